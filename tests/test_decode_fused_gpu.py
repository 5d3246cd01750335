"""The decode kernel's variants (how many tiles are asked for ahead of the grid
dependency, ring depth -- at half the ring two blocks share an SM -- and slice count)
and the sharded form whose cross-GPU exchange runs inside the slice-merge kernel,
through the C ABI against the numpy oracle.  Semantics: cuda/attention.cu:57-193 of
the engine; the knobs change summation order only."""

import numpy as np
import pytest
import torch

from oracle import attention_oracle as orc
from tests.helpers import NAN16, assert_close_per_head, dev, fill_bits, host
from whetstone_b200 import chunk, decode, workloads

pytestmark = pytest.mark.gpu

SPLITS, EARLY, STAGES = 1, 2, 4


@pytest.fixture(autouse=True)
def default_tuning_and_no_watchdog_trips():
    yield
    for key, val in ((SPLITS, 0), (EARLY, -1), (STAGES, 0)):
        decode.set_tuning(key, val)
    assert decode.device_error() == 0, "a kernel gave up waiting on a barrier"


def rand16(rng, shape):
    return workloads.f16_values(rng, shape, np.float16)


VARIANTS = [  # (early, stages, splits)
    (1, 0, 0), (0, 0, 0), (6, 6, 0), (2, 2, 0), (3, 3, 0), (3, 4, 36), (6, 0, 5), (2, 3, 64),
    (12, 12, 2),
]


@pytest.mark.parametrize("early,stages,splits", VARIANTS)
@pytest.mark.parametrize("n_q,n_kv,hd,seq", [(28, 4, 128, 1), (28, 4, 128, 65), (28, 4, 128, 700),
                                             (28, 4, 128, 9000), (14, 2, 64, 513),
                                             (14, 2, 64, 4099), (64, 2, 64, 2000),
                                             (16, 1, 128, 3100)])
def test_decode_variants_match_oracle(early, stages, splits, n_q, n_kv, hd, seq):
    decode.set_tuning(EARLY, early)
    decode.set_tuning(STAGES, stages)
    decode.set_tuning(SPLITS, splits)
    rng = np.random.default_rng(seq * 7 + n_q + early)
    max_seq = seq + 91
    cache = decode.KvCache(n_kv, n_q, hd, max_seq)
    fill_bits(cache.k, NAN16)
    fill_bits(cache.v, NAN16)
    fill_bits(cache.partials.view(torch.float16), NAN16)
    k, v = rand16(rng, (n_kv, seq, hd)), rand16(rng, (n_kv, seq, hd))
    cache.k[:, :seq] = dev(k)
    cache.v[:, :seq] = dev(v)
    want = None
    # three calls in a row on one scratch
    for rep in range(3):
        q = workloads.f16_values(rng, (n_q, hd))
        out = torch.zeros(n_q * hd, dtype=torch.float16, device="cuda")
        decode.attn_decode(dev(q), cache, out, n_q, decode.DeviceCursor(seq - 1))
        want = orc.decode_attention(q, k, v, seq)
        assert_close_per_head(host(out).astype(np.float64).reshape(n_q, hd), want,
                              f"decode variant {(early, stages, splits)} seq {seq} call {rep}")


@pytest.mark.parametrize("early,stages", [(6, 6), (2, 0), (3, 3), (0, 0)])
@pytest.mark.parametrize("prefix", [3, 200, 1500, 5000])
def test_append_then_decode_back_to_back(early, stages, prefix):
    """One-row appends and decode attention back to back with no synchronize: the
    decode kernel asks for tiles before the append ahead of it has finished and must
    still see the row it wrote (the newest row is patched after the dependency)."""
    decode.set_tuning(EARLY, early)
    decode.set_tuning(STAGES, stages)
    n_q, n_kv, hd, theta = 28, 4, 128, 1e6
    rng = np.random.default_rng(prefix + early)
    steps = 70   # crosses a 64-row tile boundary
    max_seq = prefix + steps + 9
    width = (n_q + 2 * n_kv) * hd
    table = decode.RopeTable(max_seq, hd, theta)
    cache = decode.KvCache(n_kv, n_q, hd, max_seq)
    fill_bits(cache.k, NAN16)
    fill_bits(cache.v, NAN16)
    pre = workloads.f16_values(rng, (prefix, width))
    rows = workloads.f16_values(rng, (steps, width))
    outs = torch.zeros(steps, n_q * hd, dtype=torch.float16, device="cuda")
    pre_d, rows_d = dev(pre), dev(rows)
    cur = decode.DeviceCursor(prefix)
    chunk.rope_cache(pre_d, cache, table, n_q, 0, prefix)
    for j in range(steps):
        decode.rope_cache(rows_d[j], cache, table, n_q, cur)
        decode.attn_decode(rows_d[j], cache, outs[j], n_q, cur)
        cur.advance(max_seq)
    torch.cuda.synchronize()
    _, k_pre, v_pre = orc.rope_append(pre, np.arange(prefix), n_q, n_kv, hd, theta)
    qr, k_new, v_new = orc.rope_append(rows, prefix + np.arange(steps), n_q, n_kv, hd, theta)
    k_all, v_all = np.concatenate([k_pre, k_new]), np.concatenate([v_pre, v_new])
    want = orc.attention_blocked(qr, k_all, v_all, prefix + 1 + np.arange(steps))
    assert_close_per_head(host(outs).astype(np.float64).reshape(steps, n_q, hd), want,
                          f"append + decode, prefix {prefix}, early {early}, stages {stages}")


def test_partial_output_is_the_reference_triple():
    """wst_attn_decode_partial: the (m, l, acc) triple of cuda/attention.cu:50-55."""
    rng = np.random.default_rng(8)
    n_q, n_kv, hd, seq = 28, 4, 128, 2500
    k, v = rand16(rng, (n_kv, seq, hd)), rand16(rng, (n_kv, seq, hd))
    q = workloads.f16_values(rng, (n_q, hd))
    cache = decode.KvCache(n_kv, n_q, hd, seq + 5)
    cache.k[:, :seq] = dev(k)
    cache.v[:, :seq] = dev(v)
    part = torch.zeros(n_q, hd + 2, dtype=torch.float32, device="cuda")
    decode.attn_decode_partial(dev(q), cache, part, n_q,
                               torch.tensor([seq], dtype=torch.int32, device="cuda"))
    p = host(part).astype(np.float64)
    got = p[:, 2:] / p[:, 1:2]
    assert_close_per_head(got, orc.decode_attention(q, k, v, seq), "partial triple", max_abs=1e-3)
    # m is the row maximum of the scaled scores, in natural-log units
    kk = k.astype(np.float64)
    for head in (0, 13, 27):
        scores = kk[head // (n_q // n_kv)] @ q[head].astype(np.float64) / np.sqrt(hd)
        assert abs(p[head, 0] - scores.max()) < 2e-2


# ---------------------------------------------- sharded form, exchange in the kernel

def _packets(triple: np.ndarray, tag: int) -> np.ndarray:
    """[n_q][hd+2] float32 -> the 8-byte {value, tag} packets as int32 pairs."""
    out = np.empty(triple.shape + (2,), dtype=np.int32)
    out[..., 0] = triple.astype(np.float32).view(np.int32)
    out[..., 1] = tag
    return out


def test_sharded_decode_merges_a_peers_triples():
    """Two shards of one sequence, one GPU, no second kernel: the peer's triples are
    computed with wst_attn_decode_partial and laid into this rank's mailbox the way
    the peer's kernel would store them; wst_attn_decode_sharded then attends over
    shard 0 and its merge kernel publishes, finds the peer's packets, merges and writes
    the fp16 result.
    Two calls: both mailbox halves and the call counter."""
    rng = np.random.default_rng(17)
    n_q, n_kv, hd, world = 28, 4, 128, 2
    stride = hd + 2
    seqs = (3000, 1777)
    boxes_np = np.zeros((2, 2, world, n_q, stride, 2), dtype=np.int32)   # [rank][parity]...
    own = torch.zeros(2 * world * n_q * stride * 2, dtype=torch.int32, device="cuda")
    peer = torch.zeros_like(own)
    boxes = torch.tensor([own.data_ptr(), peer.data_ptr()], dtype=torch.int64, device="cuda")
    state = torch.zeros(n_q, dtype=torch.int32, device="cuda")
    for call, seq in enumerate(seqs):
        tag = call + 1
        cut = seq // 2 + 5
        k, v = rand16(rng, (n_kv, seq, hd)), rand16(rng, (n_kv, seq, hd))
        q = workloads.f16_values(rng, (n_q, hd))
        qd = dev(q)
        shard0 = decode.KvCache(n_kv, n_q, hd, cut + 3)
        shard1 = decode.KvCache(n_kv, n_q, hd, seq - cut + 3)
        for c in (shard0, shard1):
            fill_bits(c.k, NAN16)
            fill_bits(c.v, NAN16)
        shard0.k[:, :cut], shard0.v[:, :cut] = dev(k[:, :cut]), dev(v[:, :cut])
        shard1.k[:, :seq - cut], shard1.v[:, :seq - cut] = dev(k[:, cut:]), dev(v[:, cut:])
        theirs = torch.zeros(n_q, stride, dtype=torch.float32, device="cuda")
        decode.attn_decode_partial(qd, shard1, theirs, n_q,
                                   torch.tensor([seq - cut], dtype=torch.int32, device="cuda"))
        torch.cuda.synchronize()
        box = host(own).reshape(2, world, n_q, stride, 2).copy()
        box[tag & 1, 1] = _packets(host(theirs), tag)
        own.copy_(dev(box.reshape(-1)))
        out = torch.zeros(n_q * hd, dtype=torch.float16, device="cuda")
        decode.attn_decode_sharded(qd, shard0, out, n_q,
                                   torch.tensor([cut], dtype=torch.int32, device="cuda"),
                                   boxes, state, 0, world)
        torch.cuda.synchronize()
        assert decode.device_error() == 0
        assert_close_per_head(host(out).astype(np.float64).reshape(n_q, hd),
                              orc.decode_attention(q, k, v, seq), f"sharded call {call}")
        assert torch.all(state == tag)
        # what this rank published for the peer: its own triples, tagged
        sent = host(peer).reshape(2, world, n_q, stride, 2)[tag & 1, 0]
        assert np.all(sent[..., 1] == tag)
        mine = torch.zeros(n_q, stride, dtype=torch.float32, device="cuda")
        decode.attn_decode_partial(qd, shard0, mine, n_q,
                                   torch.tensor([cut], dtype=torch.int32, device="cuda"))
        np.testing.assert_allclose(sent[..., 0].view(np.float32), host(mine), rtol=2e-5, atol=1e-6)


def test_sharded_decode_wait_runs_out_and_reports():
    """A peer that never publishes: the polls give up after their bound (about a
    second), the device error word says so, `out` stays as it was, the counters still
    advance and the context stays usable.  Local buffers only, one rank's launches."""
    rng = np.random.default_rng(4)
    n_q, n_kv, hd, world, seq = 14, 2, 64, 2, 900
    stride = hd + 2
    own = torch.zeros(2 * world * n_q * stride * 2, dtype=torch.int32, device="cuda")
    silent = torch.zeros_like(own)
    boxes = torch.tensor([own.data_ptr(), silent.data_ptr()], dtype=torch.int64, device="cuda")
    state = torch.zeros(n_q, dtype=torch.int32, device="cuda")
    cache = decode.KvCache(n_kv, n_q, hd, seq)
    cache.k.copy_(dev(rand16(rng, (n_kv, seq, hd))))
    cache.v.copy_(dev(rand16(rng, (n_kv, seq, hd))))
    q = dev(workloads.f16_values(rng, (n_q, hd)))
    out = torch.full((n_q * hd,), 7.0, dtype=torch.float16, device="cuda")
    assert decode.device_error() == 0
    decode.attn_decode_sharded(q, cache, out, n_q,
                               torch.tensor([seq], dtype=torch.int32, device="cuda"), boxes,
                               state, 0, world)
    torch.cuda.synchronize()
    assert decode.device_error() == 0x401
    assert torch.all(out == 7.0)
    assert torch.all(state == 1)
    # the same launch with world = 1 is an ordinary decode over the shard
    out1 = torch.zeros(n_q * hd, dtype=torch.float16, device="cuda")
    one = torch.tensor([own.data_ptr()], dtype=torch.int64, device="cuda")
    decode.attn_decode_sharded(q, cache, out1, n_q,
                               torch.tensor([seq], dtype=torch.int32, device="cuda"), one, state,
                               0, 1)
    ref = torch.zeros(n_q * hd, dtype=torch.float16, device="cuda")
    decode.attn_decode(q, cache, ref, n_q, decode.DeviceCursor(seq - 1))
    torch.cuda.synchronize()
    assert decode.device_error() == 0
    assert torch.equal(out1, ref) or (out1.float() - ref.float()).abs().max().item() <= 1e-3


# ------------------------------------------------ switches and the chunk workspace

def test_decode_with_the_early_requests_switched_off():
    """wst_b200_set_decode_overlap(0): no cache row is asked for before everything ahead
    in the stream has finished (for hosts that cannot keep the stream-order rule); the
    results do not change."""
    from whetstone_b200._ffi import check, lib
    check(lib.wst_b200_set_decode_overlap(0))
    try:
        n_q, n_kv, hd, theta, prefix, steps = 28, 4, 128, 1e6, 900, 8
        rng = np.random.default_rng(77)
        max_seq = prefix + steps + 3
        width = (n_q + 2 * n_kv) * hd
        table = decode.RopeTable(max_seq, hd, theta)
        cache = decode.KvCache(n_kv, n_q, hd, max_seq)
        pre, rows = workloads.f16_values(rng, (prefix, width)), workloads.f16_values(rng, (steps, width))
        rows_d = dev(rows)
        outs = torch.zeros(steps, n_q * hd, dtype=torch.float16, device="cuda")
        cur = decode.DeviceCursor(prefix)
        chunk.rope_cache(dev(pre), cache, table, n_q, 0, prefix)
        for j in range(steps):
            decode.rope_cache(rows_d[j], cache, table, n_q, cur)
            decode.attn_decode(rows_d[j], cache, outs[j], n_q, cur)
            cur.advance(max_seq)
        torch.cuda.synchronize()
        _, k_pre, v_pre = orc.rope_append(pre, np.arange(prefix), n_q, n_kv, hd, theta)
        qr, k_new, v_new = orc.rope_append(rows, prefix + np.arange(steps), n_q, n_kv, hd, theta)
        want = orc.attention_blocked(qr, np.concatenate([k_pre, k_new]), np.concatenate([v_pre, v_new]),
                                     prefix + 1 + np.arange(steps))
        assert_close_per_head(host(outs).astype(np.float64).reshape(steps, n_q, hd), want,
                              "decode without early requests")
    finally:
        check(lib.wst_b200_set_decode_overlap(1))


def test_chunk_call_without_a_workspace_runs_unsplit_and_says_so():
    """A thread's first wst_attn_chunk that wants to split the KV range, made under
    stream capture: no workspace can be allocated, so the launch runs unsplit, returns
    WST_OK and leaves a note in the thread's error text; the captured graph still
    computes the right thing.  After wst_b200_reserve_chunk_workspace the same call
    leaves no note."""
    import ctypes
    import threading

    from whetstone_b200._ffi import lib

    n_q, n_kv, hd, pos0, n = 28, 4, 128, 3000, 6
    rng = np.random.default_rng(41)
    max_seq = pos0 + n + 10
    k, v = rand16(rng, (n_kv, pos0 + n, hd)), rand16(rng, (n_kv, pos0 + n, hd))
    cache = decode.KvCache(n_kv, n_q, hd, max_seq)
    cache.k[:, :pos0 + n], cache.v[:, :pos0 + n] = dev(k), dev(v)
    width = (n_q + 2 * n_kv) * hd
    qkv = np.zeros((n, width), np.float32)
    q = workloads.f16_values(rng, (n, n_q, hd))
    qkv[:, : n_q * hd] = q.reshape(n, -1)
    qd = dev(qkv)
    out = torch.zeros(n * n_q * hd, dtype=torch.float16, device="cuda")
    torch.cuda.synchronize()
    notes = {}

    def worker():
        P = ctypes.c_void_p
        args = (P(qd.data_ptr()), P(cache.k.data_ptr()), P(cache.v.data_ptr()), P(out.data_ptr()),
                n_q, n_kv, hd, pos0, n, max_seq, ctypes.c_float(1.0 / np.sqrt(hd)))
        assert lib.wst_device_set(torch.cuda.current_device()) == 0
        assert lib.wst_b200_set_stream(None) == 0          # this thread's own default stream
        assert lib.wst_graph_capture_begin() == 0, lib.wst_last_error()
        status = lib.wst_attn_chunk(*args)
        notes["captured"] = (status, lib.wst_last_error().decode())
        graph = ctypes.c_void_p()
        assert lib.wst_graph_capture_end(ctypes.byref(graph)) == 0, lib.wst_last_error()
        assert lib.wst_graph_launch(graph) == 0 and lib.wst_stream_sync() == 0
        assert lib.wst_graph_destroy(graph) == 0
        notes["reserve"] = lib.wst_b200_reserve_chunk_workspace()
        lib.wst_attn_decode_noscratch(None, None, None, None, 1, 1, 64, None, 1, 0.0)  # resets the text
        status = lib.wst_attn_chunk(*args)
        notes["eager"] = (status, lib.wst_last_error().decode())
        assert lib.wst_stream_sync() == 0

    t = threading.Thread(target=worker)
    t.start()
    t.join()
    assert notes["captured"][0] == 0 and "without splitting" in notes["captured"][1], notes
    assert notes["reserve"] == 0
    assert notes["eager"][0] == 0 and "without splitting" not in notes["eager"][1], notes
    want = orc.chunk_attention(q.astype(np.float64), k, v, pos0, 1.0 / np.sqrt(hd))
    assert_close_per_head(host(out).astype(np.float64).reshape(n, n_q, hd), want,
                          "chunk through the unsplit and the split launch")
