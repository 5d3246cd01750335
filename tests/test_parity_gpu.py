"""GPU parity tests: the CUDA path, called through the C ABI, against the numpy
oracle on the same seeded inputs.  Bar: max abs error <= 2e-3 and cosine >=
0.9999 per head vector; KV-append indexing bit-exact."""

import numpy as np
import pytest
import torch

from oracle import attention_oracle as orc
from tests.helpers import (NAN16, SENTINEL, assert_close_per_head, bits16, dev, f16_ulp_distance,
                           fill_bits, host)
from whetstone_b200 import chunk, decode, paged, workloads
from whetstone_b200._ffi import InvalidArg, check, lib

pytestmark = pytest.mark.gpu


@pytest.fixture(params=[0, 1], ids=["auto", "portable"])
def kernel_choice(request):
    check(lib.wst_b200_set_kernel_choice(request.param))
    yield request.param
    check(lib.wst_b200_set_kernel_choice(0))


@pytest.fixture(autouse=True)
def no_watchdog_trips():
    yield
    assert decode.device_error() == 0, "a kernel gave up waiting on a barrier"


def rand16(rng, shape):
    return workloads.f16_values(rng, shape, np.float16)


# ------------------------------------------------------------------ set 1

@pytest.mark.parametrize("n_q,n_kv,hd", [(14, 2, 64), (28, 4, 128), (4, 4, 256), (6, 2, 96),
                                         (3, 1, 34)])
@pytest.mark.parametrize("norm", [False, True])
def test_append_indexing_is_bit_exact(n_q, n_kv, hd, norm):
    """Sentinel-filled caches: exactly rows pos0..pos0+n-1 of every KV head
    change; V equals fp16(v) bit for bit; K is within 1 fp16 ulp of the f64
    oracle; q is rotated in place."""
    rng = np.random.default_rng(11)
    max_seq, pos0, n, theta = 48, 17, 7, 1e6
    width = (n_q + 2 * n_kv) * hd
    qkv = workloads.f16_values(rng, (n, width))
    cache = decode.KvCache(n_kv, n_q, hd, max_seq)
    fill_bits(cache.k, SENTINEL)
    fill_bits(cache.v, SENTINEL)
    table = decode.RopeTable(max_seq, hd, theta)
    gains = None
    gq = gk = None
    if norm:
        gq, gk = workloads.qk_gains(rng, hd)
        gains = decode.QkNorm(dev(gq), dev(gk), 1e-6)
    qd = dev(qkv)
    chunk.rope_cache(qd, cache, table, n_q, pos0, n, gains)
    qr, kr, vv = orc.rope_append(qkv, pos0 + np.arange(n), n_q, n_kv, hd, theta, gq, gk, 1e-6)

    kb, vb = bits16(cache.k), bits16(cache.v)
    untouched = np.ones(max_seq, bool)
    untouched[pos0:pos0 + n] = False
    assert np.all(kb[:, untouched] == SENTINEL) and np.all(vb[:, untouched] == SENTINEL)
    want_v = vv.transpose(1, 0, 2).astype(np.float16).view(np.uint16)
    assert np.array_equal(vb[:, pos0:pos0 + n], want_v), "V must be the exact fp16 of v"
    want_k = kr.transpose(1, 0, 2).astype(np.float16).view(np.uint16)
    assert f16_ulp_distance(kb[:, pos0:pos0 + n], want_k).max() <= 1
    got_q = host(qd)[:, : n_q * hd].reshape(n, n_q, hd)
    np.testing.assert_allclose(got_q, qr, rtol=0, atol=2e-5 if norm else 4e-6)
    # k and v parts of the projection buffer are inputs only
    assert np.array_equal(host(qd)[:, n_q * hd:], qkv[:, n_q * hd:])


def test_decode_append_clamps_the_cursor():
    """*pos < 0 writes row 0, *pos >= max_seq writes the last row (decode.cu:132)."""
    n_q, n_kv, hd, max_seq = 2, 1, 64, 8
    rng = np.random.default_rng(5)
    table = decode.RopeTable(max_seq, hd, 1e6)
    for raw, row in ((-3, 0), (8, 7), (1000, 7)):
        cache = decode.KvCache(n_kv, n_q, hd, max_seq)
        fill_bits(cache.v, SENTINEL)
        qkv = workloads.f16_values(rng, ((n_q + 2 * n_kv) * hd,))
        decode.rope_cache(dev(qkv), cache, table, n_q, decode.DeviceCursor(raw))
        vb = bits16(cache.v)
        changed = [r for r in range(max_seq) if not np.all(vb[0, r] == SENTINEL)]
        assert changed == [row]


def test_advance_pos_saturates():
    cur = decode.DeviceCursor(5)
    cur.advance(7)
    assert cur.get() == 6
    cur.advance(7)
    cur.advance(7)
    assert cur.get() == 7


# ------------------------------------------------------------- set 2: decode

DECODE_SHAPES = [(14, 2, 64), (28, 4, 128), (32, 8, 128), (8, 8, 64), (16, 1, 128), (64, 2, 64)]


@pytest.mark.parametrize("n_q,n_kv,hd", DECODE_SHAPES)
@pytest.mark.parametrize("seq", [1, 2, 7, 63, 64, 65, 129, 513, 4099])
def test_decode_matches_oracle(kernel_choice, n_q, n_kv, hd, seq):
    rng = np.random.default_rng(seq * 131 + n_q)
    max_seq = seq + 77
    cache = decode.KvCache(n_kv, n_q, hd, max_seq)
    fill_bits(cache.k, NAN16)   # nothing past `seq` may influence the result
    fill_bits(cache.v, NAN16)
    k, v = rand16(rng, (n_kv, seq, hd)), rand16(rng, (n_kv, seq, hd))
    cache.k[:, :seq] = dev(k)
    cache.v[:, :seq] = dev(v)
    fill_bits(cache.partials.view(torch.float16), NAN16)  # scratch need not be clean
    q = workloads.f16_values(rng, (n_q, hd))
    out = torch.zeros(n_q * hd, dtype=torch.float16, device="cuda")
    decode.attn_decode(dev(q), cache, out, n_q, decode.DeviceCursor(seq - 1))
    want = orc.decode_attention(q, k, v, seq)
    assert_close_per_head(host(out).astype(np.float64).reshape(n_q, hd), want,
                          f"decode {n_q}/{n_kv}/{hd} seq {seq}")


@pytest.mark.parametrize("prefix", [3, 200, 1500])
def test_decode_right_after_a_chunk_append(prefix):
    """A multi-row append, a one-row append and the decode attention back to back on
    one stream, repeated without a synchronize in between: the decode kernel asks for
    its first tiles before its grid dependency is resolved, and must still see every
    row the launches ahead of it wrote (and re-read the tile with the newest row)."""
    n_q, n_kv, hd, theta = 28, 4, 128, 1e6
    rng = np.random.default_rng(prefix)
    steps = 6
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
                          f"decode after chunk append, prefix {prefix}")


@pytest.mark.parametrize("hd", [32, 96, 160, 192, 224, 256])
def test_decode_other_head_widths(hd):
    rng = np.random.default_rng(hd)
    n_q, n_kv, seq, max_seq = 6, 2, 70, 96
    cache = decode.KvCache(n_kv, n_q, hd, max_seq)
    k, v = rand16(rng, (n_kv, seq, hd)), rand16(rng, (n_kv, seq, hd))
    cache.k[:, :seq] = dev(k)
    cache.v[:, :seq] = dev(v)
    q = workloads.f16_values(rng, (n_q, hd))
    out = torch.zeros(n_q * hd, dtype=torch.float16, device="cuda")
    decode.attn_decode(dev(q), cache, out, n_q, decode.DeviceCursor(seq - 1))
    assert_close_per_head(host(out).astype(np.float64).reshape(n_q, hd),
                          orc.decode_attention(q, k, v, seq), f"decode head_dim {hd}")


def test_decode_cursor_is_clamped():
    """seq = min(max(*pos, 0) + 1, max_seq) (attention.cu:62-65)."""
    rng = np.random.default_rng(9)
    n_q, n_kv, hd, max_seq = 14, 2, 64, 100
    cache = decode.KvCache(n_kv, n_q, hd, max_seq)
    k, v = rand16(rng, (n_kv, max_seq, hd)), rand16(rng, (n_kv, max_seq, hd))
    cache.k.copy_(dev(k))
    cache.v.copy_(dev(v))
    q = workloads.f16_values(rng, (n_q, hd))
    for raw, seq in ((-5, 1), (99, 100), (5000, 100)):
        out = torch.zeros(n_q * hd, dtype=torch.float16, device="cuda")
        decode.attn_decode(dev(q), cache, out, n_q, decode.DeviceCursor(raw))
        assert_close_per_head(host(out).astype(np.float64).reshape(n_q, hd),
                              orc.decode_attention(q, k, v, seq), f"cursor {raw}")


def test_repeated_decode_calls_share_scratch():
    """Back-to-back launches on one stream reuse one split scratch: each launch
    must be ordered after the merge of the one before it."""
    rng = np.random.default_rng(21)
    n_q, n_kv, hd, seq = 28, 4, 128, 3000
    cache = decode.KvCache(n_kv, n_q, hd, seq)
    k, v = rand16(rng, (n_kv, seq, hd)), rand16(rng, (n_kv, seq, hd))
    cache.k.copy_(dev(k))
    cache.v.copy_(dev(v))
    qs = [workloads.f16_values(rng, (n_q, hd)) for _ in range(40)]
    outs = [torch.zeros(n_q * hd, dtype=torch.float16, device="cuda") for _ in qs]
    cur = decode.DeviceCursor(seq - 1)
    for q, o in zip(qs, outs):
        decode.attn_decode(dev(q), cache, o, n_q, cur)
    for i in (0, 17, 39):
        assert_close_per_head(host(outs[i]).astype(np.float64).reshape(n_q, hd),
                              orc.decode_attention(qs[i], k, v, seq), f"call {i}")


# ------------------------------------------- cross-GPU form: partial + merge

@pytest.mark.parametrize("shards", [2, 4, 8])
def test_partial_triples_merge_to_the_full_result(kernel_choice, shards):
    rng = np.random.default_rng(shards)
    n_q, n_kv, hd, seq = 28, 4, 128, 2048 + 13
    k, v = rand16(rng, (n_kv, seq, hd)), rand16(rng, (n_kv, seq, hd))
    q = workloads.f16_values(rng, (n_q, hd))
    qd = dev(q)
    per = (seq + shards - 1) // shards
    parts = torch.zeros((shards + 1, n_q, hd + 2), dtype=torch.float32, device="cuda")
    for g in range(shards):
        lo, hi = g * per, min(seq, (g + 1) * per)
        cache = decode.KvCache(n_kv, n_q, hd, per)
        fill_bits(cache.k, NAN16)
        fill_bits(cache.v, NAN16)
        cache.k[:, : hi - lo] = dev(k[:, lo:hi])
        cache.v[:, : hi - lo] = dev(v[:, lo:hi])
        length = torch.tensor([hi - lo], dtype=torch.int32, device="cuda")
        decode.attn_decode_partial(qd, cache, parts[g], n_q, length)
    # one more shard with nothing in it must not disturb the merge
    empty = decode.KvCache(n_kv, n_q, hd, per)
    decode.attn_decode_partial(qd, empty, parts[shards], n_q,
                               torch.zeros(1, dtype=torch.int32, device="cuda"))
    ph = host(parts[shards])
    assert np.all(ph[:, 0] == -np.inf) and np.all(ph[:, 1:] == 0)
    out = torch.zeros(n_q * hd, dtype=torch.float16, device="cuda")
    decode.attn_merge_partials(parts, out, n_q, hd)
    assert_close_per_head(host(out).astype(np.float64).reshape(n_q, hd),
                          orc.decode_attention(q, k, v, seq), f"{shards} shards")


# -------------------------------------------- sets 3/4: chunk (contiguous)

@pytest.fixture(params=[0, 1, 2, 3, 4], ids=["auto", "portable", "splitkv", "tcgen05", "tcgen05pair"])
def chunk_kernel_choice(request):
    check(lib.wst_b200_set_kernel_choice(request.param))
    yield request.param
    check(lib.wst_b200_set_kernel_choice(0))


@pytest.mark.parametrize("n_q,n_kv,hd", [(14, 2, 64), (28, 4, 128), (32, 8, 128)])
@pytest.mark.parametrize("pos0,n", [(0, 1), (0, 5), (0, 64), (20, 5), (1000, 5), (1000, 17),
                                    (37, 130), (0, 257), (4000, 6), (100, 128), (511, 300),
                                    (3000, 16)])
def test_chunk_matches_oracle(chunk_kernel_choice, n_q, n_kv, hd, pos0, n):
    """append + causal attention of a chunk, prefix written by earlier appends."""
    rng = np.random.default_rng(pos0 * 7 + n + hd)
    theta = 1e6
    max_seq = pos0 + n + 29
    width = (n_q + 2 * n_kv) * hd
    cache = decode.KvCache(n_kv, n_q, hd, max_seq)
    fill_bits(cache.k, NAN16)
    fill_bits(cache.v, NAN16)
    table = decode.RopeTable(max_seq, hd, theta)
    k_all = np.zeros((pos0 + n, n_kv, hd))
    v_all = np.zeros((pos0 + n, n_kv, hd))
    if pos0:
        pre = workloads.f16_values(rng, (pos0, width))
        chunk.rope_cache(dev(pre), cache, table, n_q, 0, pos0)
        _, k_all[:pos0], v_all[:pos0] = orc.rope_append(pre, np.arange(pos0), n_q, n_kv, hd, theta)
    qkv = workloads.f16_values(rng, (n, width))
    qd = dev(qkv)
    chunk.rope_cache(qd, cache, table, n_q, pos0, n)
    out = torch.zeros(n * n_q * hd, dtype=torch.float16, device="cuda")
    chunk.attn(qd, cache, out, n_q, pos0, n)
    qr, k_all[pos0:], v_all[pos0:] = orc.rope_append(qkv, pos0 + np.arange(n), n_q, n_kv, hd, theta)
    want = orc.attention_blocked(qr, k_all, v_all, pos0 + 1 + np.arange(n))
    assert_close_per_head(host(out).astype(np.float64).reshape(n, n_q, hd), want,
                          f"chunk {n_q}/{n_kv}/{hd} pos0 {pos0} n {n}")


@pytest.mark.parametrize("ramp", [0.0, 0.02, 0.3, -0.3])
def test_chunk_with_scores_that_drift_along_the_sequence(chunk_kernel_choice, ramp):
    """Scores that grow (or fall) steadily along the cache: the running exponent
    offset has to move many times (ramp 0.3: by some 50 units of log2 per 128-position
    tile), which is where a lazily or optimistically kept offset is put to the test."""
    if chunk_kernel_choice == 1:
        pytest.skip("one path per case is enough for the portable kernel")
    n_q, n_kv, hd, pos0, n = 8, 2, 128, 256, 384
    rng = np.random.default_rng(int(1000 * abs(ramp)) + 5)
    top = pos0 + n
    direction = rng.standard_normal(hd)
    direction /= np.linalg.norm(direction)
    # k(pos) = noise + ramp * pos * direction, q = noise + 4 * direction: the score
    # of a late position exceeds an early one's by about ramp * 4 * distance / sqrt(hd)
    k = (0.3 * rng.standard_normal((n_kv, top, hd)) +
         ramp * np.arange(top)[None, :, None] * direction[None, None, :] * np.sqrt(hd)).astype(np.float16)
    v = workloads.f16_values(rng, (n_kv, top, hd), np.float16)
    cache = decode.KvCache(n_kv, n_q, hd, top + 13)
    fill_bits(cache.k, NAN16)
    fill_bits(cache.v, NAN16)
    cache.k[:, :top] = dev(k)
    cache.v[:, :top] = dev(v)
    qkv = np.zeros((n, (n_q + 2 * n_kv) * hd), np.float32)
    q = (0.3 * rng.standard_normal((n, n_q, hd)) + 4.0 * direction).astype(np.float16).astype(np.float32)
    qkv[:, : n_q * hd] = q.reshape(n, -1)
    out = torch.zeros(n * n_q * hd, dtype=torch.float16, device="cuda")
    chunk.attn(dev(qkv), cache, out, n_q, pos0, n)
    want = orc.chunk_attention(q.astype(np.float64), k, v, pos0, 1.0 / np.sqrt(hd))
    assert_close_per_head(host(out).astype(np.float64).reshape(n, n_q, hd), want,
                          f"drifting scores, ramp {ramp}")


def _cache_view(batch, s_idx):
    """One sequence of a KvCacheBatch as a single-sequence KvCache (no copy)."""
    view = decode.KvCache.__new__(decode.KvCache)
    view.k, view.v = batch.k[s_idx], batch.v[s_idx]
    view.n_kv, view.head_dim, view.max_seq = batch.n_kv, batch.head_dim, batch.max_seq
    view.partials = torch.zeros(1, dtype=torch.float32, device="cuda")
    return view


@pytest.mark.parametrize("n_q,n_kv,hd", [(14, 2, 64), (32, 8, 128)])
@pytest.mark.parametrize("n", [5, 130])
def test_chunk_batch_matches_oracle(chunk_kernel_choice, n_q, n_kv, hd, n):
    """Three sequences at different positions in one launch (batched chunked prefill
    and its few-token form), against the oracle per sequence."""
    if chunk_kernel_choice == 1:
        pytest.skip("the batched entry point has no portable-kernel form")
    rng = np.random.default_rng(n * 3 + hd)
    theta, starts = 1e6, [0, 100, 517]
    n_seq, max_seq = len(starts), 700
    width = (n_q + 2 * n_kv) * hd
    batch = chunk.KvCacheBatch(n_seq, n_kv, hd, max_seq)
    fill_bits(batch.k, NAN16)
    fill_bits(batch.v, NAN16)
    table = decode.RopeTable(max_seq, hd, theta)
    prefix = []
    for s_idx, p0 in enumerate(starts):
        pre = workloads.f16_values(rng, (p0, width)) if p0 else np.zeros((0, width), np.float32)
        if p0:
            chunk.rope_cache(dev(pre), _cache_view(batch, s_idx), table, n_q, 0, p0)
        prefix.append(pre)
    qkv = workloads.f16_values(rng, (n_seq, n, width))
    qd = dev(qkv)
    pos0 = dev(np.asarray(starts, np.int32))
    chunk.rope_cache_batch(qd, batch, table, n_q, pos0, n)
    out = torch.zeros(n_seq * n * n_q * hd, dtype=torch.float16, device="cuda")
    chunk.attn_batch(qd, batch, out, n_q, pos0, n)
    got = host(out).astype(np.float64).reshape(n_seq, n, n_q, hd)
    for s_idx, p0 in enumerate(starts):
        k_all = np.zeros((p0 + n, n_kv, hd))
        v_all = np.zeros((p0 + n, n_kv, hd))
        if p0:
            _, k_all[:p0], v_all[:p0] = orc.rope_append(prefix[s_idx], np.arange(p0), n_q, n_kv, hd,
                                                        theta)
        qr, k_all[p0:], v_all[p0:] = orc.rope_append(qkv[s_idx], p0 + np.arange(n), n_q, n_kv, hd,
                                                     theta)
        want = orc.attention_blocked(qr, k_all, v_all, p0 + 1 + np.arange(n))
        assert_close_per_head(got[s_idx], want, f"batch seq {s_idx} pos0 {p0} n {n}")
        vb = bits16(batch.v[s_idx])
        assert np.array_equal(vb[:, p0:p0 + n],
                              v_all[p0:].transpose(1, 0, 2).astype(np.float16).view(np.uint16))
        assert np.all(vb[:, p0 + n:] == NAN16)


def test_chunk_argument_errors_launch_nothing():
    cache = decode.KvCache(2, 14, 64, 32)
    qkv = torch.zeros(4 * 18 * 64, dtype=torch.float32, device="cuda")
    out = torch.zeros(4 * 14 * 64, dtype=torch.float16, device="cuda")
    with pytest.raises(InvalidArg):
        check(lib.wst_attn_chunk(qkv.data_ptr(), cache.k.data_ptr(), cache.v.data_ptr(),
                                 out.data_ptr(), 14, 2, 64, 30, 4, 32, 0.125))
    assert torch.count_nonzero(out) == 0


# ---------------------------------------------------- set 4: paged verify

def build_paged_case(rng, shape, lengths, drafts, theta=1e6, with_nan=True):
    n_q, n_kv, hd = shape.n_q, shape.n_kv, shape.head_dim
    n_seq = len(lengths)
    table_np, n_pages = workloads.c5_page_table(np.asarray(lengths, np.int32), drafts, seed=77)
    cache = paged.PagedKvCache(n_pages + 3, n_kv, hd, n_seq, table_np.shape[1])
    if with_nan:
        fill_bits(cache.k, NAN16)
        fill_bits(cache.v, NAN16)
    cache.page_table.copy_(dev(table_np))
    k_ctx, v_ctx = [], []
    pool_k = host(cache.k).copy()
    pool_v = host(cache.v).copy()
    for s, L in enumerate(lengths):
        k = rand16(rng, (n_kv, L, hd))
        v = rand16(rng, (n_kv, L, hd))
        for p0 in range(0, L, 16):
            pid = table_np[s, p0 // 16]
            rows = min(16, L - p0)
            pool_k[pid, :, :rows] = k[:, p0:p0 + rows]
            pool_v[pid, :, :rows] = v[:, p0:p0 + rows]
        k_ctx.append(k)
        v_ctx.append(v)
    cache.k.copy_(dev(pool_k))
    cache.v.copy_(dev(pool_v))
    return cache, table_np, k_ctx, v_ctx


@pytest.fixture(params=[0, 2, 3], ids=["auto", "rows", "slices"])
def verify_kernel_choice(request):
    """0: when every query row of a (sequence, KV head) fits one 128-row tile, the
    persistent tcgen05 kernel over equal spans of all units' KV tiles; 3: the same tile
    pipeline with one CTA per slice of the KV range; 2: the mma.sync row-block kernel."""
    check(lib.wst_b200_set_kernel_choice(request.param))
    yield request.param
    check(lib.wst_b200_set_kernel_choice(0))


@pytest.mark.parametrize("lengths,drafts", [([100, 700, 16, 333], 5), ([1, 15, 17, 64, 65], 3),
                                            ([2050, 1024], 5), ([40], 9), ([5000, 129, 4100], 4),
                                            ([300, 77], 20)])
def test_paged_verify_matches_oracle(verify_kernel_choice, lengths, drafts):
    shape = workloads.QWEN25_7B
    n_q, n_kv, hd, theta = shape.n_q, shape.n_kv, shape.head_dim, 1e6
    rng = np.random.default_rng(sum(lengths))
    cache, table_np, k_ctx, v_ctx = build_paged_case(rng, shape, lengths, drafts)
    n_seq = len(lengths)
    total = n_seq * drafts
    qkv = workloads.f16_values(rng, (total, shape.qkv_width))
    qd = dev(qkv)
    pos0 = dev(np.asarray(lengths, np.int32))
    cu = dev(np.arange(n_seq + 1, dtype=np.int32) * drafts)
    max_len = max(lengths) + drafts
    rtab = decode.RopeTable(max_len, hd, theta)
    paged.rope_cache(qd, cache, rtab, n_q, pos0, cu, total)
    scratch = torch.empty(paged.verify_scratch_floats(n_seq, drafts, n_q, n_kv, hd, max_len),
                          dtype=torch.float32, device="cuda")
    fill_bits(scratch.view(torch.float16), NAN16)
    out = torch.zeros(total * n_q * hd, dtype=torch.float16, device="cuda")
    paged.attn_verify(qd, cache, out, scratch, n_q, pos0, cu, total, drafts, max_len)
    got = host(out).astype(np.float64).reshape(n_seq, drafts, n_q, hd)
    pool_k, pool_v = host(cache.k), host(cache.v)
    for s, L in enumerate(lengths):
        rows = qkv[s * drafts:(s + 1) * drafts]
        qr, kr, vv = orc.rope_append(rows, L + np.arange(drafts), n_q, n_kv, hd, theta)
        # appended rows landed in the mapped pages, bit-exact V, K within 1 ulp
        kc = orc.gather_pages(pool_k, table_np[s], L + drafts)
        vc = orc.gather_pages(pool_v, table_np[s], L + drafts)
        assert np.array_equal(vc[:, L:].view(np.uint16),
                              vv.transpose(1, 0, 2).astype(np.float16).view(np.uint16))
        assert f16_ulp_distance(kc[:, L:].view(np.uint16),
                                kr.transpose(1, 0, 2).astype(np.float16).view(np.uint16)).max() <= 1
        assert np.array_equal(kc[:, :L].view(np.uint16), k_ctx[s].view(np.uint16))
        k_all = np.concatenate([k_ctx[s].astype(np.float64).transpose(1, 0, 2), kr])
        v_all = np.concatenate([v_ctx[s].astype(np.float64).transpose(1, 0, 2), vv])
        want = orc.attention_blocked(qr, k_all, v_all, L + 1 + np.arange(drafts))
        assert_close_per_head(got[s], want, f"verify seq {s} (len {L})")


def test_paged_verify_ragged_token_counts(verify_kernel_choice):
    """Sequences verify different numbers of draft tokens (cu_tokens is ragged)."""
    shape = workloads.QWEN25_7B
    n_q, n_kv, hd, theta = shape.n_q, shape.n_kv, shape.head_dim, 1e6
    lengths, counts = [90, 300, 47], [1, 6, 3]
    rng = np.random.default_rng(3)
    cache, table_np, k_ctx, v_ctx = build_paged_case(rng, shape, lengths, max(counts))
    total = sum(counts)
    cu_np = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
    qkv = workloads.f16_values(rng, (total, shape.qkv_width))
    qd, pos0, cu = dev(qkv), dev(np.asarray(lengths, np.int32)), dev(cu_np)
    max_len = max(l + c for l, c in zip(lengths, counts))
    rtab = decode.RopeTable(max_len, hd, theta)
    paged.rope_cache(qd, cache, rtab, n_q, pos0, cu, total)
    scratch = torch.zeros(paged.verify_scratch_floats(3, max(counts), n_q, n_kv, hd, max_len),
                          dtype=torch.float32, device="cuda")
    out = torch.zeros(total * n_q * hd, dtype=torch.float16, device="cuda")
    paged.attn_verify(qd, cache, out, scratch, n_q, pos0, cu, total, max(counts), max_len)
    got = host(out).astype(np.float64).reshape(total, n_q, hd)
    for s, (L, c) in enumerate(zip(lengths, counts)):
        rows = qkv[cu_np[s]:cu_np[s + 1]]
        qr, kr, vv = orc.rope_append(rows, L + np.arange(c), n_q, n_kv, hd, theta)
        k_all = np.concatenate([k_ctx[s].astype(np.float64).transpose(1, 0, 2), kr])
        v_all = np.concatenate([v_ctx[s].astype(np.float64).transpose(1, 0, 2), vv])
        want = orc.attention_blocked(qr, k_all, v_all, L + 1 + np.arange(c))
        assert_close_per_head(got[cu_np[s]:cu_np[s + 1]], want, f"ragged seq {s}")


# ------------------------------------------- bounded waits report, never hang

def test_exchange_wait_runs_out_and_reports():
    """wst_attn_exchange_merge with a second "rank" that never publishes: every
    block's poll gives up after its bound (about a second), the device error word
    says so, nothing is written to `out`, and the context stays usable.  Both
    mailboxes are plain local buffers: no second kernel, no second GPU."""
    n_q, hd, world = 4, 64, 2
    packets = 2 * world * n_q * (hd + 2)
    own = torch.zeros(packets * 2, dtype=torch.int32, device="cuda")
    silent_peer = torch.zeros(packets * 2, dtype=torch.int32, device="cuda")
    boxes = torch.tensor([own.data_ptr(), silent_peer.data_ptr()], dtype=torch.int64, device="cuda")
    state = torch.zeros(n_q, dtype=torch.int32, device="cuda")
    mine = torch.ones(n_q, hd + 2, dtype=torch.float32, device="cuda")
    out = torch.full((n_q * hd,), 7.0, dtype=torch.float16, device="cuda")
    assert decode.device_error() == 0
    decode.attn_exchange_merge(mine, out, boxes, state, 0, world, n_q, hd)
    torch.cuda.synchronize()
    assert decode.device_error() == 0x401
    assert torch.all(out == 7.0)                      # no head was merged
    assert torch.all(state == 1)                      # the call is closed all the same
    assert decode.device_error() == 0                 # reading the word cleared it
    # with world = 1 the same buffers work at once
    out1 = torch.zeros(n_q * hd, dtype=torch.float16, device="cuda")
    boxes1 = torch.tensor([own.data_ptr()], dtype=torch.int64, device="cuda")
    mine[:, 0] = 0.0   # m = 0, l = 1, acc = 1  ->  out = 1
    decode.attn_exchange_merge(mine, out1, boxes1, state, 0, 1, n_q, hd)
    torch.cuda.synchronize()
    assert decode.device_error() == 0
    assert torch.allclose(out1.float(), torch.ones_like(out1.float()))
