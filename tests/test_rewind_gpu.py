"""Speculative decoding rewinds the cursor and writes over rows a rejected draft left
in the cache (crates/whetstone-core/src/engine.rs:865-880,
crates/whetstone-core/src/speculate.rs:227-239): the append must be overwrite-safe and
the attention that follows must see the NEW row, although stale finite data sits at and
behind it.  Back to back on one stream, no synchronize, against the numpy oracle."""

import numpy as np
import pytest
import torch

from oracle import attention_oracle as orc
from tests.helpers import assert_close_per_head, bits16, dev, host
from tests.test_parity_gpu import build_paged_case
from whetstone_b200 import chunk, decode, paged, workloads

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def no_watchdog_trips():
    yield
    assert decode.device_error() == 0


@pytest.mark.parametrize("n_q,n_kv,hd", [(28, 4, 128), (14, 2, 64)])
@pytest.mark.parametrize("pos0", [7, 60, 1021, 4090])
def test_rewind_then_decode_over_stale_rows(n_q, n_kv, hd, pos0):
    theta = 1e6
    rng = np.random.default_rng(pos0 + hd)
    drafts = 5
    max_seq = pos0 + 1 + drafts + 40
    width = (n_q + 2 * n_kv) * hd
    table = decode.RopeTable(max_seq, hd, theta)
    cache = decode.KvCache(n_kv, n_q, hd, max_seq)
    pre = workloads.f16_values(rng, (pos0, width))
    blk = workloads.f16_values(rng, (1 + drafts, width))
    chunk.rope_cache(dev(pre), cache, table, n_q, 0, pos0)
    _, k_pre, v_pre = orc.rope_append(pre, np.arange(pos0), n_q, n_kv, hd, theta)

    # verify round: 1 + drafts rows at pos0, attended as a chunk
    blk_d = dev(blk)
    chunk.rope_cache(blk_d, cache, table, n_q, pos0, 1 + drafts)
    out_blk = torch.zeros((1 + drafts) * n_q * hd, dtype=torch.float16, device="cuda")
    chunk.attn(blk_d, cache, out_blk, n_q, pos0, 1 + drafts)
    qb, kb, vb = orc.rope_append(blk, pos0 + np.arange(1 + drafts), n_q, n_kv, hd, theta)
    want = orc.attention_blocked(qb, np.concatenate([k_pre, kb]), np.concatenate([v_pre, vb]),
                                 pos0 + 1 + np.arange(1 + drafts))
    assert_close_per_head(host(out_blk).astype(np.float64).reshape(1 + drafts, n_q, hd), want,
                          f"verify block at {pos0}")

    # two drafts accepted: the cursor goes back to pos0 + 2, where (and behind which) the
    # rejected drafts' rows still sit; a DIFFERENT token is appended there and attended
    accepted = 2
    cur = decode.DeviceCursor(pos0 + accepted)
    steps = 3
    new = workloads.f16_values(rng, (steps, width))
    new_d = dev(new)
    outs = torch.zeros(steps, n_q * hd, dtype=torch.float16, device="cuda")
    for j in range(steps):   # no synchronize anywhere in this loop
        decode.rope_cache(new_d[j], cache, table, n_q, cur)
        decode.attn_decode(new_d[j], cache, outs[j], n_q, cur)
        cur.advance(max_seq)
    torch.cuda.synchronize()
    qn, kn, vn = orc.rope_append(new, pos0 + accepted + np.arange(steps), n_q, n_kv, hd, theta)
    k_all = np.concatenate([k_pre, kb[:accepted], kn])
    v_all = np.concatenate([v_pre, vb[:accepted], vn])
    want = orc.attention_blocked(qn, k_all, v_all, pos0 + accepted + 1 + np.arange(steps))
    assert_close_per_head(host(outs).astype(np.float64).reshape(steps, n_q, hd), want,
                          f"decode after rewind to {pos0 + accepted}")
    # the overwritten rows hold the new values, bit for bit in V
    vbits = bits16(cache.v)[:, pos0 + accepted:pos0 + accepted + steps]
    assert np.array_equal(vbits, vn.transpose(1, 0, 2).astype(np.float16).view(np.uint16))
    # the rejected draft row beyond the new tokens is still the stale one (nothing else moved)
    if accepted + steps < 1 + drafts:
        stale = bits16(cache.v)[:, pos0 + accepted + steps]
        assert np.array_equal(stale, vb[accepted + steps].astype(np.float16).view(np.uint16))


def test_second_verify_round_over_the_same_pages():
    """Paged batch: a verify round appends 5 drafts per sequence and attends; every
    sequence accepts a different number of them; the next round appends new tokens
    over the rejected rows of the same pages and attends again."""
    shape = workloads.QWEN25_7B
    n_q, n_kv, hd, theta = shape.n_q, shape.n_kv, shape.head_dim, 1e6
    lengths = [100, 2040, 16, 777]
    accepted = [0, 3, 5, 1]
    drafts = 5
    rng = np.random.default_rng(31)
    cache, table_np, k_ctx, v_ctx = build_paged_case(rng, shape, lengths, 2 * drafts + 1,
                                                     with_nan=False)
    n_seq = len(lengths)
    total = n_seq * drafts
    cu = dev(np.arange(n_seq + 1, dtype=np.int32) * drafts)
    max_len = max(lengths) + 2 * drafts + 1
    rtab = decode.RopeTable(max_len, hd, theta)
    scratch = torch.empty(paged.verify_scratch_floats(n_seq, drafts, n_q, n_kv, hd, max_len),
                          dtype=torch.float32, device="cuda")
    k_live = [k.astype(np.float64).transpose(1, 0, 2) for k in k_ctx]
    v_live = [v.astype(np.float64).transpose(1, 0, 2) for v in v_ctx]
    pos = np.asarray(lengths, np.int32)
    for rnd in range(2):
        qkv = workloads.f16_values(rng, (total, shape.qkv_width))
        qd, pos0 = dev(qkv), dev(pos)
        out = torch.zeros(total * n_q * hd, dtype=torch.float16, device="cuda")
        paged.rope_cache(qd, cache, rtab, n_q, pos0, cu, total)
        paged.attn_verify(qd, cache, out, scratch, n_q, pos0, cu, total, drafts, max_len)
        got = host(out).astype(np.float64).reshape(n_seq, drafts, n_q, hd)
        for s in range(n_seq):
            L = int(pos[s])
            qr, kr, vv = orc.rope_append(qkv[s * drafts:(s + 1) * drafts], L + np.arange(drafts),
                                         n_q, n_kv, hd, theta)
            want = orc.attention_blocked(qr, np.concatenate([k_live[s], kr]),
                                         np.concatenate([v_live[s], vv]),
                                         L + 1 + np.arange(drafts))
            assert_close_per_head(got[s], want, f"round {rnd} sequence {s} at {L}")
            keep = accepted[s]
            k_live[s] = np.concatenate([k_live[s], kr[:keep]])
            v_live[s] = np.concatenate([v_live[s], vv[:keep]])
        pos = pos + np.asarray(accepted, np.int32)


@pytest.mark.parametrize("hd", [96, 160])
def test_single_token_append_of_other_head_widths_right_after_its_producer(hd):
    """Head widths that take the generic append kernel (96, 160): the append is
    launched right behind the kernels that write its inputs (the projection row and the
    cursor), with no synchronize, many times in a row; rows and q must come out as the
    oracle says."""
    n_q, n_kv, theta, max_seq, steps = 6, 2, 1e6, 40, 24
    rng = np.random.default_rng(hd)
    width = (n_q + 2 * n_kv) * hd
    table = decode.RopeTable(max_seq, hd, theta)
    cache = decode.KvCache(n_kv, n_q, hd, max_seq)
    src = workloads.f16_values(rng, (steps, width))
    src_d = dev(src)
    row = torch.zeros(width, dtype=torch.float32, device="cuda")
    rotated = torch.zeros(steps, width, dtype=torch.float32, device="cuda")
    cur = decode.DeviceCursor(3)
    decode.use_torch_stream()
    for j in range(steps):
        row.copy_(src_d[j])            # producer of qkv, same stream
        decode.rope_cache(row, cache, table, n_q, cur)
        rotated[j].copy_(row)
        cur.advance(max_seq)           # producer of the next cursor value
    torch.cuda.synchronize()
    qr, kr, vv = orc.rope_append(src, 3 + np.arange(steps), n_q, n_kv, hd, theta)
    got_q = host(rotated)[:, : n_q * hd].reshape(steps, n_q, hd)
    np.testing.assert_allclose(got_q, qr, rtol=0, atol=4e-6)
    vbits = bits16(cache.v)[:, 3:3 + steps]
    assert np.array_equal(vbits, vv.transpose(1, 0, 2).astype(np.float16).view(np.uint16))
    from tests.helpers import assert_k_cache_matches
    assert_k_cache_matches(bits16(cache.k)[:, 3:3 + steps], kr.transpose(1, 0, 2), f"K rows, hd {hd}")
