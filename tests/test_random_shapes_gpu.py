"""Seeded random shapes through the three attention entry points, against the
oracle: head layouts, cache lengths, chunk offsets and draft counts the fixed
parametrisations of the parity tests do not list (tile-boundary straddles, GQA
groups of 1..8, slices with ragged tails).  Each seed draws a few dozen cases."""
import numpy as np
import pytest
import torch

from oracle import attention_oracle as orc
from whetstone_b200 import chunk, decode, paged, workloads
from .helpers import NAN16, assert_close_per_head, dev, fill_bits, host
from .test_parity_gpu import build_paged_case, rand16

pytestmark = pytest.mark.gpu

THETA = 1e6


def draw_layout(rng):
    hd = int(rng.choice([64, 128]))
    n_kv = int(rng.choice([1, 2, 4, 8]))
    gqa = int(rng.choice([1, 2, 4, 7, 8]))
    return n_kv * gqa, n_kv, hd


def decode_case(rng, seq_hi):
    n_q, n_kv, hd = draw_layout(rng)
    seq = int(rng.integers(1, seq_hi))
    max_seq = seq + int(rng.integers(0, 300))
    cache = decode.KvCache(n_kv, n_q, hd, max_seq)
    fill_bits(cache.k, NAN16)
    fill_bits(cache.v, NAN16)
    k, v = rand16(rng, (n_kv, seq, hd)), rand16(rng, (n_kv, seq, hd))
    cache.k[:, :seq] = dev(k)
    cache.v[:, :seq] = dev(v)
    fill_bits(cache.partials.view(torch.float16), NAN16)
    q = workloads.f16_values(rng, (n_q, hd))
    out = torch.zeros(n_q * hd, dtype=torch.float16, device="cuda")
    decode.attn_decode(dev(q), cache, out, n_q, decode.DeviceCursor(seq - 1))
    assert_close_per_head(host(out).astype(np.float64).reshape(n_q, hd),
                          orc.decode_attention(q, k, v, seq),
                          f"decode {n_q}/{n_kv}/{hd} seq {seq} max_seq {max_seq}")


def chunk_case(rng, pos_hi, n_hi):
    n_q, n_kv, hd = draw_layout(rng)
    pos0 = int(rng.integers(0, pos_hi)) if rng.random() < 0.8 else 0
    n = int(rng.integers(1, n_hi))
    max_seq = pos0 + n + int(rng.integers(0, 100))
    width = (n_q + 2 * n_kv) * hd
    cache = decode.KvCache(n_kv, n_q, hd, max_seq)
    fill_bits(cache.k, NAN16)
    fill_bits(cache.v, NAN16)
    table = decode.RopeTable(max_seq, hd, THETA)
    k_all = np.zeros((pos0 + n, n_kv, hd))
    v_all = np.zeros((pos0 + n, n_kv, hd))
    if pos0:
        pre = workloads.f16_values(rng, (pos0, width))
        chunk.rope_cache(dev(pre), cache, table, n_q, 0, pos0)
        _, k_all[:pos0], v_all[:pos0] = orc.rope_append(pre, np.arange(pos0), n_q, n_kv, hd, THETA)
    qkv = workloads.f16_values(rng, (n, width))
    qd = dev(qkv)
    chunk.rope_cache(qd, cache, table, n_q, pos0, n)
    out = torch.zeros(n * n_q * hd, dtype=torch.float16, device="cuda")
    chunk.attn(qd, cache, out, n_q, pos0, n)
    qr, k_all[pos0:], v_all[pos0:] = orc.rope_append(qkv, pos0 + np.arange(n), n_q, n_kv, hd, THETA)
    want = orc.attention_blocked(qr, k_all, v_all, pos0 + 1 + np.arange(n))
    assert_close_per_head(host(out).astype(np.float64).reshape(n, n_q, hd), want,
                          f"chunk {n_q}/{n_kv}/{hd} pos0 {pos0} n {n}")


def verify_case(rng, len_hi, drafts_hi):
    n_q, n_kv, hd = draw_layout(rng)
    shape = workloads.Shape("random", n_q, n_kv, hd, 1)
    n_seq = int(rng.integers(1, 6))
    drafts = int(rng.integers(1, drafts_hi))
    lengths = [int(x) for x in rng.integers(1, len_hi, size=n_seq)]
    cache, _, k_ctx, v_ctx = build_paged_case(rng, shape, lengths, drafts)
    total = n_seq * drafts
    qkv = workloads.f16_values(rng, (total, shape.qkv_width))
    qd = dev(qkv)
    pos0 = dev(np.asarray(lengths, np.int32))
    cu = dev(np.arange(n_seq + 1, dtype=np.int32) * drafts)
    max_len = max(lengths) + drafts
    paged.rope_cache(qd, cache, decode.RopeTable(max_len, hd, THETA), n_q, pos0, cu, total)
    scratch = torch.empty(paged.verify_scratch_floats(n_seq, drafts, n_q, n_kv, hd, max_len),
                          dtype=torch.float32, device="cuda")
    fill_bits(scratch.view(torch.float16), NAN16)
    out = torch.zeros(total * n_q * hd, dtype=torch.float16, device="cuda")
    paged.attn_verify(qd, cache, out, scratch, n_q, pos0, cu, total, drafts, max_len)
    got = host(out).astype(np.float64).reshape(n_seq, drafts, n_q, hd)
    for s, L in enumerate(lengths):
        rows = qkv[s * drafts:(s + 1) * drafts]
        qr, kr, vv = orc.rope_append(rows, L + np.arange(drafts), n_q, n_kv, hd, THETA)
        k_all = np.concatenate([k_ctx[s].astype(np.float64).transpose(1, 0, 2), kr])
        v_all = np.concatenate([v_ctx[s].astype(np.float64).transpose(1, 0, 2), vv])
        want = orc.attention_blocked(qr, k_all, v_all, L + 1 + np.arange(drafts))
        assert_close_per_head(got[s], want,
                              f"verify {n_q}/{n_kv}/{hd} lengths {lengths} drafts {drafts} seq {s}")


@pytest.mark.parametrize("seed", [1, 2, 3])
def test_random_small_shapes(seed):
    rng = np.random.default_rng(seed)
    for _ in range(30):
        kind = int(rng.integers(0, 3))
        if kind == 0:
            decode_case(rng, 9000)
        elif kind == 1:
            chunk_case(rng, 3000, 700)
        else:
            verify_case(rng, 5000, 12)
    torch.cuda.synchronize()
    assert decode.device_error() == 0


@pytest.mark.parametrize("seed", [11, 12])
def test_random_large_shapes(seed):
    """Cache lengths past 32k, chunks of several query tiles, draft counts whose
    rows exceed one 128-row tile (the row-block kernel takes those)."""
    rng = np.random.default_rng(seed)
    for _ in range(15):
        kind = int(rng.integers(0, 3))
        if kind == 0:
            decode_case(rng, 40000)
        elif kind == 1:
            chunk_case(rng, 9000, 1500)
        else:
            verify_case(rng, 17000, 40)
    torch.cuda.synchronize()
    assert decode.device_error() == 0
