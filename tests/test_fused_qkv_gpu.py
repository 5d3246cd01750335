"""wst_b200_qkv_rope_append_batch (the qkv projection with RoPE, head norm and cache
append in its epilogue) and wst_b200_attn_chunk_batch_q16, against the oracle --
exact fp64 projection (oracle.gemm_fp16, cuda/chunk_gemm.cu:184-258), then the RoPE /
norm / append of cuda/chunk_ops.cu:101-181 (oracle.rope_append), then the attention of
cuda/chunk_ops.cu:187-264 -- and against this library's own two-launch chain
(wst_gemm_fp16 + wst_rope_cache_chunk_batch + wst_attn_chunk_batch).

q, k and v come out of an fp32 tensor-core accumulation here where the oracle sums in
fp64, so a stored fp16 value may sit on the neighbouring fp16 number, and a value that
is tiny next to the row's terms carries the sum's absolute error (2e-4 at contraction
length 512 with unit-scale terms)."""

import numpy as np
import pytest
import torch

from oracle import attention_oracle as orc
from tests.helpers import NAN16, assert_close_per_head, bits16, dev, f16_ulp_distance, fill_bits, host
from whetstone_b200 import chunk, decode

pytestmark = pytest.mark.gpu


def assert_half_rows(got_bits, want_f64, what):
    want_bits = want_f64.astype(np.float16).view(np.uint16)
    ulp = f16_ulp_distance(got_bits, want_bits)
    diff = np.abs(got_bits.view(np.float16).astype(np.float64) - want_f64)
    bad = (ulp > 1) & (diff > 2e-4)
    assert not bad.any(), f"{what}: {int(bad.sum())} values off; worst {diff[bad].max():.3e}"


@pytest.mark.parametrize("n_seq,n,in_f,n_q,n_kv,hd,gains,bias", [
    (2, 130, 512, 4, 2, 128, True, True),     # ragged second token tile, gains and bias
    (3, 70, 256, 8, 2, 64, False, False),     # head_dim 64: four heads per feature tile
    (1, 300, 1000, 6, 3, 128, True, False),   # in_f not a multiple of 64, odd head counts
    (4, 64, 128, 2, 1, 64, True, True),       # feature tile wider than the qkv row (256 > 4 * 64)
])
def test_fused_projection_against_the_oracle(n_seq, n, in_f, n_q, n_kv, hd, gains, bias):
    rng = np.random.default_rng(n * 7 + in_f)
    width = (n_q + 2 * n_kv) * hd
    theta, eps, max_seq = 1e6, 1e-6, 600
    w = (rng.standard_normal((width, in_f)) / np.sqrt(in_f)).astype(np.float16)
    x = rng.standard_normal((n_seq * n, in_f)).astype(np.float16)
    b = (0.1 * rng.standard_normal(width)).astype(np.float16) if bias else None
    gq = (1 + 0.1 * rng.standard_normal(hd)).astype(np.float16) if gains else None
    gk = (1 + 0.1 * rng.standard_normal(hd)).astype(np.float16) if gains else None
    starts_np = rng.integers(0, max_seq - n, size=n_seq).astype(np.int32)
    table = decode.RopeTable(max_seq, hd, theta)
    cache = chunk.KvCacheBatch(n_seq, n_kv, hd, max_seq)
    fill_bits(cache.k, NAN16)
    fill_bits(cache.v, NAN16)
    q16 = torch.zeros((n_seq * n, n_q * hd), dtype=torch.float16, device="cuda")
    norm = decode.QkNorm(dev(gq), dev(gk), eps) if gains else None
    starts = dev(starts_np)
    chunk.qkv_rope_append_batch(dev(w), dev(x), dev(b) if bias else None, q16, cache, table, n_q,
                                starts, n, norm)
    torch.cuda.synchronize()
    assert decode.device_error() == 0

    y = orc.gemm_fp16(w, x, b)
    k_bits, v_bits = bits16(cache.k), bits16(cache.v)
    for s in range(n_seq):
        pos = starts_np[s] + np.arange(n)
        q_rot, k_rot, v = orc.rope_append(y[s * n:(s + 1) * n], pos, n_q, n_kv, hd, theta, gq, gk, eps)
        assert_half_rows(bits16(q16[s * n:(s + 1) * n]).reshape(n, n_q, hd), q_rot, f"q, sequence {s}")
        assert_half_rows(k_bits[s][:, pos], k_rot.transpose(1, 0, 2), f"k, sequence {s}")
        assert_half_rows(v_bits[s][:, pos], v.transpose(1, 0, 2), f"v, sequence {s}")
        untouched = np.ones(max_seq, dtype=bool)
        untouched[pos] = False
        assert (k_bits[s][:, untouched] == NAN16).all() and (v_bits[s][:, untouched] == NAN16).all()


def test_fused_chain_agrees_with_the_two_launch_chain_and_the_oracle():
    """One chunk step of a c4-shaped layer at reduced size: 2 sequences x 256 tokens at
    cache row 384, 8 q / 2 kv heads of 128, hidden 1024, QK-norm."""
    n_seq, n, in_f, n_q, n_kv, hd, pos0, max_seq = 2, 256, 1024, 8, 2, 128, 384, 640
    theta, eps = 1e6, 1e-6
    width = (n_q + 2 * n_kv) * hd
    rng = np.random.default_rng(99)
    w = (rng.standard_normal((width, in_f)) / np.sqrt(in_f)).astype(np.float16)
    x = rng.standard_normal((n_seq * n, in_f)).astype(np.float16)
    gq = (1 + 0.05 * rng.standard_normal(hd)).astype(np.float16)
    gk = (1 + 0.05 * rng.standard_normal(hd)).astype(np.float16)
    prefix_k = (0.5 * rng.standard_normal((n_seq, n_kv, pos0, hd))).astype(np.float16)
    prefix_v = rng.standard_normal((n_seq, n_kv, pos0, hd)).astype(np.float16)
    table = decode.RopeTable(max_seq, hd, theta)
    norm = decode.QkNorm(dev(gq), dev(gk), eps)
    starts = torch.full((n_seq,), pos0, dtype=torch.int32, device="cuda")
    wd, xd = dev(w), dev(x)

    def fresh():
        c = chunk.KvCacheBatch(n_seq, n_kv, hd, max_seq)
        fill_bits(c.k, NAN16)
        fill_bits(c.v, NAN16)
        c.k[:, :, :pos0] = dev(prefix_k)
        c.v[:, :, :pos0] = dev(prefix_v)
        return c

    fused, plain = fresh(), fresh()
    q16 = torch.zeros((n_seq * n, n_q * hd), dtype=torch.float16, device="cuda")
    out_f = torch.zeros(n_seq * n * n_q * hd, dtype=torch.float16, device="cuda")
    chunk.qkv_rope_append_batch(wd, xd, None, q16, fused, table, n_q, starts, n, norm)
    chunk.attn_batch_q16(q16, fused, out_f, n_q, starts, n)

    y = torch.zeros((n_seq * n, width), dtype=torch.float32, device="cuda")
    out_p = torch.zeros_like(out_f)
    chunk.gemm_fp16(wd, xd, None, y, in_f, width, n_seq * n)
    chunk.rope_cache_batch(y, plain, table, n_q, starts, n, norm)
    chunk.attn_batch(y, plain, out_p, n_q, starts, n)
    torch.cuda.synchronize()
    assert decode.device_error() == 0

    # the caches of the two chains: the same values up to the fp16 neighbour
    for a_, b_ in ((fused.k, plain.k), (fused.v, plain.v)):
        ulp = f16_ulp_distance(bits16(a_[:, :, : pos0 + n]), bits16(b_[:, :, : pos0 + n]))
        assert ulp.max() <= 1
    got_f = host(out_f).astype(np.float64).reshape(n_seq, n, n_q, hd)
    got_p = host(out_p).astype(np.float64).reshape(n_seq, n, n_q, hd)
    y64 = orc.gemm_fp16(w, x)
    for s in range(n_seq):
        q_rot, k_rot, v = orc.rope_append(y64[s * n:(s + 1) * n], pos0 + np.arange(n), n_q, n_kv, hd,
                                          theta, gq, gk, eps)
        k_all = np.concatenate([prefix_k[s].astype(np.float64).transpose(1, 0, 2), k_rot])
        v_all = np.concatenate([prefix_v[s].astype(np.float64).transpose(1, 0, 2), v])
        want = orc.attention_blocked(q_rot, k_all, v_all, pos0 + 1 + np.arange(n), 1.0 / np.sqrt(hd))
        assert_close_per_head(got_f[s], want, f"fused chain, sequence {s}")
        assert_close_per_head(got_p[s], want, f"two-launch chain, sequence {s}")


def test_q16_needs_the_tensor_core_kernels():
    cache = chunk.KvCacheBatch(1, 2, 128, 64)
    q16 = torch.zeros((4, 4 * 128), dtype=torch.float16, device="cuda")
    out = torch.zeros(4 * 4 * 128, dtype=torch.float16, device="cuda")
    starts = torch.zeros(1, dtype=torch.int32, device="cuda")
    with pytest.raises(Exception) as err:
        chunk.attn_batch_q16(q16, cache, out, 4, starts, 4)
    assert "fp16 query rows" in str(err.value)


def test_fused_projection_with_int4_weights():
    """wst_b200_qkv_int4_rope_append_batch against the oracle: dequantized weights
    (cuda/hier.cuh:8-13) -> exact projection -> RoPE / norm / append."""
    from tests.test_gemm_int4_gpu import fast_packed_weights
    n_seq, n, in_f, n_q, n_kv, hd, max_seq = 2, 140, 512, 4, 2, 128, 400
    theta, eps = 1e6, 1e-6
    width = (n_q + 2 * n_kv) * hd
    rng = np.random.default_rng(41)
    qw, si, sb = fast_packed_weights(in_f, width, 41)
    x = rng.uniform(-1, 1, (n_seq * n, in_f)).astype(np.float16)
    gq = (1 + 0.1 * rng.standard_normal(hd)).astype(np.float16)
    gk = (1 + 0.1 * rng.standard_normal(hd)).astype(np.float16)
    starts_np = np.array([7, 200], dtype=np.int32)
    table = decode.RopeTable(max_seq, hd, theta)
    cache = chunk.KvCacheBatch(n_seq, n_kv, hd, max_seq)
    fill_bits(cache.k, NAN16)
    fill_bits(cache.v, NAN16)
    q16 = torch.zeros((n_seq * n, n_q * hd), dtype=torch.float16, device="cuda")
    chunk.qkv_int4_rope_append_batch(dev(qw.view(np.int32)), dev(si), dev(sb.view(np.float16)), dev(x),
                                     None, q16, cache, table, n_q, dev(starts_np), n,
                                     decode.QkNorm(dev(gq), dev(gk), eps))
    torch.cuda.synchronize()
    assert decode.device_error() == 0
    y = orc.gemm_int4_hier(qw, si, sb, x, in_f, width)
    k_bits, v_bits = bits16(cache.k), bits16(cache.v)
    for s in range(n_seq):
        pos = starts_np[s] + np.arange(n)
        q_rot, k_rot, v = orc.rope_append(y[s * n:(s + 1) * n], pos, n_q, n_kv, hd, theta, gq, gk, eps)
        # the weights are rounded to fp16 once (3e-3 of the engine's test at this length)
        for got, want, what in ((bits16(q16[s * n:(s + 1) * n]).reshape(n, n_q, hd), q_rot, "q"),
                                (k_bits[s][:, pos], k_rot.transpose(1, 0, 2), "k"),
                                (v_bits[s][:, pos], v.transpose(1, 0, 2), "v")):
            diff = np.abs(got.view(np.float16).astype(np.float64) - want)
            assert (diff <= 3e-3 * np.maximum(np.abs(want), 1.0)).all(), f"{what}, sequence {s}: {diff.max()}"
