"""8-bit KV cache: wst_b200_rope_cache_fp8 and wst_b200_attn_decode_fp8.

The append is checked against the oracle's RoPE / norm (cuda/decode.cu:112-178) followed by
the oracle's e4m3 rounding (nearest, ties to even, saturating: oracle.e4m3_quantize, itself
checked against torch's float8_e4m3fn in the CPU suite): V bytes exact with a power-of-two
scale, K bytes equal or adjacent (the device rotates in fp32).  The attention is checked
against the oracle's attention (cuda/attention.cu:57-193) over the dequantized bytes the
cache really holds, with the bar of the fp16 path (2e-3 absolute, cosine 0.9999 per head):
every e4m3 number is an fp16 number, so nothing but the cache's contents differs."""

import numpy as np
import pytest
import torch

from oracle import attention_oracle as orc
from tests.helpers import assert_close_per_head, dev, host
from whetstone_b200 import decode
from whetstone_b200._ffi import ShapeError

pytestmark = pytest.mark.gpu


def random_e4m3(rng, shape, scale):
    """Unit-variance values as the e4m3 bytes a cache with this scale would hold."""
    return orc.e4m3_quantize(rng.standard_normal(shape) / scale)


@pytest.fixture(params=[1, 2], ids=["row-block kernel", "tensor-memory kernel"])
def fp8_kernel(request):
    """Both decode kernels of the e4m3 cache, whatever the cache's capacity would pick."""
    decode.set_tuning(6, request.param)
    yield request.param
    decode.set_tuning(6, 0)


@pytest.mark.parametrize("n_q,n_kv", [(28, 4), (8, 8), (32, 2)])
@pytest.mark.parametrize("seq", [1, 17, 128, 129, 1000, 4097, 20000])
def test_decode_over_an_fp8_cache(n_q, n_kv, seq, fp8_kernel):
    run_decode_case(n_q, n_kv, seq, seq + 7)


@pytest.mark.parametrize("seq,max_seq", [(300, 50000), (1, 12288), (12287, 12287), (70000, 70016), (16385, 40000)])
def test_decode_picks_a_kernel_by_capacity(seq, max_seq):
    """No tuning: the capacity decides, and slices past the live rows hold nothing."""
    run_decode_case(28, 4, seq, max_seq)


def test_sixteen_heads_per_kv_head(fp8_kernel):
    run_decode_case(16, 1, 2500, 2560)


def run_decode_case(n_q, n_kv, seq, max_seq):
    hd = 128
    rng = np.random.default_rng(seq * 31 + n_q)
    cache = decode.KvCacheFp8(n_kv, n_q, hd, max_seq, k_scale=0.0625, v_scale=0.5)
    kb = random_e4m3(rng, (n_kv, max_seq, hd), cache.k_scale)
    vb = random_e4m3(rng, (n_kv, max_seq, hd), cache.v_scale)
    kb[:, seq:] = 0x7F                    # rows past the live data hold NaN: nothing may read them
    vb[:, seq:] = 0x7F
    cache.k.copy_(dev(kb))
    cache.v.copy_(dev(vb))
    q = rng.standard_normal(n_q * hd).astype(np.float32)
    out = torch.zeros(n_q * hd, dtype=torch.float16, device="cuda")
    decode.attn_decode_fp8(dev(q), cache, out, n_q, decode.DeviceCursor(seq - 1))
    torch.cuda.synchronize()
    assert decode.device_error() == 0
    k = orc.e4m3_dequantize(kb[:, :seq], cache.k_scale)
    v = orc.e4m3_dequantize(vb[:, :seq], cache.v_scale)
    want = orc.decode_attention(q.reshape(n_q, hd), k, v, seq)
    assert_close_per_head(host(out).astype(np.float64).reshape(n_q, hd), want, f"fp8 decode, seq {seq}")


@pytest.mark.parametrize("gains", [False, True])
def test_append_into_an_fp8_cache(gains):
    n_q, n_kv, hd, max_seq, theta, eps = 8, 2, 128, 96, 1e6, 1e-6
    rng = np.random.default_rng(5)
    table = decode.RopeTable(max_seq, hd, theta)
    cache = decode.KvCacheFp8(n_kv, n_q, hd, max_seq, k_scale=0.25, v_scale=0.5)
    cache.k.fill_(0x7F)
    cache.v.fill_(0x7F)
    gq = (1 + 0.1 * rng.standard_normal(hd)).astype(np.float16) if gains else None
    gk = (1 + 0.1 * rng.standard_normal(hd)).astype(np.float16) if gains else None
    norm = decode.QkNorm(dev(gq), dev(gk), eps) if gains else None
    # a chunk of 40 tokens at row 3, then one token at the cursor
    n, pos0 = 40, 3
    qkv = (3 * rng.standard_normal((n + 1, (n_q + 2 * n_kv) * hd))).astype(np.float32)
    qd = dev(qkv[:n].copy())
    decode.rope_cache_fp8(qd, cache, table, n_q, pos0=pos0, n=n, qk_norm=norm)
    q1 = dev(qkv[n].copy())
    decode.rope_cache_fp8(q1, cache, table, n_q, pos=decode.DeviceCursor(pos0 + n), qk_norm=norm)
    torch.cuda.synchronize()
    pos = pos0 + np.arange(n + 1)
    q_rot, k_rot, v = orc.rope_append(qkv, pos, n_q, n_kv, hd, theta, gq, gk, eps)
    got_q = np.concatenate([host(qd), host(q1)[None, :]])[:, : n_q * hd].reshape(n + 1, n_q, hd)
    np.testing.assert_allclose(got_q, q_rot, rtol=0, atol=2e-5)
    kb, vb = host(cache.k), host(cache.v)
    want_v = orc.e4m3_quantize(v.transpose(1, 0, 2) / cache.v_scale)
    assert np.array_equal(vb[:, pos], want_v)
    want_k = orc.e4m3_quantize(k_rot.transpose(1, 0, 2) / cache.k_scale)
    step = np.abs((kb[:, pos] & 0x7F).astype(int) - (want_k & 0x7F).astype(int))
    assert step.max() <= 1 and (step > 0).mean() < 0.01
    assert ((kb[:, pos] ^ want_k) & 0x80)[step == 0].max() == 0      # signs agree where magnitudes do
    untouched = np.ones(max_seq, dtype=bool)
    untouched[pos] = False
    assert (kb[:, untouched] == 0x7F).all() and (vb[:, untouched] == 0x7F).all()


def test_decode_steps_through_both_entry_points(fp8_kernel):
    """Append + attend for a few tokens, the oracle reading back what the cache holds."""
    n_q, n_kv, hd, max_seq, theta = 28, 4, 128, 300, 1e6
    rng = np.random.default_rng(9)
    table = decode.RopeTable(max_seq, hd, theta)
    cache = decode.KvCacheFp8(n_kv, n_q, hd, max_seq, k_scale=0.125, v_scale=0.0625)
    start = 257
    cache.k[:, :start] = dev(random_e4m3(rng, (n_kv, start, hd), cache.k_scale))
    cache.v[:, :start] = dev(random_e4m3(rng, (n_kv, start, hd), cache.v_scale))
    cur = decode.DeviceCursor(start)
    out = torch.zeros(n_q * hd, dtype=torch.float16, device="cuda")
    for step in range(4):
        qkv = dev(rng.standard_normal((n_q + 2 * n_kv) * hd).astype(np.float32))
        decode.rope_cache_fp8(qkv, cache, table, n_q, pos=cur)
        decode.attn_decode_fp8(qkv, cache, out, n_q, cur)
        torch.cuda.synchronize()
        seq = start + step + 1
        k = orc.e4m3_dequantize(host(cache.k)[:, :seq], cache.k_scale)
        v = orc.e4m3_dequantize(host(cache.v)[:, :seq], cache.v_scale)
        want = orc.decode_attention(host(qkv)[: n_q * hd].reshape(n_q, hd), k, v, seq)
        assert_close_per_head(host(out).astype(np.float64).reshape(n_q, hd), want, f"step {step}")
        cur.advance(max_seq)
    assert decode.device_error() == 0


def test_the_row_just_appended_is_the_row_attended_to(fp8_kernel):
    """The attention may request its tiles while the append ahead of it is still running;
    whatever it fetched that early, the newest row must be the appended one.  Queries
    aligned with the new key put nearly all of the weight on that row, so a stale copy
    (the zeros the row held before) would show in every head."""
    n_q, n_kv, hd, max_seq, theta = 28, 4, 128, 8300, 1e6
    rng = np.random.default_rng(21)
    table = decode.RopeTable(max_seq, hd, theta)
    cache = decode.KvCacheFp8(n_kv, n_q, hd, max_seq, k_scale=0.0625, v_scale=0.0625)
    start = 8100
    cache.k[:, :start] = dev(random_e4m3(rng, (n_kv, start, hd), cache.k_scale * 4))   # small keys
    cache.v[:, :start] = dev(random_e4m3(rng, (n_kv, start, hd), cache.v_scale))
    cur = decode.DeviceCursor(start)
    out = torch.zeros(n_q * hd, dtype=torch.float16, device="cuda")
    group = n_q // n_kv
    for step in range(8):
        k_new = rng.standard_normal((n_kv, hd)).astype(np.float32)
        v_new = rng.standard_normal((n_kv, hd)).astype(np.float32)
        q = np.repeat(k_new, group, axis=0) * 3.0            # head h looks for its group's new key
        qkv = dev(np.concatenate([q.reshape(-1), k_new.reshape(-1), v_new.reshape(-1)]))
        decode.rope_cache_fp8(qkv, cache, table, n_q, pos=cur)   # no synchronisation in between
        decode.attn_decode_fp8(qkv, cache, out, n_q, cur)
        torch.cuda.synchronize()
        seq = start + step + 1
        k = orc.e4m3_dequantize(host(cache.k)[:, :seq], cache.k_scale)
        v = orc.e4m3_dequantize(host(cache.v)[:, :seq], cache.v_scale)
        got = host(out).astype(np.float64).reshape(n_q, hd)
        want = orc.decode_attention(host(qkv)[: n_q * hd].reshape(n_q, hd), k, v, seq)
        assert_close_per_head(got, want, f"step {step}")
        newest = np.repeat(v[:, seq - 1], group, axis=0)
        assert np.abs(got - newest).max() < 0.05, "the output is the appended value row"
        cur.advance(max_seq)
    assert decode.device_error() == 0


def test_shapes_the_fp8_path_does_not_take():
    cache = decode.KvCacheFp8(2, 4, 64, 32)
    out = torch.zeros(4 * 64, dtype=torch.float16, device="cuda")
    q = torch.zeros(4 * 64, dtype=torch.float32, device="cuda")
    with pytest.raises(ShapeError):
        decode.attn_decode_fp8(q, cache, out, 4, decode.DeviceCursor(3))
