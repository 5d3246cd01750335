"""The reference's own kernel tests for this path, restated against this
library's C ABI through the decode/chunk wrappers:

  crates/whetstone-kernels/tests/decode_kernels.rs:91-410
  crates/whetstone-kernels/tests/chunk_kernels.rs:263-360

Same inputs (closed-form sequences and the LCG), same tolerances."""

import numpy as np
import pytest
import torch

from oracle import attention_oracle as orc
from tests.helpers import dev, host
from whetstone_b200 import chunk, decode
from whetstone_b200._ffi import check, lib

pytestmark = pytest.mark.gpu


@pytest.fixture(params=[0, 1], ids=["auto", "portable"])
def kernel_choice(request):
    check(lib.wst_b200_set_kernel_choice(request.param))
    yield request.param
    check(lib.wst_b200_set_kernel_choice(0))


def seq_f32(n, mod, div):
    return np.array([(i % mod) / div - 1.0 for i in range(n)], dtype=np.float32)


def test_rope_uses_the_half_rotation_layout():
    n_q, n_kv, hd, max_seq, pos, theta = 2, 1, 64, 8, 3, 1e6
    q, k, v = seq_f32(n_q * hd, 31, 15.0), seq_f32(n_kv * hd, 23, 11.0), seq_f32(n_kv * hd, 19, 9.0)
    table = decode.RopeTable(max_seq, hd, theta)
    cache = decode.KvCache(n_kv, n_q, hd, max_seq)
    qd = dev(np.concatenate([q, k, v]))
    decode.rope_cache(qd, cache, table, n_q, decode.DeviceCursor(pos))
    got = host(qd)
    half = hd // 2
    for h in range(n_q):
        for j in range(half):
            inv = theta ** (-j / half)
            s, c = np.sin(pos * inv), np.cos(pos * inv)
            x1, x2 = float(q[h * hd + j]), float(q[h * hd + j + half])
            assert abs(got[h * hd + j] - np.float32(x1 * c - x2 * s)) < 1e-5
            assert abs(got[h * hd + j + half] - np.float32(x2 * c + x1 * s)) < 1e-5


def test_qk_norm_is_per_head_and_precedes_the_rotation():
    n_q, n_kv, hd, max_seq, pos, theta, eps = 4, 2, 64, 8, 5, 1e6, 1e-6
    q, k, v = seq_f32(n_q * hd, 31, 15.0), seq_f32(n_kv * hd, 23, 11.0), seq_f32(n_kv * hd, 19, 9.0)
    gq = np.array([0.5 + (i % 7) * 0.1 for i in range(hd)], dtype=np.float32)
    gk = np.array([1.5 - (i % 5) * 0.2 for i in range(hd)], dtype=np.float32)
    table = decode.RopeTable(max_seq, hd, theta)
    cache = decode.KvCache(n_kv, n_q, hd, max_seq)
    qd = dev(np.concatenate([q, k, v]))
    norm = decode.QkNorm(dev(gq.astype(np.float16)), dev(gk.astype(np.float16)), eps)
    decode.rope_cache(qd, cache, table, n_q, decode.DeviceCursor(pos), norm)
    got = host(qd)
    qr, kr, _ = orc.rope_append(np.concatenate([q, k, v])[None], np.array([pos]), n_q, n_kv, hd,
                                theta, gq, gk, eps)
    want_q = qr[0].reshape(-1)
    tol = 1e-4 * np.maximum(np.abs(want_q), 1.0)
    assert np.all(np.abs(got[: n_q * hd] - want_q) < tol)
    kc = host(cache.keys()).astype(np.float64)
    vc = host(cache.values()).astype(np.float64)
    for h in range(n_kv):
        assert np.all(np.abs(kc[h, pos] - kr[0, h]) < 3e-3), f"k head {h}"
        assert np.all(np.abs(vc[h, pos] - v[h * hd:(h + 1) * hd]) < 3e-3), f"v head {h} modified"


def test_qk_norm_with_unit_gain_on_a_unit_rms_head_is_the_identity():
    n_q, n_kv, hd, max_seq, pos = 2, 1, 64, 8, 2
    q = np.array([-1.0 if i % 3 == 0 else 1.0 for i in range(n_q * hd)], dtype=np.float32)
    k = np.array([-1.0 if i % 5 == 0 else 1.0 for i in range(n_kv * hd)], dtype=np.float32)
    v = seq_f32(n_kv * hd, 19, 9.0)
    ones = dev(np.ones(hd, dtype=np.float16))
    table = decode.RopeTable(max_seq, hd, 1e6)
    qkv = np.concatenate([q, k, v])
    cur = decode.DeviceCursor(pos)
    off = dev(qkv)
    decode.rope_cache(off, decode.KvCache(n_kv, n_q, hd, max_seq), table, n_q, cur)
    on = dev(qkv)
    decode.rope_cache(on, decode.KvCache(n_kv, n_q, hd, max_seq), table, n_q, cur,
                      decode.QkNorm(ones, ones.clone(), 0.0))
    assert np.all(np.abs(host(off) - host(on)) < 1e-6)


def test_attention_over_one_position_returns_that_value(kernel_choice):
    n_q, n_kv, hd, max_seq = 14, 2, 64, 32
    table = decode.RopeTable(max_seq, hd, 1e6)
    cache = decode.KvCache(n_kv, n_q, hd, max_seq)
    q, k, v = seq_f32(n_q * hd, 29, 14.0), seq_f32(n_kv * hd, 13, 6.0), seq_f32(n_kv * hd, 17, 8.0)
    qd = dev(np.concatenate([q, k, v]))
    cur = decode.DeviceCursor(0)
    decode.rope_cache(qd, cache, table, n_q, cur)
    out = torch.zeros(n_q * hd, dtype=torch.float16, device="cuda")
    decode.attn_decode(qd, cache, out, n_q, cur)
    got = host(out).astype(np.float32)
    for h in range(n_q):
        want = v[(h // 7) * hd:(h // 7 + 1) * hd].astype(np.float16).astype(np.float32)
        assert np.all(np.abs(got[h * hd:(h + 1) * hd] - want) < 2e-3), f"head {h}"


def test_attention_over_two_positions_matches_an_explicit_softmax(kernel_choice):
    n_q, n_kv, hd, max_seq, theta = 2, 1, 64, 16, 1e6
    cache = decode.KvCache(n_kv, n_q, hd, max_seq)
    table = decode.RopeTable(max_seq, hd, theta)
    ks, vs = [], []
    for p in range(2):
        k = np.array([((i + 7 * p) % 11) / 5.0 - 1.0 for i in range(hd)], dtype=np.float32)
        v = np.array([((i + 3 * p) % 7) / 3.0 - 1.0 for i in range(hd)], dtype=np.float32)
        qd = dev(np.concatenate([np.zeros(n_q * hd, np.float32), k, v]))
        decode.rope_cache(qd, cache, table, n_q, decode.DeviceCursor(p))
        kr = orc.rope(k.astype(np.float64)[None, None], np.array([p]), theta)[0, 0]
        ks.append(kr.astype(np.float32).astype(np.float16).astype(np.float64))
        vs.append(v.astype(np.float16).astype(np.float64))
    q = np.array([(i % 5) / 2.0 - 1.0 for i in range(n_q * hd)], dtype=np.float32)
    out = torch.zeros(n_q * hd, dtype=torch.float16, device="cuda")
    decode.attn_decode(dev(q), cache, out, n_q, decode.DeviceCursor(1))
    got = host(out).astype(np.float64)
    for h in range(n_q):
        s = np.array([q[h * hd:(h + 1) * hd].astype(np.float64) @ ks[p] for p in range(2)]) / 8.0
        e = np.exp(s - s.max())
        want = (e[0] * vs[0] + e[1] * vs[1]) / e.sum()
        assert np.all(np.abs(got[h * hd:(h + 1) * hd] - want) < 3e-3), f"head {h}"


def _close(got, want, tol, what):
    bound = tol * np.maximum(np.abs(want), 1.0)
    bad = np.abs(got - want) > bound
    assert not bad.any(), f"{what}: {int(bad.sum())} elements off, worst {np.abs(got - want).max()}"


def _sequential(qkv_rows, cache, table, n_q, positions):
    outs = []
    hd = cache.head_dim
    cur = decode.DeviceCursor(0)
    for row, p in zip(qkv_rows, positions):
        cur.set(int(p))
        q1 = dev(row)
        decode.rope_cache(q1, cache, table, n_q, cur)
        o1 = torch.zeros(n_q * hd, dtype=torch.float16, device="cuda")
        decode.attn_decode(q1, cache, o1, n_q, cur)
        outs.append(host(o1).astype(np.float32))
    return np.stack(outs)


def test_rope_and_attention_chunk_match_sequential_decode(kernel_choice):
    n_q, n_kv, hd, max_seq, n = 14, 2, 64, 128, 9
    stride = (n_q + 2 * n_kv) * hd
    table = decode.RopeTable(max_seq, hd, 1e6)
    qkv_all = orc.lcg_noise(stride * n, 303).reshape(n, stride)
    cache_a = decode.KvCache(n_kv, n_q, hd, max_seq)
    qkv_c = dev(qkv_all)
    chunk.rope_cache(qkv_c, cache_a, table, n_q, 0, n)
    out_c = torch.zeros(n * n_q * hd, dtype=torch.float16, device="cuda")
    chunk.attn(qkv_c, cache_a, out_c, n_q, 0, n)
    got = host(out_c).astype(np.float32).reshape(n, n_q * hd)
    cache_b = decode.KvCache(n_kv, n_q, hd, max_seq)
    want = _sequential(qkv_all, cache_b, table, n_q, range(n))
    _close(got, want, 4e-3, "attention token")
    assert torch.equal(cache_a.k, cache_b.k) and torch.equal(cache_a.v, cache_b.v)


def test_attention_chunk_resumes_mid_cache(kernel_choice):
    n_q, n_kv, hd, max_seq, prefix, n = 14, 2, 64, 128, 20, 5
    stride = (n_q + 2 * n_kv) * hd
    table = decode.RopeTable(max_seq, hd, 1e6)
    qkv_all = orc.lcg_noise(stride * (prefix + n), 404).reshape(prefix + n, stride)
    cache_a = decode.KvCache(n_kv, n_q, hd, max_seq)
    cache_b = decode.KvCache(n_kv, n_q, hd, max_seq)
    cur = decode.DeviceCursor(0)
    for j in range(prefix):
        cur.set(j)
        for cache in (cache_a, cache_b):
            decode.rope_cache(dev(qkv_all[j]), cache, table, n_q, cur)
    tail = qkv_all[prefix:]
    qkv_c = dev(tail)
    chunk.rope_cache(qkv_c, cache_a, table, n_q, prefix, n)
    out_c = torch.zeros(n * n_q * hd, dtype=torch.float16, device="cuda")
    chunk.attn(qkv_c, cache_a, out_c, n_q, prefix, n)
    got = host(out_c).astype(np.float32).reshape(n, n_q * hd)
    want = _sequential(tail, cache_b, table, n_q, range(prefix, prefix + n))
    _close(got, want, 4e-3, "resumed attention token")
