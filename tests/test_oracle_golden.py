"""Pins oracle/attention_oracle.py (CPU only).

1. Against tests/golden/reference_numpy_vectors.npz, which make_golden.py
   produced by running the reference's own rope / softmax / rms_norm and its
   attention statements (bench/reference_numpy.py:74-117, 170-181).
2. Against the closed forms used by the reference's kernel tests
   (crates/whetstone-kernels/tests/decode_kernels.rs:91-410).
"""

from pathlib import Path

import numpy as np
import pytest

from oracle import attention_oracle as orc

GOLD = np.load(Path(__file__).parent / "golden" / "reference_numpy_vectors.npz")


@pytest.mark.parametrize("tag", ["rope_a", "rope_b"])
def test_rope_matches_reference(tag):
    y = orc.rope(GOLD[f"{tag}_x"], GOLD[f"{tag}_pos"], float(GOLD[f"{tag}_theta"]))
    np.testing.assert_allclose(y, GOLD[f"{tag}_y"], rtol=0, atol=1e-12)


def test_rms_norm_matches_reference():
    y = orc.rms_norm(GOLD["norm_x"], GOLD["norm_w"], float(GOLD["norm_eps"]))
    np.testing.assert_allclose(y, GOLD["norm_y"], rtol=0, atol=1e-14)


def test_softmax_matches_reference():
    y = orc.softmax(GOLD["softmax_x"], axis=-1)
    np.testing.assert_allclose(y, GOLD["softmax_y"], rtol=0, atol=1e-15)
    assert np.all(y[:, :, 6:] == 0.0)


@pytest.mark.parametrize("tag", ["attn_q14", "attn_q8"])
def test_causal_attention_matches_reference(tag):
    seq, n_q, n_kv, hd = (int(x) for x in GOLD[f"{tag}_shape"])
    theta = float(GOLD[f"{tag}_theta"])
    q = GOLD[f"{tag}_q"].astype(np.float64)
    k = GOLD[f"{tag}_k"].astype(np.float64)
    v = GOLD[f"{tag}_v"].astype(np.float64)
    qkv = np.concatenate([q, k, v], axis=1)
    pos = np.arange(seq)
    qr, kr, vv = orc.rope_append(qkv, pos, n_q, n_kv, hd, theta)
    np.testing.assert_allclose(qr, GOLD[f"{tag}_qrot"], rtol=0, atol=1e-12)
    np.testing.assert_allclose(kr, GOLD[f"{tag}_krot"], rtol=0, atol=1e-12)
    want = GOLD[f"{tag}_ctx"].reshape(seq, n_q, hd)
    for fn in (orc.attention, orc.attention_blocked):
        got = fn(qr, kr, vv, pos + 1)
        np.testing.assert_allclose(got, want, rtol=0, atol=1e-12)
    # the cache-shaped helpers are the same math on [n_kv][pos][hd] arrays
    kc = kr.transpose(1, 0, 2)
    vc = vv.transpose(1, 0, 2)
    np.testing.assert_allclose(orc.chunk_attention(qr, kc, vc, 0), want, rtol=0, atol=1e-12)
    np.testing.assert_allclose(orc.decode_attention(qr[-1], kc, vc, seq), want[-1], rtol=0,
                               atol=1e-12)


def test_attention_resumes_mid_cache():
    """pos0 != 0: rows of a later chunk against the whole-prompt result."""
    seq, n_q, n_kv, hd = (int(x) for x in GOLD["attn_q8_shape"])
    qr, kr = GOLD["attn_q8_qrot"], GOLD["attn_q8_krot"]
    v = GOLD["attn_q8_v"].astype(np.float64).reshape(seq, n_kv, hd)
    want = GOLD["attn_q8_ctx"].reshape(seq, n_q, hd)
    got = orc.chunk_attention(qr[7:], kr.transpose(1, 0, 2), v.transpose(1, 0, 2), 7)
    np.testing.assert_allclose(got, want[7:], rtol=0, atol=1e-12)


def test_rope_table_is_the_f64_rotation_in_f32():
    """decode.rs:95-147: angles in f64, stored fp32; rope() and the table agree."""
    cos, sin = orc.rope_table(40, 64, 1e6)
    assert cos.dtype == np.float32 and cos.shape == (40, 32)
    x = np.random.default_rng(3).standard_normal((5, 2, 64))
    pos = np.array([0, 3, 17, 38, 39])
    np.testing.assert_allclose(orc.rope_from_table(x, pos, cos, sin), orc.rope(x, pos, 1e6),
                               rtol=0, atol=1e-6)


def test_rope_table_llama3_schedule():
    """High frequencies untouched, low ones divided by `factor`, a blend between."""
    sc = dict(factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0, original_max_position=8192)
    half = 64
    plain = np.power(5e5, -np.arange(half) / half)
    cos, sin = orc.rope_table(2, 128, 5e5, llama3=sc)
    inv = np.arctan2(sin[1].astype(np.float64), cos[1].astype(np.float64))  # angle at pos 1
    wl = 2 * np.pi / plain
    hi = wl < 8192 / 4.0
    lo = wl > 8192 / 1.0
    assert hi.any() and lo.any() and (~hi & ~lo).any()
    np.testing.assert_allclose(inv[hi & (plain < 3)], plain[hi & (plain < 3)], rtol=1e-6)
    np.testing.assert_allclose(inv[lo], plain[lo] / 8.0, rtol=1e-5, atol=1e-9)
    mid = ~hi & ~lo
    assert np.all(inv[mid] < plain[mid] * (1 + 1e-6)) and np.all(inv[mid] > plain[mid] / 8.0 * (1 - 1e-6))


def test_half_rotation_closed_form():
    """decode_kernels.rs:91-126: pairs are (j, j+half), angle pos*theta^(-j/half)."""
    n_q, n_kv, hd, pos, theta = 2, 1, 64, 3, 1e6
    q = np.array([(i % 31) / 15.0 - 1.0 for i in range(n_q * hd)], dtype=np.float32)
    k = np.array([(i % 23) / 11.0 - 1.0 for i in range(n_kv * hd)], dtype=np.float32)
    v = np.array([(i % 19) / 9.0 - 1.0 for i in range(n_kv * hd)], dtype=np.float32)
    qkv = np.concatenate([q, k, v])[None]
    qr, kr, vv = orc.rope_append(qkv, np.array([pos]), n_q, n_kv, hd, theta)
    half = hd // 2
    for h in range(n_q):
        for j in range(half):
            inv = theta ** (-j / half)
            s, c = np.sin(pos * inv), np.cos(pos * inv)
            x1, x2 = float(q[h * hd + j]), float(q[h * hd + j + half])
            assert abs(qr[0, h, j] - (x1 * c - x2 * s)) < 1e-12
            assert abs(qr[0, h, j + half] - (x2 * c + x1 * s)) < 1e-12
    np.testing.assert_array_equal(vv[0].ravel(), v.astype(np.float64))


def test_qk_norm_precedes_rotation_and_skips_v():
    """decode_kernels.rs:140-239."""
    n_q, n_kv, hd, pos, theta, eps = 4, 2, 64, 5, 1e6, 1e-6
    q = np.array([(i % 31) / 15.0 - 1.0 for i in range(n_q * hd)], dtype=np.float32)
    k = np.array([(i % 23) / 11.0 - 1.0 for i in range(n_kv * hd)], dtype=np.float32)
    v = np.array([(i % 19) / 9.0 - 1.0 for i in range(n_kv * hd)], dtype=np.float32)
    gq = np.array([0.5 + (i % 7) * 0.1 for i in range(hd)], dtype=np.float32)
    gk = np.array([1.5 - (i % 5) * 0.2 for i in range(hd)], dtype=np.float32)
    qkv = np.concatenate([q, k, v])[None]
    qr, kr, vv = orc.rope_append(qkv, np.array([pos]), n_q, n_kv, hd, theta, gq, gk, eps)
    half = hd // 2
    for name, src, gain, got, heads in (("q", q, gq, qr, n_q), ("k", k, gk, kr, n_kv)):
        g16 = gain.astype(np.float16).astype(np.float64)
        for h in range(heads):
            head = src[h * hd:(h + 1) * hd].astype(np.float64)
            inv_rms = 1.0 / np.sqrt(np.mean(head * head) + eps)
            for j in range(half):
                f = theta ** (-j / half)
                s, c = np.sin(pos * f), np.cos(pos * f)
                x1, x2 = head[j] * inv_rms * g16[j], head[j + half] * inv_rms * g16[j + half]
                assert abs(got[0, h, j] - (x1 * c - x2 * s)) < 1e-12, name
                assert abs(got[0, h, j + half] - (x2 * c + x1 * s)) < 1e-12, name
    np.testing.assert_array_equal(vv[0].ravel(), v.astype(np.float64))


def test_one_position_returns_value_and_two_match_explicit_softmax():
    """decode_kernels.rs:294-410."""
    rng = np.random.default_rng(0)
    n_q, n_kv, hd = 14, 2, 64
    q = rng.standard_normal((n_q, hd))
    kc = rng.standard_normal((n_kv, 4, hd))
    vc = rng.standard_normal((n_kv, 4, hd))
    one = orc.decode_attention(q, kc, vc, 1)
    for h in range(n_q):
        np.testing.assert_allclose(one[h], vc[h // 7, 0], atol=1e-13)
    two = orc.decode_attention(q, kc, vc, 2)
    for h in range(n_q):
        g = h // 7
        s = np.array([q[h] @ kc[g, 0], q[h] @ kc[g, 1]]) / np.sqrt(hd)
        e = np.exp(s - s.max())
        np.testing.assert_allclose(two[h], (e[0] * vc[g, 0] + e[1] * vc[g, 1]) / e.sum(),
                                   atol=1e-13)


def test_lcg_noise_known_values():
    """chunk_kernels.rs:31-39: first outputs computed by hand from the recurrence."""
    mask = (1 << 64) - 1
    s = (303 * 6364136223846793005 + 1) & mask
    want = []
    for _ in range(4):
        s = (s * 6364136223846793005 + 1442695040888963407) & mask
        want.append(np.float32(np.float32(s >> 33) / np.float32(2 ** 31)) - np.float32(1.0))
    got = orc.lcg_noise(4, 303)
    np.testing.assert_array_equal(got, np.array(want, dtype=np.float32))
    big = orc.lcg_noise(4096, 404)
    # (s >> 33) has 31 bits, so the generator as written covers [-1, 0), not the
    # [-1, 1) its comment promises; the restatement keeps what the code does.
    assert big.min() >= -1.0 and big.max() < 0.0 and abs(float(big.mean()) + 0.5) < 0.02


def test_gather_pages_round_trip():
    rng = np.random.default_rng(1)
    n_kv, hd, page, length = 2, 8, 16, 37
    contiguous = rng.standard_normal((n_kv, length, hd))
    ids = np.array([5, 0, 3])
    pool = np.zeros((6, n_kv, page, hd))
    for i, pid in enumerate(ids):
        rows = contiguous[:, i * page:(i + 1) * page]
        pool[pid, :, : rows.shape[1]] = rows
    np.testing.assert_array_equal(orc.gather_pages(pool, ids, length), contiguous)


def test_error_stats():
    a = np.array([[1.0, 0.0], [0.0, 2.0]])
    b = np.array([[1.0, 0.001], [0.0, 2.0]])
    mx, cs = orc.error_stats(b, a)
    assert abs(mx - 0.001) < 1e-15 and 0.9999 < cs <= 1.0


def test_int4_hier_dequant_layout():
    """One group by hand: nibble c of the 16-byte word is weight c; w = q * (d * ls) -
    dmin * lm (cuda/hier.cuh:8-13)."""
    in_f, out_f = 32, 1
    q = np.arange(32) % 16
    words = np.zeros(4, dtype=np.uint32)
    for c in range(32):
        words[c // 8] |= np.uint32(q[c]) << np.uint32(4 * (c % 8))
    si = np.array([3 | (5 << 4)], dtype=np.uint8)
    d, dmin = np.float16(0.25), np.float16(0.5)
    sb = np.array([int(d.view(np.uint16)) | (int(dmin.view(np.uint16)) << 16)], dtype=np.uint32)
    w = orc.dequant_int4_hier(words, si, sb, in_f, out_f)
    assert np.array_equal(w[0], q * (0.25 * 3) - 0.5 * 5)
    x = np.ones((2, 32), dtype=np.float16)
    assert np.allclose(orc.gemm_int4_hier(words, si, sb, x, in_f, out_f), w.sum())


def test_e4m3_rounding_matches_torch():
    """oracle.e4m3_quantize against torch's float8_e4m3fn (round to nearest even) wherever the
    value is inside the finite range; beyond it the oracle saturates at 448 like the device's
    cvt.rn.satfinite."""
    import torch
    x = (np.random.default_rng(0).standard_normal(200000) * 40).astype(np.float32)
    x = x[np.abs(x) <= 448]
    want = torch.tensor(x).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(orc.e4m3_quantize(x), want)
    assert list(orc.e4m3_quantize(np.array([500.0, -1000.0, 464.0], dtype=np.float32))) == [126, 254, 126]
    table = orc.e4m3_values()
    assert table[0x7E] == 448 and table[0x38] == 1 and table[0x01] == 2.0 ** -9 and np.isnan(table[0x7F])
    back = torch.arange(256, dtype=torch.uint8).view(torch.float8_e4m3fn).float().numpy()
    assert np.array_equal(np.nan_to_num(table, nan=-1), np.nan_to_num(back, nan=-1))
