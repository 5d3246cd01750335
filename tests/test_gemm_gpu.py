"""wst_gemm_fp16: the projection either side of the attention path, against the exact
float64 product of the same fp16 inputs (oracle.attention_oracle.gemm_fp16), against the
reference's own kernel (oracle/_ref, built unmodified from cuda/chunk_gemm.cu) and on the
reference's own test shapes and inputs (crates/whetstone-kernels/tests/chunk_kernels.rs:
51-108: the LCG, 896 x 320 x 7 with bias, 256 x 96 x 5 accumulating).

Bound, as in the reference's tests: |got - want| <= 2e-3 * max(|want|, 1).  Against the
exact product this library's kernel (fp32 products and sums) is held to 2e-4 at
contraction lengths in the thousands and to 1e-5 on the reference's own small cases."""

import ctypes
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import attention_oracle as orc
from tests.helpers import dev, host
from whetstone_b200 import chunk, decode
from whetstone_b200._ffi import SIGNATURES, ShapeError, check, lib

pytestmark = pytest.mark.gpu

REF_PATH = Path(__file__).resolve().parent.parent / "oracle" / "_ref" / "libwhetstone_ref.so"


def lcg_noise(n, seed):
    """`noise` of tests/chunk_kernels.rs:31-40: floats in [-1, 1) from a fixed LCG."""
    mask = (1 << 64) - 1
    s = (seed * 6364136223846793005 + 1) & mask
    out = np.empty(n, dtype=np.float32)
    for i in range(n):
        s = (s * 6364136223846793005 + 1442695040888963407) & mask
        out[i] = np.float32(np.float32(s >> 33) / np.float32(1 << 31)) - np.float32(1.0)
    return out


def close(got, want, tol, what):
    scale = np.maximum(np.abs(want), 1.0)
    bad = np.abs(got - want) > tol * scale
    assert not bad.any(), f"{what}: {int(bad.sum())} of {bad.size} outside {tol}, worst " \
                          f"{np.abs(got - want).max()}"


def run(w, x, bias, y0, accum):
    out_f, in_f = w.shape
    n = x.shape[0]
    wd, xd = dev(w.astype(np.float16)), dev(x.astype(np.float16))
    bd = dev(bias.astype(np.float16)) if bias is not None else None
    yd = dev(y0.astype(np.float32)) if y0 is not None else \
        torch.full((n, out_f), float("nan"), dtype=torch.float32, device="cuda")
    chunk.gemm_fp16(wd, xd, bd, yd, in_f, out_f, n, accum)
    torch.cuda.synchronize()
    assert decode.device_error() == 0
    return host(yd)


def test_reference_case_with_bias():
    in_f, out_f, n = 896, 320, 7
    w, x, b = lcg_noise(in_f * out_f, 11).reshape(out_f, in_f), lcg_noise(in_f * n, 22).reshape(n, in_f), \
        lcg_noise(out_f, 33)
    got = run(w, x, b, None, False)
    close(got, orc.gemm_fp16(w, x, b), 1e-5, "896 x 320 x 7 with bias")


def test_reference_case_accumulating():
    in_f, out_f, n = 256, 96, 5
    w, x = lcg_noise(in_f * out_f, 44).reshape(out_f, in_f), lcg_noise(in_f * n, 55).reshape(n, in_f)
    y0 = lcg_noise(n * out_f, 66).reshape(n, out_f)
    got = run(w, x, None, y0, True)
    close(got, orc.gemm_fp16(w, x, None, y0), 1e-5, "256 x 96 x 5 accumulating")


@pytest.mark.parametrize("in_f,out_f,n,bias,accum", [
    (64, 8, 1, False, False),          # one token, one k-block, a sliver of one tile
    (4096, 6144, 512, True, False),    # the qkv projection of a 512-token chunk (32/8/8 heads of 128)
    (4096, 4096, 300, False, True),    # o_proj into the residual, ragged token tile
    (896, 1152, 2048, True, False),    # 0.5B-shaped qkv, 16 token tiles
    (1000, 333, 130, True, True),      # nothing a multiple of the tile: ragged k-block, odd out_f
    (72, 40, 17, False, False),        # in_f a multiple of 8 only
    (4096, 256, 129, False, False),    # exactly one feature tile, two token tiles
    (128, 70000, 3, True, False),      # lm_head-like: many feature tiles, few tokens
])
def test_against_the_exact_product(in_f, out_f, n, bias, accum):
    rng = np.random.default_rng(in_f * 31 + out_f * 7 + n)
    w = (rng.standard_normal((out_f, in_f)) / np.sqrt(in_f)).astype(np.float16)
    x = rng.standard_normal((n, in_f)).astype(np.float16)
    b = rng.standard_normal(out_f).astype(np.float16) if bias else None
    y0 = rng.standard_normal((n, out_f)).astype(np.float32) if accum else None
    got = run(w, x, b, y0, accum)
    close(got, orc.gemm_fp16(w, x, b, y0), 2e-4, f"{in_f} x {out_f} x {n}")


@pytest.mark.parametrize("in_f", [7, 100, 4100])
def test_widths_the_tensor_maps_cannot_describe(in_f):
    """in_f not a multiple of 8: the plain kernel."""
    rng = np.random.default_rng(in_f)
    out_f, n = 50, 9
    w = (rng.standard_normal((out_f, in_f)) / np.sqrt(in_f)).astype(np.float16)
    x = rng.standard_normal((n, in_f)).astype(np.float16)
    b = rng.standard_normal(out_f).astype(np.float16)
    got = run(w, x, b, None, False)
    close(got, orc.gemm_fp16(w, x, b), 1e-5, f"in_f {in_f}")


def test_rows_past_n_and_columns_past_out_f_are_not_written():
    in_f, out_f, n = 512, 200, 5
    rng = np.random.default_rng(1)
    w = rng.standard_normal((out_f, in_f)).astype(np.float16)
    x = rng.standard_normal((n, in_f)).astype(np.float16)
    guard = torch.full(((n + 3) * out_f + 64,), 12345.0, dtype=torch.float32, device="cuda")
    y = guard[: n * out_f]
    chunk.gemm_fp16(dev(w), dev(x), None, y, in_f, out_f, n, False)
    torch.cuda.synchronize()
    assert (host(guard[n * out_f:]) == 12345.0).all()
    close(host(y).reshape(n, out_f), orc.gemm_fp16(w, x), 2e-4, "guarded")


def test_against_the_reference_kernel():
    if not REF_PATH.exists():
        pytest.skip("oracle/_ref/libwhetstone_ref.so not built")
    ref = ctypes.CDLL(str(REF_PATH))
    for name in ("wst_gemm_fp16", "wst_device_synchronize"):
        fn = getattr(ref, name)
        fn.restype, fn.argtypes = SIGNATURES[name]
    P = lambda t: ctypes.c_void_p(t.data_ptr() if t is not None else 0)
    for in_f, out_f, n, accum in ((896, 320, 7, 0), (256, 96, 5, 1), (4096, 1024, 40, 0)):
        rng = np.random.default_rng(n)
        w = dev((rng.standard_normal((out_f, in_f)) / np.sqrt(in_f)).astype(np.float16))
        x = dev(rng.standard_normal((n, in_f)).astype(np.float16))
        b = dev(rng.standard_normal(out_f).astype(np.float16))
        y0 = rng.standard_normal((n, out_f)).astype(np.float32)
        mine, theirs = dev(y0), dev(y0)
        chunk.gemm_fp16(w, x, b, mine, in_f, out_f, n, bool(accum))
        torch.cuda.synchronize()
        assert ref.wst_gemm_fp16(P(w), P(x), P(b), P(theirs), in_f, out_f, n, accum) == 0
        assert ref.wst_device_synchronize() == 0
        close(host(mine), host(theirs), 2e-3, f"reference kernel, {in_f} x {out_f} x {n}")


def test_bad_arguments_launch_nothing():
    y = torch.full((4,), 7.0, dtype=torch.float32, device="cuda")
    w = torch.zeros(8, dtype=torch.float16, device="cuda")
    for args in ((None, w, None, y, 2, 2, 1, 0), (w, w, None, y, 0, 2, 1, 0), (w, w, None, y, 2, 2, 0, 0)):
        ptrs = [ctypes.c_void_p(a.data_ptr()) if isinstance(a, torch.Tensor) else a for a in args]
        assert lib.wst_gemm_fp16(*ptrs) == 2   # WST_ERR_INVALID_ARG
        assert b"wst_gemm_fp16" in lib.wst_last_error()
    torch.cuda.synchronize()
    assert (host(y) == 7.0).all()
    with pytest.raises(ShapeError):
        chunk.gemm_fp16(w, w, None, y, 4, 4, 1)
    assert chunk.max_tokens() == 512


def test_random_shapes_against_the_exact_product():
    """Seeded random shapes through all feature-tile choices (few tokens: 32, 48, 64 rows
    and one or four slabs of K per request; many tokens: 256 rows), bias and accumulate at
    random."""
    rng = np.random.default_rng(2026)
    for case in range(24):
        n = int(rng.choice([1, 3, 16, 17, 64, 65, 128, 129, 200, 600]))
        in_f = int(rng.choice([64, 72, 128, 320, 1000, 1024, 2048]))
        out_f = int(rng.integers(1, 40)) * int(rng.choice([1, 7, 32, 48]))
        bias, accum = bool(rng.integers(2)), bool(rng.integers(2))
        w = (rng.standard_normal((out_f, in_f)) / np.sqrt(in_f)).astype(np.float16)
        x = rng.standard_normal((n, in_f)).astype(np.float16)
        b = rng.standard_normal(out_f).astype(np.float16) if bias else None
        y0 = rng.standard_normal((n, out_f)).astype(np.float32) if accum else None
        got = run(w, x, b, y0, accum)
        close(got, orc.gemm_fp16(w, x, b, y0), 2e-4, f"case {case}: {in_f} x {out_f} x {n}")


def test_projection_replays_in_a_graph():
    """The entry point under stream capture (after one ordinary call): same result on replay
    with new activations."""
    in_f, out_f, n = 512, 768, 300
    rng = np.random.default_rng(3)
    w = dev((rng.standard_normal((out_f, in_f)) / np.sqrt(in_f)).astype(np.float16))
    x = dev(rng.standard_normal((n, in_f)).astype(np.float16))
    y = torch.zeros((n, out_f), dtype=torch.float32, device="cuda")
    chunk.gemm_fp16(w, x, None, y, in_f, out_f, n)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        chunk.gemm_fp16(w, x, None, y, in_f, out_f, n)
    x2 = rng.standard_normal((n, in_f)).astype(np.float16)
    x.copy_(dev(x2))
    g.replay()
    torch.cuda.synchronize()
    close(host(y), orc.gemm_fp16(host(w), x2), 2e-4, "graph replay")
    assert decode.device_error() == 0
