"""wst_gemm_int4_hier: the projection with weights in the engine's hierarchical int4
format, against the exact fp64 product with the dequantized weights
(oracle.gemm_int4_hier, cuda/hier.cuh:8-13) and against the engine's own kernel
(oracle/_ref, cuda/chunk_gemm.cu:65-176), on the engine's test recipe
(tests/chunk_kernels.rs:114-167: xorshift bits, ls in 1..8, lm in 0..15, d and dmin per
row, 896 x 256 x 19) and on chunk-sized shapes.

Bound against the exact product, as in that test: |got - want| <= 3e-3 * max(|want|, 1)
at its contraction length of 896, grown with the square root of the length beyond it:
this kernel rounds every weight to fp16 once, an error that is random in sign.  Measured
here 1.3e-3 on the engine's case.  The engine's own kernel rounds partial dot products
to fp16 and sits 6e-3 to 1.4e-2 from the exact product on the same inputs (its test
compares it with its GEMV, which rounds the same way), so the comparison with it checks
that this kernel is the closer of the two and that the two agree to the engine's
distance."""

import ctypes
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import attention_oracle as orc
from tests.helpers import dev, host
from tests.test_gemm_gpu import REF_PATH, close, lcg_noise
from whetstone_b200 import chunk, decode
from whetstone_b200._ffi import SIGNATURES, lib

pytestmark = pytest.mark.gpu


def packed_weights(in_f, out_f, seed=0x12345678):
    """The packed arrays of tests/chunk_kernels.rs:121-147 for any shape."""
    n_words, n_groups = out_f * in_f // 8, out_f * in_f // 32
    total = n_words + n_groups
    s = np.uint32(seed)
    stream = np.empty(total, dtype=np.uint32)
    with np.errstate(over="ignore"):
        for i in range(total):
            s ^= np.uint32(s << np.uint32(13))
            s ^= np.uint32(s >> np.uint32(17))
            s ^= np.uint32(s << np.uint32(5))
            stream[i] = s
    qw = stream[:n_words].copy()
    v = stream[n_words:]
    si = ((1 + (v & 0x7)) | (((v >> 8) & 0xF) << 4)).astype(np.uint8)
    rows = np.arange(out_f)
    d = (0.002 + (rows % 7) * 1e-4).astype(np.float32).astype(np.float16).view(np.uint16).astype(np.uint32)
    dm = (0.01 + (rows % 5) * 1e-3).astype(np.float32).astype(np.float16).view(np.uint16).astype(np.uint32)
    return qw, si, d | (dm << 16)


def fast_packed_weights(in_f, out_f, seed):
    """Same value ranges from numpy's generator, for shapes where the scalar xorshift
    would take minutes."""
    rng = np.random.default_rng(seed)
    qw = rng.integers(0, 2 ** 32, size=out_f * in_f // 8, dtype=np.uint64).astype(np.uint32)
    si = (rng.integers(1, 9, size=out_f * in_f // 32) | (rng.integers(0, 16, size=out_f * in_f // 32) << 4)).astype(np.uint8)
    d = rng.uniform(0.002, 0.003, out_f).astype(np.float16).view(np.uint16).astype(np.uint32)
    dm = rng.uniform(0.01, 0.015, out_f).astype(np.float16).view(np.uint16).astype(np.uint32)
    return qw, si, d | (dm << 16)


def run(qw, si, sb, x, bias, y0, in_f, out_f, accum):
    n = x.shape[0]
    qd = dev(qw.view(np.int32))
    sd = dev(si)
    bd = dev(sb.view(np.uint32).astype(np.uint32).view(np.float16))   # (d, dmin) pairs as fp16
    yd = dev(y0.astype(np.float32)) if y0 is not None else \
        torch.full((n, out_f), float("nan"), dtype=torch.float32, device="cuda")
    chunk.gemm_int4_hier(qd, sd, bd, dev(x.astype(np.float16)),
                         dev(bias.astype(np.float16)) if bias is not None else None, yd, in_f, out_f,
                         n, accum)
    torch.cuda.synchronize()
    assert decode.device_error() == 0
    return host(yd), (qd, sd, bd)


def test_the_engines_case():
    in_f, out_f, n = 896, 256, 19
    qw, si, sb = packed_weights(in_f, out_f)
    x = lcg_noise(in_f * n, 77).reshape(n, in_f)
    got, _ = run(qw, si, sb, x, None, None, in_f, out_f, False)
    close(got, orc.gemm_int4_hier(qw, si, sb, x, in_f, out_f), 3e-3, "896 x 256 x 19")


@pytest.mark.parametrize("in_f,out_f,n,bias,accum", [
    (4096, 6144, 512, True, False),    # a qkv projection of a 512-token chunk
    (4096, 1024, 300, False, True),    # accumulating, ragged token tile
    (2080, 520, 130, True, False),     # in_f a multiple of 32 only: half a k-block at the end
    (64, 40, 3, False, False),         # one k-block, a sliver of a tile
    (1024, 3000, 16, True, False),     # few tokens: the narrow feature tile
])
def test_against_the_exact_product(in_f, out_f, n, bias, accum):
    qw, si, sb = fast_packed_weights(in_f, out_f, in_f + out_f + n)
    rng = np.random.default_rng(n)
    x = rng.uniform(-1, 1, (n, in_f)).astype(np.float16)   # the range of the engine's test inputs
    b = rng.standard_normal(out_f).astype(np.float16) if bias else None
    y0 = rng.standard_normal((n, out_f)).astype(np.float32) if accum else None
    got, _ = run(qw, si, sb, x, b, y0, in_f, out_f, accum)
    close(got, orc.gemm_int4_hier(qw, si, sb, x, in_f, out_f, b, y0),
          3e-3 * max(1.0, (in_f / 896) ** 0.5), f"{in_f} x {out_f} x {n}")


def test_against_the_reference_kernel():
    if not REF_PATH.exists():
        pytest.skip("oracle/_ref/libwhetstone_ref.so not built")
    ref = ctypes.CDLL(str(REF_PATH))
    for name in ("wst_gemm_int4_hier", "wst_device_synchronize"):
        fn = getattr(ref, name)
        fn.restype, fn.argtypes = SIGNATURES[name]
    P = lambda t: ctypes.c_void_p(t.data_ptr() if t is not None else 0)
    for in_f, out_f, n in ((896, 256, 19), (4096, 512, 40)):
        qw, si, sb = fast_packed_weights(in_f, out_f, n)
        x = np.random.default_rng(n).uniform(-1, 1, (n, in_f)).astype(np.float16)
        mine, (qd, sd, bd) = run(qw, si, sb, x, None, None, in_f, out_f, False)
        theirs = torch.zeros((n, out_f), dtype=torch.float32, device="cuda")
        xd = dev(x)
        assert ref.wst_gemm_int4_hier(P(qd), P(sd), P(bd), P(xd), None, P(theirs), in_f, out_f, n, 0) == 0
        assert ref.wst_device_synchronize() == 0
        theirs = host(theirs)
        want = orc.gemm_int4_hier(qw, si, sb, x, in_f, out_f)
        scale = np.maximum(np.abs(want), 1.0)
        err_mine, err_theirs = (np.abs(mine - want) / scale).max(), (np.abs(theirs - want) / scale).max()
        assert err_mine <= err_theirs, (err_mine, err_theirs)
        close(mine, theirs, 2e-2, f"reference kernel, {in_f} x {out_f} x {n}")


def test_bad_arguments_launch_nothing():
    y = torch.full((4,), 7.0, dtype=torch.float32, device="cuda")
    w = torch.zeros(64, dtype=torch.float16, device="cuda")
    p = ctypes.c_void_p(w.data_ptr())
    assert lib.wst_gemm_int4_hier(p, p, p, p, None, ctypes.c_void_p(y.data_ptr()), 48, 2, 1, 0) == 2
    assert b"multiple of 32" in lib.wst_last_error()
    torch.cuda.synchronize()
    assert (host(y) == 7.0).all()
