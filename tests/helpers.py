"""Small utilities shared by the GPU parity tests."""

from __future__ import annotations

import numpy as np
import torch

from oracle import attention_oracle as orc

NAN16 = 0x7E00      # fp16 quiet NaN: the filler for cache rows nothing may read
SENTINEL = 0x7BCD   # an arbitrary finite pattern for "was this slot written?" checks

MAX_ABS = 2e-3      # acceptance: max abs error per head vector
MIN_COS = 0.9999    # acceptance: cosine per head vector


def dev(x: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


def host(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().numpy()


def fill_bits(t: torch.Tensor, bits: int) -> None:
    """Fill an fp16 tensor with a raw bit pattern."""
    t.view(torch.int16).fill_(np.array(bits, dtype=np.uint16).astype(np.int16).item())


def fill_rows_from(t: torch.Tensor, bits: int, start: int) -> None:
    """Same for rows [start:] of every head of a [heads][rows][dim] cache."""
    t.view(torch.int16)[:, start:] = np.array(bits, dtype=np.uint16).astype(np.int16).item()


def bits16(t: torch.Tensor) -> np.ndarray:
    return host(t.view(torch.int16)).view(np.uint16)


def assert_close_per_head(got: np.ndarray, want: np.ndarray, what: str,
                          max_abs: float = MAX_ABS, min_cos: float = MIN_COS) -> None:
    """got/want: [..., head_dim]; the north-star bar, per head vector."""
    assert got.shape == want.shape, f"{what}: shape {got.shape} vs {want.shape}"
    assert np.all(np.isfinite(got)), f"{what}: non-finite output"
    mx, cs = orc.error_stats(got, want)
    assert mx <= max_abs, f"{what}: max abs error {mx:.3e} > {max_abs}"
    assert cs >= min_cos, f"{what}: min cosine {cs:.6f} < {min_cos}"


def assert_k_cache_matches(got_bits: np.ndarray, want_f64: np.ndarray, what: str) -> None:
    """K rows against fp16(oracle).  The device rotates in fp32 from an fp32 table,
    so a value may land on the neighbouring fp16 number (1 ulp); where the two
    rotation terms cancel, the fp32 rounding of the terms (~1e-7 absolute) can be
    several ulps of a tiny result, so an absolute 3e-6 is accepted there.  (The
    reference's own test allows 3e-3 absolute, decode_kernels.rs:219.)"""
    want_bits = want_f64.astype(np.float16).view(np.uint16)
    ulp = f16_ulp_distance(got_bits, want_bits)
    diff = np.abs(got_bits.view(np.float16).astype(np.float64) - want_f64)
    bad = (ulp > 1) & (diff > 3e-6)
    assert not bad.any(), (f"{what}: {int(bad.sum())} K values off; worst {diff[bad].max():.3e} "
                           f"({int(ulp[bad].max())} ulp)")


def f16_ulp_distance(a_bits: np.ndarray, b_bits: np.ndarray) -> np.ndarray:
    """Distance in representable fp16 values between two bit arrays (same sign or
    across zero)."""
    def key(u):
        u = u.astype(np.int32)
        return np.where(u & 0x8000, -(u & 0x7FFF), u & 0x7FFF)
    return np.abs(key(a_bits) - key(b_bits))
