"""Single-token side of the attention path: the owner types and checked wrappers
the engine keeps in crates/whetstone-kernels/src/decode.rs, over this library's
C ABI.  Same names, same argument meaning, same shape errors; device memory is
a torch CUDA tensor instead of the engine's DeviceBuffer.
"""

from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass

import numpy as np
import torch

from . import _ffi
from ._ffi import ShapeError, check, lib

_CUDA_STREAM_LEGACY = 0x1  # cudaStreamLegacy: torch's default stream reports handle 0


def use_torch_stream() -> None:
    """Enqueue this thread's wst_* calls on torch's current CUDA stream, so that
    torch ops and the kernels are ordered without extra synchronisation."""
    handle = torch.cuda.current_stream().cuda_stream
    check(lib.wst_b200_set_stream(ctypes.c_void_p(handle if handle else _CUDA_STREAM_LEGACY)))


def _ptr(t: torch.Tensor | None) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _require_cuda(t: torch.Tensor, what: str, dtype: torch.dtype) -> None:
    if not t.is_cuda:
        raise ShapeError(5, f"{what}: expected a CUDA tensor")
    if t.dtype != dtype:
        raise ShapeError(5, f"{what}: expected dtype {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise ShapeError(5, f"{what}: expected a contiguous tensor")


@dataclass(frozen=True)
class RopeScaling:
    """Frequency schedule (decode.rs:64-86).  kind 'none' or 'llama3'."""

    kind: str = "none"
    factor: float = 1.0
    low_freq_factor: float = 1.0
    high_freq_factor: float = 4.0
    original_max_position: int = 8192


class RopeTable:
    """cos/sin ``[max_seq][head_dim/2]`` fp32, built on the host in f64 by the
    library (wst_rope_table_host) and uploaded once (decode.rs:50-153)."""

    def __init__(self, max_seq: int, head_dim: int, theta: float,
                 scaling: RopeScaling | None = None, device: torch.device | str = "cuda"):
        if head_dim % 2 != 0 or head_dim == 0:
            raise ShapeError(5, f"rope: head_dim {head_dim} must be even")
        scaling = scaling or RopeScaling()
        half = head_dim // 2
        cos = np.empty((max_seq, half), dtype=np.float32)
        sin = np.empty((max_seq, half), dtype=np.float32)
        check(lib.wst_rope_table_host(
            cos.ctypes.data_as(ctypes.c_void_p), sin.ctypes.data_as(ctypes.c_void_p),
            max_seq, head_dim, float(theta), 1 if scaling.kind == "llama3" else 0,
            float(scaling.factor), float(scaling.low_freq_factor),
            float(scaling.high_freq_factor), int(scaling.original_max_position)))
        self.cos_host, self.sin_host = cos, sin
        self.cos = torch.from_numpy(cos).to(device)
        self.sin = torch.from_numpy(sin).to(device)
        self.max_seq = max_seq
        self.half_dim = half

    def bytes(self) -> int:
        return self.cos.numel() * 4 + self.sin.numel() * 4


class KvCache:
    """One layer's cache, ``[n_kv][max_seq][head_dim]`` fp16 for K and V, plus the
    split scratch sized by wst_attn_partial_floats (decode.rs:162-212)."""

    def __init__(self, n_kv: int, n_q: int, head_dim: int, max_seq: int,
                 device: torch.device | str = "cuda"):
        floats = lib.wst_attn_partial_floats(n_q, head_dim, max_seq)
        self.k = torch.zeros((n_kv, max_seq, head_dim), dtype=torch.float16, device=device)
        self.v = torch.zeros((n_kv, max_seq, head_dim), dtype=torch.float16, device=device)
        self.partials = torch.zeros(max(floats, 1), dtype=torch.float32, device=device)
        self.n_kv, self.head_dim, self.max_seq = n_kv, head_dim, max_seq

    def keys(self) -> torch.Tensor:
        return self.k

    def values(self) -> torch.Tensor:
        return self.v

    def bytes(self) -> int:
        return self.k.numel() * 2 + self.v.numel() * 2 + self.partials.numel() * 4


class DeviceCursor:
    """A device-resident int32 for the per-token position (decode.rs:221-256)."""

    def __init__(self, value: int, device: torch.device | str = "cuda"):
        self.buf = torch.tensor([value], dtype=torch.int32, device=device)

    def set(self, value: int) -> None:
        self.buf.fill_(value)

    def get(self) -> int:
        return int(self.buf.item())

    def advance(self, max_seq: int) -> None:
        use_torch_stream()
        check(lib.wst_advance_pos(_ptr(self.buf), max_seq))


@dataclass
class QkNorm:
    """Per-head RMSNorm gains, ``head_dim`` fp16 each (decode.rs:269-290)."""

    q: torch.Tensor
    k: torch.Tensor
    eps: float

    def check(self, hd: int) -> None:
        if self.q.numel() != hd or self.k.numel() != hd:
            raise ShapeError(5, f"qk_norm: gains are q[{self.q.numel()}], k[{self.k.numel()}]; "
                                f"both must be head_dim {hd}")
        _require_cuda(self.q, "qk_norm.q", torch.float16)
        _require_cuda(self.k, "qk_norm.k", torch.float16)


def norm_ptrs(qk: QkNorm | None):
    if qk is None:
        return ctypes.c_void_p(0), ctypes.c_void_p(0), 0.0
    return _ptr(qk.q), _ptr(qk.k), float(qk.eps)


def rope_cache(qkv: torch.Tensor, cache: KvCache, table: RopeTable, n_q: int,
               pos: DeviceCursor, qk_norm: QkNorm | None = None) -> None:
    """RoPE (+ QK-norm) on q in place, k into the cache, v copied (decode.rs:305-354)."""
    hd = cache.head_dim
    want = (n_q + 2 * cache.n_kv) * hd
    _require_cuda(qkv, "rope_cache: qkv", torch.float32)
    if qkv.numel() != want:
        raise ShapeError(5, f"rope_cache: qkv[{qkv.numel()}] should be ({n_q} + 2*{cache.n_kv}) "
                            f"* {hd} = {want}")
    if table.half_dim != hd // 2 or table.max_seq < cache.max_seq:
        raise ShapeError(5, "rope_cache: rotary table does not match the cache geometry")
    if qk_norm is not None:
        qk_norm.check(hd)
    qw, kw, eps = norm_ptrs(qk_norm)
    use_torch_stream()
    check(lib.wst_rope_cache(_ptr(qkv), _ptr(cache.k), _ptr(cache.v), _ptr(table.cos),
                             _ptr(table.sin), n_q, cache.n_kv, hd, _ptr(pos.buf),
                             cache.max_seq, qw, kw, eps))


def attn_decode(qkv: torch.Tensor, cache: KvCache, out: torch.Tensor, n_q: int,
                pos: DeviceCursor) -> None:
    """Batch-1 GQA attention over cache rows 0..=pos (decode.rs:368-405)."""
    hd = cache.head_dim
    _require_cuda(qkv, "attn_decode: qkv", torch.float32)
    _require_cuda(out, "attn_decode: out", torch.float16)
    if qkv.numel() < n_q * hd or out.numel() != n_q * hd:
        raise ShapeError(5, f"attn_decode: qkv[{qkv.numel()}] must hold at least {n_q}*{hd} "
                            f"queries and out[{out.numel()}] exactly that")
    scale = 1.0 / math.sqrt(hd)
    use_torch_stream()
    check(lib.wst_attn_decode(_ptr(qkv), _ptr(cache.k), _ptr(cache.v), _ptr(cache.partials),
                              _ptr(out), n_q, cache.n_kv, hd, _ptr(pos.buf), cache.max_seq,
                              scale))


def attn_decode_partial(qkv: torch.Tensor, cache: KvCache, out_partial: torch.Tensor, n_q: int,
                        length: torch.Tensor, scale: float | None = None) -> None:
    """Unnormalised (m, l, acc) per head over rows [0, *length) of a cache shard."""
    hd = cache.head_dim
    _require_cuda(qkv, "attn_decode_partial: qkv", torch.float32)
    _require_cuda(out_partial, "attn_decode_partial: out", torch.float32)
    _require_cuda(length, "attn_decode_partial: length", torch.int32)
    if qkv.numel() < n_q * hd or out_partial.numel() != n_q * (hd + 2):
        raise ShapeError(5, "attn_decode_partial: qkv must hold n_q*head_dim queries and out "
                            "n_q*(head_dim+2) floats")
    use_torch_stream()
    check(lib.wst_attn_decode_partial(
        _ptr(qkv), _ptr(cache.k), _ptr(cache.v), _ptr(cache.partials), _ptr(out_partial), n_q,
        cache.n_kv, hd, _ptr(length), cache.max_seq,
        float(scale if scale is not None else 1.0 / math.sqrt(hd))))


def attn_merge_partials(parts: torch.Tensor, out: torch.Tensor, n_q: int, head_dim: int) -> None:
    """[n_parts][n_q][head_dim+2] gathered triples -> [n_q][head_dim] fp16."""
    _require_cuda(parts, "attn_merge_partials: parts", torch.float32)
    _require_cuda(out, "attn_merge_partials: out", torch.float16)
    per = n_q * (head_dim + 2)
    if parts.numel() % per != 0 or parts.numel() == 0 or out.numel() != n_q * head_dim:
        raise ShapeError(5, "attn_merge_partials: parts must be [n_parts][n_q][head_dim+2] "
                            "and out [n_q][head_dim]")
    use_torch_stream()
    check(lib.wst_attn_merge_partials(_ptr(parts), _ptr(out), parts.numel() // per, n_q,
                                      head_dim))


def attn_exchange_merge(mine: torch.Tensor, out: torch.Tensor, mailboxes: torch.Tensor,
                        state: torch.Tensor, rank: int, world: int, n_q: int,
                        head_dim: int) -> None:
    """This rank's [n_q][head_dim+2] triples -> [n_q][head_dim] fp16 merged over all
    ranks, exchanged through peer memory inside the kernel.  `mailboxes` is an int64
    device array of the ranks' mailbox addresses (see sharded.PeerExchange)."""
    _require_cuda(mine, "attn_exchange_merge: triples", torch.float32)
    _require_cuda(out, "attn_exchange_merge: out", torch.float16)
    _require_cuda(mailboxes, "attn_exchange_merge: mailboxes", torch.int64)
    _require_cuda(state, "attn_exchange_merge: state", torch.int32)
    if mine.numel() != n_q * (head_dim + 2) or out.numel() != n_q * head_dim:
        raise ShapeError(5, "attn_exchange_merge: triples must be [n_q][head_dim+2] and out "
                            "[n_q][head_dim]")
    if mailboxes.numel() != world or state.numel() < n_q:
        raise ShapeError(5, "attn_exchange_merge: one mailbox address per rank, one counter "
                            "per head")
    use_torch_stream()
    check(lib.wst_attn_exchange_merge(_ptr(mine), _ptr(out), _ptr(mailboxes), _ptr(state), rank,
                                      world, n_q, head_dim))


def attn_decode_sharded(qkv: torch.Tensor, cache: KvCache, out: torch.Tensor, n_q: int,
                        length: torch.Tensor, mailboxes: torch.Tensor, state: torch.Tensor,
                        rank: int, world: int, scale: float | None = None) -> None:
    """attn_decode_partial and the cross-GPU exchange in one kernel: rows [0, *length) of
    this rank's shard -> out [n_q*head_dim] fp16 merged over all ranks."""
    hd = cache.head_dim
    _require_cuda(qkv, "attn_decode_sharded: qkv", torch.float32)
    _require_cuda(out, "attn_decode_sharded: out", torch.float16)
    _require_cuda(length, "attn_decode_sharded: length", torch.int32)
    _require_cuda(mailboxes, "attn_decode_sharded: mailboxes", torch.int64)
    _require_cuda(state, "attn_decode_sharded: state", torch.int32)
    if qkv.numel() < n_q * hd or out.numel() != n_q * hd:
        raise ShapeError(5, "attn_decode_sharded: qkv must hold n_q*head_dim queries and out "
                            "exactly n_q*head_dim")
    if mailboxes.numel() != world or state.numel() < n_q:
        raise ShapeError(5, "attn_decode_sharded: one mailbox address per rank, one counter "
                            "per head")
    use_torch_stream()
    check(lib.wst_attn_decode_sharded(
        _ptr(qkv), _ptr(cache.k), _ptr(cache.v), _ptr(cache.partials), _ptr(out), n_q,
        cache.n_kv, hd, _ptr(length), cache.max_seq,
        float(scale if scale is not None else 1.0 / math.sqrt(hd)), _ptr(mailboxes),
        _ptr(state), rank, world))


def set_tuning(key: int, value: int) -> None:
    """Measurement knobs of the decode kernel (wst_b200_set_tuning)."""
    check(lib.wst_b200_set_tuning(key, value))


class KvCacheFp8:
    """One layer's cache in e4m3 bytes, ``[n_kv][max_seq][head_dim]`` uint8 for K and V, with
    the two scales (a stored byte times the scale is the value) and the split scratch."""

    def __init__(self, n_kv: int, n_q: int, head_dim: int, max_seq: int, k_scale: float = 1.0,
                 v_scale: float = 1.0, device: str = "cuda"):
        floats = lib.wst_attn_partial_floats(n_q, head_dim, max_seq)
        self.k = torch.zeros((n_kv, max_seq, head_dim), dtype=torch.uint8, device=device)
        self.v = torch.zeros((n_kv, max_seq, head_dim), dtype=torch.uint8, device=device)
        self.partials = torch.zeros(max(floats, 1), dtype=torch.float32, device=device)
        self.n_kv, self.head_dim, self.max_seq = n_kv, head_dim, max_seq
        self.k_scale, self.v_scale = float(k_scale), float(v_scale)


def rope_cache_fp8(qkv: torch.Tensor, cache: KvCacheFp8, table: "RopeTable", n_q: int,
                   pos: "DeviceCursor | None" = None, pos0: int = 0, n: int = 1,
                   qk_norm: "QkNorm | None" = None) -> None:
    """rope_cache (``pos`` given: one token at the cursor) or its chunk form (``pos0``,
    ``n``) into an e4m3 cache."""
    hd = cache.head_dim
    _require_cuda(qkv, "rope_cache_fp8: qkv", torch.float32)
    if qkv.numel() < n * (n_q + 2 * cache.n_kv) * hd:
        raise ShapeError(5, f"rope_cache_fp8: qkv[{qkv.numel()}] is too short")
    if table.half_dim != hd // 2 or table.max_seq < cache.max_seq:
        raise ShapeError(5, "rope_cache_fp8: rotary table does not match the cache geometry")
    if qk_norm is not None:
        qk_norm.check(hd)
    qw, kw, eps = norm_ptrs(qk_norm)
    use_torch_stream()
    check(lib.wst_b200_rope_cache_fp8(_ptr(qkv), _ptr(cache.k), _ptr(cache.v), _ptr(table.cos),
                                      _ptr(table.sin), n_q, cache.n_kv, hd,
                                      _ptr(pos.buf) if pos is not None else None, pos0, n,
                                      cache.max_seq, qw, kw, eps, cache.k_scale, cache.v_scale))


def attn_decode_fp8(qkv: torch.Tensor, cache: KvCacheFp8, out: torch.Tensor, n_q: int,
                    pos: "DeviceCursor") -> None:
    """attn_decode over an e4m3 cache."""
    hd = cache.head_dim
    _require_cuda(qkv, "attn_decode_fp8: q", torch.float32)
    _require_cuda(out, "attn_decode_fp8: out", torch.float16)
    if qkv.numel() < n_q * hd or out.numel() != n_q * hd:
        raise ShapeError(5, f"attn_decode_fp8: q[{qkv.numel()}], out[{out.numel()}] need {n_q} * {hd}")
    use_torch_stream()
    check(lib.wst_b200_attn_decode_fp8(_ptr(qkv), _ptr(cache.k), _ptr(cache.v), _ptr(cache.partials),
                                       _ptr(out), n_q, cache.n_kv, hd, _ptr(pos.buf), cache.max_seq,
                                       1.0 / math.sqrt(hd), cache.k_scale, cache.v_scale))


def device_error() -> int:
    """Read and clear the device watchdog word (0 = no kernel gave up a wait)."""
    use_torch_stream()
    code = ctypes.c_uint32(0)
    check(lib.wst_b200_device_error(ctypes.byref(code)))
    return int(code.value)


__all__ = [
    "RopeScaling", "RopeTable", "KvCache", "DeviceCursor", "QkNorm", "rope_cache",
    "attn_decode", "attn_decode_partial", "attn_merge_partials", "attn_decode_sharded",
    "set_tuning", "use_torch_stream",
    "device_error", "_ffi",
]
