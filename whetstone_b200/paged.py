"""Paged KV cache and the ragged batch entry points (wst_rope_cache_paged,
wst_attn_verify_paged).  The engine has a contiguous single-sequence cache only
(crates/whetstone-kernels/src/decode.rs:162-212); this is the batched form its
speculative-verify loop (crates/whetstone-core/src/speculate.rs:185-256) needs
when many sequences are verified at once.
"""

from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass

import numpy as np
import torch

from ._ffi import ShapeError, check, lib
from .decode import QkNorm, RopeTable, _ptr, _require_cuda, norm_ptrs, use_torch_stream

PAGE_SIZE = 16


class PagedKvCache:
    """Page pool ``[n_pages][n_kv][16][head_dim]`` fp16 for K and V plus a page
    table ``[n_seq][max_pages]`` int32 (-1 = unmapped)."""

    def __init__(self, n_pages: int, n_kv: int, head_dim: int, n_seq: int, max_pages: int,
                 device: torch.device | str = "cuda"):
        shape = (n_pages, n_kv, PAGE_SIZE, head_dim)
        self.k = torch.zeros(shape, dtype=torch.float16, device=device)
        self.v = torch.zeros(shape, dtype=torch.float16, device=device)
        self.page_table = torch.full((n_seq, max_pages), -1, dtype=torch.int32, device=device)
        self.n_pages, self.n_kv, self.head_dim = n_pages, n_kv, head_dim
        self.n_seq, self.max_pages = n_seq, max_pages

    def bytes(self) -> int:
        return 2 * self.k.numel() * 2 + self.page_table.numel() * 4


def rope_cache(qkv: torch.Tensor, cache: PagedKvCache, table: RopeTable, n_q: int,
               seq_pos0: torch.Tensor, cu_tokens: torch.Tensor, total_tokens: int,
               qk_norm: QkNorm | None = None) -> None:
    """QK-norm + RoPE + append of a ragged batch into the page pool."""
    hd = cache.head_dim
    stride = (n_q + 2 * cache.n_kv) * hd
    _require_cuda(qkv, "rope_cache_paged: qkv", torch.float32)
    _require_cuda(seq_pos0, "rope_cache_paged: seq_pos0", torch.int32)
    _require_cuda(cu_tokens, "rope_cache_paged: cu_tokens", torch.int32)
    if qkv.numel() < total_tokens * stride:
        raise ShapeError(5, f"rope_cache_paged: qkv[{qkv.numel()}] needs {total_tokens} * {stride}")
    n_seq = seq_pos0.numel()     # the batch may use fewer rows than the table has
    if n_seq == 0 or n_seq > cache.n_seq or cu_tokens.numel() != n_seq + 1:
        raise ShapeError(5, "rope_cache_paged: seq_pos0 needs n_seq <= the table's rows and "
                            "cu_tokens n_seq+1 entries")
    if table.half_dim != hd // 2:
        raise ShapeError(5, "rope_cache_paged: rotary table does not match head_dim")
    if qk_norm is not None:
        qk_norm.check(hd)
    qw, kw, eps = norm_ptrs(qk_norm)
    use_torch_stream()
    check(lib.wst_rope_cache_paged(
        _ptr(qkv), _ptr(cache.k), _ptr(cache.v), _ptr(table.cos), _ptr(table.sin),
        _ptr(cache.page_table), _ptr(seq_pos0), _ptr(cu_tokens), n_seq, total_tokens,
        cache.max_pages, PAGE_SIZE, cache.n_pages, n_q, cache.n_kv, hd, table.max_seq, qw, kw,
        eps))


def verify_scratch_floats(n_seq: int, max_tokens_per_seq: int, n_q: int, n_kv: int,
                          head_dim: int, max_len: int) -> int:
    return int(lib.wst_attn_verify_scratch_floats(n_seq, max_tokens_per_seq, n_q, n_kv,
                                                  head_dim, max_len))


def attn_verify(qkv: torch.Tensor, cache: PagedKvCache, out: torch.Tensor, scratch: torch.Tensor,
                n_q: int, seq_pos0: torch.Tensor, cu_tokens: torch.Tensor, total_tokens: int,
                max_tokens_per_seq: int, max_len: int, scale: float | None = None) -> None:
    """Token j of sequence s attends to positions [0, seq_pos0[s] + j] of its pages."""
    hd = cache.head_dim
    stride = (n_q + 2 * cache.n_kv) * hd
    _require_cuda(qkv, "attn_verify: qkv", torch.float32)
    _require_cuda(out, "attn_verify: out", torch.float16)
    _require_cuda(scratch, "attn_verify: scratch", torch.float32)
    if qkv.numel() < total_tokens * stride:
        raise ShapeError(5, f"attn_verify: qkv[{qkv.numel()}] needs {total_tokens} * {stride}")
    if out.numel() < total_tokens * n_q * hd:
        raise ShapeError(5, f"attn_verify: out[{out.numel()}] needs {total_tokens} * {n_q} * {hd}")
    n_seq = seq_pos0.numel()
    if n_seq == 0 or n_seq > cache.n_seq or cu_tokens.numel() != n_seq + 1:
        raise ShapeError(5, "attn_verify: seq_pos0 needs n_seq <= the table's rows and cu_tokens "
                            "n_seq+1 entries")
    need = verify_scratch_floats(n_seq, max_tokens_per_seq, n_q, cache.n_kv, hd, max_len)
    if scratch.numel() < need:
        raise ShapeError(5, f"attn_verify: scratch[{scratch.numel()}] needs {need} floats")
    use_torch_stream()
    check(lib.wst_attn_verify_paged(
        _ptr(qkv), _ptr(cache.k), _ptr(cache.v), _ptr(cache.page_table), _ptr(seq_pos0),
        _ptr(cu_tokens), _ptr(scratch), _ptr(out), n_seq, total_tokens,
        max_tokens_per_seq, cache.max_pages, PAGE_SIZE, cache.n_pages, n_q, cache.n_kv, hd,
        max_len, float(scale if scale is not None else 1.0 / math.sqrt(hd))))


# ------------------------------------------- host side: page manager and scheduler

@dataclass
class Step:
    """Host arrays of one launch, as wst_rope_cache_paged / wst_attn_verify_paged take
    them (whetstone::paged_kv::StepArrays)."""

    entries: list            # [(seq id, n_tokens)] in batch order
    page_table: np.ndarray   # int32 [n_seq][max_pages], -1 = unmapped
    seq_pos0: np.ndarray     # int32 [n_seq]
    cu_tokens: np.ndarray    # int32 [n_seq + 1]
    total_tokens: int
    max_tokens_per_seq: int
    max_len: int

    @property
    def n_seq(self) -> int:
        return len(self.entries)

    def upload(self, cache: PagedKvCache):
        """Copies the page table into the cache's device table (batch slot i = row i) and
        returns (seq_pos0, cu_tokens) as device tensors."""
        dev = cache.page_table.device
        cache.page_table[: self.n_seq].copy_(torch.from_numpy(self.page_table).to(dev))
        return torch.from_numpy(self.seq_pos0).to(dev), torch.from_numpy(self.cu_tokens).to(dev)


def _i32(values) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(values, dtype=np.int32))


def _p(a: np.ndarray) -> ctypes.c_void_p:
    return a.ctypes.data_as(ctypes.c_void_p)


class PagedKvManager:
    """The C++ page manager (whetstone_b200/host/paged_kv.hpp) through its C bindings:
    a pool of 16-token pages, per-sequence page lists and committed lengths; reserve /
    commit / rewind / trim as the engine's speculative loop needs them
    (crates/whetstone-core/src/speculate.rs:185-256).  Host bookkeeping only."""

    def __init__(self, n_pool_pages: int, max_len: int):
        handle = ctypes.c_void_p()
        check(lib.wst_pkv_create(n_pool_pages, max_len, ctypes.byref(handle)))
        self._h = handle
        self.n_pool_pages, self.max_len = n_pool_pages, max_len
        self.max_pages = (max_len + PAGE_SIZE - 1) // PAGE_SIZE

    def __del__(self):
        if getattr(self, "_h", None) and lib is not None:   # lib is gone at interpreter exit
            lib.wst_pkv_destroy(self._h)
            self._h = None

    def open(self) -> int:
        seq = ctypes.c_int32(-1)
        check(lib.wst_pkv_open(self._h, ctypes.byref(seq)))
        return int(seq.value)

    def close(self, seq: int) -> None:
        check(lib.wst_pkv_close(self._h, seq))

    def _query(self, seq: int):
        length, pages, free = ctypes.c_int32(0), ctypes.c_int32(0), ctypes.c_int32(0)
        check(lib.wst_pkv_query(self._h, seq, ctypes.byref(length), ctypes.byref(pages),
                                ctypes.byref(free)))
        return int(length.value), int(pages.value), int(free.value)

    def length(self, seq: int) -> int:
        return self._query(seq)[0]

    def pages(self, seq: int) -> int:
        return self._query(seq)[1]

    def free_pages(self) -> int:
        return self._query(-1)[2]

    def reserve(self, seq: int, n_tokens: int) -> None:
        check(lib.wst_pkv_reserve(self._h, seq, n_tokens))

    def commit(self, seq: int, n_tokens: int) -> None:
        check(lib.wst_pkv_commit(self._h, seq, n_tokens))

    def rewind(self, seq: int, pos: int) -> None:
        check(lib.wst_pkv_rewind(self._h, seq, pos))

    def trim(self, seq: int, keep_tokens: int = 0) -> int:
        n = ctypes.c_int32(0)
        check(lib.wst_pkv_trim(self._h, seq, keep_tokens, ctypes.byref(n)))
        return int(n.value)

    def schedule(self, waiting, max_tokens_per_step: int, max_sequences_per_step: int):
        """waiting: [(seq, n_tokens)].  Returns this step's entries, longest context first."""
        if not waiting:
            return []
        seqs, toks = _i32([w[0] for w in waiting]), _i32([w[1] for w in waiting])
        chosen = np.zeros(len(waiting), dtype=np.int32)
        n = ctypes.c_int32(0)
        check(lib.wst_pkv_schedule(self._h, _p(seqs), _p(toks), len(waiting), max_tokens_per_step,
                                   max_sequences_per_step, _p(chosen), ctypes.byref(n)))
        return [tuple(waiting[i]) for i in chosen[: n.value]]

    def build_step(self, entries) -> Step:
        """Reserves the entries' rows (all or none: OutOfMemory leaves everything as it was)
        and lays out the launch arrays."""
        seqs, toks = _i32([e[0] for e in entries]), _i32([e[1] for e in entries])
        n = len(entries)
        table = np.empty((n, self.max_pages), dtype=np.int32)
        pos0 = np.empty(n, dtype=np.int32)
        cu = np.empty(n + 1, dtype=np.int32)
        totals = np.zeros(4, dtype=np.int32)
        check(lib.wst_pkv_build_step(self._h, _p(seqs), _p(toks), n, _p(table), _p(pos0), _p(cu),
                                     _p(totals)))
        return Step([tuple(e) for e in entries], table, pos0, cu, int(totals[0]), int(totals[1]),
                    int(totals[2]))


def assign_units(step: Step, n_kv: int, world: int) -> np.ndarray:
    """Rank of every (batch slot, KV head) unit, heaviest first to the least loaded rank:
    int32 [n_seq * n_kv], unit = slot * n_kv + kv_head."""
    out = np.zeros(step.n_seq * n_kv, dtype=np.int32)
    check(lib.wst_pkv_assign_units(_p(step.seq_pos0), _p(step.cu_tokens), step.n_seq, n_kv, world,
                                   _p(out)))
    return out


__all__ = ["PAGE_SIZE", "PagedKvCache", "rope_cache", "verify_scratch_floats", "attn_verify",
           "PagedKvManager", "Step", "assign_units"]
