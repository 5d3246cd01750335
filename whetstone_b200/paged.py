"""Paged KV cache and the ragged batch entry points (wst_rope_cache_paged,
wst_attn_verify_paged).  The engine has a contiguous single-sequence cache only
(crates/whetstone-kernels/src/decode.rs:162-212); this is the batched form its
speculative-verify loop (crates/whetstone-core/src/speculate.rs:185-256) needs
when many sequences are verified at once.
"""

from __future__ import annotations

import math

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
    if seq_pos0.numel() != cache.n_seq or cu_tokens.numel() != cache.n_seq + 1:
        raise ShapeError(5, "rope_cache_paged: seq_pos0 needs n_seq and cu_tokens n_seq+1 entries")
    if table.half_dim != hd // 2:
        raise ShapeError(5, "rope_cache_paged: rotary table does not match head_dim")
    if qk_norm is not None:
        qk_norm.check(hd)
    qw, kw, eps = norm_ptrs(qk_norm)
    use_torch_stream()
    check(lib.wst_rope_cache_paged(
        _ptr(qkv), _ptr(cache.k), _ptr(cache.v), _ptr(table.cos), _ptr(table.sin),
        _ptr(cache.page_table), _ptr(seq_pos0), _ptr(cu_tokens), cache.n_seq, total_tokens,
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
    need = verify_scratch_floats(cache.n_seq, max_tokens_per_seq, n_q, cache.n_kv, hd, max_len)
    if scratch.numel() < need:
        raise ShapeError(5, f"attn_verify: scratch[{scratch.numel()}] needs {need} floats")
    use_torch_stream()
    check(lib.wst_attn_verify_paged(
        _ptr(qkv), _ptr(cache.k), _ptr(cache.v), _ptr(cache.page_table), _ptr(seq_pos0),
        _ptr(cu_tokens), _ptr(scratch), _ptr(out), cache.n_seq, total_tokens,
        max_tokens_per_seq, cache.max_pages, PAGE_SIZE, cache.n_pages, n_q, cache.n_kv, hd,
        max_len, float(scale if scale is not None else 1.0 / math.sqrt(hd))))


__all__ = ["PAGE_SIZE", "PagedKvCache", "rope_cache", "verify_scratch_floats", "attn_verify"]
