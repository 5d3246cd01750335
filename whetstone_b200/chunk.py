"""Multi-token side of the attention path: the checked wrappers the engine keeps
in crates/whetstone-kernels/src/chunk.rs (`rope_cache` :140-201, `attn`
:207-254), over this library's C ABI.  Used for chunked prefill and for
speculative verification (a chunk of 1 + drafts tokens at pos0 = current pos).
"""

from __future__ import annotations

import math

import torch

from ._ffi import ShapeError, check, lib
from .decode import KvCache, QkNorm, RopeTable, _ptr, _require_cuda, norm_ptrs, use_torch_stream


def rope_cache(qkv: torch.Tensor, cache: KvCache, table: RopeTable, n_q: int, pos0: int, n: int,
               qk_norm: QkNorm | None = None) -> None:
    """Rotary embedding (+ QK-norm) and KV append for n positions from pos0."""
    hd = cache.head_dim
    stride = (n_q + 2 * cache.n_kv) * hd
    _require_cuda(qkv, "rope_cache_chunk: qkv", torch.float32)
    if qkv.numel() < n * stride:
        raise ShapeError(5, f"rope_cache_chunk: qkv[{qkv.numel()}] needs {n} * {stride}")
    if table.half_dim != hd // 2 or table.max_seq < cache.max_seq:
        raise ShapeError(5, "rope_cache_chunk: rotary table does not match the cache geometry")
    if pos0 + n > cache.max_seq:
        raise ShapeError(5, f"rope_cache_chunk: chunk [{pos0}, {pos0 + n}) runs past the "
                            f"{cache.max_seq} token cache")
    if qk_norm is not None and (qk_norm.q.numel() != hd or qk_norm.k.numel() != hd):
        raise ShapeError(5, f"rope_cache_chunk: gains are q[{qk_norm.q.numel()}], "
                            f"k[{qk_norm.k.numel()}]; both must be head_dim {hd}")
    qw, kw, eps = norm_ptrs(qk_norm)
    use_torch_stream()
    check(lib.wst_rope_cache_chunk(_ptr(qkv), _ptr(cache.k), _ptr(cache.v), _ptr(table.cos),
                                   _ptr(table.sin), n_q, cache.n_kv, hd, pos0, n,
                                   cache.max_seq, qw, kw, eps))


def attn(qkv: torch.Tensor, cache: KvCache, out: torch.Tensor, n_q: int, pos0: int,
         n: int) -> None:
    """Causal GQA attention: query j sees cache rows 0 ..= pos0+j."""
    hd = cache.head_dim
    stride = (n_q + 2 * cache.n_kv) * hd
    _require_cuda(qkv, "attn_chunk: qkv", torch.float32)
    _require_cuda(out, "attn_chunk: out", torch.float16)
    if qkv.numel() < n * stride:
        raise ShapeError(5, f"attn_chunk: qkv[{qkv.numel()}] needs {n} * {stride}")
    if out.numel() < n * n_q * hd:
        raise ShapeError(5, f"attn_chunk: out[{out.numel()}] needs {n} * {n_q} * {hd}")
    if pos0 + n > cache.max_seq:
        raise ShapeError(5, f"attn_chunk: chunk [{pos0}, {pos0 + n}) runs past the "
                            f"{cache.max_seq} token cache")
    scale = 1.0 / math.sqrt(hd)
    use_torch_stream()
    check(lib.wst_attn_chunk(_ptr(qkv), _ptr(cache.k), _ptr(cache.v), _ptr(out), n_q,
                             cache.n_kv, hd, pos0, n, cache.max_seq, scale))


def gemm_fp16(w: torch.Tensor, x: torch.Tensor, bias: torch.Tensor | None, y: torch.Tensor,
              in_features: int, out_features: int, n: int, accumulate: bool = False) -> None:
    """``y[j] = W x[j] + b`` for every ``j < n``, or ``+=`` when ``accumulate``
    (src/chunk.rs:55-99): w ``[out][in]`` and x ``[n][in]`` fp16, y ``[n][out]`` fp32."""
    _require_cuda(w, "gemm_fp16: w", torch.float16)
    _require_cuda(x, "gemm_fp16: x", torch.float16)
    _require_cuda(y, "gemm_fp16: y", torch.float32)
    if x.numel() != n * in_features or y.numel() != n * out_features:
        raise ShapeError(5, f"gemm_fp16: x[{x.numel()}], y[{y.numel()}] do not match n={n}, "
                            f"in={in_features}, out={out_features}")
    if w.numel() != in_features * out_features:
        raise ShapeError(5, f"gemm_fp16: weights have {w.numel()} elements, expected "
                            f"{in_features}*{out_features}")
    if bias is not None:
        _require_cuda(bias, "gemm_fp16: bias", torch.float16)
        if bias.numel() != out_features:
            raise ShapeError(5, f"gemm_fp16: bias has {bias.numel()} elements, expected "
                                f"{out_features}")
    use_torch_stream()
    check(lib.wst_gemm_fp16(_ptr(w), _ptr(x), _ptr(bias) if bias is not None else None, _ptr(y),
                            in_features, out_features, n, int(accumulate)))


def gemm_int4_hier(qw: torch.Tensor, si: torch.Tensor, sb: torch.Tensor, x: torch.Tensor,
                   bias: torch.Tensor | None, y: torch.Tensor, in_features: int,
                   out_features: int, n: int, accumulate: bool = False) -> None:
    """gemm_fp16 with weights in the hierarchical int4 format (QuantLinearHier::gemm_ex,
    src/gemv.rs): qw ``[out][in/32]`` 16-byte words as int32 x 4, si ``[out][in/32]`` uint8,
    sb ``[out]`` (d, dmin) fp16 pairs."""
    _require_cuda(qw, "gemm_int4_hier: qw", torch.int32)
    _require_cuda(si, "gemm_int4_hier: si", torch.uint8)
    _require_cuda(sb, "gemm_int4_hier: sb", torch.float16)
    _require_cuda(x, "gemm_int4_hier: x", torch.float16)
    _require_cuda(y, "gemm_int4_hier: y", torch.float32)
    if in_features % 32 != 0:
        raise ShapeError(5, "gemm_int4_hier: in_features must be a multiple of 32")
    groups = out_features * in_features // 32
    if qw.numel() != groups * 4 or si.numel() != groups or sb.numel() != 2 * out_features:
        raise ShapeError(5, f"gemm_int4_hier: qw[{qw.numel()}], si[{si.numel()}], sb[{sb.numel()}] "
                            f"do not match in={in_features}, out={out_features}")
    if x.numel() != n * in_features or y.numel() != n * out_features:
        raise ShapeError(5, f"gemm_int4_hier: x[{x.numel()}], y[{y.numel()}] do not match n={n}")
    if bias is not None:
        _require_cuda(bias, "gemm_int4_hier: bias", torch.float16)
        if bias.numel() != out_features:
            raise ShapeError(5, f"gemm_int4_hier: bias has {bias.numel()} elements")
    use_torch_stream()
    check(lib.wst_gemm_int4_hier(_ptr(qw), _ptr(si), _ptr(sb), _ptr(x),
                                 _ptr(bias) if bias is not None else None, _ptr(y), in_features,
                                 out_features, n, int(accumulate)))


def max_tokens() -> int:
    """Tokens one weight pass serves (src/chunk.rs:20)."""
    return max(1, lib.wst_chunk_max_tokens())


class KvCacheBatch:
    """Caches of n_seq sequences in one allocation, ``[n_seq][n_kv][max_seq][head_dim]``
    fp16 for K and V: what the batched chunk entry points take."""

    def __init__(self, n_seq: int, n_kv: int, head_dim: int, max_seq: int,
                 device: torch.device | str = "cuda"):
        shape = (n_seq, n_kv, max_seq, head_dim)
        self.k = torch.zeros(shape, dtype=torch.float16, device=device)
        self.v = torch.zeros(shape, dtype=torch.float16, device=device)
        self.n_seq, self.n_kv, self.head_dim, self.max_seq = n_seq, n_kv, head_dim, max_seq


def rope_cache_batch(qkv: torch.Tensor, cache: KvCacheBatch, table: RopeTable, n_q: int,
                     seq_pos0: torch.Tensor, n: int, qk_norm: QkNorm | None = None) -> None:
    """rope_cache for n tokens of each of the batch's sequences (qkv [n_seq][n][width])."""
    hd = cache.head_dim
    stride = (n_q + 2 * cache.n_kv) * hd
    _require_cuda(qkv, "rope_cache_chunk_batch: qkv", torch.float32)
    _require_cuda(seq_pos0, "rope_cache_chunk_batch: seq_pos0", torch.int32)
    if qkv.numel() < cache.n_seq * n * stride:
        raise ShapeError(5, f"rope_cache_chunk_batch: qkv[{qkv.numel()}] needs "
                            f"{cache.n_seq} * {n} * {stride}")
    if seq_pos0.numel() != cache.n_seq:
        raise ShapeError(5, "rope_cache_chunk_batch: seq_pos0 needs one entry per sequence")
    if table.half_dim != hd // 2 or table.max_seq < cache.max_seq:
        raise ShapeError(5, "rope_cache_chunk_batch: rotary table does not match the cache geometry")
    if qk_norm is not None:
        qk_norm.check(hd)
    qw, kw, eps = norm_ptrs(qk_norm)
    use_torch_stream()
    check(lib.wst_rope_cache_chunk_batch(_ptr(qkv), _ptr(cache.k), _ptr(cache.v), _ptr(table.cos),
                                         _ptr(table.sin), _ptr(seq_pos0), cache.n_seq, n_q,
                                         cache.n_kv, hd, n, cache.max_seq, qw, kw, eps))


def attn_batch(qkv: torch.Tensor, cache: KvCacheBatch, out: torch.Tensor, n_q: int,
               seq_pos0: torch.Tensor, n: int) -> None:
    """Causal attention of n tokens per sequence; out [n_seq][n][n_q*head_dim] fp16."""
    hd = cache.head_dim
    stride = (n_q + 2 * cache.n_kv) * hd
    _require_cuda(qkv, "attn_chunk_batch: qkv", torch.float32)
    _require_cuda(out, "attn_chunk_batch: out", torch.float16)
    _require_cuda(seq_pos0, "attn_chunk_batch: seq_pos0", torch.int32)
    if qkv.numel() < cache.n_seq * n * stride:
        raise ShapeError(5, f"attn_chunk_batch: qkv[{qkv.numel()}] needs {cache.n_seq} * {n} * {stride}")
    if out.numel() < cache.n_seq * n * n_q * hd:
        raise ShapeError(5, f"attn_chunk_batch: out[{out.numel()}] needs {cache.n_seq} * {n} * {n_q} * {hd}")
    use_torch_stream()
    check(lib.wst_attn_chunk_batch(_ptr(qkv), _ptr(cache.k), _ptr(cache.v), _ptr(out),
                                   _ptr(seq_pos0), cache.n_seq, n_q, cache.n_kv, hd, n,
                                   cache.max_seq, 1.0 / math.sqrt(hd)))


__all__ = ["rope_cache", "attn", "KvCacheBatch", "rope_cache_batch", "attn_batch"]


def qkv_rope_append_batch(w: torch.Tensor, x: torch.Tensor, bias: torch.Tensor | None,
                          q_out: torch.Tensor, cache: KvCacheBatch, table: RopeTable, n_q: int,
                          seq_pos0: torch.Tensor, n: int, qk_norm: QkNorm | None = None) -> None:
    """The qkv projection of n tokens per sequence with RoPE, head norm and cache append in
    its epilogue: x [n_seq * n][in] fp16, w [(n_q + 2 n_kv) * hd][in] fp16; the rotated
    queries land in q_out [n_seq * n][n_q * hd] fp16, k and v in the batched cache."""
    hd = cache.head_dim
    width = (n_q + 2 * cache.n_kv) * hd
    tokens = cache.n_seq * n
    _require_cuda(w, "qkv_rope_append_batch: w", torch.float16)
    _require_cuda(x, "qkv_rope_append_batch: x", torch.float16)
    _require_cuda(q_out, "qkv_rope_append_batch: q_out", torch.float16)
    _require_cuda(seq_pos0, "qkv_rope_append_batch: seq_pos0", torch.int32)
    if x.numel() % tokens != 0:
        raise ShapeError(5, f"qkv_rope_append_batch: x[{x.numel()}] is not {tokens} rows")
    in_f = x.numel() // tokens
    if w.numel() != width * in_f:
        raise ShapeError(5, f"qkv_rope_append_batch: w[{w.numel()}] needs {width} * {in_f}")
    if q_out.numel() < tokens * n_q * hd:
        raise ShapeError(5, f"qkv_rope_append_batch: q_out[{q_out.numel()}] needs {tokens} * {n_q} * {hd}")
    if bias is not None:
        _require_cuda(bias, "qkv_rope_append_batch: bias", torch.float16)
        if bias.numel() != width:
            raise ShapeError(5, f"qkv_rope_append_batch: bias has {bias.numel()} elements, expected {width}")
    if seq_pos0.numel() != cache.n_seq:
        raise ShapeError(5, "qkv_rope_append_batch: seq_pos0 needs one entry per sequence")
    if table.half_dim != hd // 2:
        raise ShapeError(5, "qkv_rope_append_batch: rotary table does not match the head width")
    if qk_norm is not None:
        qk_norm.check(hd)
    qw, kw, eps = norm_ptrs(qk_norm)
    use_torch_stream()
    check(lib.wst_b200_qkv_rope_append_batch(
        _ptr(w), _ptr(x), _ptr(bias) if bias is not None else None, _ptr(q_out), _ptr(cache.k),
        _ptr(cache.v), _ptr(table.cos), _ptr(table.sin), _ptr(seq_pos0), in_f, cache.n_seq, n, n_q,
        cache.n_kv, hd, cache.max_seq, table.max_seq, qw, kw, eps))


def qkv_int4_rope_append_batch(qw: torch.Tensor, si: torch.Tensor, sb: torch.Tensor, x: torch.Tensor,
                               bias: torch.Tensor | None, q_out: torch.Tensor, cache: KvCacheBatch,
                               table: RopeTable, n_q: int, seq_pos0: torch.Tensor, n: int,
                               qk_norm: QkNorm | None = None) -> None:
    """qkv_rope_append_batch with the qkv weights in the hierarchical int4 format
    (gemm_int4_hier's qw, si, sb)."""
    hd = cache.head_dim
    width = (n_q + 2 * cache.n_kv) * hd
    tokens = cache.n_seq * n
    _require_cuda(qw, "qkv_int4_rope_append_batch: qw", torch.int32)
    _require_cuda(si, "qkv_int4_rope_append_batch: si", torch.uint8)
    _require_cuda(sb, "qkv_int4_rope_append_batch: sb", torch.float16)
    _require_cuda(x, "qkv_int4_rope_append_batch: x", torch.float16)
    _require_cuda(q_out, "qkv_int4_rope_append_batch: q_out", torch.float16)
    if x.numel() % tokens != 0:
        raise ShapeError(5, f"qkv_int4_rope_append_batch: x[{x.numel()}] is not {tokens} rows")
    in_f = x.numel() // tokens
    groups = width * in_f // 32
    if in_f % 32 != 0 or qw.numel() != groups * 4 or si.numel() != groups or sb.numel() != 2 * width:
        raise ShapeError(5, "qkv_int4_rope_append_batch: packed weights do not match the shape")
    if q_out.numel() < tokens * n_q * hd:
        raise ShapeError(5, f"qkv_int4_rope_append_batch: q_out[{q_out.numel()}] is too short")
    if qk_norm is not None:
        qk_norm.check(hd)
    qwp, kwp, eps = norm_ptrs(qk_norm)
    use_torch_stream()
    check(lib.wst_b200_qkv_int4_rope_append_batch(
        _ptr(qw), _ptr(si), _ptr(sb), _ptr(x), _ptr(bias) if bias is not None else None, _ptr(q_out),
        _ptr(cache.k), _ptr(cache.v), _ptr(table.cos), _ptr(table.sin), _ptr(seq_pos0), in_f,
        cache.n_seq, n, n_q, cache.n_kv, hd, cache.max_seq, table.max_seq, qwp, kwp, eps))


def attn_batch_q16(q16: torch.Tensor, cache: KvCacheBatch, out: torch.Tensor, n_q: int,
                   seq_pos0: torch.Tensor, n: int) -> None:
    """attn_batch over fp16 query rows [n_seq * n][n_q * head_dim] (what
    qkv_rope_append_batch leaves)."""
    hd = cache.head_dim
    _require_cuda(q16, "attn_chunk_batch_q16: q", torch.float16)
    _require_cuda(out, "attn_chunk_batch_q16: out", torch.float16)
    _require_cuda(seq_pos0, "attn_chunk_batch_q16: seq_pos0", torch.int32)
    need = cache.n_seq * n * n_q * hd
    if q16.numel() < need or out.numel() < need:
        raise ShapeError(5, f"attn_chunk_batch_q16: q[{q16.numel()}] and out[{out.numel()}] need {need}")
    use_torch_stream()
    check(lib.wst_b200_attn_chunk_batch_q16(_ptr(q16), _ptr(cache.k), _ptr(cache.v), _ptr(out),
                                            _ptr(seq_pos0), cache.n_seq, n_q, cache.n_kv, hd, n,
                                            cache.max_seq, 1.0 / math.sqrt(hd)))

