"""The five benchmark workloads as seeded synthetic inputs.

Only the layer SHAPES come from the named model architectures; every tensor is
drawn from numpy's PCG64 (``default_rng(seed)``), rounded through fp16 and
widened, so that the CUDA path and any checker consume bit-identical numbers.
No weights, prompts or dataset items are involved.

    c1  Qwen2.5-0.5B decode, 24 layers, 14 q / 2 kv heads, head_dim 64, 512 cached tokens
    c2  Qwen2.5-0.5B chunked prefill, 2048 tokens as 8 chunks of 256
    c3  Qwen2.5-7B long-context decode, 28 layers, 28/4/128, context 32768
    c4  Qwen3-8B batched chunked prefill, 36 layers, 32/8/128, 4 x 8192 tokens, 512-token
        chunks, QK-norm (eps 1e-6, gains ~ N(1, 0.02))
    c5  Qwen2.5-7B speculative verify, 28/4/128, 16 sequences x 5 draft tokens over a paged
        cache (16-token pages), lengths uniform in [1024, 16384]
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np


@dataclass(frozen=True)
class Shape:
    name: str
    n_q: int
    n_kv: int
    head_dim: int
    layers: int
    theta: float = 1e6

    @property
    def gqa(self) -> int:
        return self.n_q // self.n_kv

    @property
    def qkv_width(self) -> int:
        return (self.n_q + 2 * self.n_kv) * self.head_dim

    @property
    def scale(self) -> float:
        return 1.0 / float(np.sqrt(self.head_dim))


QWEN25_05B = Shape("qwen2.5-0.5b", 14, 2, 64, 24)
QWEN25_7B = Shape("qwen2.5-7b", 28, 4, 128, 28)
QWEN3_8B = Shape("qwen3-8b", 32, 8, 128, 36)

C1 = dict(shape=QWEN25_05B, cached=512, max_seq=1024, seed=1000)
C2 = dict(shape=QWEN25_05B, prompt=2048, chunk=256, max_seq=2048, seed=2000)
C3 = dict(shape=QWEN25_7B, context=32768, seed=3000)
C4 = dict(shape=QWEN3_8B, n_seq=4, prompt=8192, chunk=512, eps=1e-6, seed=4000)
C5 = dict(shape=QWEN25_7B, n_seq=16, drafts=5, page=16, len_lo=1024, len_hi=16384, seed=5000)


def f16_values(rng: np.random.Generator, shape, dtype=np.float32) -> np.ndarray:
    """N(0,1) rounded through fp16, returned in `dtype` (fp32 for the ABI's qkv,
    fp16 for caches)."""
    x = rng.standard_normal(shape, dtype=np.float32).astype(np.float16)
    return x if dtype == np.float16 else x.astype(dtype)


def qk_gains(rng: np.random.Generator, head_dim: int):
    """QK-norm gains ~ N(1, 0.02), fp16 (config c4)."""
    q = (1.0 + 0.02 * rng.standard_normal(head_dim)).astype(np.float16)
    k = (1.0 + 0.02 * rng.standard_normal(head_dim)).astype(np.float16)
    return q, k


def c1_layer(layer: int):
    """qkv [18*64] fp32, K/V cache [2][1024][64] fp16 with rows 0..511 filled."""
    s, cfg = QWEN25_05B, C1
    rng = np.random.default_rng(cfg["seed"] + layer)
    qkv = f16_values(rng, (s.qkv_width,))
    k = np.zeros((s.n_kv, cfg["max_seq"], s.head_dim), dtype=np.float16)
    v = np.zeros_like(k)
    k[:, : cfg["cached"]] = f16_values(rng, (s.n_kv, cfg["cached"], s.head_dim), np.float16)
    v[:, : cfg["cached"]] = f16_values(rng, (s.n_kv, cfg["cached"], s.head_dim), np.float16)
    return qkv, k, v


def c2_layer(layer: int):
    """qkv for the whole 2048-token prompt, [2048][18*64] fp32."""
    s, cfg = QWEN25_05B, C2
    rng = np.random.default_rng(cfg["seed"] + layer)
    return f16_values(rng, (cfg["prompt"], s.qkv_width))


def c3_layer(layer: int, context: int | None = None):
    """q [28][128] fp32 and a fully populated K/V cache [4][context][128] fp16
    (treated as already rotated)."""
    s, cfg = QWEN25_7B, C3
    ctx = context or cfg["context"]
    rng = np.random.default_rng(cfg["seed"] + layer)
    q = f16_values(rng, (s.n_q, s.head_dim))
    k = f16_values(rng, (s.n_kv, ctx, s.head_dim), np.float16)
    v = f16_values(rng, (s.n_kv, ctx, s.head_dim), np.float16)
    return q, k, v


def c4_chunk(layer: int, seq: int, chunk_idx: int, chunk: int | None = None):
    """qkv [chunk][48*128] fp32 for one (layer, sequence, chunk)."""
    s, cfg = QWEN3_8B, C4
    n = chunk or cfg["chunk"]
    rng = np.random.default_rng([cfg["seed"] + layer, seq, chunk_idx])
    return f16_values(rng, (n, s.qkv_width))


def c4_gains(layer: int):
    rng = np.random.default_rng([C4["seed"] + layer, 9999])
    return qk_gains(rng, QWEN3_8B.head_dim)


def c5_lengths(n_seq: int | None = None, lo: int | None = None, hi: int | None = None,
               seed: int | None = None) -> np.ndarray:
    """Per-sequence context lengths, uniform on the inclusive range."""
    cfg = C5
    rng = np.random.default_rng(cfg["seed"] if seed is None else seed)
    return rng.integers(lo or cfg["len_lo"], (hi or cfg["len_hi"]) + 1,
                        size=n_seq or cfg["n_seq"]).astype(np.int32)


def c5_page_table(lengths: np.ndarray, drafts: int, page: int = 16, seed: int | None = None):
    """A page table whose pages are a seeded permutation of the pool, so that no
    sequence is contiguous.  Returns (table [n_seq][max_pages] int32, n_pages)."""
    need = (lengths.astype(np.int64) + drafts + page - 1) // page
    max_pages = int(need.max())
    total = int(need.sum())
    rng = np.random.default_rng((C5["seed"] if seed is None else seed) + 1)
    perm = rng.permutation(total).astype(np.int32)
    table = np.full((len(lengths), max_pages), -1, dtype=np.int32)
    at = 0
    for s, n in enumerate(need):
        table[s, :n] = perm[at:at + n]
        at += int(n)
    return table, total


def c5_fill_manager(manager, lengths: np.ndarray, seed: int | None = None):
    """Brings one sequence per entry of `lengths` up to its length in a page manager
    (whetstone_b200.paged.PagedKvManager), growing the sequences in seeded random turns
    of one to four pages so that their pages interleave in the pool (no sequence is
    contiguous).  Returns the sequence ids in the order of `lengths`."""
    rng = np.random.default_rng((C5["seed"] if seed is None else seed) + 2)
    ids = [manager.open() for _ in lengths]
    left = [int(n) for n in lengths]
    while any(left):
        i = int(rng.integers(0, len(left)))
        if not left[i]:
            continue
        n = min(left[i], 16 * int(rng.integers(1, 5)))
        manager.reserve(ids[i], n)
        manager.commit(ids[i], n)
        left[i] -= n
    return ids


def prefill_flops(n_q: int, head_dim: int, pos0: int, n: int) -> int:
    """Causal-exact FLOPs of one chunk: 4 * head_dim * n_q * sum_j (pos0 + j + 1)."""
    pairs = n * pos0 + n * (n + 1) // 2
    return 4 * head_dim * n_q * pairs


def decode_bytes(n_q: int, n_kv: int, head_dim: int, seq: int) -> int:
    """Algorithmic bytes of one decode-attention layer step: K and V rows read
    once (fp16), q read (fp32), out written (fp16)."""
    return 2 * n_kv * seq * head_dim * 2 + n_q * head_dim * 4 + n_q * head_dim * 2
