"""The five benchmark configurations at their full sizes, CUDA path against the
numpy oracle on the same seeded inputs (whetstone_b200/workloads.py).  Where the
oracle for a whole configuration would take minutes, a stated subset of layers /
sequences / chunks is checked against it and the rest through size-independent
properties (chunk path == single-token path; sharded == unsharded)."""

import numpy as np
import pytest
import torch

from oracle import attention_oracle as orc
from tests.helpers import (NAN16, SENTINEL, assert_close_per_head, assert_k_cache_matches, bits16,
                           dev, f16_ulp_distance, fill_bits, fill_rows_from, host)
from whetstone_b200 import chunk, decode, paged, workloads as wl

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def no_watchdog_trips():
    yield
    assert decode.device_error() == 0


def test_c1_decode_all_24_layers():
    s, cfg = wl.QWEN25_05B, wl.C1
    pos, max_seq = cfg["cached"], cfg["max_seq"]
    table = decode.RopeTable(max_seq, s.head_dim, s.theta)
    cur = decode.DeviceCursor(pos)
    for layer in range(s.layers):
        qkv, k, v = wl.c1_layer(layer)
        cache = decode.KvCache(s.n_kv, s.n_q, s.head_dim, max_seq)
        cache.k.copy_(dev(k))
        cache.v.copy_(dev(v))
        fill_rows_from(cache.k, NAN16, pos)
        fill_rows_from(cache.v, NAN16, pos)
        qd = dev(qkv)
        out = torch.zeros(s.n_q * s.head_dim, dtype=torch.float16, device="cuda")
        decode.rope_cache(qd, cache, table, s.n_q, cur)
        decode.attn_decode(qd, cache, out, s.n_q, cur)
        qr, kr, vv = orc.rope_append(qkv[None], np.array([pos]), s.n_q, s.n_kv, s.head_dim, s.theta)
        k_all = np.concatenate([k[:, :pos].astype(np.float64), kr.transpose(1, 0, 2)], axis=1)
        v_all = np.concatenate([v[:, :pos].astype(np.float64), vv.transpose(1, 0, 2)], axis=1)
        want = orc.decode_attention(qr[0], k_all, v_all, pos + 1, s.scale)
        assert_close_per_head(host(out).astype(np.float64).reshape(s.n_q, s.head_dim), want,
                              f"c1 layer {layer}")
        # the append touched row `pos` only
        kb = bits16(cache.k)
        assert np.array_equal(kb[:, :pos], k[:, :pos].view(np.uint16))
        assert np.all(kb[:, pos + 1:] == NAN16)


@pytest.mark.parametrize("layer", [0, 23])
def test_c2_chunked_prefill_2048_tokens(layer):
    s, cfg = wl.QWEN25_05B, wl.C2
    n, prompt = cfg["chunk"], cfg["prompt"]
    qkv = wl.c2_layer(layer)
    table = decode.RopeTable(prompt, s.head_dim, s.theta)
    cache = decode.KvCache(s.n_kv, s.n_q, s.head_dim, prompt)
    fill_bits(cache.k, SENTINEL)
    fill_bits(cache.v, SENTINEL)
    qd = dev(qkv)
    out = torch.zeros(prompt * s.n_q * s.head_dim, dtype=torch.float16, device="cuda")
    width = s.n_q * s.head_dim
    for c in range(prompt // n):
        rows = qd[c * n:(c + 1) * n]
        chunk.rope_cache(rows, cache, table, s.n_q, c * n, n)
        # rows beyond the chunk are still untouched
        if c + 1 < prompt // n:
            assert int(bits16(cache.k[:, (c + 1) * n])[0, 0]) == SENTINEL
        chunk.attn(rows, cache, out[c * n * width:], s.n_q, c * n, n)
    qr, kr, vv = orc.rope_append(qkv, np.arange(prompt), s.n_q, s.n_kv, s.head_dim, s.theta)
    want = orc.attention_blocked(qr, kr, vv, 1 + np.arange(prompt), s.scale)
    assert_close_per_head(host(out).astype(np.float64).reshape(prompt, s.n_q, s.head_dim), want,
                          f"c2 layer {layer}")
    assert np.array_equal(bits16(cache.v), vv.transpose(1, 0, 2).astype(np.float16).view(np.uint16))
    assert f16_ulp_distance(bits16(cache.k),
                            kr.transpose(1, 0, 2).astype(np.float16).view(np.uint16)).max() <= 1


@pytest.mark.parametrize("layer", [0, 27])
def test_c3_decode_at_32k_context(layer):
    s = wl.QWEN25_7B
    ctx = wl.C3["context"]
    q, k, v = wl.c3_layer(layer)
    cache = decode.KvCache(s.n_kv, s.n_q, s.head_dim, ctx)
    cache.k.copy_(dev(k))
    cache.v.copy_(dev(v))
    out = torch.zeros(s.n_q * s.head_dim, dtype=torch.float16, device="cuda")
    decode.attn_decode(dev(q), cache, out, s.n_q, decode.DeviceCursor(ctx - 1))
    want = orc.decode_attention(q, k, v, ctx, s.scale)
    got = host(out).astype(np.float64).reshape(s.n_q, s.head_dim)
    assert_close_per_head(got, want, f"c3 layer {layer}")

    # the same sequence sharded 8 ways gives the same answer after the merge
    shards = 8
    per = ctx // shards
    parts = torch.zeros((shards, s.n_q, s.head_dim + 2), dtype=torch.float32, device="cuda")
    qd = dev(q)
    for g in range(shards):
        shard = decode.KvCache(s.n_kv, s.n_q, s.head_dim, per)
        shard.k.copy_(cache.k[:, g * per:(g + 1) * per])
        shard.v.copy_(cache.v[:, g * per:(g + 1) * per])
        decode.attn_decode_partial(qd, shard, parts[g], s.n_q,
                                   torch.tensor([per], dtype=torch.int32, device="cuda"))
    merged = torch.zeros(s.n_q * s.head_dim, dtype=torch.float16, device="cuda")
    decode.attn_merge_partials(parts, merged, s.n_q, s.head_dim)
    assert_close_per_head(host(merged).astype(np.float64).reshape(s.n_q, s.head_dim), want,
                          f"c3 layer {layer}, 8 shards")


def test_c4_batched_prefill_with_qk_norm():
    """Layer 0.  Sequence 1 is appended in full (16 chunks of 512, QK-norm) and its
    chunks 0, 1 and 15 are checked against the oracle; sequence 3 is checked
    through the property that a chunk row equals the single-token path."""
    s, cfg = wl.QWEN3_8B, wl.C4
    n, prompt, eps = cfg["chunk"], cfg["prompt"], cfg["eps"]
    chunks = prompt // n
    gq, gk = wl.c4_gains(0)
    norm = decode.QkNorm(dev(gq), dev(gk), eps)
    table = decode.RopeTable(prompt, s.head_dim, s.theta)
    width = s.n_q * s.head_dim

    # ---- sequence 1 against the oracle
    seq = 1
    cache = decode.KvCache(s.n_kv, s.n_q, s.head_dim, prompt)
    fill_bits(cache.k, NAN16)
    fill_bits(cache.v, NAN16)
    k_all = np.zeros((prompt, s.n_kv, s.head_dim))
    v_all = np.zeros((prompt, s.n_kv, s.head_dim))
    for c in range(chunks):
        qkv = wl.c4_chunk(0, seq, c)
        qd = dev(qkv)
        chunk.rope_cache(qd, cache, table, s.n_q, c * n, n, norm)
        qr, k_all[c * n:(c + 1) * n], v_all[c * n:(c + 1) * n] = orc.rope_append(
            qkv, c * n + np.arange(n), s.n_q, s.n_kv, s.head_dim, s.theta, gq, gk, eps)
        if c in (0, 1, chunks - 1):
            out = torch.zeros(n * width, dtype=torch.float16, device="cuda")
            chunk.attn(qd, cache, out, s.n_q, c * n, n)
            want = orc.attention_blocked(qr, k_all[:(c + 1) * n], v_all[:(c + 1) * n],
                                         c * n + 1 + np.arange(n), s.scale)
            assert_close_per_head(host(out).astype(np.float64).reshape(n, s.n_q, s.head_dim),
                                  want, f"c4 seq {seq} chunk {c}")
    assert np.array_equal(bits16(cache.v), v_all.transpose(1, 0, 2).astype(np.float16).view(np.uint16))
    assert_k_cache_matches(bits16(cache.k), k_all.transpose(1, 0, 2), "c4 K cache")

    # ---- sequence 3: chunk rows == single-token decode on the same cache
    seq = 3
    cache3 = decode.KvCache(s.n_kv, s.n_q, s.head_dim, prompt)
    last = None
    for c in range(chunks):
        last = dev(wl.c4_chunk(0, seq, c))
        chunk.rope_cache(last, cache3, table, s.n_q, c * n, n, norm)
    c = chunks - 1
    out = torch.zeros(n * width, dtype=torch.float16, device="cuda")
    chunk.attn(last, cache3, out, s.n_q, c * n, n)
    got = host(out).astype(np.float64).reshape(n, s.n_q, s.head_dim)
    for j in (0, 257, n - 1):
        one = torch.zeros(width, dtype=torch.float16, device="cuda")
        decode.attn_decode(last[j].contiguous(), cache3, one, s.n_q, decode.DeviceCursor(c * n + j))
        assert_close_per_head(got[j], host(one).astype(np.float64).reshape(s.n_q, s.head_dim),
                              f"c4 seq {seq} token {c * n + j} vs single-token path")


def test_c4_through_the_batched_entry_points_at_full_size():
    """Layer 0 the way the benchmark runs it: one batched cache [4][8][8192][128], every
    chunk step ONE wst_rope_cache_chunk_batch (QK-norm gains of the config) and ONE
    wst_attn_chunk_batch over the four sequences, chunk starts in device memory.
    Chunks 0, 1 and 15 of sequences 0 and 2 against the oracle (chunk 15 on a spread of
    its 512 rows: the oracle needs seconds per 100 rows at 8192 keys); V bits exact and K
    within one fp16 ulp over the whole batched cache of those sequences."""
    s, cfg = wl.QWEN3_8B, wl.C4
    n, prompt, eps, n_seq = cfg["chunk"], cfg["prompt"], cfg["eps"], cfg["n_seq"]
    chunks = prompt // n
    gq, gk = wl.c4_gains(0)
    norm = decode.QkNorm(dev(gq), dev(gk), eps)
    table = decode.RopeTable(prompt, s.head_dim, s.theta)
    batch = chunk.KvCacheBatch(n_seq, s.n_kv, s.head_dim, prompt)
    fill_bits(batch.k, NAN16)
    fill_bits(batch.v, NAN16)
    checked = (0, 2)
    k_all = {q: np.zeros((prompt, s.n_kv, s.head_dim)) for q in checked}
    v_all = {q: np.zeros((prompt, s.n_kv, s.head_dim)) for q in checked}
    out = torch.zeros(n_seq * n * s.n_q * s.head_dim, dtype=torch.float16, device="cuda")
    spread = np.unique(np.concatenate([np.arange(0, 40), np.arange(250, 262), np.arange(n - 36, n)]))
    for c in range(chunks):
        qkv = np.stack([wl.c4_chunk(0, q, c) for q in range(n_seq)])
        qd = dev(qkv)
        starts = torch.full((n_seq,), c * n, dtype=torch.int32, device="cuda")
        chunk.rope_cache_batch(qd, batch, table, s.n_q, starts, n, norm)
        rotated = {}
        for q in checked:
            rotated[q], k_all[q][c * n:(c + 1) * n], v_all[q][c * n:(c + 1) * n] = orc.rope_append(
                qkv[q], c * n + np.arange(n), s.n_q, s.n_kv, s.head_dim, s.theta, gq, gk, eps)
        if c not in (0, 1, chunks - 1):
            continue
        chunk.attn_batch(qd, batch, out, s.n_q, starts, n)
        got = host(out).astype(np.float64).reshape(n_seq, n, s.n_q, s.head_dim)
        rows = np.arange(n) if c < 2 else spread
        for q in checked:
            want = orc.attention_blocked(rotated[q][rows], k_all[q][:(c + 1) * n],
                                         v_all[q][:(c + 1) * n], c * n + 1 + rows, s.scale)
            assert_close_per_head(got[q][rows], want, f"c4 batched, sequence {q}, chunk {c}")
    for q in checked:
        assert np.array_equal(bits16(batch.v[q]),
                              v_all[q].transpose(1, 0, 2).astype(np.float16).view(np.uint16))
        assert_k_cache_matches(bits16(batch.k[q]), k_all[q].transpose(1, 0, 2),
                               f"c4 batched K cache, sequence {q}")
    assert decode.device_error() == 0


def test_c5_paged_verify_16_sequences():
    s, cfg = wl.QWEN25_7B, wl.C5
    drafts = cfg["drafts"]
    lengths = wl.c5_lengths()
    assert lengths.min() >= cfg["len_lo"] and lengths.max() <= cfg["len_hi"] and len(lengths) == 16
    table_np, n_pages = wl.c5_page_table(lengths, drafts)
    n_seq = len(lengths)
    rng = np.random.default_rng(cfg["seed"] + 2)
    cache = paged.PagedKvCache(n_pages, s.n_kv, s.head_dim, n_seq, table_np.shape[1])
    pool_k = wl.f16_values(rng, tuple(cache.k.shape), np.float16)
    pool_v = wl.f16_values(rng, tuple(cache.v.shape), np.float16)
    # rows at and beyond each sequence's length are not live: poison them
    for q_, L in enumerate(lengths):
        for p in range(int(L), int(-(-(L + drafts) // 16) * 16)):
            pool_k[table_np[q_, p // 16], :, p % 16] = np.float16(np.nan)
            pool_v[table_np[q_, p // 16], :, p % 16] = np.float16(np.nan)
    cache.k.copy_(dev(pool_k))
    cache.v.copy_(dev(pool_v))
    cache.page_table.copy_(dev(table_np))
    total = n_seq * drafts
    qkv = wl.f16_values(rng, (total, s.qkv_width))
    qd = dev(qkv)
    pos0 = dev(lengths)
    cu = dev(np.arange(n_seq + 1, dtype=np.int32) * drafts)
    max_len = int(lengths.max()) + drafts
    rtab = decode.RopeTable(max_len, s.head_dim, s.theta)
    paged.rope_cache(qd, cache, rtab, s.n_q, pos0, cu, total)
    scratch = torch.empty(paged.verify_scratch_floats(n_seq, drafts, s.n_q, s.n_kv, s.head_dim,
                                                      max_len), dtype=torch.float32, device="cuda")
    out = torch.zeros(total * s.n_q * s.head_dim, dtype=torch.float16, device="cuda")
    paged.attn_verify(qd, cache, out, scratch, s.n_q, pos0, cu, total, drafts, max_len)
    got = host(out).astype(np.float64).reshape(n_seq, drafts, s.n_q, s.head_dim)
    for q_, L in enumerate(lengths):
        L = int(L)
        rows = qkv[q_ * drafts:(q_ + 1) * drafts]
        qr, kr, vv = orc.rope_append(rows, L + np.arange(drafts), s.n_q, s.n_kv, s.head_dim, s.theta)
        kc = orc.gather_pages(pool_k, table_np[q_], L).astype(np.float64).transpose(1, 0, 2)
        vc = orc.gather_pages(pool_v, table_np[q_], L).astype(np.float64).transpose(1, 0, 2)
        want = orc.attention_blocked(qr, np.concatenate([kc, kr]), np.concatenate([vc, vv]),
                                     L + 1 + np.arange(drafts), s.scale)
        assert_close_per_head(got[q_], want, f"c5 sequence {q_} (length {L})")
