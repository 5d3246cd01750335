"""A serving loop driven through the host-side page manager and scheduler
(whetstone_b200/host/paged_kv.hpp): ragged prefill steps picked by the scheduler, then
rounds of propose / verify / rewind as in crates/whetstone-core/src/speculate.rs:185-256
-- for several sequences over one page pool, with a sequence that finishes and a new
one that inherits its pages (stale rows and all).  Every attention output is checked
against the numpy oracle; every appended row lands in the pages the manager handed out."""

import numpy as np
import pytest
import torch

from oracle import attention_oracle as orc
from tests.helpers import NAN16, assert_close_per_head, dev, fill_bits, host
from whetstone_b200 import decode, paged, workloads

pytestmark = pytest.mark.gpu


def test_prefill_verify_rewind_loop_over_a_shared_pool():
    shape = workloads.QWEN25_7B
    n_q, n_kv, hd, theta = shape.n_q, shape.n_kv, shape.head_dim, 1e6
    rng = np.random.default_rng(2024)
    max_len, pool_pages, slots, drafts = 700, 150, 6, 5
    kv = paged.PagedKvManager(pool_pages, max_len)
    cache = paged.PagedKvCache(pool_pages, n_kv, hd, slots, kv.max_pages)
    fill_bits(cache.k, NAN16)       # a row nobody appended must never be read
    fill_bits(cache.v, NAN16)
    rtab = decode.RopeTable(max_len, hd, theta)
    scratch = torch.empty(paged.verify_scratch_floats(slots, 18, n_q, n_kv, hd, max_len),
                          dtype=torch.float32, device="cuda")

    live = {}        # seq id -> dict(k, v: committed rows [len][n_kv][hd] f64, todo: prompt rows left)

    def new_sequence(prompt_len):
        s = kv.open()
        live[s] = dict(k=np.zeros((0, n_kv, hd)), v=np.zeros((0, n_kv, hd)), todo=prompt_len)
        return s

    def run_step(entries, accept=None):
        """Append + attend for `entries`; commit; rewind each sequence to pos0 + accept + 1
        when `accept` is given (speculative round), keep everything otherwise (prefill)."""
        step = kv.build_step(entries)
        pos0, cu = step.upload(cache)
        qkv = workloads.f16_values(rng, (step.total_tokens, shape.qkv_width))
        qd = dev(qkv)
        out = torch.zeros(step.total_tokens * n_q * hd, dtype=torch.float16, device="cuda")
        paged.rope_cache(qd, cache, rtab, n_q, pos0, cu, step.total_tokens)
        paged.attn_verify(qd, cache, out, scratch, n_q, pos0, cu, step.total_tokens,
                          step.max_tokens_per_seq, step.max_len)
        got = host(out).astype(np.float64).reshape(step.total_tokens, n_q, hd)
        for i, (s, n) in enumerate(step.entries):
            L = int(step.seq_pos0[i])
            assert L == kv.length(s) == len(live[s]["k"])
            rows = qkv[step.cu_tokens[i]:step.cu_tokens[i + 1]]
            qr, kr, vv = orc.rope_append(rows, L + np.arange(n), n_q, n_kv, hd, theta)
            k_all = np.concatenate([live[s]["k"], kr])
            v_all = np.concatenate([live[s]["v"], vv])
            want = orc.attention_blocked(qr, k_all, v_all, L + 1 + np.arange(n))
            assert_close_per_head(got[step.cu_tokens[i]:step.cu_tokens[i + 1]], want,
                                  f"sequence {s} at {L}, {n} tokens")
            kv.commit(s, n)
            keep = n if accept is None else accept[s] + 1
            kv.rewind(s, L + keep)
            live[s]["k"], live[s]["v"] = k_all[:L + keep], v_all[:L + keep]
        assert decode.device_error() == 0

    # ---- prefill: five prompts, at most 40 tokens and 4 sequences per step, 18 per sequence
    for plen in (130, 17, 300, 64, 201):
        new_sequence(plen)
    steps = 0
    while any(st["todo"] for st in live.values()):
        waiting = [(s, min(st["todo"], 18)) for s, st in live.items() if st["todo"]]
        entries = kv.schedule(waiting, max_tokens_per_step=40, max_sequences_per_step=4)
        assert entries and sum(n for _, n in entries) <= 40
        lens = [kv.length(s) + n for s, n in entries]
        assert lens == sorted(lens, reverse=True)          # longest context first
        run_step(entries)
        for s, n in entries:
            live[s]["todo"] -= n
        steps += 1
    assert steps >= 18 and {kv.length(s) for s in live} == {130, 17, 300, 64, 201}

    # ---- speculative rounds: 1 + 5 rows per sequence, a random number of drafts accepted
    for rnd in range(4):
        ids = sorted(live)
        accept = {s: int(rng.integers(0, drafts + 1)) for s in ids}
        before = {s: kv.length(s) for s in ids}
        run_step(kv.schedule([(s, 1 + drafts) for s in ids], 1000, slots), accept)
        for s in ids:
            assert kv.length(s) == before[s] + accept[s] + 1
        if rnd == 1:
            # the longest sequence finishes; a new one takes over its pages, stale rows included
            gone = max(ids, key=kv.length)
            free = kv.free_pages()
            kv.close(gone)
            del live[gone]
            assert kv.free_pages() > free
            fresh = new_sequence(33)
            assert fresh == gone                            # the id is reused
            run_step([(fresh, 18)])
            run_step([(fresh, 15)])
            live[fresh]["todo"] = 0
    # every page is either free or owned by exactly one live sequence
    owned = sum(kv.pages(s) for s in live)
    assert owned + kv.free_pages() == pool_pages
