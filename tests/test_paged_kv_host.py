"""The host-side paged KV-cache manager and batch scheduler
(whetstone_b200/host/paged_kv.hpp through its C bindings): page accounting, all-or-nothing
reservation, rewind semantics of the engine's speculative loop
(crates/whetstone-core/src/speculate.rs:227-239, engine.rs:865-880), the launch arrays
and the unit assignment.  No GPU involved."""

import numpy as np
import pytest

from whetstone_b200 import paged
from whetstone_b200._ffi import InvalidArg, OutOfMemory, ShapeError


def test_pages_follow_reserve_commit_rewind_trim_close():
    kv = paged.PagedKvManager(n_pool_pages=10, max_len=200)
    a, b = kv.open(), kv.open()
    assert (a, b) == (0, 1) and kv.free_pages() == 10
    kv.reserve(a, 17)                       # rows 0..16 -> two pages
    assert kv.pages(a) == 2 and kv.free_pages() == 8 and kv.length(a) == 0
    kv.commit(a, 17)
    assert kv.length(a) == 17
    kv.reserve(a, 6)                        # 1 + 5 drafts at row 17: rows 17..22 fit page 1
    assert kv.pages(a) == 2
    kv.commit(a, 6)
    kv.rewind(a, 17 + 3)                    # two drafts accepted; nothing is given back
    assert kv.length(a) == 20 and kv.pages(a) == 2 and kv.free_pages() == 8
    with pytest.raises(InvalidArg):
        kv.rewind(a, 21)                    # ahead of the cursor, like Engine::rewind
    with pytest.raises(InvalidArg):
        kv.commit(a, 20)                    # rows that were never reserved
    kv.reserve(b, 16 * 8)
    assert kv.free_pages() == 0
    with pytest.raises(OutOfMemory):
        kv.reserve(a, 13)                   # needs a third page: refused, nothing changed
    assert kv.pages(a) == 2 and kv.length(a) == 20
    kv.rewind(b, 0)
    assert kv.trim(b, keep_tokens=16) == 7 and kv.free_pages() == 7
    with pytest.raises(ShapeError):
        kv.reserve(a, 181)                  # past max_len
    kv.close(a)
    assert kv.free_pages() == 9
    assert kv.open() == a                   # ids are reused
    with pytest.raises(InvalidArg):
        kv.length(7)


def test_build_step_arrays_and_all_or_nothing():
    kv = paged.PagedKvManager(n_pool_pages=64, max_len=2000)
    lens = [100, 16, 37]
    ids = []
    for L in lens:
        s = kv.open()
        kv.reserve(s, L)
        kv.commit(s, L)
        ids.append(s)
    used = kv.free_pages()
    step = kv.build_step([(ids[0], 5), (ids[1], 5), (ids[2], 3)])
    assert step.total_tokens == 13 and step.max_tokens_per_seq == 5 and step.max_len == 105
    assert list(step.cu_tokens) == [0, 5, 10, 13] and list(step.seq_pos0) == lens
    assert step.page_table.shape == (3, 125)
    seen = set()
    for i, L in enumerate(lens):
        n_tok = step.entries[i][1]
        need = -(-(L + n_tok) // 16)
        row = step.page_table[i]
        assert np.all(row[:need] >= 0) and np.all(row[need:] == -1)
        assert not (set(row[:need].tolist()) & seen)       # no page belongs to two sequences
        seen |= set(row[:need].tolist())
    assert kv.free_pages() == used - 1                      # only sequence 1 (16 -> 21 rows) grew
    # a step the pool cannot hold changes nothing, not even for the entries that would fit
    big = kv.open()
    free = kv.free_pages()
    with pytest.raises(OutOfMemory):
        kv.build_step([(ids[0], 20), (big, 16 * free)])
    assert kv.free_pages() == free and kv.pages(ids[0]) == 7
    with pytest.raises(InvalidArg):
        kv.build_step([(ids[0], 1), (ids[0], 1)])
    with pytest.raises(ShapeError):          # an entry past max_len: refused before any page moves
        kv.build_step([(ids[1], 20), (ids[0], 1950)])
    assert kv.free_pages() == free and kv.pages(ids[1]) == 2


def test_scheduler_takes_longest_first_within_budgets():
    kv = paged.PagedKvManager(n_pool_pages=60, max_len=400)
    lens = [10, 300, 150, 299]
    ids = []
    for L in lens:
        s = kv.open()
        kv.reserve(s, L)
        kv.commit(s, L)
        ids.append(s)
    waiting = [(ids[0], 6), (ids[1], 6), (ids[2], 6), (ids[3], 6)]
    got = kv.schedule(waiting, max_tokens_per_step=18, max_sequences_per_step=8)
    assert got == [(ids[1], 6), (ids[3], 6), (ids[2], 6)]          # 18 tokens: the shortest waits
    got = kv.schedule(waiting, max_tokens_per_step=100, max_sequences_per_step=2)
    assert got == [(ids[1], 6), (ids[3], 6)]
    assert kv.free_pages() == 60 - sum(-(-L // 16) for L in lens)     # scheduling moves no page
    # a request that needs more pages than are free is skipped, the others still run
    free = kv.free_pages()
    hungry = (ids[0], 16 * (free + 1))
    got = kv.schedule([hungry, (ids[2], 6)], 10_000, 8)
    assert got == [(ids[2], 6)]
    # a sequence that would pass max_len is left out instead of failing the step
    assert kv.schedule([(ids[1], 101)], 10_000, 8) == []


def test_unit_assignment_balances_rows_and_is_deterministic():
    rng = np.random.default_rng(3)
    lens = rng.integers(1024, 16385, size=16)
    step = paged.Step([(i, 5) for i in range(16)], np.zeros((16, 1), np.int32),
                      lens.astype(np.int32), (np.arange(17) * 5).astype(np.int32), 80, 5,
                      int(lens.max()) + 5)
    for world in (1, 2, 4, 8):
        ranks = paged.assign_units(step, n_kv=4, world=world)
        assert ranks.shape == (64,) and set(ranks.tolist()) == set(range(world))
        load = np.zeros(world)
        for u, r in enumerate(ranks):
            load[r] += lens[u // 4] + 5
        assert load.max() / load.mean() < 1.06
        assert np.array_equal(ranks, paged.assign_units(step, n_kv=4, world=world))
