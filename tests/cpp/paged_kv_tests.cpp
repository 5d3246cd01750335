/* CPU-only checks of the host-side page manager and scheduler
 * (whetstone_b200/host/paged_kv.hpp) used directly from C++, the way an engine would:
 * the propose / verify / rewind bookkeeping of
 * crates/whetstone-core/src/speculate.rs:185-256 for several sequences over one pool. */
#include <cstdio>
#include <set>
#include <stdexcept>

#include "paged_kv.hpp"

using namespace whetstone::paged_kv;

static int failures = 0;
#define CHECK(cond)                                                        \
  do {                                                                     \
    if (!(cond)) {                                                         \
      std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond);        \
      ++failures;                                                          \
    }                                                                      \
  } while (0)

static void speculative_rounds_keep_the_pool_consistent() {
  PagedKvManager kv(64, 400);
  BatchScheduler sched(/*tokens*/ 24, /*sequences*/ 3);
  std::vector<int> ids;
  const int prompt[4] = {70, 9, 33, 120};
  for (int i = 0; i < 4; ++i) {
    ids.push_back(kv.open());
    CHECK(kv.reserve(ids[i], prompt[i]));
    kv.commit(ids[i], prompt[i]);
  }
  for (int round = 0; round < 6; ++round) {
    std::vector<Waiting> waiting;
    for (int id : ids) waiting.push_back({id, 6}); /* 1 + 5 drafts */
    const std::vector<StepEntry> pick = sched.pick(kv, waiting);
    CHECK(pick.size() == 3);                       /* three sequences of six fit 24 tokens */
    for (size_t i = 1; i < pick.size(); ++i)
      CHECK(kv.length(pick[i - 1].seq) >= kv.length(pick[i].seq));
    const StepArrays a = build_step(kv, pick);
    CHECK(a.n_seq == 3 && a.total_tokens == 18 && a.max_tokens_per_seq == 6);
    std::set<int32_t> seen;
    for (int i = 0; i < a.n_seq; ++i) {
      const int need = pages_for(a.seq_pos0[i] + 6);
      for (int p = 0; p < a.max_pages; ++p) {
        const int32_t page = a.page_table[static_cast<size_t>(i) * a.max_pages + p];
        CHECK((p < need) == (page >= 0));
        if (page >= 0) CHECK(seen.insert(page).second);
      }
    }
    for (const StepEntry &e : pick) {
      const int pos0 = kv.length(e.seq);
      kv.commit(e.seq, e.n_tokens);
      kv.rewind(e.seq, pos0 + 1 + (round + e.seq) % 6); /* accepted drafts + the confirmed token */
    }
  }
  int owned = 0;
  for (int id : ids) owned += static_cast<int>(kv.pages(id).size());
  CHECK(owned + kv.free_pages() == kv.pool_pages());
  kv.close(ids[3]);
  CHECK(kv.open() == ids[3]);
  bool threw = false;
  try {
    kv.rewind(ids[0], kv.length(ids[0]) + 1);
  } catch (const std::invalid_argument &) {
    threw = true;
  }
  CHECK(threw);
}

static void units_are_dealt_heaviest_first() {
  StepArrays a;
  a.n_seq = 3;
  a.seq_pos0 = {1000, 10, 500};
  a.cu_tokens = {0, 5, 10, 15};
  const auto owned = assign_units(a, /*n_kv=*/2, /*world=*/2);
  CHECK(owned.size() == 2 && owned[0].size() + owned[1].size() == 6);
  long long load[2] = {0, 0};
  for (int r = 0; r < 2; ++r)
    for (int u : owned[r]) load[r] += a.seq_pos0[u / 2] + 5;
  CHECK(load[0] == load[1]); /* two KV heads per sequence split evenly */
}

int main() {
  speculative_rounds_keep_the_pool_consistent();
  units_are_dealt_heaviest_first();
  std::printf("%d failed\n", failures);
  return failures ? 1 : 0;
}
