/* Host-side paged KV-cache manager and batch scheduler for the ragged entry points
 * (wst_rope_cache_paged, wst_attn_verify_paged).  Header-only, no CUDA in it: the
 * bookkeeping runs and is tested on the CPU; `StepArrays` holds exactly the host
 * arrays those two entry points take once copied to the device.
 *
 * The Whetstone engine has one sequence with one contiguous cache and keeps the
 * cursor itself (crates/whetstone-kernels/src/decode.rs:162-212 `KvCache`,
 * crates/whetstone-core/src/engine.rs:264-286 `Engine.pos`, :865-880 `rewind`); its
 * speculative loop (crates/whetstone-core/src/speculate.rs:185-256) appends
 * 1 + drafts rows at the cursor, verifies, and rewinds to pos0 + accepted + 1 --
 * rejected rows are not erased, the next append writes over them.  This file is
 * that bookkeeping for MANY sequences over one page pool:
 *
 *   PagePool         fixed pool of 16-token pages with a free list
 *   PagedKvManager   per-sequence page lists and lengths: open / reserve / commit /
 *                    rewind / trim / close, all-or-nothing reservation
 *   StepArrays       page_table [n_seq][max_pages], seq_pos0 [n_seq],
 *                    cu_tokens [n_seq + 1], totals and bounds for one launch
 *   BatchScheduler   picks which waiting sequences run this step under a token and a
 *                    page budget, longest context first, and deals (sequence, KV head)
 *                    units to GPUs longest-first
 */
#pragma once

#include <algorithm>
#include <cstdint>
#include <numeric>
#include <stdexcept>
#include <string>
#include <vector>

namespace whetstone {
namespace paged_kv {

constexpr int kPageTokens = 16; /* the kernels take page_size == 16 only */

inline int pages_for(int64_t tokens) {
  return static_cast<int>((tokens + kPageTokens - 1) / kPageTokens);
}

/* ---------------------------------------------------------------- the pool */

class PagePool {
 public:
  explicit PagePool(int n_pages) : n_pages_(n_pages) {
    if (n_pages <= 0) throw std::invalid_argument("PagePool: needs at least one page");
    free_.resize(static_cast<size_t>(n_pages));
    /* lowest ids are handed out first */
    for (int i = 0; i < n_pages; ++i) free_[static_cast<size_t>(i)] = n_pages - 1 - i;
  }
  int capacity() const { return n_pages_; }
  int free_pages() const { return static_cast<int>(free_.size()); }

  /* `n` pages appended to `out`, or nothing at all and false. */
  bool take(int n, std::vector<int32_t> *out) {
    if (n < 0 || static_cast<size_t>(n) > free_.size()) return false;
    for (int i = 0; i < n; ++i) {
      out->push_back(free_.back());
      free_.pop_back();
    }
    return true;
  }
  void give_back(int32_t page) {
    if (page < 0 || page >= n_pages_) throw std::invalid_argument("PagePool: foreign page id");
    free_.push_back(page);
  }

 private:
  int n_pages_;
  std::vector<int32_t> free_;
};

/* ------------------------------------------------------------ the manager */

class PagedKvManager {
 public:
  /* `max_len`: longest context any sequence may reach (sizes a page-table row). */
  PagedKvManager(int n_pool_pages, int max_len)
      : pool_(n_pool_pages), max_len_(max_len), max_pages_(pages_for(max_len)) {
    if (max_len <= 0) throw std::invalid_argument("PagedKvManager: max_len must be positive");
  }

  int max_len() const { return max_len_; }
  int max_pages() const { return max_pages_; }
  int pool_pages() const { return pool_.capacity(); }
  int free_pages() const { return pool_.free_pages(); }
  int open_sequences() const { return live_; }

  /* A new, empty sequence; ids of closed sequences are reused. */
  int open() {
    int id;
    if (!free_ids_.empty()) {
      id = free_ids_.back();
      free_ids_.pop_back();
    } else {
      id = static_cast<int>(seqs_.size());
      seqs_.emplace_back();
    }
    seqs_[static_cast<size_t>(id)] = Seq{};
    seqs_[static_cast<size_t>(id)].open = true;
    ++live_;
    return id;
  }

  /* Tokens committed to the cache (the engine's `pos`). */
  int length(int seq) const { return at(seq).len; }
  /* Rows reserved beyond the length (appended or about to be, not yet committed). */
  int reserved(int seq) const {
    return static_cast<int>(at(seq).pages.size()) * kPageTokens - at(seq).len;
  }
  const std::vector<int32_t> &pages(int seq) const { return at(seq).pages; }

  /* Pages a reserve(seq, n_tokens) would take from the pool. */
  int pages_needed(int seq, int n_tokens) const {
    const Seq &s = at(seq);
    const int want = pages_for(static_cast<int64_t>(s.len) + n_tokens);
    return std::max(0, want - static_cast<int>(s.pages.size()));
  }

  /* Makes room for rows [len, len + n_tokens).  All or nothing: false (and no change)
   * if the pool cannot cover it; throws if the sequence would pass max_len -- the
   * engine reports a full context as an error too (engine.rs:519-523). */
  bool reserve(int seq, int n_tokens) {
    Seq &s = at(seq);
    if (n_tokens < 0) throw std::invalid_argument("reserve: negative token count");
    if (static_cast<int64_t>(s.len) + n_tokens > max_len_)
      throw std::length_error("reserve: sequence " + std::to_string(seq) + " would reach " +
                              std::to_string(s.len + n_tokens) + " tokens, the limit is " +
                              std::to_string(max_len_));
    return pool_.take(pages_needed(seq, n_tokens), &s.pages);
  }

  /* The append kernel has written n_tokens rows at the cursor: they are part of the
   * context now. */
  void commit(int seq, int n_tokens) {
    Seq &s = at(seq);
    if (n_tokens < 0 || s.len + n_tokens > static_cast<int>(s.pages.size()) * kPageTokens)
      throw std::logic_error("commit: rows were not reserved");
    s.len += n_tokens;
  }

  /* Discards everything after `pos` (speculate.rs:227-239, engine.rs:865-880).  Nothing
   * is erased and no page is returned: the rejected rows are overwritten by the next
   * append, which finds its pages still mapped. */
  void rewind(int seq, int pos) {
    Seq &s = at(seq);
    if (pos < 0 || pos > s.len)
      throw std::invalid_argument("rewind: " + std::to_string(pos) +
                                  " is ahead of the current position " + std::to_string(s.len));
    s.len = pos;
  }

  /* Returns the pages beyond the committed length (plus `keep_tokens` of slack) to the
   * pool; the number returned. */
  int trim(int seq, int keep_tokens = 0) {
    Seq &s = at(seq);
    const size_t keep = static_cast<size_t>(pages_for(static_cast<int64_t>(s.len) + keep_tokens));
    int n = 0;
    while (s.pages.size() > keep) {
      pool_.give_back(s.pages.back());
      s.pages.pop_back();
      ++n;
    }
    return n;
  }

  void close(int seq) {
    Seq &s = at(seq);
    for (int32_t p : s.pages) pool_.give_back(p);
    s = Seq{};
    free_ids_.push_back(seq);
    --live_;
  }

 private:
  struct Seq {
    bool open = false;
    int len = 0;
    std::vector<int32_t> pages;
  };
  const Seq &at(int seq) const {
    if (seq < 0 || static_cast<size_t>(seq) >= seqs_.size() || !seqs_[static_cast<size_t>(seq)].open)
      throw std::out_of_range("PagedKvManager: no open sequence " + std::to_string(seq));
    return seqs_[static_cast<size_t>(seq)];
  }
  Seq &at(int seq) { return const_cast<Seq &>(static_cast<const PagedKvManager *>(this)->at(seq)); }

  PagePool pool_;
  int max_len_, max_pages_;
  std::vector<Seq> seqs_;
  std::vector<int> free_ids_;
  int live_ = 0;
};

/* ------------------------------------------------------- one launch's arrays */

struct StepEntry {
  int seq;      /* PagedKvManager id */
  int n_tokens; /* rows this sequence appends and attends with in this step */
};

/* What wst_rope_cache_paged and wst_attn_verify_paged take, in host memory; batch
 * slot i is entries[i].  Copy page_table / seq_pos0 / cu_tokens to the device as they
 * are (int32). */
struct StepArrays {
  std::vector<StepEntry> entries;
  std::vector<int32_t> page_table; /* [n_seq][max_pages], -1 = unmapped */
  std::vector<int32_t> seq_pos0;   /* [n_seq]: cache row of each sequence's first token */
  std::vector<int32_t> cu_tokens;  /* [n_seq + 1] */
  int n_seq = 0, max_pages = 0, total_tokens = 0, max_tokens_per_seq = 0;
  int max_len = 0; /* bound on seq_pos0[s] + tokens of s: sizes the grid and the scratch */
};

/* Reserves the rows of every entry (all entries or none: on a shortfall, or when an
 * entry is refused, no page has moved; a shortfall gives an empty result) and lays the
 * arrays out.
 * The caller launches append + attention, then commit()s what it keeps and rewind()s
 * what verification rejected. */
inline StepArrays build_step(PagedKvManager &kv, const std::vector<StepEntry> &entries) {
  StepArrays a;
  /* everything that can fail is checked before the first page moves */
  int64_t need = 0;
  for (size_t i = 0; i < entries.size(); ++i) {
    const StepEntry &e = entries[i];
    if (e.n_tokens <= 0) throw std::invalid_argument("build_step: empty entry");
    for (size_t j = 0; j < i; ++j)
      if (entries[j].seq == e.seq)
        throw std::invalid_argument("build_step: a sequence appears twice in one step");
    if (static_cast<int64_t>(kv.length(e.seq)) + e.n_tokens > kv.max_len())
      throw std::length_error("build_step: sequence " + std::to_string(e.seq) + " would reach " +
                              std::to_string(kv.length(e.seq) + e.n_tokens) +
                              " tokens, the limit is " + std::to_string(kv.max_len()));
    need += kv.pages_needed(e.seq, e.n_tokens);
  }
  if (need > kv.free_pages()) return StepArrays{};
  for (const StepEntry &e : entries)
    if (!kv.reserve(e.seq, e.n_tokens)) throw std::logic_error("build_step: pool accounting");
  a.entries = entries;
  a.n_seq = static_cast<int>(entries.size());
  a.max_pages = kv.max_pages();
  a.page_table.assign(static_cast<size_t>(a.n_seq) * a.max_pages, -1);
  a.seq_pos0.resize(static_cast<size_t>(a.n_seq));
  a.cu_tokens.resize(static_cast<size_t>(a.n_seq) + 1);
  a.cu_tokens[0] = 0;
  for (int i = 0; i < a.n_seq; ++i) {
    const StepEntry &e = entries[static_cast<size_t>(i)];
    const std::vector<int32_t> &pg = kv.pages(e.seq);
    std::copy(pg.begin(), pg.end(), a.page_table.begin() + static_cast<size_t>(i) * a.max_pages);
    a.seq_pos0[static_cast<size_t>(i)] = kv.length(e.seq);
    a.cu_tokens[static_cast<size_t>(i) + 1] = a.cu_tokens[static_cast<size_t>(i)] + e.n_tokens;
    a.max_tokens_per_seq = std::max(a.max_tokens_per_seq, e.n_tokens);
    a.max_len = std::max(a.max_len, kv.length(e.seq) + e.n_tokens);
  }
  a.total_tokens = a.cu_tokens.back();
  return a;
}

/* ----------------------------------------------------------- the scheduler */

struct Waiting {
  int seq;
  int n_tokens; /* what it wants to run next: a prefill chunk, or 1 + drafts */
};

/* Chooses the sequences of one step.  Longest context first -- the kernels hand out
 * (sequence, KV head, slice) blocks in batch order, so the longest streams start
 * first and the short ones fill the tail -- under a budget of tokens per step and of
 * pages the pool can still give.  A sequence that does not fit is skipped this step,
 * never split. */
class BatchScheduler {
 public:
  BatchScheduler(int max_tokens_per_step, int max_sequences_per_step)
      : max_tokens_(max_tokens_per_step), max_seqs_(max_sequences_per_step) {}

  std::vector<StepEntry> pick(const PagedKvManager &kv, const std::vector<Waiting> &waiting) const {
    std::vector<size_t> order(waiting.size());
    std::iota(order.begin(), order.end(), size_t{0});
    std::stable_sort(order.begin(), order.end(), [&](size_t x, size_t y) {
      return kv.length(waiting[x].seq) + waiting[x].n_tokens >
             kv.length(waiting[y].seq) + waiting[y].n_tokens;
    });
    std::vector<StepEntry> chosen;
    int tokens = 0, pages = kv.free_pages();
    for (size_t idx : order) {
      const Waiting &w = waiting[idx];
      if (static_cast<int>(chosen.size()) >= max_seqs_) break;
      if (w.n_tokens <= 0 || tokens + w.n_tokens > max_tokens_) continue;
      if (kv.length(w.seq) + w.n_tokens > kv.max_len()) continue;
      const int need = kv.pages_needed(w.seq, w.n_tokens);
      if (need > pages) continue;
      chosen.push_back(StepEntry{w.seq, w.n_tokens});
      tokens += w.n_tokens;
      pages -= need;
    }
    return chosen;
  }

 private:
  int max_tokens_, max_seqs_;
};

/* (batch slot, KV head) units dealt to `world` GPUs, heaviest first, each to the
 * least loaded rank (ties to the lower rank, so every rank computes the same answer
 * without talking).  weight = rows the unit streams.  Returns, per rank, its units as
 * slot * n_kv + kv_head, ascending. */
inline std::vector<std::vector<int>> assign_units(const StepArrays &a, int n_kv, int world) {
  if (world <= 0 || n_kv <= 0) throw std::invalid_argument("assign_units: world and n_kv must be positive");
  const int n_units = a.n_seq * n_kv;
  std::vector<int> order(static_cast<size_t>(n_units));
  std::iota(order.begin(), order.end(), 0);
  auto weight = [&](int u) {
    const int slot = u / n_kv;
    return static_cast<int64_t>(a.seq_pos0[static_cast<size_t>(slot)]) +
           (a.cu_tokens[static_cast<size_t>(slot) + 1] - a.cu_tokens[static_cast<size_t>(slot)]);
  };
  std::stable_sort(order.begin(), order.end(), [&](int x, int y) { return weight(x) > weight(y); });
  std::vector<int64_t> load(static_cast<size_t>(world), 0);
  std::vector<std::vector<int>> owned(static_cast<size_t>(world));
  for (int u : order) {
    size_t best = 0;
    for (size_t r = 1; r < load.size(); ++r)
      if (load[r] < load[best]) best = r;
    owned[best].push_back(u);
    load[best] += weight(u);
  }
  for (auto &v : owned) std::sort(v.begin(), v.end());
  return owned;
}

}  // namespace paged_kv
}  // namespace whetstone
