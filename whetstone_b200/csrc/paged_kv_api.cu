/* C ABI over the host-side paged KV-cache manager and batch scheduler
 * (whetstone_b200/host/paged_kv.hpp).  Pure host bookkeeping: nothing here touches the
 * GPU, so these entry points also work in a process without a CUDA device.  Exceptions
 * of the C++ layer become status codes plus the thread's error text. */

#include <exception>
#include <new>

#include "../host/paged_kv.hpp"
#include "wst_common.cuh"

namespace {

using whetstone::paged_kv::PagedKvManager;
using whetstone::paged_kv::StepArrays;
using whetstone::paged_kv::StepEntry;

template <class F>
wst_status_t guarded(const char *who, F &&body) {
  try {
    return body();
  } catch (const std::length_error &e) {
    return wst::fail(WST_ERR_SHAPE, "%s: %s", who, e.what());
  } catch (const std::bad_alloc &) {
    return wst::fail(WST_ERR_OOM, "%s: out of host memory", who);
  } catch (const std::exception &e) {
    return wst::fail(WST_ERR_INVALID_ARG, "%s: %s", who, e.what());
  }
}

PagedKvManager *mgr(void *p) { return static_cast<PagedKvManager *>(p); }

}  // namespace

extern "C" wst_status_t wst_pkv_create(int32_t n_pool_pages, int32_t max_len, void **out_mgr) {
  WST_CHECK_ARG(out_mgr, "wst_pkv_create: null out pointer");
  *out_mgr = nullptr;
  return guarded("wst_pkv_create", [&] {
    *out_mgr = new PagedKvManager(n_pool_pages, max_len);
    return WST_OK;
  });
}

extern "C" wst_status_t wst_pkv_destroy(void *m) {
  delete mgr(m);
  return WST_OK;
}

extern "C" wst_status_t wst_pkv_open(void *m, int32_t *out_seq) {
  WST_CHECK_ARG(m && out_seq, "wst_pkv_open: null pointer");
  return guarded("wst_pkv_open", [&] {
    *out_seq = mgr(m)->open();
    return WST_OK;
  });
}

extern "C" wst_status_t wst_pkv_close(void *m, int32_t seq) {
  WST_CHECK_ARG(m, "wst_pkv_close: null manager");
  return guarded("wst_pkv_close", [&] {
    mgr(m)->close(seq);
    return WST_OK;
  });
}

extern "C" wst_status_t wst_pkv_query(void *m, int32_t seq, int32_t *out_length,
                                      int32_t *out_pages, int32_t *out_free_pages) {
  WST_CHECK_ARG(m, "wst_pkv_query: null manager");
  return guarded("wst_pkv_query", [&] {
    if (out_free_pages) *out_free_pages = mgr(m)->free_pages();
    if (seq >= 0) {
      if (out_length) *out_length = mgr(m)->length(seq);
      if (out_pages) *out_pages = static_cast<int32_t>(mgr(m)->pages(seq).size());
    }
    return WST_OK;
  });
}

extern "C" wst_status_t wst_pkv_reserve(void *m, int32_t seq, int32_t n_tokens) {
  WST_CHECK_ARG(m, "wst_pkv_reserve: null manager");
  return guarded("wst_pkv_reserve", [&] {
    if (!mgr(m)->reserve(seq, n_tokens))
      return wst::fail(WST_ERR_OOM, "wst_pkv_reserve: the pool has %d free pages, sequence %d needs %d",
                       mgr(m)->free_pages(), seq, mgr(m)->pages_needed(seq, n_tokens));
    return WST_OK;
  });
}

extern "C" wst_status_t wst_pkv_commit(void *m, int32_t seq, int32_t n_tokens) {
  WST_CHECK_ARG(m, "wst_pkv_commit: null manager");
  return guarded("wst_pkv_commit", [&] {
    mgr(m)->commit(seq, n_tokens);
    return WST_OK;
  });
}

extern "C" wst_status_t wst_pkv_rewind(void *m, int32_t seq, int32_t pos) {
  WST_CHECK_ARG(m, "wst_pkv_rewind: null manager");
  return guarded("wst_pkv_rewind", [&] {
    mgr(m)->rewind(seq, pos);
    return WST_OK;
  });
}

extern "C" wst_status_t wst_pkv_trim(void *m, int32_t seq, int32_t keep_tokens,
                                     int32_t *out_returned) {
  WST_CHECK_ARG(m, "wst_pkv_trim: null manager");
  return guarded("wst_pkv_trim", [&] {
    const int n = mgr(m)->trim(seq, keep_tokens);
    if (out_returned) *out_returned = n;
    return WST_OK;
  });
}

extern "C" wst_status_t wst_pkv_schedule(void *m, const int32_t *seqs, const int32_t *n_tokens,
                                         int32_t n_waiting, int32_t max_tokens_per_step,
                                         int32_t max_sequences_per_step, int32_t *chosen_out,
                                         int32_t *n_chosen_out) {
  WST_CHECK_ARG(m && n_chosen_out && (n_waiting == 0 || (seqs && n_tokens && chosen_out)),
                "wst_pkv_schedule: null pointer");
  return guarded("wst_pkv_schedule", [&] {
    std::vector<whetstone::paged_kv::Waiting> w;
    for (int i = 0; i < n_waiting; ++i) w.push_back({seqs[i], n_tokens[i]});
    whetstone::paged_kv::BatchScheduler sched(max_tokens_per_step, max_sequences_per_step);
    const std::vector<StepEntry> pick = sched.pick(*mgr(m), w);
    /* report positions in the caller's list, in launch order */
    int n = 0;
    for (const StepEntry &e : pick)
      for (int i = 0; i < n_waiting; ++i)
        if (seqs[i] == e.seq) {
          chosen_out[n++] = i;
          break;
        }
    *n_chosen_out = n;
    return WST_OK;
  });
}

extern "C" wst_status_t wst_pkv_build_step(void *m, const int32_t *seqs, const int32_t *n_tokens,
                                           int32_t n_seq, int32_t *page_table_host,
                                           int32_t *seq_pos0_host, int32_t *cu_tokens_host,
                                           int32_t *totals_out4) {
  WST_CHECK_ARG(m && seqs && n_tokens && page_table_host && seq_pos0_host && cu_tokens_host &&
                    totals_out4 && n_seq > 0,
                "wst_pkv_build_step: null pointer or empty batch");
  return guarded("wst_pkv_build_step", [&] {
    std::vector<StepEntry> entries;
    for (int i = 0; i < n_seq; ++i) entries.push_back({seqs[i], n_tokens[i]});
    const StepArrays a = whetstone::paged_kv::build_step(*mgr(m), entries);
    if (a.n_seq == 0)
      return wst::fail(WST_ERR_OOM, "wst_pkv_build_step: the pool cannot hold this step (%d free pages)",
                       mgr(m)->free_pages());
    std::copy(a.page_table.begin(), a.page_table.end(), page_table_host);
    std::copy(a.seq_pos0.begin(), a.seq_pos0.end(), seq_pos0_host);
    std::copy(a.cu_tokens.begin(), a.cu_tokens.end(), cu_tokens_host);
    totals_out4[0] = a.total_tokens;
    totals_out4[1] = a.max_tokens_per_seq;
    totals_out4[2] = a.max_len;
    totals_out4[3] = a.max_pages;
    return WST_OK;
  });
}

extern "C" wst_status_t wst_pkv_assign_units(const int32_t *seq_pos0_host,
                                             const int32_t *cu_tokens_host, int32_t n_seq,
                                             int32_t n_kv, int32_t world, int32_t *rank_of_unit_out) {
  WST_CHECK_ARG(seq_pos0_host && cu_tokens_host && rank_of_unit_out && n_seq > 0,
                "wst_pkv_assign_units: null pointer or empty batch");
  return guarded("wst_pkv_assign_units", [&] {
    StepArrays a;
    a.n_seq = n_seq;
    a.seq_pos0.assign(seq_pos0_host, seq_pos0_host + n_seq);
    a.cu_tokens.assign(cu_tokens_host, cu_tokens_host + n_seq + 1);
    const auto owned = whetstone::paged_kv::assign_units(a, n_kv, world);
    for (size_t r = 0; r < owned.size(); ++r)
      for (int u : owned[r]) rank_of_unit_out[u] = static_cast<int32_t>(r);
    return WST_OK;
  });
}
