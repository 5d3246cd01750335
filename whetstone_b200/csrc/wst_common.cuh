/* Host-side plumbing shared by every translation unit of the library: the
 * thread-local error message, the status helpers and the calling thread's
 * stream.  Not part of the C ABI. */
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "whetstone.h"
#include "whetstone_b200.h"

namespace wst {

/* ---- error reporting --------------------------------------------------- */

}  // namespace wst

#ifdef WST_DROPIN
/* Linked INTO the engine's kernel library (make DROPIN=1): messages go to the engine's
 * own per-thread buffer, the one its wst_last_error returns
 * (cuda/common.cuh:16, cuda/runtime.cu:5-7), so the Rust side's check() reads them. */
extern __attribute__((visibility("default"))) thread_local char wst_err_buf[512];
#define WST_ERROR_TEXT ::wst_err_buf
#else
namespace wst {
/* 512 bytes per thread, like the engine's own buffer; wst_last_error returns it. */
extern thread_local char g_error_text[512];
}
#define WST_ERROR_TEXT ::wst::g_error_text
#endif

namespace wst {

inline wst_status_t fail(wst_status_t code, const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(WST_ERROR_TEXT, sizeof(WST_ERROR_TEXT), fmt, ap);
  va_end(ap);
  return code;
}

inline wst_status_t cuda_fail(const char *what, cudaError_t e) {
  return fail(WST_ERR_CUDA, "%s: %s (%s)", what, cudaGetErrorString(e), cudaGetErrorName(e));
}

/* Argument check: message + WST_ERR_INVALID_ARG, nothing launched. */
#define WST_CHECK_ARG(cond, msg)                                      \
  do {                                                                \
    if (!(cond)) return ::wst::fail(WST_ERR_INVALID_ARG, "%s", msg);  \
  } while (0)

/* A CUDA runtime call that must succeed. */
#define WST_CUDA(expr)                                                \
  do {                                                                \
    cudaError_t e_ = (expr);                                          \
    if (e_ != cudaSuccess) return ::wst::cuda_fail(#expr, e_);        \
  } while (0)

/* After a launch: report a launch-time failure without synchronising. */
#define WST_LAUNCHED(name)                                            \
  do {                                                                \
    cudaError_t e_ = cudaGetLastError();                              \
    if (e_ != cudaSuccess) return ::wst::cuda_fail(name " (launch)", e_); \
  } while (0)

/* ---- stream ------------------------------------------------------------ */

/* The stream every entry point of this thread enqueues on: the per-thread
 * default stream unless wst_b200_set_stream installed another one. */
cudaStream_t current_stream();

/* ---- per-device facts, queried once ------------------------------------ */

struct DeviceFacts {
  int sm_count = 0;
  int smem_optin = 0; /* max dynamic shared memory per block, bytes */
  int cc_major = 0;
};
/* Facts of the CURRENT device (cached per ordinal). Returns false on failure
 * with the error text set. */
bool device_facts(DeviceFacts *out);

/* ---- device-side watchdog ---------------------------------------------- */

/* Kernels that wait on an mbarrier give up after a bounded number of polls and
 * record where in one 32-bit word per device; the host reads it back with
 * wst_b200_device_error. 0 = no failure.  This returns the DEVICE address of
 * that word for the current device (resolved once per device), or nullptr with
 * the error text set. */
unsigned int *device_error_word();

}  // namespace wst
