/* The non-kernel part of the C ABI: error text, the calling thread's stream,
 * device/memory/graph/event wrappers, the position cursor and the host-side
 * RoPE table.  Behaviour follows crates/whetstone-kernels/cuda/runtime.cu and
 * cuda/graph.cu of the engine (status codes, NULL handling, no aborts). */

#include <cmath>
#include <mutex>

#include <cstring>

#include "wst_common.cuh"

namespace wst {

#ifndef WST_DROPIN
thread_local char g_error_text[512] = "no error";
#endif
static thread_local cudaStream_t t_stream = cudaStreamPerThread;

cudaStream_t current_stream() { return t_stream; }

static constexpr int kMaxDevices = 64;

bool device_facts(DeviceFacts *out) {
  static DeviceFacts cache[kMaxDevices];
  static bool have[kMaxDevices] = {};
  static std::mutex mu;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    cuda_fail("cudaGetDevice", e);
    return false;
  }
  if (dev < 0 || dev >= kMaxDevices) {
    fail(WST_ERR_CUDA, "device ordinal %d out of range", dev);
    return false;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (!have[dev]) {
    DeviceFacts f;
    if ((e = cudaDeviceGetAttribute(&f.sm_count, cudaDevAttrMultiProcessorCount, dev)) ||
        (e = cudaDeviceGetAttribute(&f.smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev)) ||
        (e = cudaDeviceGetAttribute(&f.cc_major, cudaDevAttrComputeCapabilityMajor, dev))) {
      cuda_fail("cudaDeviceGetAttribute", e);
      return false;
    }
    cache[dev] = f;
    have[dev] = true;
  }
  *out = cache[dev];
  return true;
}

/* One watchdog word per device.  The symbol's name is a host-side handle, not a
 * device address: the address is resolved per device with
 * cudaGetSymbolAddress and handed to kernels as an argument. */
static __device__ unsigned int g_watchdog_word;

unsigned int *device_error_word() {
  static unsigned int *ptrs[kMaxDevices] = {};
  static std::mutex mu;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    cuda_fail("cudaGetDevice", e);
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (!ptrs[dev]) {
    void *p = nullptr;
    e = cudaGetSymbolAddress(&p, g_watchdog_word);
    if (e != cudaSuccess) {
      cuda_fail("cudaGetSymbolAddress(watchdog)", e);
      return nullptr;
    }
    ptrs[dev] = static_cast<unsigned int *>(p);
  }
  return ptrs[dev];
}

}  // namespace wst

using namespace wst;

#ifndef WST_DROPIN
extern "C" const char *wst_last_error(void) { return g_error_text; }
#endif

extern "C" const char *wst_b200_version(void) { return "0.1.0"; }

extern "C" wst_status_t wst_b200_set_stream(void *stream) {
  t_stream = stream ? static_cast<cudaStream_t>(stream) : cudaStreamPerThread;
  return WST_OK;
}

extern "C" wst_status_t wst_b200_device_error(uint32_t *out_code) {
  WST_CHECK_ARG(out_code, "wst_b200_device_error: null out pointer");
  unsigned int *word = device_error_word();
  if (!word) return WST_ERR_CUDA;
  WST_CUDA(cudaStreamSynchronize(current_stream()));
  unsigned int v = 0;
  WST_CUDA(cudaMemcpy(&v, word, sizeof(v), cudaMemcpyDeviceToHost));
  if (v != 0) WST_CUDA(cudaMemset(word, 0, sizeof(v)));
  *out_code = v;
  return WST_OK;
}

/* Everything from here to the next #endif is the engine's own runtime half of the ABI
 * (cuda/runtime.cu:80-190): present so that a host can run on this library alone,
 * left out of the drop-in archive, where the engine's objects define it. */
#ifndef WST_DROPIN
/* ----------------------------------------------------- device and memory */

extern "C" wst_status_t wst_device_count(int32_t *out_count) {
  WST_CHECK_ARG(out_count, "wst_device_count: null out_count");
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e == cudaErrorNoDevice || e == cudaErrorInsufficientDriver) {
    *out_count = 0;
    cudaGetLastError();
    return WST_OK;
  }
  if (e != cudaSuccess) return cuda_fail("cudaGetDeviceCount", e);
  *out_count = n;
  return WST_OK;
}

extern "C" wst_status_t wst_device_set(int32_t ordinal) {
  WST_CUDA(cudaSetDevice(ordinal));
  return WST_OK;
}

extern "C" wst_status_t wst_device_synchronize(void) {
  WST_CUDA(cudaDeviceSynchronize());
  return WST_OK;
}

extern "C" wst_status_t wst_malloc(void **out_ptr, size_t bytes) {
  WST_CHECK_ARG(out_ptr, "wst_malloc: null out_ptr");
  *out_ptr = nullptr;
  if (bytes == 0) return WST_OK;
  void *p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e == cudaErrorMemoryAllocation) {
    size_t free_b = 0, total_b = 0;
    cudaMemGetInfo(&free_b, &total_b);
    cudaGetLastError();
    return fail(WST_ERR_OOM, "wst_malloc: out of memory requesting %.1f MB (%.1f MB free of %.1f MB)",
                bytes / 1e6, free_b / 1e6, total_b / 1e6);
  }
  if (e != cudaSuccess) return cuda_fail("wst_malloc", e);
  *out_ptr = p;
  return WST_OK;
}

extern "C" wst_status_t wst_free(void *ptr) {
  if (!ptr) return WST_OK;
  WST_CUDA(cudaFree(ptr));
  return WST_OK;
}

extern "C" wst_status_t wst_memset(void *dst, int32_t value, size_t bytes) {
  if (bytes == 0) return WST_OK;
  WST_CHECK_ARG(dst, "wst_memset: null dst");
  WST_CUDA(cudaMemset(dst, value, bytes));
  return WST_OK;
}

#endif /* !WST_DROPIN */

/* Sharing one device allocation with the other processes of the box (one process
 * per GPU): the owner exports a 64-byte handle of a buffer it got from wst_malloc,
 * another process imports it WITH ITS OWN DEVICE CURRENT, so that the mapping
 * belongs to the context whose kernels will use it (peer access is switched on as
 * part of the import). */
extern "C" wst_status_t wst_b200_ipc_export(const void *dev_ptr, void *handle_out_host) {
  WST_CHECK_ARG(dev_ptr && handle_out_host, "wst_b200_ipc_export: null pointer");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  cudaIpcMemHandle_t h;
  WST_CUDA(cudaIpcGetMemHandle(&h, const_cast<void *>(dev_ptr)));
  memcpy(handle_out_host, &h, sizeof(h));
  return WST_OK;
}

extern "C" wst_status_t wst_b200_ipc_import(const void *handle_host, void **out_dev_ptr) {
  WST_CHECK_ARG(handle_host && out_dev_ptr, "wst_b200_ipc_import: null pointer");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle_host, sizeof(h));
  void *p = nullptr;
  WST_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
  *out_dev_ptr = p;
  return WST_OK;
}

extern "C" wst_status_t wst_b200_ipc_close(void *dev_ptr) {
  if (!dev_ptr) return WST_OK;
  WST_CUDA(cudaIpcCloseMemHandle(dev_ptr));
  return WST_OK;
}

/* the rest of the engine's runtime, graph (cuda/graph.cu:47-145) and cursor entry points */
#ifndef WST_DROPIN
extern "C" wst_status_t wst_memcpy_h2d(void *dst, const void *src_host, size_t bytes) {
  if (bytes == 0) return WST_OK;
  WST_CHECK_ARG(dst && src_host, "wst_memcpy_h2d: null pointer");
  WST_CUDA(cudaMemcpy(dst, src_host, bytes, cudaMemcpyHostToDevice));
  return WST_OK;
}

extern "C" wst_status_t wst_memcpy_d2h(void *dst_host, const void *src, size_t bytes) {
  if (bytes == 0) return WST_OK;
  WST_CHECK_ARG(dst_host && src, "wst_memcpy_d2h: null pointer");
  WST_CUDA(cudaMemcpy(dst_host, src, bytes, cudaMemcpyDeviceToHost));
  return WST_OK;
}

extern "C" wst_status_t wst_memcpy_d2d(void *dst, const void *src, size_t bytes) {
  if (bytes == 0) return WST_OK;
  WST_CHECK_ARG(dst && src, "wst_memcpy_d2d: null pointer");
  WST_CUDA(cudaMemcpy(dst, src, bytes, cudaMemcpyDeviceToDevice));
  return WST_OK;
}

/* ------------------------------------------------------ graphs and events */

extern "C" wst_status_t wst_graph_capture_begin(void) {
  WST_CUDA(cudaStreamBeginCapture(current_stream(), cudaStreamCaptureModeThreadLocal));
  return WST_OK;
}

extern "C" wst_status_t wst_graph_capture_end(void **out_exec) {
  WST_CHECK_ARG(out_exec, "wst_graph_capture_end: null out pointer");
  *out_exec = nullptr;
  cudaGraph_t graph = nullptr;
  WST_CUDA(cudaStreamEndCapture(current_stream(), &graph));
  if (!graph) return fail(WST_ERR_CUDA, "wst_graph_capture_end: capture produced no graph");
  cudaGraphExec_t exec = nullptr;
  cudaError_t e = cudaGraphInstantiateWithFlags(&exec, graph, 0);
  cudaGraphDestroy(graph);
  if (e != cudaSuccess) return cuda_fail("cudaGraphInstantiate", e);
  *out_exec = exec;
  return WST_OK;
}

extern "C" wst_status_t wst_graph_launch(void *exec) {
  WST_CHECK_ARG(exec, "wst_graph_launch: null graph");
  WST_CUDA(cudaGraphLaunch(static_cast<cudaGraphExec_t>(exec), current_stream()));
  return WST_OK;
}

extern "C" wst_status_t wst_graph_destroy(void *exec) {
  if (!exec) return WST_OK;
  WST_CUDA(cudaGraphExecDestroy(static_cast<cudaGraphExec_t>(exec)));
  return WST_OK;
}

extern "C" wst_status_t wst_stream_sync(void) {
  WST_CUDA(cudaStreamSynchronize(current_stream()));
  return WST_OK;
}

extern "C" wst_status_t wst_event_create(void **out) {
  WST_CHECK_ARG(out, "wst_event_create: null out pointer");
  cudaEvent_t ev = nullptr;
  WST_CUDA(cudaEventCreate(&ev));
  *out = ev;
  return WST_OK;
}

extern "C" wst_status_t wst_event_record(void *ev) {
  WST_CHECK_ARG(ev, "wst_event_record: null event");
  WST_CUDA(cudaEventRecord(static_cast<cudaEvent_t>(ev), current_stream()));
  return WST_OK;
}

extern "C" wst_status_t wst_event_elapsed_ms(void *a, void *b, float *out) {
  WST_CHECK_ARG(a && b && out, "wst_event_elapsed_ms: null pointer");
  WST_CUDA(cudaEventElapsedTime(out, static_cast<cudaEvent_t>(a), static_cast<cudaEvent_t>(b)));
  return WST_OK;
}

extern "C" wst_status_t wst_event_destroy(void *ev) {
  if (!ev) return WST_OK;
  WST_CUDA(cudaEventDestroy(static_cast<cudaEvent_t>(ev)));
  return WST_OK;
}

/* ------------------------------------------------------------ the cursor */

__global__ void advance_cursor_kernel(int32_t *pos, int32_t cap) {
  const int32_t next = *pos + 1;
  *pos = next < cap ? next : cap;
}

extern "C" wst_status_t wst_advance_pos(void *pos, int32_t max_seq) {
  WST_CHECK_ARG(pos, "wst_advance_pos: null pointer");
  WST_CHECK_ARG(max_seq > 0, "wst_advance_pos: empty cache");
  advance_cursor_kernel<<<1, 1, 0, current_stream()>>>(static_cast<int32_t *>(pos), max_seq);
  WST_LAUNCHED("wst_advance_pos");
  return WST_OK;
}

#endif /* !WST_DROPIN */

/* ----------------------------------------------------------- RoPE table */

extern "C" wst_status_t wst_rope_table_host(float *cos_host, float *sin_host, int32_t max_seq,
                                            int32_t head_dim, double theta, int32_t scaling_kind,
                                            double factor, double low_freq_factor,
                                            double high_freq_factor,
                                            int32_t original_max_position) {
  WST_CHECK_ARG(cos_host && sin_host, "wst_rope_table_host: null pointer");
  WST_CHECK_ARG(max_seq >= 0, "wst_rope_table_host: negative max_seq");
  if (head_dim <= 0 || head_dim % 2 != 0)
    return fail(WST_ERR_SHAPE, "rope: head_dim %d must be even", head_dim);
  WST_CHECK_ARG(scaling_kind == 0 || scaling_kind == 1, "wst_rope_table_host: unknown scaling kind");
  const int half = head_dim / 2;
  const double two_pi = 6.283185307179586476925286766559;
  for (int j = 0; j < half; ++j) {
    double inv_freq = std::pow(theta, -static_cast<double>(j) / half);
    if (scaling_kind == 1) {
      const double orig = static_cast<double>(original_max_position);
      const double wavelength = two_pi / inv_freq;
      if (wavelength > orig / low_freq_factor) {
        inv_freq /= factor;
      } else if (wavelength > orig / high_freq_factor) {
        const double t = (orig / wavelength - low_freq_factor) / (high_freq_factor - low_freq_factor);
        inv_freq = (1.0 - t) * (inv_freq / factor) + t * inv_freq;
      }
    }
    for (int p = 0; p < max_seq; ++p) {
      const double a = static_cast<double>(p) * inv_freq;
      cos_host[static_cast<size_t>(p) * half + j] = static_cast<float>(std::cos(a));
      sin_host[static_cast<size_t>(p) * half + j] = static_cast<float>(std::sin(a));
    }
  }
  return WST_OK;
}
