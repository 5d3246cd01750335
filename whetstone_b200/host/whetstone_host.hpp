/* C++ host layer over the wst_* C ABI: the owner types and checked wrappers the
 * Whetstone engine keeps in Rust (crates/whetstone-kernels/src/lib.rs,
 * src/decode.rs, src/chunk.rs), with the same names, argument meaning, shape
 * checks and error mapping.  Header-only; link against libwhetstone_b200.so.
 *
 *   Error / check()          src/lib.rs:47-98
 *   DeviceBuffer<T>          src/lib.rs:235-504 (the subset the attention path uses)
 *   RopeScaling, RopeTable   src/decode.rs:50-153
 *   KvCache                  src/decode.rs:162-212
 *   DeviceCursor             src/decode.rs:221-256
 *   QkNorm                   src/decode.rs:269-290
 *   decode::rope_cache       src/decode.rs:305-354
 *   decode::attn_decode      src/decode.rs:368-405
 *   chunk::rope_cache        src/chunk.rs:140-201
 *   chunk::attn              src/chunk.rs:207-254
 *   Graph, Event             src/decode.rs:543-655
 * PagedKvCache and the paged:: / sharded decode wrappers have no counterpart in
 * the engine (it has one contiguous sequence on one GPU).  The host-side page manager
 * and batch scheduler that produce the paged entry points' arrays are in paged_kv.hpp.
 */
#pragma once

#include <cmath>
#include <cstdint>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "whetstone.h"
#include "whetstone_b200.h"

namespace whetstone {

/* ------------------------------------------------------------------ errors */

class Error : public std::runtime_error {
 public:
  enum class Kind { Cuda, InvalidArg, UnsupportedArch, OutOfMemory, Shape, Unknown };
  Error(Kind kind, const std::string &what) : std::runtime_error(what), kind_(kind) {}
  Kind kind() const { return kind_; }
  static Error shape(const std::string &what) { return Error(Kind::Shape, what); }

 private:
  Kind kind_;
};

/* Maps a status to a typed exception carrying the library's message. */
inline void check(wst_status_t st) {
  if (st == WST_OK) return;
  const std::string msg = wst_last_error();
  switch (st) {
    case WST_ERR_CUDA: throw Error(Error::Kind::Cuda, msg);
    case WST_ERR_INVALID_ARG: throw Error(Error::Kind::InvalidArg, msg);
    case WST_ERR_UNSUPPORTED_ARCH: throw Error(Error::Kind::UnsupportedArch, msg);
    case WST_ERR_OOM: throw Error(Error::Kind::OutOfMemory, msg);
    case WST_ERR_SHAPE: throw Error(Error::Kind::Shape, msg);
    default: throw Error(Error::Kind::Unknown, msg);
  }
}

/* ---------------------------------------------------------- device memory */

template <class T>
class DeviceBuffer {
 public:
  DeviceBuffer() = default;
  static DeviceBuffer zeros(size_t n) {
    DeviceBuffer b;
    b.len_ = n;
    if (n) {
      check(wst_malloc(&b.ptr_, n * sizeof(T)));
      check(wst_memset(b.ptr_, 0, n * sizeof(T)));
    }
    return b;
  }
  static DeviceBuffer from_slice(const std::vector<T> &host) {
    DeviceBuffer b;
    b.len_ = host.size();
    if (b.len_) {
      check(wst_malloc(&b.ptr_, b.len_ * sizeof(T)));
      check(wst_memcpy_h2d(b.ptr_, host.data(), b.len_ * sizeof(T)));
    }
    return b;
  }
  DeviceBuffer(DeviceBuffer &&o) noexcept : ptr_(o.ptr_), len_(o.len_) { o.ptr_ = nullptr; o.len_ = 0; }
  DeviceBuffer &operator=(DeviceBuffer &&o) noexcept {
    if (this != &o) {
      release();
      ptr_ = o.ptr_; len_ = o.len_;
      o.ptr_ = nullptr; o.len_ = 0;
    }
    return *this;
  }
  DeviceBuffer(const DeviceBuffer &) = delete;
  DeviceBuffer &operator=(const DeviceBuffer &) = delete;
  ~DeviceBuffer() { release(); }

  size_t len() const { return len_; }
  size_t bytes() const { return len_ * sizeof(T); }
  void *as_mut_ptr() { return ptr_; }
  const void *as_ptr() const { return ptr_; }

  std::vector<T> to_vec() const {
    std::vector<T> out(len_);
    if (len_) check(wst_memcpy_d2h(out.data(), ptr_, bytes()));
    return out;
  }
  void copy_from_host(const std::vector<T> &host) {
    if (host.size() != len_) throw Error::shape("copy_from_host: length mismatch");
    if (len_) check(wst_memcpy_h2d(ptr_, host.data(), bytes()));
  }
  void fill_bytes(int value) {
    if (len_) check(wst_memset(ptr_, value, bytes()));
  }

 private:
  void release() {
    if (ptr_) wst_free(ptr_);
    ptr_ = nullptr;
  }
  void *ptr_ = nullptr;
  size_t len_ = 0;
};

/* -------------------------------------------------------------- RoPE table */

struct RopeScaling {
  enum class Kind { None, Llama3 } kind = Kind::None;
  double factor = 1.0, low_freq_factor = 1.0, high_freq_factor = 4.0;
  size_t original_max_position = 8192;
};

struct RopeTable {
  DeviceBuffer<float> cos, sin;
  size_t max_seq = 0, half_dim = 0;

  RopeTable(size_t max_seq_, size_t head_dim, double theta, RopeScaling scaling = {})
      : max_seq(max_seq_), half_dim(head_dim / 2) {
    if (head_dim % 2 != 0 || head_dim == 0)
      throw Error::shape("rope: head_dim " + std::to_string(head_dim) + " must be even");
    std::vector<float> c(max_seq * half_dim), s(max_seq * half_dim);
    check(wst_rope_table_host(c.data(), s.data(), static_cast<int32_t>(max_seq),
                              static_cast<int32_t>(head_dim), theta,
                              scaling.kind == RopeScaling::Kind::Llama3 ? 1 : 0, scaling.factor,
                              scaling.low_freq_factor, scaling.high_freq_factor,
                              static_cast<int32_t>(scaling.original_max_position)));
    cos = DeviceBuffer<float>::from_slice(c);
    sin = DeviceBuffer<float>::from_slice(s);
  }
  size_t bytes() const { return cos.bytes() + sin.bytes(); }
};

/* ---------------------------------------------------------------- KV cache */

struct KvCache {
  DeviceBuffer<uint16_t> k, v;   /* [n_kv][max_seq][head_dim] fp16 */
  DeviceBuffer<float> partials;  /* split scratch, sized by the library */
  size_t n_kv, head_dim, max_seq;

  KvCache(size_t n_kv_, size_t n_q, size_t head_dim_, size_t max_seq_)
      : n_kv(n_kv_), head_dim(head_dim_), max_seq(max_seq_) {
    const size_t n = n_kv * max_seq * head_dim;
    const int32_t floats = wst_attn_partial_floats(static_cast<int32_t>(n_q),
                                                   static_cast<int32_t>(head_dim),
                                                   static_cast<int32_t>(max_seq));
    k = DeviceBuffer<uint16_t>::zeros(n);
    v = DeviceBuffer<uint16_t>::zeros(n);
    partials = DeviceBuffer<float>::zeros(static_cast<size_t>(floats > 1 ? floats : 1));
  }
  const DeviceBuffer<uint16_t> &keys() const { return k; }
  const DeviceBuffer<uint16_t> &values() const { return v; }
  size_t bytes() const { return k.bytes() + v.bytes() + partials.bytes(); }
};

/* One layer's cache in e4m3 bytes (the engine's roadmap names an 8-bit cache,
 * docs/ROADMAP.md:206; it has no type for it yet): a stored byte times k_scale / v_scale is
 * the key / value.  Same shape and scratch as KvCache. */
struct KvCacheFp8 {
  DeviceBuffer<uint8_t> k, v;    /* [n_kv][max_seq][head_dim] e4m3 */
  DeviceBuffer<float> partials;  /* split scratch, sized by the library */
  size_t n_kv, head_dim, max_seq;
  float k_scale, v_scale;

  KvCacheFp8(size_t n_kv_, size_t n_q, size_t head_dim_, size_t max_seq_, float k_scale_ = 1.f,
             float v_scale_ = 1.f)
      : n_kv(n_kv_), head_dim(head_dim_), max_seq(max_seq_), k_scale(k_scale_), v_scale(v_scale_) {
    const size_t n = n_kv * max_seq * head_dim;
    const int32_t floats = wst_attn_partial_floats(static_cast<int32_t>(n_q),
                                                   static_cast<int32_t>(head_dim),
                                                   static_cast<int32_t>(max_seq));
    k = DeviceBuffer<uint8_t>::zeros(n);
    v = DeviceBuffer<uint8_t>::zeros(n);
    partials = DeviceBuffer<float>::zeros(static_cast<size_t>(floats > 1 ? floats : 1));
  }
  size_t bytes() const { return k.bytes() + v.bytes() + partials.bytes(); }
};

struct DeviceCursor {
  DeviceBuffer<int32_t> buf;
  explicit DeviceCursor(int32_t value) : buf(DeviceBuffer<int32_t>::from_slice({value})) {}
  void set(int32_t value) { buf.copy_from_host({value}); }
  int32_t get() const { return buf.to_vec()[0]; }
  void advance(size_t max_seq) { check(wst_advance_pos(buf.as_mut_ptr(), static_cast<int32_t>(max_seq))); }
};

struct QkNorm {
  const DeviceBuffer<uint16_t> *q = nullptr;
  const DeviceBuffer<uint16_t> *k = nullptr;
  float eps = 0.f;
};

namespace detail {
struct NormPtrs { const void *q; const void *k; float eps; };
inline NormPtrs norm_ptrs(const QkNorm *n) {
  if (!n) return {nullptr, nullptr, 0.f};
  return {n->q->as_ptr(), n->k->as_ptr(), n->eps};
}
inline std::string S(size_t v) { return std::to_string(v); }
}  // namespace detail

/* ------------------------------------------------------------------ decode */

namespace decode {

inline void rope_cache(DeviceBuffer<float> &qkv, KvCache &cache, const RopeTable &table, size_t n_q,
                       const DeviceCursor &pos, const QkNorm *qk_norm = nullptr) {
  using detail::S;
  const size_t hd = cache.head_dim, want = (n_q + 2 * cache.n_kv) * hd;
  if (qkv.len() != want)
    throw Error::shape("rope_cache: qkv[" + S(qkv.len()) + "] should be (" + S(n_q) + " + 2*" +
                       S(cache.n_kv) + ") * " + S(hd) + " = " + S(want));
  if (table.half_dim != hd / 2 || table.max_seq < cache.max_seq)
    throw Error::shape("rope_cache: rotary table does not match the cache geometry");
  if (qk_norm && (qk_norm->q->len() != hd || qk_norm->k->len() != hd))
    throw Error::shape("qk_norm: gains are q[" + S(qk_norm->q->len()) + "], k[" +
                       S(qk_norm->k->len()) + "]; both must be head_dim " + S(hd));
  const auto n = detail::norm_ptrs(qk_norm);
  check(wst_rope_cache(qkv.as_mut_ptr(), cache.k.as_mut_ptr(), cache.v.as_mut_ptr(),
                       table.cos.as_ptr(), table.sin.as_ptr(), static_cast<int32_t>(n_q),
                       static_cast<int32_t>(cache.n_kv), static_cast<int32_t>(hd),
                       pos.buf.as_ptr(), static_cast<int32_t>(cache.max_seq), n.q, n.k, n.eps));
}

inline void attn_decode(const DeviceBuffer<float> &qkv, KvCache &cache, DeviceBuffer<uint16_t> &out,
                        size_t n_q, const DeviceCursor &pos) {
  using detail::S;
  const size_t hd = cache.head_dim;
  if (qkv.len() < n_q * hd || out.len() != n_q * hd)
    throw Error::shape("attn_decode: qkv[" + S(qkv.len()) + "] must hold at least " + S(n_q) + "*" +
                       S(hd) + " queries and out[" + S(out.len()) + "] exactly that");
  check(wst_attn_decode(qkv.as_ptr(), cache.k.as_ptr(), cache.v.as_ptr(),
                        cache.partials.as_mut_ptr(), out.as_mut_ptr(), static_cast<int32_t>(n_q),
                        static_cast<int32_t>(cache.n_kv), static_cast<int32_t>(hd),
                        pos.buf.as_ptr(), static_cast<int32_t>(cache.max_seq),
                        1.0f / std::sqrt(static_cast<float>(hd))));
}

/* The same two steps over an 8-bit cache: the append stores round-to-nearest-even e4m3 of
 * value / scale, the attention reads the bytes back times the scale (head_dim 128, at most
 * 16 query heads per KV head). */
inline void rope_cache_fp8(DeviceBuffer<float> &qkv, KvCacheFp8 &cache, const RopeTable &table,
                           size_t n_q, const DeviceCursor &pos, const QkNorm *qk_norm = nullptr) {
  using detail::S;
  const size_t hd = cache.head_dim, want = (n_q + 2 * cache.n_kv) * hd;
  if (qkv.len() != want)
    throw Error::shape("rope_cache_fp8: qkv[" + S(qkv.len()) + "] should be (" + S(n_q) + " + 2*" +
                       S(cache.n_kv) + ") * " + S(hd) + " = " + S(want));
  if (table.half_dim != hd / 2 || table.max_seq < cache.max_seq)
    throw Error::shape("rope_cache_fp8: rotary table does not match the cache geometry");
  const auto n = detail::norm_ptrs(qk_norm);
  check(wst_b200_rope_cache_fp8(qkv.as_mut_ptr(), cache.k.as_mut_ptr(), cache.v.as_mut_ptr(),
                                table.cos.as_ptr(), table.sin.as_ptr(), static_cast<int32_t>(n_q),
                                static_cast<int32_t>(cache.n_kv), static_cast<int32_t>(hd),
                                pos.buf.as_ptr(), 0, 1, static_cast<int32_t>(cache.max_seq), n.q, n.k,
                                n.eps, cache.k_scale, cache.v_scale));
}

inline void attn_decode_fp8(const DeviceBuffer<float> &qkv, KvCacheFp8 &cache,
                            DeviceBuffer<uint16_t> &out, size_t n_q, const DeviceCursor &pos) {
  using detail::S;
  const size_t hd = cache.head_dim;
  if (qkv.len() < n_q * hd || out.len() != n_q * hd)
    throw Error::shape("attn_decode_fp8: qkv[" + S(qkv.len()) + "] must hold at least " + S(n_q) +
                       "*" + S(hd) + " queries and out[" + S(out.len()) + "] exactly that");
  check(wst_b200_attn_decode_fp8(qkv.as_ptr(), cache.k.as_ptr(), cache.v.as_ptr(),
                                 cache.partials.as_mut_ptr(), out.as_mut_ptr(),
                                 static_cast<int32_t>(n_q), static_cast<int32_t>(cache.n_kv),
                                 static_cast<int32_t>(hd), pos.buf.as_ptr(),
                                 static_cast<int32_t>(cache.max_seq),
                                 1.0f / std::sqrt(static_cast<float>(hd)), cache.k_scale,
                                 cache.v_scale));
}

/* One shard of a KV sequence split over GPUs: (m, l, acc) per head over rows [0, *len). */
inline void attn_decode_partial(const DeviceBuffer<float> &qkv, KvCache &shard,
                                DeviceBuffer<float> &out_partial, size_t n_q,
                                const DeviceCursor &len) {
  const size_t hd = shard.head_dim;
  if (qkv.len() < n_q * hd || out_partial.len() != n_q * (hd + 2))
    throw Error::shape("attn_decode_partial: qkv must hold n_q*head_dim queries and out "
                       "n_q*(head_dim+2) floats");
  check(wst_attn_decode_partial(qkv.as_ptr(), shard.k.as_ptr(), shard.v.as_ptr(),
                                shard.partials.as_mut_ptr(), out_partial.as_mut_ptr(),
                                static_cast<int32_t>(n_q), static_cast<int32_t>(shard.n_kv),
                                static_cast<int32_t>(hd), len.buf.as_ptr(),
                                static_cast<int32_t>(shard.max_seq),
                                1.0f / std::sqrt(static_cast<float>(hd))));
}

inline void attn_merge_partials(const DeviceBuffer<float> &parts, DeviceBuffer<uint16_t> &out,
                                size_t n_q, size_t head_dim) {
  const size_t per = n_q * (head_dim + 2);
  if (parts.len() == 0 || parts.len() % per != 0 || out.len() != n_q * head_dim)
    throw Error::shape("attn_merge_partials: parts must be [n_parts][n_q][head_dim+2] and out "
                       "[n_q][head_dim]");
  check(wst_attn_merge_partials(parts.as_ptr(), out.as_mut_ptr(),
                                static_cast<int32_t>(parts.len() / per),
                                static_cast<int32_t>(n_q), static_cast<int32_t>(head_dim)));
}

}  // namespace decode

/* ------------------------------------------------------------------- chunk */

namespace chunk {

inline void rope_cache(DeviceBuffer<float> &qkv, KvCache &cache, const RopeTable &table, size_t n_q,
                       size_t pos0, size_t n, const QkNorm *qk_norm = nullptr) {
  using detail::S;
  const size_t hd = cache.head_dim, stride = (n_q + 2 * cache.n_kv) * hd;
  if (qkv.len() < n * stride)
    throw Error::shape("rope_cache_chunk: qkv[" + S(qkv.len()) + "] needs " + S(n) + " * " + S(stride));
  if (table.half_dim != hd / 2 || table.max_seq < cache.max_seq)
    throw Error::shape("rope_cache_chunk: rotary table does not match the cache geometry");
  if (pos0 + n > cache.max_seq)
    throw Error::shape("rope_cache_chunk: chunk [" + S(pos0) + ", " + S(pos0 + n) +
                       ") runs past the " + S(cache.max_seq) + " token cache");
  if (qk_norm && (qk_norm->q->len() != hd || qk_norm->k->len() != hd))
    throw Error::shape("rope_cache_chunk: gains are q[" + S(qk_norm->q->len()) + "], k[" +
                       S(qk_norm->k->len()) + "]; both must be head_dim " + S(hd));
  const auto np = detail::norm_ptrs(qk_norm);
  check(wst_rope_cache_chunk(qkv.as_mut_ptr(), cache.k.as_mut_ptr(), cache.v.as_mut_ptr(),
                             table.cos.as_ptr(), table.sin.as_ptr(), static_cast<int32_t>(n_q),
                             static_cast<int32_t>(cache.n_kv), static_cast<int32_t>(hd),
                             static_cast<int32_t>(pos0), static_cast<int32_t>(n),
                             static_cast<int32_t>(cache.max_seq), np.q, np.k, np.eps));
}

inline void attn(const DeviceBuffer<float> &qkv, const KvCache &cache, DeviceBuffer<uint16_t> &out,
                 size_t n_q, size_t pos0, size_t n) {
  using detail::S;
  const size_t hd = cache.head_dim, stride = (n_q + 2 * cache.n_kv) * hd;
  if (qkv.len() < n * stride)
    throw Error::shape("attn_chunk: qkv[" + S(qkv.len()) + "] needs " + S(n) + " * " + S(stride));
  if (out.len() < n * n_q * hd)
    throw Error::shape("attn_chunk: out[" + S(out.len()) + "] needs " + S(n) + " * " + S(n_q) + " * " + S(hd));
  if (pos0 + n > cache.max_seq)
    throw Error::shape("attn_chunk: chunk [" + S(pos0) + ", " + S(pos0 + n) + ") runs past the " +
                       S(cache.max_seq) + " token cache");
  check(wst_attn_chunk(qkv.as_ptr(), cache.k.as_ptr(), cache.v.as_ptr(), out.as_mut_ptr(),
                       static_cast<int32_t>(n_q), static_cast<int32_t>(cache.n_kv),
                       static_cast<int32_t>(hd), static_cast<int32_t>(pos0),
                       static_cast<int32_t>(n), static_cast<int32_t>(cache.max_seq),
                       1.0f / std::sqrt(static_cast<float>(hd))));
}

/* Several sequences per launch: caches [n_seq][n_kv][max_seq][head_dim], qkv
 * [n_seq][n][stride], out [n_seq][n][n_q*head_dim], one chunk start per sequence in
 * device memory (no counterpart in the engine, which runs one sequence). */
struct KvCacheBatch {
  DeviceBuffer<uint16_t> k, v;
  size_t n_seq, n_kv, head_dim, max_seq;
  KvCacheBatch(size_t n_seq_, size_t n_kv_, size_t head_dim_, size_t max_seq_)
      : n_seq(n_seq_), n_kv(n_kv_), head_dim(head_dim_), max_seq(max_seq_) {
    k = DeviceBuffer<uint16_t>::zeros(n_seq * n_kv * max_seq * head_dim);
    v = DeviceBuffer<uint16_t>::zeros(n_seq * n_kv * max_seq * head_dim);
  }
};

inline void rope_cache_batch(DeviceBuffer<float> &qkv, KvCacheBatch &cache, const RopeTable &table,
                             size_t n_q, const DeviceBuffer<int32_t> &seq_pos0, size_t n,
                             const QkNorm *qk_norm = nullptr) {
  using detail::S;
  const size_t hd = cache.head_dim, stride = (n_q + 2 * cache.n_kv) * hd;
  if (qkv.len() < cache.n_seq * n * stride)
    throw Error::shape("rope_cache_chunk_batch: qkv[" + S(qkv.len()) + "] needs " +
                       S(cache.n_seq) + " * " + S(n) + " * " + S(stride));
  if (seq_pos0.len() != cache.n_seq)
    throw Error::shape("rope_cache_chunk_batch: one chunk start per sequence");
  if (table.half_dim != hd / 2 || table.max_seq < cache.max_seq)
    throw Error::shape("rope_cache_chunk_batch: rotary table does not match the cache geometry");
  const auto np = detail::norm_ptrs(qk_norm);
  check(wst_rope_cache_chunk_batch(qkv.as_mut_ptr(), cache.k.as_mut_ptr(), cache.v.as_mut_ptr(),
                                   table.cos.as_ptr(), table.sin.as_ptr(), seq_pos0.as_ptr(),
                                   static_cast<int32_t>(cache.n_seq), static_cast<int32_t>(n_q),
                                   static_cast<int32_t>(cache.n_kv), static_cast<int32_t>(hd),
                                   static_cast<int32_t>(n), static_cast<int32_t>(cache.max_seq),
                                   np.q, np.k, np.eps));
}

inline void attn_batch(const DeviceBuffer<float> &qkv, const KvCacheBatch &cache,
                       DeviceBuffer<uint16_t> &out, size_t n_q,
                       const DeviceBuffer<int32_t> &seq_pos0, size_t n) {
  using detail::S;
  const size_t hd = cache.head_dim, stride = (n_q + 2 * cache.n_kv) * hd;
  if (qkv.len() < cache.n_seq * n * stride)
    throw Error::shape("attn_chunk_batch: qkv[" + S(qkv.len()) + "] needs " + S(cache.n_seq) +
                       " * " + S(n) + " * " + S(stride));
  if (out.len() < cache.n_seq * n * n_q * hd) throw Error::shape("attn_chunk_batch: out too small");
  if (seq_pos0.len() != cache.n_seq)
    throw Error::shape("attn_chunk_batch: one chunk start per sequence");
  check(wst_attn_chunk_batch(qkv.as_ptr(), cache.k.as_ptr(), cache.v.as_ptr(), out.as_mut_ptr(),
                             seq_pos0.as_ptr(), static_cast<int32_t>(cache.n_seq),
                             static_cast<int32_t>(n_q), static_cast<int32_t>(cache.n_kv),
                             static_cast<int32_t>(hd), static_cast<int32_t>(n),
                             static_cast<int32_t>(cache.max_seq),
                             1.0f / std::sqrt(static_cast<float>(hd))));
}

/* y[j] = W x[j] + b for every j < n, or += when `accumulate` (src/chunk.rs:55-99). */
inline void gemm_fp16(const DeviceBuffer<uint16_t> &w, const DeviceBuffer<uint16_t> &x,
                      const DeviceBuffer<uint16_t> *bias, DeviceBuffer<float> &y, size_t in_features,
                      size_t out_features, size_t n, bool accumulate) {
  using detail::S;
  if (x.len() != n * in_features || y.len() != n * out_features)
    throw Error::shape("gemm_fp16: x[" + S(x.len()) + "], y[" + S(y.len()) + "] do not match n=" +
                       S(n) + ", in=" + S(in_features) + ", out=" + S(out_features));
  if (w.len() != in_features * out_features)
    throw Error::shape("gemm_fp16: weights have " + S(w.len()) + " elements, expected " +
                       S(in_features) + "*" + S(out_features));
  if (bias && bias->len() != out_features)
    throw Error::shape("gemm_fp16: bias has " + S(bias->len()) + " elements, expected " +
                       S(out_features));
  check(wst_gemm_fp16(w.as_ptr(), x.as_ptr(), bias ? bias->as_ptr() : nullptr, y.as_mut_ptr(),
                      static_cast<int32_t>(in_features), static_cast<int32_t>(out_features),
                      static_cast<int32_t>(n), accumulate ? 1 : 0));
}

/* Tokens one weight pass serves (src/chunk.rs:20). */
inline size_t max_tokens() {
  const int32_t m = wst_chunk_max_tokens();
  return m < 1 ? 1 : static_cast<size_t>(m);
}

/* The qkv projection with RoPE, head norm and cache append in its epilogue; the rotated
 * queries land in q_out [n_seq * n][n_q * head_dim] (no counterpart in the engine). */
inline void qkv_rope_append_batch(const DeviceBuffer<uint16_t> &w, const DeviceBuffer<uint16_t> &x,
                                  const DeviceBuffer<uint16_t> *bias, DeviceBuffer<uint16_t> &q_out,
                                  KvCacheBatch &cache, const RopeTable &table, size_t n_q,
                                  const DeviceBuffer<int32_t> &seq_pos0, size_t n,
                                  const QkNorm *qk_norm = nullptr) {
  using detail::S;
  const size_t hd = cache.head_dim, width = (n_q + 2 * cache.n_kv) * hd, tokens = cache.n_seq * n;
  if (tokens == 0 || x.len() % tokens != 0)
    throw Error::shape("qkv_rope_append_batch: x[" + S(x.len()) + "] is not " + S(tokens) + " rows");
  const size_t in_f = x.len() / tokens;
  if (w.len() != width * in_f)
    throw Error::shape("qkv_rope_append_batch: w[" + S(w.len()) + "] needs " + S(width) + " * " + S(in_f));
  if (q_out.len() < tokens * n_q * hd)
    throw Error::shape("qkv_rope_append_batch: q_out[" + S(q_out.len()) + "] needs " + S(tokens) +
                       " * " + S(n_q) + " * " + S(hd));
  if (bias && bias->len() != width)
    throw Error::shape("qkv_rope_append_batch: bias has " + S(bias->len()) + " elements, expected " + S(width));
  if (seq_pos0.len() != cache.n_seq)
    throw Error::shape("qkv_rope_append_batch: seq_pos0 needs one entry per sequence");
  if (table.half_dim != hd / 2)
    throw Error::shape("qkv_rope_append_batch: rotary table does not match the head width");
  if (qk_norm && (qk_norm->q->len() != hd || qk_norm->k->len() != hd))
    throw Error::shape("qkv_rope_append_batch: gains must be head_dim " + S(hd));
  const auto np = detail::norm_ptrs(qk_norm);
  check(wst_b200_qkv_rope_append_batch(
      w.as_ptr(), x.as_ptr(), bias ? bias->as_ptr() : nullptr, q_out.as_mut_ptr(), cache.k.as_mut_ptr(),
      cache.v.as_mut_ptr(), table.cos.as_ptr(), table.sin.as_ptr(), seq_pos0.as_ptr(),
      static_cast<int32_t>(in_f), static_cast<int32_t>(cache.n_seq), static_cast<int32_t>(n),
      static_cast<int32_t>(n_q), static_cast<int32_t>(cache.n_kv), static_cast<int32_t>(hd),
      static_cast<int32_t>(cache.max_seq), static_cast<int32_t>(table.max_seq), np.q, np.k, np.eps));
}

/* attn_batch over the fp16 query rows that qkv_rope_append_batch leaves. */
inline void attn_batch_q16(const DeviceBuffer<uint16_t> &q16, const KvCacheBatch &cache,
                           DeviceBuffer<uint16_t> &out, size_t n_q,
                           const DeviceBuffer<int32_t> &seq_pos0, size_t n) {
  using detail::S;
  const size_t hd = cache.head_dim, need = cache.n_seq * n * n_q * hd;
  if (q16.len() < need || out.len() < need)
    throw Error::shape("attn_chunk_batch_q16: q[" + S(q16.len()) + "] and out[" + S(out.len()) +
                       "] need " + S(need));
  check(wst_b200_attn_chunk_batch_q16(q16.as_ptr(), cache.k.as_ptr(), cache.v.as_ptr(),
                                      out.as_mut_ptr(), seq_pos0.as_ptr(),
                                      static_cast<int32_t>(cache.n_seq), static_cast<int32_t>(n_q),
                                      static_cast<int32_t>(cache.n_kv), static_cast<int32_t>(hd),
                                      static_cast<int32_t>(n), static_cast<int32_t>(cache.max_seq),
                                      1.0f / std::sqrt(static_cast<float>(hd))));
}

}  // namespace chunk

/* --------------------------------------- one long sequence over several GPUs */

/* This rank's mailbox for wst_attn_exchange_merge and the other ranks' mapped into
 * this process.  The 64-byte handles travel between the processes by whatever
 * channel the host has (`handle()` out, `import_peer()` in, rank order). */
class PeerMailbox {
 public:
  PeerMailbox(int rank, int world, size_t n_q, size_t head_dim)
      : rank_(rank), world_(world), n_q_(n_q), head_dim_(head_dim), addr_(world, nullptr) {
    const size_t bytes = 2 * static_cast<size_t>(world) * n_q * (head_dim + 2) * 8;
    check(wst_malloc(&own_, bytes));
    check(wst_memset(own_, 0, bytes));
    check(wst_device_synchronize());
    addr_[rank] = own_;
    state_ = DeviceBuffer<uint32_t>::zeros(n_q);
  }
  PeerMailbox(const PeerMailbox &) = delete;
  PeerMailbox &operator=(const PeerMailbox &) = delete;
  ~PeerMailbox() {
    for (int g = 0; g < world_; ++g)
      if (g != rank_ && addr_[g]) wst_b200_ipc_close(addr_[g]);
    if (own_) wst_free(own_);
  }
  std::vector<uint8_t> handle() const {
    std::vector<uint8_t> h(64);
    check(wst_b200_ipc_export(own_, h.data()));
    return h;
  }
  void import_peer(int g, const std::vector<uint8_t> &handle64) {
    if (g == rank_ || g < 0 || g >= world_ || handle64.size() != 64)
      throw Error::shape("PeerMailbox::import_peer: bad rank or handle");
    check(wst_b200_ipc_import(handle64.data(), &addr_[g]));
  }
  /* after every peer has been imported */
  void seal() {
    std::vector<uint64_t> a(world_);
    for (int g = 0; g < world_; ++g) {
      if (!addr_[g]) throw Error::shape("PeerMailbox::seal: a rank is missing");
      a[g] = reinterpret_cast<uint64_t>(addr_[g]);
    }
    table_ = DeviceBuffer<uint64_t>::from_slice(a);
  }
  /* Attention over this rank's shard (rows [0, *len) of `shard`) and the exchange as one
   * call: wst_attn_decode_sharded.  q replicated on every rank; every rank gets `out`. */
  void decode(const DeviceBuffer<float> &qkv, KvCache &shard, DeviceBuffer<uint16_t> &out,
              const DeviceCursor &len) {
    const size_t hd = shard.head_dim;
    if (hd != head_dim_ || qkv.len() < n_q_ * hd || out.len() != n_q_ * hd)
      throw Error::shape("PeerMailbox::decode: qkv must hold n_q*head_dim queries, out exactly that");
    check(wst_attn_decode_sharded(qkv.as_ptr(), shard.k.as_ptr(), shard.v.as_ptr(),
                                  shard.partials.as_mut_ptr(), out.as_mut_ptr(),
                                  static_cast<int32_t>(n_q_), static_cast<int32_t>(shard.n_kv),
                                  static_cast<int32_t>(hd), len.buf.as_ptr(),
                                  static_cast<int32_t>(shard.max_seq),
                                  1.0f / std::sqrt(static_cast<float>(hd)), table_.as_ptr(),
                                  state_.as_mut_ptr(), rank_, world_));
  }
  void merge(const DeviceBuffer<float> &my_triples, DeviceBuffer<uint16_t> &out) {
    if (my_triples.len() != n_q_ * (head_dim_ + 2) || out.len() != n_q_ * head_dim_)
      throw Error::shape("PeerMailbox::merge: triples [n_q][head_dim+2], out [n_q][head_dim]");
    check(wst_attn_exchange_merge(my_triples.as_ptr(), out.as_mut_ptr(), table_.as_ptr(),
                                  state_.as_mut_ptr(), rank_, world_, static_cast<int32_t>(n_q_),
                                  static_cast<int32_t>(head_dim_)));
  }

 private:
  int rank_, world_;
  size_t n_q_, head_dim_;
  void *own_ = nullptr;
  std::vector<void *> addr_;
  DeviceBuffer<uint64_t> table_;
  DeviceBuffer<uint32_t> state_;
};

/* ------------------------------------------------------------ paged batch */

struct PagedKvCache {
  static constexpr size_t kPage = 16;
  DeviceBuffer<uint16_t> k, v;          /* [n_pages][n_kv][16][head_dim] */
  DeviceBuffer<int32_t> page_table;     /* [n_seq][max_pages], -1 = unmapped */
  size_t n_pages, n_kv, head_dim, n_seq, max_pages;

  PagedKvCache(size_t n_pages_, size_t n_kv_, size_t head_dim_, size_t n_seq_, size_t max_pages_)
      : n_pages(n_pages_), n_kv(n_kv_), head_dim(head_dim_), n_seq(n_seq_), max_pages(max_pages_) {
    k = DeviceBuffer<uint16_t>::zeros(n_pages * n_kv * kPage * head_dim);
    v = DeviceBuffer<uint16_t>::zeros(n_pages * n_kv * kPage * head_dim);
    page_table = DeviceBuffer<int32_t>::from_slice(std::vector<int32_t>(n_seq * max_pages, -1));
  }
};

namespace paged {

inline void rope_cache(DeviceBuffer<float> &qkv, PagedKvCache &cache, const RopeTable &table,
                       size_t n_q, const DeviceBuffer<int32_t> &seq_pos0,
                       const DeviceBuffer<int32_t> &cu_tokens, size_t total_tokens,
                       const QkNorm *qk_norm = nullptr) {
  const size_t hd = cache.head_dim, stride = (n_q + 2 * cache.n_kv) * hd;
  if (qkv.len() < total_tokens * stride) throw Error::shape("rope_cache_paged: qkv too short");
  if (seq_pos0.len() != cache.n_seq || cu_tokens.len() != cache.n_seq + 1)
    throw Error::shape("rope_cache_paged: seq_pos0 needs n_seq and cu_tokens n_seq+1 entries");
  if (table.half_dim != hd / 2) throw Error::shape("rope_cache_paged: rotary table does not match head_dim");
  const auto np = detail::norm_ptrs(qk_norm);
  check(wst_rope_cache_paged(qkv.as_mut_ptr(), cache.k.as_mut_ptr(), cache.v.as_mut_ptr(),
                             table.cos.as_ptr(), table.sin.as_ptr(), cache.page_table.as_ptr(),
                             seq_pos0.as_ptr(), cu_tokens.as_ptr(), static_cast<int32_t>(cache.n_seq),
                             static_cast<int32_t>(total_tokens), static_cast<int32_t>(cache.max_pages),
                             static_cast<int32_t>(PagedKvCache::kPage), static_cast<int32_t>(cache.n_pages),
                             static_cast<int32_t>(n_q), static_cast<int32_t>(cache.n_kv),
                             static_cast<int32_t>(hd), static_cast<int32_t>(table.max_seq), np.q,
                             np.k, np.eps));
}

inline void attn_verify(const DeviceBuffer<float> &qkv, const PagedKvCache &cache,
                        DeviceBuffer<uint16_t> &out, DeviceBuffer<float> &scratch, size_t n_q,
                        const DeviceBuffer<int32_t> &seq_pos0, const DeviceBuffer<int32_t> &cu_tokens,
                        size_t total_tokens, size_t max_tokens_per_seq, size_t max_len) {
  const size_t hd = cache.head_dim;
  const int64_t need = wst_attn_verify_scratch_floats(
      static_cast<int32_t>(cache.n_seq), static_cast<int32_t>(max_tokens_per_seq),
      static_cast<int32_t>(n_q), static_cast<int32_t>(cache.n_kv), static_cast<int32_t>(hd),
      static_cast<int32_t>(max_len));
  if (static_cast<int64_t>(scratch.len()) < need) throw Error::shape("attn_verify: scratch too small");
  if (out.len() < total_tokens * n_q * hd) throw Error::shape("attn_verify: out too small");
  check(wst_attn_verify_paged(qkv.as_ptr(), cache.k.as_ptr(), cache.v.as_ptr(),
                              cache.page_table.as_ptr(), seq_pos0.as_ptr(), cu_tokens.as_ptr(),
                              scratch.as_mut_ptr(), out.as_mut_ptr(), static_cast<int32_t>(cache.n_seq),
                              static_cast<int32_t>(total_tokens),
                              static_cast<int32_t>(max_tokens_per_seq),
                              static_cast<int32_t>(cache.max_pages),
                              static_cast<int32_t>(PagedKvCache::kPage),
                              static_cast<int32_t>(cache.n_pages), static_cast<int32_t>(n_q),
                              static_cast<int32_t>(cache.n_kv), static_cast<int32_t>(hd),
                              static_cast<int32_t>(max_len), 1.0f / std::sqrt(static_cast<float>(hd))));
}

}  // namespace paged

/* ------------------------------------------------------- graphs and events */

class Graph {
 public:
  /* Runs `body` once eagerly (lazy initialisation), then captures it. */
  template <class F>
  static Graph capture(F &&body) {
    body();
    check(wst_stream_sync());
    check(wst_graph_capture_begin());
    try {
      body();
    } catch (...) {
      void *dead = nullptr;
      wst_graph_capture_end(&dead);
      wst_graph_destroy(dead);
      throw;
    }
    Graph g;
    check(wst_graph_capture_end(&g.exec_));
    return g;
  }
  Graph(Graph &&o) noexcept : exec_(o.exec_) { o.exec_ = nullptr; }
  Graph(const Graph &) = delete;
  ~Graph() { wst_graph_destroy(exec_); }
  void launch() const { check(wst_graph_launch(exec_)); }

 private:
  Graph() = default;
  void *exec_ = nullptr;
};

class Event {
 public:
  Event() { check(wst_event_create(&ev_)); }
  Event(const Event &) = delete;
  ~Event() { wst_event_destroy(ev_); }
  void record() { check(wst_event_record(ev_)); }
  static float elapsed_ms(const Event &a, const Event &b) {
    float ms = 0.f;
    check(wst_event_elapsed_ms(a.ev_, b.ev_, &ms));
    return ms;
  }

 private:
  void *ev_ = nullptr;
};

}  // namespace whetstone
