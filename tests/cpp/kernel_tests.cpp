/* The reference's kernel tests for the attention path, written against the C++
 * host layer (whetstone_b200/host/whetstone_host.hpp) the way the originals are
 * written against the Rust one:
 *
 *   crates/whetstone-kernels/tests/decode_kernels.rs:91-410
 *   crates/whetstone-kernels/tests/chunk_kernels.rs:51-108 (the fp16 projection), :263-360
 *
 * Same closed-form inputs, same LCG, same tolerances.  Prints one line per test
 * and exits non-zero if any failed; needs a B200.
 */
#include <cmath>
#include <cstdio>
#include <cstring>
#include <functional>
#include <string>
#include <vector>

#include "whetstone_host.hpp"

using namespace whetstone;

/* ---- fp16 <-> fp32 on the host (round to nearest even), like the `half` crate */
static uint16_t f32_to_f16(float f) {
  uint32_t x;
  std::memcpy(&x, &f, 4);
  const uint32_t sign = (x >> 16) & 0x8000u;
  int32_t exp = static_cast<int32_t>((x >> 23) & 0xff) - 127 + 15;
  uint32_t man = x & 0x7fffffu;
  if (((x >> 23) & 0xff) == 0xff) return static_cast<uint16_t>(sign | 0x7c00u | (man ? 0x200u : 0));
  if (exp >= 31) return static_cast<uint16_t>(sign | 0x7c00u);
  if (exp <= 0) {
    if (exp < -10) return static_cast<uint16_t>(sign);
    man |= 0x800000u;
    const int shift = 14 - exp;
    uint32_t half = man >> shift;
    const uint32_t rem = man & ((1u << shift) - 1), mid = 1u << (shift - 1);
    if (rem > mid || (rem == mid && (half & 1))) ++half;
    return static_cast<uint16_t>(sign | half);
  }
  uint32_t half = (static_cast<uint32_t>(exp) << 10) | (man >> 13);
  const uint32_t rem = man & 0x1fffu;
  if (rem > 0x1000u || (rem == 0x1000u && (half & 1))) ++half;
  return static_cast<uint16_t>(sign | half);
}
static float f16_to_f32(uint16_t h) {
  const uint32_t sign = (h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1f, man = h & 0x3ffu, x;
  if (exp == 0) {
    if (man == 0) {
      x = sign;
    } else {
      int e = -1;
      do { ++e; man <<= 1; } while (!(man & 0x400u));
      x = sign | ((127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
    }
  } else if (exp == 31) {
    x = sign | 0x7f800000u | (man << 13);
  } else {
    x = sign | ((exp - 15 + 127) << 23) | (man << 13);
  }
  float f;
  std::memcpy(&f, &x, 4);
  return f;
}
static std::vector<uint16_t> f16v(const std::vector<float> &v) {
  std::vector<uint16_t> o(v.size());
  for (size_t i = 0; i < v.size(); ++i) o[i] = f32_to_f16(v[i]);
  return o;
}
static std::vector<float> from_f16(const std::vector<uint16_t> &v) {
  std::vector<float> o(v.size());
  for (size_t i = 0; i < v.size(); ++i) o[i] = f16_to_f32(v[i]);
  return o;
}

/* chunk_kernels.rs:31-39 */
static std::vector<float> noise(size_t n, uint64_t seed) {
  uint64_t s = seed * 6364136223846793005ull + 1ull;
  std::vector<float> o(n);
  for (auto &x : o) {
    s = s * 6364136223846793005ull + 1442695040888963407ull;
    x = static_cast<float>(s >> 33) / static_cast<float>(1ull << 31) - 1.0f;
  }
  return o;
}

struct Failure { std::string what; };
#define REQUIRE(cond, msg) do { if (!(cond)) throw Failure{std::string(msg)}; } while (0)

static std::vector<float> seq(size_t n, int mod, float div) {
  std::vector<float> v(n);
  for (size_t i = 0; i < n; ++i) v[i] = static_cast<float>(i % mod) / div - 1.0f;
  return v;
}
static std::vector<float> cat3(const std::vector<float> &a, const std::vector<float> &b,
                               const std::vector<float> &c) {
  std::vector<float> o(a);
  o.insert(o.end(), b.begin(), b.end());
  o.insert(o.end(), c.begin(), c.end());
  return o;
}

static void rope_uses_the_half_rotation_layout() {
  const size_t n_q = 2, n_kv = 1, hd = 64, max_seq = 8, pos = 3;
  const double theta = 1e6;
  auto q = seq(n_q * hd, 31, 15.f), k = seq(n_kv * hd, 23, 11.f), v = seq(n_kv * hd, 19, 9.f);
  RopeTable table(max_seq, hd, theta);
  KvCache cache(n_kv, n_q, hd, max_seq);
  auto qd = DeviceBuffer<float>::from_slice(cat3(q, k, v));
  DeviceCursor cursor(static_cast<int32_t>(pos));
  decode::rope_cache(qd, cache, table, n_q, cursor);
  auto got = qd.to_vec();
  const size_t half = hd / 2;
  for (size_t h = 0; h < n_q; ++h)
    for (size_t j = 0; j < half; ++j) {
      const double inv = std::pow(theta, -static_cast<double>(j) / half);
      const double s = std::sin(pos * inv), c = std::cos(pos * inv);
      const double x1 = q[h * hd + j], x2 = q[h * hd + j + half];
      REQUIRE(std::fabs(got[h * hd + j] - static_cast<float>(x1 * c - x2 * s)) < 1e-5f, "lo");
      REQUIRE(std::fabs(got[h * hd + j + half] - static_cast<float>(x2 * c + x1 * s)) < 1e-5f, "hi");
    }
}

static void qk_norm_is_per_head_and_precedes_the_rotation() {
  const size_t n_q = 4, n_kv = 2, hd = 64, max_seq = 8, pos = 5;
  const double theta = 1e6;
  const float eps = 1e-6f;
  auto q = seq(n_q * hd, 31, 15.f), k = seq(n_kv * hd, 23, 11.f), v = seq(n_kv * hd, 19, 9.f);
  std::vector<float> gq(hd), gk(hd);
  for (size_t i = 0; i < hd; ++i) {
    gq[i] = 0.5f + static_cast<float>(i % 7) * 0.1f;
    gk[i] = 1.5f - static_cast<float>(i % 5) * 0.2f;
  }
  auto gqd = DeviceBuffer<uint16_t>::from_slice(f16v(gq));
  auto gkd = DeviceBuffer<uint16_t>::from_slice(f16v(gk));
  RopeTable table(max_seq, hd, theta);
  KvCache cache(n_kv, n_q, hd, max_seq);
  auto qd = DeviceBuffer<float>::from_slice(cat3(q, k, v));
  DeviceCursor cursor(static_cast<int32_t>(pos));
  QkNorm norm{&gqd, &gkd, eps};
  decode::rope_cache(qd, cache, table, n_q, cursor, &norm);
  auto got = qd.to_vec();
  const size_t half = hd / 2;
  auto reference = [&](const std::vector<float> &src, const std::vector<float> &gain, size_t h,
                       size_t j, float &w1, float &w2) {
    double ms = 0;
    for (size_t i = 0; i < hd; ++i) ms += static_cast<double>(src[h * hd + i]) * src[h * hd + i];
    const double inv = 1.0 / std::sqrt(ms / hd + eps);
    const double f = std::pow(theta, -static_cast<double>(j) / half);
    const double s = std::sin(pos * f), c = std::cos(pos * f);
    const double x1 = src[h * hd + j] * inv * f16_to_f32(f32_to_f16(gain[j]));
    const double x2 = src[h * hd + j + half] * inv * f16_to_f32(f32_to_f16(gain[j + half]));
    w1 = static_cast<float>(x1 * c - x2 * s);
    w2 = static_cast<float>(x2 * c + x1 * s);
  };
  for (size_t h = 0; h < n_q; ++h)
    for (size_t j = 0; j < half; ++j) {
      float w1, w2;
      reference(q, gq, h, j, w1, w2);
      const float tol = 1e-4f * std::fmax(std::fmax(std::fabs(w1), std::fabs(w2)), 1.0f);
      REQUIRE(std::fabs(got[h * hd + j] - w1) < tol, "q lo");
      REQUIRE(std::fabs(got[h * hd + j + half] - w2) < tol, "q hi");
    }
  auto kc = from_f16(cache.keys().to_vec());
  auto vc = from_f16(cache.values().to_vec());
  for (size_t h = 0; h < n_kv; ++h) {
    const size_t slot = (h * max_seq + pos) * hd;
    for (size_t j = 0; j < half; ++j) {
      float w1, w2;
      reference(k, gk, h, j, w1, w2);
      REQUIRE(std::fabs(kc[slot + j] - w1) < 3e-3f, "k lo");
      REQUIRE(std::fabs(kc[slot + j + half] - w2) < 3e-3f, "k hi");
    }
    for (size_t j = 0; j < hd; ++j)
      REQUIRE(std::fabs(vc[slot + j] - v[h * hd + j]) < 3e-3f, "v was modified");
  }
}

static void qk_norm_with_unit_gain_on_a_unit_rms_head_is_the_identity() {
  const size_t n_q = 2, n_kv = 1, hd = 64, max_seq = 8, pos = 2;
  std::vector<float> q(n_q * hd), k(n_kv * hd);
  for (size_t i = 0; i < q.size(); ++i) q[i] = i % 3 == 0 ? -1.f : 1.f;
  for (size_t i = 0; i < k.size(); ++i) k[i] = i % 5 == 0 ? -1.f : 1.f;
  auto v = seq(n_kv * hd, 19, 9.f);
  auto ones = f16v(std::vector<float>(hd, 1.f));
  auto gqd = DeviceBuffer<uint16_t>::from_slice(ones);
  auto gkd = DeviceBuffer<uint16_t>::from_slice(ones);
  RopeTable table(max_seq, hd, 1e6);
  const auto qkv = cat3(q, k, v);
  DeviceCursor cursor(static_cast<int32_t>(pos));
  KvCache cache_off(n_kv, n_q, hd, max_seq), cache_on(n_kv, n_q, hd, max_seq);
  auto off = DeviceBuffer<float>::from_slice(qkv);
  decode::rope_cache(off, cache_off, table, n_q, cursor);
  auto on = DeviceBuffer<float>::from_slice(qkv);
  QkNorm norm{&gqd, &gkd, 0.f};
  decode::rope_cache(on, cache_on, table, n_q, cursor, &norm);
  auto a = off.to_vec(), b = on.to_vec();
  for (size_t i = 0; i < a.size(); ++i) REQUIRE(std::fabs(a[i] - b[i]) < 1e-6f, "norm-on differs");
}

static void attention_over_one_position_returns_that_value() {
  const size_t n_q = 14, n_kv = 2, hd = 64, max_seq = 32;
  RopeTable table(max_seq, hd, 1e6);
  KvCache cache(n_kv, n_q, hd, max_seq);
  auto q = seq(n_q * hd, 29, 14.f), k = seq(n_kv * hd, 13, 6.f), v = seq(n_kv * hd, 17, 8.f);
  auto qd = DeviceBuffer<float>::from_slice(cat3(q, k, v));
  DeviceCursor cursor(0);
  decode::rope_cache(qd, cache, table, n_q, cursor);
  auto out = DeviceBuffer<uint16_t>::zeros(n_q * hd);
  decode::attn_decode(qd, cache, out, n_q, cursor);
  auto got = from_f16(out.to_vec());
  for (size_t h = 0; h < n_q; ++h) {
    const size_t kv = h / (n_q / n_kv);
    for (size_t d = 0; d < hd; ++d)
      REQUIRE(std::fabs(got[h * hd + d] - f16_to_f32(f32_to_f16(v[kv * hd + d]))) < 2e-3f, "value");
  }
}

static void attention_over_two_positions_matches_an_explicit_softmax() {
  const size_t n_q = 2, n_kv = 1, hd = 64, max_seq = 16, half = hd / 2;
  const double theta = 1e6;
  KvCache cache(n_kv, n_q, hd, max_seq);
  RopeTable table(max_seq, hd, theta);
  std::vector<std::vector<float>> ks, vs;
  for (size_t p = 0; p < 2; ++p) {
    std::vector<float> k(hd), v(hd);
    for (size_t i = 0; i < hd; ++i) {
      k[i] = static_cast<float>((i + 7 * p) % 11) / 5.f - 1.f;
      v[i] = static_cast<float>((i + 3 * p) % 7) / 3.f - 1.f;
    }
    auto qd = DeviceBuffer<float>::from_slice(cat3(std::vector<float>(n_q * hd, 0.f), k, v));
    DeviceCursor cursor(static_cast<int32_t>(p));
    decode::rope_cache(qd, cache, table, n_q, cursor);
    std::vector<float> kr(k);
    for (size_t j = 0; j < half; ++j) {
      const double inv = std::pow(theta, -static_cast<double>(j) / half);
      const double s = std::sin(p * inv), c = std::cos(p * inv);
      kr[j] = static_cast<float>(k[j] * c - k[j + half] * s);
      kr[j + half] = static_cast<float>(k[j + half] * c + k[j] * s);
    }
    ks.push_back(kr);
    vs.push_back(v);
  }
  std::vector<float> q(n_q * hd);
  for (size_t i = 0; i < q.size(); ++i) q[i] = static_cast<float>(i % 5) / 2.f - 1.f;
  auto qd = DeviceBuffer<float>::from_slice(q);
  auto out = DeviceBuffer<uint16_t>::zeros(n_q * hd);
  DeviceCursor at(1);
  decode::attn_decode(qd, cache, out, n_q, at);
  auto got = from_f16(out.to_vec());
  const double scale = 1.0 / std::sqrt(static_cast<double>(hd));
  for (size_t h = 0; h < n_q; ++h) {
    double s[2];
    for (size_t p = 0; p < 2; ++p) {
      s[p] = 0;
      for (size_t d = 0; d < hd; ++d)
        s[p] += static_cast<double>(q[h * hd + d]) * f16_to_f32(f32_to_f16(ks[p][d]));
      s[p] *= scale;
    }
    const double m = std::fmax(s[0], s[1]), e0 = std::exp(s[0] - m), e1 = std::exp(s[1] - m);
    for (size_t d = 0; d < hd; ++d) {
      const double want = (e0 * f16_to_f32(f32_to_f16(vs[0][d])) + e1 * f16_to_f32(f32_to_f16(vs[1][d]))) / (e0 + e1);
      REQUIRE(std::fabs(got[h * hd + d] - want) < 3e-3, "two positions");
    }
  }
}

static void close(float got, float want, float tol, const char *what) {
  REQUIRE(std::fabs(got - want) <= tol * std::fmax(std::fabs(want), 1.0f), what);
}

static void rope_and_attention_chunk_match_sequential_decode() {
  const size_t n_q = 14, n_kv = 2, hd = 64, max_seq = 128, n = 9;
  const size_t stride = (n_q + 2 * n_kv) * hd;
  RopeTable rope(max_seq, hd, 1e6);
  const auto all = noise(stride * n, 303);
  KvCache cache_a(n_kv, n_q, hd, max_seq);
  auto qkv_c = DeviceBuffer<float>::from_slice(all);
  chunk::rope_cache(qkv_c, cache_a, rope, n_q, 0, n);
  auto out_c = DeviceBuffer<uint16_t>::zeros(n * n_q * hd);
  chunk::attn(qkv_c, cache_a, out_c, n_q, 0, n);
  auto got = from_f16(out_c.to_vec());
  KvCache cache_b(n_kv, n_q, hd, max_seq);
  DeviceCursor cursor(0);
  for (size_t j = 0; j < n; ++j) {
    cursor.set(static_cast<int32_t>(j));
    auto q1 = DeviceBuffer<float>::from_slice(std::vector<float>(all.begin() + j * stride, all.begin() + (j + 1) * stride));
    decode::rope_cache(q1, cache_b, rope, n_q, cursor);
    auto o1 = DeviceBuffer<uint16_t>::zeros(n_q * hd);
    decode::attn_decode(q1, cache_b, o1, n_q, cursor);
    auto want = from_f16(o1.to_vec());
    for (size_t i = 0; i < n_q * hd; ++i) close(got[j * n_q * hd + i], want[i], 4e-3f, "attention token");
  }
}

static void attention_chunk_resumes_mid_cache() {
  const size_t n_q = 14, n_kv = 2, hd = 64, max_seq = 128, prefix = 20, n = 5;
  const size_t stride = (n_q + 2 * n_kv) * hd;
  RopeTable rope(max_seq, hd, 1e6);
  const auto all = noise(stride * (prefix + n), 404);
  KvCache cache_a(n_kv, n_q, hd, max_seq), cache_b(n_kv, n_q, hd, max_seq);
  DeviceCursor cursor(0);
  auto row = [&](size_t j) { return std::vector<float>(all.begin() + j * stride, all.begin() + (j + 1) * stride); };
  for (size_t j = 0; j < prefix; ++j) {
    cursor.set(static_cast<int32_t>(j));
    for (KvCache *c : {&cache_a, &cache_b}) {
      auto q1 = DeviceBuffer<float>::from_slice(row(j));
      decode::rope_cache(q1, *c, rope, n_q, cursor);
    }
  }
  auto qkv_c = DeviceBuffer<float>::from_slice(std::vector<float>(all.begin() + prefix * stride, all.end()));
  chunk::rope_cache(qkv_c, cache_a, rope, n_q, prefix, n);
  auto out_c = DeviceBuffer<uint16_t>::zeros(n * n_q * hd);
  chunk::attn(qkv_c, cache_a, out_c, n_q, prefix, n);
  auto got = from_f16(out_c.to_vec());
  for (size_t j = 0; j < n; ++j) {
    cursor.set(static_cast<int32_t>(prefix + j));
    auto q1 = DeviceBuffer<float>::from_slice(row(prefix + j));
    decode::rope_cache(q1, cache_b, rope, n_q, cursor);
    auto o1 = DeviceBuffer<uint16_t>::zeros(n_q * hd);
    decode::attn_decode(q1, cache_b, o1, n_q, cursor);
    auto want = from_f16(o1.to_vec());
    for (size_t i = 0; i < n_q * hd; ++i) close(got[j * n_q * hd + i], want[i], 4e-3f, "resumed attention token");
  }
}

/* Not in the engine's tests (it has no batched form): three sequences appended and
 * attended in one launch each must equal the same sequences run one by one. */
static void batched_chunk_matches_one_sequence_at_a_time() {
  const size_t n_seq = 3, n_q = 8, n_kv = 2, hd = 128, max_seq = 96, n = 40;
  const size_t stride = (n_q + 2 * n_kv) * hd;
  const int32_t starts[n_seq] = {0, 17, 50};
  RopeTable rope(max_seq, hd, 1e6);
  const auto prefix = noise(stride * 50, 505);
  const auto all = noise(stride * n * n_seq, 606);
  chunk::KvCacheBatch batch(n_seq, n_kv, hd, max_seq);
  std::vector<std::vector<float>> want(n_seq);
  std::vector<uint16_t> k_host(n_seq * n_kv * max_seq * hd), v_host(k_host.size());
  for (size_t s = 0; s < n_seq; ++s) {
    KvCache one(n_kv, n_q, hd, max_seq);
    if (starts[s] > 0) {
      auto pre = DeviceBuffer<float>::from_slice(std::vector<float>(prefix.begin(), prefix.begin() + starts[s] * stride));
      chunk::rope_cache(pre, one, rope, n_q, 0, starts[s]);
    }
    /* the batch's cache starts from the same prefix rows */
    auto k1 = one.k.to_vec(), v1 = one.v.to_vec();
    std::copy(k1.begin(), k1.end(), k_host.begin() + s * k1.size());
    std::copy(v1.begin(), v1.end(), v_host.begin() + s * v1.size());
    auto q1 = DeviceBuffer<float>::from_slice(std::vector<float>(all.begin() + s * n * stride, all.begin() + (s + 1) * n * stride));
    chunk::rope_cache(q1, one, rope, n_q, starts[s], n);
    auto o1 = DeviceBuffer<uint16_t>::zeros(n * n_q * hd);
    chunk::attn(q1, one, o1, n_q, starts[s], n);
    want[s] = from_f16(o1.to_vec());
  }
  batch.k.copy_from_host(k_host);
  batch.v.copy_from_host(v_host);
  auto pos = DeviceBuffer<int32_t>::from_slice(std::vector<int32_t>(starts, starts + n_seq));
  auto qkv = DeviceBuffer<float>::from_slice(all);
  chunk::rope_cache_batch(qkv, batch, rope, n_q, pos, n);
  auto out = DeviceBuffer<uint16_t>::zeros(n_seq * n * n_q * hd);
  chunk::attn_batch(qkv, batch, out, n_q, pos, n);
  const auto got = from_f16(out.to_vec());
  for (size_t s = 0; s < n_seq; ++s)
    for (size_t i = 0; i < n * n_q * hd; ++i)
      close(got[s * n * n_q * hd + i], want[s][i], 4e-3f, "batched attention element");
}

static void shape_errors_are_typed_and_launch_nothing() {
  KvCache cache(2, 14, 64, 32);
  RopeTable table(32, 64, 1e6);
  auto qkv = DeviceBuffer<float>::zeros(17 * 64);
  DeviceCursor cursor(0);
  bool threw = false;
  try {
    decode::rope_cache(qkv, cache, table, 14, cursor);
  } catch (const Error &e) {
    threw = e.kind() == Error::Kind::Shape && std::string(e.what()).find("should be (14 + 2*2) * 64") != std::string::npos;
  }
  REQUIRE(threw, "wrong qkv length must raise a Shape error");
  threw = false;
  auto ok = DeviceBuffer<float>::zeros(4 * 18 * 64);
  try {
    chunk::rope_cache(ok, cache, table, 14, 30, 4);
  } catch (const Error &e) {
    threw = e.kind() == Error::Kind::Shape;
  }
  REQUIRE(threw, "chunk past the cache must raise a Shape error");
  REQUIRE(wst_attn_decode(nullptr, nullptr, nullptr, nullptr, nullptr, 14, 2, 64, nullptr, 32, 0.125f) == WST_ERR_INVALID_ARG, "null pointers");
}

static void decode_step_replays_as_a_graph() {
  /* src/decode.rs:543-607 / engine.rs:357-393: append + attend + advance captured once */
  const size_t n_q = 14, n_kv = 2, hd = 64, max_seq = 64;
  RopeTable table(max_seq, hd, 1e6);
  KvCache cache(n_kv, n_q, hd, max_seq);
  auto qkv = DeviceBuffer<float>::from_slice(noise((n_q + 2 * n_kv) * hd, 7));
  auto out = DeviceBuffer<uint16_t>::zeros(n_q * hd);
  DeviceCursor cursor(0);
  auto step = [&] {
    decode::rope_cache(qkv, cache, table, n_q, cursor);
    decode::attn_decode(qkv, cache, out, n_q, cursor);
    cursor.advance(max_seq);
  };
  Graph g = Graph::capture(step);   /* one eager step + one captured (not launched) */
  REQUIRE(cursor.get() == 1, "capture must not execute");
  for (int i = 0; i < 5; ++i) g.launch();
  check(wst_stream_sync());
  REQUIRE(cursor.get() == 6, "five replays advance the cursor five times");
  auto o = from_f16(out.to_vec());
  for (float x : o) REQUIRE(std::isfinite(x), "finite output");
}

/* e4m3 (1-4-3, bias 7, no infinities): the value of a byte */
static float e4m3_to_f32(uint8_t b) {
  const int e = (b >> 3) & 15, m = b & 7;
  const float mag = e == 0 ? std::ldexp(static_cast<float>(m) / 8.f, -6)
                           : std::ldexp(1.f + static_cast<float>(m) / 8.f, e - 7);
  return (b & 0x80) ? -mag : mag;
}

/* The 8-bit cache against the fp16 cache holding the same numbers: every e4m3 value times
 * a power-of-two scale is an fp16 number, so both caches describe the same keys and values
 * and the two decode paths must agree to fp16 rounding of the output.  Capacity 600 goes
 * to the row-block kernel, 9000 to the tensor-memory kernel. */
static void fp8_cache_case(size_t max_seq, size_t seq) {
  const size_t n_q = 28, n_kv = 4, hd = 128;
  const float k_scale = 0.25f, v_scale = 0.5f;
  KvCache c16(n_kv, n_q, hd, max_seq);
  KvCacheFp8 c8(n_kv, n_q, hd, max_seq, k_scale, v_scale);
  std::vector<uint8_t> kb(n_kv * max_seq * hd, 0x7F), vb(kb.size(), 0x7F); /* dead rows: NaN bytes */
  std::vector<uint16_t> kh(kb.size(), 0x7E00), vh(kb.size(), 0x7E00);     /* and fp16 NaN */
  uint64_t x = 0x9E3779B97F4A7C15ull;
  auto next = [&x] { x ^= x << 13; x ^= x >> 7; x ^= x << 17; return x; };
  for (size_t h = 0; h < n_kv; ++h)
    for (size_t p = 0; p < seq; ++p)
      for (size_t d = 0; d < hd; ++d) {
        const size_t at = (h * max_seq + p) * hd + d;
        const uint64_t r = next();
        /* sign, exponent field 0..8 (magnitudes below 4), mantissa */
        kb[at] = static_cast<uint8_t>(((r & 1) << 7) | (((r >> 1) % 9) << 3) | ((r >> 8) & 7));
        vb[at] = static_cast<uint8_t>((((r >> 16) & 1) << 7) | (((r >> 17) % 9) << 3) | ((r >> 24) & 7));
        kh[at] = f32_to_f16(e4m3_to_f32(kb[at]) * k_scale);
        vh[at] = f32_to_f16(e4m3_to_f32(vb[at]) * v_scale);
      }
  c8.k = DeviceBuffer<uint8_t>::from_slice(kb);
  c8.v = DeviceBuffer<uint8_t>::from_slice(vb);
  c16.k = DeviceBuffer<uint16_t>::from_slice(kh);
  c16.v = DeviceBuffer<uint16_t>::from_slice(vh);
  auto qd = DeviceBuffer<float>::from_slice(noise((n_q + 2 * n_kv) * hd, 91));
  auto o8 = DeviceBuffer<uint16_t>::zeros(n_q * hd), o16 = DeviceBuffer<uint16_t>::zeros(n_q * hd);
  DeviceCursor cursor(static_cast<int32_t>(seq - 1));
  decode::attn_decode(qd, c16, o16, n_q, cursor);
  decode::attn_decode_fp8(qd, c8, o8, n_q, cursor);
  auto a = from_f16(o8.to_vec()), b = from_f16(o16.to_vec());
  for (size_t i = 0; i < a.size(); ++i) {
    REQUIRE(std::isfinite(a[i]) && std::isfinite(b[i]), "finite output");
    REQUIRE(std::fabs(a[i] - b[i]) <= 2e-3f, "the two caches hold the same numbers");
  }
}
static void fp8_cache_decodes_like_the_fp16_cache_holding_the_same_numbers() {
  fp8_cache_case(600, 600);
  fp8_cache_case(600, 77);
  fp8_cache_case(9000, 9000);
  fp8_cache_case(9000, 1031);
}

/* chunk_kernels.rs:51-108.  The engine pins its chunk GEMM against its own GEMV; the
 * GEMV is not part of this library, so the yardstick here is the same sum in double on
 * the host, with the engine's tolerance. */
static void gemm_case(size_t in_f, size_t out_f, size_t n, bool with_bias, bool accumulate,
                      uint64_t sw, uint64_t sx, uint64_t sb) {
  auto w = f16v(noise(in_f * out_f, sw)), x = f16v(noise(in_f * n, sx));
  auto bias = f16v(noise(out_f, sb));
  auto seed_y = noise(n * out_f, 66);
  auto wd = DeviceBuffer<uint16_t>::from_slice(w), xd = DeviceBuffer<uint16_t>::from_slice(x);
  auto bd = DeviceBuffer<uint16_t>::from_slice(bias);
  auto yd = accumulate ? DeviceBuffer<float>::from_slice(seed_y) : DeviceBuffer<float>::zeros(n * out_f);
  chunk::gemm_fp16(wd, xd, with_bias ? &bd : nullptr, yd, in_f, out_f, n, accumulate);
  auto got = yd.to_vec();
  auto wf = from_f16(w), xf = from_f16(x), bf = from_f16(bias);
  for (size_t j = 0; j < n; ++j)
    for (size_t r = 0; r < out_f; ++r) {
      double want = accumulate ? seed_y[j * out_f + r] : 0.0;
      for (size_t c = 0; c < in_f; ++c) want += static_cast<double>(xf[j * in_f + c]) * wf[r * in_f + c];
      if (with_bias) want += bf[r];
      const double scale = std::fmax(std::fabs(want), 1.0);
      REQUIRE(std::fabs(got[j * out_f + r] - want) <= 2e-3 * scale, "gemm_fp16 output");
    }
}
static void gemm_fp16_matches_the_sum_per_token() { gemm_case(896, 320, 7, true, false, 11, 22, 33); }
static void gemm_fp16_accumulates_the_same_way() { gemm_case(256, 96, 5, false, true, 44, 55, 0); }
static void gemm_fp16_takes_a_whole_chunk_in_one_pass() {
  REQUIRE(chunk::max_tokens() >= 512, "one pass covers a 512-token chunk");
  gemm_case(512, 384, 300, true, false, 7, 8, 9);
}

int main() {
  int32_t devices = 0;
  if (wst_device_count(&devices) != WST_OK || devices == 0) {
    std::printf("skip: no CUDA device\n");
    return 0;
  }
  struct Case { const char *name; std::function<void()> fn; };
  const Case cases[] = {
      {"rope_uses_the_half_rotation_layout", rope_uses_the_half_rotation_layout},
      {"qk_norm_is_per_head_and_precedes_the_rotation", qk_norm_is_per_head_and_precedes_the_rotation},
      {"qk_norm_with_unit_gain_on_a_unit_rms_head_is_the_identity", qk_norm_with_unit_gain_on_a_unit_rms_head_is_the_identity},
      {"attention_over_one_position_returns_that_value", attention_over_one_position_returns_that_value},
      {"attention_over_two_positions_matches_an_explicit_softmax", attention_over_two_positions_matches_an_explicit_softmax},
      {"rope_and_attention_chunk_match_sequential_decode", rope_and_attention_chunk_match_sequential_decode},
      {"attention_chunk_resumes_mid_cache", attention_chunk_resumes_mid_cache},
      {"batched_chunk_matches_one_sequence_at_a_time", batched_chunk_matches_one_sequence_at_a_time},
      {"gemm_fp16_matches_the_sum_per_token", gemm_fp16_matches_the_sum_per_token},
      {"gemm_fp16_accumulates_the_same_way", gemm_fp16_accumulates_the_same_way},
      {"gemm_fp16_takes_a_whole_chunk_in_one_pass", gemm_fp16_takes_a_whole_chunk_in_one_pass},
      {"fp8_cache_decodes_like_the_fp16_cache_holding_the_same_numbers",
       fp8_cache_decodes_like_the_fp16_cache_holding_the_same_numbers},
      {"shape_errors_are_typed_and_launch_nothing", shape_errors_are_typed_and_launch_nothing},
      {"decode_step_replays_as_a_graph", decode_step_replays_as_a_graph},
  };
  int failed = 0;
  for (const auto &c : cases) {
    try {
      c.fn();
      std::printf("ok   %s\n", c.name);
    } catch (const Failure &f) {
      std::printf("FAIL %s: %s\n", c.name, f.what.c_str());
      ++failed;
    } catch (const std::exception &e) {
      std::printf("FAIL %s: exception %s\n", c.name, e.what());
      ++failed;
    }
  }
  uint32_t code = 0;
  if (wst_b200_device_error(&code) != WST_OK || code != 0) {
    std::printf("FAIL device watchdog word = 0x%x\n", code);
    ++failed;
  }
  std::printf("%d failed\n", failed);
  return failed ? 1 : 0;
}
