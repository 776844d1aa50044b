// CPU kernel tiers: scalar reference and AVX2 (+FMA) bodies for the packed-weight GEMV / GEMM and the
// float ops, a row-parallel driver, and the tier dispatcher.
//
// Reference: crates/oxibonsai-kernels/src/dispatch.rs:26-201 (KernelTier Reference / Avx2 / Avx512 /
// Neon / Gpu with auto detection), simd_avx2.rs:29-789 (Q1 and TQ2 dequant / GEMV / GEMM),
// simd_float_ops.rs:27-254 (rms_norm, rope, swiglu, silu, softmax with scalar bodies), parallel.rs and
// parallel_tiled.rs (row-parallel GEMV, batch GEMM that decodes a weight block once for all batch
// rows), aligned.rs / prefetch.rs (64-byte aligned buffers, prefetch hints).  The scalar bodies here
// keep the reference's summation order (sequential inside a block, then `sum += d * block_sum`), so
// tier 0 is bit-identical to the oracle in cpu/oracle.cpp; the AVX2 and AVX-512 bodies reorder additions
// and are the timed CPU baseline (the reference's simd_avx512.rs tier: 16-lane masks instead of a decode).  The serving path of this project is the GPU; these kernels exist for the
// CPU fallback, for tests and for the CPU side of benchmarks.
#include <immintrin.h>

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <thread>
#include <vector>

#include "../core/blocks.hpp"

namespace bonsai {
namespace {

enum Tier { kReference = 0, kAvx2 = 1, kAvx512 = 2 };

int detect_tier() {
  __builtin_cpu_init();
  if (__builtin_cpu_supports("avx512f") && __builtin_cpu_supports("avx512bw")) return kAvx512;
  if (__builtin_cpu_supports("avx2") && __builtin_cpu_supports("fma")) return kAvx2;
  return kReference;
}
std::atomic<int> g_tier{-1};
int active_tier() {
  int t = g_tier.load();
  if (t < 0) {
    t = detect_tier();
    g_tier.store(t);
  }
  return t;
}

// ---- scalar bodies -----------------------------------------------------------------------------
float dot_tq2_ref(const uint8_t* row, uint64_t nblk, const float* x) {
  float sum = 0.0f;
  for (uint64_t b = 0; b < nblk; ++b, row += 34, x += 128) {
    float bs = 0.0f;
    for (int i = 0; i < 32; ++i)
      for (int l = 0; l < 4; ++l) bs += (float)tq2_decode((row[i] >> (2 * l)) & 3) * x[4 * i + l];
    sum += f16_to_f32(ld_u16(row + 32)) * bs;
  }
  return sum;
}
float dot_q1_ref(const uint8_t* row, uint64_t nblk, const float* x) {
  float sum = 0.0f;
  for (uint64_t b = 0; b < nblk; ++b, row += 18, x += 128) {
    float bs = 0.0f;
    for (int j = 0; j < 128; ++j) bs += ((row[2 + j / 8] >> (j % 8)) & 1) ? x[j] : -x[j];
    sum += f16_to_f32(ld_u16(row)) * bs;
  }
  return sum;
}

// ---- AVX2 bodies ---------------------------------------------------------------------------------
__attribute__((target("avx2,fma"))) inline float hsum256(__m256 v) {
  __m128 s = _mm_add_ps(_mm256_castps256_ps128(v), _mm256_extractf128_ps(v, 1));
  s = _mm_add_ps(s, _mm_movehl_ps(s, s));
  s = _mm_add_ss(s, _mm_shuffle_ps(s, s, 1));
  return _mm_cvtss_f32(s);
}

alignas(32) int8_t g_tq2_lut[256][4];
std::atomic<bool> g_lut_ready{false};
void init_lut() {
  if (g_lut_ready.load()) return;
  for (int b = 0; b < 256; ++b)
    for (int l = 0; l < 4; ++l) g_tq2_lut[b][l] = (int8_t)tq2_decode((b >> (2 * l)) & 3);
  g_lut_ready.store(true);
}

__attribute__((target("avx2,fma"))) float dot_tq2_avx2(const uint8_t* row, uint64_t nblk, const float* x) {
  init_lut();
  __m256 total = _mm256_setzero_ps();
  for (uint64_t b = 0; b < nblk; ++b, row += 34, x += 128) {
    alignas(32) int8_t w[128];
    for (int i = 0; i < 32; ++i) std::memcpy(w + 4 * i, g_tq2_lut[row[i]], 4);
    __m256 acc = _mm256_setzero_ps();
    for (int i = 0; i < 128; i += 8) {
      const __m256 wf = _mm256_cvtepi32_ps(_mm256_cvtepi8_epi32(_mm_loadl_epi64(reinterpret_cast<const __m128i*>(w + i))));
      acc = _mm256_fmadd_ps(wf, _mm256_loadu_ps(x + i), acc);
    }
    total = _mm256_fmadd_ps(acc, _mm256_set1_ps(f16_to_f32(ld_u16(row + 32))), total);
  }
  return hsum256(total);
}

__attribute__((target("avx2,fma"))) float dot_q1_avx2(const uint8_t* row, uint64_t nblk, const float* x) {
  const __m256i bits = _mm256_setr_epi32(1, 2, 4, 8, 16, 32, 64, 128);
  const __m256 signbit = _mm256_castsi256_ps(_mm256_set1_epi32((int)0x80000000u));
  __m256 total = _mm256_setzero_ps();
  for (uint64_t b = 0; b < nblk; ++b, row += 18, x += 128) {
    __m256 acc = _mm256_setzero_ps();
    for (int i = 0; i < 16; ++i) {
      const __m256i set = _mm256_cmpeq_epi32(_mm256_and_si256(_mm256_set1_epi32(row[2 + i]), bits), bits);
      // bit set -> +x, clear -> -x: flip the sign where the bit is clear
      const __m256 flip = _mm256_andnot_ps(_mm256_castsi256_ps(set), signbit);
      acc = _mm256_add_ps(acc, _mm256_xor_ps(_mm256_loadu_ps(x + 8 * i), flip));
    }
    total = _mm256_fmadd_ps(acc, _mm256_set1_ps(f16_to_f32(ld_u16(row))), total);
  }
  return hsum256(total);
}

// ---- AVX-512 bodies ------------------------------------------------------------------------------
// The weights never become numbers: sixteen 2-bit codes (or sixteen sign bits) turn into two mask registers and the
// activations are added or subtracted under them, sixteen lanes per instruction.
#define BONSAI_AVX512 __attribute__((target("avx512f,avx512bw,avx512vl,avx2,fma")))

BONSAI_AVX512 float dot_tq2_avx512(const uint8_t* row, uint64_t nblk, const float* x) {
  const __m512i shifts = _mm512_setr_epi32(0, 2, 4, 6, 8, 10, 12, 14, 16, 18, 20, 22, 24, 26, 28, 30);
  const __m512i three = _mm512_set1_epi32(3), two = _mm512_set1_epi32(2);
  __m512 total = _mm512_setzero_ps();
  for (uint64_t b = 0; b < nblk; ++b, row += 34, x += 128) {
    __m512 acc0 = _mm512_setzero_ps(), acc1 = _mm512_setzero_ps();
    for (int c = 0; c < 8; c += 2) {
      uint32_t w0, w1;
      std::memcpy(&w0, row + 4 * c, 4);
      std::memcpy(&w1, row + 4 * c + 4, 4);
      const __m512i c0 = _mm512_and_si512(_mm512_srlv_epi32(_mm512_set1_epi32((int)w0), shifts), three);
      const __m512i c1 = _mm512_and_si512(_mm512_srlv_epi32(_mm512_set1_epi32((int)w1), shifts), three);
      const __m512 x0 = _mm512_loadu_ps(x + 16 * c), x1 = _mm512_loadu_ps(x + 16 * c + 16);
      acc0 = _mm512_mask_add_ps(acc0, _mm512_cmpeq_epi32_mask(c0, two), acc0, x0);                    // code 2 = +1
      acc0 = _mm512_mask_sub_ps(acc0, _mm512_cmpeq_epi32_mask(c0, _mm512_setzero_si512()), acc0, x0);  // code 0 = -1
      acc1 = _mm512_mask_add_ps(acc1, _mm512_cmpeq_epi32_mask(c1, two), acc1, x1);
      acc1 = _mm512_mask_sub_ps(acc1, _mm512_cmpeq_epi32_mask(c1, _mm512_setzero_si512()), acc1, x1);
    }
    total = _mm512_fmadd_ps(_mm512_add_ps(acc0, acc1), _mm512_set1_ps(f16_to_f32(ld_u16(row + 32))), total);
  }
  return _mm512_reduce_add_ps(total);
}

BONSAI_AVX512 float dot_q1_avx512(const uint8_t* row, uint64_t nblk, const float* x) {
  __m512 total = _mm512_setzero_ps();
  for (uint64_t b = 0; b < nblk; ++b, row += 18, x += 128) {
    __m512 acc0 = _mm512_setzero_ps(), acc1 = _mm512_setzero_ps();
    for (int c = 0; c < 8; c += 2) {
      const __mmask16 m0 = (__mmask16)ld_u16(row + 2 + 2 * c), m1 = (__mmask16)ld_u16(row + 4 + 2 * c);
      const __m512 x0 = _mm512_loadu_ps(x + 16 * c), x1 = _mm512_loadu_ps(x + 16 * c + 16);
      acc0 = _mm512_mask_add_ps(acc0, m0, acc0, x0);   // bit set = +x
      acc0 = _mm512_mask_sub_ps(acc0, (__mmask16)~m0, acc0, x0);
      acc1 = _mm512_mask_add_ps(acc1, m1, acc1, x1);
      acc1 = _mm512_mask_sub_ps(acc1, (__mmask16)~m1, acc1, x1);
    }
    total = _mm512_fmadd_ps(_mm512_add_ps(acc0, acc1), _mm512_set1_ps(f16_to_f32(ld_u16(row))), total);
  }
  return _mm512_reduce_add_ps(total);
}

BONSAI_AVX512 float dot_f32_avx512(const float* a, const float* b, uint64_t n) {
  __m512 s0 = _mm512_setzero_ps(), s1 = _mm512_setzero_ps();
  uint64_t i = 0;
  for (; i + 32 <= n; i += 32) {
    s0 = _mm512_fmadd_ps(_mm512_loadu_ps(a + i), _mm512_loadu_ps(b + i), s0);
    s1 = _mm512_fmadd_ps(_mm512_loadu_ps(a + i + 16), _mm512_loadu_ps(b + i + 16), s1);
  }
  float s = _mm512_reduce_add_ps(_mm512_add_ps(s0, s1));
  for (; i < n; ++i) s += a[i] * b[i];
  return s;
}

__attribute__((target("avx2,fma"))) float dot_f32_avx2(const float* a, const float* b, uint64_t n) {
  __m256 s0 = _mm256_setzero_ps(), s1 = _mm256_setzero_ps();
  uint64_t i = 0;
  for (; i + 16 <= n; i += 16) {
    s0 = _mm256_fmadd_ps(_mm256_loadu_ps(a + i), _mm256_loadu_ps(b + i), s0);
    s1 = _mm256_fmadd_ps(_mm256_loadu_ps(a + i + 8), _mm256_loadu_ps(b + i + 8), s1);
  }
  float s = hsum256(_mm256_add_ps(s0, s1));
  for (; i < n; ++i) s += a[i] * b[i];
  return s;
}

float dot_f32_ref(const float* a, const float* b, uint64_t n) {
  float s = 0.0f;
  for (uint64_t k = 0; k < n; ++k) s += a[k] * b[k];
  return s;
}

BONSAI_AVX512 float sumsq_avx512(const float* x, uint64_t n) {
  __m512 a = _mm512_setzero_ps();
  uint64_t i = 0;
  for (; i + 16 <= n; i += 16) {
    const __m512 v = _mm512_loadu_ps(x + i);
    a = _mm512_fmadd_ps(v, v, a);
  }
  float s = _mm512_reduce_add_ps(a);
  for (; i < n; ++i) s += x[i] * x[i];
  return s;
}

using RowDot = float (*)(const uint8_t*, uint64_t, const float*);
RowDot pick(uint32_t type, int tier) {
  if (type == 42) return tier >= kAvx512 ? dot_tq2_avx512 : (tier >= kAvx2 ? dot_tq2_avx2 : dot_tq2_ref);
  if (type == 41) return tier >= kAvx512 ? dot_q1_avx512 : (tier >= kAvx2 ? dot_q1_avx2 : dot_q1_ref);
  return nullptr;
}
using VecDot = float (*)(const float*, const float*, uint64_t);
VecDot pick_f32(int tier) { return tier >= kAvx512 ? dot_f32_avx512 : (tier >= kAvx2 ? dot_f32_avx2 : dot_f32_ref); }

template <typename F>
void parallel_rows(uint64_t n, int threads, F f) {
  if (threads <= 1 || n < 64) {
    f(0, n);
    return;
  }
  std::vector<std::thread> pool;
  const uint64_t per = (n + threads - 1) / threads;
  for (int t = 0; t < threads; ++t) {
    const uint64_t lo = t * per, hi = std::min(n, lo + per);
    if (lo < hi) pool.emplace_back([=] { f(lo, hi); });
  }
  for (auto& th : pool) th.join();
}

}  // namespace
}  // namespace bonsai

extern "C" {

// 0 reference, 1 AVX2+FMA, 2 AVX-512 (F + BW + VL).
int bcpu_detect_tier() { return bonsai::detect_tier(); }
int bcpu_active_tier() { return bonsai::active_tier(); }
// Forces a tier not above what the CPU supports; -1 returns to auto detection.  Returns the tier now active.
int bcpu_set_tier(int tier) {
  const int best = bonsai::detect_tier();
  bonsai::g_tier.store(tier < 0 ? best : std::min(tier, best));
  return bonsai::g_tier.load();
}
const char* bcpu_tier_name(int tier) { return tier == 0 ? "reference" : (tier == 1 ? "avx2" : (tier == 2 ? "avx512" : "unknown")); }

// out[rows] = W x for Q1_0_g128 (41) / TQ2_0_g128 (42) rows; tier < 0 uses the active tier; threads <= 0 = all cores.
int bcpu_gemv_tiered(uint32_t type, const uint8_t* data, uint64_t rows, uint64_t cols, const float* x, float* out, int tier, int threads) {
  using namespace bonsai;
  if (cols % 128 != 0) return -12;
  RowDot dot = pick(type, tier < 0 ? active_tier() : std::min(tier, detect_tier()));
  if (dot == nullptr) return -7;
  const uint64_t rb = (cols / 128) * (type == 42 ? 34 : 18);
  if (threads <= 0) threads = (int)std::max(1u, std::thread::hardware_concurrency());
  parallel_rows(rows, threads, [=](uint64_t lo, uint64_t hi) {
    for (uint64_t r = lo; r < hi; ++r) {
      if (r + 1 < hi) __builtin_prefetch(data + (r + 1) * rb);
      out[r] = dot(data + r * rb, cols / 128, x);
    }
  });
  return 0;
}

// out[batch][rows] = X W^T: every weight row is decoded once into f32 and reused for all batch rows
// (the batch GEMM of the prefill path on CPU).
int bcpu_gemm_tiered(uint32_t type, const uint8_t* data, uint64_t rows, uint64_t cols, const float* x, uint64_t batch, float* out, int threads) {
  using namespace bonsai;
  if (cols % 128 != 0) return -12;
  if (type != 41 && type != 42) return -7;
  const uint64_t rb = (cols / 128) * (type == 42 ? 34 : 18);
  if (threads <= 0) threads = (int)std::max(1u, std::thread::hardware_concurrency());
  const VecDot vdot = pick_f32(active_tier());
  parallel_rows(rows, threads, [=](uint64_t lo, uint64_t hi) {
    std::vector<float> w(cols);
    for (uint64_t r = lo; r < hi; ++r) {
      if (type == 42) dequant_tq2(data + r * rb, cols / 128, w.data()); else dequant_q1(data + r * rb, cols / 128, w.data());
      for (uint64_t b = 0; b < batch; ++b) {
        out[b * rows + r] = vdot(w.data(), x + b * cols, cols);
      }
    }
  });
  return 0;
}

// ---- float ops; `tier` 0 = scalar bodies in the oracle's order, >= 1 = vectorised -----------------------------
__attribute__((target("avx2,fma"))) static float sumsq_avx2(const float* x, uint64_t n) {
  __m256 a = _mm256_setzero_ps();
  uint64_t i = 0;
  for (; i + 8 <= n; i += 8) {
    const __m256 v = _mm256_loadu_ps(x + i);
    a = _mm256_fmadd_ps(v, v, a);
  }
  float s = bonsai::hsum256(a);
  for (; i < n; ++i) s += x[i] * x[i];
  return s;
}

void bcpu_rmsnorm_tiered(const float* x, const float* w, float* out, uint64_t n, float eps, int tier) {
  float ss = 0.0f;
  const int have = std::min(tier, bonsai::detect_tier());
  if (have >= 2) ss = bonsai::sumsq_avx512(x, n);
  else if (have >= 1) ss = sumsq_avx2(x, n);
  else for (uint64_t i = 0; i < n; ++i) ss += x[i] * x[i];
  const float inv = 1.0f / std::sqrt(ss / (float)n + eps);
  for (uint64_t i = 0; i < n; ++i) out[i] = w[i] * x[i] * inv;
}

void bcpu_silu(const float* x, float* out, uint64_t n) {
  for (uint64_t i = 0; i < n; ++i) out[i] = x[i] / (1.0f + std::exp(-x[i]));
}

void bcpu_swiglu_tiered(const float* gate, const float* up, float* out, uint64_t n) {
  for (uint64_t i = 0; i < n; ++i) out[i] = gate[i] / (1.0f + std::exp(-gate[i])) * up[i];
}

void bcpu_softmax(const float* x, float* out, uint64_t n) {
  float m = -INFINITY;
  for (uint64_t i = 0; i < n; ++i) m = std::max(m, x[i]);
  float s = 0.0f;
  for (uint64_t i = 0; i < n; ++i) {
    out[i] = std::exp(x[i] - m);
    s += out[i];
  }
  for (uint64_t i = 0; i < n; ++i) out[i] /= s;
}

// Half-split rotation of `heads` vectors of head_dim at one position; cos / sin hold head_dim / 2 entries.
void bcpu_rope_apply(float* x, uint64_t heads, uint64_t head_dim, const float* cos, const float* sin) {
  const uint64_t h = head_dim / 2;
  for (uint64_t hd = 0; hd < heads; ++hd) {
    float* v = x + hd * head_dim;
    for (uint64_t i = 0; i < h; ++i) {
      const float a = v[i], b = v[h + i];
      v[i] = a * cos[i] - b * sin[i];
      v[h + i] = a * sin[i] + b * cos[i];
    }
  }
}

// 64-byte aligned host buffers (for SIMD loads and for pinned-memory staging).
void* bcpu_aligned_alloc(uint64_t bytes) {
  void* p = nullptr;
  return posix_memalign(&p, 64, ((bytes + 63) / 64) * 64) == 0 ? p : nullptr;
}
void bcpu_aligned_free(void* p) { std::free(p); }

}  // extern "C"
