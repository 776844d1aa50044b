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

// ---- FP8 rows (blocks of 32: 32 codes + f16 scale; GGUF types 43 = E4M3, 44 = E5M2) -----------------------------
// The reference's FP8 tiers decode through a 256-entry table (crates/oxibonsai-kernels/src/fp8_lut.rs, simd_fp8_avx2.rs,
// simd_fp8_avx512.rs); here the table feeds vector gathers: eight (AVX2) or sixteen (AVX-512) codes become floats with
// one gather and meet the activations in one fused multiply-add.
alignas(64) float g_fp8_lut[2][256];
std::atomic<bool> g_fp8_lut_ready{false};
void init_fp8_lut() {
  if (g_fp8_lut_ready.load(std::memory_order_acquire)) return;
  for (int q = 0; q < 256; ++q) {
    g_fp8_lut[0][q] = fp8_e4m3_decode((uint8_t)q);
    g_fp8_lut[1][q] = fp8_e5m2_decode((uint8_t)q);
    // NaN codes contribute nothing to a dot product here (the scalar body skips them the same way)
    if (g_fp8_lut[0][q] != g_fp8_lut[0][q]) g_fp8_lut[0][q] = 0.0f;
    if (g_fp8_lut[1][q] != g_fp8_lut[1][q] || std::isinf(g_fp8_lut[1][q])) g_fp8_lut[1][q] = 0.0f;
  }
  g_fp8_lut_ready.store(true, std::memory_order_release);
}
template <int FMT>
float dot_fp8_ref(const uint8_t* row, uint64_t nblk32, const float* x) {
  const float* lut = g_fp8_lut[FMT];
  float sum = 0.0f;
  for (uint64_t b = 0; b < nblk32; ++b, row += kFp8Bytes, x += 32) {
    float bs = 0.0f;
    for (int i = 0; i < 32; ++i) bs += lut[row[i]] * x[i];
    sum += f16_to_f32(ld_u16(row + 32)) * bs;
  }
  return sum;
}
template <int FMT>
__attribute__((target("avx2,fma"))) float dot_fp8_avx2(const uint8_t* row, uint64_t nblk32, const float* x) {
  const float* lut = g_fp8_lut[FMT];
  __m256 acc = _mm256_setzero_ps();
  for (uint64_t b = 0; b < nblk32; ++b, row += kFp8Bytes, x += 32) {
    __m256 bs = _mm256_setzero_ps();
    for (int i = 0; i < 32; i += 8) {
      const __m256i idx = _mm256_cvtepu8_epi32(_mm_loadl_epi64(reinterpret_cast<const __m128i*>(row + i)));
      bs = _mm256_fmadd_ps(_mm256_i32gather_ps(lut, idx, 4), _mm256_loadu_ps(x + i), bs);
    }
    acc = _mm256_fmadd_ps(_mm256_set1_ps(f16_to_f32(ld_u16(row + 32))), bs, acc);
  }
  return hsum256(acc);
}
template <int FMT>
__attribute__((target("avx512f,avx512bw,avx512vl"))) float dot_fp8_avx512(const uint8_t* row, uint64_t nblk32, const float* x) {
  const float* lut = g_fp8_lut[FMT];
  __m512 acc = _mm512_setzero_ps();
  for (uint64_t b = 0; b < nblk32; ++b, row += kFp8Bytes, x += 32) {
    __m512 bs = _mm512_setzero_ps();
    for (int i = 0; i < 32; i += 16) {
      const __m512i idx = _mm512_cvtepu8_epi32(_mm_loadu_si128(reinterpret_cast<const __m128i*>(row + i)));
      bs = _mm512_fmadd_ps(_mm512_i32gather_ps(idx, lut, 4), _mm512_loadu_ps(x + i), bs);
    }
    acc = _mm512_fmadd_ps(_mm512_set1_ps(f16_to_f32(ld_u16(row + 32))), bs, acc);
  }
  return _mm512_reduce_add_ps(acc);
}

using RowDot = float (*)(const uint8_t*, uint64_t, const float*);
RowDot pick(uint32_t type, int tier) {
  if (type == 42) return tier >= kAvx512 ? dot_tq2_avx512 : (tier >= kAvx2 ? dot_tq2_avx2 : dot_tq2_ref);
  if (type == 41) return tier >= kAvx512 ? dot_q1_avx512 : (tier >= kAvx2 ? dot_q1_avx2 : dot_q1_ref);
  if (type == 43 || type == 44) {
    init_fp8_lut();
    if (type == 43) return tier >= kAvx512 ? dot_fp8_avx512<0> : (tier >= kAvx2 ? dot_fp8_avx2<0> : dot_fp8_ref<0>);
    return tier >= kAvx512 ? dot_fp8_avx512<1> : (tier >= kAvx2 ? dot_fp8_avx2<1> : dot_fp8_ref<1>);
  }
  return nullptr;
}
// elements and bytes of one block of a row format the tiers know
bool row_format(uint32_t type, uint64_t* elems, uint64_t* bytes) {
  switch (type) {
    case 41: *elems = kQ1Block; *bytes = kQ1Bytes; return true;
    case 42: *elems = kTq2Block; *bytes = kTq2Bytes; return true;
    case 43: case 44: *elems = kFp8Block; *bytes = kFp8Bytes; return true;
    default: return false;
  }
}
void dequant_row(uint32_t type, const uint8_t* src, uint64_t nblk, float* dst) {
  if (type == 42) dequant_tq2(src, nblk, dst);
  else if (type == 41) dequant_q1(src, nblk, dst);
  else dequant_fp8(src, nblk, dst, type == 44);
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
  uint64_t be = 0, bb = 0;
  if (!row_format(type, &be, &bb)) return -7;
  if (cols % be != 0) return -12;
  RowDot dot = pick(type, tier < 0 ? active_tier() : std::min(tier, detect_tier()));
  if (dot == nullptr) return -7;
  const uint64_t nblk = cols / be, rb = nblk * bb;
  if (threads <= 0) threads = (int)std::max(1u, std::thread::hardware_concurrency());
  parallel_rows(rows, threads, [=](uint64_t lo, uint64_t hi) {
    for (uint64_t r = lo; r < hi; ++r) {
      if (r + 1 < hi) __builtin_prefetch(data + (r + 1) * rb);
      out[r] = dot(data + r * rb, nblk, x);
    }
  });
  return 0;
}

// out[batch][rows] = X W^T: every weight row is decoded once into f32 and reused for all batch rows
// (the batch GEMM of the prefill path on CPU).
int bcpu_gemm_tiered(uint32_t type, const uint8_t* data, uint64_t rows, uint64_t cols, const float* x, uint64_t batch, float* out, int threads) {
  using namespace bonsai;
  uint64_t be = 0, bb = 0;
  if (!row_format(type, &be, &bb)) return -7;
  if (cols % be != 0) return -12;
  const uint64_t nblk = cols / be, rb = nblk * bb;
  if (threads <= 0) threads = (int)std::max(1u, std::thread::hardware_concurrency());
  const VecDot vdot = pick_f32(active_tier());
  parallel_rows(rows, threads, [=](uint64_t lo, uint64_t hi) {
    std::vector<float> w(cols);
    for (uint64_t r = lo; r < hi; ++r) {
      dequant_row(type, data + r * rb, nblk, w.data());
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

// ---- vectorised float ops (reference: rope_apply_simd / swiglu_simd / silu_simd / softmax_simd,
// crates/oxibonsai-kernels/src/simd_float_ops.rs:27-180).  tier 0 = the scalar bodies above; tier >= 1 = AVX2 + FMA where
// the CPU has it.  The rotation is mul / sub / add only and equals the scalar result bit for bit; the ops that need exp() use
// a degree-5 polynomial after range reduction (relative error below 2e-7), so they agree with the scalar bodies to
// rounding, not bitwise.
__attribute__((target("avx2,fma"))) static inline __m256 exp256(__m256 x) {
  x = _mm256_min_ps(_mm256_max_ps(x, _mm256_set1_ps(-87.33654f)), _mm256_set1_ps(88.72283f));
  __m256 fx = _mm256_floor_ps(_mm256_fmadd_ps(x, _mm256_set1_ps(1.44269504088896341f), _mm256_set1_ps(0.5f)));
  x = _mm256_fnmadd_ps(fx, _mm256_set1_ps(0.693359375f), x);
  x = _mm256_fnmadd_ps(fx, _mm256_set1_ps(-2.12194440e-4f), x);
  __m256 y = _mm256_set1_ps(1.9875691500e-4f);
  y = _mm256_fmadd_ps(y, x, _mm256_set1_ps(1.3981999507e-3f));
  y = _mm256_fmadd_ps(y, x, _mm256_set1_ps(8.3334519073e-3f));
  y = _mm256_fmadd_ps(y, x, _mm256_set1_ps(4.1665795894e-2f));
  y = _mm256_fmadd_ps(y, x, _mm256_set1_ps(1.6666665459e-1f));
  y = _mm256_fmadd_ps(y, x, _mm256_set1_ps(5.0000001201e-1f));
  y = _mm256_fmadd_ps(y, _mm256_mul_ps(x, x), _mm256_add_ps(x, _mm256_set1_ps(1.0f)));
  const __m256i e = _mm256_slli_epi32(_mm256_add_epi32(_mm256_cvtps_epi32(fx), _mm256_set1_epi32(127)), 23);
  return _mm256_mul_ps(y, _mm256_castsi256_ps(e));
}

__attribute__((target("avx2,fma"))) static void silu_avx2(const float* x, const float* up, float* out, uint64_t n) {
  uint64_t i = 0;
  const __m256 one = _mm256_set1_ps(1.0f);
  for (; i + 8 <= n; i += 8) {
    const __m256 v = _mm256_loadu_ps(x + i);
    __m256 r = _mm256_div_ps(v, _mm256_add_ps(one, exp256(_mm256_sub_ps(_mm256_setzero_ps(), v))));
    if (up) r = _mm256_mul_ps(r, _mm256_loadu_ps(up + i));
    _mm256_storeu_ps(out + i, r);
  }
  for (; i < n; ++i) out[i] = x[i] / (1.0f + std::exp(-x[i])) * (up ? up[i] : 1.0f);
}

__attribute__((target("avx2,fma"))) static void softmax_avx2(const float* x, float* out, uint64_t n) {
  __m256 vm = _mm256_set1_ps(-INFINITY);
  uint64_t i = 0;
  for (; i + 8 <= n; i += 8) vm = _mm256_max_ps(vm, _mm256_loadu_ps(x + i));
  float lanes[8];
  _mm256_storeu_ps(lanes, vm);
  float m = -INFINITY;
  for (float l : lanes) m = std::max(m, l);
  for (; i < n; ++i) m = std::max(m, x[i]);
  const __m256 mm = _mm256_set1_ps(m);
  __m256 acc = _mm256_setzero_ps();
  for (i = 0; i + 8 <= n; i += 8) {
    const __m256 e = exp256(_mm256_sub_ps(_mm256_loadu_ps(x + i), mm));
    _mm256_storeu_ps(out + i, e);
    acc = _mm256_add_ps(acc, e);
  }
  float s = bonsai::hsum256(acc);
  for (; i < n; ++i) {
    out[i] = std::exp(x[i] - m);
    s += out[i];
  }
  const __m256 inv = _mm256_set1_ps(1.0f / s);
  for (i = 0; i + 8 <= n; i += 8) _mm256_storeu_ps(out + i, _mm256_mul_ps(_mm256_loadu_ps(out + i), inv));
  for (; i < n; ++i) out[i] *= 1.0f / s;
}

__attribute__((target("avx2"))) static void rope_avx2(float* x, uint64_t heads, uint64_t head_dim, const float* cos, const float* sin) {
  const uint64_t h = head_dim / 2;
  for (uint64_t hd = 0; hd < heads; ++hd) {
    float* v = x + hd * head_dim;
    uint64_t i = 0;
    for (; i + 8 <= h; i += 8) {
      const __m256 a = _mm256_loadu_ps(v + i), b = _mm256_loadu_ps(v + h + i), c = _mm256_loadu_ps(cos + i), s = _mm256_loadu_ps(sin + i);
      _mm256_storeu_ps(v + i, _mm256_sub_ps(_mm256_mul_ps(a, c), _mm256_mul_ps(b, s)));        // no fused multiply-add: same
      _mm256_storeu_ps(v + h + i, _mm256_add_ps(_mm256_mul_ps(a, s), _mm256_mul_ps(b, c)));    // roundings as the scalar body
    }
    for (; i < h; ++i) {
      const float a = v[i], b = v[h + i];
      v[i] = a * cos[i] - b * sin[i];
      v[h + i] = a * sin[i] + b * cos[i];
    }
  }
}

void bcpu_silu_t(const float* x, float* out, uint64_t n, int tier) {
  if (std::min(tier, bonsai::detect_tier()) >= 1) silu_avx2(x, nullptr, out, n);
  else bcpu_silu(x, out, n);
}
void bcpu_swiglu_t(const float* gate, const float* up, float* out, uint64_t n, int tier) {
  if (std::min(tier, bonsai::detect_tier()) >= 1) silu_avx2(gate, up, out, n);
  else bcpu_swiglu_tiered(gate, up, out, n);
}
void bcpu_softmax_t(const float* x, float* out, uint64_t n, int tier) {
  if (n > 0 && std::min(tier, bonsai::detect_tier()) >= 1) softmax_avx2(x, out, n);
  else bcpu_softmax(x, out, n);
}
void bcpu_rope_apply_t(float* x, uint64_t heads, uint64_t head_dim, const float* cos, const float* sin, int tier) {
  if (std::min(tier, bonsai::detect_tier()) >= 1) rope_avx2(x, heads, head_dim, cos, sin);
  else bcpu_rope_apply(x, heads, head_dim, cos, sin);
}

// 64-byte aligned host buffers (for SIMD loads and for pinned-memory staging).
void* bcpu_aligned_alloc(uint64_t bytes) {
  void* p = nullptr;
  return posix_memalign(&p, 64, ((bytes + 63) / 64) * 64) == 0 ? p : nullptr;
}
void bcpu_aligned_free(void* p) { std::free(p); }

// ---- cache-aware tiling, adaptive strategy, block packing, prefetch (reference: tiled.rs, parallel_tiled.rs, packing.rs,
// prefetch.rs of crates/oxibonsai-kernels) -------------------------------------------------------------------------------------

// Bytes a GEMV over `rows` rows touches: packed weights + input + output.
uint64_t bcpu_working_set_bytes(uint32_t type, uint64_t rows, uint64_t cols) {
  uint64_t be = 0, bb = 0;
  if (!bonsai::row_format(type, &be, &bb) || cols % be != 0) return 0;
  return rows * (cols / be) * bb + cols * 4 + rows * 4;
}
// Rows per tile so that a tile's weights and the input vector stay in `cache_bytes` (0 = 32 KB, an L1 data cache), clamped
// to [4, 256].
uint64_t bcpu_optimal_tile_rows(uint32_t type, uint64_t cols, uint64_t cache_bytes) {
  uint64_t be = 0, bb = 0;
  if (!bonsai::row_format(type, &be, &bb) || cols % be != 0 || cols == 0) return 0;
  if (cache_bytes == 0) cache_bytes = 32 * 1024;
  const uint64_t row_bytes = (cols / be) * bb, input = cols * 4;
  const uint64_t room = cache_bytes > input ? cache_bytes - input : 0;
  return std::min<uint64_t>(256, std::max<uint64_t>(4, room / row_bytes));
}
// 0 = direct (one thread, no tiling), 1 = parallel rows, 2 = parallel tiles.
int bcpu_select_strategy(uint64_t rows, uint64_t cols, uint64_t batch) {
  (void)cols;
  if (rows * std::max<uint64_t>(1, batch) <= 32) return 0;
  if (rows <= 256 && batch <= 1) return 1;
  return 2;
}
// Prefetch hints over a byte range, one per cache line.  locality 0 (streamed once) .. 3 (keep in all levels).
void bcpu_prefetch_range(const void* ptr, uint64_t bytes, int locality, int write) {
  const char* p = static_cast<const char*>(ptr);
  for (uint64_t off = 0; off < bytes; off += 64) {
    if (write) {
      switch (locality) { case 0: __builtin_prefetch(p + off, 1, 0); break; case 1: __builtin_prefetch(p + off, 1, 1); break;
                          case 2: __builtin_prefetch(p + off, 1, 2); break; default: __builtin_prefetch(p + off, 1, 3); }
    } else {
      switch (locality) { case 0: __builtin_prefetch(p + off, 0, 0); break; case 1: __builtin_prefetch(p + off, 0, 1); break;
                          case 2: __builtin_prefetch(p + off, 0, 2); break; default: __builtin_prefetch(p + off, 0, 3); }
    }
  }
}
// Tile-interleaved block order for a GEMV that walks a tile of rows block column by block column: inside every tile of
// `tile` rows the blocks are stored [block 0 of every row, block 1 of every row, ...].  `unpack` is the inverse.
int bcpu_pack_rows_tiled(const uint8_t* src, uint64_t rows, uint64_t blocks_per_row, uint64_t block_bytes, uint64_t tile, uint8_t* dst, int unpack) {
  if (tile == 0 || block_bytes == 0) return -12;
  uint64_t at = 0;   // running block index in the tiled order
  for (uint64_t r0 = 0; r0 < rows; r0 += tile) {
    const uint64_t tr = std::min(tile, rows - r0);
    for (uint64_t b = 0; b < blocks_per_row; ++b)
      for (uint64_t r = 0; r < tr; ++r, ++at) {
        const uint64_t plain = ((r0 + r) * blocks_per_row + b) * block_bytes, tiled = at * block_bytes;
        if (unpack) std::memcpy(dst + plain, src + tiled, block_bytes);
        else std::memcpy(dst + tiled, src + plain, block_bytes);
      }
  }
  return 0;
}

// out[rows] = W x with the rows cut into tiles (tile_rows = 0: bcpu_optimal_tile_rows): threads take tiles from a shared
// counter and ask for the next tile's weights while they work on the current one.
int bcpu_gemv_tiled(uint32_t type, const uint8_t* data, uint64_t rows, uint64_t cols, const float* x, float* out, uint64_t tile_rows, int threads) {
  using namespace bonsai;
  uint64_t be = 0, bb = 0;
  if (!row_format(type, &be, &bb)) return -7;
  if (cols % be != 0) return -12;
  RowDot dot = pick(type, active_tier());
  if (tile_rows == 0) tile_rows = bcpu_optimal_tile_rows(type, cols, 0);
  const uint64_t nblk = cols / be, rb = nblk * bb, ntiles = (rows + tile_rows - 1) / tile_rows;
  if (threads <= 0) threads = (int)std::max(1u, std::thread::hardware_concurrency());
  threads = (int)std::min<uint64_t>(threads, ntiles);
  std::atomic<uint64_t> next{0};
  auto work = [&] {
    for (;;) {
      const uint64_t t = next.fetch_add(1);
      if (t >= ntiles) return;
      const uint64_t lo = t * tile_rows, hi = std::min(rows, lo + tile_rows);
      if (hi < rows) bcpu_prefetch_range(data + hi * rb, std::min<uint64_t>(rb * tile_rows, 4096), 1, 0);
      for (uint64_t r = lo; r < hi; ++r) out[r] = dot(data + r * rb, nblk, x);
    }
  };
  if (threads <= 1) {
    work();
  } else {
    std::vector<std::thread> pool;
    for (int i = 0; i < threads; ++i) pool.emplace_back(work);
    for (auto& th : pool) th.join();
  }
  return 0;
}

// out[batch][rows] = X W^T, tiled both ways: a tile of weight rows is decoded to f32 once (it then sits in L2) and is
// multiplied with the batch in groups of tile_batch rows, so that the decoded tile is reused from cache by every group.
int bcpu_gemm_tiled(uint32_t type, const uint8_t* data, uint64_t rows, uint64_t cols, const float* x, uint64_t batch, float* out,
                    uint64_t tile_rows, uint64_t tile_batch, int threads) {
  using namespace bonsai;
  uint64_t be = 0, bb = 0;
  if (!row_format(type, &be, &bb)) return -7;
  if (cols % be != 0) return -12;
  if (tile_rows == 0) tile_rows = std::max<uint64_t>(4, std::min<uint64_t>(64, (256 * 1024) / (cols * 4)));   // decoded tile within ~256 KB
  if (tile_batch == 0) tile_batch = 8;
  const uint64_t nblk = cols / be, rb = nblk * bb, ntiles = (rows + tile_rows - 1) / tile_rows;
  if (threads <= 0) threads = (int)std::max(1u, std::thread::hardware_concurrency());
  threads = (int)std::min<uint64_t>(threads, ntiles);
  const VecDot vdot = pick_f32(active_tier());
  std::atomic<uint64_t> next{0};
  auto work = [&] {
    std::vector<float> w(tile_rows * cols);
    for (;;) {
      const uint64_t t = next.fetch_add(1);
      if (t >= ntiles) return;
      const uint64_t lo = t * tile_rows, hi = std::min(rows, lo + tile_rows);
      for (uint64_t r = lo; r < hi; ++r) dequant_row(type, data + r * rb, nblk, w.data() + (r - lo) * cols);
      for (uint64_t b0 = 0; b0 < batch; b0 += tile_batch) {
        const uint64_t b1 = std::min(batch, b0 + tile_batch);
        for (uint64_t r = lo; r < hi; ++r)
          for (uint64_t b = b0; b < b1; ++b) out[b * rows + r] = vdot(w.data() + (r - lo) * cols, x + b * cols, cols);
      }
    }
  };
  if (threads <= 1) {
    work();
  } else {
    std::vector<std::thread> pool;
    for (int i = 0; i < threads; ++i) pool.emplace_back(work);
    for (auto& th : pool) th.join();
  }
  return 0;
}

// Picks direct / parallel-row / parallel-tiled by problem size (bcpu_select_strategy) and runs it; returns the strategy
// (>= 0) or a negative error.
int bcpu_gemv_adaptive(uint32_t type, const uint8_t* data, uint64_t rows, uint64_t cols, const float* x, float* out) {
  const int st = bcpu_select_strategy(rows, cols, 1);
  const int rc = st == 0 ? bcpu_gemv_tiered(type, data, rows, cols, x, out, -1, 1)
               : st == 1 ? bcpu_gemv_tiered(type, data, rows, cols, x, out, -1, 0)
                         : bcpu_gemv_tiled(type, data, rows, cols, x, out, 0, 0);
  return rc < 0 ? rc : st;
}
int bcpu_gemm_adaptive(uint32_t type, const uint8_t* data, uint64_t rows, uint64_t cols, const float* x, uint64_t batch, float* out) {
  const int st = bcpu_select_strategy(rows, cols, batch);
  const int rc = st == 0 ? bcpu_gemm_tiered(type, data, rows, cols, x, batch, out, 1)
               : st == 1 ? bcpu_gemm_tiered(type, data, rows, cols, x, batch, out, 0)
                         : bcpu_gemm_tiled(type, data, rows, cols, x, batch, out, 0, 0, 0);
  return rc < 0 ? rc : st;
}

}  // extern "C"
