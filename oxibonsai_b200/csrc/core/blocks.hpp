// Block codecs for the GGUF weight formats the engine loads.
//
//   Q1_0_g128   18 B  [d f16][qs 16 B]   weight j = +d if bit (qs[j/8] >> (j%8)) & 1 else -d
//   TQ2_0_g128  34 B  [qs 32 B][d f16]   weight j = d * map((qs[j/4] >> 2(j%4)) & 3),
//                                         map = {0:-1, 1:0, 2:+1, 3:0}
//   TQ2_0       66 B  [qs 64 B][d f16]   same code map over 256 weights
//   Q4_0        18 B  [d f16][qs 16 B]   weight j = d * (nibble(j) - 8); even j = low nibble of qs[j/2]
//   Q8_0        34 B  [d f16][qs 32 i8]  weight j = d * qs[j]
//   F8_E4M3/E5M2 34 B [qs 32 B][d f16]   weight j = d * fp8_decode(qs[j]); E4M3 is the FN variant
// (reference: crates/oxibonsai-core/src/tensor.rs:11-75, quant_ternary.rs:58-200,207-320,
//  quant_std.rs:23-53,61-135,210-290, quant_fp8.rs:19-28,351-440)
//
// Quantisers follow the loader's polarity (bit set = +d), not the reference's export helper
// that encodes the opposite sign.
#pragma once
#include <cmath>
#include <cstdint>
#include <cstring>

namespace bonsai {

// ---- IEEE half / bfloat16 conversions (bit exact, round to nearest even) ---------------------
inline float f16_to_f32(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1Fu;
  uint32_t man = h & 0x3FFu;
  uint32_t bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else {
      int e = -1;
      do { man <<= 1; ++e; } while (!(man & 0x400u));
      man &= 0x3FFu;
      bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
    }
  } else if (exp == 31) {
    bits = sign | 0x7F800000u | (man << 13);
  } else {
    bits = sign | ((exp + 112u) << 23) | (man << 13);
  }
  float f;
  std::memcpy(&f, &bits, 4);
  return f;
}

inline uint16_t f32_to_f16(float f) {
  uint32_t x;
  std::memcpy(&x, &f, 4);
  uint32_t sign = (x >> 16) & 0x8000u;
  uint32_t absx = x & 0x7FFFFFFFu;
  if (absx >= 0x7F800000u) return (uint16_t)(sign | 0x7C00u | ((absx > 0x7F800000u) ? 0x200u : 0u));
  if (absx >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u);  // rounds to inf
  if (absx < 0x33000001u) return (uint16_t)sign;               // rounds to zero
  int32_t exp = (int32_t)(absx >> 23) - 127;
  uint32_t man = (absx & 0x7FFFFFu) | 0x800000u;
  int shift;
  uint32_t base;
  if (exp < -14) {  // subnormal half
    shift = 13 + (-14 - exp);
    base = 0;
  } else {
    shift = 13;
    base = (uint32_t)(exp + 15) << 10;
    man &= 0x7FFFFFu;
  }
  uint32_t q = man >> shift;
  uint32_t rem = man & ((1u << shift) - 1u);
  uint32_t half = 1u << (shift - 1);
  if (rem > half || (rem == half && (q & 1u))) ++q;
  return (uint16_t)(sign | (base + q));
}

inline float bf16_to_f32(uint16_t h) {
  uint32_t bits = (uint32_t)h << 16;
  float f;
  std::memcpy(&f, &bits, 4);
  return f;
}

inline uint16_t f32_to_bf16(float f) {
  uint32_t x;
  std::memcpy(&x, &f, 4);
  if ((x & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((x >> 16) | 0x40u);
  uint32_t lsb = (x >> 16) & 1u;
  x += 0x7FFFu + lsb;
  return (uint16_t)(x >> 16);
}

// ---- FP8 (E4M3FN max 448, E5M2 max 57344) ---------------------------------------------------
inline float fp8_e4m3_decode(uint8_t q) {
  uint32_t s = q >> 7, e = (q >> 3) & 0xF, m = q & 7;
  float v;
  if (e == 0) v = std::ldexp((float)m, -9);
  else if (e == 15 && m == 7) v = NAN;
  else v = std::ldexp((float)(8 + m), (int)e - 10);
  return s ? -v : v;
}

inline float fp8_e5m2_decode(uint8_t q) {
  uint32_t s = q >> 7, e = (q >> 2) & 0x1F, m = q & 3;
  float v;
  if (e == 0) v = std::ldexp((float)m, -16);
  else if (e == 31) v = m ? NAN : INFINITY;
  else v = std::ldexp((float)(4 + m), (int)e - 17);
  return s ? -v : v;
}

// Generic RNE encoder for a sign/exponent/mantissa format with saturation to max finite.
inline uint8_t fp8_encode_generic(float f, int ebits, int mbits, int bias, float max_finite, uint8_t nan_code) {
  if (std::isnan(f)) return nan_code;
  uint8_t sign = std::signbit(f) ? 0x80 : 0;
  float a = std::fabs(f);
  if (a >= max_finite) {
    // largest finite code
    int e;
    float fr = std::frexp(max_finite, &e);  // max = fr * 2^e, fr in [0.5,1)
    int E = e - 1 + bias;
    int M = (int)std::lround((fr * 2.0f - 1.0f) * (1 << mbits));
    return (uint8_t)(sign | (E << mbits) | M);
  }
  if (a == 0.0f) return sign;
  int e;
  std::frexp(a, &e);
  int E = e - 1;  // a = 1.x * 2^E
  int emin = 1 - bias;
  int qexp = (E < emin ? emin : E) - mbits;  // quantum exponent
  float scaled = std::ldexp(a, -qexp);
  float r = std::nearbyint(scaled);  // RNE in default rounding mode
  int q = (int)r;
  if (E < emin) {
    // subnormal (q < 2^mbits) or rounds up into the first normal
    return (uint8_t)(sign | q);
  }
  if (q == (2 << mbits)) {  // mantissa overflow
    q >>= 1;
    ++E;
  }
  int code = ((E + bias) << mbits) | (q - (1 << mbits));
  (void)ebits;
  return (uint8_t)(sign | code);
}

inline uint8_t fp8_e4m3_encode(float f) { return fp8_encode_generic(f, 4, 3, 7, 448.0f, 0x7F); }
inline uint8_t fp8_e5m2_encode(float f) { return fp8_encode_generic(f, 5, 2, 15, 57344.0f, 0x7F); }

// ---- constants ------------------------------------------------------------------------------
constexpr int kQ1Block = 128, kQ1Bytes = 18;
constexpr int kTq2Block = 128, kTq2Bytes = 34;
constexpr int kTq2LBlock = 256, kTq2LBytes = 66;
constexpr int kQ40Block = 32, kQ40Bytes = 18;
constexpr int kQ80Block = 32, kQ80Bytes = 34;
constexpr int kFp8Block = 32, kFp8Bytes = 34;

inline uint16_t ld_u16(const uint8_t* p) {
  uint16_t v;
  std::memcpy(&v, p, 2);
  return v;
}
inline void st_u16(uint8_t* p, uint16_t v) { std::memcpy(p, &v, 2); }

inline int tq2_decode(uint32_t code) { return code == 0 ? -1 : (code == 2 ? 1 : 0); }

// ---- dequantisers: `n_blocks` blocks at `src` -> n_blocks * block floats at `dst` -------------
inline void dequant_q1(const uint8_t* src, size_t n_blocks, float* dst) {
  for (size_t b = 0; b < n_blocks; ++b, src += kQ1Bytes, dst += kQ1Block) {
    float d = f16_to_f32(ld_u16(src));
    const uint8_t* qs = src + 2;
    for (int j = 0; j < kQ1Block; ++j) dst[j] = ((qs[j >> 3] >> (j & 7)) & 1) ? d : -d;
  }
}

inline void dequant_tq2(const uint8_t* src, size_t n_blocks, float* dst) {
  for (size_t b = 0; b < n_blocks; ++b, src += kTq2Bytes, dst += kTq2Block) {
    float d = f16_to_f32(ld_u16(src + 32));
    for (int j = 0; j < kTq2Block; ++j) dst[j] = d * (float)tq2_decode((src[j >> 2] >> (2 * (j & 3))) & 3);
  }
}

inline void dequant_tq2_256(const uint8_t* src, size_t n_blocks, float* dst) {
  for (size_t b = 0; b < n_blocks; ++b, src += kTq2LBytes, dst += kTq2LBlock) {
    float d = f16_to_f32(ld_u16(src + 64));
    for (int j = 0; j < kTq2LBlock; ++j) dst[j] = d * (float)tq2_decode((src[j >> 2] >> (2 * (j & 3))) & 3);
  }
}

inline void dequant_q4_0(const uint8_t* src, size_t n_blocks, float* dst) {
  for (size_t b = 0; b < n_blocks; ++b, src += kQ40Bytes, dst += kQ40Block) {
    float d = f16_to_f32(ld_u16(src));
    const uint8_t* qs = src + 2;
    for (int j = 0; j < kQ40Block; ++j) {
      int nib = (j & 1) ? (qs[j >> 1] >> 4) : (qs[j >> 1] & 0xF);
      dst[j] = d * ((float)nib - 8.0f);
    }
  }
}

inline void dequant_q8_0(const uint8_t* src, size_t n_blocks, float* dst) {
  for (size_t b = 0; b < n_blocks; ++b, src += kQ80Bytes, dst += kQ80Block) {
    float d = f16_to_f32(ld_u16(src));
    const int8_t* qs = reinterpret_cast<const int8_t*>(src + 2);
    for (int j = 0; j < kQ80Block; ++j) dst[j] = d * (float)qs[j];
  }
}

inline void dequant_fp8(const uint8_t* src, size_t n_blocks, float* dst, bool e5m2) {
  for (size_t b = 0; b < n_blocks; ++b, src += kFp8Bytes, dst += kFp8Block) {
    float d = f16_to_f32(ld_u16(src + 32));
    for (int j = 0; j < kFp8Block; ++j) dst[j] = d * (e5m2 ? fp8_e5m2_decode(src[j]) : fp8_e4m3_decode(src[j]));
  }
}

// ---- quantisers -----------------------------------------------------------------------------
inline float absmax_ignoring_nan(const float* x, int n) {
  float m = 0.0f;
  for (int j = 0; j < n; ++j) {
    float a = std::fabs(x[j]);
    if (!std::isnan(a) && a > m) m = a;
  }
  return m;
}

// Scale = mean |w| (the least-squares optimum for sign quantisation) or absmax when asked.
inline void quant_q1(const float* src, size_t n_blocks, uint8_t* dst, bool use_absmax) {
  for (size_t b = 0; b < n_blocks; ++b, src += kQ1Block, dst += kQ1Bytes) {
    float s = 0.0f;
    if (use_absmax) {
      s = absmax_ignoring_nan(src, kQ1Block);
    } else {
      for (int j = 0; j < kQ1Block; ++j) s += std::fabs(src[j]);
      s /= (float)kQ1Block;
    }
    st_u16(dst, f32_to_f16(s));
    std::memset(dst + 2, 0, 16);
    for (int j = 0; j < kQ1Block; ++j)
      if (src[j] >= 0.0f) dst[2 + (j >> 3)] |= (uint8_t)(1u << (j & 7));
  }
}

inline void quant_tq2_any(const float* src, size_t n_blocks, uint8_t* dst, int block, int bytes) {
  int qbytes = block / 4;
  for (size_t b = 0; b < n_blocks; ++b, src += block, dst += bytes) {
    float amax = 0.0f;
    for (int j = 0; j < block; ++j) amax = std::fmax(amax, std::fabs(src[j]));
    if (amax == 0.0f) {
      std::memset(dst, 0x55, qbytes);
      st_u16(dst + qbytes, 0);
      continue;
    }
    std::memset(dst, 0, qbytes);
    float thr = 0.5f * amax;
    for (int j = 0; j < block; ++j) {
      uint8_t code = src[j] >= thr ? 2 : (src[j] <= -thr ? 0 : 1);
      dst[j >> 2] |= (uint8_t)(code << (2 * (j & 3)));
    }
    st_u16(dst + qbytes, f32_to_f16(amax));
  }
}
inline void quant_tq2(const float* s, size_t n, uint8_t* d) { quant_tq2_any(s, n, d, kTq2Block, kTq2Bytes); }
inline void quant_tq2_256(const float* s, size_t n, uint8_t* d) { quant_tq2_any(s, n, d, kTq2LBlock, kTq2LBytes); }

inline void quant_q4_0(const float* src, size_t n_blocks, uint8_t* dst) {
  for (size_t b = 0; b < n_blocks; ++b, src += kQ40Block, dst += kQ40Bytes) {
    float amax = absmax_ignoring_nan(src, kQ40Block);
    if (amax == 0.0f) {
      st_u16(dst, 0);
      std::memset(dst + 2, 0x88, 16);
      continue;
    }
    uint16_t dh = f32_to_f16(amax / 7.0f);
    float d = f16_to_f32(dh);
    float inv = d == 0.0f ? 0.0f : 1.0f / d;
    st_u16(dst, dh);
    std::memset(dst + 2, 0, 16);
    for (int j = 0; j < kQ40Block; ++j) {
      float v = std::isnan(src[j]) ? 0.0f : src[j];
      int q = (int)std::lround(v * inv) + 8;
      q = q < 0 ? 0 : (q > 15 ? 15 : q);
      dst[2 + (j >> 1)] |= (uint8_t)((j & 1) ? (q << 4) : q);
    }
  }
}

inline void quant_q8_0(const float* src, size_t n_blocks, uint8_t* dst) {
  for (size_t b = 0; b < n_blocks; ++b, src += kQ80Block, dst += kQ80Bytes) {
    float amax = absmax_ignoring_nan(src, kQ80Block);
    if (amax == 0.0f) {
      std::memset(dst, 0, kQ80Bytes);
      continue;
    }
    uint16_t dh = f32_to_f16(amax / 127.0f);
    float d = f16_to_f32(dh);
    float inv = d == 0.0f ? 0.0f : 1.0f / d;
    st_u16(dst, dh);
    for (int j = 0; j < kQ80Block; ++j) {
      float v = std::isnan(src[j]) ? 0.0f : src[j];
      int q = (int)std::lround(v * inv);
      q = q < -127 ? -127 : (q > 127 ? 127 : q);
      reinterpret_cast<int8_t*>(dst + 2)[j] = (int8_t)q;
    }
  }
}

inline void quant_fp8(const float* src, size_t n_blocks, uint8_t* dst, bool e5m2) {
  float fmax = e5m2 ? 57344.0f : 448.0f;
  for (size_t b = 0; b < n_blocks; ++b, src += kFp8Block, dst += kFp8Bytes) {
    float amax = absmax_ignoring_nan(src, kFp8Block);
    if (amax == 0.0f) {
      std::memset(dst, 0, kFp8Bytes);
      continue;
    }
    uint16_t dh = f32_to_f16(amax / fmax);
    float d = f16_to_f32(dh);
    for (int j = 0; j < kFp8Block; ++j) {
      float s = d == 0.0f ? 0.0f : src[j] / d;
      dst[j] = e5m2 ? fp8_e5m2_encode(s) : fp8_e4m3_encode(s);
    }
    st_u16(dst + 32, dh);
  }
}

}  // namespace bonsai
