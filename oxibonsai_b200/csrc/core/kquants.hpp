// K-quant super-block codecs (256 weights per block), little endian, in this project's layouts:
//
//   Q2_K  84 B: scales[16] (low nibble scale, high nibble min) | qs[64] (2 bits, LSB first) | d f16 | dmin f16
//               w[i] = d * sc[i/16] * q - dmin * mn[i/16]
//   Q3_K 110 B: hmask[32] (bit 2 of each weight) | qs[64] (low 2 bits) | scales[12] (4-bit nibbles, value - 8) | d f16
//               w[i] = d * (nibble[i/16] - 8) * (q3 - 4)          (nibble scales, not llama.cpp's 6-bit packing)
//   Q4_K 144 B: d f16 | dmin f16 | scales[12] (8 six-bit scales + 8 six-bit mins) | qs[128] (nibbles)
//               w[i] = d * sc[i/32] * q - dmin * mn[i/32]
//   Q5_K 176 B: d | dmin | scales[12] (as Q4_K) | qh[32] (bit 4) | qs[128] (low nibbles)
//   Q6_K 210 B: ql[128] (low nibbles) | qh[64] (high 2 bits) | scales[16] int8 | d f16;  w[i] = d * scales[i/16] * (q6 - 32)
//   Q8_K 292 B: d f32 | qs[256] int8 | bsums[16] int16 (sums of each 16 weights);        w[i] = d * qs[i]
//
// Weight i of a block always sits at bit offset i * bits inside its packed array (byte i*bits/8,
// LSB first).  Reference: crates/oxibonsai-core/src/quant_k.rs:21-33,50-60,270-280,494-504,782-790 and
// quant_k_ext.rs:20-23,112-124,359-369.
#pragma once
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>

#include "blocks.hpp"

namespace bonsai {

constexpr int kQK = 256;

inline void k6_unpack(const uint8_t* s, uint8_t* sc, uint8_t* mn) {
  for (int i = 0; i < 4; ++i) {
    sc[2 * i] = s[i] & 15; sc[2 * i + 1] = s[i] >> 4;
    mn[2 * i] = s[4 + i] & 15; mn[2 * i + 1] = s[4 + i] >> 4;
  }
  for (int i = 0; i < 4; ++i) {
    sc[i] |= ((s[8] >> (2 * i)) & 3) << 4; sc[4 + i] |= ((s[9] >> (2 * i)) & 3) << 4;
    mn[i] |= ((s[10] >> (2 * i)) & 3) << 4; mn[4 + i] |= ((s[11] >> (2 * i)) & 3) << 4;
  }
}
inline void k6_pack(const uint8_t* sc, const uint8_t* mn, uint8_t* s) {
  std::memset(s, 0, 12);
  for (int i = 0; i < 4; ++i) {
    s[i] = (sc[2 * i] & 15) | ((sc[2 * i + 1] & 15) << 4);
    s[4 + i] = (mn[2 * i] & 15) | ((mn[2 * i + 1] & 15) << 4);
    s[8] |= ((sc[i] >> 4) & 3) << (2 * i); s[9] |= ((sc[4 + i] >> 4) & 3) << (2 * i);
    s[10] |= ((mn[i] >> 4) & 3) << (2 * i); s[11] |= ((mn[4 + i] >> 4) & 3) << (2 * i);
  }
}

// ---- dequantise ------------------------------------------------------------------------------
inline void dequant_q2k(const uint8_t* p, size_t nb, float* o) {
  for (size_t b = 0; b < nb; ++b, p += 84, o += kQK) {
    const float d = f16_to_f32(ld_u16(p + 80)), dm = f16_to_f32(ld_u16(p + 82));
    for (int i = 0; i < kQK; ++i) {
      const int q = (p[16 + i / 4] >> ((i % 4) * 2)) & 3;
      o[i] = d * (float)(p[i / 16] & 15) * (float)q - dm * (float)(p[i / 16] >> 4);
    }
  }
}
inline void dequant_q3k(const uint8_t* p, size_t nb, float* o) {
  for (size_t b = 0; b < nb; ++b, p += 110, o += kQK) {
    const float d = f16_to_f32(ld_u16(p + 108));
    for (int i = 0; i < kQK; ++i) {
      const int q = ((p[32 + i / 4] >> ((i % 4) * 2)) & 3) | (((p[i / 8] >> (i % 8)) & 1) << 2);
      const int sub = i / 16, sc = ((p[96 + sub / 2] >> (4 * (sub % 2))) & 15) - 8;
      o[i] = d * (float)sc * (float)(q - 4);
    }
  }
}
inline void dequant_q4k(const uint8_t* p, size_t nb, float* o) {
  for (size_t b = 0; b < nb; ++b, p += 144, o += kQK) {
    const float d = f16_to_f32(ld_u16(p)), dm = f16_to_f32(ld_u16(p + 2));
    uint8_t sc[8], mn[8];
    k6_unpack(p + 4, sc, mn);
    for (int i = 0; i < kQK; ++i) {
      const int q = (p[16 + i / 2] >> ((i % 2) * 4)) & 15;
      o[i] = d * (float)sc[i / 32] * (float)q - dm * (float)mn[i / 32];
    }
  }
}
inline void dequant_q5k(const uint8_t* p, size_t nb, float* o) {
  for (size_t b = 0; b < nb; ++b, p += 176, o += kQK) {
    const float d = f16_to_f32(ld_u16(p)), dm = f16_to_f32(ld_u16(p + 2));
    uint8_t sc[8], mn[8];
    k6_unpack(p + 4, sc, mn);
    for (int i = 0; i < kQK; ++i) {
      const int q = ((p[48 + i / 2] >> ((i % 2) * 4)) & 15) | (((p[16 + i / 8] >> (i % 8)) & 1) << 4);
      o[i] = d * (float)sc[i / 32] * (float)q - dm * (float)mn[i / 32];
    }
  }
}
inline void dequant_q6k(const uint8_t* p, size_t nb, float* o) {
  for (size_t b = 0; b < nb; ++b, p += 210, o += kQK) {
    const float d = f16_to_f32(ld_u16(p + 208));
    for (int i = 0; i < kQK; ++i) {
      const int q = ((p[i / 2] >> ((i % 2) * 4)) & 15) | (((p[128 + i / 4] >> (2 * (i % 4))) & 3) << 4);
      o[i] = d * (float)(int8_t)p[192 + i / 16] * (float)(q - 32);
    }
  }
}
inline void dequant_q8k(const uint8_t* p, size_t nb, float* o) {
  for (size_t b = 0; b < nb; ++b, p += 292, o += kQK) {
    float d;
    std::memcpy(&d, p, 4);
    for (int i = 0; i < kQK; ++i) o[i] = d * (float)(int8_t)p[4 + i];
  }
}

// ---- quantise --------------------------------------------------------------------------------
// Affine sub-blocks (Q2_K / Q4_K / Q5_K): w ~ s_j * q - m_j with s_j, m_j >= 0 quantised against the
// super-block d = max s_j / smax and dmin = max m_j / mmax.
template <int SUB, int QMAX, int SMAX>
inline void affine_plan(const float* x, float& d, float& dm, uint8_t* sc, uint8_t* mn) {
  constexpr int NS = kQK / SUB;
  float s[NS], m[NS], smax = 0.0f, mmax = 0.0f;
  for (int j = 0; j < NS; ++j) {
    float lo = x[j * SUB], hi = lo;
    for (int i = 1; i < SUB; ++i) { lo = std::min(lo, x[j * SUB + i]); hi = std::max(hi, x[j * SUB + i]); }
    lo = std::min(lo, 0.0f);                      // mins are stored unsigned: the offset can only be <= 0
    s[j] = (hi - lo) / (float)QMAX;
    m[j] = -lo;
    smax = std::max(smax, s[j]);
    mmax = std::max(mmax, m[j]);
  }
  d = f16_to_f32(f32_to_f16(smax / (float)SMAX));
  dm = f16_to_f32(f32_to_f16(mmax / (float)SMAX));
  for (int j = 0; j < NS; ++j) {
    sc[j] = d > 0 ? (uint8_t)std::min((float)SMAX, std::nearbyint(s[j] / d)) : 0;
    mn[j] = dm > 0 ? (uint8_t)std::min((float)SMAX, std::nearbyint(m[j] / dm)) : 0;
  }
}
template <int SUB, int QMAX>
inline int affine_code(float v, float d, float dm, uint8_t sc, uint8_t mn) {
  const float s = d * (float)sc;
  if (s <= 0.0f) return 0;
  return (int)std::min((float)QMAX, std::max(0.0f, std::nearbyint((v + dm * (float)mn) / s)));
}

inline void quant_q2k(const float* x, size_t nb, uint8_t* p) {
  for (size_t b = 0; b < nb; ++b, x += kQK, p += 84) {
    std::memset(p, 0, 84);
    float d, dm;
    uint8_t sc[16], mn[16];
    affine_plan<16, 3, 15>(x, d, dm, sc, mn);
    for (int j = 0; j < 16; ++j) p[j] = sc[j] | (mn[j] << 4);
    for (int i = 0; i < kQK; ++i) p[16 + i / 4] |= affine_code<16, 3>(x[i], d, dm, sc[i / 16], mn[i / 16]) << ((i % 4) * 2);
    st_u16(p + 80, f32_to_f16(d));
    st_u16(p + 82, f32_to_f16(dm));
  }
}
inline void quant_q4k(const float* x, size_t nb, uint8_t* p) {
  for (size_t b = 0; b < nb; ++b, x += kQK, p += 144) {
    std::memset(p, 0, 144);
    float d, dm;
    uint8_t sc[8], mn[8];
    affine_plan<32, 15, 63>(x, d, dm, sc, mn);
    st_u16(p, f32_to_f16(d));
    st_u16(p + 2, f32_to_f16(dm));
    k6_pack(sc, mn, p + 4);
    for (int i = 0; i < kQK; ++i) p[16 + i / 2] |= affine_code<32, 15>(x[i], d, dm, sc[i / 32], mn[i / 32]) << ((i % 2) * 4);
  }
}
inline void quant_q5k(const float* x, size_t nb, uint8_t* p) {
  for (size_t b = 0; b < nb; ++b, x += kQK, p += 176) {
    std::memset(p, 0, 176);
    float d, dm;
    uint8_t sc[8], mn[8];
    affine_plan<32, 31, 63>(x, d, dm, sc, mn);
    st_u16(p, f32_to_f16(d));
    st_u16(p + 2, f32_to_f16(dm));
    k6_pack(sc, mn, p + 4);
    for (int i = 0; i < kQK; ++i) {
      const int q = affine_code<32, 31>(x[i], d, dm, sc[i / 32], mn[i / 32]);
      p[48 + i / 2] |= (q & 15) << ((i % 2) * 4);
      p[16 + i / 8] |= (q >> 4) << (i % 8);
    }
  }
}
// Symmetric sub-blocks (Q3_K / Q6_K): w ~ d * s_j * (q - zero) with signed integer sub-block scales.
inline void quant_q3k(const float* x, size_t nb, uint8_t* p) {
  for (size_t b = 0; b < nb; ++b, x += kQK, p += 110) {
    std::memset(p, 0, 110);
    float am[16], amax = 0.0f;
    for (int j = 0; j < 16; ++j) {
      am[j] = absmax_ignoring_nan(x + j * 16, 16);
      amax = std::max(amax, am[j]);
    }
    const float d = f16_to_f32(f32_to_f16(amax / (4.0f * 7.0f)));   // q in [-4, 3], scale nibble in [-8, 7]
    for (int j = 0; j < 16; ++j) {
      int s = d > 0 ? (int)std::min(7.0f, std::max(1.0f, std::ceil(am[j] / (4.0f * d)))) : 1;
      if (am[j] == 0.0f) s = 1;
      p[96 + j / 2] |= (uint8_t)(s + 8) << (4 * (j % 2));
      for (int i = 0; i < 16; ++i) {
        const int idx = j * 16 + i;
        const float step = d * (float)s;
        const int q = step > 0 ? (int)std::min(3.0f, std::max(-4.0f, std::nearbyint(x[idx] / step))) + 4 : 4;
        p[32 + idx / 4] |= (q & 3) << ((idx % 4) * 2);
        p[idx / 8] |= (q >> 2) << (idx % 8);
      }
    }
    st_u16(p + 108, f32_to_f16(d));
  }
}
inline void quant_q6k(const float* x, size_t nb, uint8_t* p) {
  for (size_t b = 0; b < nb; ++b, x += kQK, p += 210) {
    std::memset(p, 0, 210);
    float am[16], amax = 0.0f;
    for (int j = 0; j < 16; ++j) {
      am[j] = absmax_ignoring_nan(x + j * 16, 16);
      amax = std::max(amax, am[j]);
    }
    const float d = f16_to_f32(f32_to_f16(amax / (32.0f * 127.0f)));
    for (int j = 0; j < 16; ++j) {
      int s = d > 0 ? (int)std::min(127.0f, std::max(1.0f, std::ceil(am[j] / (32.0f * d)))) : 1;
      p[192 + j] = (uint8_t)(int8_t)s;
      for (int i = 0; i < 16; ++i) {
        const int idx = j * 16 + i;
        const float step = d * (float)s;
        const int q = step > 0 ? (int)std::min(31.0f, std::max(-32.0f, std::nearbyint(x[idx] / step))) + 32 : 32;
        p[idx / 2] |= (q & 15) << ((idx % 2) * 4);
        p[128 + idx / 4] |= (q >> 4) << (2 * (idx % 4));
      }
    }
    st_u16(p + 208, f32_to_f16(d));
  }
}
inline void quant_q8k(const float* x, size_t nb, uint8_t* p) {
  for (size_t b = 0; b < nb; ++b, x += kQK, p += 292) {
    const float amax = absmax_ignoring_nan(x, kQK);
    const float d = amax / 127.0f;
    std::memcpy(p, &d, 4);
    for (int g = 0; g < 16; ++g) {
      int sum = 0;
      for (int i = 0; i < 16; ++i) {
        const int q = d > 0 ? (int)std::min(127.0f, std::max(-127.0f, std::nearbyint(x[g * 16 + i] / d))) : 0;
        p[4 + g * 16 + i] = (uint8_t)(int8_t)q;
        sum += q;
      }
      const int16_t s16 = (int16_t)sum;
      std::memcpy(p + 260 + 2 * g, &s16, 2);
    }
  }
}

}  // namespace bonsai
