// Decode GEMV straight from GGUF blocks for the formats that have no planar repack: Q4_0, Q8_0,
// FP8 E4M3 / E5M2 blocks, the K-quants Q2_K .. Q8_K, the 256-wide TQ2_0, F16, BF16 and F32 rows.
//
// Replaces the reference's per-format single-GEMV wrappers cuda_gemv_q4_0 / q8_0, cuda_gemv_q{2..8}k
// and cuda_gemv_fp8_* (crates/oxibonsai-kernels/src/gpu_backend/cuda_q_std_kernels.rs:200-,
// cuda_k_quant_kernels.rs:640-, cuda_fp8_kernels.rs:300-) with one kernel templated on the block
// decoder.  One warp owns a row: for 32-element blocks every lane decodes a whole block per step
// (32 blocks = 1024 inputs per warp step), for 256-element super-blocks the 32 lanes share a block,
// eight elements each.  Accumulation is f32, lanes are folded with shuffles, optional fused RMSNorm
// of the input (every warp recomputes the mean square from L1/L2-resident x) and residual add.
// Block layouts are the ones documented in csrc/core/blocks.hpp and csrc/core/kquants.hpp.
#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "common.cuh"

namespace bonsai {

__device__ __forceinline__ float ld_f16(const uint8_t* p) { return __half2float(__ushort_as_half((unsigned short)(p[0] | (p[1] << 8)))); }
__device__ __forceinline__ float fp8_to_f32(uint8_t q, bool e5m2) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)q, e5m2 ? __NV_E5M2 : __NV_E4M3);
  return __half2float(*reinterpret_cast<const __half*>(&h));
}

// Decoders: value of element i (0 <= i < kElems) of the block at p.
struct DecQ4_0 { static constexpr int kElems = 32, kBytes = 18;
  static __device__ float at(const uint8_t* p, int i) { const int q = (p[2 + (i >> 1)] >> ((i & 1) * 4)) & 15; return ld_f16(p) * (float)(q - 8); } };
struct DecQ8_0 { static constexpr int kElems = 32, kBytes = 34;
  static __device__ float at(const uint8_t* p, int i) { return ld_f16(p) * (float)(int8_t)p[2 + i]; } };
template <bool E5M2> struct DecFp8 { static constexpr int kElems = 32, kBytes = 34;
  static __device__ float at(const uint8_t* p, int i) { return ld_f16(p + 32) * fp8_to_f32(p[i], E5M2); } };
struct DecTq2_256 { static constexpr int kElems = 256, kBytes = 66;
  static __device__ float at(const uint8_t* p, int i) { const int c = (p[i >> 2] >> (2 * (i & 3))) & 3; return ld_f16(p + 64) * (c == 0 ? -1.0f : (c == 2 ? 1.0f : 0.0f)); } };
struct DecQ2K { static constexpr int kElems = 256, kBytes = 84;
  static __device__ float at(const uint8_t* p, int i) {
    const int q = (p[16 + (i >> 2)] >> ((i & 3) * 2)) & 3;
    return ld_f16(p + 80) * (float)(p[i >> 4] & 15) * (float)q - ld_f16(p + 82) * (float)(p[i >> 4] >> 4); } };
struct DecQ3K { static constexpr int kElems = 256, kBytes = 110;
  static __device__ float at(const uint8_t* p, int i) {
    const int q = ((p[32 + (i >> 2)] >> ((i & 3) * 2)) & 3) | (((p[i >> 3] >> (i & 7)) & 1) << 2);
    const int sub = i >> 4, sc = ((p[96 + (sub >> 1)] >> (4 * (sub & 1))) & 15) - 8;
    return ld_f16(p + 108) * (float)sc * (float)(q - 4); } };
__device__ __forceinline__ void k6_at(const uint8_t* s, int j, int& sc, int& mn) {
  sc = ((s[j >> 1] >> (4 * (j & 1))) & 15) | (((s[8 + (j >> 2)] >> (2 * (j & 3))) & 3) << 4);
  mn = ((s[4 + (j >> 1)] >> (4 * (j & 1))) & 15) | (((s[10 + (j >> 2)] >> (2 * (j & 3))) & 3) << 4);
}
struct DecQ4K { static constexpr int kElems = 256, kBytes = 144;
  static __device__ float at(const uint8_t* p, int i) {
    int sc, mn; k6_at(p + 4, i >> 5, sc, mn);
    const int q = (p[16 + (i >> 1)] >> ((i & 1) * 4)) & 15;
    return ld_f16(p) * (float)sc * (float)q - ld_f16(p + 2) * (float)mn; } };
struct DecQ5K { static constexpr int kElems = 256, kBytes = 176;
  static __device__ float at(const uint8_t* p, int i) {
    int sc, mn; k6_at(p + 4, i >> 5, sc, mn);
    const int q = ((p[48 + (i >> 1)] >> ((i & 1) * 4)) & 15) | (((p[16 + (i >> 3)] >> (i & 7)) & 1) << 4);
    return ld_f16(p) * (float)sc * (float)q - ld_f16(p + 2) * (float)mn; } };
struct DecQ6K { static constexpr int kElems = 256, kBytes = 210;
  static __device__ float at(const uint8_t* p, int i) {
    const int q = ((p[i >> 1] >> ((i & 1) * 4)) & 15) | (((p[128 + (i >> 2)] >> (2 * (i & 3))) & 3) << 4);
    return ld_f16(p + 208) * (float)(int8_t)p[192 + (i >> 4)] * (float)(q - 32); } };
struct DecQ8K { static constexpr int kElems = 256, kBytes = 292;
  static __device__ float at(const uint8_t* p, int i) { float d; memcpy(&d, p, 4); return d * (float)(int8_t)p[4 + i]; } };
struct DecF16 { static constexpr int kElems = 32, kBytes = 64;
  static __device__ float at(const uint8_t* p, int i) { return ld_f16(p + 2 * i); } };
struct DecBF16 { static constexpr int kElems = 32, kBytes = 64;
  static __device__ float at(const uint8_t* p, int i) { return __uint_as_float((uint32_t)(p[2 * i] | (p[2 * i + 1] << 8)) << 16); } };
struct DecF32 { static constexpr int kElems = 32, kBytes = 128;
  static __device__ float at(const uint8_t* p, int i) { float v; memcpy(&v, p + 4 * i, 4); return v; } };

template <typename D>
__global__ void __launch_bounds__(256) quant_gemv_kernel(const uint8_t* __restrict__ w, const float* __restrict__ x,
                                                        const float* __restrict__ norm_w, float eps, float* __restrict__ out,
                                                        const float* __restrict__ residual, int N, int K) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nblk = K / D::kElems;
  const size_t row_bytes = (size_t)nblk * D::kBytes;
  float inv = 1.0f;
  if (norm_w != nullptr) {
    float ss = 0.0f;
    for (int k = lane; k < K; k += 32) ss += x[k] * x[k];
    inv = 1.0f / sqrtf(warp_sum(ss) / (float)K + eps);
  }
  for (int row = blockIdx.x * 8 + warp; row < N; row += gridDim.x * 8) {
    const uint8_t* rp = w + (size_t)row * row_bytes;
    float acc = 0.0f;
    if (D::kElems == 32) {
      for (int b = lane; b < nblk; b += 32) {
        const uint8_t* p = rp + (size_t)b * D::kBytes;
        const float* xp = x + b * 32;
        const float* nw = norm_w ? norm_w + b * 32 : nullptr;
#pragma unroll 8
        for (int i = 0; i < 32; ++i) acc = fmaf(D::at(p, i), nw ? xp[i] * nw[i] : xp[i], acc);
      }
    } else {
      for (int b = 0; b < nblk; ++b) {
        const uint8_t* p = rp + (size_t)b * D::kBytes;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int i = lane * 8 + j, k = b * 256 + i;
          acc = fmaf(D::at(p, i), norm_w ? x[k] * norm_w[k] : x[k], acc);
        }
      }
    }
    acc = warp_sum(acc) * inv;
    if (lane == 0) out[row] = (residual ? residual[row] : 0.0f) + acc;
  }
}

template <typename D>
static int launch_quant_gemv(const void* w, const float* x, const float* norm_w, float eps, float* out, const float* residual, int N, int K,
                             cudaStream_t st) {
  if (K % D::kElems != 0) return BONSAI_CUDA_BAD_ARG;
  int grid = (N + 7) / 8;
  if (grid > 148 * 8) grid = 148 * 8;
  quant_gemv_kernel<D><<<grid, 256, 0, st>>>((const uint8_t*)w, x, norm_w, eps, out, residual, N, K);
  return launch_status();
}

// The same product for NB activation rows at once (a decode batch): every weight element is decoded once and multiplied into
// NB accumulators.  x: [B][x_ld], out / residual: [B][out_ld]; rows b >= B of the NB-wide template are computed on row B - 1's
// input and not stored.
template <typename D, int NB>
__global__ void __launch_bounds__(256) quant_gemv_batched_kernel(const uint8_t* __restrict__ w, const float* __restrict__ x, int x_ld,
                                                                const float* __restrict__ norm_w, float eps, float* __restrict__ out,
                                                                const float* __restrict__ residual, int out_ld, int N, int K, int B) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nblk = K / D::kElems;
  const size_t row_bytes = (size_t)nblk * D::kBytes;
  const float* xs[NB];
  float inv[NB];
#pragma unroll
  for (int t = 0; t < NB; ++t) {
    xs[t] = x + (size_t)(t < B ? t : B - 1) * x_ld;
    inv[t] = 1.0f;
    if (norm_w != nullptr) {
      float ss = 0.0f;
      for (int k = lane; k < K; k += 32) ss += xs[t][k] * xs[t][k];
      inv[t] = 1.0f / sqrtf(warp_sum(ss) / (float)K + eps);
    }
  }
  for (int row = blockIdx.x * 8 + warp; row < N; row += gridDim.x * 8) {
    const uint8_t* rp = w + (size_t)row * row_bytes;
    float acc[NB];
#pragma unroll
    for (int t = 0; t < NB; ++t) acc[t] = 0.0f;
    if (D::kElems == 32) {
      for (int b = lane; b < nblk; b += 32) {
        const uint8_t* p = rp + (size_t)b * D::kBytes;
#pragma unroll 4
        for (int i = 0; i < 32; ++i) {
          const int k = b * 32 + i;
          const float wv = D::at(p, i) * (norm_w ? norm_w[k] : 1.0f);
#pragma unroll
          for (int t = 0; t < NB; ++t) acc[t] = fmaf(wv, xs[t][k], acc[t]);
        }
      }
    } else {
      for (int b = 0; b < nblk; ++b) {
        const uint8_t* p = rp + (size_t)b * D::kBytes;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int i = lane * 8 + j, k = b * 256 + i;
          const float wv = D::at(p, i) * (norm_w ? norm_w[k] : 1.0f);
#pragma unroll
          for (int t = 0; t < NB; ++t) acc[t] = fmaf(wv, xs[t][k], acc[t]);
        }
      }
    }
#pragma unroll
    for (int t = 0; t < NB; ++t) {
      const float v = warp_sum(acc[t]) * inv[t];
      if (lane == 0 && t < B) out[(size_t)t * out_ld + row] = (residual ? residual[(size_t)t * out_ld + row] : 0.0f) + v;
    }
  }
}

template <typename D>
static int launch_quant_gemv_batched(const void* w, const float* x, int x_ld, const float* norm_w, float eps, float* out, const float* residual,
                                     int out_ld, int N, int K, int B, cudaStream_t st) {
  if (K % D::kElems != 0) return BONSAI_CUDA_BAD_ARG;
  int grid = (N + 7) / 8;
  if (grid > 148 * 8) grid = 148 * 8;
  const uint8_t* wp = (const uint8_t*)w;
  // groups of up to eight rows: the weights of a later group come from L2 when the matrix fits there
  for (int b0 = 0; b0 < B; b0 += 8) {
    const int nb = B - b0 < 8 ? B - b0 : 8;
    const float* xb = x + (size_t)b0 * x_ld;
    float* ob = out + (size_t)b0 * out_ld;
    const float* rb = residual ? residual + (size_t)b0 * out_ld : nullptr;
    if (nb == 1) quant_gemv_kernel<D><<<grid, 256, 0, st>>>(wp, xb, norm_w, eps, ob, rb, N, K);
    else if (nb == 2) quant_gemv_batched_kernel<D, 2><<<grid, 256, 0, st>>>(wp, xb, x_ld, norm_w, eps, ob, rb, out_ld, N, K, nb);
    else if (nb <= 4) quant_gemv_batched_kernel<D, 4><<<grid, 256, 0, st>>>(wp, xb, x_ld, norm_w, eps, ob, rb, out_ld, N, K, nb);
    else quant_gemv_batched_kernel<D, 8><<<grid, 256, 0, st>>>(wp, xb, x_ld, norm_w, eps, ob, rb, out_ld, N, K, nb);
  }
  return launch_status();
}

// Decodes an [N][K] matrix of blocks into row-major f16 for the dense tensor-core GEMM of the prompt path.  One thread
// owns eight consecutive inputs and stores them as one 16-byte word.  With `paired` the eight values are written in the
// K order of the GEMM's activation operand (inside every 16 inputs: position (j & 8) | ((j & 3) * 2 + ((j >> 2) & 1))
// for input j), so the prompt path's normalisation and attention kernels can feed the GEMM without a transpose.
template <typename D>
__global__ void __launch_bounds__(256) quant_to_f16_kernel(const uint8_t* __restrict__ w, __half* __restrict__ out, int N, int K, int paired) {
  const int nblk = K / D::kElems, per_row = K / 8;
  const size_t row_bytes = (size_t)nblk * D::kBytes;
  const size_t total = (size_t)N * per_row;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const int row = (int)(idx / per_row), k0 = (int)(idx % per_row) * 8;
    const uint8_t* bp = w + (size_t)row * row_bytes + (size_t)(k0 / D::kElems) * D::kBytes;
    const int i0 = k0 % D::kElems;
    __align__(16) __half v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int dst = paired ? ((j & 3) * 2 + ((j >> 2) & 1)) : j;
      v[dst] = __float2half_rn(D::at(bp, i0 + j));
    }
    *reinterpret_cast<uint4*>(out + (size_t)row * K + k0) = *reinterpret_cast<const uint4*>(v);
  }
}

template <typename D>
static int launch_quant_to_f16(const void* w, void* out, int N, int K, int paired, cudaStream_t st) {
  if (K % D::kElems != 0 || K % 16 != 0) return BONSAI_CUDA_BAD_ARG;
  const size_t total = (size_t)N * (K / 8);
  int grid = (int)((total + 255) / 256 < (size_t)(148 * 16) ? (total + 255) / 256 : (size_t)(148 * 16));
  quant_to_f16_kernel<D><<<grid, 256, 0, st>>>((const uint8_t*)w, (__half*)out, N, K, paired);
  return launch_status();
}

// out[t][i] = silu(gu[t][i]) * gu[t][inter + i]: the activation after a fused gate || up projection of T rows
__global__ void swiglu_rows_kernel(const float* __restrict__ gu, int gu_ld, float* __restrict__ out, int out_ld, int inter, int T) {
  const size_t total = (size_t)T * inter;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const int t = (int)(idx / inter), i = (int)(idx % inter);
    const float g = gu[(size_t)t * gu_ld + i];
    out[(size_t)t * out_ld + i] = g / (1.0f + __expf(-g)) * gu[(size_t)t * gu_ld + inter + i];
  }
}

__global__ void swiglu_kernel(const float* __restrict__ gate, const float* __restrict__ up, float* __restrict__ out, int n) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    const float g = gate[i];
    out[i] = g / (1.0f + __expf(-g)) * up[i];
  }
}

}  // namespace bonsai

extern "C" {

// out[N] = (residual or 0) + W (rmsnorm(x) or x) for a row-major matrix of GGUF blocks of `type`
// (GGUF type ids: 0 F32, 1 F16, 30 BF16, 2 Q4_0, 8 Q8_0, 10-15 Q2_K..Q8_K, 35 TQ2_0, 43 / 44 FP8 E4M3 / E5M2).
int bonsai_quant_gemv(int type, const void* w, const float* x, const float* norm_w, float eps, float* out, const float* residual,
                      int N, int K, cudaStream_t stream) {
  using namespace bonsai;
  if (N <= 0 || K <= 0) return BONSAI_CUDA_BAD_ARG;
  switch (type) {
    case 0: return launch_quant_gemv<DecF32>(w, x, norm_w, eps, out, residual, N, K, stream);
    case 1: return launch_quant_gemv<DecF16>(w, x, norm_w, eps, out, residual, N, K, stream);
    case 30: return launch_quant_gemv<DecBF16>(w, x, norm_w, eps, out, residual, N, K, stream);
    case 2: return launch_quant_gemv<DecQ4_0>(w, x, norm_w, eps, out, residual, N, K, stream);
    case 8: return launch_quant_gemv<DecQ8_0>(w, x, norm_w, eps, out, residual, N, K, stream);
    case 10: return launch_quant_gemv<DecQ2K>(w, x, norm_w, eps, out, residual, N, K, stream);
    case 11: return launch_quant_gemv<DecQ3K>(w, x, norm_w, eps, out, residual, N, K, stream);
    case 12: return launch_quant_gemv<DecQ4K>(w, x, norm_w, eps, out, residual, N, K, stream);
    case 13: return launch_quant_gemv<DecQ5K>(w, x, norm_w, eps, out, residual, N, K, stream);
    case 14: return launch_quant_gemv<DecQ6K>(w, x, norm_w, eps, out, residual, N, K, stream);
    case 15: return launch_quant_gemv<DecQ8K>(w, x, norm_w, eps, out, residual, N, K, stream);
    case 35: return launch_quant_gemv<DecTq2_256>(w, x, norm_w, eps, out, residual, N, K, stream);
    case 43: return launch_quant_gemv<DecFp8<false>>(w, x, norm_w, eps, out, residual, N, K, stream);
    case 44: return launch_quant_gemv<DecFp8<true>>(w, x, norm_w, eps, out, residual, N, K, stream);
    default: return BONSAI_CUDA_BAD_ARG;
  }
}

// The same for B activation rows (a decode batch): x [B][x_ld], out and residual [B][out_ld].
int bonsai_quant_gemv_batched(int type, const void* w, const float* x, int x_ld, const float* norm_w, float eps, float* out,
                              const float* residual, int out_ld, int N, int K, int B, cudaStream_t stream) {
  using namespace bonsai;
  if (N <= 0 || K <= 0 || B <= 0 || x_ld < K || out_ld < N) return BONSAI_CUDA_BAD_ARG;
#define BONSAI_QGB(D) return launch_quant_gemv_batched<D>(w, x, x_ld, norm_w, eps, out, residual, out_ld, N, K, B, stream)
  switch (type) {
    case 0: BONSAI_QGB(DecF32);
    case 1: BONSAI_QGB(DecF16);
    case 30: BONSAI_QGB(DecBF16);
    case 2: BONSAI_QGB(DecQ4_0);
    case 8: BONSAI_QGB(DecQ8_0);
    case 10: BONSAI_QGB(DecQ2K);
    case 11: BONSAI_QGB(DecQ3K);
    case 12: BONSAI_QGB(DecQ4K);
    case 13: BONSAI_QGB(DecQ5K);
    case 14: BONSAI_QGB(DecQ6K);
    case 15: BONSAI_QGB(DecQ8K);
    case 35: BONSAI_QGB(DecTq2_256);
    case 43: BONSAI_QGB(DecFp8<false>);
    case 44: BONSAI_QGB(DecFp8<true>);
    default: return BONSAI_CUDA_BAD_ARG;
  }
#undef BONSAI_QGB
}

int bonsai_swiglu_rows(const float* gu, int gu_ld, float* out, int out_ld, int inter, int T, cudaStream_t stream) {
  if (inter <= 0 || T <= 0 || gu_ld < 2 * inter || out_ld < inter) return BONSAI_CUDA_BAD_ARG;
  const size_t total = (size_t)T * inter;
  int grid = (int)((total + 255) / 256 < (size_t)(148 * 8) ? (total + 255) / 256 : (size_t)(148 * 8));
  bonsai::swiglu_rows_kernel<<<grid, 256, 0, stream>>>(gu, gu_ld, out, out_ld, inter, T);
  return bonsai::launch_status();
}

// out f16 [N][K] = the decoded matrix (same type ids as bonsai_quant_gemv); `paired` selects the activation K order of
// the tcgen05 GEMM instead of the natural one.  `out` must be 16-byte aligned.
int bonsai_quant_to_f16(int type, const void* w, void* out, int N, int K, int paired, cudaStream_t stream) {
  using namespace bonsai;
  if (N <= 0 || K <= 0 || (reinterpret_cast<uintptr_t>(out) & 15) != 0) return BONSAI_CUDA_BAD_ARG;
  switch (type) {
    case 0: return launch_quant_to_f16<DecF32>(w, out, N, K, paired, stream);
    case 1: return launch_quant_to_f16<DecF16>(w, out, N, K, paired, stream);
    case 30: return launch_quant_to_f16<DecBF16>(w, out, N, K, paired, stream);
    case 2: return launch_quant_to_f16<DecQ4_0>(w, out, N, K, paired, stream);
    case 8: return launch_quant_to_f16<DecQ8_0>(w, out, N, K, paired, stream);
    case 10: return launch_quant_to_f16<DecQ2K>(w, out, N, K, paired, stream);
    case 11: return launch_quant_to_f16<DecQ3K>(w, out, N, K, paired, stream);
    case 12: return launch_quant_to_f16<DecQ4K>(w, out, N, K, paired, stream);
    case 13: return launch_quant_to_f16<DecQ5K>(w, out, N, K, paired, stream);
    case 14: return launch_quant_to_f16<DecQ6K>(w, out, N, K, paired, stream);
    case 15: return launch_quant_to_f16<DecQ8K>(w, out, N, K, paired, stream);
    case 35: return launch_quant_to_f16<DecTq2_256>(w, out, N, K, paired, stream);
    case 43: return launch_quant_to_f16<DecFp8<false>>(w, out, N, K, paired, stream);
    case 44: return launch_quant_to_f16<DecFp8<true>>(w, out, N, K, paired, stream);
    default: return BONSAI_CUDA_BAD_ARG;
  }
}

int bonsai_swiglu(const float* gate, const float* up, float* out, int n, cudaStream_t stream) {
  if (n <= 0) return BONSAI_CUDA_BAD_ARG;
  int grid = (n + 255) / 256;
  if (grid > 148 * 4) grid = 148 * 4;
  bonsai::swiglu_kernel<<<grid, 256, 0, stream>>>(gate, up, out, n);
  return bonsai::launch_status();
}

}  // extern "C"
