// Batch-1 decode GEMV on the warp-level fp8 tensor-core instruction, weights decoded in two
// instructions per four and never staged through shared memory.
//
// The CUDA-core GEMV kernels spend ~2.4 thread instructions per weight and are bound by instruction
// issue, not by HBM.  Here the weights are stored in a *fragment* layout whose 32-bit words are the
// A operand of `mma.sync.m16n8k32` (e4m3) before decoding: a word holds, for one lane, the sixteen
// weights of its A fragment as (sign, magnitude) bit pairs, pair q of byte b at bits (7-2q, 6-2q) of
// that byte.  `(w << 2q) & 0xC0C0C0C0` is then register a_q of the fragment: every byte is an e4m3
// number with only its sign bit and top exponent bit taken from the code, i.e. +-2.0 or 0.  A lane
// reads one 16-byte vector per 128-column group (four k32 steps, one group scale), so a warp streams
// 512 contiguous bytes per (16-row tile, group).
//
// The activation vector is the B operand: x (RMS-normalised when asked) is scaled to the e4m3 range
// and split into three e4m3 terms x ~ (q0 + q1/16 + q2/256)/S, which occupy columns 0..2 of B, so one
// MMA multiplies a fragment by all three terms at once; the three accumulator columns are recombined
// in f32 at the end.  Three terms carry 12 significant bits, one more than f16.  Accumulation is f32
// inside the tensor core per 128-column group, then `acc += c * group_scale` in f32.
//
// Work split: a task is (16-row tile, K slice); the eight warps of a CTA take `tiles_per_cta` tiles x
// `ksplit` slices, every warp issues all of its weight loads before the programmatic dependency wait,
// slice partials meet in shared memory and are added in slice order (results do not depend on
// timing).  Epilogues: store, residual add, SwiGLU over interleaved gate/up rows.
//
// Reference counterpart: decode GEMV kernels gemv_tq2_g128_v1 / gemv_q1_g128_v7..v9
// (crates/oxibonsai-kernels/src/gpu_backend/cuda_kernels.rs:76-776).
#include <cuda_fp8.h>

#include "common.cuh"

namespace bonsai {

enum { MEPI_STORE = 0, MEPI_RESID = 1, MEPI_SWIGLU = 2 };

constexpr int kMmaMaxGroups = 16;   // 128-column groups one warp may own (K slice <= 2048 columns)

// planar-SM word (row, 16-column block): weight i < 8 has sign bit 4i+3 and magnitude bit 4i+1, weight
// 8+i has sign bit 4i+2 and magnitude bit 4i.
__device__ __forceinline__ uint32_t planar_sm_bits(uint32_t w, int k) {   // -> (S << 1) | M
  const int i = k & 7, lo = (k >> 3) & 1;
  const uint32_t s = (w >> (4 * i + 3 - lo)) & 1u, m = (w >> (4 * i + 1 - lo)) & 1u;
  return (s << 1) | m;
}

// One thread per output word.  out_codes: [tile][group][lane] uint4; out_scales: [tile][group][8] half2
// = (scale of row g, scale of row g + 8).  Rows >= N decode to zero.
__global__ void repack_frag_kernel(const uint32_t* __restrict__ codes, const __half* __restrict__ scales, int N, int K,
                                   uint32_t* __restrict__ out_codes, __half2* __restrict__ out_scales) {
  const int ngroups = K >> 7, ntiles = (N + 15) >> 4;
  const size_t total = (size_t)ntiles * ngroups * 128;
  for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const int j = idx & 3, lane = (idx >> 2) & 31;
    const size_t tg = idx >> 7;
    const int kg = (int)(tg % ngroups), rt = (int)(tg / ngroups);
    const int g = lane >> 2, t = lane & 3;
    uint32_t w = 0;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int row = rt * 16 + g + 8 * (q & 1);
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const int k = kg * 128 + j * 32 + 16 * (q >> 1) + 4 * t + b;
        uint32_t sm = 0;
        if (row < N) sm = planar_sm_bits(codes[(size_t)row * (K >> 4) + (k >> 4)], k & 15);
        if (!(sm & 1u)) sm = 0;   // a zero weight carries no sign
        w |= sm << (8 * b + 6 - 2 * q);
      }
    }
    out_codes[idx] = w;
    if (j == 0 && t == 0) {
      const int r0 = rt * 16 + g, r1 = r0 + 8;
      const __half z = __float2half(0.0f);
      out_scales[tg * 8 + g] = __halves2half2(r0 < N ? scales[(size_t)r0 * ngroups + kg] : z, r1 < N ? scales[(size_t)r1 * ngroups + kg] : z);
    }
  }
}

__device__ __forceinline__ void mma_e4m3(float (&c)[4], const uint32_t (&a)[4], const uint2 b) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b.x), "r"(b.y));
}

__device__ __forceinline__ uint32_t to_e4m3(float v) { return (uint32_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3); }
__device__ __forceinline__ float from_e4m3(uint32_t q) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)q, __NV_E4M3);
  return __half2float(*reinterpret_cast<const __half*>(&h));
}

// GPW: groups per warp (compile-time bound of the register arrays).
template <int GPW>
__global__ void __launch_bounds__(256, 2) bitgemv_mma_kernel(const uint4* __restrict__ codes, const __half2* __restrict__ scales,
                                                            const float* __restrict__ x, const float* __restrict__ norm_w,
                                                            float eps, float* __restrict__ out, const float* __restrict__ residual,
                                                            int N, int K, int epi, int ksplit) {
  extern __shared__ __align__(16) uint8_t xq[];            // [3 terms][K] e4m3, k order permuted per 32 so a lane's B fragment is 8 contiguous bytes
  __shared__ float s_red[64];
  __shared__ float part[2][8][16];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int ngroups = K >> 7;
  const int tiles_per_cta = 8 / ksplit;
  const int slice = warp % ksplit;
  const int ntiles = (N + 15) >> 4;
  const int ntg = (ntiles + tiles_per_cta - 1) / tiles_per_cta;   // tile groups; one per CTA iteration
  const int per = (ngroups + ksplit - 1) / ksplit;
  const int g0 = slice * per, g1 = min(ngroups, g0 + per);

  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  uint4 w[GPW];
  __half2 d[GPW];
  auto load_tile = [&](int tgi) {
    const int tile = tgi * tiles_per_cta + warp / ksplit;
    const bool live = tgi < ntg && tile < ntiles;
#pragma unroll
    for (int i = 0; i < GPW; ++i) {
      const int kg = g0 + i;
      const bool ok = live && kg < g1;
      const size_t tg = (size_t)tile * ngroups + kg;
      w[i] = ok ? __ldg(codes + tg * 32 + lane) : make_uint4(0, 0, 0, 0);
      d[i] = ok ? scales[tg * 8 + g] : __float2half2_rn(0.0f);
    }
  };
  // weights and scales do not depend on the previous kernel: request the first tile's now
  load_tile(blockIdx.x);
  asm volatile("griddepcontrol.wait;" ::: "memory");

  // ---- activations -> three e4m3 terms in shared memory ----
  float ss = 0.0f, amax = 0.0f;
  for (int i = tid; i < (K >> 2); i += 256) {
    float4 v = reinterpret_cast<const float4*>(x)[i];
    if (norm_w != nullptr) {
      ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
      const float4 nw = reinterpret_cast<const float4*>(norm_w)[i];
      v.x *= nw.x; v.y *= nw.y; v.z *= nw.z; v.w *= nw.w;
    }
    amax = fmaxf(fmaxf(amax, fmaxf(fabsf(v.x), fabsf(v.y))), fmaxf(fabsf(v.z), fabsf(v.w)));
  }
  ss = warp_sum(ss);
  amax = warp_max(amax);
  if (lane == 0) {
    s_red[warp] = ss;
    s_red[32 + warp] = amax;
  }
  __syncthreads();
  ss = 0.0f;
  amax = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    ss += s_red[i];
    amax = fmaxf(amax, s_red[32 + i]);
  }
  const float inv = norm_w != nullptr ? 1.0f / sqrtf(ss / (float)K + eps) : 1.0f;
  // largest magnitude maps to 224 (e4m3 tops out at 448); S folds the RMS factor in
  const float S = amax > 0.0f ? 224.0f / amax : 1.0f;
  for (int i = tid; i < (K >> 2); i += 256) {
    float4 v = reinterpret_cast<const float4*>(x)[i];
    if (norm_w != nullptr) {
      const float4 nw = reinterpret_cast<const float4*>(norm_w)[i];
      v.x *= nw.x; v.y *= nw.y; v.z *= nw.z; v.w *= nw.w;
    }
    const float xv[4] = {v.x * S, v.y * S, v.z * S, v.w * S};
    uint32_t q0 = 0, q1 = 0, q2 = 0;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const uint32_t a = to_e4m3(xv[e]);
      const float r1 = (xv[e] - from_e4m3(a)) * 16.0f;
      const uint32_t b = to_e4m3(r1);
      const float r2 = (r1 - from_e4m3(b)) * 16.0f;
      const uint32_t c = to_e4m3(r2);
      q0 |= a << (8 * e); q1 |= b << (8 * e); q2 |= c << (8 * e);
    }
    // element k = 4i..4i+3 of a 32-block: quad index u = (k & 31) >> 2; fragment order puts quad u at
    // byte offset (u & 3) * 8 + (u >> 2) * 4
    const int k = i << 2, u = (k & 31) >> 2;
    const int pos = (k & ~31) + (u & 3) * 8 + (u >> 2) * 4;
    *reinterpret_cast<uint32_t*>(xq + pos) = q0;
    *reinterpret_cast<uint32_t*>(xq + K + pos) = q1;
    *reinterpret_cast<uint32_t*>(xq + 2 * K + pos) = q2;
  }
  __syncthreads();

  // ---- main loop: four MMAs per group, one tile group per iteration ----
  const uint8_t* xb = xq + (g < 3 ? g : 0) * K + t * 8;
  const float unscale = inv / (2.0f * S);    // weights decode as +-2
  int par = 0;
  for (int tgi = blockIdx.x; tgi < ntg; tgi += gridDim.x, par ^= 1) {
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
    for (int i = 0; i < GPW; ++i) {
      const int kg = g0 + i;
      if (kg < g1) {   // uniform across the warp
        float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        const uint32_t w4[4] = {w[i].x, w[i].y, w[i].z, w[i].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint2 b = *reinterpret_cast<const uint2*>(xb + (kg * 4 + j) * 32);
          if (g >= 3) b = make_uint2(0u, 0u);
          const uint32_t a[4] = {w4[j] & 0xC0C0C0C0u, (w4[j] << 2) & 0xC0C0C0C0u, (w4[j] << 4) & 0xC0C0C0C0u, (w4[j] << 6) & 0xC0C0C0C0u};
          mma_e4m3(c, a, b);
        }
        const float2 df = __half22float2(d[i]);
        acc[0] = fmaf(c[0], df.x, acc[0]);
        acc[1] = fmaf(c[1], df.x, acc[1]);
        acc[2] = fmaf(c[2], df.y, acc[2]);
        acc[3] = fmaf(c[3], df.y, acc[3]);
      }
    }
    load_tile(tgi + gridDim.x);   // next tile streams while this one is reduced and written
    // columns: lane t = 0 holds terms 0 and 1, lane t = 1 holds term 2 (its second column is zero)
    float r_lo = (t == 0) ? acc[0] + acc[1] * 0.0625f : (t == 1 ? acc[0] * 0.00390625f : 0.0f);
    float r_hi = (t == 0) ? acc[2] + acc[3] * 0.0625f : (t == 1 ? acc[2] * 0.00390625f : 0.0f);
    r_lo += __shfl_xor_sync(0xffffffffu, r_lo, 1);
    r_hi += __shfl_xor_sync(0xffffffffu, r_hi, 1);
    if (t == 0) {
      part[par][warp][g] = r_lo * unscale;
      part[par][warp][g + 8] = r_hi * unscale;
    }
    __syncthreads();   // every warp runs the same number of iterations; parity keeps one barrier per iteration enough
    const int tile = tgi * tiles_per_cta + warp / ksplit;
    if (slice == 0 && tile < ntiles && lane < 16) {
      float v = 0.0f;
      for (int s = 0; s < ksplit; ++s) v += part[par][warp + s][lane];
      const int row = tile * 16 + lane;
      if (epi == MEPI_SWIGLU) {
        const float up = __shfl_down_sync(0x0000ffffu, v, 1);
        if ((lane & 1) == 0 && row + 1 < N) out[row >> 1] = v / (1.0f + __expf(-v)) * up;
      } else if (row < N) {
        out[row] = (epi == MEPI_RESID ? residual[row] : 0.0f) + v;
      }
    }
  }
}

template <int GPW>
static int launch_mma(const void* codes, const void* scales, const float* x, const float* norm_w, float eps, float* out,
                      const float* residual, int N, int K, int epi, int ksplit, cudaStream_t stream) {
  const int ntiles = (N + 15) / 16, tiles_per_cta = 8 / ksplit;
  int grid = (ntiles + tiles_per_cta - 1) / tiles_per_cta;
  if (grid > 148 * 2) grid = 148 * 2;
  static bool smem_opt_in = false;   // K > 16128 needs more than the default 48 KB of dynamic shared memory
  if (!smem_opt_in) {
    cudaFuncSetAttribute(bitgemv_mma_kernel<GPW>, cudaFuncAttributeMaxDynamicSharedMemorySize, 3 * 16384);
    smem_opt_in = true;
  }
  cudaError_t e = launch_pdl(bitgemv_mma_kernel<GPW>, dim3(grid), dim3(256), (size_t)3 * K, stream, (const uint4*)codes,
                             (const __half2*)scales, x, norm_w, eps, out, residual, N, K, epi, ksplit);
  return e == cudaSuccess ? BONSAI_CUDA_OK : BONSAI_CUDA_LAUNCH_FAILED;
}

}  // namespace bonsai

extern "C" {

// Bytes of the fragment layout for an N x K matrix: codes, then scales.
void bonsai_frag_sizes(int N, int K, size_t* code_bytes, size_t* scale_bytes) {
  const size_t ntiles = (size_t)(N + 15) / 16, ngroups = (size_t)K / 128;
  *code_bytes = ntiles * ngroups * 512;
  *scale_bytes = ntiles * ngroups * 8 * sizeof(__half2);
}

// planar-SM (codes uint32 [N][K/16], scales f16 [N][K/128]) -> fragment layout.
int bonsai_repack_frag(const void* codes, const void* scales, int N, int K, void* out_codes, void* out_scales, cudaStream_t stream) {
  if (K % 128 != 0 || N <= 0) return BONSAI_CUDA_BAD_ARG;
  bonsai::repack_frag_kernel<<<148 * 8, 256, 0, stream>>>((const uint32_t*)codes, (const __half*)scales, N, K, (uint32_t*)out_codes,
                                                         (__half2*)out_scales);
  return bonsai::launch_status();
}

// out[N] (or out[N/2] with epi = 2, gate/up rows interleaved) = W x on fragment-layout weights; x f32[K], optionally
// RMS-normalised with norm_w.  K % 128 == 0, K <= 16384 (three K-byte term rows must fit in 48 KB of shared memory).
int bonsai_bitgemv_mma(const void* codes, const void* scales, const float* x, const float* norm_w, float eps, float* out,
                       const float* residual, int N, int K, int epi, cudaStream_t stream) {
  using namespace bonsai;
  if (K % 128 != 0 || K < 128 || K > 16384 || N <= 0 || epi < 0 || epi > 2) return BONSAI_CUDA_BAD_ARG;
  if (epi == MEPI_RESID && residual == nullptr) return BONSAI_CUDA_BAD_ARG;
  if (epi == MEPI_SWIGLU && (N & 1)) return BONSAI_CUDA_BAD_ARG;
  const int ngroups = K / 128, ntiles = (N + 15) / 16;
  // enough (tile, slice) tasks for ~2400 warps, slices no longer than kMmaMaxGroups
  int ksplit = 1;
  while (ksplit < 8 && ((long long)ntiles * ksplit < 2400 || (ngroups + ksplit - 1) / ksplit > kMmaMaxGroups)) ksplit *= 2;
  const int per = (ngroups + ksplit - 1) / ksplit;
  if (per > kMmaMaxGroups) return BONSAI_CUDA_BAD_ARG;
  if (per <= 4) return launch_mma<4>(codes, scales, x, norm_w, eps, out, residual, N, K, epi, ksplit, stream);
  if (per <= 8) return launch_mma<8>(codes, scales, x, norm_w, eps, out, residual, N, K, epi, ksplit, stream);
  if (per <= 12) return launch_mma<12>(codes, scales, x, norm_w, eps, out, residual, N, K, epi, ksplit, stream);
  return launch_mma<16>(codes, scales, x, norm_w, eps, out, residual, N, K, epi, ksplit, stream);
}

}  // extern "C"
