// Batch-1 decode GEMV, warp-per-row: out = W x for a planar-SM packed matrix with packed-half FMAs.
//
// Same contract and arithmetic as bonsai_bitgemv_h2 (bitgemv.cu), different work split.  There a
// thread owns a 64-input chunk and the chunk sums of a row meet in shared memory behind two block
// barriers per tile; with a handful of tiles per CTA the kernel spends its time in those barriers and
// in the cold start of every tile.  Here a warp owns whole rows: lane l holds inputs
// [step*2048 + l*64, +64) of up to two 2048-input steps as 64 half2 registers, streams R rows at a
// time with 16-byte loads (R x NS independent loads per lane in flight), reduces each row with
// shuffles and writes it.  Warps never wait for one another when K <= 4096.  For longer rows KS warps
// share a row (each a 4096-input slice); their partial sums meet in shared memory behind a named
// barrier of just those warps and are added in slice order, so results do not depend on the grid.
//
// x is read once per CTA: all threads convert it (with the optional fused RMSNorm) to half2 in the
// pairing order of the packed words and park it in shared memory in a [step][quad][lane] layout that
// the warps read back conflict free.  The first rows' weights are requested before the programmatic
// dependency wait, so they stream while the previous kernel drains.
//
// Reference counterpart: the per-format decode GEMV kernels gemv_tq2_g128_v1 / gemv_q1_g128_v7..v9
// (crates/oxibonsai-kernels/src/gpu_backend/cuda_kernels.rs:76-776).
#include "common.cuh"

namespace bonsai {

enum { WEPI_STORE = 0, WEPI_RESID = 1, WEPI_SWIGLU = 2 };

constexpr int kWgMaxWarps = 8;

// 64 weights (one uint4 of planar-SM words) against 32 half2 activations: four chains of depth eight.
__device__ __forceinline__ float dot64_h2(const uint4 q, const __half2* __restrict__ xh) {
  const uint32_t w4[4] = {q.x, q.y, q.z, q.w};
  __half2 a0 = __float2half2_rn(0.0f), a1 = a0, a2 = a0, a3 = a0;
#pragma unroll
  for (int wd = 0; wd < 4; ++wd) {
    const uint32_t w = w4[wd];
    uint32_t m;
    m = (w << 12) & 0xA000A000u; a0 = __hfma2(*reinterpret_cast<__half2*>(&m), xh[wd * 8 + 0], a0);
    m = (w << 8) & 0xA000A000u;  a1 = __hfma2(*reinterpret_cast<__half2*>(&m), xh[wd * 8 + 1], a1);
    m = (w << 4) & 0xA000A000u;  a2 = __hfma2(*reinterpret_cast<__half2*>(&m), xh[wd * 8 + 2], a2);
    m = w & 0xA000A000u;         a3 = __hfma2(*reinterpret_cast<__half2*>(&m), xh[wd * 8 + 3], a3);
    m = (w << 13) & 0xA000A000u; a0 = __hfma2(*reinterpret_cast<__half2*>(&m), xh[wd * 8 + 4], a0);
    m = (w << 9) & 0xA000A000u;  a1 = __hfma2(*reinterpret_cast<__half2*>(&m), xh[wd * 8 + 5], a1);
    m = (w << 5) & 0xA000A000u;  a2 = __hfma2(*reinterpret_cast<__half2*>(&m), xh[wd * 8 + 6], a2);
    m = (w << 1) & 0xA000A000u;  a3 = __hfma2(*reinterpret_cast<__half2*>(&m), xh[wd * 8 + 7], a3);
  }
  const float2 f0 = __half22float2(a0), f1 = __half22float2(a1), f2 = __half22float2(a2), f3 = __half22float2(a3);
  return ((f0.x + f0.y) + (f1.x + f1.y)) + ((f2.x + f2.y) + (f3.x + f3.y));
}

// NS: 2048-input steps per warp (1 or 2).  R: rows per warp iteration (even).  KS: warps per row.
template <int NS, int R>
__global__ void __launch_bounds__(256, 2) bitgemv_warp_kernel(const uint4* __restrict__ codes, const __half* __restrict__ scales,
                                                             const float* __restrict__ x, const float* __restrict__ norm_w,
                                                             float eps, float* __restrict__ out, const float* __restrict__ residual,
                                                             int N, int K, int epi, int KS) {
  extern __shared__ uint4 xs[];                            // [steps][8][32] uint4 = half2 activations, paired order
  __shared__ float s32[32];
  __shared__ float part[2][kWgMaxWarps][R];
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  const int nwarps = blockDim.x >> 5;
  const int RG = nwarps / KS;                              // row groups per CTA
  const int rg = warp / KS, slice = warp - rg * KS;
  const int cpr = K >> 6, nsc = K >> 7;
  const int nrb = (N + R - 1) / R;                         // row blocks
  const int rb_stride = gridDim.x * RG;
  int rb = blockIdx.x * RG + rg;

  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  uint4 q[R][NS];
  float d[R][NS];
  bool ok_step[NS];
  int col[NS];
#pragma unroll
  for (int s = 0; s < NS; ++s) {
    col[s] = (slice * NS + s) * 32 + lane;                 // uint4 column of this lane in step s
    ok_step[s] = col[s] < cpr;
  }
  auto load_rows = [&](int rblock) {
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const int row = rblock * R + i;
#pragma unroll
      for (int s = 0; s < NS; ++s) {
        const bool ok = ok_step[s] && rblock < nrb && row < N;
        q[i][s] = ok ? __ldg(codes + (size_t)row * cpr + col[s]) : make_uint4(0, 0, 0, 0);
        d[i][s] = ok ? __half2float(scales[(size_t)row * nsc + (col[s] >> 1)]) : 0.0f;
      }
    }
  };
  load_rows(rb);                                           // weights do not depend on the previous kernel
  asm volatile("griddepcontrol.wait;" ::: "memory");

  // ---- activations: f32 -> (normalised) half2 pairs in shared memory ----
  {
    const int nwords = K >> 4;
    auto park = [&](int wd, const float* xr) {            // 16 activations of word wd -> paired half2, [step][quad][lane]
      __half2 h[8];
#pragma unroll
      for (int p = 0; p < 4; ++p) {
        h[p] = __floats2half2_rn(xr[p], xr[p + 4]);             // (a_p, a_{p+4})
        h[4 + p] = __floats2half2_rn(xr[8 + p], xr[12 + p]);    // (b_p, b_{p+4})
      }
      const int step = wd >> 7, owner = (wd & 127) >> 2, w4 = wd & 3;
      uint4* dst = xs + ((size_t)step * 8 + w4 * 2) * 32 + owner;
      dst[0] = *reinterpret_cast<uint4*>(&h[0]);
      dst[32] = *reinterpret_cast<uint4*>(&h[4]);
    };
    if (norm_w != nullptr && nwords <= (int)blockDim.x) {
      // one word per thread: x and the norm weights are requested together and x stays in registers across the
      // block-wide sum, so the prologue is one memory round trip instead of three
      float4 xv[4], wv[4];
      const bool mine = t < nwords;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        xv[j] = mine ? reinterpret_cast<const float4*>(x + (size_t)t * 16)[j] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        wv[j] = mine ? reinterpret_cast<const float4*>(norm_w + (size_t)t * 16)[j] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      }
      float ss = 0.0f;
#pragma unroll
      for (int j = 0; j < 4; ++j) ss += xv[j].x * xv[j].x + xv[j].y * xv[j].y + xv[j].z * xv[j].z + xv[j].w * xv[j].w;
      ss = block_sum(ss, s32);
      const float inv = 1.0f / sqrtf(ss / (float)K + eps);
      if (mine) {
        float xr[16];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          xr[4 * j] = xv[j].x * wv[j].x * inv; xr[4 * j + 1] = xv[j].y * wv[j].y * inv;
          xr[4 * j + 2] = xv[j].z * wv[j].z * inv; xr[4 * j + 3] = xv[j].w * wv[j].w * inv;
        }
        park(t, xr);
      }
    } else {
      float ss = 0.0f;
      if (norm_w != nullptr) {
        for (int i = t; i < (K >> 2); i += blockDim.x) {
          const float4 v = reinterpret_cast<const float4*>(x)[i];
          ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
        ss = block_sum(ss, s32);
      }
      const float inv = norm_w != nullptr ? 1.0f / sqrtf(ss / (float)K + eps) : 1.0f;
      for (int wd = t; wd < nwords; wd += blockDim.x) {
        float xr[16];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float4 v = reinterpret_cast<const float4*>(x + (size_t)wd * 16)[j];
          if (norm_w != nullptr) {
            const float4 w = reinterpret_cast<const float4*>(norm_w + (size_t)wd * 16)[j];
            v.x *= w.x * inv; v.y *= w.y * inv; v.z *= w.z * inv; v.w *= w.w * inv;
          }
          xr[4 * j] = v.x; xr[4 * j + 1] = v.y; xr[4 * j + 2] = v.z; xr[4 * j + 3] = v.w;
        }
        park(wd, xr);
      }
    }
  }
  __syncthreads();
  __half2 xh[NS][32];
#pragma unroll
  for (int s = 0; s < NS; ++s) {
    const int step = slice * NS + s;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      uint4 v = ok_step[s] ? xs[((size_t)step * 8 + j) * 32 + lane] : make_uint4(0, 0, 0, 0);
      *reinterpret_cast<uint4*>(&xh[s][4 * j]) = v;
    }
  }

  int par = 0;
  for (; rb < nrb; rb += rb_stride) {   // all warps of a row group share rb, so their trip counts agree
    float sum[R];
#pragma unroll
    for (int i = 0; i < R; ++i) {
      float a = 0.0f;
#pragma unroll
      for (int s = 0; s < NS; ++s) a += dot64_h2(q[i][s], xh[s]) * d[i][s];
      sum[i] = a;
    }
    const int row0 = rb * R;
    load_rows(rb + rb_stride);          // next rows stream while this block is reduced and written
#pragma unroll
    for (int i = 0; i < R; ++i) sum[i] = warp_sum(sum[i]);
    if (KS > 1) {
      if (lane == 0) {
#pragma unroll
        for (int i = 0; i < R; ++i) part[par][warp][i] = sum[i];
      }
      asm volatile("bar.sync %0, %1;" ::"r"(1 + rg), "r"(KS * 32) : "memory");
      if (slice == 0) {
#pragma unroll
        for (int i = 0; i < R; ++i) {
          float a = 0.0f;
          for (int s = 0; s < KS; ++s) a += part[par][warp + s][i];
          sum[i] = a;
        }
      }
      par ^= 1;
    }
    if (slice == 0 && lane == 0) {
      if (epi == WEPI_SWIGLU) {
#pragma unroll
        for (int i = 0; i < R; i += 2) {
          const float a = sum[i] * 128.0f, b = sum[i + 1] * 128.0f;
          if (row0 + i + 1 < N) out[(row0 + i) >> 1] = a / (1.0f + __expf(-a)) * b;
        }
      } else {
#pragma unroll
        for (int i = 0; i < R; ++i) {
          const int row = row0 + i;
          if (row < N) out[row] = (epi == WEPI_RESID ? residual[row] : 0.0f) + sum[i] * 128.0f;
        }
      }
    }
  }
}

template <int NS, int R>
static int launch_warp_gemv(const void* codes, const void* scales, const float* x, const float* norm_w, float eps, float* out,
                            const float* residual, int N, int K, int epi, int KS, cudaStream_t stream) {
  const int RG = KS == 3 ? 2 : 8 / KS;
  const int threads = RG * KS * 32;
  const int steps = (K + 2047) / 2048;
  const size_t smem = (size_t)steps * 8 * 32 * sizeof(uint4);
  const int nrb = (N + R - 1) / R;
  int grid = (nrb + RG - 1) / RG;
  if (grid > 148 * 2) grid = 148 * 2;
  cudaError_t e = launch_pdl(bitgemv_warp_kernel<NS, R>, dim3(grid), dim3(threads), smem, stream, (const uint4*)codes,
                             (const __half*)scales, x, norm_w, eps, out, residual, N, K, epi, KS);
  return e == cudaSuccess ? BONSAI_CUDA_OK : BONSAI_CUDA_LAUNCH_FAILED;
}

}  // namespace bonsai

extern "C" {

// Same contract as bonsai_bitgemv_h2: out[N] (or out[N/2] for epi = 2 with gate/up rows interleaved) = W x,
// x f32[K] optionally RMS-normalised with norm_w first.  K % 128 == 0, 128 <= K <= 16384.
int bonsai_bitgemv_warp(const void* codes, const void* scales, const float* x, const float* norm_w, float eps, float* out,
                        const float* residual, int N, int K, int epi, cudaStream_t stream) {
  using namespace bonsai;
  if (K % 128 != 0 || K < 128 || K > 16384 || N <= 0 || epi < 0 || epi > 2) return BONSAI_CUDA_BAD_ARG;
  if (epi == WEPI_RESID && residual == nullptr) return BONSAI_CUDA_BAD_ARG;
  if (epi == WEPI_SWIGLU && (N & 1)) return BONSAI_CUDA_BAD_ARG;
  const int steps = (K + 2047) / 2048;
  if (steps == 1) {
    // short rows: one step per warp
    return N >= 148 * 2 * 8 * 4 ? launch_warp_gemv<1, 4>(codes, scales, x, norm_w, eps, out, residual, N, K, epi, 1, stream)
                               : launch_warp_gemv<1, 2>(codes, scales, x, norm_w, eps, out, residual, N, K, epi, 1, stream);
  }
  const int KS = (steps + 1) / 2;
  const int RG = KS == 3 ? 2 : 8 / KS;
  // four rows per warp iteration once that still gives every warp of a full grid work
  if ((long long)N >= 148LL * 2 * RG * 4)
    return launch_warp_gemv<2, 4>(codes, scales, x, norm_w, eps, out, residual, N, K, epi, KS, stream);
  return launch_warp_gemv<2, 2>(codes, scales, x, norm_w, eps, out, residual, N, K, epi, KS, stream);
}

}  // extern "C"
