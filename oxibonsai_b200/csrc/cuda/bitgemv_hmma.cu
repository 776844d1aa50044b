// Batch-1 decode GEMV on the warp-level f16 tensor cores: out = W x for a planar-SM packed matrix.
//
// The warp-per-row kernel (bitgemv_warp.cu) spends ~2.5 thread instructions per weight: a shift and a mask to turn
// two 2-bit codes into a half2, an HFMA2 against the activations, and shuffle reductions per row; `ncu` shows it
// issue-bound at about half of the memory roofline.  Here the multiply-accumulate and the reduction go to
// mma.sync.m16n8k16 and only the shift + mask remain on the CUDA cores (~1.4 instructions per weight):
//   * a warp owns a tile of 16 weight rows; lane (g, c) = (lane / 4, lane % 4) expands the codes of rows g and g + 8;
//   * one 8-byte load per row covers the two packed words 2c, 2c+1 of a 128-input group, so a quad reads the 32
//     contiguous bytes of the group and every lane's weights of one MMA share their (row, group) scale;
//   * MMA step (j, p) multiplies, for every lane c, the four weights {p, p+4, p+8, p+12} of its word j with the
//     matching activations: A = (a_p, a_{p+4}) and (b_p, b_{p+4}) pairs straight from shift + mask, B = the same
//     pairing of x from shared memory (one 16-byte load per two steps).  All eight B columns carry x, so every
//     lane ends up with the dot products of its two rows;
//   * eight MMAs accumulate a 128-input group, then the group scale is applied in f32.
// KS warps share a tile along K when there are too few tiles to fill the GPU; their partial sums meet in shared
// memory behind a named barrier and are added in slice order.  Contract and epilogues are those of
// bonsai_bitgemv_warp.  Reference counterpart: gemv_tq2_g128_v1 / gemv_q1_g128_v7..v9
// (crates/oxibonsai-kernels/src/gpu_backend/cuda_kernels.rs:76-776).
#include "common.cuh"

namespace bonsai {

enum { HEPI_STORE = 0, HEPI_RESID = 1, HEPI_SWIGLU = 2 };

constexpr int kHmWarps = 8;
constexpr int kHmBlk = 4;   // 128-input groups per load round (and per scale vector)

__device__ __forceinline__ void hmma_16816(float* d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

constexpr int kHmDepth = 3; // load rounds in flight per warp: 3 x 2 KB; one round ahead left the SMs latency-bound (measured)

struct HmBlock {
  uint2 lo[kHmBlk], hi[kHmBlk];   // packed words (2c, 2c+1) of rows g and g + 8, per group
  uint2 slo, shi;                 // the four f16 group scales of the two rows
};

__device__ __forceinline__ float hm_scale(const uint2& s, int i) {
  const uint32_t w = i < 2 ? s.x : s.y;
  return __half2float(__ushort_as_half((unsigned short)((i & 1) ? (w >> 16) : (w & 0xFFFFu))));
}

__global__ void __launch_bounds__(kHmWarps * 32, 2) bitgemv_hmma_kernel(const uint32_t* __restrict__ codes, const __half* __restrict__ scales,
                                                                       const float* __restrict__ x, const float* __restrict__ norm_w,
                                                                       float eps, float* __restrict__ out, const float* __restrict__ residual,
                                                                       int N, int K, int epi, int KS) {
  extern __shared__ uint4 xs[];                            // [K / 16 words][2] uint4: (h0,h4,h1,h5), (h2,h6,h3,h7) of a word
  __shared__ float s32[32];
  __shared__ float part[2][kHmWarps][16];
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  const int g = lane >> 2, c = lane & 3;
  const int RG = kHmWarps / KS;                            // tiles in flight per CTA
  const int rg = warp / KS, slice = warp - rg * KS;
  const int wpr = K >> 4, ng = K >> 7;                     // words and groups per row
  const int nblk = (ng + kHmBlk - 1) / kHmBlk;
  const int b0 = (slice * nblk) / KS, b1 = ((slice + 1) * nblk) / KS;   // this warp's blocks of groups
  const int ntiles = (N + 15) >> 4;
  const int tile_stride = gridDim.x * RG;
  int tile = rg * gridDim.x + blockIdx.x;                  // tiles go round the CTAs first, so a short grid of tiles still covers every SM
  const bool vec_scales = (ng & 3) == 0;

  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  auto load_block = [&](HmBlock& bk, int tl, int blk) {
    const int r_lo = tl * 16 + g, r_hi = r_lo + 8;
    const bool ok_lo = tl < ntiles && r_lo < N && blk < b1, ok_hi = tl < ntiles && r_hi < N && blk < b1;
#pragma unroll
    for (int i = 0; i < kHmBlk; ++i) {
      const int grp = blk * kHmBlk + i;
      const bool in = grp < ng;
      bk.lo[i] = ok_lo && in ? __ldg(reinterpret_cast<const uint2*>(codes + (size_t)r_lo * wpr + grp * 8) + c) : make_uint2(0u, 0u);
      bk.hi[i] = ok_hi && in ? __ldg(reinterpret_cast<const uint2*>(codes + (size_t)r_hi * wpr + grp * 8) + c) : make_uint2(0u, 0u);
    }
    if (vec_scales) {
      bk.slo = ok_lo ? __ldg(reinterpret_cast<const uint2*>(scales + (size_t)r_lo * ng) + blk) : make_uint2(0u, 0u);
      bk.shi = ok_hi ? __ldg(reinterpret_cast<const uint2*>(scales + (size_t)r_hi * ng) + blk) : make_uint2(0u, 0u);
    } else {
      unsigned short hl[kHmBlk], hh[kHmBlk];
#pragma unroll
      for (int i = 0; i < kHmBlk; ++i) {
        const int grp = blk * kHmBlk + i;
        hl[i] = ok_lo && grp < ng ? __half_as_ushort(scales[(size_t)r_lo * ng + grp]) : (unsigned short)0;
        hh[i] = ok_hi && grp < ng ? __half_as_ushort(scales[(size_t)r_hi * ng + grp]) : (unsigned short)0;
      }
      bk.slo = make_uint2((uint32_t)hl[0] | ((uint32_t)hl[1] << 16), (uint32_t)hl[2] | ((uint32_t)hl[3] << 16));
      bk.shi = make_uint2((uint32_t)hh[0] | ((uint32_t)hh[1] << 16), (uint32_t)hh[2] | ((uint32_t)hh[3] << 16));
    }
  };
  // this warp's stream of blocks: its slice [b0, b1) of every tile it owns, tile after tile
  const int nb = b1 - b0;
  const int my_tiles = tile < ntiles ? (ntiles - 1 - tile) / tile_stride + 1 : 0;
  const int total = my_tiles * nb;
  int ld_tile = tile, ld_blk = b0, ld_q = 0;               // load cursor (loads are issued in stream order)
  auto load_next = [&](HmBlock& bk) {
    load_block(bk, ld_q < total ? ld_tile : ntiles, ld_blk);
    ++ld_q;
    if (++ld_blk == b1) { ld_blk = b0; ld_tile += tile_stride; }
  };
  HmBlock ring[kHmDepth];
#pragma unroll
  for (int d = 0; d < kHmDepth; ++d) load_next(ring[d]);   // weights do not depend on the previous kernel
  asm volatile("griddepcontrol.wait;" ::: "memory");

  // ---- activations: f32 -> (normalised) half2 pairs in shared memory, in the pairing of the packed words ----
  {
    float ss = 0.0f;
    if (norm_w != nullptr) {
      for (int i = t; i < (K >> 2); i += blockDim.x) {
        const float4 v = reinterpret_cast<const float4*>(x)[i];
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
      }
      ss = block_sum(ss, s32);
    }
    const float inv = norm_w != nullptr ? 1.0f / sqrtf(ss / (float)K + eps) : 1.0f;
    for (int wd = t; wd < wpr; wd += blockDim.x) {
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
      __half2 h[8];   // (h0,h4), (h1,h5), (h2,h6), (h3,h7): a-pair and b-pair of position p side by side
#pragma unroll
      for (int p = 0; p < 4; ++p) {
        h[2 * p] = __floats2half2_rn(xr[p], xr[p + 4]);              // (a_p, a_{p+4})
        h[2 * p + 1] = __floats2half2_rn(xr[8 + p], xr[12 + p]);     // (b_p, b_{p+4})
      }
      xs[2 * wd] = *reinterpret_cast<uint4*>(&h[0]);
      xs[2 * wd + 1] = *reinterpret_cast<uint4*>(&h[4]);
    }
  }
  __syncthreads();

  int par = 0, blk = b0;
  float tot_lo = 0.0f, tot_hi = 0.0f;
  for (int q0 = 0; q0 < total; q0 += kHmDepth) {
#pragma unroll
  for (int d = 0; d < kHmDepth; ++d) {
    if (q0 + d >= total) break;
    {
      const HmBlock& cur = ring[d];
#pragma unroll
      for (int i = 0; i < kHmBlk; ++i) {
        float acc[2][4] = {{0.0f, 0.0f, 0.0f, 0.0f}, {0.0f, 0.0f, 0.0f, 0.0f}};   // one chain of dependent MMAs per word
        const int w0 = (blk * kHmBlk + i) * 8 + 2 * c;       // first of this lane's two words of the group
        const uint32_t wl[2] = {cur.lo[i].x, cur.lo[i].y}, wh[2] = {cur.hi[i].x, cur.hi[i].y};
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int wi = min(w0 + j, wpr - 1);                // groups past K carry zero weights; keep the read in range
          const uint4 v0 = xs[2 * wi], v1 = xs[2 * wi + 1];
          const uint32_t xb[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
          for (int p = 0; p < 4; ++p) {
            const uint32_t a0 = (wl[j] << (12 - 4 * p)) & 0xA000A000u, a1 = (wh[j] << (12 - 4 * p)) & 0xA000A000u;
            const uint32_t a2 = (wl[j] << (13 - 4 * p)) & 0xA000A000u, a3 = (wh[j] << (13 - 4 * p)) & 0xA000A000u;
            hmma_16816(acc[j], a0, a1, a2, a3, xb[2 * p], xb[2 * p + 1]);
          }
        }
        tot_lo = fmaf(hm_scale(cur.slo, i), acc[0][0] + acc[1][0], tot_lo);
        tot_hi = fmaf(hm_scale(cur.shi, i), acc[0][2] + acc[1][2], tot_hi);
      }
    }
    load_next(ring[d]);                                       // refill the slot: kHmDepth rounds ahead of use
    if (++blk < b1) continue;
    blk = b0;                                                 // the tile's slice is done
    if (KS > 1) {
      if (c == 0) {
        part[par][warp][g] = tot_lo;
        part[par][warp][g + 8] = tot_hi;
      }
      asm volatile("bar.sync %0, %1;" ::"r"(1 + rg), "r"(KS * 32) : "memory");
      if (slice == 0) {
        float a = 0.0f, b = 0.0f;
        for (int s = 0; s < KS; ++s) {
          a += part[par][warp + s][g];
          b += part[par][warp + s][g + 8];
        }
        tot_lo = a;
        tot_hi = b;
      }
      par ^= 1;
    }
    if (slice == 0) {
      const float v_lo = tot_lo * 128.0f, v_hi = tot_hi * 128.0f;
      const int r_lo = tile * 16 + g, r_hi = r_lo + 8;
      if (epi == HEPI_SWIGLU) {
        // gate / up rows are interleaved: even row = gate, odd row = up, one row apart = four lanes apart
        const float up_lo = __shfl_down_sync(0xffffffffu, v_lo, 4), up_hi = __shfl_down_sync(0xffffffffu, v_hi, 4);
        if (c == 0 && (g & 1) == 0) {
          if (r_lo + 1 < N) out[r_lo >> 1] = v_lo / (1.0f + __expf(-v_lo)) * up_lo;
          if (r_hi + 1 < N) out[r_hi >> 1] = v_hi / (1.0f + __expf(-v_hi)) * up_hi;
        }
      } else if (c == 0) {
        if (r_lo < N) out[r_lo] = (epi == HEPI_RESID ? residual[r_lo] : 0.0f) + v_lo;
        if (r_hi < N) out[r_hi] = (epi == HEPI_RESID ? residual[r_hi] : 0.0f) + v_hi;
      }
    }
    tot_lo = tot_hi = 0.0f;
    tile += tile_stride;
  }
  }
}

}  // namespace bonsai

extern "C" {

// Same contract as bonsai_bitgemv_warp: out[N] (or out[N/2] for epi = 2 with gate/up rows interleaved) = W x,
// x f32[K] optionally RMS-normalised with norm_w first.  K % 128 == 0, 128 <= K <= 16384.
int bonsai_bitgemv_hmma(const void* codes, const void* scales, const float* x, const float* norm_w, float eps, float* out,
                        const float* residual, int N, int K, int epi, cudaStream_t stream) {
  using namespace bonsai;
  if (K % 128 != 0 || K < 128 || K > 16384 || N <= 0 || epi < 0 || epi > 2) return BONSAI_CUDA_BAD_ARG;
  if (epi == HEPI_RESID && residual == nullptr) return BONSAI_CUDA_BAD_ARG;
  if (epi == HEPI_SWIGLU && (N & 1)) return BONSAI_CUDA_BAD_ARG;
  const int ntiles = (N + 15) / 16, ng = K / 128, nblk = (ng + kHmBlk - 1) / kHmBlk;
  // warps per tile: fewest rounds of (blocks per warp + fixed cost) over a grid of at most two CTAs per SM
  int best_ks = 1;
  long long best_cost = -1;
  for (int ks = 1; ks <= kHmWarps; ks *= 2) {
    if (ks > nblk) break;
    const int rgn = kHmWarps / ks;
    const long long grid = ntiles < 296 ? ntiles : 296;
    const long long rounds = (ntiles + grid * rgn - 1) / (grid * rgn);
    const long long cost = rounds * ((nblk + ks - 1) / ks + 2) * 16 + (grid < 148 ? (148 - grid) / 8 : 0);
    if (best_cost < 0 || cost < best_cost) {
      best_cost = cost;
      best_ks = ks;
    }
  }
  const int KS = best_ks, RG = kHmWarps / KS;
  const int grid = ntiles < 296 ? ntiles : 296;
  const size_t smem = (size_t)(K / 16) * 2 * sizeof(uint4);
  cudaError_t e = launch_pdl(bitgemv_hmma_kernel, dim3(grid), dim3(kHmWarps * 32), smem, stream, (const uint32_t*)codes,
                             (const __half*)scales, x, norm_w, eps, out, residual, N, K, epi, KS);
  return e == cudaSuccess ? BONSAI_CUDA_OK : BONSAI_CUDA_LAUNCH_FAILED;
}

}  // extern "C"

extern "C" {

// The decode path's packed-half GEMV: rows longer than 8192 inputs (the down projection) go to the tensor-core kernel,
// which measured faster there (9.8 vs 12.1 us for 4096 x 12288), everything else to the warp-per-row kernel
// (13.7 vs 15.4 us for 24576 x 4096): both are bound by the shift + mask expansion on the integer pipe, and the
// tensor-core kernel only wins where its longer per-warp streams amortise its fixed costs.
int bonsai_bitgemv_warp(const void*, const void*, const float*, const float*, float, float*, const float*, int, int, int, cudaStream_t);
int bonsai_bitgemv_fast(const void* codes, const void* scales, const float* x, const float* norm_w, float eps, float* out,
                        const float* residual, int N, int K, int epi, cudaStream_t stream) {
  return K >= 8192 ? bonsai_bitgemv_hmma(codes, scales, x, norm_w, eps, out, residual, N, K, epi, stream)
                   : bonsai_bitgemv_warp(codes, scales, x, norm_w, eps, out, residual, N, K, epi, stream);
}

}  // extern "C"
