// Decode-batch GEMM (up to 64 tokens) for packed ternary / 1-bit weights on the warp-level f16 tensor cores.
//
//   out[t][n] = sum_k X[t][k] * W[n][k]        t < T <= 64 tokens, n < N rows
//
// The tcgen05 kernel (bitgemm_prefill.cu) has to put the expanded weights into shared memory for the tensor core
// and to hand every 64-input block over through mbarriers; with 64 columns of tensor work per block those fixed
// costs dominate (26 / 26 / 43 / 39 us for the four GEMMs of an 8B layer at 64 tokens).  mma.sync takes its A
// operand from registers, so here the 2-bit -> f16 expansion (one shift + one mask per two weights, as in
// bitgemv_hmma.cu) feeds the MMA directly:
//   * a warp owns 16 weight rows x one 128-input group per step; lane (g, c) expands words 2c, 2c+1 of rows g, g+8;
//   * MMA step (j, p) uses, for every c, the four weights {p, p+4, p+8, p+12} of word 2c+j as its 16 k-slots;
//   * the activations arrive in that same order ("hmma-K": hmma_k_pos below, a permutation inside each 128-input
//     group written by the producers of decode-batch activations), one 128-input chunk of all tokens per step through
//     cp.async into padded shared-memory rows, double buffered; B fragments come from ldmatrix;
//   * eight n-tiles of 8 tokens share every expanded A fragment; the group scale is applied in f32 per group.
// A CTA is RW row-warps x KW k-warps (RW * KW = 8): the k-warps walk different K ranges (their own chunk of the
// stage) and their partial sums are added in k order through shared memory at the end, so few-row projections still
// fill the GPU.  Reference counterpart: the batch kernels gemm_q1_g128_v7 / gemm_tq2_g128_v7 and their fused forms
// (crates/oxibonsai-kernels/src/gpu_backend/cuda_prefill_kernels.rs:74-827).
#include <cuda_fp16.h>

#include "../comm/tp_comm.cuh"
#include "common.cuh"

namespace bonsai {

constexpr int kGhWarps = 8;
constexpr int kGhMaxTok = 64;
constexpr int kGhRow = 272;                       // bytes per token row of a chunk: 128 f16 + 16 (bank spread)
constexpr int kGhChunk = kGhMaxTok * kGhRow;      // 17408 bytes: one 128-input chunk of 64 tokens
constexpr int kGhDepth = 3;                       // weight groups in flight per warp

__device__ __forceinline__ uint32_t gh_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void gh_cp_async16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void gh_ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void gh_mma(float* d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

struct GhParams {
  const uint32_t* codes;
  const __half* scales;
  const __half* x;         // [T][x_ld] f16, hmma-K order
  float* out_f32;          // [T][out_ld]  (epi 0, 1)
  const float* residual;   // [T][out_ld]  (epi 1)
  __half* out_f16;         // [T][out_ld]  (epi 2: SwiGLU over interleaved gate / up rows, hmma-K order)
  int n_rows, K, T, epi, x_ld, out_ld, KW;
};

struct GhGroup {
  uint2 lo, hi;     // packed words (2c, 2c+1) of rows g and g + 8
  float slo, shi;   // group scales
};

template <int NT>   // n-tiles of 8 tokens (T <= 8 * NT)
__global__ void __launch_bounds__(kGhWarps * 32) bitgemm_hmma_kernel(GhParams p, TpComm tp) {
  extern __shared__ __align__(16) uint8_t gh_smem[];   // [2 stages][KW chunks][64 tokens][272 bytes]; later the k-warp partial sums
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  const int g = lane >> 2, c = lane & 3;
  const int KW = p.KW, RW = kGhWarps / KW;
  const int kw = warp / RW, rw = warp - kw * RW;         // k-warp and row-warp of this warp
  const int wpr = p.K >> 4, ng = p.K >> 7;
  const int nsteps = (ng + KW - 1) / KW;                  // groups per k-warp (the last k-warp may own fewer)
  const int g0 = kw * nsteps;                             // first group of this k-warp
  const int row0 = (blockIdx.x * RW + rw) * 16;
  const int r_lo = row0 + g, r_hi = r_lo + 8;
  const bool ok_lo = r_lo < p.n_rows, ok_hi = r_hi < p.n_rows;
  const uint32_t smem0 = gh_smem_u32(gh_smem);

  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  auto load_group = [&](GhGroup& w, int s) {              // step s of this k-warp
    const int grp = g0 + s;
    const bool in = s < nsteps && grp < ng;
    w.lo = in && ok_lo ? __ldg(reinterpret_cast<const uint2*>(p.codes + (size_t)r_lo * wpr + grp * 8) + c) : make_uint2(0u, 0u);
    w.hi = in && ok_hi ? __ldg(reinterpret_cast<const uint2*>(p.codes + (size_t)r_hi * wpr + grp * 8) + c) : make_uint2(0u, 0u);
    w.slo = in && ok_lo ? __half2float(p.scales[(size_t)r_lo * ng + grp]) : 0.0f;
    w.shi = in && ok_hi ? __half2float(p.scales[(size_t)r_hi * ng + grp]) : 0.0f;
  };
  GhGroup ring[kGhDepth];
#pragma unroll
  for (int d = 0; d < kGhDepth; ++d) load_group(ring[d], d);   // weights do not depend on the previous kernel
  asm volatile("griddepcontrol.wait;" ::: "memory");

  // activations of step s: chunk k of the stage is the 128-input group of k-warp k, all tokens
  auto issue_stage = [&](int s, int buf) {
    constexpr int kTok = 8 * NT;                           // token rows that the MMAs read
    const int pieces = KW * kTok * 16;                     // 16-byte pieces of the stage
    for (int i = t; i < pieces; i += kGhWarps * 32) {
      const int k = i / (kTok * 16), rem = i - k * (kTok * 16), tok = rem >> 4, c16 = rem & 15;
      const int grp = k * nsteps + s;
      const bool in = s < nsteps && grp < ng && tok < p.T;   // rows past T are zero-filled
      const __half* src = p.x + (size_t)(in ? tok : 0) * p.x_ld + (size_t)(in ? grp : 0) * 128 + c16 * 8;
      gh_cp_async16(smem0 + (uint32_t)((buf * KW + k) * kGhChunk + tok * kGhRow + c16 * 16), src, in ? 16 : 0);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  float tot[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) tot[nt][0] = tot[nt][1] = tot[nt][2] = tot[nt][3] = 0.0f;

  issue_stage(0, 0);
  for (int s0 = 0; s0 < nsteps; s0 += kGhDepth) {
#pragma unroll
    for (int d = 0; d < kGhDepth; ++d) {
      const int s = s0 + d;
      if (s >= nsteps) break;                              // uniform over the CTA
      const int buf = s & 1;
      asm volatile("cp.async.wait_group 0;" ::: "memory");
      __syncthreads();                                     // stage s has landed for everyone; stage buffer buf ^ 1 is free
      issue_stage(s + 1, buf ^ 1);
      const GhGroup cur = ring[d];
      load_group(ring[d], s + kGhDepth);
      float acc[NT][4];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.0f;
      const uint32_t chunk = smem0 + (uint32_t)((buf * KW + kw) * kGhChunk);
      const uint32_t wl[2] = {cur.lo.x, cur.lo.y}, wh[2] = {cur.hi.x, cur.hi.y};
      const int mi = lane >> 3, r8 = lane & 7;
#pragma unroll
      for (int j = 0; j < 2; ++j) {
#pragma unroll
        for (int pp = 0; pp < 4; ++pp) {
          const uint32_t a0 = (wl[j] << (12 - 4 * pp)) & 0xA000A000u, a1 = (wh[j] << (12 - 4 * pp)) & 0xA000A000u;
          const uint32_t a2 = (wl[j] << (13 - 4 * pp)) & 0xA000A000u, a3 = (wh[j] << (13 - 4 * pp)) & 0xA000A000u;
#pragma unroll
          for (int nt = 0; nt < NT; nt += 2) {
            // matrices: (tokens of n-tile nt, k-slots 0-7), (nt, slots 8-15), (nt + 1, 0-7), (nt + 1, 8-15)
            uint32_t b0, b1, b2, b3;
            gh_ldmatrix_x4(chunk + (uint32_t)(((nt + (mi >> 1)) * 8 + r8) * kGhRow + (j * 4 + pp) * 32 + (mi & 1) * 16), b0, b1, b2, b3);
            gh_mma(acc[nt], a0, a1, a2, a3, b0, b1);
            if (nt + 1 < NT) gh_mma(acc[nt + 1], a0, a1, a2, a3, b2, b3);
          }
        }
      }
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        tot[nt][0] = fmaf(cur.slo, acc[nt][0], tot[nt][0]);
        tot[nt][1] = fmaf(cur.slo, acc[nt][1], tot[nt][1]);
        tot[nt][2] = fmaf(cur.shi, acc[nt][2], tot[nt][2]);
        tot[nt][3] = fmaf(cur.shi, acc[nt][3], tot[nt][3]);
      }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();                                         // every warp is done with the stages: the memory is reused below

  // ---- partial sums of the k-warps meet in shared memory and are added in k order --------------------
  float* part = reinterpret_cast<float*>(gh_smem);          // [KW][RW][NT][32 lanes][4]
  if (KW > 1) {
    float4* dst = reinterpret_cast<float4*>(part) + ((size_t)(kw * RW + rw) * NT) * 32 + lane;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) dst[nt * 32] = make_float4(tot[nt][0], tot[nt][1], tot[nt][2], tot[nt][3]);
    __syncthreads();
    if (kw == 0) {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        float4 a = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        for (int k = 0; k < KW; ++k) {
          const float4 v = reinterpret_cast<const float4*>(part)[((size_t)(k * RW + rw) * NT + nt) * 32 + lane];
          a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w;
        }
        tot[nt][0] = a.x; tot[nt][1] = a.y; tot[nt][2] = a.z; tot[nt][3] = a.w;
      }
    }
  }
  if (kw != 0) return;

  // ---- epilogue: lane holds (row g | g + 8) x (tokens nt * 8 + 2c, + 1) -------------------------------
  // The residual usually aliases the output (h += W x): inside a store loop every load would have to wait for the
  // previous store, a chain of exposed memory latencies, so the residuals are loaded as a block first.
  // epi 3 (row-parallel shard of a tensor-parallel group): every value goes to all peers as one 8-byte {value, tag}
  // store into slot [parity][my rank][token][row] before the residuals are even requested, and is summed with the
  // peers' values in rank order below - the all-reduce and the residual add are this epilogue.
  int tp_epoch = 0;
  if (p.epi == 3) {
    tp_epoch = ld_volatile(tp.epoch);
    const unsigned long long tag_hi = (unsigned long long)((uint32_t)tp_epoch + 1u) << 32;
    const int parity = tp_epoch & 1;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int tok = nt * 8 + 2 * c + e;
        if (tok >= p.T) continue;
        const size_t i_lo = (size_t)tok * p.n_rows + r_lo, i_hi = (size_t)tok * p.n_rows + r_hi;
        const unsigned long long m_lo = tag_hi | __float_as_uint(tot[nt][e] * 128.0f), m_hi = tag_hi | __float_as_uint(tot[nt][2 + e] * 128.0f);
        if (tp.mc != nullptr) {   // one multicast store per message: the switch replicates it into every rank's slot
          unsigned long long* dst = tp_ll_big_slot_mc(tp, parity, tp.rank);
          if (ok_lo) tp_mc_st_msg(dst + i_lo, m_lo);
          if (ok_hi) tp_mc_st_msg(dst + i_hi, m_hi);
        } else {
          for (int q = 0; q < tp.size; ++q) {
            if (q == tp.rank) continue;
            unsigned long long* dst = tp_ll_big_slot(tp, q, parity, tp.rank);
            if (ok_lo) tp_st_msg(dst + i_lo, m_lo);
            if (ok_hi) tp_st_msg(dst + i_hi, m_hi);
          }
        }
      }
  }
  float res[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int tok = nt * 8 + 2 * c + e;
      const bool rd = (p.epi == 1 || (p.epi == 3 && p.residual != nullptr)) && tok < p.T;
      res[nt][e] = rd && ok_lo ? p.residual[(size_t)tok * p.out_ld + r_lo] : 0.0f;
      res[nt][2 + e] = rd && ok_hi ? p.residual[(size_t)tok * p.out_ld + r_hi] : 0.0f;
    }
  bool tp_alive = true;
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int tok = nt * 8 + 2 * c + e;
      const float v_lo = tot[nt][e] * 128.0f, v_hi = tot[nt][2 + e] * 128.0f;
      if (p.epi == 2) {
        // gate / up rows are interleaved: even row = gate, odd row = up, one row apart = four lanes apart
        const float up_lo = __shfl_down_sync(0xffffffffu, v_lo, 4), up_hi = __shfl_down_sync(0xffffffffu, v_hi, 4);
        if ((g & 1) == 0 && tok < p.T) {
          if (r_lo + 1 < p.n_rows) p.out_f16[(size_t)tok * p.out_ld + hmma_k_pos(r_lo >> 1)] = __float2half_rn(v_lo / (1.0f + __expf(-v_lo)) * up_lo);
          if (r_hi + 1 < p.n_rows) p.out_f16[(size_t)tok * p.out_ld + hmma_k_pos(r_hi >> 1)] = __float2half_rn(v_hi / (1.0f + __expf(-v_hi)) * up_hi);
        }
      } else if (p.epi == 3) {
        if (tok < p.T) {
          const uint32_t tag = (uint32_t)tp_epoch + 1u;
          const int parity = tp_epoch & 1;
          const size_t i_lo = (size_t)tok * p.n_rows + r_lo, i_hi = (size_t)tok * p.n_rows + r_hi;
          // all peers' slots of an element are requested together and added in rank order once they are all there
          if (ok_lo)
            p.out_f32[(size_t)tok * p.out_ld + r_lo] =
                tp_recv_sum(tp, [&](int q) { return tp_ll_big_slot(tp, tp.rank, parity, q) + i_lo; }, tag, v_lo, res[nt][e], tp_alive);
          if (ok_hi)
            p.out_f32[(size_t)tok * p.out_ld + r_hi] =
                tp_recv_sum(tp, [&](int q) { return tp_ll_big_slot(tp, tp.rank, parity, q) + i_hi; }, tag, v_hi, res[nt][2 + e], tp_alive);
        }
      } else if (tok < p.T) {
        if (ok_lo) p.out_f32[(size_t)tok * p.out_ld + r_lo] = res[nt][e] + v_lo;
        if (ok_hi) p.out_f32[(size_t)tok * p.out_ld + r_hi] = res[nt][2 + e] + v_hi;
      }
    }
  }
  if (p.epi == 3) {
    // the last row-warp of the grid to finish moves the exchange counter on (every one has read it by then)
    __syncwarp();
    if (lane == 0) {
      __threadfence();
      const int prev = atomicAdd(tp.done_ctr, 1);
      if (prev == (int)gridDim.x * RW - 1) {
        *tp.done_ctr = 0;
        *tp.epoch = tp_epoch + 1;
        __threadfence();
      }
    }
  }
}

// One block per token: y = rmsnorm(x) * w (or a plain copy when w is null) as f16 in hmma-K order.
__global__ void norm_to_f16_hmma_kernel(const float* __restrict__ x, int x_ld, const float* __restrict__ w, float eps, int K,
                                        __half* __restrict__ out, int out_ld, int vec) {
  __shared__ float s32[32];
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const float* xr = x + (size_t)blockIdx.x * x_ld;
  __half* orow = out + (size_t)blockIdx.x * out_ld;
  if (vec) {
    norm_row_to_f16(xr, w, eps, K, orow, s32, [](int k) { return hmma_k_pos(k); });
    return;
  }
  float inv = 1.0f;
  if (w != nullptr) {
    float ss = 0.0f;
    for (int k = threadIdx.x; k < K; k += blockDim.x) ss += xr[k] * xr[k];
    ss = block_sum(ss, s32);
    inv = 1.0f / sqrtf(ss / (float)K + eps);
  }
  for (int k = threadIdx.x; k < K; k += blockDim.x) orow[hmma_k_pos(k)] = __float2half_rn(w ? w[k] * xr[k] * inv : xr[k]);
}

template <int NT>
static int launch_gh(const GhParams& p, const TpComm& tp, int grid, size_t smem, cudaStream_t st) {
  static bool configured[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return BONSAI_CUDA_LAUNCH_FAILED;
  if (!configured[dev]) {
    if (cudaFuncSetAttribute(bitgemm_hmma_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 2 * 4 * kGhChunk) != cudaSuccess)
      return BONSAI_CUDA_LAUNCH_FAILED;
    configured[dev] = true;
  }
  const cudaError_t e = launch_pdl(bitgemm_hmma_kernel<NT>, dim3(grid), dim3(kGhWarps * 32), smem, st, p, tp);
  return e == cudaSuccess ? BONSAI_CUDA_OK : BONSAI_CUDA_LAUNCH_FAILED;
}

}  // namespace bonsai

extern "C" {

// x_f16: activations [T][x_ld] f16 in hmma-K order (bonsai_norm_to_f16_hmma, or epi 2 of this kernel), T <= 64,
// K % 128 == 0.  epi 0: out_f32 = W x; 1: out_f32 = residual + W x; 2: out_f16 = SwiGLU over interleaved gate / up rows
// in hmma-K order (out_ld >= N / 2, N / 2 a multiple of 128 for a following GEMM).
static int bitgemm_hmma_launch(const void* codes, const void* scales, const void* x_f16, int x_ld, float* out_f32, const float* residual,
                               void* out_f16, int n_rows, int K, int T, int epi, int out_ld, const bonsai::TpComm& tp, cudaStream_t stream) {
  using namespace bonsai;
  if (K % 128 != 0 || K < 128 || n_rows < 1 || T < 1 || T > kGhMaxTok || epi < 0 || epi > 3 || x_ld % 8 != 0) return BONSAI_CUDA_BAD_ARG;
  if (epi == 3 && (out_f32 == nullptr || (size_t)T * n_rows > tp.lay.ll_big_elems)) return BONSAI_CUDA_BAD_ARG;
  if (((epi <= 1 || epi == 3) && out_f32 == nullptr) || (epi == 1 && residual == nullptr) || (epi == 2 && (out_f16 == nullptr || (n_rows & 1)))) return BONSAI_CUDA_BAD_ARG;
  const int tiles16 = (n_rows + 15) / 16, ng = K / 128;
  // k-warps per CTA: the fewest waves of (steps per k-warp + fixed cost), CTAs per SM bounded by the stage memory
  int best_kw = 1;
  long long best_cost = -1;
  for (int kwn = 1; kwn <= 4; kwn *= 2) {
    if (kwn > ng) break;
    const int rwn = kGhWarps / kwn;
    const long long ctas = (tiles16 + rwn - 1) / rwn;
    const long long per_sm = (220 * 1024) / (2 * kwn * kGhChunk);
    const long long slots = 148 * (per_sm < 1 ? 1 : per_sm);
    const long long waves = (ctas + slots - 1) / slots;
    const long long busy = ctas < 148 ? ctas : 148;
    const long long cost = waves * ((ng + kwn - 1) / kwn + 4) * 148 / busy;
    if (best_cost < 0 || cost < best_cost) {
      best_cost = cost;
      best_kw = kwn;
    }
  }
  const int KW = best_kw, RW = kGhWarps / KW;
  const int grid = (tiles16 + RW - 1) / RW;
  const size_t smem = (size_t)2 * KW * kGhChunk;
  GhParams p{(const uint32_t*)codes, (const __half*)scales, (const __half*)x_f16, out_f32, residual, (__half*)out_f16,
             n_rows, K, T, epi, x_ld, out_ld, KW};
  const int nt = (T + 7) / 8;
  if (epi == 3 && grid > 148) return BONSAI_CUDA_BAD_ARG;   // its CTAs wait on peers: all of them must be resident (one per SM at 130 registers)
  if (nt <= 2) return launch_gh<2>(p, tp, grid, smem, stream);
  if (nt <= 4) return launch_gh<4>(p, tp, grid, smem, stream);
  return launch_gh<8>(p, tp, grid, smem, stream);
}

int bonsai_bitgemm_hmma(const void* codes, const void* scales, const void* x_f16, int x_ld, float* out_f32, const float* residual,
                        void* out_f16, int n_rows, int K, int T, int epi, int out_ld, cudaStream_t stream) {
  if (epi == 3) return BONSAI_CUDA_BAD_ARG;
  return bitgemm_hmma_launch(codes, scales, x_f16, x_ld, out_f32, residual, out_f16, n_rows, K, T, epi, out_ld, bonsai::TpComm{}, stream);
}

// Row-parallel shard of a tensor-parallel group: out_f32[T][out_ld] = residual + sum over the ranks of `comm` of their
// W x, the exchange being part of the GEMM's epilogue ({value, tag} stores into the peers' memory).  Every rank
// launches the same call on its K shard; T * n_rows <= 64 * hidden.  residual may be null or alias out_f32.
int bonsai_bitgemm_hmma_tp(const void* comm, const void* codes, const void* scales, const void* x_f16, int x_ld, float* out_f32,
                           const float* residual, int n_rows, int K, int T, int out_ld, cudaStream_t stream) {
  if (comm == nullptr) return BONSAI_CUDA_BAD_ARG;
  return bitgemm_hmma_launch(codes, scales, x_f16, x_ld, out_f32, residual, nullptr, n_rows, K, T, 3, out_ld,
                             *static_cast<const bonsai::TpComm*>(comm), stream);
}

int bonsai_norm_to_f16_hmma(const float* x, int x_ld, const float* w, float eps, int T, int K, void* out, int out_ld, cudaStream_t stream) {
  if (T < 1 || K % 128 != 0) return BONSAI_CUDA_BAD_ARG;
  // one block per token: a block as wide as the row allows keeps the two passes short (few tokens = few blocks)
  const int threads = K >= 4096 ? 1024 : (K >= 2048 ? 512 : 256);
  const int vec = (x_ld % 4 == 0) && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) % 16 == 0);   // 16-byte loads
  const cudaError_t e = bonsai::launch_pdl(bonsai::norm_to_f16_hmma_kernel, dim3(T), dim3(threads), 0, stream, x, x_ld, w, eps, K, (__half*)out,
                                           out_ld, vec);
  return e == cudaSuccess ? BONSAI_CUDA_OK : BONSAI_CUDA_LAUNCH_FAILED;
}

}  // extern "C"
