// Tensor-core decode GEMV/GEMM for packed ternary / 1-bit weights (tcgen05 + TMEM, sm_100a).
//
// out[t][n] = sum_k X[t][k] * W[n][k] for a handful of tokens t (batch-1 decode, small batches,
// speculative verification).  On CUDA cores this op costs ~3 instructions per weight and is
// ALU-bound far below the HBM roofline (see bitgemv.cu); here the 2-bit codes are widened to fp4
// (e2m1) with two mask/shift operations per SIXTEEN weights and multiplied on the tensor cores:
//
//   * A operand = 128 weight rows x 128 inputs of one scale group, e2m1 in the padded 4-bit shared
//     memory format of kind::f8f6f4 (16 elements in 8 bytes + 8 bytes of padding per 16-byte chunk),
//     written by the expander threads straight from registers: (w & 0xAAAAAAAA) and
//     ((w & 0x55555555) << 1) are the two 32-bit halves of a chunk (planar-SM layout, common.cuh);
//   * B operand = activations as e4m3 "terms": x ~ s * (t0 + t1/16 + t2/256 + ...), each term an
//     fp8 number, one MMA column per (token, term).  Products of {-1,0,+1} with fp8 values are exact
//     and accumulate in f32.  The terms are either built inside the kernel from f32 activations
//     (with the RMSNorm fused in) or read from tiles prepared by act_prep_fp8_kernel;
//   * one 128-input group is accumulated per TMEM buffer (4 MMAs of K = 32); the owning thread of
//     each weight row then drains the buffer with tcgen05.ld and applies that row's f16 group scale.
//
// The kernel is persistent: one CTA per SM column walks over row tiles of a fixed K slab, so TMEM,
// barriers and the activation operand are set up once per launch.  It is launched with
// programmatic dependent launch: everything that does not depend on the previous kernel (TMEM
// allocation, barrier init, zeroing the padding, prefetching and expanding the first weight
// groups) runs before griddepcontrol.wait and overlaps the predecessor's tail.
//
// Roles: warps 0-3 expand weights and drain accumulators (thread = weight row), warp 4 issues the
// MMAs, warps 5-8 build the activation operand.  K can be split over CTA columns; the last CTA to
// finish a row tile sums the partials in split order (deterministic) and applies the epilogue
// (store / residual add / SwiGLU over interleaved gate-up rows).
//
// This kernel supersedes, for decode, the reference's gemv_tq2_g128_v1, gemv_q1_g128_v7/_v8/_v9,
// their _residual forms, fused_gate_up_swiglu_q1 and rmsnorm_weighted_v2
// (crates/oxibonsai-kernels/src/gpu_backend/cuda_kernels.rs:76-776), none of which uses tensor cores.
#include <cuda_fp8.h>

#include <cstdlib>

#include "common.cuh"
#include "tcgen05.cuh"

namespace bonsai {

constexpr int kTcGS = 4;          // scale groups per super-step (one commit per super-step)
constexpr int kTcStages = 2;      // A-operand ring, each stage holds kTcGS groups = 64 KB
constexpr int kTcStageBytes = kTcGS * 16384;
constexpr int kTcThreads = 416;   // 8 expander warps, 4 operand-build/epilogue warps, 1 MMA warp
constexpr int kTcMmaWarp = 12;
constexpr int kTcMaxInKernelTokens = 4;

enum { TC_ERR_NONE = 0, TC_ERR_TIMEOUT = 1 };

struct TcGemvParams {
  const uint32_t* codes;   // planar SM [N_rows][K/16]
  const __half* scales;    // [N_rows][K/128]
  const uint8_t* xq;       // prepared activations [K/128][ncols][128 B] (null: build from x)
  const float* colscale;   // [ncols] factor of each MMA column (with xq)
  const float* x;          // f32 activations [T][x_ld] (in-kernel operand build)
  const float* norm_w;     // optional RMSNorm weight [K]
  float* out;              // [T][out_ld]
  const float* residual;   // [T][out_ld] or null
  float* partial;          // [ksplit][T][N_rows] workspace (ksplit > 1)
  int* counters;           // [row tiles] arrival counters (ksplit > 1), zero between launches
  int* status;             // error word
  float eps;
  int n_rows, K, T, nterms, ncols, ksplit, epi, out_ld, x_ld;
  int dbg;  // experiment switches (0 in production)
  long long* ts;  // optional timestamp trace of CTA 0 (null in production)
};

__device__ __forceinline__ uint8_t to_e4m3(float v, float* back) {
  __nv_fp8_storage_t q = __nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
  *back = __half2float(__half(__nv_cvt_fp8_to_halfraw(q, __NV_E4M3)));
  return (uint8_t)q;
}

#define TC_TS(id)                                                                  \
  do {                                                                             \
    if (p.ts != nullptr && blockIdx.x == 0 && (threadIdx.x & 31) == 0) {           \
      int _i = atomicAdd((int*)p.ts, 1);                                           \
      if (_i < 4000) { p.ts[1 + 2 * _i] = (id); p.ts[2 + 2 * _i] = clock64(); }    \
    }                                                                              \
  } while (0)

template <int NCOLS>
__global__ void __launch_bounds__(kTcThreads) bitgemv_tc_kernel(TcGemvParams p) {
  // accumulator ring: each super-step owns kTcGS column blocks of NCOLS columns
  constexpr int kRing = (512 / (kTcGS * NCOLS)) < 4 ? (512 / (kTcGS * NCOLS)) : 4;
  constexpr uint32_t kTmemCols = kRing * kTcGS * NCOLS;   // 256 (NCOLS 16) or 512
  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sA = base;                                  // kTcStages x 64 KB
  uint8_t* sB = base + kTcStages * kTcStageBytes;      // groups_local x NCOLS x 128 B
  __shared__ uint64_t full_bar[kTcStages], done_bar[4], accfree_bar[4], b_bar;
  __shared__ uint32_t tmem_slot;
  __shared__ int s_last;
  __shared__ float s_colscale[64];
  __shared__ float s_red[2][kTcMaxInKernelTokens][4];

  const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
  const int split = blockIdx.x % p.ksplit, col_id = blockIdx.x / p.ksplit, ncolumns = gridDim.x / p.ksplit;
  const int ngroups = p.K >> 7;
  const int gps = (ngroups + p.ksplit - 1) / p.ksplit;
  const int g0 = split * gps, g1 = min(ngroups, g0 + gps);
  const int ng = max(0, g1 - g0);
  const int nss = (ng + kTcGS - 1) / kTcGS;            // super-steps per tile
  const int ntiles = (p.n_rows + 127) >> 7;
  const int my_tiles = col_id < ntiles ? (ntiles - col_id + ncolumns - 1) / ncolumns : 0;
  const int total = my_tiles * nss;                    // super-steps this CTA executes
  const bool build_b = p.xq == nullptr;

  // Allow the next kernel in the stream to start its own prologue right away; it blocks in its
  // griddepcontrol.wait until this grid has completed and flushed.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  TC_TS(1000 + warp);

  if (warp == kTcMmaWarp) {
    tc::tmem_alloc(&tmem_slot, kTmemCols);
    tc::tmem_relinquish();
  }
  if (t == 0) {
    for (int i = 0; i < kTcStages; ++i) tc::mbar_init(&full_bar[i], 8);   // one arrival per expander warp
    for (int i = 0; i < 4; ++i) {
      tc::mbar_init(&done_bar[i], 1);                                      // tcgen05.commit
      tc::mbar_init(&accfree_bar[i], 4);                                   // one arrival per epilogue warp
    }
    tc::mbar_init(&b_bar, build_b ? 4 : 1);
    tc::mbar_fence_init();
  }
  // padding halves of the A chunks and unused activation columns must hold zeros
  {
    const int nvec = (kTcStages * kTcStageBytes + (build_b ? ng * NCOLS * 128 : 0)) / 16;
    for (int i = t; i < nvec; i += kTcThreads) reinterpret_cast<uint4*>(sA)[i] = make_uint4(0, 0, 0, 0);
  }
  tc::fence_proxy_async();
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t taddr = tmem_slot;
  bool failed = false;
  TC_TS(2000 + warp);

  if (warp == kTcMmaWarp) {
    // ------------------------------- MMA issuer ------------------------------------------------
    if (lane == 0 && total > 0) {
      if (!build_b) {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        tc::mbar_arrive_expect_tx(&b_bar, (uint32_t)ng * NCOLS * 128);
        for (int g = 0; g < ng; ++g)
          tc::bulk_g2s(sB + (size_t)g * NCOLS * 128, p.xq + (size_t)(g0 + g) * NCOLS * 128, NCOLS * 128, &b_bar);
      }
      TC_TS(3000);
      if (!tc::mbar_wait(&b_bar, 0)) failed = true;
      TC_TS(3001);
      constexpr uint32_t idesc = tc::idesc_f32acc(tc::FMT_E2M1, tc::FMT_E4M3, 128, NCOLS);
      for (int it = 0; it < total && !failed; ++it) {
        const int ssl = it % nss;                       // super-step within the tile
        const int s = it % kTcStages, ab = it % kRing;
        const int gcount = min(kTcGS, ng - ssl * kTcGS);
        if (!tc::mbar_wait(&full_bar[s], (it / kTcStages) & 1)) { failed = true; break; }
        if (!tc::mbar_wait(&accfree_bar[ab], ((it / kRing) & 1) ^ 1)) { failed = true; break; }
        tc::tc_fence_after();
        if (!(p.dbg & 4)) {
          for (int gi = 0; gi < gcount; ++gi) {
            const uint64_t da = tc::smem_desc_sw128(tc::smem_u32(sA + s * kTcStageBytes + gi * 16384));
            const uint64_t db = tc::smem_desc_sw128(tc::smem_u32(sB + (size_t)(ssl * kTcGS + gi) * NCOLS * 128));
            const uint32_t d = taddr + (ab * kTcGS + gi) * NCOLS;
#pragma unroll
            for (uint32_t k = 0; k < 4; ++k) tc::mma_f8f6f4(d, da + 2 * k, db + 2 * k, idesc, k);
          }
        }
        // a single commit per super-step: it frees the A stage for the expanders and publishes the
        // accumulator blocks to the epilogue
        tc::mma_commit(&done_bar[it & 3]);
        TC_TS(4000 + it);
      }
      if (failed) atomicExch(p.status, TC_ERR_TIMEOUT);
    }
  } else if (warp < 8) {
    // ------------------------------- weight expanders ------------------------------------------
    // thread = (weight row r, half h): it widens groups 2h and 2h+1 of every super-step
    const int r = t & 127, h = t >> 7;
    const int words_per_row = p.K >> 4;
    auto load_ss = [&](int it, uint4* q) {
      const int row = (col_id + (it / nss) * ncolumns) * 128 + r;
      const int gl = (it % nss) * kTcGS + 2 * h;        // first local group of this thread
      const bool ok = it < total && row < p.n_rows && !(p.dbg & 16);
      const uint4* wp = reinterpret_cast<const uint4*>(p.codes + (size_t)(ok ? row : 0) * words_per_row) + (size_t)(g0 + gl) * 2;
#pragma unroll
      for (int j = 0; j < 4; ++j) q[j] = (ok && gl + (j >> 1) < ng) ? __ldg(wp + j) : make_uint4(0, 0, 0, 0);
    };
    uint4 cur[4], nxt[4];
    load_ss(0, cur);
    load_ss(1, nxt);
    for (int it = 0; it < total && !failed; ++it) {
      const int s = it % kTcStages;
      // the stage is free once the commit of the super-step that last used it has landed
      if (it >= kTcStages && !tc::mbar_wait(&done_bar[(it - kTcStages) & 3], ((it - kTcStages) >> 2) & 1)) { failed = true; break; }
      uint8_t* stage = sA + s * kTcStageBytes + (2 * h) * 16384;
      if (!(p.dbg & 8)) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint32_t w[4] = {cur[j].x, cur[j].y, cur[j].z, cur[j].w};
          uint8_t* gbase = stage + (j >> 1) * 16384;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint2 v = make_uint2(w[c] & 0xAAAAAAAAu, (w[c] & 0x55555555u) << 1);
            *reinterpret_cast<uint2*>(gbase + tc::sw128_offset(r, (j & 1) * 4 + c)) = v;
          }
        }
      }
      tc::fence_proxy_async();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(&full_bar[s]);
      if (warp == 0) TC_TS(5000 + it);
#pragma unroll
      for (int j = 0; j < 4; ++j) cur[j] = nxt[j];
      load_ss(it + 2, nxt);
    }
    if (failed && t == 0) atomicExch(p.status, TC_ERR_TIMEOUT);
  } else {
    // ------------------------------- operand build, then drain + epilogue ----------------------
    const int a = t - 256;  // 0..127 = weight row within the tile
    if (build_b && total > 0) {
      asm volatile("griddepcontrol.wait;" ::: "memory");
      const int T = p.T, NT = p.nterms, K = p.K;
      float ss[kTcMaxInKernelTokens], mx[kTcMaxInKernelTokens];
#pragma unroll
      for (int tk = 0; tk < kTcMaxInKernelTokens; ++tk) { ss[tk] = 0.0f; mx[tk] = 0.0f; }
      for (int k = a * 4; k < K; k += 512) {
        float4 w = p.norm_w ? *reinterpret_cast<const float4*>(p.norm_w + k) : make_float4(1.f, 1.f, 1.f, 1.f);
#pragma unroll
        for (int tk = 0; tk < kTcMaxInKernelTokens; ++tk) {
          if (tk < T) {
            float4 v = *reinterpret_cast<const float4*>(p.x + (size_t)tk * p.x_ld + k);
            ss[tk] += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
            mx[tk] = fmaxf(mx[tk], fmaxf(fmaxf(fabsf(w.x * v.x), fabsf(w.y * v.y)), fmaxf(fabsf(w.z * v.z), fabsf(w.w * v.w))));
          }
        }
      }
#pragma unroll
      for (int tk = 0; tk < kTcMaxInKernelTokens; ++tk) {
        ss[tk] = warp_sum(ss[tk]);
        mx[tk] = warp_max(mx[tk]);
        if (lane == 0) { s_red[0][tk][warp - 8] = ss[tk]; s_red[1][tk][warp - 8] = mx[tk]; }
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      float inv[kTcMaxInKernelTokens], rs[kTcMaxInKernelTokens];
#pragma unroll
      for (int tk = 0; tk < kTcMaxInKernelTokens; ++tk) {
        float s_sum = s_red[0][tk][0] + s_red[0][tk][1] + s_red[0][tk][2] + s_red[0][tk][3];
        float m = fmaxf(fmaxf(s_red[1][tk][0], s_red[1][tk][1]), fmaxf(s_red[1][tk][2], s_red[1][tk][3]));
        inv[tk] = p.norm_w ? 1.0f / sqrtf(s_sum / (float)K + p.eps) : 1.0f;
        float amax = m * inv[tk];
        float sc = (tk < T && amax > 0.0f) ? amax * (1.0f / 256.0f) : 1.0f;
        rs[tk] = 1.0f / sc;
        if (a < NT && tk < T) s_colscale[tk * NT + a] = sc * exp2f(-4.0f * (float)a);
      }
      const int k_lo = g0 * 128, k_hi = g1 * 128;
      for (int k = k_lo + a; k < k_hi; k += 128) {
        const int gl = (k - k_lo) >> 7, kk = k & 127;
        const float w = p.norm_w ? p.norm_w[k] : 1.0f;
        uint8_t* tile = sB + (size_t)gl * NCOLS * 128;
#pragma unroll
        for (int tk = 0; tk < kTcMaxInKernelTokens; ++tk) {
          if (tk < T) {
            float v = w * p.x[(size_t)tk * p.x_ld + k] * inv[tk] * rs[tk];
            for (int term = 0; term < NT; ++term) {
              float back;
              uint8_t q = to_e4m3(v, &back);
              tile[tc::sw128_offset(tk * NT + term, kk >> 4) + (kk & 15)] = q;
              v = (v - back) * 16.0f;
            }
          }
        }
      }
      tc::fence_proxy_async();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(&b_bar);
    }

    float acc[NCOLS];
#pragma unroll
    for (int c = 0; c < NCOLS; ++c) acc[c] = 0.0f;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    bool waited_dep = build_b;
    // group scales of this thread's row for one super-step: kTcGS consecutive f16 values
    auto load_scales = [&](int it) -> uint2 {
      const int row = (col_id + (it / nss) * ncolumns) * 128 + a;
      const int gl = (it % nss) * kTcGS;
      if (it >= total || row >= p.n_rows || (p.dbg & 1)) return make_uint2(0, 0);
      const __half* sp = p.scales + (size_t)row * ngroups + g0 + gl;
      if (gl + kTcGS <= ng && ((g0 + gl) & 3) == 0 && (ngroups & 3) == 0) return *reinterpret_cast<const uint2*>(sp);
      __half hv[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) hv[j] = (gl + j < ng) ? sp[j] : __float2half(0.0f);
      return *reinterpret_cast<uint2*>(hv);
    };
    uint2 sc_cur = load_scales(0);
    for (int it = 0; it < total && !failed; ++it) {
      const uint2 sc_nxt = load_scales(it + 1);
      const int ab = it % kRing;
      if (!tc::mbar_wait(&done_bar[it & 3], (it >> 2) & 1)) { failed = true; break; }
      tc::tc_fence_after();
      const int ssl = it % nss;
      const int tile_idx = col_id + (it / nss) * ncolumns;
      const int row = tile_idx * 128 + a;
      const bool row_ok = row < p.n_rows;
      const int gcount = min(kTcGS, ng - ssl * kTcGS);
      const __half2 s01 = *reinterpret_cast<const __half2*>(&sc_cur.x), s23 = *reinterpret_cast<const __half2*>(&sc_cur.y);
      const float dsc[4] = {__low2float(s01), __high2float(s01), __low2float(s23), __high2float(s23)};
      if (!(p.dbg & 2)) {
#pragma unroll
        for (int gi = 0; gi < kTcGS; ++gi) {
          if (gi < gcount) {
#pragma unroll
            for (int c0 = 0; c0 < NCOLS; c0 += 16) {
              uint32_t rr[16];
              tc::tmem_ld16(taddr + lane_base + (ab * kTcGS + gi) * NCOLS + c0, rr);
              tc::tmem_wait_ld();
#pragma unroll
              for (int j = 0; j < 16; ++j) acc[c0 + j] = fmaf(dsc[gi], __uint_as_float(rr[j]), acc[c0 + j]);
            }
          }
        }
      }
      tc::tc_fence_before();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(&accfree_bar[ab]);
      if (warp == 8) TC_TS(6000 + it);
      sc_cur = sc_nxt;
      if (ssl != nss - 1) continue;

      // ---- tile finished: combine the term columns, split-K fix-up, epilogue ----
      if (!waited_dep) {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        waited_dep = true;
      }
      const int T = p.T, NT = p.nterms;
      const float* cs = build_b ? s_colscale : p.colscale;
      for (int tok = 0; tok < T; ++tok) {
        float v = 0.0f;
#pragma unroll
        for (int c = 0; c < NCOLS; ++c)
          if (c >= tok * NT && c < (tok + 1) * NT) v = fmaf(cs[c], acc[c], v);
        if (p.ksplit > 1) {
          if (row_ok) p.partial[((size_t)split * T + tok) * p.n_rows + row] = v;
        } else if (p.epi == 2) {
          float other = __shfl_xor_sync(0xffffffffu, v, 1);
          if (row_ok && (a & 1) == 0) p.out[(size_t)tok * p.out_ld + (row >> 1)] = v / (1.0f + __expf(-v)) * other;
        } else if (row_ok) {
          size_t o = (size_t)tok * p.out_ld + row;
          p.out[o] = p.epi == 1 ? p.residual[o] + v : v;
        }
      }
#pragma unroll
      for (int c = 0; c < NCOLS; ++c) acc[c] = 0.0f;
      if (p.ksplit > 1) {
        // the last CTA to arrive for this row tile reduces the partials in split order
        __threadfence();
        asm volatile("bar.sync 2, 128;" ::: "memory");
        if (a == 0) {
          int prev = atomicAdd(p.counters + tile_idx, 1);
          s_last = (prev == p.ksplit - 1);
          if (s_last) p.counters[tile_idx] = 0;
        }
        asm volatile("bar.sync 2, 128;" ::: "memory");
        if (s_last) {
          __threadfence();
          for (int tok = 0; tok < T; ++tok) {
            float v = 0.0f;
            if (row_ok)
              for (int s = 0; s < p.ksplit; ++s) v += __ldcg(p.partial + ((size_t)s * T + tok) * p.n_rows + row);
            if (p.epi == 2) {
              float other = __shfl_xor_sync(0xffffffffu, v, 1);
              if (row_ok && (a & 1) == 0) p.out[(size_t)tok * p.out_ld + (row >> 1)] = v / (1.0f + __expf(-v)) * other;
            } else if (row_ok) {
              size_t o = (size_t)tok * p.out_ld + row;
              p.out[o] = p.epi == 1 ? p.residual[o] + v : v;
            }
          }
        }
        asm volatile("bar.sync 2, 128;" ::: "memory");
      }
      if (warp == 8) TC_TS(7000 + it);
    }
    if (failed && a == 0) atomicExch(p.status, TC_ERR_TIMEOUT);
  }

  TC_TS(8000 + warp);
  tc::tc_fence_before();
  __syncthreads();
  if (warp == kTcMmaWarp) tc::tmem_dealloc(taddr, kTmemCols);
  TC_TS(9000 + warp);
}

// One block per token: optional RMSNorm, then split x into e4m3 terms and write the swizzled B tiles.
// xq layout: [K/128][ncols][128 B]; column of (token, term) = token * nterms + term.
__global__ void __launch_bounds__(256) act_prep_fp8_kernel(const float* __restrict__ x, int x_ld, const float* __restrict__ norm_w,
                                                          float eps, int K, int nterms, int ncols, uint8_t* __restrict__ xq,
                                                          float* __restrict__ colscale) {
  __shared__ float s32[32];
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int tok = blockIdx.x, t = threadIdx.x;
  const float* xr = x + (size_t)tok * x_ld;
  float ss = 0.0f, amax = 0.0f;
  for (int k = t; k < K; k += blockDim.x) {
    float v = xr[k];
    ss += v * v;
    amax = fmaxf(amax, fabsf(norm_w ? norm_w[k] * v : v));
  }
  float inv = 1.0f;
  if (norm_w != nullptr) {
    ss = block_sum(ss, s32);
    inv = 1.0f / sqrtf(ss / (float)K + eps);
  }
  amax = warp_max(amax);
  __syncthreads();
  if ((t & 31) == 0) s32[t >> 5] = amax;
  __syncthreads();
  amax = 0.0f;
  for (int w = 0; w < (blockDim.x >> 5); ++w) amax = fmaxf(amax, s32[w]);
  amax *= inv;
  const float s = amax > 0.0f ? amax * (1.0f / 256.0f) : 1.0f;
  const float rs = 1.0f / s;
  for (int k = t; k < K; k += blockDim.x) {
    float v = (norm_w ? norm_w[k] : 1.0f) * xr[k] * inv * rs;
    const int g = k >> 7, kk = k & 127;
    for (int term = 0; term < nterms; ++term) {
      float back;
      uint8_t q = to_e4m3(v, &back);
      const int col = tok * nterms + term;
      xq[(size_t)g * ncols * 128 + tc::sw128_offset(col, kk >> 4) + (kk & 15)] = q;
      v = (v - back) * 16.0f;
    }
  }
  if (t < nterms) colscale[tok * nterms + t] = s * exp2f(-4.0f * (float)t);
}

}  // namespace bonsai

extern "C" {

// Quantises T rows of x (f32, leading dimension x_ld) into the fp8-term operand consumed by
// bonsai_bitgemv_tc.  xq must hold (K/128)*ncols*128 bytes and be zero in the unused columns;
// colscale holds ncols floats.  ncols = multiple of 16 >= T*nterms, at most 64.
int bonsai_act_prep_fp8(const float* x, int x_ld, const float* norm_w, float eps, int T, int K, int nterms, int ncols, void* xq,
                        float* colscale, cudaStream_t stream) {
  if (K % 128 != 0 || T < 1 || nterms < 1 || nterms > 4 || T * nterms > ncols || ncols % 16 != 0 || ncols > 64) return BONSAI_CUDA_BAD_ARG;
  cudaError_t e = bonsai::launch_pdl(bonsai::act_prep_fp8_kernel, dim3(T), dim3(256), 0, stream, x, x_ld, norm_w, eps, K, nterms, ncols,
                                     (uint8_t*)xq, colscale);
  return e == cudaSuccess ? BONSAI_CUDA_OK : BONSAI_CUDA_LAUNCH_FAILED;
}

// out[T][out_ld] = epilogue(W x) on the tensor cores.
//   xq / colscale : operand prepared by bonsai_act_prep_fp8, or null to build it in the kernel from
//                   x (f32 [T][x_ld], T <= 4) with an optional fused RMSNorm (norm_w, eps);
//   partial       : ksplit*T*n_rows floats, counters: ceil(n_rows/128) zeroed ints (ksplit > 1);
//   *status       : set non-zero if a bounded wait expired;
//   sms           : number of SMs to spread over (grid = largest multiple of ksplit <= sms).
int bonsai_bitgemv_tc(const void* codes, const void* scales, const void* xq, const float* colscale, const float* x, int x_ld,
                      const float* norm_w, float eps, float* out, const float* residual, float* partial, int* counters, int* status,
                      int n_rows, int K, int T, int nterms, int ncols, int ksplit, int epi, int out_ld, int sms,
                      cudaStream_t stream) {
  using namespace bonsai;
  if (K % 128 != 0 || n_rows < 1 || T < 1 || nterms < 1 || nterms > 4 || T * nterms > ncols ||
      (ncols != 16 && ncols != 32 && ncols != 64) || ksplit < 1 || epi < 0 || epi > 2 || sms < 1)
    return BONSAI_CUDA_BAD_ARG;
  if (epi == 1 && residual == nullptr) return BONSAI_CUDA_BAD_ARG;
  if (xq == nullptr && (x == nullptr || T > kTcMaxInKernelTokens || K % 512 != 0)) return BONSAI_CUDA_BAD_ARG;
  if (xq != nullptr && colscale == nullptr) return BONSAI_CUDA_BAD_ARG;
  const int ngroups = K / 128;
  if (ksplit > ngroups) ksplit = ngroups;
  if (ksplit > 1 && (partial == nullptr || counters == nullptr)) return BONSAI_CUDA_BAD_ARG;
  const int gps = (ngroups + ksplit - 1) / ksplit;
  ksplit = (ngroups + gps - 1) / gps;   // no empty K slab: every CTA of a tile must arrive at its counter
  const int ntiles = (n_rows + 127) / 128;
  int columns = sms / ksplit;
  if (columns < 1) columns = 1;
  if (columns > ntiles) columns = ntiles;
  TcGemvParams p{(const uint32_t*)codes, (const __half*)scales, (const uint8_t*)xq, colscale, x, norm_w, out, residual, partial,
                 counters, status, eps, n_rows, K, T, nterms, ncols, ksplit, epi, out_ld, x_ld, 0, nullptr};
  if (const char* dv = getenv("BONSAI_TC_DBG")) p.dbg = atoi(dv);
  if (const char* tv = getenv("BONSAI_TC_TS")) p.ts = (long long*)strtoull(tv, nullptr, 0);
  dim3 grid(columns * ksplit);
  size_t smem = 1024 + (size_t)kTcStages * kTcStageBytes + (size_t)gps * ncols * 128;
  if (smem > 220 * 1024) return BONSAI_CUDA_BAD_ARG;
  cudaError_t e;
  switch (ncols) {
    case 16:
      e = cudaFuncSetAttribute(bitgemv_tc_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e == cudaSuccess) { bitgemv_tc_kernel<16><<<grid, kTcThreads, smem, stream>>>(p); e = cudaGetLastError(); }
      break;
    case 32:
      e = cudaFuncSetAttribute(bitgemv_tc_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e == cudaSuccess) { bitgemv_tc_kernel<32><<<grid, kTcThreads, smem, stream>>>(p); e = cudaGetLastError(); }
      break;
    default:
      e = cudaFuncSetAttribute(bitgemv_tc_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e == cudaSuccess) { bitgemv_tc_kernel<64><<<grid, kTcThreads, smem, stream>>>(p); e = cudaGetLastError(); }
      break;
  }
  return e == cudaSuccess ? BONSAI_CUDA_OK : BONSAI_CUDA_LAUNCH_FAILED;
}

}  // extern "C"
