// Prefill / batched-decode GEMM for packed ternary / 1-bit weights on the 5th-generation tensor cores.
//
//   out[t][n] = sum_k X[t][k] * W[n][k]        t < T tokens (one to thousands), n < N rows
//
// The reference's prefill kernels (gemm_q1_g128_v7, gemm_tq2_g128_v7, their _residual forms and
// fused_gate_up_swiglu_gemm_q1/_tq2; crates/oxibonsai-kernels/src/gpu_backend/cuda_prefill_kernels.rs:74-827)
// walk the batch eight columns at a time on CUDA cores and re-read the weights for every chunk.
// Here an output tile is 128 weight rows x TOK tokens (TOK = 256 for prompt chunks, 64 for decode batches):
//   * A operand (weights): sixteen expander warps in two groups of 256 threads; a thread owns one weight row of
//     the tile and one 64-input k-block of a pair (one 16-byte load).  Every two weights become a half2 with one
//     shift, one mask and one HMUL2 by the group scale (+-2^-7 * 128*d = +-d exactly, d being an f16), stored
//     into the 128-byte-swizzled shared-memory stage.  The groups take alternate pairs of k-blocks;
//   * B operand (activations): f16 tiles fetched by TMA (cp.async.bulk.tensor, no multicast);
//   * tcgen05.mma kind::f16 accumulates in TMEM (double buffered so the epilogue of one segment overlaps the main
//     loop of the next); 64-token tiles spread the MMA and TMA issue over four warps each, one per pipeline slot,
//     every MMA issuer with its own accumulator (the comments at the issuer loops give the measurements behind it);
//   * epilogue warps read TMEM back and store f32 (plain / residual add) or f16 (SwiGLU / plain) outputs.
//
// Work distribution ("stream-K"): the (tile, k-block pair) index space is cut into one contiguous, equally long
// range per CTA, so every SM streams the same number of weight bytes whatever the tile count (32 row tiles of a
// 4096-row projection still keep 148 SMs busy).  A tile whose K extent spans several CTAs is finished by the
// last of them to arrive: each writes its partial accumulator to a workspace slot, bumps the tile's counter, and
// the CTA that observes the final count adds the partials in CTA order (a fixed order: results do not depend on
// timing) and applies the epilogue.  Without a workspace every CTA gets whole tiles.
//
// K order: the expansion naturally yields the weights of a 16-input word in the order
// [0,4,1,5,2,6,3,7, 8,12,9,13,10,14,11,15]; instead of un-shuffling them the activation operand is
// kept in the same order ("paired-K" layout), which every producer of a prefill activation writes
// (norm_to_f16_paired_kernel, the SwiGLU epilogue here, the prefill attention output).
#include <cuda.h>
#include <cuda_fp16.h>

#include "common.cuh"
#include "tcgen05.cuh"

namespace bonsai {

constexpr int kPfGroups = 4;                          // expander warp quartets (128 rows x one k-block each)
constexpr int kPfAhead = 3;                           // 16-byte code loads each expander thread keeps in flight
constexpr int kPfABytes = 128 * 128;                  // 128 rows x 64 f16
constexpr int kPfExpThreads = 128 * kPfGroups;        // warps 0-15 expand
constexpr int kPfEpiWarp0 = kPfExpThreads / 32;       // warps 16-19: epilogue (TMEM lane quarter = warp & 3)
constexpr int kPfMmaWarp = kPfEpiWarp0 + 4;           // warps 20-23: MMA issuers (64-token tiles use all four, 256-token tiles one)
constexpr int kPfTmaWarp = kPfMmaWarp + 4;            // warps 24-27: TMA issuers (likewise)
constexpr int kPfThreads = kPfExpThreads + 128 + 256; // 896
constexpr int kPfCounterBytes = 64 * 1024;            // per-tile arrival counters at the head of the workspace
constexpr int kPfMaxCtas = 160;
constexpr int kPfPollNs = 100;                        // back-off between polls of producers waiting for a free stage

// position of logical input k inside its 16-element block in the paired-K layout
__host__ __device__ inline int paired_k(int k) {
  int j = k & 15, hi = j & 8, p = j & 3, q = (j >> 2) & 1;
  return (k & ~15) | hi | (p * 2 + q);
}

struct PfParams {
  const uint32_t* codes;
  const __half* scales;
  float* out_f32;          // [T][out_ld]  (epi 0, 1)
  const float* residual;   // [T][out_ld]  (epi 1)
  __half* out_f16;         // [T][out_ld]  (epi 2: SwiGLU, paired-K order; epi 3: plain f16 store)
  int* status;
  int n_rows, K, T, epi, out_ld;
  int dense;               // 1: A is a dense f16 matrix fetched by TMA (natural K order), no expansion
  int streamk;             // 1: ranges cut anywhere in (tile, pair) space, partial tiles meet in the workspace
  float* ws_part;          // [2 * grid][TOK][128] partial accumulators
  int* ws_count;           // [tiles] arrival counters, zero between launches
};


__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                   tc::smem_u32(dst)),
               "l"(map), "r"(x), "r"(y), "r"(tc::smem_u32(bar))
               : "memory");
}

// first flattened (tile, pair) index of CTA c
__device__ __forceinline__ long long pf_range_start(int streamk, int c, int grid, int ntiles, int npairs) {
  return streamk ? ((long long)c * ntiles * npairs) / grid : (((long long)c * ntiles) / grid) * (long long)npairs;
}

// codes (16 bytes = 64 inputs) of k-block hh of (tile row r, pair), and the pair's group scale
__device__ __forceinline__ void pf_fetch(const PfParams& p, int tile, int pair, int row_tiles, int r, int hh, uint4& cv, __half& sc) {
  const int row = (tile % row_tiles) * 128 + r;
  if (row < p.n_rows) {
    cv = __ldg(reinterpret_cast<const uint4*>(p.codes + (size_t)row * (p.K >> 4) + pair * 8) + hh);
    sc = p.scales[(size_t)row * (p.K >> 7) + pair];
  } else {
    cv = make_uint4(0, 0, 0, 0);
    sc = __float2half(0.0f);
  }
}

// 64 weights of row r (one 16-byte code vector) -> 64 f16 in the swizzled stage
__device__ __forceinline__ void pf_expand(uint8_t* stage, int r, const uint4& cur, __half2 d2) {
  const uint32_t w4[4] = {cur.x, cur.y, cur.z, cur.w};
#pragma unroll
  for (int wd = 0; wd < 4; ++wd) {
    const uint32_t w = w4[wd];
    uint32_t o[8];
#pragma unroll
    for (int pi = 0; pi < 4; ++pi) {
      uint32_t ma = (w << (12 - 4 * pi)) & 0xA000A000u;   // (a_p, a_{p+4}) as +-2^-7
      uint32_t mb = (w << (13 - 4 * pi)) & 0xA000A000u;   // (b_p, b_{p+4})
      __half2 ha = __hmul2(*reinterpret_cast<__half2*>(&ma), d2);
      __half2 hb = __hmul2(*reinterpret_cast<__half2*>(&mb), d2);
      o[pi] = *reinterpret_cast<uint32_t*>(&ha);
      o[4 + pi] = *reinterpret_cast<uint32_t*>(&hb);
    }
    // a word's 16 halves are two 16-byte chunks: chunk 2*wd (a pairs) and 2*wd+1 (b pairs)
    *reinterpret_cast<uint4*>(stage + tc::sw128_offset(r, 2 * wd)) = make_uint4(o[0], o[1], o[2], o[3]);
    *reinterpret_cast<uint4*>(stage + tc::sw128_offset(r, 2 * wd + 1)) = make_uint4(o[4], o[5], o[6], o[7]);
  }
}

// residual input of one output element (epi 1), 0 otherwise.  Callers load a block of these before storing the block:
// the output usually aliases the residual (h += W x), so inside a store loop the compiler has to order every load
// after the previous store and the loop becomes a chain of exposed memory latencies.
__device__ __forceinline__ float pf_residual(const PfParams& p, int tok, int row, bool row_ok) {
  return p.epi == 1 && row_ok && tok < p.T ? p.residual[(size_t)tok * p.out_ld + row] : 0.0f;
}

// epilogue for one accumulator value; every lane of the warp calls it (epi 2 exchanges gate / up between lanes)
__device__ __forceinline__ void pf_store(const PfParams& p, float v, float res, int tok, int row, int a, bool row_ok) {
  if (p.epi == 2) {
    float other = __shfl_xor_sync(0xffffffffu, v, 1);
    if (row_ok && tok < p.T && (a & 1) == 0)
      p.out_f16[(size_t)tok * p.out_ld + paired_k(row >> 1)] = __float2half_rn(v / (1.0f + __expf(-v)) * other);
  } else if (row_ok && tok < p.T) {
    const size_t o = (size_t)tok * p.out_ld + row;
    if (p.epi == 0) p.out_f32[o] = v;
    else if (p.epi == 1) p.out_f32[o] = res + v;
    else p.out_f16[o] = __float2half_rn(v);
  }
}

__device__ __forceinline__ void pf_epi_barrier() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// TOK = tokens per tile (MMA N): 256 for prompt chunks, 64 for batched decode / verification.
template <int TOK>
__global__ void __launch_bounds__(kPfThreads, 1) bitgemm_prefill_kernel(const __grid_constant__ CUtensorMap xmap,
                                                                     const __grid_constant__ CUtensorMap amap, PfParams p) {
  constexpr int S = TOK == 64 ? 8 : 4;   // pipeline stages (one 64-input k-block each)
  // Accumulators per tile.  Back-to-back tcgen05.mma into one accumulator form a dependent chain, and with only 64
  // columns each instruction is far shorter than the pipeline's latency (measured: ~190 cycles per instruction
  // whatever N).  The four K=16 steps of a k-block therefore go to four accumulators that the epilogue adds up.
  constexpr int NACC = TOK == 64 ? 4 : 1;
  constexpr int NISS = TOK == 64 ? 4 : 1;   // MMA issuer warps, and as many TMA issuer warps
  // Barrier granularity: GK k-blocks share one full / empty barrier (index (it / GK) % NBS, phase (it / GK) / NBS).
  constexpr int GK = TOK == 64 ? 2 : 1;
  constexpr int NBS = S / GK;
  constexpr int kAccCols = NACC * TOK;   // TMEM columns of one buffer; two buffers = 512 columns in both shapes
  constexpr int kPfBBytes = TOK * 128;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sA = base;
  uint8_t* sB = base + S * kPfABytes;
  __shared__ uint64_t full_bar[S], empty_bar[S], accf_bar[2], acce_bar[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int s_info[4];
  __shared__ int s_slots[kPfMaxCtas];
  __shared__ uint64_t red_bar;   // completion of the bulk copies that bring partial tiles in for the final reduction
  const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
  const int npairs = p.K >> 7;
  const int row_tiles = (p.n_rows + 127) >> 7, tok_tiles = (p.T + TOK - 1) / TOK;
  const int ntiles = row_tiles * tok_tiles;
  const int grid = gridDim.x;
  const long long I0 = pf_range_start(p.streamk, blockIdx.x, grid, ntiles, npairs);
  const int n = (int)(pf_range_start(p.streamk, blockIdx.x + 1, grid, ntiles, npairs) - I0);   // pairs of this CTA
  const int tile0 = (int)(I0 / npairs), pair0 = (int)(I0 - (long long)tile0 * npairs);

  // Programmatic dependent launch: this CTA may start while the previous kernel of the stream is still running.  Set-up,
  // TMEM allocation and the expanders' first weight loads depend on nothing it writes; the warps that touch its outputs
  // (activation copies, epilogue reads and writes, the work-split workspace) wait for it below.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (warp == kPfMmaWarp) {
    tc::tmem_alloc(&tmem_slot, 2 * kAccCols);
    tc::tmem_relinquish();
  }
  if (t == 0) {
    for (int i = 0; i < S; ++i) {
      tc::mbar_init(&full_bar[i], p.dense ? 1 : 4 * GK + 1);   // four expander warps per k-block + the TMA issuer's expect_tx arrival
      tc::mbar_init(&empty_bar[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      tc::mbar_init(&accf_bar[i], NISS);
      tc::mbar_init(&acce_bar[i], 4);
    }
    tc::mbar_init(&red_bar, 1);
    tc::mbar_fence_init();
  }
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t taddr = tmem_slot;
  bool failed = false;

  // Issuer warps run their loops with all 32 lanes (uniform control flow, every lane waits on the barriers) and elect
  // lane 0 only for the single-thread instructions.
  //
  // Measured cost model behind the role layout: each barrier / TMA / MMA / commit instruction occupies its issuing
  // thread for roughly 100-250 cycles whatever the operand size, so one thread that waits, issues four MMAs and
  // commits needs ~1000 cycles per 64-input k-block even when nothing it waits for is late.  A 256-token k-block
  // holds ~500 cycles of tensor work, which hides most of that; a 64-token k-block holds ~130.  64-token tiles
  // therefore (a) hand over a pair of k-blocks per barrier (one wait, one expect_tx, one commit per 128 inputs) and
  // (b) spread pairs over four MMA issuers and four TMA issuers: issuer m owns barrier stage m (pairs q with
  // q % 4 == m) and, for MMA, accumulator m, so the four instruction streams never touch the same TMEM columns and
  // the epilogue adds the accumulators that were written.
  if (warp >= kPfTmaWarp && warp < kPfTmaWarp + NISS) {
    // ------------------------------- TMA issuers (activations; dense weights) -------------------
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int tw = warp - kPfTmaWarp;
    int tile = tile0, pair = pair0;
    for (int q = 0; q < n && !failed; ++q) {
      if (NISS == 1 || (q % NISS) == tw) {
        const int tok0 = (tile / row_tiles) * TOK, row0 = (tile % row_tiles) * 128;
        for (int g0 = 0; g0 < 2 && !failed; g0 += GK) {   // one barrier per GK k-blocks
          const int it = 2 * q + g0, bs = (it / GK) % NBS;
          if (!__all_sync(0xffffffffu, tc::mbar_wait(&empty_bar[bs], (((it / GK) / NBS) & 1) ^ 1))) { failed = true; break; }
          if (lane == 0) {
            tc::mbar_arrive_expect_tx(&full_bar[bs], GK * (kPfBBytes + (p.dense ? kPfABytes : 0)));
#pragma unroll
            for (int h = 0; h < GK; ++h) {
              const int s = (it + h) % S, kb = 2 * pair + g0 + h;
              tma_load_2d(sB + s * kPfBBytes, &xmap, kb * 64, tok0, &full_bar[bs]);
              if (p.dense) tma_load_2d(sA + s * kPfABytes, &amap, kb * 64, row0, &full_bar[bs]);
            }
          }
          __syncwarp();
        }
      }
      if (++pair == npairs) { pair = 0; ++tile; }
    }
    if (failed && lane == 0) atomicExch(p.status, 1);
  } else if (warp >= kPfMmaWarp && warp < kPfMmaWarp + NISS) {
    // ------------------------------- MMA issuers ------------------------------------------------
    constexpr uint32_t idesc = tc::idesc_f32acc(tc::FMT_F16, tc::FMT_F16, 128, TOK);
    const int mw = warp - kPfMmaWarp;
    int pair = pair0, seg = 0;
    bool fresh = true;   // this issuer's next MMA starts its accumulator of the segment: overwrite instead of accumulate
    for (int q = 0; q < n && !failed; ++q) {
      const int ab = seg & 1;
      if (q == 0 || pair == 0) {   // a new segment: its accumulator buffer must have been drained
        if (!__all_sync(0xffffffffu, tc::mbar_wait(&acce_bar[ab], ((seg >> 1) & 1) ^ 1))) { failed = true; break; }
        tc::tc_fence_after();
        fresh = true;
      }
      if (NISS == 1 || (q % NISS) == mw) {
        for (int g0 = 0; g0 < 2 && !failed; g0 += GK) {
          const int it = 2 * q + g0, bs = (it / GK) % NBS;
          if (!__all_sync(0xffffffffu, tc::mbar_wait(&full_bar[bs], ((it / GK) / NBS) & 1))) { failed = true; break; }
          tc::tc_fence_after();
          if (lane == 0) {
#pragma unroll
            for (int h = 0; h < GK; ++h) {
              const int s = (it + h) % S;
              const uint64_t da = tc::smem_desc_sw128(tc::smem_u32(sA + s * kPfABytes));
              const uint64_t db = tc::smem_desc_sw128(tc::smem_u32(sB + s * kPfBBytes));
#pragma unroll
              for (uint32_t k = 0; k < 4; ++k)
                tc::mma_f16(taddr + ab * kAccCols + (NACC == 1 ? 0 : mw) * TOK, da + 2 * k, db + 2 * k, idesc,
                            !(fresh && h == 0 && k == 0));
              fresh = false;
            }
            tc::mma_commit(&empty_bar[bs]);
          }
          fresh = false;
          __syncwarp();
        }
      }
      if (failed) break;
      if (pair == npairs - 1 || q == n - 1) {   // end of the segment: every issuer reports its MMAs of it done
        if (lane == 0) {
          tc::mma_commit(&accf_bar[ab]);
        }
        __syncwarp();
        ++seg;
      }
      if (++pair == npairs) pair = 0;
    }
    if (failed && lane == 0) atomicExch(p.status, 1);
  } else if (warp < kPfEpiWarp0) {
    // ------------------------------- weight expanders (thread = weight row) ---------------------
    // Two pair-groups of 256 threads; group pg expands the pairs q with q % 2 == pg, thread (r, hh) of it the 64
    // inputs of k-block hh of weight row r.  Pair q lives in stages 2 * (q % (S/2)) and +1, so a group always refills
    // the stages it filled before (its wait on an empty barrier is then never more than one phase behind; a parity
    // wait two phases behind would pass at once).  With eight stages a group has two pairs of stages to alternate
    // between: it expands pair q + 2 while the tensor core consumes pair q.  Polls back off between tries: sixteen
    // warps polling back to back take issue slots from the issuer warps (measured: 232 vs 207 us for the 1024-token
    // gate/up GEMM); so does running the 256-token tile with a single group of 128 or 256 threads (241 / 229 us).
    constexpr int KH = 2;    // threads that share a weight row's pair of k-blocks
    constexpr int NPG = 2;   // pair-groups
    constexpr int NV = 2 / KH;               // 16-byte code vectors per thread and pair
    static_assert((S / 2) % NPG == 0, "a pair of stages is always refilled by the same group");
    if (!p.dense && warp < 4 * KH * NPG) {
      const int pg = warp / (4 * KH), hh0 = KH == 2 ? (warp >> 2) & 1 : 0, r = t & 127;
      // a thread's loads walk one weight row per tile: a dependent chain of cache misses unless several are in
      // flight, so the codes of kPfAhead of its pairs (NPG * kPfAhead pairs of the CTA) are requested ahead of use
      uint4 cv[kPfAhead][NV];
      __half sc[kPfAhead];
      int ftile = tile0, fpair = pair0 + pg;   // fetch cursor
      while (fpair >= npairs) { fpair -= npairs; ++ftile; }
#pragma unroll
      for (int j = 0; j < kPfAhead; ++j) {
#pragma unroll
        for (int v = 0; v < NV; ++v) cv[j][v] = make_uint4(0, 0, 0, 0);
        sc[j] = __float2half(0.0f);
        if (pg + j * NPG < n) {
#pragma unroll
          for (int v = 0; v < NV; ++v) pf_fetch(p, ftile, fpair, row_tiles, r, hh0 + v, cv[j][v], sc[j]);
        }
        fpair += NPG;
        while (fpair >= npairs) { fpair -= npairs; ++ftile; }
      }
      for (int q = pg; q < n && !failed; q += kPfAhead * NPG) {
#pragma unroll
        for (int j = 0; j < kPfAhead; ++j) {
          const int qq = q + j * NPG;
          if (qq < n && !failed) {   // guarded body rather than a break: the unrolled loop keeps the buffers in registers
            uint4 cur[NV];
#pragma unroll
            for (int v = 0; v < NV; ++v) cur[v] = cv[j][v];
            const __half2 d2 = __half2half2(__hmul(sc[j], __float2half(128.0f)));
            if (qq + kPfAhead * NPG < n) {
#pragma unroll
              for (int v = 0; v < NV; ++v) pf_fetch(p, ftile, fpair, row_tiles, r, hh0 + v, cv[j][v], sc[j]);
            }
            fpair += NPG;
            while (fpair >= npairs) { fpair -= npairs; ++ftile; }
#pragma unroll
            for (int v = 0; v < NV; ++v) {
              const int it = 2 * qq + hh0 + v, s = it % S, bs = (it / GK) % NBS;
              const uint32_t par = (((it / GK) / NBS) & 1) ^ 1;
              if (!failed && !tc::mbar_wait_sleep<kPfPollNs>(&empty_bar[bs], par)) failed = true;
              if (!failed) {
                pf_expand(sA + s * kPfABytes, r, cur[v], d2);
                tc::fence_proxy_async();
                __syncwarp();
                if (lane == 0) tc::mbar_arrive(&full_bar[bs]);
              }
            }
          }
        }
      }
      if (failed && lane == 0) atomicExch(p.status, 1);
    }
  } else if (warp < kPfMmaWarp) {
    // ------------------------------- epilogue (thread = weight row) ------------------------------
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int a = t - kPfExpThreads;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    int seg = 0;
    uint32_t red_phase = 0;
    for (int q = 0; q < n && !failed; ++seg) {
      const long long I = I0 + q;
      const int tile = (int)(I / npairs), pair_b = (int)(I - (long long)tile * npairs);
      const int len = min(n - q, npairs - pair_b);
      const bool whole = len == npairs;
      const int ab = seg & 1;
      const int row = (tile % row_tiles) * 128 + a;
      const int tok0 = (tile / row_tiles) * TOK;
      const bool row_ok = row < p.n_rows;
      const int ncols = min(TOK, p.T - tok0);
      float* part = p.ws_part + (size_t)(2 * blockIdx.x + (q == 0 ? 0 : 1)) * (128 * TOK);
      if (!tc::mbar_wait_warp<64>(&accf_bar[ab], (seg >> 1) & 1, lane)) { failed = true; break; }
      tc::tc_fence_after();
      constexpr int CB = 16;   // columns per step: accumulator block + second operand block + residual block in registers
#pragma unroll 1
      for (int c0 = 0; c0 < TOK; c0 += CB) {
        uint32_t rr[CB];
        if (NACC == 1) {
          tc::tmem_ld16(taddr + lane_base + ab * kAccCols + c0, rr);
          tc::tmem_wait_ld();
        } else {
#pragma unroll
          for (int j = 0; j < CB; ++j) rr[j] = 0u;
        }
#pragma unroll
        for (int acc = 0; acc < (NACC == 1 ? 0 : NACC); ++acc) {
          // issuer `acc` wrote its accumulator only if one of its pairs (q % NACC == acc) lies in this segment
          if (len < NACC && ((acc - q) & (NACC - 1)) >= len) continue;
          uint32_t r2[CB];
          tc::tmem_ld16(taddr + lane_base + ab * kAccCols + acc * TOK + c0, r2);
          tc::tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < CB; ++j) rr[j] = __float_as_uint(__uint_as_float(rr[j]) + __uint_as_float(r2[j]));
        }
        if (c0 >= ncols) continue;
        if (whole) {
          float res[CB];
#pragma unroll
          for (int j = 0; j < CB; ++j) res[j] = pf_residual(p, tok0 + c0 + j, row, row_ok);
#pragma unroll
          for (int j = 0; j < CB; ++j) pf_store(p, __uint_as_float(rr[j]), res[j], tok0 + c0 + j, row, a, row_ok);
        } else {
          // a slot is [TOK columns][128 rows]: a warp's store and the reducer's reads run along the rows
#pragma unroll
          for (int j = 0; j < CB; ++j)
            if (c0 + j < ncols) part[(c0 + j) * 128 + a] = __uint_as_float(rr[j]);
        }
      }
      tc::tc_fence_before();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(&acce_bar[ab]);
      if (!whole) {
        // the tile's K extent is shared with neighbouring CTAs: the last one to arrive sums the partials
        __threadfence();
        pf_epi_barrier();
        if (a == 0) {
          const long long X0 = (long long)tile * npairs, X1 = X0 + npairs - 1;
          const long long total = (long long)ntiles * npairs;
          int cf = (int)((X0 * grid) / total), cl = (int)((X1 * grid) / total);
          while (cf + 1 < grid && pf_range_start(1, cf + 1, grid, ntiles, npairs) <= X0) ++cf;
          while (cf > 0 && pf_range_start(1, cf, grid, ntiles, npairs) > X0) --cf;
          while (cl + 1 < grid && pf_range_start(1, cl + 1, grid, ntiles, npairs) <= X1) ++cl;
          while (cl > 0 && pf_range_start(1, cl, grid, ntiles, npairs) > X1) --cl;
          const int old = atomicAdd(&p.ws_count[tile], 1);
          s_info[0] = old == cl - cf ? 1 : 0;
          s_info[1] = cf;
          s_info[2] = cl;
        }
        pf_epi_barrier();
        if (s_info[0]) {
          const int cf = s_info[1], nc = s_info[2] - cf + 1;
          __threadfence();
          for (int i = a; i < nc; i += 128)
            s_slots[i] = 2 * (cf + i) + (pf_range_start(1, cf + i, grid, ntiles, npairs) >= (long long)tile * npairs ? 0 : 1);
          pf_epi_barrier();
          if (TOK == 64 && q + len == n) {
            // The CTA's last segment: its producers and MMAs are done, so the 192 KB of stage memory are idle.  One
            // thread pulls the partial tiles in with bulk copies (five 32 KB slots per round, the sixth holds the
            // running sum between rounds) and every thread adds its row from shared memory, contributors in CTA order.
            // Summing straight from global memory instead is a chain of exposed L2 latencies (measured 15 us here).
            float* stage = reinterpret_cast<float*>(base);
            float* carry = stage + 5 * (128 * TOK);
            for (int i0 = 0; i0 < nc && !failed; i0 += 5) {
              const int cnt = min(5, nc - i0);
              if (a == 0) {
                asm volatile("fence.proxy.async.global;" ::: "memory");   // the partials were written through the generic proxy
                tc::mbar_arrive_expect_tx(&red_bar, (uint32_t)(cnt * ncols * 128 * sizeof(float)));
                for (int i = 0; i < cnt; ++i)
                  tc::bulk_g2s(stage + i * (128 * TOK), p.ws_part + (size_t)s_slots[i0 + i] * (128 * TOK),
                               (uint32_t)(ncols * 128 * sizeof(float)), &red_bar);
              }
              // every thread polls the same barrier with the same limit, so they agree on the outcome
              const bool landed = tc::mbar_wait_sleep<32>(&red_bar, red_phase & 1);
              ++red_phase;
              const bool last = i0 + cnt >= nc;
              for (int cb = 0; cb < ncols && landed; cb += 8) {
                float v[8], res[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) res[j] = last ? pf_residual(p, tok0 + cb + j, row, row_ok) : 0.0f;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  const int c = cb + j < ncols ? cb + j : ncols - 1;
                  // all five slots are read unconditionally (independent loads; a slot beyond cnt holds stale but
                  // readable data) and the unused ones are dropped in the sum, which runs in CTA order
                  float x[5];
#pragma unroll
                  for (int i = 0; i < 5; ++i) x[i] = stage[i * (128 * TOK) + c * 128 + a];
                  v[j] = i0 == 0 ? 0.0f : carry[c * 128 + a];
#pragma unroll
                  for (int i = 0; i < 5; ++i) v[j] += i < cnt ? x[i] : 0.0f;
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  if (last) pf_store(p, v[j], res[j], tok0 + cb + j, row, a, row_ok && cb + j < ncols);
                  else if (cb + j < ncols) carry[(cb + j) * 128 + a] = v[j];
                }
              }
              pf_epi_barrier();   // every thread has read the slots before the next round overwrites them
              if (!landed) failed = true;
            }
          } else {
            for (int c = 0; c < ncols; ++c) {
              float v = 0.0f;
              for (int i = 0; i < nc; ++i) v += __ldcg(p.ws_part + (size_t)s_slots[i] * (128 * TOK) + c * 128 + a);
              pf_store(p, v, pf_residual(p, tok0 + c, row, row_ok), tok0 + c, row, a, row_ok);
            }
          }
          if (a == 0) p.ws_count[tile] = 0;
        }
        pf_epi_barrier();   // s_info / s_slots are free for the next segment
      }
      q += len;
    }
    if (failed && a == 0) atomicExch(p.status, 1);
  }
  tc::tc_fence_before();
  __syncthreads();
  if (warp == kPfMmaWarp) tc::tmem_dealloc(taddr, 2 * kAccCols);
}

// One block per token: y = rmsnorm(x) * w (or a plain copy when w is null), written as f16 in the
// paired-K order consumed by bitgemm_prefill.
__global__ void norm_to_f16_paired_kernel(const float* __restrict__ x, int x_ld, const float* __restrict__ w, float eps, int K,
                                          __half* __restrict__ out, int out_ld, int natural, int vec) {
  __shared__ float s32[32];
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int tok = blockIdx.x;
  const float* xr = x + (size_t)tok * x_ld;
  __half* orow = out + (size_t)tok * out_ld;
  if (vec) {
    if (natural) norm_row_to_f16(xr, w, eps, K, orow, s32, [](int k) { return k; });
    else norm_row_to_f16(xr, w, eps, K, orow, s32, [](int k) { return paired_k(k); });
    return;
  }
  float inv = 1.0f;
  if (w != nullptr) {
    float ss = 0.0f;
    for (int k = threadIdx.x; k < K; k += blockDim.x) ss += xr[k] * xr[k];
    ss = block_sum(ss, s32);
    inv = 1.0f / sqrtf(ss / (float)K + eps);
  }
  for (int k = threadIdx.x; k < K; k += blockDim.x) {
    float v = w ? w[k] * xr[k] * inv : xr[k];
    orow[natural ? k : paired_k(k)] = __float2half_rn(v);
  }
}

}  // namespace bonsai

static bool make_map_f16(CUtensorMap* map, const void* base, uint64_t inner, uint64_t outer, uint64_t ld_elems, uint32_t box_rows) {
  cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
  cuuint64_t strides[1] = {(cuuint64_t)ld_elems * 2};
  cuuint32_t box[2] = {64, box_rows};
  cuuint32_t estr[2] = {1, 1};
  return cuTensorMapEncodeTiled(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int TOK>
static int launch_prefill(const CUtensorMap& xmap, const CUtensorMap& amap, bonsai::PfParams p, int sms, void* ws, size_t ws_bytes,
                          int balance, cudaStream_t stream) {
  using namespace bonsai;
  constexpr int S = TOK == 64 ? 8 : 4;
  const long long ntiles = (long long)((p.n_rows + 127) / 128) * ((p.T + TOK - 1) / TOK);
  const long long total = ntiles * (p.K >> 7);
  if (total >= (1ll << 31)) return BONSAI_CUDA_BAD_ARG;
  if (sms > kPfMaxCtas) sms = kPfMaxCtas;
  if (sms < 1) sms = 1;
  // stream-K needs a counter per tile and two partial slots per CTA; otherwise CTAs take whole tiles.  Finishing a
  // shared tile costs every contributor a few microseconds (partial store, fence, counter) and the last one a
  // reduction, so the balanced split is taken where measurements show it pays: few tiles with a long K extent (the
  // down projection of a decode batch: 32 tiles x 192 k-blocks), or so many tiles that partial tiles are a small
  // fraction of the work (the LM head over a decode batch), or at most 32 tokens (partial tiles are then small).  256-token partial tiles (128 KB each) cost more than the
  // imbalance they remove.  balance: 0 = never, 1 = by this rule, 2 = whenever possible.
  int grid = (int)(total < sms ? total : sms);
  const size_t need = (size_t)kPfCounterBytes + (size_t)2 * grid * 128 * TOK * sizeof(float);
  const bool can = ws != nullptr && ws_bytes >= need && ntiles * (long long)sizeof(int) <= kPfCounterBytes && ntiles % grid != 0;
  const bool pays = TOK == 64 && ((ntiles < grid && (p.K >> 7) >= 64) || ntiles >= 4ll * grid || p.T <= 32);
  p.streamk = can && (balance == 2 || (balance == 1 && pays)) ? 1 : 0;
  if (!p.streamk) grid = (int)(ntiles < sms ? ntiles : sms);
  p.ws_count = static_cast<int*>(ws);
  p.ws_part = ws != nullptr ? reinterpret_cast<float*>(static_cast<char*>(ws) + kPfCounterBytes) : nullptr;
  size_t smem = 1024 + (size_t)S * (kPfABytes + TOK * 128);
  cudaError_t e = cudaFuncSetAttribute(bitgemm_prefill_kernel<TOK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return BONSAI_CUDA_LAUNCH_FAILED;
  e = launch_pdl(bitgemm_prefill_kernel<TOK>, dim3(grid), dim3(kPfThreads), smem, stream, xmap, amap, p);
  return e == cudaSuccess ? BONSAI_CUDA_OK : BONSAI_CUDA_LAUNCH_FAILED;
}

extern "C" {

// bytes of workspace that lets every shape this library launches use the balanced (stream-K) distribution
size_t bonsai_bitgemm_prefill_ws_bytes() {
  return (size_t)bonsai::kPfCounterBytes + (size_t)2 * bonsai::kPfMaxCtas * 128 * 256 * sizeof(float);
}

// x_f16: activations [T][K] f16 (row stride x_ld elements, 16-byte aligned rows), in paired-K order for packed
// weights and natural order for dense ones.
// epi 0: out_f32 = W x; 1: out_f32 = residual + W x; 2: out_f16 = SwiGLU over interleaved gate/up rows
// (paired-K order, out_ld = N/2 or more); 3: out_f16 = W x in natural order.
// dense_w != null: W is a dense f16 row-major [n_rows][K] matrix (codes / scales ignored), e.g. the LM head.
// ws / ws_bytes: optional workspace (zero-filled once by the caller, left zeroed by every launch; one launch at a
// time may use it) for the balanced work distribution; null = whole tiles per CTA.  balance: 0 = whole tiles, 1 = balanced
// where it is expected to pay, 2 = balanced whenever the workspace allows.
int bonsai_bitgemm_prefill_ws(const void* codes, const void* scales, const void* x_f16, int x_ld, float* out_f32,
                              const float* residual, void* out_f16, int* status, int n_rows, int K, int T, int epi, int out_ld,
                              int sms, const void* dense_w, void* ws, size_t ws_bytes, int balance, cudaStream_t stream) {
  using namespace bonsai;
  if (K % 128 != 0 || n_rows < 1 || T < 1 || epi < 0 || epi > 3 || x_ld % 8 != 0) return BONSAI_CUDA_BAD_ARG;
  if ((epi <= 1 && out_f32 == nullptr) || (epi == 1 && residual == nullptr) || (epi >= 2 && out_f16 == nullptr)) return BONSAI_CUDA_BAD_ARG;
  const int tok = T <= 64 ? 64 : 256;
  CUtensorMap xmap, amap;
  if (!make_map_f16(&xmap, x_f16, K, T, x_ld, tok)) return BONSAI_CUDA_BAD_ARG;
  if (dense_w != nullptr) {
    if (!make_map_f16(&amap, dense_w, K, n_rows, K, 128)) return BONSAI_CUDA_BAD_ARG;
  } else {
    amap = xmap;
  }
  PfParams p{(const uint32_t*)codes, (const __half*)scales, out_f32, residual, (__half*)out_f16, status, n_rows, K, T, epi, out_ld,
             dense_w != nullptr ? 1 : 0, 0, nullptr, nullptr};
  return tok == 64 ? launch_prefill<64>(xmap, amap, p, sms, ws, ws_bytes, balance, stream)
                   : launch_prefill<256>(xmap, amap, p, sms, ws, ws_bytes, balance, stream);
}

int bonsai_bitgemm_prefill(const void* codes, const void* scales, const void* x_f16, int x_ld, float* out_f32,
                           const float* residual, void* out_f16, int* status, int n_rows, int K, int T, int epi, int out_ld,
                           int sms, const void* dense_w, cudaStream_t stream) {
  return bonsai_bitgemm_prefill_ws(codes, scales, x_f16, x_ld, out_f32, residual, out_f16, status, n_rows, K, T, epi, out_ld, sms,
                                   dense_w, nullptr, 0, 0, stream);
}

int bonsai_norm_to_f16_paired(const float* x, int x_ld, const float* w, float eps, int T, int K, void* out, int out_ld, int natural,
                              cudaStream_t stream) {
  if (T < 1 || K % 16 != 0) return BONSAI_CUDA_BAD_ARG;
  // one block per token; with few tokens (decode batches) a wide block keeps the two passes short
  const int threads = T <= 128 ? (K >= 4096 ? 1024 : (K >= 2048 ? 512 : 256)) : 256;
  const int vec = (x_ld % 4 == 0) && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) % 16 == 0);   // 16-byte loads
  const cudaError_t e = bonsai::launch_pdl(bonsai::norm_to_f16_paired_kernel, dim3(T), dim3(threads), 0, stream, x, x_ld, w, eps, K, (__half*)out,
                                           out_ld, natural, vec);
  return e == cudaSuccess ? BONSAI_CUDA_OK : BONSAI_CUDA_LAUNCH_FAILED;
}

}  // extern "C"
