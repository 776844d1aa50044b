// Batch-1 decode GEMV that streams packed weights through shared memory with bulk async copies and multiplies on
// the warp-level f16 tensor cores with a one-instruction weight decode.
//
// Why another GEMV: the planar-layout kernels (bitgemv_warp.cu, bitgemv_hmma.cu) spend ~2.5 thread instructions per
// weight on shift + mask + FMA and hold their loads in registers, which leaves them issue- and latency-bound at a
// quarter of the memory roofline.  Here
//   * weights live in the "S16" layout: tiles of 16 output rows, one 544-byte block per (tile, 128-input group) =
//     32 lanes x 16 bytes of 2-bit codes in MMA-fragment order + 16 f16 group scales.  A CTA owns a contiguous range
//     of tiles, i.e. one contiguous byte range of the matrix, and a producer lane streams it into a shared-memory
//     ring with cp.async.bulk (by default four stages of 17 KB: 70 KB in flight per SM).  The copies are issued before
//     griddepcontrol.wait: under programmatic dependent launch the next GEMV's weights stream in while the previous
//     kernel is still running;
//   * a code c = w + 1 in {0, 1, 2} sitting at bits p, p+1 of a 16-bit half becomes the f16 number 2^(10-p) + c with
//     one LOP3: (word & mask) | magic, where magic is the exponent pattern of 2^(10-p) and the code lands in the
//     mantissa.  Two codes (both halves of a word) per instruction, no sign handling, no conversion.  Three shifted
//     views of a word (x << 6, x, x >> 6) bring its eight code slots to p in {4, 6, 8}, so the offsets are 64, 16, 4;
//   * mma.sync.m16n8k16 multiplies the offset weights with the f16 activations and accumulates in f32; the offset
//     part, sum_k (2^(10-p(k)) + 1) x_k, is the same for every row, is computed once per 128-input group in the
//     prologue and subtracted before the group's f16 scale is applied in f32;
//   * sixteen consumer warps take two blocks each per stage, keep per-tile partial sums in registers and meet in
//     shared memory once at the end; partials are added in warp order, so results do not depend on timing.
// That is ~0.95 thread instructions per weight (0.5 LOP3, 0.125 shift, 0.125 MMA, the rest loads and bookkeeping).
//
// Epilogues: store, residual add, SwiGLU over interleaved gate/up rows, and the tensor-parallel one: every finished
// row goes to all peers as one 8-byte {value, tag} store and the same thread polls its own slots for the peers'
// values (flag-in-data: no fence, no separate flag round trip), then adds them in rank order with the residual.
//
// Reference counterpart: the per-format decode GEMVs gemv_tq2_g128_v1 / gemv_q1_g128_v7..v9
// (crates/oxibonsai-kernels/src/gpu_backend/cuda_kernels.rs:76-776) and the row-parallel all-reduce of
// tensor_parallel_forward (crates/oxibonsai-model/src/tensor_parallel.rs:338-386).
#include "../comm/tp_comm.cuh"
#include "common.cuh"
#include "tcgen05.cuh"

namespace bonsai {

enum { SEPI_STORE = 0, SEPI_RESID = 1, SEPI_SWIGLU = 2, SEPI_TP = 3 };

constexpr int kS16Warps = 16;                                    // consumer warps; warp 16 is the copy producer
constexpr int kS16Threads = (kS16Warps + 1) * 32;
constexpr int kS16BlockBytes = 544;                              // 512 B codes + 32 B scales
constexpr int kS16MaxStages = 16;
constexpr int kS16MaxTiles = 12;                                 // tiles per CTA (size of the partial-sum area)
constexpr uint32_t kS16WaitLimit = 1u << 21;                     // polls (with a short sleep in between): about a second

// Pipeline shape, settable through bonsai_s16_tune: blocks per warp per stage (1 or 2), ring stages, and the sleep
// between two polls of a ring barrier.  Back-to-back polling by sixteen waiting warps saturates the shared-memory
// pipe and delays the copy completions and the producer's own barrier traffic.
static int g_s16_bpw = 2, g_s16_stages = 4, g_s16_sleep_ns = 32, g_s16_pdl = 1;

// offset + 1 of MMA step mm (= code slot mm): slots reach mantissa position 6, 8 | 4, 6, 8 | 4, 6, 8
__device__ __constant__ float kS16Off[8] = {17.0f, 5.0f, 65.0f, 17.0f, 5.0f, 65.0f, 17.0f, 5.0f};

__device__ __forceinline__ void s16_mma(float* d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// 512 consumer threads only (the producer warp never joins)
__device__ __forceinline__ void s16_bar() { asm volatile("bar.sync 1, %0;" ::"n"(kS16Warps * 32) : "memory"); }

// Bounded wait on a ring barrier: lane 0 polls, the outcome is broadcast.  Returns false on expiry or when another
// warp has already given up (*abort set).
__device__ __forceinline__ bool s16_poll(uint64_t* bar, uint32_t parity, volatile int* abort, int sleep_ns) {
  for (uint32_t i = 0; i < kS16WaitLimit; ++i) {
    if (tc::mbar_try_wait(bar, parity)) return true;
    if ((i & 63u) == 63u && *abort) break;
    if (sleep_ns > 0) __nanosleep(sleep_ns);
  }
  *abort = 1;
  return false;
}
__device__ __forceinline__ bool s16_wait(uint64_t* bar, uint32_t parity, int lane, volatile int* abort, int sleep_ns) {
  int ok = 1;
  if (lane == 0) ok = s16_poll(bar, parity, abort, sleep_ns) ? 1 : 0;
  return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

__device__ __forceinline__ void st_relaxed_sys_u64(unsigned long long* p, unsigned long long v) {
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_relaxed_sys_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

// One (tile, group) block against the group's 128 activations.  Adds scale * (W x) of rows g and g + 8 to tot.
__device__ __forceinline__ void s16_block(const uint8_t* __restrict__ blk, const __half* __restrict__ xg, float og, int lane,
                                          float& tot_lo, float& tot_hi) {
  const int g = lane >> 2, t = lane & 3;
  const uint4 cw = *reinterpret_cast<const uint4*>(blk + lane * 16);
  const uint32_t sc = *reinterpret_cast<const uint32_t*>(blk + 512 + 4 * g);
  const uint32_t w[4] = {cw.x, cw.y, cw.z, cw.w};
  uint32_t lo[4], hi[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    lo[i] = w[i] << 6;
    hi[i] = w[i] >> 6;
  }
  float accA[4] = {0.0f, 0.0f, 0.0f, 0.0f}, accB[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  const uint4* xv4 = reinterpret_cast<const uint4*>(xg + 8 * t);
  constexpr uint32_t M4 = 0x00300030u, M6 = 0x00C000C0u, M8 = 0x03000300u;
  constexpr uint32_t E4 = 0x54005400u, E6 = 0x4C004C00u, E8 = 0x44004400u;   // 64, 16, 4
  {
    const uint4 xv = xv4[0];    // inputs 8t .. 8t+7 of the group
    s16_mma(accA, (lo[0] & M6) | E6, (lo[1] & M6) | E6, (lo[2] & M6) | E6, (lo[3] & M6) | E6, xv.x, xv.y);
    s16_mma(accB, (lo[0] & M8) | E8, (lo[1] & M8) | E8, (lo[2] & M8) | E8, (lo[3] & M8) | E8, xv.z, xv.w);
  }
  {
    const uint4 xv = xv4[4];    // 32 + 8t ..
    s16_mma(accA, (w[0] & M4) | E4, (w[1] & M4) | E4, (w[2] & M4) | E4, (w[3] & M4) | E4, xv.x, xv.y);
    s16_mma(accB, (w[0] & M6) | E6, (w[1] & M6) | E6, (w[2] & M6) | E6, (w[3] & M6) | E6, xv.z, xv.w);
  }
  {
    const uint4 xv = xv4[8];    // 64 + 8t ..
    s16_mma(accA, (w[0] & M8) | E8, (w[1] & M8) | E8, (w[2] & M8) | E8, (w[3] & M8) | E8, xv.x, xv.y);
    s16_mma(accB, (hi[0] & M4) | E4, (hi[1] & M4) | E4, (hi[2] & M4) | E4, (hi[3] & M4) | E4, xv.z, xv.w);
  }
  {
    const uint4 xv = xv4[12];   // 96 + 8t ..
    s16_mma(accA, (hi[0] & M6) | E6, (hi[1] & M6) | E6, (hi[2] & M6) | E6, (hi[3] & M6) | E6, xv.x, xv.y);
    s16_mma(accB, (hi[0] & M8) | E8, (hi[1] & M8) | E8, (hi[2] & M8) | E8, (hi[3] & M8) | E8, xv.z, xv.w);
  }
  const __half2 s2 = *reinterpret_cast<const __half2*>(&sc);
  tot_lo = fmaf(__low2float(s2), (accA[0] + accB[0]) - og, tot_lo);
  tot_hi = fmaf(__high2float(s2), (accA[2] + accB[2]) - og, tot_hi);
}

struct S16Args {
  const uint8_t* w;          // S16 blocks [tile][group]
  const float* x;            // f32 [K]
  const float* norm_w;       // f32 [K] or null
  float* out;
  const float* residual;
  int* status;               // device int, set non-zero when a bounded wait expired (may be null)
  float eps;
  int N, K, epi;
  int nstages, sleep_ns;     // ring depth and poll back-off
};

template <int BPW>
__global__ void __launch_bounds__(kS16Threads, 2) bitgemv_s16_kernel(S16Args a, TpComm tp) {
  constexpr int kS16StageBlocks = BPW * kS16Warps;
  constexpr int kS16StageBytes = kS16StageBlocks * kS16BlockBytes;   // 8704 or 17408
  extern __shared__ __align__(128) uint8_t smem[];
  const int K = a.K, ng = K >> 7;
  const int kS16Stages = a.nstages;
  uint8_t* ring = smem;
  __half* xs = reinterpret_cast<__half*>(smem + kS16Stages * kS16StageBytes);
  float* og = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(xs) + (size_t)K * 2);
  float* part = og + ((ng + 3) & ~3);                      // [kS16MaxTiles][kS16Warps][16]
  uint64_t* full = reinterpret_cast<uint64_t*>(part + kS16MaxTiles * kS16Warps * 16);
  uint64_t* empty = full + kS16MaxStages;
  float* s32 = reinterpret_cast<float*>(empty + kS16MaxStages);   // [32]
  volatile int* abort_flag = reinterpret_cast<volatile int*>(s32 + 32);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int ntiles = (a.N + 15) >> 4;
  const int tile_lo = (int)(((long long)blockIdx.x * ntiles) / gridDim.x);
  const int tile_hi = (int)(((long long)(blockIdx.x + 1) * ntiles) / gridDim.x);
  const int nb_total = (tile_hi - tile_lo) * ng;           // blocks of this CTA's stream
  const int nstage_total = (nb_total + kS16StageBlocks - 1) / kS16StageBlocks;
  const uint8_t* wbase = a.w + (size_t)tile_lo * ng * kS16BlockBytes;

  if (tid == 0) {
    for (int s = 0; s < kS16Stages; ++s) {
      tc::mbar_init(&full[s], 1);
      tc::mbar_init(&empty[s], kS16Warps);
    }
    *abort_flag = 0;
    tc::mbar_fence_init();
  }
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  __syncthreads();

  if (warp == kS16Warps) {
    // ---- producer: one lane streams the CTA's byte range through the ring (weights depend on no earlier kernel) ----
    if (lane == 0) {
      for (int s = 0; s < nstage_total; ++s) {
        const int slot = s % kS16Stages;
        if (s >= kS16Stages && !s16_poll(&empty[slot], ((s / kS16Stages) - 1) & 1, abort_flag, a.sleep_ns)) break;
        const int b0 = s * kS16StageBlocks;
        const int nb = min(kS16StageBlocks, nb_total - b0);
        const uint32_t bytes = (uint32_t)nb * kS16BlockBytes;
        tc::mbar_arrive_expect_tx(&full[slot], bytes);
        tc::bulk_g2s(ring + (size_t)slot * kS16StageBytes, wbase + (size_t)b0 * kS16BlockBytes, bytes, &full[slot]);
      }
      // The consumers wait for every stage that was issued, so all copies have landed when they finish.  After an
      // abort they no longer do: give outstanding copies a bounded time to land before this CTA's memory is released.
      if (*abort_flag) {
        for (int slot = 0; slot < kS16Stages; ++slot)
          for (uint32_t i = 0; i < (1u << 16); ++i)
            if (tc::mbar_try_wait(&full[slot], 0) || tc::mbar_try_wait(&full[slot], 1)) break;
      }
    }
    return;
  }

  // ---- consumers ----
  constexpr int NT = kS16Warps * 32;
  for (int i = tid; i < kS16MaxTiles * kS16Warps * 16; i += NT) part[i] = 0.0f;   // nothing here depends on an earlier kernel
  asm volatile("griddepcontrol.wait;" ::: "memory");
  {
    // activations: f32 -> (RMS-normalised) f16 in natural order, and the per-group offset sums
    //   og[g] = sum over the group's inputs of (offset + 1) * x,
    // taken from the rounded values while they are written: thread tid + i * NT holds inputs 4c..4c+3 of chunk c, a
    // warp's 32 chunks are one 128-input group, and lane l's four inputs all belong to MMA step 2 * (l / 8) + (l & 1)
    const int nch = K >> 2;
    const float4* x4 = reinterpret_cast<const float4*>(a.x);
    float4 keep[2];
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int c = tid + i * NT;
      keep[i] = c < nch ? x4[c] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      ss += keep[i].x * keep[i].x + keep[i].y * keep[i].y + keep[i].z * keep[i].z + keep[i].w * keep[i].w;
    }
    float inv = 1.0f;
    if (a.norm_w != nullptr) {
      for (int c = tid + 2 * NT; c < nch; c += NT) {
        const float4 v = x4[c];
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
      }
      ss = warp_sum(ss);
      if (lane == 0) s32[warp] = ss;
      s16_bar();
      float tsum = lane < kS16Warps ? s32[lane] : 0.0f;
      tsum = warp_sum(tsum);
      inv = 1.0f / sqrtf(tsum / (float)K + a.eps);
    }
    const float off = kS16Off[2 * (lane >> 3) + (lane & 1)];
    auto emit = [&](int c, float4 v) {      // whole warps enter (K % 128 == 0): c / 32 is the warp's group
      if (a.norm_w != nullptr) {
        const float4 ww = reinterpret_cast<const float4*>(a.norm_w)[c];
        v.x *= ww.x * inv; v.y *= ww.y * inv; v.z *= ww.z * inv; v.w *= ww.w * inv;
      }
      const __half2 h0 = __floats2half2_rn(v.x, v.y), h1 = __floats2half2_rn(v.z, v.w);
      uint2 u;
      u.x = *reinterpret_cast<const uint32_t*>(&h0);
      u.y = *reinterpret_cast<const uint32_t*>(&h1);
      reinterpret_cast<uint2*>(xs)[c] = u;
      const float2 f0 = __half22float2(h0), f1 = __half22float2(h1);
      const float sg = warp_sum(off * ((f0.x + f0.y) + (f1.x + f1.y)));
      if (lane == 0) og[c >> 5] = sg;
    };
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int c = tid + i * NT;
      if (c < nch) emit(c, keep[i]);
    }
    for (int c = tid + 2 * NT; c < nch; c += NT) emit(c, x4[c]);
    s16_bar();
  }

  // ---- main loop: BPW consecutive blocks per warp per stage ----
  {
    int cur_tile = -1;
    float tot_lo = 0.0f, tot_hi = 0.0f;
    const int g = lane >> 2, t = lane & 3;
    auto flush = [&]() {
      if (cur_tile >= 0 && t == 0) {
        float* p = part + ((size_t)cur_tile * kS16Warps + warp) * 16;
        p[g] += tot_lo;
        p[g + 8] += tot_hi;
      }
      tot_lo = tot_hi = 0.0f;
    };
    for (int s = 0; s < nstage_total; ++s) {
      const int slot = s % kS16Stages;
      if (!s16_wait(&full[slot], (s / kS16Stages) & 1, lane, abort_flag, a.sleep_ns)) break;
      const uint8_t* st = ring + (size_t)slot * kS16StageBytes + (size_t)(BPW * warp) * kS16BlockBytes;
      const int idx0 = s * kS16StageBlocks + BPW * warp;
      int tl = idx0 / ng, grp = idx0 - tl * ng;
#pragma unroll
      for (int i = 0; i < BPW; ++i) {
        if (idx0 + i < nb_total) {
          if (tl != cur_tile) {
            flush();
            cur_tile = tl;
          }
          s16_block(st + (size_t)i * kS16BlockBytes, xs + (size_t)grp * 128, og[grp], lane, tot_lo, tot_hi);
        }
        if (++grp == ng) {
          grp = 0;
          ++tl;
        }
      }
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(&empty[slot]);
    }
    flush();
  }
  s16_bar();
  const bool aborted = *abort_flag != 0;
  if (aborted && tid == 0 && a.status != nullptr) atomicExch(a.status, 5);
  if (aborted && a.epi != SEPI_TP) return;   // the tensor-parallel form still counts itself out below

  // ---- reduce over warps (fixed order) and epilogue ----
  const int rows_local = (tile_hi - tile_lo) * 16;
  const int row_base = tile_lo * 16;
  if (a.epi == SEPI_SWIGLU) {
    for (int pi = tid; pi < rows_local / 2; pi += kS16Warps * 32) {
      const int r0 = 2 * pi, tl = r0 >> 4, rr = r0 & 15;
      float gate = 0.0f, up = 0.0f;
#pragma unroll
      for (int w = 0; w < kS16Warps; ++w) {
        gate += part[((size_t)tl * kS16Warps + w) * 16 + rr];
        up += part[((size_t)tl * kS16Warps + w) * 16 + rr + 1];
      }
      const int row = row_base + r0;
      if (row + 1 < a.N) a.out[row >> 1] = gate / (1.0f + __expf(-gate)) * up;
    }
    return;
  }
  int tp_epoch = 0;
  if (a.epi == SEPI_TP) tp_epoch = ld_volatile(tp.epoch);
  for (int i = tid; i < (aborted ? 0 : rows_local); i += kS16Warps * 32) {
    const int tl = i >> 4, rr = i & 15;
    float v = 0.0f;
#pragma unroll
    for (int w = 0; w < kS16Warps; ++w) v += part[((size_t)tl * kS16Warps + w) * 16 + rr];
    const int row = row_base + i;
    if (row >= a.N) continue;
    if (a.epi == SEPI_STORE) {
      a.out[row] = v;
    } else if (a.epi == SEPI_RESID) {
      a.out[row] = a.residual[row] + v;
    } else {
      // flag-in-data exchange: {value, tag} as one 8-byte store into slot [parity][my rank][row] of every peer
      const uint32_t tag = (uint32_t)tp_epoch + 1u;
      const int parity = tp_epoch & 1;
      const unsigned long long msg = ((unsigned long long)tag << 32) | (unsigned long long)__float_as_uint(v);
      for (int p = 0; p < tp.size; ++p)
        if (p != tp.rank) st_relaxed_sys_u64(tp_ll_slot(tp, p, parity, tp.rank) + row, msg);
      float sum = a.residual != nullptr ? a.residual[row] : 0.0f;
      for (int s = 0; s < tp.size; ++s) {
        float pv = v;
        if (s != tp.rank) {
          const unsigned long long* src = tp_ll_slot(tp, tp.rank, parity, s) + row;
          bool got = false;
          for (uint32_t it = 0; it < tp.spin_limit; ++it) {
            const unsigned long long m = ld_relaxed_sys_u64(src);
            if ((uint32_t)(m >> 32) == tag) {
              pv = __uint_as_float((uint32_t)m);
              got = true;
              break;
            }
          }
          if (!got) {
            atomicExch(tp.status, 2);
            pv = 0.0f;
          }
        }
        sum += pv;
      }
      a.out[row] = sum;
    }
  }
  if (a.epi == SEPI_TP) {
    // last CTA bumps the exchange counter (every CTA has read it by then)
    s16_bar();
    if (tid == 0) {
      __threadfence();
      const int prev = atomicAdd(tp.done_ctr, 1);
      if (prev == (int)gridDim.x - 1) {
        *tp.done_ctr = 0;
        *tp.epoch = tp_epoch + 1;
        __threadfence();
      }
    }
  }
}

// Planar-SM -> S16.  One thread per output 32-bit word (code words and scale pairs).
__global__ void repack_s16_kernel(const uint32_t* __restrict__ codes, const __half* __restrict__ scales, int N, int K,
                                  uint32_t* __restrict__ out) {
  const int ng = K >> 7, wpr = K >> 4;
  const long long ntiles = (N + 15) >> 4;
  const long long total = ntiles * ng * (kS16BlockBytes / 4);
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    const int wi_blk = (int)(idx % (kS16BlockBytes / 4));
    const long long blk = idx / (kS16BlockBytes / 4);
    const int grp = (int)(blk % ng);
    const int tile = (int)(blk / ng);
    uint32_t o = 0;
    if (wi_blk < 128) {
      const int lane = wi_blk >> 2, wi = wi_blk & 3;
      const int g = lane >> 2, t = lane & 3;
      const int row = tile * 16 + g + ((wi & 1) ? 8 : 0);
#pragma unroll
      for (int mm = 0; mm < 8; ++mm) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t c = 1u;   // zero weight
          if (row < N) {
            const int k = grp * 128 + 32 * (mm >> 1) + 8 * t + 4 * (mm & 1) + ((wi & 2) ? 2 : 0) + h;
            const uint32_t pw = codes[(size_t)row * wpr + (k >> 4)];
            const int j = k & 15, i = j & 7;
            const uint32_t nib = (pw >> (4 * i)) & 0xFu;
            const uint32_t m = j < 8 ? (nib >> 1) & 1u : nib & 1u;
            const uint32_t sgn = j < 8 ? (nib >> 3) & 1u : (nib >> 2) & 1u;
            c = m ? (sgn ? 0u : 2u) : 1u;
          }
          o |= c << (2 * mm + 16 * h);
        }
      }
    } else {
      const int g = wi_blk - 128;   // 0..7: scales of rows g and g + 8
      const int r0 = tile * 16 + g, r1 = r0 + 8;
      const uint32_t s0 = r0 < N ? (uint32_t)__half_as_ushort(scales[(size_t)r0 * ng + grp]) : 0u;
      const uint32_t s1 = r1 < N ? (uint32_t)__half_as_ushort(scales[(size_t)r1 * ng + grp]) : 0u;
      o = s0 | (s1 << 16);
    }
    out[idx] = o;
  }
}

static inline size_t s16_smem_bytes(int K, int bpw, int stages) {
  const int ng = K / 128;
  return (size_t)stages * bpw * kS16Warps * kS16BlockBytes + (size_t)K * 2 + (size_t)((ng + 3) & ~3) * 4 +
         (size_t)kS16MaxTiles * kS16Warps * 16 * 4 + 2 * kS16MaxStages * 8 + 32 * 4 + 16;
}

}  // namespace bonsai

extern "C" {

// Bytes of the S16 form of an N x K packed matrix.
size_t bonsai_s16_bytes(int N, int K) { return (size_t)((N + 15) / 16) * (K / 128) * bonsai::kS16BlockBytes; }

int bonsai_repack_s16(const void* codes, const void* scales, int N, int K, void* out, cudaStream_t stream) {
  using namespace bonsai;
  if (N <= 0 || K <= 0 || K % 128 != 0) return BONSAI_CUDA_BAD_ARG;
  const long long total = (long long)((N + 15) / 16) * (K / 128) * (kS16BlockBytes / 4);
  const int grid = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  repack_s16_kernel<<<grid, 256, 0, stream>>>((const uint32_t*)codes, (const __half*)scales, N, K, (uint32_t*)out);
  return launch_status();
}

// Pipeline shape of bonsai_bitgemv_s16 for later launches of this process: blocks per warp per stage (1 or 2), ring
// stages (2..16), nanoseconds of sleep between two polls of a ring barrier, and whether the kernel is launched with
// programmatic dependent launch (its weight copies then start while the previous kernel still runs).  Returns 0, or
// the bad-argument code.
int bonsai_s16_tune(int blocks_per_warp, int stages, int sleep_ns, int pdl) {
  if ((blocks_per_warp != 1 && blocks_per_warp != 2) || stages < 2 || stages > bonsai::kS16MaxStages || sleep_ns < 0) return BONSAI_CUDA_BAD_ARG;
  bonsai::g_s16_pdl = pdl != 0;
  bonsai::g_s16_bpw = blocks_per_warp;
  bonsai::g_s16_stages = stages;
  bonsai::g_s16_sleep_ns = sleep_ns;
  return BONSAI_CUDA_OK;
}

// out = W x for an S16 matrix (see the head of this file): out[N] for epi 0 / 1 (1 adds residual[N]), out[N/2] for
// epi 2 (SwiGLU over interleaved gate/up rows), and for epi 3 out[N] = residual[N] + sum over the ranks of `comm` of
// their W x (every rank launches the same call on its shard; residual may be null).  x is f32[K], RMS-normalised with
// norm_w first when that is non-null.  K % 128 == 0, 128 <= K <= 16384, at most 12 row tiles per CTA.  `status`
// (device int, may be null) is set to 5 if a bounded wait on the copy pipeline expired.
int bonsai_bitgemv_s16(const void* w16, const float* x, const float* norm_w, float eps, float* out, const float* residual,
                       int N, int K, int epi, const void* comm, int* status, cudaStream_t stream) {
  using namespace bonsai;
  if (K % 128 != 0 || K < 128 || K > 16384 || N <= 0 || epi < 0 || epi > 3) return BONSAI_CUDA_BAD_ARG;
  if (epi == SEPI_RESID && residual == nullptr) return BONSAI_CUDA_BAD_ARG;
  if (epi == SEPI_SWIGLU && (N & 1)) return BONSAI_CUDA_BAD_ARG;
  if (epi == SEPI_TP && comm == nullptr) return BONSAI_CUDA_BAD_ARG;
  const int ntiles = (N + 15) / 16;
  int grid = ntiles < 148 ? ntiles : 148;
  if ((ntiles + grid - 1) / grid > kS16MaxTiles) {
    if (epi == SEPI_TP) return BONSAI_CUDA_BAD_ARG;       // waits on peers: the grid must stay co-resident
    grid = (ntiles + kS16MaxTiles - 1) / kS16MaxTiles;
  }
  TpComm tp{};
  if (epi == SEPI_TP) {
    tp = *static_cast<const TpComm*>(comm);
    if ((size_t)N > tp.lay.recv_elems) return BONSAI_CUDA_BAD_ARG;
  }
  const int bpw = g_s16_bpw, stages = g_s16_stages;
  const size_t smem = s16_smem_bytes(K, bpw, stages);
  if (smem > 200 * 1024) return BONSAI_CUDA_BAD_ARG;
  static bool attr_set[64] = {};   // per device: the attribute belongs to the device's copy of the function
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return BONSAI_CUDA_LAUNCH_FAILED;
  if (!attr_set[dev]) {
    if (cudaFuncSetAttribute(bitgemv_s16_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess ||
        cudaFuncSetAttribute(bitgemv_s16_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess)
      return BONSAI_CUDA_LAUNCH_FAILED;
    attr_set[dev] = true;
  }
  S16Args a;
  a.w = static_cast<const uint8_t*>(w16);
  a.x = x;
  a.norm_w = norm_w;
  a.out = out;
  a.residual = residual;
  a.status = status;
  a.eps = eps;
  a.N = N;
  a.K = K;
  a.epi = epi;
  a.nstages = stages;
  a.sleep_ns = g_s16_sleep_ns;
  cudaError_t e;
  if (g_s16_pdl) {
    e = bpw == 1 ? launch_pdl(bitgemv_s16_kernel<1>, dim3(grid), dim3(kS16Threads), smem, stream, a, tp)
                 : launch_pdl(bitgemv_s16_kernel<2>, dim3(grid), dim3(kS16Threads), smem, stream, a, tp);
  } else {
    if (bpw == 1) bitgemv_s16_kernel<1><<<grid, kS16Threads, smem, stream>>>(a, tp);
    else bitgemv_s16_kernel<2><<<grid, kS16Threads, smem, stream>>>(a, tp);
    e = cudaGetLastError();
  }
  return e == cudaSuccess ? BONSAI_CUDA_OK : BONSAI_CUDA_LAUNCH_FAILED;
}

}  // extern "C"
