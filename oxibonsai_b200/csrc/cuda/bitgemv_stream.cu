// Batch-1 decode GEMV that streams packed weights through shared memory with bulk async copies and multiplies on
// the warp-level integer tensor cores with a one-instruction decode of four weights.
//
// Why another GEMV: the planar-layout kernels (bitgemv_warp.cu, bitgemv_hmma.cu) spend ~2.5 thread instructions per
// weight on shift + mask + FMA.  On this GPU the integer/logic pipe issues one warp instruction every two cycles, so
// those kernels are bound by their decode instructions at a quarter of the memory roofline (measured: the same time
// with the weights resident in L2).  Here
//   * weights live in the "S16" layout: tiles of 16 output rows, one 544-byte block per (tile, 128-input group) =
//     32 lanes x 16 bytes of 2-bit codes in MMA-fragment order + 16 f16 group scales.  A CTA owns a contiguous range
//     of tiles, i.e. one contiguous byte range of the matrix, and a producer lane streams it into a three-stage
//     shared-memory ring with cp.async.bulk (34 KB per copy, 104 KB in flight per SM);
//   * a code c = w + 1 in {0, 1, 2} occupies one 2-bit field of a byte; `word & (0x03030303 << 2j)` is the u8 vector
//     (4^j c) of four weights: ONE logic instruction per four weights, no shift, no sign handling.  The 4^j is not
//     undone on the weights: MMA step j of a group uses field j of every word, and the activations are laid out so
//     that step j only reaches output columns 2j and 2j+1 of mma.sync.m16n8k32 (u8 x s8 -> s32) - every other column
//     of its B operand is zero.  After the group's four steps, column 2j (+1) holds 4^j times the dot product of
//     step j's 32 inputs, the lane that owns the column scales it by 4^-j in f32, and a quad reduction at the end of
//     the tile adds the four partial sums;
//   * activations are quantised per 128-input group to two int8 terms, x = s (q1 + q2 / 254), |q| <= 127 - sixteen
//     bits relative to the group's largest value; the terms are the even and odd output columns.  Products and sums
//     are exact integers; the +1 of the codes is removed by starting the accumulators at -4^j * sum(q) of the step;
//   * sixteen consumer warps take four consecutive blocks each per stage - four independent MMA chains, issued
//     interleaved and without a branch in between when the blocks belong to one tile - keep per-tile partial sums
//     in registers and meet in shared memory once at the end; partials are added in warp order, so results do not
//     depend on timing.
// Per (tile, group) block a thread issues 16 logic ops, 4 MMAs, 4 loads, 8 integer multiplies that build the
// zero-padded B operands and a dozen f32 ops: ~0.8 instructions per weight.
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
constexpr int kS16Bpw = 4;                                       // consecutive blocks per warp per stage
constexpr int kS16StageBlocks = kS16Bpw * kS16Warps;
constexpr int kS16StageBytes = kS16StageBlocks * kS16BlockBytes; // 34816
constexpr int kS16Stages = 3;
constexpr int kS16MaxTiles = 12;                                 // tiles per CTA (size of the partial-sum area)
constexpr uint32_t kS16WaitLimit = 1u << 21;                     // polls with a short sleep in between: about a second
constexpr float kS16Term2 = 254.0f;                              // x = s * (q1 + q2 / 254)

// Launched with programmatic dependent launch (the prologue of the next kernel overlaps the tail of this one) unless
// switched off through bonsai_s16_tune.
static int g_s16_pdl = 1;

__device__ __forceinline__ void s16_imma(int* d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Integer multiply (runs on the FMA pipe, which this kernel leaves idle; the logic pipe is the scarce one).
__device__ __forceinline__ uint32_t s16_mul(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.lo.u32 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

// 512 consumer threads only (the producer warp never joins)
__device__ __forceinline__ void s16_bar() { asm volatile("bar.sync 1, %0;" ::"n"(kS16Warps * 32) : "memory"); }

// Bounded wait on a ring barrier.  Returns false on expiry or when another warp has already given up (*abort set).
__device__ __forceinline__ bool s16_poll(uint64_t* bar, uint32_t parity, volatile int* abort) {
  for (uint32_t i = 0; i < kS16WaitLimit; ++i) {
    if (tc::mbar_try_wait(bar, parity)) return true;
    if ((i & 63u) == 63u && *abort) break;
    __nanosleep(32);
  }
  *abort = 1;
  return false;
}
__device__ __forceinline__ bool s16_wait(uint64_t* bar, uint32_t parity, int lane, volatile int* abort) {
  int ok = 1;
  if (lane == 0) ok = s16_poll(bar, parity, abort) ? 1 : 0;
  return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

// Per (group, step) record of the activation side: the step's accumulator start values and f32 factor.
struct __align__(16) S16Step {
  int og0, og1;      // -4^j * sum of the step's q1 (q2) values: takes out what the +1 of the codes adds to the integer dot product
  float sx;          // group scale of the activations times 4^-j
  float pad;
};

// One (tile, group) block.  xq_lane: the lane's eight int8 activations of its own step (g / 2) and term (g & 1) of the
// group; st_lane: the S16Step record of the lane's accumulator columns (step t of the group).  sel[j] is 1
// when this lane's B column belongs to step j, else 0.  Adds the lane's share (its step, both terms) of
// scale * (W x) of rows g and g + 8 to tot.
__device__ __forceinline__ void s16_block(const uint8_t* __restrict__ blk, const int8_t* __restrict__ xq_lane, const S16Step* __restrict__ st_lane,
                                          int lane, const uint32_t (&sel)[4], float& tot_lo, float& tot_hi) {
  const int g = lane >> 2;
  const uint4 cw = *reinterpret_cast<const uint4*>(blk + lane * 16);
  const uint32_t sc = *reinterpret_cast<const uint32_t*>(blk + 512 + 4 * g);
  const S16Step st = *st_lane;
  int acc[4] = {st.og0, st.og1, st.og0, st.og1};
  const uint2 xb = *reinterpret_cast<const uint2*>(xq_lane);            // the lane's eight activations of its own step
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    // B operand of step j: those activations if the lane's column belongs to step j, else zeros
    const uint32_t m = 0x03030303u << (2 * j);
    s16_imma(acc, cw.x & m, cw.y & m, cw.z & m, cw.w & m, s16_mul(xb.x, sel[j]), s16_mul(xb.y, sel[j]));
  }
  const __half2 s2 = *reinterpret_cast<const __half2*>(&sc);
  // columns 2t and 2t+1 are the two terms of the lane's step: x = s (q1 + q2 / 254)
  const float v_lo = fmaf((float)acc[1], 1.0f / kS16Term2, (float)acc[0]);
  const float v_hi = fmaf((float)acc[3], 1.0f / kS16Term2, (float)acc[2]);
  tot_lo = fmaf(__low2float(s2) * st.sx, v_lo, tot_lo);
  tot_hi = fmaf(__high2float(s2) * st.sx, v_hi, tot_hi);
}

// NB consecutive blocks of one tile (groups grp .. grp + NB - 1), their MMA chains issued interleaved.
template <int NB>
__device__ __forceinline__ void s16_blocks(const uint8_t* __restrict__ blk, const int8_t* __restrict__ xq_lane, const S16Step* __restrict__ st_lane,
                                           int lane, const uint32_t (&sel)[4], float& tot_lo, float& tot_hi) {
  const int g = lane >> 2;
  uint4 cw[NB];
  uint2 xb[NB];
  uint32_t sc[NB];
  float sx[NB];
  int acc[NB][4];
#pragma unroll
  for (int b = 0; b < NB; ++b) {
    cw[b] = *reinterpret_cast<const uint4*>(blk + b * kS16BlockBytes + lane * 16);
    xb[b] = *reinterpret_cast<const uint2*>(xq_lane + 128 * b);
    sc[b] = *reinterpret_cast<const uint32_t*>(blk + b * kS16BlockBytes + 512 + 4 * g);
    const S16Step st = st_lane[4 * b];
    acc[b][0] = acc[b][2] = st.og0;
    acc[b][1] = acc[b][3] = st.og1;
    sx[b] = st.sx;
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint32_t m = 0x03030303u << (2 * j);
#pragma unroll
    for (int b = 0; b < NB; ++b) {
      s16_imma(acc[b], cw[b].x & m, cw[b].y & m, cw[b].z & m, cw[b].w & m, s16_mul(xb[b].x, sel[j]), s16_mul(xb[b].y, sel[j]));
    }
  }
#pragma unroll
  for (int b = 0; b < NB; ++b) {
    const __half2 s2 = *reinterpret_cast<const __half2*>(&sc[b]);
    const float v_lo = fmaf((float)acc[b][1], 1.0f / kS16Term2, (float)acc[b][0]);
    const float v_hi = fmaf((float)acc[b][3], 1.0f / kS16Term2, (float)acc[b][2]);
    tot_lo = fmaf(__low2float(s2) * sx[b], v_lo, tot_lo);
    tot_hi = fmaf(__high2float(s2) * sx[b], v_hi, tot_hi);
  }
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
  const uint8_t* next_w;     // weights the following kernel will stream (may be null): requested into L2 from here
  unsigned long long next_bytes;
};

__global__ void __launch_bounds__(kS16Threads, 1) bitgemv_s16_kernel(S16Args a, TpComm tp) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int K = a.K, ng = K >> 7;
  const int term_stride = K + 32;                              // second term sits 32 bytes off a multiple of 128: no bank clash
  uint8_t* ring = smem;
  int8_t* xq = reinterpret_cast<int8_t*>(smem + kS16Stages * kS16StageBytes);      // [2][K + 32]
  S16Step* steps = reinterpret_cast<S16Step*>(xq + 2 * term_stride);                // [ng][4]
  float* part = reinterpret_cast<float*>(steps + (size_t)ng * 4);                   // [kS16MaxTiles][kS16Warps][16]
  uint64_t* full = reinterpret_cast<uint64_t*>(part + kS16MaxTiles * kS16Warps * 16);
  uint64_t* empty = full + kS16Stages;
  float* s32 = reinterpret_cast<float*>(empty + kS16Stages);   // [32]
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
      // slice of the next kernel's weights that this CTA requests into L2 (16-byte units)
      const unsigned long long pf_units = a.next_w != nullptr ? a.next_bytes / 16 : 0;
      const unsigned long long pf_lo = pf_units * blockIdx.x / gridDim.x, pf_hi = pf_units * (blockIdx.x + 1) / gridDim.x;
      const uint8_t* pf_ptr = a.next_w + pf_lo * 16;
      unsigned long long pf_left = (pf_hi - pf_lo) * 16;
      const unsigned long long pf_piece = 32768;
      int slot = 0;
      uint32_t phase = 1;      // parity of the use of a slot that must have been released: none for the first round
      for (int s = 0; s < nstage_total; ++s, slot = slot + 1 == kS16Stages ? 0 : slot + 1) {
        if (slot == 0) phase ^= 1u;
        if (s >= kS16Stages && !s16_poll(&empty[slot], phase ^ 1u, abort_flag)) break;
        const int b0 = s * kS16StageBlocks;
        const int nb = min(kS16StageBlocks, nb_total - b0);
        const uint32_t bytes = (uint32_t)nb * kS16BlockBytes;
        tc::mbar_arrive_expect_tx(&full[slot], bytes);
        tc::bulk_g2s(ring + (size_t)slot * kS16StageBytes, wbase + (size_t)b0 * kS16BlockBytes, bytes, &full[slot]);
        // This kernel is bound by instruction issue, not by HBM: the idle bandwidth brings the next kernel's weights
        // into L2, a slice per CTA and a piece per stage, so that its first stage does not start with a trip to DRAM.
        if (pf_left > 0) {
          const unsigned long long n = pf_left < pf_piece ? pf_left : pf_piece;
          asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(pf_ptr), "r"((uint32_t)n) : "memory");
          pf_ptr += n;
          pf_left -= n;
        }
      }
      while (pf_left > 0) {
        const unsigned long long n = pf_left < pf_piece ? pf_left : pf_piece;
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(pf_ptr), "r"((uint32_t)n) : "memory");
        pf_ptr += n;
        pf_left -= n;
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
    // Activations: f32 -> (RMS-normalised) -> two int8 terms per 128-input group.  Thread tid + i * NT holds the four
    // inputs of chunk c; a warp's 32 chunks are one group and lanes 8j..8j+7 hold the 32 inputs of MMA step j.
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
    auto emit = [&](int c, float4 v) {      // whole warps enter (K % 128 == 0): c / 32 is the warp's group
      if (a.norm_w != nullptr) {
        const float4 ww = reinterpret_cast<const float4*>(a.norm_w)[c];
        v.x *= ww.x * inv; v.y *= ww.y * inv; v.z *= ww.z * inv; v.w *= ww.w * inv;
      }
      const float amax = warp_max(fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
      const float sx = amax > 0.0f ? amax * (1.0f / 127.0f) : 1.0f;
      const float rs = 1.0f / sx;
      // Round with the 1.5 * 2^23 trick: (f + magic) holds rint(f) in its low mantissa bits (two's complement, so the low
      // byte is the int8 value) and (f + magic) - magic is rint(f) as a float.  |f| <= 127 and |f - rint(f)| * 254 <= 127
      // by construction, so nothing needs clamping.
      constexpr float kMagic = 12582912.0f;
      const float f[4] = {v.x * rs, v.y * rs, v.z * rs, v.w * rs};
      uint32_t w1 = 0, w2 = 0;
      float fs1 = 0.0f, fs2 = 0.0f;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float m1 = f[e] + kMagic, r1 = m1 - kMagic;
        const float m2 = (f[e] - r1) * kS16Term2 + kMagic, r2 = m2 - kMagic;
        w1 |= (__float_as_uint(m1) & 255u) << (8 * e);
        w2 |= (__float_as_uint(m2) & 255u) << (8 * e);
        fs1 += r1;
        fs2 += r2;
      }
      reinterpret_cast<uint32_t*>(xq)[c] = w1;
      reinterpret_cast<uint32_t*>(xq + term_stride)[c] = w2;
      // sums over the eight lanes of a step
#pragma unroll
      for (int o = 4; o > 0; o >>= 1) {      // sums of small integers: exact in f32
        fs1 += __shfl_xor_sync(0xffffffffu, fs1, o);
        fs2 += __shfl_xor_sync(0xffffffffu, fs2, o);
      }
      if ((lane & 7) == 0) {
        const int j = lane >> 3;
        const int s1 = (int)fs1, s2 = (int)fs2;
        S16Step r;
        r.og0 = -s1 * (1 << (2 * j));
        r.og1 = -s2 * (1 << (2 * j));
        r.sx = sx * (1.0f / (float)(1 << (2 * j)));
        r.pad = 0.0f;
        steps[(size_t)(c >> 5) * 4 + j] = r;
      }
    };
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int c = tid + i * NT;
      if (c < nch) emit(c, keep[i]);
    }
    for (int c = tid + 2 * NT; c < nch; c += NT) emit(c, x4[c]);
    s16_bar();
  }

  // ---- main loop: kS16Bpw consecutive blocks per warp per stage ----
  {
    const int g = lane >> 2, t = lane & 3;
    // this lane supplies output column n = g = 2 * step + term of every B operand
    const int my_step = g >> 1;
    const uint32_t sel[4] = {my_step == 0 ? 1u : 0u, my_step == 1 ? 1u : 0u, my_step == 2 ? 1u : 0u, my_step == 3 ? 1u : 0u};
    const int8_t* xq_lane = xq + (g & 1) * term_stride + 32 * my_step + 8 * t;   // + 128 * group
    const S16Step* st_lane = steps + t;                                  // + 4 * group: the lane's accumulator columns belong to step t
    const bool aligned = (ng % kS16Bpw) == 0;                            // a warp's blocks of a stage then share their tile
    int cur_tile = -1;
    float tot_lo = 0.0f, tot_hi = 0.0f;
    auto flush = [&]() {
      // the four lanes of a quad hold the four steps' shares of rows g and g + 8
      tot_lo += __shfl_xor_sync(0xffffffffu, tot_lo, 1);
      tot_hi += __shfl_xor_sync(0xffffffffu, tot_hi, 1);
      tot_lo += __shfl_xor_sync(0xffffffffu, tot_lo, 2);
      tot_hi += __shfl_xor_sync(0xffffffffu, tot_hi, 2);
      if (cur_tile >= 0 && t == 0) {
        float* p = part + ((size_t)cur_tile * kS16Warps + warp) * 16;
        p[g] += tot_lo;
        p[g + 8] += tot_hi;
      }
      tot_lo = tot_hi = 0.0f;
    };
    // (tile, group) of the warp's first block of the current stage, advanced by one stage's blocks per iteration
    int tl = (kS16Bpw * warp) / ng, grp = (kS16Bpw * warp) - tl * ng;
    int slot = 0;
    uint32_t phase = 0;
    for (int s = 0; s < nstage_total; ++s) {
      if (!s16_wait(&full[slot], phase, lane, abort_flag)) break;
      const uint8_t* st = ring + (size_t)slot * kS16StageBytes + (size_t)(kS16Bpw * warp) * kS16BlockBytes;
      const int left = nb_total - (s * kS16StageBlocks + kS16Bpw * warp);   // blocks of the stream from the warp's first one on
      if (aligned && left >= kS16Bpw) {
        if (tl != cur_tile) {           // warp-uniform
          flush();
          cur_tile = tl;
        }
        s16_blocks<kS16Bpw>(st, xq_lane + (size_t)grp * 128, st_lane + (size_t)grp * 4, lane, sel, tot_lo, tot_hi);
      } else {
        int tl_i = tl, grp_i = grp;
        for (int i = 0; i < kS16Bpw && i < left; ++i) {
          if (tl_i != cur_tile) {
            flush();
            cur_tile = tl_i;
          }
          s16_block(st + (size_t)i * kS16BlockBytes, xq_lane + (size_t)grp_i * 128, st_lane + (size_t)grp_i * 4, lane, sel, tot_lo, tot_hi);
          if (++grp_i == ng) {
            grp_i = 0;
            ++tl_i;
          }
        }
      }
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(&empty[slot]);
      if (++slot == kS16Stages) {
        slot = 0;
        phase ^= 1u;
      }
      grp += kS16StageBlocks;
      while (grp >= ng) {
        grp -= ng;
        ++tl;
      }
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
      if (tp.mc != nullptr) {   // one multicast store: the switch replicates it into every rank's slot
        tp_mc_st_msg(tp_ll_slot_mc(tp, parity, tp.rank) + row, msg);
      } else {
        for (int p = 0; p < tp.size; ++p)
          if (p != tp.rank) tp_st_msg(tp_ll_slot(tp, p, parity, tp.rank) + row, msg);
      }
      const float res = a.residual != nullptr ? a.residual[row] : 0.0f;
      bool alive = true;
      a.out[row] = tp_recv_sum(tp, [&](int s) { return tp_ll_slot(tp, tp.rank, parity, s) + row; }, tag, v, res, alive);
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
// Code word i (0..3) of lane (g, t): rows g (i even) or g + 8 (i odd) of the tile; byte b, 2-bit field j = the code of
// input 128 * group + 32 * j + 8 * t + (i >= 2 ? 4 : 0) + b.
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
      for (int b = 0; b < 4; ++b) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint32_t c = 1u;   // zero weight
          if (row < N) {
            const int k = grp * 128 + 32 * j + 8 * t + ((wi & 2) ? 4 : 0) + b;
            const uint32_t pw = codes[(size_t)row * wpr + (k >> 4)];
            const int jj = k & 15, i = jj & 7;
            const uint32_t nib = (pw >> (4 * i)) & 0xFu;
            const uint32_t m = jj < 8 ? (nib >> 1) & 1u : nib & 1u;
            const uint32_t sgn = jj < 8 ? (nib >> 3) & 1u : (nib >> 2) & 1u;
            c = m ? (sgn ? 0u : 2u) : 1u;
          }
          o |= c << (8 * b + 2 * j);
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

static inline size_t s16_smem_bytes(int K) {
  const int ng = K / 128;
  return (size_t)kS16Stages * kS16StageBytes + 2 * (size_t)(K + 32) + (size_t)ng * 4 * sizeof(S16Step) +
         (size_t)kS16MaxTiles * kS16Warps * 16 * 4 + 2 * kS16Stages * 8 + 32 * 4 + 16;
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

// Whether later launches of bonsai_bitgemv_s16 in this process use programmatic dependent launch (default: yes).
int bonsai_s16_tune(int pdl) {
  bonsai::g_s16_pdl = pdl != 0;
  return BONSAI_CUDA_OK;
}

// out = W x for an S16 matrix (see the head of this file): out[N] for epi 0 / 1 (1 adds residual[N]), out[N/2] for
// epi 2 (SwiGLU over interleaved gate/up rows), and for epi 3 out[N] = residual[N] + sum over the ranks of `comm` of
// their W x (every rank launches the same call on its shard; residual may be null).  x is f32[K], RMS-normalised with
// norm_w first when that is non-null.  K % 128 == 0, 128 <= K <= 16384, at most 12 row tiles per CTA.  `status`
// (device int, may be null) is set to 5 if a bounded wait on the copy pipeline expired.
static int bitgemv_s16_launch(const void* w16, const float* x, const float* norm_w, float eps, float* out, const float* residual,
                              int N, int K, int epi, const void* comm, int* status, const void* next_w, size_t next_bytes,
                              cudaStream_t stream) {
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
  const size_t smem = s16_smem_bytes(K);
  static bool attr_set[64] = {};   // per device: the attribute belongs to the device's copy of the function
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return BONSAI_CUDA_LAUNCH_FAILED;
  if (!attr_set[dev]) {
    if (cudaFuncSetAttribute(bitgemv_s16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024) != cudaSuccess)
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
  a.next_w = static_cast<const uint8_t*>(next_w);
  a.next_bytes = next_w != nullptr ? next_bytes : 0;
  cudaError_t e;
  if (g_s16_pdl) {
    e = launch_pdl(bitgemv_s16_kernel, dim3(grid), dim3(kS16Threads), smem, stream, a, tp);
  } else {
    bitgemv_s16_kernel<<<grid, kS16Threads, smem, stream>>>(a, tp);
    e = cudaGetLastError();
  }
  return e == cudaSuccess ? BONSAI_CUDA_OK : BONSAI_CUDA_LAUNCH_FAILED;
}

int bonsai_bitgemv_s16(const void* w16, const float* x, const float* norm_w, float eps, float* out, const float* residual,
                       int N, int K, int epi, const void* comm, int* status, cudaStream_t stream) {
  return bitgemv_s16_launch(w16, x, norm_w, eps, out, residual, N, K, epi, comm, status, nullptr, 0, stream);
}

// The same, and while it runs the kernel requests `next_bytes` bytes at `next_w` (16-byte aligned; the weights of the
// GEMV that follows in the stream) into L2.
int bonsai_bitgemv_s16_pf(const void* w16, const float* x, const float* norm_w, float eps, float* out, const float* residual,
                          int N, int K, int epi, const void* comm, int* status, const void* next_w, size_t next_bytes,
                          cudaStream_t stream) {
  if (next_w != nullptr && (reinterpret_cast<uintptr_t>(next_w) & 15) != 0) return BONSAI_CUDA_BAD_ARG;
  return bitgemv_s16_launch(w16, x, norm_w, eps, out, residual, N, K, epi, comm, status, next_w, next_bytes, stream);
}

}  // extern "C"
