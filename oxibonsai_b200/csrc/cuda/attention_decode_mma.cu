// Split-KV decode attention for head_dim 128 over f16 pages on the warp-level tensor-core path.
//
// The CUDA-core decode kernel (attention_decode.cu, half a warp per token) executes ~190 warp instructions per
// (token, kv head): dot-product FMAs, 16-lane shuffle reductions and the online-softmax bookkeeping of every token.
// With 16 warps resident per SM that instruction stream, not HBM, bounds it (6.3 M warp instructions for 4096 tokens x 8
// kv heads; 0.39 of the measured copy bandwidth at 64 x 1024 tokens).  Here a warp handles 16 tokens at a time:
//   S = Q K^T      m16n8k16 MMAs, the query heads of the group as rows 0..G-1 of the 16-row A operand (rest zero)
//   P = softmax    on the accumulator fragments (a row lives in four lanes: two shuffles per reduction)
//   O += P V       m16n8k16 MMAs, P re-used from registers as the A operand, V through ldmatrix.trans
// K and V tiles (16 tokens x 256 bytes) come in through cp.async into padded shared-memory rows, double buffered per
// warp.  That is ~10 warp instructions per (token, kv head).  The work decomposition, the workspace format and the
// last-CTA merge over splits are those of the CUDA-core kernel, so the two are interchangeable behind
// bonsai_attn_decode.  Reference behaviour: crates/oxibonsai-kernels/src/gpu_backend/cuda_attn_kernels.rs
// (single-query attention over the cached K/V of one sequence), which walks one head per block on CUDA cores.
#include <cuda_fp16.h>

#include <cooperative_groups.h>

#include "common.cuh"

namespace bonsai {

constexpr int kMmaTile = 16;                          // tokens per warp tile
constexpr int kMmaRow = 272;                          // bytes per token row in shared memory: 256 + 16 (bank spread)
constexpr int kMmaTileBytes = kMmaTile * kMmaRow;     // 4352
constexpr int kMmaHd = 128;

__device__ __forceinline__ uint32_t mma_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
// 16-byte asynchronous copy; src_bytes = 0 writes zeros without reading the source
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
// D (16x8, f32) += A (16x16, f16, row) * B (16x8, f16, col)
__device__ __forceinline__ void mma_16816(float* d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
  const __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}

struct MmaAttnParams {
  const float* q;            // [batch][nq][128] f32
  const int* positions;
  const int* block_table;    // [batch][max_pages]
  const uint8_t* k;          // this layer's pools, f16 rows of 256 bytes: [(page * nkv + kvh) * page_size + slot]
  const uint8_t* v;
  float* ws_acc;             // [batch][nq][nsplit][128]
  float* ws_ml;              // [batch][nq][nsplit][2]
  int* counters;             // [batch][nkv], zero between launches
  float* out;                // [batch][nq][128]
  int max_pages, nq, nkv, page_size, extra_len;
  float sm_scale;
  // Fused mode (qkv != null, extra_len == 0): the kernel takes the raw projections of the new token
  // ([batch][qkv_stride] f32: q heads | k heads | v heads), applies QK-RMSNorm and RoPE itself, and the CTA whose split
  // holds the new position appends the K and V rows to the cache before it reads them.  One launch per layer less.
  const float* qkv;
  const float* q_norm;
  const float* k_norm;
  const float* rope_cos;     // [position][64]
  const float* rope_sin;
  int qkv_stride;
  float eps;
};

__device__ __forceinline__ float mma_warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// NW warps per CTA: 8 when the grid is about one CTA per SM (a single sequence: each warp then walks half as many
// tiles; 479 vs 466 tok/s end to end), 4 with two CTAs per SM when many sequences fill the GPU (57 vs 63-70 us for
// 64 x 1024 tokens).
// CL: the splits of one (sequence, kv head) form a thread-block cluster (cluster dimension = the grid's y extent) and meet
// in the shared memory of the cluster's first CTA instead of in global memory.
template <int G, int NW, bool CL>
__global__ void __launch_bounds__(NW * 32, 8 / NW) attn_decode_mma_kernel(MmaAttnParams p) {
  constexpr int kMmaWarps = NW;
  constexpr int hd = kMmaHd;
  extern __shared__ __align__(16) uint8_t smem_raw[];
  // [warp][buffer][K | V] tiles, then the warp-merge staging area [warp][G][hd + 2] floats
  uint8_t* tiles = smem_raw;
  float* sh = reinterpret_cast<float*>(smem_raw + kMmaWarps * 4 * kMmaTileBytes);
  __shared__ int s_last;
  const int kvh = blockIdx.x, split = blockIdx.y, nsplit = gridDim.y, b = blockIdx.z;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int row = lane >> 2, cq = lane & 3;   // accumulator row (query head of the group) and column pair of this lane
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  // Distributed shared memory may only be touched once every CTA of the cluster runs: all threads arrive here and wait
  // just before the remote writes, by which time the barrier has long completed.
  if constexpr (CL) asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
  // Fused mode: the kernel before this one in the stream is the QKV projection, which writes nothing but the raw
  // projections - positions, block table and the cached K/V rows of earlier tokens are older than it.  The wait
  // therefore comes after the page lookups and the first K/V tile requests, just before the projections are read.
  // Otherwise (the queries and the new K/V rows come from the kernel before) it comes first.
  if (p.qkv == nullptr) asm volatile("griddepcontrol.wait;" ::: "memory");
  const int len = p.positions[b] + 1 + p.extra_len;
  int chunk = (len + nsplit - 1) / nsplit;
  chunk = (chunk + kMmaTile - 1) & ~(kMmaTile - 1);   // tiles never straddle a split boundary or (page_size >= 16) a page
  const int t0 = split * chunk, t1 = min(len, t0 + chunk);
  const int ntiles = t1 > t0 ? (t1 - t0 + kMmaTile - 1) / kMmaTile : 0;
  const int* bt = p.block_table + (size_t)b * p.max_pages;
  const int pshift = 31 - __clz(p.page_size), pmask = p.page_size - 1;

  uint8_t* wt = tiles + (size_t)warp * 4 * kMmaTileBytes;
  auto issue_tile = [&](int j, int buf) {   // tile j of the CTA -> K, V buffers `buf` of this warp
    const int tb = t0 + j * kMmaTile;
    const int page = bt[tb >> pshift];
    const size_t rowbase = ((size_t)page * p.nkv + kvh) * p.page_size + (tb & pmask);
    const uint32_t kd = mma_smem_u32(wt + (2 * buf) * kMmaTileBytes), vd = kd + kMmaTileBytes;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int c = i * 32 + lane, r = c >> 4, c16 = c & 15;
      // rows past the end of the sequence are zero-filled: their scores are masked, but 0 x (stale NaN in V) is NaN
      const int nb = tb + r < t1 ? 16 : 0;
      cp_async16(kd + r * kMmaRow + c16 * 16, p.k + (rowbase + r) * 256 + c16 * 16, nb);
      cp_async16(vd + r * kMmaRow + c16 * 16, p.v + (rowbase + r) * 256 + c16 * 16, nb);
    }
  };
  // The first tile of every warp is requested before the queries are prepared, so the two latencies overlap - unless
  // it holds the position whose K and V rows are appended below.
  const int first_tb = t0 + warp * kMmaTile;
  const bool early = warp < ntiles && !(p.qkv != nullptr && len - 1 >= first_tb && len - 1 < first_tb + kMmaTile);
  if (early) issue_tile(warp, 0);
  if (p.qkv != nullptr) asm volatile("griddepcontrol.wait;" ::: "memory");

  // Q as A-operand fragments: rows 0..G-1 hold the group's query heads (scaled), rows G..15 are zero
  uint32_t qa[8][2];   // per 16-wide k step: a0 (row, k lo pair) and a2 (row, k hi pair); a1 = a3 = 0 (rows 8..15)
  const float* qp = p.q + ((size_t)b * p.nq + kvh * G + (row < G ? row : 0)) * hd;
  float q_mul = p.sm_scale;
  if (p.qkv != nullptr) {
    // a warp per item: the G query heads, plus the new token's K and V rows in the CTA that owns position len - 1
    float* qs = sh;                                          // [G][128] normalised, rotated, scaled queries
    const int pos = len - 1;
    const bool owner = pos >= t0 && pos < t1;
    const float* raw = p.qkv + (size_t)b * p.qkv_stride;
    for (int it = warp; it < G + (owner ? 2 : 0); it += kMmaWarps) {
      const bool is_q = it < G, is_v = it == G + 1;
      const float* src = raw + (size_t)(is_q ? kvh * G + it : (is_v ? p.nq + p.nkv + kvh : p.nq + kvh)) * hd;
      float y0 = src[lane], y1 = src[lane + 32], y2 = src[lane + 64], y3 = src[lane + 96];
      if (!is_v) {
        const float inv = 1.0f / sqrtf(mma_warp_sum(y0 * y0 + y1 * y1 + y2 * y2 + y3 * y3) / (float)hd + p.eps);
        const float* w = is_q ? p.q_norm : p.k_norm;
        const float n0 = w[lane] * y0 * inv, n1 = w[lane + 32] * y1 * inv, n2 = w[lane + 64] * y2 * inv, n3 = w[lane + 96] * y3 * inv;
        const float c0 = p.rope_cos[(size_t)pos * 64 + lane], s0 = p.rope_sin[(size_t)pos * 64 + lane];
        const float c1 = p.rope_cos[(size_t)pos * 64 + lane + 32], s1 = p.rope_sin[(size_t)pos * 64 + lane + 32];
        y0 = n0 * c0 - n2 * s0; y2 = n0 * s0 + n2 * c0;      // dims (lane, lane + 64)
        y1 = n1 * c1 - n3 * s1; y3 = n1 * s1 + n3 * c1;      // dims (lane + 32, lane + 96)
      }
      if (is_q) {
        float* dst = qs + it * hd;
        dst[lane] = y0 * p.sm_scale; dst[lane + 32] = y1 * p.sm_scale; dst[lane + 64] = y2 * p.sm_scale; dst[lane + 96] = y3 * p.sm_scale;
      } else {
        const int page = bt[pos >> pshift];
        const size_t crow = ((size_t)page * p.nkv + kvh) * p.page_size + (pos & pmask);
        __half* dst = reinterpret_cast<__half*>(const_cast<uint8_t*>(is_v ? p.v : p.k)) + crow * hd;
        dst[lane] = __float2half_rn(y0); dst[lane + 32] = __float2half_rn(y1); dst[lane + 64] = __float2half_rn(y2); dst[lane + 96] = __float2half_rn(y3);
      }
    }
    if (owner) __threadfence();                              // the appended rows are read back through cp.async below
    __syncthreads();
    qp = qs + (row < G ? row : 0) * hd;
    q_mul = 1.0f;
  }
  {
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      const float2 lo = *reinterpret_cast<const float2*>(qp + ks * 16 + 2 * cq);
      const float2 hi = *reinterpret_cast<const float2*>(qp + ks * 16 + 8 + 2 * cq);
      qa[ks][0] = row < G ? pack_h2(lo.x * q_mul, lo.y * q_mul) : 0u;
      qa[ks][1] = row < G ? pack_h2(hi.x * q_mul, hi.y * q_mul) : 0u;
    }
  }
  if (p.qkv != nullptr) __syncthreads();                     // the staging area is reused for the warp merge later
  float o[16][4];   // O accumulators: 16 column tiles of 8 dims; [.][0..1] = this lane's row, [.][2..3] = row + 8 (unused)
#pragma unroll
  for (int nt = 0; nt < 16; ++nt) o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.0f;
  float m = -INFINITY, l = 0.0f;   // running max of the row (same in the row's four lanes) and this lane's share of the sum

  int buf = 0;
  if (warp < ntiles && !early) issue_tile(warp, 0);
  cp_async_commit();
  for (int j = warp; j < ntiles; j += kMmaWarps, buf ^= 1) {
    if (j + kMmaWarps < ntiles) issue_tile(j + kMmaWarps, buf ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncwarp();
    const uint32_t kb = mma_smem_u32(wt + (2 * buf) * kMmaTileBytes), vb = kb + kMmaTileBytes;
    // ---- S = Q K^T for 16 tokens: two 8-token column tiles --------------------------------------
    float s[2][4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.0f;
#pragma unroll
      for (int ks = 0; ks < 8; ks += 2) {
        // matrices: (k lo, ks), (k hi, ks), (k lo, ks + 1), (k hi, ks + 1) of tokens nt*8 .. nt*8+7
        const int mi = lane >> 3, r = lane & 7;
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4(kb + (nt * 8 + r) * kMmaRow + ((ks + (mi >> 1)) * 16 + (mi & 1) * 8) * 2, b0, b1, b2, b3);
        mma_16816(s[nt], qa[ks][0], 0u, qa[ks][1], 0u, b0, b1);
        mma_16816(s[nt], qa[ks + 1][0], 0u, qa[ks + 1][1], 0u, b2, b3);
      }
    }
    // ---- online softmax on the row of this lane (tokens tb + nt*8 + 2*cq + {0,1}) ------------------
    const int tb = t0 + j * kMmaTile;
    float mx = m;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        if (tb + nt * 8 + 2 * cq + e >= t1) s[nt][e] = -INFINITY;
        mx = fmaxf(mx, s[nt][e]);
      }
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float resc = (mx == -INFINITY) ? 1.0f : __expf(m - mx);   // exp(-inf) = 0 before the first token
    float pr[2][2], ps = 0.0f;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        pr[nt][e] = (mx == -INFINITY) ? 0.0f : __expf(s[nt][e] - mx);
        ps += pr[nt][e];
      }
    l = l * resc + ps;
    m = mx;
#pragma unroll
    for (int nt = 0; nt < 16; ++nt) {
      o[nt][0] *= resc;
      o[nt][1] *= resc;
    }
    // ---- O += P V: P (16 x 16 tokens) straight from the score fragments ------------------------------
    const uint32_t pa0 = pack_h2(pr[0][0], pr[0][1]), pa2 = pack_h2(pr[1][0], pr[1][1]);
#pragma unroll
    for (int nt = 0; nt < 16; nt += 2) {
      // matrices: (tokens 0-7, dims nt), (tokens 8-15, dims nt), (tokens 0-7, dims nt + 1), (tokens 8-15, dims nt + 1)
      const int mi = lane >> 3, r = lane & 7;
      uint32_t b0, b1, b2, b3;
      ldmatrix_x4_trans(vb + ((mi & 1) * 8 + r) * kMmaRow + ((nt + (mi >> 1)) * 8) * 2, b0, b1, b2, b3);
      mma_16816(o[nt], pa0, 0u, pa2, 0u, b0, b1);
      mma_16816(o[nt + 1], pa0, 0u, pa2, 0u, b2, b3);
    }
    __syncwarp();   // every lane is done with this buffer before the next iteration's copies overwrite it
  }
  cp_async_wait<0>();
  l += __shfl_xor_sync(0xffffffffu, l, 1);
  l += __shfl_xor_sync(0xffffffffu, l, 2);

  // ---- combine the warps of the CTA ----------------------------------------------------------------
  const int stride = hd + 2;
  if (row < G) {
    float* dst = sh + ((size_t)warp * G + row) * stride;
#pragma unroll
    for (int nt = 0; nt < 16; ++nt) {
      dst[nt * 8 + 2 * cq] = o[nt][0];
      dst[nt * 8 + 2 * cq + 1] = o[nt][1];
    }
    if (cq == 0) {
      dst[hd] = m;
      dst[hd + 1] = l;
    }
  }
  __syncthreads();
  if constexpr (CL) {
    // ---- the splits meet in the first CTA's shared memory --------------------------------------------------------------
    // Every CTA of the cluster writes its (partial sum, max, sum) rows into slot [its rank] of the merge area of CTA 0
    // through distributed shared memory, the cluster barrier (release / acquire) orders the writes before CTA 0's reads,
    // and CTA 0 folds the slots.  Every thread of every CTA passes the same two barrier phases on every path (there is
    // no early exit before them).  No global workspace, fence, counter or reload.
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    const unsigned rank = cluster.block_rank();                 // = split: the cluster spans the grid's y extent
    float* merge = sh + (size_t)kMmaWarps * G * stride;         // [nsplit][G][hd + 2], used in CTA 0 only
    float* lead = cluster.map_shared_rank(merge, 0);
    asm volatile("barrier.cluster.wait.aligned;" ::: "memory");   // the arrival at the top of the kernel: every CTA runs
    for (int idx = threadIdx.x; idx < G * hd; idx += blockDim.x) {
      const int g = idx / hd, d = idx - g * hd;
      float M = -INFINITY;
#pragma unroll
      for (int w = 0; w < kMmaWarps; ++w) M = fmaxf(M, sh[((size_t)w * G + g) * stride + hd]);
      float a = 0.0f, L = 0.0f;
#pragma unroll
      for (int w = 0; w < kMmaWarps; ++w) {
        const float* src = sh + ((size_t)w * G + g) * stride;
        const float f = (src[hd] == -INFINITY) ? 0.0f : __expf(src[hd] - M);
        a += f * src[d];
        L += f * src[hd + 1];
      }
      float* dst = lead + ((size_t)rank * G + g) * stride;
      dst[d] = a;
      if (d == 0) {
        dst[hd] = M;
        dst[hd + 1] = L;
      }
    }
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (rank != 0) return;
    float* s_f = sh;                                            // [G][nsplit] normalised weights of the splits
    for (int g = warp; g < G; g += kMmaWarps) {
      float M = -INFINITY;
      for (int sp = lane; sp < nsplit; sp += 32) M = fmaxf(M, merge[((size_t)sp * G + g) * stride + hd]);
#pragma unroll
      for (int o2 = 16; o2 > 0; o2 >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o2));
      float L = 0.0f;
      for (int sp = lane; sp < nsplit; sp += 32) {
        const float ms = merge[((size_t)sp * G + g) * stride + hd];
        const float f = (ms == -INFINITY) ? 0.0f : __expf(ms - M);
        L += f * merge[((size_t)sp * G + g) * stride + hd + 1];
        s_f[g * nsplit + sp] = f;
      }
#pragma unroll
      for (int o2 = 16; o2 > 0; o2 >>= 1) L += __shfl_xor_sync(0xffffffffu, L, o2);
      const float inv = L > 0.0f ? 1.0f / L : 0.0f;
      __syncwarp();
      for (int sp = lane; sp < nsplit; sp += 32) s_f[g * nsplit + sp] *= inv;
    }
    __syncthreads();
    const size_t hb = (size_t)b * p.nq + kvh * G;
    for (int idx = threadIdx.x; idx < G * hd; idx += blockDim.x) {
      const int g = idx / hd, d = idx - g * hd;
      float a = 0.0f;
      for (int sp = 0; sp < nsplit; ++sp) a += s_f[g * nsplit + sp] * merge[((size_t)sp * G + g) * stride + d];
      p.out[hb * hd + idx] = a;
    }
    return;
  }
  for (int idx = threadIdx.x; idx < G * hd; idx += blockDim.x) {
    const int g = idx / hd, d = idx - g * hd;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kMmaWarps; ++w) M = fmaxf(M, sh[((size_t)w * G + g) * stride + hd]);
    float a = 0.0f, L = 0.0f;
#pragma unroll
    for (int w = 0; w < kMmaWarps; ++w) {
      const float* src = sh + ((size_t)w * G + g) * stride;
      const float f = (src[hd] == -INFINITY) ? 0.0f : __expf(src[hd] - M);
      a += f * src[d];
      L += f * src[hd + 1];
    }
    const size_t oi = (((size_t)b * p.nq + kvh * G + g) * nsplit + split);
    p.ws_acc[oi * hd + d] = a;
    if (d == 0) {
      p.ws_ml[oi * 2] = M;
      p.ws_ml[oi * 2 + 1] = L;
    }
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    int* ctr = p.counters + (size_t)b * p.nkv + kvh;
    const int prev = atomicAdd(ctr, 1);
    s_last = (prev == nsplit - 1);
    if (s_last) *ctr = 0;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  // ---- merge of the splits by the last CTA of this (sequence, kv head): see attention_decode.cu -----
  float* s_f = sh;
  float* s_l = sh + G * nsplit;
  const size_t hb0 = (size_t)b * p.nq + kvh * G;
  constexpr int NI = (G * hd + kMmaWarps * 32 - 1) / (kMmaWarps * 32);   // outputs per thread
  constexpr int SB = NI >= 4 ? 5 : 20 / NI;                             // splits per step: ~20 loads in flight
  // The first SB splits' partial sums are requested together with the (max, sum) pairs: one trip to L2 instead of two.
  float av[NI][SB];
  auto load_acc = [&](int sp0) {
#pragma unroll
    for (int k = 0; k < NI; ++k) {
      const int idx = min((int)threadIdx.x + k * kMmaWarps * 32, G * hd - 1);
#pragma unroll
      for (int i = 0; i < SB; ++i)
        av[k][i] = sp0 + i < nsplit ? __ldcg(p.ws_acc + ((hb0 + idx / hd) * nsplit + sp0 + i) * hd + (idx % hd)) : 0.0f;
    }
  };
  load_acc(0);
  for (int i = threadIdx.x; i < G * nsplit; i += blockDim.x) {
    const float2 v = __ldcg(reinterpret_cast<const float2*>(p.ws_ml) + hb0 * nsplit + i);
    s_f[i] = v.x;
    s_l[i] = v.y;
  }
  __syncthreads();
  for (int g = warp; g < G; g += kMmaWarps) {   // one warp per query head of the group
    float M = -INFINITY;
    for (int sp = lane; sp < nsplit; sp += 32) M = fmaxf(M, s_f[g * nsplit + sp]);
#pragma unroll
    for (int o2 = 16; o2 > 0; o2 >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o2));
    float L = 0.0f;
    for (int sp = lane; sp < nsplit; sp += 32) {
      const float ms = s_f[g * nsplit + sp];
      const float f = (ms == -INFINITY) ? 0.0f : __expf(ms - M);
      L += f * s_l[g * nsplit + sp];
      s_f[g * nsplit + sp] = f;
    }
#pragma unroll
    for (int o2 = 16; o2 > 0; o2 >>= 1) L += __shfl_xor_sync(0xffffffffu, L, o2);
    const float inv = L > 0.0f ? 1.0f / L : 0.0f;
    __syncwarp();
    for (int sp = lane; sp < nsplit; sp += 32) s_f[g * nsplit + sp] *= inv;
  }
  __syncthreads();
  float a[NI];
#pragma unroll
  for (int k = 0; k < NI; ++k) a[k] = 0.0f;
  for (int sp0 = 0; sp0 < nsplit; sp0 += SB) {
    if (sp0 > 0) load_acc(sp0);
#pragma unroll
    for (int k = 0; k < NI; ++k) {
      const int idx = min((int)threadIdx.x + k * kMmaWarps * 32, G * hd - 1);
#pragma unroll
      for (int i = 0; i < SB; ++i) a[k] += (sp0 + i < nsplit ? s_f[(idx / hd) * nsplit + sp0 + i] : 0.0f) * av[k][i];
    }
  }
#pragma unroll
  for (int k = 0; k < NI; ++k) {
    const int idx = threadIdx.x + k * kMmaWarps * 32;
    if (idx < G * hd) p.out[hb0 * hd + idx] = a[k];
  }
}

template <int G, int NW>
static int launch_mma(const MmaAttnParams& p, dim3 grid, cudaStream_t st) {
  constexpr int kMmaWarps = NW;
  const size_t smem = (size_t)kMmaWarps * 4 * kMmaTileBytes + (size_t)kMmaWarps * G * (kMmaHd + 2) * sizeof(float);
  static bool configured[64] = {};   // per template instance and device: the attribute belongs to the function in a context
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return BONSAI_CUDA_LAUNCH_FAILED;
  if (!configured[dev]) {
    if (cudaFuncSetAttribute(attn_decode_mma_kernel<G, NW, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return BONSAI_CUDA_LAUNCH_FAILED;
    configured[dev] = true;
  }
  const cudaError_t e = launch_pdl(attn_decode_mma_kernel<G, NW, false>, grid, dim3(kMmaWarps * 32), smem, st, p);
  return e == cudaSuccess ? BONSAI_CUDA_OK : BONSAI_CUDA_LAUNCH_FAILED;
}

// 0 = let the launcher decide, 1 = never use the cluster merge, 2 = use it wherever it can be launched
static int g_cluster_mode = 0;
// form of the last launch: 0 = splits merged through global memory, 8 / 4 = cluster merge with that many warps per CTA
static int g_last_form = 0;

// The cluster form: the grid's y extent (the splits) is the cluster dimension, 2 to 16 CTAs (more than 8 needs the
// non-portable opt-in).  Returns BONSAI_CUDA_BAD_ARG when the device cannot hold one such cluster, and the caller
// launches the plain form instead.
template <int G, int NW>
static int launch_mma_cluster(const MmaAttnParams& p, dim3 grid, cudaStream_t st) {
  const int nsplit = (int)grid.y;
  const size_t smem = (size_t)NW * 4 * kMmaTileBytes + (size_t)NW * G * (kMmaHd + 2) * sizeof(float) +
                      (size_t)nsplit * G * (kMmaHd + 2) * sizeof(float);
  if (smem > 227 * 1024) return BONSAI_CUDA_BAD_ARG;
  auto kernel = attn_decode_mma_kernel<G, NW, true>;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(NW * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = (unsigned)nsplit;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  // per (device, cluster size): attributes set; the number of clusters the device holds at once (-1 = none / refused)
  static int fits[64][17] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return BONSAI_CUDA_LAUNCH_FAILED;
  if (fits[dev][nsplit] == 0) {
    bool ok = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) == cudaSuccess;
    if (ok && nsplit > 8) ok = cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess;
    int n = 0;
    cudaLaunchConfig_t probe = cfg;
    probe.numAttrs = 1;                 // the occupancy query takes the cluster dimension only
    if (ok) ok = cudaOccupancyMaxActiveClusters(&n, kernel, &probe) == cudaSuccess && n >= 1;
    if (!ok) (void)cudaGetLastError();  // a refused attribute or query must not poison the next launch check
    fits[dev][nsplit] = ok ? n : -1;
  }
  // a second wave of clusters would cost more than the merge through global memory that this form saves
  if (fits[dev][nsplit] < (int)(grid.x * grid.z)) return BONSAI_CUDA_BAD_ARG;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, p);
  if (e == cudaSuccess) g_last_form = NW;
  return e == cudaSuccess ? BONSAI_CUDA_OK : BONSAI_CUDA_LAUNCH_FAILED;
}

struct MmaFused {
  const float* qkv = nullptr;
  const float* q_norm = nullptr;
  const float* k_norm = nullptr;
  const float* rope_cos = nullptr;
  const float* rope_sin = nullptr;
  int qkv_stride = 0;
  float eps = 0.0f;
};

static int attn_decode_mma_launch(const float* q, const MmaFused& f, const int* positions, const int* block_table, int max_pages, int batch,
                                  int nq, int nkv, int page_size, const void* kpool, const void* vpool, int nsplit, float* ws_acc,
                                  float* ws_ml, int* counters, float* out, int extra_len, float sm_scale, cudaStream_t stream) {
  const int G = nq / nkv;
  if (page_size < kMmaTile || (page_size & (page_size - 1)) != 0 || 2 * G * nsplit > 4 * G * (kMmaHd + 2)) return BONSAI_CUDA_BAD_ARG;
  MmaAttnParams p{q, positions, block_table, (const uint8_t*)kpool, (const uint8_t*)vpool, ws_acc, ws_ml, counters, out,
                  max_pages, nq, nkv, page_size, extra_len, sm_scale, f.qkv, f.q_norm, f.k_norm, f.rope_cos, f.rope_sin, f.qkv_stride, f.eps};
  const dim3 grid(nkv, nsplit, batch);
  const bool wide = (long long)nkv * nsplit * batch <= 296;   // about one CTA per SM: eight warps each
  // Few CTAs (one sequence, or a handful): the splits of a (sequence, kv head) run as one cluster and merge through
  // distributed shared memory, which takes the global round trip (partial store, fence, counter, reload) out of a
  // kernel that is all latency at this size.
  if (g_cluster_mode != 1 && wide && (nsplit == 2 || nsplit == 4 || nsplit == 8 || nsplit == 16)) {
    // Eight warps per CTA, one CTA per SM: a cluster of 16 needs 16 SMs of one GPC, so eight such clusters (one sequence,
    // eight kv heads) do not all fit and that shape keeps the global merge unless it is launched with 8 splits.  A
    // four-warp form at two CTAs per SM does fit but measured slower inside a decode step (1.633 against 1.613 ms).
    int rc = BONSAI_CUDA_BAD_ARG;
    switch (G) {
      case 1: rc = launch_mma_cluster<1, 8>(p, grid, stream); break;
      case 2: rc = launch_mma_cluster<2, 8>(p, grid, stream); break;
      case 4: rc = launch_mma_cluster<4, 8>(p, grid, stream); break;
      case 8: rc = launch_mma_cluster<8, 8>(p, grid, stream); break;
      default: break;
    }
    if (rc != BONSAI_CUDA_BAD_ARG) return rc;
  }
  g_last_form = 0;
  switch (G) {
    case 1: return wide ? launch_mma<1, 8>(p, grid, stream) : launch_mma<1, 4>(p, grid, stream);
    case 2: return wide ? launch_mma<2, 8>(p, grid, stream) : launch_mma<2, 4>(p, grid, stream);
    case 4: return wide ? launch_mma<4, 8>(p, grid, stream) : launch_mma<4, 4>(p, grid, stream);
    case 8: return wide ? launch_mma<8, 8>(p, grid, stream) : launch_mma<8, 4>(p, grid, stream);
    default: return BONSAI_CUDA_BAD_ARG;
  }
}

// Returns BONSAI_CUDA_BAD_ARG for shapes it does not cover; the caller then uses the CUDA-core kernel.
int attn_decode_mma_f16(const float* q, const int* positions, const int* block_table, int max_pages, int batch, int nq, int nkv,
                        int page_size, const void* kpool, const void* vpool, int nsplit, float* ws_acc, float* ws_ml, int* counters,
                        float* out, int extra_len, float sm_scale, cudaStream_t stream) {
  return attn_decode_mma_launch(q, MmaFused{}, positions, block_table, max_pages, batch, nq, nkv, page_size, kpool, vpool, nsplit, ws_acc,
                                ws_ml, counters, out, extra_len, sm_scale, stream);
}

}  // namespace bonsai

extern "C" {

// 0 = cluster merge where the launcher finds it fits (default), 1 = never, 2 = same as 0 (kept for symmetry of the A/B switch).
void bonsai_attn_decode_cluster_mode(int mode) { bonsai::g_cluster_mode = mode; }
int bonsai_attn_decode_last_form() { return bonsai::g_last_form; }

// QK-RMSNorm + RoPE + KV append + split-KV attention of one new token per sequence in a single launch, for f16 pages
// and head_dim 128.  qkv: f32 [batch][qkv_stride] raw projections (q heads | k heads | v heads); positions[b] is the
// position of the new token, whose K and V rows are appended to the pools.  Returns BONSAI_CUDA_BAD_ARG for shapes it
// does not cover (the caller then runs bonsai_qknorm_rope_kvstore + bonsai_attn_decode).
int bonsai_attn_decode_qkv_f16(const float* qkv, int qkv_stride, const float* q_norm, const float* k_norm, float eps,
                               const float* rope_cos, const float* rope_sin, const int* positions, const int* block_table,
                               int max_pages, int batch, int nq, int nkv, int hd, int page_size, void* kpool, void* vpool, int nsplit,
                               float* ws_acc, float* ws_ml, int* counters, float* out, cudaStream_t stream) {
  using namespace bonsai;
  if (hd != kMmaHd || nq % nkv != 0 || nsplit < 1 || batch <= 0 || counters == nullptr || qkv == nullptr) return BONSAI_CUDA_BAD_ARG;
  MmaFused f;
  f.qkv = qkv; f.q_norm = q_norm; f.k_norm = k_norm; f.rope_cos = rope_cos; f.rope_sin = rope_sin; f.qkv_stride = qkv_stride; f.eps = eps;
  return attn_decode_mma_launch(nullptr, f, positions, block_table, max_pages, batch, nq, nkv, page_size, kpool, vpool, nsplit, ws_acc,
                                ws_ml, counters, out, 0, 1.0f / sqrtf((float)hd), stream);
}

}  // extern "C"
