// Causal GQA attention for prefill chunks over the paged KV cache.
//
// The reference's "batch" prefill runs attention one token at a time, re-launching the decode
// attention kernels per token per layer (crates/oxibonsai-kernels/src/gpu_backend/cuda_prefill/encode_ternary.rs:209-274),
// about a million launches for a 4096-token prompt.  This kernel processes a chunk of T new tokens
// of one sequence at once: a CTA owns 64 query rows of one head, streams the keys/values of the
// sequence (everything before the chunk plus the causal part of the chunk) in blocks of 64 from the
// page pool, and keeps the online-softmax state in registers (flash-attention style).  The score
// and value products run on the tensor cores through warp-level mma (m16n8k16, f16 in / f32
// accumulate); the matrix sizes per CTA (64 x 64 x head_dim) are too small to amortise a
// TMEM-resident tcgen05 pipeline, and the prefill time is dominated by the GEMMs.
//
// q: f32 [T][nq][hd] (already normalised and rotated); output: f16 [T][nq*hd] in the paired-K order
// that the attention-output GEMM consumes.  KV formats: F32 / F16 / Q8 / Q4 pages (dequantised to
// f16 while staging a block in shared memory).
#include <cuda_fp16.h>

#include "common.cuh"

namespace bonsai {

__host__ __device__ inline int pf_paired_k(int k) {
  int j = k & 15, hi = j & 8, p = j & 3, q = (j >> 2) & 1;
  return (k & ~15) | hi | (p * 2 + q);
}

// position of logical input k in the K order of the mma.sync decode-batch GEMM (a permutation inside every 128 inputs;
// the same map as hmma_k_pos in bitgemm_hmma.cu)
__host__ __device__ inline int pf_hmma_k(int k) {
  const int r = k & 127, wq = r >> 4, e = r & 15;
  const int c = wq >> 1, j = wq & 1, plane = e >> 3, p = e & 3, h = (e >> 2) & 1;
  return (k & ~127) | ((j * 4 + p) * 16 + plane * 8 + 2 * c + h);
}
__host__ __device__ inline int pf_out_k(int k, int order) { return order == 1 ? pf_hmma_k(k) : pf_paired_k(k); }

struct PfKvPool {
  const uint8_t* k;
  const uint8_t* v;
  const float* k_scale;
  const float* v_scale;
  int page_size, kv_heads, hd, kvt;
};

__device__ __forceinline__ void ldmatrix_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
  uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
  uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void mma16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Stage rows [t0, t0+64) of one kv head into shared memory as f16 [64][HD + 8].
template <int HD>
__device__ __forceinline__ void stage_kv(__half* __restrict__ dst, const uint8_t* __restrict__ pool, const float* __restrict__ scales,
                                         const PfKvPool& kv, const int* __restrict__ bt, int kvh, int t0, int t_end) {
  constexpr int LD = HD + 8;
  // 64 rows x HD/8 chunks of eight elements; the block has 128 threads
#pragma unroll 4
  for (int i = 0; i < 64 * (HD / 8) / 128; ++i) {
    const int idx = threadIdx.x + i * 128;
    const int r = idx / (HD / 8), c8 = (idx % (HD / 8)) * 8;
    const int t = t0 + r;
    __half h[8];
    if (t < t_end) {
      const int page = bt[t / kv.page_size];
      const size_t row = ((size_t)page * kv.kv_heads + kvh) * kv.page_size + (t % kv.page_size);
      if (kv.kvt == 1) {
        *reinterpret_cast<uint4*>(h) = *reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(pool) + row * HD + c8);
      } else if (kv.kvt == 0) {
        const float* p = reinterpret_cast<const float*>(pool) + row * HD + c8;
#pragma unroll
        for (int j = 0; j < 8; ++j) h[j] = __float2half_rn(p[j]);
      } else if (kv.kvt == 2) {
        const int8_t* p = reinterpret_cast<const int8_t*>(pool) + row * HD + c8;
        const float s = scales[row];
#pragma unroll
        for (int j = 0; j < 8; ++j) h[j] = __float2half_rn(s * (float)p[j]);
      } else {
        const uint8_t* p = pool + row * (HD / 2) + c8 / 2;
        const float s = scales[row];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          h[2 * j] = __float2half_rn(s * (float)((int)(p[j] & 15u) - 8));
          h[2 * j + 1] = __float2half_rn(s * (float)((int)(p[j] >> 4) - 8));
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) h[j] = __float2half(0.0f);
    }
    *reinterpret_cast<uint4*>(dst + r * LD + c8) = *reinterpret_cast<uint4*>(h);
  }
}

__device__ __forceinline__ void pf_cp_async16(void* dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src), "r"(src_bytes)
               : "memory");
}
__device__ __forceinline__ void pf_cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void pf_cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// f16 pages: rows [t0, t0+64) of one kv head go straight from the pool into shared memory with 16-byte asynchronous copies
// (rows past t_end are zero-filled), all of a thread's copies in flight at once.
template <int HD>
__device__ __forceinline__ void stage_kv_async(__half* dst, const __half* pool, const PfKvPool& kv, const int* __restrict__ bt, int kvh,
                                               int t0, int t_end) {
  constexpr int LD = HD + 8;
#pragma unroll
  for (int i = 0; i < 64 * (HD / 8) / 128; ++i) {
    const int idx = threadIdx.x + i * 128;
    const int r = idx / (HD / 8), c8 = (idx % (HD / 8)) * 8;
    const int t = t0 + r;
    const bool ok = t < t_end;
    const int page = ok ? bt[t / kv.page_size] : 0;
    const size_t row = ((size_t)page * kv.kv_heads + kvh) * kv.page_size + (ok ? t % kv.page_size : 0);
    pf_cp_async16(dst + r * LD + c8, pool + row * HD + c8, ok ? 16 : 0);
  }
}

__device__ __forceinline__ float pf_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// grid (nq, ceil(T/64)); block 128.  Query row i of the chunk sits at absolute position pos0 + i.
template <int HD>
__global__ void __launch_bounds__(128, 3) attn_prefill_kernel(const float* __restrict__ q, int T, int pos0, const int* __restrict__ bt,
                                                          PfKvPool kv, int nq, float sm_scale, __half* __restrict__ out, int out_ld,
                                                          int k_order) {
  constexpr int LD = HD + 8;
  extern __shared__ __align__(16) __half smem_h[];
  // four regions of [64][LD]: K and V tiles of two stages.  The scaled queries are staged through region 0 and live in
  // registers from then on, so the first K tile may overwrite them.
  __half* sQ = smem_h;
  auto stage_k = [&](int st) { return smem_h + (2 * st) * 64 * LD; };
  auto stage_v = [&](int st) { return smem_h + (2 * st + 1) * 64 * LD; };
  // blocks are dispatched in linear order: the query blocks with the most keys (the last ones) go first, the short ones
  // fill the tail of the grid
  const int qb = gridDim.y - 1 - blockIdx.y, head = blockIdx.x;
  const int kvh = head / (nq / kv.kv_heads);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q0 = qb * 64;

  // stage Q as f16, scaled by sm_scale * log2(e): the softmax below works in base 2 (one ex2 per score, no multiply)
  sm_scale *= 1.4426950408889634f;
  for (int idx = threadIdx.x; idx < 64 * (HD / 4); idx += blockDim.x) {
    const int r = idx / (HD / 4), c4 = (idx % (HD / 4)) * 4;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (q0 + r < T) v = *reinterpret_cast<const float4*>(q + ((size_t)(q0 + r) * nq + head) * HD + c4);
    __half2 a = __floats2half2_rn(v.x * sm_scale, v.y * sm_scale), b = __floats2half2_rn(v.z * sm_scale, v.w * sm_scale);
    *reinterpret_cast<__half2*>(sQ + r * LD + c4) = a;
    *reinterpret_cast<__half2*>(sQ + r * LD + c4 + 2) = b;
  }
  __syncthreads();
  // Q fragments of this warp's 16 rows: HD/16 k-steps x 4 registers
  uint32_t qf[HD / 16][4];
#pragma unroll
  for (int ks = 0; ks < HD / 16; ++ks) {
    const __half* p = sQ + (warp * 16 + (lane & 15)) * LD + ks * 16 + (lane >> 4) * 8;
    ldmatrix_x4(qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], p);
  }
  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.0f, l1 = 0.0f;
  const int row0 = q0 + warp * 16 + (lane >> 2), row1 = row0 + 8;   // chunk-relative query rows of this thread
  const int kv_end = min(pos0 + q0 + 64, pos0 + T);                  // keys needed by this query block

  // Tile it + 1 is requested before tile it is used: asynchronous copies for f16 pages (they land while the MMAs of the
  // current tile run), register staging with conversion for the other page formats.
  auto fetch = [&](int kb, int st) {
    if (kv.kvt == 1) {
      stage_kv_async<HD>(stage_k(st), reinterpret_cast<const __half*>(kv.k), kv, bt, kvh, kb, kv_end);
      stage_kv_async<HD>(stage_v(st), reinterpret_cast<const __half*>(kv.v), kv, bt, kvh, kb, kv_end);
    } else {
      stage_kv<HD>(stage_k(st), kv.k, kv.k_scale, kv, bt, kvh, kb, kv_end);
      stage_kv<HD>(stage_v(st), kv.v, kv.v_scale, kv, bt, kvh, kb, kv_end);
    }
  };
  __syncthreads();             // every warp has its query fragments: region 0 is free
  fetch(0, 0);
  pf_cp_commit();
  for (int kb = 0, it = 0; kb < kv_end; kb += 64, ++it) {
    if (kb + 64 < kv_end) fetch(kb + 64, (it + 1) & 1);   // that stage was released by the barrier that ended iteration it - 1
    pf_cp_commit();
    pf_cp_wait<1>();           // everything but the newest group: tile it has landed
    __syncthreads();
    const __half* sK = stage_k(it & 1);
    const __half* sV = stage_v(it & 1);
    // S = Q K^T : 16 x 64 per warp -> 8 n-tiles of 8 keys
    float s[8][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.0f;
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        // two n-tiles (16 keys) x 16 dims per ldmatrix.x4
        uint32_t b0, b1, b2, b3;
        const __half* p = sK + (np * 16 + (lane & 7) + ((lane >> 4) << 3)) * LD + ks * 16 + ((lane >> 3) & 1) * 8;
        ldmatrix_x4(b0, b1, b2, b3, p);
        mma16816(s[2 * np], qf[ks], b0, b1);
        mma16816(s[2 * np + 1], qf[ks], b2, b3);
      }
    }
    // causal mask + online softmax (rows row0 and row1 of this thread).  Only tiles that reach past the first query row
    // of this warp (the diagonal, and the zero-filled keys after the last one) need the mask.
    float mx0 = m0, mx1 = m1;
    if (kb + 63 > pos0 + q0 + warp * 16) {
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int key = kb + nt * 8 + (lane & 3) * 2 + (e & 1);
          const int qrow = (e < 2) ? row0 : row1;
          const bool ok = key <= pos0 + qrow && qrow < T;
          if (!ok) s[nt][e] = -INFINITY;
        }
      }
    }
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      mx0 = fmaxf(mx0, fmaxf(s[nt][0], s[nt][1]));
      mx1 = fmaxf(mx1, fmaxf(s[nt][2], s[nt][3]));
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    // a row with nothing visible yet (rows past T) keeps max = -inf; subtracting 0 instead leaves every term ex2(-inf) = 0
    const float e0 = (mx0 == -INFINITY) ? 0.0f : mx0, e1 = (mx1 == -INFINITY) ? 0.0f : mx1;
    const float r0 = pf_ex2(m0 - e0), r1 = pf_ex2(m1 - e1);
    float ps0 = 0.0f, ps1 = 0.0f;
    uint32_t pf[8][2];   // P as f16 pairs: [n-tile][row0 pair, row1 pair]
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      const float p0 = pf_ex2(s[nt][0] - e0), p1 = pf_ex2(s[nt][1] - e0);
      const float p2 = pf_ex2(s[nt][2] - e1), p3 = pf_ex2(s[nt][3] - e1);
      ps0 += p0 + p1;
      ps1 += p2 + p3;
      __half2 h01 = __floats2half2_rn(p0, p1), h23 = __floats2half2_rn(p2, p3);
      pf[nt][0] = *reinterpret_cast<uint32_t*>(&h01);
      pf[nt][1] = *reinterpret_cast<uint32_t*>(&h23);
    }
    l0 = l0 * r0 + ps0;
    l1 = l1 * r1 + ps1;
    m0 = mx0;
    m1 = mx1;
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) {
      o[i][0] *= r0; o[i][1] *= r0; o[i][2] *= r1; o[i][3] *= r1;
    }
    // O += P V : k runs over the 64 keys (4 k-steps of 16), n over HD (HD/8 n-tiles)
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
      const uint32_t a[4] = {pf[2 * ks][0], pf[2 * ks][1], pf[2 * ks + 1][0], pf[2 * ks + 1][1]};
#pragma unroll
      for (int np = 0; np < HD / 16; ++np) {
        uint32_t b0, b1, b2, b3;
        const __half* p = sV + (ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + np * 16 + (lane >> 4) * 8;
        ldmatrix_x4_trans(b0, b1, b2, b3, p);
        mma16816(o[2 * np], a, b0, b1);
        mma16816(o[2 * np + 1], a, b2, b3);
      }
    }
    __syncthreads();           // all warps are done with this stage before the next iteration refills it
  }
  pf_cp_wait<0>();
  // the row sums are spread over the four lanes that share a row
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const float i0 = l0 > 0.0f ? 1.0f / l0 : 0.0f, i1 = l1 > 0.0f ? 1.0f / l1 : 0.0f;
#pragma unroll
  for (int nt = 0; nt < HD / 8; ++nt) {
    const int d = nt * 8 + (lane & 3) * 2;
    const int n0 = head * HD + d;
    if (row0 < T) {
      out[(size_t)row0 * out_ld + pf_out_k(n0, k_order)] = __float2half_rn(o[nt][0] * i0);
      out[(size_t)row0 * out_ld + pf_out_k(n0 + 1, k_order)] = __float2half_rn(o[nt][1] * i0);
    }
    if (row1 < T) {
      out[(size_t)row1 * out_ld + pf_out_k(n0, k_order)] = __float2half_rn(o[nt][2] * i1);
      out[(size_t)row1 * out_ld + pf_out_k(n0 + 1, k_order)] = __float2half_rn(o[nt][3] * i1);
    }
  }
}

}  // namespace bonsai

extern "C" {

// q f32 [T][nq][hd]; block_table: the sequence's page list; the chunk's first token sits at pos0.
// out f16 [T][out_ld]; k_order 0 = paired-K (operand order of the tcgen05 GEMM), 1 = hmma-K (the mma.sync GEMM; needs
// nq * hd to be a multiple of 128).
int bonsai_attn_prefill_order(const float* q, int T, int pos0, const int* block_table, int nq, int nkv, int hd, int kvt, int page_size,
                              const void* kpool, const void* vpool, const float* kscale, const float* vscale, void* out, int out_ld,
                              int k_order, cudaStream_t stream) {
  using namespace bonsai;
  if (k_order < 0 || k_order > 1 || (k_order == 1 && (nq * hd) % 128 != 0)) return BONSAI_CUDA_BAD_ARG;
  if (T < 1 || (hd != 64 && hd != 128) || nq % nkv != 0 || kvt < 0 || kvt > 3) return BONSAI_CUDA_BAD_ARG;
  PfKvPool kv{(const uint8_t*)kpool, (const uint8_t*)vpool, kscale, vscale, page_size, nkv, hd, kvt};
  dim3 grid(nq, (T + 63) / 64);
  const float sc = 1.0f / sqrtf((float)hd);
  size_t smem = (size_t)4 * 64 * (hd + 8) * sizeof(__half);
  cudaError_t e;
  if (hd == 128) {
    e = cudaFuncSetAttribute(attn_prefill_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    // three CTAs of 68 KB per SM need the largest shared-memory carve-out; the default picks a smaller one that fits two
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(attn_prefill_kernel<128>, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) return BONSAI_CUDA_LAUNCH_FAILED;
    attn_prefill_kernel<128><<<grid, 128, smem, stream>>>(q, T, pos0, block_table, kv, nq, sc, (__half*)out, out_ld, k_order);
  } else {
    e = cudaFuncSetAttribute(attn_prefill_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return BONSAI_CUDA_LAUNCH_FAILED;
    attn_prefill_kernel<64><<<grid, 128, smem, stream>>>(q, T, pos0, block_table, kv, nq, sc, (__half*)out, out_ld, k_order);
  }
  return launch_status();
}

// out f16 [T][out_ld] in paired-K order.
int bonsai_attn_prefill(const float* q, int T, int pos0, const int* block_table, int nq, int nkv, int hd, int kvt, int page_size,
                        const void* kpool, const void* vpool, const float* kscale, const float* vscale, void* out, int out_ld,
                        cudaStream_t stream) {
  return bonsai_attn_prefill_order(q, T, pos0, block_table, nq, nkv, hd, kvt, page_size, kpool, vpool, kscale, vscale, out, out_ld, 0, stream);
}

}  // extern "C"
