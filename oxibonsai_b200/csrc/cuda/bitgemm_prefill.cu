// Prefill GEMM for packed ternary / 1-bit weights on the 5th-generation tensor cores.
//
//   out[t][n] = sum_k X[t][k] * W[n][k]        t < T tokens (hundreds to thousands), n < N rows
//
// The reference's prefill kernels (gemm_q1_g128_v7, gemm_tq2_g128_v7, their _residual forms and
// fused_gate_up_swiglu_gemm_q1/_tq2; crates/oxibonsai-kernels/src/gpu_backend/cuda_prefill_kernels.rs:74-827)
// walk the batch eight columns at a time on CUDA cores and re-read the weights for every chunk.
// Here a CTA owns a 128-row weight tile x 256-token tile:
//   * A operand (weights): four expander warps read the packed words (one 16-byte load = one
//     64-input k-block of a row), turn every two weights into a half2 with one shift, one mask
//     and one HMUL2 by the group scale (+-2^-7 * 128*d = +-d exactly, d being an f16), and
//     store the row into the 128-byte-swizzled shared-memory tile;
//   * B operand (activations): f16 tiles fetched by TMA (cp.async.bulk.tensor, no multicast);
//   * tcgen05.mma kind::f16 accumulates the whole K extent in TMEM (128 lanes x 256 columns,
//     double buffered so the epilogue of one tile overlaps the main loop of the next);
//   * epilogue warps read TMEM back and store f32 (plain / residual add) or f16 SwiGLU outputs.
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

constexpr int kPfStages = 4;
constexpr int kPfAhead = 8;                   // code vectors each expander thread keeps in flight
constexpr int kPfABytes = 128 * 128;          // 128 rows x 64 f16
constexpr int kPfThreads = 320;               // warps 0-3 expand, 4-7 epilogue, 8 = MMA, 9 = TMA

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
};

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                   tc::smem_u32(dst)),
               "l"(map), "r"(x), "r"(y), "r"(tc::smem_u32(bar))
               : "memory");
}

// TOK = tokens per tile (MMA N): 256 for prompt chunks, 64 for batched decode / verification.
template <int TOK>
__global__ void __launch_bounds__(kPfThreads, 1) bitgemm_prefill_kernel(const __grid_constant__ CUtensorMap xmap,
                                                                     const __grid_constant__ CUtensorMap amap, PfParams p) {
  constexpr int kPfTokTile = TOK;
  constexpr int kPfBBytes = TOK * 128;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sA = base;
  uint8_t* sB = base + kPfStages * kPfABytes;
  __shared__ uint64_t full_bar[kPfStages], empty_bar[kPfStages], accf_bar[2], acce_bar[2];
  __shared__ uint32_t tmem_slot;
  const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
  const int kblocks = p.K >> 6;
  const int row_tiles = (p.n_rows + 127) >> 7, tok_tiles = (p.T + kPfTokTile - 1) / kPfTokTile;
  const int ntiles = row_tiles * tok_tiles;

  if (warp == 8) {
    tc::tmem_alloc(&tmem_slot, 2 * TOK);
    tc::tmem_relinquish();
  }
  if (t == 0) {
    for (int i = 0; i < kPfStages; ++i) {
      tc::mbar_init(&full_bar[i], p.dense ? 1 : 5);   // 4 expander warps + the TMA issuer's expect_tx arrival
      tc::mbar_init(&empty_bar[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      tc::mbar_init(&accf_bar[i], 1);
      tc::mbar_init(&acce_bar[i], 4);
    }
    tc::mbar_fence_init();
  }
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t taddr = tmem_slot;
  bool failed = false;

  if (warp == 9) {
    // ------------------------------- TMA issuer (activations) ----------------------------------
    if (lane == 0) {
      int it = 0;
      for (int tile = blockIdx.x; tile < ntiles && !failed; tile += gridDim.x) {
        const int tok0 = (tile / row_tiles) * kPfTokTile;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % kPfStages;
          if (!tc::mbar_wait(&empty_bar[s], ((it / kPfStages) & 1) ^ 1)) { failed = true; break; }
          tc::mbar_arrive_expect_tx(&full_bar[s], kPfBBytes + (p.dense ? kPfABytes : 0));
          tma_load_2d(sB + s * kPfBBytes, &xmap, kb * 64, tok0, &full_bar[s]);
          if (p.dense) tma_load_2d(sA + s * kPfABytes, &amap, kb * 64, (tile % row_tiles) * 128, &full_bar[s]);
        }
      }
      if (failed) atomicExch(p.status, 1);
    }
  } else if (warp == 8) {
    // ------------------------------- MMA issuer -------------------------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = tc::idesc_f32acc(tc::FMT_F16, tc::FMT_F16, 128, kPfTokTile);
      int it = 0, tcount = 0;
      for (int tile = blockIdx.x; tile < ntiles && !failed; tile += gridDim.x, ++tcount) {
        const int ab = tcount & 1;
        if (!tc::mbar_wait(&acce_bar[ab], ((tcount >> 1) & 1) ^ 1)) { failed = true; break; }
        tc::tc_fence_after();
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % kPfStages;
          if (!tc::mbar_wait(&full_bar[s], (it / kPfStages) & 1)) { failed = true; break; }
          tc::tc_fence_after();
          const uint64_t da = tc::smem_desc_sw128(tc::smem_u32(sA + s * kPfABytes));
          const uint64_t db = tc::smem_desc_sw128(tc::smem_u32(sB + s * kPfBBytes));
#pragma unroll
          for (uint32_t k = 0; k < 4; ++k) tc::mma_f16(taddr + ab * kPfTokTile, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0);
          tc::mma_commit(&empty_bar[s]);
        }
        if (!failed) tc::mma_commit(&accf_bar[ab]);
      }
      if (failed) atomicExch(p.status, 1);
    }
  } else if (warp < 4) {
    // ------------------------------- weight expanders (thread = weight row) ---------------------
    if (p.dense) goto done;
    {
    const int words_per_row = p.K >> 4, ngroups = p.K >> 7;
    int it = 0;
    for (int tile = blockIdx.x; tile < ntiles && !failed; tile += gridDim.x) {
      const int row = (tile % row_tiles) * 128 + t;
      const bool row_ok = row < p.n_rows;
      const uint4* wp = reinterpret_cast<const uint4*>(p.codes + (size_t)(row_ok ? row : 0) * words_per_row);
      const __half* sp = p.scales + (size_t)(row_ok ? row : 0) * ngroups;
      // a thread walks its own weight row, so its loads are a dependent chain of cache misses unless several
      // are in flight: keep kPfAhead 16-byte code vectors (and their group scales) requested ahead of use
      uint4 cbuf[kPfAhead];
      __half sbuf[kPfAhead];
#pragma unroll
      for (int j = 0; j < kPfAhead; ++j) {
        const bool ok = row_ok && j < kblocks;
        cbuf[j] = ok ? __ldg(wp + j) : make_uint4(0, 0, 0, 0);
        sbuf[j] = ok ? sp[j >> 1] : __float2half(0.0f);
      }
      for (int kb0 = 0; kb0 < kblocks && !failed; kb0 += kPfAhead) {
#pragma unroll
      for (int j = 0; j < kPfAhead; ++j) {
        const int kb = kb0 + j;
        if (kb < kblocks && !failed) {   // no break: the unrolled loop keeps cbuf / sbuf in registers
        const uint4 cur = cbuf[j];
        const __half dh = __hmul(sbuf[j], __float2half(128.0f));
        if (row_ok && kb + kPfAhead < kblocks) {
          cbuf[j] = __ldg(wp + kb + kPfAhead);
          sbuf[j] = sp[(kb + kPfAhead) >> 1];
        }
        const __half2 d2 = __half2half2(dh);
        const int s = it % kPfStages;
        if (!tc::mbar_wait(&empty_bar[s], ((it / kPfStages) & 1) ^ 1)) failed = true;
        if (!failed) {
        uint8_t* stage = sA + s * kPfABytes;
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
          *reinterpret_cast<uint4*>(stage + tc::sw128_offset(t, 2 * wd)) = make_uint4(o[0], o[1], o[2], o[3]);
          *reinterpret_cast<uint4*>(stage + tc::sw128_offset(t, 2 * wd + 1)) = make_uint4(o[4], o[5], o[6], o[7]);
        }
        tc::fence_proxy_async();
        __syncwarp();
        if (lane == 0) tc::mbar_arrive(&full_bar[s]);
        ++it;
        }
        }
      }
      }
    }
    if (failed && t == 0) atomicExch(p.status, 1);
    }
  } else {
    // ------------------------------- epilogue (thread = weight row) ------------------------------
    const int a = t - 128;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    int tcount = 0;
    for (int tile = blockIdx.x; tile < ntiles && !failed; tile += gridDim.x, ++tcount) {
      const int ab = tcount & 1;
      const int row = (tile % row_tiles) * 128 + a;
      const int tok0 = (tile / row_tiles) * kPfTokTile;
      const bool row_ok = row < p.n_rows;
      if (!tc::mbar_wait(&accf_bar[ab], (tcount >> 1) & 1)) { failed = true; break; }
      tc::tc_fence_after();
#pragma unroll 1
      for (int c0 = 0; c0 < kPfTokTile; c0 += 32) {
        uint32_t r[32];
        tc::tmem_ld32(taddr + lane_base + ab * kPfTokTile + c0, r);
        tc::tmem_wait_ld();
        if (tok0 + c0 >= p.T) continue;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int tok = tok0 + c0 + j;
          float v = __uint_as_float(r[j]);
          if (p.epi == 2) {
            float other = __shfl_xor_sync(0xffffffffu, v, 1);
            if (row_ok && tok < p.T && (a & 1) == 0)
              p.out_f16[(size_t)tok * p.out_ld + paired_k(row >> 1)] = __float2half_rn(v / (1.0f + __expf(-v)) * other);
          } else if (row_ok && tok < p.T) {
            const size_t o = (size_t)tok * p.out_ld + row;
            if (p.epi == 0) p.out_f32[o] = v;
            else if (p.epi == 1) p.out_f32[o] = p.residual[o] + v;
            else p.out_f16[o] = __float2half_rn(v);
          }
        }
      }
      tc::tc_fence_before();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(&acce_bar[ab]);
    }
    if (failed && a == 0) atomicExch(p.status, 1);
  }
done:
  tc::tc_fence_before();
  __syncthreads();
  if (warp == 8) tc::tmem_dealloc(taddr, 2 * TOK);
}

// One block per token: y = rmsnorm(x) * w (or a plain copy when w is null), written as f16 in the
// paired-K order consumed by bitgemm_prefill.
__global__ void norm_to_f16_paired_kernel(const float* __restrict__ x, int x_ld, const float* __restrict__ w, float eps, int K,
                                          __half* __restrict__ out, int out_ld, int natural) {
  __shared__ float s32[32];
  const int tok = blockIdx.x;
  const float* xr = x + (size_t)tok * x_ld;
  float inv = 1.0f;
  if (w != nullptr) {
    float ss = 0.0f;
    for (int k = threadIdx.x; k < K; k += blockDim.x) ss += xr[k] * xr[k];
    ss = block_sum(ss, s32);
    inv = 1.0f / sqrtf(ss / (float)K + eps);
  }
  for (int k = threadIdx.x; k < K; k += blockDim.x) {
    float v = w ? w[k] * xr[k] * inv : xr[k];
    out[(size_t)tok * out_ld + (natural ? k : paired_k(k))] = __float2half_rn(v);
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
static int launch_prefill(const CUtensorMap& xmap, const CUtensorMap& amap, const bonsai::PfParams& p, int sms, cudaStream_t stream) {
  using namespace bonsai;
  const int ntiles = ((p.n_rows + 127) / 128) * ((p.T + TOK - 1) / TOK);
  int grid = ntiles < sms ? ntiles : sms;
  size_t smem = 1024 + (size_t)kPfStages * (kPfABytes + TOK * 128);
  cudaError_t e = cudaFuncSetAttribute(bitgemm_prefill_kernel<TOK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return BONSAI_CUDA_LAUNCH_FAILED;
  bitgemm_prefill_kernel<TOK><<<grid, kPfThreads, smem, stream>>>(xmap, amap, p);
  return launch_status();
}

extern "C" {

// x_f16: activations [T][K] f16 (row stride x_ld elements, 16-byte aligned rows), in paired-K order for packed
// weights and natural order for dense ones.
// epi 0: out_f32 = W x; 1: out_f32 = residual + W x; 2: out_f16 = SwiGLU over interleaved gate/up rows
// (paired-K order, out_ld = N/2 or more); 3: out_f16 = W x in natural order.
// dense_w != null: W is a dense f16 row-major [n_rows][K] matrix (codes / scales ignored), e.g. the LM head.
int bonsai_bitgemm_prefill(const void* codes, const void* scales, const void* x_f16, int x_ld, float* out_f32,
                           const float* residual, void* out_f16, int* status, int n_rows, int K, int T, int epi, int out_ld,
                           int sms, const void* dense_w, cudaStream_t stream) {
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
             dense_w != nullptr ? 1 : 0};
  return tok == 64 ? launch_prefill<64>(xmap, amap, p, sms, stream) : launch_prefill<256>(xmap, amap, p, sms, stream);
}

int bonsai_norm_to_f16_paired(const float* x, int x_ld, const float* w, float eps, int T, int K, void* out, int out_ld, int natural,
                              cudaStream_t stream) {
  if (T < 1 || K % 16 != 0) return BONSAI_CUDA_BAD_ARG;
  bonsai::norm_to_f16_paired_kernel<<<T, 256, 0, stream>>>(x, x_ld, w, eps, K, (__half*)out, out_ld, natural);
  return bonsai::launch_status();
}

}  // extern "C"
