// Single-tile tensor-core self-test: D[128][N] = A[128][K] * B[N][K]^T with one CTA, operands given
// as row-major 128-byte rows that the kernel places into swizzled shared memory.  It exists to pin
// down, on hardware, the operand encodings the production kernels rely on (f16 / bf16, and e2m1 x e4m3
// under kind::f8f6f4); the unit tests compare it against a PyTorch fp32 matmul of the decoded operands.
#include "common.cuh"
#include "tcgen05.cuh"

namespace bonsai {

// kind: 0 = f16, 1 = bf16, 2 = f8f6f4 (A e2m1, B e4m3)
__global__ void __launch_bounds__(128) tc_tile_kernel(const uint8_t* __restrict__ A, const uint8_t* __restrict__ B,
                                                     float* __restrict__ out, int N, int kind, int* __restrict__ status) {
  extern __shared__ uint8_t raw[];
  uint8_t* base = (uint8_t*)(((uintptr_t)raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sA = base;           // 128 rows x 128 B
  uint8_t* sB = base + 16384;   // up to 256 rows x 128 B
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_slot;
  const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
  const uint32_t ncols = 512;

  if (warp == 0) {
    tc::tmem_alloc(&tmem_slot, ncols);
    tc::tmem_relinquish();
  }
  if (t == 0) {
    tc::mbar_init(&bar, 1);
    tc::mbar_fence_init();
  }
  for (int c = 0; c < 8; ++c) {
    *reinterpret_cast<uint4*>(sA + tc::sw128_offset(t, c)) = *reinterpret_cast<const uint4*>(A + (size_t)t * 128 + c * 16);
  }
  for (int r = t; r < N; r += 128)
    for (int c = 0; c < 8; ++c)
      *reinterpret_cast<uint4*>(sB + tc::sw128_offset(r, c)) = *reinterpret_cast<const uint4*>(B + (size_t)r * 128 + c * 16);
  tc::fence_proxy_async();
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t taddr = tmem_slot;
  const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
  if (t == 0) {
    uint64_t da = tc::smem_desc_sw128(tc::smem_u32(sA)), db = tc::smem_desc_sw128(tc::smem_u32(sB));
    for (uint32_t k = 0; k < 4; ++k) {
      if (kind == 0) tc::mma_f16(taddr, da + 2 * k, db + 2 * k, tc::idesc_f32acc(tc::FMT_F16, tc::FMT_F16, 128, N), k);
      else if (kind == 1) tc::mma_f16(taddr, da + 2 * k, db + 2 * k, tc::idesc_f32acc(tc::FMT_BF16, tc::FMT_BF16, 128, N), k);
      else tc::mma_f8f6f4(taddr, da + 2 * k, db + 2 * k, tc::idesc_f32acc(tc::FMT_E2M1, tc::FMT_E4M3, 128, N), k);
    }
    tc::mma_commit(&bar);
  }
  bool ok = tc::mbar_wait(&bar, 0);
  tc::tc_fence_after();
  if (!ok) {
    if (t == 0) atomicExch(status, 1);
  } else {
    for (int c0 = 0; c0 < N; c0 += 8) {
      uint32_t r[8];
      tc::tmem_ld8(taddr + lane_base + c0, r);
      tc::tmem_wait_ld();
#pragma unroll
      for (int j = 0; j < 8; ++j) out[(size_t)(warp * 32 + lane) * N + c0 + j] = __uint_as_float(r[j]);
    }
  }
  tc::tc_fence_before();
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(taddr, ncols);
}

}  // namespace bonsai

extern "C" int bonsai_tc_tile(const void* A, const void* B, float* out, int N, int kind, int* status, cudaStream_t stream) {
  if (N < 16 || N > 256 || N % 16 != 0 || kind < 0 || kind > 2) return BONSAI_CUDA_BAD_ARG;
  size_t smem = 1024 + 16384 + 32768;
  cudaFuncSetAttribute(bonsai::tc_tile_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  bonsai::tc_tile_kernel<<<1, 128, smem, stream>>>((const uint8_t*)A, (const uint8_t*)B, out, N, kind, status);
  return bonsai::launch_status();
}
