// Shared device helpers and the packed weight layout used by every kernel in this library.
//
// Device weight layout ("planar SM"): a quantised matrix of N output rows by K inputs is stored as
//   codes  : uint32 [N][K/16]  - one word per 16 consecutive inputs k0..k0+15
//   scales : f16    [N][K/128] - one scale per 128-input group (the GGUF block scale)
// Inside a word, nibble i (bits 4i..4i+3) = { S(k0+i), S(k0+8+i), M(k0+i), M(k0+8+i) } from bit 3
// down to bit 0, where M = 1 for a non-zero weight and S = 1 for a negative one.  Two masks turn a
// word into sixteen e2m1 (fp4) values for the tensor cores:  (w & 0xAAAAAAAA) holds inputs
// k0..k0+7 and ((w & 0x55555555) << 1) holds k0+8..k0+15, each nibble being S0M0 = +-1.0 or 0.
// The same two bits, moved to bits 31 and 29 of a word, are the float +-2^-63 (or 0), which is
// how the CUDA-core kernels multiply without any integer-to-float conversion.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define BONSAI_CUDA_OK 0
#define BONSAI_CUDA_BAD_ARG (-13)
#define BONSAI_CUDA_LAUNCH_FAILED (-18)

namespace bonsai {

constexpr float kPow2_63 = 9223372036854775808.0f;  // 2^63

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over the whole block (blockDim.x <= 1024, multiple of 32); every thread gets the result.
__device__ __forceinline__ float block_sum(float v, float* smem32) {
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) smem32[wid] = v;
  __syncthreads();
  float t = (lane < nw) ? smem32[lane] : 0.0f;
  t = warp_sum(t);
  return t;
}

// One row: y = rmsnorm(x) * w (a plain copy when w is null), written as f16 at position pos(k) of the output row.
// The row is read once with 16-byte loads and kept in registers between the sum of squares and the scaling (up to
// 16 * blockDim.x elements; longer rows are read twice).  Needs 16-byte aligned rows and K % 4 == 0.
template <class PosFn>
__device__ __forceinline__ void norm_row_to_f16(const float* __restrict__ xr, const float* __restrict__ w, float eps, int K,
                                                __half* __restrict__ orow, float* s32, PosFn pos) {
  constexpr int kKeep = 4;
  const int nch = K >> 2;
  const float4* x4 = reinterpret_cast<const float4*>(xr);
  float4 v[kKeep];
  float ss = 0.0f;
#pragma unroll
  for (int i = 0; i < kKeep; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    v[i] = c < nch ? x4[c] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
  }
  for (int c = threadIdx.x + kKeep * blockDim.x; c < nch; c += blockDim.x) {
    const float4 t = x4[c];
    ss += t.x * t.x + t.y * t.y + t.z * t.z + t.w * t.w;
  }
  float inv = 1.0f;
  if (w != nullptr) {
    ss = block_sum(ss, s32);
    inv = 1.0f / sqrtf(ss / (float)K + eps);
  }
  auto emit = [&](int c, float4 t) {
    if (w != nullptr) {
      const float4 ww = reinterpret_cast<const float4*>(w)[c];
      t.x *= ww.x * inv; t.y *= ww.y * inv; t.z *= ww.z * inv; t.w *= ww.w * inv;
    }
    orow[pos(4 * c)] = __float2half_rn(t.x);
    orow[pos(4 * c + 1)] = __float2half_rn(t.y);
    orow[pos(4 * c + 2)] = __float2half_rn(t.z);
    orow[pos(4 * c + 3)] = __float2half_rn(t.w);
  };
#pragma unroll
  for (int i = 0; i < kKeep; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    if (c < nch) emit(c, v[i]);
  }
  for (int c = threadIdx.x + kKeep * blockDim.x; c < nch; c += blockDim.x) emit(c, x4[c]);
}

// Dot of one packed word (16 ternary weights, scaled by 2^-63) with 16 floats.
__device__ __forceinline__ float dot_word16(uint32_t w, const float* x) {
  float acc = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    float wa = __uint_as_float((w << (28 - 4 * i)) & 0xA0000000u);
    float wb = __uint_as_float((w << (29 - 4 * i)) & 0xA0000000u);
    acc = fmaf(wa, x[i], acc);
    acc = fmaf(wb, x[8 + i], acc);
  }
  return acc;
}

// position of logical input k inside its 128-input group in the hmma-K order
__host__ __device__ inline int hmma_k_pos(int k) {
  const int r = k & 127, wq = r >> 4, e = r & 15;
  const int c = wq >> 1, j = wq & 1, plane = e >> 3, p = e & 3, h = (e >> 2) & 1;
  return (k & ~127) | ((j * 4 + p) * 16 + plane * 8 + 2 * c + h);
}

// Launch with programmatic dependent launch enabled: the kernel may start while its predecessor in
// the stream is still running and must execute griddepcontrol.wait before touching anything the
// predecessor writes (or writing anything it reads).
template <typename Kern, typename... Args>
static inline cudaError_t launch_pdl(Kern kernel, dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, args...);
}

inline int launch_status() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? BONSAI_CUDA_OK : BONSAI_CUDA_LAUNCH_FAILED;
}

}  // namespace bonsai
