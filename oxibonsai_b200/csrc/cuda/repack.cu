// GGUF block bytes -> planar SM device layout (see common.cuh).
//
// The reference re-lays its weights out on upload as well (array-of-blocks to structure-of-
// arrays, crates/oxibonsai-kernels/src/gpu_backend/cuda_graph/cudagraph_reformat_tq2_blocks_to_soa_group.rs:16-74);
// here the target layout is the one the sm_100a kernels consume, and a sub-matrix can be
// selected (row range for column-parallel shards, 128-input block range for row-parallel
// shards) and scattered with a row stride so that gate/up rows interleave and q/k/v rows
// concatenate into one fused matrix.
#include "common.cuh"

namespace bonsai {

// src_type: 42 = TQ2_0_g128 ([qs 32][d f16], 34 B), 41 = Q1_0_g128 ([d f16][qs 16], 18 B)
__global__ void repack_planar_kernel(const uint8_t* __restrict__ src, int src_type, int src_blocks_per_row,
                                     int row0, int nrows, int blk0, int nblk, uint32_t* __restrict__ codes,
                                     __half* __restrict__ scales, int dst_row0, int dst_row_stride,
                                     int dst_words_per_row, int dst_blk0) {
  long long words_per_row = (long long)nblk * 8;
  long long total = (long long)nrows * words_per_row;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    int r = (int)(idx / words_per_row);
    int wi = (int)(idx % words_per_row);
    int blk = wi >> 3, sub = wi & 7;  // 8 words per 128-input block
    const int bbytes = src_type == 42 ? 34 : 18;
    const uint8_t* b = src + ((long long)(row0 + r) * src_blocks_per_row + (blk0 + blk)) * bbytes;
    uint32_t m = 0, s = 0;  // bit j = weight j of this word
    if (src_type == 42) {
      const uint8_t* q = b + sub * 4;
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        uint32_t c = (q[j >> 2] >> (2 * (j & 3))) & 3u;
        m |= (uint32_t)(c == 0u || c == 2u) << j;
        s |= (uint32_t)(c == 0u) << j;
      }
    } else {
      const uint8_t* q = b + 2 + sub * 2;
      uint32_t bits = q[0] | ((uint32_t)q[1] << 8);
      m = 0xFFFFu;
      s = (~bits) & 0xFFFFu;
    }
    uint32_t w = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      uint32_t nib = (((s >> i) & 1u) << 3) | (((s >> (8 + i)) & 1u) << 2) | (((m >> i) & 1u) << 1) | ((m >> (8 + i)) & 1u);
      w |= nib << (4 * i);
    }
    long long drow = dst_row0 + (long long)r * dst_row_stride;
    codes[drow * dst_words_per_row + (long long)(dst_blk0 + blk) * 8 + sub] = w;
    if (sub == 0) {
      const uint8_t* dp = src_type == 42 ? b + 32 : b;
      uint16_t d = (uint16_t)dp[0] | ((uint16_t)dp[1] << 8);
      scales[drow * (dst_words_per_row / 8) + dst_blk0 + blk] = __ushort_as_half(d);
    }
  }
}

// Planar SM -> dense f32 (row-major [nrows][K]); used by tests and by the cuBLAS baseline path.
__global__ void planar_to_f32_kernel(const uint32_t* __restrict__ codes, const __half* __restrict__ scales, int nrows,
                                     int words_per_row, float* __restrict__ out) {
  long long total = (long long)nrows * words_per_row;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    long long r = idx / words_per_row;
    int wi = (int)(idx % words_per_row);
    uint32_t w = codes[idx];
    float d = __half2float(scales[r * (words_per_row / 8) + (wi >> 3)]);
    float* o = out + idx * 16;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      uint32_t nib = (w >> (4 * i)) & 0xFu;
      float a = (nib & 2u) ? ((nib & 8u) ? -d : d) : 0.0f;
      float b = (nib & 1u) ? ((nib & 4u) ? -d : d) : 0.0f;
      o[i] = a;
      o[8 + i] = b;
    }
  }
}

}  // namespace bonsai

extern "C" {

// Repack rows [row0, row0+nrows) and 128-input blocks [blk0, blk0+nblk) of a GGUF matrix that has
// `src_blocks_per_row` blocks per row.  Destination row i lands at dst_row0 + i*dst_row_stride of a
// planar matrix with dst_words_per_row words per row, starting at block dst_blk0 within the row.
int bonsai_repack_planar(const void* src, int src_type, int src_blocks_per_row, int row0, int nrows, int blk0, int nblk,
                         void* codes, void* scales, int dst_row0, int dst_row_stride, int dst_words_per_row, int dst_blk0,
                         cudaStream_t stream) {
  if ((src_type != 41 && src_type != 42) || nrows <= 0 || nblk <= 0 || dst_words_per_row % 8) return BONSAI_CUDA_BAD_ARG;
  long long total = (long long)nrows * nblk * 8;
  int grid = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  bonsai::repack_planar_kernel<<<grid, 256, 0, stream>>>((const uint8_t*)src, src_type, src_blocks_per_row, row0, nrows, blk0, nblk,
                                                         (uint32_t*)codes, (__half*)scales, dst_row0, dst_row_stride,
                                                         dst_words_per_row, dst_blk0);
  return bonsai::launch_status();
}

int bonsai_planar_to_f32(const void* codes, const void* scales, int nrows, int words_per_row, void* out, cudaStream_t stream) {
  long long total = (long long)nrows * words_per_row;
  int grid = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  bonsai::planar_to_f32_kernel<<<grid, 256, 0, stream>>>((const uint32_t*)codes, (const __half*)scales, nrows, words_per_row, (float*)out);
  return bonsai::launch_status();
}

}  // extern "C"
