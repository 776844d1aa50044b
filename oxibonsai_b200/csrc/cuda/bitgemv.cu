// Batch-1 decode GEMV on CUDA cores, exact in f32: out = W x for a planar-SM packed matrix, with
// optional fused RMSNorm prologue and residual / SwiGLU epilogues, plus the f16 LM-head GEMV.
//
// This is the numerically exact path (f32 activations, f32 accumulation) used for the greedy
// token-stream gate and as the fallback of the tensor-core decode path.  It replaces the
// reference's per-format decode kernels gemv_tq2_g128_v1, gemv_q1_g128_v7/_v8/_v9(+_residual),
// fused_gate_up_swiglu_q1, rmsnorm_weighted_v2, residual_add and swiglu_fused
// (crates/oxibonsai-kernels/src/gpu_backend/cuda_kernels.rs:76-776), folding the norm, the
// residual add and the activation into the GEMV launch.
//
// Work split: a thread owns one 64-input chunk of x in registers for the whole launch and
// streams that chunk of R rows at a time with 16-byte loads (R independent loads in flight);
// the chunk partial sums of a row are reduced through shared memory in a fixed order, so the
// result does not depend on the grid size.
#include "common.cuh"
#include "../comm/tp_comm.cuh"

namespace bonsai {

// EPI_TP_ALLREDUCE: row-parallel partial sums are pushed to every tensor-parallel peer and reduced
// with the residual inside this kernel (see comm/tp_comm.cuh).
enum { EPI_STORE = 0, EPI_RESID = 1, EPI_SWIGLU = 2, EPI_TP_ALLREDUCE = 3 };

template <int R>
__global__ void __launch_bounds__(256) bitgemv_kernel(const uint4* __restrict__ codes, const __half* __restrict__ scales,
                                                     const float* __restrict__ x, const float* __restrict__ norm_w, float eps,
                                                     float* __restrict__ out, const float* __restrict__ residual, int N, int K,
                                                     int epi, TpComm tp) {
  __shared__ float red[R][256];
  __shared__ float s32[32];
  const int t = threadIdx.x;
  const int tp_epoch = epi == EPI_TP_ALLREDUCE ? ld_volatile(tp.epoch) : 0;
  const int cpr = K >> 6;        // 64-input chunks per row
  const int G = 256 / cpr;       // row groups handled side by side
  const int g = t / cpr, c = t - g * cpr;
  const bool active = g < G;

  float xr[64];
  if (active) {
    const float4* xp = reinterpret_cast<const float4*>(x + (size_t)c * 64);
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      float4 v = xp[j];
      xr[4 * j] = v.x; xr[4 * j + 1] = v.y; xr[4 * j + 2] = v.z; xr[4 * j + 3] = v.w;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 64; ++j) xr[j] = 0.0f;
  }
  if (norm_w != nullptr) {
    float ss = 0.0f;
    if (active && g == 0) {
#pragma unroll
      for (int j = 0; j < 64; ++j) ss += xr[j] * xr[j];
    }
    ss = block_sum(ss, s32);
    float inv = 1.0f / sqrtf(ss / (float)K + eps);
    if (active) {
      const float4* wp = reinterpret_cast<const float4*>(norm_w + (size_t)c * 64);
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        float4 w = wp[j];
        xr[4 * j] = w.x * xr[4 * j] * inv;
        xr[4 * j + 1] = w.y * xr[4 * j + 1] * inv;
        xr[4 * j + 2] = w.z * xr[4 * j + 2] * inv;
        xr[4 * j + 3] = w.w * xr[4 * j + 3] * inv;
      }
    }
  }

  const int rows_per_tile = G * R;
  const int ntiles = (N + rows_per_tile - 1) / rows_per_tile;
  const int nsc = K >> 7;
  const int lane = t & 31, warp = t >> 5;

  for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
    const int row_base = tile * rows_per_tile + g * R;
    uint4 q[R];
    float d[R];
#pragma unroll
    for (int i = 0; i < R; ++i) {
      int row = row_base + i;
      if (active && row < N) {
        q[i] = __ldg(codes + (size_t)row * cpr + c);
        d[i] = __half2float(scales[(size_t)row * nsc + (c >> 1)]);
      } else {
        q[i] = make_uint4(0, 0, 0, 0);
        d[i] = 0.0f;
      }
    }
#pragma unroll
    for (int i = 0; i < R; ++i) {
      float acc = dot_word16(q[i].x, xr) + dot_word16(q[i].y, xr + 16) + dot_word16(q[i].z, xr + 32) + dot_word16(q[i].w, xr + 48);
      red[i][t] = acc * d[i];
    }
    __syncthreads();
    if (epi == EPI_SWIGLU) {
      for (int pr = warp; pr < rows_per_tile / 2; pr += 8) {
        int rr = pr * 2;
        int gg = rr / R, ii = rr - gg * R;
        float a = 0.0f, b = 0.0f;
        for (int j = lane; j < cpr; j += 32) {
          a += red[ii][gg * cpr + j];
          b += red[ii + 1][gg * cpr + j];
        }
        a = warp_sum(a) * kPow2_63;
        b = warp_sum(b) * kPow2_63;
        int row = tile * rows_per_tile + rr;
        if (lane == 0 && row + 1 < N) out[row >> 1] = a / (1.0f + expf(-a)) * b;
      }
    } else {
      for (int rr = warp; rr < rows_per_tile; rr += 8) {
        int gg = rr / R, ii = rr - gg * R;
        float a = 0.0f;
        for (int j = lane; j < cpr; j += 32) a += red[ii][gg * cpr + j];
        a = warp_sum(a) * kPow2_63;
        int row = tile * rows_per_tile + rr;
        if (lane == 0 && row < N) {
          if (epi == EPI_TP_ALLREDUCE) {
            for (int r = 0; r < tp.size; ++r) tp_recv_slot(tp, r, tp_epoch & 1, tp.rank)[row] = a;
          } else {
            out[row] = (epi == EPI_RESID) ? residual[row] + a : a;
          }
        }
      }
    }
    if (epi == EPI_TP_ALLREDUCE) tp_tile_allreduce(tp, tp_epoch, tile, tile * rows_per_tile, rows_per_tile, N, 0, residual, out);
    __syncthreads();
  }
  if (epi == EPI_TP_ALLREDUCE) tp_finish_kernel(tp, tp_epoch);
}

// Fast variant: activations held as half2 pairs, packed half-precision FMAs.  In the planar-SM word
// the sign and magnitude bits of weight a_p sit two bits apart (4p+3, 4p+1), exactly the spacing of
// the sign bit (15) and exponent bit 13 of a half, whose lone value is 2^-7.  One shift and one
// mask therefore turn a word into the half2 (a_p, a_{p+4}) = (+-2^-7 or 0, +-2^-7 or 0); the same
// holds for (b_p, b_{p+4}) one bit lower.  Three instructions (shift, mask, HFMA2) handle two
// weights.  A 64-input chunk is accumulated in four half2 chains of depth eight, widened to f32
// once per chunk, scaled by the group scale times 2^7 and reduced across chunks in f32.
template <int R>
__global__ void __launch_bounds__(256, 2) bitgemv_h2_kernel(const uint4* __restrict__ codes, const __half* __restrict__ scales,
                                                           const float* __restrict__ x, const float* __restrict__ norm_w,
                                                           float eps, float* __restrict__ out, const float* __restrict__ residual,
                                                           int N, int K, int epi, TpComm tp) {
  __shared__ float red[R][256];
  __shared__ float s32[32];
  const int t = threadIdx.x;
  const int cpr = K >> 6;
  const int G = 256 / cpr;
  const int g = t / cpr, c = t - g * cpr;
  const bool active = g < G;
  const int rows_per_tile = G * R;
  const int ntiles = (N + rows_per_tile - 1) / rows_per_tile;
  const int nsc = K >> 7;
  const int lane = t & 31, warp = t >> 5;

  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  // the first tile's weights do not depend on the previous kernel: fetch them before waiting
  uint4 q[R];
  float d[R];
  {
    const int row_base = blockIdx.x * rows_per_tile + g * R;
#pragma unroll
    for (int i = 0; i < R; ++i) {
      int row = row_base + i;
      bool ok = active && row < N && blockIdx.x < ntiles;
      q[i] = ok ? __ldg(codes + (size_t)row * cpr + c) : make_uint4(0, 0, 0, 0);
      d[i] = ok ? __half2float(scales[(size_t)row * nsc + (c >> 1)]) : 0.0f;
    }
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int tp_epoch = epi == EPI_TP_ALLREDUCE ? ld_volatile(tp.epoch) : 0;

  // activations: 64 floats -> 32 half2 in the pairing order of the packed words
  __half2 xh[32];
  {
    float xr[64];
    if (active) {
      const float4* xp = reinterpret_cast<const float4*>(x + (size_t)c * 64);
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        float4 v = xp[j];
        xr[4 * j] = v.x; xr[4 * j + 1] = v.y; xr[4 * j + 2] = v.z; xr[4 * j + 3] = v.w;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 64; ++j) xr[j] = 0.0f;
    }
    if (norm_w != nullptr) {
      float ss = 0.0f;
      if (active && g == 0) {
#pragma unroll
        for (int j = 0; j < 64; ++j) ss += xr[j] * xr[j];
      }
      ss = block_sum(ss, s32);
      float inv = 1.0f / sqrtf(ss / (float)K + eps);
      if (active) {
        const float4* wp = reinterpret_cast<const float4*>(norm_w + (size_t)c * 64);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          float4 w = wp[j];
          xr[4 * j] = w.x * xr[4 * j] * inv;
          xr[4 * j + 1] = w.y * xr[4 * j + 1] * inv;
          xr[4 * j + 2] = w.z * xr[4 * j + 2] * inv;
          xr[4 * j + 3] = w.w * xr[4 * j + 3] * inv;
        }
      }
    }
#pragma unroll
    for (int wd = 0; wd < 4; ++wd) {
#pragma unroll
      for (int p = 0; p < 4; ++p) {
        xh[wd * 8 + p] = __floats2half2_rn(xr[wd * 16 + p], xr[wd * 16 + p + 4]);           // (a_p, a_{p+4})
        xh[wd * 8 + 4 + p] = __floats2half2_rn(xr[wd * 16 + 8 + p], xr[wd * 16 + 12 + p]);  // (b_p, b_{p+4})
      }
    }
  }

  for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
    // issue the next tile's loads before consuming this one
    uint4 qn[R];
    float dn[R];
    {
      const int ntile = tile + gridDim.x;
      const int row_base = ntile * rows_per_tile + g * R;
#pragma unroll
      for (int i = 0; i < R; ++i) {
        int row = row_base + i;
        bool ok = active && ntile < ntiles && row < N;
        qn[i] = ok ? __ldg(codes + (size_t)row * cpr + c) : make_uint4(0, 0, 0, 0);
        dn[i] = ok ? __half2float(scales[(size_t)row * nsc + (c >> 1)]) : 0.0f;
      }
    }
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const uint32_t w4[4] = {q[i].x, q[i].y, q[i].z, q[i].w};
      __half2 a0 = __float2half2_rn(0.0f), a1 = a0, a2 = a0, a3 = a0;
#pragma unroll
      for (int wd = 0; wd < 4; ++wd) {
        const uint32_t w = w4[wd];
        uint32_t m;
        m = (w << 12) & 0xA000A000u; a0 = __hfma2(*reinterpret_cast<__half2*>(&m), xh[wd * 8 + 0], a0);
        m = (w << 8) & 0xA000A000u;  a1 = __hfma2(*reinterpret_cast<__half2*>(&m), xh[wd * 8 + 1], a1);
        m = (w << 4) & 0xA000A000u;  a2 = __hfma2(*reinterpret_cast<__half2*>(&m), xh[wd * 8 + 2], a2);
        m = w & 0xA000A000u;         a3 = __hfma2(*reinterpret_cast<__half2*>(&m), xh[wd * 8 + 3], a3);
        m = (w << 13) & 0xA000A000u; a0 = __hfma2(*reinterpret_cast<__half2*>(&m), xh[wd * 8 + 4], a0);
        m = (w << 9) & 0xA000A000u;  a1 = __hfma2(*reinterpret_cast<__half2*>(&m), xh[wd * 8 + 5], a1);
        m = (w << 5) & 0xA000A000u;  a2 = __hfma2(*reinterpret_cast<__half2*>(&m), xh[wd * 8 + 6], a2);
        m = (w << 1) & 0xA000A000u;  a3 = __hfma2(*reinterpret_cast<__half2*>(&m), xh[wd * 8 + 7], a3);
      }
      float2 f0 = __half22float2(a0), f1 = __half22float2(a1), f2 = __half22float2(a2), f3 = __half22float2(a3);
      float s = ((f0.x + f0.y) + (f1.x + f1.y)) + ((f2.x + f2.y) + (f3.x + f3.y));
      red[i][t] = s * d[i];
    }
    __syncthreads();
    if (epi == EPI_SWIGLU) {
      for (int pr = warp; pr < rows_per_tile / 2; pr += 8) {
        int rr = pr * 2;
        int gg = rr / R, ii = rr - gg * R;
        float a = 0.0f, b = 0.0f;
        for (int j = lane; j < cpr; j += 32) {
          a += red[ii][gg * cpr + j];
          b += red[ii + 1][gg * cpr + j];
        }
        a = warp_sum(a) * 128.0f;
        b = warp_sum(b) * 128.0f;
        int row = tile * rows_per_tile + rr;
        if (lane == 0 && row + 1 < N) out[row >> 1] = a / (1.0f + __expf(-a)) * b;
      }
    } else {
      for (int rr = warp; rr < rows_per_tile; rr += 8) {
        int gg = rr / R, ii = rr - gg * R;
        float a = 0.0f;
        for (int j = lane; j < cpr; j += 32) a += red[ii][gg * cpr + j];
        a = warp_sum(a) * 128.0f;
        int row = tile * rows_per_tile + rr;
        if (lane == 0 && row < N) {
          if (epi == EPI_TP_ALLREDUCE) {
            for (int r = 0; r < tp.size; ++r) tp_recv_slot(tp, r, tp_epoch & 1, tp.rank)[row] = a;
          } else {
            out[row] = (epi == EPI_RESID) ? residual[row] + a : a;
          }
        }
      }
    }
    if (epi == EPI_TP_ALLREDUCE) tp_tile_allreduce(tp, tp_epoch, tile, tile * rows_per_tile, rows_per_tile, N, 0, residual, out);
    __syncthreads();
#pragma unroll
    for (int i = 0; i < R; ++i) { q[i] = qn[i]; d[i] = dn[i]; }
  }
  if (epi == EPI_TP_ALLREDUCE) tp_finish_kernel(tp, tp_epoch);
}

// f16 row-major matrix [N][K] times f32 x, optional fused RMSNorm prologue.  Thread t owns the
// 8-input chunks t, t+256, ... (CH of them) of x.
template <int CH, int R>
__global__ void __launch_bounds__(256) f16gemv_kernel(const uint4* __restrict__ w, const float* __restrict__ x,
                                                     const float* __restrict__ norm_w, float eps, float* __restrict__ out,
                                                     int N, int K) {
  __shared__ float red[R][256];
  __shared__ float s32[32];
  const int t = threadIdx.x;
  const int cpr = K >> 3;
  float xr[CH][8];
  float ss = 0.0f;
#pragma unroll
  for (int h = 0; h < CH; ++h) {
    int c = t + h * 256;
    if (c < cpr) {
      const float4* xp = reinterpret_cast<const float4*>(x + (size_t)c * 8);
      float4 a = xp[0], b = xp[1];
      xr[h][0] = a.x; xr[h][1] = a.y; xr[h][2] = a.z; xr[h][3] = a.w;
      xr[h][4] = b.x; xr[h][5] = b.y; xr[h][6] = b.z; xr[h][7] = b.w;
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) xr[h][j] = 0.0f;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += xr[h][j] * xr[h][j];
  }
  if (norm_w != nullptr) {
    ss = block_sum(ss, s32);
    float inv = 1.0f / sqrtf(ss / (float)K + eps);
#pragma unroll
    for (int h = 0; h < CH; ++h) {
      int c = t + h * 256;
      if (c < cpr) {
        const float4* wp = reinterpret_cast<const float4*>(norm_w + (size_t)c * 8);
        float4 a = wp[0], b = wp[1];
        xr[h][0] = a.x * xr[h][0] * inv; xr[h][1] = a.y * xr[h][1] * inv;
        xr[h][2] = a.z * xr[h][2] * inv; xr[h][3] = a.w * xr[h][3] * inv;
        xr[h][4] = b.x * xr[h][4] * inv; xr[h][5] = b.y * xr[h][5] * inv;
        xr[h][6] = b.z * xr[h][6] * inv; xr[h][7] = b.w * xr[h][7] * inv;
      }
    }
  }
  const int ntiles = (N + R - 1) / R;
  const int lane = t & 31, warp = t >> 5;
  uint4 q[R][CH];
  auto load_tile = [&](int tile) {
#pragma unroll
    for (int i = 0; i < R; ++i) {
      int row = tile * R + i;
#pragma unroll
      for (int h = 0; h < CH; ++h) {
        int c = t + h * 256;
        q[i][h] = (tile < ntiles && row < N && c < cpr) ? __ldg(w + (size_t)row * cpr + c) : make_uint4(0, 0, 0, 0);
      }
    }
  };
  load_tile(blockIdx.x);
  for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
    float acc[R];
#pragma unroll
    for (int i = 0; i < R; ++i) {
      float a = 0.0f;
#pragma unroll
      for (int h = 0; h < CH; ++h) {
        const __half2* hp = reinterpret_cast<const __half2*>(&q[i][h]);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 f = __half22float2(hp[j]);
          a = fmaf(f.x, xr[h][2 * j], a);
          a = fmaf(f.y, xr[h][2 * j + 1], a);
        }
      }
      acc[i] = a;
    }
    load_tile(tile + gridDim.x);   // the next tile's rows stream in while this one is reduced across the block
#pragma unroll
    for (int i = 0; i < R; ++i) red[i][t] = acc[i];
    __syncthreads();
    for (int rr = warp; rr < R; rr += 8) {
      float a = 0.0f;
#pragma unroll
      for (int j = 0; j < 8; ++j) a += red[rr][lane + 32 * j];
      a = warp_sum(a);
      int row = tile * R + rr;
      if (lane == 0 && row < N) out[row] = a;
    }
    __syncthreads();
  }
}

// h[0..hidden) = f16 embedding row of token *token_ptr (token id read on the device).
__global__ void embed_f16_kernel(const __half* __restrict__ table, const int* __restrict__ token_ptr, float* __restrict__ h,
                                 int hidden, int vocab) {
  int tok = *token_ptr;
  tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);
  const __half* row = table + (size_t)tok * hidden;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < hidden; i += gridDim.x * blockDim.x) h[i] = __half2float(row[i]);
}

// h[t][0..hidden) = f16 embedding row of tokens[t], one block per token.
__global__ void embed_rows_f16_kernel(const __half* __restrict__ table, const int* __restrict__ tokens, float* __restrict__ h,
                                      int hidden, int vocab) {
  int tok = tokens[blockIdx.x];
  tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);
  const __half* row = table + (size_t)tok * hidden;
  float* o = h + (size_t)blockIdx.x * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = __half2float(row[i]);
}

}  // namespace bonsai

extern "C" {

int bonsai_embed_rows_f16(const void* table, const int* tokens, float* h, int T, int hidden, int vocab, cudaStream_t stream) {
  bonsai::embed_rows_f16_kernel<<<T, 256, 0, stream>>>((const __half*)table, tokens, h, hidden, vocab);
  return bonsai::launch_status();
}


// out[N] (or out[N/2] for epi = 2 with gate/up rows interleaved) = W x.  x is f32[K]; when norm_w is
// non-null x is first RMS-normalised with that weight.  K must be a multiple of 128 and <= 16384.
int bonsai_bitgemv(const void* codes, const void* scales, const float* x, const float* norm_w, float eps, float* out,
                   const float* residual, int N, int K, int epi, cudaStream_t stream) {
  using namespace bonsai;
  if (K % 128 != 0 || K < 128 || K > 16384 || N <= 0 || epi < 0 || epi > 2) return BONSAI_CUDA_BAD_ARG;
  if (epi == EPI_RESID && residual == nullptr) return BONSAI_CUDA_BAD_ARG;
  int cpr = K / 64, G = 256 / cpr;
  int tiles8 = (N + G * 8 - 1) / (G * 8);
  if (tiles8 >= 2 * 148) {
    int grid = tiles8 < 148 * 2 ? tiles8 : 148 * 2;
    bitgemv_kernel<8><<<grid, 256, 0, stream>>>((const uint4*)codes, (const __half*)scales, x, norm_w, eps, out, residual, N, K, epi, TpComm{});
  } else {
    int tiles4 = (N + G * 4 - 1) / (G * 4);
    int grid = tiles4 < 148 * 3 ? tiles4 : 148 * 3;
    bitgemv_kernel<4><<<grid, 256, 0, stream>>>((const uint4*)codes, (const __half*)scales, x, norm_w, eps, out, residual, N, K, epi, TpComm{});
  }
  return launch_status();
}

// Same contract as bonsai_bitgemv, computed with packed half-precision FMAs (activations rounded to
// f16, 8-deep f16 accumulation chains widened to f32).  Launched with programmatic dependent launch.
int bonsai_bitgemv_h2(const void* codes, const void* scales, const float* x, const float* norm_w, float eps, float* out,
                      const float* residual, int N, int K, int epi, cudaStream_t stream) {
  using namespace bonsai;
  if (K % 128 != 0 || K < 128 || K > 16384 || N <= 0 || epi < 0 || epi > 2) return BONSAI_CUDA_BAD_ARG;
  if (epi == EPI_RESID && residual == nullptr) return BONSAI_CUDA_BAD_ARG;
  int cpr = K / 64, G = 256 / cpr;
  int tiles8 = (N + G * 8 - 1) / (G * 8);
  cudaError_t e;
  if (tiles8 >= 2 * 148) {
    int grid = tiles8 < 148 * 2 ? tiles8 : 148 * 2;
    e = launch_pdl(bitgemv_h2_kernel<8>, dim3(grid), dim3(256), 0, stream, (const uint4*)codes, (const __half*)scales, x, norm_w, eps,
                   out, residual, N, K, epi, TpComm{});
  } else {
    int tiles4 = (N + G * 4 - 1) / (G * 4);
    int grid = tiles4 < 148 * 2 ? tiles4 : 148 * 2;
    e = launch_pdl(bitgemv_h2_kernel<4>, dim3(grid), dim3(256), 0, stream, (const uint4*)codes, (const __half*)scales, x, norm_w, eps,
                   out, residual, N, K, epi, TpComm{});
  }
  return e == cudaSuccess ? BONSAI_CUDA_OK : BONSAI_CUDA_LAUNCH_FAILED;
}

// Fused row-parallel GEMV -> all-reduce + residual over the tensor-parallel group `comm`:
// out[N] = residual[N] + sum over ranks of (W_rank x_rank).  Every rank must launch it with the same N
// and the same tiling (same K shard size and `fast` flag).  fast != 0 selects the packed-half kernel.
int bonsai_bitgemv_tp(const void* comm, const void* codes, const void* scales, const float* x, float eps, float* out,
                      const float* residual, int N, int K, int fast, cudaStream_t stream) {
  using namespace bonsai;
  if (comm == nullptr || K % 128 != 0 || K < 128 || K > 16384 || N <= 0) return BONSAI_CUDA_BAD_ARG;
  const TpComm tp = *static_cast<const TpComm*>(comm);
  if ((size_t)N > tp.lay.recv_elems) return BONSAI_CUDA_BAD_ARG;
  int cpr = K / 64, G = 256 / cpr;
  int tiles4 = (N + G * 4 - 1) / (G * 4);
  if (tiles4 > kTpMaxTiles) return BONSAI_CUDA_BAD_ARG;
  // every CTA waits on its peers: keep the whole grid co-resident (two CTAs per SM at most)
  int grid = tiles4 < 148 * 2 ? tiles4 : 148 * 2;
  cudaError_t e = cudaSuccess;
  if (fast) {
    e = launch_pdl(bitgemv_h2_kernel<4>, dim3(grid), dim3(256), 0, stream, (const uint4*)codes, (const __half*)scales, x,
                   (const float*)nullptr, eps, out, residual, N, K, (int)EPI_TP_ALLREDUCE, tp);
  } else {
    if (grid > 148) grid = 148;
    bitgemv_kernel<4><<<grid, 256, 0, stream>>>((const uint4*)codes, (const __half*)scales, x, nullptr, eps, out, residual, N, K,
                                                (int)EPI_TP_ALLREDUCE, tp);
    e = cudaGetLastError();
  }
  return e == cudaSuccess ? BONSAI_CUDA_OK : BONSAI_CUDA_LAUNCH_FAILED;
}

// out[N] = W x for an f16 row-major matrix (LM head); optional fused RMSNorm.  K % 8 == 0, K <= 8192.
int bonsai_f16gemv(const void* w, const float* x, const float* norm_w, float eps, float* out, int N, int K,
                   cudaStream_t stream) {
  using namespace bonsai;
  if (K % 8 != 0 || K <= 0 || K > 8192 || N <= 0) return BONSAI_CUDA_BAD_ARG;
  int ch = (K / 8 + 255) / 256;
  int ntiles = (N + 7) / 8;
  int grid = ntiles < 148 * 4 ? ntiles : 148 * 4;
  switch (ch) {
    case 1: f16gemv_kernel<1, 8><<<grid, 256, 0, stream>>>((const uint4*)w, x, norm_w, eps, out, N, K); break;
    case 2: f16gemv_kernel<2, 8><<<grid, 256, 0, stream>>>((const uint4*)w, x, norm_w, eps, out, N, K); break;
    case 3: f16gemv_kernel<3, 8><<<grid, 256, 0, stream>>>((const uint4*)w, x, norm_w, eps, out, N, K); break;
    default: f16gemv_kernel<4, 8><<<grid, 256, 0, stream>>>((const uint4*)w, x, norm_w, eps, out, N, K); break;
  }
  return launch_status();
}

int bonsai_embed_f16(const void* table, const int* token_ptr, float* h, int hidden, int vocab, cudaStream_t stream) {
  bonsai::embed_f16_kernel<<<(hidden + 255) / 256, 256, 0, stream>>>((const __half*)table, token_ptr, h, hidden, vocab);
  return bonsai::launch_status();
}

}  // extern "C"
