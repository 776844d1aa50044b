// Stand-alone forms of the small ops that the serving path folds into its GEMV / GEMM kernels: weighted RMSNorm over rows
// and residual add.  The reference launches them as kernels of their own in every layer (rmsnorm_weighted_v2, residual_add;
// crates/oxibonsai-kernels/src/gpu_backend/cuda_kernels.rs:335-393); here they serve library callers, tests and the
// engines of the generic block formats.
#include "common.cuh"

namespace bonsai {

// One block per row: y = x * rsqrt(mean(x^2) + eps) * w.  Rows of up to 16 * blockDim.x elements are read once.
__global__ void __launch_bounds__(256) rmsnorm_rows_kernel(const float* __restrict__ x, int x_ld, const float* __restrict__ w, float eps, int K,
                                                          float* __restrict__ out, int out_ld) {
  __shared__ float s32[32];
  const float* xr = x + (size_t)blockIdx.x * x_ld;
  float* orow = out + (size_t)blockIdx.x * out_ld;
  float ss = 0.0f;
  for (int k = threadIdx.x; k < K; k += blockDim.x) ss += xr[k] * xr[k];
  ss = block_sum(ss, s32);
  const float inv = 1.0f / sqrtf(ss / (float)K + eps);
  for (int k = threadIdx.x; k < K; k += blockDim.x) orow[k] = xr[k] * inv * (w != nullptr ? w[k] : 1.0f);
}

__global__ void residual_add_kernel(float* __restrict__ a, const float* __restrict__ b, size_t n) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) a[i] += b[i];
}

}  // namespace bonsai

extern "C" {

// out[T][out_ld] = rmsnorm(x[T][x_ld]) * w (w may be null: plain normalisation); out may alias x.
int bonsai_rmsnorm_rows(const float* x, int x_ld, const float* w, float eps, int T, int K, float* out, int out_ld, cudaStream_t stream) {
  if (T < 1 || K < 1 || x_ld < K || out_ld < K) return BONSAI_CUDA_BAD_ARG;
  bonsai::rmsnorm_rows_kernel<<<T, 256, 0, stream>>>(x, x_ld, w, eps, K, out, out_ld);
  return bonsai::launch_status();
}

// a[n] += b[n]
int bonsai_residual_add(float* a, const float* b, size_t n, cudaStream_t stream) {
  if (n == 0) return BONSAI_CUDA_BAD_ARG;
  size_t blocks = (n + 255) / 256;
  const int grid = (int)(blocks < (size_t)(148 * 8) ? blocks : (size_t)(148 * 8));
  bonsai::residual_add_kernel<<<grid, 256, 0, stream>>>(a, b, n);
  return bonsai::launch_status();
}

}  // extern "C"
