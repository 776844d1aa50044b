// bonsai_attn_decode_static: split-KV decode attention whose scratch is a static device array.
// Contract, limits and caller rules are in attention_decode_static.h.
#include "attention_decode_static.h"

#include <cstdio>
#include <mutex>

#include "common.cuh"

extern "C" int bonsai_attn_decode(const float* q, const int* positions, const int* block_table, int max_pages, int batch, int nq,
                                  int nkv, int hd, int kvt, int page_size, const void* kpool, const void* vpool,
                                  const float* kscale, const float* vscale, int nsplit, float* ws_acc, float* ws_ml,
                                  int* counters, float* out, int extra_len, cudaStream_t stream);

namespace {

struct AttnScratch {
  float acc[BONSAI_ATTN_STATIC_MAX_ACC_FLOATS];  // [batch][nq][nsplit][hd] partial numerators
  float ml[BONSAI_ATTN_STATIC_MAX_ML_FLOATS];    // [batch][nq][nsplit][2] partial max / sum
  int counters[BONSAI_ATTN_STATIC_MAX_COUNTERS]; // [batch][nkv] split arrival counters, zero between launches
};

// 4 MiB + 128 KiB + 16 KiB per device, zero-initialised when the module loads.
static __device__ __align__(256) unsigned char g_attn_scratch[sizeof(AttnScratch)];

constexpr int kMaxDevices = 64;
std::mutex g_mu;
AttnScratch* g_ptr[kMaxDevices] = {};

int fail(char* err, size_t cap, const char* fmt, long long a = 0, long long b = 0) {
  if (err != nullptr && cap > 0) std::snprintf(err, cap, fmt, a, b);
  return BONSAI_CUDA_BAD_ARG;
}

// Device address of the scratch array on the current device; resolved once per device.
int scratch_for_current_device(AttnScratch** out, char* err, size_t cap) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(err, cap, "cudaGetDevice failed (cuda error %lld)", (long long)e);
  if (dev < 0 || dev >= kMaxDevices) return fail(err, cap, "device ordinal %lld is outside the supported range 0..%lld", dev, kMaxDevices - 1);
  std::lock_guard<std::mutex> g(g_mu);
  if (g_ptr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_attn_scratch);
    if (e != cudaSuccess || p == nullptr) {
      (void)cudaGetLastError();
      return fail(err, cap, "cudaGetSymbolAddress for the attention scratch array failed (cuda error %lld)", (long long)e);
    }
    g_ptr[dev] = static_cast<AttnScratch*>(p);
  }
  *out = g_ptr[dev];
  return BONSAI_CUDA_OK;
}

}  // namespace

extern "C" int bonsai_attn_decode_static(const float* q, const int* positions, const int* block_table, int max_pages, int batch,
                                         int nq, int nkv, int hd, int kvt, int page_size, const void* kpool, const void* vpool,
                                         const float* kscale, const float* vscale, int nsplit, float* out, int extra_len,
                                         cudaStream_t stream, char* err, size_t err_cap) {
  if (err != nullptr && err_cap > 0) err[0] = '\0';
  if (batch <= 0 || nq <= 0 || nkv <= 0 || hd <= 0 || nsplit <= 0)
    return fail(err, err_cap, "batch, nq, nkv, hd and nsplit must be positive");
  const unsigned long long acc_floats = (unsigned long long)batch * nq * nsplit * hd;
  const unsigned long long ml_floats = (unsigned long long)batch * nq * nsplit * 2;
  const unsigned long long n_counters = (unsigned long long)batch * nkv;
  if (acc_floats > BONSAI_ATTN_STATIC_MAX_ACC_FLOATS)
    return fail(err, err_cap, "batch*nq*nsplit*hd = %lld floats exceeds the built-in scratch of %lld floats; use bonsai_attn_decode with caller buffers",
                (long long)acc_floats, (long long)BONSAI_ATTN_STATIC_MAX_ACC_FLOATS);
  if (ml_floats > BONSAI_ATTN_STATIC_MAX_ML_FLOATS)
    return fail(err, err_cap, "batch*nq*nsplit*2 = %lld floats exceeds the built-in max/sum scratch of %lld floats",
                (long long)ml_floats, (long long)BONSAI_ATTN_STATIC_MAX_ML_FLOATS);
  if (n_counters > BONSAI_ATTN_STATIC_MAX_COUNTERS)
    return fail(err, err_cap, "batch*nkv = %lld exceeds the %lld built-in arrival counters", (long long)n_counters,
                (long long)BONSAI_ATTN_STATIC_MAX_COUNTERS);
  AttnScratch* s = nullptr;
  int rc = scratch_for_current_device(&s, err, err_cap);
  if (rc != BONSAI_CUDA_OK) return rc;
  cudaError_t e = cudaMemsetAsync(s->counters, 0, n_counters * sizeof(int), stream);
  if (e != cudaSuccess) return fail(err, err_cap, "clearing the arrival counters failed (cuda error %lld)", (long long)e);
  rc = bonsai_attn_decode(q, positions, block_table, max_pages, batch, nq, nkv, hd, kvt, page_size, kpool, vpool, kscale, vscale,
                          nsplit, s->acc, s->ml, s->counters, out, extra_len, stream);
  if (rc != BONSAI_CUDA_OK) fail(err, err_cap, "bonsai_attn_decode rejected the arguments or the launch failed (code %lld)", rc);
  return rc;
}
