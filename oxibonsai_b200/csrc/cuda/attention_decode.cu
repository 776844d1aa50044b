// Decode-side attention: fused per-head QK RMSNorm + half-split RoPE + paged KV append, and
// split-KV (flash-decode) GQA attention over paged F32 / F16 / Q8 / Q4 caches.
//
// Replaces the reference's seven attention launches per layer - fused_qk_norm, fused_qk_rope,
// fused_qk_norm_rope, fused_kv_store, batched_attn_scores_v2, batched_softmax and
// batched_attn_weighted_sum (crates/oxibonsai-kernels/src/gpu_backend/cuda_attn_kernels.rs:63-439) -
// with two kernels plus a small merge.  Unlike the reference, whose score grid is sized for the
// maximum sequence length, work is proportional to the live context, pages are looked up through
// a block table (crates/oxibonsai-model/src/paged_kv_cache.rs:33-240), the KV heads of a GQA
// group share every K/V load, and the cache can be stored as INT8 with one f32 scale per
// (token, head) row (scale = absmax/127, crates/oxibonsai-model/src/kv_cache_quant.rs:46-71) or as
// INT4 (scale = absmax/7, nibble = q + 8), a format the reference names in its policy levels but
// never stores.
//
// Pool layout, per layer and separately for K and V:  data [page][kv_head][slot][row bytes],
// scales f32 [page][kv_head][slot] (quantised formats only).  Position and block tables live in
// device memory so a captured CUDA graph stays valid as sequences grow.
#include "common.cuh"

namespace bonsai {

enum { KV_F32 = 0, KV_F16 = 1, KV_Q8 = 2, KV_Q4 = 3 };

__host__ __device__ inline int kv_row_bytes(int kvt, int hd) {
  return kvt == KV_F32 ? hd * 4 : (kvt == KV_F16 ? hd * 2 : (kvt == KV_Q8 ? hd : hd / 2));
}

struct KvPool {
  uint8_t* k;       // this layer's K pool
  uint8_t* v;       // this layer's V pool
  float* k_scale;   // may be null for F32 / F16
  float* v_scale;
  int page_size;
  int kv_heads;
  int hd;
  int kvt;
};

// One block per (head, sequence); blockDim.x == head_dim.  Heads [0, nq) are queries, [nq, nq+nkv)
// keys, [nq+nkv, nq+2nkv) values.
__global__ void qknorm_rope_kvstore_kernel(const float* __restrict__ qkv, int qkv_stride, const float* __restrict__ q_norm,
                                           const float* __restrict__ k_norm, float eps, const float* __restrict__ rope_cos,
                                           const float* __restrict__ rope_sin, const int* __restrict__ positions,
                                           const int* __restrict__ block_table, int max_pages, float* __restrict__ q_out,
                                           int nq, KvPool pool) {
  extern __shared__ float sh[];  // hd floats + 32
  const int hd = pool.hd, nkv = pool.kv_heads;
  const int head = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
  const int pos = positions[b];
  const float* src = qkv + (size_t)b * qkv_stride + (size_t)head * hd;
  float x = src[d];
  const bool is_q = head < nq, is_k = !is_q && head < nq + nkv;
  float y = x;
  if (is_q || is_k) {
    float ss = block_sum(x * x, sh + hd);
    float inv = 1.0f / sqrtf(ss / (float)hd + eps);
    float w = is_q ? q_norm[d] : k_norm[d];
    float n = w * x * inv;
    sh[d] = n;
    __syncthreads();
    int half = hd >> 1;
    int i = d < half ? d : d - half;
    float c = rope_cos[(size_t)pos * half + i], s = rope_sin[(size_t)pos * half + i];
    float x0 = sh[i], x1 = sh[half + i];
    y = d < half ? x0 * c - x1 * s : x0 * s + x1 * c;
  }
  if (is_q) {
    q_out[((size_t)b * nq + head) * hd + d] = y;
    return;
  }
  const int kvh = is_k ? head - nq : head - nq - nkv;
  const int page = block_table[(size_t)b * max_pages + pos / pool.page_size];
  const int slot = pos % pool.page_size;
  const size_t row = ((size_t)page * nkv + kvh) * pool.page_size + slot;
  uint8_t* base = is_k ? pool.k : pool.v;
  float* sc = is_k ? pool.k_scale : pool.v_scale;
  if (pool.kvt == KV_F32) {
    reinterpret_cast<float*>(base)[row * hd + d] = y;
  } else if (pool.kvt == KV_F16) {
    reinterpret_cast<__half*>(base)[row * hd + d] = __float2half_rn(y);
  } else {
    // quantised rows: absmax over the head, then round to nearest
    __syncthreads();
    float m = warp_max(fabsf(y));
    if ((d & 31) == 0) sh[hd + (d >> 5)] = m;
    __syncthreads();
    float amax = 0.0f;
    for (int w = 0; w < (hd + 31) / 32; ++w) amax = fmaxf(amax, sh[hd + w]);
    float qmax = pool.kvt == KV_Q8 ? 127.0f : 7.0f;
    float scale = fmaxf(amax / qmax, 1e-12f);
    int q = __float2int_rn(y / scale);
    q = max(-(int)qmax, min((int)qmax, q));
    if (d == 0) sc[row] = scale;
    if (pool.kvt == KV_Q8) {
      reinterpret_cast<int8_t*>(base)[row * hd + d] = (int8_t)q;
    } else {
      int other = __shfl_xor_sync(0xffffffffu, q, 1);
      if ((d & 1) == 0) base[row * (hd / 2) + (d >> 1)] = (uint8_t)((q + 8) | ((other + 8) << 4));
    }
  }
}

template <int KVT, int DPL>
__device__ __forceinline__ void load_row(const uint8_t* base, const float* scales, size_t row, int hd, int lane, float* out) {
  if (KVT == KV_F32) {
    const float* p = reinterpret_cast<const float*>(base) + row * hd + lane * DPL;
#pragma unroll
    for (int j = 0; j < DPL; ++j) out[j] = p[j];
  } else if (KVT == KV_F16) {
    const __half2* p = reinterpret_cast<const __half2*>(reinterpret_cast<const __half*>(base) + row * hd + lane * DPL);
#pragma unroll
    for (int j = 0; j < DPL / 2; ++j) {
      float2 f = __half22float2(p[j]);
      out[2 * j] = f.x;
      out[2 * j + 1] = f.y;
    }
  } else if (KVT == KV_Q8) {
    const int8_t* p = reinterpret_cast<const int8_t*>(base) + row * hd + lane * DPL;
    float s = scales[row];
#pragma unroll
    for (int j = 0; j < DPL; ++j) out[j] = s * (float)p[j];
  } else {
    const uint8_t* p = base + row * (hd / 2) + lane * (DPL / 2);
    float s = scales[row];
#pragma unroll
    for (int j = 0; j < DPL / 2; ++j) {
      uint32_t v = p[j];
      out[2 * j] = s * (float)((int)(v & 15u) - 8);
      out[2 * j + 1] = s * (float)((int)(v >> 4) - 8);
    }
  }
}

// grid (kv_heads, splits, batch), block 256 (8 warps).  Each warp walks its share of the split's
// tokens four at a time (independent K/V loads in flight), the warps are combined in shared
// memory and the split's partial (max, sum, weighted V) goes to the workspace; the last CTA of a
// (sequence, kv head) to finish merges all splits in split order and writes the attention output.
constexpr int kAttnWarps = 8;
constexpr int kAttnUnroll = 4;

template <int KVT, int DPL, int G>
__global__ void __launch_bounds__(256) attn_decode_kernel(const float* __restrict__ q, const int* __restrict__ positions,
                                                         const int* __restrict__ block_table, int max_pages, KvPool pool,
                                                         int nq, float sm_scale, float* __restrict__ ws_acc,
                                                         float* __restrict__ ws_ml, int* __restrict__ counters,
                                                         float* __restrict__ out, int extra_len) {
  extern __shared__ float sh[];  // [8 warps][G][hd + 2]
  __shared__ int s_last;
  const int hd = pool.hd, nkv = pool.kv_heads;
  const int kvh = blockIdx.x, split = blockIdx.y, nsplit = gridDim.y, b = blockIdx.z;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int len = positions[b] + 1 + extra_len;
  const int chunk = (len + nsplit - 1) / nsplit;
  const int t0 = split * chunk, t1 = min(len, t0 + chunk);

  float qr[G][DPL], acc[G][DPL], m[G], l[G];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const float* qp = q + ((size_t)b * nq + kvh * G + g) * hd + lane * DPL;
#pragma unroll
    for (int j = 0; j < DPL; ++j) {
      qr[g][j] = qp[j] * sm_scale;
      acc[g][j] = 0.0f;
    }
    m[g] = -INFINITY;
    l[g] = 0.0f;
  }
  const int* bt = block_table + (size_t)b * max_pages;
  for (int tb = t0 + warp; tb < t1; tb += kAttnWarps * kAttnUnroll) {
    float kr[kAttnUnroll][DPL], vr[kAttnUnroll][DPL];
    bool valid[kAttnUnroll];
#pragma unroll
    for (int u = 0; u < kAttnUnroll; ++u) {
      const int t = tb + u * kAttnWarps;
      valid[u] = t < t1;
      const int tt = valid[u] ? t : t0;
      const int page = bt[tt / pool.page_size];
      const size_t row = ((size_t)page * nkv + kvh) * pool.page_size + (tt % pool.page_size);
      load_row<KVT, DPL>(pool.k, pool.k_scale, row, hd, lane, kr[u]);
      load_row<KVT, DPL>(pool.v, pool.v_scale, row, hd, lane, vr[u]);
    }
    float s[kAttnUnroll][G];
#pragma unroll
    for (int u = 0; u < kAttnUnroll; ++u)
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float a = 0.0f;
#pragma unroll
        for (int j = 0; j < DPL; ++j) a = fmaf(qr[g][j], kr[u][j], a);
        s[u][g] = a;
      }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
#pragma unroll
      for (int u = 0; u < kAttnUnroll; ++u)
#pragma unroll
        for (int g = 0; g < G; ++g) s[u][g] += __shfl_xor_sync(0xffffffffu, s[u][g], o);
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float mn = m[g];
#pragma unroll
      for (int u = 0; u < kAttnUnroll; ++u)
        if (valid[u]) mn = fmaxf(mn, s[u][g]);
      const float r = expf(m[g] - mn);  // exp(-inf) = 0 before the first token
      float p[kAttnUnroll], ps = 0.0f;
#pragma unroll
      for (int u = 0; u < kAttnUnroll; ++u) {
        p[u] = valid[u] ? expf(s[u][g] - mn) : 0.0f;
        ps += p[u];
      }
      l[g] = l[g] * r + ps;
#pragma unroll
      for (int j = 0; j < DPL; ++j) {
        float a = acc[g][j] * r;
#pragma unroll
        for (int u = 0; u < kAttnUnroll; ++u) a = fmaf(p[u], vr[u][j], a);
        acc[g][j] = a;
      }
      m[g] = mn;
    }
  }
  // combine the warps
  const int stride = hd + 2;
#pragma unroll
  for (int g = 0; g < G; ++g) {
    float* dst = sh + ((size_t)warp * G + g) * stride;
#pragma unroll
    for (int j = 0; j < DPL; ++j) dst[lane * DPL + j] = acc[g][j];
    if (lane == 0) {
      dst[hd] = m[g];
      dst[hd + 1] = l[g];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * hd; idx += blockDim.x) {
    int g = idx / hd, d = idx - g * hd;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) M = fmaxf(M, sh[((size_t)w * G + g) * stride + hd]);
    float a = 0.0f, L = 0.0f;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) {
      const float* src = sh + ((size_t)w * G + g) * stride;
      float f = (src[hd] == -INFINITY) ? 0.0f : expf(src[hd] - M);
      a += f * src[d];
      L += f * src[hd + 1];
    }
    size_t o = (((size_t)b * nq + kvh * G + g) * nsplit + split);
    ws_acc[o * hd + d] = a;
    if (d == 0) {
      ws_ml[o * 2] = M;
      ws_ml[o * 2 + 1] = L;
    }
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    int* ctr = counters + (size_t)b * nkv + kvh;
    int prev = atomicAdd(ctr, 1);
    s_last = (prev == nsplit - 1);
    if (s_last) *ctr = 0;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  for (int idx = threadIdx.x; idx < G * hd; idx += blockDim.x) {
    int g = idx / hd, d = idx - g * hd;
    size_t hb = ((size_t)b * nq + kvh * G + g);
    // eight splits per step with all loads issued before the first use: a loop that consumes each load at once is a
    // chain of exposed L2 round trips (2 x nsplit of them)
    const float2* ml = reinterpret_cast<const float2*>(ws_ml) + hb * nsplit;
    const float* ac = ws_acc + hb * nsplit * hd + d;
    float M = -INFINITY;
    for (int sp0 = 0; sp0 < nsplit; sp0 += 8) {
      float x[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) x[i] = sp0 + i < nsplit ? __ldcg(ml + sp0 + i).x : -INFINITY;
#pragma unroll
      for (int i = 0; i < 8; ++i) M = fmaxf(M, x[i]);
    }
    float a = 0.0f, L = 0.0f;
    for (int sp0 = 0; sp0 < nsplit; sp0 += 8) {
      float2 mlv[8];
      float av[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const bool ok = sp0 + i < nsplit;
        mlv[i] = ok ? __ldcg(ml + sp0 + i) : make_float2(-INFINITY, 0.0f);
        av[i] = ok ? __ldcg(ac + (size_t)(sp0 + i) * hd) : 0.0f;
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float f = (mlv[i].x == -INFINITY) ? 0.0f : expf(mlv[i].x - M);
        a += f * av[i];
        L += f * mlv[i].y;
      }
    }
    out[hb * hd + d] = L > 0.0f ? a / L : 0.0f;
  }
}

// ---- head_dim 128, compressed caches: half a warp per token --------------------------------------------
// A 128-wide f16 row is 256 bytes = 16 lanes x 16 bytes, so the two halves of a warp walk two tokens
// at once with full-width loads; kH128Unroll such pairs are requested before any is consumed (8
// tokens x 2 rows in flight per warp).  Each half keeps its own online-softmax state, the halves are
// folded with shuffles at the end, and from there on the warp / split merges are those of the
// generic kernel above.  Q8 rows are 8-byte loads plus the row scale, Q4 rows 4-byte loads.
constexpr int kH128Unroll = 4;

template <int KVT>
struct RawRow8 {
  uint4 v;   // F16: 8 halves; Q8: x,y = 8 int8; Q4: x = 8 nibbles
  float s;
};

template <int KVT>
__device__ __forceinline__ void load_raw8(const uint8_t* base, const float* scales, size_t row, int sub, RawRow8<KVT>& r) {
  if (KVT == KV_F16) {
    r.v = *reinterpret_cast<const uint4*>(base + row * 256 + sub * 16);
    r.s = 1.0f;
  } else if (KVT == KV_Q8) {
    const uint2 t = *reinterpret_cast<const uint2*>(base + row * 128 + sub * 8);
    r.v = make_uint4(t.x, t.y, 0u, 0u);
    r.s = scales[row];
  } else {
    r.v = make_uint4(*reinterpret_cast<const uint32_t*>(base + row * 64 + sub * 4), 0u, 0u, 0u);
    r.s = scales[row];
  }
}

template <int KVT>
__device__ __forceinline__ void unpack8(const RawRow8<KVT>& r, float* out) {
  if (KVT == KV_F16) {
    const uint32_t w[4] = {r.v.x, r.v.y, r.v.z, r.v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
      out[2 * j] = f.x;
      out[2 * j + 1] = f.y;
    }
  } else if (KVT == KV_Q8) {
    const uint32_t w[2] = {r.v.x, r.v.y};
#pragma unroll
    for (int j = 0; j < 8; ++j) out[j] = r.s * (float)(int)(int8_t)((w[j >> 2] >> (8 * (j & 3))) & 0xFFu);
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) out[j] = r.s * (float)((int)((r.v.x >> (4 * j)) & 15u) - 8);
  }
}

template <int KVT, int G>
__global__ void __launch_bounds__(256, 2) attn_decode_h128_kernel(const float* __restrict__ q, const int* __restrict__ positions,
                                                                 const int* __restrict__ block_table, int max_pages, KvPool pool,
                                                                 int nq, float sm_scale, float* __restrict__ ws_acc,
                                                                 float* __restrict__ ws_ml, int* __restrict__ counters,
                                                                 float* __restrict__ out, int extra_len) {
  extern __shared__ float sh[];  // [8 warps][G][hd + 2]
  __shared__ int s_last;
  constexpr int hd = 128;
  const int nkv = pool.kv_heads;
  const int kvh = blockIdx.x, split = blockIdx.y, nsplit = gridDim.y, b = blockIdx.z;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int half = lane >> 4, sub = lane & 15;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int* bt = block_table + (size_t)b * max_pages;
  const int pshift = 31 - __clz(pool.page_size), pmask = pool.page_size - 1;   // the launcher admits power-of-two pages only
  {
    // Ask L2 for this CTA's K and V rows while the previous kernel is still running.  Rows of earlier tokens do not
    // depend on it; the position and block-table entries read here may be one step old (they are re-read after the
    // wait), which only shifts what gets prefetched.  With ~110 tokens per CTA the loop below is two load rounds, so
    // without this it pays the DRAM latency twice, after the dependency wait.
    constexpr int kRowBytes = KVT == KV_F16 ? 256 : (KVT == KV_Q8 ? 128 : 64);
    constexpr int kLines = kRowBytes >= 128 ? kRowBytes / 128 : 1;
    const int plen = positions[b] + 1 + extra_len;
    const int pchunk = (plen + nsplit - 1) / nsplit;
    const int p0 = split * pchunk, p1 = min(plen, p0 + pchunk);
    for (int i = threadIdx.x; i < (p1 - p0) * 2 * kLines; i += blockDim.x) {
      const int tok = p0 + i / (2 * kLines), which = (i / kLines) & 1, line = i % kLines;
      const int page = bt[tok >> pshift];
      if (page < 0) continue;
      const size_t row = ((size_t)page * nkv + kvh) * pool.page_size + (tok & pmask);
      const uint8_t* ptr = (which ? pool.v : pool.k) + row * kRowBytes + line * 128;
      asm volatile("prefetch.global.L2 [%0];" ::"l"(ptr));
    }
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int len = positions[b] + 1 + extra_len;
  const int chunk = (len + nsplit - 1) / nsplit;
  const int t0 = split * chunk, t1 = min(len, t0 + chunk);

  float qr[G][8], acc[G][8], m[G], l[G];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const float4* qp = reinterpret_cast<const float4*>(q + ((size_t)b * nq + kvh * G + g) * hd + sub * 8);
    const float4 a = qp[0], c = qp[1];
    qr[g][0] = a.x * sm_scale; qr[g][1] = a.y * sm_scale; qr[g][2] = a.z * sm_scale; qr[g][3] = a.w * sm_scale;
    qr[g][4] = c.x * sm_scale; qr[g][5] = c.y * sm_scale; qr[g][6] = c.z * sm_scale; qr[g][7] = c.w * sm_scale;
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[g][j] = 0.0f;
    m[g] = -INFINITY;
    l[g] = 0.0f;
  }
  constexpr int kTok = 2 * kH128Unroll;   // tokens per warp iteration
  for (int tb = t0 + warp * kTok; tb < t1; tb += kAttnWarps * kTok) {
    RawRow8<KVT> kr[kH128Unroll], vr[kH128Unroll];
    bool valid[kH128Unroll];
#pragma unroll
    for (int u = 0; u < kH128Unroll; ++u) {
      const int t = tb + 2 * u + half;
      valid[u] = t < t1;
      const int tt = valid[u] ? t : t0;
      const int page = bt[tt >> pshift];
      const size_t row = ((size_t)page * nkv + kvh) * pool.page_size + (tt & pmask);
      load_raw8<KVT>(pool.k, pool.k_scale, row, sub, kr[u]);
      load_raw8<KVT>(pool.v, pool.v_scale, row, sub, vr[u]);
    }
    float s[kH128Unroll][G];
#pragma unroll
    for (int u = 0; u < kH128Unroll; ++u) {
      float kf[8];
      unpack8<KVT>(kr[u], kf);
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float a = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) a = fmaf(qr[g][j], kf[j], a);
        s[u][g] = a;
      }
    }
#pragma unroll
    for (int o = 8; o > 0; o >>= 1)
#pragma unroll
      for (int u = 0; u < kH128Unroll; ++u)
#pragma unroll
        for (int g = 0; g < G; ++g) s[u][g] += __shfl_xor_sync(0xffffffffu, s[u][g], o);
    float p[kH128Unroll][G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float mn = m[g];
#pragma unroll
      for (int u = 0; u < kH128Unroll; ++u)
        if (valid[u]) mn = fmaxf(mn, s[u][g]);
      const float r = __expf(m[g] - mn);   // exp(-inf) = 0 before the first token; a half with no token yet keeps m = -inf
      float ps = 0.0f;
#pragma unroll
      for (int u = 0; u < kH128Unroll; ++u) {
        p[u][g] = valid[u] ? __expf(s[u][g] - mn) : 0.0f;
        ps += p[u][g];
      }
      const float rr = (mn == -INFINITY) ? 1.0f : r;
      l[g] = l[g] * rr + ps;
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[g][j] *= rr;
      m[g] = mn;
    }
#pragma unroll
    for (int u = 0; u < kH128Unroll; ++u) {
      float vf[8];
      unpack8<KVT>(vr[u], vf);
#pragma unroll
      for (int g = 0; g < G; ++g)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[g][j] = fmaf(p[u][g], vf[j], acc[g][j]);
    }
  }
  // fold the two halves of the warp (they saw different tokens)
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const float mo = __shfl_xor_sync(0xffffffffu, m[g], 16), lo = __shfl_xor_sync(0xffffffffu, l[g], 16);
    const float M = fmaxf(m[g], mo);
    const float fa = (m[g] == -INFINITY) ? 0.0f : __expf(m[g] - M), fb = (mo == -INFINITY) ? 0.0f : __expf(mo - M);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float ao = __shfl_xor_sync(0xffffffffu, acc[g][j], 16);
      acc[g][j] = fa * acc[g][j] + fb * ao;
    }
    l[g] = fa * l[g] + fb * lo;
    m[g] = M;
  }
  // combine the warps (same scheme as the generic kernel)
  const int stride = hd + 2;
  if (half == 0) {
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float* dst = sh + ((size_t)warp * G + g) * stride;
#pragma unroll
      for (int j = 0; j < 8; ++j) dst[sub * 8 + j] = acc[g][j];
      if (sub == 0) {
        dst[hd] = m[g];
        dst[hd + 1] = l[g];
      }
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * hd; idx += blockDim.x) {
    int g = idx / hd, d = idx - g * hd;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) M = fmaxf(M, sh[((size_t)w * G + g) * stride + hd]);
    float a = 0.0f, L = 0.0f;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) {
      const float* src = sh + ((size_t)w * G + g) * stride;
      float f = (src[hd] == -INFINITY) ? 0.0f : __expf(src[hd] - M);
      a += f * src[d];
      L += f * src[hd + 1];
    }
    size_t o = (((size_t)b * nq + kvh * G + g) * nsplit + split);
    ws_acc[o * hd + d] = a;
    if (d == 0) {
      ws_ml[o * 2] = M;
      ws_ml[o * 2 + 1] = L;
    }
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    int* ctr = counters + (size_t)b * nkv + kvh;
    int prev = atomicAdd(ctr, 1);
    s_last = (prev == nsplit - 1);
    if (s_last) *ctr = 0;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  // Merge of the splits by the last CTA of this (sequence, kv head).  Every dependent trip to L2 costs ~600 cycles
  // here, so the (max, sum) pairs go to shared memory in one trip, one warp per query head turns them into weights
  // f[sp] = exp(m_sp - M) / L, and each thread then sums its outputs over the splits with twenty loads in flight.
  float* s_f = sh;                    // [G][nsplit] weights (the warp-merge staging area is free by now)
  float* s_l = sh + G * nsplit;       // [G][nsplit] partial sums
  const size_t hb0 = (size_t)b * nq + kvh * G;
  for (int i = threadIdx.x; i < G * nsplit; i += blockDim.x) {
    const float2 v = __ldcg(reinterpret_cast<const float2*>(ws_ml) + hb0 * nsplit + i);   // heads of a group are adjacent
    s_f[i] = v.x;
    s_l[i] = v.y;
  }
  __syncthreads();
  if (warp < G) {
    float M = -INFINITY;
    for (int sp = lane; sp < nsplit; sp += 32) M = fmaxf(M, s_f[warp * nsplit + sp]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
    float L = 0.0f;
    for (int sp = lane; sp < nsplit; sp += 32) {
      const float ms = s_f[warp * nsplit + sp];
      const float f = (ms == -INFINITY) ? 0.0f : __expf(ms - M);
      L += f * s_l[warp * nsplit + sp];
      s_f[warp * nsplit + sp] = f;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) L += __shfl_xor_sync(0xffffffffu, L, o);
    const float inv = L > 0.0f ? 1.0f / L : 0.0f;
    for (int sp = lane; sp < nsplit; sp += 32) s_f[warp * nsplit + sp] *= inv;
  }
  __syncthreads();
  constexpr int NI = (G * hd + 255) / 256;   // outputs per thread
  float a[NI];
  const float* ac[NI];
  const float* fw[NI];
#pragma unroll
  for (int k = 0; k < NI; ++k) {
    const int idx = min(threadIdx.x + k * 256, G * hd - 1);
    const int g = idx / hd, d = idx - g * hd;
    ac[k] = ws_acc + (hb0 + g) * nsplit * hd + d;
    fw[k] = s_f + g * nsplit;
    a[k] = 0.0f;
  }
  constexpr int SB = 20 / NI;   // splits per step
  for (int sp0 = 0; sp0 < nsplit; sp0 += SB) {
    float av[NI][SB];
#pragma unroll
    for (int k = 0; k < NI; ++k)
#pragma unroll
      for (int i = 0; i < SB; ++i) av[k][i] = sp0 + i < nsplit ? __ldcg(ac[k] + (size_t)(sp0 + i) * hd) : 0.0f;
#pragma unroll
    for (int k = 0; k < NI; ++k)
#pragma unroll
      for (int i = 0; i < SB; ++i) a[k] += (sp0 + i < nsplit ? fw[k][sp0 + i] : 0.0f) * av[k][i];
  }
#pragma unroll
  for (int k = 0; k < NI; ++k) {
    const int idx = threadIdx.x + k * 256;
    if (idx < G * hd) out[hb0 * hd + idx] = a[k];
  }
}

template <int KVT>
int launch_decode_h128(int G, dim3 grid, size_t smem, cudaStream_t st, const float* q, const int* pos, const int* bt, int max_pages,
                       KvPool pool, int nq, float sc, float* wa, float* wm, int* ctr, float* out, int extra) {
  cudaError_t e;
  switch (G) {
    case 1: e = launch_pdl(attn_decode_h128_kernel<KVT, 1>, grid, dim3(256), smem, st, q, pos, bt, max_pages, pool, nq, sc, wa, wm, ctr, out, extra); break;
    case 2: e = launch_pdl(attn_decode_h128_kernel<KVT, 2>, grid, dim3(256), smem, st, q, pos, bt, max_pages, pool, nq, sc, wa, wm, ctr, out, extra); break;
    case 4: e = launch_pdl(attn_decode_h128_kernel<KVT, 4>, grid, dim3(256), smem, st, q, pos, bt, max_pages, pool, nq, sc, wa, wm, ctr, out, extra); break;
    default: return BONSAI_CUDA_BAD_ARG;
  }
  return e == cudaSuccess ? BONSAI_CUDA_OK : BONSAI_CUDA_LAUNCH_FAILED;
}

template <int KVT, int DPL>
int launch_decode_g(int G, dim3 grid, size_t smem, cudaStream_t st, const float* q, const int* pos, const int* bt, int max_pages,
                    KvPool pool, int nq, float sc, float* wa, float* wm, int* ctr, float* out, int extra) {
  cudaError_t e;
  switch (G) {
    case 1: e = launch_pdl(attn_decode_kernel<KVT, DPL, 1>, grid, dim3(256), smem, st, q, pos, bt, max_pages, pool, nq, sc, wa, wm, ctr, out, extra); break;
    case 2: e = launch_pdl(attn_decode_kernel<KVT, DPL, 2>, grid, dim3(256), smem, st, q, pos, bt, max_pages, pool, nq, sc, wa, wm, ctr, out, extra); break;
    case 4: e = launch_pdl(attn_decode_kernel<KVT, DPL, 4>, grid, dim3(256), smem, st, q, pos, bt, max_pages, pool, nq, sc, wa, wm, ctr, out, extra); break;
    case 8: e = launch_pdl(attn_decode_kernel<KVT, DPL, 8>, grid, dim3(256), smem, st, q, pos, bt, max_pages, pool, nq, sc, wa, wm, ctr, out, extra); break;
    default: return BONSAI_CUDA_BAD_ARG;
  }
  return e == cudaSuccess ? BONSAI_CUDA_OK : BONSAI_CUDA_LAUNCH_FAILED;
}

template <int KVT>
int launch_decode_d(int dpl, int G, dim3 grid, size_t smem, cudaStream_t st, const float* q, const int* pos, const int* bt,
                    int max_pages, KvPool pool, int nq, float sc, float* wa, float* wm, int* ctr, float* out, int extra) {
  switch (dpl) {
    case 2: return launch_decode_g<KVT, 2>(G, grid, smem, st, q, pos, bt, max_pages, pool, nq, sc, wa, wm, ctr, out, extra);
    case 4: return launch_decode_g<KVT, 4>(G, grid, smem, st, q, pos, bt, max_pages, pool, nq, sc, wa, wm, ctr, out, extra);
    case 8: return launch_decode_g<KVT, 8>(G, grid, smem, st, q, pos, bt, max_pages, pool, nq, sc, wa, wm, ctr, out, extra);
    default: return BONSAI_CUDA_BAD_ARG;
  }
}

int attn_decode_mma_f16(const float* q, const int* positions, const int* block_table, int max_pages, int batch, int nq, int nkv,
                        int page_size, const void* kpool, const void* vpool, int nsplit, float* ws_acc, float* ws_ml, int* counters,
                        float* out, int extra_len, float sm_scale, cudaStream_t stream);
static int g_attn_force_cuda_cores = 0;

}  // namespace bonsai

extern "C" {

// 1: f16 caches with head_dim 128 use the CUDA-core kernel instead of the tensor-core one (comparisons, tests)
void bonsai_attn_decode_force_cuda_cores(int on) { bonsai::g_attn_force_cuda_cores = on; }

// qkv: f32 [batch][qkv_stride] holding q | k | v heads.  Writes normalised+rotated q to q_out
// [batch][nq][hd] and appends k, v at positions[b] through block_table [batch][max_pages].
int bonsai_qknorm_rope_kvstore(const float* qkv, int qkv_stride, const float* q_norm, const float* k_norm, float eps,
                               const float* rope_cos, const float* rope_sin, const int* positions, const int* block_table,
                               int max_pages, float* q_out, int batch, int nq, int nkv, int hd, int kvt, int page_size,
                               void* kpool, void* vpool, float* kscale, float* vscale, cudaStream_t stream) {
  using namespace bonsai;
  if (hd % 32 != 0 || hd < 64 || hd > 256 || kvt < 0 || kvt > 3 || batch <= 0) return BONSAI_CUDA_BAD_ARG;
  KvPool pool{(uint8_t*)kpool, (uint8_t*)vpool, kscale, vscale, page_size, nkv, hd, kvt};
  dim3 grid(nq + 2 * nkv, batch);
  qknorm_rope_kvstore_kernel<<<grid, hd, (hd + 32) * sizeof(float), stream>>>(qkv, qkv_stride, q_norm, k_norm, eps, rope_cos, rope_sin,
                                                                              positions, block_table, max_pages, q_out, nq, pool);
  return launch_status();
}

// q: f32 [batch][nq][hd] -> out f32 [batch][nq][hd].  Context length of sequence b is
// positions[b] + 1 + extra_len.  ws_acc needs batch*nq*nsplit*hd floats, ws_ml batch*nq*nsplit*2,
// counters batch*nkv ints that are zero between launches (the kernel resets them).
int bonsai_attn_decode(const float* q, const int* positions, const int* block_table, int max_pages, int batch, int nq, int nkv,
                       int hd, int kvt, int page_size, const void* kpool, const void* vpool, const float* kscale,
                       const float* vscale, int nsplit, float* ws_acc, float* ws_ml, int* counters, float* out, int extra_len,
                       cudaStream_t stream) {
  using namespace bonsai;
  if (hd % 32 != 0 || hd < 64 || hd > 256 || nq % nkv != 0 || nsplit < 1 || batch <= 0 || counters == nullptr) return BONSAI_CUDA_BAD_ARG;
  int G = nq / nkv, dpl = hd / 32;
  KvPool pool{(uint8_t*)kpool, (uint8_t*)vpool, (float*)kscale, (float*)vscale, page_size, nkv, hd, kvt};
  dim3 grid(nkv, nsplit, batch);
  size_t smem = (size_t)kAttnWarps * G * (hd + 2) * sizeof(float);
  if (smem > 48 * 1024) return BONSAI_CUDA_BAD_ARG;
  float sc = 1.0f / sqrtf((float)hd);
  if (hd == 128 && kvt == KV_F16 && !g_attn_force_cuda_cores) {
    // tensor-core path; it declines (BAD_ARG) shapes it does not cover and the CUDA-core kernels below take over
    const int rc = attn_decode_mma_f16(q, positions, block_table, max_pages, batch, nq, nkv, page_size, kpool, vpool, nsplit, ws_acc,
                                       ws_ml, counters, out, extra_len, sc, stream);
    if (rc != BONSAI_CUDA_BAD_ARG) return rc;
  }
  if (hd == 128 && kvt != KV_F32 && (G == 1 || G == 2 || G == 4) && (page_size & (page_size - 1)) == 0) {
    switch (kvt) {
      case KV_F16: return launch_decode_h128<KV_F16>(G, grid, smem, stream, q, positions, block_table, max_pages, pool, nq, sc, ws_acc, ws_ml, counters, out, extra_len);
      case KV_Q8: return launch_decode_h128<KV_Q8>(G, grid, smem, stream, q, positions, block_table, max_pages, pool, nq, sc, ws_acc, ws_ml, counters, out, extra_len);
      default: return launch_decode_h128<KV_Q4>(G, grid, smem, stream, q, positions, block_table, max_pages, pool, nq, sc, ws_acc, ws_ml, counters, out, extra_len);
    }
  }
  switch (kvt) {
    case KV_F32: return launch_decode_d<KV_F32>(dpl, G, grid, smem, stream, q, positions, block_table, max_pages, pool, nq, sc, ws_acc, ws_ml, counters, out, extra_len);
    case KV_F16: return launch_decode_d<KV_F16>(dpl, G, grid, smem, stream, q, positions, block_table, max_pages, pool, nq, sc, ws_acc, ws_ml, counters, out, extra_len);
    case KV_Q8: return launch_decode_d<KV_Q8>(dpl, G, grid, smem, stream, q, positions, block_table, max_pages, pool, nq, sc, ws_acc, ws_ml, counters, out, extra_len);
    case KV_Q4: return launch_decode_d<KV_Q4>(dpl, G, grid, smem, stream, q, positions, block_table, max_pages, pool, nq, sc, ws_acc, ws_ml, counters, out, extra_len);
    default: return BONSAI_CUDA_BAD_ARG;
  }
}

}  // extern "C"
