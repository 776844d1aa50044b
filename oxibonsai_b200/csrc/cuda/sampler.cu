// Token sampler: one block per sequence picks the next token from a row of logits.
//
// Semantics follow the reference's host sampler (crates/oxibonsai-runtime/src/sampling.rs:73-189):
//   temperature < 1e-6 -> argmax, LAST index among ties (Rust `max_by`);
//   else logits / T -> keep the top-k (k > 0) -> softmax -> sort descending -> keep the prefix
//   whose cumulative probability first exceeds top_p (inclusive) -> renormalise -> draw
//   r = (xorshift64() / u64::MAX) as f32 and take the first token whose cumulative sum reaches r.
// The xorshift state (x ^= x<<13; x ^= x>>7; x ^= x<<17) lives in device memory, seeded with the
// raw seed, so the whole decode step stays on the device.  The reference's GPU path only has a
// single-block first-max argmax (cuda_kernels.rs:407-431) and downloads all logits otherwise.
//
// Two candidate strategies: with 1 <= k <= 1024 an exact radix select gathers the k largest logits
// (ties at the threshold taken in index order), which are then sorted in shared memory; with
// k = 0 (or k > 1024) the whole vocabulary is the candidate set, the top-p threshold is found by a
// radix select over probability mass and the draw walks tokens in index order (the same
// distribution as walking them in sorted order).
#include "common.cuh"

namespace bonsai {

constexpr int kSampThreads = 1024;

__device__ __forceinline__ uint32_t order_key(float v) {
  uint32_t b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ unsigned long long xorshift64(unsigned long long x) {
  x ^= x << 13;
  x ^= x >> 7;
  x ^= x << 17;
  return x;
}

// Exclusive scan over the block of one int per thread; returns the exclusive prefix, total in *total.
__device__ int block_excl_scan_int(int v, int* sh /* >= 33 ints */, int* total) {
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  int inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    int n = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += n;
  }
  __syncthreads();
  if (lane == 31) sh[wid] = inc;
  __syncthreads();
  if (wid == 0) {
    int w = sh[lane];
    int winc = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int n = __shfl_up_sync(0xffffffffu, winc, o);
      if (lane >= o) winc += n;
    }
    sh[lane] = winc - w;
    if (lane == 31) sh[32] = winc;
  }
  __syncthreads();
  *total = sh[32];
  return sh[wid] + inc - v;
}

__device__ float block_excl_scan_float(float v, float* sh /* >= 33 floats */, float* total) {
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  float inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    float n = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += n;
  }
  __syncthreads();
  if (lane == 31) sh[wid] = inc;
  __syncthreads();
  if (wid == 0) {
    float w = sh[lane];
    float winc = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      float n = __shfl_up_sync(0xffffffffu, winc, o);
      if (lane >= o) winc += n;
    }
    sh[lane] = winc - w;
    if (lane == 31) sh[32] = winc;
  }
  __syncthreads();
  *total = sh[32];
  return sh[wid] + inc - v;
}

__device__ float block_max_f(float v, float* sh) {
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) sh[wid] = v;
  __syncthreads();
  float t = sh[lane];
  t = warp_max(t);
  return t;
}

__device__ float block_sum_f(float v, float* sh) {
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) sh[wid] = v;
  __syncthreads();
  float t = sh[lane];
  t = warp_sum(t);
  return t;
}

// Greedy rows of small batches are scanned by kArgmaxBlocks CTAs each (a 152k-entry row is 608 KB: one CTA needs ~10
// dependent trips to L2 for it); the CTAs leave their candidates here and the last one to arrive picks the winner.
constexpr int kArgmaxBlocks = 32, kArgmaxRows = 64;
struct ArgmaxCand { float v; int i; };
__device__ ArgmaxCand g_argmax_cand[kArgmaxRows][kArgmaxBlocks];
__device__ int g_argmax_count[kArgmaxRows];   // zero between launches

// grid = (batch, 1 or kArgmaxBlocks), block = 1024
__global__ void __launch_bounds__(kSampThreads) sample_kernel(const float* __restrict__ logits, int vocab, int stride,
                                                             const float* __restrict__ temps, const int* __restrict__ topks,
                                                             const float* __restrict__ topps,
                                                             unsigned long long* __restrict__ rng, int* __restrict__ out_tokens,
                                                             int* __restrict__ positions, int advance,
                                                             const uint32_t* __restrict__ allow_mask, int mask_words) {
  __shared__ float s_val[kSampThreads];
  __shared__ int s_idx[kSampThreads];
  __shared__ float s_f[40];
  __shared__ int s_i[40];
  __shared__ int s_hist[256];
  __shared__ float s_fhist[256];
  __shared__ int s_pick;

  const int b = blockIdx.x, t = threadIdx.x;
  const int nby = gridDim.y, by = blockIdx.y;
  const float* lg = logits + (size_t)b * stride;
  const uint32_t* am = allow_mask ? allow_mask + (size_t)b * mask_words : nullptr;
  const float T = temps ? temps[b] : 0.0f;
  const int per = (vocab + kSampThreads - 1) / kSampThreads;
  const int i0 = t * per, i1 = min(vocab, i0 + per);
  auto allowed = [&](int i) -> bool { return am == nullptr || ((am[i >> 5] >> (i & 31)) & 1u); };

  int result = 0;
  if (by > 0 && !(T < 1e-6f)) return;      // only the greedy scan is split over several CTAs
  if (T < 1e-6f) {
    // ---- greedy: last maximal index ----
    // Threads stride through the row with 16-byte loads (a warp reads 512 contiguous bytes); a thread that walks its
    // own contiguous range instead touches 32 cache lines per warp load and the scan of a 152k-entry row took 39 us.
    // Candidates therefore do not arrive in index order: ties are resolved by index explicitly.
    float bv = -INFINITY;
    int bi = -1;
    auto consider = [&](float v, int i) {
      if (allowed(i) && !(v < bv) && (v != bv || i > bi)) { bv = v; bi = i; }
    };
    const int nv4 = ((stride & 3) == 0 && (reinterpret_cast<uintptr_t>(logits) & 15) == 0) ? vocab >> 2 : 0;
    const float4* lg4 = reinterpret_cast<const float4*>(lg);
    const int per4 = (nv4 + nby - 1) / nby, lo4 = by * per4, hi4 = min(nv4, lo4 + per4);
#pragma unroll 4
    for (int i4 = lo4 + t; i4 < hi4; i4 += kSampThreads) {
      const float4 v = lg4[i4];
      consider(v.x, 4 * i4);
      consider(v.y, 4 * i4 + 1);
      consider(v.z, 4 * i4 + 2);
      consider(v.w, 4 * i4 + 3);
    }
    if (by == nby - 1)
      for (int i = 4 * nv4 + t; i < vocab; i += kSampThreads) consider(lg[i], i);
    s_val[t] = bv;
    s_idx[t] = bi;
    __syncthreads();
    for (int o = kSampThreads / 2; o > 0; o >>= 1) {
      if (t < o) {
        float ov = s_val[t + o];
        int oi = s_idx[t + o];
        // equal values: the larger index wins (last maximal index overall)
        if (oi >= 0 && (s_idx[t] < 0 || ov > s_val[t] || (ov == s_val[t] && oi > s_idx[t]))) { s_val[t] = ov; s_idx[t] = oi; }
      }
      __syncthreads();
    }
    if (nby > 1) {
      // leave this CTA's candidate; the last CTA of the row to arrive reduces them (ties: the larger index)
      if (t == 0) {
        g_argmax_cand[b][by] = ArgmaxCand{s_val[0], s_idx[0]};
        __threadfence();
        const int prev = atomicAdd(&g_argmax_count[b], 1);
        s_pick = prev == nby - 1;
        if (s_pick) g_argmax_count[b] = 0;
      }
      __syncthreads();
      if (!s_pick) return;
      __threadfence();
      if (t < 32) {
        float v = -INFINITY;
        int i = -1;
        for (int c = t; c < nby; c += 32) {
          const float cv = __ldcg(&g_argmax_cand[b][c].v);
          const int ci = __ldcg(&g_argmax_cand[b][c].i);
          if (ci >= 0 && (i < 0 || cv > v || (cv == v && ci > i))) { v = cv; i = ci; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          const float ov = __shfl_xor_sync(0xffffffffu, v, o);
          const int oi = __shfl_xor_sync(0xffffffffu, i, o);
          if (oi >= 0 && (i < 0 || ov > v || (ov == v && oi > i))) { v = ov; i = oi; }
        }
        if (t == 0) s_idx[0] = i;
      }
      __syncthreads();
    }
    result = s_idx[0] < 0 ? 0 : s_idx[0];
  } else {
    const float invT = 1.0f / T;
    int k = topks ? topks[b] : 0;
    float top_p = topps ? topps[b] : 1.0f;
    unsigned long long st = xorshift64(rng[b]);
    float r = (float)((double)st / 18446744073709551615.0);
    float mx = -INFINITY;
    for (int i = i0; i < i1; ++i)
      if (allowed(i)) mx = fmaxf(mx, lg[i] * invT);
    mx = block_max_f(mx, s_f);

    if (k >= 1 && k <= kSampThreads && k < vocab) {
      // ---- radix select of the k largest keys ----
      uint32_t prefix = 0, mask = 0;
      int need = k;
      for (int pass = 3; pass >= 0; --pass) {
        int shift = pass * 8;
        if (t < 256) s_hist[t] = 0;
        __syncthreads();
        for (int i = i0; i < i1; ++i) {
          if (!allowed(i)) continue;
          uint32_t key = order_key(lg[i] * invT);
          if ((key & mask) == prefix) atomicAdd(&s_hist[(key >> shift) & 255u], 1);
        }
        __syncthreads();
        if (t == 0) {
          int cum = 0, bin = 255;
          for (; bin > 0; --bin) {
            if (cum + s_hist[bin] >= need) break;
            cum += s_hist[bin];
          }
          s_i[0] = bin;
          s_i[1] = need - cum;
        }
        __syncthreads();
        prefix |= (uint32_t)s_i[0] << shift;
        mask |= 255u << shift;
        need = s_i[1];
        __syncthreads();
      }
      // prefix is the k-th largest key; `need` of the elements equal to it are kept (index order)
      int ngt = 0, neq = 0;
      for (int i = i0; i < i1; ++i) {
        if (!allowed(i)) continue;
        uint32_t key = order_key(lg[i] * invT);
        ngt += key > prefix;
        neq += key == prefix;
      }
      int tot_gt, tot_eq;
      int off_gt = block_excl_scan_int(ngt, s_i, &tot_gt);
      int off_eq = block_excl_scan_int(neq, s_i, &tot_eq);
      int n_eq_keep = min(need, tot_eq);
      int ncand = tot_gt + n_eq_keep;
      s_val[t] = -INFINITY;
      s_idx[t] = 0x7fffffff;
      __syncthreads();
      for (int i = i0; i < i1; ++i) {
        if (!allowed(i)) continue;
        float v = lg[i] * invT;
        uint32_t key = order_key(v);
        if (key > prefix) {
          s_val[off_gt] = v;
          s_idx[off_gt] = i;
          ++off_gt;
        } else if (key == prefix) {
          if (off_eq < n_eq_keep) {
            s_val[tot_gt + off_eq] = v;
            s_idx[tot_gt + off_eq] = i;
          }
          ++off_eq;
        }
      }
      __syncthreads();
      // softmax over candidates
      float e = t < ncand ? expf(s_val[t] - mx) : 0.0f;
      float Z = block_sum_f(e, s_f);
      __syncthreads();
      s_val[t] = t < ncand ? e / Z : -1.0f;
      __syncthreads();
      // bitonic sort, descending by probability, ascending index on ties
      for (int size = 2; size <= kSampThreads; size <<= 1) {
        for (int strd = size >> 1; strd > 0; strd >>= 1) {
          int partner = t ^ strd;
          if (partner > t) {
            bool desc = (t & size) == 0;
            float a = s_val[t], c = s_val[partner];
            int ai = s_idx[t], ci = s_idx[partner];
            bool a_first = (a > c) || (a == c && ai < ci);
            if (desc != a_first) {
              s_val[t] = c; s_val[partner] = a;
              s_idx[t] = ci; s_idx[partner] = ai;
            }
          }
          __syncthreads();
        }
      }
      float p = t < ncand ? s_val[t] : 0.0f;
      float tot;
      float excl = block_excl_scan_float(p, s_f, &tot);
      float inc = excl + p;
      // top-p cutoff: first position whose inclusive cumulative sum exceeds top_p
      if (t == 0) s_pick = ncand - 1;
      __syncthreads();
      if (top_p < 1.0f && t < ncand && inc > top_p && !(excl > top_p)) atomicMin(&s_pick, t);
      __syncthreads();
      int cutoff = s_pick;
      __syncthreads();
      float keep = t <= cutoff ? p : 0.0f;
      float ksum;
      float kexcl = block_excl_scan_float(keep, s_f, &ksum);
      float kinc = (kexcl + keep) / ksum;
      if (t == 0) s_pick = 0x7fffffff;
      __syncthreads();
      if (t <= cutoff && r <= kinc) atomicMin(&s_pick, t);
      __syncthreads();
      int pick = s_pick == 0x7fffffff ? 0 : s_pick;
      result = s_idx[pick];
      if (t == 0) rng[b] = st;
    } else {
      // ---- whole vocabulary: threshold by probability mass, then walk in index order ----
      float zs = 0.0f;
      for (int i = i0; i < i1; ++i)
        if (allowed(i)) zs += expf(lg[i] * invT - mx);
      float Z = block_sum_f(zs, s_f);
      uint32_t prefix = 0, mask = 0;
      float target = top_p * Z, above = 0.0f;
      bool use_p = top_p < 1.0f;
      if (use_p) {
        for (int pass = 3; pass >= 0; --pass) {
          int shift = pass * 8;
          if (t < 256) { s_fhist[t] = 0.0f; s_hist[t] = 0; }
          __syncthreads();
          for (int i = i0; i < i1; ++i) {
            if (!allowed(i)) continue;
            float v = lg[i] * invT;
            uint32_t key = order_key(v);
            if ((key & mask) == prefix) {
              atomicAdd(&s_fhist[(key >> shift) & 255u], expf(v - mx));
              atomicAdd(&s_hist[(key >> shift) & 255u], 1);
            }
          }
          __syncthreads();
          if (t == 0) {
            float cum = above;
            int bin = 255;
            for (; bin > 0; --bin) {
              if (s_hist[bin] > 0 && cum + s_fhist[bin] > target) break;
              cum += s_fhist[bin];
            }
            s_i[0] = bin;
            s_f[34] = cum;
          }
          __syncthreads();
          prefix |= (uint32_t)s_i[0] << shift;
          mask |= 255u << shift;
          above = s_f[34];
          __syncthreads();
        }
      }
      // elements with key > prefix are kept; of those equal to prefix keep the first n_eq (index order)
      float e_thr = 0.0f;
      int n_eq_keep = 0x7fffffff;
      if (use_p) {
        // value of the threshold key
        uint32_t kb = (prefix & 0x80000000u) ? (prefix & 0x7fffffffu) : ~prefix;
        e_thr = expf(__uint_as_float(kb) - mx);
        n_eq_keep = e_thr > 0.0f ? (int)floorf(fmaxf(target - above, 0.0f) / e_thr) + 1 : 0x7fffffff;
      }
      float ksum = 0.0f;
      int neq = 0;
      for (int i = i0; i < i1; ++i) {
        if (!allowed(i)) continue;
        float v = lg[i] * invT;
        uint32_t key = order_key(v);
        if (!use_p || key > prefix) ksum += expf(v - mx);
        else if (key == prefix) ++neq;
      }
      int tot_eq;
      int off_eq = block_excl_scan_int(neq, s_i, &tot_eq);
      int my_eq = max(0, min(neq, n_eq_keep - off_eq));
      ksum += (float)my_eq * e_thr;
      float total;
      float excl = block_excl_scan_float(ksum, s_f, &total);
      float goal = r * total;
      if (t == 0) s_pick = 0x7fffffff;
      __syncthreads();
      // the first thread whose inclusive mass reaches the goal owns the draw
      bool mine = (ksum > 0.0f) && (goal <= excl + ksum) && !(goal <= excl && excl > 0.0f);
      if (mine) atomicMin(&s_pick, t);
      __syncthreads();
      if (s_pick == t) {
        float cum = excl;
        int eqc = off_eq, last = -1, chosen = -1;
        for (int i = i0; i < i1 && chosen < 0; ++i) {
          if (!allowed(i)) continue;
          float v = lg[i] * invT;
          uint32_t key = order_key(v);
          bool kept = !use_p || key > prefix || (key == prefix && eqc++ < n_eq_keep);
          if (!kept) continue;
          cum += expf(v - mx);
          last = i;
          if (goal <= cum) chosen = i;
        }
        s_idx[0] = chosen >= 0 ? chosen : (last >= 0 ? last : 0);
      }
      __syncthreads();
      if (s_pick == 0x7fffffff) {
        // numerical corner: fall back to the most likely token
        float bv = -INFINITY;
        int bi = 0;
        for (int i = i0; i < i1; ++i)
          if (allowed(i) && lg[i] > bv) { bv = lg[i]; bi = i; }
        s_val[t] = bv;
        s_idx[t] = bi;
        __syncthreads();
        for (int o = kSampThreads / 2; o > 0; o >>= 1) {
          if (t < o && s_val[t + o] > s_val[t]) { s_val[t] = s_val[t + o]; s_idx[t] = s_idx[t + o]; }
          __syncthreads();
        }
      }
      result = s_idx[0];
      if (t == 0) rng[b] = st;
    }
  }
  if (t == 0) {
    out_tokens[b] = result;
    if (advance) positions[b] += 1;
  }
}

}  // namespace bonsai

extern "C" {

// logits f32 [batch][stride]; temps / topks / topps per sequence (null temps = greedy for all);
// rng: one xorshift64 state per sequence; out_tokens int32 [batch]; positions[b] += 1 when
// advance != 0; allow_mask (optional) has mask_words uint32 per sequence, bit i set = token i allowed.
int bonsai_sample(const float* logits, int batch, int vocab, int stride, const float* temps, const int* topks,
                  const float* topps, unsigned long long* rng, int* out_tokens, int* positions, int advance,
                  const uint32_t* allow_mask, int mask_words, cudaStream_t stream) {
  if (batch <= 0 || vocab <= 0 || stride < vocab) return BONSAI_CUDA_BAD_ARG;
  if (temps != nullptr && rng == nullptr) return BONSAI_CUDA_BAD_ARG;
  // a few rows: split every greedy row's scan over kArgmaxBlocks CTAs (their meeting place is a fixed-size device array)
  const int nby = (batch <= 4 && batch <= bonsai::kArgmaxRows && vocab >= 32768) ? bonsai::kArgmaxBlocks : 1;
  bonsai::sample_kernel<<<dim3(batch, nby), bonsai::kSampThreads, 0, stream>>>(logits, vocab, stride, temps, topks, topps, rng, out_tokens,
                                                                    positions, advance, allow_mask, mask_words);
  return bonsai::launch_status();
}

}  // extern "C"
