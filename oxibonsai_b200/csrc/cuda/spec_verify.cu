// Speculative-decoding verification on the device: the rejection test of every drafted token and the replacement sample,
// from the target's and the draft's logits, without bringing a distribution to the host.
//
// The reference's SpeculativeDecoder verifies with a mock draft probability and synthetic target logits on the host
// (crates/oxibonsai-runtime/src/speculative.rs:220-404).  Here, for k drafted tokens d_0..d_{k-1} and k+1 rows of target
// logits (row i = the target's distribution p_i for the position of d_i; row k = the position after the last draft) and
// k rows of draft logits (q_i, the distribution d_i was drawn from), both at temperature T:
//   accept d_i while u_i <= p_i(d_i) / q_i(d_i);
//   at the first rejection i emit a token drawn from normalise(max(0, p_i - q_i)) with the uniform v_i;
//   if all k are accepted emit a token drawn from p_k with v_k.
// The output stream is then distributed exactly as the target's own sampling at temperature T.
//
// Kernel 1, one CTA per row: softmax statistics of both rows, p_i(d_i), q_i(d_i), the residual mass and the replacement
// token by inverse CDF over the row in index order (row k: q = 0, so the residual is p_k itself).  Kernel 2, one thread:
// walks the rows in order and writes {accepted count, next token}.  Uniforms come from the caller (2 per row).
#include "common.cuh"

namespace bonsai {

constexpr int kSvThreads = 1024;

struct SvRow {
  float p_tok, q_tok;   // probabilities of the drafted token under target and draft
  int repl;             // replacement / bonus token of this row
  int pad;
};

__device__ __forceinline__ float block_max(float v, float* s32) {
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) s32[wid] = v;
  __syncthreads();
  float t = lane < nw ? s32[lane] : -INFINITY;
  return warp_max(t);
}

__global__ void __launch_bounds__(kSvThreads) spec_rows_kernel(const float* __restrict__ target, int t_ld, const float* __restrict__ draft,
                                                              int d_ld, const int* __restrict__ draft_tokens, int k, int vocab,
                                                              float inv_temp, const float* __restrict__ uniforms, SvRow* __restrict__ rows) {
  __shared__ float s32[32];
  __shared__ float chunk_sum[kSvThreads];
  __shared__ int pick_thread;
  const int i = blockIdx.x, tid = threadIdx.x;
  const float* p = target + (size_t)i * t_ld;
  const float* q = i < k ? draft + (size_t)i * d_ld : nullptr;
  // every thread owns one contiguous chunk of the row, so that the inverse CDF runs in index order
  const int per = (vocab + kSvThreads - 1) / kSvThreads;
  const int lo = min(vocab, tid * per), hi = min(vocab, lo + per);
  float pm = -INFINITY, qm = -INFINITY;
  for (int j = lo; j < hi; ++j) {
    pm = fmaxf(pm, p[j]);
    if (q) qm = fmaxf(qm, q[j]);
  }
  pm = block_max(pm, s32);
  qm = q ? block_max(qm, s32) : 0.0f;
  float ps = 0.0f, qs = 0.0f;
  for (int j = lo; j < hi; ++j) {
    ps += __expf((p[j] - pm) * inv_temp);
    if (q) qs += __expf((q[j] - qm) * inv_temp);
  }
  ps = block_sum(ps, s32);
  qs = q ? block_sum(qs, s32) : 1.0f;
  const float pinv = 1.0f / ps, qinv = q ? 1.0f / qs : 0.0f;
  // residual mass of the chunk, then of the row
  float r = 0.0f;
  for (int j = lo; j < hi; ++j) {
    const float pv = __expf((p[j] - pm) * inv_temp) * pinv;
    const float qv = q ? __expf((q[j] - qm) * inv_temp) * qinv : 0.0f;
    r += fmaxf(0.0f, pv - qv);
  }
  chunk_sum[tid] = r;
  if (tid == 0) pick_thread = -1;
  __syncthreads();
  if (tid == 0) {
    // serial prefix over 1024 partial sums: a few microseconds, and the same order as a cumulative sum over the row
    float total = 0.0f;
    for (int t = 0; t < kSvThreads; ++t) total += chunk_sum[t];
    const float want = uniforms[2 * i + 1] * total;
    float acc = 0.0f;
    int pick = -1;
    for (int t = 0; t < kSvThreads; ++t) {
      if (chunk_sum[t] > 0.0f) {
        if (acc + chunk_sum[t] >= want) { pick = t; break; }
        pick = t;              // the last chunk with mass takes what rounding leaves over
      }
      acc += chunk_sum[t];
    }
    pick_thread = pick;
    s32[0] = acc;              // mass before the picked chunk (unused when the walk ran off the end)
    s32[1] = want;
    s32[2] = total;
  }
  __syncthreads();
  if (tid == pick_thread) {
    float acc = 0.0f;
    for (int t = 0; t < tid; ++t) acc += chunk_sum[t];
    const float want = s32[1];
    int tok = -1;
    for (int j = lo; j < hi; ++j) {
      const float pv = __expf((p[j] - pm) * inv_temp) * pinv;
      const float qv = q ? __expf((q[j] - qm) * inv_temp) * qinv : 0.0f;
      const float d = fmaxf(0.0f, pv - qv);
      if (d > 0.0f) {
        tok = j;
        acc += d;
        if (acc >= want) break;
      }
    }
    rows[i].repl = tok;
  }
  if (tid == 0) {
    if (pick_thread < 0) {
      // p == q everywhere (no residual mass): a rejection cannot happen (the ratio is 1); keep the draft's own token
      rows[i].repl = i < k ? draft_tokens[i] : 0;
    }
    if (i < k) {
      const int d = draft_tokens[i];
      const bool ok = d >= 0 && d < vocab;
      rows[i].p_tok = ok ? __expf((p[d] - pm) * inv_temp) * pinv : 0.0f;
      rows[i].q_tok = ok ? __expf((q[d] - qm) * inv_temp) * qinv : 1.0f;
    } else {
      rows[i].p_tok = rows[i].q_tok = 1.0f;
    }
  }
}

__global__ void spec_decide_kernel(const SvRow* __restrict__ rows, int k, const float* __restrict__ uniforms, int* __restrict__ out) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  int n = 0;
  while (n < k) {
    const float ratio = rows[n].q_tok > 0.0f ? rows[n].p_tok / rows[n].q_tok : 1.0f;
    if (uniforms[2 * n] <= fminf(1.0f, ratio)) ++n;
    else break;
  }
  out[0] = n;
  out[1] = rows[n].repl;
}

}  // namespace bonsai

extern "C" {

// target: f32 [k+1][t_ld] logits, draft: f32 [k][d_ld] logits, draft_tokens int32 [k], uniforms f32 [2*(k+1)] in [0,1)
// (entry 2i: acceptance test of row i, 2i+1: replacement draw of row i), scratch: 16*(k+1) bytes, out int32 [2] =
// {number of accepted drafts, the token that follows them}.  temperature > 0.
int bonsai_spec_verify(const float* target, int t_ld, const float* draft, int d_ld, const int* draft_tokens, int k, int vocab,
                       float temperature, const float* uniforms, void* scratch, int* out, cudaStream_t stream) {
  using namespace bonsai;
  if (k < 0 || k > 64 || vocab < 1 || t_ld < vocab || (k > 0 && d_ld < vocab) || !(temperature > 0.0f)) return BONSAI_CUDA_BAD_ARG;
  if (target == nullptr || uniforms == nullptr || scratch == nullptr || out == nullptr || (k > 0 && (draft == nullptr || draft_tokens == nullptr)))
    return BONSAI_CUDA_BAD_ARG;
  static_assert(sizeof(SvRow) == 16, "scratch layout");
  spec_rows_kernel<<<k + 1, kSvThreads, 0, stream>>>(target, t_ld, draft, d_ld, draft_tokens, k, vocab, 1.0f / temperature, uniforms,
                                                     static_cast<SvRow*>(scratch));
  spec_decide_kernel<<<1, 32, 0, stream>>>(static_cast<const SvRow*>(scratch), k, uniforms, out);
  return launch_status();
}

}  // extern "C"
