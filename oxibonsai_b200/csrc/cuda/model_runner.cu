// Native decode-step runner: enqueues every kernel of one Qwen3 decoder step on a stream.
//
// The host loop of the reference builds per-layer parameter structs and issues 14 launches per
// layer plus host round trips for the hidden state, the RoPE row and the logits on every token
// (crates/oxibonsai-kernels/src/gpu_backend/cuda_full_layer/encode_ternary.rs:395-826).  Here a step
// is: embed (token id read on the device) -> per layer { norm+QKV GEMV, QK-norm+RoPE+KV append,
// split-KV attention, O-proj+residual, norm+gate/up+SwiGLU, down+residual } -> norm+LM head ->
// sampler (writes the next token id and advances the position on the device).  Nothing crosses
// the PCIe bus inside a step, so the whole step can be captured in one CUDA graph and replayed;
// positions, block tables and sampler state are device buffers the graph reads.
//
// Tensor parallelism: q/k/v and gate/up are column-parallel (local heads / local intermediate
// rows), attn-output and down are row-parallel (local K slice).  With tp_size > 1 the row-parallel
// GEMVs write partial sums and the fused all-reduce+residual kernel of csrc/comm combines them.
#include <vector>

#include "common.cuh"

extern "C" {
int bonsai_bitgemv(const void*, const void*, const float*, const float*, float, float*, const float*, int, int, int, cudaStream_t);
int bonsai_f16gemv(const void*, const float*, const float*, float, float*, int, int, cudaStream_t);
int bonsai_embed_f16(const void*, const int*, float*, int, int, cudaStream_t);
int bonsai_qknorm_rope_kvstore(const float*, int, const float*, const float*, float, const float*, const float*, const int*,
                               const int*, int, float*, int, int, int, int, int, int, void*, void*, float*, float*, cudaStream_t);
int bonsai_attn_decode(const float*, const int*, const int*, int, int, int, int, int, int, int, const void*, const void*,
                       const float*, const float*, int, float*, float*, int*, float*, int, cudaStream_t);
int bonsai_bitgemv_h2(const void*, const void*, const float*, const float*, float, float*, const float*, int, int, int, cudaStream_t);
int bonsai_bitgemv_warp(const void*, const void*, const float*, const float*, float, float*, const float*, int, int, int, cudaStream_t);
int bonsai_bitgemv_hmma(const void*, const void*, const float*, const float*, float, float*, const float*, int, int, int, cudaStream_t);
int bonsai_bitgemv_fast(const void*, const void*, const float*, const float*, float, float*, const float*, int, int, int, cudaStream_t);
int bonsai_sample(const float*, int, int, int, const float*, const int*, const float*, unsigned long long*, int*, int*, int,
                  const uint32_t*, int, cudaStream_t);
int bonsai_bitgemv_tp(const void*, const void*, const void*, const float*, float, float*, const float*, int, int, int, cudaStream_t);
int bonsai_tp_allgather_logits(void*, const float*, int, int, int, int, cudaStream_t);
int bonsai_tp_allreduce_big_add(void*, float*, size_t, cudaStream_t);
void* bonsai_tp_big_ptr(void*);
int bonsai_tp_allgather_logits_at(void*, const float*, int, int, int, int, int, cudaStream_t);
int bonsai_tp_allreduce_oneshot_add(void*, float*, size_t, int, cudaStream_t);
void* bonsai_tp_big_half_ptr(void*, int);
int bonsai_tp_barrier(void*, cudaStream_t);
int bonsai_bitgemm_prefill_ws(const void*, const void*, const void*, int, float*, const float*, void*, int*, int, int, int, int, int,
                              int, const void*, void*, size_t, int, cudaStream_t);
int bonsai_norm_to_f16_paired(const float*, int, const float*, float, int, int, void*, int, int, cudaStream_t);
int bonsai_attn_decode_qkv_f16(const float*, int, const float*, const float*, float, const float*, const float*, const int*, const int*,
                               int, int, int, int, int, int, void*, void*, int, float*, float*, int*, float*, cudaStream_t);
int bonsai_norm_to_f16_hmma(const float*, int, const float*, float, int, int, void*, int, cudaStream_t);
int bonsai_bitgemm_hmma(const void*, const void*, const void*, int, float*, const float*, void*, int, int, int, int, int, cudaStream_t);
int bonsai_bitgemm_hmma_tp(const void*, const void*, const void*, const void*, int, float*, const float*, int, int, int, int, cudaStream_t);
int bonsai_attn_prefill_order(const float*, int, int, const int*, int, int, int, int, int, const void*, const void*, const float*,
                              const float*, void*, int, int, cudaStream_t);
int bonsai_embed_rows_f16(const void*, const int*, float*, int, int, int, cudaStream_t);
int bonsai_bitgemv_s16_pf(const void*, const float*, const float*, float, float*, const float*, int, int, int, const void*, int*, const void*,
                          size_t, cudaStream_t);
size_t bonsai_s16_bytes(int, int);
}

namespace bonsai {

enum LayerPtr {
  LP_QKV_CODES = 0, LP_QKV_SCALES, LP_O_CODES, LP_O_SCALES, LP_GU_CODES, LP_GU_SCALES, LP_DOWN_CODES, LP_DOWN_SCALES,
  LP_ATTN_NORM, LP_FFN_NORM, LP_Q_NORM, LP_K_NORM, LP_KPOOL, LP_VPOOL, LP_KSCALE, LP_VSCALE,
  LP_QKV_S16, LP_O_S16, LP_GU_S16, LP_DOWN_S16,   // the same four matrices in the streamed decode layout (0 = not built)
  LP_COUNT
};
enum GlobalPtr {
  GP_EMBD = 0, GP_LM_HEAD, GP_OUT_NORM, GP_ROPE_COS, GP_ROPE_SIN, GP_COUNT
};
enum IntCfg {
  IC_HIDDEN = 0, IC_INTER_LOCAL, IC_LAYERS, IC_HEADS_LOCAL, IC_KV_HEADS_LOCAL, IC_HEAD_DIM, IC_VOCAB, IC_LM_ROWS_LOCAL,
  IC_KVT, IC_PAGE_SIZE, IC_MAX_PAGES, IC_NSPLIT, IC_TP_SIZE, IC_TP_RANK, IC_FAST, IC_NSPLIT_BATCHED, IC_COUNT
};
enum StepPtr {
  SP_TOKENS = 0, SP_POSITIONS, SP_BLOCK_TABLE, SP_H, SP_QKV, SP_Q, SP_ATTN, SP_ACT, SP_LOGITS, SP_WS_ACC, SP_WS_ML,
  SP_TEMPS, SP_TOPKS, SP_TOPPS, SP_RNG, SP_OUT_TOKENS, SP_PARTIAL, SP_ALLOW_MASK, SP_ATTN_COUNTERS,
  SP_STATUS,   // device int: non-zero after a bounded wait inside a kernel of the step expired
  SP_COUNT
};

// K / V pools of one layer in one page format.
struct KvPoolPtrs { uint64_t k = 0, v = 0, ks = 0, vs = 0; };

struct Runner {
  // Page formats beside the default one (ic[IC_KVT]): pools[kvt][layer], empty when that format has no pool.  slot_fmt[s] is
  // the page format of the sequence in slot s (slots beyond its size use the default): a KV-pressure policy admits new
  // sequences in a denser format while the old ones keep theirs, so one decode batch can mix formats.
  std::vector<KvPoolPtrs> pools[4];
  std::vector<int> slot_fmt;
  int ic[IC_COUNT];
  float eps;
  uint64_t gp[GP_COUNT];
  std::vector<uint64_t> lp;  // [layers][LP_COUNT]
  void* comm = nullptr;      // tensor-parallel communicator (csrc/comm), null when tp_size == 1
  void* gemm_ws = nullptr;   // set from the prefill pointer table at every call
  size_t gemm_ws_bytes = 0;
};

template <typename T>
static inline T* P(uint64_t v) { return reinterpret_cast<T*>(v); }

#define RC(expr) do { int _rc = (expr); if (_rc != 0) return _rc; } while (0)

static inline int slot_format(const Runner& r, int slot) {
  return slot < (int)r.slot_fmt.size() ? r.slot_fmt[slot] : r.ic[IC_KVT];
}
static inline KvPoolPtrs layer_pool(const Runner& r, const uint64_t* lp, int layer, int kvt) {
  if (kvt != r.ic[IC_KVT] && !r.pools[kvt].empty()) return r.pools[kvt][layer];
  KvPoolPtrs p;
  p.k = lp[LP_KPOOL]; p.v = lp[LP_VPOOL]; p.ks = lp[LP_KSCALE]; p.vs = lp[LP_VSCALE];
  return p;
}

// QK-norm + RoPE + KV append + decode attention of one new token per sequence: one fused launch for f16 pages with
// head_dim 128 on the packed-half path, otherwise (other page formats, exact mode, shapes the fused kernel declines)
// the two separate kernels.  Slots b0 .. b0+n-1 of the step buffers, all in page format kvt.
static int qkv_attention_run(Runner& r, const uint64_t* lp, const uint64_t* sp, const KvPoolPtrs& pool, int kvt, const float* qkv, int qkv_n,
                             float* q, float* attn, const int* positions, const int* bt, int b0, int n, int nsplit, cudaStream_t st) {
  const int nq = r.ic[IC_HEADS_LOCAL], nkv = r.ic[IC_KV_HEADS_LOCAL], hd = r.ic[IC_HEAD_DIM], mp = r.ic[IC_MAX_PAGES];
  qkv += (size_t)b0 * qkv_n;
  q += (size_t)b0 * nq * hd;
  attn += (size_t)b0 * nq * hd;
  positions += b0;
  bt += (size_t)b0 * mp;
  float* ws_acc = P<float>(sp[SP_WS_ACC]) + (size_t)b0 * nq * nsplit * hd;
  float* ws_ml = P<float>(sp[SP_WS_ML]) + (size_t)b0 * nq * nsplit * 2;
  int* counters = P<int>(sp[SP_ATTN_COUNTERS]) + (size_t)b0 * nkv;
  if (kvt == 1 && hd == 128 && r.ic[IC_FAST] != 0) {
    const int rc = bonsai_attn_decode_qkv_f16(qkv, qkv_n, P<float>(lp[LP_Q_NORM]), P<float>(lp[LP_K_NORM]), r.eps, P<float>(r.gp[GP_ROPE_COS]),
                                              P<float>(r.gp[GP_ROPE_SIN]), positions, bt, mp, n, nq, nkv, hd, r.ic[IC_PAGE_SIZE],
                                              P<void>(pool.k), P<void>(pool.v), nsplit, ws_acc, ws_ml, counters, attn, st);
    if (rc != BONSAI_CUDA_BAD_ARG) return rc;   // bad argument = not a shape of the fused kernel
  }
  RC(bonsai_qknorm_rope_kvstore(qkv, qkv_n, P<float>(lp[LP_Q_NORM]), P<float>(lp[LP_K_NORM]), r.eps, P<float>(r.gp[GP_ROPE_COS]),
                                P<float>(r.gp[GP_ROPE_SIN]), positions, bt, mp, q, n, nq, nkv, hd, kvt, r.ic[IC_PAGE_SIZE], P<void>(pool.k),
                                P<void>(pool.v), P<float>(pool.ks), P<float>(pool.vs), st));
  return bonsai_attn_decode(q, positions, bt, mp, n, nq, nkv, hd, kvt, r.ic[IC_PAGE_SIZE], P<void>(pool.k), P<void>(pool.v),
                            P<float>(pool.ks), P<float>(pool.vs), nsplit, ws_acc, ws_ml, counters, attn, 0, st);
}

// The same for slots 0 .. batch-1: one launch (pair) per run of consecutive slots that share a page format.
static int qkv_attention(Runner& r, int layer, const uint64_t* lp, const uint64_t* sp, const float* qkv, int qkv_n, float* q, float* attn,
                         const int* positions, const int* bt, int batch, int nsplit, cudaStream_t st) {
  int b0 = 0;
  while (b0 < batch) {
    const int kvt = slot_format(r, b0);
    int b1 = b0 + 1;
    while (b1 < batch && slot_format(r, b1) == kvt) ++b1;
    RC(qkv_attention_run(r, lp, sp, layer_pool(r, lp, layer, kvt), kvt, qkv, qkv_n, q, attn, positions, bt, b0, b1 - b0, nsplit, st));
    b0 = b1;
  }
  return 0;
}

// flags: bit 0 = run the sampler and advance positions, bit 1 = skip the LM head
static int decode_step(Runner& r, const uint64_t* sp, int batch, int flags, int mask_words, cudaStream_t st) {
  const int hidden = r.ic[IC_HIDDEN], inter = r.ic[IC_INTER_LOCAL], nq = r.ic[IC_HEADS_LOCAL], nkv = r.ic[IC_KV_HEADS_LOCAL];
  const int hd = r.ic[IC_HEAD_DIM], vocab = r.ic[IC_VOCAB], lm_rows = r.ic[IC_LM_ROWS_LOCAL];
  const int qd = nq * hd, kvd = nkv * hd, qkv_n = qd + 2 * kvd;
  const bool tp = r.ic[IC_TP_SIZE] > 1;
  // IC_FAST: 0 exact f32, 1 packed-half (warp-per-row or tensor-core kernel by shape), 2 packed-half tile kernel,
  // 3 warp-level tensor cores for every shape, 4 warp-per-row for every shape
  auto gemv = r.ic[IC_FAST] == 0 ? bonsai_bitgemv
              : (r.ic[IC_FAST] == 2 ? bonsai_bitgemv_h2
                 : (r.ic[IC_FAST] == 3 ? bonsai_bitgemv_hmma : (r.ic[IC_FAST] == 4 ? bonsai_bitgemv_warp : bonsai_bitgemv_fast)));
  int* tokens = P<int>(sp[SP_TOKENS]);
  int* positions = P<int>(sp[SP_POSITIONS]);
  const int* bt = P<int>(sp[SP_BLOCK_TABLE]);
  float* h = P<float>(sp[SP_H]);
  float* qkv = P<float>(sp[SP_QKV]);
  float* q = P<float>(sp[SP_Q]);
  float* attn = P<float>(sp[SP_ATTN]);
  float* act = P<float>(sp[SP_ACT]);
  float* logits = P<float>(sp[SP_LOGITS]);
  float* partial = P<float>(sp[SP_PARTIAL]);

  // One linear layer of one sequence.  The packed-half mode streams the matrix in its S16 form through the tensor-core
  // GEMV (bitgemv_stream.cu) when that form was built and the shape fits; epi 3 = row-parallel sum over the
  // tensor-parallel group + residual inside the same kernel.
  int* status = P<int>(sp[SP_STATUS]);
  // (next, next_n, next_k): the S16 matrix of the GEMV that follows in the stream, which this one requests into L2.
  auto linear = [&](const uint64_t* lp, int w_codes, int w_s16, const float* x, const float* norm_w, float* out, const float* residual,
                    int n, int k, int epi, uint64_t next, int next_n, int next_k) -> int {
    if (r.ic[IC_FAST] == 1 && lp[w_s16] != 0) {
      const int rc = bonsai_bitgemv_s16_pf(P<void>(lp[w_s16]), x, norm_w, r.eps, out, residual, n, k, epi, r.comm, status, P<void>(next),
                                           next != 0 ? bonsai_s16_bytes(next_n, next_k) : 0, st);
      if (rc != BONSAI_CUDA_BAD_ARG) return rc;   // bad argument = a shape the streamed kernel declines
    }
    if (epi == 3)
      return bonsai_bitgemv_tp(r.comm, P<void>(lp[w_codes]), P<void>(lp[w_codes + 1]), x, r.eps, out, residual, n, k, r.ic[IC_FAST], st);
    return gemv(P<void>(lp[w_codes]), P<void>(lp[w_codes + 1]), x, norm_w, r.eps, out, residual, n, k, epi, st);
  };

  for (int b = 0; b < batch; ++b)
    RC(bonsai_embed_f16(P<void>(r.gp[GP_EMBD]), tokens + b, h + (size_t)b * hidden, hidden, vocab, st));
  for (int l = 0; l < r.ic[IC_LAYERS]; ++l) {
    const uint64_t* lp = &r.lp[(size_t)l * LP_COUNT];
    const uint64_t next_qkv = l + 1 < r.ic[IC_LAYERS] ? r.lp[(size_t)(l + 1) * LP_COUNT + LP_QKV_S16] : 0;
    for (int b = 0; b < batch; ++b)
      RC(linear(lp, LP_QKV_CODES, LP_QKV_S16, h + (size_t)b * hidden, P<float>(lp[LP_ATTN_NORM]), qkv + (size_t)b * qkv_n, nullptr,
                qkv_n, hidden, 0, lp[LP_O_S16], hidden, qd));
    RC(qkv_attention(r, l, lp, sp, qkv, qkv_n, q, attn, positions, bt, batch, r.ic[IC_NSPLIT], st));
    for (int b = 0; b < batch; ++b)
      RC(linear(lp, LP_O_CODES, LP_O_S16, attn + (size_t)b * qd, nullptr, h + (size_t)b * hidden, h + (size_t)b * hidden, hidden, qd,
                tp ? 3 : 1, lp[LP_GU_S16], 2 * inter, hidden));
    for (int b = 0; b < batch; ++b)
      RC(linear(lp, LP_GU_CODES, LP_GU_S16, h + (size_t)b * hidden, P<float>(lp[LP_FFN_NORM]), act + (size_t)b * inter, nullptr,
                2 * inter, hidden, 2, lp[LP_DOWN_S16], hidden, inter));
    for (int b = 0; b < batch; ++b)
      RC(linear(lp, LP_DOWN_CODES, LP_DOWN_S16, act + (size_t)b * inter, nullptr, h + (size_t)b * hidden, h + (size_t)b * hidden, hidden,
                inter, tp ? 3 : 1, next_qkv, qkv_n, hidden));
  }
  if (!(flags & 2)) {
    if (!tp) {
      for (int b = 0; b < batch; ++b)
        RC(bonsai_f16gemv(P<void>(r.gp[GP_LM_HEAD]), h + (size_t)b * hidden, P<float>(r.gp[GP_OUT_NORM]), r.eps,
                          logits + (size_t)b * vocab, lm_rows, hidden, st));
    } else {
      // vocab-parallel head: local slice, then every rank pushes its slice into all logits areas
      // (`logits` is this rank's area of the symmetric buffer)
      const int rows_per_rank = (vocab + r.ic[IC_TP_SIZE] - 1) / r.ic[IC_TP_SIZE];
      for (int b = 0; b < batch; ++b)
        if (lm_rows > 0)
          RC(bonsai_f16gemv(P<void>(r.gp[GP_LM_HEAD]), h + (size_t)b * hidden, P<float>(r.gp[GP_OUT_NORM]), r.eps,
                            partial + (size_t)b * lm_rows, lm_rows, hidden, st));
      RC(bonsai_tp_allgather_logits(r.comm, partial, batch, lm_rows, r.ic[IC_TP_RANK] * rows_per_rank, vocab, st));
    }
  }
  if (flags & 1) {
    RC(bonsai_sample(logits, batch, vocab, vocab, P<float>(sp[SP_TEMPS]), P<int>(sp[SP_TOPKS]), P<float>(sp[SP_TOPPS]),
                     P<unsigned long long>(sp[SP_RNG]), P<int>(sp[SP_OUT_TOKENS]), positions, 1,
                     mask_words > 0 ? P<uint32_t>(sp[SP_ALLOW_MASK]) : nullptr, mask_words, st));
  }
  return 0;
}

enum PrefillPtr {
  PP_TOKENS = 0, PP_POSITIONS, PP_H, PP_XN, PP_QKV, PP_Q, PP_ATTN, PP_ACT, PP_STATUS,
  PP_SM_ATTN, PP_SM_ACC, PP_SM_ML, PP_SM_CTR,   // small chunks: f32 attention output and split-KV workspace for kSmallChunk rows
  PP_GEMM_WS, PP_GEMM_WS_BYTES,   // workspace of the GEMM's balanced work distribution (pointer, size as a plain integer)
  PP_COUNT
};

// Chunks of at most this many tokens run like a decode batch (mma.sync GEMMs, split-KV attention); the small-chunk
// workspace holds kSmallChunk rows of kSmallSplits splits.
constexpr int kSmallChunk = 32, kSmallSplits = 16;

static inline int pf_gemm(Runner& r, const void* codes, const void* scales, const void* x, int x_ld, float* out_f32, const float* residual,
                          void* out_f16, int* status, int n_rows, int K, int T, int epi, int out_ld, int sms, const void* dense_w,
                          cudaStream_t st) {
  return bonsai_bitgemm_prefill_ws(codes, scales, x, x_ld, out_f32, residual, out_f16, status, n_rows, K, T, epi, out_ld, sms, dense_w,
                                   r.gemm_ws, r.gemm_ws_bytes, 1, st);
}

// One chunk of T prompt tokens of the sequence in `slot`, starting at position pos0: batched
// embed -> per layer { norm -> QKV GEMM -> QK-norm+RoPE+KV append -> causal attention over the
// paged cache -> O GEMM + residual -> norm -> gate/up GEMM + SwiGLU -> down GEMM + residual }.
// With want_logits the last token's hidden state goes through the final norm and LM head into
// the slot's logits row.
static int prefill_chunk(Runner& r, const uint64_t* sp, const uint64_t* pp, int T, int pos0, int slot, int want_logits,
                         cudaStream_t st) {
  const int hidden = r.ic[IC_HIDDEN], inter = r.ic[IC_INTER_LOCAL], nq = r.ic[IC_HEADS_LOCAL], nkv = r.ic[IC_KV_HEADS_LOCAL];
  const int hd = r.ic[IC_HEAD_DIM], vocab = r.ic[IC_VOCAB], lm_rows = r.ic[IC_LM_ROWS_LOCAL];
  const int qd = nq * hd, kvd = nkv * hd, qkv_n = qd + 2 * kvd;
  const bool tp = r.ic[IC_TP_SIZE] > 1;
  float* big = tp ? static_cast<float*>(bonsai_tp_big_ptr(r.comm)) : nullptr;
  const int sms = 148;
  const int* tokens = P<int>(pp[PP_TOKENS]);
  const int* positions = P<int>(pp[PP_POSITIONS]);
  float* h = P<float>(pp[PP_H]);
  void* xn = P<void>(pp[PP_XN]);
  float* qkv = P<float>(pp[PP_QKV]);
  float* q = P<float>(pp[PP_Q]);
  void* attn = P<void>(pp[PP_ATTN]);
  void* act = P<void>(pp[PP_ACT]);
  int* status = P<int>(pp[PP_STATUS]);
  r.gemm_ws = P<void>(pp[PP_GEMM_WS]);
  r.gemm_ws_bytes = (size_t)pp[PP_GEMM_WS_BYTES];
  const int xn_ld = hidden > qd ? hidden : qd;
  const int* bt = P<int>(sp[SP_BLOCK_TABLE]) + (size_t)slot * r.ic[IC_MAX_PAGES];

  // Chunks of up to 32 tokens (speculative verification, short prompts) run like a decode batch: the packed GEMMs on
  // mma.sync with register-expanded weights (activations in hmma-K order) and, once the chunk's K/V rows are appended,
  // the split-KV decode attention with one "sequence" per token (all share the page list; token i sees positions
  // <= pos0 + i), which spreads a long context over the GPU where the prompt kernel would run one CTA per head.
  // Larger chunks use the tcgen05 GEMM (paired-K order) and the prompt attention kernel.
  const bool hm = r.ic[IC_FAST] != 5 && T <= kSmallChunk && hidden % 128 == 0 && qd % 128 == 0 && inter % 128 == 0;
  // Tensor parallel, up to 16 tokens (a speculative verification pass): the row-parallel GEMMs exchange their partial sums
  // in the epilogue, as in the batched decode step, instead of GEMM + two-shot all-reduce (three more launches and two flag
  // barriers per exchange).
  const bool tp_fused = tp && hm && T <= 16;
  int sm_splits = (4 * 148) / (nkv * T);
  if (sm_splits < 1) sm_splits = 1;
  if (sm_splits > kSmallSplits) sm_splits = kSmallSplits;
  while (sm_splits & (sm_splits - 1)) sm_splits &= sm_splits - 1;   // a power of two: 2 to 16 splits can run as one cluster
  auto to_f16 = [&](const float* w) {
    return hm ? bonsai_norm_to_f16_hmma(h, hidden, w, r.eps, T, hidden, xn, xn_ld, st)
              : bonsai_norm_to_f16_paired(h, hidden, w, r.eps, T, hidden, xn, xn_ld, 0, st);
  };
  auto gemm = [&](const void* codes, const void* scales, const void* x, int x_ld, float* out_f32, const float* residual, void* out_f16,
                  int n_rows, int K, int epi, int out_ld) {
    return hm ? bonsai_bitgemm_hmma(codes, scales, x, x_ld, out_f32, residual, out_f16, n_rows, K, T, epi, out_ld, st)
              : pf_gemm(r, codes, scales, x, x_ld, out_f32, residual, out_f16, status, n_rows, K, T, epi, out_ld, sms, nullptr, st);
  };

  const int kvt = slot_format(r, slot);                   // page format of this sequence
  RC(bonsai_embed_rows_f16(P<void>(r.gp[GP_EMBD]), tokens, h, T, hidden, vocab, st));
  for (int l = 0; l < r.ic[IC_LAYERS]; ++l) {
    const uint64_t* lp = &r.lp[(size_t)l * LP_COUNT];
    const KvPoolPtrs pool = layer_pool(r, lp, l, kvt);
    RC(to_f16(P<float>(lp[LP_ATTN_NORM])));
    RC(gemm(P<void>(lp[LP_QKV_CODES]), P<void>(lp[LP_QKV_SCALES]), xn, xn_ld, qkv, nullptr, nullptr, qkv_n, hidden, 0, qkv_n));
    // every row of the chunk uses the same page list: a block-table stride of zero
    RC(bonsai_qknorm_rope_kvstore(qkv, qkv_n, P<float>(lp[LP_Q_NORM]), P<float>(lp[LP_K_NORM]), r.eps, P<float>(r.gp[GP_ROPE_COS]),
                                  P<float>(r.gp[GP_ROPE_SIN]), positions, bt, 0, q, T, nq, nkv, hd, kvt,
                                  r.ic[IC_PAGE_SIZE], P<void>(pool.k), P<void>(pool.v), P<float>(pool.ks),
                                  P<float>(pool.vs), st));
    if (hm) {
      float* attn32 = P<float>(pp[PP_SM_ATTN]);
      RC(bonsai_attn_decode(q, positions, bt, 0, T, nq, nkv, hd, kvt, r.ic[IC_PAGE_SIZE], P<void>(pool.k),
                            P<void>(pool.v), P<float>(pool.ks), P<float>(pool.vs), sm_splits, P<float>(pp[PP_SM_ACC]),
                            P<float>(pp[PP_SM_ML]), P<int>(pp[PP_SM_CTR]), attn32, 0, st));
      RC(bonsai_norm_to_f16_hmma(attn32, qd, nullptr, r.eps, T, qd, attn, qd, st));
    } else {
      RC(bonsai_attn_prefill_order(q, T, pos0, bt, nq, nkv, hd, kvt, r.ic[IC_PAGE_SIZE], P<void>(pool.k),
                                   P<void>(pool.v), P<float>(pool.ks), P<float>(pool.vs), attn, qd, 0, st));
    }
    if (!tp) {
      RC(gemm(P<void>(lp[LP_O_CODES]), P<void>(lp[LP_O_SCALES]), attn, qd, h, h, nullptr, hidden, qd, 1, hidden));
    } else if (tp_fused) {
      RC(bonsai_bitgemm_hmma_tp(r.comm, P<void>(lp[LP_O_CODES]), P<void>(lp[LP_O_SCALES]), attn, qd, h, h, hidden, qd, T, hidden, st));
    } else {
      RC(gemm(P<void>(lp[LP_O_CODES]), P<void>(lp[LP_O_SCALES]), attn, qd, big, nullptr, nullptr, hidden, qd, 0, hidden));
      RC(bonsai_tp_allreduce_big_add(r.comm, h, (size_t)T * hidden, st));
    }
    RC(to_f16(P<float>(lp[LP_FFN_NORM])));
    RC(gemm(P<void>(lp[LP_GU_CODES]), P<void>(lp[LP_GU_SCALES]), xn, xn_ld, nullptr, nullptr, act, 2 * inter, hidden, 2, inter));
    if (!tp) {
      RC(gemm(P<void>(lp[LP_DOWN_CODES]), P<void>(lp[LP_DOWN_SCALES]), act, inter, h, h, nullptr, hidden, inter, 1, hidden));
    } else if (tp_fused) {
      RC(bonsai_bitgemm_hmma_tp(r.comm, P<void>(lp[LP_DOWN_CODES]), P<void>(lp[LP_DOWN_SCALES]), act, inter, h, h, hidden, inter, T, hidden, st));
    } else {
      RC(gemm(P<void>(lp[LP_DOWN_CODES]), P<void>(lp[LP_DOWN_SCALES]), act, inter, big, nullptr, nullptr, hidden, inter, 0, hidden));
      RC(bonsai_tp_allreduce_big_add(r.comm, h, (size_t)T * hidden, st));
    }
  }
  if (want_logits) {
    float* hs = P<float>(sp[SP_H]) + (size_t)slot * hidden;
    if (cudaMemcpyAsync(hs, h + (size_t)(T - 1) * hidden, (size_t)hidden * sizeof(float), cudaMemcpyDeviceToDevice, st) != cudaSuccess)
      return BONSAI_CUDA_LAUNCH_FAILED;
    if (!tp) {
      RC(bonsai_f16gemv(P<void>(r.gp[GP_LM_HEAD]), hs, P<float>(r.gp[GP_OUT_NORM]), r.eps, P<float>(sp[SP_LOGITS]) + (size_t)slot * vocab,
                        lm_rows, hidden, st));
    } else {
      const int rows_per_rank = (vocab + r.ic[IC_TP_SIZE] - 1) / r.ic[IC_TP_SIZE];
      float* partial = P<float>(sp[SP_PARTIAL]) + (size_t)slot * lm_rows;
      if (lm_rows > 0) RC(bonsai_f16gemv(P<void>(r.gp[GP_LM_HEAD]), hs, P<float>(r.gp[GP_OUT_NORM]), r.eps, partial, lm_rows, hidden, st));
      RC(bonsai_tp_allgather_logits_at(r.comm, partial, slot, 1, lm_rows, r.ic[IC_TP_RANK] * rows_per_rank, vocab, st));
    }
  }
  return 0;
}

// Batched decode step for `batch` live sequences (slots 0..batch-1): every linear layer is one
// tcgen05 GEMM over all sequences (the packed weights are expanded once per step, not once per
// sequence), attention stays the per-sequence split-KV kernel, and the LM head is a dense f16
// tcgen05 GEMM.  The reference's continuous batching re-runs a full single-sequence generate per
// request per step (crates/oxibonsai-runtime/src/continuous_batch.rs:283-293).
//
// Tensor parallel: up to 16 sequences, the row-parallel O and down GEMMs run on the mma.sync kernel and their epilogue
// is the all-reduce + residual add ({value, tag} stores into the peers' memory, summed in rank order).  Larger batches
// write partial sums into alternating halves of the symmetric big area and one kernel per all-reduce (entry flag
// barrier + peer loads + residual add) folds them into h; every step issues an even number of those, so the
// alternation of halves continues across replays of a captured step.  The vocab-parallel LM head writes
// [batch][local rows] and the slices are pushed into every rank's logits area.
static int decode_step_batched(Runner& r, const uint64_t* sp, const uint64_t* pp, int batch, int flags, int mask_words,
                               cudaStream_t st) {
  const int hidden = r.ic[IC_HIDDEN], inter = r.ic[IC_INTER_LOCAL], nq = r.ic[IC_HEADS_LOCAL], nkv = r.ic[IC_KV_HEADS_LOCAL];
  const int hd = r.ic[IC_HEAD_DIM], vocab = r.ic[IC_VOCAB], lm_rows = r.ic[IC_LM_ROWS_LOCAL];
  const int qd = nq * hd, kvd = nkv * hd, qkv_n = qd + 2 * kvd;
  const bool tp = r.ic[IC_TP_SIZE] > 1;
  float* big[2] = {tp ? static_cast<float*>(bonsai_tp_big_half_ptr(r.comm, 0)) : nullptr,
                   tp ? static_cast<float*>(bonsai_tp_big_half_ptr(r.comm, 1)) : nullptr};
  const int sms = 148;
  int* tokens = P<int>(sp[SP_TOKENS]);
  int* positions = P<int>(sp[SP_POSITIONS]);
  const int* bt = P<int>(sp[SP_BLOCK_TABLE]);
  float* h = P<float>(sp[SP_H]);
  float* qkv = P<float>(sp[SP_QKV]);
  float* q = P<float>(sp[SP_Q]);
  float* attn = P<float>(sp[SP_ATTN]);
  float* logits = P<float>(sp[SP_LOGITS]);
  void* xn = P<void>(pp[PP_XN]);
  void* attn16 = P<void>(pp[PP_ATTN]);
  void* act = P<void>(pp[PP_ACT]);
  int* status = P<int>(pp[PP_STATUS]);
  r.gemm_ws = P<void>(pp[PP_GEMM_WS]);
  r.gemm_ws_bytes = (size_t)pp[PP_GEMM_WS_BYTES];
  const int xn_ld = hidden > qd ? hidden : qd;
  // Small batches run the packed GEMMs on mma.sync with register-expanded weights (bitgemm_hmma.cu, activations in
  // hmma-K order); the tcgen05 kernel (paired-K order) takes over where it measured faster.  QKV / O / gate-up / down
  // of the 8B model in us: 8 tokens 15.7 / 8.3 / 24.6 / 20.9 against 17.8 / 17.6 / 32.8 / 24.7, 32 tokens 23.9 / 12.7 /
  // 40.2 / 33.3 against 21.8 / 25.0 / 38.4 / 30.7, 64 tokens 39.6 / 20.6 / 66.0 / 51.7 against 26.3 / 26.1 / 43.4 / 39.0:
  // everything up to 32 sequences, and the O projection (few rows, short K) up to 64.
  const bool hm_ok = r.ic[IC_FAST] != 5 && hidden % 128 == 0 && qd % 128 == 0 && inter % 128 == 0;
  // Tensor parallel, up to 16 sequences: the two row-parallel GEMMs carry the all-reduce + residual add in their epilogue
  // ({value, tag} messages).  That doubles the bytes on the wire, which is right while the exchange is latency-bound;
  // measured at 64 sequences (2 MB per peer per exchange) it lost to partial sums + the one-shot all-reduce kernel
  // (TP = 2: 7.3 against 6.2 ms per step), so larger batches keep that path.
  const bool tp_fused = tp && hm_ok && batch <= 16;
  const bool hm_all = hm_ok && batch <= 32, hm_o = hm_ok && batch <= 64;
  auto to_f16 = [&](bool hm, const float* src, int src_ld, const float* w, int K, void* dst, int dst_ld) {
    return hm ? bonsai_norm_to_f16_hmma(src, src_ld, w, r.eps, batch, K, dst, dst_ld, st)
              : bonsai_norm_to_f16_paired(src, src_ld, w, r.eps, batch, K, dst, dst_ld, 0, st);
  };
  auto gemm = [&](bool hm, const void* codes, const void* scales, const void* x, int x_ld, float* out_f32, const float* residual,
                  void* out_f16, int n_rows, int K, int epi, int out_ld) {
    return hm ? bonsai_bitgemm_hmma(codes, scales, x, x_ld, out_f32, residual, out_f16, n_rows, K, batch, epi, out_ld, st)
              : pf_gemm(r, codes, scales, x, x_ld, out_f32, residual, out_f16, status, n_rows, K, batch, epi, out_ld, sms, nullptr, st);
  };
  // about four CTAs per SM over all (sequence, kv head, split) triples, within the workspace's split count
  int attn_splits = (4 * 148) / (nkv * batch);
  if (attn_splits < 1) attn_splits = 1;
  if (attn_splits > r.ic[IC_NSPLIT_BATCHED]) attn_splits = r.ic[IC_NSPLIT_BATCHED];

  RC(bonsai_embed_rows_f16(P<void>(r.gp[GP_EMBD]), tokens, h, batch, hidden, vocab, st));
  for (int l = 0; l < r.ic[IC_LAYERS]; ++l) {
    const uint64_t* lp = &r.lp[(size_t)l * LP_COUNT];
    RC(to_f16(hm_all, h, hidden, P<float>(lp[LP_ATTN_NORM]), hidden, xn, xn_ld));
    RC(gemm(hm_all, P<void>(lp[LP_QKV_CODES]), P<void>(lp[LP_QKV_SCALES]), xn, xn_ld, qkv, nullptr, nullptr, qkv_n, hidden, 0, qkv_n));
    RC(qkv_attention(r, l, lp, sp, qkv, qkv_n, q, attn, positions, bt, batch, attn_splits, st));
    RC(to_f16(hm_o, attn, qd, nullptr, qd, attn16, qd));
    if (!tp) {
      RC(gemm(hm_o, P<void>(lp[LP_O_CODES]), P<void>(lp[LP_O_SCALES]), attn16, qd, h, h, nullptr, hidden, qd, 1, hidden));
    } else if (tp_fused) {
      RC(bonsai_bitgemm_hmma_tp(r.comm, P<void>(lp[LP_O_CODES]), P<void>(lp[LP_O_SCALES]), attn16, qd, h, h, hidden, qd, batch, hidden, st));
    } else {
      RC(gemm(hm_o, P<void>(lp[LP_O_CODES]), P<void>(lp[LP_O_SCALES]), attn16, qd, big[0], nullptr, nullptr, hidden, qd, 0, hidden));
      RC(bonsai_tp_allreduce_oneshot_add(r.comm, h, (size_t)batch * hidden, 0, st));
    }
    RC(to_f16(hm_all, h, hidden, P<float>(lp[LP_FFN_NORM]), hidden, xn, xn_ld));
    RC(gemm(hm_all, P<void>(lp[LP_GU_CODES]), P<void>(lp[LP_GU_SCALES]), xn, xn_ld, nullptr, nullptr, act, 2 * inter, hidden, 2, inter));
    if (!tp) {
      RC(gemm(hm_all, P<void>(lp[LP_DOWN_CODES]), P<void>(lp[LP_DOWN_SCALES]), act, inter, h, h, nullptr, hidden, inter, 1, hidden));
    } else if (tp_fused) {
      RC(bonsai_bitgemm_hmma_tp(r.comm, P<void>(lp[LP_DOWN_CODES]), P<void>(lp[LP_DOWN_SCALES]), act, inter, h, h, hidden, inter, batch, hidden, st));
    } else {
      RC(gemm(hm_all, P<void>(lp[LP_DOWN_CODES]), P<void>(lp[LP_DOWN_SCALES]), act, inter, big[1], nullptr, nullptr, hidden, inter, 0, hidden));
      RC(bonsai_tp_allreduce_oneshot_add(r.comm, h, (size_t)batch * hidden, 1, st));
    }
  }
  if (!(flags & 2)) {
    RC(bonsai_norm_to_f16_paired(h, hidden, P<float>(r.gp[GP_OUT_NORM]), r.eps, batch, hidden, xn, xn_ld, 1, st));
    if (!tp) {
      RC(pf_gemm(r, nullptr, nullptr, xn, xn_ld, logits, nullptr, nullptr, status, lm_rows, hidden, batch, 0, vocab, sms,
                                P<void>(r.gp[GP_LM_HEAD]), st));
    } else {
      float* partial = P<float>(sp[SP_PARTIAL]);
      const int rows_per_rank = (vocab + r.ic[IC_TP_SIZE] - 1) / r.ic[IC_TP_SIZE];
      if (lm_rows > 0)
        RC(pf_gemm(r, nullptr, nullptr, xn, xn_ld, partial, nullptr, nullptr, status, lm_rows, hidden, batch, 0, lm_rows, sms,
                                  P<void>(r.gp[GP_LM_HEAD]), st));
      RC(bonsai_tp_allgather_logits_at(r.comm, partial, 0, batch, lm_rows, r.ic[IC_TP_RANK] * rows_per_rank, vocab, st));
    }
  } else if (tp) {
    // no logits gather (and hence no barrier) in this step: close it so that a following prefill
    // cannot overwrite the big area while a peer still reads it
    RC(bonsai_tp_barrier(r.comm, st));
  }
  if (flags & 1) {
    RC(bonsai_sample(logits, batch, vocab, vocab, P<float>(sp[SP_TEMPS]), P<int>(sp[SP_TOPKS]), P<float>(sp[SP_TOPPS]),
                     P<unsigned long long>(sp[SP_RNG]), P<int>(sp[SP_OUT_TOKENS]), positions, 1,
                     mask_words > 0 ? P<uint32_t>(sp[SP_ALLOW_MASK]) : nullptr, mask_words, st));
  }
  return 0;
}

}  // namespace bonsai

extern "C" {

void* bonsai_runner_create(const int* icfg, float eps, const uint64_t* global_ptrs, const uint64_t* layer_ptrs) {
  using namespace bonsai;
  Runner* r = new Runner();
  for (int i = 0; i < IC_COUNT; ++i) r->ic[i] = icfg[i];
  r->eps = eps;
  for (int i = 0; i < GP_COUNT; ++i) r->gp[i] = global_ptrs[i];
  r->lp.assign(layer_ptrs, layer_ptrs + (size_t)icfg[IC_LAYERS] * LP_COUNT);
  return r;
}

// Registers the K / V pools of `layer` in page format kvt (0 f32, 1 f16, 2 int8, 3 int4) beside the runner's default format.
int bonsai_runner_set_pool(void* rp, int kvt, int layer, const void* k, const void* v, const void* ks, const void* vs) {
  bonsai::Runner& r = *static_cast<bonsai::Runner*>(rp);
  if (kvt < 0 || kvt > 3 || layer < 0 || layer >= r.ic[bonsai::IC_LAYERS]) return BONSAI_CUDA_BAD_ARG;
  if (r.pools[kvt].empty()) r.pools[kvt].resize(r.ic[bonsai::IC_LAYERS]);
  bonsai::KvPoolPtrs p;
  p.k = (uint64_t)k; p.v = (uint64_t)v; p.ks = (uint64_t)ks; p.vs = (uint64_t)vs;
  r.pools[kvt][layer] = p;
  return 0;
}
// Page format of the sequences in slots 0 .. n-1 for the launches that follow (and the graphs captured from them).
int bonsai_runner_set_slot_formats(void* rp, const int* fmts, int n) {
  bonsai::Runner& r = *static_cast<bonsai::Runner*>(rp);
  for (int i = 0; i < n; ++i)
    if (fmts[i] < 0 || fmts[i] > 3 || (fmts[i] != r.ic[bonsai::IC_KVT] && r.pools[fmts[i]].empty())) return BONSAI_CUDA_BAD_ARG;
  r.slot_fmt.assign(fmts, fmts + n);
  return 0;
}

void bonsai_runner_destroy(void* r) { delete static_cast<bonsai::Runner*>(r); }
void bonsai_runner_set_comm(void* r, void* comm) { static_cast<bonsai::Runner*>(r)->comm = comm; }
void bonsai_runner_set_nsplit(void* r, int nsplit) { static_cast<bonsai::Runner*>(r)->ic[bonsai::IC_NSPLIT] = nsplit; }
void bonsai_runner_set_fast(void* r, int fast) { static_cast<bonsai::Runner*>(r)->ic[bonsai::IC_FAST] = fast; }
int bonsai_runner_layer_ptr_count() { return bonsai::LP_COUNT; }
int bonsai_runner_step_ptr_count() { return bonsai::SP_COUNT; }
int bonsai_runner_prefill_ptr_count() { return bonsai::PP_COUNT; }

int bonsai_runner_decode_step_batched(void* r, const uint64_t* step_ptrs, const uint64_t* prefill_ptrs, int batch, int flags,
                                      int mask_words, cudaStream_t stream) {
  return bonsai::decode_step_batched(*static_cast<bonsai::Runner*>(r), step_ptrs, prefill_ptrs, batch, flags, mask_words, stream);
}

int bonsai_runner_prefill_chunk(void* r, const uint64_t* step_ptrs, const uint64_t* prefill_ptrs, int T, int pos0, int slot,
                                int want_logits, cudaStream_t stream) {
  return bonsai::prefill_chunk(*static_cast<bonsai::Runner*>(r), step_ptrs, prefill_ptrs, T, pos0, slot, want_logits, stream);
}

int bonsai_runner_decode_step(void* r, const uint64_t* step_ptrs, int batch, int flags, int mask_words, cudaStream_t stream) {
  return bonsai::decode_step(*static_cast<bonsai::Runner*>(r), step_ptrs, batch, flags, mask_words, stream);
}

int bonsai_runner_small_chunk() { return bonsai::kSmallChunk; }
int bonsai_runner_small_splits() { return bonsai::kSmallSplits; }

}  // extern "C"
