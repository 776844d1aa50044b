// CPU oracle: the Qwen3 decoder forward in plain f32 with sequential sums, restating the
// reference's scalar path (reference: crates/oxibonsai-model/src/model/types/mod.rs:633-934,
// block/types/forward.rs:33-419, crates/oxibonsai-kernels/src/gemv_ternary.rs:48-104, gemv.rs:25-88,
// simd_float_ops.rs:187-254, crates/oxibonsai-model/src/layers/attention_fused.rs:184-226,
// layers/rope.rs:27-46, crates/oxibonsai-runtime/src/sampling.rs:182-189, engine.rs:401-422).
//
// Per token: embed -> [RMSNorm -> q,k,v GEMV -> per-head QK RMSNorm -> half-split RoPE -> append
// to an f32 KV cache -> causal GQA with position-ordered online softmax -> o-proj + residual ->
// RMSNorm -> gate,up GEMV -> silu(gate)*up -> down + residual] x L -> RMSNorm -> LM head.
// Greedy sampling returns the LAST maximal index; token 151645 ends generation before being
// emitted.  Rows of a GEMV are independent, so they are spread over threads without changing
// any row's arithmetic.
#pragma once
#include <cstdint>
#include <memory>
#include <string>
#include <vector>

#include "../core/config.hpp"
#include "../core/gguf.hpp"

namespace bonsai {

constexpr uint32_t kEosToken = 151645;

// Row-major quantised (or float) matrix: `rows` output features of `cols` inputs each.
struct MatrixRef {
  const uint8_t* data = nullptr;
  uint32_t type = 0;
  uint64_t rows = 0, cols = 0;
};

// out[r] = sum_k W[r][k] * x[k], block-sequential as the reference's scalar kernels.
void cpu_gemv(const MatrixRef& w, const float* x, float* out);
// Dequantise a row range into f32 (row-major).
void cpu_dequant_rows(const MatrixRef& w, uint64_t row0, uint64_t nrows, float* out);

void cpu_rmsnorm(const float* x, const float* w, float* out, size_t n, float eps);
void cpu_rope_halfsplit(float* x, size_t head_dim, uint32_t pos, float base);
void cpu_swiglu(const float* gate, const float* up, float* out, size_t n);
int cpu_argmax_last(const float* x, size_t n);

class OracleModel {
 public:
  OracleModel(const GgufFile& f, uint32_t max_seq);
  const Qwen3Config& config() const { return cfg_; }
  // Runs one token at `pos` (appending to the KV cache) and writes vocab logits.
  void forward(uint32_t token, uint32_t pos, float* logits);
  // Prefill is a loop of single-token forwards, then greedy decode.  Returns generated ids;
  // `gaps` (optional) receives top1 - top2 logit per generated step.
  std::vector<uint32_t> generate_greedy(const std::vector<uint32_t>& prompt, uint32_t max_new,
                                        std::vector<float>* gaps, bool stop_at_eos = true);
  // Hidden state after the final norm of the last forward (for parity tests).
  const std::vector<float>& last_hidden() const { return normed_; }
  // When enabled, the residual stream after every layer of the last forward is kept ([layers][hidden]).
  void keep_layer_hidden(bool on) { layer_hidden_.assign(on ? (size_t)cfg_.layers * cfg_.hidden : 0, 0.0f); }
  const std::vector<float>& layer_hidden() const { return layer_hidden_; }

 private:
  struct Layer {
    MatrixRef wq, wk, wv, wo, wgate, wup, wdown;
    const float* attn_norm;
    const float* ffn_norm;
    const float* q_norm;
    const float* k_norm;
  };
  Qwen3Config cfg_;
  uint32_t max_seq_;
  MatrixRef embd_, lm_head_;
  const float* out_norm_;
  std::vector<Layer> layers_;
  std::vector<float> kcache_, vcache_;  // [layer][kv_head][max_seq][hd]
  std::vector<float> x_, normed_, q_, k_, v_, attn_, proj_, gate_, up_, act_;
  std::vector<float> layer_hidden_;
  std::vector<std::vector<float>> owned_f32_;  // norm vectors converted from non-f32 storage

  const float* norm_vector(const GgufFile& f, const std::string& name, uint64_t n);
  MatrixRef matrix(const GgufFile& f, const std::string& name, uint64_t rows, uint64_t cols);
};

struct SyntheticSpec {
  Qwen3Config cfg;
  uint32_t weight_type = 42;   // 42 = TQ2_0_g128, 41 = Q1_0_g128
  uint32_t embd_type = 1;      // F16
  bool tied = true;            // output.weight duplicates token_embd.weight
  uint64_t seed = 42;
  float embd_std = 0.02f;
  float scale_mean = 0.02f, scale_std = 0.002f;
  bool llm_keys = false;       // write `llm.*` metadata instead of `{arch}.*`
};

// Writes a seeded random-init checkpoint of the given shape: embeddings ~ N(0, embd_std) in f16,
// norm weights 1.0 (f32), ternary codes iid uniform over {-1,0,+1} (or Bernoulli(0.5) sign bits),
// one f16 scale |N(scale_mean, scale_std)| per 128 weights.
void write_synthetic_gguf(const std::string& path, const SyntheticSpec& spec);

}  // namespace bonsai
