// Qwen3 decoder hyper-parameters read from GGUF metadata.
//
// Keys are looked up as `{general.architecture}.<key>` first and `llm.<key>` second, with the
// reference's defaults (4096 / 36 / 32 / 8 / 14336 / 151936 / 65536 / 1e-6 / 1e6) when both are
// missing (reference: crates/oxibonsai-core/src/config.rs:41-116).  Two deliberate differences:
// `attention.key_length` overrides head_dim = hidden / heads when present, which Qwen3-4B
// shapes (hidden 2560, 32 heads, head_dim 128) need, and the vocabulary size is corrected from
// the embedding tensor's shape when that tensor exists.
#pragma once
#include <cstdint>
#include <string>

#include "gguf.hpp"

namespace bonsai {

struct Qwen3Config {
  uint32_t hidden = 4096;
  uint32_t inter = 14336;
  uint32_t layers = 36;
  uint32_t heads = 32;
  uint32_t kv_heads = 8;
  uint32_t head_dim = 128;
  uint32_t vocab = 151936;
  uint32_t context = 65536;
  float eps = 1e-6f;
  float rope_base = 1e6f;
  std::string arch = "qwen3";
  std::string name = "Bonsai-8B";
};

inline bool meta_u32(const GgufFile& f, const std::string& arch, const char* key, uint32_t* out) {
  const MetaValue* v = f.find(arch + "." + key);
  if (!v) v = f.find(std::string("llm.") + key);
  uint64_t u;
  if (v && v->as_u64(&u)) {
    *out = static_cast<uint32_t>(u);
    return true;
  }
  return false;
}

inline bool meta_f32(const GgufFile& f, const std::string& arch, const char* key, float* out) {
  const MetaValue* v = f.find(arch + "." + key);
  if (!v) v = f.find(std::string("llm.") + key);
  double d;
  if (v && v->as_f64(&d)) {
    *out = static_cast<float>(d);
    return true;
  }
  return false;
}

inline Qwen3Config config_from_gguf(const GgufFile& f) {
  Qwen3Config c;
  if (const MetaValue* a = f.find("general.architecture"); a && a->type == MetaType::String) c.arch = a->s;
  if (const MetaValue* n = f.find("general.name"); n && n->type == MetaType::String) c.name = n->s;
  meta_u32(f, c.arch, "embedding_length", &c.hidden);
  meta_u32(f, c.arch, "block_count", &c.layers);
  meta_u32(f, c.arch, "attention.head_count", &c.heads);
  meta_u32(f, c.arch, "attention.head_count_kv", &c.kv_heads);
  meta_u32(f, c.arch, "feed_forward_length", &c.inter);
  meta_u32(f, c.arch, "vocab_size", &c.vocab);
  meta_u32(f, c.arch, "context_length", &c.context);
  meta_f32(f, c.arch, "attention.layer_norm_rms_epsilon", &c.eps);
  meta_f32(f, c.arch, "rope.freq_base", &c.rope_base);
  if (c.heads == 0) fail(ErrorCode::MissingMetadata, "attention.head_count is zero");
  c.head_dim = c.hidden / c.heads;
  meta_u32(f, c.arch, "attention.key_length", &c.head_dim);
  int e = f.tensor_index("token_embd.weight");
  if (e >= 0 && f.tensors[e].dims.size() == 2) c.vocab = static_cast<uint32_t>(f.tensors[e].dims[1]);
  if (c.kv_heads == 0 || c.heads % c.kv_heads != 0) fail(ErrorCode::ShapeMismatch, "head_count must be a multiple of head_count_kv");
  return c;
}

}  // namespace bonsai
