// C ABI of the host library (GGUF container, block codecs, CPU oracle, synthetic checkpoints).
// Every function returns 0 / a valid handle on success and a negative code / null on failure;
// the message of the last failure on the calling thread is available from bonsai_last_error().
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <string>

#include "core/blocks.hpp"
#include "core/kquants.hpp"
#include "core/config.hpp"
#include "core/gguf.hpp"
#include "cpu/oracle.hpp"

using namespace bonsai;

namespace {
thread_local std::string g_err;
thread_local int g_code = 0;

int set_error(const BonsaiError& e) {
  g_err = e.what();
  g_code = static_cast<int>(e.code());
  return -g_code;
}
int set_error(const std::exception& e) {
  g_err = e.what();
  g_code = static_cast<int>(ErrorCode::Internal);
  return -g_code;
}
}  // namespace

#define BONSAI_TRY try {
#define BONSAI_CATCH_INT \
  } catch (const BonsaiError& e) { return set_error(e); } catch (const std::exception& e) { return set_error(e); }
#define BONSAI_CATCH_PTR \
  } catch (const BonsaiError& e) { set_error(e); return nullptr; } catch (const std::exception& e) { set_error(e); return nullptr; }

extern "C" {

const char* bonsai_last_error() { return g_err.c_str(); }
int bonsai_last_error_code() { return g_code; }
const char* bonsai_error_name(int code) { return error_code_name(static_cast<ErrorCode>(code)); }
int bonsai_error_retryable(int code) { return error_is_retryable(static_cast<ErrorCode>(code)) ? 1 : 0; }
void bonsai_free(void* p) { std::free(p); }

// ---- type table -----------------------------------------------------------------------------
int bonsai_type_info(uint32_t id, uint32_t* block_elems, uint32_t* block_bytes, char* name, size_t cap) {
  TypeTraits t;
  if (!tensor_type_traits(id, &t)) return -static_cast<int>(ErrorCode::UnsupportedQuantType);
  if (block_elems) *block_elems = t.block_elems;
  if (block_bytes) *block_bytes = t.block_bytes;
  if (name && cap) {
    std::strncpy(name, t.name, cap - 1);
    name[cap - 1] = 0;
  }
  return 0;
}

// ---- GGUF reader ----------------------------------------------------------------------------
void* bgguf_open(const char* path) {
  BONSAI_TRY
  return GgufFile::open(path).release();
  BONSAI_CATCH_PTR
}
void* bgguf_parse(const uint8_t* data, size_t size) {
  BONSAI_TRY
  return GgufFile::parse(data, size).release();
  BONSAI_CATCH_PTR
}
void bgguf_close(void* h) { delete static_cast<GgufFile*>(h); }
uint32_t bgguf_version(void* h) { return static_cast<GgufFile*>(h)->version; }
uint32_t bgguf_alignment(void* h) { return static_cast<GgufFile*>(h)->alignment; }
uint64_t bgguf_data_offset(void* h) { return static_cast<GgufFile*>(h)->data_offset; }
uint64_t bgguf_n_tensors(void* h) { return static_cast<GgufFile*>(h)->tensors.size(); }
uint64_t bgguf_n_kv(void* h) { return static_cast<GgufFile*>(h)->kv.size(); }
uint64_t bgguf_file_size(void* h) { return static_cast<GgufFile*>(h)->size(); }

char* bgguf_metadata_json(void* h, uint64_t max_array_items) {
  BONSAI_TRY
  std::string s = static_cast<GgufFile*>(h)->metadata_json(max_array_items);
  char* out = static_cast<char*>(std::malloc(s.size() + 1));
  std::memcpy(out, s.c_str(), s.size() + 1);
  return out;
  BONSAI_CATCH_PTR
}

int bgguf_find_tensor(void* h, const char* name) { return static_cast<GgufFile*>(h)->tensor_index(name); }

int bgguf_tensor_info(void* h, uint64_t idx, char* name, size_t cap, uint64_t* dims, uint32_t* ndims, uint32_t* type,
                      uint64_t* offset, uint64_t* nbytes) {
  BONSAI_TRY
  GgufFile* f = static_cast<GgufFile*>(h);
  if (idx >= f->tensors.size()) fail(ErrorCode::TensorNotFound, "tensor index out of range");
  const TensorInfo& t = f->tensors[idx];
  if (name && cap) {
    std::strncpy(name, t.name.c_str(), cap - 1);
    name[cap - 1] = 0;
  }
  *ndims = static_cast<uint32_t>(t.dims.size());
  for (size_t d = 0; d < t.dims.size() && d < 8; ++d) dims[d] = t.dims[d];
  *type = t.type;
  *offset = t.offset;
  TypeTraits tt;
  *nbytes = tensor_type_traits(t.type, &tt) ? t.data_size() : 0;
  return 0;
  BONSAI_CATCH_INT
}

const uint8_t* bgguf_tensor_data(void* h, uint64_t idx, uint64_t* nbytes) {
  BONSAI_TRY
  return static_cast<GgufFile*>(h)->tensor_data(idx, nbytes);
  BONSAI_CATCH_PTR
}

// cfg_u32 = {hidden, inter, layers, heads, kv_heads, head_dim, vocab, context}; cfg_f32 = {eps, rope_base}
int bgguf_config(void* h, uint32_t* cfg_u32, float* cfg_f32, char* arch, size_t arch_cap, char* name, size_t name_cap) {
  BONSAI_TRY
  Qwen3Config c = config_from_gguf(*static_cast<GgufFile*>(h));
  uint32_t v[8] = {c.hidden, c.inter, c.layers, c.heads, c.kv_heads, c.head_dim, c.vocab, c.context};
  std::memcpy(cfg_u32, v, sizeof v);
  cfg_f32[0] = c.eps;
  cfg_f32[1] = c.rope_base;
  if (arch && arch_cap) { std::strncpy(arch, c.arch.c_str(), arch_cap - 1); arch[arch_cap - 1] = 0; }
  if (name && name_cap) { std::strncpy(name, c.name.c_str(), name_cap - 1); name[name_cap - 1] = 0; }
  return 0;
  BONSAI_CATCH_INT
}

// ---- GGUF writer ----------------------------------------------------------------------------
void* bggufw_new(uint32_t version, uint32_t alignment) { return new GgufWriter(version, alignment); }
void bggufw_free(void* h) { delete static_cast<GgufWriter*>(h); }
void bggufw_add_u32(void* h, const char* k, uint32_t v) { static_cast<GgufWriter*>(h)->add_kv(k, MetaValue::of_u32(v)); }
void bggufw_add_u64(void* h, const char* k, uint64_t v) { static_cast<GgufWriter*>(h)->add_kv(k, MetaValue::of_u64(v)); }
void bggufw_add_i32(void* h, const char* k, int32_t v) { static_cast<GgufWriter*>(h)->add_kv(k, MetaValue::of_i32(v)); }
void bggufw_add_f32(void* h, const char* k, float v) { static_cast<GgufWriter*>(h)->add_kv(k, MetaValue::of_f32(v)); }
void bggufw_add_f64(void* h, const char* k, double v) { static_cast<GgufWriter*>(h)->add_kv(k, MetaValue::of_f64(v)); }
void bggufw_add_bool(void* h, const char* k, int v) { static_cast<GgufWriter*>(h)->add_kv(k, MetaValue::of_bool(v != 0)); }
void bggufw_add_str(void* h, const char* k, const char* v) { static_cast<GgufWriter*>(h)->add_kv(k, MetaValue::of_str(v)); }
// Generic scalar with an explicit metadata type id (0..7, 10..12); value passed as i64/f64.
void bggufw_add_scalar(void* h, const char* k, uint32_t type, int64_t iv, double fv) {
  MetaValue m;
  m.type = static_cast<MetaType>(type);
  m.u = static_cast<uint64_t>(iv);
  m.i = iv;
  m.f = fv;
  static_cast<GgufWriter*>(h)->add_kv(k, std::move(m));
}
void bggufw_add_str_array(void* h, const char* k, const char* const* items, const uint64_t* lens, uint64_t n) {
  MetaValue m;
  m.type = MetaType::Array;
  m.elem_type = MetaType::String;
  m.arr.reserve(n);
  for (uint64_t i = 0; i < n; ++i) m.arr.push_back(MetaValue::of_str(std::string(items[i], lens[i])));
  static_cast<GgufWriter*>(h)->add_kv(k, std::move(m));
}
void bggufw_add_num_array(void* h, const char* k, uint32_t elem_type, const int64_t* iv, const double* fv, uint64_t n) {
  MetaValue m;
  m.type = MetaType::Array;
  m.elem_type = static_cast<MetaType>(elem_type);
  m.arr.reserve(n);
  for (uint64_t i = 0; i < n; ++i) {
    MetaValue e;
    e.type = m.elem_type;
    if (iv) { e.i = iv[i]; e.u = static_cast<uint64_t>(iv[i]); }
    if (fv) e.f = fv[i];
    m.arr.push_back(std::move(e));
  }
  static_cast<GgufWriter*>(h)->add_kv(k, std::move(m));
}
int bggufw_add_tensor(void* h, const char* name, const uint64_t* dims, uint32_t ndims, uint32_t type, const uint8_t* data,
                      uint64_t nbytes, int copy) {
  BONSAI_TRY
  std::vector<uint64_t> d(dims, dims + ndims);
  static_cast<GgufWriter*>(h)->add_tensor(name, d, type, data, nbytes, copy != 0);
  return 0;
  BONSAI_CATCH_INT
}
int bggufw_write(void* h, const char* path) {
  BONSAI_TRY
  static_cast<GgufWriter*>(h)->write(path);
  return 0;
  BONSAI_CATCH_INT
}
// Serialises into a malloc'd buffer (caller frees with bonsai_free).
uint8_t* bggufw_to_bytes(void* h, uint64_t* size) {
  BONSAI_TRY
  std::vector<uint8_t> b = static_cast<GgufWriter*>(h)->to_bytes();
  uint8_t* out = static_cast<uint8_t*>(std::malloc(b.size() ? b.size() : 1));
  std::memcpy(out, b.data(), b.size());
  *size = b.size();
  return out;
  BONSAI_CATCH_PTR
}

// ---- streaming parser -----------------------------------------------------------------------
void* bggufs_new() { return new GgufStreamParser(); }
void bggufs_free(void* h) { delete static_cast<GgufStreamParser*>(h); }
// 0 = need more, 1 = header complete, 2 = failed
int bggufs_feed(void* h, const uint8_t* chunk, size_t n) { return static_cast<int>(static_cast<GgufStreamParser*>(h)->feed(chunk, n)); }
// Borrowed GgufFile handle (valid while the parser lives); null until the header is complete.
void* bggufs_file(void* h) { return const_cast<GgufFile*>(static_cast<GgufStreamParser*>(h)->file()); }
uint64_t bggufs_bytes_consumed(void* h) { return static_cast<GgufStreamParser*>(h)->bytes_consumed(); }
uint64_t bggufs_data_seen(void* h) { return static_cast<GgufStreamParser*>(h)->data_bytes_seen(); }
uint64_t bggufs_data_expected(void* h) { return static_cast<GgufStreamParser*>(h)->data_bytes_expected(); }
const char* bggufs_error(void* h) { return static_cast<GgufStreamParser*>(h)->error().c_str(); }

// ---- codecs ---------------------------------------------------------------------------------
int bonsai_dequant(uint32_t type, const uint8_t* src, uint64_t n_blocks, float* dst) {
  switch (type) {
    case 41: dequant_q1(src, n_blocks, dst); return 0;
    case 42: dequant_tq2(src, n_blocks, dst); return 0;
    case 35: dequant_tq2_256(src, n_blocks, dst); return 0;
    case 2: dequant_q4_0(src, n_blocks, dst); return 0;
    case 8: dequant_q8_0(src, n_blocks, dst); return 0;
    case 43: dequant_fp8(src, n_blocks, dst, false); return 0;
    case 44: dequant_fp8(src, n_blocks, dst, true); return 0;
    case 10: dequant_q2k(src, n_blocks, dst); return 0;
    case 11: dequant_q3k(src, n_blocks, dst); return 0;
    case 12: dequant_q4k(src, n_blocks, dst); return 0;
    case 13: dequant_q5k(src, n_blocks, dst); return 0;
    case 14: dequant_q6k(src, n_blocks, dst); return 0;
    case 15: dequant_q8k(src, n_blocks, dst); return 0;
    case 1: for (uint64_t i = 0; i < n_blocks; ++i) dst[i] = f16_to_f32(ld_u16(src + 2 * i)); return 0;
    case 30: for (uint64_t i = 0; i < n_blocks; ++i) dst[i] = bf16_to_f32(ld_u16(src + 2 * i)); return 0;
    case 0: std::memcpy(dst, src, n_blocks * 4); return 0;
    default: g_err = "dequant: unsupported type"; g_code = 7; return -7;
  }
}

// flags: bit 0 = Q1 absmax scale instead of mean |w|
int bonsai_quant(uint32_t type, const float* src, uint64_t n_blocks, uint8_t* dst, uint32_t flags) {
  switch (type) {
    case 41: quant_q1(src, n_blocks, dst, flags & 1); return 0;
    case 42: quant_tq2(src, n_blocks, dst); return 0;
    case 35: quant_tq2_256(src, n_blocks, dst); return 0;
    case 2: quant_q4_0(src, n_blocks, dst); return 0;
    case 8: quant_q8_0(src, n_blocks, dst); return 0;
    case 43: quant_fp8(src, n_blocks, dst, false); return 0;
    case 44: quant_fp8(src, n_blocks, dst, true); return 0;
    case 10: quant_q2k(src, n_blocks, dst); return 0;
    case 11: quant_q3k(src, n_blocks, dst); return 0;
    case 12: quant_q4k(src, n_blocks, dst); return 0;
    case 13: quant_q5k(src, n_blocks, dst); return 0;
    case 14: quant_q6k(src, n_blocks, dst); return 0;
    case 15: quant_q8k(src, n_blocks, dst); return 0;
    case 1: for (uint64_t i = 0; i < n_blocks; ++i) st_u16(dst + 2 * i, f32_to_f16(src[i])); return 0;
    case 30: for (uint64_t i = 0; i < n_blocks; ++i) st_u16(dst + 2 * i, f32_to_bf16(src[i])); return 0;
    case 0: std::memcpy(dst, src, n_blocks * 4); return 0;
    default: g_err = "quant: unsupported type"; g_code = 7; return -7;
  }
}

uint8_t bonsai_fp8_encode(float v, int e5m2) { return e5m2 ? fp8_e5m2_encode(v) : fp8_e4m3_encode(v); }
float bonsai_fp8_decode(uint8_t q, int e5m2) { return e5m2 ? fp8_e5m2_decode(q) : fp8_e4m3_decode(q); }
uint16_t bonsai_f32_to_f16(float v) { return f32_to_f16(v); }
float bonsai_f16_to_f32(uint16_t v) { return f16_to_f32(v); }

// ---- CPU ops --------------------------------------------------------------------------------
int bcpu_gemv(uint32_t type, const uint8_t* data, uint64_t rows, uint64_t cols, const float* x, float* out) {
  BONSAI_TRY
  switch (type) {
    case 0: case 1: case 30: case 2: case 8: case 35: case 41: case 42: case 43: case 44:
    case 10: case 11: case 12: case 13: case 14: case 15: break;
    default: fail(ErrorCode::UnsupportedQuantType, "cpu gemv: unsupported type " + std::to_string(type));
  }
  cpu_gemv(MatrixRef{data, type, rows, cols}, x, out);
  return 0;
  BONSAI_CATCH_INT
}
void bcpu_rmsnorm(const float* x, const float* w, float* out, uint64_t n, float eps) { cpu_rmsnorm(x, w, out, n, eps); }
void bcpu_rope(float* x, uint64_t head_dim, uint32_t pos, float base) { cpu_rope_halfsplit(x, head_dim, pos, base); }
void bcpu_swiglu(const float* g, const float* u, float* out, uint64_t n) { cpu_swiglu(g, u, out, n); }
int bcpu_argmax_last(const float* x, uint64_t n) { return cpu_argmax_last(x, n); }
// cos/sin tables [max_pos][head_dim/2] computed exactly as the oracle does per token:
// freq = 1 / powf(base, 2i/head_dim), angle = (float)pos * freq, cosf / sinf.
void bcpu_rope_table(uint32_t head_dim, uint32_t max_pos, float base, float* cos_out, float* sin_out) {
  uint32_t half = head_dim / 2;
  for (uint32_t p = 0; p < max_pos; ++p)
    for (uint32_t i = 0; i < half; ++i) {
      float freq = 1.0f / std::pow(base, 2.0f * (float)i / (float)head_dim);
      float ang = (float)p * freq;
      cos_out[(size_t)p * half + i] = std::cos(ang);
      sin_out[(size_t)p * half + i] = std::sin(ang);
    }
}

// ---- oracle ---------------------------------------------------------------------------------
void* boracle_new(void* gguf, uint32_t max_seq) {
  BONSAI_TRY
  return new OracleModel(*static_cast<GgufFile*>(gguf), max_seq);
  BONSAI_CATCH_PTR
}
void boracle_free(void* h) { delete static_cast<OracleModel*>(h); }
int boracle_forward(void* h, uint32_t token, uint32_t pos, float* logits) {
  BONSAI_TRY
  static_cast<OracleModel*>(h)->forward(token, pos, logits);
  return 0;
  BONSAI_CATCH_INT
}
int boracle_last_hidden(void* h, float* out, uint64_t n) {
  const std::vector<float>& v = static_cast<OracleModel*>(h)->last_hidden();
  if (n < v.size()) return -14;
  std::memcpy(out, v.data(), v.size() * 4);
  return 0;
}
void boracle_keep_layer_hidden(void* h, int on) { static_cast<OracleModel*>(h)->keep_layer_hidden(on != 0); }
int boracle_layer_hidden(void* h, float* out, uint64_t n) {
  const std::vector<float>& v = static_cast<OracleModel*>(h)->layer_hidden();
  if (v.empty() || n < v.size()) return -14;
  std::memcpy(out, v.data(), v.size() * 4);
  return 0;
}
// Returns the number of generated tokens (<= max_new) or a negative error code.
int boracle_generate(void* h, const uint32_t* prompt, uint32_t n_prompt, uint32_t max_new, uint32_t* out, float* gaps,
                     int stop_at_eos) {
  BONSAI_TRY
  std::vector<uint32_t> p(prompt, prompt + n_prompt);
  std::vector<float> g;
  std::vector<uint32_t> r = static_cast<OracleModel*>(h)->generate_greedy(p, max_new, gaps ? &g : nullptr, stop_at_eos != 0);
  for (size_t i = 0; i < r.size(); ++i) out[i] = r[i];
  if (gaps) for (size_t i = 0; i < g.size() && i < max_new; ++i) gaps[i] = g[i];
  return static_cast<int>(r.size());
  BONSAI_CATCH_INT
}

// ---- synthetic checkpoints ------------------------------------------------------------------
int bonsai_write_synthetic(const char* path, const uint32_t* cfg_u32, const float* cfg_f32, const char* name,
                           uint32_t weight_type, int tied, uint64_t seed, int llm_keys) {
  BONSAI_TRY
  SyntheticSpec s;
  s.cfg.hidden = cfg_u32[0];
  s.cfg.inter = cfg_u32[1];
  s.cfg.layers = cfg_u32[2];
  s.cfg.heads = cfg_u32[3];
  s.cfg.kv_heads = cfg_u32[4];
  s.cfg.head_dim = cfg_u32[5];
  s.cfg.vocab = cfg_u32[6];
  s.cfg.context = cfg_u32[7];
  s.cfg.eps = cfg_f32[0];
  s.cfg.rope_base = cfg_f32[1];
  if (name) s.cfg.name = name;
  s.weight_type = weight_type;
  s.tied = tied != 0;
  s.seed = seed;
  s.llm_keys = llm_keys != 0;
  write_synthetic_gguf(path, s);
  return 0;
  BONSAI_CATCH_INT
}

}  // extern "C"
