#include "oracle.hpp"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <thread>

#include "../core/blocks.hpp"
#include "../core/kquants.hpp"

namespace bonsai {

namespace {

// Splits [0, n) over hardware threads.  Each index is processed by exactly one thread with the
// same arithmetic as a serial loop, so results do not depend on the thread count.
template <typename F>
void parallel_for(uint64_t n, uint64_t min_chunk, F&& fn) {
  unsigned hw = std::thread::hardware_concurrency();
  if (hw == 0) hw = 1;
  uint64_t nthreads = std::min<uint64_t>(hw, (n + min_chunk - 1) / min_chunk);
  if (nthreads <= 1) {
    fn(0, n);
    return;
  }
  std::vector<std::thread> th;
  uint64_t per = (n + nthreads - 1) / nthreads;
  for (uint64_t t = 0; t < nthreads; ++t) {
    uint64_t a = t * per, b = std::min(n, a + per);
    if (a >= b) break;
    th.emplace_back([&fn, a, b] { fn(a, b); });
  }
  for (auto& t : th) t.join();
}

inline float row_dot_tq2(const uint8_t* row, uint64_t nblk, const float* x) {
  float sum = 0.0f;
  for (uint64_t b = 0; b < nblk; ++b, row += kTq2Bytes, x += kTq2Block) {
    float d = f16_to_f32(ld_u16(row + 32));
    float bs = 0.0f;
    for (int byte = 0; byte < 32; ++byte) {
      uint32_t q = row[byte];
      for (int lane = 0; lane < 4; ++lane) {
        float w = (float)tq2_decode((q >> (2 * lane)) & 3);
        bs += w * x[byte * 4 + lane];
      }
    }
    sum += d * bs;
  }
  return sum;
}

inline float row_dot_tq2_256(const uint8_t* row, uint64_t nblk, const float* x) {
  float sum = 0.0f;
  for (uint64_t b = 0; b < nblk; ++b, row += kTq2LBytes, x += kTq2LBlock) {
    float d = f16_to_f32(ld_u16(row + 64));
    float bs = 0.0f;
    for (int j = 0; j < kTq2LBlock; ++j) bs += (float)tq2_decode((row[j >> 2] >> (2 * (j & 3))) & 3) * x[j];
    sum += d * bs;
  }
  return sum;
}

inline float row_dot_q1(const uint8_t* row, uint64_t nblk, const float* x) {
  float sum = 0.0f;
  for (uint64_t b = 0; b < nblk; ++b, row += kQ1Bytes, x += kQ1Block) {
    float d = f16_to_f32(ld_u16(row));
    const uint8_t* qs = row + 2;
    float bs = 0.0f;
    for (int j = 0; j < kQ1Block; ++j) {
      float s = ((qs[j >> 3] >> (j & 7)) & 1) ? 1.0f : -1.0f;
      bs += s * x[j];
    }
    sum += d * bs;
  }
  return sum;
}

template <int BLOCK, int BYTES, typename DQ>
inline float row_dot_generic(const uint8_t* row, uint64_t nblk, const float* x, DQ dq) {
  float sum = 0.0f;
  float tmp[BLOCK];
  for (uint64_t b = 0; b < nblk; ++b, row += BYTES, x += BLOCK) {
    dq(row, tmp);
    for (int j = 0; j < BLOCK; ++j) sum += tmp[j] * x[j];
  }
  return sum;
}

uint64_t row_bytes(uint32_t type, uint64_t cols) {
  TypeTraits t;
  if (!tensor_type_traits(type, &t)) fail(ErrorCode::UnsupportedQuantType, "unsupported matrix type " + std::to_string(type));
  if (cols % t.block_elems != 0)
    fail(ErrorCode::NotBlockAligned, "row length " + std::to_string(cols) + " is not a multiple of the block size " + std::to_string(t.block_elems));
  return cols / t.block_elems * t.block_bytes;
}

}  // namespace

void cpu_gemv(const MatrixRef& w, const float* x, float* out) {
  uint64_t rb = row_bytes(w.type, w.cols);
  uint64_t cols = w.cols;
  const uint8_t* base = w.data;
  uint32_t type = w.type;
  parallel_for(w.rows, 64, [=](uint64_t r0, uint64_t r1) {
    for (uint64_t r = r0; r < r1; ++r) {
      const uint8_t* row = base + r * rb;
      float s = 0.0f;
      switch (type) {
        case 42: s = row_dot_tq2(row, cols / 128, x); break;
        case 41: s = row_dot_q1(row, cols / 128, x); break;
        case 35: s = row_dot_tq2_256(row, cols / 256, x); break;
        case 0: {
          const float* wr = reinterpret_cast<const float*>(row);
          for (uint64_t k = 0; k < cols; ++k) s += wr[k] * x[k];
          break;
        }
        case 1: {
          for (uint64_t k = 0; k < cols; ++k) s += f16_to_f32(ld_u16(row + 2 * k)) * x[k];
          break;
        }
        case 30: {
          for (uint64_t k = 0; k < cols; ++k) s += bf16_to_f32(ld_u16(row + 2 * k)) * x[k];
          break;
        }
        case 2: s = row_dot_generic<32, 18>(row, cols / 32, x, [](const uint8_t* p, float* o) { dequant_q4_0(p, 1, o); }); break;
        case 8: s = row_dot_generic<32, 34>(row, cols / 32, x, [](const uint8_t* p, float* o) { dequant_q8_0(p, 1, o); }); break;
        case 43: s = row_dot_generic<32, 34>(row, cols / 32, x, [](const uint8_t* p, float* o) { dequant_fp8(p, 1, o, false); }); break;
        case 44: s = row_dot_generic<32, 34>(row, cols / 32, x, [](const uint8_t* p, float* o) { dequant_fp8(p, 1, o, true); }); break;
        case 10: s = row_dot_generic<256, 84>(row, cols / 256, x, [](const uint8_t* p, float* o) { dequant_q2k(p, 1, o); }); break;
        case 11: s = row_dot_generic<256, 110>(row, cols / 256, x, [](const uint8_t* p, float* o) { dequant_q3k(p, 1, o); }); break;
        case 12: s = row_dot_generic<256, 144>(row, cols / 256, x, [](const uint8_t* p, float* o) { dequant_q4k(p, 1, o); }); break;
        case 13: s = row_dot_generic<256, 176>(row, cols / 256, x, [](const uint8_t* p, float* o) { dequant_q5k(p, 1, o); }); break;
        case 14: s = row_dot_generic<256, 210>(row, cols / 256, x, [](const uint8_t* p, float* o) { dequant_q6k(p, 1, o); }); break;
        case 15: s = row_dot_generic<256, 292>(row, cols / 256, x, [](const uint8_t* p, float* o) { dequant_q8k(p, 1, o); }); break;
        default: fail(ErrorCode::UnsupportedQuantType, "cpu_gemv: unsupported type " + std::to_string(type));
      }
      out[r] = s;
    }
  });
}

void cpu_dequant_rows(const MatrixRef& w, uint64_t row0, uint64_t nrows, float* out) {
  uint64_t rb = row_bytes(w.type, w.cols);
  if (row0 + nrows > w.rows) fail(ErrorCode::InvalidArgument, "row range out of bounds");
  for (uint64_t r = 0; r < nrows; ++r) {
    const uint8_t* row = w.data + (row0 + r) * rb;
    float* o = out + r * w.cols;
    switch (w.type) {
      case 42: dequant_tq2(row, w.cols / 128, o); break;
      case 41: dequant_q1(row, w.cols / 128, o); break;
      case 35: dequant_tq2_256(row, w.cols / 256, o); break;
      case 0: std::memcpy(o, row, w.cols * 4); break;
      case 1: for (uint64_t k = 0; k < w.cols; ++k) o[k] = f16_to_f32(ld_u16(row + 2 * k)); break;
      case 30: for (uint64_t k = 0; k < w.cols; ++k) o[k] = bf16_to_f32(ld_u16(row + 2 * k)); break;
      case 2: dequant_q4_0(row, w.cols / 32, o); break;
      case 8: dequant_q8_0(row, w.cols / 32, o); break;
      case 43: dequant_fp8(row, w.cols / 32, o, false); break;
      case 44: dequant_fp8(row, w.cols / 32, o, true); break;
      case 10: dequant_q2k(row, w.cols / 256, o); break;
      case 11: dequant_q3k(row, w.cols / 256, o); break;
      case 12: dequant_q4k(row, w.cols / 256, o); break;
      case 13: dequant_q5k(row, w.cols / 256, o); break;
      case 14: dequant_q6k(row, w.cols / 256, o); break;
      case 15: dequant_q8k(row, w.cols / 256, o); break;
      default: fail(ErrorCode::UnsupportedQuantType, "cpu_dequant_rows: unsupported type " + std::to_string(w.type));
    }
  }
}

void cpu_rmsnorm(const float* x, const float* w, float* out, size_t n, float eps) {
  float ss = 0.0f;
  for (size_t i = 0; i < n; ++i) ss += x[i] * x[i];
  float inv = 1.0f / std::sqrt(ss / (float)n + eps);
  for (size_t i = 0; i < n; ++i) out[i] = w[i] * x[i] * inv;
}

void cpu_rope_halfsplit(float* x, size_t head_dim, uint32_t pos, float base) {
  size_t half = head_dim / 2;
  for (size_t i = 0; i < half; ++i) {
    float freq = 1.0f / std::pow(base, 2.0f * (float)i / (float)head_dim);
    float ang = (float)pos * freq;
    float c = std::cos(ang), s = std::sin(ang);
    float x0 = x[i], x1 = x[half + i];
    x[i] = x0 * c - x1 * s;
    x[half + i] = x0 * s + x1 * c;
  }
}

void cpu_swiglu(const float* gate, const float* up, float* out, size_t n) {
  for (size_t i = 0; i < n; ++i) out[i] = gate[i] / (1.0f + std::exp(-gate[i])) * up[i];
}

int cpu_argmax_last(const float* x, size_t n) {
  size_t best = 0;
  for (size_t i = 1; i < n; ++i)
    if (!(x[i] < x[best])) best = i;  // ties move to the later index
  return (int)best;
}

// ---------------------------------------------------------------------------------------------
// model
// ---------------------------------------------------------------------------------------------
const float* OracleModel::norm_vector(const GgufFile& f, const std::string& name, uint64_t n) {
  int idx = f.tensor_index(name);
  if (idx < 0) fail(ErrorCode::TensorNotFound, "missing tensor " + name);
  const TensorInfo& ti = f.tensors[idx];
  if (ti.n_elements() != n) fail(ErrorCode::ShapeMismatch, name + ": expected " + std::to_string(n) + " elements");
  const uint8_t* p = f.tensor_data(idx);
  if (ti.type == 0 && reinterpret_cast<uintptr_t>(p) % 4 == 0) return reinterpret_cast<const float*>(p);
  owned_f32_.emplace_back(n);
  MatrixRef m{p, ti.type, 1, n};
  cpu_dequant_rows(m, 0, 1, owned_f32_.back().data());
  return owned_f32_.back().data();
}

MatrixRef OracleModel::matrix(const GgufFile& f, const std::string& name, uint64_t rows, uint64_t cols) {
  int idx = f.tensor_index(name);
  if (idx < 0) fail(ErrorCode::TensorNotFound, "missing tensor " + name);
  const TensorInfo& ti = f.tensors[idx];
  if (ti.dims.size() != 2 || ti.dims[0] != cols || ti.dims[1] != rows)
    fail(ErrorCode::ShapeMismatch, name + ": expected [" + std::to_string(cols) + ", " + std::to_string(rows) + "]");
  row_bytes(ti.type, cols);
  return MatrixRef{f.tensor_data(idx), ti.type, rows, cols};
}

OracleModel::OracleModel(const GgufFile& f, uint32_t max_seq) : cfg_(config_from_gguf(f)), max_seq_(max_seq) {
  const Qwen3Config& c = cfg_;
  uint64_t qd = (uint64_t)c.heads * c.head_dim, kvd = (uint64_t)c.kv_heads * c.head_dim;
  embd_ = matrix(f, "token_embd.weight", c.vocab, c.hidden);
  if (f.tensor_index("output.weight") >= 0) lm_head_ = matrix(f, "output.weight", c.vocab, c.hidden);
  else lm_head_ = embd_;  // tied checkpoint without a duplicate
  out_norm_ = norm_vector(f, "output_norm.weight", c.hidden);
  owned_f32_.reserve(4 * c.layers + 4);
  layers_.resize(c.layers);
  for (uint32_t l = 0; l < c.layers; ++l) {
    std::string p = "blk." + std::to_string(l) + ".";
    Layer& L = layers_[l];
    L.wq = matrix(f, p + "attn_q.weight", qd, c.hidden);
    L.wk = matrix(f, p + "attn_k.weight", kvd, c.hidden);
    L.wv = matrix(f, p + "attn_v.weight", kvd, c.hidden);
    L.wo = matrix(f, p + "attn_output.weight", c.hidden, qd);
    L.wgate = matrix(f, p + "ffn_gate.weight", c.inter, c.hidden);
    L.wup = matrix(f, p + "ffn_up.weight", c.inter, c.hidden);
    L.wdown = matrix(f, p + "ffn_down.weight", c.hidden, c.inter);
    L.attn_norm = norm_vector(f, p + "attn_norm.weight", c.hidden);
    L.ffn_norm = norm_vector(f, p + "ffn_norm.weight", c.hidden);
    L.q_norm = norm_vector(f, p + "attn_q_norm.weight", c.head_dim);
    L.k_norm = norm_vector(f, p + "attn_k_norm.weight", c.head_dim);
  }
  size_t kv = (size_t)c.layers * c.kv_heads * max_seq_ * c.head_dim;
  kcache_.assign(kv, 0.0f);
  vcache_.assign(kv, 0.0f);
  x_.resize(c.hidden);
  normed_.resize(c.hidden);
  q_.resize(qd);
  k_.resize(kvd);
  v_.resize(kvd);
  attn_.resize(qd);
  proj_.resize(std::max<uint64_t>(c.hidden, 1));
  gate_.resize(c.inter);
  up_.resize(c.inter);
  act_.resize(c.inter);
}

void OracleModel::forward(uint32_t token, uint32_t pos, float* logits) {
  const Qwen3Config& c = cfg_;
  if (token >= c.vocab) fail(ErrorCode::InvalidArgument, "token id out of range");
  if (pos >= max_seq_) fail(ErrorCode::InvalidArgument, "position exceeds max_seq");
  const uint32_t hd = c.head_dim, nq = c.heads, nkv = c.kv_heads, group = nq / nkv;
  cpu_dequant_rows(embd_, token, 1, x_.data());
  const float scale = 1.0f / std::sqrt((float)hd);
  for (uint32_t l = 0; l < c.layers; ++l) {
    Layer& L = layers_[l];
    cpu_rmsnorm(x_.data(), L.attn_norm, normed_.data(), c.hidden, c.eps);
    cpu_gemv(L.wq, normed_.data(), q_.data());
    cpu_gemv(L.wk, normed_.data(), k_.data());
    cpu_gemv(L.wv, normed_.data(), v_.data());
    for (uint32_t h = 0; h < nq; ++h) {
      float* qh = q_.data() + (size_t)h * hd;
      cpu_rmsnorm(qh, L.q_norm, qh, hd, c.eps);
      cpu_rope_halfsplit(qh, hd, pos, c.rope_base);
    }
    for (uint32_t h = 0; h < nkv; ++h) {
      float* kh = k_.data() + (size_t)h * hd;
      cpu_rmsnorm(kh, L.k_norm, kh, hd, c.eps);
      cpu_rope_halfsplit(kh, hd, pos, c.rope_base);
      size_t off = (((size_t)l * nkv + h) * max_seq_ + pos) * hd;
      std::memcpy(&kcache_[off], kh, hd * 4);
      std::memcpy(&vcache_[off], v_.data() + (size_t)h * hd, hd * 4);
    }
    // causal GQA, online softmax in position order
    parallel_for(nq, 1, [&](uint64_t h0, uint64_t h1) {
      std::vector<float> acc(hd);
      for (uint64_t h = h0; h < h1; ++h) {
        const float* qh = q_.data() + h * hd;
        size_t kvh = h / group;
        const float* kb = &kcache_[((size_t)l * nkv + kvh) * max_seq_ * hd];
        const float* vb = &vcache_[((size_t)l * nkv + kvh) * max_seq_ * hd];
        float m = -INFINITY, sum = 0.0f;
        std::fill(acc.begin(), acc.end(), 0.0f);
        for (uint32_t t = 0; t <= pos; ++t) {
          const float* kt = kb + (size_t)t * hd;
          float s = 0.0f;
          for (uint32_t d = 0; d < hd; ++d) s += qh[d] * kt[d];
          s *= scale;
          if (s > m) {
            float r = (m == -INFINITY) ? 0.0f : std::exp(m - s);
            sum *= r;
            for (uint32_t d = 0; d < hd; ++d) acc[d] *= r;
            m = s;
          }
          float e = std::exp(s - m);
          sum += e;
          const float* vt = vb + (size_t)t * hd;
          for (uint32_t d = 0; d < hd; ++d) acc[d] += e * vt[d];
        }
        float inv = sum > 0.0f ? 1.0f / sum : 0.0f;
        float* o = attn_.data() + h * hd;
        for (uint32_t d = 0; d < hd; ++d) o[d] = acc[d] * inv;
      }
    });
    cpu_gemv(L.wo, attn_.data(), proj_.data());
    for (uint32_t i = 0; i < c.hidden; ++i) x_[i] += proj_[i];
    cpu_rmsnorm(x_.data(), L.ffn_norm, normed_.data(), c.hidden, c.eps);
    cpu_gemv(L.wgate, normed_.data(), gate_.data());
    cpu_gemv(L.wup, normed_.data(), up_.data());
    cpu_swiglu(gate_.data(), up_.data(), act_.data(), c.inter);
    cpu_gemv(L.wdown, act_.data(), proj_.data());
    for (uint32_t i = 0; i < c.hidden; ++i) x_[i] += proj_[i];
    if (!layer_hidden_.empty()) std::memcpy(&layer_hidden_[(size_t)l * c.hidden], x_.data(), (size_t)c.hidden * 4);
  }
  cpu_rmsnorm(x_.data(), out_norm_, normed_.data(), c.hidden, c.eps);
  if (logits) cpu_gemv(lm_head_, normed_.data(), logits);
}

std::vector<uint32_t> OracleModel::generate_greedy(const std::vector<uint32_t>& prompt, uint32_t max_new,
                                                   std::vector<float>* gaps, bool stop_at_eos) {
  std::vector<uint32_t> out;
  if (prompt.empty()) return out;
  std::vector<float> logits(cfg_.vocab);
  uint32_t pos = 0;
  for (uint32_t t : prompt) forward(t, pos++, logits.data());
  for (uint32_t step = 0; step < max_new && pos < max_seq_; ++step) {
    int best = cpu_argmax_last(logits.data(), logits.size());
    if (gaps) {
      float second = -INFINITY;
      for (size_t i = 0; i < logits.size(); ++i)
        if ((int)i != best && logits[i] > second) second = logits[i];
      gaps->push_back(logits[best] - second);
    }
    if (stop_at_eos && (uint32_t)best == kEosToken) break;
    out.push_back((uint32_t)best);
    forward((uint32_t)best, pos++, logits.data());
  }
  return out;
}

// ---------------------------------------------------------------------------------------------
// synthetic checkpoints
// ---------------------------------------------------------------------------------------------
namespace {

struct SplitMix {
  uint64_t s;
  explicit SplitMix(uint64_t seed) : s(seed) {}
  uint64_t next() {
    uint64_t z = (s += 0x9E3779B97F4A7C15ull);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
  }
  double uniform() { return (double)(next() >> 11) * (1.0 / 9007199254740992.0); }
  float normal() {
    double u1 = uniform(), u2 = uniform();
    if (u1 < 1e-300) u1 = 1e-300;
    return (float)(std::sqrt(-2.0 * std::log(u1)) * std::cos(6.283185307179586 * u2));
  }
};

uint64_t mix_seed(uint64_t seed, uint64_t a, uint64_t b) {
  SplitMix m(seed ^ (a * 0xD1B54A32D192ED03ull) ^ (b * 0x8CB92BA72F3D8DD7ull));
  m.next();
  return m.next();
}

std::vector<uint8_t> random_quant_matrix(uint32_t type, uint64_t rows, uint64_t cols, uint64_t seed, uint64_t tid,
                                         float smean, float sstd) {
  uint64_t nblk = cols / 128;
  uint64_t bbytes = type == 42 ? kTq2Bytes : kQ1Bytes;
  std::vector<uint8_t> out(rows * nblk * bbytes);
  parallel_for(rows, 16, [&](uint64_t r0, uint64_t r1) {
    for (uint64_t r = r0; r < r1; ++r) {
      SplitMix rng(mix_seed(seed, tid, r));
      uint8_t* p = out.data() + r * nblk * bbytes;
      for (uint64_t b = 0; b < nblk; ++b, p += bbytes) {
        uint16_t d = f32_to_f16(std::fabs(smean + sstd * rng.normal()));
        if (type == 42) {
          for (int i = 0; i < 32; ++i) {
            uint8_t byte = 0;
            for (int lane = 0; lane < 4; ++lane) {
              uint32_t t = (uint32_t)(rng.next() >> 33) % 3u;  // 0,1,2 -> -1,0,+1
              byte |= (uint8_t)(t << (2 * lane));
            }
            p[i] = byte;
          }
          st_u16(p + 32, d);
        } else {
          st_u16(p, d);
          for (int i = 0; i < 16; i += 8) {
            uint64_t bits = rng.next();
            std::memcpy(p + 2 + i, &bits, 8);
          }
        }
      }
    }
  });
  return out;
}

std::vector<uint8_t> random_f16_matrix(uint64_t rows, uint64_t cols, uint64_t seed, uint64_t tid, float stdv) {
  std::vector<uint8_t> out(rows * cols * 2);
  parallel_for(rows, 16, [&](uint64_t r0, uint64_t r1) {
    for (uint64_t r = r0; r < r1; ++r) {
      SplitMix rng(mix_seed(seed, tid, r));
      uint8_t* p = out.data() + r * cols * 2;
      for (uint64_t k = 0; k < cols; ++k) st_u16(p + 2 * k, f32_to_f16(stdv * rng.normal()));
    }
  });
  return out;
}

}  // namespace

void write_synthetic_gguf(const std::string& path, const SyntheticSpec& spec) {
  const Qwen3Config& c = spec.cfg;
  if (spec.weight_type != 41 && spec.weight_type != 42) fail(ErrorCode::InvalidArgument, "weight_type must be 41 (Q1_0_g128) or 42 (TQ2_0_g128)");
  uint64_t qd = (uint64_t)c.heads * c.head_dim, kvd = (uint64_t)c.kv_heads * c.head_dim;
  if (c.hidden % 128 || c.inter % 128 || qd % 128) fail(ErrorCode::NotBlockAligned, "hidden, intermediate and heads*head_dim must be multiples of 128");
  GgufWriter w(3);
  std::string a = spec.llm_keys ? "llm" : c.arch;
  w.add_kv("general.architecture", MetaValue::of_str(c.arch));
  w.add_kv("general.name", MetaValue::of_str(c.name));
  w.add_kv(a + ".embedding_length", MetaValue::of_u32(c.hidden));
  w.add_kv(a + ".block_count", MetaValue::of_u32(c.layers));
  w.add_kv(a + ".attention.head_count", MetaValue::of_u32(c.heads));
  w.add_kv(a + ".attention.head_count_kv", MetaValue::of_u32(c.kv_heads));
  w.add_kv(a + ".attention.key_length", MetaValue::of_u32(c.head_dim));
  w.add_kv(a + ".feed_forward_length", MetaValue::of_u32(c.inter));
  w.add_kv(a + ".vocab_size", MetaValue::of_u32(c.vocab));
  w.add_kv(a + ".context_length", MetaValue::of_u32(c.context));
  w.add_kv(a + ".attention.layer_norm_rms_epsilon", MetaValue::of_f32(c.eps));
  w.add_kv(a + ".rope.freq_base", MetaValue::of_f32(c.rope_base));
  w.add_kv("bonsai.synthetic_seed", MetaValue::of_u64(spec.seed));

  uint64_t tid = 0;
  auto ones = [&](const std::string& name, uint64_t n) {
    std::vector<float> v(n, 1.0f);
    w.add_tensor(name, {n}, 0, reinterpret_cast<const uint8_t*>(v.data()), n * 4, true);
  };
  auto qmat = [&](const std::string& name, uint64_t rows, uint64_t cols) {
    std::vector<uint8_t> d = random_quant_matrix(spec.weight_type, rows, cols, spec.seed, ++tid, spec.scale_mean, spec.scale_std);
    w.add_tensor(name, {cols, rows}, spec.weight_type, d.data(), d.size(), true);
  };
  std::vector<uint8_t> embd = random_f16_matrix(c.vocab, c.hidden, spec.seed, ++tid, spec.embd_std);
  w.add_tensor("token_embd.weight", {c.hidden, c.vocab}, 1, embd.data(), embd.size(), false);
  ones("output_norm.weight", c.hidden);
  std::vector<uint8_t> head;
  if (spec.tied) {
    w.add_tensor("output.weight", {c.hidden, c.vocab}, 1, embd.data(), embd.size(), false);
  } else {
    head = random_f16_matrix(c.vocab, c.hidden, spec.seed, ++tid, spec.embd_std);
    w.add_tensor("output.weight", {c.hidden, c.vocab}, 1, head.data(), head.size(), false);
  }
  for (uint32_t l = 0; l < c.layers; ++l) {
    std::string p = "blk." + std::to_string(l) + ".";
    ones(p + "attn_norm.weight", c.hidden);
    qmat(p + "attn_q.weight", qd, c.hidden);
    qmat(p + "attn_k.weight", kvd, c.hidden);
    qmat(p + "attn_v.weight", kvd, c.hidden);
    qmat(p + "attn_output.weight", c.hidden, qd);
    ones(p + "attn_q_norm.weight", c.head_dim);
    ones(p + "attn_k_norm.weight", c.head_dim);
    ones(p + "ffn_norm.weight", c.hidden);
    qmat(p + "ffn_gate.weight", c.inter, c.hidden);
    qmat(p + "ffn_up.weight", c.inter, c.hidden);
    qmat(p + "ffn_down.weight", c.hidden, c.inter);
  }
  w.write(path);
}

}  // namespace bonsai
