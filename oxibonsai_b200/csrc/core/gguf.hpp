// GGUF v2/v3 container: zero-copy reader, writer and an incremental (streaming) parser.
//
// File layout (little endian): magic u32 "GGUF" | version u32 | tensor_count u64 | kv_count u64 |
// kv_count x { key string, value-type u32, value } | tensor_count x { name string, n_dims u32,
// dims u64 x n (innermost first), type u32, offset u64 } | padding to `general.alignment`
// (default 32) | tensor data.  A string is u64 length + bytes.  Tensor bytes live at
// data_offset + offset and span ceil(n_elements / block) * block_bytes.
// (reference: crates/oxibonsai-core/src/gguf/header.rs:17-81, metadata.rs:15-186,
//  tensor_info.rs:20-186, reader.rs:12-99, writer.rs:212-323, streaming.rs:42-219)
//
// The writer keeps the reference's convention that tensor offsets are a running sum with no
// per-tensor padding; the reader never assumes it and always uses the explicit offsets.
#pragma once
#include <cstdint>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <utility>
#include <vector>

#include "errors.hpp"

namespace bonsai {

constexpr uint32_t kGgufMagic = 0x46554747u;  // "GGUF"
constexpr uint64_t kMaxStringLen = 256ull << 20;
constexpr uint64_t kMaxArrayLen = 16ull << 20;
constexpr uint32_t kDefaultAlignment = 32;

enum class MetaType : uint32_t {
  U8 = 0, I8 = 1, U16 = 2, I16 = 3, U32 = 4, I32 = 5, F32 = 6, Bool = 7, String = 8,
  Array = 9, U64 = 10, I64 = 11, F64 = 12,
};

// Tensor storage types (ids are the on-disk GGUF type ids).
enum class TensorType : uint32_t {
  F32 = 0, F16 = 1, Q4_0 = 2, Q4_1 = 3, Q5_0 = 6, Q5_1 = 7, Q8_0 = 8, Q8_1 = 9,
  Q2_K = 10, Q3_K = 11, Q4_K = 12, Q5_K = 13, Q6_K = 14, Q8_K = 15, BF16 = 30,
  TQ2_0 = 35, Q1_0_g128 = 41, TQ2_0_g128 = 42, F8_E4M3 = 43, F8_E5M2 = 44,
};

struct TypeTraits {
  const char* name;
  uint32_t block_elems;
  uint32_t block_bytes;
};

// Returns false for ids that are not in the table.
bool tensor_type_traits(uint32_t id, TypeTraits* out);
const char* tensor_type_name(uint32_t id);
// Bytes needed to store `n_elements` of type `id`; throws on unknown types.
uint64_t tensor_data_size(uint32_t id, uint64_t n_elements);

struct MetaValue {
  MetaType type = MetaType::U32;
  uint64_t u = 0;   // unsigned / bool payload
  int64_t i = 0;    // signed payload
  double f = 0.0;   // float payload
  std::string s;    // string payload
  MetaType elem_type = MetaType::U32;  // arrays
  std::vector<MetaValue> arr;

  static MetaValue of_u32(uint32_t v) { MetaValue m; m.type = MetaType::U32; m.u = v; return m; }
  static MetaValue of_u64(uint64_t v) { MetaValue m; m.type = MetaType::U64; m.u = v; return m; }
  static MetaValue of_i32(int32_t v) { MetaValue m; m.type = MetaType::I32; m.i = v; return m; }
  static MetaValue of_f32(float v) { MetaValue m; m.type = MetaType::F32; m.f = v; return m; }
  static MetaValue of_f64(double v) { MetaValue m; m.type = MetaType::F64; m.f = v; return m; }
  static MetaValue of_bool(bool v) { MetaValue m; m.type = MetaType::Bool; m.u = v; return m; }
  static MetaValue of_str(std::string v) { MetaValue m; m.type = MetaType::String; m.s = std::move(v); return m; }

  bool is_integer() const;
  // Lossy typed getters (any integer type -> u64 / any numeric -> double).
  bool as_u64(uint64_t* out) const;
  bool as_f64(double* out) const;
};

struct TensorInfo {
  std::string name;
  std::vector<uint64_t> dims;  // innermost first: [in_features, out_features]
  uint32_t type = 0;
  uint64_t offset = 0;  // relative to the data section

  uint64_t n_elements() const {
    uint64_t n = 1;
    for (uint64_t d : dims) n *= d;
    return n;
  }
  uint64_t data_size() const { return tensor_data_size(type, n_elements()); }
};

class GgufFile {
 public:
  // Parses headers over an existing buffer; the buffer must outlive the object.
  static std::unique_ptr<GgufFile> parse(const uint8_t* data, size_t size);
  // mmap()s the file read-only and parses it; the mapping is owned by the object.
  static std::unique_ptr<GgufFile> open(const std::string& path);
  ~GgufFile();

  uint32_t version = 0;
  uint32_t alignment = kDefaultAlignment;
  uint64_t data_offset = 0;
  std::vector<std::pair<std::string, MetaValue>> kv;
  std::vector<TensorInfo> tensors;

  const MetaValue* find(const std::string& key) const;
  int tensor_index(const std::string& name) const;  // -1 if absent
  // Pointer to the tensor's bytes; bounds-checked against the buffer.
  const uint8_t* tensor_data(size_t index, uint64_t* nbytes = nullptr) const;
  const uint8_t* base() const { return base_; }
  size_t size() const { return size_; }
  std::string metadata_json(size_t max_array_items) const;

 private:
  const uint8_t* base_ = nullptr;
  size_t size_ = 0;
  bool owns_map_ = false;
  std::map<std::string, size_t> kv_index_;
  std::map<std::string, size_t> tensor_index_;
  void build_indexes();
  friend class GgufStreamParser;
};

class GgufWriter {
 public:
  explicit GgufWriter(uint32_t version = 3, uint32_t alignment = kDefaultAlignment)
      : version_(version), alignment_(alignment) {}
  void add_kv(const std::string& key, MetaValue v) { kv_.emplace_back(key, std::move(v)); }
  // The bytes are referenced, not copied, unless `copy` is true.
  void add_tensor(const std::string& name, const std::vector<uint64_t>& dims, uint32_t type,
                  const uint8_t* data, uint64_t nbytes, bool copy);
  std::vector<uint8_t> header_bytes() const;  // everything up to and including the pad
  void write(const std::string& path) const;
  std::vector<uint8_t> to_bytes() const;

 private:
  struct Pending {
    TensorInfo info;
    const uint8_t* data;
    uint64_t nbytes;
    std::shared_ptr<std::vector<uint8_t>> owned;
  };
  uint32_t version_, alignment_;
  std::vector<std::pair<std::string, MetaValue>> kv_;
  std::vector<Pending> tensors_;
};

// Incremental parser: feed() arbitrary chunks; once headers are complete the parsed file is
// available and remaining bytes are tensor data counted by data_bytes_seen().
class GgufStreamParser {
 public:
  enum class State { NeedMore, HeaderComplete, Failed };
  State feed(const uint8_t* chunk, size_t n);
  State state() const { return state_; }
  const GgufFile* file() const { return file_.get(); }
  uint64_t bytes_consumed() const { return total_; }
  uint64_t data_bytes_seen() const;
  uint64_t data_bytes_expected() const;
  const std::string& error() const { return error_; }

 private:
  State state_ = State::NeedMore;
  std::vector<uint8_t> buf_;
  std::unique_ptr<GgufFile> file_;
  uint64_t total_ = 0;
  std::string error_;
};

}  // namespace bonsai
