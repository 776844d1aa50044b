#include "gguf.hpp"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cmath>
#include <cstdio>
#include <sstream>

namespace bonsai {

// ---------------------------------------------------------------------------------------------
// type table
// ---------------------------------------------------------------------------------------------
bool tensor_type_traits(uint32_t id, TypeTraits* out) {
  TypeTraits t{nullptr, 0, 0};
  switch (id) {
    case 0: t = {"F32", 1, 4}; break;
    case 1: t = {"F16", 1, 2}; break;
    case 2: t = {"Q4_0", 32, 18}; break;
    case 3: t = {"Q4_1", 32, 20}; break;
    case 6: t = {"Q5_0", 32, 22}; break;
    case 7: t = {"Q5_1", 32, 24}; break;
    case 8: t = {"Q8_0", 32, 34}; break;
    case 9: t = {"Q8_1", 32, 40}; break;   // f32 scale + f32 sum + 32 bytes, as the reference sizes it (ggml itself uses two f16: 36)
    case 10: t = {"Q2_K", 256, 84}; break;
    case 11: t = {"Q3_K", 256, 110}; break;
    case 12: t = {"Q4_K", 256, 144}; break;
    case 13: t = {"Q5_K", 256, 176}; break;
    case 14: t = {"Q6_K", 256, 210}; break;
    case 15: t = {"Q8_K", 256, 292}; break;
    case 30: t = {"BF16", 1, 2}; break;
    case 35: t = {"TQ2_0", 256, 66}; break;
    case 41: t = {"Q1_0_g128", 128, 18}; break;
    case 42: t = {"TQ2_0_g128", 128, 34}; break;
    case 43: t = {"F8_E4M3", 32, 34}; break;
    case 44: t = {"F8_E5M2", 32, 34}; break;
    default: return false;
  }
  if (out) *out = t;
  return true;
}

const char* tensor_type_name(uint32_t id) {
  TypeTraits t;
  return tensor_type_traits(id, &t) ? t.name : "UNKNOWN";
}

uint64_t tensor_data_size(uint32_t id, uint64_t n) {
  TypeTraits t;
  if (!tensor_type_traits(id, &t)) fail(ErrorCode::UnsupportedQuantType, "unsupported tensor type id " + std::to_string(id));
  uint64_t blocks = (n + t.block_elems - 1) / t.block_elems;
  return blocks * t.block_bytes;
}

// ---------------------------------------------------------------------------------------------
// metadata values
// ---------------------------------------------------------------------------------------------
bool MetaValue::is_integer() const {
  switch (type) {
    case MetaType::U8: case MetaType::I8: case MetaType::U16: case MetaType::I16:
    case MetaType::U32: case MetaType::I32: case MetaType::U64: case MetaType::I64:
      return true;
    default: return false;
  }
}

bool MetaValue::as_u64(uint64_t* out) const {
  switch (type) {
    case MetaType::U8: case MetaType::U16: case MetaType::U32: case MetaType::U64: case MetaType::Bool:
      *out = u; return true;
    case MetaType::I8: case MetaType::I16: case MetaType::I32: case MetaType::I64:
      if (i < 0) return false;
      *out = static_cast<uint64_t>(i); return true;
    default: return false;
  }
}

bool MetaValue::as_f64(double* out) const {
  switch (type) {
    case MetaType::F32: case MetaType::F64: *out = f; return true;
    case MetaType::U8: case MetaType::U16: case MetaType::U32: case MetaType::U64: case MetaType::Bool:
      *out = static_cast<double>(u); return true;
    case MetaType::I8: case MetaType::I16: case MetaType::I32: case MetaType::I64:
      *out = static_cast<double>(i); return true;
    default: return false;
  }
}

// ---------------------------------------------------------------------------------------------
// reader
// ---------------------------------------------------------------------------------------------
namespace {

struct Cursor {
  const uint8_t* p;
  size_t size;
  size_t pos = 0;

  void need(uint64_t n) const {
    if (n > size - pos) fail(ErrorCode::UnexpectedEof, "unexpected end of GGUF data at offset " + std::to_string(pos));
  }
  template <typename T>
  T rd() {
    need(sizeof(T));
    T v;
    std::memcpy(&v, p + pos, sizeof(T));
    pos += sizeof(T);
    return v;
  }
  std::string rd_string() {
    uint64_t len = rd<uint64_t>();
    if (len > kMaxStringLen) fail(ErrorCode::LimitExceeded, "GGUF string longer than 256 MiB");
    need(len);
    std::string s(reinterpret_cast<const char*>(p + pos), static_cast<size_t>(len));
    pos += len;
    return s;
  }
};

MetaValue read_value(Cursor& c, uint32_t type_id, int depth) {
  if (type_id > 12) fail(ErrorCode::InvalidMetadataType, "invalid metadata value type " + std::to_string(type_id));
  MetaValue v;
  v.type = static_cast<MetaType>(type_id);
  switch (v.type) {
    case MetaType::U8: v.u = c.rd<uint8_t>(); break;
    case MetaType::I8: v.i = c.rd<int8_t>(); break;
    case MetaType::U16: v.u = c.rd<uint16_t>(); break;
    case MetaType::I16: v.i = c.rd<int16_t>(); break;
    case MetaType::U32: v.u = c.rd<uint32_t>(); break;
    case MetaType::I32: v.i = c.rd<int32_t>(); break;
    case MetaType::F32: v.f = c.rd<float>(); break;
    case MetaType::Bool: v.u = c.rd<uint8_t>() != 0; break;
    case MetaType::String: v.s = c.rd_string(); break;
    case MetaType::U64: v.u = c.rd<uint64_t>(); break;
    case MetaType::I64: v.i = c.rd<int64_t>(); break;
    case MetaType::F64: v.f = c.rd<double>(); break;
    case MetaType::Array: {
      if (depth > 4) fail(ErrorCode::LimitExceeded, "metadata arrays nested too deeply");
      uint32_t et = c.rd<uint32_t>();
      if (et > 12) fail(ErrorCode::InvalidMetadataType, "invalid array element type " + std::to_string(et));
      uint64_t n = c.rd<uint64_t>();
      if (n > kMaxArrayLen) fail(ErrorCode::LimitExceeded, "metadata array longer than 16 Mi entries");
      // every element takes at least one byte; reject counts the buffer cannot hold
      c.need(n);
      v.elem_type = static_cast<MetaType>(et);
      v.arr.reserve(static_cast<size_t>(n));
      for (uint64_t k = 0; k < n; ++k) v.arr.push_back(read_value(c, et, depth + 1));
      break;
    }
  }
  return v;
}

void parse_headers(Cursor& c, GgufFile& f) {
  uint32_t magic = c.rd<uint32_t>();
  if (magic != kGgufMagic) {
    char b[64];
    std::snprintf(b, sizeof b, "bad GGUF magic 0x%08x", magic);
    fail(ErrorCode::InvalidMagic, b);
  }
  f.version = c.rd<uint32_t>();
  if (f.version != 2 && f.version != 3) fail(ErrorCode::UnsupportedVersion, "unsupported GGUF version " + std::to_string(f.version));
  uint64_t n_tensors = c.rd<uint64_t>();
  uint64_t n_kv = c.rd<uint64_t>();
  if (n_tensors > (1ull << 24) || n_kv > (1ull << 24)) fail(ErrorCode::LimitExceeded, "implausible tensor / kv count");
  f.kv.reserve(static_cast<size_t>(n_kv));
  for (uint64_t k = 0; k < n_kv; ++k) {
    std::string key = c.rd_string();
    uint32_t t = c.rd<uint32_t>();
    f.kv.emplace_back(std::move(key), read_value(c, t, 0));
  }
  f.tensors.reserve(static_cast<size_t>(n_tensors));
  for (uint64_t k = 0; k < n_tensors; ++k) {
    TensorInfo ti;
    ti.name = c.rd_string();
    uint32_t nd = c.rd<uint32_t>();
    if (nd > 8) fail(ErrorCode::LimitExceeded, "tensor with more than 8 dimensions");
    uint64_t total = 1;
    for (uint32_t d = 0; d < nd; ++d) {
      uint64_t dim = c.rd<uint64_t>();
      if (dim != 0 && total > (1ull << 62) / dim) fail(ErrorCode::LimitExceeded, "tensor element count overflows");
      total *= dim;
      ti.dims.push_back(dim);
    }
    ti.type = c.rd<uint32_t>();
    ti.offset = c.rd<uint64_t>();
    f.tensors.push_back(std::move(ti));
  }
  f.alignment = kDefaultAlignment;
  for (auto& e : f.kv) {
    if (e.first == "general.alignment") {
      uint64_t a;
      if (e.second.as_u64(&a) && a > 0 && a <= (1u << 20)) f.alignment = static_cast<uint32_t>(a);
    }
  }
  uint64_t a = f.alignment;
  f.data_offset = (c.pos + a - 1) / a * a;
}

void json_escape(std::ostringstream& o, const std::string& s) {
  o << '"';
  for (unsigned char ch : s) {
    switch (ch) {
      case '"': o << "\\\""; break;
      case '\\': o << "\\\\"; break;
      case '\n': o << "\\n"; break;
      case '\r': o << "\\r"; break;
      case '\t': o << "\\t"; break;
      default:
        if (ch < 0x20) {
          char b[8];
          std::snprintf(b, sizeof b, "\\u%04x", ch);
          o << b;
        } else {
          o << static_cast<char>(ch);
        }
    }
  }
  o << '"';
}

void json_value(std::ostringstream& o, const MetaValue& v, size_t max_items) {
  switch (v.type) {
    case MetaType::U8: case MetaType::U16: case MetaType::U32: case MetaType::U64: o << v.u; break;
    case MetaType::I8: case MetaType::I16: case MetaType::I32: case MetaType::I64: o << v.i; break;
    case MetaType::Bool: o << (v.u ? "true" : "false"); break;
    case MetaType::F32: case MetaType::F64:
      if (std::isfinite(v.f)) {
        char b[40];
        std::snprintf(b, sizeof b, "%.17g", v.f);
        o << b;
      } else {
        o << "null";
      }
      break;
    case MetaType::String: json_escape(o, v.s); break;
    case MetaType::Array: {
      o << '[';
      size_t n = v.arr.size();
      size_t lim = (max_items && n > max_items) ? max_items : n;
      for (size_t k = 0; k < lim; ++k) {
        if (k) o << ',';
        json_value(o, v.arr[k], max_items);
      }
      o << ']';
      break;
    }
  }
}

}  // namespace

void GgufFile::build_indexes() {
  kv_index_.clear();
  tensor_index_.clear();
  for (size_t k = 0; k < kv.size(); ++k) kv_index_.emplace(kv[k].first, k);
  for (size_t k = 0; k < tensors.size(); ++k) tensor_index_.emplace(tensors[k].name, k);
}

std::unique_ptr<GgufFile> GgufFile::parse(const uint8_t* data, size_t size) {
  std::unique_ptr<GgufFile> f(new GgufFile());
  Cursor c{data, size};
  parse_headers(c, *f);
  f->base_ = data;
  f->size_ = size;
  f->build_indexes();
  return f;
}

std::unique_ptr<GgufFile> GgufFile::open(const std::string& path) {
  int fd = ::open(path.c_str(), O_RDONLY);
  if (fd < 0) fail(ErrorCode::Io, "cannot open " + path);
  struct stat st;
  if (fstat(fd, &st) != 0) {
    ::close(fd);
    fail(ErrorCode::Io, "cannot stat " + path);
  }
  size_t size = static_cast<size_t>(st.st_size);
  if (size < 24) {
    ::close(fd);
    fail(ErrorCode::UnexpectedEof, "file too small to be GGUF: " + path);
  }
  void* m = mmap(nullptr, size, PROT_READ, MAP_PRIVATE, fd, 0);
  ::close(fd);
  if (m == MAP_FAILED) fail(ErrorCode::Io, "mmap failed for " + path);
  std::unique_ptr<GgufFile> f;
  try {
    f = parse(static_cast<const uint8_t*>(m), size);
  } catch (...) {
    munmap(m, size);
    throw;
  }
  f->owns_map_ = true;
  return f;
}

GgufFile::~GgufFile() {
  if (owns_map_ && base_) munmap(const_cast<uint8_t*>(base_), size_);
}

const MetaValue* GgufFile::find(const std::string& key) const {
  auto it = kv_index_.find(key);
  return it == kv_index_.end() ? nullptr : &kv[it->second].second;
}

int GgufFile::tensor_index(const std::string& name) const {
  auto it = tensor_index_.find(name);
  return it == tensor_index_.end() ? -1 : static_cast<int>(it->second);
}

const uint8_t* GgufFile::tensor_data(size_t index, uint64_t* nbytes) const {
  if (index >= tensors.size()) fail(ErrorCode::TensorNotFound, "tensor index out of range");
  const TensorInfo& ti = tensors[index];
  uint64_t n = ti.data_size();
  uint64_t start = data_offset + ti.offset;
  if (start < data_offset || start > size_ || n > size_ - start)
    fail(ErrorCode::UnexpectedEof, "tensor '" + ti.name + "' extends past the end of the file");
  if (nbytes) *nbytes = n;
  return base_ + start;
}

std::string GgufFile::metadata_json(size_t max_array_items) const {
  std::ostringstream o;
  o << '{';
  for (size_t k = 0; k < kv.size(); ++k) {
    if (k) o << ',';
    json_escape(o, kv[k].first);
    o << ':';
    json_value(o, kv[k].second, max_array_items);
  }
  o << '}';
  return o.str();
}

// ---------------------------------------------------------------------------------------------
// writer
// ---------------------------------------------------------------------------------------------
namespace {

struct Out {
  std::vector<uint8_t> b;
  template <typename T>
  void wr(T v) {
    size_t n = b.size();
    b.resize(n + sizeof(T));
    std::memcpy(b.data() + n, &v, sizeof(T));
  }
  void wr_string(const std::string& s) {
    wr<uint64_t>(s.size());
    b.insert(b.end(), s.begin(), s.end());
  }
};

void write_value(Out& o, const MetaValue& v) {
  switch (v.type) {
    case MetaType::U8: o.wr<uint8_t>(static_cast<uint8_t>(v.u)); break;
    case MetaType::I8: o.wr<int8_t>(static_cast<int8_t>(v.i)); break;
    case MetaType::U16: o.wr<uint16_t>(static_cast<uint16_t>(v.u)); break;
    case MetaType::I16: o.wr<int16_t>(static_cast<int16_t>(v.i)); break;
    case MetaType::U32: o.wr<uint32_t>(static_cast<uint32_t>(v.u)); break;
    case MetaType::I32: o.wr<int32_t>(static_cast<int32_t>(v.i)); break;
    case MetaType::F32: o.wr<float>(static_cast<float>(v.f)); break;
    case MetaType::Bool: o.wr<uint8_t>(v.u ? 1 : 0); break;
    case MetaType::String: o.wr_string(v.s); break;
    case MetaType::U64: o.wr<uint64_t>(v.u); break;
    case MetaType::I64: o.wr<int64_t>(v.i); break;
    case MetaType::F64: o.wr<double>(v.f); break;
    case MetaType::Array:
      o.wr<uint32_t>(static_cast<uint32_t>(v.elem_type));
      o.wr<uint64_t>(v.arr.size());
      for (auto& e : v.arr) write_value(o, e);
      break;
  }
}

}  // namespace

void GgufWriter::add_tensor(const std::string& name, const std::vector<uint64_t>& dims, uint32_t type,
                            const uint8_t* data, uint64_t nbytes, bool copy) {
  Pending p;
  p.info.name = name;
  p.info.dims = dims;
  p.info.type = type;
  uint64_t expect = p.info.data_size();
  if (expect != nbytes)
    fail(ErrorCode::ShapeMismatch, "tensor '" + name + "': " + std::to_string(nbytes) + " bytes given, " +
                                       std::to_string(expect) + " expected for its shape and type");
  if (copy) {
    p.owned = std::make_shared<std::vector<uint8_t>>(data, data + nbytes);
    p.data = p.owned->data();
  } else {
    p.data = data;
  }
  p.nbytes = nbytes;
  tensors_.push_back(std::move(p));
}

std::vector<uint8_t> GgufWriter::header_bytes() const {
  Out o;
  o.wr<uint32_t>(kGgufMagic);
  o.wr<uint32_t>(version_);
  o.wr<uint64_t>(tensors_.size());
  bool has_align = false;
  for (auto& e : kv_) has_align |= (e.first == "general.alignment");
  bool emit_align = !has_align && alignment_ != kDefaultAlignment;
  o.wr<uint64_t>(kv_.size() + (emit_align ? 1 : 0));
  if (emit_align) {
    o.wr_string("general.alignment");
    o.wr<uint32_t>(static_cast<uint32_t>(MetaType::U32));
    o.wr<uint32_t>(alignment_);
  }
  for (auto& e : kv_) {
    o.wr_string(e.first);
    o.wr<uint32_t>(static_cast<uint32_t>(e.second.type));
    write_value(o, e.second);
  }
  uint64_t off = 0;
  for (auto& t : tensors_) {
    o.wr_string(t.info.name);
    o.wr<uint32_t>(static_cast<uint32_t>(t.info.dims.size()));
    for (uint64_t d : t.info.dims) o.wr<uint64_t>(d);
    o.wr<uint32_t>(t.info.type);
    o.wr<uint64_t>(off);
    off += t.nbytes;  // running sum, no per-tensor padding
  }
  uint64_t a = alignment_;
  for (auto& e : kv_) {
    uint64_t v;
    if (e.first == "general.alignment" && e.second.as_u64(&v) && v > 0) a = v;
  }
  size_t padded = (o.b.size() + a - 1) / a * a;
  o.b.resize(padded, 0);
  return o.b;
}

void GgufWriter::write(const std::string& path) const {
  std::vector<uint8_t> h = header_bytes();
  FILE* fp = std::fopen(path.c_str(), "wb");
  if (!fp) fail(ErrorCode::Io, "cannot create " + path);
  bool ok = std::fwrite(h.data(), 1, h.size(), fp) == h.size();
  for (auto& t : tensors_) {
    if (!ok) break;
    ok = std::fwrite(t.data, 1, t.nbytes, fp) == t.nbytes;
  }
  ok = (std::fclose(fp) == 0) && ok;
  if (!ok) fail(ErrorCode::Io, "short write to " + path);
}

std::vector<uint8_t> GgufWriter::to_bytes() const {
  std::vector<uint8_t> h = header_bytes();
  for (auto& t : tensors_) h.insert(h.end(), t.data, t.data + t.nbytes);
  return h;
}

// ---------------------------------------------------------------------------------------------
// streaming parser
// ---------------------------------------------------------------------------------------------
GgufStreamParser::State GgufStreamParser::feed(const uint8_t* chunk, size_t n) {
  total_ += n;
  if (state_ != State::NeedMore) return state_;
  buf_.insert(buf_.end(), chunk, chunk + n);
  std::unique_ptr<GgufFile> f(new GgufFile());
  try {
    Cursor c{buf_.data(), buf_.size()};
    parse_headers(c, *f);
  } catch (const BonsaiError& e) {
    if (e.code() == ErrorCode::UnexpectedEof) return state_;
    state_ = State::Failed;
    error_ = e.what();
    buf_.clear();
    return state_;
  }
  f->build_indexes();
  file_ = std::move(f);
  state_ = State::HeaderComplete;
  buf_.clear();
  buf_.shrink_to_fit();
  return state_;
}

uint64_t GgufStreamParser::data_bytes_seen() const {
  if (state_ != State::HeaderComplete) return 0;
  return total_ > file_->data_offset ? total_ - file_->data_offset : 0;
}

uint64_t GgufStreamParser::data_bytes_expected() const {
  if (state_ != State::HeaderComplete) return 0;
  uint64_t end = 0;
  for (auto& t : file_->tensors) {
    uint64_t e = t.offset + t.data_size();
    if (e > end) end = e;
  }
  return end;
}

}  // namespace bonsai
