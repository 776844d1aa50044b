// Error model of the host library.
//
// One exception type with a stable numeric code and a retryable bit, the same split the
// reference makes between its error enum, `error_code()` and `is_retryable()`
// (reference: crates/oxibonsai-core/src/error.rs:10-92).  The C ABI converts every
// exception into a negative return code plus a thread-local message.
#pragma once
#include <stdexcept>
#include <string>

namespace bonsai {

enum class ErrorCode : int {
  Ok = 0,
  InvalidMagic = 1,
  UnsupportedVersion = 2,
  UnexpectedEof = 3,
  InvalidMetadataType = 4,
  InvalidString = 5,
  LimitExceeded = 6,
  UnsupportedQuantType = 7,
  TensorNotFound = 8,
  MissingMetadata = 9,
  ShapeMismatch = 10,
  NotBlockAligned = 11,
  Io = 12,
  InvalidArgument = 13,
  BufferTooSmall = 14,
  Unsupported = 15,
  Timeout = 16,   // retryable
  Busy = 17,      // retryable
  Internal = 18,
};

inline const char* error_code_name(ErrorCode c) {
  switch (c) {
    case ErrorCode::Ok: return "ok";
    case ErrorCode::InvalidMagic: return "invalid_magic";
    case ErrorCode::UnsupportedVersion: return "unsupported_version";
    case ErrorCode::UnexpectedEof: return "unexpected_eof";
    case ErrorCode::InvalidMetadataType: return "invalid_metadata_type";
    case ErrorCode::InvalidString: return "invalid_string";
    case ErrorCode::LimitExceeded: return "limit_exceeded";
    case ErrorCode::UnsupportedQuantType: return "unsupported_quant_type";
    case ErrorCode::TensorNotFound: return "tensor_not_found";
    case ErrorCode::MissingMetadata: return "missing_metadata";
    case ErrorCode::ShapeMismatch: return "shape_mismatch";
    case ErrorCode::NotBlockAligned: return "not_block_aligned";
    case ErrorCode::Io: return "io";
    case ErrorCode::InvalidArgument: return "invalid_argument";
    case ErrorCode::BufferTooSmall: return "buffer_too_small";
    case ErrorCode::Unsupported: return "unsupported";
    case ErrorCode::Timeout: return "timeout";
    case ErrorCode::Busy: return "busy";
    case ErrorCode::Internal: return "internal";
  }
  return "unknown";
}

inline bool error_is_retryable(ErrorCode c) {
  return c == ErrorCode::Timeout || c == ErrorCode::Busy || c == ErrorCode::Io;
}

class BonsaiError : public std::runtime_error {
 public:
  BonsaiError(ErrorCode code, const std::string& what) : std::runtime_error(what), code_(code) {}
  ErrorCode code() const { return code_; }
  bool retryable() const { return error_is_retryable(code_); }

 private:
  ErrorCode code_;
};

[[noreturn]] inline void fail(ErrorCode c, const std::string& msg) { throw BonsaiError(c, msg); }

}  // namespace bonsai
