// A stand-in for jaxlib's xla/ffi/api/ffi.h with just the names csrc/fo_ffi.cc uses, so that the shim
// can be type-checked (g++ -fsyntax-only) on a machine without jaxlib.  Declarations only; it cannot
// run anything.  The signatures follow the published header of XLA's typed FFI.
#pragma once
#include <cstddef>
#include <cstdint>
#include <string>
#include <utility>

namespace xla {
namespace ffi {

enum class DataType { PRED, S8, S16, S32, S64, U8, U16, U32, U64, F16, F32, F64, BF16 };
enum class ErrorCode { kOk, kInvalidArgument, kInternal };

class Error {
 public:
  Error() = default;
  Error(ErrorCode code, std::string message) : code_(code), message_(std::move(message)) {}
  static Error Success() { return Error(); }
  static Error Internal(std::string m) { return Error(ErrorCode::kInternal, std::move(m)); }

 private:
  ErrorCode code_ = ErrorCode::kOk;
  std::string message_;
};

template <typename T>
class ErrorOr {
 public:
  bool has_value() const;
  T& operator*();
  T* operator->();
  Error error() const;
};

class AnyBuffer {
 public:
  void* untyped_data() const;
  size_t element_count() const;
  DataType element_type() const;
};

template <typename T>
class Result {
 public:
  T* operator->() const;
  T& operator*() const;
};

template <typename T>
class Span {
 public:
  size_t size() const;
  const T& operator[](size_t i) const;
};

class RemainingArgs {
 public:
  size_t size() const;
  template <typename T>
  ErrorOr<T> get(size_t index) const;
};

class RemainingRets {
 public:
  size_t size() const;
  template <typename T>
  ErrorOr<Result<T>> get(size_t index) const;
};

template <typename T>
struct PlatformStream {};

class Binding {
 public:
  template <typename T>
  Binding& Ctx() { return *this; }
  Binding& RemainingArgs() { return *this; }
  Binding& RemainingRets() { return *this; }
  template <typename T>
  Binding& Attr(const char*) { return *this; }
};

struct Ffi {
  static Binding Bind() { return Binding(); }
};

}  // namespace ffi
}  // namespace xla

#define XLA_FFI_DEFINE_HANDLER_SYMBOL(symbol, fn, binding)          \
  extern "C" void* symbol(void* call_frame) {                       \
    (void)(binding);                                                \
    (void)&fn;                                                      \
    return call_frame;                                              \
  }
