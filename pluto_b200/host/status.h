// Minimal Status / StatusOr for the C++ host adapter.  The reference uses absl::Status with
// exceptions disabled (src/util/status_macros.h:11-38); Abseil is not available to this build, so
// the adapter carries the same codes in a small value type and the same two macros.
#pragma once

#include <optional>
#include <string>
#include <utility>

namespace pluto {

enum class StatusCode { kOk = 0, kCancelled = 1, kInvalidArgument = 3, kResourceExhausted = 8,
                        kUnimplemented = 12, kInternal = 13 };

class Status {
 public:
  Status() = default;
  Status(StatusCode code, std::string message) : code_(code), message_(std::move(message)) {}
  bool ok() const { return code_ == StatusCode::kOk; }
  StatusCode code() const { return code_; }
  const std::string& message() const { return message_; }

 private:
  StatusCode code_ = StatusCode::kOk;
  std::string message_;
};

inline Status OkStatus() { return Status(); }
inline Status InvalidArgumentError(std::string m) { return {StatusCode::kInvalidArgument, std::move(m)}; }
inline Status UnimplementedError(std::string m) { return {StatusCode::kUnimplemented, std::move(m)}; }
inline Status ResourceExhaustedError(std::string m) { return {StatusCode::kResourceExhausted, std::move(m)}; }
inline Status InternalError(std::string m) { return {StatusCode::kInternal, std::move(m)}; }

template <class T>
class StatusOr {
 public:
  StatusOr(Status status) : status_(std::move(status)) {}
  StatusOr(T value) : value_(std::move(value)) {}
  bool ok() const { return status_.ok() && value_.has_value(); }
  const Status& status() const { return status_; }
  T& value() { return *value_; }
  const T& value() const { return *value_; }
  T& operator*() { return *value_; }
  T* operator->() { return &*value_; }

 private:
  Status status_;
  std::optional<T> value_;
};

// Maps a return value of the C ABI (include/pluto_b200.h) to a Status.
Status FromEngine(int code, const char* operation);

}  // namespace pluto

#define PLUTO_RETURN_IF_ERROR(expression)              \
  do {                                                 \
    ::pluto::Status pluto_status_ = (expression);      \
    if (!pluto_status_.ok()) return pluto_status_;     \
  } while (false)

#define PLUTO_CONCAT_INNER_(a, b) a##b
#define PLUTO_CONCAT_(a, b) PLUTO_CONCAT_INNER_(a, b)
#define PLUTO_ASSIGN_OR_RETURN(lhs, expression)                         \
  auto PLUTO_CONCAT_(pluto_or_, __LINE__) = (expression);               \
  if (!PLUTO_CONCAT_(pluto_or_, __LINE__).ok())                         \
    return PLUTO_CONCAT_(pluto_or_, __LINE__).status();                 \
  lhs = std::move(PLUTO_CONCAT_(pluto_or_, __LINE__).value())
