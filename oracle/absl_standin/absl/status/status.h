// Stand-in for absl::Status: a code plus a message, enough for the reference's
// RETURN_IF_ERROR / ASSIGN_OR_RETURN macros and its error constructors.
#pragma once
#include <ostream>
#include <string>
#include <string_view>
#include <utility>
namespace absl {
enum class StatusCode : int {
  kOk = 0, kCancelled = 1, kUnknown = 2, kInvalidArgument = 3, kNotFound = 5,
  kResourceExhausted = 8, kFailedPrecondition = 9, kAborted = 10, kOutOfRange = 11,
  kUnimplemented = 12, kInternal = 13,
};
class Status {
 public:
  Status() = default;
  Status(StatusCode code, std::string_view message) : code_(code), message_(message) {}
  bool ok() const { return code_ == StatusCode::kOk; }
  StatusCode code() const { return code_; }
  std::string_view message() const { return message_; }
  std::string ToString() const {
    return ok() ? "OK" : "error " + std::to_string(static_cast<int>(code_)) + ": " + message_;
  }
 private:
  StatusCode code_ = StatusCode::kOk;
  std::string message_;
};
inline std::ostream& operator<<(std::ostream& out, const Status& s) { return out << s.ToString(); }
inline Status OkStatus() { return Status(); }
inline Status InvalidArgumentError(std::string_view m) { return Status(StatusCode::kInvalidArgument, m); }
inline Status UnimplementedError(std::string_view m) { return Status(StatusCode::kUnimplemented, m); }
inline Status ResourceExhaustedError(std::string_view m) { return Status(StatusCode::kResourceExhausted, m); }
inline Status InternalError(std::string_view m) { return Status(StatusCode::kInternal, m); }
inline Status FailedPreconditionError(std::string_view m) { return Status(StatusCode::kFailedPrecondition, m); }
inline bool IsInvalidArgument(const Status& s) { return s.code() == StatusCode::kInvalidArgument; }
inline bool IsUnimplemented(const Status& s) { return s.code() == StatusCode::kUnimplemented; }
inline bool IsResourceExhausted(const Status& s) { return s.code() == StatusCode::kResourceExhausted; }
inline bool IsInternal(const Status& s) { return s.code() == StatusCode::kInternal; }
inline bool IsFailedPrecondition(const Status& s) { return s.code() == StatusCode::kFailedPrecondition; }
}  // namespace absl
