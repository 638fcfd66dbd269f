// Status codes and canned errors shared by the runtime, the transports and the
// Python bindings.  Same vocabulary as the reference (bluefog/common/common.h:145-185):
// OK / UNKNOWN_ERROR / PRECONDITION_ERROR / ABORTED / INVALID_ARGUMENT / IN_PROGRESS.
#pragma once
#include <stdexcept>
#include <string>

namespace bfb {

enum class StatusType : int {
  OK = 0,
  UNKNOWN_ERROR = 1,
  PRECONDITION_ERROR = 2,
  ABORTED = 3,
  INVALID_ARGUMENT = 4,
  IN_PROGRESS = 5,
};

class Status {
 public:
  Status() = default;
  static Status OK() { return Status(); }
  static Status UnknownError(std::string m) { return Status(StatusType::UNKNOWN_ERROR, std::move(m)); }
  static Status PreconditionError(std::string m) { return Status(StatusType::PRECONDITION_ERROR, std::move(m)); }
  static Status Aborted(std::string m) { return Status(StatusType::ABORTED, std::move(m)); }
  static Status InvalidArgument(std::string m) { return Status(StatusType::INVALID_ARGUMENT, std::move(m)); }
  static Status InProgress() { return Status(StatusType::IN_PROGRESS, ""); }
  bool ok() const { return type_ == StatusType::OK; }
  bool in_progress() const { return type_ == StatusType::IN_PROGRESS; }
  StatusType type() const { return type_; }
  const std::string& reason() const { return reason_; }

 private:
  Status(StatusType t, std::string m) : type_(t), reason_(std::move(m)) {}
  StatusType type_ = StatusType::OK;
  std::string reason_;
};

// Error mapping used at the Python boundary (reference: bluefog/torch/adapter.cc:260-274):
// PRECONDITION_ERROR / INVALID_ARGUMENT -> ValueError, ABORTED / UNKNOWN -> RuntimeError.
inline void ThrowIfError(const Status& s) {
  switch (s.type()) {
    case StatusType::OK:
    case StatusType::IN_PROGRESS:
      return;
    case StatusType::PRECONDITION_ERROR:
    case StatusType::INVALID_ARGUMENT:
      throw std::invalid_argument(s.reason());
    default:
      throw std::runtime_error(s.reason());
  }
}

inline const char* kNotInitializedError() {
  return "BlueFog-B200 has not been initialized; use bf.init().";
}
inline const char* kShutDownError() {
  return "BlueFog-B200 has been shut down. This was caused by an exception on one of the "
         "ranks or an attempt to run a collective after one of the ranks finished execution.";
}
inline const char* kSuspendError() {
  return "BlueFog-B200 background thread is suspended; call bf.resume() first.";
}
inline std::string DuplicateNameError(const std::string& name) {
  return "Requested to enqueue an operation with the same name as another operation that is "
         "currently in flight: " + name;
}

}  // namespace bfb
