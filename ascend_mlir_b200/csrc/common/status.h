// Error value used across the host runtime: empty message = success.
#pragma once

#include <string>
#include <utility>

namespace afir {

class Status {
public:
  Status() = default;
  static Status success() { return Status(); }
  static Status error(std::string message) {
    Status s;
    s.failed_ = true;
    s.message_ = std::move(message);
    return s;
  }
  bool ok() const { return !failed_; }
  explicit operator bool() const { return !failed_; }
  const std::string &message() const { return message_; }
  // Prefixes the message with a pipeline stage tag such as "[cuda:kernel_launch] ".
  Status withStage(const std::string &stage) const {
    if (!failed_) return *this;
    return Status::error("[" + stage + "] " + message_);
  }

private:
  bool failed_ = false;
  std::string message_;
};

} // namespace afir
