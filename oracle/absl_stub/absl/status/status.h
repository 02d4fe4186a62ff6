// Two-function stand-in for abseil's Status, only so that the reference's own
// src/core/quants.h compiles into oracle/_ref without abseil-cpp installed.
// Test infrastructure only.
#pragma once
namespace absl {
class Status {
 public:
  bool ok() const { return true; }
};
inline Status OkStatus() { return Status(); }
}  // namespace absl
