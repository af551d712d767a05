// Whole-microsecond durations and the {cpuOverhead, kernelRuntime} pair profile() returns
// (the reference's tc/core/utils/time.h:21-80).  profileUnchecked additionally keeps the
// sub-microsecond CUDA-event time: three of the five benchmark kernels run in 1-100 us.
#pragma once

#include <chrono>
#include <cstddef>
#include <cstdint>

namespace tc {

struct Duration {
 private:
  explicit Duration(std::chrono::microseconds us) : val_(us) {}

 public:
  Duration() : val_(0) {}
  Duration(const Duration&) = default;
  Duration& operator=(const Duration&) = default;
  static Duration since(std::chrono::time_point<std::chrono::system_clock> begin) {
    return Duration(std::chrono::duration_cast<std::chrono::microseconds>(
        std::chrono::system_clock::now() - begin));
  }
  static Duration fromMicroSeconds(size_t us) { return Duration(std::chrono::microseconds(us)); }
  size_t toMicroSeconds() const { return (size_t)val_.count(); }
  static Duration zero() { return Duration(std::chrono::microseconds(0)); }
  static Duration max() { return Duration(std::chrono::microseconds::max()); }
  friend Duration operator-(Duration a, const Duration& b) { a.val_ -= b.val_; return a; }
  friend Duration operator+(Duration a, const Duration& b) { a.val_ += b.val_; return a; }
  friend Duration operator/(Duration a, uint32_t d) { return Duration(a.val_ / d); }
  friend Duration operator*(Duration a, uint32_t m) { return Duration(a.val_ * m); }
  friend bool operator>=(const Duration& a, const Duration& b) { return a.val_ >= b.val_; }
  friend bool operator<(const Duration& a, const Duration& b) { return a.val_ < b.val_; }
  friend bool operator==(const Duration& a, const Duration& b) { return a.val_ == b.val_; }

 private:
  std::chrono::microseconds val_;
};

struct ProfilingInfo {
  Duration cpuOverhead;
  Duration kernelRuntime;
  double kernelRuntimeUs = 0.0;  // same measurement, not truncated to whole microseconds
};

}  // namespace tc
