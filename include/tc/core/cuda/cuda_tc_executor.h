// CudaTcExecutor — what tc::compile<CudaBackend> returns (the reference's
// tc/core/cuda/cuda_tc_executor.h:27-66).  Holds, per device, one immutable tcb200 plan per matched launch;
// run() enqueues them in statement order on the caller's stream of the CURRENT device.  The plans of a device
// are created the first time the executor runs there, under a lock, the way the reference loads its module
// lazily per device (tc/core/cuda/cuda_rtc.cc:308-329): one executor may be run from several host threads,
// each bound to its own device (tc/autotuner/autotuner-inl.h:291-295).
#pragma once

#include <array>
#include <atomic>
#include <mutex>
#include <string>
#include <vector>

#include "tc/core/cuda/cuda_backend.h"
#include "tc/core/tc_executor.h"

namespace tc {

class CudaTcExecutor : public TcExecutor<CudaBackend> {
 public:
  CudaTcExecutor(const std::vector<TensorInfo>& inputsInfo, const std::vector<TensorInfo>& outputsInfo,
                 const DefAnalysis& def, const CudaCompilationResult& result);
  ~CudaTcExecutor();

  // No shape checks: the caller guarantees the pointers match the compiled shapes.
  void uncheckedRun(const std::vector<const void*>& inputs, const std::vector<void*>& outputs,
                    CudaBackend::RuntimeInformation info = {}) const;
  // Runs between two device events and synchronises; kernelRuntime is the device time of all launches of
  // the def.  A def that takes less than ~100 us is then replayed from a captured graph, enough times to
  // fill a window of ~200 us, and the time per run of that window is reported (a 4 us kernel timed with one
  // event pair measures the host's launch rate); defs that accumulate into their outputs ("+=" without "!")
  // are never run more than once.  Throws if a kernel's bounded wait gave up during the runs.
  ProfilingInfo profileUnchecked(const std::vector<const void*>& inputs,
                                 const std::vector<void*>& outputs) const;
  // Waits for `stream` of the current device and throws std::runtime_error if any launch of this executor
  // on that device reported a device-side wait that gave up since the last check.
  void checkDeviceStatus(tcb200_stream_t stream = nullptr) const;

  const Grid& grid() const { return grid_; }
  const Block& block() const { return block_; }
  size_t numLaunches() const { return launches_.size(); }
  const std::vector<MatchedLaunch>& launches() const { return launches_; }
  const std::vector<tcb200_tile_t>& tiles() const { return tiles_; }
  // the device the executor was compiled on (its plans exist from the start there)
  int device() const { return device_; }

 private:
  struct DeviceState {
    std::vector<tcb200_plan_t*> plans;
    int* status = nullptr;  // device word the kernels' bounded waits report into
  };
  static constexpr int kMaxDevices = 64;
  const DeviceState& stateForCurrentDevice() const;

  std::vector<MatchedLaunch> launches_;
  std::vector<tcb200_tile_t> tiles_;
  Grid grid_;
  Block block_;
  int device_;
  bool accumulates_ = false;
  mutable std::mutex mu_;
  mutable std::array<std::atomic<DeviceState*>, kMaxDevices> states_;
};

}  // namespace tc
