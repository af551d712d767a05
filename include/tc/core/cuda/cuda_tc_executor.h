// CudaTcExecutor — what tc::compile<CudaBackend> returns (the reference's
// tc/core/cuda/cuda_tc_executor.h:27-66).  Holds one immutable tcb200 plan per matched launch;
// run() enqueues them in statement order on the caller's stream of the current device.
#pragma once

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
  // Runs between two device events and synchronises; kernelRuntime is the device time of all
  // launches of the def.
  ProfilingInfo profileUnchecked(const std::vector<const void*>& inputs,
                                 const std::vector<void*>& outputs) const;

  const Grid& grid() const { return grid_; }
  const Block& block() const { return block_; }
  size_t numLaunches() const { return plans_.size(); }
  const std::vector<MatchedLaunch>& launches() const { return launches_; }
  const std::vector<tcb200_tile_t>& tiles() const { return tiles_; }
  int device() const { return device_; }

 private:
  std::vector<MatchedLaunch> launches_;
  std::vector<tcb200_tile_t> tiles_;
  std::vector<tcb200_plan_t*> plans_;
  Grid grid_;
  Block block_;
  int device_;
};

}  // namespace tc
