// The backend trait struct the templated API is instantiated with
// (the reference's tc/core/cuda/cuda_backend.h:34-87).
#pragma once

#include <string>
#include <vector>

#include "tc/core/cuda/cuda.h"
#include "tc/core/cuda/cuda_mapping_options.h"
#include "tc/core/kernel_matcher.h"
#include "tc/core/tc_analysis.h"
#include "tc/core/tensor.h"

namespace tc {

// What "compilation" produces here: the matched launches with their resolved tiles.
struct CudaCompilationResult {
  std::string source;           // human-readable description (-> TcExecutor::compiledSource)
  std::string specializedName;  // <tcName>_<size0>_<size1>...
  std::vector<long> parameters; // values of the size symbols, in name order
  Grid grid;                    // geometry of the (last) launch
  Block block;
  std::vector<MatchedLaunch> launches;
  std::vector<tcb200_tile_t> tiles;  // resolved tile per launch
  int device = 0;
};

// Per-call runtime information: the stream to enqueue on (the reference's only field,
// tc/core/cuda/cuda_backend.h:46-52; its Caffe2 operators pass their own stream through it).
struct CudaRuntimeInformation {
  CudaRuntimeInformation() : stream(nullptr) {}
  explicit CudaRuntimeInformation(tcb200_stream_t s) : stream(s) {}
  tcb200_stream_t stream;
  // Optional device int that a kernel's bounded wait reports into instead of spinning forever.
  int* deviceStatus = nullptr;
};

class CudaTcExecutor;
class CudaRTCFunction;

struct CudaBackend {
  using ExecutorType = CudaTcExecutor;
  using MappingOptionsType = CudaMappingOptions;
  using CompilationResultType = CudaCompilationResult;
  using RTCFunctionType = CudaRTCFunction;
  using WithDevice = WithCudaDevice;
  using RuntimeInformation = CudaRuntimeInformation;

  static std::string backendString() { return CudaGPUInfo::GPUInfo().getCudaDeviceStr(); }
  static std::string makeDeviceFilename(const std::string& fn) { return fn + ".cuda"; }

  // Pattern-matches the analysed def to kernel launches and resolves a tile for each from
  // `options` (CudaMappingOptions::toTile) or the family default.  Throws lang::ErrorReport when a
  // statement matches no family.
  static CompilationResultType compileWithTcMapper(const std::string& tcName, const DefAnalysis& def,
                                                   const std::vector<const DLConstTensor*>& inputs,
                                                   const MappingOptionsType& options);
};

}  // namespace tc
