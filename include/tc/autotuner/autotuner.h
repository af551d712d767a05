// Autotuner: same entry point and return contract as the reference's
// (tc/autotuner/autotuner.h:123-168, autotuner-inl.h:420-518: a possibly empty vector of mapping
// options, fastest first, every element accepted by compile), implemented as a sweep over the
// candidate tiles the kernel library reports for the matched launches.  Each candidate is compiled,
// warmed up once and profiled `tuner_profile_iterations` times; the median device time ranks it
// (the reference records the median of 10 as well, autotuner-inl.h:195-221).
#pragma once

#include <memory>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "tc/autotuner/genetic_search.h"
#include "tc/autotuner/options_cache.h"
#include "tc/core/cuda/cuda_backend.h"
#include "tc/core/tensor.h"
#include "tc/core/utils/time.h"
#include "tc/lang/canonicalize.h"

namespace tc {
namespace autotune {

// Values the caller pins before tuning (the reference's TuningParameterFixer,
// tc/autotuner/parameters.h:200-236).  Pinned tile sizes / CTA sizes / unroll (= pipeline depth)
// filter the sweep; the remaining setters are accepted for source compatibility and ignored.
class TuningParameterFixer {
 public:
  TuningParameterFixer& fixOuterScheduleFusionStrategy(const FusionStrategy&) { return *this; }
  TuningParameterFixer& fixIntraTileScheduleFusionStrategy(const FusionStrategy&) { return *this; }
  TuningParameterFixer& fixFixParametersBeforeScheduling(bool) { return *this; }
  TuningParameterFixer& fixUnrollFactor(uint32_t val) { unroll = (int)val; return *this; }
  TuningParameterFixer& fixTilingParameters(std::vector<uint32_t> vals) { tiling = std::move(vals); return *this; }
  TuningParameterFixer& fixBlockParameters(std::vector<uint32_t> vals) { blockDims = std::move(vals); return *this; }
  TuningParameterFixer& fixGridParameters(std::vector<uint32_t> vals) { gridDims = std::move(vals); return *this; }
  TuningParameterFixer& fixTileImperfectlyNested(bool) { return *this; }
  TuningParameterFixer& fixUseSharedMemory(bool) { return *this; }
  TuningParameterFixer& fixUsePrivateMemory(bool val) { split3 = val ? 1 : 0; return *this; }
  TuningParameterFixer& fixUnrollCopyShared(bool) { return *this; }
  TuningParameterFixer& fixUseReadOnlyCache(bool) { return *this; }
  TuningParameterFixer& fixMatchLibraryCalls(bool) { return *this; }
  bool admits(const tcb200_tile_t& t) const;

  int unroll = -1, split3 = -1;
  std::vector<uint32_t> tiling, blockDims, gridDims;
};

struct TunedCandidate {
  CudaMappingOptions options;
  double medianUs;
  std::string description;
};

// The sweep itself (CUDA backend): returns every candidate that compiled and ran, fastest first.
// inputs/outputs: device tensors of the current device.
std::vector<TunedCandidate> sweepTiles(const std::string& tc, const std::string& entryPoint,
                                       const std::vector<const DLConstTensor*>& inputs,
                                       const std::vector<const DLTensor*>& outputs,
                                       const TuningParameterFixer& fixed);

template <typename Backend, typename SearchStrategy>
class Autotuner {
 public:
  using MappingOptionsType = typename Backend::MappingOptionsType;
  Autotuner() : optionsCache(new OptionsCache<Backend>()) {}

  // inputs/outputs are keyed by device id, as in the reference; the sweep runs on the first device.
  std::vector<MappingOptionsType> tune(
      const std::string& tc, const std::string& tcEntryPoint,
      const std::unordered_map<size_t, std::vector<const DLConstTensor*>>& inputs,
      std::unordered_map<size_t, std::vector<const DLTensor*>>& outputs,
      const std::vector<MappingOptionsType>& baseMappings, size_t topK = 1,
      const TuningParameterFixer& fixedParams = TuningParameterFixer());

  std::shared_ptr<OptionsCache<Backend>> optionsCache;
};

}  // namespace autotune
}  // namespace tc

#include "tc/autotuner/autotuner-inl.h"
