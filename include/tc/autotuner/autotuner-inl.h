#pragma once

#include <algorithm>
#include <fstream>
#include <sstream>

#include "tc/core/compiler.h"
#include "tc/core/cuda/cuda_tc_executor.h"

namespace tc {
namespace autotune {

// options_cache-inl.h:336-367 of the reference: look a (tc, sizes) up in a cache file / merge the k best
// of every key of a cache into a cache file.
template <typename Backend>
std::vector<typename Backend::MappingOptionsType> loadTopKFromCacheFile(
    const std::string& tc, const std::string& entryPoint, const std::string& cacheFilename,
    const std::vector<const DLConstTensor*>& inputs, size_t count) {
  OptionsCache<Backend> optionsCache;
  optionsCache.loadCacheFromFile(cacheFilename);
  auto outputs = tc::inferOutputTensorInfo(tc, entryPoint, inputs);
  return optionsCache.getTopKOptions(lang::canonicalTc(tc::detail::parse(tc).at(entryPoint)),
                                     makeTensorInfoVector(inputs), outputs,
                                     Backend::backendString(), count);
}

template <typename Backend>
void appendTopKToCacheFile(const OptionsCache<Backend>& cache, const std::string& cacheFilename, uint32_t count) {
  OptionsCache<Backend> copy(cache);
  copy.pruneKeepTopK(count);
  OptionsCache<Backend> onDisk;
  onDisk.loadCacheFromFile(cacheFilename);
  onDisk.fromProtobuf(copy.toProtobuf());
  onDisk.storeCacheToFile(cacheFilename);
}

template <typename Backend, typename SearchStrategy>
std::vector<typename Backend::MappingOptionsType> Autotuner<Backend, SearchStrategy>::tune(
    const std::string& tc, const std::string& tcEntryPoint,
    const std::unordered_map<size_t, std::vector<const DLConstTensor*>>& inputs,
    std::unordered_map<size_t, std::vector<const DLTensor*>>& outputs,
    const std::vector<MappingOptionsType>& baseMappings, size_t topK,
    const TuningParameterFixer& fixedParams) {
  (void)baseMappings;  // every family default is part of the sweep already
  if (inputs.empty()) return {};
  // lowest device id first
  size_t dev = inputs.begin()->first;
  for (const auto& kv : inputs) dev = std::min(dev, kv.first);
  const auto& in = inputs.at(dev);
  const auto& out = outputs.at(dev);
  typename Backend::WithDevice guard(dev);
  std::vector<TunedCandidate> ranked = sweepTiles(tc, tcEntryPoint, in, out, fixedParams);

  auto parsed = tc::detail::parse(tc);
  const lang::CanonicalTcString canonical = lang::canonicalTc(parsed.at(tcEntryPoint));
  const std::vector<TensorInfo> inInfo = makeTensorInfoVector(in), outInfo = makeTensorInfoVector(out);
  const std::string device = Backend::backendString();
  for (const auto& c : ranked)
    optionsCache->recordRuntime(canonical, inInfo, outInfo, device, c.options,
                                Duration::fromMicroSeconds((size_t)(c.medianUs + 0.5)));
  std::vector<MappingOptionsType> result;
  for (size_t i = 0; i < ranked.size() && i < topK; ++i) result.push_back(ranked[i].options);
  return result;
}

}  // namespace autotune
}  // namespace tc
