// ATenAutotuner (the reference's tc/aten/aten_autotuner.h:44-90): tune over at::Tensors.
#pragma once

#include <ATen/ATen.h>

#include <string>
#include <unordered_map>
#include <vector>

#include "tc/aten/aten_compiler.h"
#include "tc/autotuner/autotuner.h"

namespace tc {
namespace aten {

template <typename Backend, typename SearchStrategy>
class ATenAutotuner : public tc::autotune::Autotuner<Backend, SearchStrategy> {
 public:
  using MappingOptionsType = typename Backend::MappingOptionsType;
  explicit ATenAutotuner(const std::string& tc) : tc_(tc) {}

  // Returns up to topK options, fastest first; possibly empty.  The candidates are timed on the
  // device the inputs live on; outputs are allocated with prepareOutputs.
  std::vector<MappingOptionsType> tune(const std::string& tcEntryPoint, const std::vector<at::Tensor>& inputs,
                                       const std::vector<MappingOptionsType>& baseMappings, size_t topK = 1,
                                       const tc::autotune::TuningParameterFixer& fixedParams = {}) {
    std::vector<at::Tensor> outputs = prepareOutputs(tc_, tcEntryPoint, inputs);
    auto in = makeDLConstTensors(inputs);
    auto out = makeDLTensors(outputs);
    const size_t dev = inputs[0].is_cuda() ? (size_t)inputs[0].get_device() : 0;
    std::unordered_map<size_t, std::vector<const DLConstTensor*>> inMap{{dev, extractRawPtrs(in)}};
    std::unordered_map<size_t, std::vector<const DLTensor*>> outMap{{dev, extractRawPtrs(out)}};
    return tc::autotune::Autotuner<Backend, SearchStrategy>::tune(tc_, tcEntryPoint, inMap, outMap, baseMappings,
                                                                  topK, fixedParams);
  }

 private:
  std::string tc_;
};

}  // namespace aten
}  // namespace tc
