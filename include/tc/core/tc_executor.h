// Backend-agnostic executor base (the reference's tc/core/tc_executor.h:70-116): remembers the
// TensorInfo of inputs and outputs, checks every run against them, then dispatches statically to
// Backend::ExecutorType::uncheckedRun / profileUnchecked.  Tensor data is always borrowed.
#pragma once

#include <chrono>
#include <memory>
#include <string>
#include <tuple>
#include <vector>

#include "tc/core/tc_analysis.h"
#include "tc/core/tensor.h"
#include "tc/core/utils/time.h"
#include "tc/lang/error_report.h"
#include "tc/lang/sema.h"

namespace tc {

namespace detail {
template <typename DLTensorType, typename ParamList>
void checkSizesAndStridesAreCompliant(const std::vector<const DLTensorType*>& actualVec,
                                      const std::vector<TensorInfo>& expectedVec, const ParamList& dbg) {
  if (actualVec.size() != expectedVec.size())
    throw lang::ErrorReport(dbg) << "expected " << expectedVec.size() << " parameters but found "
                                 << actualVec.size() << " parameters";
  for (size_t i = 0; i < actualVec.size(); ++i) {
    const auto* actual = actualVec[i];
    const TensorInfo& expected = expectedVec[i];
    if ((size_t)actual->ndim != expected.shape.size())
      throw lang::ErrorReport(dbg) << "expected " << expected.shape.size()
                                   << " dimensions but found tensor with " << actual->ndim
                                   << " dimensions";
    const int atype = toScalarKind(actual->dtype), etype = toScalarKind(expected.dtype);
    if (atype != etype)
      throw lang::ErrorReport(dbg) << "expected " << lang::kindToString(etype) << " for dim " << i
                                   << " but found " << lang::kindToString(atype);
    for (int d = 0; d < actual->ndim; ++d)
      if (actual->shape[d] != expected.shape[d])
        throw lang::ErrorReport(dbg) << "expected size " << expected.shape[d] << " for dim " << d
                                     << " but found " << actual->shape[d];
  }
}
}  // namespace detail

template <typename Backend>
class TcExecutor {
 protected:
  TcExecutor(const std::vector<TensorInfo>& inputsInfo, const std::vector<TensorInfo>& outputsInfo,
             const DefAnalysis& def, const typename Backend::CompilationResultType& result)
      : compiledSource(result.source), inputsInfo_(inputsInfo), outputsInfo_(outputsInfo), def_(def),
        parameters_(result.parameters) {}

 public:
  TcExecutor(TcExecutor&&) = delete;
  TcExecutor& operator=(TcExecutor&&) = delete;
  TcExecutor(const TcExecutor&) = delete;
  TcExecutor& operator=(const TcExecutor&) = delete;

  // Checks shapes/types, then launches on info.stream.  Does not synchronise.
  void run(const std::vector<const DLConstTensor*>& inputs, const std::vector<const DLTensor*>& outputs,
           typename Backend::RuntimeInformation info = {}) const {
    std::vector<const void*> rawIn;
    std::vector<void*> rawOut;
    std::tie(rawIn, rawOut) = prepareRun(inputs, outputs);
    static_cast<const typename Backend::ExecutorType&>(*this).uncheckedRun(rawIn, rawOut, info);
  }

  // Same, timed with device events; synchronises on the stop event.
  ProfilingInfo profile(const std::vector<const DLConstTensor*>& inputs,
                        const std::vector<const DLTensor*>& outputs) const {
    auto start = std::chrono::system_clock::now();
    std::vector<const void*> rawIn;
    std::vector<void*> rawOut;
    std::tie(rawIn, rawOut) = prepareRun(inputs, outputs);
    ProfilingInfo pi(
        static_cast<const typename Backend::ExecutorType&>(*this).profileUnchecked(rawIn, rawOut));
    Duration cpuOverhead(Duration::since(start));
    cpuOverhead = cpuOverhead - pi.kernelRuntime;
    return ProfilingInfo{cpuOverhead, pi.kernelRuntime, pi.kernelRuntimeUs};
  }

  const std::vector<TensorInfo>& inputsInfo() const { return inputsInfo_; }
  const std::vector<TensorInfo>& outputsInfo() const { return outputsInfo_; }

  // One line per launch: matched family, problem sizes, tile, launch geometry.
  const std::string compiledSource;

 protected:
  std::pair<std::vector<const void*>, std::vector<void*>> prepareRun(
      const std::vector<const DLConstTensor*>& inputs, const std::vector<const DLTensor*>& outputs) const {
    lang::Def d(def_.def);
    detail::checkSizesAndStridesAreCompliant(inputs, inputsInfo_, d.params());
    detail::checkSizesAndStridesAreCompliant(outputs, outputsInfo_, d.returns());
    std::vector<const void*> rawIn;
    std::vector<void*> rawOut;
    for (auto* t : inputs) rawIn.push_back(static_cast<const char*>(t->data) + t->byte_offset);
    for (auto* t : outputs) rawOut.push_back(static_cast<char*>(t->data) + t->byte_offset);
    return {rawIn, rawOut};
  }

  std::vector<TensorInfo> inputsInfo_;
  std::vector<TensorInfo> outputsInfo_;
  DefAnalysis def_;
  std::vector<long> parameters_;
};

}  // namespace tc
