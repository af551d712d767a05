// The ATen-facing API: the exact entry points of the reference's tc/aten/aten_compiler.h:35-92.
//
//   auto exe  = tc::aten::compile<tc::CudaBackend>(tc, "name", {I0, I1}, options);
//   auto outs = tc::aten::prepareOutputs(tc, "name", {I0, I1});
//   tc::aten::run(*exe, {I0, I1}, outs);          // or profile(...) / uncheckedRun(...)
#pragma once

#include <ATen/ATen.h>

#include <memory>
#include <string>
#include <vector>

#include "tc/aten/aten.h"
#include "tc/core/compiler.h"
#include "tc/core/cuda/cuda_backend.h"
#include "tc/core/cuda/cuda_tc_executor.h"
#include "tc/core/utils/time.h"
#include "tc/utils/compiler_options.h"

namespace tc {
namespace aten {

// Contiguous output metadata for these input shapes.
inline std::vector<tc::DLTensorUPtr> inferOutputTensorInfo(const std::string& tc, const std::string& entryPoint,
                                                           const std::vector<at::Tensor>& inputs) {
  auto in = makeDLConstTensors(inputs);
  std::vector<tc::DLTensorUPtr> out;
  for (const auto& info : tc::inferOutputTensorInfo(tc, entryPoint, extractRawPtrs(in)))
    out.push_back(tc::makeDLTensor(info));
  return out;
}

// Fresh, uninitialised outputs on the device of inputs[0] (at least one input is required, like the
// reference: tc/aten/aten_compiler.cc:55-65).
inline std::vector<at::Tensor> prepareOutputs(const std::string& tc, const std::string& entryPoint,
                                              const std::vector<at::Tensor>& inputs) {
  TC_CHECK_GE(inputs.size(), 1u) << "NYI: Need >= 1 input tensors to determine backend and prepare ATen outputs.";
  auto in = makeDLConstTensors(inputs);
  std::vector<at::Tensor> out;
  for (const auto& info : tc::inferOutputTensorInfo(tc, entryPoint, extractRawPtrs(in)))
    out.push_back(at::empty(info.shape, inputs[0].options().dtype(toScalarType(info.dtype))));
  return out;
}

template <typename Backend>
std::unique_ptr<typename Backend::ExecutorType> compile(const std::string& tc, const std::string& entryPoint,
                                                        const std::vector<at::Tensor>& inputs,
                                                        const typename Backend::MappingOptionsType& options,
                                                        const CompilerOptions& compilerOptions = CompilerOptions()) {
  auto in = makeDLConstTensors(inputs);
  return tc::compile<Backend>(tc, entryPoint, extractRawPtrs(in), options, compilerOptions);
}

template <typename Executor>
void run(const Executor& executor, const std::vector<at::Tensor>& inputs, std::vector<at::Tensor>& outputs) {
  auto in = makeDLConstTensors(inputs);
  auto out = makeDLTensors(outputs);
  executor.run(extractRawPtrs(in), extractRawPtrs(out));
}

template <typename Executor>
ProfilingInfo profile(const Executor& executor, const std::vector<at::Tensor>& inputs,
                      std::vector<at::Tensor>& outputs) {
  auto start = std::chrono::system_clock::now();
  auto in = makeDLConstTensors(inputs);
  auto out = makeDLTensors(outputs);
  ProfilingInfo pi(executor.profile(extractRawPtrs(in), extractRawPtrs(out)));
  Duration cpuOverhead(Duration::since(start));
  cpuOverhead = cpuOverhead - pi.kernelRuntime;
  return ProfilingInfo{cpuOverhead, pi.kernelRuntime, pi.kernelRuntimeUs};
}

// "Low-latency" mode: raw pointers, no shape checks (tc/aten/aten_compiler-inl.h:71-86).
template <typename Executor>
void uncheckedRun(const Executor& executor, const std::vector<at::Tensor>& inputs,
                  std::vector<at::Tensor>& outputs) {
  std::vector<const void*> rawIn;
  std::vector<void*> rawOut;
  for (const auto& t : inputs) rawIn.push_back(t.data_ptr());
  for (auto& t : outputs) rawOut.push_back(t.data_ptr());
  executor.uncheckedRun(rawIn, rawOut);
}

}  // namespace aten
}  // namespace tc
