// tc::compile<Backend> and friends (the reference's tc/core/compiler.h:71-98, compiler-inl.h).
#pragma once

#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include "tc/core/tc_analysis.h"
#include "tc/core/tensor.h"
#include "tc/lang/parser.h"
#include "tc/utils/compiler_options.h"

namespace tc {

// Strides that are not "contiguous-like" (non-increasing, innermost >= 1); the kernels of this
// backend additionally require dense tensors and say so in the message.
struct InvalidStrideException : public std::runtime_error {
  explicit InvalidStrideException(const std::string& s) : std::runtime_error(s) {}
};

namespace detail {
// name -> parsed (not yet sema-checked) def, for every def in the TC string.
std::map<std::string, lang::TreeRef> parse(const std::string& tc);
void checkInputsCompliant(const DefAnalysis& def, const std::vector<const DLConstTensor*>& inputs);
std::vector<TensorInfo> inferOutputTensorInfo(const lang::TreeRef& parsedDef,
                                              const std::vector<const DLConstTensor*>& inputs,
                                              const CompilerOptions& options = CompilerOptions());

template <typename Backend>
std::unique_ptr<typename Backend::ExecutorType> compile(
    const lang::TreeRef& parsedDef, const std::vector<const DLConstTensor*>& inputs,
    const typename Backend::MappingOptionsType& options,
    const CompilerOptions& compilerOptions = CompilerOptions()) {
  DefAnalysis def = analyzeDef(parsedDef, inputs, compilerOptions);
  checkInputsCompliant(def, inputs);
  std::vector<TensorInfo> inInfo = makeTensorInfoVector(inputs);
  std::vector<TensorInfo> outInfo;
  for (const auto& o : def.outputs)
    outInfo.emplace_back(toDLDataType(o.scalarKind), 0, o.shape, makeStridesFromSizes(o.shape));
  auto result = Backend::compileWithTcMapper(def.name, def, inputs, options);
  return std::unique_ptr<typename Backend::ExecutorType>(
      new typename Backend::ExecutorType(inInfo, outInfo, def, result));
}
}  // namespace detail

// Output metadata (contiguous) of `entryPoint` for these input shapes.
std::vector<TensorInfo> inferOutputTensorInfo(const std::string& tc, const std::string& entryPoint,
                                              const std::vector<const DLConstTensor*>& inputs,
                                              const CompilerOptions& options = CompilerOptions());

// Compiles one def of a TC string for concrete input shapes.  Re-entrant.
template <typename Backend>
std::unique_ptr<typename Backend::ExecutorType> compile(
    const std::string& tc, const std::string& entryPoint,
    const std::vector<const DLConstTensor*>& inputs,
    const typename Backend::MappingOptionsType& options,
    const CompilerOptions& compilerOptions = CompilerOptions()) {
  auto parsed = detail::parse(tc);
  auto it = parsed.find(entryPoint);
  if (it == parsed.end())
    throw std::runtime_error("Check failed: attempting to access undefined function " + entryPoint);
  return detail::compile<Backend>(it->second, inputs, options, compilerOptions);
}

}  // namespace tc
