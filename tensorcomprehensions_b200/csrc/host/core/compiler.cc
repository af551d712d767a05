// tc::detail::parse / checkInputsCompliant / inferOutputTensorInfo, CudaBackend::compileWithTcMapper
// and CudaTcExecutor.
#include "tc/core/compiler.h"

#include <iostream>
#include <sstream>

#include "tc/core/check.h"
#include "tc/core/cuda/cuda_backend.h"
#include "tc/core/cuda/cuda_tc_executor.h"
#include "tc/core/flags.h"
#include "tc/lang/error_report.h"

namespace tc {
namespace detail {

std::map<std::string, lang::TreeRef> parse(const std::string& tc) {
  lang::Parser parser(tc);
  std::map<std::string, lang::TreeRef> parsed;
  while (parser.L.cur().kind != lang::TK_EOF) {
    lang::TreeRef t = parser.parseFunction();
    parsed.emplace(lang::Def(t).name().name(), t);
  }
  return parsed;
}

void checkInputsCompliant(const DefAnalysis& def, const std::vector<const DLConstTensor*>& inputs) {
  lang::Def d(def.def);
  if (inputs.size() != def.inputs.size())
    throw lang::ErrorReport(def.def) << "expected " << def.inputs.size() << " inputs but found "
                                     << inputs.size();
  for (size_t i = 0; i < inputs.size(); ++i) {
    const DLConstTensor* t = inputs[i];
    const int got = toScalarKind(t->dtype);
    int want = def.inputs[i].scalarKind;
    want = lang::TypeInfo(lang::Tree::compound(want, d.params()[i].range())).toScalarToken();
    if (got != want)
      throw lang::ErrorReport(d.params()[i]) << "expected type " << lang::kindToString(want)
                                             << " but found " << lang::kindToString(got);
    if ((size_t)t->ndim != def.inputs[i].shape.size())
      throw lang::ErrorReport(d.params()[i])
          << "expected a tensor with " << def.inputs[i].shape.size() << " dimensions but found "
          << t->ndim << " dimensions.";
    if (t->ndim && t->strides) {
      bool ok = t->strides[t->ndim - 1] >= 1;
      for (int j = 0; ok && j < t->ndim - 1; ++j)
        ok = t->strides[j] >= t->strides[j + 1] * t->shape[j + 1];
      // The reference's generated code silently assumes dense tensors even when it accepts padded
      // outer strides (test/cuda/test_tc_mapper.cc:306-335); this backend requires them outright.
      bool dense = TensorInfo(t).isContiguous();
      if (!ok || !dense) {
        std::ostringstream err;
        err << lang::ErrorReport(d.params()[i]).what() << "compilation aborted: invalid strides in tensor "
            << (ok ? "(the B200 kernels need dense row-major tensors) " : "") << std::endl
            << *t << std::endl;
        throw InvalidStrideException(err.str());
      }
    }
  }
}

std::vector<TensorInfo> inferOutputTensorInfo(const lang::TreeRef& parsedDef,
                                              const std::vector<const DLConstTensor*>& inputs,
                                              const CompilerOptions& options) {
  DefAnalysis def = analyzeDef(parsedDef, inputs, options);
  std::vector<TensorInfo> r;
  for (const auto& o : def.outputs)
    r.emplace_back(toDLDataType(o.scalarKind), 0, o.shape, makeStridesFromSizes(o.shape));
  return r;
}

}  // namespace detail

std::vector<TensorInfo> inferOutputTensorInfo(const std::string& tc, const std::string& entryPoint,
                                              const std::vector<const DLConstTensor*>& inputs,
                                              const CompilerOptions& options) {
  auto parsed = detail::parse(tc);
  auto it = parsed.find(entryPoint);
  if (it == parsed.end())
    throw std::runtime_error("Check failed: attempting to access undefined function " + entryPoint);
  return detail::inferOutputTensorInfo(it->second, inputs, options);
}

// ------------------------------------------------------------------------------------------------
CudaCompilationResult CudaBackend::compileWithTcMapper(const std::string& tcName, const DefAnalysis& def,
                                                       const std::vector<const DLConstTensor*>& inputs,
                                                       const CudaMappingOptions& options) {
  CudaCompilationResult res;
  res.launches = matchKernels(def);
  res.device = 0;
  if (!inputs.empty() && inputs[0]->device.device_type == kDLCUDA) res.device = inputs[0]->device.device_id;

  std::stringstream name;
  name << tcName;
  for (const auto& kv : def.sizes) {
    res.parameters.push_back((long)kv.second);
    name << "_" << kv.second;
  }
  res.specializedName = name.str();

  tcb200_tile_t wanted;
  const bool hasTile = options.toTile(&wanted);
  std::stringstream src;
  src << "// " << res.specializedName << ": " << res.launches.size() << " launch(es)\n";
  for (auto& l : res.launches) {
    tcb200_plan_t* plan = nullptr;
    int st = TCB200_ERR_UNSUPPORTED;
    if (hasTile) st = tcb200_plan_create(&l.problem, &wanted, res.device, &plan);
    if (st != TCB200_OK) st = tcb200_plan_create(&l.problem, nullptr, res.device, &plan);
    if (st != TCB200_OK) {
      const lang::TreeRef where = def.statements[l.statements.front()].tree;
      throw lang::ErrorReport(where) << "the " << l.family() << " kernel family rejected this problem: "
                                     << tcb200_strerror(st);
    }
    tcb200_tile_t tile;
    tcb200_plan_tile(plan, &tile);
    res.tiles.push_back(tile);
    char buf[640];
    tcb200_plan_describe(plan, buf, sizeof(buf));
    src << buf << "\n";
    int64_t g[3], b[3];
    tcb200_plan_geometry(plan, g, b);
    res.grid = Grid(CudaDim((uint64_t)g[0], (uint64_t)g[1], (uint64_t)g[2]));
    res.block = Block(CudaDim((uint64_t)b[0], (uint64_t)b[1], (uint64_t)b[2]));
    tcb200_plan_destroy(plan);
  }
  res.source = src.str();
  if (flags().debug_tc_mapper || flags().dump_cuda) std::cerr << res.source;
  return res;
}

CudaTcExecutor::CudaTcExecutor(const std::vector<TensorInfo>& inputsInfo,
                               const std::vector<TensorInfo>& outputsInfo, const DefAnalysis& def,
                               const CudaCompilationResult& result)
    : TcExecutor<CudaBackend>(inputsInfo, outputsInfo, def, result), launches_(result.launches),
      tiles_(result.tiles), grid_(result.grid), block_(result.block), device_(result.device) {
  for (size_t i = 0; i < launches_.size(); ++i) {
    tcb200_plan_t* plan = nullptr;
    TC_TCB200_ENFORCE(tcb200_plan_create(&launches_[i].problem, &tiles_[i], device_, &plan));
    plans_.push_back(plan);
  }
}

CudaTcExecutor::~CudaTcExecutor() {
  for (auto* p : plans_) tcb200_plan_destroy(p);
}

void CudaTcExecutor::uncheckedRun(const std::vector<const void*>& inputs, const std::vector<void*>& outputs,
                                  CudaBackend::RuntimeInformation info) const {
  const size_t nIn = inputs.size();
  auto value = [&](int idx) -> const void* {
    return (size_t)idx < nIn ? inputs[idx] : outputs[idx - nIn];
  };
  for (size_t i = 0; i < plans_.size(); ++i) {
    const MatchedLaunch& l = launches_[i];
    const void* ins[3];
    for (size_t j = 0; j < l.inputs.size(); ++j) ins[j] = value(l.inputs[j]);
    void* outs[1] = {outputs[l.output - nIn]};
    TC_TCB200_ENFORCE(tcb200_launch(plans_[i], ins, (int)l.inputs.size(), outs, 1, info.stream, info.deviceStatus));
  }
}

ProfilingInfo CudaTcExecutor::profileUnchecked(const std::vector<const void*>& inputs,
                                               const std::vector<void*>& outputs) const {
  auto start = std::chrono::system_clock::now();
  tcb200_timer_t* timer = nullptr;
  TC_TCB200_ENFORCE(tcb200_timer_start(nullptr, &timer));
  try {
    uncheckedRun(inputs, outputs, CudaBackend::RuntimeInformation());
  } catch (...) {
    float ignored;
    tcb200_timer_stop(timer, nullptr, &ignored);
    throw;
  }
  float us = 0.f;
  TC_TCB200_ENFORCE(tcb200_timer_stop(timer, nullptr, &us));
  Duration kernel = Duration::fromMicroSeconds((size_t)us);
  Duration cpu = Duration::since(start);
  cpu = cpu - kernel;
  return ProfilingInfo{cpu, kernel, (double)us};
}

}  // namespace tc
