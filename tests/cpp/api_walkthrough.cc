// The reference's own API walk-through (tc/examples/tensordot.cc:41-69) written against this
// repository's headers: tune from naive options, compile with the best, prepareOutputs, profile,
// then reuse the options on other sizes.  With no GPU it stops after the compile-time part
// (parse, shape inference, matching, error reporting), which needs no device.
#include <iostream>

#include <ATen/ATen.h>

#include "tc/aten/aten_autotuner.h"
#include "tc/aten/aten_compiler.h"
#include "tc/core/check.h"
#include "tc/core/cuda/cuda_mapping_options.h"
#include "tc/core/cuda/cuda_tc_executor.h"
#include "tc/core/flags.h"

template <typename Backend>
int walkthrough(bool haveGpu) {
  std::string tc = R"TC(
def tensordot(float(N, C1, C2, H, W) I0,
              float(N, C2, C3, H, W) I1)  -> (O)
{
    O(n, c1, c3, h, w) +=! I0(n, c1, r_c2, h, w) * I1(n, r_c2, c3, h, w)
}
  )TC";
  auto opts = haveGpu ? at::TensorOptions().dtype(at::kFloat).device(at::kCUDA)
                      : at::TensorOptions().dtype(at::kFloat);
  at::Tensor I0 = at::rand({16, 8, 16, 17, 25}, opts);
  at::Tensor I1 = at::rand({16, 16, 2, 17, 25}, opts);

  auto naiveOptions = Backend::MappingOptionsType::makeNaiveMappingOptions();
  std::vector<typename Backend::MappingOptionsType> best{naiveOptions};
  if (haveGpu) {
    tc::aten::ATenAutotuner<Backend, tc::autotune::GeneticSearch> tuner(tc);
    best = tuner.tune("tensordot", {I0, I1}, {naiveOptions});
    TC_CHECK_GT(best.size(), 0u);
  }
  auto pExecutor = tc::aten::compile<Backend>(tc, "tensordot", {I0, I1}, best[0]);
  std::cout << pExecutor->compiledSource;
  auto info = tc::aten::inferOutputTensorInfo(tc, "tensordot", {I0, I1});
  TC_CHECK_EQ(info.size(), 1u);
  TC_CHECK_EQ(info[0]->ndim, 5);
  TC_CHECK_EQ(info[0]->shape[1], 8);
  TC_CHECK_EQ(info[0]->shape[2], 2);

  if (haveGpu) {
    auto outputs = tc::aten::prepareOutputs(tc, "tensordot", {I0, I1});
    auto timings = tc::aten::profile(*pExecutor, {I0, I1}, outputs);
    std::cout << "tensordot ran in: " << timings.kernelRuntime.toMicroSeconds() << "us\n";
    at::Tensor ref = at::einsum("nakhw,nkchw->nachw", {I0, I1});
    const double err = (outputs[0] - ref).abs().max().item<double>();
    TC_CHECK_LT(err, 16 * 5e-7 * 1.0) << "precision";
    tc::aten::run(*pExecutor, {I0, I1}, outputs);
    tc::aten::uncheckedRun(*pExecutor, {I0, I1}, outputs);
    for (auto sizes : std::vector<std::pair<std::vector<int64_t>, std::vector<int64_t>>>{
             {{4, 9, 7, 16, 14}, {4, 7, 3, 16, 14}}, {{8, 5, 11, 10, 10}, {8, 11, 16, 10, 10}}}) {
      at::Tensor A = at::rand(sizes.first, opts), B = at::rand(sizes.second, opts);
      auto exe = tc::aten::compile<Backend>(tc, "tensordot", {A, B}, best[0]);
      auto outs = tc::aten::prepareOutputs(tc, "tensordot", {A, B});
      auto t = tc::aten::profile(*exe, {A, B}, outs);
      std::cout << "tensordot " << A.sizes() << " ran in: " << t.kernelRuntime.toMicroSeconds() << "us\n";
    }
  }

  // error behaviour at the boundary (test/cuda/test_corner_cases.cc:56-80 style)
  int caught = 0;
  try {
    tc::aten::compile<Backend>(tc, "tensordot", {I0}, naiveOptions);
  } catch (const lang::ErrorReport& e) {
    TC_CHECK(std::string(e.what()).find("expected 2 inputs") != std::string::npos) << e.what();
    ++caught;
  }
  try {
    tc::aten::compile<Backend>(tc, "tensordot", {I0.to(at::kInt), I1}, naiveOptions);
  } catch (const lang::ErrorReport& e) {
    TC_CHECK(std::string(e.what()).find("expected type float but found int32") != std::string::npos) << e.what();
    ++caught;
  }
  try {
    tc::aten::compile<Backend>("def f(float(N) A) -> (O) { O(i) = A(i) * 2 }", "f", {at::rand({4}, opts)}, naiveOptions);
  } catch (const lang::ErrorReport& e) {
    TC_CHECK(std::string(e.what()).find("no kernel family") != std::string::npos) << e.what();
    ++caught;
  }
  TC_CHECK_EQ(caught, 3);
  std::cout << "api walkthrough ok (gpu=" << haveGpu << ")\n";
  return 0;
}

int main(int argc, char** argv) {
  tc::parseFlags(argc, argv);
  int n = 0;
  const bool haveGpu = tcb200_device_count(&n) == TCB200_OK && n > 0;
  return walkthrough<tc::CudaBackend>(haveGpu);
}
