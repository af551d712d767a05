// One executor, several devices: compiled once (on device 0), then run from one host thread per device, each
// thread with its own current device, inputs and outputs there.  The executor creates the plans of a device
// the first time it runs on it, under a lock, as the reference loads its module per device
// (tc/core/cuda/cuda_rtc.cc:308-329; its tuner runs one executor from a thread per GPU,
// tc/autotuner/autotuner-inl.h:279-295).  Needs two GPUs; with fewer it says so and exits 0.
#include <atomic>
#include <iostream>
#include <thread>

#include <ATen/ATen.h>

#include "tc/aten/aten_compiler.h"
#include "tc/core/check.h"
#include "tc/core/cuda/cuda_mapping_options.h"
#include "tc/core/cuda/cuda_tc_executor.h"

int main() {
  int n = 0;
  if (tcb200_device_count(&n) != TCB200_OK || n < 2) {
    std::cout << "multi device skipped (gpus=" << n << ")\n";
    return 0;
  }
  const int devices = std::min(n, 4);
  const std::string tc = R"TC(
def fcrelu(float(B, N) I, float(O, N) W, float(O) Bias) -> (Out) {
    Out(b, o) +=! I(b, n) * W(o, n)
    Out(b, o)  = Out(b, o) + Bias(o)
    Out(b, o)  = fmax(Out(b, o), 0)
}
def tensordot(float(N, C1, C2, H, W) I0, float(N, C2, C3, H, W) I1) -> (O) {
    O(n, c1, c3, h, w) +=! I0(n, c1, r_c2, h, w) * I1(n, r_c2, c3, h, w)
}
  )TC";
  auto on = [](int d) { return at::TensorOptions().dtype(at::kFloat).device(at::Device(at::kCUDA, d)); };
  at::Tensor I = at::randn({512, 640}, on(0)), W = at::randn({384, 640}, on(0)), Bias = at::randn({384}, on(0));
  at::Tensor I0 = at::rand({4, 24, 8, 6, 20}, on(0)), I1 = at::rand({4, 8, 2, 6, 20}, on(0));
  auto naive = tc::CudaMappingOptions::makeNaiveMappingOptions();
  auto fc = tc::aten::compile<tc::CudaBackend>(tc, "fcrelu", {I, W, Bias}, naive);
  auto td = tc::aten::compile<tc::CudaBackend>(tc, "tensordot", {I0, I1}, naive);
  std::atomic<int> failures{0};
  std::vector<std::thread> threads;
  for (int d = 0; d < devices; ++d) {
    threads.emplace_back([&, d]() {
      try {
        tc::WithCudaDevice here((size_t)d);
        for (int round = 0; round < 3; ++round) {
          at::Tensor i = I.to(on(d)), w = W.to(on(d)), b = Bias.to(on(d));
          std::vector<at::Tensor> outs{at::empty({512, 384}, on(d))};
          tc::aten::run(*fc, {i, w, b}, outs);
          at::Tensor ref = at::clamp_min(at::mm(i.to(at::kDouble), w.to(at::kDouble).t()) + b.to(at::kDouble), 0).to(at::kFloat);
          const double err = (outs[0] - ref).abs().max().item<double>() / ref.abs().max().item<double>();
          if (!(err < 1e-5 * 640)) { ++failures; std::cerr << "device " << d << " fcrelu err " << err << "\n"; }
          at::Tensor a0 = I0.to(on(d)), a1 = I1.to(on(d));
          std::vector<at::Tensor> o2{at::empty({4, 24, 2, 6, 20}, on(d))};
          tc::aten::run(*td, {a0, a1}, o2);
          at::Tensor r2 = at::einsum("nakhw,nkchw->nachw", {a0, a1});
          const double e2 = (o2[0] - r2).abs().max().item<double>();
          if (!(e2 < 8 * 5e-7 * 8)) { ++failures; std::cerr << "device " << d << " tensordot err " << e2 << "\n"; }
          fc->checkDeviceStatus();
          td->checkDeviceStatus();
        }
      } catch (const std::exception& e) {
        ++failures;
        std::cerr << "device " << d << ": " << e.what() << "\n";
      }
    });
  }
  for (auto& t : threads) t.join();
  TC_CHECK_EQ(failures.load(), 0);
  std::cout << "multi device ok (gpus=" << devices << ")\n";
  return 0;
}
