// The operator library (tc/library/*.h of the reference) and the reference benchmarks' other cases
// (tc/benchmarks/MLP_model.cc:423-426,479-483; group_convolution.cc:186-217) compiled and, with a
// GPU, run through tc::aten and compared with ATen the way the reference's harness does it
// (test/test_harness_aten.h checkRtol: max|diff| < L * prec * max|inputs|).  The ATen side is evaluated
// in float64 and rounded once: an fp32 library GEMM over 2000 positive terms is itself a few 1e-3 away
// from the exact sum, more than the bound allows for both sides together.
#include <iostream>

#include <ATen/ATen.h>

#include "tc/aten/aten_compiler.h"
#include "tc/core/check.h"
#include "tc/core/cuda/cuda_mapping_options.h"
#include "tc/core/cuda/cuda_tc_executor.h"
#include "tc/core/flags.h"
#include "tc/library/2fcrelu.h"
#include "tc/library/3fcrelu.h"
#include "tc/library/4fcrelu.h"
#include "tc/library/batch_matmul.h"
#include "tc/library/common.h"
#include "tc/library/convolution.h"
#include "tc/library/fcrelu.h"
#include "tc/library/group_convolution.h"
#include "tc/library/matmul.h"

namespace {

bool gpu = false;
int cases = 0;

at::Tensor rnd(std::vector<int64_t> sizes) {
  auto opts = gpu ? at::TensorOptions().dtype(at::kFloat).device(at::kCUDA) : at::TensorOptions().dtype(at::kFloat);
  return at::rand(sizes, opts);
}

void checkRtol(const at::Tensor& out, const at::Tensor& ref, const std::vector<at::Tensor>& inputs, double L,
               double prec, const std::string& what) {
  TC_CHECK(out.sizes() == ref.sizes()) << what << ": shape " << out.sizes() << " vs " << ref.sizes();
  double maxIn = 0;
  for (const auto& t : inputs) maxIn = std::max(maxIn, t.abs().max().item<double>());
  const double err = (out - ref).abs().max().item<double>();
  TC_CHECK_LE(err, L * prec * maxIn) << what << ": max|diff| " << err;
}

// One expected output: the ATen result and the operation count its bound is formed with.
struct Expect {
  at::Tensor ref;
  double L;
};

// Compile (always); run and compare every output (GPU only).
void runCase(const std::string& tc, const std::string& entry, const std::vector<at::Tensor>& inputs,
             const std::vector<Expect>& refs, double prec, const std::string& expectKernel) {
  auto exe = tc::aten::compile<tc::CudaBackend>(tc, entry, inputs, tc::CudaMappingOptions::makeNaiveMappingOptions());
  TC_CHECK(exe->compiledSource.find(expectKernel) != std::string::npos) << entry << ": " << exe->compiledSource;
  auto info = tc::aten::inferOutputTensorInfo(tc, entry, inputs);
  TC_CHECK_EQ(info.size(), refs.size()) << entry;
  for (size_t i = 0; i < refs.size(); ++i) {
    TC_CHECK_EQ((size_t)info[i]->ndim, (size_t)refs[i].ref.dim()) << entry;
    for (int d = 0; d < info[i]->ndim; ++d)
      TC_CHECK_EQ(info[i]->shape[d], refs[i].ref.size(d)) << entry << " output " << i;
  }
  if (gpu) {
    auto outputs = tc::aten::prepareOutputs(tc, entry, inputs);
    tc::aten::run(*exe, inputs, outputs);
    for (size_t i = 0; i < refs.size(); ++i)
      checkRtol(outputs[i], refs[i].ref, inputs, refs[i].L, prec, entry);
  }
  ++cases;
}

at::Tensor d(const at::Tensor& t) { return t.to(at::kDouble); }
at::Tensor f(const at::Tensor& t) { return t.to(at::kFloat); }

at::Tensor fcrelu(const at::Tensor& I, const at::Tensor& W, const at::Tensor& B) {
  return f(d(I).mm(d(W).t()).add(d(B)).clamp_min(0));
}

}  // namespace

int main(int argc, char** argv) {
  tc::parseFlags(argc, argv);
  int n = 0;
  gpu = tcb200_device_count(&n) == TCB200_OK && n > 0;

  // matmul, four transpose forms (test/test_cuda_mapper.cc uses makeMatmulTc())
  for (int ta = 0; ta < 2; ++ta)
    for (int tb = 0; tb < 2; ++tb) {
      at::Tensor A = ta ? rnd({72, 100}) : rnd({100, 72}), B = tb ? rnd({50, 72}) : rnd({72, 50});
      runCase(tc::makeMatmulTc(ta, tb), tc::TC_MATMUL_NAME, {A, B}, {{f(d(ta ? A.t() : A).mm(d(tb ? B.t() : B))), 72}}, 3e-7,
              "tcb200::contraction");
    }
  {
    at::Tensor X = rnd({7, 26, 72}), Y = rnd({7, 72, 26});
    runCase(tc::TC_BATCH_MATMUL, tc::TC_BATCH_MATMUL_NAME, {X, Y}, {{f(d(X).bmm(d(Y))), 72}}, 3e-7, "tcb200::contraction");
  }
  // fully-connected chains at the benchmark's sizes (MLP_model.cc: B=128, M=2000, N=128, O=64, P=32, Q=2)
  {
    at::Tensor I = rnd({128, 2000}), W1 = rnd({128, 2000}), B1 = rnd({128}), W2 = rnd({64, 128}), B2 = rnd({64}),
               W3 = rnd({32, 64}), B3 = rnd({32}), W4 = rnd({2, 32}), B4 = rnd({2});
    at::Tensor O1 = fcrelu(I, W1, B1), O2 = fcrelu(O1, W2, B2), O3 = fcrelu(O2, W3, B3), O4 = fcrelu(O3, W4, B4);
    // bounds as the benchmark forms them: one layer M + 1 operations at 1e-6 (MLP_model.cc:469-473), a
    // chain the product of the reduction sizes so far plus the layer number (MLP_model.cc:536-542)
    const double prec = 1e-6;
    const Expect e1{O1, 2000 + 1}, e2{O2, 2000. * 128 + 2}, e3{O3, 2000. * 128 * 64 + 3},
        e4{O4, 2000. * 128 * 64 * 32 + 4};
    runCase(tc::TC_FCRELU, tc::TC_FCRELU_NAME, {I, W1, B1}, {e1}, prec, "tcb200::contraction");
    runCase(tc::TC_2FCRELU, tc::TC_2FCRELU_NAME, {I, W1, B1, W2, B2}, {e1, e2}, prec, "epilogue=+bias,relu");
    runCase(tc::TC_3FCRELU, tc::TC_3FCRELU_NAME, {I, W1, B1, W2, B2, W3, B3}, {e1, e2, e3}, prec, "relu");
    runCase(tc::TC_4FCRELU, tc::TC_4FCRELU_NAME, {I, W1, B1, W2, B2, W3, B3, W4, B4}, {e1, e2, e3, e4}, prec, "relu");
    {
      // the benchmark's own three-layer case: B=128, 128 -> 64 -> 32 -> 2 at 3e-7 (MLP_model.cc:883-886)
      at::Tensor J = rnd({128, 128});
      at::Tensor P2 = fcrelu(J, W2, B2), P3 = fcrelu(P2, W3, B3), P4 = fcrelu(P3, W4, B4);
      const std::string mlp3 = tc::replaceString(tc::TC_3FCRELU, tc::TC_3FCRELU_NAME, "mlp3");
      runCase(mlp3, "mlp3", {J, W2, B2, W3, B3, W4, B4},
              {{P2, 128 + 1}, {P3, 128. * 64 + 2}, {P4, 128. * 64 * 32 + 3}}, 3e-7, "relu");
    }
    // MLP1 of the benchmark: W1 stored (M, N) and read W1(r_m, n)
    const std::string mlp1 =
        "def mlp1(float(B,M) I, float(M, N) W1, float(N) B1) -> (O1) {\n"
        "  O1(b, n) +=! I(b, r_m) * W1(r_m, n)\n  O1(b, n) = O1(b, n) + B1(n)\n  O1(b, n) = fmax(O1(b, n), 0)\n}\n";
    at::Tensor W1t = W1.t().contiguous();
    runCase(mlp1, "mlp1", {I, W1t, B1}, {e1}, prec, "B=n-major");
    // C3 of the benchmark: B=128, WX=1000, WY=1024
    const std::string c3 = "def _C3(float(B,WX) I, float(WY, WX) W) -> (C3) {\n  C3(b, wy) +=! I(b, r_wx) * W(wy, r_wx)\n}\n";
    at::Tensor Ic = rnd({128, 1000}), Wc = rnd({1024, 1000});
    runCase(c3, "_C3", {Ic, Wc}, {{f(d(Ic).mm(d(Wc).t())), 1024 + 1}}, 1e-6, "tcb200::contraction");  // MLP_model.cc:413-417
  }
  // convolutions: library texts with strides, and the benchmark's four group-convolution cases
  for (auto s : std::vector<std::pair<int, int>>{{1, 1}, {2, 2}, {3, 2}}) {
    at::Tensor I = rnd({4, 8, 33, 30}), W = rnd({16, 8, 3, 3}), B = rnd({16});
    runCase(tc::makeConvolution2DTc(s.first, s.second), tc::CONVOLUTION2D_TC_NAME, {I, W, B},
            {{f(at::conv2d(d(I), d(W), d(B), at::IntArrayRef({(int64_t)s.first, (int64_t)s.second}))), 72}}, 1e-6,
            "tcb200::group_conv");
    at::Tensor Ig = rnd({2, 3, 4, 17, 19}), Wg = rnd({3, 8, 4, 3, 3}), Bg = rnd({3, 8});
    at::Tensor ref = at::conv2d(d(Ig).reshape({2, 12, 17, 19}), d(Wg).reshape({24, 4, 3, 3}), d(Bg).reshape({24}),
                                at::IntArrayRef({(int64_t)s.first, (int64_t)s.second}), at::IntArrayRef({0, 0}),
                                at::IntArrayRef({1, 1}), 3);
    runCase(tc::makeGroupConvolution2DTc(s.first, s.second), tc::GROUP_CONVOLUTION2D_TC_NAME, {Ig, Wg, Bg},
            {{f(ref).reshape({2, 3, 8, ref.size(2), ref.size(3)}), 36}}, 1e-6, "tcb200::group_conv");
  }
  for (auto c : std::vector<std::vector<int64_t>>{{32, 32, 4, 4, 56, 56}, {32, 32, 8, 8, 28, 28},
                                                 {32, 32, 16, 16, 14, 14}, {32, 32, 32, 32, 7, 7}}) {
    const int64_t N = c[0], G = c[1], C = c[2], F = c[3], H = c[4], W = c[5];
    at::Tensor I = rnd({N, G, C, H, W}), W1 = rnd({G, F, C, 3, 3}), B = rnd({G, F});
    at::Tensor ref = at::conv2d(d(I).reshape({N, G * C, H, W}), d(W1).reshape({G * F, C, 3, 3}), d(B).reshape({G * F}), at::IntArrayRef({1, 1}),
                               at::IntArrayRef({0, 0}), at::IntArrayRef({1, 1}), G);
    runCase(tc::makeGroupConvolution2DTc(1, 1), tc::GROUP_CONVOLUTION2D_TC_NAME, {I, W1, B},
            {{f(ref).reshape({N, G, F, H - 2, W - 2}), (double)C * 9}}, 1e-6, "tcb200::group_conv");
  }
  // replaceString keeps its contract (used by callers that template their own texts)
  TC_CHECK_EQ(tc::replaceString("a<x>b<x>", "<x>", "<x><x>"), std::string("a<x><x>b<x><x>"));
  std::cout << "library cases ok: " << cases << " (gpu=" << gpu << ")\n";
  return 0;
}
