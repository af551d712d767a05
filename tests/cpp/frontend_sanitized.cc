// The C++ host front-end and analysis under AddressSanitizer + UndefinedBehaviorSanitizer: every TC of the golden
// corpus is parsed, checked and canonicalised; every rejected text of the error corpus must throw (and nothing
// else); the five benchmark comprehensions and the library's texts go through size binding, range inference and
// the pattern matcher with shape-only inputs.  No device is touched.  Built by tests/test_sanitized_cpu.py from the
// host sources with -fsanitize=address,undefined; a sanitizer report makes the process exit non-zero.
#include <fstream>
#include <iostream>
#include <sstream>

#include "tc/core/compiler.h"
#include "tc/core/cuda/cuda_backend.h"
#include "tc/core/kernel_matcher.h"
#include "tc/core/tc_analysis.h"
#include "tc/lang/canonicalize.h"
#include "tc/lang/parser.h"
#include "tc/lang/sema.h"
#include "tc/library/3fcrelu.h"
#include "tc/library/batch_matmul.h"
#include "tc/library/group_convolution.h"
#include "tc/library/matmul.h"

static std::string slurp(const std::string& path) {
  std::ifstream f(path);
  std::stringstream ss;
  ss << f.rdbuf();
  return ss.str();
}

static int checked = 0, rejected = 0, matched = 0;

static void frontEnd(const std::string& text) {
  lang::Parser parser(text);
  while (parser.L.cur().kind != lang::TK_EOF) {
    auto def = parser.parseFunction();
    std::stringstream out;
    out << def;
    lang::Sema sema;
    auto typed = sema.checkFunction(def);
    out << typed << sema.dumpEnv() << lang::canonicalize(typed);
    if (out.str().empty()) throw std::runtime_error("empty print");
    ++checked;
  }
}

static void analyseAndMatch(const std::string& text, const std::string& entry,
                            const std::vector<std::vector<int64_t>>& shapes) {
  std::vector<tc::DLConstTensorUPtr> owned;
  std::vector<const DLConstTensor*> inputs;
  for (const auto& s : shapes) {
    owned.push_back(tc::makeDLConstTensor(DLDataType{kDLFloat, 32, 1}, DLDevice{kDLCUDA, 0}, s,
                                          tc::makeStridesFromSizes(s), nullptr));
    inputs.push_back(owned.back().get());
  }
  auto parsed = tc::detail::parse(text);
  auto def = tc::analyzeDef(parsed.at(entry), inputs);
  tc::detail::checkInputsCompliant(def, inputs);
  auto launches = tc::matchKernels(def);
  if (launches.empty()) throw std::runtime_error("no launch for " + entry);
  matched += (int)launches.size();
}

int main(int argc, char** argv) {
  if (argc < 2) return 2;
  const std::string dir = argv[1];
  for (const char* f : {"contraction_family.tc", "conv_and_mlp.tc", "language_features.tc"}) frontEnd(slurp(dir + "/" + f));
  // rejected texts: blocks separated by a line of '----'
  {
    std::stringstream all(slurp(dir + "/errors.txt"));
    std::string line, block;
    auto flush = [&]() {
      if (block.find("def ") == std::string::npos) { block.clear(); return; }
      try {
        frontEnd(block);
        std::cerr << "accepted a text that must be rejected:\n" << block;
        exit(3);
      } catch (const lang::ErrorReport&) {
        ++rejected;
      }
      block.clear();
    };
    while (std::getline(all, line)) {
      if (line.rfind("----", 0) == 0) flush();
      else if (line.rfind("#", 0) != 0) block += line + "\n";
    }
    flush();
  }
  analyseAndMatch("def tensordot(float(N, C1, C2, H, W) I0, float(N, C2, C3, H, W) I1) -> (O) {\n"
                  "  O(n, c1, c3, h, w) +=! I0(n, c1, r_c2, h, w) * I1(n, r_c2, c3, h, w)\n}\n",
                  "tensordot", {{32, 512, 8, 28, 28}, {32, 8, 2, 28, 28}});
  analyseAndMatch(tc::TC_BATCH_MATMUL, tc::TC_BATCH_MATMUL_NAME, {{500, 26, 72}, {500, 72, 26}});
  analyseAndMatch(tc::makeMatmulTc(false, true), "matmul", {{128, 4096}, {16384, 4096}});
  analyseAndMatch(tc::makeGroupConvolution2DTc(1, 1), "group_convolution",
                  {{32, 32, 16, 16, 16}, {32, 16, 16, 3, 3}, {32, 16}});
  analyseAndMatch(tc::TC_3FCRELU, tc::TC_3FCRELU_NAME,
                  {{16384, 2048}, {1024, 2048}, {1024}, {512, 1024}, {512}, {256, 512}, {256}});
  // the convolution gradients of the autograd example: unit-range index differences, reduced batch index, copy
  const std::string grads =
      "def convolution_igrad(float(M,C,KH,KW) W1, float(N,M,H,W) d_O) -> (d_I) {\n"
      "  d_I(n, c, h, w) +=! d_O(n, r_m, h - r_kh, w - r_kw) * W1(r_m, c, r_kh, r_kw)\n}\n"
      "def convolution_wgrad(float(N,C,H,W) I, float(N,M,H,W) d_O) -> (d_W1) {\n"
      "  d_W1(m, c, kh, kw) +=! d_O(r_n, m, r_h - kh, r_w - kw) * I(r_n, c, r_h, r_w)\n}\n"
      "def convolution_biasgrad(float(M) Bias) -> (d_Bias) { d_Bias(m) = Bias(m) }\n";
  analyseAndMatch(grads, "convolution_igrad", {{16, 4, 1, 1}, {32, 16, 56, 56}});
  analyseAndMatch(grads, "convolution_wgrad", {{32, 4, 56, 56}, {32, 16, 56, 56}});
  analyseAndMatch(grads, "convolution_biasgrad", {{16}});
  // an unmatched comprehension is an ErrorReport, not a crash
  try {
    analyseAndMatch("def f(float(N) A) -> (O) { O(i) = A(i) * 2 }", "f", {{4}});
    return 4;
  } catch (const lang::ErrorReport&) {
  }
  std::cout << "sanitized front-end ok: " << checked << " defs, " << rejected << " rejected, " << matched << " launches\n";
  return 0;
}
