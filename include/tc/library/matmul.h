// tc/library/matmul.h:22-45 of the reference: O(i, j) +=! A * B in the four transpose forms.
#pragma once

#include <string>

namespace tc {

static constexpr auto TC_MATMUL_NAME = "matmul";

// transposeFirst: A is stored (K, N) and read A(k, i); transposeSecond: B is stored (M, K) and read B(j, k).
inline std::string makeMatmulTc(bool transposeFirst = false, bool transposeSecond = false) {
  const std::string a = transposeFirst ? "float(K, N) A" : "float(N, K) A", ai = transposeFirst ? "A(k, i)" : "A(i, k)";
  const std::string b = transposeSecond ? "float(M, K) B" : "float(K, M) B", bi = transposeSecond ? "B(j, k)" : "B(k, j)";
  return "def matmul(" + a + ", " + b + ") -> (O) {\n  O(i, j) +=! " + ai + " * " + bi + "\n}\n";
}

}  // namespace tc
