// tc/library/matmul.h:22-45 of the reference: O(i, j) +=! A * B in the four transpose forms.
#pragma once

#include <string>

#include "tc/library/tc_text.h"

namespace tc {

static constexpr auto TC_MATMUL_NAME = "matmul";

// transposeFirst: A is stored (K, N) and read A(k, i); transposeSecond: B is stored (M, K) and read B(j, k).
inline std::string makeMatmulTc(bool transposeFirst = false, bool transposeSecond = false) {
  return library_detail::matmulText(TC_MATMUL_NAME, false, transposeFirst, transposeSecond, "A", "B", "O", "N", "K", "M",
                                    "i", "k", "j");
}

}  // namespace tc
