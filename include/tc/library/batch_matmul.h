// tc/library/batch_matmul.h:20-28 of the reference: Z(b, n, k) +=! X(b, n, mm) * Y(b, mm, k).
#pragma once

#include <string>

#include "tc/library/tc_text.h"

namespace tc {

static constexpr auto TC_BATCH_MATMUL_NAME = "batch_matmul";

inline const std::string TC_BATCH_MATMUL = library_detail::matmulText(
    TC_BATCH_MATMUL_NAME, true, false, false, "X", "Y", "Z", "N", "M", "K", "n", "mm", "k");

}  // namespace tc
