// tc/library/batch_matmul.h:20-28 of the reference.
#pragma once

namespace tc {

static constexpr auto TC_BATCH_MATMUL_NAME = "batch_matmul";

static constexpr auto TC_BATCH_MATMUL =
    "def batch_matmul(float(B, N, M) X, float(B, M, K) Y) -> (Z) {\n"
    "  Z(b, n, k) +=! X(b, n, mm) * Y(b, mm, k)\n"
    "}\n";

}  // namespace tc
