// Pattern matcher: the statements of an analysed def -> a chain of launches of the hand-written
// kernel families behind the tcb200 C ABI.
//
// This is what replaces the polyhedral mapper + code generator
// (CudaBackend::compileWithTcMapper, tc/core/cuda/cuda_tc_executor.cc:71-109).  Matching is done
// on the sema-checked tree by STRUCTURE (which index appears in which operand, at which
// position), never by name, so `r_c2` vs `c2` or `mm` vs `r_m` match alike
// (tc/examples/tensordot.cc:45 vs README.md:18; tc/library/batch_matmul.h:24 vs
// tc/benchmarks/batchmatmul.cc:82).
//
//   reduction statement  O(out...) +=! A(...) * B(...)   (or += without "!": accumulate)
//     indices in O, A and B          -> batch        indices in O and A only -> M
//     indices in O and B only        -> N            reduction indices in A and B -> K
//     * trailing batch indices that are the innermost dims of all three tensors
//       (O = [outer, M, N, inner], A = [outer, M, K, inner], B = [outer, K, N, inner])
//                                    -> TENSORDOT family
//     * otherwise each group must flatten to one strided dimension
//                                    -> CONTRACTION family (any operand major-ness)
//     * A(n,g,c,h+kh,w+kw) * W(g,f,c,kh,kw)  (or without g)
//                                    -> GROUP_CONV family
//   followed on the same tensor by
//     O(idx) = O(idx) + Bias(subset of idx)        -> +bias epilogue
//     O(idx) = fmax(O(idx), 0)                      -> ReLU epilogue
//   fused into the launch of the reduction.
// Anything else is a hard error (lang::ErrorReport on the statement); there is no fallback.
#pragma once

#include <string>
#include <vector>

#include "tc/core/tc_analysis.h"
#include "tcb200.h"

namespace tc {

struct MatchedLaunch {
  tcb200_problem_t problem;
  // Positions in the value table [inputs..., outputs...] of the def.
  std::vector<int> inputs;  // {A, B[, bias]}
  int output = -1;
  std::vector<int> statements;  // indices of the statements this launch covers
  std::string family() const;
};

std::vector<MatchedLaunch> matchKernels(const DefAnalysis& def);

}  // namespace tc
