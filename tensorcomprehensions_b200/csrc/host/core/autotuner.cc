// The tile sweep behind Autotuner::tune (CUDA backend).
#include "tc/autotuner/autotuner.h"

#include <algorithm>
#include <iostream>
#include <tuple>

#include "tc/core/compiler.h"
#include "tc/core/cuda/cuda_tc_executor.h"
#include "tc/core/flags.h"

namespace tc {
namespace autotune {

bool TuningParameterFixer::admits(const tcb200_tile_t& t) const {
  if (unroll >= 0 && t.stages != unroll) return false;
  if (split3 >= 0 && t.variant == TCB200_VARIANT_TCGEN05 && (t.split_tf32 == 3) != (split3 == 1)) return false;
  if (!tiling.empty()) {
    const int want[3] = {tiling.size() > 0 ? (int)tiling[0] : t.bm, tiling.size() > 1 ? (int)tiling[1] : t.bn,
                         tiling.size() > 2 ? (int)tiling[2] : t.bk};
    if (want[0] != t.bm || want[1] != t.bn || want[2] != t.bk) return false;
  }
  if (!blockDims.empty() && (int)blockDims[0] != t.threads) return false;
  return true;
}

std::vector<TunedCandidate> sweepTiles(const std::string& tc, const std::string& entryPoint,
                                       const std::vector<const DLConstTensor*>& inputs,
                                       const std::vector<const DLTensor*>& outputs,
                                       const TuningParameterFixer& fixed) {
  // Family-default compile tells us which launches the def consists of.
  auto base = tc::compile<CudaBackend>(tc, entryPoint, inputs, CudaMappingOptions::makeNaiveMappingOptions());
  std::vector<tcb200_tile_t> candidates;
  auto key = [](const tcb200_tile_t& t) {
    return std::make_tuple(t.variant, t.bm, t.bn, t.bk, t.stages, t.threads, t.split_tf32, t.split_k > 1 ? t.split_k : 1);
  };
  for (const auto& l : base->launches()) {
    tcb200_tile_t tiles[32];
    int n = 0;
    if (tcb200_query(&l.problem, tiles, 32, &n) != TCB200_OK) continue;
    for (int i = 0; i < std::min(n, 32); ++i) {
      // A plan fills in what a listed tile leaves open (threads, rows per CTA ...): sweep the tile as the
      // plan will report it, so that the "was it applied" test below compares like with like.
      tcb200_plan_t* probe = nullptr;
      if (tcb200_plan_create(&l.problem, &tiles[i], 0, &probe) != TCB200_OK) continue;
      tcb200_plan_tile(probe, &tiles[i]);
      tcb200_plan_destroy(probe);
      if (!fixed.admits(tiles[i])) continue;
      bool seen = false;
      for (const auto& c : candidates) seen = seen || key(c) == key(tiles[i]);
      if (!seen) candidates.push_back(tiles[i]);
    }
  }
  const uint32_t iters = std::max<uint32_t>(1, flags().tuner_profile_iterations);
  std::vector<TunedCandidate> ranked;
  for (const auto& tile : candidates) {
    CudaMappingOptions opts = CudaMappingOptions::fromTile(tile);
    try {
      auto exe = tc::compile<CudaBackend>(tc, entryPoint, inputs, opts);
      // a candidate whose tile no launch accepted is the default configuration again: skip it
      bool applied = false;
      for (const auto& t : exe->tiles()) applied = applied || key(t) == key(tile);
      if (!applied) continue;
      exe->profile(inputs, outputs);  // warm-up (first launch configures the kernel)
      std::vector<double> us;
      for (uint32_t i = 0; i < iters; ++i) us.push_back(exe->profile(inputs, outputs).kernelRuntimeUs);
      std::sort(us.begin(), us.end());
      ranked.push_back(TunedCandidate{opts, us[us.size() / 2], exe->compiledSource});
      if (flags().tuner_print_progress)
        std::cerr << "[tune] " << us[us.size() / 2] << " us  " << exe->compiledSource;
    } catch (const std::exception& e) {
      // an invalid candidate is skipped, like the reference marks it invalid (autotuner-inl.h:91-109)
      if (flags().tuner_print_progress) std::cerr << "[tune] candidate rejected: " << e.what() << "\n";
    }
  }
  std::stable_sort(ranked.begin(), ranked.end(),
                   [](const TunedCandidate& a, const TunedCandidate& b) { return a.medianUs < b.medianUs; });
  return ranked;
}

}  // namespace autotune
}  // namespace tc
