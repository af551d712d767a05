// Search-strategy tag.  The reference's GeneticSearch (tc/autotuner/genetic_search.h:51-111) breeds
// mapping options for its polyhedral mapper over generations; with hand-written kernel families the
// search space is a handful of tile configurations per family, so the "search" is an exhaustive
// sweep and this type only selects it in ATenAutotuner<CudaBackend, GeneticSearch>.
#pragma once

namespace tc {
namespace autotune {
class GeneticSearch {};
}  // namespace autotune
}  // namespace tc
