#include "common.cuh"
namespace tcb200 {
int contraction_tc_query(const tcb200_problem_t&, tcb200_tile_t*, int, int* n) { *n = 0; return TCB200_OK; }
int contraction_tc_plan(Plan&) { return TCB200_ERR_UNSUPPORTED; }
int contraction_tc_launch(const Plan&, const float*, const float*, const float*, float*, cudaStream_t, int*) { return TCB200_ERR_UNSUPPORTED; }
}
