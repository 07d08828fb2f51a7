// Second translation unit of the GEMM: the kernel instantiations with the run-time switches (bf16 activations, e4m3 weights,
// low-rank blocks, row-sharded destinations).  Same source as scaled_mm.cu; only the explicit instantiations of
// launch_tn<TN, true> are emitted here, so that the two halves compile in parallel.
#define FEATHER_TU_EXT 1
#include "scaled_mm.cu"
