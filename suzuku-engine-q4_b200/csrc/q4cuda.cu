// The whole library as one translation unit: the codebook lives in one
// __constant__ array that every kernel file reads.
#include "q4b_internal.cuh"

#include "q4b_runtime.cu"
#include "q4b_decode.cu"
#include "q4b_synth.cu"
#include "q4b_stack.cu"
#include "q4b_mmq_tc.cu"
#include "q4b_few.cu"
#include "q4b_grouped.cu"
#include "q4b_elem.cu"
#include "q4b_mmvq.cu"
#include "q4b_compat.cu"
#include "q4b_noalloc.cu"
