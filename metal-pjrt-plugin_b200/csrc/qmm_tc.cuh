// The tensor-core route of the int4 dequant-matmul (qmm_tc.cu), as seen by qmm.cu.
#pragma once
#include "common.cuh"

namespace b200 {
// Whether the tcgen05 route takes this problem: sequential int4 in groups of 64, up to 8 rows of x,
// K a multiple of 256, aligned operands, and a working set that fits one CTA's shared memory.
bool QmmTcEligible(const b200_context* ctx, const b200_qmm_params* p);
// Enqueues it (the parameters have been validated and found eligible).
b200_status QmmTcRun(b200_context* ctx, cudaStream_t stream, const b200_qmm_params* p);
}  // namespace b200
