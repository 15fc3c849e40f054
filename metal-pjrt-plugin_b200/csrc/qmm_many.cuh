// b200_qmm for more than 32 rows of x (qmm_many.cu), as seen by qmm.cu.
#pragma once
#include "common.cuh"

namespace b200 {
// Dequantises the weights panel by panel into the context's bf16 workspace and runs the
// tensor-core GEMM on each panel.  The parameters have passed b200_qmm_validate.
b200_status QmmManyRows(b200_context* ctx, cudaStream_t stream, const b200_qmm_params* p);
}  // namespace b200
