// placeholder until the tensor-core kernel lands
#include "common.cuh"
namespace b200 {
bool Tcgen05Supports(const b200_gemm_params*, const b200_epilogue*) { return false; }
b200_status RunTcgen05(b200_context*, cudaStream_t, const b200_gemm_params*, const b200_epilogue*) {
  return Fail(B200_UNIMPLEMENTED, "tcgen05 GEMM not built");
}
}  // namespace b200
