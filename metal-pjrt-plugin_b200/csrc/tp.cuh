// Tensor-parallel group internals shared by tp.cu and decoder.cu.
#pragma once
#include "common.cuh"

struct b200_tp {
  b200_context* ctx = nullptr;
  void* comm = nullptr;  // ncclComm_t
  int rank = 0, world = 1;
};

namespace b200 {
// In-place sum over ranks; dtype B200_F32 or B200_BF16.
b200_status TpAllReduce(b200_tp* tp, cudaStream_t stream, void* buf, int64_t count, int dtype);
b200_status TpAllGather(b200_tp* tp, cudaStream_t stream, const void* send, void* recv, int64_t count_per_rank,
                        int dtype);
}  // namespace b200
