// Tensor-parallel group internals shared by tp.cu and decoder.cu.
#pragma once
#include "common.cuh"

constexpr int kTpMaxWorld = 8;

// One rank's peer-exchange block (device memory, mapped into every peer by CUDA IPC):
//   float partial[2][cap]          two alternating slots of this rank's partial sums
//   uint32 flags[kTpMaxWorld]      flags[r]: last exchange for which rank r's partial is ready
//                                  (written by rank r over NVLink)
//   uint32 seq                     exchanges this rank has completed
//   uint32 done                    CTAs of the running exchange that have finished
struct b200_tp {
  b200_context* ctx = nullptr;
  void* comm = nullptr;  // ncclComm_t
  int rank = 0, world = 1;
  bool peer = false;               // peer exchange connected
  int64_t cap = 0;                 // floats per slot
  void* block = nullptr;           // this rank's block
  void* peer_block[kTpMaxWorld] = {};   // every rank's block as mapped here (own: block)
};

namespace b200 {
// In-place sum over ranks; dtype B200_F32 or B200_BF16.
b200_status TpAllReduce(b200_tp* tp, cudaStream_t stream, void* buf, int64_t count, int dtype);
b200_status TpAllGather(b200_tp* tp, cudaStream_t stream, const void* send, void* recv, int64_t count_per_rank,
                        int dtype);
// This rank's slot (0/1) of the peer-exchange block, where a K-sharded projection writes
// its f32 partial sums; null when the exchange is not connected.
float* TpPeerPartial(b200_tp* tp, int slot);
// x (bf16 [batch, hidden]) += bf16(sum over ranks of slot `slot`), h = rms_norm(x) * gain:
// one kernel that signals the peers, waits (bounded) for theirs and reads their partials
// over NVLink.
b200_status TpSumResidualNorm(b200_tp* tp, cudaStream_t stream, int slot, void* x, const void* gain, void* h,
                              int64_t batch, int64_t hidden, double eps);
}  // namespace b200
