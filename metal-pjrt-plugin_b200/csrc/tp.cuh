// Tensor-parallel group internals shared by tp.cu and decoder.cu.
#pragma once
#include "common.cuh"

constexpr int kTpMaxWorld = 8;

// One rank's peer-exchange block (device memory, mapped into every peer by CUDA IPC):
//   float partial[2][cap]          two alternating slots of this rank's partial sums (pulled by the peers)
//   uint2 pushed[2][world][cap]    two alternating slots of EVERY rank's partial sums, stored here by
//                                  the projections of those ranks (rank r writes sub-slot r) as 8-byte
//                                  lines {f32 bits, number of the push exchange the value belongs to}
//   uint2 bcast[2][cap / 2]        two alternating slots of this rank's OWN summed rows, published by the CTAs of
//                                  the consuming projection for one another: lines {two bf16, exchange number}
//   uint32 flags[kTpMaxWorld]      flags[r]: last pull exchange for which rank r's partial is ready
//                                  (written by rank r over NVLink)
//   uint32 seq                     pull exchanges this rank has completed
//   uint32 done                    CTAs of the running pull exchange that have finished
//   uint32 unused[kTpMaxWorld]
//   uint32 pcount                  push exchanges this rank has pushed
//   uint32 pdone                   CTAs of the pushing projection that have finished
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
// How one projection (b200_qmm) takes part in the push exchange of a K-sharded product's
// partial sums.  push: its epilogue stores each raw f32 partial sum, together with the number
// of the exchange, as one 8-byte line into sub-slot `rank` of every rank's block (plain
// stores over NVLink; no flag, no fence: the line itself says when it is there).  At their
// end the CTAs of the same kernel form the sum over ranks once per rank: each owns some runs
// of 8 values, adds the ranks' lines from THIS rank's memory in rank order (waiting, bounded,
// for lines that have not landed) and the old residual x_old, writes the new residual rows to
// x_out and publishes them as {two bf16, exchange number} lines.  Not push: the projection
// that follows reads those published rows as the input of its RMSNorm prologue.  Slots
// alternate with the exchange number, which lives in device memory (a captured graph replays).
struct QmmTp {
  int world = 0, rank = 0;
  int64_t cap = 0;                        // lines per sub-slot
  uint32_t* count = nullptr;              // push exchanges so far
  bool push = false;
  uint2* dst[kTpMaxWorld] = {};           // this rank's sub-slot (of slot 0) on every rank
  uint32_t* done = nullptr;
  const uint2* src = nullptr;             // slot 0 of pushed[][][] in this rank's memory
  uint2* bcast = nullptr;                 // slot 0 of bcast[][] in this rank's memory
  const void* x_old = nullptr;            // push: residual rows [M, N] the sum is added to
  void* x_out = nullptr;                  // push: where the new residual rows go
};
b200_status QmmRunEx(b200_context* ctx, cudaStream_t stream, const b200_qmm_params* p, const QmmTp* tp);
// Fills the fields above (push and consume sides) from a connected group; false when the exchange is not connected.
bool TpPushLink(b200_tp* tp, QmmTp* out);

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
