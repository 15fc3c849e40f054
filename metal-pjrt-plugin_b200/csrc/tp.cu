// Tensor-parallel group over NCCL (NVLink 5 / NVSwitch), one process per GPU.
// The reference is single-device (its collectives are a stub,
// metal_pjrt/compiler/metal_collectives_registration.cc:10-17); this is new.
// NCCL is looked up with dlopen when the first group is made, so the library
// itself links nothing but the CUDA runtime.  The caller moves the 128-byte
// group id between processes by whatever transport it has.
//
// Peer exchange: the all-reduce that follows a K-sharded projection (o, down) moves
// batch x hidden f32 values, 16 KB at batch 1, so its cost is launch and handshake
// latency, not bandwidth.  With the exchange connected, every rank's partial sums live in
// a block that CUDA IPC maps into all peers, and ONE kernel per rank does signal ->
// bounded wait -> read all peers' partials with plain peer loads (no multimem, no
// multicast) -> sum in rank order (every rank gets the same bits) -> residual add ->
// RMSNorm, in place of ncclAllReduce + a separate residual/norm kernel.
#include <dlfcn.h>
#include <nccl.h>

#include <algorithm>
#include <cstring>

#include "tp.cuh"

using namespace b200;

namespace {

struct NcclApi {
  void* handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
};

NcclApi* Api() {
  static NcclApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    // A process that already loaded NCCL (e.g. through torch) gets that copy.
    const char* names[] = {"libnccl.so.2", "libnccl.so"};
    for (const char* n : names) {
      api.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
      if (api.handle != nullptr) break;
    }
    if (api.handle == nullptr) return;
    auto sym = [&](const char* s) { return dlsym(api.handle, s); };
    api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(sym("ncclGetUniqueId"));
    api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(sym("ncclCommInitRank"));
    api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(sym("ncclCommDestroy"));
    api.AllReduce = reinterpret_cast<decltype(api.AllReduce)>(sym("ncclAllReduce"));
    api.AllGather = reinterpret_cast<decltype(api.AllGather)>(sym("ncclAllGather"));
    api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(sym("ncclGetErrorString"));
    if (!api.GetUniqueId || !api.CommInitRank || !api.CommDestroy || !api.AllReduce || !api.AllGather ||
        !api.GetErrorString)
      api.handle = nullptr;
  });
  return api.handle != nullptr ? &api : nullptr;
}

b200_status NcclFail(b200_context* ctx, const char* what, ncclResult_t r) {
  return Stick(ctx, Fail(B200_INTERNAL, "%s: %s", what, Api()->GetErrorString(r)));
}


struct PeerArgs {
  const float* partial[kTpMaxWorld];   // slot base of every rank, rank order
  uint32_t* peer_flags[kTpMaxWorld];   // flags array inside every rank's block
  uint32_t* flags;                     // this rank's flags
  uint32_t* seq;
  uint32_t* done;
  int rank, world;
  __nv_bfloat16* x;
  const __nv_bfloat16* gain;
  __nv_bfloat16* h;
  int n;
  float eps;
  int* status;
};

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ float4 ld_relaxed_sys_f4(const float* p) {
  float4 v;
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

// One CTA per batch row, up to 1024 threads (a float4 of every rank's partial each), n a multiple of 4.
__global__ void __launch_bounds__(1024) peer_sum_residual_norm_kernel(const PeerArgs a) {
  extern __shared__ float row[];
  __shared__ float scratch[32];
  __shared__ uint32_t seq_s;
  __shared__ int gave_up;
  pdl_wait();   // this rank's partial comes from the kernel before
  pdl_launch_dependents();
  const int tid = threadIdx.x;
  if (tid == 0) gave_up = 0;
  if (tid == 0) seq_s = ld_acquire_sys(a.seq) + 1u;   // the number of this exchange
  __syncthreads();
  const uint32_t seq = seq_s;
  // tell every peer that this rank's partial for exchange `seq` is complete ...
  if (blockIdx.x == 0 && tid < a.world && tid != a.rank) {
    __threadfence_system();
    st_release_sys(a.peer_flags[tid] + a.rank, seq);
  }
  // ... and wait, bounded, for theirs
  if (tid < a.world && tid != a.rank) {
    const uint32_t* f = a.flags + tid;
    bool ok = false;
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
      for (int i = 0; i < 256 && !ok; ++i) ok = static_cast<int32_t>(ld_acquire_sys(f) - seq) >= 0;
      if (ok || clock64() - t0 > 4000000000ll) break;
    }
    if (!ok) {
      report_timeout(a.status, 400 + tid);
      gave_up = 1;
    }
  }
  __syncthreads();
  // A peer that did not answer may be gone, and its memory with it: after a wait that ran out
  // nothing of any peer is read and nothing is written; the status word tells the host.
  if (gave_up) return;
  const int64_t base = static_cast<int64_t>(blockIdx.x) * a.n;
  float ss = 0.0f;
  for (int i = tid * 4; i < a.n; i += blockDim.x * 4) {
    // every rank's four values requested before any is used (one NVLink round trip, not `world`)
    float4 v[kTpMaxWorld];
#pragma unroll
    for (int r = 0; r < kTpMaxWorld; ++r)
      v[r] = r < a.world ? ld_relaxed_sys_f4(a.partial[r] + base + i) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    const uint2 xraw = *reinterpret_cast<const uint2*>(a.x + base + i);
    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
    for (int r = 0; r < kTpMaxWorld; ++r) {   // rank order on every rank: identical sums everywhere
      if (r < a.world) {
        acc.x += v[r].x;
        acc.y += v[r].y;
        acc.z += v[r].z;
        acc.w += v[r].w;
      }
    }
    const float y[4] = {acc.x, acc.y, acc.z, acc.w};
    const float xo[4] = {bf16_lo(xraw.x), bf16_hi(xraw.x), bf16_lo(xraw.y), bf16_hi(xraw.y)};
    float o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      o[j] = bf16_round(xo[j] + bf16_round(y[j]));
      row[i + j] = o[j];
      ss = fmaf(o[j], o[j], ss);
    }
    *reinterpret_cast<uint2*>(a.x + base + i) = make_uint2(pack_bf16(o[0], o[1]), pack_bf16(o[2], o[3]));
  }
  ss = warp_sum(ss);
  if ((tid & 31) == 0) scratch[tid >> 5] = ss;
  __syncthreads();
  float t = (tid & 31) < (blockDim.x >> 5) ? scratch[tid & 31] : 0.0f;
  t = warp_sum(t);
  const float r = 1.0f / sqrtf(t / static_cast<float>(a.n) + a.eps);
  for (int i = tid; i < a.n; i += blockDim.x)
    a.h[base + i] = __float2bfloat16_rn((row[i] * r) * __bfloat162float(a.gain[i]));
  // the last CTA to finish closes the exchange
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    if (atomicAdd(a.done, 1u) == gridDim.x - 1) {
      *a.done = 0u;
      __threadfence();
      st_release_sys(a.seq, seq);
    }
  }
}

size_t BlockBytes(int64_t cap, int world) {
  return static_cast<size_t>(2 + 4 * world + 2) * cap * sizeof(float) + 2 * (kTpMaxWorld + 2) * sizeof(uint32_t);
}
uint2* PushedOf(void* block, int64_t cap) { return reinterpret_cast<uint2*>(static_cast<float*>(block) + 2 * cap); }
uint2* BcastOf(void* block, int64_t cap, int world) {
  return reinterpret_cast<uint2*>(static_cast<float*>(block) + static_cast<size_t>(2 + 4 * world) * cap);
}
uint32_t* FlagsOf(void* block, int64_t cap, int world) {
  return reinterpret_cast<uint32_t*>(static_cast<float*>(block) + static_cast<size_t>(2 + 4 * world + 2) * cap);
}
uint32_t* PushFlagsOf(void* block, int64_t cap, int world) { return FlagsOf(block, cap, world) + kTpMaxWorld + 2; }

}  // namespace

namespace b200 {

b200_status TpAllReduce(b200_tp* tp, cudaStream_t stream, void* buf, int64_t count, int dtype) {
  if (tp == nullptr || tp->comm == nullptr) return Fail(B200_INVALID_ARGUMENT, "all-reduce: null group");
  b200_status s = BeginLaunch(tp->ctx);
  if (s != B200_OK) return s;
  if (count < 0) return Fail(B200_INVALID_ARGUMENT, "all-reduce: negative count");
  if (count == 0) return B200_OK;
  if (buf == nullptr) return Fail(B200_INVALID_ARGUMENT, "all-reduce: null buffer");
  ncclResult_t r = Api()->AllReduce(buf, buf, static_cast<size_t>(count), dtype == B200_F32 ? ncclFloat32 : ncclBfloat16,
                                    ncclSum, static_cast<ncclComm_t>(tp->comm), stream);
  if (r != ncclSuccess) return NcclFail(tp->ctx, "ncclAllReduce", r);
  return B200_OK;
}

b200_status TpAllGather(b200_tp* tp, cudaStream_t stream, const void* send, void* recv, int64_t count_per_rank,
                        int dtype) {
  if (tp == nullptr || tp->comm == nullptr) return Fail(B200_INVALID_ARGUMENT, "all-gather: null group");
  b200_status s = BeginLaunch(tp->ctx);
  if (s != B200_OK) return s;
  if (count_per_rank < 0) return Fail(B200_INVALID_ARGUMENT, "all-gather: negative count");
  if (count_per_rank == 0) return B200_OK;
  if (send == nullptr || recv == nullptr) return Fail(B200_INVALID_ARGUMENT, "all-gather: null buffer");
  ncclResult_t r = Api()->AllGather(send, recv, static_cast<size_t>(count_per_rank),
                                    dtype == B200_F32 ? ncclFloat32 : ncclBfloat16,
                                    static_cast<ncclComm_t>(tp->comm), stream);
  if (r != ncclSuccess) return NcclFail(tp->ctx, "ncclAllGather", r);
  return B200_OK;
}

bool TpPushLink(b200_tp* tp, QmmTp* out) {
  if (tp == nullptr || !tp->peer || out == nullptr || tp->cap % 8 != 0) return false;   // (16-byte reads of the lines)
  *out = QmmTp();
  out->world = tp->world;
  out->rank = tp->rank;
  out->cap = tp->cap;
  uint32_t* pf = PushFlagsOf(tp->block, tp->cap, tp->world);
  out->count = pf + kTpMaxWorld;
  out->done = pf + kTpMaxWorld + 1;
  out->src = PushedOf(tp->block, tp->cap);
  out->bcast = BcastOf(tp->block, tp->cap, tp->world);
  for (int r = 0; r < tp->world; ++r) {
    out->dst[r] = PushedOf(tp->peer_block[r], tp->cap) + static_cast<int64_t>(tp->rank) * tp->cap;
  }
  return true;
}

float* TpPeerPartial(b200_tp* tp, int slot) {
  if (tp == nullptr || !tp->peer || slot < 0 || slot > 1) return nullptr;
  return static_cast<float*>(tp->block) + static_cast<int64_t>(slot) * tp->cap;
}

b200_status TpSumResidualNorm(b200_tp* tp, cudaStream_t stream, int slot, void* x, const void* gain, void* h,
                              int64_t batch, int64_t hidden, double eps) {
  if (tp == nullptr || !tp->peer) return Fail(B200_FAILED_PRECONDITION, "peer exchange is not connected");
  b200_status s = BeginLaunch(tp->ctx);
  if (s != B200_OK) return s;
  if (slot < 0 || slot > 1 || batch < 1 || hidden < 4 || hidden % 4 != 0 || batch * hidden > tp->cap)
    return Fail(B200_INVALID_ARGUMENT, "peer exchange: batch %lld x hidden %lld does not fit (capacity %lld floats, hidden %% 4)",
                static_cast<long long>(batch), static_cast<long long>(hidden), static_cast<long long>(tp->cap));
  if (x == nullptr || gain == nullptr || h == nullptr || !Aligned(x, 8))
    return Fail(B200_INVALID_ARGUMENT, "peer exchange: null or misaligned buffer");
  PeerArgs a = {};
  for (int r = 0; r < tp->world; ++r) {
    a.partial[r] = static_cast<const float*>(tp->peer_block[r]) + static_cast<int64_t>(slot) * tp->cap;
    a.peer_flags[r] = FlagsOf(tp->peer_block[r], tp->cap, tp->world);
  }
  a.flags = FlagsOf(tp->block, tp->cap, tp->world);
  a.seq = a.flags + kTpMaxWorld;
  a.done = a.flags + kTpMaxWorld + 1;
  a.rank = tp->rank;
  a.world = tp->world;
  a.x = static_cast<__nv_bfloat16*>(x);
  a.gain = static_cast<const __nv_bfloat16*>(gain);
  a.h = static_cast<__nv_bfloat16*>(h);
  a.n = static_cast<int>(hidden);
  a.eps = static_cast<float>(eps);
  a.status = tp->ctx->dev_status;
  LaunchCfg lc;
  lc.grid = dim3(static_cast<unsigned>(batch));
  lc.block = dim3(static_cast<unsigned>(std::min<int64_t>(1024, (hidden / 4 + 31) / 32 * 32)));
  lc.smem = static_cast<size_t>(hidden) * sizeof(float);
  lc.stream = stream;
  lc.pdl = true;
  cudaError_t e = cudaFuncSetAttribute(peer_sum_residual_norm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(lc.smem));
  if (e == cudaSuccess) e = Launch(lc, peer_sum_residual_norm_kernel, a);
  if (e != cudaSuccess) return Stick(tp->ctx, Fail(B200_INTERNAL, "peer exchange launch: %s", cudaGetErrorString(e)));
  return EndLaunch(tp->ctx, "peer exchange");
}

}  // namespace b200

extern "C" {

b200_status b200_tp_peer_alloc(b200_tp* tp, int64_t max_floats, void* handle_out) {
  static_assert(sizeof(cudaIpcMemHandle_t) == B200_TP_PEER_HANDLE_BYTES, "IPC handle size");
  if (tp == nullptr || handle_out == nullptr) return Fail(B200_INVALID_ARGUMENT, "b200_tp_peer_alloc: null argument");
  b200_status s = BeginLaunch(tp->ctx);
  if (s != B200_OK) return s;
  if (tp->block != nullptr) return Fail(B200_FAILED_PRECONDITION, "b200_tp_peer_alloc: already allocated");
  if (max_floats < 4 || tp->world > kTpMaxWorld)
    return Fail(B200_INVALID_ARGUMENT, "b200_tp_peer_alloc: capacity %lld, world %d (at most %d ranks)",
                static_cast<long long>(max_floats), tp->world, kTpMaxWorld);
  const int64_t cap = (max_floats + 3) / 4 * 4;
  void* block = nullptr;
  cudaError_t e = cudaMalloc(&block, BlockBytes(cap, tp->world));
  if (e == cudaSuccess) e = cudaMemset(block, 0, BlockBytes(cap, tp->world));
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, block);
  if (e != cudaSuccess) {
    if (block != nullptr) cudaFree(block);
    (void)cudaGetLastError();
    return Fail(B200_RESOURCE_EXHAUSTED, "b200_tp_peer_alloc: %s", cudaGetErrorString(e));
  }
  tp->block = block;
  tp->cap = cap;
  std::memcpy(handle_out, &h, sizeof(h));
  return B200_OK;
}

b200_status b200_tp_peer_connect(b200_tp* tp, const void* handles) {
  if (tp == nullptr || handles == nullptr) return Fail(B200_INVALID_ARGUMENT, "b200_tp_peer_connect: null argument");
  b200_status s = BeginLaunch(tp->ctx);
  if (s != B200_OK) return s;
  if (tp->block == nullptr) return Fail(B200_FAILED_PRECONDITION, "b200_tp_peer_connect before b200_tp_peer_alloc");
  if (tp->peer) return Fail(B200_FAILED_PRECONDITION, "b200_tp_peer_connect: already connected");
  for (int r = 0; r < tp->world; ++r) {
    if (r == tp->rank) {
      tp->peer_block[r] = tp->block;
      continue;
    }
    cudaIpcMemHandle_t h;
    std::memcpy(&h, static_cast<const char*>(handles) + static_cast<size_t>(r) * sizeof(h), sizeof(h));
    void* mapped = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&mapped, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
      (void)cudaGetLastError();
      for (int q = 0; q < r; ++q)
        if (q != tp->rank && tp->peer_block[q] != nullptr) cudaIpcCloseMemHandle(tp->peer_block[q]);
      for (void*& pb : tp->peer_block) pb = nullptr;
      return Fail(B200_FAILED_PRECONDITION, "b200_tp_peer_connect: rank %d's block cannot be mapped: %s", r,
                  cudaGetErrorString(e));
    }
    tp->peer_block[r] = mapped;
  }
  tp->peer = true;
  return B200_OK;
}

void* b200_tp_peer_partial(b200_tp* tp, int slot) { return TpPeerPartial(tp, slot); }

b200_status b200_tp_sum_residual_norm(b200_tp* tp, b200_stream stream, int slot, void* x, const void* gain, void* h,
                                      int64_t batch, int64_t hidden, double eps) {
  return TpSumResidualNorm(tp, stream, slot, x, gain, h, batch, hidden, eps);
}

b200_status b200_tp_make_id(void* id_bytes) {
  static_assert(sizeof(ncclUniqueId) == B200_TP_ID_BYTES, "group id size");
  if (id_bytes == nullptr) return Fail(B200_INVALID_ARGUMENT, "b200_tp_make_id: null buffer");
  NcclApi* api = Api();
  if (api == nullptr) return Fail(B200_FAILED_PRECONDITION, "NCCL (libnccl.so.2) could not be loaded: %s", dlerror());
  ncclUniqueId id;
  ncclResult_t r = api->GetUniqueId(&id);
  if (r != ncclSuccess) return Fail(B200_INTERNAL, "ncclGetUniqueId: %s", api->GetErrorString(r));
  std::memcpy(id_bytes, &id, sizeof(id));
  return B200_OK;
}

b200_status b200_tp_create(b200_context* ctx, const void* id_bytes, int rank, int world, b200_tp** out) {
  if (out == nullptr) return Fail(B200_INVALID_ARGUMENT, "b200_tp_create: null out");
  *out = nullptr;
  b200_status s = BeginLaunch(ctx);
  if (s != B200_OK) return s;
  if (id_bytes == nullptr || world < 1 || rank < 0 || rank >= world)
    return Fail(B200_INVALID_ARGUMENT, "b200_tp_create: bad rank %d / world %d", rank, world);
  NcclApi* api = Api();
  if (api == nullptr) return Fail(B200_FAILED_PRECONDITION, "NCCL (libnccl.so.2) could not be loaded");
  ncclUniqueId id;
  std::memcpy(&id, id_bytes, sizeof(id));
  ncclComm_t comm = nullptr;
  ncclResult_t r = api->CommInitRank(&comm, world, id, rank);
  if (r != ncclSuccess) return NcclFail(ctx, "ncclCommInitRank", r);
  b200_tp* tp = new b200_tp();
  tp->ctx = ctx;
  tp->comm = comm;
  tp->rank = rank;
  tp->world = world;
  *out = tp;
  return B200_OK;
}

void b200_tp_destroy(b200_tp* tp) {
  if (tp == nullptr) return;
  if (tp->block != nullptr) {
    cudaSetDevice(tp->ctx->device);
    for (int r = 0; r < tp->world; ++r)
      if (r != tp->rank && tp->peer_block[r] != nullptr) cudaIpcCloseMemHandle(tp->peer_block[r]);
    cudaFree(tp->block);
  }
  if (tp->comm != nullptr && Api() != nullptr) Api()->CommDestroy(static_cast<ncclComm_t>(tp->comm));
  delete tp;
}

b200_status b200_tp_all_reduce_bf16(b200_tp* tp, b200_stream stream, void* buf, int64_t count) {
  return TpAllReduce(tp, stream, buf, count, B200_BF16);
}

b200_status b200_tp_all_gather_f32(b200_tp* tp, b200_stream stream, const void* send, void* recv,
                                   int64_t count_per_rank) {
  return TpAllGather(tp, stream, send, recv, count_per_rank, B200_F32);
}

}  // extern "C"
