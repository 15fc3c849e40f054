// Tensor-parallel group over NCCL (NVLink 5 / NVSwitch), one process per GPU.
// The reference is single-device (its collectives are a stub,
// metal_pjrt/compiler/metal_collectives_registration.cc:10-17); this is new.
// NCCL is looked up with dlopen when the first group is made, so the library
// itself links nothing but the CUDA runtime.  The caller moves the 128-byte
// group id between processes by whatever transport it has.
#include <dlfcn.h>
#include <nccl.h>

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

}  // namespace b200

extern "C" {

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
