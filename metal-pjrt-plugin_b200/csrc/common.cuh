// Shared host/device helpers for the b200graft library (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <mutex>
#include <string>

#include "b200graft.h"

// ---------------------------------------------------------------------------
// Context and status plumbing
// ---------------------------------------------------------------------------

// Device status word layout (int32[4], zeroed at context creation):
//   [0] first error code reported by a kernel (b200_status), 0 = none
//   [1] id of the wait that gave up (kernel specific), [2],[3] spare
struct b200_context {
  int device = 0;
  int sm_count = 0;
  int max_smem_optin = 0;
  int* dev_status = nullptr;      // device memory, 4 ints
  int* host_status = nullptr;     // pinned mirror for asynchronous read-back
  std::atomic<int> sticky{0};     // b200_status
  std::atomic<int64_t> launches{0};
  std::atomic<int64_t> fail_at{0};  // absolute launch index to refuse, 0 = disarmed
  std::atomic<int> force_route{0};
  std::atomic<int> qmm_route{0};   // b200_qmm_force_route
  void* qmm_ws = nullptr;          // bf16 panel of dequantised weights (b200_qmm above 32 rows), grown on first use
  size_t qmm_ws_bytes = 0;
  // scratch of the tensor-core dequant-matmul: partial rows of tiles shared between CTAs, and per
  // tile how many CTAs have delivered theirs (zero between launches)
  float* qtc_parts = nullptr;
  size_t qtc_parts_floats = 0;
  unsigned* qtc_counters = nullptr;
  int qtc_tiles_max = 0;
  std::mutex mu;
  std::string sticky_message;
};

namespace b200 {

void SetError(const char* fmt, ...);
b200_status Fail(b200_status code, const char* fmt, ...);
// Records `code` as the context's sticky error (first one wins) and returns it.
b200_status Stick(b200_context* ctx, b200_status code);
// attention.cu: caches the device address of the built-in attention scratch for this context's device.
b200_status AttnStaticScratchInit(b200_context* ctx);
// Called by every entry point before it enqueues: returns the sticky error if
// one is set, applies host-side fault injection, makes the device current.
b200_status BeginLaunch(b200_context* ctx);
// Called after a launch: maps cudaGetLastError to a status (sticky on failure)
// and counts the launch.
b200_status EndLaunch(b200_context* ctx, const char* what, int kernels = 1);

inline int64_t CeilDiv(int64_t a, int64_t b) { return (a + b - 1) / b; }
inline bool Aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }
inline int DtypeSize(int dt) { return dt == B200_F32 ? 4 : 2; }

// B200_NO_PDL=1 launches every kernel with plain stream ordering (an A/B switch).
bool PdlDisabled();

// Launch helper: optional programmatic dependent launch (the kernel must call
// pdl_wait() before touching anything an earlier kernel wrote) and optional
// thread-block cluster along y.
struct LaunchCfg {
  dim3 grid, block;
  size_t smem = 0;
  cudaStream_t stream = nullptr;
  bool pdl = false;
  int cluster_y = 1;
};

template <typename... KArgs, typename... Args>
cudaError_t Launch(const LaunchCfg& lc, void (*kernel)(KArgs...), Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = lc.grid;
  cfg.blockDim = lc.block;
  cfg.dynamicSmemBytes = lc.smem;
  cfg.stream = lc.stream;
  cudaLaunchAttribute attrs[2];
  unsigned n = 0;
  if (lc.pdl && !PdlDisabled()) {
    attrs[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  if (lc.cluster_y > 1) {
    attrs[n].id = cudaLaunchAttributeClusterDimension;
    attrs[n].val.clusterDim.x = 1;
    attrs[n].val.clusterDim.y = lc.cluster_y;
    attrs[n].val.clusterDim.z = 1;
    ++n;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace b200

// ---------------------------------------------------------------------------
// Device helpers
// ---------------------------------------------------------------------------
#ifdef __CUDACC__
namespace b200 {

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ float bf16_bits_to_f32(uint32_t lo16) { return __uint_as_float(lo16 << 16); }
__device__ __forceinline__ float bf16_lo(uint32_t packed) { return __uint_as_float(packed << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t packed) { return __uint_as_float(packed & 0xffff0000u); }
__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float ldg_bf16(const void* p) {
  return bf16_bits_to_f32(__ldg(reinterpret_cast<const unsigned short*>(p)));
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// ---- mbarrier / bulk-copy wrappers (all waits are bounded) -----------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(0x989680u)   // let the hardware park the thread (hint: 10 ms)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// Waits for the phase with the given parity, bounded by ~4e9 SM cycles (about
// two seconds).  Returns false when it gave up; the caller reports B200_TIMEOUT
// through the status word and leaves the pipeline.  The SM cycle counter is
// read only after a few thousand failed polls (each poll may itself suspend the
// thread for a while), so the common case costs nothing but the polls.
// kSleepNs > 0 parks the warp between polls (a producer that is far ahead of its consumers
// should not compete with them for issue slots).
template <int kSleepNs = 0>
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
#pragma unroll 1
  for (int i = 0; i < 4096; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if (kSleepNs > 0) __nanosleep(kSleepNs);
  }
  const long long t0 = clock64();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 1024; ++i) {
      if (mbar_try_wait(bar, parity)) return true;
      if (kSleepNs > 0) __nanosleep(kSleepNs);
    }
    if (clock64() - t0 > 4000000000ll) return false;
  }
}
// Cluster-scope pair: one arrival (with release) on the same barrier in CTA `rank` of
// this cluster, and a bounded acquire-wait on this CTA's own barrier.  Used where CTAs
// of a cluster hand tiles to one another through distributed shared memory.
__device__ __forceinline__ void mbar_arrive_cluster(uint64_t* bar, uint32_t rank) {
  asm volatile(
      "{\n\t.reg .b32 ra;\n\t"
      "mapa.shared::cluster.u32 ra, %0, %1;\n\t"
      "mbarrier.arrive.release.cluster.shared::cluster.b64 _, [ra];\n\t}" ::"r"(smem_u32(bar)),
      "r"(rank)
      : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(0x989680u)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_bounded_cluster(uint64_t* bar, uint32_t parity) {
#pragma unroll 1
  for (int i = 0; i < 4096; ++i)
    if (mbar_try_wait_cluster(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 1024; ++i)
      if (mbar_try_wait_cluster(bar, parity)) return true;
    if (clock64() - t0 > 4000000000ll) return false;
  }
}
// 1-D bulk copy global -> this CTA's shared memory, completion on `bar`.
// dst, src 16-byte aligned; bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(dst)),
      "l"(src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
// First report wins: status[0] = code, status[1] = where (an id the reporting kernel chooses:
// 1xx/2xx/3xx the ring and cluster waits of the streaming kernels, 4xx peer exchanges,
// 5xx argument checks made on the device, 6xx the decode-stream kernel, 9xx the wait probe).
__device__ __forceinline__ void report_status(int* status, int code, int where) {
  if (status != nullptr && atomicCAS(status, 0, code) == 0) status[1] = where;
}
__device__ __forceinline__ void report_timeout(int* status, int where) {
  report_status(status, (int)B200_TIMEOUT, where);
}

// mma.sync m16n8k16, bf16 inputs, f32 accumulate (the few-row streaming path:
// weights are the 16-row operand, the batch is the 8-column operand).
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                               uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// d = a . b (no accumulator input: the zero registers cost no instruction)
__device__ __forceinline__ void mma_bf16_16816_z(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                 uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%10,%10,%10,%10};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
}

// Epilogue activation in f32 (formulas of metal_pjrt/kernels/steel_gemm.metal:58-66).
__device__ __forceinline__ float apply_act(int act, float x) {
  if (act == 1) return isnan(x) ? x : (x > 0.0f ? x : 0.0f);
  if (act == 2) {
    const float k = 0.7978845608028654f;
    return 0.5f * x * (1.0f + tanhf(k * (x + 0.044715f * x * x * x)));
  }
  if (act == 3) return x / (1.0f + expf(-x));
  return x;
}

template <typename T>
__device__ __forceinline__ float load_as_f32(const T* p);
template <>
__device__ __forceinline__ float load_as_f32<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float load_as_f32<__half>(const __half* p) { return __half2float(*p); }
template <>
__device__ __forceinline__ float load_as_f32<__nv_bfloat16>(const __nv_bfloat16* p) {
  return __bfloat162float(*p);
}
template <typename T>
__device__ __forceinline__ T store_from_f32(float v);
template <>
__device__ __forceinline__ float store_from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half store_from_f32<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 store_from_f32<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

}  // namespace b200
#endif  // __CUDACC__
