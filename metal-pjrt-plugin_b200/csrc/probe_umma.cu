// Measurement only: how many SM cycles one tcgen05.mma costs, by shape.  One CTA, one issuing
// thread, `count` instructions back to back, then a commit and a bounded wait on its mbarrier.
// The answer on B200 (about 194 cycles whatever N, M, kind or A source) is why the int4 product
// for a handful of rows stays on mma.sync (see qmm_tc.cu).
#include "common.cuh"

using namespace b200;

namespace {

__device__ __forceinline__ uint64_t probe_desc(uint32_t a, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((a & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>(lbo >> 4) << 16;
  d |= static_cast<uint64_t>(sbo >> 4) << 32;
  d |= 1ull << 46;
  return d;
}

template <int KIND>   // 0: kind::f8f6f4 (e4m3), 1: kind::f16 (bf16)
__global__ void umma_rate_kernel(int M, int N, int a_tmem, int nd, int count, long long* out, int* status) {
  extern __shared__ __align__(1024) uint8_t smem[];
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_s;
  const int tid = threadIdx.x;
  for (int i = tid; i < 48 * 1024 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = KIND ? 0x3c003c00u : 0x38383838u;
  if (tid == 0) {
    mbar_init(&bar, 1);
    mbar_fence_init();
  }
  if (tid < 32) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_s)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = tmem_s;
  if (tid == 0) {
    const uint32_t idesc = (1u << 4) | (KIND ? ((1u << 7) | (1u << 10)) : 0u) | (static_cast<uint32_t>(N >> 3) << 17) |
                           (static_cast<uint32_t>(M >> 4) << 24);
    const uint64_t db = probe_desc(smem_u32(smem), 128, 256);
    const uint64_t da = probe_desc(smem_u32(smem) + 16384, 128, 256);
    const uint32_t d_cols = static_cast<uint32_t>(N > 16 ? N : 16);
    const long long t0 = clock64();
    for (int i = 0; i < count; ++i) {
      const uint32_t d = tmem + 256u + (static_cast<uint32_t>(i % nd) * d_cols) % 256u;
      const uint32_t acc = i >= nd ? 1u : 0u;
      if (a_tmem) {
        const uint32_t at = tmem + static_cast<uint32_t>(i % 4) * 8u;
        if (KIND == 0)
          asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d), "r"(at), "l"(db), "r"(idesc), "r"(acc) : "memory");
        else
          asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d), "r"(at), "l"(db), "r"(idesc), "r"(acc) : "memory");
      } else {
        if (KIND == 0)
          asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}" ::"r"(d), "l"(da), "l"(db), "r"(idesc), "r"(acc) : "memory");
        else
          asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d), "l"(da), "l"(db), "r"(idesc), "r"(acc) : "memory");
      }
    }
    const long long t1 = clock64();
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&bar)) : "memory");
    if (!mbar_wait_bounded(&bar, 0)) report_timeout(status, 910);
    const long long t2 = clock64();
    out[0] = t1 - t0;
    out[1] = t2 - t0;
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (tid < 32) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
  }
}

}  // namespace

extern "C" b200_status b200_probe_umma_rate(b200_context* ctx, b200_stream stream, int kind, int m, int n, int a_from_tmem,
                                            int accumulators, int count, int64_t* cycles_device) {
  b200_status s = BeginLaunch(ctx);
  if (s != B200_OK) return s;
  const bool shape_ok = (m == 128 && n % 16 == 0 && n >= 16 && n <= 256) || (m == 64 && n % 8 == 0 && n >= 8 && n <= 256);
  if ((kind != 0 && kind != 1) || !shape_ok || accumulators < 1 || accumulators > 8 || count < 1 || count > 4096 ||
      cycles_device == nullptr || accumulators * (n > 16 ? n : 16) > 256)
    return Fail(B200_INVALID_ARGUMENT, "b200_probe_umma_rate: kind 0/1, M 64 (N %% 8) or 128 (N %% 16), N <= 256, 1..8 accumulators within 256 columns, 1..4096 instructions");
  auto k0 = umma_rate_kernel<0>;
  auto k1 = umma_rate_kernel<1>;
  cudaError_t e = cudaFuncSetAttribute(kind == 0 ? k0 : k1, cudaFuncAttributeMaxDynamicSharedMemorySize, 60 * 1024);
  if (e != cudaSuccess) return Stick(ctx, Fail(B200_INTERNAL, "b200_probe_umma_rate: %s", cudaGetErrorString(e)));
  if (kind == 0)
    umma_rate_kernel<0><<<1, 128, 60 * 1024, stream>>>(m, n, a_from_tmem, accumulators, count, reinterpret_cast<long long*>(cycles_device), ctx->dev_status);
  else
    umma_rate_kernel<1><<<1, 128, 60 * 1024, stream>>>(m, n, a_from_tmem, accumulators, count, reinterpret_cast<long long*>(cycles_device), ctx->dev_status);
  return EndLaunch(ctx, "b200_probe_umma_rate");
}
