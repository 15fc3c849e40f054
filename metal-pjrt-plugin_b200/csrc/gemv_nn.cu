// Few-row dense product with the weights stored [K][N] (N contiguous):
//   D[m, n] = act(alpha * sum_k A[m, k] B[k, n] + bias[n]),  m < M <= 8.
// This is the NN layout of the benchmark's bf16 GEMM sweep at M = 1 and 16, where the
// op is a stream over B (bandwidth-bound), not a contraction for the tensor cores: the
// counterpart of the reference's few-row kernel (metal_pjrt/kernels/gemv.metal:72-176),
// which only takes the K-contiguous (NT) layout.
//
// A warp reads whole rows of B with coalesced 4/8/16-byte loads (a lane owns 2/4/8
// adjacent columns and all M rows of the output for them: 64 f32 accumulators), the
// eight warps of a CTA split the CTA's K range, a cluster of CTAs splits K further;
// partial sums meet in shared memory and then across the cluster's distributed shared
// memory, where the fused epilogue (steel_gemm.metal:217-225) is applied once.
#include <cooperative_groups.h>

#include <algorithm>

#include "common.cuh"

namespace cg = cooperative_groups;
using namespace b200;

namespace {

// Small CTAs (several fit an SM), so that the clusters of 8 pack onto every GPC in one wave.
constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;

struct NnArgs {
  const void* a;      // [M][lda]
  const void* b;      // [K][ldb]
  void* d;            // [M][ldd]
  const void* bias;
  void* aux;
  int m, n, k;
  int64_t lda, ldb, ldd;
  int k_per_cta;
  float alpha;
  int act;
};

// CT adjacent elements of a row of B as one 4/8/16-byte load, kept raw until used.
template <int CT> struct RawCols;
template <> struct RawCols<8> { uint4 v; };
template <> struct RawCols<4> { uint2 v; };
template <> struct RawCols<2> { uint32_t v; };

template <typename T, int CT>
__device__ __forceinline__ RawCols<CT> load_raw(const T* p) {
  RawCols<CT> r;
  if constexpr (CT == 8) r.v = __ldg(reinterpret_cast<const uint4*>(p));
  else if constexpr (CT == 4) r.v = __ldg(reinterpret_cast<const uint2*>(p));
  else r.v = __ldg(reinterpret_cast<const uint32_t*>(p));
  return r;
}

template <typename T, int CT>
__device__ __forceinline__ void unpack_cols(const RawCols<CT>& r, float (&v)[CT]) {
  const T* e = reinterpret_cast<const T*>(&r.v);
#pragma unroll
  for (int i = 0; i < CT; ++i) v[i] = load_as_f32<T>(e + i);
}

template <int BYTES>
__device__ __forceinline__ void cp_async(uint32_t dst, const void* src, int src_bytes) {
  if constexpr (BYTES == 16)
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
  else
    asm volatile("cp.async.ca.shared.global [%0], [%1], %2, %3;" ::"r"(dst), "l"(src), "n"(BYTES), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <int CT>
__device__ __forceinline__ RawCols<CT> lds_raw(uint32_t addr) {
  RawCols<CT> r;
  if constexpr (CT == 8)
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(r.v.x), "=r"(r.v.y), "=r"(r.v.z), "=r"(r.v.w) : "r"(addr));
  else if constexpr (CT == 4)
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(r.v.x), "=r"(r.v.y) : "r"(addr));
  else
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(r.v) : "r"(addr));
  return r;
}

constexpr int kStages = 4;        // ring depth per thread
constexpr int kRowsPerStage = 8;  // rows of B per stage: 24 copies in flight per thread
constexpr int kRowsPerRound = kRowsPerStage * kWarps;

// MT rows of the output per thread (M <= MT), CT adjacent columns per lane.  Every
// thread streams its own CT columns of B through a private ring in shared memory
// with cp.async, so the bytes in flight do not depend on how the compiler orders loads.
template <typename TIn, typename TOut, int MT, int CT>
__global__ void __launch_bounds__(kThreads) gemv_nn_kernel(const NnArgs p) {
  constexpr int kCols = 32 * CT;   // columns per CTA
  constexpr int CTB = CT * static_cast<int>(sizeof(TIn));
  extern __shared__ __align__(16) float smem_f[];
  const int rounds = (p.k_per_cta + kRowsPerRound - 1) / kRowsPerRound;
  float* As = smem_f;                                               // [rounds * 64][MT], zero beyond k_len
  float* ring = smem_f + static_cast<size_t>(rounds) * kRowsPerRound * MT;
  float* red = ring;   // after the stream: [kWarps][MT][kCols], then the CTA's sum in warp 0's slice
  pdl_wait();
  pdl_launch_dependents();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n0 = blockIdx.x * kCols + lane * CT;
  const int k_begin = blockIdx.y * p.k_per_cta;
  const int k_len = max(0, min(p.k_per_cta, p.k - k_begin));
  const TIn* A = static_cast<const TIn*>(p.a);
  const TIn* bp = static_cast<const TIn*>(p.b) + static_cast<int64_t>(k_begin) * p.ldb + n0;
  const bool active = n0 < p.n;
  const uint32_t ring_thread = smem_u32(ring) + static_cast<uint32_t>((warp * kStages * kRowsPerStage * 32 + lane) * CTB);

  auto issue = [&](int j) {
    if (active && j < rounds) {
      const int s = j % kStages;
#pragma unroll
      for (int r = 0; r < kRowsPerStage; ++r) {
        const int kk = (j * kRowsPerStage + r) * kWarps + warp;
        const bool ok = kk < k_len;
        cp_async<CTB>(ring_thread + static_cast<uint32_t>((s * kRowsPerStage + r) * 32 * CTB),
                      bp + static_cast<int64_t>(ok ? kk : 0) * p.ldb, ok ? CTB : 0);
      }
    }
    cp_async_commit();
  };
#pragma unroll
  for (int j = 0; j < kStages - 1; ++j) issue(j);

  // this CTA's slice of A as f32, [k][MT], while the first copies fly
  const int k_pad = rounds * kRowsPerRound;
  if ((p.lda % 8) == 0 && (k_begin % 8) == 0 && (reinterpret_cast<uintptr_t>(A) & 15) == 0) {
    const int chunks = k_len / 8;
    for (int i = tid; i < chunks * MT; i += kThreads) {
      const int m = i / chunks, c = i - m * chunks;
      float v[8];
      if (m < p.m) {
        unpack_cols<TIn, 8>(load_raw<TIn, 8>(A + static_cast<int64_t>(m) * p.lda + k_begin + c * 8), v);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = 0.0f;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) As[(c * 8 + j) * MT + m] = v[j];
    }
    for (int i = chunks * 8 * MT + tid; i < k_pad * MT; i += kThreads) {
      const int kk = i / MT, m = i - kk * MT;
      As[i] = (m < p.m && kk < k_len) ? load_as_f32<TIn>(A + static_cast<int64_t>(m) * p.lda + k_begin + kk) : 0.0f;
    }
  } else {
    for (int i = tid; i < k_pad * MT; i += kThreads) {
      const int kk = i / MT, m = i - kk * MT;
      As[i] = (m < p.m && kk < k_len) ? load_as_f32<TIn>(A + static_cast<int64_t>(m) * p.lda + k_begin + kk) : 0.0f;
    }
  }
  __syncthreads();

  float acc[MT][CT];
#pragma unroll
  for (int m = 0; m < MT; ++m)
#pragma unroll
    for (int c = 0; c < CT; ++c) acc[m][c] = 0.0f;
  for (int j = 0; j < rounds; ++j) {
    cp_async_wait<kStages - 2>();
    if (active) {
      const int s = j % kStages;
#pragma unroll
      for (int r = 0; r < kRowsPerStage; ++r) {
        float bv[CT];
        unpack_cols<TIn, CT>(lds_raw<CT>(ring_thread + static_cast<uint32_t>((s * kRowsPerStage + r) * 32 * CTB)), bv);
        const float* ar = As + ((j * kRowsPerStage + r) * kWarps + warp) * MT;
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          const float av = ar[m];
#pragma unroll
          for (int c = 0; c < CT; ++c) acc[m][c] = fmaf(av, bv[c], acc[m][c]);
        }
      }
    }
    issue(j + kStages - 1);
  }
  cp_async_wait<0>();
  __syncthreads();   // every thread is done with its ring before the ring becomes `red`
  // the warps' partial tiles, then their sum into warp 0's slice
#pragma unroll
  for (int m = 0; m < MT; ++m)
#pragma unroll
    for (int c = 0; c < CT; ++c) red[(warp * MT + m) * kCols + lane * CT + c] = acc[m][c];
  __syncthreads();
  for (int i = tid; i < MT * kCols; i += kThreads) {
    float v = red[i];
#pragma unroll
    for (int w = 1; w < kWarps; ++w) v += red[w * MT * kCols + i];
    red[i] = v;
  }
  __syncthreads();

  cg::cluster_group cluster = cg::this_cluster();
  const int split = gridDim.y;
  if (split > 1) cluster.sync();
  // rank r finishes rows m = r, r + split, ... of this column block
  for (int i = tid; i < MT * kCols; i += kThreads) {
    const int m = i / kCols, c = i - m * kCols;
    const int n = blockIdx.x * kCols + c;
    if (m % split != static_cast<int>(blockIdx.y) || m >= p.m || n >= p.n) continue;
    float v = 0.0f;
    if (split > 1) {
      for (int r = 0; r < split; ++r) v += cluster.map_shared_rank(red, r)[i];
    } else {
      v = red[i];
    }
    v *= p.alpha;
    if (p.bias != nullptr) v += load_as_f32<TOut>(static_cast<const TOut*>(p.bias) + n);
    const int64_t o = static_cast<int64_t>(m) * p.ldd + n;
    if (p.aux != nullptr) static_cast<TOut*>(p.aux)[o] = store_from_f32<TOut>(v);
    static_cast<TOut*>(p.d)[o] = store_from_f32<TOut>(apply_act(p.act, v));
  }
  if (split > 1) cluster.sync();
}

template <typename TIn, typename TOut, int MT, int CT>
cudaError_t LaunchNn(const NnArgs& a, int split, size_t smem, cudaStream_t stream) {
  auto kernel = gemv_nn_kernel<TIn, TOut, MT, CT>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (e != cudaSuccess) return e;
  LaunchCfg lc;
  lc.grid = dim3(static_cast<unsigned>(CeilDiv(a.n, 32 * CT)), split, 1);
  lc.block = dim3(kThreads);
  lc.smem = smem;
  lc.stream = stream;
  lc.pdl = true;
  lc.cluster_y = split;
  return Launch(lc, kernel, a);
}

template <typename TIn, typename TOut>
cudaError_t LaunchRows(const NnArgs& a, int mt, int split, size_t smem, cudaStream_t stream) {
  if (mt == 2) return LaunchNn<TIn, TOut, 2, 8>(a, split, smem, stream);
  return LaunchNn<TIn, TOut, 8, 8>(a, split, smem, stream);
}

}  // namespace

namespace b200 {

bool FewRowNnSupports(const b200_gemm_params* p) {
  if (p->a.transpose || p->b.transpose || p->batch != 1 || p->beta != 0.0) return false;
  if (p->a.dtype != B200_BF16 && p->a.dtype != B200_F16) return false;
  if (p->m < 1 || p->m > 8 || p->k < 512 || p->n < 256) return false;
  if (p->n % 8 != 0 || p->b.ld % 8 != 0 || !Aligned(p->b.ptr, 16)) return false;
  return true;
}

b200_status RunFewRowNn(b200_context* ctx, cudaStream_t stream, const b200_gemm_params* p, const b200_epilogue* epi) {
  NnArgs a;
  a.a = p->a.ptr;
  a.b = p->b.ptr;
  a.d = p->c.ptr;
  a.bias = epi->bias;
  a.aux = epi->aux;
  a.m = static_cast<int>(p->m);
  a.n = static_cast<int>(p->n);
  a.k = static_cast<int>(p->k);
  a.lda = p->a.ld;
  a.ldb = p->b.ld;
  a.ldd = p->c.ld;
  a.alpha = static_cast<float>(p->alpha);
  a.act = epi->act;
  const int mt = a.m <= 2 ? 2 : 8;
  const int ct = mt <= 8 ? 8 : 64 / mt;
  const int cols = 32 * ct;
  const int blocks = static_cast<int>(CeilDiv(a.n, cols));
  int split = 1;
  while (split < 8 && blocks * split < 2 * ctx->sm_count && a.k / (split * 2) >= 256) split *= 2;
  a.k_per_cta = static_cast<int>(CeilDiv(a.k, split));
  const size_t a_bytes = static_cast<size_t>(CeilDiv(a.k_per_cta, kRowsPerRound)) * kRowsPerRound * mt * sizeof(float);
  const size_t ring_bytes = static_cast<size_t>(kThreads) * kStages * kRowsPerStage * ct * 2;
  const size_t red_bytes = static_cast<size_t>(kWarps) * mt * cols * sizeof(float);
  const size_t smem = a_bytes + std::max(ring_bytes, red_bytes);
  if (smem > static_cast<size_t>(ctx->max_smem_optin))
    return Fail(B200_UNIMPLEMENTED, "b200_gemm (few-row NN): K = %d needs %zu bytes of shared memory", a.k, smem);
  cudaError_t e;
  const bool bf = p->a.dtype == B200_BF16;
  if (p->c.dtype == B200_F32)
    e = bf ? LaunchRows<__nv_bfloat16, float>(a, mt, split, smem, stream) : LaunchRows<__half, float>(a, mt, split, smem, stream);
  else if (bf)
    e = LaunchRows<__nv_bfloat16, __nv_bfloat16>(a, mt, split, smem, stream);
  else
    e = LaunchRows<__half, __half>(a, mt, split, smem, stream);
  if (e != cudaSuccess) return Stick(ctx, Fail(B200_INTERNAL, "b200_gemm (few-row NN) launch: %s", cudaGetErrorString(e)));
  return EndLaunch(ctx, "b200_gemm (few-row NN)");
}

}  // namespace b200
