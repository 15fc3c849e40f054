// Row reductions over the minor dimension: RMSNorm, softmax, log_softmax,
// LayerNorm.  The reference has no kernel for these (XLA's reduction and loop
// emitters produce them from examples/llm/qwen3.py:294-297,325 and
// bench/jax_bench.py:44-46); this is one hand-written family.
//
// One pass over HBM.  Rows whose length is 32, 128, ... 1024 threads times 1, 2, 4 or 8
// 16-byte vectors (every shape of the benchmark configurations) stay in REGISTERS: all
// loads of a row are issued before the first is used, the statistics come from the
// registers (shuffles within a warp, one exchange through shared memory for a CTA per
// row), and the row is written once.  Other rows: a row is read once with 16-byte loads
// into shared memory as f32 while the first statistic is accumulated, the second statistic and
// the output come from shared memory, and the row is written once.  Short rows
// get a warp each (several rows per CTA, shuffle reductions only), long rows a
// CTA each; rows that do not fit shared memory fall back to re-reading global
// memory (L2-resident at those sizes).  Statistics are f32.
#include <type_traits>

#include "common.cuh"

using namespace b200;

namespace {

enum { kRms = 0, kSoftmax = 1, kLogSoftmax = 2, kLayerNorm = 3 };

struct RowArgs {
  const void* x;
  const void* gain;
  const void* beta;
  void* y;
  int64_t rows;
  int n;
  float eps;
};

__device__ __forceinline__ float nan_max(float a, float b) {
  return (a != a || b != b) ? __int_as_float(0x7fc00000) : fmaxf(a, b);
}

template <bool WARP>
__device__ __forceinline__ float group_sum(float v, float* scratch) {
  v = warp_sum(v);
  if (WARP) return v;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = lane < nw ? scratch[lane] : 0.0f;
  return warp_sum(r);
}

template <bool WARP>
__device__ __forceinline__ float group_nanmax(float v, float* scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = nan_max(v, __shfl_xor_sync(0xffffffffu, v, o));
  if (WARP) return v;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = lane < nw ? scratch[lane] : -INFINITY;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) r = nan_max(r, __shfl_xor_sync(0xffffffffu, r, o));
  return r;
}

template <typename T>
struct Vec {
  static constexpr int kN = 16 / sizeof(T);
};

template <typename T>
__device__ __forceinline__ void load_vec(const T* p, float (&out)[Vec<T>::kN]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
  for (int i = 0; i < Vec<T>::kN; ++i) out[i] = load_as_f32<T>(e + i);
}

template <typename T>
__device__ __forceinline__ void store_vec(T* p, const float (&v)[Vec<T>::kN]) {
  uint4 raw;
  T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
  for (int i = 0; i < Vec<T>::kN; ++i) e[i] = store_from_f32<T>(v[i]);
  *reinterpret_cast<uint4*>(p) = raw;
}

// The per-row work, done by a warp (WARP) or by the whole CTA.  `buf` holds the
// row as f32 (n floats) in shared memory.
template <typename T, int KIND, bool WARP, bool VEC>
__device__ __forceinline__ void do_row(const RowArgs& a, int64_t row, float* buf, float* scratch, int tid,
                                       int nthreads) {
  constexpr int V = Vec<T>::kN;
  const int n = a.n;
  const T* x = static_cast<const T*>(a.x) + row * n;
  T* y = static_cast<T*>(a.y) + row * n;
  const T* gain = static_cast<const T*>(a.gain);
  const T* beta = static_cast<const T*>(a.beta);

  // pass 0: global -> shared, first statistic
  float st = (KIND == kSoftmax || KIND == kLogSoftmax) ? -INFINITY : 0.0f;
  if (VEC) {
    for (int i = tid * V; i < n; i += nthreads * V) {
      float v[V];
      load_vec<T>(x + i, v);
#pragma unroll
      for (int j = 0; j < V; ++j) {
        buf[i + j] = v[j];
        if (KIND == kRms) st = fmaf(v[j], v[j], st);
        else if (KIND == kLayerNorm) st += v[j];
        else st = nan_max(st, v[j]);
      }
    }
  } else {
    for (int i = tid; i < n; i += nthreads) {
      const float v = load_as_f32<T>(x + i);
      buf[i] = v;
      if (KIND == kRms) st = fmaf(v, v, st);
      else if (KIND == kLayerNorm) st += v;
      else st = nan_max(st, v);
    }
  }
  if (KIND == kSoftmax || KIND == kLogSoftmax) st = group_nanmax<WARP>(st, scratch);
  else st = group_sum<WARP>(st, scratch);
  // buf writes of this thread are re-read only by this thread below (same
  // index pattern), so no barrier is needed between the passes.

  float scale = 1.0f, shift = 0.0f;
  if (KIND == kRms) {
    scale = 1.0f / sqrtf(st / static_cast<float>(n) + a.eps);
  } else if (KIND == kLayerNorm) {
    const float mean = st / static_cast<float>(n);
    float sq = 0.0f;
    if (VEC) {
      for (int i = tid * V; i < n; i += nthreads * V)
#pragma unroll
        for (int j = 0; j < V; ++j) {
          const float d = buf[i + j] - mean;
          sq = fmaf(d, d, sq);
        }
    } else {
      for (int i = tid; i < n; i += nthreads) {
        const float d = buf[i] - mean;
        sq = fmaf(d, d, sq);
      }
    }
    sq = group_sum<WARP>(sq, scratch);
    scale = 1.0f / sqrtf(sq / static_cast<float>(n) + a.eps);
    shift = mean;
  } else {
    float sum = 0.0f;
    if (VEC) {
      for (int i = tid * V; i < n; i += nthreads * V)
#pragma unroll
        for (int j = 0; j < V; ++j) {
          const float e = expf(buf[i + j] - st);
          if (KIND == kSoftmax) buf[i + j] = e;
          sum += e;
        }
    } else {
      for (int i = tid; i < n; i += nthreads) {
        const float e = expf(buf[i] - st);
        if (KIND == kSoftmax) buf[i] = e;
        sum += e;
      }
    }
    sum = group_sum<WARP>(sum, scratch);
    if (KIND == kSoftmax) scale = sum;  // divide, like the reference (not multiply by 1/sum)
    else { shift = st; scale = logf(sum); }
  }

  // final pass: shared -> global
  auto one = [&](int i) -> float {
    const float v = buf[i];
    if (KIND == kRms) return (v * scale) * load_as_f32<T>(gain + i);
    if (KIND == kSoftmax) return v / scale;
    if (KIND == kLogSoftmax) return (v - shift) - scale;
    float r = (v - shift) * scale;
    if (gain != nullptr) r *= load_as_f32<T>(gain + i);
    if (beta != nullptr) r += load_as_f32<T>(beta + i);
    return r;
  };
  if (VEC) {
    for (int i = tid * V; i < n; i += nthreads * V) {
      float v[V];
#pragma unroll
      for (int j = 0; j < V; ++j) v[j] = one(i + j);
      store_vec<T>(y + i, v);
    }
  } else {
    for (int i = tid; i < n; i += nthreads) y[i] = store_from_f32<T>(one(i));
  }
}

template <typename T, int KIND, bool VEC>
__global__ void rownorm_warp_kernel(const RowArgs a) {
  extern __shared__ __align__(16) float smem_f[];
  pdl_wait();
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  const int stride = (a.n + 3) & ~3;
  float* buf = smem_f + warp * stride;
  for (int64_t row = static_cast<int64_t>(blockIdx.x) * wpb + warp; row < a.rows;
       row += static_cast<int64_t>(gridDim.x) * wpb) {
    do_row<T, KIND, true, VEC>(a, row, buf, nullptr, lane, 32);
    __syncwarp();
  }
}

template <typename T, int KIND, bool VEC>
__global__ void rownorm_block_kernel(const RowArgs a) {
  extern __shared__ __align__(16) float smem_f[];
  __shared__ float scratch[32];
  pdl_wait();
  pdl_launch_dependents();
  for (int64_t row = blockIdx.x; row < a.rows; row += gridDim.x) {
    do_row<T, KIND, false, VEC>(a, row, smem_f, scratch, threadIdx.x, blockDim.x);
    __syncthreads();
  }
}

// Register-resident rows: n == threads-per-row * NV * (16 / sizeof(T)).  WARP: a warp per row,
// eight rows per CTA; else the whole CTA on one row.
template <typename T, int KIND, int NV, bool WARP>
__global__ void __launch_bounds__(WARP ? 256 : 1024) rownorm_reg_kernel(const RowArgs a) {
  constexpr int V = Vec<T>::kN;
  __shared__ float scratch[32];
  pdl_wait();
  pdl_launch_dependents();
  const int tpr = WARP ? 32 : static_cast<int>(blockDim.x);
  const int t = WARP ? static_cast<int>(threadIdx.x & 31) : static_cast<int>(threadIdx.x);
  const int wpb = blockDim.x >> 5;
  const int64_t row0 = WARP ? static_cast<int64_t>(blockIdx.x) * wpb + (threadIdx.x >> 5) : blockIdx.x;
  const int64_t rstride = WARP ? static_cast<int64_t>(gridDim.x) * wpb : gridDim.x;
  const T* gain = static_cast<const T*>(a.gain);
  const T* beta = static_cast<const T*>(a.beta);
  for (int64_t row = row0; row < a.rows; row += rstride) {
    const T* x = static_cast<const T*>(a.x) + row * a.n;
    T* y = static_cast<T*>(a.y) + row * a.n;
    float v[NV][V];
#pragma unroll
    for (int j = 0; j < NV; ++j) load_vec<T>(x + (j * tpr + t) * V, v[j]);
    float st = (KIND == kSoftmax || KIND == kLogSoftmax) ? -INFINITY : 0.0f;
#pragma unroll
    for (int j = 0; j < NV; ++j)
#pragma unroll
      for (int e = 0; e < V; ++e) {
        if (KIND == kRms) st = fmaf(v[j][e], v[j][e], st);
        else if (KIND == kLayerNorm) st += v[j][e];
        else st = nan_max(st, v[j][e]);
      }
    if (KIND == kSoftmax || KIND == kLogSoftmax) st = group_nanmax<WARP>(st, scratch);
    else st = group_sum<WARP>(st, scratch);
    float scale = 1.0f, shift = 0.0f;
    if (KIND == kRms) {
      scale = 1.0f / sqrtf(st / static_cast<float>(a.n) + a.eps);
    } else if (KIND == kLayerNorm) {
      const float mean = st / static_cast<float>(a.n);
      float sq = 0.0f;
#pragma unroll
      for (int j = 0; j < NV; ++j)
#pragma unroll
        for (int e = 0; e < V; ++e) {
          const float d = v[j][e] - mean;
          sq = fmaf(d, d, sq);
        }
      sq = group_sum<WARP>(sq, scratch);
      scale = 1.0f / sqrtf(sq / static_cast<float>(a.n) + a.eps);
      shift = mean;
    } else {
      float sum = 0.0f;
#pragma unroll
      for (int j = 0; j < NV; ++j)
#pragma unroll
        for (int e = 0; e < V; ++e) {
          const float ex = expf(v[j][e] - st);
          if (KIND == kSoftmax) v[j][e] = ex;
          sum += ex;
        }
      sum = group_sum<WARP>(sum, scratch);
      if (KIND == kSoftmax) scale = sum;   // divide, like the reference (not multiply by 1/sum)
      else { shift = st; scale = logf(sum); }
    }
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int i = (j * tpr + t) * V;
      float g[V], bt[V], o[V];
      if (KIND == kRms || (KIND == kLayerNorm && gain != nullptr)) load_vec<T>(gain + i, g);
      if (KIND == kLayerNorm && beta != nullptr) load_vec<T>(beta + i, bt);
#pragma unroll
      for (int e = 0; e < V; ++e) {
        if (KIND == kRms) o[e] = (v[j][e] * scale) * g[e];
        else if (KIND == kSoftmax) o[e] = v[j][e] / scale;
        else if (KIND == kLogSoftmax) o[e] = (v[j][e] - shift) - scale;
        else {
          float r = (v[j][e] - shift) * scale;
          if (gain != nullptr) r *= g[e];
          if (beta != nullptr) r += bt[e];
          o[e] = r;
        }
      }
      store_vec<T>(y + i, o);
    }
  }
}

// Rows too long for shared memory: statistics by re-reading global memory.
template <typename T, int KIND>
__global__ void rownorm_long_kernel(const RowArgs a) {
  __shared__ float scratch[32];
  pdl_wait();
  pdl_launch_dependents();
  const int n = a.n, tid = threadIdx.x, nt = blockDim.x;
  for (int64_t row = blockIdx.x; row < a.rows; row += gridDim.x) {
    const T* x = static_cast<const T*>(a.x) + row * n;
    T* y = static_cast<T*>(a.y) + row * n;
    const T* gain = static_cast<const T*>(a.gain);
    const T* beta = static_cast<const T*>(a.beta);
    float st = (KIND == kSoftmax || KIND == kLogSoftmax) ? -INFINITY : 0.0f;
    for (int i = tid; i < n; i += nt) {
      const float v = load_as_f32<T>(x + i);
      if (KIND == kRms) st = fmaf(v, v, st);
      else if (KIND == kLayerNorm) st += v;
      else st = nan_max(st, v);
    }
    if (KIND == kSoftmax || KIND == kLogSoftmax) st = group_nanmax<false>(st, scratch);
    else st = group_sum<false>(st, scratch);
    float scale = 1.0f, shift = 0.0f;
    if (KIND == kRms) {
      scale = 1.0f / sqrtf(st / static_cast<float>(n) + a.eps);
    } else if (KIND == kLayerNorm) {
      const float mean = st / static_cast<float>(n);
      float sq = 0.0f;
      for (int i = tid; i < n; i += nt) {
        const float d = load_as_f32<T>(x + i) - mean;
        sq = fmaf(d, d, sq);
      }
      sq = group_sum<false>(sq, scratch);
      scale = 1.0f / sqrtf(sq / static_cast<float>(n) + a.eps);
      shift = mean;
    } else {
      float sum = 0.0f;
      for (int i = tid; i < n; i += nt) sum += expf(load_as_f32<T>(x + i) - st);
      sum = group_sum<false>(sum, scratch);
      if (KIND == kSoftmax) { shift = st; scale = sum; }
      else { shift = st; scale = logf(sum); }
    }
    __syncthreads();  // y may alias x: every read of the row is done
    for (int i = tid; i < n; i += nt) {
      const float v = load_as_f32<T>(x + i);
      float r;
      if (KIND == kRms) r = (v * scale) * load_as_f32<T>(gain + i);
      else if (KIND == kSoftmax) r = expf(v - shift) / scale;
      else if (KIND == kLogSoftmax) r = (v - shift) - scale;
      else {
        r = (v - shift) * scale;
        if (gain != nullptr) r *= load_as_f32<T>(gain + i);
        if (beta != nullptr) r += load_as_f32<T>(beta + i);
      }
      y[i] = store_from_f32<T>(r);
    }
    __syncthreads();
  }
}

template <typename T, int KIND>
b200_status LaunchRows(b200_context* ctx, cudaStream_t stream, const RowArgs& a) {
  constexpr int V = Vec<T>::kN;
  const bool vec = (a.n % V == 0) && Aligned(a.x, 16) && Aligned(a.y, 16);
  const int stride = (a.n + 3) & ~3;
  LaunchCfg lc;
  lc.stream = stream;
  lc.pdl = true;
  cudaError_t e;
  // register-resident rows (f32 and bf16): threads per row x vectors per thread == vectors per row
  if (!std::is_same<T, __half>::value && vec && (a.gain == nullptr || Aligned(a.gain, 16)) && (a.beta == nullptr || Aligned(a.beta, 16))) {
    const int vecs = a.n / V;
    int tpr = 0, nv = 0;
    for (int cand : {8, 4, 2, 1})
      if (tpr == 0 && vecs == 32 * cand) { tpr = 32; nv = cand; }
    for (int cand : {8, 4, 2, 1})
      for (int th : {128, 256, 512, 1024})
        if (tpr == 0 && vecs == th * cand) { tpr = th; nv = cand; }
    if (tpr != 0) {
      const bool warp = tpr == 32;
      lc.block = dim3(warp ? 256 : tpr);
      lc.grid = dim3(static_cast<unsigned>(warp ? std::min<int64_t>(CeilDiv(a.rows, 8), ctx->sm_count * 8)
                                                : std::min<int64_t>(a.rows, static_cast<int64_t>(ctx->sm_count) * std::max(1, 2048 / tpr))));
#define B200_ROW_CASE(NVV)                                                                                         \
  case NVV: e = warp ? Launch(lc, rownorm_reg_kernel<T, KIND, NVV, true>, a) : Launch(lc, rownorm_reg_kernel<T, KIND, NVV, false>, a); break;
      switch (nv) {
        B200_ROW_CASE(8)
        B200_ROW_CASE(4)
        B200_ROW_CASE(2)
        default: e = warp ? Launch(lc, rownorm_reg_kernel<T, KIND, 1, true>, a) : Launch(lc, rownorm_reg_kernel<T, KIND, 1, false>, a); break;
      }
#undef B200_ROW_CASE
      if (e != cudaSuccess) return Stick(ctx, Fail(B200_INTERNAL, "b200_rownorm launch: %s", cudaGetErrorString(e)));
      return EndLaunch(ctx, "b200_rownorm");
    }
  }
  if (a.n <= 2048) {
    // a warp per row; 8 warps per CTA
    const int wpb = 8;
    lc.block = dim3(wpb * 32);
    lc.smem = static_cast<size_t>(wpb) * stride * 4;
    lc.grid = dim3(static_cast<unsigned>(std::min<int64_t>(CeilDiv(a.rows, wpb), ctx->sm_count * 8)));
    auto k = vec ? rownorm_warp_kernel<T, KIND, true> : rownorm_warp_kernel<T, KIND, false>;
    if (lc.smem > 48 * 1024) {
      e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(lc.smem));
      if (e != cudaSuccess) return Stick(ctx, Fail(B200_INTERNAL, "rownorm smem attribute: %s", cudaGetErrorString(e)));
    }
    e = Launch(lc, k, a);
  } else if (static_cast<size_t>(stride) * 4 <= 200 * 1024) {
    const int threads = a.n >= 16384 ? 1024 : (a.n >= 8192 ? 512 : 256);
    lc.block = dim3(threads);
    lc.smem = static_cast<size_t>(stride) * 4;
    lc.grid = dim3(static_cast<unsigned>(std::min<int64_t>(a.rows, ctx->sm_count * 8)));
    auto k = vec ? rownorm_block_kernel<T, KIND, true> : rownorm_block_kernel<T, KIND, false>;
    if (lc.smem > 48 * 1024) {
      e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(lc.smem));
      if (e != cudaSuccess) return Stick(ctx, Fail(B200_INTERNAL, "rownorm smem attribute: %s", cudaGetErrorString(e)));
    }
    e = Launch(lc, k, a);
  } else {
    lc.block = dim3(1024);
    lc.grid = dim3(static_cast<unsigned>(std::min<int64_t>(a.rows, ctx->sm_count * 2)));
    e = Launch(lc, rownorm_long_kernel<T, KIND>, a);
  }
  if (e != cudaSuccess) return Stick(ctx, Fail(B200_INTERNAL, "b200_rownorm launch: %s", cudaGetErrorString(e)));
  return EndLaunch(ctx, "b200_rownorm");
}

template <typename T>
b200_status LaunchKind(b200_context* ctx, cudaStream_t stream, int kind, const RowArgs& a) {
  switch (kind) {
    case kRms: return LaunchRows<T, kRms>(ctx, stream, a);
    case kSoftmax: return LaunchRows<T, kSoftmax>(ctx, stream, a);
    case kLogSoftmax: return LaunchRows<T, kLogSoftmax>(ctx, stream, a);
    default: return LaunchRows<T, kLayerNorm>(ctx, stream, a);
  }
}

}  // namespace

extern "C" b200_status b200_rownorm(b200_context* ctx, b200_stream stream, int kind, const void* x,
                                    const void* gain_or_null, const void* beta_or_null, void* y, int64_t rows,
                                    int64_t n, int dtype, double eps) {
  b200_status s = BeginLaunch(ctx);
  if (s != B200_OK) return s;
  if (kind < 0 || kind > 3) return Fail(B200_INVALID_ARGUMENT, "b200_rownorm: unknown kind %d", kind);
  if (dtype != B200_F32 && dtype != B200_F16 && dtype != B200_BF16)
    return Fail(B200_INVALID_ARGUMENT, "b200_rownorm: unknown dtype %d", dtype);
  if (rows < 0 || n < 0) return Fail(B200_INVALID_ARGUMENT, "b200_rownorm: negative size");
  if (rows == 0 || n == 0) return B200_OK;  // zero-sized inputs launch nothing (ffi/scan.cc:51-75)
  if (n > (1 << 30)) return Fail(B200_UNIMPLEMENTED, "b200_rownorm: row length %lld too large", static_cast<long long>(n));
  if (x == nullptr || y == nullptr) return Fail(B200_INVALID_ARGUMENT, "b200_rownorm: null buffer");
  if (kind == kRms && gain_or_null == nullptr) return Fail(B200_INVALID_ARGUMENT, "b200_rownorm: RMSNorm needs a gain");
  RowArgs a;
  a.x = x;
  a.gain = gain_or_null;
  a.beta = beta_or_null;
  a.y = y;
  a.rows = rows;
  a.n = static_cast<int>(n);
  a.eps = static_cast<float>(eps);
  switch (dtype) {
    case B200_F32: return LaunchKind<float>(ctx, stream, kind, a);
    case B200_F16: return LaunchKind<__half>(ctx, stream, kind, a);
    default: return LaunchKind<__nv_bfloat16>(ctx, stream, kind, a);
  }
}
