// Next-token sampling on the device (≙ sample, examples/llm/qwen3.py:395-418): greedy,
// temperature, top-k and top-p (nucleus) over the top-k candidates, so that a decode loop
// reads back 4 bytes per sequence instead of a row of 151936 logits.
//
// The reference draws with jax.random.categorical (Gumbel noise from a threefry key), which
// cannot be reproduced bit for bit outside JAX.  Here the caller supplies one uniform number
// u in [0, 1) per row and the draw is the inverse CDF: the first candidate whose cumulative
// probability exceeds u * (total kept probability).  Candidates are ordered as the reference
// orders them: all logits in vocabulary order when neither top-k nor top-p is set
// (categorical over the row), else the top-k values in descending order, ties by lower
// index first (jax.lax.top_k), of which top-p keeps the smallest prefix whose probability
// reaches top_p (always at least one).  One CTA per row.
#include "common.cuh"

using namespace b200;

namespace {

constexpr int kT = 1024;
constexpr int kMaxTopK = 1024;

struct SampleArgs {
  const float* logits;
  const float* uniform;
  int32_t* out;
  int V;
  float inv_temperature;   // 0: greedy
  int top_k;
  float top_p;
};

// order-preserving map of f32 onto u32 (larger float, larger key)
__device__ __forceinline__ uint32_t fkey(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// Inclusive scan over the block's kT threads (deterministic: warp scans, then the warp totals).
__device__ __forceinline__ float block_scan(float v, float* warp_tot, float* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float n = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= o) v += n;
  }
  if (lane == 31) warp_tot[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float w = warp_tot[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float n = __shfl_up_sync(0xffffffffu, w, o);
      if (lane >= o) w += n;
    }
    warp_tot[lane] = w;
  }
  __syncthreads();
  const float before = warp == 0 ? 0.0f : warp_tot[warp - 1];
  if (total != nullptr) *total = warp_tot[kT / 32 - 1];
  __syncthreads();
  return v + before;
}

__global__ void __launch_bounds__(kT) sample_kernel(const SampleArgs a) {
  __shared__ float s_val[kT / 32];
  __shared__ int s_idx[kT / 32];
  __shared__ float warp_tot[32];
  __shared__ unsigned hist[256];
  __shared__ unsigned long long cand[kMaxTopK];
  __shared__ float s_cum[kMaxTopK];
  __shared__ unsigned s_prefix, s_krem, s_count, s_choice;
  __shared__ float s_max;
  __shared__ int s_arg;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int V = a.V;
  const float* x = a.logits + static_cast<size_t>(blockIdx.x) * V;

  // ---- maximum and argmax (ties: the lowest index, like jnp.argmax)
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = tid; i < V; i += kT) {
    const float v = x[i];
    if (v > bv || (v == bv && i < bi) || bi == 0x7fffffff) {
      if (v > bv || bi == 0x7fffffff || (v == bv && i < bi)) {
        bv = v;
        bi = i;
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) {
      bv = ov;
      bi = oi;
    }
  }
  if (lane == 0) {
    s_val[warp] = bv;
    s_idx[warp] = bi;
  }
  __syncthreads();
  if (tid == 0) {
    float mv = s_val[0];
    int mi = s_idx[0];
    for (int w = 1; w < kT / 32; ++w)
      if (s_val[w] > mv || (s_val[w] == mv && s_idx[w] < mi)) {
        mv = s_val[w];
        mi = s_idx[w];
      }
    s_max = mv;
    s_arg = mi;
    s_choice = 0xffffffffu;
  }
  __syncthreads();
  const float gmax = s_max;
  if (a.inv_temperature == 0.0f) {
    if (tid == 0) a.out[blockIdx.x] = s_arg;
    return;
  }
  const float u = a.uniform[blockIdx.x];

  if (a.top_k == 0) {
    // ---- categorical over the whole row, vocabulary order: thread t owns a contiguous chunk
    const int chunk = (V + kT - 1) / kT;
    const int i0 = min(tid * chunk, V), i1 = min(i0 + chunk, V);
    float part = 0.0f;
    for (int i = i0; i < i1; ++i) part += expf((x[i] - gmax) * a.inv_temperature);
    float total;
    const float incl = block_scan(part, warp_tot, &total);
    const float target = u * total, before = incl - part;
    if (part > 0.0f && before <= target && target < incl) {
      float c = before;
      int pick = i1 - 1;
      for (int i = i0; i < i1; ++i) {
        c += expf((x[i] - gmax) * a.inv_temperature);
        if (target < c) {
          pick = i;
          break;
        }
      }
      s_choice = static_cast<unsigned>(pick);
    }
    __syncthreads();
    if (tid == 0) a.out[blockIdx.x] = s_choice != 0xffffffffu ? static_cast<int>(s_choice) : s_arg;   // u * total rounded up to the total
    return;
  }

  // ---- the k-th largest key by radix selection (four passes of eight bits)
  const int k = a.top_k;
  if (tid == 0) {
    s_prefix = 0;
    s_krem = static_cast<unsigned>(k);
  }
  unsigned mask = 0;
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int i = tid; i < 256; i += kT) hist[i] = 0;
    __syncthreads();
    const unsigned prefix = s_prefix;
    for (int i = tid; i < V; i += kT) {
      const unsigned key = fkey(x[i]);
      if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
    }
    __syncthreads();
    if (tid == 0) {
      unsigned need = s_krem, seen = 0;
      int b = 255;
      for (; b > 0; --b) {
        if (seen + hist[b] >= need) break;
        seen += hist[b];
      }
      s_krem = need - seen;
      s_prefix = prefix | (static_cast<unsigned>(b) << shift);
    }
    mask |= 255u << shift;
    __syncthreads();
  }
  const unsigned thr = s_prefix, k_eq = s_krem;   // the k-th largest key; how many of its equals belong to the top k
  // ---- collect: every key above thr (any order, sorted below), and of the keys equal to thr the k_eq lowest indices
  if (tid == 0) s_count = 0;
  for (int i = tid; i < kMaxTopK; i += kT) cand[i] = 0ull;
  __syncthreads();
  const int chunk = (V + kT - 1) / kT;
  const int i0 = min(tid * chunk, V), i1 = min(i0 + chunk, V);
  float n_eq = 0.0f;
  for (int i = i0; i < i1; ++i) {
    const unsigned key = fkey(x[i]);
    if (key > thr) {
      const unsigned slot = atomicAdd(&s_count, 1u);
      cand[slot] = (static_cast<unsigned long long>(key) << 32) | (0xffffffffu - static_cast<unsigned>(i));
    } else if (key == thr) {
      n_eq += 1.0f;
    }
  }
  const float eq_incl = block_scan(n_eq, warp_tot, nullptr);   // counts up to 2^24 are exact in f32
  {
    unsigned rank = static_cast<unsigned>(eq_incl - n_eq);
    const unsigned base = static_cast<unsigned>(k) - k_eq;     // the keys above thr
    for (int i = i0; i < i1 && rank < k_eq; ++i) {
      if (fkey(x[i]) == thr) {
        cand[base + rank] = (static_cast<unsigned long long>(thr) << 32) | (0xffffffffu - static_cast<unsigned>(i));
        ++rank;
      }
    }
  }
  __syncthreads();
  // ---- bitonic sort of the 1024 candidate slots, descending (value, then lower index first)
  for (int size = 2; size <= kMaxTopK; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      const int j = tid ^ stride;
      if (j > tid) {
        const unsigned long long lo = cand[tid], hi = cand[j];
        const bool desc = (tid & size) == 0;
        if ((lo < hi) == desc) {
          cand[tid] = hi;
          cand[j] = lo;
        }
      }
      __syncthreads();
    }
  }
  // ---- probabilities of the sorted candidates, nucleus, draw
  float pj = 0.0f;
  int idx = 0;
  if (tid < k) {
    idx = static_cast<int>(0xffffffffu - static_cast<unsigned>(cand[tid] & 0xffffffffull));
    pj = expf((x[idx] - gmax) * a.inv_temperature);
  }
  float total;
  const float cum = block_scan(pj, warp_tot, &total);
  if (tid < kMaxTopK) s_cum[tid] = cum;
  // kept: before < top_p * total (the first candidate always is)
  const bool kept = tid < k && (tid == 0 || (cum - pj) < a.top_p * total);
  float kcount;
  block_scan(kept ? 1.0f : 0.0f, warp_tot, &kcount);
  const int kk = max(1, static_cast<int>(kcount));
  const float kept_total = s_cum[kk - 1];
  const float target = u * kept_total;
  if (tid < kk && (cum - pj) <= target && target < cum) s_choice = static_cast<unsigned>(idx);
  __syncthreads();
  if (tid == kk - 1 && s_choice == 0xffffffffu) s_choice = static_cast<unsigned>(idx);   // u * total rounded up to the total
  __syncthreads();
  if (tid == 0) a.out[blockIdx.x] = static_cast<int>(s_choice);
}

}  // namespace

extern "C" {

b200_status b200_sample(b200_context* ctx, b200_stream stream, const float* logits, int64_t batch, int64_t vocab,
                        float temperature, int32_t top_k, float top_p, const float* uniform, int32_t* out) {
  b200_status s = BeginLaunch(ctx);
  if (s != B200_OK) return s;
  if (temperature < 0.0f) return Fail(B200_INVALID_ARGUMENT, "b200_sample: temperature must be >= 0, got %g", temperature);
  if (batch < 0 || vocab < 0) return Fail(B200_INVALID_ARGUMENT, "b200_sample: negative size");
  if (top_k < 0 || top_k > vocab) return Fail(B200_INVALID_ARGUMENT, "b200_sample: top_k must be in [0, %lld], got %d",
                                              static_cast<long long>(vocab), top_k);
  if (batch == 0) return B200_OK;
  if (vocab == 0) return Fail(B200_INVALID_ARGUMENT, "b200_sample: empty vocabulary");
  if (vocab > (1 << 24)) return Fail(B200_UNIMPLEMENTED, "b200_sample: vocabulary above 2^24");
  if (batch > 65535) return Fail(B200_UNIMPLEMENTED, "b200_sample: more than 65535 rows");
  if (logits == nullptr || out == nullptr) return Fail(B200_INVALID_ARGUMENT, "b200_sample: null buffer");
  if (temperature > 0.0f && uniform == nullptr)
    return Fail(B200_INVALID_ARGUMENT, "b200_sample: sampling needs one uniform number per row");
  if (temperature > 0.0f && top_k > kMaxTopK)
    return Fail(B200_UNIMPLEMENTED, "b200_sample: top_k %d (up to %d)", top_k, kMaxTopK);
  if (temperature > 0.0f && top_k == 0 && top_p < 1.0f)
    return Fail(B200_UNIMPLEMENTED, "b200_sample: top_p without top_k sorts the whole vocabulary; set top_k (up to %d)", kMaxTopK);
  SampleArgs a;
  a.logits = logits;
  a.uniform = uniform;
  a.out = out;
  a.V = static_cast<int>(vocab);
  a.inv_temperature = temperature > 0.0f ? 1.0f / temperature : 0.0f;
  a.top_k = temperature > 0.0f ? top_k : 0;
  a.top_p = top_p;
  LaunchCfg lc;
  lc.stream = stream;
  lc.grid = dim3(static_cast<unsigned>(batch));
  lc.block = dim3(kT);
  cudaError_t e = Launch(lc, sample_kernel, a);
  if (e != cudaSuccess) return Stick(ctx, Fail(B200_INTERNAL, "b200_sample launch: %s", cudaGetErrorString(e)));
  return EndLaunch(ctx, "b200_sample");
}

}  // extern "C"
