// Grouped-query decode attention over the KV cache (the decode branch of
// attention, examples/llm/qwen3.py:322-327): scores q.k over the head dim from
// K [B, KV, S, D], an f32 softmax over positions, p.v over positions from
// V [B, KV, D, S] (both caches are read along their minor axis, the layout the
// reference chose, qwen3.py:279-291).
//
// Split over positions: a CTA owns 64 cache slots of one (batch, KV head) and
// all G query heads that share it, and writes an unnormalised partial
// (sum p v, running max, sum p) to scratch; a second kernel merges the
// partials.  All K and V bytes of a CTA are requested up front (one DRAM
// latency per CTA).  In the fused form the kernel also does what precedes
// attention in the layer (qwen3.py:366-369): per-head RMSNorm and rotate-half
// RoPE of q from the fused qkv row, and - in the CTA whose slots contain the
// new position - of k, plus the cache writes of k and v.  That CTA takes the
// new key/value from shared memory, so nothing is read back after being written.
#include <mutex>

#include "common.cuh"

using namespace b200;

namespace {

constexpr int kChunk = 64;     // cache positions per CTA
constexpr int kThreads = 128;

struct AttnArgs {
  const __nv_bfloat16* q;        // [B, H, D], already normalised + rotated (plain form)
  const __nv_bfloat16* qkv;      // [B, (H + 2 KV) D] (fused form), else null
  const __nv_bfloat16* q_norm;
  const __nv_bfloat16* k_norm;
  const float* inv_freq;         // [D / 2] or null (computed in the kernel)
  __nv_bfloat16* k_cache;        // [B, KV, S, D]
  __nv_bfloat16* v_cache;        // [B, KV, D, S]
  __nv_bfloat16* out;            // [B, H, D]
  const int32_t* pos;
  float* scratch;                // [B, KV, splits, G, D + 2]
  int heads, kv_heads;
  int64_t max_len;
  int splits;
  int vec_v;                     // V rows allow 16-byte loads (max_len % 8 == 0, base aligned)
  float scale, theta, eps;
  int* status;                   // device status word
};

// RMSNorm + RoPE of one head by one warp; the results (bf16-rounded, as the
// reference rounds after rms_norm and after rope) go to dst1[i], dst2[i] for
// i < D/2 (first and second half of the head).
template <int D>
__device__ __forceinline__ void norm_rope_head(const __nv_bfloat16* src, const __nv_bfloat16* w, int pos,
                                               const AttnArgs& a, int lane, float* dst1, float* dst2) {
  constexpr int PAIRS = D / 64;
  float x1[PAIRS], x2[PAIRS];
  float ss = 0.0f;
#pragma unroll
  for (int p = 0; p < PAIRS; ++p) {
    const int i = lane + 32 * p;
    x1[p] = __bfloat162float(src[i]);
    x2[p] = __bfloat162float(src[i + D / 2]);
    ss = fmaf(x1[p], x1[p], ss);
    ss = fmaf(x2[p], x2[p], ss);
  }
  ss = warp_sum(ss);
  const float r = 1.0f / sqrtf(ss / static_cast<float>(D) + a.eps);
#pragma unroll
  for (int p = 0; p < PAIRS; ++p) {
    const int i = lane + 32 * p;
    const float n1 = bf16_round((x1[p] * r) * __bfloat162float(w[i]));
    const float n2 = bf16_round((x2[p] * r) * __bfloat162float(w[i + D / 2]));
    const float inv_freq = a.inv_freq != nullptr
                               ? a.inv_freq[i]
                               : static_cast<float>(1.0 / pow(static_cast<double>(a.theta), static_cast<double>(2 * i) / D));
    float sn, cs;
    sincosf(static_cast<float>(pos) * inv_freq, &sn, &cs);
    dst1[i] = bf16_round(n1 * cs - n2 * sn);
    dst2[i] = bf16_round(n2 * cs + n1 * sn);
  }
}

template <int D, int G>
__global__ void __launch_bounds__(kThreads) attn_partial_kernel(const AttnArgs a) {
  constexpr int HALF = D / 2;
  constexpr int KV4 = HALF / 8;   // 16-byte loads of K per thread (two threads per position)
  __shared__ __align__(16) float qs[G][2][HALF + 4];
  __shared__ __align__(16) float sc[G][kChunk];
  __shared__ float red[G][kThreads / 32];
  __shared__ float knew[2][HALF + 4];
  __shared__ float vnew[D];
  // Fused form: the position and the cache slots of earlier steps (all below *pos) do not
  // come from the kernel before this one, so they are requested before waiting for it.
  // Plain form: slot *pos itself is read, and the kernel before this one (the cache write
  // of b200_qk_norm_rope_cache) may still be storing it, so the wait comes first.
  pdl_launch_dependents();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int split = blockIdx.x, kv = blockIdx.y, b = blockIdx.z;
  const bool fused = a.qkv != nullptr;
  if (!fused) pdl_wait();
  const int pos = *a.pos;
  if (pos < 0 || pos >= a.max_len) {         // nothing may be written outside the cache
    pdl_wait();
    if (tid == 0) report_status(a.status, B200_INVALID_ARGUMENT, 500);
    return;
  }
  const int n_valid = pos + 1;
  const int n_old = fused ? pos : pos + 1;   // slots whose K/V are already in the cache
  const int s0 = split * kChunk;
  if (s0 >= n_valid) {                       // the merge only reads splits below n_valid
    pdl_wait();
    return;
  }
  const int cnt = min(kChunk, n_valid - s0);
  const bool owner = fused && pos >= s0 && pos < s0 + kChunk;
  const int64_t bkv = static_cast<int64_t>(b) * a.kv_heads + kv;

  // ---- request every K and V byte of this CTA now ------------------------------------
  const int p = tid >> 1, half = tid & 1;    // scores: position p, half of the head dim
  uint4 kreg[KV4];
  {
    const bool have = s0 + p < n_old;
    const uint4* krow = reinterpret_cast<const uint4*>(a.k_cache + (bkv * a.max_len + s0 + p) * D + half * HALF);
#pragma unroll
    for (int v = 0; v < KV4; ++v) kreg[v] = have ? krow[v] : make_uint4(0, 0, 0, 0);
  }
  uint4 vreg[kChunk / 8];
  const __nv_bfloat16* vrow = a.v_cache + (bkv * D + min(tid, D - 1)) * a.max_len + s0;
  if (a.vec_v && tid < D) {
#pragma unroll
    for (int j = 0; j < kChunk / 8; ++j)
      vreg[j] = (s0 + 8 * j < n_old) ? *reinterpret_cast<const uint4*>(vrow + 8 * j) : make_uint4(0, 0, 0, 0);
  }

  // ---- queries (and, in the owning CTA, the new key and value) -----------------------
  pdl_wait();   // q (or the fused qkv row) is the previous kernel's output
  if (fused) {
    const int total_heads = a.heads + 2 * a.kv_heads;
    const __nv_bfloat16* row = a.qkv + static_cast<int64_t>(b) * total_heads * D;
    for (int gq = warp; gq < G; gq += kThreads / 32)
      norm_rope_head<D>(row + static_cast<int64_t>(kv * G + gq) * D, a.q_norm, pos, a, lane, qs[gq][0], qs[gq][1]);
    if (owner) {
      if (warp == (G % 4)) {
        norm_rope_head<D>(row + static_cast<int64_t>(a.heads + kv) * D, a.k_norm, pos, a, lane, knew[0], knew[1]);
        __syncwarp();
        __nv_bfloat16* kdst = a.k_cache + (bkv * a.max_len + pos) * D;
        for (int i = lane; i < HALF; i += 32) {
          kdst[i] = __float2bfloat16_rn(knew[0][i]);
          kdst[i + HALF] = __float2bfloat16_rn(knew[1][i]);
        }
      } else if (warp == ((G + 1) % 4)) {
        const __nv_bfloat16* vsrc = row + static_cast<int64_t>(a.heads + a.kv_heads + kv) * D;
        __nv_bfloat16* vdst = a.v_cache + bkv * D * a.max_len + pos;
        for (int d = lane; d < D; d += 32) {
          const __nv_bfloat16 v = vsrc[d];
          vnew[d] = __bfloat162float(v);
          vdst[static_cast<int64_t>(d) * a.max_len] = v;
        }
      }
    }
  } else {
    for (int i = tid; i < G * D; i += kThreads) {
      const int gq = i / D, d = i % D;
      qs[gq][d / HALF][d % HALF] = __bfloat162float(a.q[(static_cast<int64_t>(b) * a.heads + kv * G + gq) * D + d]);
    }
  }
  __syncthreads();

  // ---- scores -------------------------------------------------------------------------
  float dot[G];
#pragma unroll
  for (int gq = 0; gq < G; ++gq) dot[gq] = 0.0f;
  const bool from_smem = owner && s0 + p == pos;
#pragma unroll
  for (int v = 0; v < KV4; ++v) {
    float kf[8];
    if (from_smem) {
#pragma unroll
      for (int j = 0; j < 8; ++j) kf[j] = knew[half][v * 8 + j];
    } else {
      const uint32_t w[4] = {kreg[v].x, kreg[v].y, kreg[v].z, kreg[v].w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        kf[2 * j] = bf16_lo(w[j]);
        kf[2 * j + 1] = bf16_hi(w[j]);
      }
    }
#pragma unroll
    for (int gq = 0; gq < G; ++gq) {
      const float4 q0 = *reinterpret_cast<const float4*>(&qs[gq][half][v * 8]);
      const float4 q1 = *reinterpret_cast<const float4*>(&qs[gq][half][v * 8 + 4]);
      dot[gq] = fmaf(q0.x, kf[0], dot[gq]);
      dot[gq] = fmaf(q0.y, kf[1], dot[gq]);
      dot[gq] = fmaf(q0.z, kf[2], dot[gq]);
      dot[gq] = fmaf(q0.w, kf[3], dot[gq]);
      dot[gq] = fmaf(q1.x, kf[4], dot[gq]);
      dot[gq] = fmaf(q1.y, kf[5], dot[gq]);
      dot[gq] = fmaf(q1.z, kf[6], dot[gq]);
      dot[gq] = fmaf(q1.w, kf[7], dot[gq]);
    }
  }
  float mx[G];
#pragma unroll
  for (int gq = 0; gq < G; ++gq) {
    dot[gq] += __shfl_xor_sync(0xffffffffu, dot[gq], 1);   // the two halves of the head dim
    const float s = p < cnt ? dot[gq] * a.scale : -INFINITY;
    if (half == 0) sc[gq][p] = s;
    mx[gq] = warp_max(s);
    if (lane == 0) red[gq][warp] = mx[gq];
  }
  __syncthreads();
  float lsum[G];
#pragma unroll
  for (int gq = 0; gq < G; ++gq) {
    float m = red[gq][0];
#pragma unroll
    for (int w = 1; w < kThreads / 32; ++w) m = fmaxf(m, red[gq][w]);
    mx[gq] = m;
    float e = 0.0f;
    if (tid < kChunk) {
      e = tid < cnt ? expf(sc[gq][tid] - m) : 0.0f;
      sc[gq][tid] = e;
    }
    lsum[gq] = warp_sum(e);
  }
  __syncthreads();   // every thread has read the maxima; sc[][] now holds p
#pragma unroll
  for (int gq = 0; gq < G; ++gq)
    if (lane == 0) red[gq][warp] = lsum[gq];
  __syncthreads();

  // ---- p . v: one output dimension per thread -------------------------------------------
  float* part = a.scratch + (bkv * a.splits + split) * G * (D + 2);
  if (tid < D) {
    float acc[G];
#pragma unroll
    for (int gq = 0; gq < G; ++gq) acc[gq] = 0.0f;
    if (a.vec_v) {
#pragma unroll
      for (int j = 0; j < kChunk / 8; ++j) {
        const uint32_t w[4] = {vreg[j].x, vreg[j].y, vreg[j].z, vreg[j].w};
        float v[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = (e & 1) ? bf16_hi(w[e >> 1]) : bf16_lo(w[e >> 1]);
        if (s0 + 8 * j + 8 > n_old) {   // only the chunk that holds the newest position has such slots
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const int s = 8 * j + e;
            if (s0 + s >= n_old) v[e] = (owner && s0 + s == pos) ? vnew[tid] : 0.0f;
          }
        }
        // the eight probabilities of a head as two 16-byte broadcast reads (the loop is bound by
        // shared-memory instructions otherwise: one scalar read per multiply-add)
#pragma unroll
        for (int gq = 0; gq < G; ++gq) {
          const float4 p0 = *reinterpret_cast<const float4*>(&sc[gq][8 * j]);
          const float4 p1 = *reinterpret_cast<const float4*>(&sc[gq][8 * j + 4]);
          acc[gq] = fmaf(p0.x, v[0], acc[gq]);
          acc[gq] = fmaf(p0.y, v[1], acc[gq]);
          acc[gq] = fmaf(p0.z, v[2], acc[gq]);
          acc[gq] = fmaf(p0.w, v[3], acc[gq]);
          acc[gq] = fmaf(p1.x, v[4], acc[gq]);
          acc[gq] = fmaf(p1.y, v[5], acc[gq]);
          acc[gq] = fmaf(p1.z, v[6], acc[gq]);
          acc[gq] = fmaf(p1.w, v[7], acc[gq]);
        }
      }
    } else {
      for (int s = 0; s < cnt; ++s) {
        const float v = s0 + s < n_old ? __bfloat162float(vrow[s]) : ((owner && s0 + s == pos) ? vnew[tid] : 0.0f);
#pragma unroll
        for (int gq = 0; gq < G; ++gq) acc[gq] = fmaf(sc[gq][s], v, acc[gq]);
      }
    }
#pragma unroll
    for (int gq = 0; gq < G; ++gq) part[gq * (D + 2) + tid] = acc[gq];
  }
  if (tid < G) {
    float l = 0.0f;
    for (int w = 0; w < kThreads / 32; ++w) l += red[tid][w];
    part[tid * (D + 2) + D] = mx[tid];
    part[tid * (D + 2) + D + 1] = l;
  }
}

// Merges the partials of one (batch, query head): out = sum_s e^{m_s - M} o_s / sum_s e^{m_s - M} l_s.
template <int D, int G>
__global__ void __launch_bounds__(kThreads) attn_combine_kernel(const AttnArgs a) {
  extern __shared__ float wsm[];   // [2][splits]: weights e^{m_s - M}, then the partial sums l_s
  __shared__ float red[kThreads / 32];
  pdl_wait();
  pdl_launch_dependents();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int h = blockIdx.x, b = blockIdx.y;
  const int kv = h / G, gq = h % G;
  if (*a.pos < 0 || *a.pos >= a.max_len) return;
  const int n_valid = *a.pos + 1;
  const int nsplit = (n_valid + kChunk - 1) / kChunk;
  const float* base = a.scratch + (static_cast<int64_t>(b) * a.kv_heads + kv) * a.splits * G * (D + 2) + gq * (D + 2);
  const int64_t stride = static_cast<int64_t>(G) * (D + 2);
  // Everything this thread needs from the partials is requested at once (one trip to L2):
  // its output dimension of the first kPre splits, and the (max, sum) pair of split `tid`.
  constexpr int kPre = 40;
  const int d0 = tid < D ? tid : 0;
  float o[kPre];
#pragma unroll
  for (int s = 0; s < kPre; ++s) o[s] = s < nsplit ? base[s * stride + d0] : 0.0f;
  float m = -INFINITY;
  for (int s = tid; s < nsplit; s += kThreads) {
    const float2 ml = *reinterpret_cast<const float2*>(&base[s * stride + D]);
    wsm[s] = ml.x;
    wsm[a.splits + s] = ml.y;
    m = fmaxf(m, ml.x);
  }
  m = warp_max(m);
  if (lane == 0) red[warp] = m;
  __syncthreads();
  m = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
  __syncthreads();
  float den = 0.0f;
  for (int s = tid; s < nsplit; s += kThreads) {
    const float w = expf(wsm[s] - m);
    wsm[s] = w;
    den = fmaf(w, wsm[a.splits + s], den);
  }
  den = warp_sum(den);
  if (lane == 0) red[warp] = den;
  __syncthreads();
  den = (red[0] + red[1]) + (red[2] + red[3]);
  for (int d = tid; d < D; d += kThreads) {
    float num = 0.0f;
    if (d == d0) {
#pragma unroll
      for (int s = 0; s < kPre; ++s)
        if (s < nsplit) num = fmaf(wsm[s], o[s], num);
    } else {
      for (int s = 0; s < min(nsplit, kPre); ++s) num = fmaf(wsm[s], base[s * stride + d], num);
    }
#pragma unroll 8
    for (int s = kPre; s < nsplit; ++s) num = fmaf(wsm[s], base[s * stride + d], num);
    a.out[(static_cast<int64_t>(b) * a.heads + h) * D + d] = __float2bfloat16_rn(num / den);
  }
}

template <int D>
b200_status LaunchAttn(b200_context* ctx, cudaStream_t stream, const AttnArgs& a, int group, int64_t batch) {
  LaunchCfg lc;
  lc.stream = stream;
  lc.pdl = true;
  lc.block = dim3(kThreads);
  lc.grid = dim3(a.splits, a.kv_heads, static_cast<unsigned>(batch));
  cudaError_t e;
  switch (group) {
    case 1: e = Launch(lc, attn_partial_kernel<D, 1>, a); break;
    case 2: e = Launch(lc, attn_partial_kernel<D, 2>, a); break;
    case 4: e = Launch(lc, attn_partial_kernel<D, 4>, a); break;
    case 8: e = Launch(lc, attn_partial_kernel<D, 8>, a); break;
    default: return Fail(B200_UNIMPLEMENTED, "attention: %d query heads per KV head (1, 2, 4 or 8)", group);
  }
  if (e != cudaSuccess) return Stick(ctx, Fail(B200_INTERNAL, "attention launch: %s", cudaGetErrorString(e)));
  lc.grid = dim3(a.heads, static_cast<unsigned>(batch));
  lc.smem = static_cast<size_t>(2 * a.splits) * sizeof(float);
  switch (group) {
    case 1: e = Launch(lc, attn_combine_kernel<D, 1>, a); break;
    case 2: e = Launch(lc, attn_combine_kernel<D, 2>, a); break;
    case 4: e = Launch(lc, attn_combine_kernel<D, 4>, a); break;
    default: e = Launch(lc, attn_combine_kernel<D, 8>, a); break;
  }
  if (e != cudaSuccess) return Stick(ctx, Fail(B200_INTERNAL, "attention merge launch: %s", cudaGetErrorString(e)));
  return EndLaunch(ctx, "b200_attention", 2);
}

b200_status Run(b200_context* ctx, cudaStream_t stream, AttnArgs a, const char* who, int64_t batch, int head_dim) {
  b200_status s = BeginLaunch(ctx);
  if (s != B200_OK) return s;
  if (batch < 0 || a.heads <= 0 || a.kv_heads <= 0 || a.max_len <= 0 || a.heads % a.kv_heads != 0)
    return Fail(B200_INVALID_ARGUMENT, "%s: bad sizes", who);
  if (head_dim != 64 && head_dim != 128) return Fail(B200_UNIMPLEMENTED, "%s: head_dim %d (64 or 128)", who, head_dim);
  if (batch > 65535 || a.kv_heads > 65535) return Fail(B200_UNIMPLEMENTED, "%s: batch or head count too large", who);
  if (a.max_len > (1 << 20)) return Fail(B200_UNIMPLEMENTED, "%s: max_len above 2^20", who);
  if (batch == 0) return B200_OK;
  if (!a.k_cache || !a.v_cache || !a.out || !a.pos || !a.scratch || (!a.q && !a.qkv))
    return Fail(B200_INVALID_ARGUMENT, "%s: null buffer", who);
  if (a.qkv && (!a.q_norm || !a.k_norm)) return Fail(B200_INVALID_ARGUMENT, "%s: null norm gain", who);
  if (!Aligned(a.k_cache, 16) || !Aligned(a.v_cache, 2))
    return Fail(B200_INVALID_ARGUMENT, "%s: the K cache must be 16-byte aligned", who);
  a.splits = static_cast<int>((a.max_len + kChunk - 1) / kChunk);
  a.vec_v = Aligned(a.v_cache, 16) && a.max_len % 8 == 0;
  a.scale = 1.0f / sqrtf(static_cast<float>(head_dim));
  a.status = ctx->dev_status;
  return head_dim == 128 ? LaunchAttn<128>(ctx, stream, a, a.heads / a.kv_heads, batch)
                         : LaunchAttn<64>(ctx, stream, a, a.heads / a.kv_heads, batch);
}

// ---- scratch that nobody has to allocate ------------------------------------------------
// Some hosts of this library may not allocate device memory when they call it: code that
// runs inside a stream capture, or a runtime whose allocator owns every byte of the device
// and forbids cudaMalloc from plugins.  For them the split-attention partials can live in
// this fixed array instead of a caller-provided buffer.  Every GPU that loads the library
// carries it until the process exits.
constexpr size_t kStaticScratchFloats = size_t(2) << 20;   // 8 MiB
static __device__ __align__(256) float g_attn_scratch[kStaticScratchFloats];

constexpr int kMaxDevices = 64;
std::mutex g_scratch_mu;
float* g_scratch_ptr[kMaxDevices] = {};   // device address of g_attn_scratch, per device ordinal

// In host code `g_attn_scratch` is only a handle for the symbol, not a device address, so
// the address is asked for once per device (with that device current) and cached.
b200_status StaticScratch(b200_context* ctx, float** out) {
  if (ctx->device < 0 || ctx->device >= kMaxDevices)
    return Fail(B200_UNIMPLEMENTED, "b200_attention_decode_static: device ordinal %d beyond %d", ctx->device, kMaxDevices);
  std::lock_guard<std::mutex> lock(g_scratch_mu);
  if (g_scratch_ptr[ctx->device] == nullptr) {
    float* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_attn_scratch);
    if (e != cudaSuccess || p == nullptr)
      return Stick(ctx, Fail(B200_INTERNAL, "cudaGetSymbolAddress(static attention scratch): %s", cudaGetErrorString(e)));
    g_scratch_ptr[ctx->device] = p;
  }
  *out = g_scratch_ptr[ctx->device];
  return B200_OK;
}

}  // namespace

namespace b200 {
// Called by b200_context_create: the address of the built-in scratch is looked up while the
// context is made, so that b200_attention_decode_static itself never calls into the runtime
// for it (it may run inside a stream capture).
b200_status AttnStaticScratchInit(b200_context* ctx) {
  if (ctx->device < 0 || ctx->device >= kMaxDevices) return B200_OK;   // (the static entry point refuses such a device itself)
  float* p = nullptr;
  return StaticScratch(ctx, &p);
}
}  // namespace b200

extern "C" {

size_t b200_attention_scratch_bytes(int64_t batch, int heads, int head_dim, int64_t max_len) {
  const int64_t splits = (max_len + kChunk - 1) / kChunk;
  return static_cast<size_t>(batch) * heads * splits * (head_dim + 2) * sizeof(float);
}

b200_status b200_attention_decode(b200_context* ctx, b200_stream stream, const void* q, const void* k_cache,
                                  const void* v_cache, void* out, const int32_t* pos, void* scratch, int64_t batch,
                                  int heads, int kv_heads, int head_dim, int64_t max_len) {
  AttnArgs a = {};
  a.q = static_cast<const __nv_bfloat16*>(q);
  a.k_cache = static_cast<__nv_bfloat16*>(const_cast<void*>(k_cache));
  a.v_cache = static_cast<__nv_bfloat16*>(const_cast<void*>(v_cache));
  a.out = static_cast<__nv_bfloat16*>(out);
  a.pos = pos;
  a.scratch = static_cast<float*>(scratch);
  a.heads = heads;
  a.kv_heads = kv_heads;
  a.max_len = max_len;
  return Run(ctx, stream, a, "b200_attention_decode", batch, head_dim);
}

b200_status b200_attention_step(b200_context* ctx, b200_stream stream, const void* qkv, const void* q_norm,
                                const void* k_norm, const float* inv_freq_or_null, void* k_cache, void* v_cache,
                                void* out, const int32_t* pos, void* scratch, int64_t batch, int heads,
                                int kv_heads, int head_dim, int64_t max_len, float theta, float eps) {
  AttnArgs a = {};
  a.qkv = static_cast<const __nv_bfloat16*>(qkv);
  a.q_norm = static_cast<const __nv_bfloat16*>(q_norm);
  a.k_norm = static_cast<const __nv_bfloat16*>(k_norm);
  a.inv_freq = inv_freq_or_null;
  a.k_cache = static_cast<__nv_bfloat16*>(k_cache);
  a.v_cache = static_cast<__nv_bfloat16*>(v_cache);
  a.out = static_cast<__nv_bfloat16*>(out);
  a.pos = pos;
  a.scratch = static_cast<float*>(scratch);
  a.heads = heads;
  a.kv_heads = kv_heads;
  a.max_len = max_len;
  a.theta = theta;
  a.eps = eps;
  return Run(ctx, stream, a, "b200_attention_step", batch, head_dim);
}

b200_status b200_attention_decode_static(b200_context* ctx, b200_stream stream, const void* q, const void* k_cache,
                                         const void* v_cache, void* out, const int32_t* pos, int64_t batch,
                                         int heads, int kv_heads, int head_dim, int64_t max_len) {
  b200_status s = BeginLaunch(ctx);   // makes the context's device current
  if (s != B200_OK) return s;
  if (batch < 0 || heads <= 0 || max_len <= 0 || (head_dim != 64 && head_dim != 128))
    return Fail(B200_INVALID_ARGUMENT, "b200_attention_decode_static: bad sizes");
  const size_t need = b200_attention_scratch_bytes(batch, heads, head_dim, max_len);
  if (need > kStaticScratchFloats * sizeof(float))
    return Fail(B200_RESOURCE_EXHAUSTED,
                "b200_attention_decode_static: batch %lld x heads %d x max_len %lld needs %zu bytes of scratch; the "
                "built-in scratch holds %zu (use b200_attention_decode with a caller buffer)",
                static_cast<long long>(batch), heads, static_cast<long long>(max_len), need,
                kStaticScratchFloats * sizeof(float));
  float* scratch = nullptr;
  s = StaticScratch(ctx, &scratch);
  if (s != B200_OK) return s;
  AttnArgs a = {};
  a.q = static_cast<const __nv_bfloat16*>(q);
  a.k_cache = static_cast<__nv_bfloat16*>(const_cast<void*>(k_cache));
  a.v_cache = static_cast<__nv_bfloat16*>(const_cast<void*>(v_cache));
  a.out = static_cast<__nv_bfloat16*>(out);
  a.pos = pos;
  a.scratch = scratch;   // every partial the merge reads is written earlier in the same call: nothing to clear
  a.heads = heads;
  a.kv_heads = kv_heads;
  a.max_len = max_len;
  return Run(ctx, stream, a, "b200_attention_decode_static", batch, head_dim);
}

}  // extern "C"
