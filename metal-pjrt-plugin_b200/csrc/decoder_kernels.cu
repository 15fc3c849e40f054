// The pieces of a decode step that sit between the projections
// (examples/llm/qwen3.py:270-331,366-376): embedding gather, per-head q/k
// RMSNorm + rotate-half RoPE + KV-cache write, grouped-query decode attention
// over the cache (K [B,KV,S,D], V [B,KV,D,S], both reduced over their minor
// axis as the reference lays them out, qwen3.py:279-291), and silu(gate)*up.
// All activations bf16, all arithmetic f32, rounded where the reference casts.
#include "common.cuh"

using namespace b200;

namespace {

// ---------------------------------------------------------------------------
__global__ void embed_kernel(const uint4* table, const int32_t* tokens, uint4* out, int vec_per_row) {
  pdl_wait();
  pdl_launch_dependents();
  const int64_t row = tokens[blockIdx.x];
  for (int i = threadIdx.x; i < vec_per_row; i += blockDim.x)
    out[static_cast<int64_t>(blockIdx.x) * vec_per_row + i] = __ldg(table + row * vec_per_row + i);
}

// ---------------------------------------------------------------------------
// One warp per head.  Heads 0..H-1 are queries, H..H+KV-1 keys, then values.
struct QkArgs {
  const __nv_bfloat16* qkv;
  const __nv_bfloat16* q_norm;
  const __nv_bfloat16* k_norm;
  __nv_bfloat16* q_out;
  __nv_bfloat16* k_cache;
  __nv_bfloat16* v_cache;
  const int32_t* pos;
  int heads, kv_heads, head_dim;
  int64_t max_len;
  float theta, eps;
};

template <int D>
__global__ void qk_norm_rope_cache_kernel(const QkArgs a) {
  pdl_wait();
  pdl_launch_dependents();
  constexpr int PAIRS = D / 64;  // rotate-half pairs (i, i + D/2) per lane
  const int lane = threadIdx.x & 31;
  const int head = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int total_heads = a.heads + 2 * a.kv_heads;
  if (head >= total_heads) return;
  const int b = blockIdx.y;
  const int pos = *a.pos;
  const __nv_bfloat16* src = a.qkv + (static_cast<int64_t>(b) * total_heads + head) * D;

  if (head >= a.heads + a.kv_heads) {  // value head: transposed cache write, V[b, kv, d, pos]
    const int kv = head - a.heads - a.kv_heads;
    __nv_bfloat16* dst = a.v_cache + (static_cast<int64_t>(b) * a.kv_heads + kv) * D * a.max_len + pos;
    for (int d = lane; d < D; d += 32) dst[static_cast<int64_t>(d) * a.max_len] = src[d];
    return;
  }
  const bool is_q = head < a.heads;
  const __nv_bfloat16* w = is_q ? a.q_norm : a.k_norm;
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
  __nv_bfloat16* dst = is_q ? a.q_out + (static_cast<int64_t>(b) * a.heads + head) * D
                            : a.k_cache + ((static_cast<int64_t>(b) * a.kv_heads + (head - a.heads)) * a.max_len + pos) * D;
#pragma unroll
  for (int p = 0; p < PAIRS; ++p) {
    const int i = lane + 32 * p;
    // rms_norm rounds to bf16 before rope widens again (qwen3.py:297,306)
    const float n1 = bf16_round((x1[p] * r) * __bfloat162float(w[i]));
    const float n2 = bf16_round((x2[p] * r) * __bfloat162float(w[i + D / 2]));
    const float inv_freq = static_cast<float>(1.0 / pow(static_cast<double>(a.theta), static_cast<double>(2 * i) / D));
    const float ang = static_cast<float>(pos) * inv_freq;
    float sn, cs;
    sincosf(ang, &sn, &cs);
    dst[i] = __float2bfloat16_rn(n1 * cs - n2 * sn);
    dst[i + D / 2] = __float2bfloat16_rn(n2 * cs + n1 * sn);
  }
}

// ---------------------------------------------------------------------------
// Decode attention, split over the cache positions (partials + combine).
constexpr int kAttnChunk = 128;    // positions per CTA
constexpr int kAttnThreads = 128;
constexpr int kMaxGroup = 8;       // query heads per KV head

struct AttnArgs {
  const __nv_bfloat16* q;        // [B, H, D]
  const __nv_bfloat16* k_cache;  // [B, KV, S, D]
  const __nv_bfloat16* v_cache;  // [B, KV, D, S]
  __nv_bfloat16* out;            // [B, H, D]
  const int32_t* pos;
  float* scratch;                // [B, KV, splits, G, D + 2]
  int heads, kv_heads;
  int64_t max_len;
  int splits;
  float scale;
};

template <int D, int G>
__global__ void __launch_bounds__(kAttnThreads) attn_partial_kernel(const AttnArgs a) {
  __shared__ float qs[G][D];
  __shared__ float sc[G][kAttnChunk];
  __shared__ float red[G][kAttnThreads / 32];
  pdl_wait();
  pdl_launch_dependents();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int split = blockIdx.x, kv = blockIdx.y, b = blockIdx.z;
  const int n_valid = *a.pos + 1;
  const int s0 = split * kAttnChunk;
  if (s0 >= n_valid) return;  // the combine pass only reads splits below n_valid
  const int cnt = min(kAttnChunk, n_valid - s0);

  for (int i = tid; i < G * D; i += kAttnThreads) {
    const int gq = i / D, d = i % D;
    qs[gq][d] = __bfloat162float(a.q[(static_cast<int64_t>(b) * a.heads + kv * G + gq) * D + d]);
  }
  __syncthreads();

  // scores: one cache position per thread, the whole K row from 16-byte loads
  float mx[G];
#pragma unroll
  for (int gq = 0; gq < G; ++gq) mx[gq] = -INFINITY;
  if (tid < cnt) {
    const uint4* krow = reinterpret_cast<const uint4*>(
        a.k_cache + ((static_cast<int64_t>(b) * a.kv_heads + kv) * a.max_len + s0 + tid) * D);
    float dot[G];
#pragma unroll
    for (int gq = 0; gq < G; ++gq) dot[gq] = 0.0f;
#pragma unroll 4
    for (int v = 0; v < D / 8; ++v) {
      const uint4 raw = __ldg(krow + v);
      const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float k0 = bf16_lo(w[j]), k1 = bf16_hi(w[j]);
#pragma unroll
        for (int gq = 0; gq < G; ++gq) {
          dot[gq] = fmaf(qs[gq][v * 8 + 2 * j], k0, dot[gq]);
          dot[gq] = fmaf(qs[gq][v * 8 + 2 * j + 1], k1, dot[gq]);
        }
      }
    }
#pragma unroll
    for (int gq = 0; gq < G; ++gq) {
      dot[gq] *= a.scale;
      sc[gq][tid] = dot[gq];
      mx[gq] = dot[gq];
    }
  }
#pragma unroll
  for (int gq = 0; gq < G; ++gq) {
    mx[gq] = warp_max(mx[gq]);
    if (lane == 0) red[gq][warp] = mx[gq];
  }
  __syncthreads();
  float lsum[G];
#pragma unroll
  for (int gq = 0; gq < G; ++gq) {
    float m = red[gq][0];
#pragma unroll
    for (int w = 1; w < kAttnThreads / 32; ++w) m = fmaxf(m, red[gq][w]);
    mx[gq] = m;
    float e = 0.0f;
    if (tid < cnt) {
      e = expf(sc[gq][tid] - m);
      sc[gq][tid] = e;
    }
    lsum[gq] = warp_sum(e);
  }
  __syncthreads();  // every thread has read red[][] (the maxima)
#pragma unroll
  for (int gq = 0; gq < G; ++gq)
    if (lane == 0) red[gq][warp] = lsum[gq];
  __syncthreads();

  // p . v: one output dimension per thread, V^T row d is contiguous over positions
  float* part = a.scratch + ((static_cast<int64_t>(b) * a.kv_heads + kv) * a.splits + split) * G * (D + 2);
  for (int d = tid; d < D; d += kAttnThreads) {
    const __nv_bfloat16* vrow = a.v_cache + ((static_cast<int64_t>(b) * a.kv_heads + kv) * D + d) * a.max_len + s0;
    float acc[G];
#pragma unroll
    for (int gq = 0; gq < G; ++gq) acc[gq] = 0.0f;
    int s = 0;
    if ((reinterpret_cast<uintptr_t>(vrow) & 15) == 0) {
      for (; s + 8 <= cnt; s += 8) {
        const uint4 raw = __ldg(reinterpret_cast<const uint4*>(vrow + s));
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float v0 = bf16_lo(w[j]), v1 = bf16_hi(w[j]);
#pragma unroll
          for (int gq = 0; gq < G; ++gq) {
            acc[gq] = fmaf(sc[gq][s + 2 * j], v0, acc[gq]);
            acc[gq] = fmaf(sc[gq][s + 2 * j + 1], v1, acc[gq]);
          }
        }
      }
    }
    for (; s < cnt; ++s) {
      const float v = __bfloat162float(vrow[s]);
#pragma unroll
      for (int gq = 0; gq < G; ++gq) acc[gq] = fmaf(sc[gq][s], v, acc[gq]);
    }
#pragma unroll
    for (int gq = 0; gq < G; ++gq) part[gq * (D + 2) + d] = acc[gq];
  }
  if (tid < G) {
    float l = 0.0f;
    for (int w = 0; w < kAttnThreads / 32; ++w) l += red[tid][w];
    part[tid * (D + 2) + D] = mx[tid];
    part[tid * (D + 2) + D + 1] = l;
  }
}

template <int D, int G>
__global__ void attn_combine_kernel(const AttnArgs a) {
  pdl_wait();
  pdl_launch_dependents();
  const int h = blockIdx.x, b = blockIdx.y;
  const int kv = h / G, gq = h % G;
  const int n_valid = *a.pos + 1;
  const int nsplit = (n_valid + kAttnChunk - 1) / kAttnChunk;
  const float* base = a.scratch + (static_cast<int64_t>(b) * a.kv_heads + kv) * a.splits * G * (D + 2) + gq * (D + 2);
  const int64_t stride = static_cast<int64_t>(G) * (D + 2);
  float m = -INFINITY;
  for (int s = 0; s < nsplit; ++s) m = fmaxf(m, base[s * stride + D]);
  float denom = 0.0f;
  for (int s = 0; s < nsplit; ++s) denom += expf(base[s * stride + D] - m) * base[s * stride + D + 1];
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float num = 0.0f;
    for (int s = 0; s < nsplit; ++s) num = fmaf(expf(base[s * stride + D] - m), base[s * stride + d], num);
    a.out[(static_cast<int64_t>(b) * a.heads + h) * D + d] = __float2bfloat16_rn(num / denom);
  }
}

// ---------------------------------------------------------------------------
__global__ void silu_mul_kernel(const __nv_bfloat16* gate_up, __nv_bfloat16* out, int64_t inter) {
  pdl_wait();
  pdl_launch_dependents();
  const int64_t b = blockIdx.y;
  const __nv_bfloat16* gp = gate_up + b * 2 * inter;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < inter;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const float g = __bfloat162float(gp[i]);
    const float u = __bfloat162float(gp[inter + i]);
    // jax.nn.silu(gate) * up on bf16: sigmoid, gate*sigmoid and the product with up each round
    const float sig = bf16_round(1.0f / (1.0f + expf(-g)));
    const float act = bf16_round(g * sig);
    out[b * inter + i] = __float2bfloat16_rn(act * u);
  }
}

template <int D>
b200_status LaunchAttn(b200_context* ctx, cudaStream_t stream, const AttnArgs& a, int group, int64_t batch) {
  LaunchCfg lc;
  lc.stream = stream;
  lc.pdl = true;
  lc.block = dim3(kAttnThreads);
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
  lc.block = dim3(D < 128 ? D : 128);
  lc.grid = dim3(a.heads, static_cast<unsigned>(batch));
  switch (group) {
    case 1: e = Launch(lc, attn_combine_kernel<D, 1>, a); break;
    case 2: e = Launch(lc, attn_combine_kernel<D, 2>, a); break;
    case 4: e = Launch(lc, attn_combine_kernel<D, 4>, a); break;
    default: e = Launch(lc, attn_combine_kernel<D, 8>, a); break;
  }
  if (e != cudaSuccess) return Stick(ctx, Fail(B200_INTERNAL, "attention combine launch: %s", cudaGetErrorString(e)));
  return EndLaunch(ctx, "b200_attention_decode", 2);
}

}  // namespace

extern "C" {

b200_status b200_embed(b200_context* ctx, b200_stream stream, const void* table, const int32_t* tokens, void* out,
                       int64_t batch, int64_t hidden) {
  b200_status s = BeginLaunch(ctx);
  if (s != B200_OK) return s;
  if (batch < 0 || hidden < 0) return Fail(B200_INVALID_ARGUMENT, "b200_embed: negative size");
  if (batch == 0 || hidden == 0) return B200_OK;
  if (table == nullptr || tokens == nullptr || out == nullptr) return Fail(B200_INVALID_ARGUMENT, "b200_embed: null buffer");
  if (hidden % 8 != 0 || !Aligned(table, 16) || !Aligned(out, 16))
    return Fail(B200_UNIMPLEMENTED, "b200_embed: hidden must be a multiple of 8 and buffers 16-byte aligned");
  LaunchCfg lc;
  lc.stream = stream;
  lc.pdl = true;
  lc.grid = dim3(static_cast<unsigned>(batch));
  lc.block = dim3(128);
  cudaError_t e = Launch(lc, embed_kernel, static_cast<const uint4*>(table), tokens, static_cast<uint4*>(out),
                         static_cast<int>(hidden / 8));
  if (e != cudaSuccess) return Stick(ctx, Fail(B200_INTERNAL, "b200_embed launch: %s", cudaGetErrorString(e)));
  return EndLaunch(ctx, "b200_embed");
}

b200_status b200_qk_norm_rope_cache(b200_context* ctx, b200_stream stream, const void* qkv, const void* q_norm,
                                    const void* k_norm, void* q_out, void* k_cache, void* v_cache,
                                    const int32_t* pos, int64_t batch, int heads, int kv_heads, int head_dim,
                                    int64_t max_len, float theta, float eps) {
  b200_status s = BeginLaunch(ctx);
  if (s != B200_OK) return s;
  if (batch < 0 || heads <= 0 || kv_heads <= 0 || max_len <= 0)
    return Fail(B200_INVALID_ARGUMENT, "b200_qk_norm_rope_cache: bad sizes");
  if (head_dim != 64 && head_dim != 128)
    return Fail(B200_UNIMPLEMENTED, "b200_qk_norm_rope_cache: head_dim %d (64 or 128)", head_dim);
  if (batch == 0) return B200_OK;
  if (!qkv || !q_norm || !k_norm || !q_out || !k_cache || !v_cache || !pos)
    return Fail(B200_INVALID_ARGUMENT, "b200_qk_norm_rope_cache: null buffer");
  QkArgs a;
  a.qkv = static_cast<const __nv_bfloat16*>(qkv);
  a.q_norm = static_cast<const __nv_bfloat16*>(q_norm);
  a.k_norm = static_cast<const __nv_bfloat16*>(k_norm);
  a.q_out = static_cast<__nv_bfloat16*>(q_out);
  a.k_cache = static_cast<__nv_bfloat16*>(k_cache);
  a.v_cache = static_cast<__nv_bfloat16*>(v_cache);
  a.pos = pos;
  a.heads = heads;
  a.kv_heads = kv_heads;
  a.head_dim = head_dim;
  a.max_len = max_len;
  a.theta = theta;
  a.eps = eps;
  const int total = heads + 2 * kv_heads;
  LaunchCfg lc;
  lc.stream = stream;
  lc.pdl = true;
  lc.block = dim3(128);
  lc.grid = dim3((total + 3) / 4, static_cast<unsigned>(batch));
  cudaError_t e = head_dim == 128 ? Launch(lc, qk_norm_rope_cache_kernel<128>, a)
                                  : Launch(lc, qk_norm_rope_cache_kernel<64>, a);
  if (e != cudaSuccess) return Stick(ctx, Fail(B200_INTERNAL, "b200_qk_norm_rope_cache launch: %s", cudaGetErrorString(e)));
  return EndLaunch(ctx, "b200_qk_norm_rope_cache");
}

size_t b200_attention_scratch_bytes(int64_t batch, int heads, int head_dim, int64_t max_len) {
  const int64_t splits = (max_len + kAttnChunk - 1) / kAttnChunk;
  return static_cast<size_t>(batch) * heads * splits * (head_dim + 2) * sizeof(float);
}

b200_status b200_attention_decode(b200_context* ctx, b200_stream stream, const void* q, const void* k_cache,
                                  const void* v_cache, void* out, const int32_t* pos, void* scratch,
                                  int64_t batch, int heads, int kv_heads, int head_dim, int64_t max_len) {
  b200_status s = BeginLaunch(ctx);
  if (s != B200_OK) return s;
  if (batch < 0 || heads <= 0 || kv_heads <= 0 || max_len <= 0 || heads % kv_heads != 0)
    return Fail(B200_INVALID_ARGUMENT, "b200_attention_decode: bad sizes");
  if (head_dim != 64 && head_dim != 128)
    return Fail(B200_UNIMPLEMENTED, "b200_attention_decode: head_dim %d (64 or 128)", head_dim);
  if (batch > 65535) return Fail(B200_UNIMPLEMENTED, "b200_attention_decode: batch too large");
  if (batch == 0) return B200_OK;
  if (!q || !k_cache || !v_cache || !out || !pos || !scratch)
    return Fail(B200_INVALID_ARGUMENT, "b200_attention_decode: null buffer");
  if (!Aligned(k_cache, 16) || !Aligned(v_cache, 16))
    return Fail(B200_INVALID_ARGUMENT, "b200_attention_decode: caches must be 16-byte aligned");
  AttnArgs a;
  a.q = static_cast<const __nv_bfloat16*>(q);
  a.k_cache = static_cast<const __nv_bfloat16*>(k_cache);
  a.v_cache = static_cast<const __nv_bfloat16*>(v_cache);
  a.out = static_cast<__nv_bfloat16*>(out);
  a.pos = pos;
  a.scratch = static_cast<float*>(scratch);
  a.heads = heads;
  a.kv_heads = kv_heads;
  a.max_len = max_len;
  a.splits = static_cast<int>((max_len + kAttnChunk - 1) / kAttnChunk);
  a.scale = 1.0f / sqrtf(static_cast<float>(head_dim));
  return head_dim == 128 ? LaunchAttn<128>(ctx, stream, a, heads / kv_heads, batch)
                         : LaunchAttn<64>(ctx, stream, a, heads / kv_heads, batch);
}

b200_status b200_silu_mul(b200_context* ctx, b200_stream stream, const void* gate_up, void* out, int64_t batch,
                          int64_t inter) {
  b200_status s = BeginLaunch(ctx);
  if (s != B200_OK) return s;
  if (batch < 0 || inter < 0) return Fail(B200_INVALID_ARGUMENT, "b200_silu_mul: negative size");
  if (batch == 0 || inter == 0) return B200_OK;
  if (batch > 65535) return Fail(B200_UNIMPLEMENTED, "b200_silu_mul: batch too large");
  if (!gate_up || !out) return Fail(B200_INVALID_ARGUMENT, "b200_silu_mul: null buffer");
  LaunchCfg lc;
  lc.stream = stream;
  lc.pdl = true;
  lc.block = dim3(256);
  lc.grid = dim3(static_cast<unsigned>(std::min<int64_t>(CeilDiv(inter, 256), 64)), static_cast<unsigned>(batch));
  cudaError_t e = Launch(lc, silu_mul_kernel, static_cast<const __nv_bfloat16*>(gate_up),
                         static_cast<__nv_bfloat16*>(out), inter);
  if (e != cudaSuccess) return Stick(ctx, Fail(B200_INTERNAL, "b200_silu_mul launch: %s", cudaGetErrorString(e)));
  return EndLaunch(ctx, "b200_silu_mul");
}

}  // extern "C"
