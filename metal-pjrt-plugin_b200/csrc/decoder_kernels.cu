// The pieces of a decode step that sit between the projections
// (examples/llm/qwen3.py:270-331,366-376): embedding gather, per-head q/k
// RMSNorm + rotate-half RoPE + KV-cache write, and silu(gate)*up (attention is
// in attention.cu).
// All activations bf16, all arithmetic f32, rounded where the reference casts.
#include "common.cuh"

using namespace b200;

namespace {

// ---------------------------------------------------------------------------
// A token id outside [0, vocab) reads row 0 instead of memory outside the table and reports
// B200_INVALID_ARGUMENT through the status word.
__global__ void embed_kernel(const uint4* table, const int32_t* tokens, uint4* out, int vec_per_row, int64_t vocab,
                             int* status) {
  pdl_wait();
  pdl_launch_dependents();
  int64_t row = tokens[blockIdx.x];
  if (row < 0 || row >= vocab) {
    if (threadIdx.x == 0) report_status(status, B200_INVALID_ARGUMENT, 501);
    row = 0;
  }
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
  int* status;
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
  if (pos < 0 || pos >= a.max_len) {   // nothing may be written outside the cache
    if (lane == 0) report_status(a.status, B200_INVALID_ARGUMENT, 502);
    return;
  }
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

}  // namespace

extern "C" {

b200_status b200_embed(b200_context* ctx, b200_stream stream, const void* table, const int32_t* tokens, void* out,
                       int64_t batch, int64_t hidden, int64_t vocab) {
  b200_status s = BeginLaunch(ctx);
  if (s != B200_OK) return s;
  if (batch < 0 || hidden < 0 || vocab < 1) return Fail(B200_INVALID_ARGUMENT, "b200_embed: bad sizes");
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
                         static_cast<int>(hidden / 8), vocab, ctx->dev_status);
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
  a.status = ctx->dev_status;
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
