// Dequantise-to-matrix and load-time quantisers.
//   b200_dequantize ≙ dequantize (examples/llm/qwen3.py:199-207): w = q*s (+ b),
//     here in f32 with one rounding per operation (no fused multiply-add), so a
//     NumPy evaluation of the same expression matches it bit for bit.
//   b200_quantize   ≙ quantize_int8 / quantize_int4 (qwen3.py:154-196) in the
//     benchmark's variants: symmetric int8 per group (or per channel), min/max
//     affine int4 with eight consecutive-k nibbles per uint32; f32 arithmetic
//     with IEEE division and round-half-even, scale/offset stored as bf16.
#include "common.cuh"

using namespace b200;

namespace {

__device__ __forceinline__ int q_at(int bits, int order, const void* q, int64_t n, int64_t k, int64_t K) {
  if (bits == 8) return static_cast<const int8_t*>(q)[n * K + k];
  if (order == 0) {
    const uint32_t w = static_cast<const uint32_t*>(q)[n * (K / 8) + k / 8];
    return (w >> (4 * (k & 7))) & 0xF;
  }
  const int64_t g = k / 64;
  const int j = static_cast<int>(k % 64);
  const uint8_t b = static_cast<const uint8_t*>(q)[n * (K / 2) + g * 32 + (j & 31)];
  return j < 32 ? (b & 0xF) : (b >> 4);
}

template <typename OutT>
__global__ void dequantize_kernel(int bits, int order, int group, const void* q, const __nv_bfloat16* scale,
                                  const __nv_bfloat16* bias, OutT* out, int64_t N, int64_t K) {
  const int64_t total = N * K;
  const int64_t spr = K / group;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t n = i / K, k = i % K;
    const float qv = static_cast<float>(q_at(bits, order, q, n, k, K));
    const float s = __bfloat162float(scale[n * spr + k / group]);
    float w = __fmul_rn(qv, s);
    if (bias != nullptr) w = __fadd_rn(w, __bfloat162float(bias[n * spr + k / group]));
    out[i] = store_from_f32<OutT>(w);
  }
}

template <typename T>
__device__ __forceinline__ float ld(const T* p, int64_t i) { return load_as_f32<T>(p + i); }

// One warp per (row, group of 64): min/max affine, sequential nibbles.
template <typename T>
__global__ void quantize_int4_kernel(const T* w, uint32_t* q, __nv_bfloat16* scale, __nv_bfloat16* bias,
                                     int64_t N, int64_t K) {
  const int lane = threadIdx.x & 31;
  const int64_t groups = K / 64;
  const int64_t total = N * groups;
  const int64_t warps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  for (int64_t wg = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5; wg < total; wg += warps) {
    const int64_t n = wg / groups, g = wg % groups;
    const int64_t base = n * K + g * 64;
    const float v0 = ld(w, base + 2 * lane), v1 = ld(w, base + 2 * lane + 1);
    float lo = fminf(v0, v1), hi = fmaxf(v0, v1);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, o));
      hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, o));
    }
    const float s = __fdiv_rn(fmaxf(__fsub_rn(hi, lo), 1e-12f), 15.0f);
    const float q0 = fminf(fmaxf(rintf(__fdiv_rn(__fsub_rn(v0, lo), s)), 0.0f), 15.0f);
    const float q1 = fminf(fmaxf(rintf(__fdiv_rn(__fsub_rn(v1, lo), s)), 0.0f), 15.0f);
    // lane holds elements 2*lane, 2*lane+1 of the group: word = lane / 4, nibbles 2*(lane%4), +1
    uint32_t word = (static_cast<uint32_t>(q0) | (static_cast<uint32_t>(q1) << 4)) << (8 * (lane & 3));
    word |= __shfl_xor_sync(0xffffffffu, word, 1);
    word |= __shfl_xor_sync(0xffffffffu, word, 2);
    if ((lane & 3) == 0) q[n * (K / 8) + g * 8 + (lane >> 2)] = word;
    if (lane == 0) {
      scale[n * groups + g] = __float2bfloat16_rn(s);
      bias[n * groups + g] = __float2bfloat16_rn(lo);
    }
  }
}

// The reference's own 4-bit grid (quantize_int4, examples/llm/qwen3.py:169-196, MLX's affine
// grid): anchored at the group's largest-magnitude edge and stretched so that zero falls on
// it; the step may be negative.  Output in the reference's layout: byte j of a group holds
// element j in its low nibble and element j + 32 in its high nibble.  One warp per (row, group),
// lane j owns byte j.  Every operation is the IEEE f32 one NumPy performs, so the result is the
// reference's bit for bit.
template <typename T>
__global__ void quantize_int4_ref_kernel(const T* w, uint8_t* q, __nv_bfloat16* scale, __nv_bfloat16* bias, int64_t N,
                                         int64_t K) {
  const int lane = threadIdx.x & 31;
  const int64_t groups = K / 64;
  const int64_t total = N * groups;
  const int64_t warps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  for (int64_t wg = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5; wg < total; wg += warps) {
    const int64_t n = wg / groups, g = wg % groups;
    const int64_t base = n * K + g * 64;
    const float v0 = ld(w, base + lane), v1 = ld(w, base + lane + 32);
    float lo = fminf(v0, v1), hi = fmaxf(v0, v1);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, o));
      hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, o));
    }
    const bool neg = fabsf(lo) > fabsf(hi);
    float s = __fdiv_rn(fmaxf(__fsub_rn(hi, lo), 1e-12f), 15.0f);
    s = neg ? s : -s;
    const float edge = neg ? lo : hi;
    const float q0 = rintf(__fdiv_rn(edge, s));
    if (q0 != 0.0f) s = __fdiv_rn(edge, q0);
    const float b = q0 == 0.0f ? 0.0f : edge;
    const float qa = fminf(fmaxf(rintf(__fdiv_rn(__fsub_rn(v0, b), s)), 0.0f), 15.0f);
    const float qb = fminf(fmaxf(rintf(__fdiv_rn(__fsub_rn(v1, b), s)), 0.0f), 15.0f);
    q[(n * groups + g) * 32 + lane] = static_cast<uint8_t>(static_cast<uint32_t>(qa) | (static_cast<uint32_t>(qb) << 4));
    if (lane == 0) {
      scale[n * groups + g] = __float2bfloat16_rn(s);
      bias[n * groups + g] = __float2bfloat16_rn(b);
    }
  }
}

// Split-half bytes [N, K/64, 32] -> sequential words [N, K/8] (element k = 8i + j at bits 4j..4j+3).
__global__ void repack_int4_kernel(const uint8_t* in, uint32_t* out, int64_t words) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < words;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t group = i >> 3;
    const int wi = static_cast<int>(i & 7);          // word of the group: elements 8 wi .. 8 wi + 7
    const uint8_t* bytes = in + group * 32;
    uint32_t word = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int e = 8 * wi + j;                       // element of the group
      const uint32_t nib = e < 32 ? (bytes[e] & 15u) : (bytes[e - 32] >> 4);
      word |= nib << (4 * j);
    }
    out[i] = word;
  }
}

// dst row d = 16 t + j: gate row 8 t + j (j < 8) or up row 8 t + j - 8, i.e. source row inter + 8 t + j - 8.
__global__ void interleave_gate_up_kernel(const uint32_t* src, uint32_t* dst, int64_t inter, int64_t row_words) {
  const int64_t total = 2 * inter * row_words;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t d = i / row_words, w = i % row_words;
    const int64_t t = d >> 4, j = d & 15;
    const int64_t srow = j < 8 ? 8 * t + j : inter + 8 * t + (j - 8);
    dst[i] = src[srow * row_words + w];
  }
}

// One warp per (row, group): symmetric int8.
template <typename T>
__global__ void quantize_int8_kernel(const T* w, int8_t* q, __nv_bfloat16* scale, int64_t N, int64_t K, int group) {
  const int lane = threadIdx.x & 31;
  const int64_t groups = K / group;
  const int64_t total = N * groups;
  const int64_t warps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  for (int64_t wg = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5; wg < total; wg += warps) {
    const int64_t n = wg / groups, g = wg % groups;
    const int64_t base = n * K + g * group;
    float amax = 0.0f;
    for (int j = lane; j < group; j += 32) amax = fmaxf(amax, fabsf(ld(w, base + j)));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float s = __fdiv_rn(fmaxf(amax, 1e-12f), 127.0f);
    for (int j = lane; j < group; j += 32) {
      const float qv = fminf(fmaxf(rintf(__fdiv_rn(ld(w, base + j), s)), -127.0f), 127.0f);
      q[base + j] = static_cast<int8_t>(qv);
    }
    if (lane == 0) scale[n * groups + g] = __float2bfloat16_rn(s);
  }
}

}  // namespace

extern "C" {

b200_status b200_dequantize(b200_context* ctx, b200_stream stream, int bits, int group, int nibble_order,
                            const void* q, const void* scale, const void* bias_or_null, void* w_out, int64_t N,
                            int64_t K, int out_dtype) {
  b200_status s = BeginLaunch(ctx);
  if (s != B200_OK) return s;
  if (bits != 4 && bits != 8) return Fail(B200_INVALID_ARGUMENT, "b200_dequantize: bits must be 4 or 8");
  if (N < 0 || K < 0) return Fail(B200_INVALID_ARGUMENT, "b200_dequantize: negative size");
  if (N == 0 || K == 0) return B200_OK;
  if (group <= 0 || K % group != 0 || (bits == 4 && (group != 64 || K % 64 != 0)))
    return Fail(B200_UNIMPLEMENTED, "b200_dequantize: group %d does not divide K=%lld (int4 needs 64)", group,
                static_cast<long long>(K));
  if (bits == 4 && bias_or_null == nullptr) return Fail(B200_INVALID_ARGUMENT, "b200_dequantize: int4 needs a bias");
  if (q == nullptr || scale == nullptr || w_out == nullptr) return Fail(B200_INVALID_ARGUMENT, "b200_dequantize: null buffer");
  if (out_dtype != B200_F32 && out_dtype != B200_BF16)
    return Fail(B200_UNIMPLEMENTED, "b200_dequantize: output must be f32 or bf16");
  const int threads = 256;
  const int blocks = static_cast<int>(std::min<int64_t>(CeilDiv(N * K, threads), 148 * 16));
  const __nv_bfloat16* sc = static_cast<const __nv_bfloat16*>(scale);
  const __nv_bfloat16* bi = bits == 4 ? static_cast<const __nv_bfloat16*>(bias_or_null) : nullptr;
  if (out_dtype == B200_F32)
    dequantize_kernel<float><<<blocks, threads, 0, stream>>>(bits, nibble_order, group, q, sc, bi,
                                                             static_cast<float*>(w_out), N, K);
  else
    dequantize_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>(bits, nibble_order, group, q, sc, bi,
                                                                     static_cast<__nv_bfloat16*>(w_out), N, K);
  return EndLaunch(ctx, "b200_dequantize");
}

b200_status b200_quantize(b200_context* ctx, b200_stream stream, int bits, int group, const void* w, int w_dtype,
                          void* q_out, void* scale_out, void* bias_out, int64_t N, int64_t K) {
  b200_status s = BeginLaunch(ctx);
  if (s != B200_OK) return s;
  if (bits != 4 && bits != 8) return Fail(B200_INVALID_ARGUMENT, "b200_quantize: bits must be 4 or 8");
  if (w_dtype != B200_F32 && w_dtype != B200_BF16) return Fail(B200_UNIMPLEMENTED, "b200_quantize: w must be f32 or bf16");
  if (N < 0 || K < 0) return Fail(B200_INVALID_ARGUMENT, "b200_quantize: negative size");
  if (N == 0 || K == 0) return B200_OK;
  if (group <= 0 || K % group != 0 || (bits == 4 && group != 64))
    return Fail(B200_UNIMPLEMENTED, "b200_quantize: group %d unsupported for K=%lld", group, static_cast<long long>(K));
  if (w == nullptr || q_out == nullptr || scale_out == nullptr || (bits == 4 && bias_out == nullptr))
    return Fail(B200_INVALID_ARGUMENT, "b200_quantize: null buffer");
  const int threads = 256;
  const int64_t warps_needed = N * (K / group);
  const int blocks = static_cast<int>(std::min<int64_t>(CeilDiv(warps_needed, threads / 32), 148 * 32));
  __nv_bfloat16* sc = static_cast<__nv_bfloat16*>(scale_out);
  if (bits == 4) {
    if (w_dtype == B200_F32)
      quantize_int4_kernel<float><<<blocks, threads, 0, stream>>>(static_cast<const float*>(w),
                                                                  static_cast<uint32_t*>(q_out), sc,
                                                                  static_cast<__nv_bfloat16*>(bias_out), N, K);
    else
      quantize_int4_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>(
          static_cast<const __nv_bfloat16*>(w), static_cast<uint32_t*>(q_out), sc,
          static_cast<__nv_bfloat16*>(bias_out), N, K);
  } else {
    if (w_dtype == B200_F32)
      quantize_int8_kernel<float><<<blocks, threads, 0, stream>>>(static_cast<const float*>(w),
                                                                  static_cast<int8_t*>(q_out), sc, N, K, group);
    else
      quantize_int8_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>(
          static_cast<const __nv_bfloat16*>(w), static_cast<int8_t*>(q_out), sc, N, K, group);
  }
  return EndLaunch(ctx, "b200_quantize");
}

b200_status b200_quantize_int4_ref(b200_context* ctx, b200_stream stream, const void* w, int w_dtype, void* q_out,
                                   void* scale_out, void* bias_out, int64_t N, int64_t K) {
  b200_status s = BeginLaunch(ctx);
  if (s != B200_OK) return s;
  if (w_dtype != B200_F32 && w_dtype != B200_BF16) return Fail(B200_UNIMPLEMENTED, "b200_quantize_int4_ref: w must be f32 or bf16");
  if (N < 0 || K < 0) return Fail(B200_INVALID_ARGUMENT, "b200_quantize_int4_ref: negative size");
  if (N == 0 || K == 0) return B200_OK;
  if (K % 64 != 0) return Fail(B200_UNIMPLEMENTED, "b200_quantize_int4_ref: K=%lld is not a multiple of the group (64)", static_cast<long long>(K));
  if (w == nullptr || q_out == nullptr || scale_out == nullptr || bias_out == nullptr)
    return Fail(B200_INVALID_ARGUMENT, "b200_quantize_int4_ref: null buffer");
  const int threads = 256;
  const int blocks = static_cast<int>(std::min<int64_t>(CeilDiv(N * (K / 64), threads / 32), 148 * 32));
  if (w_dtype == B200_F32)
    quantize_int4_ref_kernel<float><<<blocks, threads, 0, stream>>>(static_cast<const float*>(w), static_cast<uint8_t*>(q_out),
                                                                    static_cast<__nv_bfloat16*>(scale_out),
                                                                    static_cast<__nv_bfloat16*>(bias_out), N, K);
  else
    quantize_int4_ref_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(w), static_cast<uint8_t*>(q_out), static_cast<__nv_bfloat16*>(scale_out),
        static_cast<__nv_bfloat16*>(bias_out), N, K);
  return EndLaunch(ctx, "b200_quantize_int4_ref");
}

b200_status b200_repack_int4(b200_context* ctx, b200_stream stream, const void* q_split_half, void* q_sequential, int64_t N,
                             int64_t K) {
  b200_status s = BeginLaunch(ctx);
  if (s != B200_OK) return s;
  if (N < 0 || K < 0) return Fail(B200_INVALID_ARGUMENT, "b200_repack_int4: negative size");
  if (N == 0 || K == 0) return B200_OK;
  if (K % 64 != 0) return Fail(B200_UNIMPLEMENTED, "b200_repack_int4: K=%lld is not a multiple of 64", static_cast<long long>(K));
  if (q_split_half == nullptr || q_sequential == nullptr) return Fail(B200_INVALID_ARGUMENT, "b200_repack_int4: null buffer");
  const int64_t words = N * (K / 8);
  const int blocks = static_cast<int>(std::min<int64_t>(CeilDiv(words, 256), 148 * 16));
  repack_int4_kernel<<<blocks, 256, 0, stream>>>(static_cast<const uint8_t*>(q_split_half), static_cast<uint32_t*>(q_sequential), words);
  return EndLaunch(ctx, "b200_repack_int4");
}

b200_status b200_interleave_gate_up(b200_context* ctx, b200_stream stream, const void* src, void* dst, int64_t inter,
                                    int64_t row_bytes) {
  b200_status s = BeginLaunch(ctx);
  if (s != B200_OK) return s;
  if (inter < 0 || row_bytes < 0) return Fail(B200_INVALID_ARGUMENT, "b200_interleave_gate_up: negative size");
  if (inter == 0 || row_bytes == 0) return B200_OK;
  if (inter % 8 != 0 || row_bytes % 4 != 0)
    return Fail(B200_UNIMPLEMENTED, "b200_interleave_gate_up: inter must be a multiple of 8 and rows a multiple of 4 bytes");
  if (src == nullptr || dst == nullptr || src == dst || !Aligned(src, 4) || !Aligned(dst, 4))
    return Fail(B200_INVALID_ARGUMENT, "b200_interleave_gate_up: null, aliased or unaligned buffer");
  const int64_t total = 2 * inter * (row_bytes / 4);
  const int blocks = static_cast<int>(std::min<int64_t>(CeilDiv(total, 256), 148 * 32));
  interleave_gate_up_kernel<<<blocks, 256, 0, stream>>>(static_cast<const uint32_t*>(src), static_cast<uint32_t*>(dst), inter, row_bytes / 4);
  return EndLaunch(ctx, "b200_interleave_gate_up");
}

}  // extern "C"
