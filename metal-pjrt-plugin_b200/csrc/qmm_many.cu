// Weight-only quantised matmul for MORE than 32 rows of x (prefill-sized batches): the weights are
// dequantised panel by panel into a bf16 workspace that stays in L2 and each panel goes through the
// tcgen05 GEMM (≙ the reference beyond ROWS_MAX: dequantize(w, dtype), then x @ w.T,
// examples/llm/qwen3.py:199-230).  HBM sees the quantised weights once; the 4x larger bf16 panel
// is written and read back inside the 126 MB L2 (a panel is at most 32 MB, and the same buffer is
// reused for every panel, so its lines are overwritten before they are evicted).
#include <algorithm>

#include "common.cuh"
#include "qmm_many.cuh"

using namespace b200;

namespace {

constexpr int64_t kPanelBytes = 32ll << 20;

// Sequential int4 in groups of 64: one thread per 8 inputs (one word), 16-byte stores.
__global__ void dequant_int4_seq_kernel(const uint32_t* q, const __nv_bfloat16* scale, const __nv_bfloat16* bias, uint4* out,
                                        int64_t words, int words_per_row) {
  pdl_wait();   // the GEMM of the panel before still reads the workspace
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < words;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t n = i / words_per_row;
    const int w = static_cast<int>(i % words_per_row);
    const uint32_t v = __ldg(q + i);
    const int64_t g = n * (words_per_row / 8) + w / 8;
    const float s = __bfloat162float(scale[g]), b = __bfloat162float(bias[g]);
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      // w = q*s + b in f32 with one rounding per operation, then one rounding to bf16 (b200_dequantize's values)
      const float lo = __fadd_rn(__fmul_rn(static_cast<float>((v >> (8 * j)) & 15u), s), b);
      const float hi = __fadd_rn(__fmul_rn(static_cast<float>((v >> (8 * j + 4)) & 15u), s), b);
      o[j] = pack_bf16(lo, hi);
    }
    out[i] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

}  // namespace

namespace b200 {

b200_status QmmManyRows(b200_context* ctx, cudaStream_t stream, const b200_qmm_params* p) {
  if (p->prologue != B200_QMM_PRO_NONE)
    return Fail(B200_UNIMPLEMENTED, "b200_qmm: the fused input transforms take up to 32 rows (8 for RMSNorm); M = %lld",
                static_cast<long long>(p->M));
  if (p->epilogue == B200_QMM_OUT_F32)
    return Fail(B200_UNIMPLEMENTED, "b200_qmm: above 32 rows the output is bf16, bf16 + residual, or raw f32");
  const int64_t M = p->M, N = p->N, K = p->K;
  const int64_t ldx = p->ldx ? p->ldx : K, ldo = p->ldo ? p->ldo : N;
  const bool f32_out = p->epilogue == B200_QMM_OUT_F32_RAW;
  const size_t esz = f32_out ? 4 : 2;
  // bf16 weights need no workspace: one GEMM over the whole matrix
  int64_t panel = N;
  if (p->bits != 16) {
    panel = std::max<int64_t>(256, (kPanelBytes / (K * 2)) / 256 * 256);
    panel = std::min(panel, N);
    const size_t need = static_cast<size_t>(panel) * K * 2;
    std::lock_guard<std::mutex> lock(ctx->mu);
    if (ctx->qmm_ws_bytes < need) {
      // grown on first use (not inside a stream capture: reserve by running the shape once before capturing)
      if (ctx->qmm_ws != nullptr) {
        cudaStreamSynchronize(stream);
        cudaFree(ctx->qmm_ws);
        ctx->qmm_ws = nullptr;
        ctx->qmm_ws_bytes = 0;
      }
      cudaError_t e = cudaMalloc(&ctx->qmm_ws, need);
      if (e != cudaSuccess) {
        (void)cudaGetLastError();
        return Fail(B200_RESOURCE_EXHAUSTED, "b200_qmm: %zu bytes of dequantisation workspace: %s", need, cudaGetErrorString(e));
      }
      ctx->qmm_ws_bytes = need;
    }
  }
  if (p->epilogue == B200_QMM_ADD_RESIDUAL && p->residual != p->out) {
    cudaError_t e = cudaMemcpy2DAsync(p->out, ldo * 2, p->residual, ldo * 2, N * 2, M, cudaMemcpyDeviceToDevice, stream);
    if (e != cudaSuccess) return Stick(ctx, Fail(B200_INTERNAL, "b200_qmm: residual copy: %s", cudaGetErrorString(e)));
  }
  const int64_t row_bytes = p->bits == 4 ? K / 2 : (p->bits == 8 ? K : 2 * K);
  const int64_t spr = p->bits == 16 ? 0 : K / p->group;
  for (int64_t r0 = 0; r0 < N; r0 += panel) {
    const int64_t rows = std::min(panel, N - r0);
    const uint8_t* qp = static_cast<const uint8_t*>(p->q) + r0 * row_bytes;
    const void* wmat = qp;
    if (p->bits != 16) {
      const __nv_bfloat16* sp = static_cast<const __nv_bfloat16*>(p->scale) + r0 * spr;
      const __nv_bfloat16* bp = p->bits == 4 ? static_cast<const __nv_bfloat16*>(p->bias) + r0 * spr : nullptr;
      if (p->bits == 4 && p->nibble_order == 0 && Aligned(ctx->qmm_ws, 16)) {
        b200_status s = BeginLaunch(ctx);
        if (s != B200_OK) return s;
        const int64_t words = rows * (K / 8);
        LaunchCfg lc;
        lc.grid = dim3(static_cast<unsigned>(std::min<int64_t>(CeilDiv(words, 256), ctx->sm_count * 16)));
        lc.block = dim3(256);
        lc.stream = stream;
        lc.pdl = true;
        cudaError_t e = Launch(lc, dequant_int4_seq_kernel, reinterpret_cast<const uint32_t*>(qp), sp, bp,
                               static_cast<uint4*>(ctx->qmm_ws), words, static_cast<int>(K / 8));
        if (e != cudaSuccess) return Stick(ctx, Fail(B200_INTERNAL, "b200_qmm: dequantise launch: %s", cudaGetErrorString(e)));
        s = EndLaunch(ctx, "b200_qmm (dequantise)");
        if (s != B200_OK) return s;
      } else {
        b200_status s = b200_dequantize(ctx, stream, p->bits, p->group, p->nibble_order, qp, sp, bp, ctx->qmm_ws, rows, K, B200_BF16);
        if (s != B200_OK) return s;
      }
      wmat = ctx->qmm_ws;
    }
    // out[:, r0 : r0 + rows] = x . W_panel^T
    b200_gemm_params g = {};
    g.m = M;
    g.n = rows;
    g.k = K;
    g.batch = 1;
    g.alpha = 1.0;
    g.beta = p->epilogue == B200_QMM_ADD_RESIDUAL ? 1.0 : 0.0;
    g.a.ptr = const_cast<void*>(p->x);
    g.a.ld = ldx;
    g.a.dtype = B200_BF16;
    g.b.ptr = const_cast<void*>(wmat);
    g.b.ld = K;
    g.b.dtype = B200_BF16;
    g.b.transpose = 1;
    g.c.ptr = static_cast<uint8_t*>(p->out) + static_cast<size_t>(r0) * esz;
    g.c.ld = ldo;
    g.c.dtype = f32_out ? B200_F32 : B200_BF16;
    b200_epilogue epi = {};
    b200_status s = b200_gemm(ctx, stream, &g, &epi);
    if (s != B200_OK) return s;
  }
  return B200_OK;
}

}  // namespace b200
