// Dense GEMM with the fused epilogue: validation, routing and the SIMT tile
// kernel.  Semantics kept from the reference: GemmParams / SteelEpilogue
// (metal_pjrt/blas/mps_gemm.h:23-53, steel_gemm.h:38-46), the acceptance rules
// of SteelGemmSupports / RunSteelGemm (steel_gemm.cc:140-196), and the
// per-element epilogue of kernels/steel_gemm.metal:217-225:
//     v = alpha*acc (+ beta*D) (+ bias[col]);  aux = T(v);  D = T(act(v)).
// Routing replaces ChooseGemv / ChooseSteelTile (gemv.cc:68-108,
// steel_gemm.cc:115-138) with three B200 kernels:
//   tcgen05  - TMA-fed tensor-core tiles with TMEM accumulators (gemm_tcgen05.cu),
//              for 16-bit operands whose layout the TMA descriptors accept;
//   few-row  - the bandwidth-bound streaming kernel (qmm.cu, 16-bit weights), for
//              x . W^T with up to 32 rows on either side; preferred up to 8 rows, above
//              that the tensor-core route (which splits K across a cluster) is faster;
//   SIMT     - the general tile kernel below: every dtype, transpose, stride,
//              batch and beta; true f32 arithmetic for f32 operands (tensor
//              cores have no f32 multiply, and the f32 block must hold rtol 1e-5).
#include <algorithm>

#include "common.cuh"

using namespace b200;

namespace b200 {
b200_status RunFewRowNT(b200_context* ctx, cudaStream_t stream, const void* mat, const void* vecs, void* out,
                        int64_t R, int64_t V, int64_t K, int64_t ld_vec, int64_t out_row_stride,
                        int64_t out_vec_stride, float alpha, int act, const void* bias, int bias_by_vec,
                        void* aux, int out_f32);
// gemm_tcgen05.cu
bool Tcgen05Supports(const b200_gemm_params* p, const b200_epilogue* epi);
b200_status RunTcgen05(b200_context* ctx, cudaStream_t stream, const b200_gemm_params* p, const b200_epilogue* epi);
}  // namespace b200

namespace {

constexpr int64_t kMaxInt = INT32_MAX;
constexpr int64_t kMaxLd = INT32_MAX / 256;  // steel_gemm.cc:153

struct SimtArgs {
  const void* a;
  const void* b;
  void* d;
  const void* bias;
  void* aux;
  int m, n, k;
  int64_t lda, ldb, ldd;
  int64_t sa, sb, sd;  // batch strides
  int ta, tb;
  float alpha, beta;
  int act;
};

// 64x64 output tile, 16-wide K steps, 256 threads with a 4x4 micro-tile each.
template <typename TIn, typename TOut>
__global__ void __launch_bounds__(256) gemm_simt_kernel(const SimtArgs p) {
  constexpr int BM = 64, BN = 64, BK = 16;
  __shared__ float As[BK][BM + 4];
  __shared__ float Bs[BK][BN + 4];
  pdl_wait();
  pdl_launch_dependents();
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int64_t batch = blockIdx.z;
  const TIn* A = static_cast<const TIn*>(p.a) + batch * p.sa;
  const TIn* B = static_cast<const TIn*>(p.b) + batch * p.sb;
  TOut* D = static_cast<TOut*>(p.d) + batch * p.sd;
  TOut* AUX = p.aux ? static_cast<TOut*>(p.aux) + batch * p.sd : nullptr;

  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

  for (int k0 = 0; k0 < p.k; k0 += BK) {
    // A tile: BM x BK.  Thread order follows the contiguous dimension of the operand.
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      const int idx = tid + it * 256;
      int i, kk;
      if (p.ta) { i = idx % BM; kk = idx / BM; } else { kk = idx % BK; i = idx / BK; }
      const int gi = m0 + i, gk = k0 + kk;
      float v = 0.0f;
      if (gi < p.m && gk < p.k)
        v = load_as_f32<TIn>(A + (p.ta ? static_cast<int64_t>(gk) * p.lda + gi : static_cast<int64_t>(gi) * p.lda + gk));
      As[kk][i] = v;
    }
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      const int idx = tid + it * 256;
      int j, kk;
      if (p.tb) { kk = idx % BK; j = idx / BK; } else { j = idx % BN; kk = idx / BN; }
      const int gj = n0 + j, gk = k0 + kk;
      float v = 0.0f;
      if (gj < p.n && gk < p.k)
        v = load_as_f32<TIn>(B + (p.tb ? static_cast<int64_t>(gj) * p.ldb + gk : static_cast<int64_t>(gk) * p.ldb + gj));
      Bs[kk][j] = v;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      const float4 av = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
      const float4 bv = *reinterpret_cast<const float4*>(&Bs[kk][tx * 4]);
      const float a4[4] = {av.x, av.y, av.z, av.w};
      const float b4[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a4[i], b4[j], acc[i][j]);
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gi = m0 + ty * 4 + i;
    if (gi >= p.m) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gj = n0 + tx * 4 + j;
      if (gj >= p.n) continue;
      const int64_t o = static_cast<int64_t>(gi) * p.ldd + gj;
      float v = p.alpha * acc[i][j];
      if (p.beta != 0.0f) v += p.beta * load_as_f32<TOut>(D + o);
      if (p.bias != nullptr) v += load_as_f32<TOut>(static_cast<const TOut*>(p.bias) + gj);
      if (AUX != nullptr) AUX[o] = store_from_f32<TOut>(v);
      D[o] = store_from_f32<TOut>(apply_act(p.act, v));
    }
  }
}

template <typename TIn, typename TOut>
cudaError_t LaunchSimt(const SimtArgs& a, int64_t batch, cudaStream_t stream) {
  LaunchCfg lc;
  lc.grid = dim3(static_cast<unsigned>(CeilDiv(a.n, 64)), static_cast<unsigned>(CeilDiv(a.m, 64)),
                 static_cast<unsigned>(batch));
  lc.block = dim3(256);
  lc.stream = stream;
  lc.pdl = true;
  return Launch(lc, gemm_simt_kernel<TIn, TOut>, a);
}

b200_status Validate(const b200_gemm_params* p, const b200_epilogue* epi) {
  if (p == nullptr) return Fail(B200_INVALID_ARGUMENT, "b200_gemm: null params");
  if (epi != nullptr && (epi->act < 0 || epi->act > 3))
    return Fail(B200_INVALID_ARGUMENT, "b200_gemm: unknown activation %d", epi->act);
  for (const b200_operand* x : {&p->a, &p->b, &p->c})
    if (x->dtype != B200_F32 && x->dtype != B200_F16 && x->dtype != B200_BF16)
      return Fail(B200_INVALID_ARGUMENT, "b200_gemm: unknown dtype %d", x->dtype);
  if (p->a.dtype != p->b.dtype) return Fail(B200_INVALID_ARGUMENT, "b200_gemm: A and B dtypes differ");
  if (p->c.dtype != p->a.dtype && p->c.dtype != B200_F32)
    return Fail(B200_INVALID_ARGUMENT, "b200_gemm: unsupported output dtype");
  if (p->c.transpose) return Fail(B200_INVALID_ARGUMENT, "b200_gemm: transposed C");
  if (p->m < 0 || p->n < 0 || p->k < 0 || p->batch < 0) return Fail(B200_INVALID_ARGUMENT, "b200_gemm: negative size");
  if (p->m > kMaxInt || p->n > kMaxInt || p->k > kMaxInt)
    return Fail(B200_INVALID_ARGUMENT, "b200_gemm: dimension exceeds int32");
  for (const b200_operand* x : {&p->a, &p->b, &p->c}) {
    if (x->ld < 0 || x->ld > kMaxLd) return Fail(B200_INVALID_ARGUMENT, "b200_gemm: leading dimension too large");
    if (x->batch_stride < 0) return Fail(B200_INVALID_ARGUMENT, "b200_gemm: negative batch stride");
  }
  if (p->batch > kMaxInt) return Fail(B200_INVALID_ARGUMENT, "b200_gemm: batch too large");
  if (p->batch > 65535) return Fail(B200_UNIMPLEMENTED, "b200_gemm: more than 65535 batches");
  const int64_t a_cols = p->a.transpose ? p->m : p->k;
  const int64_t b_cols = p->b.transpose ? p->k : p->n;
  if ((p->k > 0 && ((p->m > 0 && p->a.ld < a_cols) || (p->n > 0 && p->b.ld < b_cols))) ||
      (p->m > 0 && p->c.ld < p->n))
    return Fail(B200_INVALID_ARGUMENT, "b200_gemm: leading dimension smaller than row length");
  if (p->m == 0 || p->n == 0 || p->batch == 0) return B200_OK;
  if (p->c.ptr == nullptr || (p->k > 0 && (p->a.ptr == nullptr || p->b.ptr == nullptr)))
    return Fail(B200_INVALID_ARGUMENT, "b200_gemm: null buffer");
  return B200_OK;
}

bool FewRowSupports(const b200_gemm_params* p, bool* vectors_are_b) {
  // x . W^T with K contiguous on both sides (the reference's gemv layout,
  // gemv.cc:71-75), widened from 2..8 to 1..32 vectors.
  if (p->a.dtype != B200_BF16 || p->a.transpose || !p->b.transpose) return false;
  if (p->c.dtype != B200_BF16 && p->c.dtype != B200_F32) return false;
  if (p->batch != 1 || p->beta != 0.0) return false;
  const bool vb = p->n < p->m;
  const int64_t vecs = vb ? p->n : p->m;
  if (vecs < 1 || vecs > 32 || p->k < 512 || p->k % 64 != 0) return false;
  const b200_operand& mat = vb ? p->a : p->b;
  if (mat.ld != p->k || !Aligned(mat.ptr, 16)) return false;
  if (vectors_are_b) *vectors_are_b = vb;
  return true;
}

int Route(const b200_gemm_params* p, const b200_epilogue* epi, int forced) {
  if (p->m == 0 || p->n == 0 || p->batch == 0) return B200_ROUTE_NONE;
  if (forced == B200_ROUTE_SIMT) return B200_ROUTE_SIMT;
  const bool few = FewRowSupports(p, nullptr);
  const bool tc = Tcgen05Supports(p, epi);
  if (forced == B200_ROUTE_FEWROW && few) return B200_ROUTE_FEWROW;
  if (forced == B200_ROUTE_TCGEN05 && tc) return B200_ROUTE_TCGEN05;
  // measured on 4096 x 4096 weights: 9 vs 13 us at 1 row, 12 vs 14 at 8, 20 vs 13 at 16, 33 vs 16 at 32
  if (few && (std::min(p->m, p->n) <= 8 || !tc)) return B200_ROUTE_FEWROW;
  if (tc) return B200_ROUTE_TCGEN05;
  return B200_ROUTE_SIMT;
}

}  // namespace

extern "C" {

b200_status b200_gemm_validate(const b200_gemm_params* p, const b200_epilogue* epi) { return Validate(p, epi); }

int b200_gemm_route(const b200_gemm_params* p, const b200_epilogue* epi) {
  if (Validate(p, epi) != B200_OK) return -1;
  return Route(p, epi, 0);
}

uint64_t b200_gemm_work(const b200_gemm_params* p) {
  if (p == nullptr) return 0;
  const uint64_t b = static_cast<uint64_t>(p->batch > 0 ? p->batch : 0);
  const uint64_t m = p->m, n = p->n, k = p->k;
  const uint64_t flops = 2 * b * m * n * k;
  const uint64_t bytes = b * (DtypeSize(p->a.dtype) * (m * k + k * n) + DtypeSize(p->c.dtype) * m * n);
  return flops > 64 * bytes ? flops : 64 * bytes;
}

b200_status b200_gemm(b200_context* ctx, b200_stream stream, const b200_gemm_params* p, const b200_epilogue* epi) {
  b200_status s = BeginLaunch(ctx);
  if (s != B200_OK) return s;
  s = Validate(p, epi);
  if (s != B200_OK) return s;
  const b200_epilogue none = {0, nullptr, nullptr};
  if (epi == nullptr) epi = &none;
  const int route = Route(p, epi, ctx->force_route.load());
  if (route == B200_ROUTE_NONE) return B200_OK;
  if (route == B200_ROUTE_TCGEN05) return RunTcgen05(ctx, stream, p, epi);
  if (route == B200_ROUTE_FEWROW) {
    bool vb = false;
    FewRowSupports(p, &vb);
    const b200_operand& mat = vb ? p->a : p->b;
    const b200_operand& vec = vb ? p->b : p->a;
    const int64_t rows = vb ? p->m : p->n, vecs = vb ? p->n : p->m;
    // D[i, j] at i*ldc + j: the vectors index i (m small) or j (n small).
    const int64_t out_vec_stride = vb ? 1 : p->c.ld;
    const int64_t out_row_stride = vb ? p->c.ld : 1;
    return RunFewRowNT(ctx, stream, mat.ptr, vec.ptr, p->c.ptr, rows, vecs, p->k, vec.ld, out_row_stride,
                       out_vec_stride, static_cast<float>(p->alpha), epi->act, epi->bias, vb ? 1 : 0, epi->aux,
                       p->c.dtype == B200_F32);
  }
  SimtArgs a;
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
  const bool batched = p->batch > 1;
  a.sa = batched ? p->a.batch_stride : 0;
  a.sb = batched ? p->b.batch_stride : 0;
  a.sd = batched ? p->c.batch_stride : 0;
  a.ta = p->a.transpose;
  a.tb = p->b.transpose;
  a.alpha = static_cast<float>(p->alpha);
  a.beta = static_cast<float>(p->beta);
  a.act = epi->act;
  if (CeilDiv(p->m, 64) > 65535) return Fail(B200_UNIMPLEMENTED, "b200_gemm: m too large for the SIMT kernel grid");
  cudaError_t e;
  const int in = p->a.dtype, out = p->c.dtype;
  if (in == B200_F32) e = LaunchSimt<float, float>(a, p->batch, stream);
  else if (in == B200_F16 && out == B200_F16) e = LaunchSimt<__half, __half>(a, p->batch, stream);
  else if (in == B200_F16) e = LaunchSimt<__half, float>(a, p->batch, stream);
  else if (out == B200_BF16) e = LaunchSimt<__nv_bfloat16, __nv_bfloat16>(a, p->batch, stream);
  else e = LaunchSimt<__nv_bfloat16, float>(a, p->batch, stream);
  if (e != cudaSuccess) return Stick(ctx, Fail(B200_INTERNAL, "b200_gemm launch: %s", cudaGetErrorString(e)));
  return EndLaunch(ctx, "b200_gemm");
}

}  // extern "C"
