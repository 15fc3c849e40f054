// The BlasLt-shaped front of the dense GEMM: what XLA hands a plugin (operand layouts that
// may be column-major, one of twelve fused epilogues, separate C and D buffers) turned into
// the row-major b200_gemm_params / b200_epilogue that the kernels take.  Host code only.
//
// ≙ DecodeEpilogue + ValidateMatmul (metal_pjrt/blas/blas_lt_support.cc:25-201) and
// MetalBlasLt::GetMatmulPlan / MatmulPlan::ExecuteOnStream / EpilogueBuffers
// (metal_pjrt/blas/metal_blas.cc:245-378).
#include <algorithm>

#include "common.cuh"

using namespace b200;

namespace {

void Transpose(b200_matrix_layout* l) {   // the same storage seen as the transposed matrix
  std::swap(l->num_rows, l->num_cols);
  l->order = l->order == B200_ROW_MAJOR ? B200_COLUMN_MAJOR : B200_ROW_MAJOR;
}

bool DtypeOk(int32_t t) { return t == B200_F32 || t == B200_F16 || t == B200_BF16; }

const char* DtypeName(int32_t t) { return t == B200_F32 ? "f32" : (t == B200_F16 ? "f16" : (t == B200_BF16 ? "bf16" : "?")); }

}  // namespace

extern "C" {

b200_status b200_decode_epilogue(int32_t epilogue, b200_epilogue_spec* out) {
  if (out == nullptr) return Fail(B200_INVALID_ARGUMENT, "b200_decode_epilogue: null out");
  b200_epilogue_spec s = {0, 0, 0};
  switch (epilogue) {
    case B200_EPI_DEFAULT: break;
    case B200_EPI_RELU: s.act = 1; break;
    case B200_EPI_BIAS: s.bias = 1; break;
    case B200_EPI_BIAS_RELU: s.bias = 1; s.act = 1; break;
    case B200_EPI_GELU: s.act = 2; break;
    case B200_EPI_GELU_AUX: s.act = 2; s.aux = 1; break;
    case B200_EPI_BIAS_GELU: s.bias = 1; s.act = 2; break;
    case B200_EPI_BIAS_GELU_AUX: s.bias = 1; s.act = 2; s.aux = 1; break;
    case B200_EPI_SILU: s.act = 3; break;
    case B200_EPI_SILU_AUX: s.act = 3; s.aux = 1; break;
    case B200_EPI_BIAS_SILU: s.bias = 1; s.act = 3; break;
    case B200_EPI_BIAS_SILU_AUX: s.bias = 1; s.act = 3; s.aux = 1; break;
    default: return Fail(B200_UNIMPLEMENTED, "matmul with fused epilogue %d is not supported", epilogue);
  }
  *out = s;
  return B200_OK;
}

b200_status b200_matmul_plan_create(const b200_matmul_config* cfg, int32_t epilogue, b200_matmul_plan* out) {
  if (cfg == nullptr || out == nullptr) return Fail(B200_INVALID_ARGUMENT, "b200_matmul_plan_create: null argument");
  b200_matmul_plan plan = {};
  b200_status st = b200_decode_epilogue(epilogue, &plan.epi);
  if (st != B200_OK) return st;
  if (cfg->alpha_imag != 0.0) return Fail(B200_UNIMPLEMENTED, "matmul with a complex scale factor is not supported");
  b200_matrix_layout lhs = cfg->lhs, rhs = cfg->rhs, c = cfg->c, o = cfg->out;
  for (const b200_matrix_layout* l : {&lhs, &rhs, &c, &o})
    if (l->transpose != 0) return Fail(B200_UNIMPLEMENTED, "matmul: layouts must not carry a transpose flag");
  // an operand without a batch dimension is broadcast (its batch stride counts as 0)
  const int64_t batch = std::max(lhs.batch_size, rhs.batch_size);
  if (o.batch_size != batch) return Fail(B200_INVALID_ARGUMENT, "matmul: batch mismatch (operands %lld, output %lld)",
                                         static_cast<long long>(batch), static_cast<long long>(o.batch_size));
  const bool lhs_bcast = lhs.batch_size <= 1, rhs_bcast = rhs.batch_size <= 1;
  // The kernels write a row-major result.  For a column-major output compute
  //   D^T = (A B)^T = B^T A^T:
  // swap the operands and view every layout transposed.
  plan.swap = o.order == B200_COLUMN_MAJOR;
  bool a_bcast = lhs_bcast, b_bcast = rhs_bcast;
  if (plan.swap) {
    std::swap(lhs, rhs);
    std::swap(a_bcast, b_bcast);
    Transpose(&lhs);
    Transpose(&rhs);
    Transpose(&c);
    Transpose(&o);
  }
  const int64_t m = o.num_rows, n = o.num_cols, k = lhs.num_cols;
  if (lhs.num_rows != m || rhs.num_rows != k || rhs.num_cols != n)
    return Fail(B200_INVALID_ARGUMENT, "matmul: inconsistent shapes lhs %lldx%lld rhs %lldx%lld out %lldx%lld",
                static_cast<long long>(lhs.num_rows), static_cast<long long>(lhs.num_cols), static_cast<long long>(rhs.num_rows),
                static_cast<long long>(rhs.num_cols), static_cast<long long>(m), static_cast<long long>(n));
  if (!(DtypeOk(lhs.dtype) && lhs.dtype == rhs.dtype && DtypeOk(o.dtype) && (o.dtype == lhs.dtype || o.dtype == B200_F32)))
    return Fail(B200_UNIMPLEMENTED,
                "matmul %s x %s -> %s is not supported: both operands must be f32, f16 or bf16 of one type, the result "
                "that type or f32. Cast the operands", DtypeName(lhs.dtype), DtypeName(rhs.dtype), DtypeName(o.dtype));
  if (cfg->beta != 0.0 && (c.dtype != o.dtype || c.order != o.order || c.leading_dim_stride != o.leading_dim_stride ||
                           c.batch_stride != o.batch_stride || c.num_rows != o.num_rows || c.num_cols != o.num_cols))
    return Fail(B200_UNIMPLEMENTED, "matmul adding an operand laid out unlike the result is not supported");
  if (lhs.dtype != B200_F32) {
    // the 16-bit kernels index in 32 bits: every dimension and the batch count within int32, every
    // leading dimension within INT32_MAX / 256
    constexpr int64_t kMaxInt = 2147483647, kMaxLd = kMaxInt / 256;
    if (batch > kMaxInt) return Fail(B200_UNIMPLEMENTED, "%s matmul too large: batch count %lld exceeds %lld", DtypeName(lhs.dtype),
                                     static_cast<long long>(batch), static_cast<long long>(kMaxInt));
    for (int64_t d : {m, n, k})
      if (d > kMaxInt) return Fail(B200_UNIMPLEMENTED, "%s matmul too large: dimension %lld exceeds %lld. Split the matmul or use float32",
                                   DtypeName(lhs.dtype), static_cast<long long>(d), static_cast<long long>(kMaxInt));
    for (const b200_matrix_layout* l : {&lhs, &rhs, &o})
      if (l->leading_dim_stride > kMaxLd)
        return Fail(B200_UNIMPLEMENTED, "%s matmul too large: leading dimension %lld exceeds %lld. Split the matmul or use float32",
                    DtypeName(lhs.dtype), static_cast<long long>(l->leading_dim_stride), static_cast<long long>(kMaxLd));
  }
  // A row-major logical matrix is its stored matrix; a column-major one is the transpose of the
  // row-major view of its storage.
  auto operand = [](const b200_matrix_layout& l, bool bcast) {
    b200_operand x = {};
    x.ld = l.leading_dim_stride;
    x.batch_stride = bcast ? 0 : l.batch_stride;
    x.dtype = l.dtype;
    x.transpose = l.order == B200_COLUMN_MAJOR;
    return x;
  };
  plan.params.m = m;
  plan.params.n = n;
  plan.params.k = k;
  plan.params.batch = batch;
  plan.params.alpha = cfg->alpha_real;
  plan.params.beta = cfg->beta;
  plan.params.a = operand(lhs, a_bcast);
  plan.params.b = operand(rhs, b_bcast);
  plan.params.c = operand(o, batch <= 1);   // row-major after the swap
  plan.params.c.transpose = 0;
  *out = plan;
  return B200_OK;
}

b200_status b200_matmul_execute(b200_context* ctx, b200_stream stream, const b200_matmul_plan* plan, const void* a, const void* b,
                                const void* c, void* d, const void* bias, void* aux, size_t d_bytes, size_t bias_bytes,
                                size_t aux_bytes) {
  if (plan == nullptr) return Fail(B200_INVALID_ARGUMENT, "b200_matmul_execute: null plan");
  b200_status s = BeginLaunch(ctx);
  if (s != B200_OK) return s;
  b200_gemm_params p = plan->params;
  if (p.m == 0 || p.n == 0 || p.batch == 0) return B200_OK;
  const uint64_t elem = static_cast<uint64_t>(DtypeSize(p.c.dtype));
  const uint64_t batch_stride = p.batch > 1 ? static_cast<uint64_t>(p.c.batch_stride) : 0;
  const uint64_t extent = static_cast<uint64_t>(p.batch - 1) * batch_stride + static_cast<uint64_t>(p.m - 1) * p.c.ld + p.n;
  if (d == nullptr || d_bytes < extent * elem)
    return Fail(B200_INVALID_ARGUMENT, "matmul: D has %zu bytes, need %llu", d_bytes, static_cast<unsigned long long>(extent * elem));
  b200_epilogue e = {plan->epi.act, nullptr, nullptr};
  if (plan->epi.bias) {
    if (bias == nullptr || bias_bytes < static_cast<uint64_t>(p.n) * elem)
      return Fail(B200_INVALID_ARGUMENT, "matmul epilogue: bias buffer (%zu bytes) must hold %lld elements of %s", bias_bytes,
                  static_cast<long long>(p.n), DtypeName(p.c.dtype));
    e.bias = bias;
  }
  if (plan->epi.aux) {
    if (aux == nullptr || aux_bytes < extent * elem)
      return Fail(B200_INVALID_ARGUMENT, "matmul epilogue: aux buffer (%zu bytes) smaller than the output (%llu bytes)", aux_bytes,
                  static_cast<unsigned long long>(extent * elem));
    e.aux = aux;
  }
  p.a.ptr = const_cast<void*>(plan->swap ? b : a);
  p.b.ptr = const_cast<void*>(plan->swap ? a : b);
  p.c.ptr = d;
  // D = alpha A B + beta C accumulates in place: seed D with C when they are distinct buffers
  // (their layouts were checked equal at plan creation)
  if (p.beta != 0.0 && c != nullptr && c != d) {
    cudaError_t err = cudaMemcpyAsync(d, c, extent * elem, cudaMemcpyDeviceToDevice, stream);
    if (err != cudaSuccess) return Stick(ctx, Fail(B200_INTERNAL, "matmul: copying C into D: %s", cudaGetErrorString(err)));
  }
  return b200_gemm(ctx, stream, &p, &e);
}

}  // extern "C"
