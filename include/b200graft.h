/* b200graft: the C ABI of the B200-native hot path (dense GEMM with fused
 * epilogue, weight-only int8/int4 dequant-matmul, row reductions, and the
 * Qwen3-shaped int4 decoder step built from them).
 *
 * Conventions, kept from the reference's XLA-free dispatch functions (the seam
 * its FFI handlers and BlasLt plan call into, e.g. metal_pjrt/ffi/scan.h:45-48,
 * metal_pjrt/blas/steel_gemm.h:72-78):
 *   - every buffer is a BORROWED raw device pointer; the library never owns or
 *     frees caller memory; the caller owns the stream;
 *   - every call only enqueues on `stream` and returns; no host sync, no hidden
 *     allocation on the hot path (the reference GEMM reports workspace 0,
 *     metal_pjrt/blas/metal_blas.cc:425-431);
 *   - errors are status codes with a thread-local message, never aborts
 *     (status vocabulary of metal_pjrt/runtime/metal_runtime.h:33-41);
 *     anything unsupported is refused before any launch;
 *   - zero-sized problems launch nothing and succeed (metal_blas.cc:383);
 *   - the first failure makes the context's error sticky: every later call on
 *     that context returns it (metal_pjrt/runtime/metal_runtime.h:43-53).
 * There is no CPU fallback anywhere behind this header.
 */
#ifndef B200GRAFT_H_
#define B200GRAFT_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200_ABI_VERSION 1

typedef enum {
  B200_OK = 0,
  B200_INVALID_ARGUMENT = 1,    /* caller mistake */
  B200_UNIMPLEMENTED = 2,       /* known gap, refused up front */
  B200_INTERNAL = 3,            /* CUDA API failure */
  B200_RESOURCE_EXHAUSTED = 4,
  B200_FAILED_PRECONDITION = 5,
  B200_TIMEOUT = 6              /* a bounded device-side wait ran out */
} b200_status;

typedef enum { B200_F32 = 0, B200_F16 = 1, B200_BF16 = 2 } b200_dtype;

typedef struct b200_context b200_context;
typedef struct CUstream_st* b200_stream; /* == cudaStream_t */

/* ---- context -------------------------------------------------------------
 * Replaces rt::Device (metal_pjrt/runtime/metal_runtime.h:276-450) with the
 * little a CUDA caller needs: device ordinal, attribute cache, a device status
 * word, the sticky error. */
int b200_abi_version(void); /* ≙ metal_pjrt_frontend_abi_version, metal_pjrt/pjrt/metal_pjrt_api.cc:390-392 */
b200_status b200_context_create(int device_ordinal, b200_context** out);
void b200_context_destroy(b200_context* ctx);
/* Message of the last failing call on this thread (valid until the next call). */
const char* b200_last_error(void);
/* The sticky error; also folds in the device status word (a kernel whose bounded
 * wait ran out reports B200_TIMEOUT here).  Synchronises nothing: call after
 * the stream was synchronised to see device-side reports. */
b200_status b200_context_error(b200_context* ctx);
/* Host-side fault injection (≙ METAL_PJRT_FAIL_COMMAND_BUFFER=n,
 * metal_pjrt/runtime/metal_runtime.cc:1646-1653): the n-th launch from now
 * (1 = next) is refused before it is enqueued and sets the sticky error.
 * n <= 0 disarms. */
void b200_context_fail_launch_after(b200_context* ctx, int64_t n);
/* Exercises the path every bounded device-side wait of this library takes when it runs out
 * (≙ what tests/test_gpu_errors.py:21-65 does for the reference's sticky device error, made
 * on purpose without faulting anything): enqueues a kernel that waits, for at most
 * `limit_cycles` SM cycles, on a barrier nobody arrives at, gives up, writes B200_TIMEOUT and
 * its wait id (900) to the status word and returns.  After the stream is synchronised
 * b200_context_error turns sticky B200_TIMEOUT; other contexts are unaffected. */
b200_status b200_context_wait_probe(b200_context* ctx, b200_stream stream, int64_t limit_cycles);
/* Measurement only: the cost of one tcgen05.mma.  One CTA issues `count` (<= 4096) instructions of
 * kind 0 (kind::f8f6f4, e4m3 operands) or 1 (kind::f16, bf16) with the given M (64, 128) and N, A from
 * tensor memory (1) or shared memory (0), cycling over `accumulators` (1..8) D regions, then commits
 * and waits (bounded).  cycles_device[0] = SM cycles spent issuing, [1] = until the commit arrived
 * (int64, device memory).  `opbench.py umma` prints the table. */
b200_status b200_probe_umma_rate(b200_context* ctx, b200_stream stream, int kind, int m, int n, int a_from_tmem,
                                 int accumulators, int count, int64_t* cycles_device);
/* Number of kernels this context has enqueued so far. */
int64_t b200_context_launch_count(b200_context* ctx);

/* ---- dense GEMM ------------------------------------------------------------
 * GemmParams / MpsOperand (metal_pjrt/blas/mps_gemm.h:23-53) and SteelEpilogue
 * (metal_pjrt/blas/steel_gemm.h:38-46): row-major
 *   D[b] (m x n) = act(alpha * op(A[b]) op(B[b]) + beta * D[b] + bias[col]),
 * aux = the pre-activation value; f32 accumulation, one rounding. */
typedef struct {
  void* ptr;            /* element (0,0) of batch 0 */
  int64_t ld;           /* elements between consecutive stored rows */
  int64_t batch_stride; /* elements between batches; 0 = broadcast */
  int32_t dtype;        /* b200_dtype */
  int32_t transpose;    /* operand is used as op(X) = X^T */
} b200_operand;

typedef struct {
  int64_t m, n, k, batch;
  double alpha, beta;
  b200_operand a, b, c; /* c is both the beta input and the output D */
} b200_gemm_params;

typedef struct {
  int32_t act;      /* 0 none, 1 ReLU (keeps NaN), 2 GELU-tanh, 3 SiLU */
  const void* bias; /* n elements of D's dtype, or NULL */
  void* aux;        /* D's layout and dtype, or NULL */
} b200_epilogue;

/* ≙ SteelGemmSupports + RunSteelGemm's argument checks
 * (metal_pjrt/blas/steel_gemm.cc:140-196) and the size limits of ValidateMatmul
 * (metal_pjrt/blas/blas_lt_support.cc:167-190).  Pure. */
b200_status b200_gemm_validate(const b200_gemm_params* p, const b200_epilogue* epi);
/* ≙ RunHalfGemm / RunSteelGemm / RunGemv / RunMpsGemm + epilogue
 * (metal_pjrt/blas/metal_blas.cc:91-118, steel_gemm.cc:163-255, gemv.cc:129-196). */
b200_status b200_gemm(b200_context* ctx, b200_stream stream, const b200_gemm_params* p,
                      const b200_epilogue* epi);
/* Which kernel b200_gemm would run (≙ ChooseGemv / ChooseSteelTile,
 * gemv.cc:68-108, steel_gemm.cc:115-138): 0 nothing (empty problem),
 * 1 tcgen05 tensor-core tile kernel, 2 few-row streaming kernel, 3 SIMT tile kernel. */
typedef enum { B200_ROUTE_NONE = 0, B200_ROUTE_TCGEN05 = 1, B200_ROUTE_FEWROW = 2,
               B200_ROUTE_SIMT = 3 } b200_gemm_route_t;
int b200_gemm_route(const b200_gemm_params* p, const b200_epilogue* epi);
/* ≙ GemmWork (metal_pjrt/blas/mps_gemm_objc.cc:57-67): max(2 b m n k, 64 * bytes). */
uint64_t b200_gemm_work(const b200_gemm_params* p);
/* A/B switch for benchmarks and tests (≙ RunSteelGemm's explicit tile argument,
 * steel_gemm.h:72-78): force a route (b200_gemm_route_t), 0 = automatic. */
void b200_gemm_force_route(b200_context* ctx, int route);

/* ---- the BlasLt front of the dense GEMM ---------------------------------------
 * What XLA's GEMM thunk hands a plugin, in plain C: operand layouts that may be
 * column-major, one of twelve fused epilogues, C and D as separate buffers.
 * b200_matrix_layout ≙ the fields of gpu::MatrixLayout that ValidateMatmul reads,
 * b200_matmul_config ≙ gpu::GemmConfig (metal_pjrt/blas/blas_lt_support.cc:102-201);
 * the epilogue codes follow the order of DecodeEpilogue's switch (:25-82), a binder
 * maps XLA's BlasLt::Epilogue values onto them. */
typedef enum { B200_ROW_MAJOR = 0, B200_COLUMN_MAJOR = 1 } b200_matrix_order;
typedef struct {
  int32_t dtype;               /* b200_dtype */
  int32_t order;               /* b200_matrix_order */
  int64_t num_rows, num_cols;  /* of the logical matrix */
  int64_t leading_dim_stride;  /* elements between consecutive rows (row-major) / columns (column-major) */
  int64_t batch_size, batch_stride;
  int32_t transpose;           /* must be 0 (blas_lt_support.cc:112-118) */
} b200_matrix_layout;
typedef struct {
  b200_matrix_layout lhs, rhs, c, out;
  double alpha_real, alpha_imag, beta;
} b200_matmul_config;
typedef enum { B200_EPI_DEFAULT = 0, B200_EPI_RELU, B200_EPI_BIAS, B200_EPI_BIAS_RELU, B200_EPI_GELU, B200_EPI_GELU_AUX,
               B200_EPI_BIAS_GELU, B200_EPI_BIAS_GELU_AUX, B200_EPI_SILU, B200_EPI_SILU_AUX, B200_EPI_BIAS_SILU,
               B200_EPI_BIAS_SILU_AUX } b200_blaslt_epilogue;
typedef struct { int32_t bias, act, aux; } b200_epilogue_spec;   /* ≙ EpilogueSpec, blas_lt_support.h:44-49; act as in b200_epilogue */
typedef struct {
  int32_t swap;                /* column-major output: A and B change places, every layout is seen transposed */
  b200_gemm_params params;     /* row-major normal form; pointers are filled in at execution */
  b200_epilogue_spec epi;
} b200_matmul_plan;
/* ≙ DecodeEpilogue (blas_lt_support.cc:25-82).  Pure. */
b200_status b200_decode_epilogue(int32_t epilogue, b200_epilogue_spec* out);
/* ≙ ValidateMatmul + GetMatmulPlan (blas_lt_support.cc:102-201, metal_blas.cc:245-281): the
 * acceptance rules (one operand type of f32/f16/bf16, result that type or f32; real alpha; no
 * transpose flags; batch = max of the operands', an operand without batch is broadcast;
 * beta != 0 needs C laid out exactly like D; the 16-bit index limits) and the normal form.
 * Unsupported requests fail here, never at execution with wrong values.  Pure. */
b200_status b200_matmul_plan_create(const b200_matmul_config* cfg, int32_t epilogue, b200_matmul_plan* out);
/* ≙ MatmulPlan::ExecuteOnStream + EpilogueBuffers (metal_blas.cc:296-378): operands swapped if
 * planned, D seeded with C when beta != 0 and they are distinct buffers, D / bias / aux sizes
 * checked (bias holds n elements of D's type, aux has D's extent), empty problems are no-ops. */
b200_status b200_matmul_execute(b200_context* ctx, b200_stream stream, const b200_matmul_plan* plan, const void* a,
                                const void* b, const void* c, void* d, const void* bias, void* aux, size_t d_bytes,
                                size_t bias_bytes, size_t aux_bytes);

/* ---- weight-only quantised matmul ------------------------------------------
 * out[M, N] = x[M, K] . dequant(W)[N, K]^T, W stored [N, K] with K contiguous
 * (the reference keeps [out, in], examples/llm/qwen3.py:102).  The reference has
 * no kernel for this; the math is that of _matvec_int8/_matvec_int4 and
 * dequantize (examples/llm/qwen3.py:199-267): w = q*s (+ b), all in f32, one
 * rounding to the activation dtype.
 *   bits 16: q is a bf16 [N, K] matrix, no scale (the LM head / bf16 weights).
 *   bits 8 : q int8 [N, K]; scale bf16 [N, K/group]; group == K is per-channel.
 *   bits 4 : nibble_order 0: q uint32 [N, K/8], element k=8i+j at bits 4j..4j+3;
 *            nibble_order 1: q uint8 [N, K/64, 32], low nibble = element j of the
 *            group, high nibble = element j+32 (qwen3.py:169-196);
 *            scale, bias bf16 [N, K/64].
 * M <= 32 runs the streaming kernel.  Larger M (prefill-sized batches) dequantises the
 * weights, panel by panel, into a bf16 workspace of the context that stays in L2 and runs the
 * tcgen05 GEMM on each panel (like the reference beyond ROWS_MAX: dequantize, then x @ w.T,
 * qwen3.py:199-230); there the weights are rounded to bf16 before the product, no prologue
 * is fused, the epilogue is OUT_BF16, ADD_RESIDUAL (one rounding of acc + residual) or
 * OUT_F32_RAW, and the workspace (at most 32 MB) is allocated on the first such call of a
 * context: make that call outside a stream capture. */
typedef enum { B200_QMM_OUT_BF16 = 0,      /* out bf16 [M, ldo] */
               B200_QMM_ADD_RESIDUAL = 1,  /* out = bf16(residual + bf16(y)), residual bf16 [M, ldo] */
               B200_QMM_OUT_F32 = 2,       /* out f32 [M, ldo] holding the bf16-rounded value */
               B200_QMM_OUT_F32_RAW = 3,   /* out f32 [M, ldo], unrounded (a partial sum of a K-sharded product) */
               B200_QMM_OUT_SILU_PAIR = 4  /* the weight rows come as 8 gate rows then 8 up rows per 16 (b200_interleave_gate_up):
                                              out bf16 [M, N/2] = silu(gate) * up with the reference's bf16 roundings
                                              (qwen3.py:376), formed in the tile's epilogue; up to 8 rows of x */
} b200_qmm_epilogue;

/* Input transforms fused into the staging of x (each CTA applies them to the
 * slice of x it reads, so the transformed activations are never written out):
 *   RMSNORM  x' = bf16(x * rsqrt(mean(x^2) + eps) * gain)  (rms_norm feeding a projection,
 *            examples/llm/qwen3.py:361-362,374-375); up to 8 rows;
 *   SILU_MUL x is [M, 2K] = [gate | up]; x' = silu(gate) * up with the reference's
 *            bf16 roundings (qwen3.py:376). */
typedef enum { B200_QMM_PRO_NONE = 0, B200_QMM_PRO_RMSNORM = 1, B200_QMM_PRO_SILU_MUL = 2 } b200_qmm_prologue;

typedef struct {
  int32_t bits;          /* 4, 8 or 16 */
  int32_t group;         /* 64, or K (per output channel; int8 only) */
  int32_t nibble_order;  /* bits == 4 only */
  int32_t epilogue;      /* b200_qmm_epilogue */
  const void* x;         /* bf16 [M, ldx] */
  const void* q;
  const void* scale;     /* NULL for bits 16 */
  const void* bias;      /* bits 4 only */
  const void* residual;  /* B200_QMM_ADD_RESIDUAL only; may alias out */
  void* out;
  int64_t M, N, K;
  int64_t ldx, ldo;      /* 0 = dense (K, or 2K under SILU_MUL; and N) */
  int32_t prologue;      /* b200_qmm_prologue */
  float eps;             /* RMSNORM */
  const void* prologue_gain; /* RMSNORM: bf16 [K] */
} b200_qmm_params;

/* Which kernel b200_qmm_run takes for sequential int4 in groups of 64 with up to 8 rows of x:
 * 0 the library's choice (the mma.sync streaming kernel, unless B200_QMM_TC=1 is set), 1 the
 * mma.sync kernel, 2 the tcgen05 kernel (nibbles spread to e4m3 bytes in tensor memory,
 * activations split into two e4m3 terms) wherever it applies.  For tests and measurements. */
void b200_qmm_force_route(b200_context* ctx, int route);
/* Rows of a [gate | up] projection (2 * inter rows: gate rows first, then up rows; any row size) rearranged so that
 * every 16 consecutive rows hold 8 gate rows followed by the 8 up rows of the same outputs: what
 * B200_QMM_OUT_SILU_PAIR consumes.  Applies to the packed weights and, with their row size, to the scale and offset
 * rows.  inter a multiple of 8, row_bytes a multiple of 4; src and dst distinct. */
b200_status b200_interleave_gate_up(b200_context* ctx, b200_stream stream, const void* src, void* dst, int64_t inter,
                                    int64_t row_bytes);
b200_status b200_qmm_validate(const b200_qmm_params* p);
b200_status b200_qmm_run(b200_context* ctx, b200_stream stream, const b200_qmm_params* p);
/* The short form: dense rows, bf16 in and out. */
b200_status b200_qmm(b200_context* ctx, b200_stream stream, int bits, int group, int nibble_order,
                     const void* x, const void* q, const void* scale, const void* bias_or_null,
                     void* out, int64_t M, int64_t N, int64_t K, int act_dtype);
/* How b200_qmm_run would tile this problem: rows per CTA, CTAs along K (cluster
 * size), batch blocks of 8.  Pure; for tests and benchmarks. */
b200_status b200_qmm_plan(const b200_qmm_params* p, int* rows_per_cta, int* split_k, int* batch_blocks);
/* Dequantised weights written out, w[N, K] = q*s (+ b) in f32 with one rounding
 * per operation, then stored as f32 (out_dtype B200_F32) or rounded once more to
 * bf16 (≙ dequantize, qwen3.py:199-207).  The bit-exactness check reads this. */
b200_status b200_dequantize(b200_context* ctx, b200_stream stream, int bits, int group, int nibble_order,
                            const void* q, const void* scale, const void* bias_or_null, void* w_out,
                            int64_t N, int64_t K, int out_dtype);
/* Load-time quantisers on the device (≙ quantize_int8/quantize_int4,
 * qwen3.py:154-196, in the benchmark's variants): w f32 or bf16 [N, K] ->
 * int8 per-group symmetric (group == K: per channel), or int4 min/max affine
 * with sequential uint32 nibbles.  scale/bias are written as bf16. */
b200_status b200_quantize(b200_context* ctx, b200_stream stream, int bits, int group, const void* w,
                          int w_dtype, void* q_out, void* scale_out, void* bias_out, int64_t N, int64_t K);

/* The reference's own load-time 4-bit quantiser on the device (≙ quantize_int4,
 * qwen3.py:169-196: the grid anchored at the group's largest-magnitude edge, stretched so
 * that zero falls on it, step possibly negative), bit for bit, in the reference's layout:
 * q uint8 [N, K/64, 32] (low nibble = element j, high nibble = element j + 32), scale and
 * bias bf16 [N, K/64].  (Its int8 quantiser, qwen3.py:154-166, is b200_quantize with bits 8
 * and group 64.)  w f32 or bf16 [N, K]. */
b200_status b200_quantize_int4_ref(b200_context* ctx, b200_stream stream, const void* w, int w_dtype, void* q_out,
                                   void* scale_out, void* bias_out, int64_t N, int64_t K);
/* Split-half bytes (nibble_order 1) -> sequential uint32 words (nibble_order 0), the layout
 * b200_decoder_create takes.  Scale and bias are shared by both layouts. */
b200_status b200_repack_int4(b200_context* ctx, b200_stream stream, const void* q_split_half, void* q_sequential,
                             int64_t N, int64_t K);

/* ---- row reductions over the minor dimension --------------------------------
 * kind 0 RMSNorm  y = x * rsqrt(mean(x^2) + eps) * gain   (examples/llm/qwen3.py:294-297)
 *      1 softmax, 2 log_softmax (max-subtract form; call sites qwen3.py:325, tests/test_scan.py:35-48)
 *      3 LayerNorm y = (x - mean) / sqrt(var + eps) [* gain + beta] (bench/jax_bench.py:44-46)
 * Statistics in f32, one rounding to the input dtype.  x, y [rows, n] dense;
 * y may alias x.  gain/beta have x's dtype. */
b200_status b200_rownorm(b200_context* ctx, b200_stream stream, int kind, const void* x,
                         const void* gain_or_null, const void* beta_or_null, void* y, int64_t rows,
                         int64_t n, int dtype, double eps);

/* ---- decoder step -------------------------------------------------------------
 * One decode step (one new token per sequence) of the Qwen3-shaped decoder of
 * examples/llm/qwen3.py:334-390, with int4-g64 projections (sequential uint32
 * nibbles), bf16 activations, a bf16 KV cache laid out as the reference's
 * (K [B, KV, S, D], V [B, KV, D, S], qwen3.py:279-291) and an untied bf16 LM
 * head.  With tp_world > 1 each rank holds its shard (see b200_tp_*). */
typedef struct {
  int32_t layers, hidden, heads, kv_heads, head_dim, inter, vocab, max_len;
  float rope_theta, rms_eps;
  int32_t max_batch;
} b200_decoder_config;

typedef struct {             /* one projection, int4-g64 sequential layout */
  const void* q;             /* uint32 [N, K/8] */
  const void* scale;         /* bf16 [N, K/64] */
  const void* bias;          /* bf16 [N, K/64] */
} b200_qweight;

typedef struct {
  const void* attn_norm;     /* bf16 [hidden] */
  b200_qweight qkv;          /* N = (heads + 2 kv_heads) * head_dim (this rank's heads) */
  const void* q_norm;        /* bf16 [head_dim] */
  const void* k_norm;
  b200_qweight o;            /* N = hidden, K = heads * head_dim (this rank's heads) */
  const void* mlp_norm;
  b200_qweight gate_up;      /* N = 2 * inter (this rank's share: gate rows then up rows) */
  b200_qweight down;         /* N = hidden, K = inter (this rank's share) */
  void* k_cache;             /* bf16 [B, kv_heads, max_len, head_dim] */
  void* v_cache;             /* bf16 [B, kv_heads, head_dim, max_len] */
} b200_decoder_layer;

typedef struct b200_decoder b200_decoder;
typedef struct b200_tp b200_tp;

/* cfg holds this rank's LOCAL head counts / inter / vocab share; `tp` may be NULL
 * (one GPU).  The layer structs are copied; the buffers they point to are borrowed.
 * The decoder owns its activation buffers and, for steps of up to 8 rows, one
 * row-interleaved copy of every gate_up matrix (b200_interleave_gate_up; the size of the
 * original), with which that projection forms silu(gate) * up in its epilogue;
 * B200_DECODER_NO_SILU_PAIR=1 leaves the copies out. */
b200_status b200_decoder_create(b200_context* ctx, const b200_decoder_config* cfg,
                                const b200_decoder_layer* layers, const void* embed /* bf16 [vocab_full, hidden] */,
                                const void* final_norm, const void* lm_head /* bf16 [vocab, hidden] */,
                                b200_tp* tp, b200_decoder** out);
void b200_decoder_destroy(b200_decoder* dec);
/* tokens: device int32 [batch]; pos: device int32 [1] (position of the new token,
 * every sequence the same, qwen3.py:356); logits: device f32 [batch, vocab_total]
 * (with tp: the all-gathered logits, rank-major).  Enqueues on `stream`.
 * The step is a sequence of kernels captured into a CUDA graph: tokens and pos are copied
 * into decoder-owned buffers first, a graph is kept per (batch, logits pointer) - pass the
 * same logits buffer every step to replay one graph - and at most 8 graphs are kept (least
 * recently used out).  Calls on one decoder are serialised by a mutex; use one decoder per
 * host thread to overlap.
 * With B200_DECODER_STREAM=1 in the environment at b200_decoder_create, one GPU and up to a
 * few rows, the whole step is instead ONE persistent kernel that reads the tokens / pos /
 * logits pointers afresh at every call.  It copies the int4 projections once, at creation,
 * into its own streaming layout (a second copy of those weights in device memory; when
 * that allocation fails the decoder keeps the graph).  It is slower than the graph today
 * (2.5 against 2.2 ms per step on the Qwen3-8B shape at batch 1) and is kept as an option. */
b200_status b200_decoder_step(b200_decoder* dec, b200_stream stream, const int32_t* tokens,
                              const int32_t* pos, float* logits, int batch);
/* Kernels enqueued by one step at this batch size (1, or the graph's node count). */
int64_t b200_decoder_launches_per_step(b200_decoder* dec, int batch);
/* CUDA graphs this decoder has captured so far (0 while every step took the single kernel). */
int64_t b200_decoder_graphs_built(b200_decoder* dec);
/* Per-stage tracing of the single-kernel step (≙ METAL_PJRT_TRACE's per-command timing,
 * metal_pjrt/runtime/metal_runtime.cc:56-59,1671, moved inside the kernel because there is
 * only one launch to time).  While enabled, thread 0 of every CTA stamps the device's
 * nanosecond timer four times per stage: 0 the stage may start (grid barrier passed),
 * 1 its inputs are staged in shared memory, 2 its share of the weight records is consumed,
 * 3 its outputs are written.  b200_decoder_trace_read copies the stamps of the last step
 * (uint64 [ctas, stages, 4]; call with out == NULL to learn the sizes) after the caller has
 * synchronised the stream, and the stage kinds (0 qkv, 1 attention, 2 o, 3 gate_up, 4 down,
 * 5 LM head; int32 [stages]).  FAILED_PRECONDITION on a decoder without the single kernel. */
b200_status b200_decoder_trace(b200_decoder* dec, int enable);
b200_status b200_decoder_trace_read(b200_decoder* dec, uint64_t* out, int64_t capacity, int32_t* ctas,
                                    int32_t* stages, int32_t* stage_types);

/* Pieces of the step, exported for parity tests (bf16 throughout). */
/* table bf16 [vocab, hidden].  A token id outside [0, vocab) reads row 0 and reports
 * B200_INVALID_ARGUMENT through the context's device status word. */
b200_status b200_embed(b200_context* ctx, b200_stream stream, const void* table, const int32_t* tokens,
                       void* out, int64_t batch, int64_t hidden, int64_t vocab);
/* Per-head RMSNorm + rotate-half RoPE of q and k, and the KV-cache write at *pos
 * (qwen3.py:366-369).  qkv bf16 [B, (H + 2 KV) * D]; q_out bf16 [B, H, D].  A *pos outside
 * [0, max_len) writes nothing and reports B200_INVALID_ARGUMENT through the status word. */
b200_status b200_qk_norm_rope_cache(b200_context* ctx, b200_stream stream, const void* qkv,
                                    const void* q_norm, const void* k_norm, void* q_out, void* k_cache,
                                    void* v_cache, const int32_t* pos, int64_t batch, int heads,
                                    int kv_heads, int head_dim, int64_t max_len, float theta, float eps);
/* Grouped-query decode attention over slots [0, *pos] (qwen3.py:322-327).
 * scratch: f32, b200_attention_scratch_bytes(...) bytes. */
size_t b200_attention_scratch_bytes(int64_t batch, int heads, int head_dim, int64_t max_len);
b200_status b200_attention_decode(b200_context* ctx, b200_stream stream, const void* q, const void* k_cache,
                                  const void* v_cache, void* out, const int32_t* pos, void* scratch,
                                  int64_t batch, int heads, int kv_heads, int head_dim, int64_t max_len);
/* The same attention for callers that cannot allocate device memory (no counterpart in
 * the reference).  Who that is: a caller in the middle of a stream capture, where
 * cudaMalloc is not allowed, or a plugin host whose own allocator has claimed the whole
 * device and gives plugins no way to ask for more.  The partials go into an 8 MiB array
 * that is part of the library image on every GPU that loads it, so there is no scratch
 * argument and the call allocates nothing; a problem whose partials
 * (b200_attention_scratch_bytes) exceed 8 MiB is refused with B200_RESOURCE_EXHAUSTED.
 * The first call on a device looks up the array's device address (once per device);
 * make that first call outside any stream capture.  All calls share the one array: it
 * keeps whatever the last call left (nothing in it needs clearing, every value read is
 * written first within the call), and two calls that overlap on the GPU - different
 * streams, or different contexts on one device - race on it. */
b200_status b200_attention_decode_static(b200_context* ctx, b200_stream stream, const void* q, const void* k_cache,
                                         const void* v_cache, void* out, const int32_t* pos, int64_t batch,
                                         int heads, int kv_heads, int head_dim, int64_t max_len);
/* The fused form the decoder uses: per-head RMSNorm + RoPE of q and of the new k,
 * the cache writes of k and v at *pos, and attention over slots [0, *pos], all
 * from the fused projection row qkv bf16 [B, (H + 2 KV) * D] (qwen3.py:363-372).
 * inv_freq: f32 [D/2] = theta^(-2i/D), or NULL to compute it in the kernel.
 * A *pos outside [0, max_len) writes nothing and reports B200_INVALID_ARGUMENT
 * through the context's device status word. */
b200_status b200_attention_step(b200_context* ctx, b200_stream stream, const void* qkv, const void* q_norm,
                                const void* k_norm, const float* inv_freq_or_null, void* k_cache, void* v_cache,
                                void* out, const int32_t* pos, void* scratch, int64_t batch, int heads,
                                int kv_heads, int head_dim, int64_t max_len, float theta, float eps);
/* silu(gate) * up with the reference's bf16 roundings (qwen3.py:376). gate_up bf16 [B, 2*inter]. */
b200_status b200_silu_mul(b200_context* ctx, b200_stream stream, const void* gate_up, void* out,
                          int64_t batch, int64_t inter);

/* ---- sampling ------------------------------------------------------------------
 * ≙ sample (examples/llm/qwen3.py:395-418): next token [batch] from f32 logits [batch, vocab].
 * temperature 0 is greedy (argmax, ties to the lowest index; `uniform` may be NULL).
 * Otherwise logits / temperature, then: neither top_k nor top_p set - a categorical draw
 * over the row; else the top_k values in descending order (ties: lower index first), of
 * which top_p < 1 keeps the smallest prefix whose probability reaches top_p (always at
 * least the most likely token), and a categorical draw over those.  The draw is the
 * inverse CDF at uniform[row] in [0, 1) (the reference draws with jax.random.categorical,
 * whose bit stream only JAX has): the first candidate, in the order above, whose cumulative
 * probability exceeds uniform[row] x the kept total.
 * Refused: temperature < 0, top_k outside [0, vocab] (INVALID_ARGUMENT, as the reference
 * raises); top_k > 1024, and top_p < 1 with top_k == 0 (UNIMPLEMENTED: that sorts the whole
 * vocabulary). */
b200_status b200_sample(b200_context* ctx, b200_stream stream, const float* logits, int64_t batch, int64_t vocab,
                        float temperature, int32_t top_k, float top_p, const float* uniform, int32_t* out);

/* ---- tensor parallel group (NEW: the reference is single-device,
 * metal_pjrt/compiler/metal_collectives_registration.cc:10-17) ------------------
 * One process per GPU.  Rank 0 makes an id, the caller distributes its bytes
 * (any transport), every rank calls b200_tp_create. */
#define B200_TP_ID_BYTES 128
b200_status b200_tp_make_id(void* id_bytes /* B200_TP_ID_BYTES */);
b200_status b200_tp_create(b200_context* ctx, const void* id_bytes, int rank, int world, b200_tp** out);
void b200_tp_destroy(b200_tp* tp);
/* In-place sum over ranks of a bf16 [count] buffer; all-gather of `count` f32 per rank. */
b200_status b200_tp_all_reduce_bf16(b200_tp* tp, b200_stream stream, void* buf, int64_t count);
b200_status b200_tp_all_gather_f32(b200_tp* tp, b200_stream stream, const void* send, void* recv,
                                   int64_t count_per_rank);
/* Peer exchange (optional; ranks are processes on GPUs of one NVLink domain, at most 8).
 * The sum over ranks that follows a K-sharded projection is a few KB, so it is done by one
 * kernel per rank over peer memory instead of a collective call: every rank allocates an
 * exchange block (two slots of max_floats f32 + flags) and gets its CUDA IPC handle; the
 * caller gathers the handles of all ranks (rank order, B200_TP_PEER_HANDLE_BYTES each) by
 * any transport and connects, then synchronises the ranks on the host before first use
 * and before b200_tp_destroy.  b200_tp_peer_partial(slot) is where the projection writes
 * its f32 partial sums; consecutive exchanges must alternate slots 0, 1, 0, ...
 * b200_tp_sum_residual_norm: x[batch, hidden] (bf16) += bf16(sum over ranks of the slot),
 * h = rms_norm(x) * gain; peers are awaited with a bounded spin (B200_TIMEOUT through the
 * context's status word; after a wait that ran out no peer memory is read).
 * A decoder created with a connected group goes one step further for up to 4 rows per step
 * (B200_TP_PUSH_ROWS, at most 8; B200_TP_PULL=1 switches it off): its o / down projections
 * store each f32 partial sum together with the exchange number as one 8-byte line into
 * every rank's block (max_floats a multiple of 8); at their end the CTAs of the same kernel
 * form the sum over ranks once, from this rank's own memory, and publish the new residual
 * rows there for the projection that follows (no exchange kernel, no flags or fences;
 * bounded waits, ids 400 + rank and 450).  No TMA, multicast or multimem
 * touches peer memory anywhere in this library: plain loads and stores only. */
#define B200_TP_PEER_HANDLE_BYTES 64
b200_status b200_tp_peer_alloc(b200_tp* tp, int64_t max_floats, void* handle_out /* B200_TP_PEER_HANDLE_BYTES */);
b200_status b200_tp_peer_connect(b200_tp* tp, const void* handles /* world x B200_TP_PEER_HANDLE_BYTES */);
void* b200_tp_peer_partial(b200_tp* tp, int slot);
b200_status b200_tp_sum_residual_norm(b200_tp* tp, b200_stream stream, int slot, void* x, const void* gain, void* h,
                                      int64_t batch, int64_t hidden, double eps);

#ifdef __cplusplus
}
#endif
#endif /* B200GRAFT_H_ */
