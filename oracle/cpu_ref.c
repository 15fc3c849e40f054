/* CPU restatement in C of the decode path: TEST / BENCHMARK INFRASTRUCTURE.
 *
 * It exists so the CPU baseline can be timed with all host threads (OpenMP)
 * and so the NumPy oracle has an independent cross-check.  It follows the
 * reference's Python, function by function:
 *   oracle_qmv_int4   <- _matvec_int4   (examples/llm/qwen3.py:243-267): per group
 *                        s*(sum x q) + b*(sum x), all f32, summed over groups
 *   oracle_qmv_int8   <- _matvec_int8   (qwen3.py:233-240)
 *   oracle_mv_bf16    <- linear / einsum for an unquantised [out, in] matrix (qwen3.py:230)
 *   oracle_rms_norm   <- rms_norm       (qwen3.py:294-297)
 *   oracle_softmax_f32, oracle_layer_norm_f32 <- jax.nn.softmax (qwen3.py:325), bench/jax_bench.py:44-46
 *   oracle_decode_step<- forward, T = 1 (qwen3.py:334-390) with rope (:300-310) and the
 *                        decode branch of attention (:322-327)
 * int4 weights use the sequential layout (eight consecutive-k nibbles per
 * uint32).  bf16 is a uint16_t holding the upper half of an f32, rounded to
 * nearest even as metal_pjrt/blas/steel_gemm_test.cc:30-35 does.
 * The library never links or calls this file.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

static inline float bf2f(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
static inline uint16_t f2bf(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40); /* NaN stays NaN */
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}
static inline float rbf(float f) { return bf2f(f2bf(f)); }

int oracle_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* Threads for the parallel loops from now on (a launcher may have exported
 * OMP_NUM_THREADS=1; the benchmark's CPU arm asks for every core instead). */
void oracle_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

/* out[m*N + n] (f32, unrounded) = sum_k x[m,k] * (q*s + b)[n,k];  M <= 32 */
void oracle_qmv_int4(const uint16_t* x, const uint32_t* q, const uint16_t* s, const uint16_t* b, float* out,
                     int M, int N, int K) {
  const int G = K / 64;
  float* xf = (float*)malloc((size_t)M * K * sizeof(float));
  float* xs = (float*)malloc((size_t)M * G * sizeof(float)); /* per-group sums of x */
  for (int m = 0; m < M; ++m)
    for (int g = 0; g < G; ++g) {
      float t = 0.0f;
      for (int j = 0; j < 64; ++j) {
        const float v = bf2f(x[(size_t)m * K + g * 64 + j]);
        xf[(size_t)m * K + g * 64 + j] = v;
        t += v;
      }
      xs[m * G + g] = t;
    }
#pragma omp parallel for schedule(static)
  for (int n = 0; n < N; ++n) {
    float acc[32];
    for (int m = 0; m < M; ++m) acc[m] = 0.0f;
    const uint32_t* qr = q + (size_t)n * (K / 8);
    for (int g = 0; g < G; ++g) {
      const float sc = bf2f(s[(size_t)n * G + g]), bi = bf2f(b[(size_t)n * G + g]);
      float qf[64];
      for (int w = 0; w < 8; ++w) {
        const uint32_t word = qr[g * 8 + w];
        for (int j = 0; j < 8; ++j) qf[w * 8 + j] = (float)((word >> (4 * j)) & 0xF);
      }
      for (int m = 0; m < M; ++m) {
        const float* xr = xf + (size_t)m * K + g * 64;
        float t = 0.0f;
#pragma omp simd reduction(+ : t)
        for (int j = 0; j < 64; ++j) t += xr[j] * qf[j];
        acc[m] += t * sc + xs[m * G + g] * bi;
      }
    }
    for (int m = 0; m < M; ++m) out[(size_t)m * N + n] = acc[m];
  }
  free(xf);
  free(xs);
}

/* int8, scale per `group` inputs (group == K: per output channel) */
void oracle_qmv_int8(const uint16_t* x, const int8_t* q, const uint16_t* s, float* out, int M, int N, int K,
                     int group) {
  const int G = K / group;
  float* xf = (float*)malloc((size_t)M * K * sizeof(float));
  for (size_t i = 0; i < (size_t)M * K; ++i) xf[i] = bf2f(x[i]);
#pragma omp parallel for schedule(static)
  for (int n = 0; n < N; ++n) {
    for (int m = 0; m < M; ++m) {
      float acc = 0.0f;
      for (int g = 0; g < G; ++g) {
        const int8_t* qr = q + (size_t)n * K + (size_t)g * group;
        const float* xr = xf + (size_t)m * K + (size_t)g * group;
        float t = 0.0f;
#pragma omp simd reduction(+ : t)
        for (int j = 0; j < group; ++j) t += xr[j] * (float)qr[j];
        acc += t * bf2f(s[(size_t)n * G + g]);
      }
      out[(size_t)m * N + n] = acc;
    }
  }
  free(xf);
}

void oracle_mv_bf16(const uint16_t* x, const uint16_t* w, float* out, int M, int N, int K) {
  float* xf = (float*)malloc((size_t)M * K * sizeof(float));
  for (size_t i = 0; i < (size_t)M * K; ++i) xf[i] = bf2f(x[i]);
#pragma omp parallel for schedule(static)
  for (int n = 0; n < N; ++n) {
    const uint16_t* wr = w + (size_t)n * K;
    for (int m = 0; m < M; ++m) {
      const float* xr = xf + (size_t)m * K;
      float t = 0.0f;
#pragma omp simd reduction(+ : t)
      for (int k = 0; k < K; ++k) t += xr[k] * bf2f(wr[k]);
      out[(size_t)m * N + n] = t;
    }
  }
  free(xf);
}

/* D = act(A[M,K] @ B[K,N] + bias), f32 (config 1) */
void oracle_gemm_f32(const float* a, const float* b, const float* bias, float* d, int M, int N, int K) {
#pragma omp parallel for schedule(static)
  for (int i = 0; i < M; ++i) {
    float* dr = d + (size_t)i * N;
    for (int j = 0; j < N; ++j) dr[j] = bias ? bias[j] : 0.0f;
    for (int k = 0; k < K; ++k) {
      const float av = a[(size_t)i * K + k];
      const float* br = b + (size_t)k * N;
      for (int j = 0; j < N; ++j) dr[j] += av * br[j];
    }
  }
}

void oracle_rms_norm_bf16(const uint16_t* x, const uint16_t* w, uint16_t* y, int rows, int n, float eps) {
#pragma omp parallel for schedule(static) if (rows > 8)
  for (int r = 0; r < rows; ++r) {
    const uint16_t* xr = x + (size_t)r * n;
    float ss = 0.0f;
    for (int i = 0; i < n; ++i) { const float v = bf2f(xr[i]); ss += v * v; }
    const float sc = 1.0f / sqrtf(ss / (float)n + eps);
    for (int i = 0; i < n; ++i) y[(size_t)r * n + i] = f2bf((bf2f(xr[i]) * sc) * bf2f(w[i]));
  }
}

void oracle_rms_norm_f32(const float* x, const float* w, float* y, int rows, int n, float eps) {
#pragma omp parallel for schedule(static) if (rows > 8)
  for (int r = 0; r < rows; ++r) {
    const float* xr = x + (size_t)r * n;
    float ss = 0.0f;
    for (int i = 0; i < n; ++i) ss += xr[i] * xr[i];
    const float sc = 1.0f / sqrtf(ss / (float)n + eps);
    for (int i = 0; i < n; ++i) y[(size_t)r * n + i] = (xr[i] * sc) * w[i];
  }
}

void oracle_softmax_f32(const float* x, float* y, int rows, int n) {
#pragma omp parallel for schedule(static) if (rows > 8)
  for (int r = 0; r < rows; ++r) {
    const float* xr = x + (size_t)r * n;
    float m = -INFINITY;
    for (int i = 0; i < n; ++i) m = xr[i] > m ? xr[i] : m;
    float sum = 0.0f;
    for (int i = 0; i < n; ++i) { const float e = expf(xr[i] - m); y[(size_t)r * n + i] = e; sum += e; }
    for (int i = 0; i < n; ++i) y[(size_t)r * n + i] /= sum;
  }
}

void oracle_layer_norm_f32(const float* x, float* y, int rows, int n, float eps) {
#pragma omp parallel for schedule(static) if (rows > 8)
  for (int r = 0; r < rows; ++r) {
    const float* xr = x + (size_t)r * n;
    float mean = 0.0f;
    for (int i = 0; i < n; ++i) mean += xr[i];
    mean /= (float)n;
    float var = 0.0f;
    for (int i = 0; i < n; ++i) var += (xr[i] - mean) * (xr[i] - mean);
    var /= (float)n;
    const float sc = 1.0f / sqrtf(var + eps);
    for (int i = 0; i < n; ++i) y[(size_t)r * n + i] = (xr[i] - mean) * sc;
  }
}

typedef struct {
  int32_t layers, hidden, heads, kv_heads, head_dim, inter, vocab, max_len;
  float theta, eps;
} oracle_cfg;

typedef struct {
  const uint16_t* attn_norm;
  const uint32_t* qkv_q; const uint16_t* qkv_s; const uint16_t* qkv_b;
  const uint16_t* q_norm; const uint16_t* k_norm;
  const uint32_t* o_q; const uint16_t* o_s; const uint16_t* o_b;
  const uint16_t* mlp_norm;
  const uint32_t* gu_q; const uint16_t* gu_s; const uint16_t* gu_b;
  const uint32_t* down_q; const uint16_t* down_s; const uint16_t* down_b;
  uint16_t* k_cache; /* [B, KV, S, D] */
  uint16_t* v_cache; /* [B, KV, D, S] */
} oracle_layer;

static void norm_rope_head(const uint16_t* src, const uint16_t* w, uint16_t* dst, int D, int pos, float theta,
                           float eps) {
  float ss = 0.0f;
  for (int i = 0; i < D; ++i) { const float v = bf2f(src[i]); ss += v * v; }
  const float r = 1.0f / sqrtf(ss / (float)D + eps);
  for (int i = 0; i < D / 2; ++i) {
    const float n1 = rbf((bf2f(src[i]) * r) * bf2f(w[i]));
    const float n2 = rbf((bf2f(src[i + D / 2]) * r) * bf2f(w[i + D / 2]));
    const float inv_freq = (float)(1.0 / pow((double)theta, (double)(2 * i) / D));
    const float ang = (float)pos * inv_freq;
    const float cs = cosf(ang), sn = sinf(ang);
    dst[i] = f2bf(n1 * cs - n2 * sn);
    dst[i + D / 2] = f2bf(n2 * cs + n1 * sn);
  }
}

/* One decode step.  Runs the first `run_layers` layers and `run_vocab` rows of
 * the LM head (the benchmark times a bounded sample and scales; parity tests
 * pass the full counts).  logits f32 [B, run_vocab]. */
void oracle_decode_step(const oracle_cfg* c, const oracle_layer* layers, const uint16_t* embed,
                        const uint16_t* final_norm, const uint16_t* lm_head, const int32_t* tokens, int pos,
                        int B, float* logits, int run_layers, int run_vocab) {
  const int E = c->hidden, H = c->heads, KV = c->kv_heads, D = c->head_dim, I = c->inter, S = c->max_len;
  const int G = H / KV, QKV = (H + 2 * KV) * D;
  uint16_t* x = (uint16_t*)malloc((size_t)B * E * 2);
  uint16_t* h = (uint16_t*)malloc((size_t)B * E * 2);
  uint16_t* qkv = (uint16_t*)malloc((size_t)B * QKV * 2);
  uint16_t* qr = (uint16_t*)malloc((size_t)B * H * D * 2);
  uint16_t* att = (uint16_t*)malloc((size_t)B * H * D * 2);
  uint16_t* act = (uint16_t*)malloc((size_t)B * I * 2);
  const size_t wide = (size_t)(2 * I > QKV ? 2 * I : QKV);
  float* y = (float*)malloc((size_t)B * (wide > (size_t)run_vocab ? wide : (size_t)run_vocab) * sizeof(float));
  const float scale = 1.0f / sqrtf((float)D);
  for (int b = 0; b < B; ++b) memcpy(x + (size_t)b * E, embed + (size_t)tokens[b] * E, (size_t)E * 2);
  for (int li = 0; li < run_layers; ++li) {
    const oracle_layer* L = &layers[li];
    oracle_rms_norm_bf16(x, L->attn_norm, h, B, E, c->eps);
    oracle_qmv_int4(h, L->qkv_q, L->qkv_s, L->qkv_b, y, B, QKV, E);
    for (size_t i = 0; i < (size_t)B * QKV; ++i) qkv[i] = f2bf(y[i]);
    for (int b = 0; b < B; ++b) {
      for (int hh = 0; hh < H; ++hh)
        norm_rope_head(qkv + (size_t)b * QKV + hh * D, L->q_norm, qr + ((size_t)b * H + hh) * D, D, pos, c->theta, c->eps);
      for (int kv = 0; kv < KV; ++kv) {
        norm_rope_head(qkv + (size_t)b * QKV + (H + kv) * D, L->k_norm,
                       L->k_cache + (((size_t)b * KV + kv) * S + pos) * D, D, pos, c->theta, c->eps);
        const uint16_t* vs = qkv + (size_t)b * QKV + (H + KV + kv) * D;
        for (int d = 0; d < D; ++d) L->v_cache[(((size_t)b * KV + kv) * D + d) * S + pos] = vs[d];
      }
    }
    const int nv = pos + 1;
#pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < B; ++b)
      for (int hh = 0; hh < H; ++hh) {
        const int kv = hh / G;
        const uint16_t* qh = qr + ((size_t)b * H + hh) * D;
        const uint16_t* kc = L->k_cache + ((size_t)b * KV + kv) * S * D;
        const uint16_t* vc = L->v_cache + ((size_t)b * KV + kv) * D * S;
        float* p = (float*)malloc((size_t)nv * sizeof(float));
        float m = -INFINITY;
        for (int s = 0; s < nv; ++s) {
          float t = 0.0f;
#pragma omp simd reduction(+ : t)
          for (int d = 0; d < D; ++d) t += bf2f(qh[d]) * bf2f(kc[(size_t)s * D + d]);
          p[s] = t * scale;
          m = p[s] > m ? p[s] : m;
        }
        float sum = 0.0f;
        for (int s = 0; s < nv; ++s) { p[s] = expf(p[s] - m); sum += p[s]; }
        for (int s = 0; s < nv; ++s) p[s] /= sum;
        for (int d = 0; d < D; ++d) {
          float t = 0.0f;
#pragma omp simd reduction(+ : t)
          for (int s = 0; s < nv; ++s) t += p[s] * bf2f(vc[(size_t)d * S + s]);
          att[((size_t)b * H + hh) * D + d] = f2bf(t);
        }
        free(p);
      }
    oracle_qmv_int4(att, L->o_q, L->o_s, L->o_b, y, B, E, H * D);
    for (size_t i = 0; i < (size_t)B * E; ++i) x[i] = f2bf(bf2f(x[i]) + rbf(y[i]));
    oracle_rms_norm_bf16(x, L->mlp_norm, h, B, E, c->eps);
    oracle_qmv_int4(h, L->gu_q, L->gu_s, L->gu_b, y, B, 2 * I, E);
    for (int b = 0; b < B; ++b)
      for (int i = 0; i < I; ++i) {
        const float g = rbf(y[(size_t)b * 2 * I + i]), u = rbf(y[(size_t)b * 2 * I + I + i]);
        const float sig = rbf(1.0f / (1.0f + expf(-g)));
        act[(size_t)b * I + i] = f2bf(rbf(g * sig) * u);
      }
    oracle_qmv_int4(act, L->down_q, L->down_s, L->down_b, y, B, E, I);
    for (size_t i = 0; i < (size_t)B * E; ++i) x[i] = f2bf(bf2f(x[i]) + rbf(y[i]));
  }
  oracle_rms_norm_bf16(x, final_norm, h, B, E, c->eps);
  oracle_mv_bf16(h, lm_head, y, B, run_vocab, E);
  for (size_t i = 0; i < (size_t)B * run_vocab; ++i) logits[i] = rbf(y[i]);
  free(x); free(h); free(qkv); free(qr); free(att); free(act); free(y);
}
