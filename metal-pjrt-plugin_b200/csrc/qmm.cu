// Weight-only quantised matmul for few rows (M <= 32), the decode path:
//   out[M, N] = x[M, K] . dequant(W)[N, K]^T
// The reference has no kernel for this; XLA turns its _matvec_int4/_matvec_int8
// (examples/llm/qwen3.py:233-267) into generic row reductions.  The math kept
// from there: w = q*s (+ b) per group of 64 inputs, all in f32, the offset term
// folded into the same reduction as  sum_g s_g (sum_j x q) + b_g (sum_j x),
// one rounding to the activation dtype.
//
// Design (HBM-bound; the weights are read exactly once):
//   * a CTA owns 16*RT weight rows and a K slice; a producer warp streams the
//     packed rows into a shared-memory ring with 1-D bulk async copies
//     (cp.async.bulk + mbarrier), so tens of KB per SM are in flight without
//     costing registers;
//   * the weight copies do not depend on the previous kernel, so they are
//     issued BEFORE griddepcontrol.wait: under programmatic dependent launch
//     the next product's weights stream while the previous kernel drains;
//   * eight consumer warps take one 64-input group each per 512-input chunk:
//     nibbles / bytes are widened to bf16 in registers (one lop3 per two
//     nibbles, 128 + q with the 128 folded into the offset term) and fed to
//     mma.sync m16n8k16 with the batch as the 8-wide operand; the inputs of x
//     are pre-permuted in shared memory to match the register order, so no
//     shuffles are needed; per-group scale/offset are applied in f32;
//   * split-K inside a CTA is reduced through shared-memory atomics, split-K
//     across CTAs through a thread-block cluster's distributed shared memory.
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;
using namespace b200;

namespace {

constexpr int kConsumerWarps = 8;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kThreads = kConsumerThreads + 32;  // + one producer warp
constexpr int kChunkK = 512;                     // inputs per pipeline stage: 8 groups
constexpr int kGroupK = 64;

enum Format { kInt4Seq = 0, kInt4Half = 1, kInt8 = 2, kBf16 = 3 };

template <int FMT>
struct Fmt {
  static constexpr int kBits = FMT == kInt8 ? 8 : (FMT == kBf16 ? 16 : 4);
  static constexpr int kChunkRowBytes = kChunkK * kBits / 8;  // 256 / 512 / 1024
  static constexpr int kPad = kBits == 4 ? 32 : 64;           // keeps the quad reads conflict-free
  static constexpr int kRowStride = kChunkRowBytes + kPad;
  static constexpr int kGroupBytes = kGroupK * kBits / 8;     // 32 / 64 / 128
};

// Which input (0..63) of a group sits in half `h` of A register `r` (0..7) of
// quad thread `t`.  x is staged in shared memory in exactly this order.
template <int FMT>
__device__ __forceinline__ int kmap(int t, int r, int h) {
  if (FMT == kInt4Seq) return 16 * t + 8 * (r >> 2) + (r & 3) + 4 * h;
  if (FMT == kInt4Half) {
    const int rr = r & 3;
    return 8 * t + 4 * (r >> 2) + (rr >> 1) + 2 * h + 32 * (rr & 1);
  }
  if (FMT == kInt8) return 16 * t + 2 * r + h;
  return 32 * (r >> 2) + 8 * t + 2 * (r & 3) + h;  // bf16: two 16-byte pieces per thread
}

struct QmmArgs {
  const uint8_t* q;
  const __nv_bfloat16* scale;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* x;
  const __nv_bfloat16* residual;
  void* out;
  int M, N, K;
  int ldx, ldo;
  int scale_ld;    // scales per row
  int k_per_cta;   // K / gridDim.y, a multiple of 64
  int epilogue;
  int stages;
  int* status;
  // dense-GEMM use (epilogue == kEpilogueGemm): D = act(alpha * acc + bias), aux = pre-activation
  int64_t out_row_stride;  // between weight rows (n)
  int64_t out_vec_stride;  // between batch vectors (m)
  float alpha;
  int act;
  int bias_by_vec;         // bias follows the batch vector, not the weight row
  int out_f32;
  const void* gemm_bias;
  void* aux;
  // fused input transforms (b200_qmm_prologue)
  int prologue;
  int x_vec;                   // x rows allow 16-byte loads
  float eps;
  const __nv_bfloat16* gain;   // RMSNorm gain [K]
};

constexpr int kEpilogueGemm = 100;

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

// Widens one thread's share of a group (for one weight row) into 8 bf16x2 registers.
template <int FMT>
__device__ __forceinline__ void load_a(const uint8_t* row_group_ptr, int t, uint32_t (&a)[8]) {
  if (FMT == kInt4Seq || FMT == kInt4Half) {
    const uint2 w = *reinterpret_cast<const uint2*>(row_group_ptr + 8 * t);
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      a[r] = lop3_and_or(w.x >> (4 * r), 0x000f000fu, 0x43004300u);      // bf16 (128 + q)
      a[4 + r] = lop3_and_or(w.y >> (4 * r), 0x000f000fu, 0x43004300u);
    }
  } else if (FMT == kInt8) {
    const uint4 w = *reinterpret_cast<const uint4*>(row_group_ptr + 16 * t);
    const uint32_t words[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t u = words[j] ^ 0x80808080u;  // q + 128 in every byte
      // 2^23 + (q + 128) as f32, minus (2^23 + 128): q exactly, no int->float unit
      const float f0 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7650)) - 8388736.0f;
      const float f1 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7651)) - 8388736.0f;
      const float f2 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7652)) - 8388736.0f;
      const float f3 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7653)) - 8388736.0f;
      a[2 * j] = pack_bf16(f0, f1);
      a[2 * j + 1] = pack_bf16(f2, f3);
    }
  } else {
    const uint4 w0 = *reinterpret_cast<const uint4*>(row_group_ptr + 16 * t);
    const uint4 w1 = *reinterpret_cast<const uint4*>(row_group_ptr + 64 + 16 * t);
    a[0] = w0.x; a[1] = w0.y; a[2] = w0.z; a[3] = w0.w;
    a[4] = w1.x; a[5] = w1.y; a[6] = w1.z; a[7] = w1.w;
  }
}

__device__ __forceinline__ void consumer_barrier() {
  asm volatile("bar.sync 1, %0;" ::"n"(kConsumerThreads) : "memory");
}

// FMT: storage format; MB: batch blocks of 8; RT: 16-row tiles per CTA;
// GROUPED: a scale (and offset) per 64 inputs, else one scale per row applied at the end.
template <int FMT, int MB, int RT, bool GROUPED>
__global__ void __launch_bounds__(kThreads) qgemv_kernel(const QmmArgs a) {
  using F = Fmt<FMT>;
  constexpr int R = 16 * RT;
  constexpr int MP = 8 * MB;
  extern __shared__ __align__(128) uint8_t smem[];

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int n0 = blockIdx.x * R;
  const int rows_valid = min(R, a.N - n0);
  const int split = gridDim.y;
  const int k_begin = blockIdx.y * a.k_per_cta;
  const int groups_cta = a.k_per_cta / kGroupK;
  const int n_chunks = (a.k_per_cta + kChunkK - 1) / kChunkK;
  const int NS = a.stages;
  const size_t row_bytes_total = static_cast<size_t>(a.K) * F::kBits / 8;

  // ---- shared memory carve-up -------------------------------------------------
  uint64_t* full = reinterpret_cast<uint64_t*>(smem);
  uint64_t* empty = full + NS;
  size_t off = (static_cast<size_t>(2 * NS) * 8 + 127) & ~static_cast<size_t>(127);
  float* red = reinterpret_cast<float*>(smem + off);                 // [R][MP]
  off += static_cast<size_t>(R) * MP * 4;
  float* xsum = reinterpret_cast<float*>(smem + off);                // [groups_cta][MP]
  off += (static_cast<size_t>(groups_cta) * MP * 4 + 127) & ~static_cast<size_t>(127);
  uint4* xs = reinterpret_cast<uint4*>(smem + off);                  // [groups_cta][2][M][4] x 16 B
  off += (static_cast<size_t>(groups_cta) * a.M * 128 + 127) & ~static_cast<size_t>(127);
  float2* so = reinterpret_cast<float2*>(smem + off);                // [groups_cta][R] (scale, offset)
  if (GROUPED) off += (static_cast<size_t>(groups_cta) * R * 8 + 127) & ~static_cast<size_t>(127);
  uint8_t* stage_base = smem + off;
  __shared__ float ss_part[kConsumerWarps][8];
  __shared__ float rinv[8];
  constexpr int kStageBytes = R * F::kRowStride;

  if (tid == 0) {
    for (int s = 0; s < NS; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], kConsumerWarps);
    }
    mbar_fence_init();
  }
  for (int i = tid; i < R * MP; i += kThreads) red[i] = 0.0f;
  for (int i = tid; i < groups_cta * MP; i += kThreads) xsum[i] = 0.0f;
  __syncthreads();

  bool dead = false;  // a bounded wait gave up: leave the pipeline, keep the barriers below

  if (warp == kConsumerWarps) {
    // ---------------- producer warp: weights only, independent of earlier kernels
    const uint8_t* src0 = a.q + static_cast<size_t>(n0) * row_bytes_total +
                          static_cast<size_t>(k_begin) * F::kBits / 8;
    for (int c = 0; c < n_chunks && !dead; ++c) {
      const int s = c % NS, use = c / NS;
      if (use > 0 && !mbar_wait_bounded(&empty[s], (use - 1) & 1)) {
        report_timeout(a.status, 100 + s);
        dead = true;
        break;
      }
      const int chunk_k = min(kChunkK, a.k_per_cta - c * kChunkK);
      const uint32_t bytes_row = static_cast<uint32_t>(chunk_k * F::kBits / 8);
      if (lane == 0) mbar_expect_tx(&full[s], bytes_row * rows_valid);
      __syncwarp();
      uint8_t* dst = stage_base + static_cast<size_t>(s) * kStageBytes;
      const uint8_t* src = src0 + static_cast<size_t>(c) * F::kChunkRowBytes;
      for (int r = lane; r < rows_valid; r += 32)
        bulk_g2s(dst + r * F::kRowStride, src + static_cast<size_t>(r) * row_bytes_total, bytes_row, &full[s]);
    }
    if (lane == 0) pdl_launch_dependents();
  } else {
    // ---------------- consumer warps
    // Scales and offsets belong to the weights: fetch them before waiting on the
    // previous kernel, as (s, b - 128 s) pairs laid out [group][row].
    if (GROUPED) {
      const int g0 = k_begin / kGroupK;
      for (int i = tid; i < R * groups_cta; i += kConsumerThreads) {
        const int r = i / groups_cta, gi = i - r * groups_cta;
        // rows past N are clamped for the load; their results are never stored
        const size_t idx = static_cast<size_t>(min(n0 + r, a.N - 1)) * a.scale_ld + g0 + gi;
        const float sc = ldg_bf16(a.scale + idx);
        // int4 registers hold 128 + q: fold the 128 into the offset
        const float of = F::kBits == 4 ? fmaf(-128.0f, sc, ldg_bf16(a.bias + idx)) : 0.0f;
        so[gi * R + r] = make_float2(sc, of);
      }
    }
    pdl_wait();  // x (and the residual) come from the previous kernel
    if (a.prologue == B200_QMM_PRO_RMSNORM) {
      // 1 / rms of every full row of x (M <= 8), recomputed by each CTA
      float ss[8];
#pragma unroll
      for (int m = 0; m < 8; ++m) {
        ss[m] = 0.0f;
        if (m < a.M) {
          const __nv_bfloat16* xr = a.x + static_cast<size_t>(m) * a.ldx;
          if (a.x_vec) {
            for (int i = tid * 8; i < a.K; i += kConsumerThreads * 8) {
              const uint4 raw = __ldg(reinterpret_cast<const uint4*>(xr + i));
              const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                ss[m] = fmaf(bf16_lo(w[j]), bf16_lo(w[j]), ss[m]);
                ss[m] = fmaf(bf16_hi(w[j]), bf16_hi(w[j]), ss[m]);
              }
            }
          } else {
            for (int i = tid; i < a.K; i += kConsumerThreads) {
              const float v = __bfloat162float(xr[i]);
              ss[m] = fmaf(v, v, ss[m]);
            }
          }
        }
        ss[m] = warp_sum(ss[m]);
        if (lane == 0) ss_part[warp][m] = ss[m];
      }
      consumer_barrier();
      if (tid < 8) {
        float tsum = 0.0f;
#pragma unroll
        for (int w = 0; w < kConsumerWarps; ++w) tsum += ss_part[w][tid];
        rinv[tid] = 1.0f / sqrtf(tsum / static_cast<float>(a.K) + a.eps);
      }
      consumer_barrier();
    }
    // Stage x in register order: unit (m, group, t) = 16 inputs = two runs of 8 (or one of 16).
    {
      const int units = a.M * groups_cta * 4;
      const int units_pad = (units + 31) & ~31;
      constexpr bool kOneRun = FMT == kInt4Seq || FMT == kInt8;
      for (int u = tid; u < units_pad; u += kConsumerThreads) {
        const bool valid = u < units;
        const int ut = u & 3;
        const int ug = (u >> 2) % groups_cta;
        const int um = (u >> 2) / groups_cta;
        float sum = 0.0f;
        if (valid) {
          const int kbase = k_begin + ug * kGroupK;
          const int run0 = kOneRun ? 16 * ut : 8 * ut;
          const int run1 = kOneRun ? 16 * ut + 8 : 32 + 8 * ut;
          float e[16];
          auto load_run = [&](const __nv_bfloat16* base, int k, float* dst) {
            if (a.x_vec) {
              const uint4 raw = __ldg(reinterpret_cast<const uint4*>(base + k));
              const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                dst[2 * j] = bf16_lo(w[j]);
                dst[2 * j + 1] = bf16_hi(w[j]);
              }
            } else {
#pragma unroll
              for (int j = 0; j < 8; ++j) dst[j] = ldg_bf16(base + k + j);
            }
          };
          const __nv_bfloat16* xr = a.x + static_cast<size_t>(um) * a.ldx;
          load_run(xr, kbase + run0, e);
          load_run(xr, kbase + run1, e + 8);
          if (a.prologue == B200_QMM_PRO_RMSNORM) {
            float gn[16];
            load_run(a.gain, kbase + run0, gn);
            load_run(a.gain, kbase + run1, gn + 8);
            const float rr = rinv[um];
#pragma unroll
            for (int j = 0; j < 16; ++j) e[j] = bf16_round((e[j] * rr) * gn[j]);
          } else if (a.prologue == B200_QMM_PRO_SILU_MUL) {
            // x is [M, 2K]: gate in the first K columns, up in the last K
            float up[16];
            load_run(xr + a.K, kbase + run0, up);
            load_run(xr + a.K, kbase + run1, up + 8);
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const float sig = bf16_round(1.0f / (1.0f + expf(-e[j])));
              e[j] = bf16_round(bf16_round(e[j] * sig) * up[j]);
            }
          }
          uint32_t regs[8];
#pragma unroll
          for (int r = 0; r < 8; ++r) {
            const int k0 = kmap<FMT>(0, r, 0), k1 = kmap<FMT>(0, r, 1);
            const int l0 = kOneRun ? k0 : (k0 & 7) + 8 * (k0 >> 5);
            const int l1 = kOneRun ? k1 : (k1 & 7) + 8 * (k1 >> 5);
            regs[r] = pack_bf16(e[l0], e[l1]);
            sum += e[l0] + e[l1];
          }
          xs[((ug * 2 + 0) * a.M + um) * 4 + ut] = make_uint4(regs[0], regs[1], regs[2], regs[3]);
          xs[((ug * 2 + 1) * a.M + um) * 4 + ut] = make_uint4(regs[4], regs[5], regs[6], regs[7]);
        }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        if (valid && ut == 0) xsum[ug * MP + um] = sum;
      }
    }
    consumer_barrier();

    float acc[RT][MB][4];
#pragma unroll
    for (int rt = 0; rt < RT; ++rt)
#pragma unroll
      for (int mb = 0; mb < MB; ++mb)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[rt][mb][i] = 0.0f;

    for (int c = 0; c < n_chunks; ++c) {
      const int s = c % NS;
      if (!mbar_wait_bounded(&full[s], (c / NS) & 1)) {
        report_timeout(a.status, 200 + s);
        dead = true;
        break;
      }
      const int chunk_groups = min(kChunkK, a.k_per_cta - c * kChunkK) / kGroupK;
      if (warp < chunk_groups) {
        const int gl = c * (kChunkK / kGroupK) + warp;   // group within this CTA's slice
        uint32_t xf[MB][8];
        float xs2[MB][2];
#pragma unroll
        for (int mb = 0; mb < MB; ++mb) {
          const int m = mb * 8 + g;
          if (m < a.M) {
            const uint4 v0 = xs[((gl * 2 + 0) * a.M + m) * 4 + t];
            const uint4 v1 = xs[((gl * 2 + 1) * a.M + m) * 4 + t];
            xf[mb][0] = v0.x; xf[mb][1] = v0.y; xf[mb][2] = v0.z; xf[mb][3] = v0.w;
            xf[mb][4] = v1.x; xf[mb][5] = v1.y; xf[mb][6] = v1.z; xf[mb][7] = v1.w;
          } else {
#pragma unroll
            for (int r = 0; r < 8; ++r) xf[mb][r] = 0u;
          }
          if (F::kBits == 4) {
            const float2 v = *reinterpret_cast<const float2*>(&xsum[gl * MP + mb * 8 + 2 * t]);
            xs2[mb][0] = v.x;
            xs2[mb][1] = v.y;
          }
        }
        const uint8_t* stage = stage_base + static_cast<size_t>(s) * kStageBytes + warp * F::kGroupBytes;
#pragma unroll
        for (int rt = 0; rt < RT; ++rt) {
          const int r0 = rt * 16 + g, r1 = r0 + 8;
          float s0 = 1.0f, s1 = 1.0f, o0 = 0.0f, o1 = 0.0f;
          if (GROUPED) {
            const float2 p0 = so[gl * R + r0], p1 = so[gl * R + r1];
            s0 = p0.x; o0 = p0.y;
            s1 = p1.x; o1 = p1.y;
          }
          uint32_t a0[8], a1[8];
          load_a<FMT>(stage + r0 * F::kRowStride, t, a0);
          load_a<FMT>(stage + r1 * F::kRowStride, t, a1);
          if (GROUPED) {
            float tmp[MB][4];
#pragma unroll
            for (int mb = 0; mb < MB; ++mb) {
              tmp[mb][0] = tmp[mb][1] = tmp[mb][2] = tmp[mb][3] = 0.0f;
#pragma unroll
              for (int i = 0; i < 4; ++i)
                mma_bf16_16816(tmp[mb], a0[2 * i], a1[2 * i], a0[2 * i + 1], a1[2 * i + 1], xf[mb][2 * i],
                               xf[mb][2 * i + 1]);
              if (F::kBits == 4) {
                acc[rt][mb][0] += fmaf(s0, tmp[mb][0], o0 * xs2[mb][0]);
                acc[rt][mb][1] += fmaf(s0, tmp[mb][1], o0 * xs2[mb][1]);
                acc[rt][mb][2] += fmaf(s1, tmp[mb][2], o1 * xs2[mb][0]);
                acc[rt][mb][3] += fmaf(s1, tmp[mb][3], o1 * xs2[mb][1]);
              } else {
                acc[rt][mb][0] = fmaf(s0, tmp[mb][0], acc[rt][mb][0]);
                acc[rt][mb][1] = fmaf(s0, tmp[mb][1], acc[rt][mb][1]);
                acc[rt][mb][2] = fmaf(s1, tmp[mb][2], acc[rt][mb][2]);
                acc[rt][mb][3] = fmaf(s1, tmp[mb][3], acc[rt][mb][3]);
              }
            }
          } else {
#pragma unroll
            for (int mb = 0; mb < MB; ++mb)
#pragma unroll
              for (int i = 0; i < 4; ++i)
                mma_bf16_16816(acc[rt][mb], a0[2 * i], a1[2 * i], a0[2 * i + 1], a1[2 * i + 1], xf[mb][2 * i],
                               xf[mb][2 * i + 1]);
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[s]);
    }
    // split-K inside the CTA: eight warps add into one [R][MP] tile
#pragma unroll
    for (int rt = 0; rt < RT; ++rt)
#pragma unroll
      for (int mb = 0; mb < MB; ++mb)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int row = rt * 16 + g + ((i & 2) ? 8 : 0);
          const int col = mb * 8 + 2 * t + (i & 1);
          atomicAdd(&red[row * MP + col], acc[rt][mb][i]);
        }
  }
  __syncthreads();

  // ---- split-K across the cluster, then the epilogue -----------------------------
  cg::cluster_group cluster = cg::this_cluster();
  if (split > 1) cluster.sync();
  const int rows_per_rank = (R + split - 1) / split;
  const int r_begin = blockIdx.y * rows_per_rank;
  const int r_end = min(min(r_begin + rows_per_rank, R), rows_valid);
  const int r_count = r_end - r_begin;
  if (r_count > 0) {
    for (int idx = tid; idx < r_count * a.M; idx += kThreads) {
      const int r = r_begin + idx % r_count;
      const int m = idx / r_count;
      float v;
      if (split > 1) {
        v = 0.0f;
        for (int c = 0; c < split; ++c) v += cluster.map_shared_rank(red, c)[r * MP + m];
      } else {
        v = red[r * MP + m];
      }
      const int n = n0 + r;
      if (!GROUPED && F::kBits != 16) v *= ldg_bf16(a.scale + n);
      if (a.epilogue == kEpilogueGemm) {
        const size_t o = static_cast<size_t>(m) * a.out_vec_stride + static_cast<size_t>(n) * a.out_row_stride;
        v *= a.alpha;
        const int bi = a.bias_by_vec ? m : n;
        if (a.out_f32) {
          if (a.gemm_bias != nullptr) v += static_cast<const float*>(a.gemm_bias)[bi];
          if (a.aux != nullptr) static_cast<float*>(a.aux)[o] = v;
          static_cast<float*>(a.out)[o] = apply_act(a.act, v);
        } else {
          if (a.gemm_bias != nullptr) v += __bfloat162float(static_cast<const __nv_bfloat16*>(a.gemm_bias)[bi]);
          if (a.aux != nullptr) static_cast<__nv_bfloat16*>(a.aux)[o] = __float2bfloat16_rn(v);
          static_cast<__nv_bfloat16*>(a.out)[o] = __float2bfloat16_rn(apply_act(a.act, v));
        }
        continue;
      }
      const float y = bf16_round(v);
      const size_t o = static_cast<size_t>(m) * a.ldo + n;
      if (a.epilogue == B200_QMM_OUT_F32_RAW) {
        reinterpret_cast<float*>(a.out)[o] = v;
      } else if (a.epilogue == B200_QMM_OUT_F32) {
        reinterpret_cast<float*>(a.out)[o] = y;
      } else if (a.epilogue == B200_QMM_ADD_RESIDUAL) {
        reinterpret_cast<__nv_bfloat16*>(a.out)[o] =
            __float2bfloat16_rn(__bfloat162float(a.residual[o]) + y);
      } else {
        reinterpret_cast<__nv_bfloat16*>(a.out)[o] = __float2bfloat16_rn(v);
      }
    }
  }
  if (split > 1) cluster.sync();  // peers may still be reading this CTA's tile
}

// ---------------------------------------------------------------------------
// Host side: plan, validation, dispatch
// ---------------------------------------------------------------------------

struct Plan {
  int fmt = 0, mb = 1, rt = 1, split = 1, stages = 2;
  bool grouped = true;
  size_t smem = 0;
};

int ChunkRowStride(int fmt) {
  switch (fmt) {
    case kInt8: return Fmt<kInt8>::kRowStride;
    case kBf16: return Fmt<kBf16>::kRowStride;
    default: return Fmt<kInt4Seq>::kRowStride;
  }
}

size_t SmemFor(const Plan& pl, int M, int k_per_cta) {
  const int R = 16 * pl.rt, MP = 8 * pl.mb, groups = k_per_cta / kGroupK;
  size_t off = (static_cast<size_t>(2 * pl.stages) * 8 + 127) & ~static_cast<size_t>(127);
  off += static_cast<size_t>(R) * MP * 4;
  off += (static_cast<size_t>(groups) * MP * 4 + 127) & ~static_cast<size_t>(127);
  off += (static_cast<size_t>(groups) * M * 128 + 127) & ~static_cast<size_t>(127);
  if (pl.grouped) off += (static_cast<size_t>(groups) * R * 8 + 127) & ~static_cast<size_t>(127);
  off += static_cast<size_t>(pl.stages) * R * ChunkRowStride(pl.fmt);
  return off;
}

b200_status Validate(const b200_qmm_params* p) {
  if (p == nullptr) return Fail(B200_INVALID_ARGUMENT, "b200_qmm: null params");
  if (p->bits != 4 && p->bits != 8 && p->bits != 16)
    return Fail(B200_INVALID_ARGUMENT, "b200_qmm: bits must be 4, 8 or 16, got %d", p->bits);
  if (p->M < 0 || p->N < 0 || p->K < 0) return Fail(B200_INVALID_ARGUMENT, "b200_qmm: negative size");
  if (p->M > 32)
    return Fail(B200_UNIMPLEMENTED,
                "b200_qmm: M = %lld rows; the streaming kernel takes up to 32 (dequantise, then b200_gemm)",
                static_cast<long long>(p->M));
  if (p->N > INT32_MAX / 2 || p->K > INT32_MAX / 2) return Fail(B200_UNIMPLEMENTED, "b200_qmm: size exceeds int32");
  if (p->K % kGroupK != 0)
    return Fail(B200_UNIMPLEMENTED, "b200_qmm: K = %lld is not a multiple of 64", static_cast<long long>(p->K));
  if (p->bits == 4 && p->group != 64) return Fail(B200_UNIMPLEMENTED, "b200_qmm: int4 group must be 64, got %d", p->group);
  if (p->bits == 8 && p->group != 64 && p->group != p->K)
    return Fail(B200_UNIMPLEMENTED, "b200_qmm: int8 group must be 64 or K, got %d", p->group);
  if (p->bits == 4 && p->nibble_order != 0 && p->nibble_order != 1)
    return Fail(B200_INVALID_ARGUMENT, "b200_qmm: nibble_order must be 0 or 1");
  if (p->epilogue < 0 || p->epilogue > 3) return Fail(B200_INVALID_ARGUMENT, "b200_qmm: unknown epilogue %d", p->epilogue);
  if (p->prologue < 0 || p->prologue > 2) return Fail(B200_INVALID_ARGUMENT, "b200_qmm: unknown prologue %d", p->prologue);
  if (p->prologue == B200_QMM_PRO_RMSNORM && p->M > 8)
    return Fail(B200_UNIMPLEMENTED, "b200_qmm: the fused RMSNorm takes up to 8 rows (run b200_rownorm first)");
  if (p->M == 0 || p->N == 0) return B200_OK;
  if (p->prologue == B200_QMM_PRO_RMSNORM && p->prologue_gain == nullptr)
    return Fail(B200_INVALID_ARGUMENT, "b200_qmm: fused RMSNorm without a gain");
  if (p->x == nullptr || p->q == nullptr || p->out == nullptr) return Fail(B200_INVALID_ARGUMENT, "b200_qmm: null buffer");
  if (p->bits != 16 && p->scale == nullptr) return Fail(B200_INVALID_ARGUMENT, "b200_qmm: null scale");
  if (p->bits == 4 && p->bias == nullptr) return Fail(B200_INVALID_ARGUMENT, "b200_qmm: int4 needs a bias (offset) buffer");
  if (p->epilogue == B200_QMM_ADD_RESIDUAL && p->residual == nullptr)
    return Fail(B200_INVALID_ARGUMENT, "b200_qmm: residual epilogue without a residual buffer");
  if (!Aligned(p->q, 16)) return Fail(B200_INVALID_ARGUMENT, "b200_qmm: q must be 16-byte aligned (bulk copies)");
  const int64_t xcols = p->prologue == B200_QMM_PRO_SILU_MUL ? 2 * p->K : p->K;
  const int64_t ldx = p->ldx ? p->ldx : xcols, ldo = p->ldo ? p->ldo : p->N;
  if (ldx < xcols || ldo < p->N) return Fail(B200_INVALID_ARGUMENT, "b200_qmm: leading dimension smaller than row length");
  if (p->K == 0) return Fail(B200_UNIMPLEMENTED, "b200_qmm: K = 0");
  return B200_OK;
}

b200_status MakePlan(const b200_qmm_params* p, int sm_count, int max_smem, Plan* out) {
  Plan pl;
  pl.fmt = p->bits == 16 ? kBf16 : (p->bits == 8 ? kInt8 : (p->nibble_order ? kInt4Half : kInt4Seq));
  pl.grouped = (p->bits == 4) || (p->bits == 8 && p->group == 64);
  const int M = static_cast<int>(p->M), N = static_cast<int>(p->N), K = static_cast<int>(p->K);
  pl.mb = M <= 8 ? 1 : (M <= 16 ? 2 : 4);
  // More rows per CTA amortise the staging of x (read once per CTA from L2):
  // keep x traffic at or below the weight traffic where the grid still fills.
  const int rt_max = pl.mb == 4 ? 4 : (pl.mb == 2 ? 4 : (M <= 2 ? 1 : (M <= 4 ? 2 : 4)));
  const int rt_min = pl.mb == 4 ? 4 : (pl.mb == 2 ? 2 : 1);
  const int target = sm_count * 3 / 2;
  const size_t x_budget = 96 * 1024;
  bool found = false;
  for (int rt = rt_max; rt >= rt_min && !found; rt >>= 1) {
    const int tiles = static_cast<int>(CeilDiv(N, 16 * rt));
    for (int split = 1; split <= 8; split <<= 1) {
      if (K % (split * kGroupK) != 0) break;
      const int kc = K / split;
      if (static_cast<size_t>(M) * kc * 2 > x_budget) continue;
      const bool fills = static_cast<int64_t>(tiles) * split >= target;
      const bool last = split == 8 || K % (2 * split * kGroupK) != 0;
      if (fills || (last && rt == rt_min)) {
        pl.rt = rt;
        pl.split = split;
        found = true;
        break;
      }
    }
  }
  if (!found)
    return Fail(B200_UNIMPLEMENTED, "b200_qmm: M=%d K=%d does not fit the shared-memory staging of x", M, K);
  const int kc = K / pl.split;
  const int chunks = static_cast<int>(CeilDiv(kc, kChunkK));
  // Ring depth: everything in flight if it fits ~100 KB, else what fits.
  const size_t budget = 100 * 1024;
  pl.stages = chunks < 2 ? 2 : chunks;
  for (;;) {
    pl.smem = SmemFor(pl, M, kc);
    if (pl.smem <= budget || pl.stages <= 2) break;
    --pl.stages;
  }
  if (pl.stages > 32) {
    pl.stages = 32;
    pl.smem = SmemFor(pl, M, kc);
  }
  if (pl.smem > static_cast<size_t>(max_smem))
    return Fail(B200_UNIMPLEMENTED, "b200_qmm: needs %zu bytes of shared memory (limit %d)", pl.smem, max_smem);
  *out = pl;
  return B200_OK;
}

template <int FMT, int MB, int RT, bool GROUPED>
cudaError_t LaunchOne(const Plan& pl, const QmmArgs& args, dim3 grid, cudaStream_t stream) {
  auto kernel = qgemv_kernel<FMT, MB, RT, GROUPED>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(pl.smem));
  if (e != cudaSuccess) return e;
  LaunchCfg lc;
  lc.grid = grid;
  lc.block = dim3(kThreads);
  lc.smem = pl.smem;
  lc.stream = stream;
  lc.pdl = true;
  lc.cluster_y = pl.split;
  return Launch(lc, kernel, args);
}

template <int FMT, bool GROUPED>
cudaError_t LaunchFmt(const Plan& pl, const QmmArgs& args, dim3 grid, cudaStream_t stream) {
  switch (pl.mb * 10 + pl.rt) {
    case 11: return LaunchOne<FMT, 1, 1, GROUPED>(pl, args, grid, stream);
    case 12: return LaunchOne<FMT, 1, 2, GROUPED>(pl, args, grid, stream);
    case 14: return LaunchOne<FMT, 1, 4, GROUPED>(pl, args, grid, stream);
    case 22: return LaunchOne<FMT, 2, 2, GROUPED>(pl, args, grid, stream);
    case 24: return LaunchOne<FMT, 2, 4, GROUPED>(pl, args, grid, stream);
    case 44: return LaunchOne<FMT, 4, 4, GROUPED>(pl, args, grid, stream);
  }
  return cudaErrorInvalidValue;
}

}  // namespace

namespace b200 {

// Dense few-row product for b200_gemm: D = act(alpha * vecs[V, K] . mat[R, K]^T + bias),
// bf16 operands with K contiguous, V <= 32.  Element (v, r) of the result is
// written at v * out_vec_stride + r * out_row_stride.
b200_status RunFewRowNT(b200_context* ctx, cudaStream_t stream, const void* mat, const void* vecs, void* out,
                        int64_t R, int64_t V, int64_t K, int64_t ld_vec, int64_t out_row_stride,
                        int64_t out_vec_stride, float alpha, int act, const void* bias, int bias_by_vec,
                        void* aux, int out_f32) {
  b200_qmm_params p = {};
  p.bits = 16;
  p.x = vecs;
  p.q = mat;
  p.out = out;
  p.M = V;
  p.N = R;
  p.K = K;
  p.ldx = ld_vec;
  p.ldo = R;  // unused by the GEMM epilogue
  b200_status s = Validate(&p);
  if (s != B200_OK) return s;
  Plan pl;
  s = MakePlan(&p, ctx->sm_count, ctx->max_smem_optin, &pl);
  if (s != B200_OK) return s;
  QmmArgs a = {};
  a.q = static_cast<const uint8_t*>(mat);
  a.x = static_cast<const __nv_bfloat16*>(vecs);
  a.out = out;
  a.M = static_cast<int>(V);
  a.N = static_cast<int>(R);
  a.K = static_cast<int>(K);
  a.ldx = static_cast<int>(ld_vec);
  a.ldo = static_cast<int>(R);
  a.x_vec = Aligned(vecs, 16) && ld_vec % 8 == 0;
  a.k_per_cta = a.K / pl.split;
  a.epilogue = kEpilogueGemm;
  a.stages = pl.stages;
  a.status = ctx->dev_status;
  a.out_row_stride = out_row_stride;
  a.out_vec_stride = out_vec_stride;
  a.alpha = alpha;
  a.act = act;
  a.bias_by_vec = bias_by_vec;
  a.out_f32 = out_f32;
  a.gemm_bias = bias;
  a.aux = aux;
  const dim3 grid(static_cast<unsigned>(CeilDiv(a.N, 16 * pl.rt)), pl.split, 1);
  cudaError_t e = LaunchFmt<kBf16, false>(pl, a, grid, stream);
  if (e != cudaSuccess) return Stick(ctx, Fail(B200_INTERNAL, "few-row GEMM launch: %s", cudaGetErrorString(e)));
  return EndLaunch(ctx, "b200_gemm (few-row)");
}

}  // namespace b200

extern "C" {

b200_status b200_qmm_validate(const b200_qmm_params* p) { return Validate(p); }

b200_status b200_qmm_plan(const b200_qmm_params* p, int* rows_per_cta, int* split_k, int* batch_blocks) {
  b200_status s = Validate(p);
  if (s != B200_OK) return s;
  Plan pl;
  s = MakePlan(p, 148, 227 * 1024, &pl);
  if (s != B200_OK) return s;
  if (rows_per_cta) *rows_per_cta = 16 * pl.rt;
  if (split_k) *split_k = pl.split;
  if (batch_blocks) *batch_blocks = pl.mb;
  return B200_OK;
}

b200_status b200_qmm_run(b200_context* ctx, b200_stream stream, const b200_qmm_params* p) {
  b200_status s = BeginLaunch(ctx);
  if (s != B200_OK) return s;
  s = Validate(p);
  if (s != B200_OK) return s;
  if (p->M == 0 || p->N == 0) return B200_OK;
  Plan pl;
  s = MakePlan(p, ctx->sm_count, ctx->max_smem_optin, &pl);
  if (s != B200_OK) return s;
  QmmArgs a;
  a.q = static_cast<const uint8_t*>(p->q);
  a.scale = static_cast<const __nv_bfloat16*>(p->scale);
  a.bias = static_cast<const __nv_bfloat16*>(p->bias);
  a.x = static_cast<const __nv_bfloat16*>(p->x);
  a.residual = static_cast<const __nv_bfloat16*>(p->residual);
  a.out = p->out;
  a.M = static_cast<int>(p->M);
  a.N = static_cast<int>(p->N);
  a.K = static_cast<int>(p->K);
  a.ldx = static_cast<int>(p->ldx ? p->ldx : (p->prologue == B200_QMM_PRO_SILU_MUL ? 2 * p->K : p->K));
  a.ldo = static_cast<int>(p->ldo ? p->ldo : p->N);
  a.prologue = p->prologue;
  a.eps = p->eps;
  a.gain = static_cast<const __nv_bfloat16*>(p->prologue_gain);
  a.x_vec = Aligned(p->x, 16) && a.ldx % 8 == 0 && (p->prologue != B200_QMM_PRO_RMSNORM || Aligned(p->prologue_gain, 16));
  a.scale_ld = p->bits == 16 ? 0 : static_cast<int>(p->K / p->group);
  a.k_per_cta = a.K / pl.split;
  a.epilogue = p->epilogue;
  a.stages = pl.stages;
  a.status = ctx->dev_status;
  a.out_row_stride = a.out_vec_stride = 0;
  a.alpha = 1.0f;
  a.act = a.bias_by_vec = a.out_f32 = 0;
  a.gemm_bias = nullptr;
  a.aux = nullptr;
  const dim3 grid(static_cast<unsigned>(CeilDiv(a.N, 16 * pl.rt)), pl.split, 1);
  cudaError_t e;
  switch (pl.fmt) {
    case kInt4Seq: e = LaunchFmt<kInt4Seq, true>(pl, a, grid, stream); break;
    case kInt4Half: e = LaunchFmt<kInt4Half, true>(pl, a, grid, stream); break;
    case kInt8:
      e = pl.grouped ? LaunchFmt<kInt8, true>(pl, a, grid, stream) : LaunchFmt<kInt8, false>(pl, a, grid, stream);
      break;
    default: e = LaunchFmt<kBf16, false>(pl, a, grid, stream); break;
  }
  if (e != cudaSuccess) return Stick(ctx, Fail(B200_INTERNAL, "b200_qmm launch: %s", cudaGetErrorString(e)));
  return EndLaunch(ctx, "b200_qmm");
}

b200_status b200_qmm(b200_context* ctx, b200_stream stream, int bits, int group, int nibble_order, const void* x,
                     const void* q, const void* scale, const void* bias_or_null, void* out, int64_t M, int64_t N,
                     int64_t K, int act_dtype) {
  if (act_dtype != B200_BF16)
    return Fail(B200_UNIMPLEMENTED, "b200_qmm: activations must be bf16 (dtype %d given)", act_dtype);
  b200_qmm_params p = {};
  p.bits = bits;
  p.group = group;
  p.nibble_order = nibble_order;
  p.epilogue = B200_QMM_OUT_BF16;
  p.x = x;
  p.q = q;
  p.scale = scale;
  p.bias = bias_or_null;
  p.out = out;
  p.M = M;
  p.N = N;
  p.K = K;
  return b200_qmm_run(ctx, stream, &p);
}

}  // extern "C"
