// int4-g64 dequant-matmul for up to 8 rows of x on the 5th-generation tensor cores
// (≙ _matvec_int4 / dequantize + dot of the reference, examples/llm/qwen3.py:199-267).
//
// Status: an alternative route, taken only with B200_QMM_TC=1.  It is correct (the parity tests
// pass on it) but slower than the mma.sync kernel for these shapes, for a reason measured on the
// device: one tcgen05.mma costs ~194 SM cycles whatever its N (16 ... 256), M (64, 128), operand
// kind (f8f6f4, f16) or A source (shared or tensor memory).  With the weights on the M side an
// instruction covers 128 rows x 32 inputs = 2 KB of nibbles, so an SM cannot stream more than
// 2 KB / 194 cycles = 10.5 B/cycle: 2.95 TB/s over 148 SMs at 1.9 GHz, below what the mma.sync
// kernel reaches (3.5 TB/s on the 24576 x 4096 projection).  The tensor core only pays once the
// batch fills the instruction's N (hundreds of columns).
//
// The idea: with mma.sync the nibbles have to be widened to bf16 in registers (4 two-cycle logic
// operations per 8 weights, plus the fragment loads and the MMA issue), and that ALU work, not
// HBM, bounds the kernel.  Here the nibbles are only spread to BYTES (3 operations per 8 weights):
// a byte 0x0q read as e4m3 is exactly q * 2^-9, so the spread bytes ARE the A operand of a
// tcgen05.mma kind::f8f6f4.  The activations are the B operand: every bf16 value x (times a
// power of two that brings the row's largest magnitude near 256) is split exactly into two e4m3
// terms x = x1 + x2 (4 significant bits each; exact for every element within 2^10 of the
// largest), which sit in the B matrix as two columns per batch row.
//
//   HBM --TMA (128 rows x 128 B boxes, 128-byte swizzle)--> shared memory ring
//   thread r of a warpgroup owns row r of the 128-row tile: LDS.128 x2 (64 nibbles = one group)
//     -> 16 registers of bytes -> tcgen05.st into TMEM (A operand: lane = row, 4 k per column)
//   one thread of the warpgroup: 2 x tcgen05.mma (M 128, N 16, K 32) -> D in TMEM, commit -> mbarrier
//   thread r again: tcgen05.ld its row of D (the group's q.x1 and q.x2 sums per batch row),
//     acc += scale[r][g] * (d1 + d2);  acc_b += offset[r][g] * sum_k x   (f32, per group: the
//     promotion out of the tensor core's accumulator every 64 inputs)
// A and D are double-buffered per warpgroup, so widening group g+1 overlaps the MMA of group g.
// The four warpgroups of a CTA take different 256-input chunks; the producer warp keeps the ring full.
//
// Work is cut into units of (128-row tile, 256-input chunk) and dealt out evenly as contiguous
// ranges: every SM streams the same number of bytes whatever N and K are.  A tile whose chunks
// are shared by several CTAs is finished by the last of them to arrive, which adds the partial
// rows of all of them in a fixed order (deterministic) from a scratch buffer of the context.
//
// Every wait is bounded; after one gives up the CTA keeps its control flow (so barriers still
// meet) but waits for nothing, frees its TMEM, and the status word reports B200_TIMEOUT.
#include <cuda.h>

#include <algorithm>

#include "common.cuh"
#include "qmm_tc.cuh"

using namespace b200;

namespace b200 {
namespace qtc {

constexpr int kWarpgroups = 4;
constexpr int kConsumerWarps = 16;
constexpr int kConsumers = kConsumerWarps * 32;
constexpr int kThreads = kConsumers + 32;      // + the producer warp
constexpr int kTileRows = 128;
constexpr int kChunkK = 256;                   // inputs per unit: one 128-byte swizzle row of nibbles
constexpr int kSlotBytes = kTileRows * 128;    // 16 KB
constexpr int kMaxSlots = 8;
constexpr uint32_t kTmemCols = 256;            // per warpgroup: A 2 x 16 columns, D 2 x 16 columns
constexpr uint32_t kIdesc = (1u << 4) /* f32 accumulate */ | (0u << 7) | (0u << 10) /* e4m3 x e4m3 */ |
                            ((16u >> 3) << 17) | ((128u >> 4) << 24);

struct Args {
  const __nv_bfloat16* scale;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* x;
  const __nv_bfloat16* residual;
  const __nv_bfloat16* gain;
  void* out;
  int M, N, K;
  int ldx, ldo;
  int epilogue, prologue;
  float eps;
  int MT;                 // rows of x per e4m3 term in shared memory: 4 or 8 (the B operand has 2 MT rows)
  int slots;
  int xchunks;            // chunks of x a CTA keeps in shared memory (its longest run of units, at most a whole row)
  int units, chunks_per_tile;
  float* parts;           // [tile][max_parts][MT][128] partial rows of tiles shared between CTAs
  unsigned* counters;     // [tile] CTAs that have delivered their part
  int max_parts;
  int* status;
};

struct Layout {
  size_t ring, xq, xsum, red, misc, total;
};
__host__ __device__ inline Layout MakeLayout(int xchunks, int MT, int slots) {
  Layout l;
  l.ring = 0;
  l.xq = static_cast<size_t>(slots) * kSlotBytes;
  l.xsum = l.xq + static_cast<size_t>(2 * MT) * kChunkK * xchunks + 256;   // (+ what a 16-row read of an 8-row operand overshoots)
  l.red = l.xsum + static_cast<size_t>(MT) * 4 * xchunks * 4;
  l.misc = l.red + static_cast<size_t>(kWarpgroups) * kTileRows * MT * 4;
  l.total = l.misc + 512;
  return l;
}

struct Misc {
  uint64_t full[kMaxSlots];
  uint64_t empty[kMaxSlots];
  uint64_t done[kWarpgroups][2];
  float stat[kConsumerWarps][8];
  float inv_p[8];       // 512 / (power-of-two scale of row m)
  float pscale[8];
  float rinv[8];
  uint32_t tmem;
  int dead;
  int last;
};
static_assert(sizeof(Misc) <= 1024 - 64, "misc block");

// ---- PTX ------------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// D[tmem_d] (+)= A[tmem_a] . B[desc_b]^T, A e4m3 from tensor memory, B e4m3 from shared memory
__device__ __forceinline__ void umma_f8_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [%1], %2, %3, p;\n\t}" ::"r"(tmem_d),
      "r"(tmem_a), "l"(desc_b), "r"(kIdesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]),
      "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
      : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
               : "r"(taddr)
               : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// K-major operand without swizzle: 8 rows x 16 bytes core matrices; `lbo` bytes between the two
// 16-byte pieces of a 32-byte K step, `sbo` bytes between groups of 8 rows.
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>(lbo >> 4) << 16;
  d |= static_cast<uint64_t>(sbo >> 4) << 32;
  d |= 1ull << 46;
  return d;
}
__device__ __forceinline__ void named_barrier(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
// two floats -> two e4m3 bytes (lo in bits 0..7), round to nearest, saturating
__device__ __forceinline__ uint32_t cvt_e4m3x2(float lo, float hi) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ float2 e4m3x2_to_f32(uint32_t v) {
  uint32_t h2;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(static_cast<uint16_t>(v)));
  const __half2 h = *reinterpret_cast<const __half2*>(&h2);
  return __half22float2(h);
}

// The CTA's contiguous range of units and the bookkeeping of tiles shared between CTAs.
__host__ __device__ inline long long UnitBegin(int cta, int ctas, int units) {
  return static_cast<long long>(cta) * units / ctas;
}
__host__ __device__ inline int UnitOwner(long long u, int ctas, int units) {
  return static_cast<int>(((u + 1) * ctas - 1) / units);
}

__global__ void __launch_bounds__(kThreads, 1) qmm_tc_kernel(const __grid_constant__ CUtensorMap wmap, const Args a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const Layout L = MakeLayout(a.xchunks, a.MT, a.slots);
  uint8_t* xq = smem + L.xq;
  float* xsum = reinterpret_cast<float*>(smem + L.xsum);     // [group of the kept chunks][MT]
  float* red = reinterpret_cast<float*>(smem + L.red);       // [warpgroup][m][128]
  Misc* mi = reinterpret_cast<Misc*>(smem + L.misc);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int ctas = gridDim.x, cta = blockIdx.x;
  const int CPT = a.chunks_per_tile, MT = a.MT, NR = 2 * a.MT;
  const long long u0 = UnitBegin(cta, ctas, a.units), u1 = UnitBegin(cta + 1, ctas, a.units);
  const int n_units = static_cast<int>(u1 - u0);

  if (tid == 0) {
    for (int s = 0; s < a.slots; ++s) {
      mbar_init(&mi->full[s], 1);
      mbar_init(&mi->empty[s], 4);    // the four warps of the warpgroup that owns the unit
    }
    for (int w = 0; w < kWarpgroups; ++w) {
      mbar_init(&mi->done[w][0], 1);
      mbar_init(&mi->done[w][1], 1);
    }
    mi->dead = 0;
    mbar_fence_init();
  }
  if (warp == kConsumerWarps) {   // the producer warp also owns the tensor memory
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&mi->tmem)), "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_launch_dependents();
  const uint32_t tmem = mi->tmem;
  volatile int* dead = &mi->dead;

  if (warp == kConsumerWarps) {
    // ---- producer: the weights do not depend on the kernel before this one -----------------
    if (lane == 0) {
      for (int i = 0; i < n_units; ++i) {
        const int s = i % a.slots;
        const int lap = i / a.slots;
        if (lap > 0 && !*dead && !mbar_wait_bounded<64>(&mi->empty[s], (lap - 1) & 1)) {
          *dead = 1;
          report_timeout(a.status, 700 + s);
        }
        const long long u = u0 + i;
        const int t = static_cast<int>(u / CPT), c = static_cast<int>(u % CPT);
        mbar_expect_tx(&mi->full[s], kSlotBytes);
        tma_load_2d(smem_u32(smem + static_cast<size_t>(s) * kSlotBytes), &wmap, c * 128, t * kTileRows, &mi->full[s]);
      }
    }
  } else {
    // ---- consumers ---------------------------------------------------------------------------
    const int wg = warp >> 2, q = warp & 3;
    const int row = 32 * q + lane;                       // row of the tile = TMEM lane
    const uint32_t lane_base = static_cast<uint32_t>(32 * q) << 16;
    const uint32_t colA = static_cast<uint32_t>(wg * 64), colD = static_cast<uint32_t>(wg * 64 + 32);

    // The chunks this CTA needs x for: everything, or a cyclic run of chunks_per_tile.
    const int need = n_units >= CPT ? CPT : n_units;
    const int c_first = n_units >= CPT ? 0 : static_cast<int>(u0 % CPT);
    pdl_wait();   // x (and the residual) come from the kernel before
    // -- pass 0: per row of x, what the e4m3 split scales by (and the RMSNorm factor) --------------
    {
      float mx[8], ss[8];
#pragma unroll
      for (int m = 0; m < 8; ++m) mx[m] = ss[m] = 0.0f;
      const int runs_row = need * (kChunkK / 8);
#pragma unroll 1
      for (int m = 0; m < a.M; ++m) {
        const __nv_bfloat16* xr = a.x + static_cast<size_t>(m) * a.ldx;
        if (a.prologue == B200_QMM_PRO_RMSNORM) {   // the norm needs the whole row
          for (int i = tid; i < a.K / 8; i += kConsumers) {
            const uint4 raw = __ldg(reinterpret_cast<const uint4*>(xr + i * 8));
            const uint4 gr = __ldg(reinterpret_cast<const uint4*>(a.gain + i * 8));
            const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w}, g[4] = {gr.x, gr.y, gr.z, gr.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float e0 = bf16_lo(w[j]), e1 = bf16_hi(w[j]);
              ss[m] = fmaf(e0, e0, ss[m]);
              ss[m] = fmaf(e1, e1, ss[m]);
              mx[m] = fmaxf(mx[m], fmaxf(fabsf(e0 * bf16_lo(g[j])), fabsf(e1 * bf16_hi(g[j]))));
            }
          }
        } else {
          for (int i = tid; i < runs_row; i += kConsumers) {
            const int k = ((c_first + i / 32) % CPT) * kChunkK + (i % 32) * 8;
            const uint4 raw = __ldg(reinterpret_cast<const uint4*>(xr + k));
            const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
            if (a.prologue == B200_QMM_PRO_SILU_MUL) {   // |silu(g) up| <= |g up|
              const uint4 ur = __ldg(reinterpret_cast<const uint4*>(xr + a.K + k));
              const uint32_t u[4] = {ur.x, ur.y, ur.z, ur.w};
#pragma unroll
              for (int j = 0; j < 4; ++j)
                mx[m] = fmaxf(mx[m], fmaxf(fabsf(bf16_lo(w[j]) * bf16_lo(u[j])), fabsf(bf16_hi(w[j]) * bf16_hi(u[j]))));
            } else {
#pragma unroll
              for (int j = 0; j < 4; ++j) mx[m] = fmaxf(mx[m], fmaxf(fabsf(bf16_lo(w[j])), fabsf(bf16_hi(w[j]))));
            }
          }
        }
      }
#pragma unroll
      for (int m = 0; m < 8; ++m) {
        mx[m] = warp_max(mx[m]);
        ss[m] = warp_sum(ss[m]);
      }
      // two rounds through the 16 x 8 table: maxima, then sums
      if (lane == 0) {
#pragma unroll
        for (int m = 0; m < 8; ++m) mi->stat[warp][m] = mx[m];
      }
      named_barrier(1, kConsumers);
      float bmax = 0.0f;
      if (tid < 8) {
        for (int w = 0; w < kConsumerWarps; ++w) bmax = fmaxf(bmax, mi->stat[w][tid]);
      }
      named_barrier(1, kConsumers);
      if (lane == 0) {
#pragma unroll
        for (int m = 0; m < 8; ++m) mi->stat[warp][m] = ss[m];
      }
      named_barrier(1, kConsumers);
      if (tid < 8) {
        float tot = 0.0f;
        for (int w = 0; w < kConsumerWarps; ++w) tot += mi->stat[w][tid];
        float rr = 1.0f;
        if (a.prologue == B200_QMM_PRO_RMSNORM) {
          rr = 1.0f / sqrtf(tot / static_cast<float>(a.K) + a.eps);
          bmax *= rr;
        }
        bmax *= 1.01f;   // the transforms round to bf16 on the way
        // power of two p with bound * p in [128, 256): e4m3 holds up to 448
        float p = 1.0f;
        if (bmax > 0.0f && bmax < 3.0e38f) {
          int e;
          frexpf(bmax, &e);                 // bmax = f * 2^e, f in [0.5, 1)
          p = ldexpf(1.0f, max(-100, min(100, 8 - e)));   // bmax * p in [128, 256)
        }
        mi->rinv[tid] = rr;
        mi->pscale[tid] = p;
        mi->inv_p[tid] = 512.0f / p;
      }
      named_barrier(1, kConsumers);
    }
    // -- pass 1: the transformed activations, split into two e4m3 terms, into the B operand ------
    // B operand, K-major without swizzle: 16-byte piece j of K holds rows 0 .. NR-1 back to back.
    // Within a 32-byte K step the bytes follow the order the nibble spreading produces:
    // position 8i + h * 4 + e <-> input 8i + 2e + h.
    {
      const int runs_row = need * (kChunkK / 8);
      const int total = a.M * runs_row;
#pragma unroll 1
      for (int idx = tid; idx < ((total + 31) & ~31); idx += kConsumers) {
        const bool valid = idx < total;
        const int m = valid ? idx / runs_row : 0;
        const int i = valid ? idx % runs_row : 0;
        const int k = ((c_first + i / 32) % CPT) * kChunkK + (i % 32) * 8;   // input
        const int kl = i * 8;                                                // ... and where it sits among the kept chunks
        float e[8];
        float sum = 0.0f;
        if (valid) {
          const __nv_bfloat16* xr = a.x + static_cast<size_t>(m) * a.ldx;
          const uint4 raw = __ldg(reinterpret_cast<const uint4*>(xr + k));
          const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            e[2 * j] = bf16_lo(w[j]);
            e[2 * j + 1] = bf16_hi(w[j]);
          }
          if (a.prologue == B200_QMM_PRO_RMSNORM) {
            const uint4 gr = __ldg(reinterpret_cast<const uint4*>(a.gain + k));
            const uint32_t g[4] = {gr.x, gr.y, gr.z, gr.w};
            const float rr = mi->rinv[m];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              e[2 * j] = bf16_round((e[2 * j] * rr) * bf16_lo(g[j]));
              e[2 * j + 1] = bf16_round((e[2 * j + 1] * rr) * bf16_hi(g[j]));
            }
          } else if (a.prologue == B200_QMM_PRO_SILU_MUL) {
            const uint4 ur = __ldg(reinterpret_cast<const uint4*>(xr + a.K + k));
            const uint32_t u[4] = {ur.x, ur.y, ur.z, ur.w};
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float up = (j & 1) ? bf16_hi(u[j >> 1]) : bf16_lo(u[j >> 1]);
              const float sig = bf16_round(__fdividef(1.0f, 1.0f + __expf(-e[j])));
              e[j] = bf16_round(bf16_round(e[j] * sig) * up);
            }
          }
          const float p = mi->pscale[m];
          uint32_t t1[4], t2[4];   // e4m3 pairs (inputs 2j, 2j+1) of the two terms
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            sum += e[2 * j] + e[2 * j + 1];
            const float s0 = e[2 * j] * p, s1 = e[2 * j + 1] * p;
            t1[j] = cvt_e4m3x2(s0, s1);
            const float2 back = e4m3x2_to_f32(t1[j]);
            t2[j] = cvt_e4m3x2(s0 - back.x, s1 - back.y);
          }
          // bytes in operand order: inputs 0, 2, 4, 6, 1, 3, 5, 7
          const uint32_t a_lo = (t1[0] & 0xff) | ((t1[1] & 0xff) << 8) | ((t1[2] & 0xff) << 16) | ((t1[3] & 0xff) << 24);
          const uint32_t a_hi = ((t1[0] >> 8) & 0xff) | (((t1[1] >> 8) & 0xff) << 8) | (((t1[2] >> 8) & 0xff) << 16) | (((t1[3] >> 8) & 0xff) << 24);
          const uint32_t b_lo = (t2[0] & 0xff) | ((t2[1] & 0xff) << 8) | ((t2[2] & 0xff) << 16) | ((t2[3] & 0xff) << 24);
          const uint32_t b_hi = ((t2[0] >> 8) & 0xff) | (((t2[1] >> 8) & 0xff) << 8) | (((t2[2] >> 8) & 0xff) << 16) | (((t2[3] >> 8) & 0xff) << 24);
          uint8_t* piece = xq + static_cast<size_t>(kl >> 4) * (NR * 16) + (kl & 8);
          *reinterpret_cast<uint2*>(piece + m * 16) = make_uint2(a_lo, a_hi);
          *reinterpret_cast<uint2*>(piece + (MT + m) * 16) = make_uint2(b_lo, b_hi);
        }
        // the eight threads of a 64-input group add up its sum of x
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        sum += __shfl_xor_sync(0xffffffffu, sum, 4);
        if (valid && (lane & 7) == 0) xsum[(kl >> 6) * MT + m] = sum;
      }
      // rows of the operand that hold no batch row: zeros (their columns of D are never read, but keep them finite)
      for (int idx = tid; idx < need * (kChunkK / 16) * (MT - a.M); idx += kConsumers) {
        const int piece_i = idx / (MT - a.M), mm = a.M + idx % (MT - a.M);
        uint8_t* piece = xq + static_cast<size_t>(piece_i) * (NR * 16);
        *reinterpret_cast<uint4*>(piece + mm * 16) = make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4*>(piece + (MT + mm) * 16) = make_uint4(0, 0, 0, 0);
      }
    }
    // make the generic-proxy writes of x visible to the tensor core's reads of shared memory
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    named_barrier(1, kConsumers);

    const uint32_t xq_addr = smem_u32(xq);
    const uint32_t lbo = static_cast<uint32_t>(NR * 16), sbo = 128u;
    uint32_t done_phase[2] = {0u, 0u};
    int issued = 0;   // groups this warpgroup has issued so far (selects the A / D buffer)

    // ---- segments: runs of this CTA's units inside one tile --------------------------------------
    int i0 = 0;
#pragma unroll 1
    while (i0 < n_units) {
      const long long ua = u0 + i0;
      const int t = static_cast<int>(ua / CPT);
      const int i1 = static_cast<int>(min(static_cast<long long>(n_units), (static_cast<long long>(t) + 1) * CPT - u0));
      const int grow = t * kTileRows + row;
      const bool row_ok = grow < a.N;
      float accA[8], accB[8];
#pragma unroll
      for (int m = 0; m < 8; ++m) accA[m] = accB[m] = 0.0f;
      // this warpgroup's units of the segment: i = wg (mod 4) counted over the CTA's whole range
      int i = i0 + ((wg - i0) & 3);
      const __nv_bfloat16* srow = a.scale + static_cast<size_t>(row_ok ? grow : 0) * (a.K / 64);
      const __nv_bfloat16* brow = a.bias + static_cast<size_t>(row_ok ? grow : 0) * (a.K / 64);
      uint2 s_next = make_uint2(0, 0), b_next = make_uint2(0, 0);
      if (i < i1) {
        const int c = static_cast<int>((u0 + i) % CPT);
        s_next = __ldg(reinterpret_cast<const uint2*>(srow + 4 * c));
        b_next = __ldg(reinterpret_cast<const uint2*>(brow + 4 * c));
      }
      // the group waiting to be drained
      bool pending = false;
      int pend_buf = 0, pend_g = 0;
      float pend_s = 0.0f, pend_b = 0.0f;
      auto drain = [&]() {
        if (!*dead && !mbar_wait_bounded(&mi->done[wg][pend_buf], done_phase[pend_buf])) {
          *dead = 1;
          report_timeout(a.status, 720 + wg);
        }
        done_phase[pend_buf] ^= 1u;
        tc_fence_after();
        uint32_t d[16];
        const uint32_t taddr = tmem + lane_base + colD + static_cast<uint32_t>(pend_buf * 16);
        if (MT == 4) {
          tmem_ld8(taddr, d);
        } else {
          tmem_ld16(taddr, d);
        }
        tc_fence_before();
        const float* xs = xsum + pend_g * MT;   // (pend_g counts groups of the kept chunks)
#pragma unroll
        for (int m = 0; m < 8; ++m) {
          if (m < MT) {
            const float dot = __uint_as_float(d[m]) + __uint_as_float(MT == 4 ? d[4 + (m & 3)] : d[8 + m]);
            accA[m] = fmaf(pend_s, dot, accA[m]);
            accB[m] = fmaf(pend_b, xs[m], accB[m]);
          }
        }
        pending = false;
      };
#pragma unroll 1
      for (; i < i1; i += 4) {
        const int s = i % a.slots;
        const int c = static_cast<int>((u0 + i) % CPT);
        const int cl = (c - c_first + CPT) % CPT;   // the chunk among the kept ones
        const uint2 s_cur = s_next, b_cur = b_next;
        if (i + 4 < i1) {
          const int cn = static_cast<int>((u0 + i + 4) % CPT);
          s_next = __ldg(reinterpret_cast<const uint2*>(srow + 4 * cn));
          b_next = __ldg(reinterpret_cast<const uint2*>(brow + 4 * cn));
        }
        if (!*dead && !mbar_wait_bounded(&mi->full[s], (i / a.slots) & 1)) {
          *dead = 1;
          report_timeout(a.status, 710 + s);
        }
        const uint32_t slot_row = smem_u32(smem + static_cast<size_t>(s) * kSlotBytes) + static_cast<uint32_t>(row) * 128u;
#pragma unroll 1
        for (int g = 0; g < 4; ++g) {
          const int buf = issued & 1;
          // 64 nibbles of this thread's row: 16-byte pieces 2g, 2g+1 of the swizzled 128-byte row
          uint4 w0, w1;
          {
            const uint32_t p0 = slot_row + (static_cast<uint32_t>((2 * g) ^ (row & 7)) << 4);
            const uint32_t p1 = slot_row + (static_cast<uint32_t>((2 * g + 1) ^ (row & 7)) << 4);
            asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(w0.x), "=r"(w0.y), "=r"(w0.z), "=r"(w0.w) : "r"(p0));
            asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(w1.x), "=r"(w1.y), "=r"(w1.z), "=r"(w1.w) : "r"(p1));
          }
          const uint32_t ws[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
          uint32_t bytes[16];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            bytes[2 * j] = ws[j] & 0x0F0F0F0Fu;             // inputs 8j + 0, 2, 4, 6
            bytes[2 * j + 1] = (ws[j] >> 4) & 0x0F0F0F0Fu;  // inputs 8j + 1, 3, 5, 7
          }
          tmem_st16(tmem + lane_base + colA + static_cast<uint32_t>(buf * 16), bytes);
          tc_fence_before();
          named_barrier(2 + wg, 128);
          if (q == 0 && lane == 0) {
            tc_fence_after();
            const uint32_t b_addr = xq_addr + static_cast<uint32_t>(4 * (4 * cl + g)) * lbo;
            const uint32_t d_t = tmem + colD + static_cast<uint32_t>(buf * 16);
            const uint32_t a_t = tmem + colA + static_cast<uint32_t>(buf * 16);
            umma_f8_ts(d_t, a_t, make_desc(b_addr, lbo, sbo), 0u);
            umma_f8_ts(d_t, a_t + 8u, make_desc(b_addr + 2u * lbo, lbo, sbo), 1u);
            umma_commit(&mi->done[wg][buf]);
          }
          // while the tensor core works on this group, fold in the one before
          if (pending) drain();
          pending = true;
          pend_buf = buf;
          pend_g = 4 * cl + g;
          const uint32_t sw = g < 2 ? s_cur.x : s_cur.y, bw = g < 2 ? b_cur.x : b_cur.y;
          pend_s = (g & 1) ? bf16_hi(sw) : bf16_lo(sw);
          pend_b = (g & 1) ? bf16_hi(bw) : bf16_lo(bw);
          ++issued;
        }
        // the slot is free once every warp of the warpgroup has read its rows
        __syncwarp();
        if (lane == 0) mbar_arrive(&mi->empty[s]);
      }
      if (pending) drain();
      // ---- end of the segment: add the warpgroups' rows, then finish or hand over ------------------
#pragma unroll
      for (int m = 0; m < 8; ++m)
        if (m < MT) red[(wg * MT + m) * kTileRows + row] = fmaf(accA[m], mi->inv_p[m], accB[m]);
      named_barrier(1, kConsumers);
      if (wg == 0) {
        float v[8];
#pragma unroll
        for (int m = 0; m < 8; ++m) {
          v[m] = 0.0f;
          if (m < MT) {
#pragma unroll
            for (int w = 0; w < kWarpgroups; ++w) v[m] += red[(w * MT + m) * kTileRows + row];
          }
        }
        const bool whole = (i1 - i0) == CPT;
        bool finish = whole;
        if (!whole) {
          // part index: CTAs before this one that share the tile
          const int first = UnitOwner(static_cast<long long>(t) * CPT, ctas, a.units);
          const int last = UnitOwner(static_cast<long long>(t + 1) * CPT - 1, ctas, a.units);
          const int nparts = last - first + 1, part = cta - first;
          float* mine = a.parts + (static_cast<size_t>(t) * a.max_parts + part) * (MT * kTileRows);
#pragma unroll
          for (int m = 0; m < 8; ++m)
            if (m < a.M) __stcg(mine + m * kTileRows + row, v[m]);
          __threadfence();
          named_barrier(2, 128);
          if (tid == 0) {
            __threadfence();
            const unsigned old = atomicAdd(a.counters + t, 1u);
            mi->last = old == static_cast<unsigned>(nparts - 1);
            if (mi->last) a.counters[t] = 0u;   // every part is in: ready for the next launch
          }
          named_barrier(2, 128);
          finish = mi->last != 0;
          if (finish) {
            __threadfence();
            const float* base = a.parts + static_cast<size_t>(t) * a.max_parts * (MT * kTileRows);
#pragma unroll
            for (int m = 0; m < 8; ++m) {
              if (m < a.M) {
                float tot = 0.0f;
                for (int pi = 0; pi < nparts; ++pi) tot += __ldcg(base + static_cast<size_t>(pi) * (MT * kTileRows) + m * kTileRows + row);
                v[m] = tot;
              }
            }
          }
        }
        if (finish && row_ok) {
#pragma unroll
          for (int m = 0; m < 8; ++m) {
            if (m < a.M) {
              const size_t o = static_cast<size_t>(m) * a.ldo + grow;
              const float y = bf16_round(v[m]);
              if (a.epilogue == B200_QMM_OUT_F32_RAW) {
                static_cast<float*>(a.out)[o] = v[m];
              } else if (a.epilogue == B200_QMM_OUT_F32) {
                static_cast<float*>(a.out)[o] = y;
              } else if (a.epilogue == B200_QMM_ADD_RESIDUAL) {
                static_cast<__nv_bfloat16*>(a.out)[o] = __float2bfloat16_rn(__bfloat162float(a.residual[o]) + y);
              } else {
                static_cast<__nv_bfloat16*>(a.out)[o] = __float2bfloat16_rn(v[m]);
              }
            }
          }
        }
      }
      named_barrier(1, kConsumers);   // `red` is free again
      i0 = i1;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kConsumerWarps) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
  }
}

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn Encoder() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

}  // namespace qtc

bool QmmTcEligible(const b200_context* ctx, const b200_qmm_params* p) {
  if (p->bits != 4 || p->nibble_order != 0 || p->group != 64) return false;
  if (p->M < 1 || p->M > 8 || p->N < 1 || p->K < qtc::kChunkK || p->K % qtc::kChunkK != 0) return false;
  if (p->prologue == B200_QMM_PRO_RMSNORM && p->prologue_gain == nullptr) return false;
  const int64_t xcols = p->prologue == B200_QMM_PRO_SILU_MUL ? 2 * p->K : p->K;
  const int64_t ldx = p->ldx ? p->ldx : xcols;
  if (!Aligned(p->x, 16) || ldx % 8 != 0 || !Aligned(p->q, 16) || !Aligned(p->scale, 8) || !Aligned(p->bias, 8)) return false;
  if (p->prologue == B200_QMM_PRO_RMSNORM && !Aligned(p->prologue_gain, 16)) return false;
  if (ctx->qtc_parts == nullptr || qtc::Encoder() == nullptr) return false;
  const int MT = p->M <= 4 ? 4 : 8;
  const int64_t tiles = CeilDiv(p->N, qtc::kTileRows);
  const int64_t cpt = p->K / qtc::kChunkK;
  if (tiles * cpt > (1ll << 30) || tiles > ctx->qtc_tiles_max) return false;
  const int64_t units = tiles * cpt;
  const int64_t ctas = std::min<int64_t>(ctx->sm_count, units);
  const int xchunks = static_cast<int>(std::min<int64_t>(cpt, CeilDiv(units, ctas)));
  if (qtc::MakeLayout(xchunks, MT, 8).total + 1024 > static_cast<size_t>(ctx->max_smem_optin)) return false;
  return true;
}

b200_status QmmTcRun(b200_context* ctx, cudaStream_t stream, const b200_qmm_params* p) {
  using namespace qtc;
  Args a = {};
  a.scale = static_cast<const __nv_bfloat16*>(p->scale);
  a.bias = static_cast<const __nv_bfloat16*>(p->bias);
  a.x = static_cast<const __nv_bfloat16*>(p->x);
  a.residual = static_cast<const __nv_bfloat16*>(p->residual);
  a.gain = static_cast<const __nv_bfloat16*>(p->prologue_gain);
  a.out = p->out;
  a.M = static_cast<int>(p->M);
  a.N = static_cast<int>(p->N);
  a.K = static_cast<int>(p->K);
  a.ldx = static_cast<int>(p->ldx ? p->ldx : (p->prologue == B200_QMM_PRO_SILU_MUL ? 2 * p->K : p->K));
  a.ldo = static_cast<int>(p->ldo ? p->ldo : p->N);
  a.epilogue = p->epilogue;
  a.prologue = p->prologue;
  a.eps = p->eps;
  a.MT = a.M <= 4 ? 4 : 8;
  a.chunks_per_tile = a.K / kChunkK;
  const int tiles = static_cast<int>(CeilDiv(a.N, kTileRows));
  a.units = tiles * a.chunks_per_tile;
  const int ctas = std::min(ctx->sm_count, a.units);
  // CTAs that can share one tile: ceil(chunks per tile / least units per CTA) + 1
  const int least = std::max(1, a.units / ctas);
  a.max_parts = std::min(ctas, static_cast<int>(CeilDiv(a.chunks_per_tile, least)) + 1);
  if (static_cast<size_t>(tiles) * a.max_parts * a.MT * kTileRows > ctx->qtc_parts_floats)
    return Fail(B200_RESOURCE_EXHAUSTED, "b200_qmm: partial-row scratch too small for N=%d K=%d", a.N, a.K);
  a.parts = ctx->qtc_parts;
  a.counters = ctx->qtc_counters;
  a.status = ctx->dev_status;
  a.xchunks = std::min(a.chunks_per_tile, static_cast<int>(CeilDiv(a.units, ctas)));
  // a multiple of four slots: a slot then always belongs to the same warpgroup, whose waits on it stay in phase order
  a.slots = 8;
  const size_t smem = MakeLayout(a.xchunks, a.MT, a.slots).total + 1024;

  CUtensorMap map;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(a.K / 2), static_cast<cuuint64_t>(a.N)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(a.K / 2)};
  const cuuint32_t box[2] = {128, static_cast<cuuint32_t>(kTileRows)};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = Encoder()(&map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(p->q), dims, strides, box, estr,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return Stick(ctx, Fail(B200_INTERNAL, "b200_qmm: cuTensorMapEncodeTiled refused the weight matrix"));

  static std::mutex mu;
  static size_t attr_set[64] = {0};   // per device: the largest dynamic shared memory size configured so far
  {
    std::lock_guard<std::mutex> lock(mu);
    const int dev = ctx->device & 63;
    if (attr_set[dev] < smem) {
      cudaError_t e = cudaFuncSetAttribute(qmm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(ctx->max_smem_optin));
      if (e != cudaSuccess) return Stick(ctx, Fail(B200_INTERNAL, "b200_qmm: shared memory attribute: %s", cudaGetErrorString(e)));
      attr_set[dev] = static_cast<size_t>(ctx->max_smem_optin);
    }
  }
  LaunchCfg lc;
  lc.grid = dim3(static_cast<unsigned>(ctas));
  lc.block = dim3(kThreads);
  lc.smem = smem;
  lc.stream = stream;
  lc.pdl = true;
  cudaError_t e = Launch(lc, qmm_tc_kernel, map, a);
  if (e != cudaSuccess) return Stick(ctx, Fail(B200_INTERNAL, "b200_qmm (tensor-core route) launch: %s", cudaGetErrorString(e)));
  return EndLaunch(ctx, "b200_qmm");
}

}  // namespace b200
