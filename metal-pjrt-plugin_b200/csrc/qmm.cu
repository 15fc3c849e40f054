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
//   * sixteen consumer warps own fixed sets of 64-input groups: nibbles / bytes
//     are widened to bf16 in registers (one lop3 per two nibbles, 128 + q with
//     the 128 folded into the offset term) and fed to mma.sync m16n8k16 with the
//     batch as the 8-wide operand; the inputs of x are pre-permuted in shared
//     memory to match the register order, so no shuffles are needed; per-group
//     scale/offset are applied in f32;
//   * the warps' partial tiles are added by rotating epilogue threads; a K split
//     across CTAs goes through a thread-block cluster's distributed shared memory.
// More than 32 rows: qmm_many.cu (dequantised panels in L2 + the tensor-core GEMM).
// An alternative route for up to 8 rows on tcgen05: qmm_tc.cu (on request; slower, and why).
// Tensor-parallel decoders: the `TP` builds of the kernel take part in the push exchange of
// partial sums (tp.cuh); their slow paths are out of line, because these kernels pay about a
// microsecond per launch for every 30-40 KB of code.
#include <cooperative_groups.h>

#include <algorithm>
#include <cstdlib>
#include <map>
#include <utility>

#include "qmm_many.cuh"
#include "qmm_tc.cuh"
#include "tp.cuh"

namespace cg = cooperative_groups;
using namespace b200;

namespace {

constexpr int kConsumerWarps = 16;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kThreads = kConsumerThreads + 32;  // + one producer warp
constexpr int kCopyBytes = 2048;                 // bytes of one weight row per bulk copy (RT = 1)
constexpr int kGroupK = 64;

enum Format { kInt4Seq = 0, kInt4Half = 1, kInt8 = 2, kBf16 = 3 };

template <int FMT>
struct Fmt {
  static constexpr int kBits = FMT == kInt8 ? 8 : (FMT == kBf16 ? 16 : 4);
  static constexpr int kPad = kBits == 4 ? 32 : 64;           // keeps the quad reads conflict-free
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
  int scale_vec;               // scale / offset rows allow 16-byte loads of eight groups
  int tiles;                   // row tiles in all (ceil(N / (16 RT)))
  float eps;
  const __nv_bfloat16* gain;   // RMSNorm gain [K]
  // tensor-parallel exchange (tp_world == 0: none), see b200::QmmTp
  int tp_world, tp_rank;
  uint2* tp_dst[kTpMaxWorld];            // epilogue kEpiloguePush: slot 0 of this rank's sub-slot on every rank
  uint32_t* tp_count;                    // exchanges this rank has pushed (device memory)
  uint32_t* tp_done;                     // CTAs of the pushing kernel that have finished
  const uint2* tp_src;                   // pusher: slot 0 of the ranks' lines in this rank's memory, [world][cap]
  long long tp_cap;                      // floats per sub-slot; a slot is world sub-slots
  int tp_nowait;                         // measurement only, wrong results: bits of B200_TP_NOWAIT: 1 take the lines as they are (no
                                         // waiting), 2 do not read the ranks' lines at all, 4 (pusher) store to this rank's own memory
                                         // only, 8 (pusher) no exchange count at the end, 16 (pusher) plain instead of volatile stores
  __nv_bfloat16* x_out;                  // pusher: where the new residual rows go
  const __nv_bfloat16* tp_x_old;         // pusher: the residual rows the sum over ranks is added to, [M, N]
  uint2* tp_bcast;                       // slot 0 of this rank's lines {two bf16 of the new residual row, exchange number}
};

constexpr int kEpilogueGemm = 100;
constexpr int kEpiloguePush = 101;   // f32 partial sums stored into every rank's exchange block

// The exchange moves 8-byte lines {f32 partial sum, exchange number}: one store carries the value
// and says which exchange it belongs to, so the reader needs no flag of its own, no fence and no
// "last CTA" on the writer's side; it just reads the line again until the number is the one it wants.
__device__ __forceinline__ void st_line(uint2* p, float v, uint32_t n) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(__float_as_uint(v)), "r"(n) : "memory");
}
__device__ __forceinline__ uint4 ld_lines2(const uint2* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
// The slow path of every wait on lines, out of line (the kernels are sensitive to their code size):
// spins, bounded, until the `quads` 16-byte pairs of lines at p (and at p + pitch, ... for `ranks`
// sub-slots) all carry exchange n.  Once any wait of this context has run out (the status word is
// set) nobody waits again.
__device__ __noinline__ void tp_wait_lines(const uint2* p, size_t pitch, int ranks, int quads, uint32_t n, int* status, int where) {
  const long long t0 = clock64();
  for (;;) {
    int late = -1;
    for (int r = ranks - 1; r >= 0; --r)
      for (int j = 0; j < quads; ++j) {
        const uint4 v = ld_lines2(p + r * pitch + 2 * j);
        if (v.y != n || v.w != n) late = r;
      }
    if (late < 0) return;
    if (*reinterpret_cast<volatile int*>(status) != 0) return;
    if (clock64() - t0 > 4000000000ll) {
      report_timeout(status, where + late);   // the first rank whose lines are missing
      return;
    }
  }
}

// Eight consecutive lines of exchange n from each of R ranks' sub-slots (p 16-byte aligned, `pitch`
// lines between sub-slots), added to sum[] in rank order.  All R x 4 loads are in flight together
// (one trip to L2 for R ranks); lines that have not landed yet are waited for out of line, and
// count as zero if that wait gives up.
template <int R>
__device__ __forceinline__ void add_lines8(const uint2* p, size_t pitch, uint32_t n, int* status, int where, float (&sum)[8],
                                           bool nowait) {
  uint4 v[R][4];
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int j = 0; j < 4; ++j) v[r][j] = ld_lines2(p + r * pitch + 2 * j);
  bool ok = true;
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int j = 0; j < 4; ++j) ok = ok && v[r][j].y == n && v[r][j].w == n;
  if (!ok && !nowait) {
    tp_wait_lines(p, pitch, R, 4, n, status, where);
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int j = 0; j < 4; ++j) v[r][j] = ld_lines2(p + r * pitch + 2 * j);
  }
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const bool have = (v[r][j].y == n && v[r][j].w == n) || nowait;
      sum[2 * j] += have ? __uint_as_float(v[r][j].x) : 0.0f;
      sum[2 * j + 1] += have ? __uint_as_float(v[r][j].z) : 0.0f;
    }
}

// One partial sum into sub-slot `rank` of every rank's block (out of line: seven call sites).
__device__ __noinline__ void tp_push_value(uint2* const* dst, int world, int rank, int mode, size_t idx, float v, uint32_t n) {
  for (int r = 0; r < world; ++r) {
    if ((mode & 4) && r != rank) continue;
    if (mode & 16) dst[r][idx] = make_uint2(__float_as_uint(v), n);
    else st_line(dst[r] + idx, v, n);
  }
}

// The first level of the sum over ranks, by the CTAs of the consuming projection together: the rows
// are cut into runs of 8 values dealt out over the CTAs (8 consecutive runs per CTA and step, so a
// quarter warp reads 512 contiguous bytes per rank); the owner of a run adds the ranks' lines in
// rank order (identical sums on every rank) and the old residual, writes the new residual row, and
// publishes the 8 bf16 values as four {two values, exchange number} lines in this rank's memory.
__device__ __noinline__ void tp_reduce_publish(const uint2* slot, size_t pitch, int world, uint32_t n, int* status, int mode,
                                               const __nv_bfloat16* x, int ldx, int M, int K, __nv_bfloat16* x_out, uint2* bc,
                                               int cta_id, int n_ctas, int tid, int threads) {
  const int runs = M * (K / 8);
  for (int run = cta_id * 8 + (tid & 7) + (tid >> 3) * n_ctas * 8; run < runs; run += (threads / 8) * n_ctas * 8) {
    const int m = run / (K / 8), k = (run % (K / 8)) * 8;
    float sum[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
    const uint2* base = slot + static_cast<size_t>(m) * K + k;
    int r = (mode & 2) ? world : 0;
    for (; r + 2 <= world; r += 2) add_lines8<2>(base + r * pitch, pitch, n, status, 400 + r, sum, (mode & 1) != 0);
    if (r < world) add_lines8<1>(base + r * pitch, pitch, n, status, 400 + r, sum, (mode & 1) != 0);
    const uint4 raw = __ldg(reinterpret_cast<const uint4*>(x + static_cast<size_t>(m) * ldx + k));
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) o[j] = pack_bf16(bf16_lo(w[j]) + bf16_round(sum[2 * j]), bf16_hi(w[j]) + bf16_round(sum[2 * j + 1]));
    if (x_out != nullptr) *reinterpret_cast<uint4*>(x_out + static_cast<size_t>(m) * K + k) = make_uint4(o[0], o[1], o[2], o[3]);
    uint2* dst = bc + (static_cast<size_t>(m) * K + k) / 2;
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "r"(o[0]), "r"(n), "r"(o[1]), "r"(n) : "memory");
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(dst + 2), "r"(o[2]), "r"(n), "r"(o[3]), "r"(n) : "memory");
  }
}

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

// v >> log2(2^32 / pow2).  (Written as a multiply-high by a power of two it would run on the FMA
// pipe, but that instruction measures 4-6 issue cycles per warp on this GPU against about one
// for a plain shift.)
__device__ __forceinline__ uint32_t mulhi_shift(uint32_t v, uint32_t pow2) { return v >> (__clz(pow2) + 1); }

// Widens one thread's share of a group (for one weight row) into 8 bf16x2 registers.
template <int FMT>
__device__ __forceinline__ void load_a(const uint8_t* row_group_ptr, int t, uint32_t (&a)[8]) {
  if (FMT == kInt4Seq || FMT == kInt4Half) {
    const uint2 w = *reinterpret_cast<const uint2*>(row_group_ptr + 8 * t);
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      // the right shifts are multiply-high by a power of two: that instruction runs on the
      // FMA pipe, which leaves the (half-rate) integer pipe to the lop3s
      a[r] = lop3_and_or(r == 0 ? w.x : mulhi_shift(w.x, 1u << (32 - 4 * r)), 0x000f000fu, 0x43004300u);  // bf16 (128 + q)
      a[4 + r] = lop3_and_or(r == 0 ? w.y : mulhi_shift(w.y, 1u << (32 - 4 * r)), 0x000f000fu, 0x43004300u);
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

__device__ __forceinline__ uint2 lds64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ float2 lds64f(uint32_t addr) {
  float2 v;
  asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(addr));
  return v;
}

// Same as load_a, from a 32-bit shared-memory address that already includes the thread's
// offset (the unrolled path keeps these offsets in registers instead of re-deriving them).
template <int FMT>
__device__ __forceinline__ void load_a32(uint32_t addr, uint32_t (&a)[8]) {
  if (FMT == kInt4Seq || FMT == kInt4Half) {
    const uint2 w = lds64(addr);
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      a[r] = lop3_and_or(r == 0 ? w.x : mulhi_shift(w.x, 1u << (32 - 4 * r)), 0x000f000fu, 0x43004300u);
      a[4 + r] = lop3_and_or(r == 0 ? w.y : mulhi_shift(w.y, 1u << (32 - 4 * r)), 0x000f000fu, 0x43004300u);
    }
  } else if (FMT == kInt8) {
    const uint4 w = lds128(addr);
    const uint32_t words[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t u = words[j] ^ 0x80808080u;
      const float f0 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7650)) - 8388736.0f;
      const float f1 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7651)) - 8388736.0f;
      const float f2 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7652)) - 8388736.0f;
      const float f3 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7653)) - 8388736.0f;
      a[2 * j] = pack_bf16(f0, f1);
      a[2 * j + 1] = pack_bf16(f2, f3);
    }
  } else {
    const uint4 w0 = lds128(addr);
    const uint4 w1 = lds128(addr + 64);
    a[0] = w0.x; a[1] = w0.y; a[2] = w0.z; a[3] = w0.w;
    a[4] = w1.x; a[5] = w1.y; a[6] = w1.z; a[7] = w1.w;
  }
}

__device__ __forceinline__ void consumer_barrier() {
  asm volatile("bar.sync 1, %0;" ::"n"(kConsumerThreads) : "memory");
}

// One output element: the per-channel scale (if any), then the epilogue.
template <int FMT, bool GROUPED, bool TP = false>
__device__ __forceinline__ void store_output(const QmmArgs& a, float v, int m, int n) {
  if (!GROUPED && Fmt<FMT>::kBits != 16) v *= ldg_bf16(a.scale + n);
  if (FMT == kBf16 && a.epilogue == kEpilogueGemm) {   // b200_gemm's few-row route: 16-bit weights only
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
    return;
  }
  const float y = bf16_round(v);
  const size_t o = static_cast<size_t>(m) * a.ldo + n;
  if (TP && a.epilogue == kEpiloguePush) {
    // one line per value into every rank's memory (its own included); the slot alternates with the exchange number
    const uint32_t n_x = *a.tp_count + 1u;
    tp_push_value(a.tp_dst, a.tp_world, a.tp_rank, a.tp_nowait, static_cast<size_t>(n_x & 1u) * a.tp_world * a.tp_cap + o, v, n_x);
    return;
  }
  if (a.epilogue == B200_QMM_OUT_F32_RAW) {
    reinterpret_cast<float*>(a.out)[o] = v;
  } else if (a.epilogue == B200_QMM_OUT_F32) {
    reinterpret_cast<float*>(a.out)[o] = y;
  } else if (a.epilogue == B200_QMM_ADD_RESIDUAL) {
    reinterpret_cast<__nv_bfloat16*>(a.out)[o] = __float2bfloat16_rn(__bfloat162float(a.residual[o]) + y);
  } else {
    reinterpret_cast<__nv_bfloat16*>(a.out)[o] = __float2bfloat16_rn(v);
  }
}

// FMT: storage format; MB: batch blocks of 8; RT: 16-row tiles per CTA tile;
// GROUPED: a scale (and offset) per 64 inputs, else one scale per row applied at the end.
//
// grid = (CTAs or clusters, split).  CTAs are persistent: a CTA walks row tiles
// blockIdx.x, blockIdx.x + gridDim.x, ... and stages its slice of x (and fused
// transforms) once.  With split > 1 the `split` CTAs of a cluster take the K
// slices of the same tiles; after every tile they meet on an mbarrier in each
// other's shared memory and each finishes a share of the rows from all the
// slices' partial tiles, read through distributed shared memory.
// KG > 0: the CTA's K slice is exactly KG groups (and MB == 1): every warp owns
// a compile-time set of KG / 16 groups, keeps their x fragments in registers for
// all row tiles, and its loop over them is fully unrolled.  KG == 0: any K.
// LEAN: launched only without a K split and with 16-byte-loadable x, gain, scales and offsets, so
// none of the code for the other cases is compiled in (the unrolled variants, KG > 0, are always lean).
// VEC: the 16-byte-load assumption alone, for the builds that do split K (LEAN implies it).
// TP: the build that takes part in the tensor-parallel exchange (sums the ranks' partial sums while it
// stages x, or pushes its own from the epilogue); the others carry none of that code.
template <int FMT, int MB, int RT, bool GROUPED, int KG, bool LEAN = (KG > 0), bool VEC = LEAN, bool TP = false>
__global__ void __launch_bounds__(kThreads, 1) qgemv_kernel(const __grid_constant__ QmmArgs a) {
  static_assert(KG == 0 || LEAN, "the unrolled variants are lean");
  static_assert(!LEAN || VEC, "lean implies 16-byte loads");
  using F = Fmt<FMT>;
  constexpr int R = 16 * RT;
  constexpr int MP = 8 * MB;
  // Row pitch of the tiles that are added into atomically: above one batch block, four words
  // more than the batch width, so that the eight rows a warp adds into fall in different banks.
  constexpr int RP = MB > 1 ? MP + 4 : MP;
  // One pipeline stage holds R rows x kChunkK inputs; a row's share arrives as ONE
  // bulk copy (small copies are bound by the copy engine's request rate, not by HBM).
  constexpr int kChunkRowBytes = MB == 1 ? kCopyBytes : kCopyBytes / RT;
  constexpr int kChunkK = kChunkRowBytes * 8 / F::kBits;
  constexpr int kRowStride = kChunkRowBytes + F::kPad;
  constexpr int kStageBytes = R * kRowStride;
  extern __shared__ __align__(128) uint8_t smem[];

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int split = gridDim.y;   // CTAs of one cluster along K; every CTA walks tiles blockIdx.x, + gridDim.x, ...
  // The unrolled variants (KG > 0) are only launched without a K split, so they carry none of
  // the cluster code (and none of its registers).
  const bool solo = LEAN || split == 1;
  // ... and are only launched with 16-byte-loadable x / scales and without the silu prologue.
  const bool x_vec = VEC || a.x_vec != 0;
  const bool scale_vec = VEC || a.scale_vec != 0;
  const int k_begin = blockIdx.y * a.k_per_cta;
  const int groups_cta = a.k_per_cta / kGroupK;
  const int n_chunks = (a.k_per_cta + kChunkK - 1) / kChunkK;
  const int NS = a.stages;
  const size_t row_bytes_total = static_cast<size_t>(a.K) * F::kBits / 8;
  const int n_my = (a.tiles - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x);
  const int n_units = n_my * n_chunks;

  // ---- shared memory carve-up -------------------------------------------------
  uint64_t* full = reinterpret_cast<uint64_t*>(smem);
  uint64_t* empty = full + NS;
  size_t off = (static_cast<size_t>(2 * NS) * 8 + 127) & ~static_cast<size_t>(127);
  // Cross-warp reduction buffer.  Small tiles (one MMA row tile, batch <= 8) without a
  // split of K: every warp stores its partial tile, [2][warps][R][MP], and the
  // epilogue threads add the 16 partials.  Otherwise: [2][R][MP] added into atomically; with
  // K split across a cluster [4][R][MP], the tiles the peers read through distributed shared memory.
  constexpr bool kPartials = MB == 1;
  const bool partials = kPartials && solo;
  float* red = reinterpret_cast<float*>(smem + off);
  off += static_cast<size_t>(kPartials ? 2 * kConsumerWarps * MP : 4 * RP) * R * 4;
  float* xsum = reinterpret_cast<float*>(smem + off);                // [groups_cta][MP]
  off += (static_cast<size_t>(groups_cta) * MP * 4 + 127) & ~static_cast<size_t>(127);
  uint4* xs = reinterpret_cast<uint4*>(smem + off);                  // [groups_cta][2][M][4] x 16 B
  off += (static_cast<size_t>(groups_cta) * a.M * 128 + 127) & ~static_cast<size_t>(127);
  float2* so = reinterpret_cast<float2*>(smem + off);                // [2][groups_cta][R] (scale, offset)
  const int so_buf = groups_cta * R;
  if (GROUPED) off += (static_cast<size_t>(2) * so_buf * 8 + 127) & ~static_cast<size_t>(127);
  uint8_t* stage_base = smem + off;
  __shared__ float ss_part[kConsumerWarps][8];
  __shared__ float rinv[8];
  __shared__ __align__(8) uint64_t tile_bar[4];   // K split: "every CTA of the cluster has finished tile ti" (ti mod 4)

  if (tid == 0) {
    for (int s = 0; s < NS; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], kConsumerWarps);
    }
    for (int i = 0; i < 4; ++i) mbar_init(&tile_bar[i], split);
    mbar_fence_init();
  }
  if (!partials)
    for (int i = tid; i < (solo ? 2 : 4) * R * RP; i += kThreads) red[i] = 0.0f;
  for (int i = tid; i < groups_cta * MP; i += kThreads) xsum[i] = 0.0f;
  __syncthreads();
  if (!solo) cg::this_cluster().sync();   // the peers' barriers exist before anyone arrives on them

  bool dead = false;  // a bounded wait gave up: skip the work, keep every barrier

  if (warp == kConsumerWarps) {
    // ---------------- producer warp: weights only, independent of earlier kernels
    const int first_fill = min(n_units, NS);
    for (int u = 0; u < n_units; ++u) {
      const int ti = u / n_chunks, c = u - ti * n_chunks;
      const int n0 = (static_cast<int>(blockIdx.x) + ti * static_cast<int>(gridDim.x)) * R;
      const int rows_valid = min(R, a.N - n0);
      const int s = u % NS, use = u / NS;
      if (!dead && use > 0 && !mbar_wait_bounded<128>(&empty[s], (use - 1) & 1)) {
        report_timeout(a.status, 100 + s);
        dead = true;
      }
      if (!dead) {
        const int chunk_k = min(kChunkK, a.k_per_cta - c * kChunkK);
        const uint32_t bytes_row = static_cast<uint32_t>(chunk_k * F::kBits / 8);
        if (lane == 0) mbar_expect_tx(&full[s], bytes_row * rows_valid);
        __syncwarp();
        uint8_t* dst = stage_base + static_cast<size_t>(s) * kStageBytes;
        const uint8_t* src = a.q + static_cast<size_t>(n0) * row_bytes_total +
                             (static_cast<size_t>(k_begin) + static_cast<size_t>(c) * kChunkK) * F::kBits / 8;
        for (int r = lane; r < rows_valid; r += 32)
          bulk_g2s(dst + r * kRowStride, src + static_cast<size_t>(r) * row_bytes_total, bytes_row, &full[s]);
      }
      if (u == first_fill - 1 && lane == 0) pdl_launch_dependents();
    }
  } else {
    // ---------------- consumer warps
    // Scales and offsets belong to the weights, so the first tile's are fetched
    // before waiting on the previous kernel; a later tile's are fetched into
    // registers while the tile before it is computed.  Stored packed (scale,
    // offset) as [group][row].
    const int g0 = k_begin / kGroupK;
    const int nch = R * (groups_cta / 8);
    uint4 sreg = make_uint4(0, 0, 0, 0), breg = make_uint4(0, 0, 0, 0);
    auto scale_load = [&](int n0) {
      if (GROUPED && scale_vec && tid < nch) {
        const int c = tid / R, r = tid - c * R;
        const size_t o = static_cast<size_t>(min(n0 + r, a.N - 1)) * a.scale_ld + g0 + 8 * c;
        sreg = __ldg(reinterpret_cast<const uint4*>(a.scale + o));
        if (F::kBits == 4) breg = __ldg(reinterpret_cast<const uint4*>(a.bias + o));
      }
    };
    // int4 registers hold 128 + q: the 128 is folded into the offset here
    auto put8 = [&](float2* dstbuf, int c, int r, const uint4& sv, const uint4& bv) {
      const uint32_t sw[4] = {sv.x, sv.y, sv.z, sv.w};
      const uint32_t bw[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float sc = (j & 1) ? bf16_hi(sw[j >> 1]) : bf16_lo(sw[j >> 1]);
        const float bi = (j & 1) ? bf16_hi(bw[j >> 1]) : bf16_lo(bw[j >> 1]);
        dstbuf[(8 * c + j) * R + r] = make_float2(sc, F::kBits == 4 ? fmaf(-128.0f, sc, bi) : 0.0f);
      }
    };
    auto scale_store = [&](int n0, float2* dstbuf) {
      if (!GROUPED) return;
      if (scale_vec) {
        if (tid < nch) put8(dstbuf, tid / R, tid % R, sreg, breg);
        for (int idx = tid + kConsumerThreads; idx < nch; idx += kConsumerThreads) {   // rarely taken
          const int c = idx / R, r = idx - c * R;
          const size_t o = static_cast<size_t>(min(n0 + r, a.N - 1)) * a.scale_ld + g0 + 8 * c;
          const uint4 sv = __ldg(reinterpret_cast<const uint4*>(a.scale + o));
          const uint4 bv = F::kBits == 4 ? __ldg(reinterpret_cast<const uint4*>(a.bias + o)) : make_uint4(0, 0, 0, 0);
          put8(dstbuf, c, r, sv, bv);
        }
      } else {
        for (int i = tid; i < R * groups_cta; i += kConsumerThreads) {
          const int r = i / groups_cta, gi = i - r * groups_cta;
          // rows past N are clamped for the load; their results are never stored
          const size_t o = static_cast<size_t>(min(n0 + r, a.N - 1)) * a.scale_ld + g0 + gi;
          const float sc = ldg_bf16(a.scale + o);
          dstbuf[gi * R + r] = make_float2(sc, F::kBits == 4 ? fmaf(-128.0f, sc, ldg_bf16(a.bias + o)) : 0.0f);
        }
      }
    };
    scale_load(static_cast<int>(blockIdx.x) * R);
    scale_store(static_cast<int>(blockIdx.x) * R, so);
    pdl_wait();  // x (and the residual) come from the previous kernel
    // Tensor parallel: x is the new residual row, bf16(old + bf16(sum over ranks of the partial sums of
    // the K-sharded projection before this one)), which the CTAs of that projection formed at their
    // end and published as {two values, exchange number} lines in this rank's memory.  That kernel
    // has finished on this rank (the wait above), so the exchange number is final and the lines are
    // there; the bounded wait behind the first read only ever runs in the measurement modes.
    const uint2* tp_bc = nullptr;
    uint32_t tp_n = 0;
    if (TP && a.tp_bcast != nullptr && a.epilogue != kEpiloguePush) {
      tp_n = *a.tp_count;
      tp_bc = a.tp_bcast + static_cast<size_t>(tp_n & 1u) * (a.tp_cap / 2);
    }
    // eight values of row m starting at k: of x, or of the new residual row as this rank published it
    auto load_x8 = [&](int m, int k, float* dst) {
      uint32_t w[4];
      if (TP && tp_bc != nullptr) {
        const uint2* src = tp_bc + (static_cast<size_t>(m) * a.K + k) / 2;
        uint4 v0 = ld_lines2(src), v1 = ld_lines2(src + 2);
        if (!(v0.y == tp_n && v0.w == tp_n && v1.y == tp_n && v1.w == tp_n) && !(a.tp_nowait & 1)) {
          tp_wait_lines(src, 0, 1, 2, tp_n, a.status, 450);
          v0 = ld_lines2(src);
          v1 = ld_lines2(src + 2);
        }
        w[0] = v0.x; w[1] = v0.z; w[2] = v1.x; w[3] = v1.z;
      } else {
        const uint4 raw = __ldg(reinterpret_cast<const uint4*>(a.x + static_cast<size_t>(m) * a.ldx + k));
        w[0] = raw.x; w[1] = raw.y; w[2] = raw.z; w[3] = raw.w;
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        dst[2 * j] = bf16_lo(w[j]);
        dst[2 * j + 1] = bf16_hi(w[j]);
      }
    };
    // RMSNorm in one pass: when every thread stages at most one 16-input unit of a whole row
    // (M * K <= 8192) and warps do not straddle rows, the sum of squares comes from the
    // values the threads hold for staging anyway (one trip to L2, one barrier).
    const int units_all = a.M * groups_cta * 4;
    const bool rms_one_pass = a.prologue == B200_QMM_PRO_RMSNORM && solo && units_all <= kConsumerThreads &&
                              (groups_cta * 4) % 32 == 0;
    if (a.prologue == B200_QMM_PRO_RMSNORM && !rms_one_pass) {
      // 1 / rms of every full row of x (M <= 8), recomputed by each CTA
      float ss[8];
#pragma unroll
      for (int m = 0; m < 8; ++m) {
        ss[m] = 0.0f;
        if (m < a.M) {
          const __nv_bfloat16* xr = a.x + static_cast<size_t>(m) * a.ldx;
          if (TP && x_vec && tp_bc != nullptr) {
            for (int i = tid * 8; i < a.K; i += kConsumerThreads * 8) {
              float e8[8];
              load_x8(m, i, e8);
#pragma unroll
              for (int j = 0; j < 8; ++j) ss[m] = fmaf(e8[j], e8[j], ss[m]);
            }
          } else if (x_vec) {
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
      const int units = units_all;
      // one pass: every consumer thread runs the body exactly once (it holds a barrier)
      const int units_pad = rms_one_pass ? kConsumerThreads : (units + 31) & ~31;
      constexpr bool kOneRun = FMT == kInt4Seq || FMT == kInt8;
      for (int u = tid; u < units_pad; u += kConsumerThreads) {
        const bool valid = u < units;
        const int ut = u & 3;
        const int ug = (u >> 2) % groups_cta;
        const int um = (u >> 2) / groups_cta;
        float sum = 0.0f;
        float e[16], gn[16];
        const int kbase = k_begin + ug * kGroupK;
        const int run0 = kOneRun ? 16 * ut : 8 * ut;
        const int run1 = kOneRun ? 16 * ut + 8 : 32 + 8 * ut;
        auto load_run = [&](const __nv_bfloat16* base, int k, float* dst) {
            if (x_vec) {
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
        const __nv_bfloat16* xr = a.x + static_cast<size_t>(valid ? um : 0) * a.ldx;
        if (TP && valid && tp_bc != nullptr) {
          load_x8(um, kbase + run0, e);
          load_x8(um, kbase + run1, e + 8);
          load_run(a.gain, kbase + run0, gn);
          load_run(a.gain, kbase + run1, gn + 8);
        } else if (valid) {
          load_run(xr, kbase + run0, e);
          load_run(xr, kbase + run1, e + 8);
          if (a.prologue == B200_QMM_PRO_RMSNORM) {
            load_run(a.gain, kbase + run0, gn);
            load_run(a.gain, kbase + run1, gn + 8);
          }
        }
        if (rms_one_pass) {
          float ss = 0.0f;
          if (valid) {
#pragma unroll
            for (int j = 0; j < 16; ++j) ss = fmaf(e[j], e[j], ss);
          }
          ss = warp_sum(ss);
          if (lane == 0) ss_part[warp][0] = ss;
          consumer_barrier();
          if (valid) {
            const int wpr = groups_cta * 4 / 32;   // warps per row of x
            float tsum = 0.0f;
            for (int w = um * wpr; w < (um + 1) * wpr; ++w) tsum += ss_part[w][0];
            const float rr = 1.0f / sqrtf(tsum / static_cast<float>(a.K) + a.eps);
#pragma unroll
            for (int j = 0; j < 16; ++j) e[j] = bf16_round((e[j] * rr) * gn[j]);
          }
        }
        if (valid) {
          if (a.prologue == B200_QMM_PRO_RMSNORM && !rms_one_pass) {
            const float rr = rinv[um];
#pragma unroll
            for (int j = 0; j < 16; ++j) e[j] = bf16_round((e[j] * rr) * gn[j]);
          } else if (KG == 0 && a.prologue == B200_QMM_PRO_SILU_MUL) {
            // x is [M, 2K]: gate in the first K columns, up in the last K
            float up[16];
            load_run(xr + a.K, kbase + run0, up);
            load_run(xr + a.K, kbase + run1, up + 8);
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              // hardware exp2 / reciprocal: their error (~1e-6 relative) sits far below the bf16
              // rounding that follows, and the accurate forms cost 3 us per launch here
              const float sig = bf16_round(__fdividef(1.0f, 1.0f + __expf(-e[j])));
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

    // Batches above 8 (MB > 1): the 16 warps split the tile's RT row tiles as well as K
    // (warp w takes row tile w % RT and every (16 / RT)-th group), so a warp keeps one row
    // tile of accumulators and adds it into the shared tile once per 16 / RT groups' worth
    // of work.  Up to 8: every warp covers all RT row tiles of its groups.
    constexpr int kRowSplit = MB > 1 ? RT : 1;    // warps along the rows of a tile
    constexpr int RTW = RT / kRowSplit;           // row tiles per warp
    const int row_base = (warp % kRowSplit) * 16;
    float acc[RTW][MB][4];
#pragma unroll
    for (int rt = 0; rt < RTW; ++rt)
#pragma unroll
      for (int mb = 0; mb < MB; ++mb)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[rt][mb][i] = 0.0f;

    // x fragments (and per-group sums of x) of one group for this lane
    auto load_x = [&](int gl, uint32_t (&xf)[MB][8], float (&xs2)[MB][2]) {
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
        xs2[mb][0] = xs2[mb][1] = 0.0f;
        if (F::kBits == 4) {
          const float2 v = *reinterpret_cast<const float2*>(&xsum[gl * MP + mb * 8 + 2 * t]);
          xs2[mb][0] = v.x;
          xs2[mb][1] = v.y;
        }
      }
    };
    // one group (64 inputs) of every row tile: widen, multiply, scale, accumulate
    auto do_group = [&](const uint8_t* stage_group, const float2* so_group, const uint32_t (&xf)[MB][8],
                        const float (&xs2)[MB][2]) {
#pragma unroll
      for (int rt = 0; rt < RTW; ++rt) {
        const int r0 = row_base + rt * 16 + g, r1 = r0 + 8;
        uint32_t a0[8], a1[8];
        load_a<FMT>(stage_group + r0 * kRowStride, t, a0);
        load_a<FMT>(stage_group + r1 * kRowStride, t, a1);
        if (GROUPED) {
          const float2 p0 = so_group[r0], p1 = so_group[r1];
#pragma unroll
          for (int mb = 0; mb < MB; ++mb) {
            float tmp[4];
            mma_bf16_16816_z(tmp, a0[0], a1[0], a0[1], a1[1], xf[mb][0], xf[mb][1]);
#pragma unroll
            for (int i = 1; i < 4; ++i)
              mma_bf16_16816(tmp, a0[2 * i], a1[2 * i], a0[2 * i + 1], a1[2 * i + 1], xf[mb][2 * i], xf[mb][2 * i + 1]);
            if (F::kBits == 4) {
              acc[rt][mb][0] = fmaf(p0.x, tmp[0], fmaf(p0.y, xs2[mb][0], acc[rt][mb][0]));
              acc[rt][mb][1] = fmaf(p0.x, tmp[1], fmaf(p0.y, xs2[mb][1], acc[rt][mb][1]));
              acc[rt][mb][2] = fmaf(p1.x, tmp[2], fmaf(p1.y, xs2[mb][0], acc[rt][mb][2]));
              acc[rt][mb][3] = fmaf(p1.x, tmp[3], fmaf(p1.y, xs2[mb][1], acc[rt][mb][3]));
            } else {
              acc[rt][mb][0] = fmaf(p0.x, tmp[0], acc[rt][mb][0]);
              acc[rt][mb][1] = fmaf(p0.x, tmp[1], acc[rt][mb][1]);
              acc[rt][mb][2] = fmaf(p1.x, tmp[2], acc[rt][mb][2]);
              acc[rt][mb][3] = fmaf(p1.x, tmp[3], acc[rt][mb][3]);
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
    };

    // the same step from 32-bit shared addresses (thread offsets already added)
    auto do_group32 = [&](uint32_t a_addr, uint32_t so_addr, const uint32_t (&xf)[MB][8], const float (&xs2)[MB][2]) {
#pragma unroll
      for (int rt = 0; rt < RTW; ++rt) {
        uint32_t a0[8], a1[8];
        load_a32<FMT>(a_addr + rt * 16 * kRowStride, a0);
        load_a32<FMT>(a_addr + (rt * 16 + 8) * kRowStride, a1);
        if (GROUPED) {
          const float2 p0 = lds64f(so_addr + rt * 16 * 8), p1 = lds64f(so_addr + (rt * 16 + 8) * 8);
#pragma unroll
          for (int mb = 0; mb < MB; ++mb) {
            float tmp[4];
            mma_bf16_16816_z(tmp, a0[0], a1[0], a0[1], a1[1], xf[mb][0], xf[mb][1]);
#pragma unroll
            for (int i = 1; i < 4; ++i)
              mma_bf16_16816(tmp, a0[2 * i], a1[2 * i], a0[2 * i + 1], a1[2 * i + 1], xf[mb][2 * i], xf[mb][2 * i + 1]);
            if (F::kBits == 4) {
              acc[rt][mb][0] = fmaf(p0.x, tmp[0], fmaf(p0.y, xs2[mb][0], acc[rt][mb][0]));
              acc[rt][mb][1] = fmaf(p0.x, tmp[1], fmaf(p0.y, xs2[mb][1], acc[rt][mb][1]));
              acc[rt][mb][2] = fmaf(p1.x, tmp[2], fmaf(p1.y, xs2[mb][0], acc[rt][mb][2]));
              acc[rt][mb][3] = fmaf(p1.x, tmp[3], fmaf(p1.y, xs2[mb][1], acc[rt][mb][3]));
            } else {
              acc[rt][mb][0] = fmaf(p0.x, tmp[0], acc[rt][mb][0]);
              acc[rt][mb][1] = fmaf(p0.x, tmp[1], acc[rt][mb][1]);
              acc[rt][mb][2] = fmaf(p1.x, tmp[2], acc[rt][mb][2]);
              acc[rt][mb][3] = fmaf(p1.x, tmp[3], acc[rt][mb][3]);
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
    };

    constexpr int GC = kChunkK / kGroupK;                       // groups per chunk
    constexpr int GPW = KG > 0 ? KG / kConsumerWarps : 1;       // groups per warp (fast path)
    uint32_t xr[GPW][MB][8];
    float xq[GPW][MB][2];
    uint32_t a_off[GPW], so_off[GPW];   // this thread's byte offsets inside a stage / a scale buffer
    const uint32_t stage0 = smem_u32(stage_base), so0 = smem_u32(so);
    if (KG > 0) {
#pragma unroll
      for (int j = 0; j < GPW; ++j) {
        load_x(warp + kConsumerWarps * j, xr[j], xq[j]);
        const int gs = warp + (kConsumerWarps * j) % GC;
        a_off[j] = static_cast<uint32_t>(gs * F::kGroupBytes + g * kRowStride + t * (F::kBits == 4 ? 8 : 16));
        so_off[j] = static_cast<uint32_t>(((warp + kConsumerWarps * j) * R + g) * 8);
      }
    }

    // K split across the cluster (consumer threads only).  Tile ti of every CTA lands in buffer
    // ti mod 4 of its own shared memory.  After its adds (and a consumer_barrier, which orders
    // them before thread 0's release-arrivals) a CTA arrives on barrier ti mod 4 of every peer;
    // it finishes its share of tile ti's rows from all peers' buffers one tile LATER, when the
    // peers' arrivals are long there, so nobody waits for the slowest CTA tile by tile.
    auto cluster_arrive = [&](int ti) {
      if (tid == 0)
        for (int c = 0; c < split; ++c) mbar_arrive_cluster(&tile_bar[ti & 3], static_cast<uint32_t>(c));
    };
    auto cluster_wait = [&](int ti) {
      if (!dead && !mbar_wait_bounded_cluster(&tile_bar[ti & 3], static_cast<uint32_t>(ti >> 2) & 1u)) {
        report_timeout(a.status, 300 + (ti & 3));
        dead = true;
      }
    };
    auto cluster_finish = [&](int ti) {
      const int n0 = (static_cast<int>(blockIdx.x) + ti * static_cast<int>(gridDim.x)) * R;
      const int rows_valid = min(R, a.N - n0);
      const float* tile = red + (ti & 3) * R * RP;
      cluster_wait(ti);
      const int rows_per_rank = (R + split - 1) / split;
      const int r_begin = static_cast<int>(blockIdx.y) * rows_per_rank;
      const int r_count = min(min(r_begin + rows_per_rank, R), rows_valid) - r_begin;
      if (r_count <= 0 || dead) return;
      cg::cluster_group cluster = cg::this_cluster();
      // adjacent threads read adjacent words of the peers' tiles ([row][batch], batch fastest);
      // four batch columns per thread and read when the batch allows it
      if (a.M % 4 == 0 && a.M >= 16) {   // below 16 rows too few (row, 4-column) items to hide the latency
        const int mq = a.M / 4;
        for (int idx = tid; idx < r_count * mq; idx += kConsumerThreads) {
          const int r = r_begin + idx / mq, m = (idx % mq) * 4;
          float4 part[8];
#pragma unroll
          for (int c = 0; c < 8; ++c)
            part[c] = c < split ? *reinterpret_cast<const float4*>(cluster.map_shared_rank(tile, c) + r * RP + m)
                                : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
          float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            v.x += part[c].x;
            v.y += part[c].y;
            v.z += part[c].z;
            v.w += part[c].w;
          }
          store_output<FMT, GROUPED, TP>(a, v.x, m, n0 + r);
          store_output<FMT, GROUPED, TP>(a, v.y, m + 1, n0 + r);
          store_output<FMT, GROUPED, TP>(a, v.z, m + 2, n0 + r);
          store_output<FMT, GROUPED, TP>(a, v.w, m + 3, n0 + r);
        }
        return;
      }
      for (int idx = tid; idx < r_count * a.M; idx += kConsumerThreads) {
        const int r = r_begin + idx / a.M, m = idx % a.M;
        float part[8];
#pragma unroll
        for (int c = 0; c < 8; ++c)   // all the remote reads in flight together
          part[c] = c < split ? cluster.map_shared_rank(tile, c)[r * RP + m] : 0.0f;
        float v = 0.0f;
#pragma unroll
        for (int c = 0; c < 8; ++c) v += part[c];
        store_output<FMT, GROUPED, TP>(a, v, m, n0 + r);
      }
    };

    for (int ti = 0; ti < n_my; ++ti) {
      const int n0 = (static_cast<int>(blockIdx.x) + ti * static_cast<int>(gridDim.x)) * R;
      const int rows_valid = min(R, a.N - n0);
      const float2* so_cur = so + (ti & 1) * so_buf;
      float* red_cur = solo ? red + (ti & 1) * R * (partials ? kConsumerWarps * MP : RP) : red + (ti & 3) * R * RP;
      const bool has_next = ti + 1 < n_my;
      if (has_next) scale_load(n0 + static_cast<int>(gridDim.x) * R);

      if (KG > 0) {
        // compile-time schedule: group j of this warp is warp + 16 j, in chunk (16 j) / GC
        int s = 0;
#pragma unroll
        for (int j = 0; j < GPW; ++j) {
          const int c = (kConsumerWarps * j) / GC;
          const bool first = j == 0 || (kConsumerWarps * (j - 1)) / GC != c;
          const bool last = j == GPW - 1 || (kConsumerWarps * (j + 1)) / GC != c;
          if (first) {
            const int u = ti * n_chunks + c;
            s = u % NS;
            if (!dead && !mbar_wait_bounded(&full[s], (u / NS) & 1)) {
              report_timeout(a.status, 200 + s);
              dead = true;
            }
          }
          // (after a timed-out wait this multiplies stale shared memory; the result is discarded
          // with the reported error, and skipping the branch keeps the loop straight-line)
          do_group32(stage0 + static_cast<uint32_t>(s) * kStageBytes + a_off[j],
                     so0 + static_cast<uint32_t>((ti & 1) * so_buf * 8) + so_off[j], xr[j], xq[j]);
          if (last) {
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);
          }
        }
      } else if (LEAN && MB == 1 && GC % kConsumerWarps == 0) {
        // any K, lean build: the warp's GC / 16 groups of a chunk unrolled, from 32-bit shared
        // addresses; the x fragments come from shared memory (they do not fit registers for K = 12288)
        constexpr int JC = GC / kConsumerWarps;
        const uint32_t a_thr = static_cast<uint32_t>(warp * F::kGroupBytes + g * kRowStride + t * (F::kBits == 4 ? 8 : 16));
        const uint32_t so_thr = so0 + static_cast<uint32_t>((ti & 1) * so_buf * 8 + (warp * R + g) * 8);
        for (int c = 0; c < n_chunks; ++c) {
          const int u = ti * n_chunks + c;
          const int s = u % NS;
          if (!dead && !mbar_wait_bounded(&full[s], (u / NS) & 1)) {
            report_timeout(a.status, 200 + s);
            dead = true;
          }
          const int chunk_groups = min(kChunkK, a.k_per_cta - c * kChunkK) / kGroupK;
          const uint32_t a_chunk = stage0 + static_cast<uint32_t>(s) * kStageBytes + a_thr;
          const uint32_t so_chunk = so_thr + static_cast<uint32_t>(c * GC * R * 8);
#pragma unroll
          for (int j = 0; j < JC; ++j) {
            if (warp + kConsumerWarps * j < chunk_groups) {   // the last chunk of a K that is no multiple of the chunk
              uint32_t xf[MB][8];
              float xs2[MB][2];
              load_x(c * GC + warp + kConsumerWarps * j, xf, xs2);
              do_group32(a_chunk + static_cast<uint32_t>(kConsumerWarps * j * F::kGroupBytes),
                         so_chunk + static_cast<uint32_t>(kConsumerWarps * j * R * 8), xf, xs2);
            }
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(&empty[s]);
        }
      } else {
        for (int c = 0; c < n_chunks; ++c) {
          const int u = ti * n_chunks + c;
          const int s = u % NS;
          if (!dead && !mbar_wait_bounded(&full[s], (u / NS) & 1)) {
            report_timeout(a.status, 200 + s);
            dead = true;
          }
          const int chunk_groups = min(kChunkK, a.k_per_cta - c * kChunkK) / kGroupK;
          for (int gs = warp / kRowSplit; gs < chunk_groups && !dead; gs += kConsumerWarps / kRowSplit) {
            const int gl = c * GC + gs;     // group within this CTA's slice
            uint32_t xf[MB][8];
            float xs2[MB][2];
            load_x(gl, xf, xs2);
            do_group(stage_base + static_cast<size_t>(s) * kStageBytes + gs * F::kGroupBytes, so_cur + gl * R, xf, xs2);
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(&empty[s]);
        }
      }
      // split-K inside the CTA
      if (partials) {
        // plain stores of this warp's partial tile: lane (g, t) holds rows g, g+8, columns 2t, 2t+1
        float* mine = red_cur + warp * R * MP;
#pragma unroll
        for (int rt = 0; rt < RTW; ++rt) {
          *reinterpret_cast<float2*>(&mine[(rt * 16 + g) * MP + 2 * t]) = make_float2(acc[rt][0][0], acc[rt][0][1]);
          *reinterpret_cast<float2*>(&mine[(rt * 16 + g + 8) * MP + 2 * t]) = make_float2(acc[rt][0][2], acc[rt][0][3]);
          acc[rt][0][0] = acc[rt][0][1] = acc[rt][0][2] = acc[rt][0][3] = 0.0f;
        }
      } else {
#pragma unroll
        for (int rt = 0; rt < RTW; ++rt)
#pragma unroll
          for (int mb = 0; mb < MB; ++mb)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int row = row_base + rt * 16 + g + ((i & 2) ? 8 : 0);
              const int col = mb * 8 + 2 * t + (i & 1);
              atomicAdd(&red_cur[row * RP + col], acc[rt][mb][i]);
              acc[rt][mb][i] = 0.0f;
            }
      }
      if (has_next) scale_store(n0 + static_cast<int>(gridDim.x) * R, so + ((ti + 1) & 1) * so_buf);
      consumer_barrier();
      if (solo) {
        if (partials) {
          // the epilogue moves to other warps every tile, so no warp is always the late one
          const int et = (tid + kConsumerThreads - ((ti * 128) % kConsumerThreads)) % kConsumerThreads;
          if (a.epilogue == B200_QMM_OUT_SILU_PAIR) {
            // rows come as 8 gate rows then 8 up rows per 16: out[m, n0 / 2 + pair] = silu(gate) * up, with the
            // reference's bf16 roundings (the projection's own output, the sigmoid, gate * sigmoid, the product)
            if (et < (rows_valid / 2) * a.M) {
              const int pr = et % (rows_valid / 2), m = et / (rows_valid / 2);
              const int rg = (pr >> 3) * 16 + (pr & 7);
              float vg = 0.0f, vu = 0.0f;
#pragma unroll
              for (int w = 0; w < kConsumerWarps; ++w) {
                vg += red_cur[(w * R + rg) * MP + m];
                vu += red_cur[(w * R + rg + 8) * MP + m];
              }
              const float g = bf16_round(vg), u = bf16_round(vu);
              const float sig = bf16_round(__fdividef(1.0f, 1.0f + __expf(-g)));
              reinterpret_cast<__nv_bfloat16*>(a.out)[static_cast<size_t>(m) * a.ldo + n0 / 2 + pr] =
                  __float2bfloat16_rn(bf16_round(g * sig) * u);
            }
          } else if (et < rows_valid * a.M) {
            const int r = et % rows_valid, m = et / rows_valid;
            float v = 0.0f;
#pragma unroll
            for (int w = 0; w < kConsumerWarps; ++w) v += red_cur[(w * R + r) * MP + m];
            store_output<FMT, GROUPED, TP>(a, v, m, n0 + r);
          }
        } else {
          for (int idx = tid; idx < rows_valid * a.M; idx += kConsumerThreads) {
            const int r = idx % rows_valid, m = idx / rows_valid;
            const float v = red_cur[r * RP + m];
            red_cur[r * RP + m] = 0.0f;   // this buffer is added into again two tiles from now
            store_output<FMT, GROUPED, TP>(a, v, m, n0 + r);
          }
        }
      } else {
        cluster_arrive(ti);
        if (ti > 0) cluster_finish(ti - 1);
        // Buffer (ti + 1) mod 4 held tile ti - 3.  Every peer read it before arriving for tile
        // ti - 1, which this CTA has just waited for: clear it for tile ti + 1.
        if (ti >= 3) {
          float* next = red + ((ti + 1) & 3) * R * RP;
          for (int i = tid; i < R * RP; i += kConsumerThreads) next[i] = 0.0f;
        }
        consumer_barrier();
      }
    }
    if (!solo) {
      cluster_finish(n_my - 1);
      // no CTA leaves while a peer may still read its last tiles
      consumer_barrier();
      cluster_arrive(n_my);
      cluster_wait(n_my);
    }
    if (TP && a.epilogue == kEpiloguePush) {
      // This CTA's lines are on their way.  Now the sum over ranks, formed ONCE per rank by the CTAs of
      // this kernel together (tp_reduce_publish): CTAs that finish their tiles early do it while the
      // others still stream weights, and the projection that follows finds the new residual row
      // published in this rank's memory (K / 2 lines instead of world * K to read).  All CTAs of the
      // grid are resident (one per SM), so waiting for lines that other CTAs of the grid, or the
      // peers, still have to store cannot deadlock; the wait is bounded like every other.
      consumer_barrier();
      const uint32_t n = *a.tp_count + 1u;
      if (a.tp_bcast != nullptr)
        tp_reduce_publish(a.tp_src + static_cast<size_t>(n & 1u) * a.tp_world * a.tp_cap, static_cast<size_t>(a.tp_cap), a.tp_world, n,
                          a.status, a.tp_nowait, a.tp_x_old, a.N, a.M, a.N, a.x_out,
                          a.tp_bcast + static_cast<size_t>(n & 1u) * (a.tp_cap / 2),
                          static_cast<int>(blockIdx.y * gridDim.x + blockIdx.x), static_cast<int>(gridDim.x * gridDim.y), tid,
                          kConsumerThreads);
      // The last CTA of this rank to finish counts the exchange (every CTA read the old count before).
      consumer_barrier();
      if (tid == 0 && !(a.tp_nowait & 8)) {
        __threadfence();
        if (atomicAdd(a.tp_done, 1u) == gridDim.x * gridDim.y - 1u) {
          *a.tp_done = 0u;
          *a.tp_count = n;
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------
// Host side: plan, validation, dispatch
// ---------------------------------------------------------------------------

struct Plan {
  int fmt = 0, mb = 1, rt = 1, split = 1, stages = 2, tiles = 0, grid_x = 0;
  bool grouped = true;
  size_t smem = 0;
};

int BitsOf(int fmt) { return fmt == kInt8 ? 8 : (fmt == kBf16 ? 16 : 4); }
int ChunkRowBytes(int mb, int rt) { return mb == 1 ? kCopyBytes : kCopyBytes / rt; }
int ChunkRowStride(int fmt, int mb, int rt) { return ChunkRowBytes(mb, rt) + (BitsOf(fmt) == 4 ? 32 : 64); }
int ChunkK(int fmt, int mb, int rt) { return ChunkRowBytes(mb, rt) * 8 / BitsOf(fmt); }

size_t SmemFor(const Plan& pl, int M, int k_per_cta) {
  const int R = 16 * pl.rt, MP = 8 * pl.mb, groups = k_per_cta / kGroupK;
  size_t off = (static_cast<size_t>(2 * pl.stages) * 8 + 127) & ~static_cast<size_t>(127);
  off += static_cast<size_t>(pl.mb == 1 ? 2 * kConsumerWarps * MP : 4 * (MP + 4)) * R * 4;
  off += (static_cast<size_t>(groups) * MP * 4 + 127) & ~static_cast<size_t>(127);
  off += (static_cast<size_t>(groups) * M * 128 + 127) & ~static_cast<size_t>(127);
  if (pl.grouped) off += (static_cast<size_t>(2) * groups * R * 8 + 127) & ~static_cast<size_t>(127);
  off += static_cast<size_t>(pl.stages) * R * ChunkRowStride(pl.fmt, pl.mb, pl.rt);
  return off;
}

b200_status Validate(const b200_qmm_params* p) {
  if (p == nullptr) return Fail(B200_INVALID_ARGUMENT, "b200_qmm: null params");
  if (p->bits != 4 && p->bits != 8 && p->bits != 16)
    return Fail(B200_INVALID_ARGUMENT, "b200_qmm: bits must be 4, 8 or 16, got %d", p->bits);
  if (p->M < 0 || p->N < 0 || p->K < 0) return Fail(B200_INVALID_ARGUMENT, "b200_qmm: negative size");
  if (p->M > 32 && p->prologue != B200_QMM_PRO_NONE)
    return Fail(B200_UNIMPLEMENTED, "b200_qmm: the fused input transforms take up to 32 rows (8 for RMSNorm); M = %lld",
                static_cast<long long>(p->M));
  if (p->M > 32 && p->epilogue == B200_QMM_OUT_F32)
    return Fail(B200_UNIMPLEMENTED, "b200_qmm: above 32 rows the output is bf16, bf16 + residual, or raw f32");
  if (p->N > INT32_MAX / 2 || p->K > INT32_MAX / 2) return Fail(B200_UNIMPLEMENTED, "b200_qmm: size exceeds int32");
  if (p->K % kGroupK != 0)
    return Fail(B200_UNIMPLEMENTED, "b200_qmm: K = %lld is not a multiple of 64", static_cast<long long>(p->K));
  if (p->bits == 4 && p->group != 64) return Fail(B200_UNIMPLEMENTED, "b200_qmm: int4 group must be 64, got %d", p->group);
  if (p->bits == 8 && p->group != 64 && p->group != p->K)
    return Fail(B200_UNIMPLEMENTED, "b200_qmm: int8 group must be 64 or K, got %d", p->group);
  if (p->bits == 4 && p->nibble_order != 0 && p->nibble_order != 1)
    return Fail(B200_INVALID_ARGUMENT, "b200_qmm: nibble_order must be 0 or 1");
  if (p->epilogue < 0 || p->epilogue > 4) return Fail(B200_INVALID_ARGUMENT, "b200_qmm: unknown epilogue %d", p->epilogue);
  if (p->epilogue == B200_QMM_OUT_SILU_PAIR && (p->M > 8 || p->N % 16 != 0 || p->bits == 16 || (p->bits == 8 && p->group != 64)))
    return Fail(B200_UNIMPLEMENTED, "b200_qmm: the silu(gate) * up epilogue takes up to 8 rows of x and grouped weights with N a multiple of 16");
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
  const int64_t ncols = p->epilogue == B200_QMM_OUT_SILU_PAIR ? p->N / 2 : p->N;
  const int64_t ldx = p->ldx ? p->ldx : xcols, ldo = p->ldo ? p->ldo : ncols;
  if (ldx < xcols || ldo < ncols) return Fail(B200_INVALID_ARGUMENT, "b200_qmm: leading dimension smaller than row length");
  if (p->K == 0) return Fail(B200_UNIMPLEMENTED, "b200_qmm: K = 0");
  return B200_OK;
}

b200_status MakePlanImpl(const b200_qmm_params* p, int sm_count, int max_smem, Plan* out, bool no_tall_tiles) {
  Plan pl;
  pl.fmt = p->bits == 16 ? kBf16 : (p->bits == 8 ? kInt8 : (p->nibble_order ? kInt4Half : kInt4Seq));
  pl.grouped = (p->bits == 4) || (p->bits == 8 && p->group == 64);
  const int M = static_cast<int>(p->M), N = static_cast<int>(p->N), K = static_cast<int>(p->K);
  pl.mb = M <= 8 ? 1 : (M <= 16 ? 2 : 4);
  // Above 8 batch rows the tile grows with the batch: its row tiles are shared out among
  // the warps, so each warp reduces into the shared tile less often.
  pl.rt = pl.mb;
  // Up to 8 rows of x: two 16-row tiles per step (two independent dequant/MMA chains per
  // warp) when 32-row tiles still give every SM one; only on the unrolled K = 4096 path.
  // ... or, up to 2 rows of x, when they cost the busiest SM no more rows than 16-row tiles would (N = 4096 on 148 SMs:
  // one 32-row tile each for 128 CTAs against two 16-row tiles for 108 of 148).
  const int64_t rows_tall = CeilDiv(CeilDiv(N, 32), sm_count) * 32, rows_short = CeilDiv(CeilDiv(N, 16), sm_count) * 16;
  // the unrolled variants take 16-byte loads of x, gain, scales and offsets for granted
  const int64_t ldx = p->ldx ? p->ldx : (p->prologue == B200_QMM_PRO_SILU_MUL ? 2 * p->K : p->K);
  const bool fast_ok = p->prologue != B200_QMM_PRO_SILU_MUL && Aligned(p->x, 16) && ldx % 8 == 0 &&
                       (p->prologue != B200_QMM_PRO_RMSNORM || Aligned(p->prologue_gain, 16)) &&
                       (!pl.grouped || (Aligned(p->scale, 16) && (p->bits != 4 || Aligned(p->bias, 16))));
  if (fast_ok && pl.mb == 1 && K == 64 * kGroupK && (CeilDiv(N, 32) >= sm_count || (M <= 2 && rows_tall <= rows_short)) && !no_tall_tiles)
    pl.rt = 2;
  if (pl.mb == 4 && no_tall_tiles) pl.rt = 2;   // the 64-row tile's buffers did not fit beside this slice of x
  pl.tiles = static_cast<int>(CeilDiv(N, 16 * pl.rt));
  // K is split across a cluster only when the row tiles alone cannot occupy the
  // GPU, or when a CTA's slice of x would not fit shared memory.
  // One persistent CTA per SM (it walks tiles blockIdx.x, + grid, ...) with a deep
  // ring: under load a bulk copy takes ~3 us to land, so ~6.5 TB/s needs well
  // over 100 KB in flight per SM.  Ring depth: as many stages as the CTA has units,
  // within ~200 KB.
  const size_t x_budget = 96 * 1024, budget = 200 * 1024;
  bool found = false;
  for (int split = 1; split <= 8 && !found; split <<= 1) {
    if (K % (split * kGroupK) != 0) break;
    const int kc = K / split;
    // Up to 8 rows of x a fifth of the SMs is "enough": measured at M = 1, 1536 x 4096 takes 3.7 us on 96 CTAs
    // against 8.4 us as 96 clusters of two, 768 x 4096 3.3 us on 48 CTAs against 8.8 us as clusters of four
    // (the exchange through distributed shared memory costs more than the idle SMs).
    const int fill_pct = pl.mb == 1 ? 20 : 100;
    const bool fills = static_cast<int64_t>(pl.tiles) * split * 100 >= static_cast<int64_t>(sm_count) * fill_pct;
    const bool last = split == 8 || K % (2 * split * kGroupK) != 0;
    const bool tall = pl.rt > pl.mb;   // the two-tile variant never splits K
    if (static_cast<size_t>(M) * kc * 2 > x_budget || !(fills || last || tall)) continue;
    pl.split = split;
    const int chunks = static_cast<int>(CeilDiv(kc, ChunkK(pl.fmt, pl.mb, pl.rt)));
    pl.grid_x = std::min(pl.tiles, std::max(1, sm_count / split));
    const int units = chunks * static_cast<int>(CeilDiv(pl.tiles, pl.grid_x));
    pl.stages = std::min(units, 12);
    const int min_stages = units < 2 ? 1 : 2;
    for (;;) {
      pl.smem = SmemFor(pl, M, kc);
      if (pl.smem <= budget || pl.stages <= min_stages) break;
      --pl.stages;
    }
    found = pl.smem <= static_cast<size_t>(max_smem);   // else: a smaller slice of K per CTA
    if (pl.rt > pl.mb) break;   // the two-tile variant exists for the whole K = 4096 only
  }
  if (!found) {
    if (((pl.mb == 1 && pl.rt == 2) || pl.mb == 4) && !no_tall_tiles) return MakePlanImpl(p, sm_count, max_smem, out, true);
    return Fail(B200_UNIMPLEMENTED, "b200_qmm: M=%d K=%d does not fit shared memory (limit %d bytes)", M, K, max_smem);
  }
  *out = pl;
  return B200_OK;
}

b200_status MakePlan(const b200_qmm_params* p, int sm_count, int max_smem, Plan* out) {
  return MakePlanImpl(p, sm_count, max_smem, out, false);
}

template <int FMT, int MB, int RT, bool GROUPED, int KG, bool LEAN = (KG > 0), bool VEC = LEAN, bool TP = false>
cudaError_t LaunchOne(const Plan& pl, const QmmArgs& args, dim3 grid, cudaStream_t stream) {
  auto kernel = qgemv_kernel<FMT, MB, RT, GROUPED, KG, LEAN, VEC, TP>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(pl.smem));
  if (e != cudaSuccess) return e;
  LaunchCfg lc;
  lc.grid = grid;
  lc.block = dim3(kThreads);
  lc.smem = pl.smem;
  lc.stream = stream;
  lc.pdl = true;
  lc.cluster_y = pl.split;
  if (pl.split > 1) {
    // Persistent clusters: no more of them than the GPU holds at once (a GPC takes only
    // whole clusters), or the surplus would run alone after the others finish.
    static std::mutex mu;
    static std::map<std::pair<int, size_t>, int> resident;   // (split, smem) -> clusters
    std::lock_guard<std::mutex> lock(mu);
    auto it = resident.find({pl.split, pl.smem});
    if (it == resident.end()) {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(64, pl.split, 1);
      cfg.blockDim = lc.block;
      cfg.dynamicSmemBytes = pl.smem;
      cudaLaunchAttribute attr;
      attr.id = cudaLaunchAttributeClusterDimension;
      attr.val.clusterDim.x = 1;
      attr.val.clusterDim.y = pl.split;
      attr.val.clusterDim.z = 1;
      cfg.attrs = &attr;
      cfg.numAttrs = 1;
      int n = 0;
      e = cudaOccupancyMaxActiveClusters(&n, kernel, &cfg);
      if (e != cudaSuccess) return e;
      it = resident.emplace(std::make_pair(pl.split, pl.smem), std::max(n, 1)).first;
    }
    lc.grid.x = std::min<unsigned>(lc.grid.x, static_cast<unsigned>(it->second));
  }
  return Launch(lc, kernel, args);
}

// What the unrolled (KG > 0) variants are compiled for.
template <bool GROUPED>
bool FastPathOk(const QmmArgs& a) {
  return a.x_vec && (!GROUPED || a.scale_vec) && a.prologue != B200_QMM_PRO_SILU_MUL;
}

template <int FMT, bool GROUPED>
cudaError_t LaunchFmt(const Plan& pl, const QmmArgs& args, dim3 grid, cudaStream_t stream) {
  const bool vec = args.x_vec && (!GROUPED || args.scale_vec);   // 16-byte loads of x, scales and offsets
  if (args.tp_world > 0) {
    // The exchange builds: sequential int4 in groups (the projections) and bf16 (the LM head), up to
    // 8 rows: what a sharded decoder has.
    if constexpr ((FMT == kInt4Seq && GROUPED) || FMT == kBf16) {
      if (pl.mb != 1) return cudaErrorInvalidValue;
      const bool fast = args.k_per_cta == 64 * kGroupK && pl.split == 1 && FastPathOk<GROUPED>(args);
      if (pl.rt == 2) return fast ? LaunchOne<FMT, 1, 2, GROUPED, 64, true, true, true>(pl, args, grid, stream) : cudaErrorInvalidValue;
      if (pl.rt != 1) return cudaErrorInvalidValue;
      if (fast) return LaunchOne<FMT, 1, 1, GROUPED, 64, true, true, true>(pl, args, grid, stream);
      if (pl.split == 1 && vec) return LaunchOne<FMT, 1, 1, GROUPED, 0, true, true, true>(pl, args, grid, stream);
      if (vec) return LaunchOne<FMT, 1, 1, GROUPED, 0, false, true, true>(pl, args, grid, stream);
      return LaunchOne<FMT, 1, 1, GROUPED, 0, false, false, true>(pl, args, grid, stream);
    } else {
      return cudaErrorInvalidValue;
    }
  }
  switch (pl.mb * 10 + pl.rt) {
    case 11:
      // the decode shape K = 4096 (64 groups, no K split) takes the unrolled register path
      if (args.k_per_cta == 64 * kGroupK && pl.split == 1 && FastPathOk<GROUPED>(args))
        return LaunchOne<FMT, 1, 1, GROUPED, 64>(pl, args, grid, stream);
      // any K (the down projection, K = 12288, with its silu prologue): the lean build when it applies
      if (pl.split == 1 && vec) return LaunchOne<FMT, 1, 1, GROUPED, 0, true>(pl, args, grid, stream);
      if (vec) return LaunchOne<FMT, 1, 1, GROUPED, 0, false, true>(pl, args, grid, stream);
      return LaunchOne<FMT, 1, 1, GROUPED, 0>(pl, args, grid, stream);
    case 12:
      if (args.k_per_cta != 64 * kGroupK || pl.split != 1 || !FastPathOk<GROUPED>(args)) return cudaErrorInvalidValue;
      return LaunchOne<FMT, 1, 2, GROUPED, 64>(pl, args, grid, stream);
    case 22:
      if (vec) return LaunchOne<FMT, 2, 2, GROUPED, 0, false, true>(pl, args, grid, stream);
      return LaunchOne<FMT, 2, 2, GROUPED, 0>(pl, args, grid, stream);
    case 42:
      if (vec) return LaunchOne<FMT, 4, 2, GROUPED, 0, false, true>(pl, args, grid, stream);
      return LaunchOne<FMT, 4, 2, GROUPED, 0>(pl, args, grid, stream);
    case 44:
      if (vec) return LaunchOne<FMT, 4, 4, GROUPED, 0, false, true>(pl, args, grid, stream);
      return LaunchOne<FMT, 4, 4, GROUPED, 0>(pl, args, grid, stream);
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
  a.tiles = pl.tiles;   // (a = {}: no tensor-parallel exchange)
  const dim3 grid(static_cast<unsigned>(pl.grid_x), pl.split, 1);
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
  if (p->M > 32) {   // not the streaming kernel: panel-wise dequantisation + GEMM
    if (rows_per_cta) *rows_per_cta = 0;
    if (split_k) *split_k = 0;
    if (batch_blocks) *batch_blocks = static_cast<int>(CeilDiv(p->M, 8));
    return B200_OK;
  }
  Plan pl;
  s = MakePlan(p, 148, 227 * 1024, &pl);
  if (s != B200_OK) return s;
  if (rows_per_cta) *rows_per_cta = 16 * pl.rt;
  if (split_k) *split_k = pl.split;
  if (batch_blocks) *batch_blocks = pl.mb;
  return B200_OK;
}

b200_status b200_qmm_run(b200_context* ctx, b200_stream stream, const b200_qmm_params* p) {
  return b200::QmmRunEx(ctx, stream, p, nullptr);
}

}  // extern "C"

namespace b200 {

static int TpMeasureMode() {
  static const int mode = [] {
    const char* v = std::getenv("B200_TP_NOWAIT");
    return v != nullptr ? atoi(v) : 0;
  }();
  return mode;
}

static bool TcRouteEnabled() {
  static const bool on = [] {
    const char* v = std::getenv("B200_QMM_TC");
    return v != nullptr && v[0] == '1';
  }();
  return on;
}

b200_status QmmRunEx(b200_context* ctx, cudaStream_t stream, const b200_qmm_params* p, const QmmTp* tp) {
  b200_status s = BeginLaunch(ctx);
  if (s != B200_OK) return s;
  s = Validate(p);
  if (s != B200_OK) return s;
  if (p->M == 0 || p->N == 0) return B200_OK;
  // int4 in groups of 64, up to 8 rows: the tcgen05 route on request (b200_qmm_force_route 2, or B200_QMM_TC=1);
  // measured slower than the mma.sync kernel at these batch sizes, see qmm_tc.cu
  if (p->M > 32) {   // prefill-sized batches: dequantise into an L2-resident panel, then the tensor-core GEMM
    if (tp != nullptr && tp->world > 1) return Fail(B200_UNIMPLEMENTED, "b200_qmm: the exchange takes up to 8 rows");
    return QmmManyRows(ctx, stream, p);
  }
  const int forced = ctx->qmm_route.load();
  if (p->epilogue == B200_QMM_OUT_SILU_PAIR) {
    Plan chk;
    b200_status ps = MakePlan(p, ctx->sm_count, ctx->max_smem_optin, &chk);
    if (ps != B200_OK) return ps;
    if (chk.split != 1 || chk.mb != 1)
      return Fail(B200_UNIMPLEMENTED, "b200_qmm: the silu(gate) * up epilogue needs a plan without a K split (M=%lld N=%lld K=%lld)",
                  static_cast<long long>(p->M), static_cast<long long>(p->N), static_cast<long long>(p->K));
  }
  if ((tp == nullptr || tp->world <= 1) && p->epilogue != B200_QMM_OUT_SILU_PAIR && (forced == 2 || (forced == 0 && TcRouteEnabled())) &&
      QmmTcEligible(ctx, p))
    return QmmTcRun(ctx, stream, p);
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
  a.ldo = static_cast<int>(p->ldo ? p->ldo : (p->epilogue == B200_QMM_OUT_SILU_PAIR ? p->N / 2 : p->N));
  a.prologue = p->prologue;
  a.eps = p->eps;
  a.gain = static_cast<const __nv_bfloat16*>(p->prologue_gain);
  a.x_vec = Aligned(p->x, 16) && a.ldx % 8 == 0 && (p->prologue != B200_QMM_PRO_RMSNORM || Aligned(p->prologue_gain, 16));
  a.scale_ld = p->bits == 16 ? 0 : static_cast<int>(p->K / p->group);
  a.k_per_cta = a.K / pl.split;
  a.scale_vec = pl.grouped && (a.k_per_cta / kGroupK) % 8 == 0 && a.scale_ld % 8 == 0 && Aligned(p->scale, 16) &&
                (p->bits != 4 || Aligned(p->bias, 16));
  a.epilogue = p->epilogue;
  a.stages = pl.stages;
  a.status = ctx->dev_status;
  a.out_row_stride = a.out_vec_stride = 0;
  a.alpha = 1.0f;
  a.act = a.bias_by_vec = a.out_f32 = 0;
  a.gemm_bias = nullptr;
  a.aux = nullptr;
  a.tiles = pl.tiles;
  a.tp_world = 0;
  a.tp_rank = 0;
  a.tp_count = a.tp_done = nullptr;
  a.tp_src = nullptr;
  a.tp_cap = 0;
  a.tp_nowait = 0;
  a.x_out = nullptr;
  a.tp_x_old = nullptr;
  a.tp_bcast = nullptr;
  for (int r = 0; r < kTpMaxWorld; ++r) {
    a.tp_dst[r] = nullptr;
  }
  static const bool force_tp_build = std::getenv("B200_QMM_FORCE_TP_BUILD") != nullptr;   // measurement only
  if (force_tp_build && tp == nullptr && pl.mb == 1 && (pl.fmt == kInt4Seq || pl.fmt == kBf16)) a.tp_world = 1;
  if (tp != nullptr && tp->world >= 1) {
    if (p->M * p->N > tp->cap && tp->push) return Fail(B200_INVALID_ARGUMENT, "b200_qmm: partial sums exceed the exchange block");
    if ((pl.fmt != kInt4Seq && pl.fmt != kBf16) || pl.mb != 1)
      return Fail(B200_UNIMPLEMENTED, "b200_qmm: the exchange takes sequential int4 or bf16 weights and up to 8 rows");
    if (tp->src == nullptr || tp->bcast == nullptr || tp->count == nullptr)
      return Fail(B200_INVALID_ARGUMENT, "b200_qmm: the exchange is not connected");
    a.tp_world = tp->world;
    a.tp_rank = tp->rank;
    a.tp_cap = tp->cap;
    a.tp_count = tp->count;
    a.tp_bcast = tp->bcast;
    a.tp_nowait = TpMeasureMode();
    if (tp->push) {
      if (p->epilogue != B200_QMM_OUT_F32_RAW || a.ldo != a.N || a.N % 8 != 0 || tp->x_old == nullptr || tp->x_out == nullptr ||
          !Aligned(tp->x_old, 16) || !Aligned(tp->x_out, 16))
        return Fail(B200_INVALID_ARGUMENT, "b200_qmm: pushed partial sums are dense raw f32 rows of a multiple of 8 values, with the residual rows they are added to");
      a.epilogue = kEpiloguePush;
      a.tp_done = tp->done;
      a.tp_src = tp->src;
      a.tp_x_old = static_cast<const __nv_bfloat16*>(tp->x_old);
      a.x_out = static_cast<__nv_bfloat16*>(tp->x_out);
      for (int r = 0; r < tp->world; ++r) a.tp_dst[r] = tp->dst[r];
    } else {
      if (p->prologue != B200_QMM_PRO_RMSNORM || !a.x_vec || a.ldx != a.K || a.K % 8 != 0 || p->M * p->K > tp->cap)
        return Fail(B200_INVALID_ARGUMENT, "b200_qmm: reading the summed rows goes with the RMSNorm prologue on dense, aligned rows");
    }
  }
  const dim3 grid(static_cast<unsigned>(pl.grid_x), pl.split, 1);
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

}  // namespace b200

extern "C" {

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
