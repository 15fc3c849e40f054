// Dense 16-bit GEMM on the 5th-generation tensor cores:
//   D = act(alpha * op(A) op(B) + beta * D + bias[col]),  aux = pre-activation,
// the semantics of the reference's steel GEMM (metal_pjrt/blas/steel_gemm.cc:163-255,
// kernels/steel_gemm.metal:217-225) with f32 accumulation and one rounding.
//
// Structure (one persistent CTA per SM, 192 threads):
//   warp 0    TMA producer: per K step one 128 x 64 tile of op(A) and one 64 x BN tile
//             of op(B), as 128-byte-swizzled boxes of cp.async.bulk.tensor (no cluster
//             multicast), into a 4- to 8-deep shared-memory ring guarded by mbarriers;
//   warp 1    allocates tensor memory and issues tcgen05.mma (cta_group::1, kind::f16,
//             M = 128, N = BN, K = 16) from shared-memory descriptors; tcgen05.commit
//             releases ring slots and signals a finished accumulator;
//   warps 2-5 epilogue: tcgen05.ld of their 32 accumulator lanes, the fused epilogue in
//             f32, one rounding, 64-byte row segments stored straight to D.
// Two accumulators (2 x BN of the 512 TMEM columns) let the epilogue of one tile overlap
// the MMAs of the next.  Every wait is bounded; a wait that gives up reports
// B200_TIMEOUT through the context's status word and the CTA unwinds (frees TMEM, returns).
//
// Either operand may be transposed: a K-contiguous operand is loaded as [rows][64 k] boxes
// (K-major descriptor), an M- or N-contiguous one as [64 k][64 rows] boxes (MN-major
// descriptor), so nothing is transposed in memory.
#include <cooperative_groups.h>
#include <cuda.h>

#include <mutex>

#include "common.cuh"

namespace cg = cooperative_groups;
using namespace b200;

namespace {

constexpr int BM = 128;
constexpr int BK = 64;          // one 128-byte swizzle row of 16-bit elements
constexpr int kThreads = 192;
constexpr int kEpilogueWarps = 4;

struct TcArgs {
  void* d;
  const void* bias;
  void* aux;
  int m, n, k;
  int64_t ldd;
  float alpha, beta;
  int act;
  int out_dtype;   // b200_dtype of D
  int ta, tb;
  int tiles_m, tiles_n;
  int split;       // CTAs of a cluster along K (grid.y); 1: persistent CTAs, no cluster
  int* status;
};

// ---- PTX wrappers --------------------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
          smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// 32 lanes x 32 consecutive columns: thread i of the warp gets lane (base + i), columns c .. c+31
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
        "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
        "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor, 128-byte swizzle.  K-major tile: rows of 128 bytes,
// 8-row groups 1024 bytes apart (SBO), LBO unused.  MN-major tile: boxes of [64 k][64 mn],
// 8-k-row groups 1024 bytes apart (SBO), the next 64 mn (next box) `lbo` bytes on.
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>(lbo_bytes >> 4) << 16;
  d |= static_cast<uint64_t>(sbo_bytes >> 4) << 32;
  d |= 1ull << 46;   // descriptor version for this architecture
  d |= 2ull << 61;   // 128-byte swizzle
  return d;
}

// Instruction descriptor for kind::f16: f32 accumulate, A/B format (0 f16, 1 bf16),
// major-ness (0 K-major, 1 MN-major), N >> 3 at bit 17, M >> 4 at bit 24.
__host__ __device__ constexpr uint32_t make_idesc(int ab_format, int a_mn_major, int b_mn_major, int n) {
  return (1u << 4) | (static_cast<uint32_t>(ab_format) << 7) | (static_cast<uint32_t>(ab_format) << 10) |
         (static_cast<uint32_t>(a_mn_major) << 15) | (static_cast<uint32_t>(b_mn_major) << 16) |
         (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(BM >> 4) << 24);
}

template <int BN>
struct Smem {
  static constexpr int kABytes = BM * BK * 2;        // 16 KB
  static constexpr int kBBytes = BN * BK * 2;        // 32 KB at BN = 256
  static constexpr int kStageBytes = kABytes + kBBytes;
  // ~192 KB of ring whatever the tile width: narrow tiles stream B and need the depth
  static constexpr int kStages = BN == 256 ? 4 : (BN == 128 ? 6 : 8);
  static constexpr int kTotal = kStages * kStageBytes + 1024 /* alignment slack */ + 256 /* barriers */;
};

template <typename TOut>
__device__ __forceinline__ void epilogue_row(const TcArgs& a, const uint32_t (&v)[32], int row, int col0) {
  TOut* D = static_cast<TOut*>(a.d);
  TOut* AUX = static_cast<TOut*>(a.aux);
  const TOut* bias = static_cast<const TOut*>(a.bias);
  const int64_t o = static_cast<int64_t>(row) * a.ldd + col0;
  const bool full = col0 + 32 <= a.n;
  constexpr int kVec = 16 / sizeof(TOut);
  const bool vec = full && (a.ldd % kVec == 0) && ((reinterpret_cast<uintptr_t>(D) & 15) == 0) &&
                   (AUX == nullptr || (reinterpret_cast<uintptr_t>(AUX) & 15) == 0);
  float x[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    x[j] = a.alpha * __uint_as_float(v[j]);
    if (a.beta != 0.0f && col0 + j < a.n) x[j] += a.beta * load_as_f32<TOut>(D + o + j);
    if (bias != nullptr && col0 + j < a.n) x[j] += load_as_f32<TOut>(bias + col0 + j);
  }
  if (vec) {
    if (AUX != nullptr) {
#pragma unroll
      for (int j = 0; j < 32; j += kVec) {
        uint4 raw;
        TOut* e = reinterpret_cast<TOut*>(&raw);
#pragma unroll
        for (int i = 0; i < kVec; ++i) e[i] = store_from_f32<TOut>(x[j + i]);
        *reinterpret_cast<uint4*>(AUX + o + j) = raw;
      }
    }
#pragma unroll
    for (int j = 0; j < 32; j += kVec) {
      uint4 raw;
      TOut* e = reinterpret_cast<TOut*>(&raw);
#pragma unroll
      for (int i = 0; i < kVec; ++i) e[i] = store_from_f32<TOut>(apply_act(a.act, x[j + i]));
      *reinterpret_cast<uint4*>(D + o + j) = raw;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      if (col0 + j < a.n) {
        if (AUX != nullptr) AUX[o + j] = store_from_f32<TOut>(x[j]);
        D[o + j] = store_from_f32<TOut>(apply_act(a.act, x[j]));
      }
    }
  }
}

// The same epilogue for 4 consecutive columns (the split-K reduction, where a warp owns a
// row and its lanes adjacent float4s, so that the reads of the peers' tiles coalesce).
template <typename TOut>
__device__ __forceinline__ void epilogue_quad(const TcArgs& a, const float (&acc)[4], int row, int col0) {
  TOut* D = static_cast<TOut*>(a.d);
  TOut* AUX = static_cast<TOut*>(a.aux);
  const TOut* bias = static_cast<const TOut*>(a.bias);
  const int64_t o = static_cast<int64_t>(row) * a.ldd + col0;
  float x[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    x[j] = a.alpha * acc[j];
    if (col0 + j < a.n) {
      if (a.beta != 0.0f) x[j] += a.beta * load_as_f32<TOut>(D + o + j);
      if (bias != nullptr) x[j] += load_as_f32<TOut>(bias + col0 + j);
    }
  }
  constexpr size_t kBytes = 4 * sizeof(TOut);
  const bool vec = col0 + 4 <= a.n && (a.ldd % 4 == 0) && (reinterpret_cast<uintptr_t>(D) % kBytes == 0) &&
                   (AUX == nullptr || reinterpret_cast<uintptr_t>(AUX) % kBytes == 0);
  if (vec) {
    struct alignas(kBytes) Pack { TOut e[4]; };
    Pack pd, pa;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      pa.e[j] = store_from_f32<TOut>(x[j]);
      pd.e[j] = store_from_f32<TOut>(apply_act(a.act, x[j]));
    }
    if (AUX != nullptr) *reinterpret_cast<Pack*>(AUX + o) = pa;
    *reinterpret_cast<Pack*>(D + o) = pd;
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (col0 + j < a.n) {
        if (AUX != nullptr) AUX[o + j] = store_from_f32<TOut>(x[j]);
        D[o + j] = store_from_f32<TOut>(apply_act(a.act, x[j]));
      }
    }
  }
}

template <int BN, typename TOut>
__global__ void __launch_bounds__(kThreads, 1)
    gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const TcArgs a,
                   const uint32_t idesc) {
  using S = Smem<BN>;
  constexpr int kStages = S::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + kStages * S::kStageBytes);
  uint64_t* empty = full + kStages;
  uint64_t* tfull = empty + kStages;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int num_tiles = a.tiles_m * a.tiles_n;
  const int k_iters = (a.k + BK - 1) / BK;
  // With K split across a cluster, grid.x is the tile count (one tile per CTA) and CTA
  // blockIdx.y accumulates k steps [ki_begin, ki_end) of it.
  const int ki_begin = a.split > 1 ? static_cast<int>(blockIdx.y) * k_iters / a.split : 0;
  const int ki_end = a.split > 1 ? (static_cast<int>(blockIdx.y) + 1) * k_iters / a.split : k_iters;
  constexpr int kPartLd = BN + 4;          // row pitch (floats) of the partial tile in shared memory
  constexpr uint32_t kTmemCols = 2 * BN;   // two accumulators; a power of two >= 32

  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull[i], 1);
      mbar_init(&tempty[i], kEpilogueWarps);
    }
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(tmem_slot, kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();               // A, B (and D under beta) may come from the previous kernel
  pdl_launch_dependents();

  if (warp == 0) {
    // ---------------- TMA producer (one lane)
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int tm = tile % a.tiles_m, tn = tile / a.tiles_m;
        for (int ki = ki_begin; ki < ki_end && ok; ++ki, ++it) {
          const int s = it % kStages, use = it / kStages;
          if (use > 0 && !mbar_wait_bounded(&empty[s], (use - 1) & 1)) {
            report_timeout(a.status, 300 + s);
            ok = false;
            break;
          }
          uint8_t* As = smem + s * S::kStageBytes;
          uint8_t* Bs = As + S::kABytes;
          mbar_expect_tx(&full[s], S::kStageBytes);
          if (!a.ta) {
            tma_load_2d(As, &tmA, ki * BK, tm * BM, &full[s]);                 // [128 m][64 k]
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)                                    // [64 k][64 m] boxes
              tma_load_2d(As + j * 8192, &tmA, tm * BM + j * 64, ki * BK, &full[s]);
          }
          if (a.tb) {
            tma_load_2d(Bs, &tmB, ki * BK, tn * BN, &full[s]);                 // [BN n][64 k]
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)                                    // [64 k][64 n] boxes
              tma_load_2d(Bs + j * 8192, &tmB, tn * BN + j * 64, ki * BK, &full[s]);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (one lane)
    if (lane == 0) {
      int it = 0, tcount = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++tcount) {
        const int acc = tcount & 1, use_acc = tcount >> 1;
        if (use_acc > 0 && !mbar_wait_bounded(&tempty[acc], (use_acc - 1) & 1)) {
          report_timeout(a.status, 310 + acc);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(acc * BN);
        for (int ki = ki_begin; ki < ki_end && ok; ++ki, ++it) {
          const int s = it % kStages;
          if (!mbar_wait_bounded(&full[s], (it / kStages) & 1)) {
            report_timeout(a.status, 320 + s);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + s * S::kStageBytes);
          const uint32_t b_addr = a_addr + S::kABytes;
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk) {
            const uint64_t da = a.ta ? make_desc(a_addr + kk * 2048, 8192, 1024) : make_desc(a_addr + kk * 32, 16, 1024);
            const uint64_t db = a.tb ? make_desc(b_addr + kk * 32, 16, 1024) : make_desc(b_addr + kk * 2048, 8192, 1024);
            umma_f16(tmem_d, da, db, idesc, (ki > ki_begin || kk > 0) ? 1u : 0u);
          }
          umma_commit(&empty[s]);     // the slot is free once these MMAs have read it
        }
        if (ok) umma_commit(&tfull[acc]);
      }
    }
  } else {
    // ---------------- epilogue warps: TMEM lanes 32 q .. 32 q + 31
    const int q = warp & 3;
    int tcount = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++tcount) {
      const int tm = tile % a.tiles_m, tn = tile / a.tiles_m;
      const int acc = tcount & 1;
      if (!mbar_wait_bounded(&tfull[acc], (tcount >> 1) & 1)) {
        report_timeout(a.status, 330 + acc);
        ok = false;
        break;
      }
      tc_fence_after();
      const int row = tm * BM + 32 * q + lane;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t v[32];
        tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(32 * q) << 16) + static_cast<uint32_t>(acc * BN + c0), v);
        const int col0 = tn * BN + c0;
        if (a.split > 1) {
          // this CTA's K slice only: park the f32 partial in the (now idle) ring
          float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(smem) + (32 * q + lane) * kPartLd + c0);
#pragma unroll
          for (int j = 0; j < 8; ++j)
            dst[j] = make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]), __uint_as_float(v[4 * j + 2]),
                                 __uint_as_float(v[4 * j + 3]));
        } else if (row < a.m && col0 < a.n) {
          epilogue_row<TOut>(a, v, row, col0);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
    }
  }
  if (a.split > 1) {
    // K split: every CTA of the cluster finishes rows [rank, rank + 1) * 128 / split of the
    // tile from all the partial tiles, read through distributed shared memory.
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();
    if (warp >= 2) {
      const int tile = blockIdx.x, tm = tile % a.tiles_m, tn = tile / a.tiles_m;
      const int rows_per_rank = BM / a.split;
      const float* part = reinterpret_cast<const float*>(smem);
      // a warp per row, lanes on adjacent float4s: 512-byte runs of every peer's tile
      for (int rr = warp - 2; rr < rows_per_rank; rr += kEpilogueWarps) {
        const int r = static_cast<int>(blockIdx.y) * rows_per_rank + rr;
        const int row = tm * BM + r;
        if (row >= a.m) break;
#pragma unroll
        for (int t = 0; t < BN / 128 + (BN < 128 ? 1 : 0); ++t) {
          const int c = t * 128 + 4 * lane;
          if (c >= BN || tn * BN + c >= a.n) continue;
          float sum[4] = {0.0f, 0.0f, 0.0f, 0.0f};
          float4 v[8];
#pragma unroll
          for (int peer = 0; peer < 8; ++peer)   // all the remote loads in flight together
            v[peer] = peer < a.split
                          ? *reinterpret_cast<const float4*>(cluster.map_shared_rank(part, peer) + r * kPartLd + c)
                          : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
          for (int peer = 0; peer < 8; ++peer) {
            sum[0] += v[peer].x;
            sum[1] += v[peer].y;
            sum[2] += v[peer].z;
            sum[3] += v[peer].w;
          }
          epilogue_quad<TOut>(a, sum, row, tn * BN + c);
        }
      }
    }
    cluster.sync();   // peers may still be reading this CTA's partial tile
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver's tensor-map encoder, looked up through the runtime so that the
// library links nothing but the CUDA runtime.
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

// A 2-D map over a row-major matrix: `inner` contiguous elements per row, `outer`
// rows `ld` elements apart; boxes of box_inner x box_outer, 128-byte swizzle.
bool MakeMap(CUtensorMap* map, int dtype, const void* base, int64_t inner, int64_t outer, int64_t ld, int box_inner,
             int box_outer) {
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(outer)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(box_inner), static_cast<cuuint32_t>(box_outer)};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = Encoder()(map, dtype == B200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                               2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

template <int BN, typename TOut>
cudaError_t LaunchTc(const CUtensorMap& ma, const CUtensorMap& mb, const TcArgs& a, uint32_t idesc, int grid,
                     cudaStream_t stream) {
  static_assert(BM * (BN + 4) * 4 <= Smem<BN>::kStages * Smem<BN>::kStageBytes, "partial tile must fit the ring");
  auto kernel = gemm_tc_kernel<BN, TOut>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem<BN>::kTotal);
  if (e != cudaSuccess) return e;
  LaunchCfg lc;
  lc.grid = dim3(grid, a.split, 1);
  lc.block = dim3(kThreads);
  lc.smem = Smem<BN>::kTotal;
  lc.stream = stream;
  lc.pdl = true;
  lc.cluster_y = a.split;
  return Launch(lc, kernel, ma, mb, a, idesc);
}

// How many clusters of `split` CTAs of this kernel the device holds at once (a GPC takes
// only whole clusters, so this can be well below SMs / split).  Cached per shape of launch.
template <int BN, typename TOut>
int ResidentClusters(int split) {
  static std::mutex mu;
  static int cached[9] = {0};
  std::lock_guard<std::mutex> lock(mu);
  if (cached[split] == 0) {
    auto kernel = gemm_tc_kernel<BN, TOut>;
    int n = 0;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem<BN>::kTotal) == cudaSuccess) {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(16, split, 1);
      cfg.blockDim = dim3(kThreads);
      cfg.dynamicSmemBytes = Smem<BN>::kTotal;
      cudaLaunchAttribute attr;
      attr.id = cudaLaunchAttributeClusterDimension;
      attr.val.clusterDim.x = 1;
      attr.val.clusterDim.y = split;
      attr.val.clusterDim.z = 1;
      cfg.attrs = &attr;
      cfg.numAttrs = 1;
      if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess) n = 0;
      (void)cudaGetLastError();
    }
    cached[split] = n > 0 ? n : -1;
  }
  return cached[split] > 0 ? cached[split] : 0;
}

template <int BN>
int ResidentClustersFor(int out_dtype, int split) {
  if (out_dtype == B200_F32) return ResidentClusters<BN, float>(split);
  if (out_dtype == B200_BF16) return ResidentClusters<BN, __nv_bfloat16>(split);
  return ResidentClusters<BN, __half>(split);
}

}  // namespace

namespace b200 {

bool Tcgen05Supports(const b200_gemm_params* p, const b200_epilogue* epi) {
  (void)epi;
  if (p->a.dtype != B200_BF16 && p->a.dtype != B200_F16) return false;
  if (p->b.dtype != p->a.dtype) return false;
  if (p->batch != 1 || p->k < 1) return false;
  if (Encoder() == nullptr) return false;
  // TMA: 16-byte aligned bases, row pitches that are multiples of 16 bytes
  if (!Aligned(p->a.ptr, 16) || !Aligned(p->b.ptr, 16)) return false;
  if (p->a.ld % 8 != 0 || p->b.ld % 8 != 0) return false;
  if (p->m > (1 << 30) || p->n > (1 << 30) || p->k > (1 << 30)) return false;
  return true;
}

b200_status RunTcgen05(b200_context* ctx, cudaStream_t stream, const b200_gemm_params* p, const b200_epilogue* epi) {
  const int ta = p->a.transpose, tb = p->b.transpose;
  const int64_t m = p->m, n = p->n, k = p->k;
  // 128 x 256 tiles; narrower ones (128, 64 columns) when that is what it takes to spread
  // a few-row problem, which only streams B, over more SMs
  const int64_t tiles_m = CeilDiv(m, BM), k_iters = CeilDiv(k, BK);
  // Tile width and K split by a small cost model (microseconds).  A k step of a 128 x bn
  // tile costs what the SM's share of L2 bandwidth or the MMAs take, whichever is longer
  // (measured: 0.55 / 0.43 / 0.375 us for bn = 256 / 128 / 64); tiles run in waves over the
  // SMs.  When the tiles leave SMs idle, a cluster of 2/4/8 CTAs splits one tile's K loop
  // (a serial chain on one SM otherwise) and adds the partial tiles through distributed
  // shared memory, for a fixed cost of the cluster barriers and the extra pass.
  int bn = 256, split = 1;
  double best = 1e30;
  for (int cand : {256, 128, 64}) {
    const double t_iter = cand == 256 ? 0.55 : (cand == 128 ? 0.43 : 0.375);
    const int64_t tiles = tiles_m * CeilDiv(n, cand);
    const double whole = static_cast<double>(CeilDiv(tiles, ctx->sm_count)) * k_iters * t_iter;
    if (whole < best) best = whole, bn = cand, split = 1;
    for (int sp = 2; sp <= 8; sp *= 2) {
      if (tiles * sp > ctx->sm_count || k_iters / sp < 4) break;
      const int resident = cand == 256 ? ResidentClustersFor<256>(p->c.dtype, sp)
                                       : (cand == 128 ? ResidentClustersFor<128>(p->c.dtype, sp) : ResidentClustersFor<64>(p->c.dtype, sp));
      if (tiles > resident) continue;   // a second wave of clusters would double the time
      const double cost = static_cast<double>(CeilDiv(k_iters, sp)) * t_iter + 4.0;
      if (cost < best) best = cost, bn = cand, split = sp;
    }
  }
  CUtensorMap ma, mb;
  bool ok;
  if (!ta) ok = MakeMap(&ma, p->a.dtype, p->a.ptr, k, m, p->a.ld, BK, BM);     // A [m][k]
  else ok = MakeMap(&ma, p->a.dtype, p->a.ptr, m, k, p->a.ld, 64, BK);         // A stored [k][m]
  if (tb) ok = ok && MakeMap(&mb, p->b.dtype, p->b.ptr, k, n, p->b.ld, BK, bn); // B stored [n][k]
  else ok = ok && MakeMap(&mb, p->b.dtype, p->b.ptr, n, k, p->b.ld, 64, BK);   // B [k][n]
  if (!ok) return Stick(ctx, Fail(B200_INTERNAL, "b200_gemm: cuTensorMapEncodeTiled refused the operand layout"));
  TcArgs a;
  a.d = p->c.ptr;
  a.bias = epi->bias;
  a.aux = epi->aux;
  a.m = static_cast<int>(m);
  a.n = static_cast<int>(n);
  a.k = static_cast<int>(k);
  a.ldd = p->c.ld;
  a.alpha = static_cast<float>(p->alpha);
  a.beta = static_cast<float>(p->beta);
  a.act = epi->act;
  a.out_dtype = p->c.dtype;
  a.ta = ta;
  a.tb = tb;
  a.tiles_m = static_cast<int>(tiles_m);
  a.tiles_n = static_cast<int>(CeilDiv(n, bn));
  a.split = split;
  a.status = ctx->dev_status;
  const int64_t tiles = static_cast<int64_t>(a.tiles_m) * a.tiles_n;
  const int grid = split > 1 ? static_cast<int>(tiles) : static_cast<int>(std::min<int64_t>(tiles, ctx->sm_count));
  const uint32_t idesc = make_idesc(p->a.dtype == B200_BF16 ? 1 : 0, ta ? 1 : 0, tb ? 0 : 1, bn);
  cudaError_t e;
  const int out = p->c.dtype;
  if (bn == 256) {
    if (out == B200_F32) e = LaunchTc<256, float>(ma, mb, a, idesc, grid, stream);
    else if (out == B200_BF16) e = LaunchTc<256, __nv_bfloat16>(ma, mb, a, idesc, grid, stream);
    else e = LaunchTc<256, __half>(ma, mb, a, idesc, grid, stream);
  } else if (bn == 128) {
    if (out == B200_F32) e = LaunchTc<128, float>(ma, mb, a, idesc, grid, stream);
    else if (out == B200_BF16) e = LaunchTc<128, __nv_bfloat16>(ma, mb, a, idesc, grid, stream);
    else e = LaunchTc<128, __half>(ma, mb, a, idesc, grid, stream);
  } else {
    if (out == B200_F32) e = LaunchTc<64, float>(ma, mb, a, idesc, grid, stream);
    else if (out == B200_BF16) e = LaunchTc<64, __nv_bfloat16>(ma, mb, a, idesc, grid, stream);
    else e = LaunchTc<64, __half>(ma, mb, a, idesc, grid, stream);
  }
  if (e != cudaSuccess) return Stick(ctx, Fail(B200_INTERNAL, "b200_gemm (tcgen05) launch: %s", cudaGetErrorString(e)));
  return EndLaunch(ctx, "b200_gemm (tcgen05)");
}

}  // namespace b200
