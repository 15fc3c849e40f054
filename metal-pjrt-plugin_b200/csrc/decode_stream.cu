// One decode step of the Qwen3-shaped int4 decoder (examples/llm/qwen3.py:334-390, T = 1) as
// ONE persistent kernel: a CTA per SM walks every stage of every layer
//   qkv projection -> attention -> o projection -> gate_up projection -> down projection
// and finally the LM head, with a grid-wide arrive/wait between stages.  Nothing of the
// reference runs this way (XLA launches one kernel per fused op, ~430 per token,
// docs/performance.md:309-317); the arithmetic, the rounding points and the cache layout are
// the reference's.
//
// Why one kernel: at batch 1 a step reads 5.4 GB and takes a few hundred dependent
// operations; launched one by one, each pays a few microseconds of fill and drain while the
// memory system idles.  Here the weights of a CTA form ONE linear stream through all stages:
// a producer warp copies it record by record (cp.async.bulk + mbarrier) into a shared-memory
// ring and is never stopped by a stage boundary, so while the consumers wait at a grid
// barrier, stage their inputs or run attention, the next projection's weights keep arriving.
//
// Weight stream.  At decoder creation the int4 projections are copied into records of
// 16 rows x 512 inputs (4096 B of nibbles + 512 B of scales and offsets), each record laid
// out in the order the consuming warp's lanes read it (one conflict-free 16-byte load per
// lane and group), and the records of a CTA are stored in the order it consumes them.  Row
// tiles are dealt round-robin to the CTAs, continuing from stage to stage where the previous
// one stopped, so every CTA streams the same number of bytes over a layer.
//
// Consumers (15 warps).  A record is one warp's work: nibbles are widened to bf16 (128 + q) by
// one lop3 per pair and fed to mma.sync m16n8k16 with the batch as the 8-wide operand; x
// lies in shared memory in its natural order (the nibble order inside a record is chosen so
// that a lane's x fragment is 32 contiguous bytes); scale and offset are applied in f32 per
// group of 64 exactly as the per-operator kernel does.  (Measured and rejected: the nibbles as
// e4m3 subnormals through mma.sync m16n8k32 e4m3 with the activations split into two e4m3
// terms - numerically fine, but on this GPU that MMA costs 30-55 issue cycles as soon as its
// operands change from one MMA to the next, against ~10 for the bf16 one; and right shifts as
// multiply-high on the FMA pipe, 4-6 cycles each against ~1.)  The records of a CTA's stream go to
// its warps round-robin; the partial tiles of a row tile are added in a fixed order after one
// barrier per stage.  A gate_up tile holds eight gate rows and their eight up rows, so
// silu(gate) * up is formed where the tile is finished and never makes a round trip.
//
// What does not depend on the stage before is requested before the grid barrier in front of a
// stage: the old residual row and the RMSNorm gain of a projection's input, the K / V bytes of
// an attention unit (which the producer warp has asked L2 to fetch a stage earlier).
#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "decode_stream.cuh"

using namespace b200;

namespace b200 {
namespace dsk {

constexpr int kNW = 15;                      // consumer warps (with the producer warp: 16 warps, 128 registers each)
constexpr int kConsumers = kNW * 32;
constexpr int kThreads = kConsumers + 32;    // + the producer warp
constexpr int kAttnThreads = 256;            // consumer threads that work in the attention stage
constexpr int kMaxM = 8;                     // batch rows: the MMA's eight batch columns
constexpr int kUnitK = 512;                  // inputs per int4 record
constexpr int kUnitGroups = kUnitK / 64;
constexpr int kUnitBytes = 16 * kUnitK / 2 + 16 * kUnitGroups * 4;   // 4608
constexpr int kHeadUnitK = 1024;             // inputs per LM-head unit (16 bf16 rows, one 2 KB copy each: 1 KB copies
                                             // reached 4.2 TB/s with nothing consuming them)
constexpr int kHeadRows = 8;                 // rows per LM-head tile: half an MMA tile, so that twice as many units
                                             // (and warps) are in flight within the same ring bytes
constexpr int kHeadRowPitch = kHeadUnitK * 2 + 16;                   // keeps the row reads conflict-free
constexpr int kHeadUnitBytes = kHeadRows * kHeadRowPitch;
constexpr int kMaxSlots = 56;
constexpr int kMaxHeadSlots = 16;
constexpr int kHeaderBytes = 3072;           // mbarriers, small reduction arrays, the RoPE table
constexpr int kAttnWindow = 128;             // cache positions per pass of the attention loop
constexpr int kMaxChunks = 64;               // position chunks per (sequence, KV head)

enum StageType { kQkv = 0, kAttn = 1, kO = 2, kGateUp = 3, kDown = 4, kHead = 5 };

struct Stage {
  int type, layer;
  int NT, C, rot, K, N;            // row tiles, records per tile, first CTA of the round-robin, sizes
  const __nv_bfloat16* gain;       // RMSNorm gain of the input staging (qkv, gate_up, LM head)
  const __nv_bfloat16* q_norm;
  const __nv_bfloat16* k_norm;
  __nv_bfloat16* k_cache;
  __nv_bfloat16* v_cache;
};

struct StreamArgs {
  const Stage* stages;
  int n_stages;
  const uint8_t* packed;           // the int4 record stream of all CTAs
  const unsigned long long* cta_off;   // [G] byte offset of a CTA's stream
  const unsigned* cta_units;       // [G] its number of records
  const uint8_t* head_w;           // LM head, bf16 [V, E]
  int M;
  const int32_t* tokens;
  const int32_t* pos;
  float* logits;
  int32_t* next_token;             // or null
  const __nv_bfloat16* embed;
  long long vocab_full;
  __nv_bfloat16* x[2];             // residual stream, double buffered (one CTA writes while all read)
  float* y;                        // f32 [M, E]: output of the last o / down projection
  __nv_bfloat16* qkv;
  __nv_bfloat16* attn;
  __nv_bfloat16* hmlp;             // bf16 [M, I]: silu(gate) * up
  float* attn_part;                // [M * KV, chunks, G, D + 2]
  unsigned* attn_cnt;              // [M * KV] chunks finished (returns to zero)
  unsigned long long* ctl;         // [0] grid barrier arrivals, [1] CTAs that finished the step
  float* best_val;                 // [G, M] per-CTA best logit (greedy sampling)
  int* best_idx;
  int E, H, KV, D, I, V;
  long long max_len;
  float eps, attn_scale;
  const float* inv_freq;
  int attn_chunks;
  int NS, NS2;                     // ring slots (int4 records / LM-head units)
  int part_units;                  // partial tiles the reduction buffer holds
  int xs_pitch;                    // bf16 elements between rows of x in shared memory
  int MP;                          // batch columns kept per partial tile (M rounded up to even)
  int off_xsum, off_part, off_ring;   // byte offsets into dynamic shared memory
  int* status;
  unsigned long long* trace;       // or null: [G, n_stages, 4] globaltimer stamps of thread 0
  int ablate;                      // measurement only: 1 = consume the records without computing on them
};

// ---------------------------------------------------------------------------------------
// small device helpers
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
// right shift by 4r.  (A multiply-high by a power of two does the same on the FMA pipe, but it
// measures 4-6 issue cycles per warp instruction on this GPU against 2 for a lop3 and less
// for a plain shift, so it is not used.)
__device__ __forceinline__ uint32_t shr4(uint32_t v, int r) { return v >> (4 * r); }
// Shared-memory loads and MMAs of the record loops are NOT volatile: the compiler may then
// issue the loads of later groups ahead of the MMAs of earlier ones and interleave the MMA
// chains of different groups.  What keeps them inside the region where the slot is valid:
// their addresses pass through pin_addresses() after the wait on the slot's full barrier, and
// their results through pin_results() before the arrival on its empty one.
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
  uint2 v;
  asm("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}
__device__ __forceinline__ float2 lds64f(uint32_t addr) {
  float2 v;
  asm("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(addr));
  return v;
}
__device__ __forceinline__ void pin_addresses(uint32_t& a0, uint32_t& a1, uint32_t& a2) {
  asm volatile("" : "+r"(a0), "+r"(a1), "+r"(a2)::"memory");
}
__device__ __forceinline__ void pin_results(const float (&acc)[4]) {
  asm volatile("" ::"f"(acc[0]), "f"(acc[1]), "f"(acc[2]), "f"(acc[3]) : "memory");
}
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma16816_z(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                           uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
}
// Ask for a piece of global memory to be brought into L2 (address 16-byte aligned, size a multiple of 16).
__device__ __forceinline__ void prefetch_l2(const void* p, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}
// Per-stage time stamps (ns) of a CTA's thread 0: 0 the stage's inputs are complete (grid
// barrier passed), 1 its own inputs are staged, 2 this warp's share of the records is done,
// 3 outputs written (just before the arrival on the next grid barrier).
__device__ __forceinline__ void stamp(const StreamArgs& a, int si, int k, int tid) {
  if (a.trace != nullptr && tid == 0)
    a.trace[(static_cast<size_t>(blockIdx.x) * a.n_stages + si) * 4 + k] = global_timer_ns();
}
__device__ __forceinline__ void consumer_bar() { asm volatile("bar.sync 1, %0;" ::"n"(kConsumers) : "memory"); }

__device__ __forceinline__ unsigned long long ld_acquire_gpu_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

// Eight bf16 (one 16-byte piece) <-> eight floats.
__device__ __forceinline__ void unpack8(const uint4& raw, float* f) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    f[2 * j] = bf16_lo(w[j]);
    f[2 * j + 1] = bf16_hi(w[j]);
  }
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  return make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]), pack_bf16(f[6], f[7]));
}

// Tiles of a stage that CTA `cta` owns: t0, t0 + G, ...  Returns their count.
__device__ __host__ __forceinline__ int tiles_of(int NT, int rot, int cta, int G, int* t0) {
  const int first = ((cta - rot) % G + G) % G;
  *t0 = first;
  return first < NT ? (NT - first - 1) / G + 1 : 0;
}

// Ring discipline.  Record u of a CTA's stream is consumed by warp u % nw, and the ns slots are
// split into nw private sub-rings (sizes differing by at most one), so a slot is always
// consumed by the same warp.  That matters: a wait on an mbarrier phase is only meaningful
// while the barrier is at most one phase behind, and a warp that consumed the slot's previous
// use knows that it is.
__device__ __forceinline__ void slot_of(unsigned u, int ns, int nw, int* slot, unsigned* use) {
  const int w = static_cast<int>(u % nw);
  const unsigned i = u / nw;
  const int k = ns / nw, r = ns % nw;
  const int n = k + (w < r ? 1 : 0), base = w * k + min(w, r);
  *slot = base + static_cast<int>(i % n);
  *use = i / n;
}

struct Shared {   // the fixed header of dynamic shared memory (kHeaderBytes)
  uint64_t full[kMaxSlots], empty[kMaxSlots];
  uint64_t full2[kMaxHeadSlots], empty2[kMaxHeadSlots];
  float red[8][16];
  float redl[8][16];
  float rinv[8];
  float rope_cos[64], rope_sin[64];   // cos / sin of pos * inv_freq[i]: the same for every head and layer of a step
  __align__(16) uint32_t zeros[8];    // what the lanes of batch columns beyond M read as their x
  int dead;
  int flag;
};
static_assert(sizeof(Shared) <= kHeaderBytes, "header too small");

// ---------------------------------------------------------------------------------------
// grid barrier: arrivals counted in ctl[0]; barrier number nb is passed when the count
// reaches nb * G.  The count returns to zero at the end of the step.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void grid_arrive(const StreamArgs& a) {   // one thread, after consumer_bar
  __threadfence();
  atomicAdd(a.ctl, 1ull);
}
__device__ __forceinline__ void grid_wait(const StreamArgs& a, Shared* sh, int nb, int tid) {
  if (nb > 0 && tid == 0 && !sh->dead) {
    const unsigned long long target = static_cast<unsigned long long>(nb) * gridDim.x;
    bool ok = false;
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
      for (int i = 0; i < 64 && !ok; ++i) ok = ld_acquire_gpu_u64(a.ctl) >= target;
      if (ok || clock64() - t0 > 4000000000ll) break;
    }
    if (!ok) {
      report_timeout(a.status, 600);
      sh->dead = 1;
    }
  }
  if (nb > 0) consumer_bar();
}

// ---------------------------------------------------------------------------------------
// Input staging of a projection: x (bf16, natural order, rows `pitch` apart, zero beyond K up
// to the padded length) and the per-group sums of x that the int4 offset term needs.
// Source kinds:
//   residual + RMSNorm (qkv, gate_up, LM head): xn = bf16(x_old + bf16(y)) (layer 0: the
//       embedding row), written back to the other residual buffer by CTA 0; staged value
//       = bf16(xn * rinv * gain).  x_old and the gain do not depend on the stage before, so
//       they are requested BEFORE the grid barrier; only y waits for it.
//   plain (o, down): the attention output / silu(gate) * up
// The grid barrier in front of the stage (number nb, 0 = none) is taken in here.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void group_sums(float* xsum, const float* v8, int m, int piece, int lane) {
  float s = 0.0f;
#pragma unroll
  for (int j = 0; j < 8; ++j) s += v8[j];
  s += __shfl_xor_sync(0xffffffffu, s, 1);
  s += __shfl_xor_sync(0xffffffffu, s, 2);
  s += __shfl_xor_sync(0xffffffffu, s, 4);
  if ((lane & 7) == 0) xsum[(piece >> 3) * 8 + m] = s;
}

__device__ void stage_inputs(const StreamArgs& a, const Stage& st, Shared* sh, uint8_t* smem, int xcur, bool first_layer,
                             bool work, int nb, int si, int tid) {
  const int lane = tid & 31, warp = tid >> 5;
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(smem + kHeaderBytes);
  float* xsum = reinterpret_cast<float*>(smem + a.off_xsum);
  const int K = st.K, Kpad = st.C * (st.type == kHead ? kHeadUnitK : kUnitK);
  const int pitch = a.xs_pitch;
  const int nvK = K / 8;       // 16-byte pieces of a row
  const int nvec = Kpad / 8;   // ... the zero tail included (a multiple of 64 pieces)
  const bool norm = st.type == kQkv || st.type == kGateUp || st.type == kHead;
  if (!norm) {
    grid_wait(a, sh, nb, tid);
    stamp(a, si, 0, tid);
    if (!work) return;
    const __nv_bfloat16* src = st.type == kO ? a.attn : a.hmlp;
    for (int m = 0; m < a.M; ++m) {
      for (int v0 = 0; v0 < nvec; v0 += 4 * kConsumers) {
        uint4 raw[4];
#pragma unroll
        for (int it = 0; it < 4; ++it) {   // all the loads of the round in flight together
          const int v = v0 + it * kConsumers + tid;
          raw[it] = v < nvK ? __ldcg(reinterpret_cast<const uint4*>(src + static_cast<long long>(m) * K) + v) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int it = 0; it < 4; ++it) {
          const int v = v0 + it * kConsumers + tid;
          if (v < nvec) {   // whole warps: nvec and the warp's first piece are multiples of 32
            float f[8];
            unpack8(raw[it], f);
            *reinterpret_cast<uint4*>(xs + m * pitch + 8 * v) = raw[it];
            group_sums(xsum, f, m, v, lane);
          }
        }
      }
    }
    consumer_bar();
    return;
  }

  // ---- residual + RMSNorm
  // what does not depend on the stage before: the old residual rows (up to 4 of them; a thread's
  // first two pieces of each) and the gain
  uint4 xo[4][2], gn[2];
#pragma unroll
  for (int it = 0; it < 2; ++it) {
    const int v = it * kConsumers + tid;
    gn[it] = make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int m = 0; m < 4; ++m) xo[m][it] = make_uint4(0, 0, 0, 0);
    if (work && v < nvK) {
      gn[it] = __ldg(reinterpret_cast<const uint4*>(st.gain) + v);
#pragma unroll
      for (int m = 0; m < 4; ++m) {
        if (m < a.M) {
          const __nv_bfloat16* xo_row;
          if (first_layer) {
            long long tok = a.tokens[m];
            if (tok < 0 || tok >= a.vocab_full) tok = 0;   // reported below; row 0 instead of memory outside the table
            xo_row = a.embed + tok * K;
          } else {
            xo_row = a.x[xcur] + static_cast<long long>(m) * K;
          }
          xo[m][it] = __ldcg(reinterpret_cast<const uint4*>(xo_row) + v);
        }
      }
    }
  }
  grid_wait(a, sh, nb, tid);
  stamp(a, si, 0, tid);
  if (!work) return;
  if (first_layer && tid < a.M) {
    const long long tok = a.tokens[tid];
    if (tok < 0 || tok >= a.vocab_full) report_status(a.status, B200_INVALID_ARGUMENT, 501);
  }
  // one piece: new residual value, written to shared memory (and by CTA 0 to the other residual buffer)
  auto piece = [&](int m, int v, const uint4& xold, float& ss) {
    float f[8];
    unpack8(xold, f);
    if (!first_layer) {
      const float4 y0 = __ldcg(reinterpret_cast<const float4*>(a.y + static_cast<long long>(m) * K) + 2 * v);
      const float4 y1 = __ldcg(reinterpret_cast<const float4*>(a.y + static_cast<long long>(m) * K) + 2 * v + 1);
      const float yy[8] = {y0.x, y0.y, y0.z, y0.w, y1.x, y1.y, y1.z, y1.w};
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = bf16_round(f[j] + bf16_round(yy[j]));
    }
    const uint4 packed = pack8(f);
    *reinterpret_cast<uint4*>(xs + m * pitch + 8 * v) = packed;
    if (blockIdx.x == 0 && st.type != kHead) *(reinterpret_cast<uint4*>(a.x[xcur ^ 1] + static_cast<long long>(m) * K) + v) = packed;
#pragma unroll
    for (int j = 0; j < 8; ++j) ss = fmaf(f[j], f[j], ss);
  };
#pragma unroll
  for (int m = 0; m < 4; ++m) {
    if (m < a.M) {
      float ss = 0.0f;
#pragma unroll
      for (int it = 0; it < 2; ++it) {
        const int v = it * kConsumers + tid;
        if (v < nvK) piece(m, v, xo[m][it], ss);
      }
      for (int v = 2 * kConsumers + tid; v < nvK; v += kConsumers) {   // rows longer than 7680
        const __nv_bfloat16* xo_row = first_layer ? a.embed + static_cast<long long>(max(0, min(a.tokens[m], static_cast<int>(a.vocab_full - 1)))) * K
                                                  : a.x[xcur] + static_cast<long long>(m) * K;
        piece(m, v, __ldcg(reinterpret_cast<const uint4*>(xo_row) + v), ss);
      }
      ss = warp_sum(ss);
      if (lane == 0) sh->red[m][warp] = ss;
    }
  }
  for (int m = 4; m < a.M; ++m) {   // rows beyond the four kept in registers
    float ss = 0.0f;
    const __nv_bfloat16* xo_row = first_layer ? a.embed + static_cast<long long>(max(0, min(a.tokens[m], static_cast<int>(a.vocab_full - 1)))) * K
                                              : a.x[xcur] + static_cast<long long>(m) * K;
    for (int v = tid; v < nvK; v += kConsumers) piece(m, v, __ldcg(reinterpret_cast<const uint4*>(xo_row) + v), ss);
    ss = warp_sum(ss);
    if (lane == 0) sh->red[m][warp] = ss;
  }
  consumer_bar();
  if (tid < a.M) {
    float t = 0.0f;
#pragma unroll
    for (int w = 0; w < kNW; ++w) t += sh->red[tid][w];
    sh->rinv[tid] = 1.0f / sqrtf(t / static_cast<float>(K) + a.eps);
  }
  consumer_bar();
  // pass 2: normalise in place (every thread revisits the pieces it wrote)
  for (int m = 0; m < a.M; ++m) {
    const float r = sh->rinv[m];
    int it = 0;
    for (int v = tid; v < nvec; v += kConsumers, ++it) {
      float f[8];
      if (v < nvK) {
        float g[8];
        unpack8(*reinterpret_cast<const uint4*>(xs + m * pitch + 8 * v), f);
        unpack8(it == 0 ? gn[0] : (it == 1 ? gn[1] : __ldg(reinterpret_cast<const uint4*>(st.gain) + v)), g);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = bf16_round((f[j] * r) * g[j]);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = 0.0f;
      }
      *reinterpret_cast<uint4*>(xs + m * pitch + 8 * v) = pack8(f);
      group_sums(xsum, f, m, v, lane);
    }
  }
  consumer_bar();
}

// ---------------------------------------------------------------------------------------
// One int4 record: 16 rows x 512 inputs against the batch.  acc: rows g / g+8, batch columns
// 2t / 2t+1 (the m16n8k16 accumulator fragment).
//
// The loads and MMAs are volatile asms in a hand-written software pipeline: per group
//   loads of group gi + 1 | widening of group gi | MMAs of group gi | scaling of group gi - 1
// so that every warp's instruction stream alternates between the pipes and nothing waits for
// the result of the instruction just before it.
// Issue cost per group and scheduler, from microbenchmarks on this GPU: 16 lop3 at 2 cycles,
// 12 shifts at ~1, four bf16 MMAs at 8-12, the loads and the f32 arithmetic ~25: about 100
// cycles, against the 102 that the measured HBM rate leaves for 16 rows x 64 inputs.
// ---------------------------------------------------------------------------------------
struct GroupRegs {
  uint4 w;       // nibbles: rows g / g + 8, 16 inputs each
  uint2 sb;      // (scale, offset) of rows g / g + 8
  uint4 x0, x1;  // 16 inputs of the lane's batch column
  float2 xs2;    // sum of x over the group for batch columns 2t, 2t + 1
};
__device__ __forceinline__ uint4 vlds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
// 16 bytes of x, only in the lanes of a real batch column (the others get zeros without
// touching shared memory)
__device__ __forceinline__ uint4 vlds128_if(uint32_t addr, uint32_t on) {
  uint4 v;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.u32 p, %5, 0;\n\t"
      "mov.u32 %0, 0;\n\tmov.u32 %1, 0;\n\tmov.u32 %2, 0;\n\tmov.u32 %3, 0;\n\t"
      "@p ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];\n\t}"
      : "=&r"(v.x), "=&r"(v.y), "=&r"(v.z), "=&r"(v.w)
      : "r"(addr), "r"(on));
  return v;
}
__device__ __forceinline__ uint2 vlds64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}
__device__ __forceinline__ float2 vlds64f(uint32_t addr) {
  float2 v;
  asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(addr));
  return v;
}
__device__ __forceinline__ void vmma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void vmma_z(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
               : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
}

// xstep: 128 (bytes of x per group) in the lanes of a real batch column, 0 in the others (which
// load nothing and multiply zeros).
template <int MODE = 0>   // MODE > 0: measurement builds that leave parts of the work out (wrong results)
__device__ __forceinline__ void int4_record(uint32_t rec, uint32_t xaddr, uint32_t xstep, uint32_t xsum_addr, int lane,
                                            float (&acc)[4]) {
  const int g = lane >> 2;
  auto load = [&](int gi, GroupRegs& r) {
    r.w = vlds128(rec + gi * 512 + lane * 16);
    r.sb = vlds64(rec + 4096 + gi * 64 + g * 8);
    r.x0 = vlds128_if(xaddr + gi * xstep, xstep);
    r.x1 = vlds128_if(xaddr + gi * xstep + 16, xstep);
    r.xs2 = vlds64f(xsum_addr + gi * 32);
  };
  auto scale = [&](const float (&tmp)[4], const uint2& sb, const float2& xs2) {
    // sum_k x (s q + b) = s * sum_k x (128 + q) + (b - 128 s) * sum_k x
    const float s0 = bf16_lo(sb.x), b0 = bf16_hi(sb.x), s1 = bf16_lo(sb.y), b1 = bf16_hi(sb.y);
    const float o0 = fmaf(-128.0f, s0, b0), o1 = fmaf(-128.0f, s1, b1);
    acc[0] = fmaf(s0, tmp[0], fmaf(o0, xs2.x, acc[0]));
    acc[1] = fmaf(s0, tmp[1], fmaf(o0, xs2.y, acc[1]));
    acc[2] = fmaf(s1, tmp[2], fmaf(o1, xs2.x, acc[2]));
    acc[3] = fmaf(s1, tmp[3], fmaf(o1, xs2.y, acc[3]));
  };
  GroupRegs r[kUnitGroups];
  float tmp[kUnitGroups][4];
  load(0, r[0]);
#pragma unroll
  for (int gi = 0; gi < kUnitGroups; ++gi) {
    if (gi + 1 < kUnitGroups) load(gi + 1, r[gi + 1]);
    const uint4 w = r[gi].w;
    if (MODE == 2) {   // loads only
      acc[0] += __uint_as_float((w.x ^ w.y ^ w.z ^ w.w ^ r[gi].sb.x ^ r[gi].sb.y ^ r[gi].x0.x ^ r[gi].x0.y ^ r[gi].x0.z ^ r[gi].x0.w ^
                                 r[gi].x1.x ^ r[gi].x1.y ^ r[gi].x1.z ^ r[gi].x1.w) & 0x3fffffffu) + r[gi].xs2.x + r[gi].xs2.y;
      continue;
    }
    uint32_t a0[8], a1[8];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      a0[q] = lop3_and_or(q == 0 ? w.x : shr4(w.x, q), 0x000f000fu, 0x43004300u);   // bf16 (128 + q) pairs
      a0[4 + q] = lop3_and_or(q == 0 ? w.y : shr4(w.y, q), 0x000f000fu, 0x43004300u);
      a1[q] = lop3_and_or(q == 0 ? w.z : shr4(w.z, q), 0x000f000fu, 0x43004300u);
      a1[4 + q] = lop3_and_or(q == 0 ? w.w : shr4(w.w, q), 0x000f000fu, 0x43004300u);
    }
    if (MODE == 3) {   // loads + widening
      uint32_t z = r[gi].sb.x ^ r[gi].sb.y ^ r[gi].x0.x ^ r[gi].x0.y ^ r[gi].x0.z ^ r[gi].x0.w ^ r[gi].x1.x ^ r[gi].x1.y ^ r[gi].x1.z ^ r[gi].x1.w;
#pragma unroll
      for (int q = 0; q < 8; ++q) z ^= a0[q] ^ a1[q];
      acc[0] += __uint_as_float(z & 0x3fffffffu) + r[gi].xs2.x + r[gi].xs2.y;
      continue;
    }
    vmma_z(tmp[gi], a0[0], a1[0], a0[1], a1[1], r[gi].x0.x, r[gi].x0.y);
    vmma(tmp[gi], a0[2], a1[2], a0[3], a1[3], r[gi].x0.z, r[gi].x0.w);
    vmma(tmp[gi], a0[4], a1[4], a0[5], a1[5], r[gi].x1.x, r[gi].x1.y);
    vmma(tmp[gi], a0[6], a1[6], a0[7], a1[7], r[gi].x1.z, r[gi].x1.w);
    if (MODE == 4) {   // no scale / offset arithmetic
      acc[0] += tmp[gi][0] + __uint_as_float((r[gi].sb.x ^ r[gi].sb.y) & 0x3fffffffu) + r[gi].xs2.x;
      acc[1] += tmp[gi][1] + r[gi].xs2.y;
      acc[2] += tmp[gi][2];
      acc[3] += tmp[gi][3];
      continue;
    }
    if (gi > 0) scale(tmp[gi - 1], r[gi - 1].sb, r[gi - 1].xs2);   // the MMAs of the group before have had a group's time to finish
  }
  if (MODE == 0) scale(tmp[kUnitGroups - 1], r[kUnitGroups - 1].sb, r[kUnitGroups - 1].xs2);
}

// 8 bf16 rows x `groups` groups of 64 inputs (one LM-head unit), accumulated into acc[0..1] (rows
// g; the MMA's rows 8..15 are fed zeros).  The same pipeline: the loads of group gi + 1 are issued
// before the MMAs of group gi.
__device__ __forceinline__ void bf16_unit(uint32_t unit, uint32_t xaddr, uint32_t xstep, int groups, int lane, float (&acc)[4]) {
  const int g = lane >> 2, t = lane & 3;
  const uint32_t r0 = unit + g * kHeadRowPitch + t * 32;
  float acc2[4] = {0.0f, 0.0f, 0.0f, 0.0f};   // a second, independent accumulation chain
  uint4 p0 = vlds128(r0), p1 = vlds128(r0 + 16);
  uint4 x0 = vlds128_if(xaddr, xstep), x1 = vlds128_if(xaddr + 16, xstep);
#pragma unroll 4
  for (int gi = 0; gi < groups; ++gi) {
    // (the last iteration loads the last group again: never used)
    const uint32_t nx = static_cast<uint32_t>(min(gi + 1, groups - 1));
    const uint4 np0 = vlds128(r0 + nx * 128), np1 = vlds128(r0 + nx * 128 + 16);
    const uint4 nx0 = vlds128_if(xaddr + nx * xstep, xstep), nx1 = vlds128_if(xaddr + nx * xstep + 16, xstep);
    vmma(acc, p0.x, 0u, p0.y, 0u, x0.x, x0.y);
    vmma(acc2, p0.z, 0u, p0.w, 0u, x0.z, x0.w);
    vmma(acc, p1.x, 0u, p1.y, 0u, x1.x, x1.y);
    vmma(acc2, p1.z, 0u, p1.w, 0u, x1.z, x1.w);
    p0 = np0; p1 = np1; x0 = nx0; x1 = nx1;
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) acc[i] += acc2[i];
}

// ---------------------------------------------------------------------------------------
// Attention stage (qwen3.py:363-372 at T = 1): per-head RMSNorm + rotate-half RoPE of q and of
// the new k, the cache writes at *pos, scores, f32 softmax, p.v.  A unit is one chunk of
// positions of one (sequence, KV head) with all G query heads; the CTA that finishes a
// (sequence, KV head)'s last chunk merges its partials.  The first 256 consumer threads do
// the arithmetic; the K and V bytes of a CTA's first window are requested before the grid
// barrier in front of the stage (they are older than this step, and the producer warp asked
// for them to be brought into L2 while the projection before was running).
// ---------------------------------------------------------------------------------------
template <int D>
__device__ __forceinline__ void norm_rope_head(const __nv_bfloat16* src, const __nv_bfloat16* w, float eps, const Shared* sh,
                                               int lane, float* dst1, float* dst2) {
  constexpr int PAIRS = D / 64;
  float x1[PAIRS], x2[PAIRS];
  float ss = 0.0f;
#pragma unroll
  for (int p = 0; p < PAIRS; ++p) {
    const int i = lane + 32 * p;
    x1[p] = bf16_bits_to_f32(__ldcg(reinterpret_cast<const unsigned short*>(src) + i));
    x2[p] = bf16_bits_to_f32(__ldcg(reinterpret_cast<const unsigned short*>(src) + i + D / 2));
    ss = fmaf(x1[p], x1[p], ss);
    ss = fmaf(x2[p], x2[p], ss);
  }
  ss = warp_sum(ss);
  const float r = 1.0f / sqrtf(ss / static_cast<float>(D) + eps);
#pragma unroll
  for (int p = 0; p < PAIRS; ++p) {
    const int i = lane + 32 * p;
    const float n1 = bf16_round((x1[p] * r) * __bfloat162float(w[i]));
    const float n2 = bf16_round((x2[p] * r) * __bfloat162float(w[i + D / 2]));
    const float cs = sh->rope_cos[i], sn = sh->rope_sin[i];
    dst1[i] = bf16_round(n1 * cs - n2 * sn);
    dst2[i] = bf16_round(n2 * cs + n1 * sn);
  }
}

template <int D, int G>
__device__ void attention_stage(const StreamArgs& a, const Stage& st, Shared* sh, uint8_t* smem, int nb, int si, int tid) {
  constexpr int HALF = D / 2;
  constexpr int KV4 = HALF / 8;                 // 16-byte loads of K per thread (two threads per position)
  constexpr int W = kAttnWindow;
  constexpr int VH = kAttnThreads / D;          // threads per output dimension (2 or 4)
  constexpr int SPAN = W / VH;                  // positions per such thread and window
  constexpr int NWA = kAttnThreads / 32;        // warps that compute
  const int lane = tid & 31, warp = tid >> 5;
  const bool act = tid < kAttnThreads;
  // scratch in the (idle) x staging area
  float* base = reinterpret_cast<float*>(smem + kHeaderBytes);
  float(*qs)[2][HALF + 4] = reinterpret_cast<float(*)[2][HALF + 4]>(base);
  base += G * 2 * (HALF + 4);
  float(*sc)[W] = reinterpret_cast<float(*)[W]>(base);
  base += G * W;
  float(*knew)[HALF + 4] = reinterpret_cast<float(*)[HALF + 4]>(base);
  base += 2 * (HALF + 4);
  float* vnew = base;
  base += D;
  float* accs = base;   // [VH][G][D]
  base += VH * G * D;
  float* wsm = base;    // [G][kMaxChunks + 1] merge weights, then 1 / denominator

  const int pos = *a.pos;
  const bool bad = pos < 0 || pos >= a.max_len;
  const int n_valid = pos + 1;
  const int chunk_len = bad ? 8 : ((n_valid + a.attn_chunks - 1) / a.attn_chunks + 7) & ~7;
  const int nch = bad ? 0 : (n_valid + chunk_len - 1) / chunk_len;
  const int units = a.M * a.KV * nch;
  const int total_heads = a.H + 2 * a.KV;
  const int p = (tid >> 1) & (W - 1), half = tid & 1;            // scores: position p of the window, half of the head dim
  const int vd = tid % D, vh = (tid / D) % VH;                    // p.v: output dimension vd, positions [vh * SPAN, + SPAN)

  uint4 kreg[KV4], vreg[SPAN / 8];
  auto load_window = [&](int bk, int w0, int cnt) {
    // slots below pos; slot pos itself comes from shared memory
    const __nv_bfloat16* kbase = st.k_cache + static_cast<long long>(bk) * a.max_len * D;
    const __nv_bfloat16* vbase = st.v_cache + static_cast<long long>(bk) * D * a.max_len;
    const bool have = act && p < cnt && w0 + p < pos;
    const uint4* krow = reinterpret_cast<const uint4*>(kbase + static_cast<long long>(w0 + p) * D + half * HALF);
#pragma unroll
    for (int v = 0; v < KV4; ++v) kreg[v] = have ? __ldcg(krow + v) : make_uint4(0, 0, 0, 0);
    const int vs0 = w0 + vh * SPAN;
    const __nv_bfloat16* vrow = vbase + static_cast<long long>(vd) * a.max_len + vs0;
#pragma unroll
    for (int j = 0; j < SPAN / 8; ++j)
      vreg[j] = (act && vs0 + 8 * j < pos) ? __ldcg(reinterpret_cast<const uint4*>(vrow + 8 * j)) : make_uint4(0, 0, 0, 0);
  };
  bool preloaded = false;
  if (static_cast<int>(blockIdx.x) < units) {
    const int u = blockIdx.x;
    const int ch = u % nch, bk = u / nch;
    const int s_begin = ch * chunk_len;
    load_window(bk, s_begin, min(W, min(n_valid, s_begin + chunk_len) - s_begin));
    preloaded = true;
  }
  grid_wait(a, sh, nb, tid);
  stamp(a, si, 0, tid);
  if (bad) {   // nothing may be written outside the cache
    if (tid == 0) report_status(a.status, B200_INVALID_ARGUMENT, 500);
    return;
  }

  for (int u = blockIdx.x; u < units; u += gridDim.x) {
    const int ch = u % nch, bk = u / nch;
    const int b = bk / a.KV, kv = bk % a.KV;
    const int s_begin = ch * chunk_len, s_end = min(n_valid, s_begin + chunk_len);
    const bool owner = pos >= s_begin && pos < s_end;
    const __nv_bfloat16* row = a.qkv + static_cast<long long>(b) * total_heads * D;

    if (warp < NWA) {
      for (int gq = warp; gq < G; gq += NWA)
        norm_rope_head<D>(row + static_cast<long long>(kv * G + gq) * D, st.q_norm, a.eps, sh, lane, qs[gq][0], qs[gq][1]);
      if (owner) {
        if (warp == (G % NWA)) {
          norm_rope_head<D>(row + static_cast<long long>(a.H + kv) * D, st.k_norm, a.eps, sh, lane, knew[0], knew[1]);
          __syncwarp();
          __nv_bfloat16* kdst = st.k_cache + (static_cast<long long>(bk) * a.max_len + pos) * D;
          for (int i = lane; i < HALF; i += 32) {
            kdst[i] = __float2bfloat16_rn(knew[0][i]);
            kdst[i + HALF] = __float2bfloat16_rn(knew[1][i]);
          }
        } else if (warp == ((G + 1) % NWA)) {
          const unsigned short* vsrc = reinterpret_cast<const unsigned short*>(row + static_cast<long long>(a.H + a.KV + kv) * D);
          unsigned short* vdst = reinterpret_cast<unsigned short*>(st.v_cache) + static_cast<long long>(bk) * D * a.max_len + pos;
          for (int d = lane; d < D; d += 32) {
            const unsigned short v = __ldcg(vsrc + d);
            vnew[d] = bf16_bits_to_f32(v);
            vdst[static_cast<long long>(d) * a.max_len] = v;
          }
        }
      }
    }
    consumer_bar();

    float m_run[G], l_run[G], acc[G];
#pragma unroll
    for (int gq = 0; gq < G; ++gq) {
      m_run[gq] = -INFINITY;
      l_run[gq] = 0.0f;
      acc[gq] = 0.0f;
    }
    for (int w0 = s_begin; w0 < s_end; w0 += W) {
      const int cnt = min(W, s_end - w0);
      if (!preloaded) load_window(bk, w0, cnt);
      preloaded = false;
      const int vs0 = w0 + vh * SPAN;
      // ---- scores
      float dot[G];
#pragma unroll
      for (int gq = 0; gq < G; ++gq) dot[gq] = 0.0f;
      const bool from_smem = owner && w0 + p == pos;
#pragma unroll
      for (int v = 0; v < KV4; ++v) {
        float kf[8];
        if (from_smem) {
#pragma unroll
          for (int j = 0; j < 8; ++j) kf[j] = knew[half][v * 8 + j];
        } else {
          unpack8(kreg[v], kf);
        }
#pragma unroll
        for (int gq = 0; gq < G; ++gq) {
          const float4 q0 = *reinterpret_cast<const float4*>(&qs[gq][half][v * 8]);
          const float4 q1 = *reinterpret_cast<const float4*>(&qs[gq][half][v * 8 + 4]);
          dot[gq] = fmaf(q0.x, kf[0], dot[gq]);
          dot[gq] = fmaf(q0.y, kf[1], dot[gq]);
          dot[gq] = fmaf(q0.z, kf[2], dot[gq]);
          dot[gq] = fmaf(q0.w, kf[3], dot[gq]);
          dot[gq] = fmaf(q1.x, kf[4], dot[gq]);
          dot[gq] = fmaf(q1.y, kf[5], dot[gq]);
          dot[gq] = fmaf(q1.z, kf[6], dot[gq]);
          dot[gq] = fmaf(q1.w, kf[7], dot[gq]);
        }
      }
#pragma unroll
      for (int gq = 0; gq < G; ++gq) {
        dot[gq] += __shfl_xor_sync(0xffffffffu, dot[gq], 1);   // the two halves of the head dim
        const float s = (act && p < cnt) ? dot[gq] * a.attn_scale : -INFINITY;
        if (act && half == 0) sc[gq][p] = s;
        const float mw = warp_max(s);
        if (lane == 0 && warp < NWA) sh->red[gq][warp] = mw;
      }
      consumer_bar();
      float corr[G];
#pragma unroll
      for (int gq = 0; gq < G; ++gq) {
        float m = sh->red[gq][0];
#pragma unroll
        for (int w = 1; w < NWA; ++w) m = fmaxf(m, sh->red[gq][w]);
        const float m_new = fmaxf(m_run[gq], m);
        corr[gq] = m_run[gq] == -INFINITY ? 0.0f : expf(m_run[gq] - m_new);
        m_run[gq] = m_new;
        float e = 0.0f;
        if (tid < W) {
          e = tid < cnt ? expf(sc[gq][tid] - m_new) : 0.0f;
          sc[gq][tid] = e;
        }
        e = warp_sum(e);
        if (lane == 0 && warp < NWA) sh->redl[gq][warp] = e;   // warps beyond W / 32 write zero
      }
      consumer_bar();
#pragma unroll
      for (int gq = 0; gq < G; ++gq) {
        float l = 0.0f;
#pragma unroll
        for (int w = 0; w < NWA; ++w) l += sh->redl[gq][w];
        l_run[gq] = l_run[gq] * corr[gq] + l;
        acc[gq] *= corr[gq];
      }
      // ---- p . v over this thread's positions of the window
      if (act) {
#pragma unroll
        for (int j = 0; j < SPAN / 8; ++j) {
          float v[8];
          unpack8(vreg[j], v);
          if (vs0 + 8 * j + 8 > pos) {   // only the window that holds the newest position has such slots
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              const int s = vs0 + 8 * j + e;
              if (s >= pos) v[e] = (owner && s == pos) ? vnew[vd] : 0.0f;
            }
          }
#pragma unroll
          for (int gq = 0; gq < G; ++gq) {
            const float4 p0 = *reinterpret_cast<const float4*>(&sc[gq][vh * SPAN + 8 * j]);
            const float4 p1 = *reinterpret_cast<const float4*>(&sc[gq][vh * SPAN + 8 * j + 4]);
            acc[gq] = fmaf(p0.x, v[0], acc[gq]);
            acc[gq] = fmaf(p0.y, v[1], acc[gq]);
            acc[gq] = fmaf(p0.z, v[2], acc[gq]);
            acc[gq] = fmaf(p0.w, v[3], acc[gq]);
            acc[gq] = fmaf(p1.x, v[4], acc[gq]);
            acc[gq] = fmaf(p1.y, v[5], acc[gq]);
            acc[gq] = fmaf(p1.z, v[6], acc[gq]);
            acc[gq] = fmaf(p1.w, v[7], acc[gq]);
          }
        }
      }
      if (w0 + W < s_end) consumer_bar();   // sc / red are rewritten by the next window
    }
    // ---- this unit's partial: sum p v (unnormalised), running max, sum p
    if (act) {
#pragma unroll
      for (int gq = 0; gq < G; ++gq) accs[(vh * G + gq) * D + vd] = acc[gq];
    }
    consumer_bar();
    float* part = a.attn_part + (static_cast<long long>(bk) * kMaxChunks + ch) * G * (D + 2);
    for (int i = tid; i < G * D; i += kConsumers) {
      const int gq = i / D, d = i % D;
      float v = 0.0f;
#pragma unroll
      for (int h2 = 0; h2 < VH; ++h2) v += accs[(h2 * G + gq) * D + d];
      part[gq * (D + 2) + d] = v;
    }
    if (tid < G) {
      part[tid * (D + 2) + D] = m_run[tid];
      part[tid * (D + 2) + D + 1] = l_run[tid];
    }
    consumer_bar();
    if (tid == 0) {
      __threadfence();
      const unsigned old = atomicAdd(a.attn_cnt + bk, 1u);
      sh->flag = old == static_cast<unsigned>(nch - 1);
      if (sh->flag) a.attn_cnt[bk] = 0u;
    }
    consumer_bar();
    if (sh->flag) {
      __threadfence();
      // merge: out = sum_c e^{m_c - M} o_c / sum_c e^{m_c - M} l_c.  Weights: one warp per query head.
      const float* pb = a.attn_part + static_cast<long long>(bk) * kMaxChunks * G * (D + 2);
      if (warp < G) {
        const int gq = warp;
        const int c0 = lane, c1 = lane + 32;
        const float m0 = c0 < nch ? __ldcg(pb + (c0 * G + gq) * (D + 2) + D) : -INFINITY;
        const float m1 = c1 < nch ? __ldcg(pb + (c1 * G + gq) * (D + 2) + D) : -INFINITY;
        const float l0 = c0 < nch ? __ldcg(pb + (c0 * G + gq) * (D + 2) + D + 1) : 0.0f;
        const float l1 = c1 < nch ? __ldcg(pb + (c1 * G + gq) * (D + 2) + D + 1) : 0.0f;
        const float mall = warp_max(fmaxf(m0, m1));
        const float w0 = c0 < nch ? expf(m0 - mall) : 0.0f, w1 = c1 < nch ? expf(m1 - mall) : 0.0f;
        wsm[gq * (kMaxChunks + 1) + c0] = w0;
        wsm[gq * (kMaxChunks + 1) + c1] = w1;
        const float den = warp_sum(fmaf(w0, l0, w1 * l1));
        if (lane == 0) wsm[gq * (kMaxChunks + 1) + kMaxChunks] = 1.0f / den;
      }
      consumer_bar();
      // outputs: every consumer thread, the partials of 16 chunks requested together
      for (int i = tid; i < G * D; i += kConsumers) {
        const int gq = i / D, d = i % D;
        const float* wq = wsm + gq * (kMaxChunks + 1);
        float num = 0.0f;
        for (int c0 = 0; c0 < nch; c0 += 16) {
          float v[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = c0 + j < nch ? __ldcg(pb + ((c0 + j) * G + gq) * (D + 2) + d) : 0.0f;
#pragma unroll
          for (int j = 0; j < 16; ++j) num = fmaf(wq[min(c0 + j, kMaxChunks - 1)], v[j], num);
        }
        a.attn[(static_cast<long long>(b) * a.H + kv * G + gq) * D + d] = __float2bfloat16_rn(num * wq[kMaxChunks]);
      }
    }
    consumer_bar();   // the scratch is reused by this CTA's next unit
  }
}

// Asks for this CTA's K and V bytes of a layer's attention stage to be brought into L2.  Called
// by the consumer threads a stage early (while the qkv projection runs); the attention stage
// then requests them before its grid barrier.
__device__ __forceinline__ void prefetch_kv(const StreamArgs& a, const Stage& st, int pos, int tid) {
  if (pos < 0 || pos >= a.max_len) return;
  const int n_valid = pos + 1, D = a.D;
  const int chunk_len = ((n_valid + a.attn_chunks - 1) / a.attn_chunks + 7) & ~7;
  const int nch = (n_valid + chunk_len - 1) / chunk_len;
  const int units = a.M * a.KV * nch;
  for (int u = blockIdx.x; u < units; u += gridDim.x) {
    const int ch = u % nch, bk = u / nch;
    const int s_begin = ch * chunk_len, cnt = min(n_valid, s_begin + chunk_len) - s_begin;
    const uint8_t* kb = reinterpret_cast<const uint8_t*>(st.k_cache + (static_cast<long long>(bk) * a.max_len + s_begin) * D);
    const int kbytes = cnt * D * 2;
    for (int off = tid * 2048; off < kbytes; off += kConsumers * 2048) prefetch_l2(kb + off, static_cast<uint32_t>(min(2048, kbytes - off)));
    const uint32_t vbytes = static_cast<uint32_t>(((cnt + 7) & ~7) * 2);
    for (int d = kConsumers - 1 - tid; d < D; d += kConsumers)
      prefetch_l2(st.v_cache + (static_cast<long long>(bk) * D + d) * a.max_len + s_begin, vbytes);
  }
}

// ---------------------------------------------------------------------------------------
// The kernel
// ---------------------------------------------------------------------------------------
template <int D, int G>
__global__ void __launch_bounds__(kThreads, 1) decode_stream_kernel(const StreamArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  Shared* sh = reinterpret_cast<Shared*>(smem);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int cta = blockIdx.x, nctas = gridDim.x;
  uint8_t* ring = smem + a.off_ring;
  const int nw2 = min(kNW, a.NS2);   // warps that take LM-head units

  if (tid == 0) {
    for (int s = 0; s < a.NS; ++s) {
      mbar_init(&sh->full[s], 1);
      mbar_init(&sh->empty[s], 1);
    }
    for (int s = 0; s < a.NS2; ++s) {
      mbar_init(&sh->full2[s], 1);
      mbar_init(&sh->empty2[s], 1);
    }
    sh->dead = 0;
    sh->flag = 0;
    for (int i = 0; i < 8; ++i) sh->zeros[i] = 0u;
    mbar_fence_init();
  }
  const int pos0 = *a.pos;
  if (tid < D / 2) {
    float sn, cs;
    sincosf(static_cast<float>(pos0) * a.inv_freq[tid], &sn, &cs);
    sh->rope_cos[tid] = cs;
    sh->rope_sin[tid] = sn;
  }
  // columns of the group sums beyond the batch are read (and multiplied into unused
  // accumulator columns): keep them finite
  for (int i = tid; i < (a.off_part - a.off_xsum) / 4; i += kThreads) reinterpret_cast<float*>(smem + a.off_xsum)[i] = 0.0f;
  __syncthreads();

  const Stage& head = a.stages[a.n_stages - 1];   // the LM head is always the last stage
  int head_t0;
  const int head_tiles = tiles_of(head.NT, head.rot, cta, nctas, &head_t0);
  const int head_chunks = head.C;

  if (warp == kNW) {
    // ================= producer warp: the CTA's weight stream, start to end =================
    // Lane w serves consumer warp w: it copies that warp's records (u = w, w + 15, ...) into the
    // warp's private slots, one bulk copy per record, never waiting for anything but those
    // slots.  (One lane for the whole stream was the bottleneck: a few hundred cycles of
    // dependent work per record.)
    bool dead = false;
    const unsigned n1 = a.cta_units[cta];
    const uint8_t* src = a.packed + a.cta_off[cta];
    if (lane < kNW) {
      const int w = lane;
      const int k = a.NS / kNW, r = a.NS % kNW;
      const int n = k + (w < r ? 1 : 0), base = w * k + min(w, r);
      const unsigned cnt = n1 > static_cast<unsigned>(w) ? (n1 - 1 - w) / kNW + 1 : 0;
      int s = 0;          // slot within the sub-ring
      unsigned use = 0;   // times the sub-ring has wrapped
      for (unsigned i = 0; i < cnt && !dead; ++i) {
        uint64_t* fullb = &sh->full[base + s];
        if (use > 0 && !mbar_wait_bounded<32>(&sh->empty[base + s], (use - 1) & 1)) {
          report_timeout(a.status, 610);
          dead = true;
          sh->dead = 1;
          break;
        }
        mbar_expect_tx(fullb, kUnitBytes);
        bulk_g2s(ring + static_cast<size_t>(base + s) * kUnitBytes, src + (static_cast<size_t>(i) * kNW + w) * kUnitBytes,
                 kUnitBytes, fullb);
        if (++s == n) {
          s = 0;
          ++use;
        }
      }
      // the LM-head units use the same bytes with another slot size: wait until this warp's last records are consumed
      for (unsigned i = cnt > static_cast<unsigned>(n) ? cnt - n : 0; i < cnt && !dead; ++i) {
        if (!mbar_wait_bounded<32>(&sh->empty[base + static_cast<int>(i % n)], (i / n) & 1)) {
          report_timeout(a.status, 611);
          dead = true;
          sh->dead = 1;
        }
      }
    }
    dead = __any_sync(0xffffffffu, dead);
    // LM head: unit u2 = (tile u2 / C, chunk u2 % C) of this CTA's 8-row tiles, a 2 KB copy per row;
    // lane w serves warp w here too
    const unsigned n2 = static_cast<unsigned>(head_tiles) * head_chunks;
    if (lane < nw2 && !dead) {
      const int w = lane;
      const int k = a.NS2 / nw2, r = a.NS2 % nw2;
      const int n = k + (w < r ? 1 : 0), base = w * k + min(w, r);
      int s = 0;
      unsigned use = 0;
      for (unsigned u2 = w; u2 < n2; u2 += nw2) {
        uint64_t* fullb = &sh->full2[base + s];
        if (use > 0 && !mbar_wait_bounded<32>(&sh->empty2[base + s], (use - 1) & 1)) {
          report_timeout(a.status, 612);
          sh->dead = 1;
          break;
        }
        const int tl = static_cast<int>(u2 / head_chunks), c = static_cast<int>(u2 % head_chunks);
        const int k0 = c * kHeadUnitK;
        const uint32_t row_bytes = static_cast<uint32_t>(min(kHeadUnitK, head.K - k0) * 2);
        const long long tile = head_t0 + static_cast<long long>(tl) * nctas;
        const int rows_valid = static_cast<int>(min(static_cast<long long>(kHeadRows), head.N - tile * kHeadRows));
        mbar_expect_tx(fullb, row_bytes * rows_valid);
        uint8_t* dst = ring + static_cast<size_t>(base + s) * kHeadUnitBytes;
        const uint8_t* row = a.head_w + (tile * kHeadRows * head.K + k0) * 2;
        for (int rr = 0; rr < rows_valid; ++rr) bulk_g2s(dst + rr * kHeadRowPitch, row + static_cast<long long>(rr) * head.K * 2, row_bytes, fullb);
        if (++s == n) {
          s = 0;
          ++use;
        }
      }
    }
    return;
  }

  // ================= consumer warps ==========================================================
  const int g = lane >> 2, t = lane & 3;
  const uint32_t ring0 = smem_u32(ring);
  const uint32_t xs0 = smem_u32(smem + kHeaderBytes);
  const uint32_t xsum0 = smem_u32(smem + a.off_xsum);
  float* part = reinterpret_cast<float*>(smem + a.off_part);
  const bool have_x = g < a.M;
  const uint32_t x_lane = have_x ? xs0 + static_cast<uint32_t>(g * a.xs_pitch * 2 + t * 32) : smem_u32(sh->zeros);
  const uint32_t xstep = have_x ? 128u : 0u;                // bytes of x per group
  const uint32_t xchunk = have_x ? kUnitK * 2u : 0u;        // ... per record
  const uint32_t xchunk2 = have_x ? kHeadUnitK * 2u : 0u;   // ... per LM-head unit
  // this warp's private part of the rings
  const int k1 = a.NS / kNW, r1 = a.NS % kNW;
  const int ns_w = k1 + (warp < r1 ? 1 : 0), base_w = warp * k1 + min(warp, r1);
  const int k2 = a.NS2 / nw2, r2 = a.NS2 % nw2;
  const int ns2_w = k2 + (warp < r2 ? 1 : 0), base2_w = warp * k2 + min(warp, r2);
  unsigned ubase = 0;   // records of this CTA consumed by earlier stages
  int nb = 0;           // grid barriers passed
  int xcur = 0;         // residual buffer holding the current x
  bool first_layer = true;

  for (int si = 0; si < a.n_stages; ++si) {
    const Stage& st = a.stages[si];
    const int wait_nb = si > 0 ? ++nb : 0;
    if (st.type == kAttn) {
      if (!sh->dead) attention_stage<D, G>(a, st, sh, smem, wait_nb, si, tid);
      else grid_wait(a, sh, wait_nb, tid);
      consumer_bar();
      stamp(a, si, 3, tid);
      if (tid == 0) grid_arrive(a);
      continue;
    }
    int t0;
    const int n_my = tiles_of(st.NT, st.rot, cta, nctas, &t0);
    const bool norm = st.type == kQkv || st.type == kGateUp || st.type == kHead;
    // (CTA 0 writes the new residual row even when it owns no tile of this stage)
    stage_inputs(a, st, sh, smem, xcur, first_layer, n_my > 0 || (cta == 0 && norm), wait_nb, si, tid);
    if (norm) {
      if (st.type != kHead) xcur ^= 1;
      first_layer = false;
    }
    stamp(a, si, 1, tid);
    if (st.type == kQkv) prefetch_kv(a, a.stages[si + 1], pos0, tid);   // the attention stage always follows

    if (st.type != kHead) {
      // ---- int4 projection: record j = (tile j / C, chunk j % C); record u of the CTA's stream
      // goes to warp u % kNW
      const int total = n_my * st.C;
      for (int j = (warp + kNW - static_cast<int>(ubase % kNW)) % kNW; j < total; j += kNW) {
        const unsigned i = (ubase + j) / kNW;
        const int s = base_w + static_cast<int>(i % ns_w);
        if (!sh->dead && !mbar_wait_bounded(&sh->full[s], (i / ns_w) & 1)) {
          report_timeout(a.status, 620);
          sh->dead = 1;
        }
        const int chunk = j % st.C;
        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        uint32_t rec = ring0 + static_cast<uint32_t>(s) * kUnitBytes, xa = x_lane + chunk * xchunk;
        uint32_t xsa = xsum0 + static_cast<uint32_t>((chunk * kUnitGroups * 8 + 2 * t) * 4);
        pin_addresses(rec, xa, xsa);
        if (a.ablate == 0) int4_record<0>(rec, xa, xstep, xsa, lane, acc);
        else if (a.ablate == 2) int4_record<2>(rec, xa, xstep, xsa, lane, acc);
        else if (a.ablate == 3) int4_record<3>(rec, xa, xstep, xsa, lane, acc);
        else if (a.ablate == 4) int4_record<4>(rec, xa, xstep, xsa, lane, acc);
        pin_results(acc);
        __syncwarp();
        if (lane == 0) mbar_arrive(&sh->empty[s]);
        if (2 * t < a.MP) {
          float* pt = part + j * 16 * a.MP;   // [16 rows][MP batch columns]
          *reinterpret_cast<float2*>(pt + g * a.MP + 2 * t) = make_float2(acc[0], acc[1]);
          *reinterpret_cast<float2*>(pt + (g + 8) * a.MP + 2 * t) = make_float2(acc[2], acc[3]);
        }
      }
      ubase += total;
      stamp(a, si, 2, tid);
      consumer_bar();
      // ---- outputs: the records of a row are added in chunk order
      if (st.type == kGateUp) {
        // a tile holds eight gate rows and the eight up rows that go with them:
        // silu(gate) * up with the reference's three roundings (qwen3.py:376), written once
        const int outs = n_my * 8 * a.M;
        for (int idx = tid; idx < outs; idx += kConsumers) {
          const int m = idx / (n_my * 8), rr = idx % (n_my * 8);
          const int tl = rr >> 3, r = rr & 7;
          float vg = 0.0f, vu = 0.0f;
          for (int c = 0; c < st.C; ++c) {
            vg += part[((tl * st.C + c) * 16 + r) * a.MP + m];
            vu += part[((tl * st.C + c) * 16 + r + 8) * a.MP + m];
          }
          const float gate = bf16_round(vg), up = bf16_round(vu);
          const float sig = bf16_round(1.0f / (1.0f + expf(-gate)));
          const long long n = (t0 + static_cast<long long>(tl) * nctas) * 8 + r;
          a.hmlp[static_cast<long long>(m) * a.I + n] = __float2bfloat16_rn(bf16_round(gate * sig) * up);
        }
      } else {
        const int outs = n_my * 16 * a.M;
        for (int idx = tid; idx < outs; idx += kConsumers) {
          const int m = idx / (n_my * 16), rr = idx % (n_my * 16);
          const int tl = rr >> 4, r = rr & 15;
          float v = 0.0f;
          for (int c = 0; c < st.C; ++c) v += part[((tl * st.C + c) * 16 + r) * a.MP + m];
          const long long n = (t0 + static_cast<long long>(tl) * nctas) * 16 + r;
          if (st.type == kQkv) a.qkv[static_cast<long long>(m) * st.N + n] = __float2bfloat16_rn(v);
          else a.y[static_cast<long long>(m) * st.N + n] = v;   // o, down: the residual add is the next staging's
        }
      }
    } else {
      // ---- LM head: the same scheme over bf16 rows, in rounds of as many tiles as the partial
      // buffer holds (a CTA has dozens of tiles here)
      const int round_tiles = a.part_units / st.C;
      for (int r0 = 0; r0 < n_my; r0 += round_tiles) {
        const int rt = min(round_tiles, n_my - r0);
        const int j0 = r0 * st.C, total = rt * st.C;
        if (warp < nw2) {
          for (int j = (warp + nw2 - (j0 % nw2)) % nw2; j < total; j += nw2) {
            const unsigned i = static_cast<unsigned>(j0 + j) / nw2;
            const int s = base2_w + static_cast<int>(i % ns2_w);
            if (!sh->dead && !mbar_wait_bounded(&sh->full2[s], (i / ns2_w) & 1)) {
              report_timeout(a.status, 621);
              sh->dead = 1;
            }
            const int chunk = j % st.C;
            const int groups = min(kHeadUnitK, st.K - chunk * kHeadUnitK) / 64;
            float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            uint32_t unit = ring0 + static_cast<uint32_t>(s) * kHeadUnitBytes, xa = x_lane + chunk * xchunk2, zero = 0;
            pin_addresses(unit, xa, zero);
            if (a.ablate != 1) bf16_unit(unit, xa, xstep, groups, lane, acc);
            pin_results(acc);
            __syncwarp();
            if (lane == 0) mbar_arrive(&sh->empty2[s]);
            if (2 * t < a.MP) *reinterpret_cast<float2*>(part + (j * 16 + g) * a.MP + 2 * t) = make_float2(acc[0], acc[1]);
          }
        }
        consumer_bar();
        // logits are the bf16-rounded products widened to f32 (qwen3.py:389-390)
        const int outs = rt * kHeadRows * a.M;
        for (int idx = tid; idx < outs; idx += kConsumers) {
          const int m = idx / (rt * kHeadRows), rr = idx % (rt * kHeadRows);
          const int tl = rr / kHeadRows, r = rr % kHeadRows;
          float v = 0.0f;
          for (int c = 0; c < st.C; ++c) v += part[((tl * st.C + c) * 16 + r) * a.MP + m];
          const long long n = (t0 + static_cast<long long>(r0 + tl) * nctas) * kHeadRows + r;
          if (n < st.N) a.logits[static_cast<long long>(m) * st.N + n] = bf16_round(v);
        }
        consumer_bar();   // the partial buffer is rewritten by the next round
      }
    }
    if (si + 1 < a.n_stages) {
      consumer_bar();
      stamp(a, si, 3, tid);
      if (tid == 0) grid_arrive(a);
    } else {
      stamp(a, si, 3, tid);
    }
  }
  // ---- end of the step: the last CTA to get here returns the barrier count to zero
  consumer_bar();
  if (tid == 0) {
    __threadfence();
    if (atomicAdd(a.ctl + 1, 1ull) == static_cast<unsigned long long>(nctas - 1)) {
      a.ctl[0] = 0ull;
      a.ctl[1] = 0ull;
      __threadfence();
    }
  }
}

// ---------------------------------------------------------------------------------------
// Repacking of one int4 projection into the record stream (runs once, at decoder creation).
// Source: q uint32 [N, K/8] (element k = 8i + j at bits 4j..4j+3), scale / offset bf16
// [N, K/64].  Block (tile, chunk) writes its 4608-byte record:
//   weights: group gi, lane (g, t): four words {row g: inputs 16t..16t+7, 16t+8..16t+15;
//            row g+8: the same}, nibble r of a word = input 2r, nibble r+4 = input 2r+1
//            (so that one lop3 yields the bf16 pair of two ADJACENT inputs);
//   then per group gi and g: {scale[g], offset[g], scale[g+8], offset[g+8]} bf16.
// Groups beyond K are zero.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t pair_nibbles(uint32_t w) {
  uint32_t o = 0;
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    o |= ((w >> (8 * r)) & 15u) << (4 * r);              // input 2r
    o |= ((w >> (8 * r + 4)) & 15u) << (16 + 4 * r);     // input 2r + 1
  }
  return o;
}

// half > 0 (the fused gate_up matrix, rows [gate; up], half = rows of each): tile t holds gate
// rows 8t..8t+7 in its rows 0..7 and up rows 8t..8t+7 in its rows 8..15.
__global__ void pack_int4_kernel(const uint32_t* q, const unsigned short* scale, const unsigned short* bias, int K, int C,
                                 int rot, int G, int half, uint8_t* packed, const unsigned long long* cta_off,
                                 const unsigned* stage_off /* [G] records of this CTA before this stage */) {
  const int tile = blockIdx.x, chunk = blockIdx.y;
  const int cta = (tile + rot) % G, local = tile / G;
  uint8_t* rec = packed + cta_off[cta] + (static_cast<size_t>(stage_off[cta]) + static_cast<size_t>(local) * C + chunk) * kUnitBytes;
  const int tid = threadIdx.x;   // 256: (group gi, lane)
  const int gi = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int k0 = chunk * kUnitK + gi * 64;
  auto src_row = [&](int r) -> size_t {   // source row of the tile's row r
    if (half > 0) return r < 8 ? static_cast<size_t>(tile) * 8 + r : static_cast<size_t>(half) + static_cast<size_t>(tile) * 8 + (r - 8);
    return static_cast<size_t>(tile) * 16 + r;
  };
  uint4 w = make_uint4(0, 0, 0, 0);
  if (k0 < K) {
    const uint32_t* r0 = q + src_row(g) * (K / 8) + (k0 + 16 * t) / 8;
    const uint32_t* r1 = q + src_row(g + 8) * (K / 8) + (k0 + 16 * t) / 8;
    w = make_uint4(pair_nibbles(r0[0]), pair_nibbles(r0[1]), pair_nibbles(r1[0]), pair_nibbles(r1[1]));
  }
  *reinterpret_cast<uint4*>(rec + gi * 512 + lane * 16) = w;
  if (tid < kUnitGroups * 8 * 4) {
    const int sgi = tid >> 5, sg = (tid >> 2) & 7, which = tid & 3;   // which: s[g], b[g], s[g+8], b[g+8]
    const int kk = chunk * kUnitK + sgi * 64;
    unsigned short v = 0;
    if (kk < K) {
      const size_t o = src_row(sg + ((which & 2) ? 8 : 0)) * (K / 64) + kk / 64;
      v = (which & 1) ? bias[o] : scale[o];
    }
    reinterpret_cast<unsigned short*>(rec + 4096)[sgi * 32 + sg * 4 + which] = v;
  }
}

template <int D, int G>
cudaError_t LaunchStream(const StreamArgs& a, int grid, size_t smem, cudaStream_t stream) {
  auto kernel = decode_stream_kernel<D, G>;
  static std::mutex mu;
  static size_t configured[64] = {};   // per device: the attribute belongs to the device's copy of the kernel
  {
    std::lock_guard<std::mutex> lock(mu);
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64 || smem > configured[dev]) {
      e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
      if (e != cudaSuccess) return e;
      if (dev >= 0 && dev < 64) configured[dev] = smem;
    }
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeCooperative;   // every CTA resident at once: they wait for one another
  attr.val.cooperative = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, a);
}

}  // namespace dsk

using namespace dsk;

struct DecodeStream {
  b200_context* ctx = nullptr;
  b200_decoder_config cfg = {};
  int G = 0;                 // CTAs
  int group = 0;             // query heads per KV head
  int max_m = 0;             // largest batch the kernel takes
  int part_units = 0;        // most records a CTA has in one projection stage
  int kmax = 0;              // longest padded input row
  size_t packed_bytes = 0;
  StreamArgs args = {};      // everything but the per-step pointers
  unsigned long long* trace = nullptr;   // device buffer of stage time stamps, allocated on first use
  bool tracing = false;
  std::vector<void*> owned;  // device allocations
};

namespace dsk {

template <typename T>
cudaError_t AllocInto(DecodeStream* ds, T** p, size_t bytes) {
  void* v = nullptr;
  cudaError_t e = cudaMalloc(&v, bytes);
  if (e != cudaSuccess) return e;
  ds->owned.push_back(v);
  *p = static_cast<T*>(v);
  return cudaMemset(v, 0, bytes);
}

// Shared-memory carve-up for a batch; false when fewer than the minimum slots would remain.
bool Layout(const DecodeStream* ds, int M, int max_smem, StreamArgs* a, size_t* total) {
  if (M > kMaxM) return false;
  a->xs_pitch = ds->kmax + 8;
  const size_t xs = static_cast<size_t>(M) * a->xs_pitch * 2;
  size_t off = kHeaderBytes + ((xs + 127) & ~static_cast<size_t>(127));
  // the attention scratch lives in the x area: make sure it fits
  const int D = ds->cfg.head_dim, Gq = ds->group;
  const size_t attn = static_cast<size_t>(Gq * 2 * (D / 2 + 4) + Gq * kAttnWindow + 2 * (D / 2 + 4) + D +
                                          (kAttnThreads / D) * Gq * D + Gq * (kMaxChunks + 1)) * 4;
  off = std::max(off, kHeaderBytes + ((attn + 127) & ~static_cast<size_t>(127)));
  a->off_xsum = static_cast<int>(off);
  off += static_cast<size_t>(ds->kmax / 64) * 8 * 4;
  a->off_part = static_cast<int>(off);
  a->MP = (M + 1) & ~1;
  off += static_cast<size_t>(ds->part_units) * 16 * a->MP * 4;
  off = (off + 127) & ~static_cast<size_t>(127);
  a->off_ring = static_cast<int>(off);
  if (off + kNW * kUnitBytes > static_cast<size_t>(max_smem)) return false;
  const size_t ring = static_cast<size_t>(max_smem) - off;
  a->NS = static_cast<int>(std::min<size_t>(kMaxSlots, ring / kUnitBytes));
  a->NS2 = static_cast<int>(std::min<size_t>(kMaxHeadSlots, ring / kHeadUnitBytes));
  if (a->NS < kNW || a->NS2 < 2) return false;   // every consumer warp owns at least one record slot
  a->part_units = ds->part_units;
  *total = off + std::max(static_cast<size_t>(a->NS) * kUnitBytes, static_cast<size_t>(a->NS2) * kHeadUnitBytes);
  return true;
}

}  // namespace dsk

b200_status DecodeStreamCreate(b200_context* ctx, const b200_decoder_config& c, const std::vector<b200_decoder_layer>& layers,
                               const void* embed, const void* final_norm, const void* lm_head, int64_t vocab_full,
                               b200_tp* tp, DecodeStream** out) {
  *out = nullptr;
  if (tp != nullptr && tp->world > 1) return B200_OK;   // sharded decoders keep the kernel-per-operator path
  const int E = c.hidden, H = c.heads, KV = c.kv_heads, D = c.head_dim, I = c.inter, V = c.vocab;
  const int QKV = (H + 2 * KV) * D, HD = H * D;
  const int Gq = H / KV;
  // shapes the single kernel is written for
  const bool group_ok = (D == 128 && (Gq == 1 || Gq == 2 || Gq == 4 || Gq == 8)) || (D == 64 && (Gq == 1 || Gq == 2 || Gq == 4));
  if (!group_ok || E % 64 != 0 || HD % 64 != 0 || I % 64 != 0 || QKV % 16 != 0 || E % 16 != 0 || I % 8 != 0 ||
      c.max_len % 8 != 0 || !Aligned(embed, 16) || !Aligned(lm_head, 16) || !Aligned(final_norm, 16))
    return B200_OK;
  for (const b200_decoder_layer& L : layers) {
    for (const void* p : {L.attn_norm, L.mlp_norm, L.qkv.q, L.qkv.scale, L.qkv.bias, L.o.q, L.o.scale, L.o.bias, L.gate_up.q,
                          L.gate_up.scale, L.gate_up.bias, L.down.q, L.down.scale, L.down.bias,
                          static_cast<const void*>(L.k_cache), static_cast<const void*>(L.v_cache)})
      if (p == nullptr || !Aligned(p, 16)) return B200_OK;
    if (L.q_norm == nullptr || L.k_norm == nullptr) return B200_OK;
  }
  DecodeStream* ds = new DecodeStream();
  ds->ctx = ctx;
  ds->cfg = c;
  ds->G = ctx->sm_count;
  ds->group = Gq;
  const int G = ds->G;
  auto fail = [&](b200_status s) {
    DecodeStreamDestroy(ds);
    return s;
  };

  // ---- the stage table and every CTA's share of the record stream -----------------------
  std::vector<Stage> stages;
  std::vector<std::vector<unsigned>> stage_off;   // per int4 stage: records of each CTA before it
  std::vector<unsigned> units(G, 0);
  int rot = 0;
  auto pad_k = [](int K, int unit) { return (K + unit - 1) / unit * unit; };
  ds->kmax = std::max({pad_k(E, kUnitK), pad_k(HD, kUnitK), pad_k(I, kUnitK), pad_k(E, kHeadUnitK)});
  auto add_proj = [&](int type, int layer, int N, int K, const void* gain) {
    Stage st = {};
    st.type = type;
    st.layer = layer;
    st.N = N;
    st.K = K;
    st.NT = type == kHead ? (N + kHeadRows - 1) / kHeadRows : (N + 15) / 16;
    st.C = type == kHead ? (K + kHeadUnitK - 1) / kHeadUnitK : (K + kUnitK - 1) / kUnitK;
    st.rot = rot;
    st.gain = static_cast<const __nv_bfloat16*>(gain);
    if (type != kHead) {
      stage_off.push_back(units);
      for (int cta = 0; cta < G; ++cta) {
        int t0;
        const int n = tiles_of(st.NT, st.rot, cta, G, &t0);
        units[cta] += static_cast<unsigned>(n * st.C);
        ds->part_units = std::max(ds->part_units, n * st.C);
      }
    }
    rot = (rot + st.NT) % G;
    stages.push_back(st);
  };
  for (int li = 0; li < c.layers; ++li) {
    const b200_decoder_layer& L = layers[li];
    add_proj(kQkv, li, QKV, E, L.attn_norm);
    Stage at = {};
    at.type = kAttn;
    at.layer = li;
    at.q_norm = static_cast<const __nv_bfloat16*>(L.q_norm);
    at.k_norm = static_cast<const __nv_bfloat16*>(L.k_norm);
    at.k_cache = static_cast<__nv_bfloat16*>(L.k_cache);
    at.v_cache = static_cast<__nv_bfloat16*>(L.v_cache);
    stages.push_back(at);
    add_proj(kO, li, E, HD, nullptr);
    add_proj(kGateUp, li, 2 * I, E, L.mlp_norm);
    add_proj(kDown, li, E, I, nullptr);
  }
  add_proj(kHead, c.layers, V, E, final_norm);
  ds->part_units = std::max(ds->part_units, stages.back().C);   // at least one LM-head tile per round

  std::vector<unsigned long long> cta_off(G);
  unsigned long long total = 0;
  for (int cta = 0; cta < G; ++cta) {
    cta_off[cta] = total;
    total += static_cast<unsigned long long>(units[cta]) * kUnitBytes;
  }
  ds->packed_bytes = static_cast<size_t>(total);

  // ---- device memory ------------------------------------------------------------------------
  b200_status s = BeginLaunch(ctx);
  if (s != B200_OK) return fail(s);
  StreamArgs& a = ds->args;
  uint8_t* packed = nullptr;
  Stage* dstages = nullptr;
  unsigned long long* doff = nullptr;
  unsigned* dunits = nullptr;
  unsigned* dstage_off = nullptr;
  float* inv_freq = nullptr;
  const size_t B = static_cast<size_t>(std::min(c.max_batch, kMaxM));
  cudaError_t e = AllocInto(ds, &packed, std::max<size_t>(ds->packed_bytes, 16));
  if (e == cudaSuccess) e = AllocInto(ds, &dstages, stages.size() * sizeof(Stage));
  if (e == cudaSuccess) e = AllocInto(ds, &doff, G * sizeof(unsigned long long));
  if (e == cudaSuccess) e = AllocInto(ds, &dunits, G * sizeof(unsigned));
  if (e == cudaSuccess) e = AllocInto(ds, &dstage_off, G * sizeof(unsigned));
  if (e == cudaSuccess) e = AllocInto(ds, &a.x[0], B * E * 2);
  if (e == cudaSuccess) e = AllocInto(ds, &a.x[1], B * E * 2);
  if (e == cudaSuccess) e = AllocInto(ds, &a.y, B * E * 4);
  if (e == cudaSuccess) e = AllocInto(ds, &a.qkv, B * QKV * 2);
  if (e == cudaSuccess) e = AllocInto(ds, &a.attn, B * HD * 2);
  if (e == cudaSuccess) e = AllocInto(ds, &a.hmlp, B * I * 2);
  if (e == cudaSuccess) e = AllocInto(ds, &a.attn_part, B * KV * kMaxChunks * Gq * (D + 2) * 4);
  if (e == cudaSuccess) e = AllocInto(ds, &a.attn_cnt, B * KV * 4);
  if (e == cudaSuccess) e = AllocInto(ds, &a.ctl, 2 * sizeof(unsigned long long));
  if (e == cudaSuccess) e = AllocInto(ds, &a.best_val, static_cast<size_t>(G) * 8 * 4);
  if (e == cudaSuccess) e = AllocInto(ds, &a.best_idx, static_cast<size_t>(G) * 8 * 4);
  if (e == cudaSuccess) e = AllocInto(ds, &inv_freq, static_cast<size_t>(D / 2) * 4);
  if (e == cudaSuccess) e = cudaMemcpy(dstages, stages.data(), stages.size() * sizeof(Stage), cudaMemcpyHostToDevice);
  if (e == cudaSuccess) e = cudaMemcpy(doff, cta_off.data(), G * sizeof(unsigned long long), cudaMemcpyHostToDevice);
  if (e == cudaSuccess) e = cudaMemcpy(dunits, units.data(), G * sizeof(unsigned), cudaMemcpyHostToDevice);
  if (e == cudaSuccess) {
    std::vector<float> f(D / 2);
    for (int i = 0; i < D / 2; ++i)
      f[i] = static_cast<float>(1.0 / pow(static_cast<double>(c.rope_theta), static_cast<double>(2 * i) / D));
    e = cudaMemcpy(inv_freq, f.data(), f.size() * sizeof(float), cudaMemcpyHostToDevice);
  }
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    // not enough memory for a second copy of the weights: the per-operator path needs none
    DecodeStreamDestroy(ds);
    return B200_OK;
  }

  // ---- repack the projections (stream order), one launch per stage ---------------------------
  size_t pi = 0;
  for (const Stage& st : stages) {
    if (st.type == kAttn || st.type == kHead) continue;
    const b200_decoder_layer& L = layers[st.layer];
    const b200_qweight& w = st.type == kQkv ? L.qkv : (st.type == kO ? L.o : (st.type == kGateUp ? L.gate_up : L.down));
    e = cudaMemcpy(dstage_off, stage_off[pi].data(), G * sizeof(unsigned), cudaMemcpyHostToDevice);
    if (e != cudaSuccess) break;
    pack_int4_kernel<<<dim3(st.NT, st.C), 256>>>(static_cast<const uint32_t*>(w.q), static_cast<const unsigned short*>(w.scale),
                                                 static_cast<const unsigned short*>(w.bias), st.K, st.C, st.rot, G,
                                                 st.type == kGateUp ? I : 0, packed, doff, dstage_off);
    e = cudaDeviceSynchronize();   // dstage_off is reused by the next stage
    if (e != cudaSuccess) break;
    ++pi;
  }
  if (e != cudaSuccess) return fail(Stick(ctx, Fail(B200_INTERNAL, "decode stream: repacking the weights: %s", cudaGetErrorString(e))));

  a.stages = dstages;
  a.n_stages = static_cast<int>(stages.size());
  a.packed = packed;
  a.cta_off = doff;
  a.cta_units = dunits;
  a.head_w = static_cast<const uint8_t*>(lm_head);
  a.embed = static_cast<const __nv_bfloat16*>(embed);
  a.vocab_full = vocab_full;
  a.E = E;
  a.H = H;
  a.KV = KV;
  a.D = D;
  a.I = I;
  a.V = V;
  a.max_len = c.max_len;
  a.eps = c.rms_eps;
  a.attn_scale = 1.0f / sqrtf(static_cast<float>(D));
  a.inv_freq = inv_freq;
  a.status = ctx->dev_status;
  // largest batch whose inputs leave room for a useful ring
  ds->max_m = 0;
  for (int M = 1; M <= std::min(c.max_batch, kMaxM); ++M) {
    StreamArgs tmp = a;
    size_t smem = 0;
    if (!Layout(ds, M, ctx->max_smem_optin, &tmp, &smem) || tmp.NS < 16) break;
    ds->max_m = M;
  }
  if (ds->max_m == 0) {
    DecodeStreamDestroy(ds);
    return B200_OK;
  }
  *out = ds;
  return B200_OK;
}

void DecodeStreamDestroy(DecodeStream* ds) {
  if (ds == nullptr) return;
  cudaSetDevice(ds->ctx->device);
  for (void* p : ds->owned) cudaFree(p);
  delete ds;
}

bool DecodeStreamSupports(const DecodeStream* ds, int batch) { return ds != nullptr && batch >= 1 && batch <= ds->max_m; }

size_t DecodeStreamPackedBytes(const DecodeStream* ds) { return ds == nullptr ? 0 : ds->packed_bytes; }

b200_status DecodeStreamTrace(DecodeStream* ds, bool enable) {
  if (ds == nullptr) return Fail(B200_FAILED_PRECONDITION, "decoder trace: this decoder has no single-kernel path");
  if (enable && ds->trace == nullptr) {
    cudaSetDevice(ds->ctx->device);
    const size_t bytes = static_cast<size_t>(ds->G) * ds->args.n_stages * 4 * sizeof(unsigned long long);
    cudaError_t e = dsk::AllocInto(ds, &ds->trace, bytes);
    if (e != cudaSuccess) return Fail(B200_RESOURCE_EXHAUSTED, "decoder trace: %s", cudaGetErrorString(e));
  }
  ds->tracing = enable;
  return B200_OK;
}

b200_status DecodeStreamTraceRead(DecodeStream* ds, unsigned long long* out, int64_t capacity, int* ctas, int* stages,
                                  int* stage_types) {
  if (ds == nullptr || ds->trace == nullptr) return Fail(B200_FAILED_PRECONDITION, "decoder trace: tracing was never enabled");
  const int64_t count = static_cast<int64_t>(ds->G) * ds->args.n_stages * 4;
  if (ctas) *ctas = ds->G;
  if (stages) *stages = ds->args.n_stages;
  if (out == nullptr) return B200_OK;
  if (capacity < count) return Fail(B200_INVALID_ARGUMENT, "decoder trace: buffer of %lld words, %lld needed",
                                    static_cast<long long>(capacity), static_cast<long long>(count));
  cudaSetDevice(ds->ctx->device);
  cudaError_t e = cudaMemcpy(out, ds->trace, count * sizeof(unsigned long long), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return Stick(ds->ctx, Fail(B200_INTERNAL, "decoder trace: %s", cudaGetErrorString(e)));
  if (stage_types != nullptr) {
    std::vector<dsk::Stage> st(ds->args.n_stages);
    e = cudaMemcpy(st.data(), ds->args.stages, st.size() * sizeof(dsk::Stage), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return Stick(ds->ctx, Fail(B200_INTERNAL, "decoder trace: %s", cudaGetErrorString(e)));
    for (int i = 0; i < ds->args.n_stages; ++i) stage_types[i] = st[i].type;
  }
  return B200_OK;
}

b200_status DecodeStreamStep(DecodeStream* ds, cudaStream_t stream, const int32_t* tokens, const int32_t* pos, float* logits,
                             int32_t* next_token, int batch) {
  b200_status s = BeginLaunch(ds->ctx);
  if (s != B200_OK) return s;
  StreamArgs a = ds->args;
  a.M = batch;
  a.tokens = tokens;
  a.pos = pos;
  a.logits = logits;
  a.next_token = next_token;
  a.trace = ds->tracing ? ds->trace : nullptr;
  {
    // B200_STREAM_ABLATE=1: the consumers release every record unread (wrong results; shows what
    // the copy pipeline alone sustains)
    static const int ablate = [] {
      const char* v = std::getenv("B200_STREAM_ABLATE");
      return v != nullptr ? std::atoi(v) : 0;
    }();
    a.ablate = ablate;
  }
  size_t smem = 0;
  if (!Layout(ds, batch, ds->ctx->max_smem_optin, &a, &smem))
    return Fail(B200_INTERNAL, "decode stream: batch %d does not fit shared memory", batch);
  a.attn_chunks = std::max(1, std::min(kMaxChunks, ds->G / (batch * ds->cfg.kv_heads)));
  cudaError_t e;
  const int D = ds->cfg.head_dim;
  if (D == 128) {
    switch (ds->group) {
      case 1: e = LaunchStream<128, 1>(a, ds->G, smem, stream); break;
      case 2: e = LaunchStream<128, 2>(a, ds->G, smem, stream); break;
      case 4: e = LaunchStream<128, 4>(a, ds->G, smem, stream); break;
      default: e = LaunchStream<128, 8>(a, ds->G, smem, stream); break;
    }
  } else {
    switch (ds->group) {
      case 1: e = LaunchStream<64, 1>(a, ds->G, smem, stream); break;
      case 2: e = LaunchStream<64, 2>(a, ds->G, smem, stream); break;
      default: e = LaunchStream<64, 4>(a, ds->G, smem, stream); break;
    }
  }
  if (e != cudaSuccess) return Stick(ds->ctx, Fail(B200_INTERNAL, "decode stream launch: %s", cudaGetErrorString(e)));
  return EndLaunch(ds->ctx, "decode stream");
}

}  // namespace b200
