// Decode-sized QMatMul::forward in the integer scheme, built to stay HBM-bound on B200.
//
//   * Persistent CTAs, two per SM: a producer warp streams device tiles (contiguous bytes) into
//     a shared-memory ring with bulk async copies (cp.async.bulk, no multicast) that complete
//     on mbarriers; 8 consumer warps each take one tile of a stage, read their fragment chunks
//     from shared memory with 128-bit loads and run the integer MMAs of gemv_tile.cuh; an
//     epilogue warp adds the consumers' partial sums and writes outputs, so consumers never
//     meet at a CTA-wide barrier. The bytes in flight per SM are set by the ring, not by
//     registers.
//   * Work split (launch_plan.h): whole row-tiles per CTA when that keeps the CTA slots busy,
//     else an even split in tiles where a CTA's range may start or end inside a row-tile. The
//     partial sums of a cut row-tile go through a small global workspace and are added in CTA
//     order by the CTA that holds the row-tile's first tile, so results are deterministic.
//   * Quantized activations (template parameter ACT): up to 4096 values the CTA quantizes
//     them itself into shared memory while the first weight stages are in flight; otherwise a
//     launch of its own quantizes them once into global scratch and the CTAs either bulk-copy
//     the planes into shared memory (up to 16 rows, when they fit) or read them from global
//     memory in the MMA loop. The GEMV that follows its quantization launch is started with
//     programmatic stream serialization: its CTAs set up while that launch still runs and
//     order themselves behind it with griddepcontrol.wait.
//   * Several weights that share x run as one launch over their concatenated row-tiles, also
//     Q4_K / Q5_K weights beside Q6_K ones (template parameter DT2).
//
// Every wait (mbarrier, cross-CTA flag) is bounded: on expiry the kernel records
// TURQ_E_TIMEOUT in the status word, stops issuing work and returns.
#include <cstdio>
#include <cstdlib>

#include "actquant.cuh"
#include "gemv_tile.cuh"
#include "launch_plan.h"
#include "tp_exchange.cuh"
#include "turq_internal.h"

namespace turq {

constexpr int NW = 8;                  // consumer warps
constexpr int THREADS = (NW + 2) * 32; // + producer warp + epilogue warp
constexpr int RED_SLOTS = 2;           // partial-sum hand-over buffers between consumers and epilogue
constexpr int MAX_STAGES = 6;
constexpr uint32_t SPIN_LIMIT = 1u << 23;
constexpr long long WAIT_CYCLES = 2000000000ll;  // about one second of SM clock

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait; returns false (and raises the CTA's abort flag) when the limit is reached.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  const long long t0 = clock64();
  for (uint32_t i = 0; i < SPIN_LIMIT; i++) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 1023u) == 1023u && (*abort_flag || clock64() - t0 > WAIT_CYCLES)) break;
  }
  *abort_flag = 1;
  return false;
}
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst_smem)),
               "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(NW * 32) : "memory"); }

#ifdef TURQ_TRACE
// Debug timeline: per CTA, global-timer stamps at a few points (built only with -DTURQ_TRACE).
__device__ unsigned long long g_trace[1024 * 8];
__device__ __forceinline__ unsigned long long gtime() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
#define TRACE(slot) do { if (lane == 0) g_trace[(blockIdx.x & 1023) * 8 + (slot)] = gtime(); } while (0)
extern "C" int turq_debug_read_trace(unsigned long long* host, int n) {
  return (int)cudaMemcpyFromSymbol(host, g_trace, sizeof(unsigned long long) * n);
}
#else
#define TRACE(slot) do { } while (0)
#endif

struct SmemPlan {
  int ring, act_qs, act_dsc, act_bs16, act_bs32, red, bars, total, qs_stride;
};

constexpr int MAX_PARTS = 4;  // weights that share one activation and one launch (q|k|v, gate|up)

struct StreamArgs {
  // part p covers row-tiles [rt_begin[p], rt_begin[p+1]) of the concatenated row space
  const uint8_t* tiles[MAX_PARTS];
  int64_t n_rows[MAX_PARTS];
  int rt_begin[MAX_PARTS + 1];
  int part_alt[MAX_PARTS];        // mixed launches: 1 = this part's tiles are of the second type (DT2)
  float* y[MAX_PARTS];            // outputs, already offset to the pass's first row
  float* y_alt[MAX_PARTS];        // second output buffer, used instead of y when (*y_toggle + 1) is odd
  const unsigned* y_toggle;       // nullptr: always y. Tensor-parallel exchange: the call counter, whose
                                  // parity selects the exchange slot this launch has to fill
  const float* bias[MAX_PARTS];
  int nparts;
  int interleave;       // 1: two parts of equal shape (ffn_gate, ffn_up) walked as row-tiles g0, u0, g1, u1, ...;
                        // the epilogue keeps silu-input g_t and writes silu(g_t) * u_t to y[0] only
  int ktiles, k;
  int KU;               // units (tiles; groups of 4 tiles for Q8_0) per row-tile
  int split_q, split_r; // CTA b owns units [b*q + min(b,r), (b+1)*q + min(b+1,r)), clamped to total_units
  int total_units;
  const void* x;        // activations of the pass (first row of the pass), f32 or bf16   [ACT_FUSED]
  int x_is_bf16;
  ActPack gact;         // planes in global scratch, already offset to the pass's first row [other modes]
  int rows;             // valid activation rows in this pass (<= 8 * MG)
  float* partial;       // [grid][MG * 128]: partial sums of a CTA's leading split row-tile
  int* flags;           // [grid], all zero between launches
  int* status;
  int stages;
  int stage_bytes;
  SmemPlan sp;
  // Row-parallel linear of a tensor-parallel group, small outputs: the CTAs that finish last
  // perform the exchange themselves (signal the peers, wait, add all ranks' partial results in rank
  // order into xchg.out) - compute and collective in one kernel. y / y_alt are then the two
  // exchange slots and y_toggle the group's call counter.
  int xchg_on;
  TpArgs xchg;
};

inline SmemPlan plan_smem(int dtype, int mg, bool fused /* planes in shared memory */, int rows_cap, int k, int stages, int stage_bytes,
                          int dtype2 = -1) {
  auto up = [](int v) { return (v + 127) & ~127; };
  SmemPlan p{};
  p.ring = 0;
  int off = up(stages * stage_bytes);
  p.qs_stride = k + 32;
  p.act_qs = off;
  if (fused) {
    off = up(off + rows_cap * p.qs_stride);
    p.act_dsc = off;
    off = up(off + rows_cap * (k / (dtype == TQ_Q8_0 ? 32 : 256)) * 4);
    p.act_bs16 = off;  // Q6_K reads the sums of 16, Q4_K / Q5_K the sums of 32
    if (dtype == TQ_Q6_K || dtype2 == TQ_Q6_K) off = up(off + rows_cap * (k / 16) * 2);
    p.act_bs32 = off;
    if (dtype == TQ_Q4_K || dtype == TQ_Q5_K) off = up(off + rows_cap * (k / 32) * 2);
  }
  p.red = off;
  off = up(off + RED_SLOTS * NW * mg * 128 * 4);
  p.bars = off;
  off += (MAX_STAGES * NW + MAX_STAGES + 2 * RED_SLOTS) * 8 + 8 /* abort flag */ + 8 /* act_full */ + 16;
  p.total = off;
  return p;
}

// Walks a CTA's unit range stage by stage (a stage never crosses a row-tile); identical in
// the producer, the consumers and the epilogue warp. No divisions on the way.
struct StageWalk {
  int rt, ku, left, KU;
  __device__ __forceinline__ void init(int u0, int u1, int ku_) {
    KU = ku_;
    rt = u0 / KU;
    ku = u0 - rt * KU;
    left = u1 - u0;
  }
  __device__ __forceinline__ bool done() const { return left <= 0; }
  __device__ __forceinline__ int count() const {
    int n = KU - ku;
    if (n > NW) n = NW;
    if (n > left) n = left;
    return n;
  }
  // advances past n units; returns true when that closed a segment (row-tile or range end)
  __device__ __forceinline__ bool advance(int n) {
    ku += n;
    left -= n;
    const bool closed = ku == KU || left == 0;
    return closed;
  }
  __device__ __forceinline__ void next_row_if_needed() {
    if (ku == KU) { ku = 0; rt++; }
  }
};

// Where the consumer warps find the quantized activation planes
constexpr int ACT_GLOBAL = 0;  // in global scratch (written by a preceding quantization launch)
constexpr int ACT_FUSED = 1;   // quantized by this CTA into shared memory
constexpr int ACT_STAGED = 2;  // bulk-copied from global scratch into shared memory at CTA start

// DT2 != DT: a mixed launch (attn_q|k in Q4_K or Q5_K beside attn_v in Q6_K, as the K-quant
// mixes store them); parts flagged in part_alt hold DT2 tiles. Both types have one tile per
// 256 elements, so the walk over tiles is the same; ring slots are sized for the larger tile.
template <int DT, int MG, int ACT, int DT2 = DT>
__global__ void __launch_bounds__(THREADS, 2) gemv_stream_kernel(const __grid_constant__ StreamArgs a) {
  constexpr bool MIXED = DT2 != DT;
  constexpr int TB = TileGeom<DT>::BYTES;
  constexpr int TB2 = TileGeom<DT2>::BYTES;
  constexpr int GROUP = TileGeom<DT>::GROUP;
  static_assert(!MIXED || (GROUP == 1 && TileGeom<DT2>::GROUP == 1 && TileGeom<DT>::ELEMS == TileGeom<DT2>::ELEMS),
                "mixed launches pair K-quant types only");
  constexpr int UNIT_BYTES = (TB2 > TB ? TB2 : TB) * GROUP;
  constexpr bool NEED16 = DT == TQ_Q6_K || DT2 == TQ_Q6_K;
  constexpr bool NEED32 = DT == TQ_Q4_K || DT == TQ_Q5_K || DT2 == TQ_Q4_K || DT2 == TQ_Q5_K;
  extern __shared__ __align__(128) uint8_t smem[];
  const SmemPlan& sp = a.sp;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + sp.bars);  // [stage][consumer warp]: one tile each
  uint64_t* empty = full + MAX_STAGES * NW;
  uint64_t* red_full = empty + MAX_STAGES;
  uint64_t* red_empty = red_full + RED_SLOTS;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(red_empty + RED_SLOTS);
  uint64_t* act_full = red_empty + RED_SLOTS + 1;  // ACT_STAGED: the planes have landed
  float* red = reinterpret_cast<float*>(smem + sp.red);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp == 0) TRACE(0);
  const int KU = a.KU;
  const int G = gridDim.x, b = blockIdx.x;
  auto start_of = [&](int bb) {
    const int u = bb * a.split_q + (bb < a.split_r ? bb : a.split_r);
    return u < a.total_units ? u : a.total_units;
  };
  const int u0 = start_of(b), u1 = start_of(b + 1);

  {
    // one barrier per thread: ~60 mbarrier.init in sequence on one thread cost most of a
    // microsecond before the first copy could be issued
    const int tid = (int)threadIdx.x;
    const int nfull = a.stages * NW;
    int i = tid;
    bool did = true;
    if (i < nfull) {
      mbar_init(&full[i], 1);
    } else if ((i -= nfull) < a.stages) {
      mbar_init(&empty[i], NW);
    } else if ((i -= a.stages) < RED_SLOTS) {
      mbar_init(&red_full[i], NW);
    } else if ((i -= RED_SLOTS) < RED_SLOTS) {
      mbar_init(&red_empty[i], 1);
    } else if (i == RED_SLOTS) {
      mbar_init(act_full, 1);
      *abort_flag = 0;
    } else {
      did = false;
    }
    if (did) asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  // Programmatic dependent launch (when the launch carries the attribute): the next kernel of
  // the stream may be scheduled once every CTA of this grid has issued launch_dependents, which
  // the producer does after its last copy - the launch latency of the next kernel then hides
  // behind this grid's tail. The weights never depend on a preceding kernel, so a producer warp
  // starts streaming at once; the warps that read activations or write outputs / the hand-over
  // workspace first wait (griddepcontrol.wait) for the preceding grid to finish.

  if (warp == NW) {
    // ------------------------------------------------------------ producer warp
    if (lane == 0) {
      // ACT_STAGED: the activation planes of this pass go first - the consumers cannot start
      // without them. They were written by the quantization launch just before this one; with
      // programmatic stream serialization this grid is already resident (barriers set up) when
      // that launch ends, and griddepcontrol.wait orders the copies after it.
      // One copy per row of quants (the shared-memory rows are padded), one per plane of
      // scales / sums (sizes rounded up to 16 bytes; the planes are padded on both sides).
      auto copy_planes = [&]() {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        const int nb = DT == TQ_Q8_0 ? a.k >> 5 : a.k >> 8;
        const uint32_t dsc_bytes = ((uint32_t)(a.rows * nb * 4) + 15u) & ~15u;
        const uint32_t s16_bytes = NEED16 ? (((uint32_t)(a.rows * (a.k >> 4) * 2) + 15u) & ~15u) : 0u;
        const uint32_t s32_bytes = NEED32 ? (((uint32_t)(a.rows * (a.k >> 5) * 2) + 15u) & ~15u) : 0u;
        mbar_expect_tx(act_full, (uint32_t)(a.rows * a.k) + dsc_bytes + s16_bytes + s32_bytes);
        for (int r = 0; r < a.rows; r++)
          bulk_g2s(smem + sp.act_qs + r * sp.qs_stride, a.gact.qs + (size_t)r * a.k, (uint32_t)a.k, act_full);
        bulk_g2s(smem + sp.act_dsc, a.gact.dsc, dsc_bytes, act_full);
        if constexpr (NEED16) bulk_g2s(smem + sp.act_bs16, a.gact.bs16, s16_bytes, act_full);
        if constexpr (NEED32) bulk_g2s(smem + sp.act_bs32, a.gact.bs32, s32_bytes, act_full);
      };
      // The first ring fill goes out before the planes: weights never depend on the preceding
      // kernels, the planes have to wait for them. The consumers cannot free a stage before they
      // have the planes, so the planes are requested before the first wait that needs a free stage.
      bool planes_pending = ACT == ACT_STAGED;
      StageWalk w;
      w.init(u0, u1, KU);
      int slot = 0, issued = 0;
      uint32_t ph = 0;
      while (!w.done()) {
        const int n = w.count();
        if (planes_pending && issued == a.stages) {
          copy_planes();
          planes_pending = false;
        }
        issued++;
        if (!mbar_wait(&empty[slot], ph ^ 1u, abort_flag)) break;
        // one copy per consumer warp (its tile, or its group of Q8_0 tiles), each completing on
        // that warp's own barrier: a warp starts as soon as its bytes are there
        int part = 0, rt_in_part;
        if (a.interleave) {
          part = w.rt & 1;
          rt_in_part = w.rt >> 1;
        } else {
          while (part + 1 < a.nparts && w.rt >= a.rt_begin[part + 1]) part++;
          rt_in_part = w.rt - a.rt_begin[part];
        }
        const int tb = (MIXED && a.part_alt[part]) ? TB2 : TB;
        const uint8_t* src = a.tiles[part] + ((int64_t)rt_in_part * a.ktiles + (int64_t)w.ku * GROUP) * tb;
        uint8_t* dst = smem + sp.ring + slot * a.stage_bytes;
        for (int i = 0; i < n; i++) {
          int nt = a.ktiles - (w.ku + i) * GROUP;
          if (nt > GROUP) nt = GROUP;
          const uint32_t bytes = (uint32_t)nt * tb;
          mbar_expect_tx(&full[slot * NW + i], bytes);
          bulk_g2s(dst + i * UNIT_BYTES, src + (size_t)i * GROUP * tb, bytes, &full[slot * NW + i]);
        }
        for (int i = n; i < NW; i++) mbar_arrive(&full[slot * NW + i]);  // unused this stage: keep phases in step
        w.advance(n);
        w.next_row_if_needed();
        if (++slot == a.stages) { slot = 0; ph ^= 1u; }
      }
      if (planes_pending) copy_planes();  // fewer stages of work than the ring holds
    }
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  } else if (warp < NW) {
    // ------------------------------------------------------------ consumer warps
    if (warp == 0) TRACE(1);
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (warp == 0) TRACE(2);
    ActPack act = a.gact;
    if constexpr (ACT == ACT_STAGED) {
      mbar_wait(act_full, 0u, abort_flag);
      act.qs = reinterpret_cast<const int8_t*>(smem + sp.act_qs);
      act.dsc = reinterpret_cast<const float*>(smem + sp.act_dsc);
      act.bs16 = reinterpret_cast<const int16_t*>(smem + sp.act_bs16);
      act.bs32 = reinterpret_cast<const int16_t*>(smem + sp.act_bs32);
      act.qs_stride = sp.qs_stride;
    }
    if constexpr (ACT == ACT_FUSED) {
      int8_t* sqs = reinterpret_cast<int8_t*>(smem + sp.act_qs);
      float* sdsc = reinterpret_cast<float*>(smem + sp.act_dsc);
      int16_t* sb16 = reinterpret_cast<int16_t*>(smem + sp.act_bs16);
      int16_t* sb32 = reinterpret_cast<int16_t*>(smem + sp.act_bs32);
      if constexpr (DT == TQ_Q8_0) {
        const int nblk = a.k >> 5, groups = (nblk + 7) >> 3;
        for (int wg = warp; wg < a.rows * groups; wg += NW) {
          const int row = wg / groups, blk = (wg - row * groups) * 8 + (lane >> 2);
          const bool live = blk < nblk;
          float v[8];
          if (live) {
            load8(a.x, a.x_is_bf16, (int64_t)row * a.k + blk * 32 + (lane & 3) * 8, v);
          } else {
#pragma unroll
            for (int e = 0; e < 8; e++) v[e] = 0.f;
          }
          uint32_t w0, w1;
          __half dh;
          quant_block_q8_0(v, w0, w1, dh);
          if (live) {
            *reinterpret_cast<uint2*>(sqs + row * sp.qs_stride + blk * 32 + (lane & 3) * 8) = make_uint2(w0, w1);
            if ((lane & 3) == 0) sdsc[row * nblk + blk] = __half2float(dh);
          }
        }
      } else {
        // Only the 256-element blocks this CTA's tiles touch: all of them when the range
        // covers a whole row-tile, else the (cyclic) run starting at the first tile's block.
        const int nblk = a.k >> 8;
        const int span = u1 - u0 >= KU ? KU : u1 - u0;
        const int first = u1 - u0 >= KU ? 0 : u0 % KU;
        const int total = a.rows * span;
        for (int base = 2 * warp; base < total; base += 2 * NW) {
          // two blocks per pass, one per half-warp (16 values per lane)
          const int i = base + (lane >> 4);
          const bool has = i < total;
          const int row = has ? i / span : 0;
          int blk = has ? first + (i - row * span) : 0;
          if (blk >= nblk) blk -= nblk;
          const int hl = lane & 15;
          float v[16];
          if (has) {
            float v0[8], v1[8];
            load8(a.x, a.x_is_bf16, (int64_t)row * a.k + blk * 256 + hl * 16, v0);
            load8(a.x, a.x_is_bf16, (int64_t)row * a.k + blk * 256 + hl * 16 + 8, v1);
#pragma unroll
            for (int e = 0; e < 8; e++) { v[e] = v0[e]; v[8 + e] = v1[e]; }
          } else {
#pragma unroll
            for (int e = 0; e < 16; e++) v[e] = 0.f;
          }
          uint32_t w4[4];
          float d;
          int s16, s32;
          quant_block_q8k_half(v, lane, w4, d, s16, s32);
          if (has) {
            *reinterpret_cast<uint4*>(sqs + row * sp.qs_stride + blk * 256 + hl * 16) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
            if (hl == 0) sdsc[row * nblk + blk] = d;
            if constexpr (NEED16) sb16[row * (a.k >> 4) + blk * 16 + hl] = (int16_t)s16;
            if constexpr (NEED32) {
              if ((hl & 1) == 0) sb32[row * (a.k >> 5) + blk * 8 + (hl >> 1)] = (int16_t)s32;
            }
          }
        }
      }
      act.qs = sqs;
      act.dsc = sdsc;
      act.bs16 = sb16;
      act.bs32 = sb32;
      act.qs_stride = sp.qs_stride;
      consumer_sync();
    }
    if (warp == 0) TRACE(3);

    const int g = lane >> 2, c = lane & 3;
    float acc[MG][4];
#pragma unroll
    for (int mg = 0; mg < MG; mg++)
#pragma unroll
      for (int e = 0; e < 4; e++) acc[mg][e] = 0.f;
    StageWalk w;
    w.init(u0, u1, KU);
    int slot = 0, rs = 0;
    uint32_t ph = 0, rph = 0;
    bool first = true;
    while (!w.done()) {
      const int n = w.count();
      // Every warp waits for its barrier of this stage, also when it has no tile in it (the
      // producer completes that phase with a plain arrive): a warp that skipped the wait could
      // run more than one phase ahead of the producer, pass a later parity test too early
      // and release the stage twice.
      if (!mbar_wait(&full[slot * NW + warp], ph, abort_flag)) break;
      if (warp == 0 && first) TRACE(4);
      first = false;
      if (warp < n) {
        const int kt = (w.ku + warp) * GROUP;
        int left = a.ktiles - kt;
        if (left > GROUP) left = GROUP;
        const uint8_t* tile = smem + sp.ring + slot * a.stage_bytes + warp * UNIT_BYTES;
        bool alt = false;
        if constexpr (MIXED) {
          int part = 0;
          while (part + 1 < a.nparts && w.rt >= a.rt_begin[part + 1]) part++;
          alt = a.part_alt[part] != 0;
        }
        // one activation row: the single-row tile function (same bits, about half the instructions)
        bool done_row1 = false;
        if constexpr (MG == 1 && DT != TQ_Q8_0 && DT2 != TQ_Q8_0) {
          if (a.rows == 1) {
            if (MIXED && alt) {
              tile_mma_row1<DT2>(tile, lane, act, a.k, kt, acc);
            } else {
              tile_mma_row1<DT>(tile, lane, act, a.k, kt, acc);
            }
            done_row1 = true;
          }
        }
        if (!done_row1) {
          if (MIXED && alt) {
            tile_mma<DT2, MG>(tile, lane, act, a.k, kt, a.rows, left, acc);
          } else {
            tile_mma<DT, MG>(tile, lane, act, a.k, kt, a.rows, left, acc);
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[slot]);  // after the tile's bytes have been consumed
      if (++slot == a.stages) { slot = 0; ph ^= 1u; }
      const bool closed = w.advance(n);
      w.next_row_if_needed();
      if (closed) {
        // ---- segment closed: hand this warp's partial sums to the epilogue warp
        if (!mbar_wait(&red_empty[rs], rph ^ 1u, abort_flag)) break;
        float* rw = red + ((rs * NW + warp) * MG) * 128;
#pragma unroll
        for (int mg = 0; mg < MG; mg++) {
          rw[mg * 128 + (2 * c) * 16 + g] = acc[mg][0];
          rw[mg * 128 + (2 * c + 1) * 16 + g] = acc[mg][1];
          rw[mg * 128 + (2 * c) * 16 + g + 8] = acc[mg][2];
          rw[mg * 128 + (2 * c + 1) * 16 + g + 8] = acc[mg][3];
          acc[mg][0] = acc[mg][1] = acc[mg][2] = acc[mg][3] = 0.f;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&red_full[rs]);
        if (++rs == RED_SLOTS) { rs = 0; rph ^= 1u; }
      }
    }
    if (warp == 0) TRACE(5);
  } else {
    // ------------------------------------------------------------ epilogue warp
    // Walks the same stage sequence to know where segments end; per segment adds the
    // consumer warps' partial sums in warp order and either writes y (this CTA owns the
    // row-tile) or parks the sums in the workspace for the owner. The CTA holding the first
    // tile of a row-tile owns it; later CTAs reach into it with the first tiles of their
    // ranges, so their sums are normally there long before the owner needs them.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const bool use_alt = a.y_toggle != nullptr && ((__ldcg(a.y_toggle) + 1u) & 1u) != 0u;
    StageWalk w;
    w.init(u0, u1, KU);
    int seg_ka = w.ku;
    int rs = 0;
    uint32_t rph = 0;
    constexpr int EPL_ALL = (MG * 128 + 31) / 32;
    float gate_keep[EPL_ALL];  // interleaved launches: the gate row-tile's sums until its up row-tile closes
#pragma unroll
    for (int j = 0; j < EPL_ALL; j++) gate_keep[j] = 0.f;
    while (!w.done()) {
      const int n = w.count();
      const int rt = w.rt;
      const bool closed = w.advance(n);
      const int kb = w.ku;
      w.next_row_if_needed();
      if (!closed) continue;
      const bool owner = seg_ka == 0;
      const bool whole = owner && kb == KU;
      const int rt_end = (rt + 1) * KU;
      const int ncols = a.rows < 8 * MG ? a.rows : 8 * MG;
      int part = 0, rt_local;
      if (a.interleave) {
        part = rt & 1;
        rt_local = rt >> 1;
      } else {
        while (part + 1 < a.nparts && rt >= a.rt_begin[part + 1]) part++;
        rt_local = rt - a.rt_begin[part];
      }
      const int64_t part_rows = a.n_rows[part];
      float* const part_y = a.interleave ? a.y[0] : (use_alt ? a.y_alt[part] : a.y[part]);
      const float* const part_bias = a.bias[part];
      constexpr int EPL = (MG * 128 + 31) / 32;  // output elements per lane
      float other[EPL];
#pragma unroll
      for (int j = 0; j < EPL; j++) other[j] = 0.f;
      int ncontrib = 0;
      if (owner && !whole) {
        for (int bp = b + 1; bp < G && start_of(bp) < rt_end; bp++) ncontrib++;
        const long long t0 = clock64();
        for (int base = 0; base < ncontrib; base += 32) {
          const int mine = base + lane;
          for (;;) {
            const int ready = mine < ncontrib ? *(volatile int*)(a.flags + b + 1 + mine) : 1;
            if (__all_sync(0xFFFFFFFFu, ready != 0)) break;
            if (*abort_flag || clock64() - t0 > WAIT_CYCLES) { *abort_flag = 1; break; }
            __nanosleep(64);
          }
        }
        __threadfence();
        for (int cb = 0; cb < ncontrib; cb++) {
#pragma unroll
          for (int j = 0; j < EPL; j++) {
            const int idx = lane + 32 * j;
            if (idx < ncols * 16) {
              const int col = idx >> 4, row = idx & 15;
              other[j] += __ldcg(a.partial + ((b + 1 + cb) * MG + (col >> 3)) * 128 + (col & 7) * 16 + row);
            }
          }
        }
      }
      if (!mbar_wait(&red_full[rs], rph, abort_flag)) break;
#pragma unroll
      for (int j = 0; j < EPL; j++) {
        const int idx = lane + 32 * j;
        if (idx < ncols * 16) {
          const int col = idx >> 4, row = idx & 15;
          const int mg = col >> 3, e = (col & 7) * 16 + row;
          float s = 0.f;
#pragma unroll
          for (int ww = 0; ww < NW; ww++) s += red[((rs * NW + ww) * MG + mg) * 128 + e];
          if (!owner) {
            a.partial[(b * MG + mg) * 128 + e] = s;
          } else {
            s += other[j];
            const int64_t nn = (int64_t)rt_local * TQ_TILE_ROWS + row;
            if (nn < part_rows) {
              if (part_bias) s += part_bias[nn];
              if (a.interleave) {
                // the split gives every CTA whole (gate, up) pairs, gate first
                if (part == 0) {
                  gate_keep[j] = s;
                } else {
                  const float gv = gate_keep[j];
                  part_y[(int64_t)col * part_rows + nn] = (gv / (1.f + expf(-gv))) * s;
                }
              } else {
                part_y[(int64_t)col * part_rows + nn] = s;
              }
            }
          }
        }
      }
      if (!owner) __threadfence();
      __syncwarp();
      if (lane == 0) mbar_arrive(&red_empty[rs]);
      if (!owner) {
        if (lane == 0) atomicExch(a.flags + b, 1);
      } else if (!whole) {
        for (int cb = lane; cb < ncontrib; cb += 32) a.flags[b + 1 + cb] = 0;  // consumed: zero again for the next launch
      }
      if (++rs == RED_SLOTS) { rs = 0; rph ^= 1u; }
      seg_ka = kb == KU ? 0 : kb;
    }
    TRACE(6);
  }
  __syncthreads();
  if (*abort_flag) {
    // a wait ran out: give copies still in flight time to land in this CTA's shared memory
    for (int i = 0; i < 64; i++) __nanosleep(2000);
    if (threadIdx.x == 0) {
      *reinterpret_cast<volatile int*>(a.status) = 7;  // TURQ_E_TIMEOUT; the word may be mapped host memory
      __threadfence_system();
    }
  }
  if (a.xchg_on) {
    // The CTAs that finish last exchange: the last `nb` tickets (nb = enough CTAs for one float4
    // group per thread, at most 16) wait the short while until every CTA of the launch has
    // written its part of the slot, then ticket order gives each its share of the result and the
    // row of flags it pairs on with the peers' CTA of the same role.
    // Two words of the dynamic shared memory behind the barriers hold the CTA-wide decisions
    // (static shared memory would eat into the opt-in maximum the launch configuration asks for).
    int* s_words = reinterpret_cast<int*>(act_full + 1);
    int& s_role = s_words[0];
    int& s_ok = s_words[1];
    const int G2 = (int)gridDim.x;
    const int64_t nvec = (a.xchg.count + 3) >> 2;
    int nb = (int)((nvec + THREADS - 1) / THREADS);
    if (nb > 16) nb = 16;
    if (nb > G2) nb = G2;
    if (nb < 1) nb = 1;
    if (threadIdx.x == 0) {
      __threadfence();  // this CTA's outputs (written before the barrier above) before its ticket
      const int ticket = (int)atomicAdd(a.xchg.counter + 2, 1u);
      s_role = ticket - (G2 - nb);
      if (s_role >= 0) {
        const long long t0 = clock64();
        while (*reinterpret_cast<volatile unsigned*>(a.xchg.counter + 2) < (unsigned)G2) {
          if (clock64() - t0 > a.xchg.wait_cycles) break;  // a CTA of this launch gave up: the rendezvous below reports it
          __nanosleep(32);
        }
        __threadfence();
      }
    }
    __syncthreads();
    if (s_role >= 0) {
      const unsigned seq = *reinterpret_cast<volatile unsigned*>(a.xchg.counter) + 1u;
      const size_t slot_off = (seq & 1u) ? a.xchg.slot_elems : 0;
      const bool ok = tp_rendezvous(a.xchg, seq, &s_ok, s_role);
      if (ok) tp_reduce_range(a.xchg, slot_off, (int64_t)s_role * THREADS + threadIdx.x, (int64_t)nb * THREADS, s_role == 0);
      __syncthreads();
      if (threadIdx.x == 0) {
        if (!ok) {
          *reinterpret_cast<volatile int*>(a.status) = TURQ_E_TIMEOUT;
          __threadfence_system();
        }
        __threadfence();
        if (atomicAdd(a.xchg.counter + 1, 1u) == (unsigned)nb - 1) {  // last of the exchanging CTAs
          a.xchg.counter[1] = 0;
          a.xchg.counter[2] = 0;
          __threadfence();
          *reinterpret_cast<volatile unsigned*>(a.xchg.counter) = seq;
        }
      }
    }
  }
}

// ------------------------------------------------------------------ host side

static int smem_budget() { return device_smem_optin(); }

// In-kernel quantization is redundant work in every CTA and every CTA reads the same few
// cache lines of x: one pass (16 Q8_K blocks, or 64 Q8_0 blocks, per CTA) costs about as much
// as the weight ring takes to fill, so it is only used for up to 4096 activation values - one
// pass of Q8_K blocks, two of Q8_0 blocks (measured at one
// row: Q4_K 5120x8192, two passes, 12.2 us fused against 11.4 us with the planes quantized by a
// launch of their own and bulk-copied; Q6_K 4096x12288, three passes, 15.0 against 12.4 us).
bool gemv_int8_fuses_act(int dtype, int64_t m, int64_t k) {
  (void)dtype;
  static const int max_elems = tuning_env("TURQ_GEMV_FUSE_ELEMS", 4096);
  return m <= 8 && m * k <= max_elems;
}

// partial sums [up to 4 CTAs per SM][4 groups of 8 rows][128] + one flag per CTA
size_t gemv_workspace_bytes(int sms) { return (size_t)sms * 4 * 4 * 128 * 4 + (size_t)sms * 4 * 4 + 256; }
// where in the workspace the ready flags live (the only part that must read zero at launch)
size_t gemv_workspace_flags_offset(int sms) { return (size_t)sms * 4 * 4 * 128 * 4; }
size_t gemv_workspace_flags_bytes(int sms) { return (size_t)sms * 4 * 4; }

// Launches with the programmatic-stream-serialization attribute (the kernel orders itself
// against its predecessor with griddepcontrol.wait).
template <int DT, int MG, int ACT, int DT2 = DT>
static cudaError_t launch_one(StreamArgs a, int grid, int smem_bytes, cudaStream_t s, bool after_quant = false) {
  static PerDeviceOnce configured;  // per instantiation; the attribute is per device function
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured.done(dev)) {
    cudaError_t e = cudaFuncSetAttribute(gemv_stream_kernel<DT, MG, ACT, DT2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         smem_budget());
    if (e != cudaSuccess) return e;
    configured.set(dev);
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = (size_t)smem_bytes;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  // Every GEMV launch carries the attribute: its CTAs may become resident, set up and start
  // streaming weights while the preceding kernel of the stream still runs (measured on B200:
  // cfg2 decode pass 1.75 -> 1.67 ms, cfg1 0.53 -> 0.42 ms, cfg4 1.33 -> 1.22 ms, nothing slower;
  // triggering from the kernel's start instead of after the last copy made no difference).
  // TURQ_GEMV_PDL=0 (tuning builds) restricts it to the launch that follows its own quantization
  // launch, TURQ_GEMV_PDL_PAIR=0 turns that off too.
  static const int pdl = tuning_env("TURQ_GEMV_PDL", 1);
  static const int pdl_pair = tuning_env("TURQ_GEMV_PDL_PAIR", 1);
  cfg.numAttrs = (pdl || (after_quant && pdl_pair)) ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, gemv_stream_kernel<DT, MG, ACT, DT2>, a);
}

// DT2 != DT: parts whose dtype field is DT2 hold tiles of that type (one launch for the K-quant
// mixes' attn_q|k|v). Returns cudaErrorNotSupported, before anything is launched, when a mixed
// call would need a variant that is not instantiated (more than 8 rows, planes in global memory).
template <int DT, int DT2 = DT>
static cudaError_t launch_dt(const GemvPart* parts, int nparts, int64_t k, const void* x, int x_dtype,
                             uint8_t* act_scratch, int64_t m, uint8_t* workspace, int* status, int sm_count,
                             cudaStream_t s, int* launches, bool x_remote, const unsigned* y_toggle, bool planes_ready,
                             const TpArgs* xchg, bool interleave = false) {
  constexpr bool MIXED = DT2 != DT;
  constexpr int GROUP = TileGeom<DT>::GROUP;
  constexpr int UNIT_BYTES = (TileGeom<DT2>::BYTES > TileGeom<DT>::BYTES ? TileGeom<DT2>::BYTES : TileGeom<DT>::BYTES) * GROUP;
  if (nparts < 1 || nparts > MAX_PARTS) return cudaErrorInvalidValue;
  const int ktiles = (int)(k / TileGeom<DT>::ELEMS);
  const int KU = (ktiles + GROUP - 1) / GROUP;
  int rt_begin[MAX_PARTS + 1] = {0};
  for (int p = 0; p < nparts; p++)
    rt_begin[p + 1] = rt_begin[p] + (int)((parts[p].n_rows + TQ_TILE_ROWS - 1) / TQ_TILE_ROWS);
  const int64_t T = (int64_t)rt_begin[nparts] * KU;
  if (T > (int64_t)1 << 30) return cudaErrorInvalidValue;
  if (interleave && (MIXED || nparts != 2 || parts[0].n_rows != parts[1].n_rows)) return cudaErrorNotSupported;
  // The tile split (hence the summation order) must not depend on M: always two CTAs per SM.
  static const int cps_env = tuning_env("TURQ_GEMV_CPS", 0);
  const int ctas_per_sm = cps_env > 0 ? cps_env : 2;
  // Each CTA may use half of the SM's shared memory.
  static const int share_env = tuning_env("TURQ_GEMV_SHARE", 0);
  const int share_div = share_env > 0 ? share_env : 2;
  const int fmt = DT == TQ_Q8_0 ? TQ_Q8_0 : TQ_Q8_K;
  const int stage_bytes = NW * UNIT_BYTES;
  // Shared memory: the ring needs at least two stages next to the activation planes. If
  // that does not fit a CTA's share of the SM, the planes stay in global memory.
  auto stages_for = [&](bool planes_in_smem, int cps, int rows, int mg) {
    if (cps < share_div) cps = share_div;
    const int share = (smem_budget() + 1024) / cps - 1024;  // 1 KB per CTA is reserved by the system
    static const int gmax = tuning_env("TURQ_GEMV_GSTAGES", MAX_STAGES);
    int st = planes_in_smem ? MAX_STAGES : (gmax < MAX_STAGES ? (gmax < 2 ? 2 : gmax) : MAX_STAGES);
    for (; st >= 2; st--)
      if (plan_smem(DT, mg, planes_in_smem, rows, (int)k, st, stage_bytes, DT2).total <= share) break;
    return st;
  };
  // Activation planes: quantized in the kernel (few rows), else quantized once by a launch of
  // their own and then either bulk-copied into every CTA's shared memory (up to 16 rows, when
  // they fit beside a two-stage ring) or read from global memory by the MMA loop.
  // x_remote: x lives in mapped host memory - every CTA reading it over the bus would cost far
  // more than the one pass of the quantization launch, so the planes are always staged.
  // planes_ready: a preceding launch of the caller (RMSNorm prologue) already left the planes of
  // these rows in act_scratch.
  int act_mode = (gemv_int8_fuses_act(DT, m, k) && !x_remote && !planes_ready) ? ACT_FUSED : ACT_GLOBAL;
  {
    const int rows0 = (int)(m < 32 ? m : 32), mg0 = rows0 <= 8 ? 1 : rows0 <= 16 ? 2 : 4;
    if (act_mode == ACT_FUSED && stages_for(true, ctas_per_sm, rows0, mg0) < 2) act_mode = ACT_GLOBAL;
    static const int stage_env = tuning_env("TURQ_GEMV_STAGED", 1);
    if (act_mode == ACT_GLOBAL && m <= 16 && stage_env && stages_for(true, ctas_per_sm, rows0, mg0) >= 2) act_mode = ACT_STAGED;
  }
  const bool fused = act_mode == ACT_FUSED, planes_in_smem = act_mode != ACT_GLOBAL;
  if (MIXED && (m > 8 || act_mode == ACT_GLOBAL)) return cudaErrorNotSupported;
  // Work split. Whole row-tiles per CTA when that keeps most CTA slots busy (or the problem
  // is small): no row-tile is shared, so no partial sums cross CTAs. Otherwise an even split
  // in tiles, with the hand-over of split row-tiles. Depends on the shape only, never on M.
  const int slots = sm_count * ctas_per_sm;
  const int row_tiles_all = rt_begin[nparts];
  static const int split_env = tuning_env("TURQ_GEMV_SPLIT", -1);
  // interleaved (gate, up) launches are split in whole pairs of row-tiles, and only when whole
  // pairs keep the CTA slots busy: a pair cut between CTAs would need both halves handed over
  GemvSplit split = interleave ? plan_gemv_split(row_tiles_all / 2, 2 * KU, slots, -1) : plan_gemv_split(row_tiles_all, KU, slots, split_env);
  if (interleave && !split.aligned) return cudaErrorNotSupported;
  const int grid = split.grid, split_q = split.split_q, split_r = split.split_r;
  const size_t x_es = x_dtype == TQ_BF16 ? 2 : 4;
  ActPackPlan plan = plan_act_pack(fmt, m, k);
  if (!fused && !planes_ready) {
    cudaError_t e = launch_quantize_act_pack(fmt, x, x_dtype, m, k, act_scratch, s);
    if (launches) (*launches)++;
    if (e != cudaSuccess) return e;
  }
  for (int64_t m0 = 0; m0 < m; m0 += 32) {
    const int rows = (int)(m - m0 < 32 ? m - m0 : 32);
    const int mg = rows <= 8 ? 1 : rows <= 16 ? 2 : 4;
    StreamArgs a{};
    for (int p = 0; p < nparts; p++) {
      a.tiles[p] = parts[p].tiles;
      a.n_rows[p] = parts[p].n_rows;
      a.y[p] = parts[p].y + m0 * parts[p].n_rows;
      a.y_alt[p] = parts[p].y_alt ? parts[p].y_alt + m0 * parts[p].n_rows : nullptr;
      a.bias[p] = parts[p].bias;
      a.part_alt[p] = (MIXED && parts[p].dtype == DT2) ? 1 : 0;
    }
    for (int p = 0; p <= nparts; p++) a.rt_begin[p] = rt_begin[p];
    a.y_toggle = y_toggle;
    if (xchg && m <= 32) {  // single pass: the launch's last CTA exchanges
      a.xchg_on = 1;
      a.xchg = *xchg;
    }
    a.interleave = interleave ? 1 : 0;
    a.nparts = nparts;
    a.ktiles = ktiles;
    a.k = (int)k;
    a.KU = KU;
    a.split_q = split_q;
    a.split_r = split_r;
    a.total_units = (int)T;
    a.x = static_cast<const uint8_t*>(x) + (size_t)m0 * k * x_es;
    a.x_is_bf16 = x_dtype == TQ_BF16;
    if (!fused) {
      const int bs = fmt == TQ_Q8_0 ? 32 : 256;
      a.gact.qs = reinterpret_cast<const int8_t*>(act_scratch + plan.off_qs) + m0 * k;
      a.gact.dsc = reinterpret_cast<const float*>(act_scratch + plan.off_dsc) + m0 * (k / bs);
      a.gact.bs16 = reinterpret_cast<const int16_t*>(act_scratch + plan.off_bs16) + m0 * (k / 16);
      a.gact.bs32 = reinterpret_cast<const int16_t*>(act_scratch + plan.off_bs32) + m0 * (k / 32);
      a.gact.qs_stride = (int)k;
    }
    a.rows = rows;
    a.partial = reinterpret_cast<float*>(workspace);
    a.flags = reinterpret_cast<int*>(workspace + gemv_workspace_flags_offset(sm_count));
    a.status = status;
    const int stages = stages_for(planes_in_smem, ctas_per_sm, rows, mg);
    if (stages < 2) return cudaErrorInvalidConfiguration;
    const SmemPlan sp = plan_smem(DT, mg, planes_in_smem, rows, (int)k, stages, stage_bytes, DT2);
    a.stages = stages;
    a.stage_bytes = stage_bytes;
    a.sp = sp;
    cudaError_t e;
    if constexpr (MIXED) {
      e = act_mode == ACT_FUSED ? launch_one<DT, 1, ACT_FUSED, DT2>(a, grid, sp.total, s)
                                : launch_one<DT, 1, ACT_STAGED, DT2>(a, grid, sp.total, s, true);
    } else if (act_mode == ACT_FUSED) {
      e = launch_one<DT, 1, ACT_FUSED>(a, grid, sp.total, s);
    } else if (act_mode == ACT_STAGED) {
      e = mg == 1 ? launch_one<DT, 1, ACT_STAGED>(a, grid, sp.total, s, true) : launch_one<DT, 2, ACT_STAGED>(a, grid, sp.total, s, true);
    } else if (mg == 1) {
      e = launch_one<DT, 1, ACT_GLOBAL>(a, grid, sp.total, s);
    } else if (mg == 2) {
      e = launch_one<DT, 2, ACT_GLOBAL>(a, grid, sp.total, s);
    } else {
      e = launch_one<DT, 4, ACT_GLOBAL>(a, grid, sp.total, s);
    }
    if (launches) (*launches)++;
    if (e != cudaSuccess) return e;
  }
  return cudaSuccess;
}

#define TQ_LAUNCH_ARGS k, x, x_dtype, act_scratch, m, workspace, status, sm_count, s, launches, x_remote, y_toggle, planes_ready, xchg

static cudaError_t launch_one_type(int dtype, const GemvPart* parts, int nparts, int64_t k, const void* x, int x_dtype,
                                   uint8_t* act_scratch, int64_t m, uint8_t* workspace, int* status, int sm_count,
                                   cudaStream_t s, int* launches, bool x_remote, const unsigned* y_toggle, bool planes_ready,
                                   const TpArgs* xchg) {
  switch (dtype) {
    case TQ_Q8_0: return launch_dt<TQ_Q8_0>(parts, nparts, TQ_LAUNCH_ARGS);
    case TQ_Q4_K: return launch_dt<TQ_Q4_K>(parts, nparts, TQ_LAUNCH_ARGS);
    case TQ_Q5_K: return launch_dt<TQ_Q5_K>(parts, nparts, TQ_LAUNCH_ARGS);
    case TQ_Q6_K: return launch_dt<TQ_Q6_K>(parts, nparts, TQ_LAUNCH_ARGS);
    default: return cudaErrorInvalidValue;
  }
}

// parts[i].dtype = 0 means `dtype`. Parts of one type go out as one launch; Q4_K or Q5_K parts
// together with Q6_K parts too, where the mixed kernel exists; anything else one launch per type.
cudaError_t launch_gemv_int8_multi(int dtype, const GemvPart* parts, int nparts, int64_t k, const void* x, int x_dtype,
                                   uint8_t* act_scratch, int64_t m, uint8_t* workspace, int* status, int sm_count,
                                   cudaStream_t s, int* launches, bool x_remote, const unsigned* y_toggle, bool planes_ready,
                                   const TpArgs* xchg) {
  if (nparts < 1 || nparts > MAX_PARTS) return cudaErrorInvalidValue;
  GemvPart p[MAX_PARTS];
  int types[MAX_PARTS], ntypes = 0;
  for (int i = 0; i < nparts; i++) {
    p[i] = parts[i];
    if (p[i].dtype == 0) p[i].dtype = dtype;
    bool seen = false;
    for (int t = 0; t < ntypes; t++) seen = seen || types[t] == p[i].dtype;
    if (!seen) types[ntypes++] = p[i].dtype;
  }
  if (ntypes == 1) return launch_one_type(types[0], p, nparts, TQ_LAUNCH_ARGS);
  static const int mixed_env = tuning_env("TURQ_GEMV_MIXED", 1);
  if (ntypes == 2 && mixed_env) {
    const int other = types[0] == TQ_Q6_K ? types[1] : types[0];
    if ((types[0] == TQ_Q6_K || types[1] == TQ_Q6_K) && (other == TQ_Q4_K || other == TQ_Q5_K)) {
      cudaError_t e = other == TQ_Q4_K ? launch_dt<TQ_Q4_K, TQ_Q6_K>(p, nparts, TQ_LAUNCH_ARGS)
                                       : launch_dt<TQ_Q5_K, TQ_Q6_K>(p, nparts, TQ_LAUNCH_ARGS);
      if (e != cudaErrorNotSupported) return e;
    }
  }
  for (int t = 0; t < ntypes; t++) {
    GemvPart q[MAX_PARTS];
    int nq = 0;
    for (int i = 0; i < nparts; i++)
      if (p[i].dtype == types[t]) q[nq++] = p[i];
    cudaError_t e = launch_one_type(types[t], q, nq, TQ_LAUNCH_ARGS);
    if (e != cudaSuccess) return e;
  }
  return cudaSuccess;
}
#define TQ_LAUNCH_ARGS_DECL k, x, x_dtype, act_scratch, m, workspace, status, sm_count, s, launches, x_remote, y_toggle, planes_ready, xchg

// silu(x . Wg^T) * (x . Wu^T) in one launch (two weights of one type and shape). Returns
// cudaErrorNotSupported, before anything is launched, where the interleaved split does not apply.
cudaError_t launch_gemv_int8_swiglu(int dtype, const uint8_t* gate_tiles, const uint8_t* up_tiles, int64_t n_rows, int64_t k,
                                    const void* x, int x_dtype, uint8_t* act_scratch, int64_t m, float* out, uint8_t* workspace,
                                    int* status, int sm_count, cudaStream_t s, int* launches) {
  GemvPart parts[2] = {{gate_tiles, n_rows, out, nullptr, dtype, nullptr}, {up_tiles, n_rows, out, nullptr, dtype, nullptr}};
  const bool x_remote = false, planes_ready = false;
  const unsigned* y_toggle = nullptr;
  const TpArgs* xchg = nullptr;
  switch (dtype) {
    case TQ_Q8_0: return launch_dt<TQ_Q8_0>(parts, 2, TQ_LAUNCH_ARGS_DECL, true);
    case TQ_Q4_K: return launch_dt<TQ_Q4_K>(parts, 2, TQ_LAUNCH_ARGS_DECL, true);
    case TQ_Q5_K: return launch_dt<TQ_Q5_K>(parts, 2, TQ_LAUNCH_ARGS_DECL, true);
    case TQ_Q6_K: return launch_dt<TQ_Q6_K>(parts, 2, TQ_LAUNCH_ARGS_DECL, true);
    default: return cudaErrorInvalidValue;
  }
}

cudaError_t launch_gemv_int8(int dtype, const uint8_t* tiles, int64_t n_rows, int64_t k, const void* x, int x_dtype,
                             uint8_t* act_scratch, int64_t m, float* y, const float* bias, uint8_t* workspace,
                             int* status, int sm_count, cudaStream_t s, int* launches) {
  GemvPart part{tiles, n_rows, y, bias, dtype, nullptr};
  return launch_gemv_int8_multi(dtype, &part, 1, k, x, x_dtype, act_scratch, m, workspace, status, sm_count, s, launches, false,
                                nullptr, false, nullptr);
}

#undef TQ_LAUNCH_ARGS
#undef TQ_LAUNCH_ARGS_DECL

}  // namespace turq
