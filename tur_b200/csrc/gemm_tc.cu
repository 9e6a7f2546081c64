// Prefill-sized QMatMul::forward on the 5th-generation tensor cores (tcgen05 / TMEM).
//
//   y[m, n] = sum_k x[m, k] * W[n, k]      W quantized (device fragment tiles), x f32 or bf16
//
// Step 1 (prep kernel): x -> f16 [M, K], each row scaled by a power of two that puts its largest
// magnitude just below the top of the f16 range (the scale is undone exactly in the epilogue).
// Step 2 (this kernel, one CTA per 128 weight rows x BN = 256 or 64 activation rows):
//   * warp 0        TMA producer: activation tiles (256 rows x 64 k, f16) into 128B-swizzled
//                   shared memory (cp.async.bulk.tensor, no multicast);
//   * warps 2..17   dequantize (two groups of eight on alternate stages) the weight tile (128 rows x 64 k) from the fragment tiles to
//                   f16 with packed half arithmetic and store it in the same K-major
//                   128B-swizzled layout, then fence to the async proxy;
//   * warp 1        one elected thread issues tcgen05.mma (M=128, N=256, K=16, f16 x f16 ->
//                   f32 in TMEM), four per stage, and commits the stage back to the producers;
//   * warps 2..17   epilogue: tcgen05.ld the accumulator, undo the row scale, add bias, store.
// MMA roles: A = weights (rows = TMEM lanes), B = activations (columns).
// Every mbarrier wait is bounded; on expiry the CTA records TURQ_E_TIMEOUT, releases its TMEM
// and returns.
#include <cstdlib>
#include <cuda.h>
#include <cuda_fp16.h>

#include <cstdio>

#include "device_utils.cuh"
#include "gemv_tile.cuh"
#include "launch_plan.h"
#include "turq_internal.h"

namespace turq {

namespace {

constexpr int BM = 128;      // weight rows per CTA (MMA M)
constexpr int BK = 64;       // k per stage (one 128-byte swizzle row of f16)
// Pipeline depth by activation-tile height: the ring must cover the L2 -> shared-memory latency of
// the TMA loads (a slot is only refilled after the MMAs that read it have completed), so the
// smaller tiles get more stages out of the same shared memory.
constexpr int stages_for_bn(int bn) { return bn == 64 ? 8 : bn == 128 ? 6 : 4; }
constexpr int A_BYTES = BM * BK * 2;  // 16 KB
constexpr int DQ_WARPS = 8;        // warps that together produce one stage of the weight operand
constexpr int DQ_GROUPS = 2;       // groups of DQ_WARPS warps working on alternate stages
constexpr int TC_THREADS = (2 + DQ_WARPS * DQ_GROUPS) * 32;
constexpr long long TC_WAIT_CYCLES = 4000000000ll;

__device__ __forceinline__ uint32_t s_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void bar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s_u32(bar)), "r"(count));
}
__device__ __forceinline__ void bar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(s_u32(bar)) : "memory");
}
__device__ __forceinline__ void bar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(s_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool bar_try(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(s_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool bar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (bar_try(bar, parity)) return true;  // the common case costs one poll, no clock read
  const long long t0 = clock64();
  for (uint32_t i = 0;; i++) {
    if (bar_try(bar, parity)) return true;
    if ((i & 255u) == 255u && (*abort_flag || clock64() - t0 > TC_WAIT_CYCLES)) break;
  }
  *abort_flag = 1;
  return false;
}

#ifdef TURQ_TRACE
// Debug timeline of CTA (0,0,0): global-timer stamps of one dequantize warp and of the MMA
// thread over a few consecutive stages (built only with -DTURQ_TRACE).
__device__ unsigned long long g_gemm_trace[64 * 8];
__device__ __forceinline__ unsigned long long gtime_tc() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
#define TC_TRACE(row, col) do { if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (row) >= 0 && (row) < 64) g_gemm_trace[(row) * 8 + (col)] = gtime_tc(); } while (0)
int read_gemm_trace(unsigned long long* host, int n) {
  return (int)cudaMemcpyFromSymbol(host, g_gemm_trace, sizeof(unsigned long long) * n);
}
#else
#define TC_TRACE(row, col) do { } while (0)
#endif

// K-major, 128-byte swizzle shared-memory matrix descriptor (8-row groups 1024 B apart).
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}

// byte offset of 16-byte chunk `ch` (8 f16 along k) of tile row r in the swizzled layout
__device__ __forceinline__ uint32_t swz(int r, int ch) {
  return (uint32_t)((r >> 3) * 1024 + (r & 7) * 128 + ((ch ^ (r & 7)) << 4));
}

// ---- dequantization to f16 with packed half arithmetic (two elements per instruction).
// An integer q <= 1023 becomes the half 1024 + q by OR-ing it under the exponent 0x6400;
// subtracting the offset is exact, so the only roundings are the f16 sub-block scale / min
// and the final multiply-add. The error stays a few 1e-4 of the value, inside the 2e-3 budget
// of the tensor-core mode (the bit-exact f32 decode lives in decode.cuh).
__device__ __forceinline__ __half2 u2h2(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }
__device__ __forceinline__ uint32_t h22u(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }
// bytes (b0, b1) / (b2, b3) of a word of small integers -> half2 (1024 + b0, 1024 + b1) / ...
__device__ __forceinline__ __half2 pair01(uint32_t w) { return u2h2(__byte_perm(w, 0x64646464u, 0x5140)); }
__device__ __forceinline__ __half2 pair23(uint32_t w) { return u2h2(__byte_perm(w, 0x64646464u, 0x5342)); }

// Raw fragment bytes of one lane for one stage (16 rows x 64 k), fetched from global memory a
// few stages ahead of their use so that the HBM/L2 latency is off the critical path.
template <int DT> struct StageRegs;
template <> struct StageRegs<TQ_Q8_0> { uint4 q[2]; uint32_t d[2]; };       // d: f16 row g | row g+8 << 16, per tile
template <> struct StageRegs<TQ_Q4_K> { uint4 q; uint4 hdr[2]; };
template <> struct StageRegs<TQ_Q5_K> { uint4 q; uint4 qh; uint4 hdr[2]; };
template <> struct StageRegs<TQ_Q6_K> { uint4 ql; uint4 qh; uint32_t sc[2]; uint32_t d; };

template <int DT>
__device__ __forceinline__ void stage_load(StageRegs<DT>& r, const uint8_t* __restrict__ tiles_rt, int kb, int lane) {
  const int g = lane >> 2;
  if constexpr (DT == TQ_Q8_0) {
#pragma unroll
    for (int tt = 0; tt < 2; tt++) {
      const uint8_t* t = tiles_rt + (size_t)(2 * kb + tt) * 544;
      r.q[tt] = ld_stream_v4(t + TQ_Q8_0_QS + 16 * lane);
      r.d[tt] = (uint32_t)ld_u16(t + 2 * g) | ((uint32_t)ld_u16(t + 2 * (g + 8)) << 16);
    }
  } else if constexpr (DT == TQ_Q4_K || DT == TQ_Q5_K) {
    constexpr int TB = DT == TQ_Q4_K ? 2304 : 2816;
    constexpr int QS = DT == TQ_Q4_K ? TQ_Q4K_QS : TQ_Q5K_QS;
    const uint8_t* t = tiles_rt + (size_t)(kb >> 2) * TB;
    r.q = ld_stream_v4(t + QS + 512 * (kb & 3) + 16 * lane);
    if constexpr (DT == TQ_Q5_K) r.qh = ld_v4(t + TQ_Q5K_QH + 16 * lane);
    r.hdr[0] = ld_v4(t + 16 * g);
    r.hdr[1] = ld_v4(t + 16 * (g + 8));
  } else {
    const uint8_t* t = tiles_rt + (size_t)(kb >> 2) * 3360;
    const int i = kb & 3;
    r.ql = ld_stream_v4(t + TQ_Q6K_QL + 512 * i + 16 * lane);
    r.qh = ld_v4(t + TQ_Q6K_QH + 512 * (i >> 1) + 16 * lane);
    r.sc[0] = ld_u32(t + 16 * g + 4 * i);
    r.sc[1] = ld_u32(t + 16 * (g + 8) + 4 * i);
    r.d = (uint32_t)ld_u16(t + TQ_Q6K_D + 2 * g) | ((uint32_t)ld_u16(t + TQ_Q6K_D + 2 * (g + 8)) << 16);
  }
}

// Dequantize one stage from registers and store it as f16: a_tile = swizzled 128 x 64 tile,
// row0 = first of this warp's 16 rows inside it.
template <int DT>
__device__ __forceinline__ void stage_dequant_store(const StageRegs<DT>& r, int kb, int lane, uint8_t* a_tile, int row0) {
  const int g = lane >> 2, c = lane & 3;
  if constexpr (DT == TQ_Q8_0) {
    const __half2 off = __float2half2_rn(1152.f);  // 1024 + 128: bytes are biased by xor 0x80
#pragma unroll
    for (int tt = 0; tt < 2; tt++) {
      const uint4 q = r.q[tt];
      const uint32_t w[2][2] = {{q.x ^ 0x80808080u, q.y ^ 0x80808080u}, {q.z ^ 0x80808080u, q.w ^ 0x80808080u}};
#pragma unroll
      for (int hr = 0; hr < 2; hr++) {
        const __half2 d2 = __half2half2(__ushort_as_half((unsigned short)((r.d[tt] >> (16 * hr)) & 0xFFFFu)));
        uint4 o;
        o.x = h22u(__hmul2(__hsub2(pair01(w[hr][0]), off), d2));
        o.y = h22u(__hmul2(__hsub2(pair23(w[hr][0]), off), d2));
        o.z = h22u(__hmul2(__hsub2(pair01(w[hr][1]), off), d2));
        o.w = h22u(__hmul2(__hsub2(pair23(w[hr][1]), off), d2));
        *reinterpret_cast<uint4*>(a_tile + swz(row0 + g + 8 * hr, 4 * tt + c)) = o;
      }
    }
  } else if constexpr (DT == TQ_Q4_K || DT == TQ_Q5_K) {
    const int i = kb & 3;  // 64-element group inside the super-block: sub-blocks 2i, 2i+1
    const uint32_t w[2][2] = {{r.q.x, r.q.y}, {r.q.z, r.q.w}};
    uint32_t qh[2][2] = {{0, 0}, {0, 0}};
    if constexpr (DT == TQ_Q5_K) {
      qh[0][0] = r.qh.x; qh[0][1] = r.qh.y; qh[1][0] = r.qh.z; qh[1][1] = r.qh.w;
    }
    const __half2 off = __float2half2_rn(1024.f);
#pragma unroll
    for (int hr = 0; hr < 2; hr++) {
      const uint4 hdr = r.hdr[hr];
      // Sub-block scales in half arithmetic only (no int->float / float->half conversions, which
      // share one narrow pipe): d * sc is exact in f32, so one f16 multiply rounds it the same way.
      const __half2 dd = u2h2(__byte_perm(hdr.x, 0u, 0x1010)), mm = u2h2(__byte_perm(hdr.x, 0u, 0x3232));
      // 6-bit scales / mins of sub-blocks 0..3 or 4..7, one per byte; this stage needs bytes
      // 2*(i&1) and 2*(i&1)+1
      const uint32_t scw = i < 2 ? (hdr.y & 0x3F3F3F3Fu) : ((hdr.w & 0x0F0F0F0Fu) | ((hdr.y >> 2) & 0x30303030u));
      const uint32_t mnw = i < 2 ? (hdr.z & 0x3F3F3F3Fu) : (((hdr.w >> 4) & 0x0F0F0F0Fu) | ((hdr.z >> 2) & 0x30303030u));
      const __half2 sc2 = __hsub2((i & 1) ? pair23(scw) : pair01(scw), off);
      const __half2 mn2 = __hsub2((i & 1) ? pair23(mnw) : pair01(mnw), off);
      const __half2 dl2 = __hmul2(dd, sc2), ml2 = __hneg2(__hmul2(mm, mn2));
#pragma unroll
      for (int nib = 0; nib < 2; nib++) {
        const int j = 2 * i + nib;
        const __half2 dl = nib ? __high2half2(dl2) : __low2half2(dl2);
        const __half2 ml = nib ? __high2half2(ml2) : __low2half2(ml2);
        uint32_t m0 = (nib ? (w[hr][0] >> 4) : w[hr][0]) & 0x0F0F0F0Fu;
        uint32_t m1 = (nib ? (w[hr][1] >> 4) : w[hr][1]) & 0x0F0F0F0Fu;
        if constexpr (DT == TQ_Q5_K) {
          m0 |= ((qh[hr][0] >> j) << 4) & 0x10101010u;
          m1 |= ((qh[hr][1] >> j) << 4) & 0x10101010u;
        }
        uint4 o;
        o.x = h22u(__hfma2(__hsub2(pair01(m0), off), dl, ml));
        o.y = h22u(__hfma2(__hsub2(pair23(m0), off), dl, ml));
        o.z = h22u(__hfma2(__hsub2(pair01(m1), off), dl, ml));
        o.w = h22u(__hfma2(__hsub2(pair23(m1), off), dl, ml));
        *reinterpret_cast<uint4*>(a_tile + swz(row0 + g + 8 * hr, 4 * nib + c)) = o;
      }
    }
  } else {  // Q6_K: the stage is sub-blocks 4i .. 4i+3 (16 elements each)
    const int i = kb & 3;
    const uint32_t qlw[2][2] = {{r.ql.x, r.ql.y}, {r.ql.z, r.ql.w}};
    const uint32_t qhw[2] = {(i & 1) ? r.qh.y : r.qh.x, (i & 1) ? r.qh.w : r.qh.z};
    const __half2 off = __float2half2_rn(1056.f);  // 1024 + 32
    const __half2 off_sc = __float2half2_rn(1152.f);  // 1024 + 128: the int8 scales are biased by xor 0x80
#pragma unroll
    for (int hr = 0; hr < 2; hr++) {
      const int rr = g + 8 * hr;
      // d * scale in half arithmetic (exact product, one rounding - as the f32 route gives)
      const __half2 dd = u2h2(__byte_perm(r.d, 0u, hr ? 0x3232 : 0x1010));
      const uint32_t scb = r.sc[hr] ^ 0x80808080u;
      const __half2 dl01 = __hmul2(dd, __hsub2(pair01(scb), off_sc)), dl23 = __hmul2(dd, __hsub2(pair23(scb), off_sc));
#pragma unroll
      for (int jj = 0; jj < 4; jj++) {
        const int tw = jj >> 1, nib = jj & 1, sh = 2 * jj;
        const __half2 dlp = jj < 2 ? dl01 : dl23;
        const __half2 dl = (jj & 1) ? __high2half2(dlp) : __low2half2(dlp);
        uint32_t m = (nib ? (qlw[hr][tw] >> 4) : qlw[hr][tw]) & 0x0F0F0F0Fu;
        m |= (sh <= 4 ? (qhw[hr] << (4 - sh)) : (qhw[hr] >> (sh - 4))) & 0x30303030u;
        // elements 16*jj + 4c .. +3 of the stage: chunk 2*jj + (c >> 1), half (c & 1)
        uint2 o;
        o.x = h22u(__hmul2(__hsub2(pair01(m), off), dl));
        o.y = h22u(__hmul2(__hsub2(pair23(m), off), dl));
        *reinterpret_cast<uint2*>(a_tile + swz(row0 + rr, 2 * jj + (c >> 1)) + 8 * (c & 1)) = o;
      }
    }
  }
}

struct GemmArgs {
  const uint8_t* tiles;
  int64_t n_rows;   // weight rows (output features)
  int ktiles;       // fragment tiles per row-tile
  int k;
  int m;            // activation rows
  const float* rscale;  // [m] factor undoing the f16 row scaling
  float* y;         // [m, n_rows]; with split-K: partial sums [splits][m][n_rows]
  const float* bias;
  int* status;
  int splits;       // CTAs along K per output tile (gridDim.z); > 1: a reduction launch follows
  // exchange slots (tp.cu): with y_toggle set, the result goes to y_alt instead of y when the
  // word it points to, plus one, is odd - read after the preceding kernels have completed
  const unsigned* y_toggle;
  float* y_alt;
};

// BN = activation rows per CTA (MMA N): 256 for prefill (128 when that is needed to give every
// SM a CTA), 64 for decode batches of a few dozen rows.
template <int DT, int BN>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap xmap, const GemmArgs a) {
  constexpr int TB = TileGeom<DT>::BYTES;
  constexpr int B_BYTES = BN * BK * 2;
  constexpr int TMEM_COLS = BN;
  constexpr int ST = stages_for_bn(BN);
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // 1024-byte alignment for the swizzled tiles
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sA = smem;
  uint8_t* sB = smem + ST * A_BYTES;
  // full[s]: stage s holds its weight tile (one arrival per dequantize warp) and its
  // activation tile (the TMA thread's arrival + transaction bytes)
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + ST * (A_BYTES + B_BYTES));
  uint64_t* empty = full + ST;
  uint64_t* accum = empty + ST;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * BM;  // first weight row
  const int m0 = blockIdx.y * BN;  // first activation row
  // this CTA's share of the K loop (split-K: an even share of the 64-element blocks)
  const int kb_all = a.k / BK;
  const int kb_begin = (int)((int64_t)kb_all * blockIdx.z / a.splits);
  const int kblocks = (int)((int64_t)kb_all * (blockIdx.z + 1) / a.splits) - kb_begin;

  if (threadIdx.x == 0) {
    for (int s = 0; s < ST; s++) {
      bar_init(&full[s], DQ_WARPS + 1);
      bar_init(&empty[s], 1);
    }
    bar_init(accum, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s_u32(tmem_slot)), "n"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (activations)
    if (lane == 0) {
      // launched with programmatic stream serialization: the f16 operand comes from the
      // conversion launch before this one (the weight side below starts without waiting)
      asm volatile("griddepcontrol.wait;" ::: "memory");
      for (int kb = 0; kb < kblocks; kb++) {
        const int s = kb % ST;
        const uint32_t ph = (uint32_t)(kb / ST) & 1u;
        if (!bar_wait(&empty[s], ph ^ 1u, abort_flag)) break;
        bar_expect_tx(&full[s], B_BYTES);
        asm volatile(
            "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                s_u32(sB + s * B_BYTES)),
            "l"(&xmap), "r"((kb_begin + kb) * BK), "r"(m0), "r"(s_u32(&full[s]))
            : "memory");
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      // instruction descriptor: f32 accumulate, f16 x f16, both K-major, N = BN, M = 128
      constexpr uint32_t idesc = (1u << 4) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
      // This one thread feeds the tensor core, so its own instruction count per stage is what
      // separates consecutive stages' MMAs: descriptors are a constant high half plus a low
      // half that advances by 2 (32 bytes >> 4) per 16-element K step, the stage index and
      // phase are carried along, and one barrier covers both operands.
      constexpr uint64_t desc_hi = (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
      const uint32_t a_lo0 = (s_u32(sA) & 0x3FFFFu) >> 4, b_lo0 = (s_u32(sB) & 0x3FFFFu) >> 4;
      bool ok = true;
      int s = 0;
      uint32_t ph = 0, accumulate = 0;  // the first MMA of the tile overwrites the accumulator
      for (int kb = 0; kb < kblocks; kb++) {
        TC_TRACE(kb, 5);
        ok = bar_wait(&full[s], ph, abort_flag);
        if (!ok) break;
        TC_TRACE(kb, 6);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint64_t da0 = desc_hi | (uint64_t)(a_lo0 + (uint32_t)s * (A_BYTES >> 4));
        const uint64_t db0 = desc_hi | (uint64_t)(b_lo0 + (uint32_t)s * (B_BYTES >> 4));
#pragma unroll
        for (int kk = 0; kk < BK / 16; kk++) {
          asm volatile(
              "{\n\t.reg .pred p;\n\t"
              "setp.ne.b32 p, %4, 0;\n\t"
              "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_base),
              "l"(da0 + 2 * kk), "l"(db0 + 2 * kk), "r"(idesc), "r"(kk > 0 ? 1u : accumulate)
              : "memory");
        }
        accumulate = 1u;
        // release the stage to the producers once these MMAs have read it
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(s_u32(&empty[s]))
                     : "memory");
        TC_TRACE(kb, 7);
        if (++s == ST) { s = 0; ph ^= 1u; }
      }
      if (ok)
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(s_u32(accum))
                     : "memory");
    }
  } else {
    // ------------------------------------------------------------ dequantize producers, then epilogue
    const int dqw = warp - 2;           // 0..15
    const int grp = dqw / DQ_WARPS;     // this warp's group takes stages kb = grp, grp + DQ_GROUPS, ...
    const int dq = dqw % DQ_WARPS;      // row-tile of 16 rows inside the 128-row tile
    const int64_t rt = (int64_t)(n0 >> 4) + dq;
    const bool live = rt * TQ_TILE_ROWS < ((a.n_rows + 15) & ~(int64_t)15);
    const uint8_t* tiles_rt = a.tiles + rt * a.ktiles * TB;
    bool ok = true;
    constexpr int PF = 4;  // stages of raw weight bytes kept in registers ahead of their use
    StageRegs<DT> pre[PF];
    // this warp's stages are kb = grp + DQ_GROUPS * t, t = 0, 1, ...
    const int nmine = (kblocks - grp + DQ_GROUPS - 1) / DQ_GROUPS;
    if (live) {
#pragma unroll
      for (int u = 0; u < PF - 1; u++)
        if (u < nmine) stage_load<DT>(pre[u], tiles_rt, kb_begin + grp + DQ_GROUPS * u, lane);
    }
    for (int t0 = 0; t0 < nmine && ok; t0 += PF) {
#pragma unroll
      for (int u = 0; u < PF; u++) {
        const int t = t0 + u;
        if (t >= nmine) break;
        const int kb = grp + DQ_GROUPS * t;
        if (live && t + PF - 1 < nmine)
          stage_load<DT>(pre[(u + PF - 1) % PF], tiles_rt, kb_begin + grp + DQ_GROUPS * (t + PF - 1), lane);
        const int s = kb % ST;
        const uint32_t ph = (uint32_t)(kb / ST) & 1u;
        if (dq == 0 && lane == 0) TC_TRACE(kb, 0);
        ok = bar_wait(&empty[s], ph ^ 1u, abort_flag);
        if (!ok) break;
        if (dq == 0 && lane == 0) TC_TRACE(kb, 1);
        uint8_t* a_tile = sA + s * A_BYTES;
        if (live) {
          stage_dequant_store<DT>(pre[u], kb_begin + kb, lane, a_tile, 16 * dq);
        } else {
          // rows beyond the tensor: zeros
          const int g = lane >> 2, c = lane & 3;
#pragma unroll
          for (int hr = 0; hr < 2; hr++)
#pragma unroll
            for (int h = 0; h < 2; h++)
              *reinterpret_cast<uint4*>(a_tile + swz(16 * dq + g + 8 * hr, 4 * h + c)) = make_uint4(0, 0, 0, 0);
        }
        if (dq == 0 && lane == 0) TC_TRACE(kb, 2);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy stores -> visible to the MMA
        __syncwarp();
        if (dq == 0 && lane == 0) TC_TRACE(kb, 3);
        if (lane == 0) bar_arrive(&full[s]);
        if (dq == 0 && lane == 0) TC_TRACE(kb, 4);
      }
    }
    // ---- epilogue: TMEM lanes 32*(warp%4).., columns split over the warps of each lane quarter
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // the next launch may set up behind this one
    asm volatile("griddepcontrol.wait;" ::: "memory");               // y / the partial sums may still be read by the predecessor
    if (ok) ok = bar_wait(accum, 0, abort_flag);
    if (ok) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int quarter = warp & 3;
      constexpr int PARTS = BN >= 128 ? 4 : 2;       // column parts shared out over the warps of a lane quarter
      const int col_part = dqw >> 2;                  // 0..3
      const int64_t n = (int64_t)n0 + 32 * quarter + lane;
      const float bv = (a.bias && a.splits == 1 && n < a.n_rows) ? a.bias[n] : 0.f;
      float* ybase = a.y;
      if (a.y_toggle && ((*reinterpret_cast<const volatile unsigned*>(a.y_toggle) + 1u) & 1u)) ybase = a.y_alt;
      float* const yout = ybase + (size_t)blockIdx.z * (size_t)a.m * (size_t)a.n_rows;
#pragma unroll 1
      for (int cb = 0; cb < BN / (32 * PARTS) && col_part < PARTS; cb++) {
        const int col0 = (BN / PARTS) * col_part + 32 * cb;
        uint32_t v[32];
        const uint32_t taddr = tmem_base + ((uint32_t)(32 * quarter) << 16) + (uint32_t)col0;
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
        if (n < a.n_rows) {
#pragma unroll
          for (int j = 0; j < 32; j++) {
            const int mrow = m0 + col0 + j;
            if (mrow < a.m) yout[(int64_t)mrow * a.n_rows + n] = __uint_as_float(v[j]) * a.rscale[mrow] + bv;
          }
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "n"(TMEM_COLS) : "memory");
  }
  if (threadIdx.x == 0 && *abort_flag) {
    *reinterpret_cast<volatile int*>(a.status) = 7;  // TURQ_E_TIMEOUT; the word may be mapped host memory
    __threadfence_system();
  }
}

// x [m, k] (f32 / bf16) -> f16 [m, k] with a per-row power-of-two scale that brings the row's
// largest magnitude into [8192, 16384): rows of large values do not overflow f16 and rows of
// tiny values do not sink into its subnormals. rscale[m] undoes the scale exactly in the
// epilogue. Rows that are all zero, or hold an infinity or NaN, are converted as they are.
// One CTA per row.
__global__ void __launch_bounds__(256) prep_act_kernel(const void* __restrict__ x, int is_bf16, int64_t k,
                                                        __half* __restrict__ xh, float* __restrict__ rscale) {
  __shared__ float wmax[8];
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // the GEMM behind may start on its weights
  asm volatile("griddepcontrol.wait;" ::: "memory");               // x may still be written, the operand buffer still read
  const int64_t row = blockIdx.x;
  float amax = 0.f;
  for (int64_t i = threadIdx.x; i < k; i += blockDim.x) amax = fmaxf(amax, fabsf(load_act_f32(x, is_bf16, row * k + i)));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
  if ((threadIdx.x & 31) == 0) wmax[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = wmax[0];
#pragma unroll
  for (int w = 1; w < 8; w++) amax = fmaxf(amax, wmax[w]);
  float s = 1.f;
  if (amax > 0.f && amax < 3.0e38f) {  // also false for NaN
    int e;
    frexpf(amax, &e);           // amax = f * 2^e, f in [0.5, 1)
    int se = 14 - e;            // scaled row maximum lands in [8192, 16384)
    if (se > 126) se = 126;     // keep the scale and its reciprocal normal numbers
    s = ldexpf(1.f, se);
  }
  if (threadIdx.x == 0) rscale[row] = 1.f / s;
  for (int64_t i = threadIdx.x; i < k; i += blockDim.x)
    xh[row * k + i] = __float2half_rn(load_act_f32(x, is_bf16, row * k + i) * s);
}

// y[i] = sum of the split-K partial sums (in split order) + bias
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float* __restrict__ part, int splits, int64_t total,
                                                             int64_t n_rows, const float* __restrict__ bias,
                                                             float* __restrict__ y, const unsigned* y_toggle, float* y_alt) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (y_toggle && ((*reinterpret_cast<const volatile unsigned*>(y_toggle) + 1u) & 1u)) y = y_alt;
  const int64_t i4 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i4 >= total) return;
  if (i4 + 4 <= total && (n_rows & 3) == 0 && (reinterpret_cast<uintptr_t>(y) & 15) == 0) {
    float4 acc = *reinterpret_cast<const float4*>(part + i4);
    for (int z = 1; z < splits; z++) {
      const float4 p = *reinterpret_cast<const float4*>(part + (size_t)z * total + i4);
      acc.x += p.x; acc.y += p.y; acc.z += p.z; acc.w += p.w;
    }
    if (bias) {
      const int64_t n = i4 % n_rows;
      acc.x += bias[n]; acc.y += bias[n + 1]; acc.z += bias[n + 2]; acc.w += bias[n + 3];
    }
    *reinterpret_cast<float4*>(y + i4) = acc;
  } else {
    for (int64_t i = i4; i < total && i < i4 + 4; i++) {
      float acc = part[i];
      for (int z = 1; z < splits; z++) acc += part[(size_t)z * total + i];
      if (bias) acc += bias[i % n_rows];
      y[i] = acc;
    }
  }
}

// Launch with programmatic stream serialization: the kernel may be scheduled while its
// predecessor in the stream still runs and orders itself with griddepcontrol.wait.
template <class... Params, class... Args>
cudaError_t launch_pdl(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, args...);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

template <int DT, int BN>
cudaError_t launch_tc_bn(const CUtensorMap& map, const GemmArgs& a, cudaStream_t s) {
  constexpr int ST = stages_for_bn(BN);
  constexpr int SMEM = ST * (A_BYTES + BN * BK * 2) + (3 * ST + 1) * 8 + 16 + 1024;
  static PerDeviceOnce configured;
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured.done(dev)) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<DT, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) return e;
    configured.set(dev);
  }
  dim3 grid((unsigned)((a.n_rows + BM - 1) / BM), (unsigned)((a.m + BN - 1) / BN), (unsigned)a.splits);
  return launch_pdl(gemm_tc_kernel<DT, BN>, grid, dim3(TC_THREADS), (size_t)SMEM, s, map, a);
}

template <int DT>
cudaError_t launch_tc_dt(const CUtensorMap& map, const GemmArgs& a, int bn, cudaStream_t s) {
  return bn == 64 ? launch_tc_bn<DT, 64>(map, a, s) : bn == 128 ? launch_tc_bn<DT, 128>(map, a, s) : launch_tc_bn<DT, 256>(map, a, s);
}

}  // namespace

static int pick_bn(int64_t n_rows, int64_t m, int sm_count) {
  static const int bn_env = tuning_env("TURQ_GEMM_BN", 0);
  return plan_gemm_bn(n_rows, m, sm_count, bn_env);
}

static int pick_splits(int64_t n_rows, int64_t m, int64_t k, int sm_count) {
  static const int env = tuning_env("TURQ_GEMM_SPLITK", -1);
  return plan_gemm_splits(n_rows, m, k, sm_count, env);
}

size_t gemm_tc_scratch_bytes(int64_t m, int64_t k, int64_t n_rows, int sm_count) {
  const int splits = pick_splits(n_rows, m, k, sm_count);
  const size_t part = splits > 1 ? (((size_t)splits * (size_t)m * (size_t)n_rows * 4 + 255) & ~(size_t)255) : 0;
  return (((size_t)m * (size_t)k * 2 + 255) & ~(size_t)255) + (((size_t)m * 4 + 255) & ~(size_t)255) + 256 + part;
}

cudaError_t launch_gemm_tc(int dtype, const uint8_t* tiles, int64_t n_rows, int64_t k, const void* x, int x_dtype,
                           int64_t m, float* y, const float* bias, uint8_t* scratch, int sm_count, cudaStream_t s,
                           int* launches, int* dev_status_word, bool x_prepared, const unsigned* y_toggle, float* y_alt) {
  if (k % BK != 0 || m <= 0 || m > INT32_MAX || k > INT32_MAX) return cudaErrorInvalidValue;
  EncodeTiledFn enc = encode_fn();
  if (!enc) return cudaErrorNotSupported;
  __half* xh = reinterpret_cast<__half*>(scratch);
  float* rscale = reinterpret_cast<float*>(scratch + (((size_t)m * (size_t)k * 2 + 255) & ~(size_t)255));
  cudaError_t e = cudaSuccess;
  if (!x_prepared) {  // several weights that read the same x share one conversion
    e = launch_pdl(prep_act_kernel, dim3((unsigned)m), dim3(256), 0, s, x, (int)(x_dtype == TQ_BF16), k, xh, rscale);
    if (launches) (*launches)++;
    if (e != cudaSuccess) return e;
  }

  CUtensorMap map;
  const cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)m};
  const cuuint64_t strides[1] = {(cuuint64_t)k * 2};
  const int bn = pick_bn(n_rows, m, sm_count);
  const int splits = pick_splits(n_rows, m, k, sm_count);
  float* partial = reinterpret_cast<float*>(scratch + (((size_t)m * (size_t)k * 2 + 255) & ~(size_t)255) +
                                            (((size_t)m * 4 + 255) & ~(size_t)255) + 256);
  const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)bn};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, xh, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;

  GemmArgs a{};
  a.tiles = tiles;
  a.n_rows = n_rows;
  a.ktiles = (int)(k / tq_block_elems(dtype));
  a.k = (int)k;
  a.m = (int)m;
  a.rscale = rscale;
  a.y = splits > 1 ? partial : y;
  a.bias = bias;
  a.status = dev_status_word;
  a.splits = splits;
  a.y_toggle = splits > 1 ? nullptr : y_toggle;  // with split-K the reduction launch picks the buffer
  a.y_alt = y_alt;
  switch (dtype) {
    case TQ_Q8_0: e = launch_tc_dt<TQ_Q8_0>(map, a, bn, s); break;
    case TQ_Q4_K: e = launch_tc_dt<TQ_Q4_K>(map, a, bn, s); break;
    case TQ_Q5_K: e = launch_tc_dt<TQ_Q5_K>(map, a, bn, s); break;
    case TQ_Q6_K: e = launch_tc_dt<TQ_Q6_K>(map, a, bn, s); break;
    default: return cudaErrorInvalidValue;
  }
  if (launches) (*launches)++;
  if (e != cudaSuccess || splits == 1) return e;
  const int64_t total = m * n_rows;
  e = launch_pdl(splitk_reduce_kernel, dim3((unsigned)((total + 1023) / 1024)), dim3(256), 0, s, (const float*)partial, splits,
                 total, n_rows, bias, y, y_toggle, y_alt);
  if (launches) (*launches)++;
  return e;
}

}  // namespace turq

#ifdef TURQ_TRACE
extern "C" int turq_debug_read_gemm_trace(unsigned long long* host, int n) { return turq::read_gemm_trace(host, n); }
#endif
