// Decode-sized QMatMul::forward in the integer scheme, built to stay HBM-bound on B200.
//
//   * One persistent CTA per SM: a producer warp streams device tiles (contiguous bytes)
//     into a shared-memory ring with bulk async copies (cp.async.bulk, no multicast) that
//     complete on mbarriers; 16 consumer warps each take one tile of a stage, read their
//     fragment chunks from shared memory with 128-bit loads and run the integer MMAs of
//     gemv_tile.cuh. The bytes in flight per SM are set by the ring, not by registers.
//   * Work is split evenly over the CTAs in units of tiles (not rows): a CTA owns a
//     contiguous tile range that may start or end inside a row-tile. The partial sums of a
//     split row-tile go through a small global workspace and are added in CTA order by the
//     CTA that holds the row-tile's first tile, so results are deterministic.
//   * For small M*K the CTA quantizes the activations itself into shared memory while the
//     first weight stages are in flight (no separate launch); otherwise it reads the planes a
//     preceding activation-quantization launch left in global scratch.
//
// Every wait (mbarrier, cross-CTA flag) is bounded: on expiry the kernel records
// TURQ_E_TIMEOUT in the status word, stops issuing work and returns.
#include <cstdio>
#include <cstdlib>

#include "actquant.cuh"
#include "gemv_tile.cuh"
#include "turq_internal.h"

namespace turq {

constexpr int NW = 16;                 // consumer warps
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

struct StreamArgs {
  const uint8_t* tiles;
  int64_t n_rows;
  int row_tiles, ktiles, k;
  const void* x;        // activations of the pass (row m_base first), f32 or bf16   [FUSED]
  int x_is_bf16;
  ActPack gact;         // planes in global scratch, already offset to row m_base     [!FUSED]
  int rows;             // valid activation rows in this pass (<= 8 * MG)
  float* y;             // output, already offset to row m_base
  const float* bias;
  float* partial;       // [grid][MG * 128]: partial sums of a CTA's leading split row-tile
  int* flags;           // [grid], all zero between launches
  int* status;
  int stages;
  int stage_bytes;
};

struct SmemPlan {
  int ring, act_qs, act_dsc, act_bs16, act_bs32, red, bars, total, qs_stride;
};

__host__ __device__ inline SmemPlan plan_smem(int dtype, int mg, bool fused, int rows_cap, int k, int stages,
                                               int stage_bytes) {
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
    p.act_bs16 = off;
    if (dtype != TQ_Q8_0) off = up(off + rows_cap * (k / 16) * 2);
    p.act_bs32 = off;
    if (dtype != TQ_Q8_0) off = up(off + rows_cap * (k / 32) * 2);
  }
  p.red = off;
  off = up(off + RED_SLOTS * NW * mg * 128 * 4);
  p.bars = off;
  off += (2 * MAX_STAGES + 2 * RED_SLOTS) * 8 + 16;
  p.total = off;
  return p;
}

template <int DT, int MG, bool FUSED>
__global__ void __launch_bounds__(THREADS, 1) gemv_stream_kernel(const StreamArgs a) {
  constexpr int TB = TileGeom<DT>::BYTES;
  constexpr int GROUP = TileGeom<DT>::GROUP;
  constexpr int UNIT_BYTES = TB * GROUP;
  extern __shared__ __align__(128) uint8_t smem[];
  const SmemPlan sp = plan_smem(DT, MG, FUSED, a.rows, a.k, a.stages, a.stage_bytes);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + sp.bars);
  uint64_t* empty = full + MAX_STAGES;
  uint64_t* red_full = empty + MAX_STAGES;
  uint64_t* red_empty = red_full + RED_SLOTS;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(red_empty + RED_SLOTS);
  float* red = reinterpret_cast<float*>(smem + sp.red);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int KU = (a.ktiles + GROUP - 1) / GROUP;  // units per row-tile
  const int64_t T = (int64_t)a.row_tiles * KU;
  const int64_t G = gridDim.x, b = blockIdx.x;
  const int64_t u0 = (b * T) / G, u1 = ((b + 1) * T) / G;

  if (threadIdx.x == 0) {
    for (int s = 0; s < a.stages; s++) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], NW);
    }
    for (int s = 0; s < RED_SLOTS; s++) {
      mbar_init(&red_full[s], NW);
      mbar_init(&red_empty[s], 1);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  if (warp == NW) {
    // ------------------------------------------------------------ producer warp
    if (lane == 0) {
      int it = 0;
      for (int64_t u = u0; u < u1;) {
        const int64_t rt = u / KU;
        const int ku = (int)(u - rt * KU);
        int n = KU - ku;
        if (n > NW) n = NW;
        if ((int64_t)n > u1 - u) n = (int)(u1 - u);
        const int slot = it % a.stages;
        const uint32_t ph = (uint32_t)(it / a.stages) & 1u;
        if (!mbar_wait(&empty[slot], ph ^ 1u, abort_flag)) break;
        int ntiles = a.ktiles - ku * GROUP;
        if (ntiles > n * GROUP) ntiles = n * GROUP;
        const uint32_t bytes = (uint32_t)ntiles * TB;
        mbar_expect_tx(&full[slot], bytes);
        bulk_g2s(smem + sp.ring + slot * a.stage_bytes, a.tiles + (rt * a.ktiles + (int64_t)ku * GROUP) * TB, bytes,
                 &full[slot]);
        u += n;
        it++;
      }
    }
  } else if (warp < NW) {
    // ------------------------------------------------------------ consumer warps
    const int ctid = threadIdx.x;  // 0 .. NW*32-1
    ActPack act = a.gact;
    if constexpr (FUSED) {
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
        const int nblk = a.k >> 8;
        for (int wb = warp; wb < a.rows * nblk; wb += NW) {
          const int row = wb / nblk, blk = wb - row * nblk;
          float v[8];
          load8(a.x, a.x_is_bf16, (int64_t)row * a.k + blk * 256 + lane * 8, v);
          uint32_t w0, w1;
          float d;
          int s16, s32;
          quant_block_q8k(v, lane, w0, w1, d, s16, s32);
          *reinterpret_cast<uint2*>(sqs + row * sp.qs_stride + blk * 256 + lane * 8) = make_uint2(w0, w1);
          if (lane == 0) sdsc[wb] = d;
          if ((lane & 1) == 0) sb16[row * (a.k >> 4) + blk * 16 + (lane >> 1)] = (int16_t)s16;
          if ((lane & 3) == 0) sb32[row * (a.k >> 5) + blk * 8 + (lane >> 2)] = (int16_t)s32;
        }
      }
      act.qs = sqs;
      act.dsc = sdsc;
      act.bs16 = sb16;
      act.bs32 = sb32;
      act.qs_stride = sp.qs_stride;
      consumer_sync();
    }

    const int g = lane >> 2, c = lane & 3;
    float acc[MG][4];
#pragma unroll
    for (int mg = 0; mg < MG; mg++)
#pragma unroll
      for (int e = 0; e < 4; e++) acc[mg][e] = 0.f;
    int it = 0, seg = 0;
    bool ok = true;
    for (int64_t u = u0; u < u1 && ok;) {
      const int64_t rt = u / KU;
      const int ku = (int)(u - rt * KU);
      int n = KU - ku;
      if (n > NW) n = NW;
      if ((int64_t)n > u1 - u) n = (int)(u1 - u);
      const int slot = it % a.stages;
      const uint32_t ph = (uint32_t)(it / a.stages) & 1u;
      ok = mbar_wait(&full[slot], ph, abort_flag);
      if (!ok) break;
      if (warp < n) {
        const int kt = (ku + warp) * GROUP;
        int left = a.ktiles - kt;
        if (left > GROUP) left = GROUP;
        TileRegs<DT> r;
        load_tile<DT, SharedLoader>(r, smem + sp.ring + slot * a.stage_bytes + warp * UNIT_BYTES, lane, left);
        tile_mma<DT, MG>(r, lane, act, a.k, kt, a.rows, left, acc);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[slot]);  // after the tile's registers have been consumed
      u += n;
      it++;
      if (ku + n == KU || u == u1) {
        // ---- segment of row-tile rt closed: hand this warp's partial sums to the epilogue warp
        const int rs = seg % RED_SLOTS;
        const uint32_t rph = (uint32_t)(seg / RED_SLOTS) & 1u;
        ok = mbar_wait(&red_empty[rs], rph ^ 1u, abort_flag);
        if (!ok) break;
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
        seg++;
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue warp
    // Walks the same stage sequence to know where segments end; per segment adds the 16
    // warps' partial sums in warp order and either writes y (the CTA owns the row-tile),
    // or parks the sums in the workspace for the owner. The CTA holding the first tile of a
    // row-tile owns it; later CTAs reach into it with the first tiles of their ranges.
    int seg = 0;
    int seg_ka = (int)(u0 % KU);
    bool ok = true;
    for (int64_t u = u0; u < u1 && ok;) {
      const int64_t rt = u / KU;
      const int ku = (int)(u - rt * KU);
      int n = KU - ku;
      if (n > NW) n = NW;
      if ((int64_t)n > u1 - u) n = (int)(u1 - u);
      u += n;
      const int kb = ku + n;
      if (kb != KU && u != u1) continue;
      const int rs = seg % RED_SLOTS;
      const uint32_t rph = (uint32_t)(seg / RED_SLOTS) & 1u;
      ok = mbar_wait(&red_full[rs], rph, abort_flag);
      if (!ok) break;
      const bool owner = seg_ka == 0;
      const bool whole = owner && kb == KU;
      const int64_t rt_end = (rt + 1) * (int64_t)KU;
      const int ncols = a.rows < 8 * MG ? a.rows : 8 * MG;
      for (int idx = lane; idx < ncols * 16; idx += 32) {
        const int col = idx >> 4, row = idx & 15;
        const int mg = col >> 3, e = (col & 7) * 16 + row;
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < NW; w++) s += red[((rs * NW + w) * MG + mg) * 128 + e];
        if (!owner) {
          a.partial[(b * MG + mg) * 128 + e] = s;
          __threadfence();
        } else {
          if (!whole) {
            for (int64_t bp = b + 1; bp < G && (bp * T) / G < rt_end; bp++) {
              volatile int* fl = a.flags + bp;
              const long long t0 = clock64();
              while (*fl == 0) {
                if (*abort_flag || clock64() - t0 > WAIT_CYCLES) { *abort_flag = 1; break; }
                __nanosleep(100);
              }
              __threadfence();
              s += __ldcg(a.partial + (bp * MG + mg) * 128 + e);
            }
          }
          const int64_t nn = rt * TQ_TILE_ROWS + row;
          if (nn < a.n_rows) {
            if (a.bias) s += a.bias[nn];
            a.y[(int64_t)col * a.n_rows + nn] = s;
          }
        }
      }
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&red_empty[rs]);
        if (!owner) {
          __threadfence();
          atomicExch(a.flags + b, 1);
        } else if (!whole) {
          for (int64_t bp = b + 1; bp < G && (bp * T) / G < rt_end; bp++)
            atomicExch(a.flags + bp, 0);  // consumed: back to zero for the next launch
        }
      }
      seg_ka = kb == KU ? 0 : kb;
      seg++;
    }
  }
  __syncthreads();
  if (*abort_flag) {
    // a wait ran out: give copies still in flight time to land in this CTA's shared memory
    for (int i = 0; i < 64; i++) __nanosleep(2000);
    if (threadIdx.x == 0) atomicExch(a.status, 7 /* TURQ_E_TIMEOUT */);
  }
}

// ------------------------------------------------------------------ host side

static int g_smem_optin = -1;

static int smem_budget() {
  if (g_smem_optin < 0) {
    int dev = 0, v = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    g_smem_optin = v > 0 ? v : 48 * 1024;
  }
  return g_smem_optin;
}

bool gemv_int8_fuses_act(int dtype, int64_t m, int64_t k) {
  if (m > 8) return false;
  const int64_t plane = m * (k + 32) + m * (k / 16) * 4 + 1024;
  (void)dtype;
  return plane <= 64 * 1024;
}

size_t gemv_workspace_bytes(int ctas) { return (size_t)ctas * 4 * 128 * 4 + (size_t)ctas * 4 + 256; }

template <int DT, int MG, bool FUSED>
static cudaError_t launch_one(StreamArgs a, int grid, int smem_bytes, cudaStream_t s) {
  static bool configured = false;  // per instantiation; the attribute is per device function
  static int configured_dev = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured || configured_dev != dev) {
    cudaError_t e = cudaFuncSetAttribute(gemv_stream_kernel<DT, MG, FUSED>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         smem_budget());
    if (e != cudaSuccess) return e;
    configured = true;
    configured_dev = dev;
  }
  gemv_stream_kernel<DT, MG, FUSED><<<grid, THREADS, smem_bytes, s>>>(a);
  return cudaGetLastError();
}

template <int DT>
static cudaError_t launch_dt(const uint8_t* tiles, int64_t n_rows, int64_t k, const void* x, int x_dtype,
                             uint8_t* act_scratch, int64_t m, float* y, const float* bias, uint8_t* workspace,
                             int* status, int sm_count, cudaStream_t s, int* launches) {
  constexpr int GROUP = TileGeom<DT>::GROUP;
  constexpr int UNIT_BYTES = TileGeom<DT>::BYTES * GROUP;
  const int ktiles = (int)(k / TileGeom<DT>::ELEMS);
  const int row_tiles = (int)((n_rows + TQ_TILE_ROWS - 1) / TQ_TILE_ROWS);
  const int KU = (ktiles + GROUP - 1) / GROUP;
  const int64_t T = (int64_t)row_tiles * KU;
  int grid = sm_count;
  if ((int64_t)grid > T) grid = (int)T;
  const int fmt = DT == TQ_Q8_0 ? TQ_Q8_0 : TQ_Q8_K;
  const bool fused = gemv_int8_fuses_act(DT, m, k);
  const size_t x_es = x_dtype == TQ_BF16 ? 2 : 4;
  ActPackPlan plan = plan_act_pack(fmt, m, k);
  if (!fused) {
    cudaError_t e = launch_quantize_act_pack(fmt, x, x_dtype, m, k, act_scratch, s);
    if (launches) (*launches)++;
    if (e != cudaSuccess) return e;
  }
  const int stage_bytes = NW * UNIT_BYTES;
  for (int64_t m0 = 0; m0 < m; m0 += 32) {
    const int rows = (int)(m - m0 < 32 ? m - m0 : 32);
    const int mg = rows <= 8 ? 1 : rows <= 16 ? 2 : 4;
    StreamArgs a{};
    a.tiles = tiles;
    a.n_rows = n_rows;
    a.row_tiles = row_tiles;
    a.ktiles = ktiles;
    a.k = (int)k;
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
    a.y = y + m0 * n_rows;
    a.bias = bias;
    a.partial = reinterpret_cast<float*>(workspace);
    a.flags = reinterpret_cast<int*>(workspace + (size_t)sm_count * 4 * 128 * 4);
    a.status = status;
    // ring depth from what the activation planes leave free
    int stages = MAX_STAGES;
    SmemPlan sp{};
    for (; stages >= 2; stages--) {
      sp = plan_smem(DT, mg, fused, rows, (int)k, stages, stage_bytes);
      if (sp.total <= smem_budget()) break;
    }
    if (stages < 2) return cudaErrorInvalidConfiguration;
    a.stages = stages;
    a.stage_bytes = stage_bytes;
    cudaError_t e;
    if (fused) {
      e = launch_one<DT, 1, true>(a, grid, sp.total, s);
    } else if (mg == 1) {
      e = launch_one<DT, 1, false>(a, grid, sp.total, s);
    } else if (mg == 2) {
      e = launch_one<DT, 2, false>(a, grid, sp.total, s);
    } else {
      e = launch_one<DT, 4, false>(a, grid, sp.total, s);
    }
    if (launches) (*launches)++;
    if (e != cudaSuccess) return e;
  }
  return cudaSuccess;
}

cudaError_t launch_gemv_int8(int dtype, const uint8_t* tiles, int64_t n_rows, int64_t k, const void* x, int x_dtype,
                             uint8_t* act_scratch, int64_t m, float* y, const float* bias, uint8_t* workspace,
                             int* status, int sm_count, cudaStream_t s, int* launches) {
  switch (dtype) {
    case TQ_Q8_0: return launch_dt<TQ_Q8_0>(tiles, n_rows, k, x, x_dtype, act_scratch, m, y, bias, workspace, status, sm_count, s, launches);
    case TQ_Q4_K: return launch_dt<TQ_Q4_K>(tiles, n_rows, k, x, x_dtype, act_scratch, m, y, bias, workspace, status, sm_count, s, launches);
    case TQ_Q5_K: return launch_dt<TQ_Q5_K>(tiles, n_rows, k, x, x_dtype, act_scratch, m, y, bias, workspace, status, sm_count, s, launches);
    case TQ_Q6_K: return launch_dt<TQ_Q6_K>(tiles, n_rows, k, x, x_dtype, act_scratch, m, y, bias, workspace, status, sm_count, s, launches);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace turq
