// Decode-sized QMatMul::forward (M up to a few dozen rows): y[m, n] = sum_k x[m, k] W[n, k].
//
// INT8 scheme (the reference CPU scheme): activations are pre-quantized to Q8_K / Q8_0
// planes; a warp owns one device tile (16 weight rows x one wire block) at a time, loads its
// fragment chunks with coalesced 128-bit streaming loads straight into registers and runs
// integer MMAs (m16n8k32 / m16n8k16, weights as the 16-row operand, up to 8 activation rows
// as the narrow operand). Sub-block scales are applied in integers, one f32 scale per
// (super-)block, f32 accumulation across blocks in a fixed order: results do not depend on
// the grid size. The kernel is HBM-bound: every weight byte is read exactly once.
//
// EXACT_F32 scheme: the same tiles are decoded to their exact f32 values and multiplied
// with f32 activations (CUDA-core FMAs).
#include "decode.cuh"
#include "turq_internal.h"

namespace turq {

constexpr int MAX_WARPS = 16;

template <int DT> struct TileGeom;
template <> struct TileGeom<TQ_Q8_0> { static constexpr int BYTES = 544, ELEMS = 32, GROUP = 4; };
template <> struct TileGeom<TQ_Q4_K> { static constexpr int BYTES = 2304, ELEMS = 256, GROUP = 1; };
template <> struct TileGeom<TQ_Q5_K> { static constexpr int BYTES = 2816, ELEMS = 256, GROUP = 1; };
template <> struct TileGeom<TQ_Q6_K> { static constexpr int BYTES = 3360, ELEMS = 256, GROUP = 1; };

// Registers holding one lane's share of a tile (or of GROUP consecutive Q8_0 tiles).
template <int DT> struct TileRegs;
template <> struct TileRegs<TQ_Q8_0> { uint4 q[4]; uint32_t d[4]; };  // d: f16 row g | f16 row g+8 << 16
template <> struct TileRegs<TQ_Q4_K> { uint4 hdr[2]; uint4 q[4]; };
template <> struct TileRegs<TQ_Q5_K> { uint4 hdr[2]; uint4 qh; uint4 q[4]; };
template <> struct TileRegs<TQ_Q6_K> { uint4 sc[2]; uint32_t d; uint4 qh[2]; uint4 ql[4]; };

template <int DT>
__device__ __forceinline__ void load_tile(TileRegs<DT>& r, const uint8_t* __restrict__ t, int lane, int ntiles_left) {
  const int g = lane >> 2;
  if constexpr (DT == TQ_Q8_0) {
#pragma unroll
    for (int u = 0; u < 4; u++) {
      if (u < ntiles_left) {
        const uint8_t* tu = t + 544 * u;
        r.q[u] = ld_stream_v4(tu + TQ_Q8_0_QS + 16 * lane);
        r.d[u] = (uint32_t)ld_u16(tu + 2 * g) | ((uint32_t)ld_u16(tu + 2 * (g + 8)) << 16);
      } else {
        r.q[u] = make_uint4(0, 0, 0, 0);
        r.d[u] = 0;
      }
    }
  } else if constexpr (DT == TQ_Q4_K) {
    r.hdr[0] = ld_v4(t + 16 * g);
    r.hdr[1] = ld_v4(t + 16 * (g + 8));
#pragma unroll
    for (int i = 0; i < 4; i++) r.q[i] = ld_stream_v4(t + TQ_Q4K_QS + 512 * i + 16 * lane);
  } else if constexpr (DT == TQ_Q5_K) {
    r.hdr[0] = ld_v4(t + 16 * g);
    r.hdr[1] = ld_v4(t + 16 * (g + 8));
    r.qh = ld_stream_v4(t + TQ_Q5K_QH + 16 * lane);
#pragma unroll
    for (int i = 0; i < 4; i++) r.q[i] = ld_stream_v4(t + TQ_Q5K_QS + 512 * i + 16 * lane);
  } else {
    r.sc[0] = ld_v4(t + 16 * g);
    r.sc[1] = ld_v4(t + 16 * (g + 8));
    r.d = (uint32_t)ld_u16(t + TQ_Q6K_D + 2 * g) | ((uint32_t)ld_u16(t + TQ_Q6K_D + 2 * (g + 8)) << 16);
    r.qh[0] = ld_stream_v4(t + TQ_Q6K_QH + 16 * lane);
    r.qh[1] = ld_stream_v4(t + TQ_Q6K_QH + 512 + 16 * lane);
#pragma unroll
    for (int i = 0; i < 4; i++) r.ql[i] = ld_stream_v4(t + TQ_Q6K_QL + 512 * i + 16 * lane);
  }
}

__device__ __forceinline__ int s16_lo(uint32_t w) { return (int)(int16_t)(w & 0xFFFFu); }
__device__ __forceinline__ int s16_hi(uint32_t w) { return ((int)w) >> 16; }
__device__ __forceinline__ int s8_at(uint32_t w, int b) { return (int)(int8_t)((w >> (8 * b)) & 0xFFu); }

// One tile (kt) against activation rows [m_base + 8*mg, +8) for mg < MG; accumulates into
// acc[mg][0..3] = (row g, act 2c), (row g, act 2c+1), (row g+8, act 2c), (row g+8, act 2c+1).
template <int DT, int MG>
__device__ __forceinline__ void tile_mma(const TileRegs<DT>& r, int lane, const ActPack& act, int64_t k, int64_t kt,
                                         int m_base, int m_end, int ntiles_left, float (&acc)[MG][4]) {
  const int g = lane >> 2, c = lane & 3;
#pragma unroll
  for (int mg = 0; mg < MG; mg++) {
    const int mb = m_base + 8 * mg + g;           // activation row feeding this lane's B fragment
    const bool bval = mb < m_end;
    const int m0 = m_base + 8 * mg + 2 * c, m1 = m0 + 1;  // activation rows of this lane's C columns
    const bool v0 = m0 < m_end, v1 = m1 < m_end;
    if constexpr (DT == TQ_Q8_0) {
#pragma unroll
      for (int u = 0; u < 4; u++) {
        if (u < ntiles_left) {
          const int64_t kb = kt + u;
          const uint32_t a[4] = {r.q[u].x, r.q[u].z, r.q[u].y, r.q[u].w};
          uint2 b = bval ? ld_v2(act.qs + (int64_t)mb * k + kb * 32 + 8 * c) : make_uint2(0, 0);
          int cc[4] = {0, 0, 0, 0};
          mma_16832<false>(cc, a, b.x, b.y);
          float dw0 = f16_bits_to_f32(r.d[u]), dw1 = f16_bits_to_f32(r.d[u] >> 16);
          float dx0 = v0 ? act.dsc[(int64_t)m0 * (k >> 5) + kb] : 0.f;
          float dx1 = v1 ? act.dsc[(int64_t)m1 * (k >> 5) + kb] : 0.f;
          acc[mg][0] += (float)cc[0] * (dw0 * dx0);
          acc[mg][1] += (float)cc[1] * (dw0 * dx1);
          acc[mg][2] += (float)cc[2] * (dw1 * dx0);
          acc[mg][3] += (float)cc[3] * (dw1 * dx1);
        }
      }
    } else if constexpr (DT == TQ_Q4_K || DT == TQ_Q5_K) {
      int aI[4] = {0, 0, 0, 0}, aM[4] = {0, 0, 0, 0};
      const int8_t* xrow = act.qs + (int64_t)mb * k + kt * 256 + 8 * c;
      uint4 bs0 = v0 ? ld_v4(act.bs32 + (int64_t)m0 * (k >> 5) + kt * 8) : make_uint4(0, 0, 0, 0);
      uint4 bs1 = v1 ? ld_v4(act.bs32 + (int64_t)m1 * (k >> 5) + kt * 8) : make_uint4(0, 0, 0, 0);
      const uint32_t bw0[4] = {bs0.x, bs0.y, bs0.z, bs0.w}, bw1[4] = {bs1.x, bs1.y, bs1.z, bs1.w};
#pragma unroll
      for (int i = 0; i < 4; i++) {
        const uint4 q = r.q[i];
        uint32_t alo[4] = {q.x & 0x0F0F0F0Fu, q.z & 0x0F0F0F0Fu, q.y & 0x0F0F0F0Fu, q.w & 0x0F0F0F0Fu};
        uint32_t ahi[4] = {(q.x >> 4) & 0x0F0F0F0Fu, (q.z >> 4) & 0x0F0F0F0Fu, (q.y >> 4) & 0x0F0F0F0Fu,
                           (q.w >> 4) & 0x0F0F0F0Fu};
        if constexpr (DT == TQ_Q5_K) {
          const uint32_t hw[4] = {r.qh.x, r.qh.z, r.qh.y, r.qh.w};
#pragma unroll
          for (int e = 0; e < 4; e++) {
            alo[e] |= ((hw[e] >> (2 * i)) & 0x01010101u) << 4;
            ahi[e] |= ((hw[e] >> (2 * i + 1)) & 0x01010101u) << 4;
          }
        }
        uint2 blo = bval ? ld_v2(xrow + 64 * i) : make_uint2(0, 0);
        uint2 bhi = bval ? ld_v2(xrow + 64 * i + 32) : make_uint2(0, 0);
        int clo[4] = {0, 0, 0, 0}, chi[4] = {0, 0, 0, 0};
        mma_16832<true>(clo, alo, blo.x, blo.y);
        mma_16832<true>(chi, ahi, bhi.x, bhi.y);
#pragma unroll
        for (int hr = 0; hr < 2; hr++) {
          int scl, mnl, sch, mnh;
          tq_k4_scale_min(r.hdr[hr].y, r.hdr[hr].z, r.hdr[hr].w, 2 * i, &scl, &mnl);
          tq_k4_scale_min(r.hdr[hr].y, r.hdr[hr].z, r.hdr[hr].w, 2 * i + 1, &sch, &mnh);
          aI[2 * hr] += scl * clo[2 * hr] + sch * chi[2 * hr];
          aI[2 * hr + 1] += scl * clo[2 * hr + 1] + sch * chi[2 * hr + 1];
          aM[2 * hr] += mnl * s16_lo(bw0[i]) + mnh * s16_hi(bw0[i]);
          aM[2 * hr + 1] += mnl * s16_lo(bw1[i]) + mnh * s16_hi(bw1[i]);
        }
      }
      float dx0 = v0 ? act.dsc[(int64_t)m0 * (k >> 8) + kt] : 0.f;
      float dx1 = v1 ? act.dsc[(int64_t)m1 * (k >> 8) + kt] : 0.f;
#pragma unroll
      for (int hr = 0; hr < 2; hr++) {
        float d = f16_bits_to_f32(r.hdr[hr].x), dmin = f16_bits_to_f32(r.hdr[hr].x >> 16);
        acc[mg][2 * hr] += (dx0 * d) * (float)aI[2 * hr] - (dx0 * dmin) * (float)aM[2 * hr];
        acc[mg][2 * hr + 1] += (dx1 * d) * (float)aI[2 * hr + 1] - (dx1 * dmin) * (float)aM[2 * hr + 1];
      }
    } else {  // Q6_K
      int aI[4] = {0, 0, 0, 0};
      const int8_t* xrow = act.qs + (int64_t)mb * k + kt * 256 + 4 * c;
      const int16_t* b0p = act.bs16 + (int64_t)m0 * (k >> 4) + kt * 16;
      const int16_t* b1p = act.bs16 + (int64_t)m1 * (k >> 4) + kt * 16;
      uint4 z = make_uint4(0, 0, 0, 0);
      uint4 bs0a = v0 ? ld_v4(b0p) : z, bs0b = v0 ? ld_v4(b0p + 8) : z;
      uint4 bs1a = v1 ? ld_v4(b1p) : z, bs1b = v1 ? ld_v4(b1p + 8) : z;
      const uint32_t bw0[8] = {bs0a.x, bs0a.y, bs0a.z, bs0a.w, bs0b.x, bs0b.y, bs0b.z, bs0b.w};
      const uint32_t bw1[8] = {bs1a.x, bs1a.y, bs1a.z, bs1a.w, bs1b.x, bs1b.y, bs1b.z, bs1b.w};
      const uint32_t qhw[2][4] = {{r.qh[0].x, r.qh[0].y, r.qh[1].x, r.qh[1].y},
                                  {r.qh[0].z, r.qh[0].w, r.qh[1].z, r.qh[1].w}};
      const uint32_t scw[2][4] = {{r.sc[0].x, r.sc[0].y, r.sc[0].z, r.sc[0].w},
                                  {r.sc[1].x, r.sc[1].y, r.sc[1].z, r.sc[1].w}};
#pragma unroll
      for (int j = 0; j < 16; j++) {
        const int i = j >> 2, tw = (j >> 1) & 1, nib = j & 1;
        const uint32_t w0 = tw ? r.ql[i].y : r.ql[i].x, w1 = tw ? r.ql[i].w : r.ql[i].z;
        uint32_t a0 = (nib ? (w0 >> 4) : w0) & 0x0F0F0F0Fu, a1 = (nib ? (w1 >> 4) : w1) & 0x0F0F0F0Fu;
        a0 |= ((qhw[0][j >> 2] >> (2 * (j & 3))) & 0x03030303u) << 4;
        a1 |= ((qhw[1][j >> 2] >> (2 * (j & 3))) & 0x03030303u) << 4;
        uint32_t b = bval ? ld_u32(xrow + 16 * j) : 0u;
        int cc[4] = {0, 0, 0, 0};
        mma_16816_u8s8(cc, a0, a1, b);
        const int sc0 = s8_at(scw[0][j >> 2], j & 3), sc1 = s8_at(scw[1][j >> 2], j & 3);
        const int o0 = 32 * ((j & 1) ? s16_hi(bw0[j >> 1]) : s16_lo(bw0[j >> 1]));
        const int o1 = 32 * ((j & 1) ? s16_hi(bw1[j >> 1]) : s16_lo(bw1[j >> 1]));
        aI[0] += sc0 * (cc[0] - o0);
        aI[1] += sc0 * (cc[1] - o1);
        aI[2] += sc1 * (cc[2] - o0);
        aI[3] += sc1 * (cc[3] - o1);
      }
      float dx0 = v0 ? act.dsc[(int64_t)m0 * (k >> 8) + kt] : 0.f;
      float dx1 = v1 ? act.dsc[(int64_t)m1 * (k >> 8) + kt] : 0.f;
      float d0 = f16_bits_to_f32(r.d), d1 = f16_bits_to_f32(r.d >> 16);
      acc[mg][0] += (dx0 * d0) * (float)aI[0];
      acc[mg][1] += (dx1 * d0) * (float)aI[1];
      acc[mg][2] += (dx0 * d1) * (float)aI[2];
      acc[mg][3] += (dx1 * d1) * (float)aI[3];
    }
  }
}

// grid: persistent CTAs over row-tiles; the CTA's warps split the K-tiles of a row-tile and
// their partial sums are added in warp order through shared memory.
template <int DT, int MG>
__global__ void __launch_bounds__(MAX_WARPS * 32)
gemv_int8_kernel(const uint8_t* __restrict__ tiles, int64_t n_rows, int64_t row_tiles, int64_t ktiles, int64_t k,
                 ActPack act, int m_base, int m_end, float* __restrict__ y, const float* __restrict__ bias) {
  constexpr int GROUP = TileGeom<DT>::GROUP;
  constexpr int TB = TileGeom<DT>::BYTES;
  __shared__ float red[MAX_WARPS][MG][128];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int g = lane >> 2, c = lane & 3;
  for (int64_t rt = blockIdx.x; rt < row_tiles; rt += gridDim.x) {
    float acc[MG][4];
#pragma unroll
    for (int mg = 0; mg < MG; mg++)
#pragma unroll
      for (int e = 0; e < 4; e++) acc[mg][e] = 0.f;
    const uint8_t* base = tiles + rt * ktiles * TB;
    int64_t kt = (int64_t)warp * GROUP;
    const int64_t step = (int64_t)nwarps * GROUP;
    TileRegs<DT> cur, nxt;
    if (kt < ktiles) load_tile<DT>(cur, base + kt * TB, lane, (int)min((int64_t)GROUP, ktiles - kt));
    for (; kt < ktiles; kt += step) {
      const int64_t kn = kt + step;
      if (kn < ktiles) load_tile<DT>(nxt, base + kn * TB, lane, (int)min((int64_t)GROUP, ktiles - kn));
      tile_mma<DT, MG>(cur, lane, act, k, kt, m_base, m_end, (int)min((int64_t)GROUP, ktiles - kt), acc);
      cur = nxt;
    }
    __syncthreads();  // previous row-tile's reduction has been read
#pragma unroll
    for (int mg = 0; mg < MG; mg++) {
      // red[..][mg][col * 16 + row]
      red[warp][mg][(2 * c) * 16 + g] = acc[mg][0];
      red[warp][mg][(2 * c + 1) * 16 + g] = acc[mg][1];
      red[warp][mg][(2 * c) * 16 + g + 8] = acc[mg][2];
      red[warp][mg][(2 * c + 1) * 16 + g + 8] = acc[mg][3];
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < MG * 128; idx += blockDim.x) {
      const int mg = idx >> 7, col = (idx >> 4) & 7, row = idx & 15;
      const int mrow = m_base + 8 * mg + col;
      const int64_t n = rt * TQ_TILE_ROWS + row;
      if (mrow < m_end && n < n_rows) {
        float s = 0.f;
        for (int w = 0; w < nwarps; w++) s += red[w][mg][idx & 127];
        if (bias) s += bias[n];
        y[(int64_t)mrow * n_rows + n] = s;
      }
    }
  }
}

static int pick_warps(int64_t row_tiles, int64_t kgroups, int sm_count) {
  int w = row_tiles >= (int64_t)sm_count * 4 ? 4 : row_tiles >= (int64_t)sm_count * 2 ? 8 : 16;
  if (w > kgroups) w = (int)kgroups;
  if (w < 1) w = 1;
  return w;
}

template <int DT>
static cudaError_t launch_int8_dt(const uint8_t* tiles, int64_t n_rows, int64_t k, const ActPack& act, int64_t m,
                                  float* y, const float* bias, int sm_count, cudaStream_t s, int* launches) {
  const int64_t ktiles = k / TileGeom<DT>::ELEMS;
  const int64_t row_tiles = (n_rows + TQ_TILE_ROWS - 1) / TQ_TILE_ROWS;
  const int64_t kgroups = (ktiles + TileGeom<DT>::GROUP - 1) / TileGeom<DT>::GROUP;
  const int warps = pick_warps(row_tiles, kgroups, sm_count);
  const int ctas_per_sm = 2048 / (warps * 32) > 8 ? 8 : 2048 / (warps * 32);
  int64_t grid = row_tiles < (int64_t)sm_count * ctas_per_sm ? row_tiles : (int64_t)sm_count * ctas_per_sm;
  for (int64_t m0 = 0; m0 < m; m0 += 16) {
    const int m_end = (int)(m0 + 16 < m ? m0 + 16 : m);
    if (m_end - m0 <= 8) {
      gemv_int8_kernel<DT, 1><<<(unsigned)grid, warps * 32, 0, s>>>(tiles, n_rows, row_tiles, ktiles, k, act, (int)m0,
                                                                     m_end, y, bias);
    } else {
      gemv_int8_kernel<DT, 2><<<(unsigned)grid, warps * 32, 0, s>>>(tiles, n_rows, row_tiles, ktiles, k, act, (int)m0,
                                                                     m_end, y, bias);
    }
    if (launches) (*launches)++;
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
  }
  return cudaSuccess;
}

cudaError_t launch_gemv_int8(int dtype, const uint8_t* tiles, int64_t n_rows, int64_t k, const uint8_t* act_scratch,
                             int64_t m, float* y, const float* bias, int sm_count, cudaStream_t s, int* launches) {
  const int fmt = dtype == TQ_Q8_0 ? TQ_Q8_0 : TQ_Q8_K;
  ActPackPlan p = plan_act_pack(fmt, m, k);
  ActPack act;
  act.qs = reinterpret_cast<const int8_t*>(act_scratch + p.off_qs);
  act.dsc = reinterpret_cast<const float*>(act_scratch + p.off_dsc);
  act.bs16 = reinterpret_cast<const int16_t*>(act_scratch + p.off_bs16);
  act.bs32 = reinterpret_cast<const int16_t*>(act_scratch + p.off_bs32);
  switch (dtype) {
    case TQ_Q8_0: return launch_int8_dt<TQ_Q8_0>(tiles, n_rows, k, act, m, y, bias, sm_count, s, launches);
    case TQ_Q4_K: return launch_int8_dt<TQ_Q4_K>(tiles, n_rows, k, act, m, y, bias, sm_count, s, launches);
    case TQ_Q5_K: return launch_int8_dt<TQ_Q5_K>(tiles, n_rows, k, act, m, y, bias, sm_count, s, launches);
    case TQ_Q6_K: return launch_int8_dt<TQ_Q6_K>(tiles, n_rows, k, act, m, y, bias, sm_count, s, launches);
    default: return cudaErrorInvalidValue;
  }
}

// ---------------------------------------------------------------- exact f32 scheme

template <int DT, int MB>
__global__ void __launch_bounds__(MAX_WARPS * 32)
gemv_f32_kernel(const uint8_t* __restrict__ tiles, int64_t n_rows, int64_t row_tiles, int64_t ktiles, int64_t k,
                const void* __restrict__ x, int x_is_bf16, int m_base, int m_end, float* __restrict__ y,
                const float* __restrict__ bias) {
  constexpr int TB = TileGeom<DT>::BYTES;
  constexpr int KE = TileGeom<DT>::ELEMS;
  __shared__ float red[MAX_WARPS][MB][16];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int g = lane >> 2, c = lane & 3;
  for (int64_t rt = blockIdx.x; rt < row_tiles; rt += gridDim.x) {
    float acc[2][MB];
#pragma unroll
    for (int hr = 0; hr < 2; hr++)
#pragma unroll
      for (int mm = 0; mm < MB; mm++) acc[hr][mm] = 0.f;
    const uint8_t* base = tiles + rt * ktiles * TB;
    for (int64_t kt = warp; kt < ktiles; kt += nwarps) {
      decode_tile<DT>(base + kt * TB, lane, [&](int hr, int off, const auto& v) {
        constexpr int NV = sizeof(v) / sizeof(float);
#pragma unroll
        for (int mm = 0; mm < MB; mm++) {
          const int mrow = m_base + mm;
          if (mrow < m_end) {
            const int64_t xi = (int64_t)mrow * k + kt * KE + off;
            float s = acc[hr][mm];
#pragma unroll
            for (int e = 0; e < NV; e++) s = fmaf(v[e], load_act_f32(x, x_is_bf16, xi + e), s);
            acc[hr][mm] = s;
          }
        }
      });
    }
#pragma unroll
    for (int hr = 0; hr < 2; hr++)
#pragma unroll
      for (int mm = 0; mm < MB; mm++) {
        float s = acc[hr][mm];
        s += __shfl_xor_sync(0xFFFFFFFFu, s, 1);
        s += __shfl_xor_sync(0xFFFFFFFFu, s, 2);
        acc[hr][mm] = s;
      }
    __syncthreads();
    if (c == 0) {
#pragma unroll
      for (int mm = 0; mm < MB; mm++) {
        red[warp][mm][g] = acc[0][mm];
        red[warp][mm][g + 8] = acc[1][mm];
      }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < MB * 16; idx += blockDim.x) {
      const int mm = idx >> 4, row = idx & 15;
      const int mrow = m_base + mm;
      const int64_t n = rt * TQ_TILE_ROWS + row;
      if (mrow < m_end && n < n_rows) {
        float s = 0.f;
        for (int w = 0; w < nwarps; w++) s += red[w][mm][row];
        if (bias) s += bias[n];
        y[(int64_t)mrow * n_rows + n] = s;
      }
    }
  }
}

template <int DT>
static cudaError_t launch_f32_dt(const uint8_t* tiles, int64_t n_rows, int64_t k, const void* x, int x_dtype, int64_t m,
                                 float* y, const float* bias, int sm_count, cudaStream_t s, int* launches) {
  constexpr int MB = 4;
  const int64_t ktiles = k / TileGeom<DT>::ELEMS;
  const int64_t row_tiles = (n_rows + TQ_TILE_ROWS - 1) / TQ_TILE_ROWS;
  const int warps = pick_warps(row_tiles, ktiles, sm_count);
  const int ctas_per_sm = 2048 / (warps * 32) > 8 ? 8 : 2048 / (warps * 32);
  int64_t grid = row_tiles < (int64_t)sm_count * ctas_per_sm ? row_tiles : (int64_t)sm_count * ctas_per_sm;
  for (int64_t m0 = 0; m0 < m; m0 += MB) {
    const int m_end = (int)(m0 + MB < m ? m0 + MB : m);
    gemv_f32_kernel<DT, MB><<<(unsigned)grid, warps * 32, 0, s>>>(tiles, n_rows, row_tiles, ktiles, k, x,
                                                                  x_dtype == TQ_BF16, (int)m0, m_end, y, bias);
    if (launches) (*launches)++;
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
  }
  return cudaSuccess;
}

cudaError_t launch_gemv_f32(int dtype, const uint8_t* tiles, int64_t n_rows, int64_t k, const void* x, int x_dtype,
                            int64_t m, float* y, const float* bias, int sm_count, cudaStream_t s, int* launches) {
  switch (dtype) {
    case TQ_Q8_0: return launch_f32_dt<TQ_Q8_0>(tiles, n_rows, k, x, x_dtype, m, y, bias, sm_count, s, launches);
    case TQ_Q4_K: return launch_f32_dt<TQ_Q4_K>(tiles, n_rows, k, x, x_dtype, m, y, bias, sm_count, s, launches);
    case TQ_Q5_K: return launch_f32_dt<TQ_Q5_K>(tiles, n_rows, k, x, x_dtype, m, y, bias, sm_count, s, launches);
    case TQ_Q6_K: return launch_f32_dt<TQ_Q6_K>(tiles, n_rows, k, x, x_dtype, m, y, bias, sm_count, s, launches);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace turq
