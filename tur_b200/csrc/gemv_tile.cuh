// Per-warp arithmetic of the integer-scheme GEMV: one device tile (16 weight rows x one wire
// block) held in shared memory against up to 8*MG quantized activation rows, with integer
// MMAs.
//
// Lane l = 4g + c holds weight rows g and g+8 (A fragment) and, as B fragment, the bytes of
// activation row g for the elements lane column c owns (8c..8c+7 of every 32-element
// sub-block; 4c..4c+3 of every 16-element one). Its C fragment is
//   c0 = (row g, act 2c)  c1 = (row g, act 2c+1)  c2 = (row g+8, act 2c)  c3 = (row g+8, act 2c+1).
// Sub-block scales stay integers; one f32 multiply per (super-)block and output element.
// Fragment chunks are read from shared memory where they are needed (128-bit loads), which
// keeps the live register set small (96 registers, no spills, two CTAs per SM).
#pragma once
#include "device_utils.cuh"
#include "layout.h"

namespace turq {

template <int DT> struct TileGeom;
template <> struct TileGeom<TQ_Q8_0> { static constexpr int BYTES = 544, ELEMS = 32, GROUP = 4; };
template <> struct TileGeom<TQ_Q4_K> { static constexpr int BYTES = 2304, ELEMS = 256, GROUP = 1; };
template <> struct TileGeom<TQ_Q5_K> { static constexpr int BYTES = 2816, ELEMS = 256, GROUP = 1; };
template <> struct TileGeom<TQ_Q6_K> { static constexpr int BYTES = 3360, ELEMS = 256, GROUP = 1; };

// Quantized activation planes (global scratch or shared memory), indexed by the row number
// relative to the first row of the pass.
//   qs    int8  [rows][qs_stride]  element order = input order
//   dsc   f32   [rows][k/bs]       bs = 256 (Q8_K) or 32 (Q8_0; the f16-rounded scale)
//   bs16  int16 [rows][k/16]       Q8_K: sums of 16 consecutive qs
//   bs32  int16 [rows][k/32]       Q8_K: sums of 32 consecutive qs
struct ActPack {
  const int8_t* qs;
  const float* dsc;
  const int16_t* bs16;
  const int16_t* bs32;
  int qs_stride;
};

__device__ __forceinline__ int sext_byte(uint32_t w, int b) { return (int)(int8_t)((w >> (8 * b)) & 0xFFu); }
__device__ __forceinline__ uint4 lds_v4(const uint8_t* p) { return *reinterpret_cast<const uint4*>(p); }
__device__ __forceinline__ uint32_t lds_u16(const uint8_t* p) { return *reinterpret_cast<const uint16_t*>(p); }

// One tile (or GROUP consecutive Q8_0 tiles) at shared-memory address t, tile index kt of its
// row, against the `rows` valid activation rows of the pass; adds into acc[mg][0..3].
template <int DT, int MG>
__device__ __forceinline__ void tile_mma(const uint8_t* __restrict__ t, int lane, const ActPack& act, int k, int kt,
                                         int rows, int ntiles_left, float (&acc)[MG][4]) {
  const int g = lane >> 2, c = lane & 3;
  const uint4 z4 = make_uint4(0, 0, 0, 0);
  if constexpr (DT == TQ_Q8_0) {
    const int nb = k >> 5;
#pragma unroll
    for (int u = 0; u < 4; u++) {
      if (u < ntiles_left) {
        const uint8_t* tu = t + 544 * u;
        const uint4 q = lds_v4(tu + TQ_Q8_0_QS + 16 * lane);
        const uint32_t a[4] = {q.x, q.z, q.y, q.w};
        const float dw0 = f16_bits_to_f32(lds_u16(tu + 2 * g)), dw1 = f16_bits_to_f32(lds_u16(tu + 2 * (g + 8)));
        const int kb = kt + u;
#pragma unroll
        for (int mg = 0; mg < MG; mg++) {
          const int mb = 8 * mg + g, m0 = 8 * mg + 2 * c, m1 = m0 + 1;
          const uint2 b = mb < rows ? ld_v2(act.qs + mb * act.qs_stride + kb * 32 + 8 * c) : make_uint2(0, 0);
          int cc[4] = {0, 0, 0, 0};
          mma_16832<false>(cc, a, b.x, b.y);
          const float dx0 = m0 < rows ? act.dsc[m0 * nb + kb] : 0.f;
          const float dx1 = m1 < rows ? act.dsc[m1 * nb + kb] : 0.f;
          acc[mg][0] += (float)cc[0] * (dw0 * dx0);
          acc[mg][1] += (float)cc[1] * (dw0 * dx1);
          acc[mg][2] += (float)cc[2] * (dw1 * dx0);
          acc[mg][3] += (float)cc[3] * (dw1 * dx1);
        }
      }
    }
  } else if constexpr (DT == TQ_Q4_K || DT == TQ_Q5_K) {
    constexpr int QS = DT == TQ_Q4_K ? TQ_Q4K_QS : TQ_Q5K_QS;
    // Integer accumulators per C-fragment element: even sub-blocks (low nibbles), odd
    // sub-blocks (Q4_K: high nibbles kept in place, i.e. 16 x the dot product) and mins.
    int aE[MG][4], aO[MG][4], aM[MG][4];
    const uint4 h0 = lds_v4(t + 16 * g), h1 = lds_v4(t + 16 * (g + 8));
    // 6-bit scales / mins of both rows, four per word, decoded with byte-parallel ops
    uint32_t scl[2], sch[2];
    {
      const uint4 hh[2] = {h0, h1};
#pragma unroll
      for (int hr = 0; hr < 2; hr++) {
        const uint32_t s0 = hh[hr].y, s1 = hh[hr].z, s2 = hh[hr].w;
        scl[hr] = s0 & 0x3F3F3F3Fu;
        sch[hr] = (s2 & 0x0F0F0F0Fu) | ((s0 >> 2) & 0x30303030u);
        const int mnl = (int)(s1 & 0x3F3F3F3Fu);
        const int mnh = (int)(((s2 >> 4) & 0x0F0F0F0Fu) | ((s1 >> 2) & 0x30303030u));
#pragma unroll
        for (int mg = 0; mg < MG; mg++) {
          const int m0 = 8 * mg + 2 * c, m1 = m0 + 1;
          const uint4 bs0 = m0 < rows ? ld_v4(act.bs32 + m0 * (k >> 5) + kt * 8) : z4;
          const uint4 bs1 = m1 < rows ? ld_v4(act.bs32 + m1 * (k >> 5) + kt * 8) : z4;
          // mins: sum_j mn_j * bsum_j, two 16-bit x 8-bit products per instruction
          aM[mg][2 * hr] = __dp2a_hi((int)bs0.w, mnh, __dp2a_lo((int)bs0.z, mnh, __dp2a_hi((int)bs0.y, mnl, __dp2a_lo((int)bs0.x, mnl, 0))));
          aM[mg][2 * hr + 1] = __dp2a_hi((int)bs1.w, mnh, __dp2a_lo((int)bs1.z, mnh, __dp2a_hi((int)bs1.y, mnl, __dp2a_lo((int)bs1.x, mnl, 0))));
        }
      }
    }
#pragma unroll
    for (int mg = 0; mg < MG; mg++)
#pragma unroll
      for (int e = 0; e < 4; e++) aE[mg][e] = aO[mg][e] = 0;
    uint4 qh = z4;
    if constexpr (DT == TQ_Q5_K) qh = lds_v4(t + TQ_Q5K_QH + 16 * lane);
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const uint4 q = lds_v4(t + QS + 512 * i + 16 * lane);
      uint32_t alo[4] = {q.x & 0x0F0F0F0Fu, q.z & 0x0F0F0F0Fu, q.y & 0x0F0F0F0Fu, q.w & 0x0F0F0F0Fu};
      uint32_t ahi[4] = {q.x & 0xF0F0F0F0u, q.z & 0xF0F0F0F0u, q.y & 0xF0F0F0F0u, q.w & 0xF0F0F0F0u};
      if constexpr (DT == TQ_Q5_K) {
        // the fifth bit would be worth 256 in place, so the odd sub-block is shifted down
        const uint32_t hw[4] = {qh.x, qh.z, qh.y, qh.w};
#pragma unroll
        for (int e = 0; e < 4; e++) {
          alo[e] |= ((hw[e] >> (2 * i)) << 4) & 0x10101010u;
          ahi[e] = (ahi[e] >> 4) | (((hw[e] >> (2 * i + 1)) << 4) & 0x10101010u);
        }
      }
      // sub-blocks 2i and 2i+1 are bytes (2i & 3), (2i+1 & 3) of the low or high scale word
      int se[2], so[2];
#pragma unroll
      for (int hr = 0; hr < 2; hr++) {
        const uint32_t sw = i < 2 ? scl[hr] : sch[hr];
        se[hr] = (int)__byte_perm(sw, 0, 0x4440 + ((2 * i) & 3));
        so[hr] = (int)__byte_perm(sw, 0, 0x4440 + ((2 * i + 1) & 3));
      }
#pragma unroll
      for (int mg = 0; mg < MG; mg++) {
        const int mb = 8 * mg + g;
        const int8_t* xrow = act.qs + mb * act.qs_stride + kt * 256 + 8 * c + 64 * i;
        const uint2 blo = mb < rows ? ld_v2(xrow) : make_uint2(0, 0);
        const uint2 bhi = mb < rows ? ld_v2(xrow + 32) : make_uint2(0, 0);
        int clo[4] = {0, 0, 0, 0}, chi[4] = {0, 0, 0, 0};
        mma_16832<true>(clo, alo, blo.x, blo.y);
        mma_16832<true>(chi, ahi, bhi.x, bhi.y);
#pragma unroll
        for (int hr = 0; hr < 2; hr++) {
          aE[mg][2 * hr] += se[hr] * clo[2 * hr];
          aE[mg][2 * hr + 1] += se[hr] * clo[2 * hr + 1];
          aO[mg][2 * hr] += so[hr] * chi[2 * hr];
          aO[mg][2 * hr + 1] += so[hr] * chi[2 * hr + 1];
        }
      }
    }
    const float d[2] = {f16_bits_to_f32(h0.x), f16_bits_to_f32(h1.x)};
    const float dmin[2] = {f16_bits_to_f32(h0.x >> 16), f16_bits_to_f32(h1.x >> 16)};
#pragma unroll
    for (int mg = 0; mg < MG; mg++) {
      const int m0 = 8 * mg + 2 * c, m1 = m0 + 1;
      const float dx0 = m0 < rows ? act.dsc[m0 * (k >> 8) + kt] : 0.f;
      const float dx1 = m1 < rows ? act.dsc[m1 * (k >> 8) + kt] : 0.f;
#pragma unroll
      for (int hr = 0; hr < 2; hr++) {
        constexpr int SH = DT == TQ_Q4_K ? 4 : 0;
        const int i0 = aE[mg][2 * hr] + (aO[mg][2 * hr] >> SH), i1 = aE[mg][2 * hr + 1] + (aO[mg][2 * hr + 1] >> SH);
        acc[mg][2 * hr] += (dx0 * d[hr]) * (float)i0 - (dx0 * dmin[hr]) * (float)aM[mg][2 * hr];
        acc[mg][2 * hr + 1] += (dx1 * d[hr]) * (float)i1 - (dx1 * dmin[hr]) * (float)aM[mg][2 * hr + 1];
      }
    }
  } else {  // Q6_K: sum_j sc_j * (dot_j(q) - 32 * bsum_j), q unsigned 0..63
    int aI[MG][4];
    const uint4 s0v = lds_v4(t + 16 * g), s1v = lds_v4(t + 16 * (g + 8));
    const uint32_t scw[2][4] = {{s0v.x, s0v.y, s0v.z, s0v.w}, {s1v.x, s1v.y, s1v.z, s1v.w}};
#pragma unroll
    for (int mg = 0; mg < MG; mg++) {
      // the -32 offset: sum_j sc_j * bsum16_j, two products per instruction
      const int m0 = 8 * mg + 2 * c, m1 = m0 + 1;
      const int16_t* b0p = act.bs16 + m0 * (k >> 4) + kt * 16;
      const int16_t* b1p = act.bs16 + m1 * (k >> 4) + kt * 16;
      const uint4 p0 = m0 < rows ? ld_v4(b0p) : z4, p1 = m0 < rows ? ld_v4(b0p + 8) : z4;
      const uint4 q0 = m1 < rows ? ld_v4(b1p) : z4, q1 = m1 < rows ? ld_v4(b1p + 8) : z4;
      const uint32_t bw0[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
      const uint32_t bw1[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
      for (int hr = 0; hr < 2; hr++) {
        int o0 = 0, o1 = 0;
#pragma unroll
        for (int w = 0; w < 4; w++) {
          o0 = __dp2a_hi((int)bw0[2 * w + 1], (int)scw[hr][w], __dp2a_lo((int)bw0[2 * w], (int)scw[hr][w], o0));
          o1 = __dp2a_hi((int)bw1[2 * w + 1], (int)scw[hr][w], __dp2a_lo((int)bw1[2 * w], (int)scw[hr][w], o1));
        }
        aI[mg][2 * hr] = -32 * o0;
        aI[mg][2 * hr + 1] = -32 * o1;
      }
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const uint4 ql = lds_v4(t + TQ_Q6K_QL + 512 * i + 16 * lane);
      const uint4 qh = lds_v4(t + TQ_Q6K_QH + 512 * (i >> 1) + 16 * lane);
      // qh word of this chunk's four sub-blocks: chunk i of ql pairs with qh word (i & 1) of each row
      const uint32_t qh0 = (i & 1) ? qh.y : qh.x, qh1 = (i & 1) ? qh.w : qh.z;
#pragma unroll
      for (int jj = 0; jj < 4; jj++) {
        const int j = 4 * i + jj;
        const int tw = jj >> 1, nib = jj & 1;
        const uint32_t w0 = tw ? ql.y : ql.x, w1 = tw ? ql.w : ql.z;
        uint32_t a0 = (nib ? (w0 >> 4) : w0) & 0x0F0F0F0Fu, a1 = (nib ? (w1 >> 4) : w1) & 0x0F0F0F0Fu;
        // 2-bit field jj of the qh word moved to bits 4..5 of every byte
        const int sh = 2 * jj;
        a0 |= (sh <= 4 ? (qh0 << (4 - sh)) : (qh0 >> (sh - 4))) & 0x30303030u;
        a1 |= (sh <= 4 ? (qh1 << (4 - sh)) : (qh1 >> (sh - 4))) & 0x30303030u;
        const int sc0 = sext_byte(scw[0][i], jj), sc1 = sext_byte(scw[1][i], jj);
#pragma unroll
        for (int mg = 0; mg < MG; mg++) {
          const int mb = 8 * mg + g;
          const uint32_t b = mb < rows ? ld_u32(act.qs + mb * act.qs_stride + kt * 256 + 4 * c + 16 * j) : 0u;
          int cc[4] = {0, 0, 0, 0};
          mma_16816_u8s8(cc, a0, a1, b);
          aI[mg][0] += sc0 * cc[0];
          aI[mg][1] += sc0 * cc[1];
          aI[mg][2] += sc1 * cc[2];
          aI[mg][3] += sc1 * cc[3];
        }
      }
    }
    const float d0 = f16_bits_to_f32(lds_u16(t + TQ_Q6K_D + 2 * g)), d1 = f16_bits_to_f32(lds_u16(t + TQ_Q6K_D + 2 * (g + 8)));
#pragma unroll
    for (int mg = 0; mg < MG; mg++) {
      const int m0 = 8 * mg + 2 * c, m1 = m0 + 1;
      const float dx0 = m0 < rows ? act.dsc[m0 * (k >> 8) + kt] : 0.f;
      const float dx1 = m1 < rows ? act.dsc[m1 * (k >> 8) + kt] : 0.f;
      acc[mg][0] += (dx0 * d0) * (float)aI[mg][0];
      acc[mg][1] += (dx1 * d0) * (float)aI[mg][1];
      acc[mg][2] += (dx0 * d1) * (float)aI[mg][2];
      acc[mg][3] += (dx1 * d1) * (float)aI[mg][3];
    }
  }
}

// The same tile against ONE activation row (decode, M = 1), K-quant types. With a single row the
// 8-wide activation operand of the MMA would carry seven rows of zeros and every lane would
// still apply the sub-block scales to all four of its C elements. Here the eight B columns carry
// the eight 32-element sub-blocks instead (16-element ones for Q6_K, in two accumulator sets):
// the MMA of sub-block s gets the activation bytes in column s only, so after the tile's MMAs
// C[row][j] is the integer dot of `row` with sub-block j. A lane then scales just its own two
// (four) sub-blocks, the four lanes of a row add their integers with two shuffles, and the
// float step is the one of the general function - same integers, same float operations, so
// the result has the bits of tile_mma<DT, 1> with rows = 1. Each lane loads one 8-byte (two
// 4-byte) activation fragment per tile instead of eight (sixteen).
template <int DT>
__device__ __forceinline__ void tile_mma_row1(const uint8_t* __restrict__ t, int lane, const ActPack& act, int k, int kt,
                                              float (&acc)[1][4]) {
  static_assert(DT == TQ_Q4_K || DT == TQ_Q5_K || DT == TQ_Q6_K, "single-row variant exists for the K-quants");
  const int g = lane >> 2, c = lane & 3;
  const float dx0 = act.dsc[kt];
  if constexpr (DT == TQ_Q4_K || DT == TQ_Q5_K) {
    constexpr int QS = DT == TQ_Q4_K ? TQ_Q4K_QS : TQ_Q5K_QS;
    constexpr int SH = DT == TQ_Q4_K ? 4 : 0;
    const uint4 h0 = lds_v4(t + 16 * g), h1 = lds_v4(t + 16 * (g + 8));
    const uint4 hh[2] = {h0, h1};
    const uint4 bs0 = ld_v4(act.bs32 + kt * 8);
    uint32_t scl[2], sch[2];
    int aM[2];
#pragma unroll
    for (int hr = 0; hr < 2; hr++) {
      const uint32_t s0 = hh[hr].y, s1 = hh[hr].z, s2 = hh[hr].w;
      scl[hr] = s0 & 0x3F3F3F3Fu;
      sch[hr] = (s2 & 0x0F0F0F0Fu) | ((s0 >> 2) & 0x30303030u);
      const int mnl = (int)(s1 & 0x3F3F3F3Fu);
      const int mnh = (int)(((s2 >> 4) & 0x0F0F0F0Fu) | ((s1 >> 2) & 0x30303030u));
      aM[hr] = __dp2a_hi((int)bs0.w, mnh, __dp2a_lo((int)bs0.z, mnh, __dp2a_hi((int)bs0.y, mnl, __dp2a_lo((int)bs0.x, mnl, 0))));
    }
    // this lane's activation fragment: elements 8c .. 8c+7 of sub-block g
    const uint2 frag = ld_v2(act.qs + kt * 256 + 32 * g + 8 * c);
    int cc[4] = {0, 0, 0, 0};
    uint4 qh = make_uint4(0, 0, 0, 0);
    if constexpr (DT == TQ_Q5_K) qh = lds_v4(t + TQ_Q5K_QH + 16 * lane);
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const uint4 q = lds_v4(t + QS + 512 * i + 16 * lane);
      uint32_t alo[4] = {q.x & 0x0F0F0F0Fu, q.z & 0x0F0F0F0Fu, q.y & 0x0F0F0F0Fu, q.w & 0x0F0F0F0Fu};
      uint32_t ahi[4] = {q.x & 0xF0F0F0F0u, q.z & 0xF0F0F0F0u, q.y & 0xF0F0F0F0u, q.w & 0xF0F0F0F0u};
      if constexpr (DT == TQ_Q5_K) {
        const uint32_t hw[4] = {qh.x, qh.z, qh.y, qh.w};
#pragma unroll
        for (int e = 0; e < 4; e++) {
          alo[e] |= ((hw[e] >> (2 * i)) << 4) & 0x10101010u;
          ahi[e] = (ahi[e] >> 4) | (((hw[e] >> (2 * i + 1)) << 4) & 0x10101010u);
        }
      }
      const bool lo_mine = g == 2 * i, hi_mine = g == 2 * i + 1;
      mma_16832<true>(cc, alo, lo_mine ? frag.x : 0u, lo_mine ? frag.y : 0u);
      mma_16832<true>(cc, ahi, hi_mine ? frag.x : 0u, hi_mine ? frag.y : 0u);
    }
    // cc[0] = (row g, sub-block 2c), cc[1] = (row g, 2c+1), cc[2] = (row g+8, 2c), cc[3] = (row g+8, 2c+1)
    const int sh_even = 8 * ((2 * c) & 3), sh_odd = sh_even + 8;
    int p[2];
#pragma unroll
    for (int hr = 0; hr < 2; hr++) {
      const uint32_t sw = c < 2 ? scl[hr] : sch[hr];
      const int s_even = (int)((sw >> sh_even) & 0xFFu), s_odd = (int)((sw >> sh_odd) & 0xFFu);
      p[hr] = s_even * cc[2 * hr] + ((s_odd * cc[2 * hr + 1]) >> SH);
      p[hr] += __shfl_xor_sync(0xFFFFFFFFu, p[hr], 1);
      p[hr] += __shfl_xor_sync(0xFFFFFFFFu, p[hr], 2);
    }
    const float d[2] = {f16_bits_to_f32(h0.x), f16_bits_to_f32(h1.x)};
    const float dmin[2] = {f16_bits_to_f32(h0.x >> 16), f16_bits_to_f32(h1.x >> 16)};
    acc[0][0] += (dx0 * d[0]) * (float)p[0] - (dx0 * dmin[0]) * (float)aM[0];
    acc[0][2] += (dx0 * d[1]) * (float)p[1] - (dx0 * dmin[1]) * (float)aM[1];
  } else {  // Q6_K: 16 sub-blocks of 16 elements -> two accumulator sets of 8 columns
    const uint4 s0v = lds_v4(t + 16 * g), s1v = lds_v4(t + 16 * (g + 8));
    const uint32_t scw[2][4] = {{s0v.x, s0v.y, s0v.z, s0v.w}, {s1v.x, s1v.y, s1v.z, s1v.w}};
    const int16_t* b0p = act.bs16 + kt * 16;
    const uint4 p0 = ld_v4(b0p), p1 = ld_v4(b0p + 8);
    const uint32_t bw0[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
    int off32[2];
#pragma unroll
    for (int hr = 0; hr < 2; hr++) {
      int o0 = 0;
#pragma unroll
      for (int w = 0; w < 4; w++) o0 = __dp2a_hi((int)bw0[2 * w + 1], (int)scw[hr][w], __dp2a_lo((int)bw0[2 * w], (int)scw[hr][w], o0));
      off32[hr] = -32 * o0;
    }
    // this lane's activation fragments: elements 4c .. 4c+3 of sub-blocks g and g + 8
    const uint32_t fa = ld_u32(act.qs + kt * 256 + 16 * g + 4 * c);
    const uint32_t fb = ld_u32(act.qs + kt * 256 + 16 * (g + 8) + 4 * c);
    int ca[4] = {0, 0, 0, 0}, cb[4] = {0, 0, 0, 0};
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const uint4 ql = lds_v4(t + TQ_Q6K_QL + 512 * i + 16 * lane);
      const uint4 qh = lds_v4(t + TQ_Q6K_QH + 512 * (i >> 1) + 16 * lane);
      const uint32_t qh0 = (i & 1) ? qh.y : qh.x, qh1 = (i & 1) ? qh.w : qh.z;
#pragma unroll
      for (int jj = 0; jj < 4; jj++) {
        const int j = 4 * i + jj;
        const int tw = jj >> 1, nib = jj & 1;
        const uint32_t w0 = tw ? ql.y : ql.x, w1 = tw ? ql.w : ql.z;
        uint32_t a0 = (nib ? (w0 >> 4) : w0) & 0x0F0F0F0Fu, a1 = (nib ? (w1 >> 4) : w1) & 0x0F0F0F0Fu;
        const int sh = 2 * jj;
        a0 |= (sh <= 4 ? (qh0 << (4 - sh)) : (qh0 >> (sh - 4))) & 0x30303030u;
        a1 |= (sh <= 4 ? (qh1 << (4 - sh)) : (qh1 >> (sh - 4))) & 0x30303030u;
        if (j < 8) {
          mma_16816_u8s8(ca, a0, a1, g == j ? fa : 0u);
        } else {
          mma_16816_u8s8(cb, a0, a1, g == j - 8 ? fb : 0u);
        }
      }
    }
    // ca: sub-blocks 2c, 2c+1 (rows g | g+8); cb: sub-blocks 8+2c, 9+2c
    const int b_even = (2 * c) & 3, b_odd = b_even + 1;
    int p[2];
#pragma unroll
    for (int hr = 0; hr < 2; hr++) {
      const uint32_t wa = (c >> 1) ? scw[hr][1] : scw[hr][0];
      const uint32_t wb = (c >> 1) ? scw[hr][3] : scw[hr][2];
      p[hr] = sext_byte(wa, b_even) * ca[2 * hr] + sext_byte(wa, b_odd) * ca[2 * hr + 1] + sext_byte(wb, b_even) * cb[2 * hr] +
              sext_byte(wb, b_odd) * cb[2 * hr + 1];
      p[hr] += __shfl_xor_sync(0xFFFFFFFFu, p[hr], 1);
      p[hr] += __shfl_xor_sync(0xFFFFFFFFu, p[hr], 2);
      p[hr] += off32[hr];
    }
    const float d0 = f16_bits_to_f32(lds_u16(t + TQ_Q6K_D + 2 * g)), d1 = f16_bits_to_f32(lds_u16(t + TQ_Q6K_D + 2 * (g + 8)));
    acc[0][0] += (dx0 * d0) * (float)p[0];
    acc[0][2] += (dx0 * d1) * (float)p[1];
  }
}

}  // namespace turq
