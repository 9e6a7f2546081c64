// Per-warp arithmetic of the integer-scheme GEMV: one device tile (16 weight rows x one wire
// block) against up to 8*MG quantized activation rows, with integer MMAs.
//
// Lane l = 4g + c holds weight rows g and g+8 (A fragment) and, as B fragment, the bytes of
// activation row g for the elements lane column c owns (8c..8c+7 of every 32-element
// sub-block; 4c..4c+3 of every 16-element one). Its C fragment is
//   c0 = (row g, act 2c)  c1 = (row g, act 2c+1)  c2 = (row g+8, act 2c)  c3 = (row g+8, act 2c+1).
// Sub-block scales stay integers; one f32 multiply per (super-)block and output element.
#pragma once
#include "device_utils.cuh"
#include "layout.h"

namespace turq {

template <int DT> struct TileGeom;
template <> struct TileGeom<TQ_Q8_0> { static constexpr int BYTES = 544, ELEMS = 32, GROUP = 4; };
template <> struct TileGeom<TQ_Q4_K> { static constexpr int BYTES = 2304, ELEMS = 256, GROUP = 1; };
template <> struct TileGeom<TQ_Q5_K> { static constexpr int BYTES = 2816, ELEMS = 256, GROUP = 1; };
template <> struct TileGeom<TQ_Q6_K> { static constexpr int BYTES = 3360, ELEMS = 256, GROUP = 1; };

// Registers holding one lane's share of a tile (of GROUP consecutive tiles for Q8_0).
template <int DT> struct TileRegs;
template <> struct TileRegs<TQ_Q8_0> { uint4 q[4]; uint32_t d[4]; };  // d: f16 row g | f16 row g+8 << 16
template <> struct TileRegs<TQ_Q4_K> { uint4 hdr[2]; uint4 q[4]; };
template <> struct TileRegs<TQ_Q5_K> { uint4 hdr[2]; uint4 qh; uint4 q[4]; };
template <> struct TileRegs<TQ_Q6_K> { uint4 sc[2]; uint32_t d; uint4 qh[2]; uint4 ql[4]; };

struct GlobalLoader {
  static __device__ __forceinline__ uint4 v4s(const uint8_t* p) { return ld_stream_v4(p); }  // quants: streaming
  static __device__ __forceinline__ uint4 v4(const uint8_t* p) { return ld_v4(p); }          // headers: shared by 4 lanes
  static __device__ __forceinline__ uint32_t u16(const uint8_t* p) { return ld_u16(p); }
};
struct SharedLoader {  // p is a generic pointer into shared memory
  static __device__ __forceinline__ uint4 v4s(const uint8_t* p) { return *reinterpret_cast<const uint4*>(p); }
  static __device__ __forceinline__ uint4 v4(const uint8_t* p) { return *reinterpret_cast<const uint4*>(p); }
  static __device__ __forceinline__ uint32_t u16(const uint8_t* p) { return *reinterpret_cast<const uint16_t*>(p); }
};

template <int DT, class L>
__device__ __forceinline__ void load_tile(TileRegs<DT>& r, const uint8_t* __restrict__ t, int lane, int ntiles_left) {
  const int g = lane >> 2;
  if constexpr (DT == TQ_Q8_0) {
#pragma unroll
    for (int u = 0; u < 4; u++) {
      if (u < ntiles_left) {
        const uint8_t* tu = t + 544 * u;
        r.q[u] = L::v4s(tu + TQ_Q8_0_QS + 16 * lane);
        r.d[u] = L::u16(tu + 2 * g) | (L::u16(tu + 2 * (g + 8)) << 16);
      } else {
        r.q[u] = make_uint4(0, 0, 0, 0);
        r.d[u] = 0;
      }
    }
  } else if constexpr (DT == TQ_Q4_K) {
    r.hdr[0] = L::v4(t + 16 * g);
    r.hdr[1] = L::v4(t + 16 * (g + 8));
#pragma unroll
    for (int i = 0; i < 4; i++) r.q[i] = L::v4s(t + TQ_Q4K_QS + 512 * i + 16 * lane);
  } else if constexpr (DT == TQ_Q5_K) {
    r.hdr[0] = L::v4(t + 16 * g);
    r.hdr[1] = L::v4(t + 16 * (g + 8));
    r.qh = L::v4s(t + TQ_Q5K_QH + 16 * lane);
#pragma unroll
    for (int i = 0; i < 4; i++) r.q[i] = L::v4s(t + TQ_Q5K_QS + 512 * i + 16 * lane);
  } else {
    r.sc[0] = L::v4(t + 16 * g);
    r.sc[1] = L::v4(t + 16 * (g + 8));
    r.d = L::u16(t + TQ_Q6K_D + 2 * g) | (L::u16(t + TQ_Q6K_D + 2 * (g + 8)) << 16);
    r.qh[0] = L::v4s(t + TQ_Q6K_QH + 16 * lane);
    r.qh[1] = L::v4s(t + TQ_Q6K_QH + 512 + 16 * lane);
#pragma unroll
    for (int i = 0; i < 4; i++) r.ql[i] = L::v4s(t + TQ_Q6K_QL + 512 * i + 16 * lane);
  }
}

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

// One tile (index kt of its row) against activation rows [8*mg, 8*mg+8) of the pass, mg < MG;
// `rows` = number of valid activation rows in the pass.
template <int DT, int MG>
__device__ __forceinline__ void tile_mma(const TileRegs<DT>& r, int lane, const ActPack& act, int k, int kt, int rows,
                                         int ntiles_left, float (&acc)[MG][4]) {
  const int g = lane >> 2, c = lane & 3;
#pragma unroll
  for (int mg = 0; mg < MG; mg++) {
    const int mb = 8 * mg + g;  // activation row feeding this lane's B fragment
    const bool bval = mb < rows;
    const int m0 = 8 * mg + 2 * c, m1 = m0 + 1;  // activation rows of this lane's C columns
    const bool v0 = m0 < rows, v1 = m1 < rows;
    if constexpr (DT == TQ_Q8_0) {
      const int nb = k >> 5;
#pragma unroll
      for (int u = 0; u < 4; u++) {
        if (u < ntiles_left) {
          const int kb = kt + u;
          const uint32_t a[4] = {r.q[u].x, r.q[u].z, r.q[u].y, r.q[u].w};
          const uint2 b = bval ? ld_v2(act.qs + mb * act.qs_stride + kb * 32 + 8 * c) : make_uint2(0, 0);
          int cc[4] = {0, 0, 0, 0};
          mma_16832<false>(cc, a, b.x, b.y);
          const float dw0 = f16_bits_to_f32(r.d[u]), dw1 = f16_bits_to_f32(r.d[u] >> 16);
          const float dx0 = v0 ? act.dsc[m0 * nb + kb] : 0.f;
          const float dx1 = v1 ? act.dsc[m1 * nb + kb] : 0.f;
          acc[mg][0] += (float)cc[0] * (dw0 * dx0);
          acc[mg][1] += (float)cc[1] * (dw0 * dx1);
          acc[mg][2] += (float)cc[2] * (dw1 * dx0);
          acc[mg][3] += (float)cc[3] * (dw1 * dx1);
        }
      }
    } else if constexpr (DT == TQ_Q4_K || DT == TQ_Q5_K) {
      // Integer accumulators per C-fragment element: even sub-blocks (low nibbles), odd
      // sub-blocks (Q4_K: high nibbles kept in place, i.e. 16 x the dot product) and mins.
      int aE[4] = {0, 0, 0, 0}, aO[4] = {0, 0, 0, 0}, aM[4];
      const int8_t* xrow = act.qs + mb * act.qs_stride + kt * 256 + 8 * c;
      const uint4 z4 = make_uint4(0, 0, 0, 0);
      const uint4 bs0 = v0 ? ld_v4(act.bs32 + m0 * (k >> 5) + kt * 8) : z4;
      const uint4 bs1 = v1 ? ld_v4(act.bs32 + m1 * (k >> 5) + kt * 8) : z4;
      // 6-bit scales / mins of both rows, four per word, decoded with byte-parallel ops
      uint32_t scl[2], sch[2];
#pragma unroll
      for (int hr = 0; hr < 2; hr++) {
        const uint32_t s0 = r.hdr[hr].y, s1 = r.hdr[hr].z, s2 = r.hdr[hr].w;
        scl[hr] = s0 & 0x3F3F3F3Fu;
        sch[hr] = (s2 & 0x0F0F0F0Fu) | ((s0 >> 2) & 0x30303030u);
        const int mnl = (int)(s1 & 0x3F3F3F3Fu);
        const int mnh = (int)(((s2 >> 4) & 0x0F0F0F0Fu) | ((s1 >> 2) & 0x30303030u));
        // mins: sum_j mn_j * bsum_j, two 16-bit x 8-bit products per instruction
        aM[2 * hr] = __dp2a_hi((int)bs0.w, mnh, __dp2a_lo((int)bs0.z, mnh, __dp2a_hi((int)bs0.y, mnl, __dp2a_lo((int)bs0.x, mnl, 0))));
        aM[2 * hr + 1] = __dp2a_hi((int)bs1.w, mnh, __dp2a_lo((int)bs1.z, mnh, __dp2a_hi((int)bs1.y, mnl, __dp2a_lo((int)bs1.x, mnl, 0))));
      }
#pragma unroll
      for (int i = 0; i < 4; i++) {
        const uint4 q = r.q[i];
        uint32_t alo[4] = {q.x & 0x0F0F0F0Fu, q.z & 0x0F0F0F0Fu, q.y & 0x0F0F0F0Fu, q.w & 0x0F0F0F0Fu};
        uint32_t ahi[4] = {q.x & 0xF0F0F0F0u, q.z & 0xF0F0F0F0u, q.y & 0xF0F0F0F0u, q.w & 0xF0F0F0F0u};
        if constexpr (DT == TQ_Q5_K) {
          // the fifth bit would be worth 256 in place, so the odd sub-block is shifted down
          const uint32_t hw[4] = {r.qh.x, r.qh.z, r.qh.y, r.qh.w};
#pragma unroll
          for (int e = 0; e < 4; e++) {
            alo[e] |= ((hw[e] >> (2 * i)) << 4) & 0x10101010u;
            ahi[e] = (ahi[e] >> 4) | (((hw[e] >> (2 * i + 1)) << 4) & 0x10101010u);
          }
        }
        const uint2 blo = bval ? ld_v2(xrow + 64 * i) : make_uint2(0, 0);
        const uint2 bhi = bval ? ld_v2(xrow + 64 * i + 32) : make_uint2(0, 0);
        int clo[4] = {0, 0, 0, 0}, chi[4] = {0, 0, 0, 0};
        mma_16832<true>(clo, alo, blo.x, blo.y);
        mma_16832<true>(chi, ahi, bhi.x, bhi.y);
#pragma unroll
        for (int hr = 0; hr < 2; hr++) {
          // sub-blocks 2i and 2i+1 are bytes (2i & 3), (2i+1 & 3) of the low or high scale word
          const uint32_t sw = i < 2 ? scl[hr] : sch[hr];
          const int se = (int)__byte_perm(sw, 0, 0x4440 + ((2 * i) & 3));
          const int so = (int)__byte_perm(sw, 0, 0x4440 + ((2 * i + 1) & 3));
          aE[2 * hr] += se * clo[2 * hr];
          aE[2 * hr + 1] += se * clo[2 * hr + 1];
          aO[2 * hr] += so * chi[2 * hr];
          aO[2 * hr + 1] += so * chi[2 * hr + 1];
        }
      }
      const float dx0 = v0 ? act.dsc[m0 * (k >> 8) + kt] : 0.f;
      const float dx1 = v1 ? act.dsc[m1 * (k >> 8) + kt] : 0.f;
#pragma unroll
      for (int hr = 0; hr < 2; hr++) {
        const float d = f16_bits_to_f32(r.hdr[hr].x), dmin = f16_bits_to_f32(r.hdr[hr].x >> 16);
        constexpr int SH = DT == TQ_Q4_K ? 4 : 0;
        const int i0 = aE[2 * hr] + (aO[2 * hr] >> SH), i1 = aE[2 * hr + 1] + (aO[2 * hr + 1] >> SH);
        acc[mg][2 * hr] += (dx0 * d) * (float)i0 - (dx0 * dmin) * (float)aM[2 * hr];
        acc[mg][2 * hr + 1] += (dx1 * d) * (float)i1 - (dx1 * dmin) * (float)aM[2 * hr + 1];
      }
    } else {  // Q6_K: sum_j sc_j * (dot_j(q) - 32 * bsum_j), q unsigned 0..63
      int aI[4] = {0, 0, 0, 0};
      const int8_t* xrow = act.qs + mb * act.qs_stride + kt * 256 + 4 * c;
      const uint32_t scw[2][4] = {{r.sc[0].x, r.sc[0].y, r.sc[0].z, r.sc[0].w},
                                  {r.sc[1].x, r.sc[1].y, r.sc[1].z, r.sc[1].w}};
      {  // the -32 offset: sum_j sc_j * bsum16_j, two products per instruction
        const uint4 z = make_uint4(0, 0, 0, 0);
        const int16_t* b0p = act.bs16 + m0 * (k >> 4) + kt * 16;
        const int16_t* b1p = act.bs16 + m1 * (k >> 4) + kt * 16;
        const uint4 p0 = v0 ? ld_v4(b0p) : z, p1 = v0 ? ld_v4(b0p + 8) : z;
        const uint4 q0 = v1 ? ld_v4(b1p) : z, q1 = v1 ? ld_v4(b1p + 8) : z;
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
          aI[2 * hr] = -32 * o0;
          aI[2 * hr + 1] = -32 * o1;
        }
      }
      const uint32_t qhw[2][4] = {{r.qh[0].x, r.qh[0].y, r.qh[1].x, r.qh[1].y},
                                  {r.qh[0].z, r.qh[0].w, r.qh[1].z, r.qh[1].w}};
#pragma unroll
      for (int j = 0; j < 16; j++) {
        const int i = j >> 2, tw = (j >> 1) & 1, nib = j & 1;
        const uint32_t w0 = tw ? r.ql[i].y : r.ql[i].x, w1 = tw ? r.ql[i].w : r.ql[i].z;
        uint32_t a0 = (nib ? (w0 >> 4) : w0) & 0x0F0F0F0Fu, a1 = (nib ? (w1 >> 4) : w1) & 0x0F0F0F0Fu;
        // 2-bit field (j & 3) of the qh word moved to bits 4..5 of every byte
        const int sh = 2 * (j & 3);
        a0 |= (sh <= 4 ? (qhw[0][j >> 2] << (4 - sh)) : (qhw[0][j >> 2] >> (sh - 4))) & 0x30303030u;
        a1 |= (sh <= 4 ? (qhw[1][j >> 2] << (4 - sh)) : (qhw[1][j >> 2] >> (sh - 4))) & 0x30303030u;
        const uint32_t b = bval ? ld_u32(xrow + 16 * j) : 0u;
        int cc[4] = {0, 0, 0, 0};
        mma_16816_u8s8(cc, a0, a1, b);
        const int sc0 = sext_byte(scw[0][j >> 2], j & 3), sc1 = sext_byte(scw[1][j >> 2], j & 3);
        aI[0] += sc0 * cc[0];
        aI[1] += sc0 * cc[1];
        aI[2] += sc1 * cc[2];
        aI[3] += sc1 * cc[3];
      }
      const float dx0 = v0 ? act.dsc[m0 * (k >> 8) + kt] : 0.f;
      const float dx1 = v1 ? act.dsc[m1 * (k >> 8) + kt] : 0.f;
      const float d0 = f16_bits_to_f32(r.d), d1 = f16_bits_to_f32(r.d >> 16);
      acc[mg][0] += (dx0 * d0) * (float)aI[0];
      acc[mg][1] += (dx1 * d0) * (float)aI[1];
      acc[mg][2] += (dx0 * d1) * (float)aI[2];
      acc[mg][3] += (dx1 * d1) * (float)aI[3];
    }
  }
}

}  // namespace turq
