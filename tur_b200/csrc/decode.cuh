// Per-lane decoding of one device tile (16 rows x one wire block) to exact f32 values.
// Used by the dequantize kernel and by the exact-f32 GEMV. The float order is the one that
// defines the format (gguf-py quants.py:513-522, 540-549, 561-572, 398-401): sub-block scale
// product first, then times the integer, then the subtraction, each separately rounded.
#pragma once
#include "device_utils.cuh"
#include "layout.h"

namespace turq {

// f(hr, elem_off, v): lane owns tile row g + 8*hr, elements [elem_off, elem_off + NV) of the
// K-tile, with exact f32 values v[0..NV).
template <int DT, class F>
__host__ __device__ __forceinline__ void decode_tile(const uint8_t* __restrict__ t, int lane, F&& f) {
  const int g = lane >> 2, c = lane & 3;
  if constexpr (DT == TQ_Q8_0) {
    uint4 q = ld_stream_v4(t + TQ_Q8_0_QS + 16 * lane);
    const uint32_t w[2][2] = {{q.x, q.y}, {q.z, q.w}};
#pragma unroll
    for (int hr = 0; hr < 2; hr++) {
      float d = f16_bits_to_f32(ld_u16(t + 2 * (g + 8 * hr)));
      float v[8];
#pragma unroll
      for (int e = 0; e < 8; e++) {
        int qi = (int)(int8_t)((w[hr][e >> 2] >> (8 * (e & 3))) & 0xFF);
        v[e] = mul_rn((float)qi, d);
      }
      f(hr, 8 * c, v);
    }
  } else if constexpr (DT == TQ_Q4_K || DT == TQ_Q5_K) {
    constexpr int QS = DT == TQ_Q4_K ? TQ_Q4K_QS : TQ_Q5K_QS;
    uint4 hdr[2] = {ld_v4(t + 16 * g), ld_v4(t + 16 * (g + 8))};
    uint32_t qh[2][2] = {{0, 0}, {0, 0}};
    if constexpr (DT == TQ_Q5_K) {
      uint4 h = ld_stream_v4(t + TQ_Q5K_QH + 16 * lane);
      qh[0][0] = h.x; qh[0][1] = h.y; qh[1][0] = h.z; qh[1][1] = h.w;
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
      uint4 q = ld_stream_v4(t + QS + 512 * i + 16 * lane);
      const uint32_t w[2][2] = {{q.x, q.y}, {q.z, q.w}};
#pragma unroll
      for (int hr = 0; hr < 2; hr++) {
        float d = f16_bits_to_f32(hdr[hr].x), dmin = f16_bits_to_f32(hdr[hr].x >> 16);
#pragma unroll
        for (int nib = 0; nib < 2; nib++) {
          const int j = 2 * i + nib;
          int sc, mn;
          tq_k4_scale_min(hdr[hr].y, hdr[hr].z, hdr[hr].w, j, &sc, &mn);
          float dl = mul_rn(d, (float)sc), ml = mul_rn(dmin, (float)mn);
          float v[8];
#pragma unroll
          for (int e = 0; e < 8; e++) {
            uint32_t qi = (w[hr][e >> 2] >> (8 * (e & 3) + 4 * nib)) & 0x0F;
            if constexpr (DT == TQ_Q5_K) qi |= ((qh[hr][e >> 2] >> (8 * (e & 3) + j)) & 1u) << 4;
            v[e] = sub_rn(mul_rn(dl, (float)qi), ml);
          }
          f(hr, 32 * j + 8 * c, v);
        }
      }
    }
  } else if constexpr (DT == TQ_Q6_K) {
    uint4 scv[2] = {ld_v4(t + 16 * g), ld_v4(t + 16 * (g + 8))};
    float d[2] = {f16_bits_to_f32(ld_u16(t + TQ_Q6K_D + 2 * g)),
                  f16_bits_to_f32(ld_u16(t + TQ_Q6K_D + 2 * (g + 8)))};
    uint4 h0 = ld_stream_v4(t + TQ_Q6K_QH + 16 * lane);
    uint4 h1 = ld_stream_v4(t + TQ_Q6K_QH + 512 + 16 * lane);
    const uint32_t qh[2][4] = {{h0.x, h0.y, h1.x, h1.y}, {h0.z, h0.w, h1.z, h1.w}};
#pragma unroll
    for (int i = 0; i < 4; i++) {
      uint4 q = ld_stream_v4(t + TQ_Q6K_QL + 512 * i + 16 * lane);
      const uint32_t ql[2][2] = {{q.x, q.y}, {q.z, q.w}};
#pragma unroll
      for (int hr = 0; hr < 2; hr++) {
        const uint32_t s4[4] = {scv[hr].x, scv[hr].y, scv[hr].z, scv[hr].w};
#pragma unroll
        for (int jj = 0; jj < 4; jj++) {
          const int j = 4 * i + jj;           // sub-block 0..15
          const int tw = jj >> 1, nib = jj & 1;  // ql word inside this chunk, nibble half
          int sc = (int)(int8_t)((s4[j >> 2] >> (8 * (j & 3))) & 0xFF);
          float dl = mul_rn(d[hr], (float)sc);
          float v[4];
#pragma unroll
          for (int e = 0; e < 4; e++) {
            uint32_t lo = (ql[hr][tw] >> (8 * e + 4 * nib)) & 0x0F;
            uint32_t hi = (qh[hr][j >> 2] >> (8 * e + 2 * (j & 3))) & 3u;
            int qi = (int)(lo | (hi << 4)) - 32;
            v[e] = mul_rn(dl, (float)qi);
          }
          f(hr, 16 * j + 4 * c, v);
        }
      }
    }
  }
}

}  // namespace turq
