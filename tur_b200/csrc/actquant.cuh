// Warp-level activation quantization shared by the stand-alone kernels and the GEMV that
// quantizes its activations in shared memory. Same arithmetic in both places, so the wire
// blocks of the public entry and the planes the GEMV consumes always agree.
#pragma once
#include "device_utils.cuh"

// The Q8_K activation quantizer has three choices on which GGML revisions and candle differ.
// They are compile-time switches here and (under the TQO_ prefix) in the CPU oracle, which
// must be built with the same values; turq_q8k_variant() reports what a library was built with.
//   TURQ_Q8K_DIVISOR          128 (default) or 127: magnitude the block maximum maps to
//   TURQ_Q8K_NEG_SCALE        1 (default): iscale = -DIVISOR / (signed element of largest
//                             magnitude, first one on ties), so that element maps to -DIVISOR
//                             and d = 1/iscale carries its sign; 0: iscale = DIVISOR / amax
//   TURQ_Q8K_ROUND_HALF_EVEN  0 (default): ties round away from zero (Rust's f32::round, which
//                             candle-core's BlockQ8K::from_float applies); 1: ties to even
//                             (GGML's nearest_int)
// The defaults are candle-core's published behaviour; the result is then clamped at 127.
#ifndef TURQ_Q8K_DIVISOR
#define TURQ_Q8K_DIVISOR 128
#endif
#ifndef TURQ_Q8K_NEG_SCALE
#define TURQ_Q8K_NEG_SCALE 1
#endif
#ifndef TURQ_Q8K_ROUND_HALF_EVEN
#define TURQ_Q8K_ROUND_HALF_EVEN 0
#endif
#if TURQ_Q8K_DIVISOR != 127 && TURQ_Q8K_DIVISOR != 128
#error "TURQ_Q8K_DIVISOR must be 127 or 128"
#endif

namespace turq {

// mx = the element of largest magnitude (signed), amax = its magnitude (> 0)
__device__ __forceinline__ float q8k_iscale(float mx, float amax) {
#if TURQ_Q8K_NEG_SCALE
  (void)amax;
  return __fdiv_rn(-(float)TURQ_Q8K_DIVISOR, mx);
#else
  (void)mx;
  return __fdiv_rn((float)TURQ_Q8K_DIVISOR, amax);
#endif
}
__device__ __forceinline__ int q8k_round(float v) {
#if TURQ_Q8K_ROUND_HALF_EVEN
  return min(127, __float2int_rn(v));
#else
  return min(127, (int)roundf(v));
#endif
}

__device__ __forceinline__ void load8(const void* x, int is_bf16, int64_t idx, float (&v)[8]) {
  if (is_bf16) {
    uint4 r = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(x) + idx);
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int e = 0; e < 4; e++) {
      v[2 * e] = __uint_as_float(w[e] << 16);
      v[2 * e + 1] = __uint_as_float(w[e] & 0xFFFF0000u);
    }
  } else {
    const float4* p = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(x) + idx);
    float4 a = p[0], b = p[1];
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
}

__device__ __forceinline__ uint32_t pack4(const int* q) {
  return (q[0] & 0xFF) | ((q[1] & 0xFF) << 8) | ((q[2] & 0xFF) << 16) | ((uint32_t)(q[3] & 0xFF) << 24);
}

// Q8_K block of 256 values held 8 per lane (lane owns elements 8*lane .. 8*lane+7).
// Default semantics: the element of largest magnitude (first on ties) maps to -128 before the
// clamp at 127, ties round away from zero, d = 1/iscale (switches above). Returns the packed quants
// (w0, w1), the block scale d and the sums of this lane's aligned group of 16 and of 32.
__device__ __forceinline__ void quant_block_q8k(const float (&v)[8], int lane, uint32_t& w0, uint32_t& w1, float& d,
                                                int& s16, int& s32) {
  // arg-max of |v| over the block with "first index wins" on ties: per-lane scan, then one
  // warp-wide integer max on the float bit patterns (monotonic for non-negative floats) and a
  // ballot to find the lowest lane that holds it.
  uint32_t umax = 0;
  float mx = 0.f;
#pragma unroll
  for (int e = 0; e < 8; e++) {
    const uint32_t ua = __float_as_uint(fabsf(v[e]));
    if (ua > umax) { umax = ua; mx = v[e]; }
  }
  const uint32_t wmax = __reduce_max_sync(0xFFFFFFFFu, umax);
  const uint32_t holders = __ballot_sync(0xFFFFFFFFu, umax == wmax);
  mx = __shfl_sync(0xFFFFFFFFu, mx, __ffs(holders) - 1);
  const float amax = __uint_as_float(wmax);
  (void)lane;
  int q[8];
  d = 0.f;
  if (amax == 0.f) {
#pragma unroll
    for (int e = 0; e < 8; e++) q[e] = 0;
  } else {
    const float iscale = q8k_iscale(mx, amax);
#pragma unroll
    for (int e = 0; e < 8; e++) q[e] = q8k_round(__fmul_rn(iscale, v[e]));
    d = __fdiv_rn(1.f, iscale);
  }
  int s8 = 0;
#pragma unroll
  for (int e = 0; e < 8; e++) s8 += q[e];
  s16 = s8 + __shfl_xor_sync(0xFFFFFFFFu, s8, 1);
  s32 = s16 + __shfl_xor_sync(0xFFFFFFFFu, s16, 2);
  w0 = pack4(q);
  w1 = pack4(q + 4);
}

// The same Q8_K block held 16 values per lane by one half of a warp (lane & 15 owns elements
// 16*(lane&15) .. +15), so a warp quantizes two blocks at once. Identical results.
__device__ __forceinline__ void quant_block_q8k_half(const float (&v)[16], int lane, uint32_t (&w)[4], float& d, int& s16,
                                                     int& s32) {
  const uint32_t half_mask = 0xFFFFu << (lane & 16);
  uint32_t umax = 0;
  float mx = 0.f;
#pragma unroll
  for (int e = 0; e < 16; e++) {
    const uint32_t ua = __float_as_uint(fabsf(v[e]));
    if (ua > umax) { umax = ua; mx = v[e]; }
  }
  const uint32_t wmax = __reduce_max_sync(half_mask, umax);
  const uint32_t holders = __ballot_sync(half_mask, umax == wmax) & half_mask;
  mx = __shfl_sync(half_mask, mx, __ffs(holders) - 1);
  int q[16];
  d = 0.f;
  if (wmax == 0u) {
#pragma unroll
    for (int e = 0; e < 16; e++) q[e] = 0;
  } else {
    const float iscale = q8k_iscale(mx, __uint_as_float(wmax));
#pragma unroll
    for (int e = 0; e < 16; e++) q[e] = q8k_round(__fmul_rn(iscale, v[e]));
    d = __fdiv_rn(1.f, iscale);
  }
  s16 = 0;
#pragma unroll
  for (int e = 0; e < 16; e++) s16 += q[e];
  s32 = s16 + __shfl_xor_sync(half_mask, s16, 1);
#pragma unroll
  for (int i = 0; i < 4; i++) w[i] = pack4(q + 4 * i);
}

// Q8_0 block of 32 values held 8 per lane by 4 consecutive lanes: d = amax/127 in f32,
// stored as f16; q = round-half-away(x * (1/d)).
__device__ __forceinline__ void quant_block_q8_0(const float (&v)[8], uint32_t& w0, uint32_t& w1, __half& dh) {
  float amax = 0.f;
#pragma unroll
  for (int e = 0; e < 8; e++) amax = fmaxf(amax, fabsf(v[e]));
  amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 2));
  float d = __fdiv_rn(amax, 127.f);
  float id = d == 0.f ? 0.f : __fdiv_rn(1.f, d);
  int q[8];
#pragma unroll
  for (int e = 0; e < 8; e++) q[e] = (int)roundf(__fmul_rn(v[e], id));
  dh = __float2half_rn(d);
  w0 = pack4(q);
  w1 = pack4(q + 4);
}

}  // namespace turq
