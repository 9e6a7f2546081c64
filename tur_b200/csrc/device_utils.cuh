// Small device-side helpers: streaming loads, f16 unpacking, integer MMA wrappers.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace turq {

// 128-bit streaming load for weights: read-only path, no L1 allocation (each weight byte is
// used exactly once per launch, activations keep L1).
// (The host branches exist so the tile decoders can be exercised by a CPU test build.)
__host__ __device__ __forceinline__ uint4 ld_stream_v4(const void* p) {
#ifdef __CUDA_ARCH__
  uint4 v;
  asm("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
      : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
      : "l"(p));
  return v;
#else
  return *reinterpret_cast<const uint4*>(p);
#endif
}

__host__ __device__ __forceinline__ uint4 ld_v4(const void* p) { return *reinterpret_cast<const uint4*>(p); }
__host__ __device__ __forceinline__ uint2 ld_v2(const void* p) { return *reinterpret_cast<const uint2*>(p); }
__host__ __device__ __forceinline__ uint32_t ld_u32(const void* p) { return *reinterpret_cast<const uint32_t*>(p); }
__host__ __device__ __forceinline__ uint16_t ld_u16(const void* p) { return *reinterpret_cast<const uint16_t*>(p); }

__host__ __device__ __forceinline__ float f16_bits_to_f32(uint32_t bits16) {
  __half_raw r;
  r.x = (unsigned short)(bits16 & 0xFFFFu);
  return __half2float(__half(r));
}

// Separately rounded f32 multiply / subtract (never contracted into an FMA).
__host__ __device__ __forceinline__ float mul_rn(float a, float b) {
#ifdef __CUDA_ARCH__
  return __fmul_rn(a, b);
#else
  volatile float r = a * b;
  return r;
#endif
}
__host__ __device__ __forceinline__ float sub_rn(float a, float b) {
#ifdef __CUDA_ARCH__
  return __fsub_rn(a, b);
#else
  volatile float r = a - b;
  return r;
#endif
}

__device__ __forceinline__ float load_act_f32(const void* x, int x_is_bf16, int64_t idx) {
  if (x_is_bf16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(x)[idx]);
  return reinterpret_cast<const float*>(x)[idx];
}

// D = A(16x32, s8 or u8) * B(32x8, s8) + C, row.col, s32 accumulate.
template <bool A_UNSIGNED>
__device__ __forceinline__ void mma_16832(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if (A_UNSIGNED) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  } else {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
}

// D = A(16x16, u8) * B(16x8, s8) + C
__device__ __forceinline__ void mma_16816_u8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
      : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
      : "r"(a0), "r"(a1), "r"(b0));
}

}  // namespace turq
