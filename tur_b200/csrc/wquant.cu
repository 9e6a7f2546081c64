// Weight quantizer: f32 rows -> GGUF wire blocks of Q4_K, Q5_K, Q6_K (Q8_0 goes through the
// activation quantizer, whose Q8_0 blocks are the same format). The counterpart of candle-core's
// QTensor::quantize, which tur itself never calls (src/weights/gguf_varbuilder.rs:73 only loads
// quantized files) but which makes the inputs of the benchmark configurations.
//
// The block search is a published-format quantizer of this library's own (any valid blocks serve:
// dequantize / matmul parity is defined on the bytes): per sub-block a min/max start followed by
// up to four rounds of "round, then refit scale and offset by least squares" (Q4_K / Q5_K), or a
// largest-magnitude-to-minus-32 start with one least-squares refit of the scale (Q6_K). It is an
// offline, load-time step, so the kernel is written for exactness, not speed: every float and
// double operation is a separately rounded IEEE operation in a fixed order (the *_rn intrinsics
// keep the compiler from fusing multiplies and adds), one thread runs a sub-block's search from
// its first element to its last, and the sums of the refit are double, as in the CPU
// restatement the tests compare the bytes with.
#include <cuda_fp16.h>

#include "layout.h"
#include "turq_internal.h"

namespace turq {

namespace {

__device__ __forceinline__ int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }
__device__ __forceinline__ uint16_t f32_to_f16_bits(float f) { return __half_as_ushort(__float2half_rn(f)); }
__device__ __forceinline__ float f16_bits_to_f32_dev(uint16_t h) { return __half2float(__ushort_as_half(h)); }

// x ~ scale * q + mn (mn <= 0), q in [0, nmax], for the n values of one sub-block.
__device__ void fit_scale_min(const float* x, int n, int nmax, float& scale_out, float& negmin_out) {
  float mn = x[0], mx = x[0];
  for (int i = 1; i < n; i++) {
    if (x[i] < mn) mn = x[i];
    if (x[i] > mx) mx = x[i];
  }
  if (mn > 0.f) mn = 0.f;
  if (mx <= mn) {
    scale_out = 0.f;
    negmin_out = -mn;
    return;
  }
  float scale = __fdiv_rn(__fsub_rn(mx, mn), (float)nmax);
  float best_err = __int_as_float(0x7F800000);  // +inf
  float best_s = scale, best_m = mn;
  for (int it = 0; it < 4; it++) {
    const float inv = __fdiv_rn(1.f, scale);
    double sq = 0, sqq = 0, sx = 0, sxq = 0, err = 0;
    for (int i = 0; i < n; i++) {
      int q = __float2int_rn(__fmul_rn(__fsub_rn(x[i], mn), inv));
      q = clampi(q, 0, nmax);
      const float r = __fsub_rn(__fadd_rn(__fmul_rn(scale, (float)q), mn), x[i]);
      err = __dadd_rn(err, __dmul_rn((double)r, (double)r));
      sq = __dadd_rn(sq, (double)q);
      sqq = __dadd_rn(sqq, __dmul_rn((double)q, (double)q));
      sx = __dadd_rn(sx, (double)x[i]);
      sxq = __dadd_rn(sxq, __dmul_rn((double)x[i], (double)q));
    }
    if (err < (double)best_err) {
      best_err = __double2float_rn(err);
      best_s = scale;
      best_m = mn;
    } else {
      break;
    }
    const double det = __dsub_rn(__dmul_rn((double)n, sqq), __dmul_rn(sq, sq));
    if (det <= 0) break;
    double s2 = __ddiv_rn(__dsub_rn(__dmul_rn((double)n, sxq), __dmul_rn(sq, sx)), det);
    double m2 = __ddiv_rn(__dsub_rn(sx, __dmul_rn(s2, sq)), (double)n);
    if (s2 <= 0) break;
    if (m2 > 0) {  // re-solve with the offset pinned at zero
      m2 = 0;
      s2 = sqq > 0 ? __ddiv_rn(sxq, sqq) : s2;
      if (s2 <= 0) break;
    }
    scale = __double2float_rn(s2);
    mn = __double2float_rn(m2);
  }
  scale_out = best_s;
  negmin_out = -best_m;
}

// Q4_K / Q5_K: eight threads per 256-block, thread j owns sub-block j. 128 threads = 16 blocks.
template <int BITS>
__global__ void __launch_bounds__(128) quant_q45k_kernel(const float* __restrict__ x, int64_t nblocks, uint8_t* __restrict__ out) {
  constexpr int NMAX = (1 << BITS) - 1;
  constexpr int BSZ = BITS == 4 ? 144 : 176;
  __shared__ uint8_t L[16][256];
  __shared__ int s_ls[16][8], s_lm[16][8];
  const int j = threadIdx.x & 7, lb = threadIdx.x >> 3;
  const unsigned gmask = 0xFFu << (8 * ((threadIdx.x & 31) >> 3));  // the eight lanes of this block
  for (int64_t b0 = (int64_t)blockIdx.x * 16; b0 < nblocks; b0 += (int64_t)gridDim.x * 16) {
    const int64_t blk = b0 + lb;
    const bool live = blk < nblocks;
    if (live) {
      const float* xs = x + blk * 256 + 32 * j;
      float v[32];
#pragma unroll
      for (int i = 0; i < 32; i += 4) {
        const float4 t = *reinterpret_cast<const float4*>(xs + i);
        v[i] = t.x; v[i + 1] = t.y; v[i + 2] = t.z; v[i + 3] = t.w;
      }
      float sc, mnv;
      fit_scale_min(v, 32, NMAX, sc, mnv);
      float max_scale = sc, max_min = mnv;
#pragma unroll
      for (int o = 4; o > 0; o >>= 1) {
        max_scale = fmaxf(max_scale, __shfl_xor_sync(gmask, max_scale, o));
        max_min = fmaxf(max_min, __shfl_xor_sync(gmask, max_min, o));
      }
      if (!(max_scale > 0.f)) max_scale = 0.f;  // also turns a -0 into the +0 a maximum over "0, ..." gives
      if (!(max_min > 0.f)) max_min = 0.f;
      const float inv_scale = max_scale > 0.f ? __fdiv_rn(63.f, max_scale) : 0.f;
      const float inv_min = max_min > 0.f ? __fdiv_rn(63.f, max_min) : 0.f;
      const int ls = clampi(__float2int_rn(__fmul_rn(inv_scale, sc)), 0, 63);
      const int lm = clampi(__float2int_rn(__fmul_rn(inv_min, mnv)), 0, 63);
      const uint16_t dh = f32_to_f16_bits(__fdiv_rn(max_scale, 63.f)), dmh = f32_to_f16_bits(__fdiv_rn(max_min, 63.f));
      const float d = f16_bits_to_f32_dev(dh), dmin = f16_bits_to_f32_dev(dmh);
      const float dl = __fmul_rn(d, (float)ls), ml = __fmul_rn(dmin, (float)lm);
#pragma unroll
      for (int i = 0; i < 32; i++) {
        int q = 0;
        if (dl != 0.f) q = clampi(__float2int_rn(__fdiv_rn(__fadd_rn(v[i], ml), dl)), 0, NMAX);
        L[lb][32 * j + i] = (uint8_t)q;
      }
      s_ls[lb][j] = ls;
      s_lm[lb][j] = lm;
      uint8_t* ob = out + blk * BSZ;
      if (j == 0) {
        ob[0] = (uint8_t)(dh & 0xFF); ob[1] = (uint8_t)(dh >> 8);
        ob[2] = (uint8_t)(dmh & 0xFF); ob[3] = (uint8_t)(dmh >> 8);
      }
    }
    __syncwarp();
    if (live) {
      uint8_t* ob = out + blk * BSZ;
      if (j == 0) {
        // twelve bytes holding eight 6-bit scales and eight 6-bit mins
        const int* sc = s_ls[lb];
        const int* m = s_lm[lb];
        uint8_t* s = ob + 4;
        for (int t = 0; t < 4; t++) {
          s[t] = (uint8_t)((sc[t] & 63) | ((sc[t + 4] >> 4) << 6));
          s[t + 4] = (uint8_t)((m[t] & 63) | ((m[t + 4] >> 4) << 6));
          s[t + 8] = (uint8_t)((sc[t + 4] & 0x0F) | ((m[t + 4] & 0x0F) << 4));
        }
      }
      // qs: byte 32 g + i holds element i of sub-block 2g (low nibble) and of 2g + 1 (high);
      // thread j writes bytes 16 j .. 16 j + 15
      uint8_t* qs = ob + (BITS == 4 ? 16 : 48);
      const int g = j >> 1, i0 = 16 * (j & 1);
      for (int i = i0; i < i0 + 16; i++) {
        const int lo = L[lb][64 * g + i], hi = L[lb][64 * g + 32 + i];
        qs[32 * g + i] = (uint8_t)((lo & 0x0F) | ((hi & 0x0F) << 4));
      }
      if (BITS == 5) {
        // qh: bit 2g of byte i = fifth bit of element i of sub-block 2g, bit 2g + 1 of sub-block 2g + 1
        uint8_t* qh = ob + 16;
        for (int i = 4 * j; i < 4 * j + 4; i++) {
          int bits = 0;
          for (int gg = 0; gg < 4; gg++) {
            const int lo = L[lb][64 * gg + i], hi = L[lb][64 * gg + 32 + i];
            bits |= ((lo >> 4) << (2 * gg)) | ((hi >> 4) << (2 * gg + 1));
          }
          qh[i] = (uint8_t)bits;
        }
      }
    }
    __syncwarp();
  }
}

// Q6_K: sixteen threads per 256-block, thread j owns the 16 elements of sub-block j. 128 threads = 8 blocks.
__global__ void __launch_bounds__(128) quant_q6k_kernel(const float* __restrict__ x, int64_t nblocks, uint8_t* __restrict__ out) {
  __shared__ uint8_t L[8][256];
  const int j = threadIdx.x & 15, lb = threadIdx.x >> 4;
  const unsigned gmask = 0xFFFFu << (16 * ((threadIdx.x & 31) >> 4));
  for (int64_t b0 = (int64_t)blockIdx.x * 8; b0 < nblocks; b0 += (int64_t)gridDim.x * 8) {
    const int64_t blk = b0 + lb;
    const bool live = blk < nblocks;
    bool zero_block = false;
    if (live) {
      const float* xs = x + blk * 256 + 16 * j;
      float v[16];
#pragma unroll
      for (int i = 0; i < 16; i += 4) {
        const float4 t = *reinterpret_cast<const float4*>(xs + i);
        v[i] = t.x; v[i + 1] = t.y; v[i + 2] = t.z; v[i + 3] = t.w;
      }
      float amax = 0.f, mx = 0.f;
      for (int i = 0; i < 16; i++) {
        const float a = fabsf(v[i]);
        if (a > amax) {
          amax = a;
          mx = v[i];
        }
      }
      float s = amax == 0.f ? 0.f : __fdiv_rn(mx, -32.f);  // largest magnitude lands on -32
      if (s != 0.f) {  // one least-squares refit of the scale on the rounded integers
        double sxq = 0, sqq = 0;
        for (int i = 0; i < 16; i++) {
          const int q = clampi(__float2int_rn(__fdiv_rn(v[i], s)), -32, 31);
          sxq = __dadd_rn(sxq, __dmul_rn((double)v[i], (double)q));
          sqq = __dadd_rn(sqq, __dmul_rn((double)q, (double)q));
        }
        if (sqq > 0 && sxq != 0) s = __double2float_rn(__ddiv_rn(sxq, sqq));
      }
      float max_abs = fabsf(s);
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) max_abs = fmaxf(max_abs, __shfl_xor_sync(gmask, max_abs, o));
      uint8_t* ob = out + blk * 210;
      zero_block = max_abs == 0.f;
      if (zero_block) {
        // q = 0 is stored as 32: low nibble 0, high two bits = 2
        for (int i = 8 * j; i < 8 * j + 8; i++) ob[i] = 0;
        for (int i = 4 * j; i < 4 * j + 4; i++) ob[128 + i] = 0xAA;
        ob[192 + j] = 0;
        if (j == 0) ob[208] = ob[209] = 0;
      } else {
        const uint16_t dh = f32_to_f16_bits(__fdiv_rn(max_abs, 127.f));
        const float d = f16_bits_to_f32_dev(dh);
        const int si = d != 0.f ? clampi(__float2int_rn(__fdiv_rn(s, d)), -128, 127) : 0;
        const float dl = __fmul_rn(d, (float)si);
        for (int i = 0; i < 16; i++) {
          int q = 0;
          if (dl != 0.f) q = clampi(__float2int_rn(__fdiv_rn(v[i], dl)), -32, 31);
          L[lb][16 * j + i] = (uint8_t)(q + 32);
        }
        ob[192 + j] = (uint8_t)(int8_t)si;
        if (j == 0) {
          ob[208] = (uint8_t)(dh & 0xFF);
          ob[209] = (uint8_t)(dh >> 8);
        }
      }
    }
    __syncwarp();
    if (live && !zero_block) {
      uint8_t* ob = out + blk * 210;
      // ql: two halves of 64 bytes, each the low nibbles of elements 0..63 of its 128 and, in the
      // high nibbles, elements 64..127; thread j writes bytes 8 j .. 8 j + 7
      for (int bi = 8 * j; bi < 8 * j + 8; bi++) {
        const int h = bi >> 6, r = bi & 63;  // r < 32: elements l and 64 + l; else 32 + l and 96 + l
        const int l = r & 31, base = 128 * h + (r < 32 ? 0 : 32);
        const int qa = L[lb][base + l], qb = L[lb][base + 64 + l];
        ob[bi] = (uint8_t)((qa & 0x0F) | ((qb & 0x0F) << 4));
      }
      // qh: two halves of 32 bytes, four 2-bit fields per byte; thread j writes bytes 4 j .. 4 j + 3
      for (int bi = 4 * j; bi < 4 * j + 4; bi++) {
        const int h = bi >> 5, l = bi & 31;
        const int q1 = L[lb][128 * h + l], q2 = L[lb][128 * h + 32 + l], q3 = L[lb][128 * h + 64 + l], q4 = L[lb][128 * h + 96 + l];
        ob[128 + bi] = (uint8_t)((q1 >> 4) | ((q2 >> 4) << 2) | ((q3 >> 4) << 4) | ((q4 >> 4) << 6));
      }
    }
    __syncwarp();
  }
}

}  // namespace

cudaError_t launch_quantize_weights(int dtype, const float* x, int64_t n_rows, int64_t k, uint8_t* wire, cudaStream_t s) {
  if (dtype == TQ_Q8_0) return launch_quantize_act_wire(TQ_Q8_0, x, TQ_F32, n_rows, k, wire, s);
  const int64_t nblocks = n_rows * (k / 256);
  if (nblocks <= 0) return cudaErrorInvalidValue;
  const int per_cta = dtype == TQ_Q6_K ? 8 : 16;
  int64_t grid = (nblocks + per_cta - 1) / per_cta;
  if (grid > 65535 * 16) grid = 65535 * 16;
  if (dtype == TQ_Q4_K) quant_q45k_kernel<4><<<(unsigned)grid, 128, 0, s>>>(x, nblocks, wire);
  else if (dtype == TQ_Q5_K) quant_q45k_kernel<5><<<(unsigned)grid, 128, 0, s>>>(x, nblocks, wire);
  else if (dtype == TQ_Q6_K) quant_q6k_kernel<<<(unsigned)grid, 128, 0, s>>>(x, nblocks, wire);
  else return cudaErrorInvalidValue;
  return cudaGetLastError();
}

}  // namespace turq
