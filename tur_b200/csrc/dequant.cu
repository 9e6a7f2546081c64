// QTensor::dequantize on the device layout: one warp per tile (16 rows x one wire block),
// output row-major [n_rows, k] in f32 (bit-exact), f16 or bf16 (rounded from the exact f32).
// HBM-bound on the writes: 4 B out per 0.56-1.06 B in.
#include "decode.cuh"
#include "turq_internal.h"

namespace turq {

template <class T> __device__ __forceinline__ T cvt_out(float v);
template <> __device__ __forceinline__ float cvt_out<float>(float v) { return v; }
template <> __device__ __forceinline__ __half cvt_out<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 cvt_out<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

template <int NV, class T>
__device__ __forceinline__ void store_run(T* dst, const float (&v)[NV]) {
  if constexpr (sizeof(T) == 4) {
#pragma unroll
    for (int e = 0; e < NV; e += 4)
      *reinterpret_cast<float4*>(dst + e) = make_float4(v[e], v[e + 1], v[e + 2], v[e + 3]);
  } else {
    T tmp[NV];
#pragma unroll
    for (int e = 0; e < NV; e++) tmp[e] = cvt_out<T>(v[e]);
    if constexpr (NV == 8) {
      *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(tmp);
    } else {
      *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(tmp);
    }
  }
}

template <int DT, class T>
__global__ void __launch_bounds__(256) dequant_kernel(const uint8_t* __restrict__ tiles, T* __restrict__ out,
                                                      int64_t n_rows, int64_t k, int64_t ktiles,
                                                      int64_t total_tiles) {
  constexpr int TB = 16 * (DT == TQ_Q8_0 ? 34 : DT == TQ_Q4_K ? 144 : DT == TQ_Q5_K ? 176 : 210);
  constexpr int KE = DT == TQ_Q8_0 ? 32 : 256;
  const int lane = threadIdx.x & 31;
  const int g = lane >> 2;
  int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t tile = warp; tile < total_tiles; tile += nwarps) {
    int64_t rt = tile / ktiles, kt = tile - rt * ktiles;
    const uint8_t* t = tiles + tile * TB;
    decode_tile<DT>(t, lane, [&](int hr, int off, const auto& v) {
      int64_t row = rt * TQ_TILE_ROWS + g + 8 * hr;
      if (row < n_rows) store_run(out + row * k + kt * KE + off, v);
    });
  }
}

template <int DT>
static cudaError_t launch_dt(const uint8_t* tiles, void* out, int out_dtype, int64_t n_rows, int64_t k,
                             cudaStream_t s) {
  int64_t ktiles = k / tq_block_elems(DT);
  int64_t row_tiles = (n_rows + TQ_TILE_ROWS - 1) / TQ_TILE_ROWS;
  int64_t total = row_tiles * ktiles;
  if (total == 0) return cudaSuccess;
  int threads = 256;
  int64_t blocks = (total + 7) / 8;
  if (blocks > (int64_t)device_sm_count() * 16) blocks = (int64_t)device_sm_count() * 16;
  switch (out_dtype) {
    case TQ_F32:
      dequant_kernel<DT, float><<<(unsigned)blocks, threads, 0, s>>>(tiles, (float*)out, n_rows, k, ktiles, total);
      break;
    case TQ_F16:
      dequant_kernel<DT, __half><<<(unsigned)blocks, threads, 0, s>>>(tiles, (__half*)out, n_rows, k, ktiles, total);
      break;
    case TQ_BF16:
      dequant_kernel<DT, __nv_bfloat16><<<(unsigned)blocks, threads, 0, s>>>(tiles, (__nv_bfloat16*)out, n_rows, k, ktiles, total);
      break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

// Embedding lookup on the quantized table: out[i, :] = dequantize(row ids[i]). Four lanes per
// (id, K-tile): in the fragment layout lane 4g + c of a full-tile decode holds rows g and g + 8,
// so the four lanes of column group c = 0..3 with g = row % 8 hold the whole row. Each quad runs
// the full dequantize's per-lane code for that lane position only (the values are the same bits)
// and reads an eighth of the tile instead of all of it. A warp serves eight (id, K-tile) pairs.
// An id outside [0, n_rows) gives a row of zeros and raises the status word.
template <int DT, class T>
__global__ void __launch_bounds__(256) gather_rows_kernel(const uint8_t* __restrict__ tiles, const int32_t* __restrict__ ids,
                                                          T* __restrict__ out, int64_t n_rows, int64_t n_ids, int64_t k,
                                                          int64_t ktiles, int* __restrict__ status) {
  constexpr int TB = 16 * (DT == TQ_Q8_0 ? 34 : DT == TQ_Q4_K ? 144 : DT == TQ_Q5_K ? 176 : 210);
  constexpr int KE = DT == TQ_Q8_0 ? 32 : 256;
  const int lane = threadIdx.x & 31;
  const int c = lane & 3;
  const int64_t quad = (((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5) * 8 + (lane >> 2);
  const int64_t nquads = (((int64_t)gridDim.x * blockDim.x) >> 5) * 8;
  const int64_t total = n_ids * ktiles;
  for (int64_t u = quad; u < total; u += nquads) {
    const int64_t i = u / ktiles, kt = u - i * ktiles;
    const int64_t row = ids[i];
    T* dst = out + i * k + kt * KE;
    if (row < 0 || row >= n_rows) {
      for (int e = c; e < KE; e += 4) dst[e] = cvt_out<T>(0.f);
      if (c == 0 && kt == 0) {
        *reinterpret_cast<volatile int*>(status) = 1;  // TURQ_E_INVALID_ARG; the word may be mapped host memory
        __threadfence_system();
      }
      continue;
    }
    const int r16 = (int)(row & 15);
    const uint8_t* t = tiles + ((row >> 4) * ktiles + kt) * TB;
    const int want_hr = r16 >> 3;
    decode_tile<DT>(t, 4 * (r16 & 7) + c, [&](int hr, int off, const auto& v) {
      if (hr == want_hr) store_run(dst + off, v);
    });
  }
}

template <int DT>
static cudaError_t launch_gather_dt(const uint8_t* tiles, const int32_t* ids, void* out, int out_dtype, int64_t n_rows,
                                    int64_t n_ids, int64_t k, int* status, cudaStream_t s) {
  const int64_t ktiles = k / tq_block_elems(DT);
  const int64_t total = n_ids * ktiles;
  if (total == 0) return cudaSuccess;
  int64_t blocks = (total + 63) / 64;  // eight (id, K-tile) pairs per warp, eight warps per block
  if (blocks > (int64_t)device_sm_count() * 16) blocks = (int64_t)device_sm_count() * 16;
  switch (out_dtype) {
    case TQ_F32:
      gather_rows_kernel<DT, float><<<(unsigned)blocks, 256, 0, s>>>(tiles, ids, (float*)out, n_rows, n_ids, k, ktiles, status);
      break;
    case TQ_F16:
      gather_rows_kernel<DT, __half><<<(unsigned)blocks, 256, 0, s>>>(tiles, ids, (__half*)out, n_rows, n_ids, k, ktiles, status);
      break;
    case TQ_BF16:
      gather_rows_kernel<DT, __nv_bfloat16><<<(unsigned)blocks, 256, 0, s>>>(tiles, ids, (__nv_bfloat16*)out, n_rows, n_ids, k, ktiles, status);
      break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

cudaError_t launch_gather_rows(int dtype, const uint8_t* dev_tiles, const int32_t* dev_ids, void* dev_out, int out_dtype,
                               int64_t n_rows, int64_t n_ids, int64_t k, int* status, cudaStream_t s) {
  switch (dtype) {
    case TQ_Q8_0: return launch_gather_dt<TQ_Q8_0>(dev_tiles, dev_ids, dev_out, out_dtype, n_rows, n_ids, k, status, s);
    case TQ_Q4_K: return launch_gather_dt<TQ_Q4_K>(dev_tiles, dev_ids, dev_out, out_dtype, n_rows, n_ids, k, status, s);
    case TQ_Q5_K: return launch_gather_dt<TQ_Q5_K>(dev_tiles, dev_ids, dev_out, out_dtype, n_rows, n_ids, k, status, s);
    case TQ_Q6_K: return launch_gather_dt<TQ_Q6_K>(dev_tiles, dev_ids, dev_out, out_dtype, n_rows, n_ids, k, status, s);
    default: return cudaErrorInvalidValue;
  }
}

cudaError_t launch_dequant(int dtype, const uint8_t* dev_tiles, void* dev_out, int out_dtype, int64_t n_rows,
                           int64_t k, cudaStream_t s) {
  switch (dtype) {
    case TQ_Q8_0: return launch_dt<TQ_Q8_0>(dev_tiles, dev_out, out_dtype, n_rows, k, s);
    case TQ_Q4_K: return launch_dt<TQ_Q4_K>(dev_tiles, dev_out, out_dtype, n_rows, k, s);
    case TQ_Q5_K: return launch_dt<TQ_Q5_K>(dev_tiles, dev_out, out_dtype, n_rows, k, s);
    case TQ_Q6_K: return launch_dt<TQ_Q6_K>(dev_tiles, dev_out, out_dtype, n_rows, k, s);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace turq
