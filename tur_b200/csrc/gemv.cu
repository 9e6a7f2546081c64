// EXACT_F32 scheme of the decode-sized QMatMul::forward: y[m, n] = sum_k x[m, k] W[n, k] with
// the device tiles decoded to their exact f32 values and multiplied with f32 activations
// (CUDA-core FMAs). Persistent CTAs over row-tiles, the warps of a CTA split the K-tiles and
// their partial sums are added in warp order, so results do not depend on the grid size.
#include <cstdio>
#include <cstdlib>

#include "decode.cuh"
#include "gemv_tile.cuh"
#include "turq_internal.h"

namespace turq {

constexpr int MAX_WARPS = 16;

static int pick_warps(int64_t row_tiles, int64_t ktiles, int sm_count) {
  int w = row_tiles >= (int64_t)sm_count * 4 ? 4 : row_tiles >= (int64_t)sm_count * 2 ? 8 : 16;
  while (w > 1 && w > ktiles) w >>= 1;
  return w;
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
