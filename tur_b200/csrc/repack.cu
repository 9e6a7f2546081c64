// GGUF wire blocks -> device fragment tiles (upload-time path), and column slicing of a
// tiled tensor for row-parallel tensor-parallel shards.
#include "turq_internal.h"

namespace turq {

__global__ void repack_kernel(int dtype, const uint8_t* __restrict__ wire, uint32_t* __restrict__ tiles,
                              int64_t n_rows, int64_t ktiles, int64_t total_words) {
  const int words_per_tile = tq_tile_bytes(dtype) / 4;
  const int block_bytes = tq_block_bytes(dtype);
  const int64_t row_bytes = ktiles * block_bytes;
  for (int64_t w = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; w < total_words;
       w += (int64_t)gridDim.x * blockDim.x) {
    int64_t tile = w / words_per_tile;
    int wi = (int)(w - tile * words_per_tile);
    int64_t rt = tile / ktiles, kt = tile - rt * ktiles;
    auto blk = [&](int r) -> const uint8_t* {
      int64_t row = rt * TQ_TILE_ROWS + r;
      return row < n_rows ? wire + row * row_bytes + kt * block_bytes : nullptr;
    };
    tiles[w] = tq_tile_word(dtype, wi, blk);
  }
}

cudaError_t launch_repack(int dtype, const uint8_t* dev_wire, uint8_t* dev_tiles, int64_t n_rows,
                          int64_t k, cudaStream_t s) {
  int64_t ktiles = k / tq_block_elems(dtype);
  int64_t row_tiles = (n_rows + TQ_TILE_ROWS - 1) / TQ_TILE_ROWS;
  int64_t total_words = row_tiles * ktiles * (tq_tile_bytes(dtype) / 4);
  if (total_words == 0) return cudaSuccess;
  int threads = 256;
  int64_t blocks = (total_words + threads - 1) / threads;
  if (blocks > (int64_t)device_sm_count() * 64) blocks = (int64_t)device_sm_count() * 64;
  repack_kernel<<<(unsigned)blocks, threads, 0, s>>>(dtype, dev_wire, reinterpret_cast<uint32_t*>(dev_tiles),
                                                      n_rows, ktiles, total_words);
  return cudaGetLastError();
}

__global__ void slice_cols_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, int64_t row_tiles,
                                  int64_t src_ktiles, int64_t kt0, int64_t nkt, int vec_per_tile) {
  int64_t total = row_tiles * nkt * vec_per_tile;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    int64_t tile = i / vec_per_tile;
    int v = (int)(i - tile * vec_per_tile);
    int64_t rt = tile / nkt, kt = tile - rt * nkt;
    dst[i] = src[((rt * src_ktiles) + kt0 + kt) * vec_per_tile + v];
  }
}

cudaError_t launch_slice_cols(int dtype, const uint8_t* src_tiles, uint8_t* dst_tiles, int64_t row_tiles,
                              int64_t src_ktiles, int64_t kt0, int64_t nkt, cudaStream_t s) {
  int vec_per_tile = tq_tile_bytes(dtype) / 16;
  int64_t total = row_tiles * nkt * vec_per_tile;
  if (total == 0) return cudaSuccess;
  int threads = 256;
  int64_t blocks = (total + threads - 1) / threads;
  if (blocks > (int64_t)device_sm_count() * 32) blocks = (int64_t)device_sm_count() * 32;
  slice_cols_kernel<<<(unsigned)blocks, threads, 0, s>>>(reinterpret_cast<const uint4*>(src_tiles),
                                                          reinterpret_cast<uint4*>(dst_tiles), row_tiles,
                                                          src_ktiles, kt0, nkt, vec_per_tile);
  return cudaGetLastError();
}

}  // namespace turq
