// C-ABI layer: argument validation, handle lifetimes, scratch memory, dispatch to kernels.
// No entry throws, aborts or falls back to a CPU path; failures come back as turq_status
// with a message stored on the context.
#include <atomic>
#include <chrono>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <new>
#include <string>

#include "../../include/turq.h"
#include "handles.h"
#include "turq_internal.h"

namespace turq {

namespace {
struct DeviceFacts {
  std::atomic<int> sms{0}, smem_optin{0};
};
DeviceFacts g_facts[64];

int fact(int which) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
  std::atomic<int>& slot = which == 0 ? g_facts[dev].sms : g_facts[dev].smem_optin;
  int v = slot.load(std::memory_order_acquire);
  if (v > 0) return v;
  if (cudaDeviceGetAttribute(&v, which == 0 ? cudaDevAttrMultiProcessorCount : cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) !=
          cudaSuccess || v <= 0) {
    cudaGetLastError();
    v = which == 0 ? 1 : 48 * 1024;
  }
  slot.store(v, std::memory_order_release);
  return v;
}
}  // namespace

int device_sm_count() { return fact(0); }
int device_smem_optin() { return fact(1); }

}  // namespace turq

namespace {

int32_t fail(turq_ctx* ctx, int32_t st, const char* fmt, ...) {
  if (ctx) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    try {
      ctx->err = buf;
    } catch (...) {
    }
  }
  return st;
}

int32_t cuda_fail(turq_ctx* ctx, cudaError_t e, const char* what) {
  return fail(ctx, TURQ_E_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

#define TQ_CUDA(ctx, call)                                   \
  do {                                                       \
    cudaError_t e__ = (call);                                \
    if (e__ != cudaSuccess) return cuda_fail(ctx, e__, #call); \
  } while (0)

// Grows a context-owned buffer. Growing synchronizes the device and reallocates, which is why
// turq_ctx_reserve exists: a caller that reserves for its largest call never gets here again.
int32_t ensure(turq_ctx* ctx, uint8_t** buf, size_t* have, size_t need) {
  if (need <= *have) return TURQ_OK;
  size_t want = need + need / 4;
  want = (want + 0xFFFFF) & ~(size_t)0xFFFFF;
  if (*buf) {
    TQ_CUDA(ctx, cudaDeviceSynchronize());
    TQ_CUDA(ctx, cudaFree(*buf));
    *buf = nullptr;
    *have = 0;
  }
  TQ_CUDA(ctx, cudaMalloc(reinterpret_cast<void**>(buf), want));
  *have = want;
  return TURQ_OK;
}

size_t tiled_bytes(int dtype, int64_t n_rows, int64_t k) {
  int64_t row_tiles = (n_rows + TQ_TILE_ROWS - 1) / TQ_TILE_ROWS;
  return (size_t)row_tiles * (size_t)(k / tq_block_elems(dtype)) * (size_t)tq_tile_bytes(dtype);
}

int32_t check_weight_args(turq_ctx* ctx, int32_t dtype, int64_t n_rows, int64_t n_cols, size_t nbytes) {
  if (!tq_is_weight_type(dtype))
    return fail(ctx, TURQ_E_DTYPE, "dtype %d is not a supported quantized weight type (Q8_0, Q4_K, Q5_K, Q6_K)", dtype);
  if (n_rows <= 0 || n_cols <= 0) return fail(ctx, TURQ_E_SHAPE, "shape [%lld, %lld] must be positive", (long long)n_rows, (long long)n_cols);
  if (n_cols % tq_block_elems(dtype) != 0)
    return fail(ctx, TURQ_E_SHAPE, "n_cols %lld is not a multiple of the block size %d", (long long)n_cols, tq_block_elems(dtype));
  size_t expect = (size_t)n_rows * (size_t)(n_cols / tq_block_elems(dtype)) * (size_t)tq_block_bytes(dtype);
  if (nbytes != expect)
    return fail(ctx, TURQ_E_SHAPE, "got %zu bytes, shape [%lld, %lld] of this type needs %zu", nbytes, (long long)n_rows, (long long)n_cols, expect);
  return TURQ_OK;
}

int32_t new_qtensor(turq_ctx* ctx, int dtype, int64_t n_rows, int64_t n_cols, turq_qtensor** out) {
  turq_qtensor* qt = new (std::nothrow) turq_qtensor();
  if (!qt) return fail(ctx, TURQ_E_INVALID_ARG, "out of host memory");
  qt->device = ctx->device;
  qt->dtype = dtype;
  qt->n_rows = n_rows;
  qt->n_cols = n_cols;
  qt->wire_bytes = (size_t)n_rows * (size_t)(n_cols / tq_block_elems(dtype)) * (size_t)tq_block_bytes(dtype);
  qt->tile_bytes = tiled_bytes(dtype, n_rows, n_cols);
  cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&qt->tiles), qt->tile_bytes);
  if (e != cudaSuccess) {
    delete qt;
    return cuda_fail(ctx, e, "cudaMalloc(weight tiles)");
  }
  *out = qt;
  return TURQ_OK;
}

}  // namespace

extern "C" {

int32_t turq_version(void) { return TURQ_VERSION; }
int32_t turq_q8k_variant(void) { return turq::q8k_variant(); }

const char* turq_status_string(int32_t st) {
  switch (st) {
    case TURQ_OK: return "ok";
    case TURQ_E_INVALID_ARG: return "invalid argument";
    case TURQ_E_SHAPE: return "shape mismatch";
    case TURQ_E_DTYPE: return "unsupported dtype";
    case TURQ_E_ALIGN: return "misaligned pointer";
    case TURQ_E_CUDA: return "CUDA error";
    case TURQ_E_NCCL: return "NCCL error";
    case TURQ_E_TIMEOUT: return "timeout";
    case TURQ_E_NO_DEVICE: return "no CUDA device (no CPU fallback exists)";
    case TURQ_E_LIMIT: return "capacity of the entry point exceeded";
    default: return "unknown status";
  }
}

int32_t turq_block_elems(int32_t dtype) { return tq_block_elems(dtype); }
int32_t turq_block_bytes(int32_t dtype) { return tq_block_bytes(dtype); }
size_t turq_row_bytes(int32_t dtype, int64_t k) {
  int be = tq_block_elems(dtype);
  if (be == 0 || k < 0 || k % be != 0) return 0;
  return (size_t)(k / be) * (size_t)tq_block_bytes(dtype);
}

int32_t turq_ctx_create(int32_t device, turq_ctx** out) {
  if (!out) return TURQ_E_INVALID_ARG;
  *out = nullptr;
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess || count <= 0) {
    cudaGetLastError();
    return TURQ_E_NO_DEVICE;
  }
  if (device < 0 || device >= count) return TURQ_E_INVALID_ARG;
  turq_ctx* ctx = new (std::nothrow) turq_ctx();
  if (!ctx) return TURQ_E_INVALID_ARG;
  ctx->device = device;
  cudaDeviceProp prop;
  if (cudaSetDevice(device) != cudaSuccess || cudaGetDeviceProperties(&prop, device) != cudaSuccess ||
      cudaStreamCreateWithFlags(&ctx->own_stream, cudaStreamNonBlocking) != cudaSuccess ||
      cudaHostAlloc(reinterpret_cast<void**>(&ctx->host_status), 128, cudaHostAllocMapped) != cudaSuccess ||
      cudaHostGetDevicePointer(reinterpret_cast<void**>(&ctx->dev_status), ctx->host_status, 0) != cudaSuccess ||
      cudaMalloc(reinterpret_cast<void**>(&ctx->done_count), sizeof(unsigned)) != cudaSuccess ||
      cudaMemset(ctx->done_count, 0, sizeof(unsigned)) != cudaSuccess) {
    cudaGetLastError();
    if (ctx->host_status) cudaFreeHost(ctx->host_status);
    if (ctx->done_count) cudaFree(ctx->done_count);
    delete ctx;
    return TURQ_E_CUDA;
  }
  *ctx->host_status = 0;
  ctx->host_done = reinterpret_cast<volatile unsigned*>(ctx->host_status) + 16;  // a cache line of its own
  ctx->dev_done = reinterpret_cast<unsigned*>(ctx->dev_status) + 16;
  *ctx->host_done = 0;
  ctx->sm_count = prop.multiProcessorCount;
  const size_t ws_bytes = turq::gemv_workspace_bytes(ctx->sm_count);
  if (cudaMalloc(reinterpret_cast<void**>(&ctx->gemv_ws), ws_bytes) != cudaSuccess ||
      cudaMemset(ctx->gemv_ws, 0, ws_bytes) != cudaSuccess) {
    cudaGetLastError();
    turq_ctx_destroy(ctx);
    return TURQ_E_CUDA;
  }
  int32_t st = ensure(ctx, &ctx->scratch, &ctx->scratch_bytes, (size_t)8 << 20);
  if (st != TURQ_OK) {
    delete ctx;
    return st;
  }
  *out = ctx;
  return TURQ_OK;
}

int32_t turq_ctx_destroy(turq_ctx* ctx) {
  if (!ctx) return TURQ_E_INVALID_ARG;
  cudaSetDevice(ctx->device);
  cudaDeviceSynchronize();
  if (ctx->scratch) cudaFree(ctx->scratch);
  if (ctx->io) cudaFree(ctx->io);
  if (ctx->tmp) cudaFree(ctx->tmp);
  if (ctx->host_status) cudaFreeHost(ctx->host_status);
  if (ctx->done_count) cudaFree(ctx->done_count);
  if (ctx->gemv_ws) cudaFree(ctx->gemv_ws);
  if (ctx->own_stream) cudaStreamDestroy(ctx->own_stream);
  delete ctx;
  return TURQ_OK;
}

int32_t turq_ctx_reserve(turq_ctx* ctx, int64_t max_m, int64_t max_k, int64_t max_n) {
  if (!ctx) return TURQ_E_INVALID_ARG;
  if (max_m <= 0 || max_k <= 0 || max_n <= 0 || max_m > INT32_MAX / 2 || max_k > INT32_MAX || max_n > INT32_MAX)
    return fail(ctx, TURQ_E_SHAPE, "reserve(%lld, %lld, %lld): sizes must be positive and fit 31 bits", (long long)max_m,
                (long long)max_k, (long long)max_n);
  TQ_CUDA(ctx, cudaSetDevice(ctx->device));
  const int64_t k256 = (max_k + 255) / 256 * 256;
  size_t need = turq::plan_act_pack(TQ_Q8_K, max_m, k256).total;
  const size_t q80 = turq::plan_act_pack(TQ_Q8_0, max_m, k256).total;
  if (q80 > need) need = q80;
  // the tensor-core path's f16 operand and split-K partial sums (decode batches split the K loop)
  for (int64_t mm : {max_m < 64 ? max_m : (int64_t)64, max_m}) {
    const size_t tc = turq::gemm_tc_scratch_bytes(mm, k256, max_n, ctx->sm_count);
    if (tc > need) need = tc;
    // the widest split happens for weights of at most 128 rows
    const size_t tc_small = turq::gemm_tc_scratch_bytes(mm, k256, max_n < 128 ? max_n : 128, ctx->sm_count);
    if (tc_small > need) need = tc_small;
  }
  int32_t st = ensure(ctx, &ctx->scratch, &ctx->scratch_bytes, need);
  if (st != TURQ_OK) return st;
  auto up = [](size_t v) { return (v + 255) & ~(size_t)255; };
  return ensure(ctx, &ctx->io, &ctx->io_bytes,
                up((size_t)max_m * max_k * 4) + 4 * up((size_t)max_m * max_n * 4) + 4 * up((size_t)max_n * 4));
}

int32_t turq_ctx_set_auto_policy(turq_ctx* ctx, int32_t mode) {
  if (!ctx) return TURQ_E_INVALID_ARG;
  if (mode < TURQ_MODE_AUTO || mode > TURQ_MODE_TENSOR_CORE) return fail(ctx, TURQ_E_INVALID_ARG, "unknown mode %d", mode);
  ctx->auto_policy = mode;
  return TURQ_OK;
}

const char* turq_last_error(const turq_ctx* ctx) { return ctx ? ctx->err.c_str() : "null context"; }
int64_t turq_ctx_launch_count(const turq_ctx* ctx) { return ctx ? ctx->launches : 0; }

int32_t turq_ctx_poll_status(turq_ctx* ctx, void* stream) {
  if (!ctx) return TURQ_E_INVALID_ARG;
  TQ_CUDA(ctx, cudaSetDevice(ctx->device));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  TQ_CUDA(ctx, cudaStreamSynchronize(s));
  // The status word lives in mapped host memory: kernels store to it (rarely), the host reads it
  // here without a copy.
  const int st = *static_cast<volatile int*>(ctx->host_status);
  if (st != 0) {
    *static_cast<volatile int*>(ctx->host_status) = 0;
    // a kernel that gave up may have left hand-over flags or claim counters set
    cudaMemsetAsync(ctx->gemv_ws, 0, turq::gemv_workspace_bytes(ctx->sm_count), s);
    cudaStreamSynchronize(s);
    if (st == TURQ_E_INVALID_ARG) return fail(ctx, st, "an embedding lookup was given an id outside the table");
    return fail(ctx, st, "a kernel gave up a bounded device-side wait (status %d)", st);
  }
  return TURQ_OK;
}

int32_t turq_qtensor_from_device(turq_ctx* ctx, int32_t dtype, int64_t n_rows, int64_t n_cols,
                                 const void* dev_blocks, size_t nbytes, void* stream, turq_qtensor** out) {
  if (!ctx || !out || !dev_blocks) return fail(ctx, TURQ_E_INVALID_ARG, "null argument");
  *out = nullptr;
  int32_t st = check_weight_args(ctx, dtype, n_rows, n_cols, nbytes);
  if (st != TURQ_OK) return st;
  TQ_CUDA(ctx, cudaSetDevice(ctx->device));
  turq_qtensor* qt = nullptr;
  st = new_qtensor(ctx, dtype, n_rows, n_cols, &qt);
  if (st != TURQ_OK) return st;
  cudaError_t e = turq::launch_repack(dtype, static_cast<const uint8_t*>(dev_blocks), qt->tiles, n_rows, n_cols,
                                      static_cast<cudaStream_t>(stream));
  ctx->launches++;
  if (e != cudaSuccess) {
    turq_qtensor_free(qt);
    return cuda_fail(ctx, e, "repack launch");
  }
  *out = qt;
  return TURQ_OK;
}

int32_t turq_qtensor_from_host(turq_ctx* ctx, int32_t dtype, int64_t n_rows, int64_t n_cols,
                               const void* host_blocks, size_t nbytes, turq_qtensor** out) {
  if (!ctx || !out || !host_blocks) return fail(ctx, TURQ_E_INVALID_ARG, "null argument");
  *out = nullptr;
  int32_t st = check_weight_args(ctx, dtype, n_rows, n_cols, nbytes);
  if (st != TURQ_OK) return st;
  TQ_CUDA(ctx, cudaSetDevice(ctx->device));
  uint8_t* tmp = nullptr;
  TQ_CUDA(ctx, cudaMalloc(reinterpret_cast<void**>(&tmp), nbytes));
  cudaError_t e = cudaMemcpyAsync(tmp, host_blocks, nbytes, cudaMemcpyHostToDevice, ctx->own_stream);
  if (e == cudaSuccess) {
    st = turq_qtensor_from_device(ctx, dtype, n_rows, n_cols, tmp, nbytes, ctx->own_stream, out);
    if (st == TURQ_OK) e = cudaStreamSynchronize(ctx->own_stream);
  }
  cudaFree(tmp);
  if (st != TURQ_OK) return st;
  if (e != cudaSuccess) {
    if (*out) turq_qtensor_free(*out);
    *out = nullptr;
    return cuda_fail(ctx, e, "weight upload");
  }
  return TURQ_OK;
}

int32_t turq_qtensor_slice_rows(turq_ctx* ctx, const turq_qtensor* src, int64_t row0, int64_t n, turq_qtensor** out) {
  if (!ctx || !src || !out) return fail(ctx, TURQ_E_INVALID_ARG, "null argument");
  *out = nullptr;
  if (row0 < 0 || n <= 0 || row0 + n > src->n_rows) return fail(ctx, TURQ_E_SHAPE, "row range [%lld, +%lld) outside [0, %lld)", (long long)row0, (long long)n, (long long)src->n_rows);
  if (row0 % TQ_TILE_ROWS != 0) return fail(ctx, TURQ_E_SHAPE, "row0 %lld must be a multiple of %d", (long long)row0, TQ_TILE_ROWS);
  TQ_CUDA(ctx, cudaSetDevice(ctx->device));
  turq_qtensor* qt = nullptr;
  int32_t st = new_qtensor(ctx, src->dtype, n, src->n_cols, &qt);
  if (st != TURQ_OK) return st;
  size_t per_row_tile = (size_t)(src->n_cols / tq_block_elems(src->dtype)) * tq_tile_bytes(src->dtype);
  size_t off = (size_t)(row0 / TQ_TILE_ROWS) * per_row_tile;
  // A trailing partial row-tile of the slice carries rows of the source beyond row0+n; they
  // are never written to an output because every kernel bounds rows by n_rows.
  size_t avail = src->tile_bytes - off;
  size_t nbytes = qt->tile_bytes < avail ? qt->tile_bytes : avail;
  cudaError_t e = cudaMemcpyAsync(qt->tiles, src->tiles + off, nbytes, cudaMemcpyDeviceToDevice, ctx->own_stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->own_stream);
  if (e != cudaSuccess) {
    turq_qtensor_free(qt);
    return cuda_fail(ctx, e, "slice_rows copy");
  }
  *out = qt;
  return TURQ_OK;
}

int32_t turq_qtensor_slice_cols(turq_ctx* ctx, const turq_qtensor* src, int64_t col0, int64_t n, turq_qtensor** out) {
  if (!ctx || !src || !out) return fail(ctx, TURQ_E_INVALID_ARG, "null argument");
  *out = nullptr;
  const int be = tq_block_elems(src->dtype);
  if (col0 < 0 || n <= 0 || col0 + n > src->n_cols) return fail(ctx, TURQ_E_SHAPE, "column range [%lld, +%lld) outside [0, %lld)", (long long)col0, (long long)n, (long long)src->n_cols);
  if (col0 % be != 0 || n % be != 0) return fail(ctx, TURQ_E_SHAPE, "column range must be whole blocks of %d", be);
  TQ_CUDA(ctx, cudaSetDevice(ctx->device));
  turq_qtensor* qt = nullptr;
  int32_t st = new_qtensor(ctx, src->dtype, src->n_rows, n, &qt);
  if (st != TURQ_OK) return st;
  int64_t row_tiles = (src->n_rows + TQ_TILE_ROWS - 1) / TQ_TILE_ROWS;
  cudaError_t e = turq::launch_slice_cols(src->dtype, src->tiles, qt->tiles, row_tiles, src->n_cols / be, col0 / be,
                                          n / be, ctx->own_stream);
  ctx->launches++;
  if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->own_stream);
  if (e != cudaSuccess) {
    turq_qtensor_free(qt);
    return cuda_fail(ctx, e, "slice_cols");
  }
  *out = qt;
  return TURQ_OK;
}

int32_t turq_qtensor_free(turq_qtensor* qt) {
  if (!qt) return TURQ_E_INVALID_ARG;
  if (qt->tiles) {
    cudaSetDevice(qt->device);
    cudaFree(qt->tiles);
  }
  delete qt;
  return TURQ_OK;
}

int32_t turq_qtensor_info(const turq_qtensor* qt, int32_t* dtype, int64_t* n_rows, int64_t* n_cols, size_t* wire_bytes) {
  if (!qt) return TURQ_E_INVALID_ARG;
  if (dtype) *dtype = qt->dtype;
  if (n_rows) *n_rows = qt->n_rows;
  if (n_cols) *n_cols = qt->n_cols;
  if (wire_bytes) *wire_bytes = qt->wire_bytes;
  return TURQ_OK;
}

int32_t turq_dequantize(turq_ctx* ctx, const turq_qtensor* qt, int32_t out_dtype, void* dev_out, void* stream) {
  if (!ctx || !qt || !dev_out) return fail(ctx, TURQ_E_INVALID_ARG, "null argument");
  if (out_dtype != TURQ_F32 && out_dtype != TURQ_F16 && out_dtype != TURQ_BF16)
    return fail(ctx, TURQ_E_DTYPE, "dequantize output must be F32, F16 or BF16 (got %d)", out_dtype);
  if (qt->device != ctx->device) return fail(ctx, TURQ_E_INVALID_ARG, "tensor lives on device %d, context on %d", qt->device, ctx->device);
  if ((uintptr_t)dev_out % 16 != 0) return fail(ctx, TURQ_E_ALIGN, "dev_out must be 16-byte aligned");
  TQ_CUDA(ctx, cudaSetDevice(ctx->device));
  cudaError_t e = turq::launch_dequant(qt->dtype, qt->tiles, dev_out, out_dtype, qt->n_rows, qt->n_cols,
                                       static_cast<cudaStream_t>(stream));
  ctx->launches++;
  if (e != cudaSuccess) return cuda_fail(ctx, e, "dequantize launch");
  return TURQ_OK;
}

int32_t turq_embedding(turq_ctx* ctx, const turq_qtensor* qt, const int32_t* dev_ids, int64_t n_ids, int32_t out_dtype,
                       void* dev_out, void* stream) {
  if (!ctx || !qt) return fail(ctx, TURQ_E_INVALID_ARG, "null argument");
  if (n_ids < 0) return fail(ctx, TURQ_E_SHAPE, "n_ids=%lld is negative", (long long)n_ids);
  if (n_ids == 0) return TURQ_OK;
  if (!dev_out || !dev_ids) return fail(ctx, TURQ_E_INVALID_ARG, "null argument");
  if (out_dtype != TURQ_F32 && out_dtype != TURQ_F16 && out_dtype != TURQ_BF16)
    return fail(ctx, TURQ_E_DTYPE, "embedding output must be F32, F16 or BF16 (got %d)", out_dtype);
  if (qt->device != ctx->device) return fail(ctx, TURQ_E_INVALID_ARG, "tensor lives on device %d, context on %d", qt->device, ctx->device);
  if ((uintptr_t)dev_out % 16 != 0 || (uintptr_t)dev_ids % 4 != 0) return fail(ctx, TURQ_E_ALIGN, "dev_out must be 16-byte, dev_ids 4-byte aligned");
  TQ_CUDA(ctx, cudaSetDevice(ctx->device));
  cudaError_t e = turq::launch_gather_rows(qt->dtype, qt->tiles, dev_ids, dev_out, out_dtype, qt->n_rows, n_ids, qt->n_cols,
                                           ctx->dev_status, static_cast<cudaStream_t>(stream));
  ctx->launches++;
  if (e != cudaSuccess) return cuda_fail(ctx, e, "embedding launch");
  return TURQ_OK;
}

int32_t turq_quantize_act(turq_ctx* ctx, int32_t fmt, const void* dev_x, int32_t x_dtype, int64_t m, int64_t k,
                          void* dev_blocks, void* stream) {
  if (!ctx || !dev_x || !dev_blocks) return fail(ctx, TURQ_E_INVALID_ARG, "null argument");
  if (fmt != TURQ_Q8_0 && fmt != TURQ_Q8_K) return fail(ctx, TURQ_E_DTYPE, "activation format must be Q8_0 or Q8_K (got %d)", fmt);
  if (x_dtype != TURQ_F32 && x_dtype != TURQ_BF16) return fail(ctx, TURQ_E_DTYPE, "activations must be F32 or BF16 (got %d)", x_dtype);
  if (m <= 0 || k <= 0 || k % tq_block_elems(fmt) != 0)
    return fail(ctx, TURQ_E_SHAPE, "m=%lld k=%lld: k must be a positive multiple of %d", (long long)m, (long long)k, tq_block_elems(fmt));
  if ((uintptr_t)dev_x % 16 != 0 || (uintptr_t)dev_blocks % 4 != 0)
    return fail(ctx, TURQ_E_ALIGN, "dev_x must be 16-byte and dev_blocks 4-byte aligned");
  TQ_CUDA(ctx, cudaSetDevice(ctx->device));
  cudaError_t e = turq::launch_quantize_act_wire(fmt, dev_x, x_dtype, m, k, dev_blocks, static_cast<cudaStream_t>(stream));
  ctx->launches++;
  if (e != cudaSuccess) return cuda_fail(ctx, e, "quantize_act launch");
  return TURQ_OK;
}

int32_t turq_quantize_weights(turq_ctx* ctx, int32_t dtype, const float* dev_x, int64_t n_rows, int64_t n_cols,
                              void* dev_blocks, void* stream) {
  if (!ctx || !dev_x || !dev_blocks) return fail(ctx, TURQ_E_INVALID_ARG, "null argument");
  if (dtype != TURQ_Q8_0 && dtype != TURQ_Q4_K && dtype != TURQ_Q5_K && dtype != TURQ_Q6_K)
    return fail(ctx, TURQ_E_DTYPE, "weight type must be Q8_0, Q4_K, Q5_K or Q6_K (got %d)", dtype);
  if (n_rows <= 0 || n_cols <= 0 || n_cols % tq_block_elems(dtype) != 0)
    return fail(ctx, TURQ_E_SHAPE, "n_rows=%lld n_cols=%lld: n_cols must be a positive multiple of %d", (long long)n_rows,
                (long long)n_cols, tq_block_elems(dtype));
  if ((uintptr_t)dev_x % 16 != 0) return fail(ctx, TURQ_E_ALIGN, "dev_x must be 16-byte aligned");
  TQ_CUDA(ctx, cudaSetDevice(ctx->device));
  cudaError_t e = turq::launch_quantize_weights(dtype, dev_x, n_rows, n_cols, static_cast<uint8_t*>(dev_blocks),
                                                static_cast<cudaStream_t>(stream));
  ctx->launches++;
  if (e != cudaSuccess) return cuda_fail(ctx, e, "quantize_weights launch");
  return TURQ_OK;
}

// TURQ_MODE_AUTO: the integer GEMV up to 16 rows, the tcgen05 GEMM above (64-row activation
// tiles with split-K for decode batches, 128/256-row tiles for prefill). Measured on B200 at 32
// and 64 rows the GEMM is ahead for every weight shape of the benchmark configurations.
// A context whose policy was pinned with turq_ctx_set_auto_policy uses that one scheme for every
// row count, so a token's result does not depend on the batch or chunk it arrives in.
static int32_t auto_mode(const turq_ctx* ctx, int64_t n_rows, int64_t n_cols, int64_t m) {
  (void)n_rows;
  if (ctx->auto_policy != TURQ_MODE_AUTO) {
    if (ctx->auto_policy == TURQ_MODE_TENSOR_CORE && n_cols % 64 != 0) return TURQ_MODE_INT8_ACT;
    return ctx->auto_policy;
  }
  return (m <= 16 || n_cols % 64 != 0) ? TURQ_MODE_INT8_ACT : TURQ_MODE_TENSOR_CORE;
}

int32_t turq_qmatmul(turq_ctx* ctx, const turq_qtensor* qt, const void* dev_x, int32_t x_dtype, int64_t m,
                     float* dev_y, int32_t mode, const float* dev_bias, void* stream) {
  if (!ctx || !qt || !dev_x || !dev_y) return fail(ctx, TURQ_E_INVALID_ARG, "null argument");
  if (x_dtype != TURQ_F32 && x_dtype != TURQ_BF16) return fail(ctx, TURQ_E_DTYPE, "activations must be F32 or BF16 (got %d)", x_dtype);
  if (m <= 0) return fail(ctx, TURQ_E_SHAPE, "m=%lld must be positive", (long long)m);
  if (m > INT32_MAX / 2) return fail(ctx, TURQ_E_SHAPE, "m=%lld too large", (long long)m);
  if (qt->device != ctx->device) return fail(ctx, TURQ_E_INVALID_ARG, "tensor lives on device %d, context on %d", qt->device, ctx->device);
  if ((uintptr_t)dev_x % 16 != 0 || (uintptr_t)dev_y % 4 != 0) return fail(ctx, TURQ_E_ALIGN, "dev_x must be 16-byte aligned");
  if (mode == TURQ_MODE_AUTO) mode = auto_mode(ctx, qt->n_rows, qt->n_cols, m);
  if (mode == TURQ_MODE_TENSOR_CORE && qt->n_cols % 64 != 0)
    return fail(ctx, TURQ_E_SHAPE, "the tensor-core mode needs in-features to be a multiple of 64 (got %lld)", (long long)qt->n_cols);
  TQ_CUDA(ctx, cudaSetDevice(ctx->device));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t k = qt->n_cols;
  int launches = 0;
  cudaError_t e = cudaSuccess;
  if (mode == TURQ_MODE_INT8_ACT) {
    const int fmt = qt->dtype == TURQ_Q8_0 ? TQ_Q8_0 : TQ_Q8_K;
    turq::ActPackPlan plan = turq::plan_act_pack(fmt, m, k);
    int32_t st = ensure(ctx, &ctx->scratch, &ctx->scratch_bytes, plan.total);
    if (st != TURQ_OK) return st;
    e = turq::launch_gemv_int8(qt->dtype, qt->tiles, qt->n_rows, k, dev_x, x_dtype, ctx->scratch, m, dev_y, dev_bias,
                               ctx->gemv_ws, ctx->dev_status, ctx->sm_count, s, &launches);
  } else if (mode == TURQ_MODE_EXACT_F32) {
    e = turq::launch_gemv_f32(qt->dtype, qt->tiles, qt->n_rows, k, dev_x, x_dtype, m, dev_y, dev_bias, ctx->sm_count, s, &launches);
  } else if (mode == TURQ_MODE_TENSOR_CORE) {
    int32_t st = ensure(ctx, &ctx->scratch, &ctx->scratch_bytes, turq::gemm_tc_scratch_bytes(m, k, qt->n_rows, ctx->sm_count));
    if (st != TURQ_OK) return st;
    e = turq::launch_gemm_tc(qt->dtype, qt->tiles, qt->n_rows, k, dev_x, x_dtype, m, dev_y, dev_bias, ctx->scratch,
                             ctx->sm_count, s, &launches, ctx->dev_status);
  } else {
    return fail(ctx, TURQ_E_INVALID_ARG, "unknown mode %d", mode);
  }
  ctx->launches += launches;
  if (e != cudaSuccess) return cuda_fail(ctx, e, "qmatmul launch");
  return TURQ_OK;
}

static int32_t qmatmul_multi_impl(turq_ctx* ctx, int32_t count, const turq_qtensor* const* qts, const void* dev_x,
                                  int32_t x_dtype, int64_t m, float* const* dev_ys, int32_t mode,
                                  const float* const* dev_biases, void* stream, bool x_remote,
                                  uint8_t* own_scratch = nullptr /* planes buffer of a bound call instead of the context's */) {
  if (!ctx || !qts || !dev_x || !dev_ys) return fail(ctx, TURQ_E_INVALID_ARG, "null argument");
  if (count < 1 || count > 4) return fail(ctx, TURQ_E_INVALID_ARG, "count %d outside 1..4", count);
  for (int i = 0; i < count; i++) {
    if (!qts[i] || !dev_ys[i]) return fail(ctx, TURQ_E_INVALID_ARG, "null argument");
    if (qts[i]->n_cols != qts[0]->n_cols) return fail(ctx, TURQ_E_SHAPE, "weights of one call must share the in-feature count");
  }
  // One activation format per call: K-quant weights (Q8_K activations) and Q8_0 weights do not mix.
  bool same = true;
  for (int i = 1; i < count; i++)
    same = same && (qts[i]->dtype == TURQ_Q8_0) == (qts[0]->dtype == TURQ_Q8_0) && qts[i]->device == qts[0]->device;
  int32_t eff = mode;
  if (eff == TURQ_MODE_AUTO) {
    int64_t rows_all = 0;
    for (int i = 0; i < count; i++) rows_all += qts[i]->n_rows;
    eff = auto_mode(ctx, rows_all, qts[0]->n_cols, m);
  }
  if (eff == TURQ_MODE_TENSOR_CORE && count > 1 && !x_remote && qts[0]->n_cols % 64 == 0 && m > 0 && m <= INT32_MAX / 2 &&
      (x_dtype == TURQ_F32 || x_dtype == TURQ_BF16) && (uintptr_t)dev_x % 16 == 0) {
    // tensor-core scheme: x is converted to the f16 operand once for all the weights
    const int64_t k = qts[0]->n_cols;
    size_t need = 0;
    for (int i = 0; i < count; i++) {
      if (qts[i]->device != ctx->device) return fail(ctx, TURQ_E_INVALID_ARG, "tensor lives on device %d, context on %d", qts[i]->device, ctx->device);
      const size_t b = turq::gemm_tc_scratch_bytes(m, k, qts[i]->n_rows, ctx->sm_count);
      if (b > need) need = b;
    }
    TQ_CUDA(ctx, cudaSetDevice(ctx->device));
    int32_t st = ensure(ctx, &ctx->scratch, &ctx->scratch_bytes, need);
    if (st != TURQ_OK) return st;
    for (int i = 0; i < count; i++) {
      int launches = 0;
      cudaError_t e = turq::launch_gemm_tc(qts[i]->dtype, qts[i]->tiles, qts[i]->n_rows, k, dev_x, x_dtype, m, dev_ys[i],
                                           dev_biases ? dev_biases[i] : nullptr, ctx->scratch, ctx->sm_count,
                                           static_cast<cudaStream_t>(stream), &launches, ctx->dev_status, i > 0);
      ctx->launches += launches;
      if (e != cudaSuccess) return cuda_fail(ctx, e, "qmatmul_multi launch");
    }
    return TURQ_OK;
  }
  if (!same || eff != TURQ_MODE_INT8_ACT || (count == 1 && !x_remote)) {
    if (x_remote) return fail(ctx, TURQ_E_INVALID_ARG, "host-mapped activations need the integer scheme and one activation format");
    for (int i = 0; i < count; i++) {
      int32_t st = turq_qmatmul(ctx, qts[i], dev_x, x_dtype, m, dev_ys[i], mode, dev_biases ? dev_biases[i] : nullptr, stream);
      if (st != TURQ_OK) return st;
    }
    return TURQ_OK;
  }
  if (x_dtype != TURQ_F32 && x_dtype != TURQ_BF16) return fail(ctx, TURQ_E_DTYPE, "activations must be F32 or BF16 (got %d)", x_dtype);
  if (m <= 0 || m > INT32_MAX / 2) return fail(ctx, TURQ_E_SHAPE, "m=%lld out of range", (long long)m);
  if (qts[0]->device != ctx->device) return fail(ctx, TURQ_E_INVALID_ARG, "tensor lives on device %d, context on %d", qts[0]->device, ctx->device);
  if ((uintptr_t)dev_x % 16 != 0) return fail(ctx, TURQ_E_ALIGN, "dev_x must be 16-byte aligned");
  TQ_CUDA(ctx, cudaSetDevice(ctx->device));
  const int64_t k = qts[0]->n_cols;
  const int fmt = qts[0]->dtype == TURQ_Q8_0 ? TQ_Q8_0 : TQ_Q8_K;
  turq::ActPackPlan plan = turq::plan_act_pack(fmt, m, k);
  if (!own_scratch) {
    int32_t st = ensure(ctx, &ctx->scratch, &ctx->scratch_bytes, plan.total);
    if (st != TURQ_OK) return st;
  }
  turq::GemvPart parts[4];
  for (int i = 0; i < count; i++)
    parts[i] = turq::GemvPart{qts[i]->tiles, qts[i]->n_rows, dev_ys[i], dev_biases ? dev_biases[i] : nullptr, qts[i]->dtype, nullptr};
  int launches = 0;
  cudaError_t e = turq::launch_gemv_int8_multi(qts[0]->dtype, parts, count, k, dev_x, x_dtype, own_scratch ? own_scratch : ctx->scratch, m, ctx->gemv_ws,
                                               ctx->dev_status, ctx->sm_count, static_cast<cudaStream_t>(stream), &launches,
                                               x_remote);
  ctx->launches += launches;
  if (e != cudaSuccess) return cuda_fail(ctx, e, "qmatmul_multi launch");
  return TURQ_OK;
}

int32_t turq_qmatmul_multi(turq_ctx* ctx, int32_t count, const turq_qtensor* const* qts, const void* dev_x,
                           int32_t x_dtype, int64_t m, float* const* dev_ys, int32_t mode,
                           const float* const* dev_biases, void* stream) {
  return qmatmul_multi_impl(ctx, count, qts, dev_x, x_dtype, m, dev_ys, mode, dev_biases, stream, false);
}

}  // extern "C"

namespace {
// Last launch of a host-buffer call: once everything before it has completed (and its stores to the
// caller's mapped buffers with it), the call number goes into the context's completion word in
// mapped host memory, where the host waits for it (wait_for_signal).
__global__ void host_signal_kernel(unsigned* count, volatile unsigned* flag) {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const unsigned v = *count + 1u;
  *count = v;
  __threadfence_system();
  *flag = v;
}

cudaError_t launch_host_signal(turq_ctx* ctx, cudaStream_t s) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(1);
  cfg.blockDim = dim3(1);
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, host_signal_kernel, ctx->done_count, static_cast<volatile unsigned*>(ctx->dev_done));
}

// Waits for the work queued on the context's stream up to and including a signal: the signal
// kernel goes behind it, and the host spins on the completion word - bounded: after two seconds
// (a kernel that gave up its own bounded wait finishes far sooner) the stream is synchronized the
// ordinary way. `launched`: the signal is part of a graph that has just been launched.
int32_t wait_for_signal(turq_ctx* ctx, bool launched) {
  if (!launched) {
    cudaError_t e = launch_host_signal(ctx, ctx->own_stream);
    ctx->launches++;
    if (e != cudaSuccess) {
      cudaGetLastError();
      return turq_ctx_poll_status(ctx, ctx->own_stream);
    }
  }
  const unsigned expected = ++ctx->done_expected;
  const auto t0 = std::chrono::steady_clock::now();
  for (unsigned spins = 0; *ctx->host_done != expected; spins++) {
    if ((spins & 0xFFFu) == 0xFFFu && std::chrono::steady_clock::now() - t0 > std::chrono::seconds(2)) {
      cudaError_t e = cudaStreamSynchronize(ctx->own_stream);
      if (e != cudaSuccess) return cuda_fail(ctx, e, "waiting for a host call");
      break;
    }
  }
  std::atomic_thread_fence(std::memory_order_acquire);
  if (*static_cast<volatile int*>(ctx->host_status) != 0) return turq_ctx_poll_status(ctx, ctx->own_stream);
  return TURQ_OK;
}
}  // namespace

extern "C" {

// Device-side alias of a host pointer when the memory is page-locked and reachable from this
// device (cudaHostAlloc / cudaHostRegister under unified addressing); nullptr otherwise.
static void* mapped_alias(const void* host_ptr) {
  cudaPointerAttributes at;
  if (cudaPointerGetAttributes(&at, host_ptr) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  if (at.type != cudaMemoryTypeHost || !at.devicePointer) return nullptr;
  return at.devicePointer;
}

int32_t turq_qmatmul_multi_host(turq_ctx* ctx, int32_t count, const turq_qtensor* const* qts, const float* host_x,
                                int64_t m, float* const* host_ys, int32_t mode, const float* const* host_biases) {
  if (!ctx || !qts || !host_x || !host_ys) return fail(ctx, TURQ_E_INVALID_ARG, "null argument");
  if (count < 1 || count > 4) return fail(ctx, TURQ_E_INVALID_ARG, "count %d outside 1..4", count);
  if (m <= 0 || m > INT32_MAX / 2) return fail(ctx, TURQ_E_SHAPE, "m=%lld out of range", (long long)m);
  bool k_quant = false, q8_0 = false;
  int64_t rows_all = 0, rows_max = 0;
  for (int i = 0; i < count; i++) {
    if (!qts[i] || !host_ys[i]) return fail(ctx, TURQ_E_INVALID_ARG, "null argument");
    if (qts[i]->n_cols != qts[0]->n_cols) return fail(ctx, TURQ_E_SHAPE, "weights of one call must share the in-feature count");
    (qts[i]->dtype == TURQ_Q8_0 ? q8_0 : k_quant) = true;
    rows_all += qts[i]->n_rows;
    if (qts[i]->n_rows > rows_max) rows_max = qts[i]->n_rows;
  }
  TQ_CUDA(ctx, cudaSetDevice(ctx->device));
  cudaStream_t s = ctx->own_stream;
  const int64_t k = qts[0]->n_cols;
  const int32_t eff = mode == TURQ_MODE_AUTO ? auto_mode(ctx, rows_all, k, m) : mode;
  auto up = [](size_t v) { return (v + 255) & ~(size_t)255; };

  // Decode-sized calls on page-locked buffers run without any copy: the quantization launch
  // reads x from the caller's memory once, the GEMV writes y straight into it, and the one
  // synchronize at the end is the only host wait. Needs the integer scheme, 16-byte aligned x
  // and little enough output that posted writes over the bus do not hold the kernel up.
  if (eff == TURQ_MODE_INT8_ACT && !(k_quant && q8_0) && (size_t)m * rows_max * 4 <= ((size_t)2 << 20)) {
    bool any_bias = false;
    for (int i = 0; host_biases && i < count; i++) any_bias = any_bias || host_biases[i] != nullptr;
    void* mx = any_bias ? nullptr : mapped_alias(host_x);  // a bias would be read element-wise over the bus
    float* mys[4] = {nullptr, nullptr, nullptr, nullptr};
    bool ok = mx != nullptr && (uintptr_t)mx % 16 == 0;
    for (int i = 0; ok && i < count; i++) {
      mys[i] = static_cast<float*>(mapped_alias(host_ys[i]));
      ok = mys[i] != nullptr;
    }
    if (ok) {
      int32_t st = qmatmul_multi_impl(ctx, count, qts, mx, TURQ_F32, m, mys, TURQ_MODE_INT8_ACT, nullptr, s, true);
      if (st != TURQ_OK) return st;
      return s == ctx->own_stream ? wait_for_signal(ctx, false) : turq_ctx_poll_status(ctx, s);
    }
  }

  // General case: one copy of x in, one launch group, one copy per output back, one synchronize.
  size_t need = up((size_t)m * k * 4);
  for (int i = 0; i < count; i++) need += up((size_t)m * qts[i]->n_rows * 4) + up((size_t)qts[i]->n_rows * 4);
  int32_t st = ensure(ctx, &ctx->io, &ctx->io_bytes, need);
  if (st != TURQ_OK) return st;
  uint8_t* p = ctx->io;
  float* dx = reinterpret_cast<float*>(p);
  p += up((size_t)m * k * 4);
  float* dys[4];
  const float* dbs[4];
  TQ_CUDA(ctx, cudaMemcpyAsync(dx, host_x, (size_t)m * k * 4, cudaMemcpyHostToDevice, s));
  for (int i = 0; i < count; i++) {
    dys[i] = reinterpret_cast<float*>(p);
    p += up((size_t)m * qts[i]->n_rows * 4);
    dbs[i] = nullptr;
    if (host_biases && host_biases[i]) {
      TQ_CUDA(ctx, cudaMemcpyAsync(p, host_biases[i], (size_t)qts[i]->n_rows * 4, cudaMemcpyHostToDevice, s));
      dbs[i] = reinterpret_cast<const float*>(p);
    }
    p += up((size_t)qts[i]->n_rows * 4);
  }
  st = qmatmul_multi_impl(ctx, count, qts, dx, TURQ_F32, m, dys, mode, dbs, s, false);
  if (st != TURQ_OK) return st;
  for (int i = 0; i < count; i++)
    TQ_CUDA(ctx, cudaMemcpyAsync(host_ys[i], dys[i], (size_t)m * qts[i]->n_rows * 4, cudaMemcpyDeviceToHost, s));
  return turq_ctx_poll_status(ctx, s);
}

int32_t turq_host_call_create(turq_ctx* ctx, int32_t count, const turq_qtensor* const* qts, const float* host_x, int64_t m,
                              float* const* host_ys, turq_host_call** out) {
  if (!ctx || !qts || !host_x || !host_ys || !out) return fail(ctx, TURQ_E_INVALID_ARG, "null argument");
  *out = nullptr;
  if (count < 1 || count > 4) return fail(ctx, TURQ_E_INVALID_ARG, "count %d outside 1..4", count);
  if (m <= 0 || m > 64) return fail(ctx, TURQ_E_LIMIT, "a bound host call takes 1..64 rows (decode batches); use turq_qmatmul_multi_host beyond");
  bool k_quant = false, q8_0 = false;
  for (int i = 0; i < count; i++) {
    if (!qts[i] || !host_ys[i]) return fail(ctx, TURQ_E_INVALID_ARG, "null argument");
    if (qts[i]->n_cols != qts[0]->n_cols || qts[i]->device != ctx->device)
      return fail(ctx, TURQ_E_SHAPE, "weights of one call must share the in-feature count and live on the context's device");
    (qts[i]->dtype == TURQ_Q8_0 ? q8_0 : k_quant) = true;
  }
  if (k_quant && q8_0) return fail(ctx, TURQ_E_DTYPE, "Q8_0 and K-quant weights do not share an activation format");
  TQ_CUDA(ctx, cudaSetDevice(ctx->device));
  turq_host_call* hc = new (std::nothrow) turq_host_call();
  if (!hc) return fail(ctx, TURQ_E_INVALID_ARG, "out of host memory");
  hc->ctx = ctx;
  void* mx = mapped_alias(host_x);
  float* mys[4] = {nullptr, nullptr, nullptr, nullptr};
  bool ok = mx != nullptr && (uintptr_t)mx % 16 == 0;
  for (int i = 0; ok && i < count; i++) {
    mys[i] = static_cast<float*>(mapped_alias(host_ys[i]));
    ok = mys[i] != nullptr;
  }
  if (!ok) {
    delete hc;
    return fail(ctx, TURQ_E_INVALID_ARG, "a bound host call needs page-locked x (16-byte aligned) and y buffers (cudaHostAlloc / cudaHostRegister)");
  }
  const int64_t k = qts[0]->n_cols;
  const int fmt = q8_0 ? TQ_Q8_0 : TQ_Q8_K;
  cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&hc->scratch), turq::plan_act_pack(fmt, m, k).total);
  if (e != cudaSuccess) {
    delete hc;
    return cuda_fail(ctx, e, "cudaMalloc(bound call planes)");
  }
  // The launches of the call, recorded once: afterwards a run is one graph launch and one synchronize.
  cudaStream_t s = ctx->own_stream;
  cudaGraph_t graph = nullptr;
  e = cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal);
  int32_t st = TURQ_OK;
  if (e == cudaSuccess) {
    st = qmatmul_multi_impl(ctx, count, qts, mx, TURQ_F32, m, mys, TURQ_MODE_INT8_ACT, nullptr, s, true, hc->scratch);
    cudaError_t es = st == TURQ_OK ? launch_host_signal(ctx, s) : cudaSuccess;
    if (st == TURQ_OK) ctx->launches++;
    e = cudaStreamEndCapture(s, &graph);
    if (e == cudaSuccess) e = es;
  }
  if (e == cudaSuccess && st == TURQ_OK) e = cudaGraphInstantiate(&hc->exec, graph, 0);
  if (graph) cudaGraphDestroy(graph);
  if (e != cudaSuccess || st != TURQ_OK) {
    cudaGetLastError();
    turq_host_call_destroy(hc);
    return st != TURQ_OK ? st : cuda_fail(ctx, e, "recording the bound call");
  }
  *out = hc;
  return TURQ_OK;
}

int32_t turq_host_call_run(turq_host_call* hc) {
  if (!hc || !hc->ctx || !hc->exec) return TURQ_E_INVALID_ARG;
  turq_ctx* ctx = hc->ctx;
  TQ_CUDA(ctx, cudaGraphLaunch(hc->exec, ctx->own_stream));
  // Wait for the call's own completion word instead of synchronizing the stream: the host sees
  // the result a few microseconds earlier. Bounded: after two seconds (a kernel that gave up its
  // own bounded wait finishes far sooner) the stream is synchronized the ordinary way.
  return wait_for_signal(ctx, true);
}

int32_t turq_host_call_destroy(turq_host_call* hc) {
  if (!hc) return TURQ_E_INVALID_ARG;
  if (hc->ctx) {
    cudaSetDevice(hc->ctx->device);
    cudaStreamSynchronize(hc->ctx->own_stream);
  }
  if (hc->exec) cudaGraphExecDestroy(hc->exec);
  if (hc->scratch) cudaFree(hc->scratch);
  delete hc;
  return TURQ_OK;
}

int32_t turq_qmatmul_host(turq_ctx* ctx, const turq_qtensor* qt, const float* host_x, int64_t m, float* host_y,
                          int32_t mode, const float* host_bias) {
  if (!ctx || !qt || !host_x || !host_y) return fail(ctx, TURQ_E_INVALID_ARG, "null argument");
  return turq_qmatmul_multi_host(ctx, 1, &qt, host_x, m, &host_y, mode, host_bias ? &host_bias : nullptr);
}

}  // extern "C"

namespace turq {

int32_t qmatmul_for_exchange(turq_ctx* ctx, const turq_qtensor* qt, const void* dev_x, int32_t x_dtype, int64_t m, float* s0,
                             float* s1, const unsigned* toggle, int32_t mode, cudaStream_t s, float** staged,
                             const TpArgs* fuse, bool* fused, const float* local_bias) {
  *staged = nullptr;
  *fused = false;
  if (x_dtype != TURQ_F32 && x_dtype != TURQ_BF16) return fail(ctx, TURQ_E_DTYPE, "activations must be F32 or BF16 (got %d)", x_dtype);
  if (qt->device != ctx->device) return fail(ctx, TURQ_E_INVALID_ARG, "tensor lives on device %d, context on %d", qt->device, ctx->device);
  if ((uintptr_t)dev_x % 16 != 0) return fail(ctx, TURQ_E_ALIGN, "dev_x must be 16-byte aligned");
  if (mode == TURQ_MODE_AUTO) mode = auto_mode(ctx, qt->n_rows, qt->n_cols, m);
  TQ_CUDA(ctx, cudaSetDevice(ctx->device));
  if (mode == TURQ_MODE_INT8_ACT) {
    const int64_t k = qt->n_cols;
    const int fmt = qt->dtype == TURQ_Q8_0 ? TQ_Q8_0 : TQ_Q8_K;
    int32_t st = ensure(ctx, &ctx->scratch, &ctx->scratch_bytes, plan_act_pack(fmt, m, k).total);
    if (st != TURQ_OK) return st;
    GemvPart part{qt->tiles, qt->n_rows, s0, local_bias, qt->dtype, s1};
    int launches = 0;
    const bool fuse_now = fuse != nullptr && m <= 32;
    cudaError_t e = launch_gemv_int8_multi(qt->dtype, &part, 1, k, dev_x, x_dtype, ctx->scratch, m, ctx->gemv_ws, ctx->dev_status,
                                           ctx->sm_count, s, &launches, false, toggle, false, fuse_now ? fuse : nullptr);
    *fused = fuse_now;
    ctx->launches += launches;
    if (e != cudaSuccess) return cuda_fail(ctx, e, "row-parallel GEMV launch");
    return TURQ_OK;
  }
  if (mode == TURQ_MODE_TENSOR_CORE && qt->n_cols % 64 == 0 && m <= INT32_MAX / 2) {
    // the GEMM's epilogue (or its split-K reduction) picks the slot itself: no staging copy
    int32_t st = ensure(ctx, &ctx->scratch, &ctx->scratch_bytes, gemm_tc_scratch_bytes(m, qt->n_cols, qt->n_rows, ctx->sm_count));
    if (st != TURQ_OK) return st;
    int launches = 0;
    cudaError_t e = launch_gemm_tc(qt->dtype, qt->tiles, qt->n_rows, qt->n_cols, dev_x, x_dtype, m, s0, local_bias, ctx->scratch,
                                   ctx->sm_count, s, &launches, ctx->dev_status, false, toggle, s1);
    ctx->launches += launches;
    if (e != cudaSuccess) return cuda_fail(ctx, e, "row-parallel GEMM launch");
    return TURQ_OK;
  }
  int32_t st = ensure(ctx, &ctx->tmp, &ctx->tmp_bytes, (size_t)m * qt->n_rows * 4);
  if (st != TURQ_OK) return st;
  st = turq_qmatmul(ctx, qt, dev_x, x_dtype, m, reinterpret_cast<float*>(ctx->tmp), mode, local_bias, s);
  if (st != TURQ_OK) return st;
  *staged = reinterpret_cast<float*>(ctx->tmp);
  return TURQ_OK;
}

// ---- helpers of this translation unit, shared with the fused entries (fused.cu)
int32_t api_fail(turq_ctx* ctx, int32_t st, const char* msg) { return fail(ctx, st, "%s", msg); }
int32_t api_cuda_fail(turq_ctx* ctx, cudaError_t e, const char* what) { return cuda_fail(ctx, e, what); }
int32_t api_ensure_scratch(turq_ctx* ctx, size_t bytes) { return ensure(ctx, &ctx->scratch, &ctx->scratch_bytes, bytes); }
int32_t api_ensure_tmp(turq_ctx* ctx, size_t bytes) { return ensure(ctx, &ctx->tmp, &ctx->tmp_bytes, bytes); }
int32_t api_auto_mode(const turq_ctx* ctx, int64_t n_rows, int64_t n_cols, int64_t m) { return auto_mode(ctx, n_rows, n_cols, m); }

}  // namespace turq
