// turq_qmatmul_static: the integer-scheme QMatMul for callers that may not allocate.
//
// Who needs it: a host that runs under a pre-reserved device-memory budget (an inference
// server whose allocator grabbed the whole GPU at start-up, a plugin loaded into somebody
// else's process) cannot let a library call cudaMalloc on its behalf - the call may fail,
// or it may synchronise the device in the middle of the host's pipeline. The regular entry
// keeps the quantized activation planes in a context-owned buffer that grows on demand; this
// variant keeps them in a fixed array that is part of the library image instead, so the
// call itself touches no allocator at all.
//
// The price: the array has a fixed size (TURQ_STATIC_SCRATCH_BYTES, resident on every GPU
// that loads the library until the process exits). Its tail holds the GEMV's hand-over
// workspace for row-tiles cut between CTAs (about 1.2 MB on a 148-SM part), the rest - about
// 2.8 MiB there - is what the activation planes of one call may use (roughly m * k * 1.2
// bytes); larger requests are refused with TURQ_E_LIMIT. All calls on one GPU share it - two calls whose kernels may overlap on
// the GPU (different streams) race on it and must be serialised by the caller.
#include <cstdio>
#include <mutex>

#include "../../include/turq.h"
#include "handles.h"
#include "turq_internal.h"

namespace {

// Quantized activation planes of the call in flight, followed by the GEMV's workspace for
// row-tiles split between CTAs. The planes need no clearing (every element read is written
// first by the same call), nor do the workspace's partial sums; its ready flags must start at
// zero and are cleared by each call before its kernels run.
static __device__ __align__(256) uint8_t g_static_scratch[TURQ_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
uint8_t* g_scratch_addr[kMaxDevices] = {};  // device address of g_static_scratch, per device

// In host code `g_static_scratch` is only a handle for the runtime, not a device address, so
// the address the kernels get is looked up once per device (with that device current).
cudaError_t scratch_for_device(int device, uint8_t** out) {
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (!g_scratch_addr[device]) {
    cudaError_t e = cudaSetDevice(device);
    if (e != cudaSuccess) return e;
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess) return e;
    g_scratch_addr[device] = static_cast<uint8_t*>(p);
  }
  *out = g_scratch_addr[device];
  return cudaSuccess;
}

int32_t fail(turq_ctx* ctx, int32_t st, const char* msg) {
  if (ctx) {
    try {
      ctx->err = msg;
    } catch (...) {
    }
  }
  return st;
}

}  // namespace

extern "C" int32_t turq_qmatmul_static(turq_ctx* ctx, const turq_qtensor* qt, const void* dev_x, int32_t x_dtype,
                                       int64_t m, float* dev_y, const float* dev_bias, void* stream) {
  if (!ctx || !qt || !dev_x || !dev_y) return fail(ctx, TURQ_E_INVALID_ARG, "null argument");
  if (x_dtype != TURQ_F32 && x_dtype != TURQ_BF16) return fail(ctx, TURQ_E_DTYPE, "activations must be F32 or BF16");
  if (m <= 0) return fail(ctx, TURQ_E_SHAPE, "m must be positive");
  if (m > INT32_MAX / 2) return fail(ctx, TURQ_E_SHAPE, "m is too large");
  if (qt->device != ctx->device || ctx->device < 0 || ctx->device >= kMaxDevices)
    return fail(ctx, TURQ_E_INVALID_ARG, "tensor and context must live on the same device");
  if ((uintptr_t)dev_x % 16 != 0 || (uintptr_t)dev_y % 4 != 0) return fail(ctx, TURQ_E_ALIGN, "dev_x must be 16-byte aligned");
  const int64_t k = qt->n_cols;
  const int fmt = qt->dtype == TURQ_Q8_0 ? TQ_Q8_0 : TQ_Q8_K;
  const turq::ActPackPlan plan = turq::plan_act_pack(fmt, m, k);
  // the tail of the array is the GEMV's split row-tile workspace (partial sums + ready flags)
  const size_t ws_bytes = (turq::gemv_workspace_bytes(ctx->sm_count) + 255) & ~(size_t)255;
  if (ws_bytes >= (size_t)TURQ_STATIC_SCRATCH_BYTES) return fail(ctx, TURQ_E_LIMIT, "this GPU's hand-over workspace alone exceeds the static buffer");
  const size_t capacity = (size_t)TURQ_STATIC_SCRATCH_BYTES - ws_bytes;
  if (plan.total > capacity) {
    char buf[240];
    snprintf(buf, sizeof(buf),
             "m=%lld x k=%lld needs %zu bytes of activation planes, the static buffer has room for %zu (%d bytes minus "
             "the %zu-byte hand-over workspace)",
             (long long)m, (long long)k, plan.total, capacity, (int)TURQ_STATIC_SCRATCH_BYTES, ws_bytes);
    return fail(ctx, TURQ_E_LIMIT, buf);
  }
  uint8_t* scratch = nullptr;
  cudaError_t e = scratch_for_device(ctx->device, &scratch);  // first call per device does the look-up
  if (e == cudaSuccess) e = cudaSetDevice(ctx->device);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int launches = 0;
  uint8_t* ws = scratch + TURQ_STATIC_SCRATCH_BYTES - ws_bytes;
  // The ready flags must read zero at kernel start. A completed call leaves them zero, but the
  // array is shared and outlives failed calls, so they are cleared every time (stream-ordered).
  if (e == cudaSuccess)
    e = cudaMemsetAsync(ws + turq::gemv_workspace_flags_offset(ctx->sm_count), 0, turq::gemv_workspace_flags_bytes(ctx->sm_count), s);
  if (e == cudaSuccess)
    e = turq::launch_gemv_int8(qt->dtype, qt->tiles, qt->n_rows, k, dev_x, x_dtype, scratch, m, dev_y, dev_bias, ws,
                               ctx->dev_status, ctx->sm_count, s, &launches);
  ctx->launches += launches;
  if (e != cudaSuccess) return fail(ctx, TURQ_E_CUDA, cudaGetErrorString(e));
  return TURQ_OK;
}
