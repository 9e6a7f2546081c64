// Tensor-parallel exchange over peer memory (NVLink / NVSwitch): the all-reduce behind the
// row-parallel linears (attn_output, ffn_down) and the all-gather behind the vocabulary-sharded
// head, as kernels of this library instead of NCCL calls, so that a whole sharded decode pass
// can live in one CUDA graph and the partial sums never take an extra copy.
//
// The reference is single-device (src/models/layers/norm.rs:50 passes Shard::default()
// everywhere); this is the multi-GPU extension of its linear layers.
//
// Memory. Every rank owns one exchange region allocated with cudaMalloc and opened on the other
// ranks through CUDA IPC handles (one process per GPU, one node):
//     [ flags: MAX_BLOCKS x MAX_RANKS u32 | counter: 4 u32 | slot 0 | slot 1 ]
// A linear's epilogue writes its partial result straight into a slot of the local region; the
// exchange kernel then tells every peer "my slot is complete" (one system-scope release store per
// peer and CTA), waits for the peers' signals, and reads the peers' slots with plain 128-bit peer
// loads in rank order - a fixed summation order, no float atomics, no multicast loads of any
// kind, no library kernel ever sees a peer pointer.
//
// Slots alternate by call parity. A rank can run at most one call ahead of the slowest peer (it
// cannot pass the next call's wait before that peer has signalled, which the peer only does
// after it finished reading), so the slot a fast rank writes next is never one a slow peer still
// reads. The call number lives in device memory (counter[0]) and is advanced by the exchange
// kernel itself, which is what lets a captured graph replay the same launches again and again;
// the GEMV picks its output slot from the same word.
//
// Every wait is bounded by a cycle limit held in the handle; when it runs out the kernel records
// TURQ_E_TIMEOUT in the context's status word, skips the exchange and returns. The sequence is
// then out of step across ranks: the host reads the status (turq_ctx_poll_status) and every
// rank calls turq_tp_reset before the group is used again.
#include <cstdio>
#include <cstring>
#include <new>

#include "../../include/turq.h"
#include "handles.h"
#include "tp_exchange.cuh"
#include "turq_internal.h"

namespace turq {

// The exchange kernels are launched with programmatic stream serialization: they let the next
// launch (a GEMV that starts by streaming weights) be scheduled at once, and wait themselves for
// the kernel that filled the slot before they tell the peers about it.
__global__ void __launch_bounds__(TP_THREADS) tp_allreduce_kernel(const TpArgs a) {
  __shared__ int s_ok;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const unsigned seq = *reinterpret_cast<volatile unsigned*>(a.counter) + 1u;
  const size_t slot_off = (seq & 1u) ? a.slot_elems : 0;
  const bool ok = tp_rendezvous(a, seq, &s_ok, blockIdx.x);
  if (ok)
    tp_reduce_range(a, slot_off, (int64_t)blockIdx.x * TP_THREADS + threadIdx.x, (int64_t)gridDim.x * TP_THREADS, blockIdx.x == 0);
  tp_finish(a, seq, ok);
}

// Large results on three or more ranks: reduce-scatter, then gather (tp_twoshot).
__global__ void __launch_bounds__(TP_THREADS) tp_allreduce2_kernel(const TpArgs a) {
  __shared__ int s_ok;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const unsigned seq = *reinterpret_cast<volatile unsigned*>(a.counter) + 1u;
  const size_t slot_off = (seq & 1u) ? a.slot_elems : 0;
  bool ok = tp_rendezvous(a, seq, &s_ok, blockIdx.x);
  if (ok) ok = tp_twoshot(a, seq, slot_off, &s_ok, blockIdx.x, gridDim.x);
  tp_finish(a, seq, ok);
}

__global__ void __launch_bounds__(TP_THREADS) tp_allgather_kernel(const TpArgs a) {
  __shared__ int s_ok;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const unsigned seq = *reinterpret_cast<volatile unsigned*>(a.counter) + 1u;
  const size_t slot_off = (seq & 1u) ? a.slot_elems : 0;
  const bool ok = tp_rendezvous(a, seq, &s_ok, blockIdx.x);
  if (ok) {
    // one (rank, row) run of columns at a time; widths are multiples of 4 floats
    const int64_t runs = (int64_t)a.world * a.m;
    for (int64_t run = blockIdx.x; run < runs; run += gridDim.x) {
      const int p = (int)(run / a.m);
      const int64_t r = run - (int64_t)p * a.m;
      const int64_t width = a.col0[p + 1] - a.col0[p];
      const float* src = a.peer_data[p] + slot_off + r * width;
      float* dst = a.out + r * a.n_total + a.col0[p];
      if ((width & 3) == 0 && ((a.col0[p] | a.n_total) & 3) == 0) {
        for (int64_t v = threadIdx.x; v < (width >> 2); v += TP_THREADS)
          *reinterpret_cast<float4*>(dst + 4 * v) = ld_peer_v4(src + 4 * v);
      } else {
        for (int64_t i = threadIdx.x; i < width; i += TP_THREADS) dst[i] = ld_peer_f32(src + i);
      }
    }
  }
  tp_finish(a, seq, ok);
}

// Copies a result that was computed elsewhere into the slot of the upcoming call.
__global__ void __launch_bounds__(256) tp_stage_kernel(const float* __restrict__ src, float* __restrict__ slots,
                                                        size_t slot_elems, const unsigned* counter, int64_t count) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const unsigned seq = *reinterpret_cast<const volatile unsigned*>(counter) + 1u;
  float* dst = slots + ((seq & 1u) ? slot_elems : 0);
  const int64_t nvec = count >> 2;
  for (int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v < nvec; v += (int64_t)gridDim.x * blockDim.x)
    reinterpret_cast<float4*>(dst)[v] = reinterpret_cast<const float4*>(src)[v];
  if (blockIdx.x == 0)
    for (int64_t i = (nvec << 2) + threadIdx.x; i < count; i += blockDim.x) dst[i] = src[i];
}

}  // namespace turq

namespace {
template <class... Params, class... Args>
cudaError_t tp_launch_pdl(void (*kernel)(Params...), unsigned grid, unsigned block, cudaStream_t s, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(block);
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, args...);
}
}  // namespace

struct turq_tp {
  turq_ctx* ctx = nullptr;
  int rank = 0, world = 1;
  size_t slot_bytes = 0;                 // bytes per slot (multiple of 256)
  uint8_t* region = nullptr;             // own region
  size_t region_bytes = 0;
  uint8_t* peers[turq::TP_MAX_RANKS] = {};  // every rank's region as this process sees it (own = region)
  bool opened[turq::TP_MAX_RANKS] = {};     // true: mapped with cudaIpcOpenMemHandle (close on destroy)
  bool loopback[turq::TP_MAX_RANKS] = {};   // true: a local stand-in allocated by turq_tp_connect_loopback
  bool connected = false;
  long long wait_cycles = 2000000000ll;  // about one second of SM clock
  size_t fuse_max_bytes = 64 << 10;      // results up to this size are exchanged by the GEMV's own last CTA
  // Results from this size on take the two-shot exchange (3+ ranks). Measured at 4 ranks: a 1.3 MB
  // result (64 decode rows) is faster one-shot (cfg5 pass 10.4 against 11.7 ms), an 84 MB result
  // (4096 prefill rows) two-shot (113 against 134 ms).
  size_t twoshot_min_bytes = 4 << 20;
  int64_t chunk_rows = 0;                // rows per chunk of a chunked row-parallel GEMM (0: not cut)
  // chunked row-parallel GEMM: the exchange of chunk j runs on `comm` while chunk j + 1 is computed
  cudaStream_t comm = nullptr;
  cudaEvent_t ev_mm[2] = {}, ev_x[2] = {};
};

namespace {

int32_t tp_fail(turq_tp* tp, int32_t st, const char* msg) {
  if (tp && tp->ctx) {
    try {
      tp->ctx->err = msg;
    } catch (...) {
    }
  }
  return st;
}
int32_t tp_cuda_fail(turq_tp* tp, cudaError_t e, const char* what) {
  char buf[256];
  snprintf(buf, sizeof(buf), "%s: %s", what, cudaGetErrorString(e));
  cudaGetLastError();
  return tp_fail(tp, TURQ_E_CUDA, buf);
}

float* slot0(const turq_tp* tp, int p) { return reinterpret_cast<float*>(tp->peers[p] + turq::TP_HEADER_BYTES); }
unsigned* flags_of(const turq_tp* tp, int p) { return reinterpret_cast<unsigned*>(tp->peers[p]); }
unsigned* counter_of(const turq_tp* tp) { return reinterpret_cast<unsigned*>(tp->region + turq::TP_FLAGS_BYTES); }

void fill_args(const turq_tp* tp, turq::TpArgs& a) {
  for (int p = 0; p < tp->world; p++) {
    a.peer_data[p] = slot0(tp, p);
    a.peer_flags[p] = flags_of(tp, p);
  }
  a.counter = counter_of(tp);
  a.slot_elems = tp->slot_bytes / 4;
  a.rank = tp->rank;
  a.world = tp->world;
  a.wait_cycles = tp->wait_cycles;
  a.status = tp->ctx->dev_status;
}

int grid_for(int64_t work_items, int sm_count) {
  int64_t g = (work_items + turq::TP_THREADS - 1) / turq::TP_THREADS;
  const int cap = sm_count < turq::TP_MAX_BLOCKS ? sm_count : turq::TP_MAX_BLOCKS;
  if (g > cap) g = cap;
  return g < 1 ? 1 : (int)g;
}

int32_t check_ready(turq_tp* tp) {
  if (!tp || !tp->ctx) return TURQ_E_INVALID_ARG;
  if (!tp->connected) return tp_fail(tp, TURQ_E_INVALID_ARG, "the tensor-parallel group is not connected yet (turq_tp_connect)");
  return TURQ_OK;
}

int32_t launch_reduce(turq_tp* tp, int64_t count, int64_t n, const float* bias, float* out, cudaStream_t s) {
  turq::TpArgs a{};
  fill_args(tp, a);
  a.count = count;
  a.n = n > 0 ? n : 1;
  a.bias = bias;
  a.out = out;
  // the same grid on every rank (CTA b pairs with CTA b of the peers): it depends on count only
  // (so does the choice of the two-shot form: size and world only)
  const bool twoshot = tp->world >= 3 && (count & 3) == 0 && (size_t)count * 4 >= tp->twoshot_min_bytes;
  const int grid = twoshot ? grid_for(((count >> 2) + tp->world - 1) / tp->world, turq::TP_MAX_BLOCKS)
                           : grid_for((count + 3) / 4, turq::TP_MAX_BLOCKS);
  cudaError_t e = twoshot ? tp_launch_pdl(turq::tp_allreduce2_kernel, (unsigned)grid, (unsigned)turq::TP_THREADS, s, a)
                          : tp_launch_pdl(turq::tp_allreduce_kernel, (unsigned)grid, (unsigned)turq::TP_THREADS, s, a);
  tp->ctx->launches++;
  if (e != cudaSuccess) return tp_cuda_fail(tp, e, "all-reduce launch");
  return TURQ_OK;
}

// Row-parallel product in chunks of rows: chunk j is computed on the caller's stream into one of
// two result buffers, copied into the slot and exchanged on the group's second stream, while the
// caller's stream goes on with chunk j + 1. The caller's stream rejoins at the end. A result
// buffer is reused after the exchange two chunks earlier has read it; the slot protocol is the
// one of separate calls (stage and exchange of a chunk follow the previous chunk's exchange on
// the same stream).
int32_t rowparallel_chunked(turq_tp* tp, const turq_qtensor* qt, const void* dev_x, int32_t x_dtype, int64_t m, float* dev_y,
                            int32_t mode, const float* dev_bias, cudaStream_t s, int64_t chunk_m) {
  turq_ctx* ctx = tp->ctx;
  const int64_t n = qt->n_rows, k = qt->n_cols;
  const int64_t nchunks = (m + chunk_m - 1) / chunk_m;
  // even chunks in multiples of 64 rows, so that no chunk is a sliver
  int64_t rows = (((m + nchunks - 1) / nchunks + 63) / 64) * 64;
  if (rows > chunk_m) rows = chunk_m;
  const size_t buf_elems = (size_t)rows * (size_t)n;
  int32_t st = turq::api_ensure_tmp(ctx, 2 * buf_elems * 4);
  if (st != TURQ_OK) return st;
  float* bufs[2] = {reinterpret_cast<float*>(ctx->tmp), reinterpret_cast<float*>(ctx->tmp) + buf_elems};
  const size_t x_es = x_dtype == TURQ_BF16 ? 2 : 4;
  cudaError_t e = cudaSuccess;
  int64_t j = 0;
  for (int64_t r0 = 0; r0 < m && e == cudaSuccess; r0 += rows, j++) {
    const int64_t mj = m - r0 < rows ? m - r0 : rows;
    const int slot = (int)(j & 1);
    if (j >= 2) e = cudaStreamWaitEvent(s, tp->ev_x[slot], 0);  // the exchange that read this buffer
    if (e != cudaSuccess) break;
    st = turq_qmatmul(ctx, qt, static_cast<const uint8_t*>(dev_x) + (size_t)r0 * (size_t)k * x_es, x_dtype, mj, bufs[slot], mode, nullptr, s);
    if (st != TURQ_OK) return st;
    e = cudaEventRecord(tp->ev_mm[slot], s);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(tp->comm, tp->ev_mm[slot], 0);
    if (e != cudaSuccess) break;
    const int64_t cnt = mj * n;
    int64_t blocks = (cnt / 4 + 255) / 256;
    if (blocks > 2 * (int64_t)ctx->sm_count) blocks = 2 * (int64_t)ctx->sm_count;
    if (blocks < 1) blocks = 1;
    turq::tp_stage_kernel<<<(unsigned)blocks, 256, 0, tp->comm>>>(bufs[slot], slot0(tp, tp->rank), tp->slot_bytes / 4, counter_of(tp), cnt);
    ctx->launches++;
    e = cudaGetLastError();
    if (e != cudaSuccess) break;
    st = launch_reduce(tp, cnt, n, dev_bias, dev_y + (size_t)r0 * (size_t)n, tp->comm);
    if (st != TURQ_OK) return st;
    e = cudaEventRecord(tp->ev_x[slot], tp->comm);
  }
  // rejoin: the caller's stream continues after the last two exchanges
  if (e == cudaSuccess && j >= 2) e = cudaStreamWaitEvent(s, tp->ev_x[(int)((j - 2) & 1)], 0);
  if (e == cudaSuccess && j >= 1) e = cudaStreamWaitEvent(s, tp->ev_x[(int)((j - 1) & 1)], 0);
  if (e != cudaSuccess) return tp_cuda_fail(tp, e, "chunked row-parallel product");
  return TURQ_OK;
}

}  // namespace

extern "C" {

int32_t turq_tp_create(turq_ctx* ctx, int32_t rank, int32_t world, size_t max_bytes, turq_tp** out) {
  if (!ctx || !out) return TURQ_E_INVALID_ARG;
  *out = nullptr;
  auto bad = [&](int32_t st, const char* m) {
    try { ctx->err = m; } catch (...) {}
    return st;
  };
  if (world < 1 || world > turq::TP_MAX_RANKS || rank < 0 || rank >= world) return bad(TURQ_E_INVALID_ARG, "rank / world out of range (at most 8 ranks)");
  if (max_bytes == 0 || max_bytes > ((size_t)1 << 31)) return bad(TURQ_E_LIMIT, "exchange slot size must be between 1 byte and 2 GiB");
  turq_tp* tp = new (std::nothrow) turq_tp();
  if (!tp) return bad(TURQ_E_INVALID_ARG, "out of host memory");
  tp->ctx = ctx;
  tp->rank = rank;
  tp->world = world;
  tp->slot_bytes = (max_bytes + 255) & ~(size_t)255;
  tp->region_bytes = turq::TP_HEADER_BYTES + 2 * tp->slot_bytes;
  cudaError_t e = cudaSetDevice(ctx->device);
  if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&tp->region), tp->region_bytes);
  if (e == cudaSuccess) e = cudaMemset(tp->region, 0, turq::TP_HEADER_BYTES);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    if (tp->region) cudaFree(tp->region);
    delete tp;
    cudaGetLastError();
    return bad(TURQ_E_CUDA, cudaGetErrorString(e));
  }
  e = cudaStreamCreateWithFlags(&tp->comm, cudaStreamNonBlocking);
  for (int i = 0; i < 2 && e == cudaSuccess; i++) {
    e = cudaEventCreateWithFlags(&tp->ev_mm[i], cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&tp->ev_x[i], cudaEventDisableTiming);
  }
  if (e != cudaSuccess) {
    turq_tp_destroy(tp);
    cudaGetLastError();
    return bad(TURQ_E_CUDA, cudaGetErrorString(e));
  }
  tp->peers[rank] = tp->region;
  if (world == 1) tp->connected = true;
  *out = tp;
  return TURQ_OK;
}

int32_t turq_tp_export(const turq_tp* tp, void* handle_out) {
  if (!tp || !handle_out) return TURQ_E_INVALID_ARG;
  static_assert(sizeof(cudaIpcMemHandle_t) <= TURQ_TP_HANDLE_BYTES, "handle blob too small");
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaSetDevice(tp->ctx->device);
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, tp->region);
  if (e != cudaSuccess) return tp_cuda_fail(const_cast<turq_tp*>(tp), e, "cudaIpcGetMemHandle");
  memset(handle_out, 0, TURQ_TP_HANDLE_BYTES);
  memcpy(handle_out, &h, sizeof(h));
  return TURQ_OK;
}

int32_t turq_tp_connect(turq_tp* tp, const void* handles) {
  if (!tp || !handles) return TURQ_E_INVALID_ARG;
  if (tp->connected) return tp_fail(tp, TURQ_E_INVALID_ARG, "the group is connected already");
  cudaError_t e = cudaSetDevice(tp->ctx->device);
  if (e != cudaSuccess) return tp_cuda_fail(tp, e, "cudaSetDevice");
  for (int p = 0; p < tp->world; p++) {
    if (p == tp->rank) continue;
    cudaIpcMemHandle_t h;
    memcpy(&h, static_cast<const uint8_t*>(handles) + (size_t)p * TURQ_TP_HANDLE_BYTES, sizeof(h));
    void* ptr = nullptr;
    e = cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return tp_cuda_fail(tp, e, "cudaIpcOpenMemHandle (is peer access between the GPUs available?)");
    tp->peers[p] = static_cast<uint8_t*>(ptr);
    tp->opened[p] = true;
  }
  tp->connected = true;
  return TURQ_OK;
}

int32_t turq_tp_connect_loopback(turq_tp* tp) {
  if (!tp) return TURQ_E_INVALID_ARG;
  if (tp->connected) return tp_fail(tp, TURQ_E_INVALID_ARG, "the group is connected already");
  cudaError_t e = cudaSetDevice(tp->ctx->device);
  for (int p = 0; p < tp->world && e == cudaSuccess; p++) {
    if (p == tp->rank) continue;
    e = cudaMalloc(reinterpret_cast<void**>(&tp->peers[p]), tp->region_bytes);
    if (e == cudaSuccess) {
      tp->loopback[p] = true;
      e = cudaMemset(tp->peers[p], 0, tp->region_bytes);
    }
  }
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return tp_cuda_fail(tp, e, "loopback allocation");
  tp->connected = true;
  return TURQ_OK;
}

int32_t turq_tp_loopback_fill(turq_tp* tp, int32_t peer, const float* dev_src, int64_t count, int32_t signal, void* stream) {
  int32_t st = check_ready(tp);
  if (st != TURQ_OK) return st;
  if (peer < 0 || peer >= tp->world || !tp->loopback[peer]) return tp_fail(tp, TURQ_E_INVALID_ARG, "not a loopback stand-in rank");
  if (count < 0 || (size_t)count * 4 > tp->slot_bytes) return tp_fail(tp, TURQ_E_LIMIT, "more elements than an exchange slot holds");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaSetDevice(tp->ctx->device);
  // The stand-in plays the peer's part for the NEXT call: data into the slot of that call and,
  // with `signal`, its "slot complete" flags for every CTA. Needs the current call number.
  unsigned done = 0;
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  if (e == cudaSuccess) e = cudaMemcpy(&done, counter_of(tp), 4, cudaMemcpyDeviceToHost);
  const unsigned seq = done + 1u;
  if (e == cudaSuccess && dev_src && count > 0)
    e = cudaMemcpyAsync(slot0(tp, peer) + ((seq & 1u) ? tp->slot_bytes / 4 : 0), dev_src, (size_t)count * 4, cudaMemcpyDeviceToDevice, s);
  if (e == cudaSuccess && signal) {
    unsigned host_flags[turq::TP_MAX_BLOCKS * turq::TP_MAX_RANKS];
    e = cudaMemcpy(host_flags, flags_of(tp, tp->rank), sizeof(host_flags), cudaMemcpyDeviceToHost);
    // both meeting points of that call (a stand-in that plays a two-shot peer has its reduced
    // slice in the data already)
    // `signal` = how many upcoming calls the stand-in has "arrived" at (1: the next one)
    for (int b = 0; b < turq::TP_MAX_BLOCKS; b++) host_flags[b * turq::TP_MAX_RANKS + peer] = 2u * (done + (unsigned)signal) + 1u;
    if (e == cudaSuccess) e = cudaMemcpy(flags_of(tp, tp->rank), host_flags, sizeof(host_flags), cudaMemcpyHostToDevice);
  }
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  if (e != cudaSuccess) return tp_cuda_fail(tp, e, "loopback fill");
  return TURQ_OK;
}

int32_t turq_tp_set_wait_limit(turq_tp* tp, int64_t cycles) {
  if (!tp || cycles <= 0) return TURQ_E_INVALID_ARG;
  tp->wait_cycles = cycles;
  return TURQ_OK;
}

int32_t turq_tp_set_fuse_limit(turq_tp* tp, int64_t bytes) {
  if (!tp || bytes < 0) return TURQ_E_INVALID_ARG;
  tp->fuse_max_bytes = (size_t)bytes;
  return TURQ_OK;
}

int32_t turq_tp_set_twoshot_limit(turq_tp* tp, int64_t bytes) {
  if (!tp || bytes < 0) return TURQ_E_INVALID_ARG;
  tp->twoshot_min_bytes = (size_t)bytes;
  return TURQ_OK;
}

int32_t turq_tp_set_chunk_rows(turq_tp* tp, int64_t rows) {
  if (!tp || rows < 0) return TURQ_E_INVALID_ARG;
  tp->chunk_rows = rows;
  return TURQ_OK;
}

int32_t turq_tp_reset(turq_tp* tp) {
  if (!tp) return TURQ_E_INVALID_ARG;
  cudaError_t e = cudaSetDevice(tp->ctx->device);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e == cudaSuccess) e = cudaMemset(tp->region, 0, turq::TP_HEADER_BYTES);
  for (int p = 0; p < tp->world && e == cudaSuccess; p++)
    if (tp->loopback[p]) e = cudaMemset(tp->peers[p], 0, turq::TP_HEADER_BYTES);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return tp_cuda_fail(tp, e, "tp reset");
  return TURQ_OK;
}

int32_t turq_tp_destroy(turq_tp* tp) {
  if (!tp) return TURQ_E_INVALID_ARG;
  cudaSetDevice(tp->ctx->device);
  cudaDeviceSynchronize();
  for (int p = 0; p < tp->world; p++) {
    if (tp->opened[p]) cudaIpcCloseMemHandle(tp->peers[p]);
    if (tp->loopback[p]) cudaFree(tp->peers[p]);
  }
  if (tp->region) cudaFree(tp->region);
  for (int i = 0; i < 2; i++) {
    if (tp->ev_mm[i]) cudaEventDestroy(tp->ev_mm[i]);
    if (tp->ev_x[i]) cudaEventDestroy(tp->ev_x[i]);
  }
  if (tp->comm) cudaStreamDestroy(tp->comm);
  cudaGetLastError();
  delete tp;
  return TURQ_OK;
}

int32_t turq_tp_allreduce(turq_tp* tp, const float* dev_in, float* dev_out, int64_t count, void* stream) {
  int32_t st = check_ready(tp);
  if (st != TURQ_OK) return st;
  if (!dev_in || !dev_out) return tp_fail(tp, TURQ_E_INVALID_ARG, "null argument");
  if (count <= 0) return tp_fail(tp, TURQ_E_SHAPE, "count must be positive");
  if ((size_t)count * 4 > tp->slot_bytes) return tp_fail(tp, TURQ_E_LIMIT, "more elements than an exchange slot holds (turq_tp_create max_bytes)");
  if ((uintptr_t)dev_in % 16 != 0 || (uintptr_t)dev_out % 16 != 0) return tp_fail(tp, TURQ_E_ALIGN, "buffers must be 16-byte aligned");
  cudaError_t e = cudaSetDevice(tp->ctx->device);
  if (e != cudaSuccess) return tp_cuda_fail(tp, e, "cudaSetDevice");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int64_t blocks = (count / 4 + 255) / 256;
  if (blocks > 2 * (int64_t)tp->ctx->sm_count) blocks = 2 * (int64_t)tp->ctx->sm_count;
  if (blocks < 1) blocks = 1;
  turq::tp_stage_kernel<<<(unsigned)blocks, 256, 0, s>>>(dev_in, slot0(tp, tp->rank), tp->slot_bytes / 4, counter_of(tp), count);
  tp->ctx->launches++;
  e = cudaGetLastError();
  if (e != cudaSuccess) return tp_cuda_fail(tp, e, "stage launch");
  return launch_reduce(tp, count, 1, nullptr, dev_out, s);
}

int32_t turq_tp_allgather(turq_tp* tp, const float* dev_in, int64_t m, const int64_t* widths, float* dev_out, void* stream) {
  int32_t st = check_ready(tp);
  if (st != TURQ_OK) return st;
  if (!dev_in || !dev_out || !widths) return tp_fail(tp, TURQ_E_INVALID_ARG, "null argument");
  if (m <= 0) return tp_fail(tp, TURQ_E_SHAPE, "m must be positive");
  turq::TpArgs a{};
  fill_args(tp, a);
  int64_t widest = 0;
  a.col0[0] = 0;
  for (int p = 0; p < tp->world; p++) {
    if (widths[p] <= 0) return tp_fail(tp, TURQ_E_SHAPE, "every rank's width must be positive");
    a.col0[p + 1] = a.col0[p] + widths[p];
    if (widths[p] > widest) widest = widths[p];
  }
  if ((size_t)m * (size_t)widest * 4 > tp->slot_bytes) return tp_fail(tp, TURQ_E_LIMIT, "a rank's share exceeds an exchange slot (turq_tp_create max_bytes)");
  if ((uintptr_t)dev_in % 16 != 0 || (uintptr_t)dev_out % 16 != 0) return tp_fail(tp, TURQ_E_ALIGN, "buffers must be 16-byte aligned");
  cudaError_t e = cudaSetDevice(tp->ctx->device);
  if (e != cudaSuccess) return tp_cuda_fail(tp, e, "cudaSetDevice");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t count = m * widths[tp->rank];
  int64_t blocks = (count / 4 + 255) / 256;
  if (blocks > 2 * (int64_t)tp->ctx->sm_count) blocks = 2 * (int64_t)tp->ctx->sm_count;
  if (blocks < 1) blocks = 1;
  turq::tp_stage_kernel<<<(unsigned)blocks, 256, 0, s>>>(dev_in, slot0(tp, tp->rank), tp->slot_bytes / 4, counter_of(tp), count);
  tp->ctx->launches++;
  a.m = m;
  a.n_total = a.col0[tp->world];
  a.out = dev_out;
  // the same grid on every rank: it depends on (world, m) only
  const int grid = grid_for((int64_t)tp->world * m * turq::TP_THREADS, turq::TP_MAX_BLOCKS);
  e = tp_launch_pdl(turq::tp_allgather_kernel, (unsigned)grid, (unsigned)turq::TP_THREADS, s, a);
  tp->ctx->launches++;
  if (e != cudaSuccess) return tp_cuda_fail(tp, e, "all-gather launch");
  return TURQ_OK;
}

int32_t turq_qmatmul_rowparallel(turq_tp* tp, const turq_qtensor* qt, const void* dev_x, int32_t x_dtype, int64_t m,
                                 float* dev_y, int32_t mode, const float* dev_bias, void* stream) {
  int32_t st = check_ready(tp);
  if (st != TURQ_OK) return st;
  turq_ctx* ctx = tp->ctx;
  if (!qt || !dev_x || !dev_y) return tp_fail(tp, TURQ_E_INVALID_ARG, "null argument");
  if (m <= 0 || m > INT32_MAX / 2) return tp_fail(tp, TURQ_E_SHAPE, "m out of range");
  const int64_t count = m * qt->n_rows;
  // Prefill-sized products in the dequantizing modes are cut into chunks of rows: the exchange of
  // a chunk runs on a second stream while the next chunk is computed, and a slot only has to
  // hold one chunk.
  const int32_t mode_resolved = mode == TURQ_MODE_AUTO ? turq::api_auto_mode(ctx, qt->n_rows, qt->n_cols, m) : mode;
  // Off unless turq_tp_set_chunk_rows asks for it: measured at 4 ranks on the cfg5 prefill pass
  // (M = 4096) the uncut product with the two-shot exchange took 113 ms, chunks of 2048 / 1024 / 768
  // rows 116 / 126 / 135 ms - the GEMM's last wave of CTAs gets emptier with every cut.
  int64_t chunk_m = tp->chunk_rows;
  if (chunk_m > 0 && chunk_m < 64) chunk_m = 64;
  while (chunk_m > 64 && (size_t)chunk_m * (size_t)qt->n_rows * 4 > tp->slot_bytes) chunk_m -= 64;
  const bool chunked = chunk_m > 0 && tp->world > 1 && mode_resolved != TURQ_MODE_INT8_ACT && m >= 2 * chunk_m &&
                       (size_t)chunk_m * (size_t)qt->n_rows * 4 <= tp->slot_bytes;
  if (!chunked && (size_t)count * 4 > tp->slot_bytes) return tp_fail(tp, TURQ_E_LIMIT, "m x out-features exceeds an exchange slot (turq_tp_create max_bytes)");
  if ((uintptr_t)dev_y % 16 != 0) return tp_fail(tp, TURQ_E_ALIGN, "dev_y must be 16-byte aligned");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  float* s0 = slot0(tp, tp->rank);
  float* s1 = s0 + tp->slot_bytes / 4;
  float* staged = nullptr;
  if (chunked) return rowparallel_chunked(tp, qt, dev_x, x_dtype, m, dev_y, mode_resolved, dev_bias, s, chunk_m);
  // Small results (decode): the GEMV's last CTA does the exchange - one kernel computes and
  // reduces. Larger ones get the multi-CTA exchange launch.
  turq::TpArgs fuse{};
  fill_args(tp, fuse);
  fuse.count = count;
  fuse.n = qt->n_rows;
  fuse.bias = dev_bias;
  fuse.out = dev_y;
  bool fused = false;
  st = turq::qmatmul_for_exchange(ctx, qt, dev_x, x_dtype, m, s0, s1, counter_of(tp), mode, s, &staged,
                                  (size_t)count * 4 <= tp->fuse_max_bytes ? &fuse : nullptr, &fused);
  if (st != TURQ_OK) return st;
  if (fused) return TURQ_OK;
  if (staged) {
    int64_t blocks = (count / 4 + 255) / 256;
    if (blocks > 2 * (int64_t)ctx->sm_count) blocks = 2 * (int64_t)ctx->sm_count;
    if (blocks < 1) blocks = 1;
    turq::tp_stage_kernel<<<(unsigned)blocks, 256, 0, s>>>(staged, s0, tp->slot_bytes / 4, counter_of(tp), count);
    ctx->launches++;
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return tp_cuda_fail(tp, e, "stage launch");
  }
  return launch_reduce(tp, count, qt->n_rows, dev_bias, dev_y, s);
}

int32_t turq_qmatmul_gather(turq_tp* tp, const turq_qtensor* qt, const void* dev_x, int32_t x_dtype, int64_t m,
                            const int64_t* widths, float* dev_out, int32_t mode, const float* dev_bias, void* stream) {
  int32_t st = check_ready(tp);
  if (st != TURQ_OK) return st;
  turq_ctx* ctx = tp->ctx;
  if (!qt || !dev_x || !dev_out || !widths) return tp_fail(tp, TURQ_E_INVALID_ARG, "null argument");
  if (m <= 0 || m > INT32_MAX / 2) return tp_fail(tp, TURQ_E_SHAPE, "m out of range");
  if (widths[tp->rank] != qt->n_rows) return tp_fail(tp, TURQ_E_SHAPE, "widths[rank] must equal the shard's out-features");
  turq::TpArgs a{};
  fill_args(tp, a);
  int64_t widest = 0;
  a.col0[0] = 0;
  for (int p = 0; p < tp->world; p++) {
    if (widths[p] <= 0) return tp_fail(tp, TURQ_E_SHAPE, "every rank's width must be positive");
    a.col0[p + 1] = a.col0[p] + widths[p];
    if (widths[p] > widest) widest = widths[p];
  }
  if ((size_t)m * (size_t)widest * 4 > tp->slot_bytes) return tp_fail(tp, TURQ_E_LIMIT, "a rank's share exceeds an exchange slot (turq_tp_create max_bytes)");
  if ((uintptr_t)dev_out % 16 != 0) return tp_fail(tp, TURQ_E_ALIGN, "dev_out must be 16-byte aligned");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  float* s0 = slot0(tp, tp->rank);
  float* s1 = s0 + tp->slot_bytes / 4;
  const int64_t count = m * qt->n_rows;
  float* staged = nullptr;
  bool fused = false;
  st = turq::qmatmul_for_exchange(ctx, qt, dev_x, x_dtype, m, s0, s1, counter_of(tp), mode, s, &staged, nullptr, &fused, dev_bias);
  if (st != TURQ_OK) return st;
  if (staged) {
    int64_t blocks = (count / 4 + 255) / 256;
    if (blocks > 2 * (int64_t)ctx->sm_count) blocks = 2 * (int64_t)ctx->sm_count;
    if (blocks < 1) blocks = 1;
    turq::tp_stage_kernel<<<(unsigned)blocks, 256, 0, s>>>(staged, s0, tp->slot_bytes / 4, counter_of(tp), count);
    ctx->launches++;
  }
  a.m = m;
  a.n_total = a.col0[tp->world];
  a.out = dev_out;
  const int grid = grid_for((int64_t)tp->world * m * turq::TP_THREADS, turq::TP_MAX_BLOCKS);
  cudaError_t e = tp_launch_pdl(turq::tp_allgather_kernel, (unsigned)grid, (unsigned)turq::TP_THREADS, s, a);
  ctx->launches++;
  if (e != cudaSuccess) return tp_cuda_fail(tp, e, "gather launch");
  return TURQ_OK;
}

}  // extern "C"
