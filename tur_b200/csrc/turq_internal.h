// Internal declarations shared by the kernel translation units and the C-ABI layer.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "layout.h"

#include <atomic>
#include <cstdlib>

namespace turq {

// Facts about the current CUDA device, looked up once per device (safe from any thread).
int device_sm_count();
int device_smem_optin();
// Q8_K quantizer switches of this build: divisor | 0x100 (negative scale) | 0x200 (ties to even)
int q8k_variant();

// Tuning knobs read from the environment exist only in -DTURQ_TUNING builds: several of them
// change how a sum is split (hence its last bits), which a shipped library must not allow.
inline int tuning_env(const char* name, int dflt) {
#ifdef TURQ_TUNING
  const char* v = getenv(name);
  return v ? atoi(v) : dflt;
#else
  (void)name;
  return dflt;
#endif
}

// "cudaFuncSetAttribute was applied on device d" for one kernel instantiation: a bit per
// device, set after the call succeeded (the call is idempotent, so a race only repeats it).
struct PerDeviceOnce {
  std::atomic<unsigned long long> mask{0};
  bool done(int dev) const { return dev >= 0 && dev < 64 && ((mask.load(std::memory_order_acquire) >> dev) & 1ull); }
  void set(int dev) { if (dev >= 0 && dev < 64) mask.fetch_or(1ull << dev, std::memory_order_release); }
};

struct ActPackPlan {
  size_t off_qs, off_dsc, off_bs16, off_bs32, total;
};
ActPackPlan plan_act_pack(int fmt, int64_t m, int64_t k);

// wire -> device tiles. n_rows may be any positive value; rows are padded to 16.
cudaError_t launch_repack(int dtype, const uint8_t* dev_wire, uint8_t* dev_tiles, int64_t n_rows,
                          int64_t k, cudaStream_t s);
// device tiles -> row-major [n_rows, k]
cudaError_t launch_dequant(int dtype, const uint8_t* dev_tiles, void* dev_out, int out_dtype,
                           int64_t n_rows, int64_t k, cudaStream_t s);
// out[i, :] = dequantize(row dev_ids[i]) for an embedding table kept quantized; ids outside the
// table give zero rows and raise the status word (TURQ_E_INVALID_ARG).
cudaError_t launch_gather_rows(int dtype, const uint8_t* dev_tiles, const int32_t* dev_ids, void* dev_out, int out_dtype,
                               int64_t n_rows, int64_t n_ids, int64_t k, int* status, cudaStream_t s);
// copy K-tile range [kt0, kt0+nkt) of every row-tile into a new tiled tensor
cudaError_t launch_slice_cols(int dtype, const uint8_t* src_tiles, uint8_t* dst_tiles,
                              int64_t row_tiles, int64_t src_ktiles, int64_t kt0, int64_t nkt,
                              cudaStream_t s);

// activations -> wire-format Q8_0 / Q8_K blocks
// f32 rows -> GGUF wire blocks of a weight type (Q8_0, Q4_K, Q5_K, Q6_K); x 16-byte aligned.
cudaError_t launch_quantize_weights(int dtype, const float* x, int64_t n_rows, int64_t k, uint8_t* wire, cudaStream_t s);
cudaError_t launch_quantize_act_wire(int fmt, const void* x, int x_dtype, int64_t m, int64_t k,
                                     void* blocks, cudaStream_t s);
// activations -> ActPack planes at `scratch` (laid out by plan_act_pack)
cudaError_t launch_quantize_act_pack(int fmt, const void* x, int x_dtype, int64_t m, int64_t k,
                                     uint8_t* scratch, cudaStream_t s);

// y[m, n] = quantize(x) . W^T in the integer scheme (gemv_stream.cu). Quantizes the
// activations inside the kernel when they are small, else into `act_scratch` (which must hold
// plan_act_pack(fmt, m, k).total bytes) with a preceding launch. `workspace` holds
// gemv_workspace_bytes(sm_count) bytes, zero-initialised once; `status` is a device int.
size_t gemv_workspace_bytes(int sms);
size_t gemv_workspace_flags_offset(int sms);  // the ready flags inside the workspace: the only
size_t gemv_workspace_flags_bytes(int sms);   // part that has to read zero when a launch starts
bool gemv_int8_fuses_act(int dtype, int64_t m, int64_t k);
cudaError_t launch_gemv_int8(int dtype, const uint8_t* tiles, int64_t n_rows, int64_t k, const void* x,
                             int x_dtype, uint8_t* act_scratch, int64_t m, float* y, const float* bias,
                             uint8_t* workspace, int* status, int sm_count, cudaStream_t s, int* launches);
// The same for several weights of one in-feature count that share x: one launch over the
// concatenated rows (q|k|v, gate|up) per weight type - and a single one for Q4_K or Q5_K parts
// beside Q6_K parts at up to 8 rows - each part with its own output and bias. x_remote: x is
// mapped host memory; it is then read exactly once, by the quantization launch. planes_ready: the
// caller's own prologue launch already wrote the quantized planes of these rows to act_scratch.
struct TpArgs;  // tp_exchange.cuh: xchg != nullptr (one part, m <= 32) makes the launch's last CTA run
                // the tensor-parallel all-reduce of the result itself
struct GemvPart {
  const uint8_t* tiles;
  int64_t n_rows;
  float* y;
  const float* bias;
  int dtype;  // TQ_* of this part's tiles; 0 = the launch's dtype argument
  float* y_alt = nullptr;  // with y_toggle: the output buffer to use when (*y_toggle + 1) is odd
};
cudaError_t launch_gemv_int8_multi(int dtype, const GemvPart* parts, int nparts, int64_t k, const void* x,
                                   int x_dtype, uint8_t* act_scratch, int64_t m, uint8_t* workspace, int* status,
                                   int sm_count, cudaStream_t s, int* launches, bool x_remote = false,
                                   const unsigned* y_toggle = nullptr, bool planes_ready = false,
                                   const struct TpArgs* xchg = nullptr);
// out[m, n] = silu(x . Wg^T) * (x . Wu^T) as ONE integer-scheme launch over the row-tiles of both
// weights interleaved (same type and shape). cudaErrorNotSupported = not applicable, nothing launched.
cudaError_t launch_gemv_int8_swiglu(int dtype, const uint8_t* gate_tiles, const uint8_t* up_tiles, int64_t n_rows, int64_t k,
                                    const void* x, int x_dtype, uint8_t* act_scratch, int64_t m, float* out, uint8_t* workspace,
                                    int* status, int sm_count, cudaStream_t s, int* launches);
// y[m, n] = x . dequant(W)^T with f32 FMAs on exact f32 weights.
cudaError_t launch_gemv_f32(int dtype, const uint8_t* tiles, int64_t n_rows, int64_t k,
                            const void* x, int x_dtype, int64_t m, float* y, const float* bias,
                            int sm_count, cudaStream_t s, int* launches);

// Tensor-core GEMM (tcgen05): x [m, k] -> f16 operand in scratch, then the fused
// dequantize + MMA kernel. scratch must hold gemm_tc_scratch_bytes(m, k, n_rows, sm_count).
// x_prepared: the f16 operand of this x (same m, k) is already in scratch from a preceding call.
// y_toggle / y_alt: the result goes to y_alt instead of y when *y_toggle + 1 is odd (read on the
// device after the preceding kernels have completed: the exchange slots of tp.cu).
size_t gemm_tc_scratch_bytes(int64_t m, int64_t k, int64_t n_rows, int sm_count);
cudaError_t launch_gemm_tc(int dtype, const uint8_t* tiles, int64_t n_rows, int64_t k,
                           const void* x, int x_dtype, int64_t m, float* y, const float* bias,
                           uint8_t* scratch, int sm_count, cudaStream_t s, int* launches,
                           int* dev_status_word, bool x_prepared = false, const unsigned* y_toggle = nullptr,
                           float* y_alt = nullptr);

// QMatMul (no bias) whose result has to land in one of two buffers picked on the device: s1 when
// (*toggle + 1) is odd, else s0 (the exchange slots of tp.cu). In the integer scheme the GEMV's
// epilogue writes there itself and *staged comes back null; the other schemes compute into
// context memory, returned in *staged, which the caller still has to copy into the slot. With
// `fuse` (the exchange's arguments) an integer-scheme launch of at most 32 rows performs the
// exchange in its last CTA and *fused comes back true: no exchange launch is needed then.
// local_bias is added by the matmul itself (column-parallel shards own their bias rows).
}  // namespace turq
struct turq_ctx;
struct turq_qtensor;
namespace turq {
int32_t api_fail(turq_ctx* ctx, int32_t st, const char* msg);
int32_t api_cuda_fail(turq_ctx* ctx, cudaError_t e, const char* what);
int32_t api_ensure_scratch(turq_ctx* ctx, size_t bytes);  // the context's growable activation scratch
int32_t api_ensure_tmp(turq_ctx* ctx, size_t bytes);      // the context's growable result staging
int32_t api_auto_mode(const turq_ctx* ctx, int64_t n_rows, int64_t n_cols, int64_t m);
int32_t qmatmul_for_exchange(turq_ctx* ctx, const turq_qtensor* qt, const void* dev_x, int32_t x_dtype, int64_t m, float* s0,
                             float* s1, const unsigned* toggle, int32_t mode, cudaStream_t s, float** staged,
                             const TpArgs* fuse, bool* fused, const float* local_bias = nullptr);

}  // namespace turq
