/*
 * turq - B200 (sm_100a) kernels for GGUF quantized linear layers behind a flat C ABI.
 *
 * This is the drop-in boundary for the one path tur runs through candle:
 *   LinearX::Quantized -> QMatMul::forward          (src/models/layers/linear.rs:19-32)
 *   QVarBuilder::get   -> Arc<QTensor> on a device  (src/weights/gguf_varbuilder.rs:52-94)
 *   QTensor::dequantize                             (src/weights/mod.rs:150,161)
 * A Rust `-sys` crate binds exactly these symbols; candle's names map as noted per entry.
 *
 * Conventions
 *   - every entry returns a turq_status (0 = OK); nothing throws or aborts across the ABI;
 *   - `turq_last_error(ctx)` returns the message of the last failing call on that context;
 *   - pointers named dev_* are CUDA device pointers on the context's device, host_* are
 *     host pointers; `stream` is a cudaStream_t passed as void* (NULL = default stream);
 *   - calls are asynchronous on `stream` unless stated otherwise; the library never frees
 *     caller memory and never falls back to a CPU implementation;
 *   - dtype arguments use the GGUF wire-format type ids (enum turq_dtype).
 */
#ifndef TURQ_H
#define TURQ_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TURQ_VERSION 100 /* major*10000 + minor*100 + patch */

typedef enum {
  TURQ_OK = 0,
  TURQ_E_INVALID_ARG = 1, /* null pointer, bad handle, bad enum value */
  TURQ_E_SHAPE = 2,       /* K not a multiple of the block size, M <= 0, size mismatch */
  TURQ_E_DTYPE = 3,       /* type not supported by this entry */
  TURQ_E_ALIGN = 4,       /* pointer alignment requirement not met */
  TURQ_E_CUDA = 5,        /* a CUDA runtime call or kernel launch failed */
  TURQ_E_NCCL = 6,
  TURQ_E_TIMEOUT = 7,
  TURQ_E_NO_DEVICE = 8, /* no CUDA device: there is no CPU fallback */
  TURQ_E_LIMIT = 9      /* request exceeds a fixed capacity of the entry point */
} turq_status;

/* GGUF tensor type ids (candle: GgmlDType) */
typedef enum {
  TURQ_F32 = 0,
  TURQ_F16 = 1,
  TURQ_Q8_0 = 8,
  TURQ_Q4_K = 12,
  TURQ_Q5_K = 13,
  TURQ_Q6_K = 14,
  TURQ_Q8_K = 15,
  TURQ_BF16 = 30
} turq_dtype;

/* How QMatMul::forward computes.
 *   INT8_ACT    the reference CPU scheme: activation rows are quantized to Q8_0 (Q8_0 weights)
 *               or Q8_K (K-quant weights) and block dots run in integers.
 *   EXACT_F32   weights are dequantized on the fly to their exact f32 values, f32 FMA.
 *   TENSOR_CORE tcgen05 f16 MMA with f32 accumulation (prefill-sized M).
 *   AUTO        INT8_ACT for M <= 16, TENSOR_CORE above (when in-features are a multiple of 64).
 *               The two schemes differ by the rounding of the activations to int8 (5-8e-3
 *               relative), so under the default policy a row's result changes when its batch
 *               grows from 16 to 17 rows. A host that needs a token's result to be independent
 *               of the batch or chunk it arrives in (tur's tests/pipeline_integration.rs:275-369
 *               do) pins one scheme for all row counts with turq_ctx_set_auto_policy or passes
 *               an explicit mode. Within one mode results never depend on the other rows. */
typedef enum {
  TURQ_MODE_AUTO = 0,
  TURQ_MODE_INT8_ACT = 1,
  TURQ_MODE_EXACT_F32 = 2,
  TURQ_MODE_TENSOR_CORE = 3
} turq_mode;

typedef struct turq_ctx turq_ctx;         /* one device + its scratch memory */
typedef struct turq_qtensor turq_qtensor; /* immutable quantized weight on the device */

int32_t turq_version(void);
/* How this build quantizes activations to Q8_K (compile-time switches TURQ_Q8K_*): the divisor
 * (127 or 128) | 0x100 when the scale is -divisor / (signed element of largest magnitude)
 * | 0x200 when ties round to even. Default 0x180: candle-core's published quantizer
 * (-128 / max, ties away from zero, clamp at 127). */
int32_t turq_q8k_variant(void);
const char* turq_status_string(int32_t status);

/* Block geometry of the wire format (candle: GgmlDType::block_size / type_size). */
int32_t turq_block_elems(int32_t dtype);
int32_t turq_block_bytes(int32_t dtype);
/* bytes of one row of k elements, 0 if k is not a whole number of blocks */
size_t turq_row_bytes(int32_t dtype, int64_t k);

/* Context: binds to CUDA device `device`. Fails with TURQ_E_NO_DEVICE when none exists. */
int32_t turq_ctx_create(int32_t device, turq_ctx** out);
int32_t turq_ctx_destroy(turq_ctx* ctx);
const char* turq_last_error(const turq_ctx* ctx);
/* The context owns scratch memory that grows on demand: a call with more rows (or a wider weight)
 * than any before it synchronizes the device, frees the old buffer and allocates a larger one.
 * That is not allowed during stream capture and stalls a serving thread, so a host that knows
 * its largest call reserves once, up front: afterwards no call with m <= max_m rows, in-features
 * <= max_k and out-features <= max_n allocates (turq_qmatmul, _multi, _host, _multi_host). */
int32_t turq_ctx_reserve(turq_ctx* ctx, int64_t max_m, int64_t max_k, int64_t max_n);
/* What TURQ_MODE_AUTO means on this context: TURQ_MODE_AUTO (default) = by row count as described
 * above; INT8_ACT, EXACT_F32 or TENSOR_CORE = that scheme for every row count (TENSOR_CORE still
 * falls back to INT8_ACT for in-features that are not a multiple of 64). */
int32_t turq_ctx_set_auto_policy(turq_ctx* ctx, int32_t mode);
/* Kernels never trap: a device-side wait that runs out (mbarrier, cross-CTA hand-over) stops
 * the kernel and records a status word. This call synchronizes `stream`, returns TURQ_OK or
 * the recorded status (TURQ_E_TIMEOUT) and clears it. */
int32_t turq_ctx_poll_status(turq_ctx* ctx, void* stream);
/* Number of kernels this context has launched so far (bookkeeping for benchmarks). */
int64_t turq_ctx_launch_count(const turq_ctx* ctx);

/* QTensor from GGUF wire-format blocks in host memory: uploads and converts to the device
 * layout. Replaces gguf_file::Content::tensor(reader, name, device)
 * (src/weights/gguf_varbuilder.rs:73) / QTensor::new. Synchronous. */
int32_t turq_qtensor_from_host(turq_ctx* ctx, int32_t dtype, int64_t n_rows, int64_t n_cols,
                               const void* host_blocks, size_t nbytes, turq_qtensor** out);
/* Same, blocks already in device memory (copied; the caller keeps ownership of dev_blocks). */
int32_t turq_qtensor_from_device(turq_ctx* ctx, int32_t dtype, int64_t n_rows, int64_t n_cols,
                                 const void* dev_blocks, size_t nbytes, void* stream,
                                 turq_qtensor** out);
/* Tensor-parallel shards (no counterpart in the reference, which is single-device):
 * rows [row0, row0+n) for column-parallel linears, columns [col0, col0+n) for row-parallel
 * ones. row0 must be a multiple of 16, col0 and n (columns) multiples of the block size.
 * The result owns its own memory. */
int32_t turq_qtensor_slice_rows(turq_ctx* ctx, const turq_qtensor* src, int64_t row0, int64_t n,
                                turq_qtensor** out);
int32_t turq_qtensor_slice_cols(turq_ctx* ctx, const turq_qtensor* src, int64_t col0, int64_t n,
                                turq_qtensor** out);
int32_t turq_qtensor_free(turq_qtensor* qt);
/* candle: QTensor::{dtype, shape, storage_size_in_bytes}; any out pointer may be NULL */
int32_t turq_qtensor_info(const turq_qtensor* qt, int32_t* dtype, int64_t* n_rows,
                          int64_t* n_cols, size_t* wire_bytes);

/* QTensor::dequantize (src/weights/mod.rs:150): dev_out is [n_rows, n_cols] row-major of
 * out_dtype (F32, F16 or BF16). F32 output is bit-exact with the GGUF definition. */
int32_t turq_dequantize(turq_ctx* ctx, const turq_qtensor* qt, int32_t out_dtype, void* dev_out,
                        void* stream);

/* Embedding lookup on a table that stays quantized (src/models/layers/mod.rs:30-48 dequantizes
 * the whole token_embd tensor and indexes it; qwen3.rs:691-700): dev_out[i, :] =
 * dequantize(row dev_ids[i]), [n_ids, n_cols] row-major of out_dtype, the same bits as
 * turq_dequantize gives for that row. dev_ids are int32 on the device. An id outside the table
 * gives a row of zeros and turq_ctx_poll_status then reports TURQ_E_INVALID_ARG. */
int32_t turq_embedding(turq_ctx* ctx, const turq_qtensor* qt, const int32_t* dev_ids, int64_t n_ids,
                       int32_t out_dtype, void* dev_out, void* stream);

/* QTensor::quantize (candle-core; tur only loads quantized files, src/weights/gguf_varbuilder.rs:73,
 * but the benchmark configurations quantize synthetic weights with it): f32 rows
 * [n_rows, n_cols] -> wire-format blocks of dtype (Q8_0, Q4_K, Q5_K or Q6_K), n_rows rows of
 * turq_row_bytes(dtype, n_cols) bytes, ready for turq_qtensor_from_device. Q8_0 is the GGML
 * reference quantizer; the K-quant search is this library's own (valid blocks, not candle's
 * bytes): min/max start plus least-squares refits per sub-block. dev_x 16-byte aligned. */
int32_t turq_quantize_weights(turq_ctx* ctx, int32_t dtype, const float* dev_x, int64_t n_rows,
                              int64_t n_cols, void* dev_blocks, void* stream);

/* Activation quantization used inside QMatMul::forward (entered at
 * src/models/layers/linear.rs:24): x [m, k] (F32 or BF16) -> wire-format Q8_0 or Q8_K blocks,
 * m rows of turq_row_bytes(fmt, k) bytes. */
int32_t turq_quantize_act(turq_ctx* ctx, int32_t fmt, const void* dev_x, int32_t x_dtype,
                          int64_t m, int64_t k, void* dev_blocks, void* stream);

/* QMatMul::forward (src/models/layers/linear.rs:24) with the optional bias add of
 * LinearX::forward (linear.rs:25-28): y[m, n] = sum_k x[m, k] * W[n, k] (+ bias[n]).
 * x is [m, n_cols] row-major F32 or BF16, y is [m, n_rows] row-major F32,
 * dev_bias is NULL or n_rows f32 values. */
int32_t turq_qmatmul(turq_ctx* ctx, const turq_qtensor* qt, const void* dev_x, int32_t x_dtype,
                     int64_t m, float* dev_y, int32_t mode, const float* dev_bias, void* stream);

/* Several linears that read the same x (attn_q|k|v: src/models/qwen3.rs:272-274; ffn_gate|up:
 * qwen3.rs:162-166) in one call: count <= 4 weights with the same in-feature count, y[i] is
 * [m, rows of qts[i]], biases may be NULL or hold NULL entries. In the integer scheme, weights
 * of the same type run as ONE kernel launch over their concatenated rows, and so do Q4_K or
 * Q5_K weights together with Q6_K ones (the K-quant mixes keep attn_v in Q6_K) up to m = 8;
 * other combinations get one launch per type, other modes one call per weight. Results equal
 * those of separate turq_qmatmul calls up to the f32 summation order. */
int32_t turq_qmatmul_multi(turq_ctx* ctx, int32_t count, const turq_qtensor* const* qts,
                           const void* dev_x, int32_t x_dtype, int64_t m, float* const* dev_ys,
                           int32_t mode, const float* const* dev_biases, void* stream);

/* The same call for a caller that keeps activations in host memory, as tur does today
 * (Device::Cpu everywhere: tests/common.rs:5): x in, y out, one synchronize; x and y are f32.
 * With page-locked buffers (cudaHostAlloc / cudaHostRegister), 16-byte aligned x, no bias, the
 * integer scheme and at most 2 MiB per output, nothing is copied: one small launch reads x from
 * the caller's memory and the GEMV writes y into it. Otherwise x is copied in and y copied
 * back. Runs on the context's own stream. */
int32_t turq_qmatmul_host(turq_ctx* ctx, const turq_qtensor* qt, const float* host_x, int64_t m,
                          float* host_y, int32_t mode, const float* host_bias);
/* turq_qmatmul_multi with host buffers: attn_q|k|v or ffn_gate|up read one host x and cost one
 * round trip instead of three or two. host_ys[i] is [m, rows of qts[i]]. */
int32_t turq_qmatmul_multi_host(turq_ctx* ctx, int32_t count, const turq_qtensor* const* qts,
                                const float* host_x, int64_t m, float* const* host_ys, int32_t mode,
                                const float* const* host_biases);

/* A host-buffer call bound to its buffers, for a decoder that calls the same linears with the
 * same page-locked x / y buffers token after token (it rewrites x in place between runs):
 * create resolves the buffers' device aliases, allocates the call's own activation scratch and
 * records its launches once; run is then one graph launch and one wait (on a completion word the
 * call's last kernel stores into mapped host memory; bounded, then a stream synchronize), with the results
 * of turq_qmatmul_multi_host(..., TURQ_MODE_INT8_ACT, no biases). 1 <= m <= 64. The buffers
 * and the weights must stay alive until destroy; runs of calls of one context are serialised by
 * the caller (they share the context's stream and hand-over workspace). Fails with
 * TURQ_E_INVALID_ARG when a buffer is not page-locked: use turq_qmatmul_multi_host then. */
typedef struct turq_host_call turq_host_call;
int32_t turq_host_call_create(turq_ctx* ctx, int32_t count, const turq_qtensor* const* qts, const float* host_x,
                              int64_t m, float* const* host_ys, turq_host_call** out);
int32_t turq_host_call_run(turq_host_call* call);
int32_t turq_host_call_destroy(turq_host_call* call);

/* Integer-scheme QMatMul for hosts that must not allocate device memory during a call
 * (a process whose memory pool already owns the GPU, a plugin inside a foreign runtime).
 * No counterpart in the reference. Same arguments and results as turq_qmatmul with
 * TURQ_MODE_INT8_ACT, but the quantized activation planes live in a fixed buffer inside the
 * library image (TURQ_STATIC_SCRATCH_BYTES on every GPU that loads the library) instead of
 * the context's growable scratch: the call performs no cudaMalloc/cudaFree. The tail of the
 * buffer is the GEMV's hand-over workspace (about 1.2 MB on a 148-SM GPU), so the planes of one
 * call (about m * k * 1.2 bytes) may use the remaining ~2.8 MiB; larger requests fail with
 * TURQ_E_LIMIT and the message gives both figures. All calls on a GPU
 * share that buffer, so calls that can overlap on the GPU (different streams) race and must
 * be ordered by the caller. The first call on each device looks up the buffer's device
 * address; make that call before starting any stream capture. */
#define TURQ_STATIC_SCRATCH_BYTES (4 << 20)
int32_t turq_qmatmul_static(turq_ctx* ctx, const turq_qtensor* qt, const void* dev_x,
                            int32_t x_dtype, int64_t m, float* dev_y, const float* dev_bias,
                            void* stream);

/* ---- Fused neighbours of the linears

 * The MLP's first half (src/models/qwen3.rs:160-166: x.apply(gate_proj).apply(act_fn) *
 * x.apply(up_proj)) as one call: dev_out[m, n] = silu(x . Wg^T) * (x . Wu^T), silu(v) =
 * v / (1 + exp(-v)). In the integer scheme, for weights of one type, this is ONE kernel launch
 * over the interleaved row-tiles of both weights whose epilogue applies SiLU and the product;
 * the two [m, n] intermediates are never written. Other cases compute both products into
 * context memory and finish with an elementwise launch. */
int32_t turq_qmatmul_swiglu(turq_ctx* ctx, const turq_qtensor* gate, const turq_qtensor* up, const void* dev_x,
                            int32_t x_dtype, int64_t m, float* dev_out, int32_t mode, void* stream);

/* RMSNorm feeding linears (src/models/qwen3.rs:633-638: ln1 -> attn_q|k|v, ln2 -> ffn_gate|up;
 * candle_nn::RmsNorm behind src/models/layers/norm.rs:25-41): h = x / sqrt(mean(x^2) + eps) *
 * weight per row in f32, then turq_qmatmul_multi on h. One prologue launch normalises and writes
 * the quantized activation planes the GEMV reads; h itself is only written when dev_h_out (f32
 * [m, k]) is given. dev_norm_weight holds k f32 values. */
int32_t turq_rmsnorm_qmatmul_multi(turq_ctx* ctx, int32_t count, const turq_qtensor* const* qts, const void* dev_x,
                                   int32_t x_dtype, int64_t m, const float* dev_norm_weight, float eps,
                                   float* dev_h_out, float* const* dev_ys, int32_t mode,
                                   const float* const* dev_biases, void* stream);

/* The k largest values of every row with their ids, best first, equal values by lower id (what a
 * sequential arg-max scan returns; NaN ranks lowest). dev_vals is [m, n]; ids are the positions
 * plus id_offset, or dev_ids[m, n] when given (merging candidates of several shards). k <= 64.
 * Rows with fewer than k candidates are padded with (-inf, INT32_MAX). */
int32_t turq_topk(turq_ctx* ctx, const float* dev_vals, const int32_t* dev_ids, int64_t m, int64_t n, int32_t k,
                  int32_t id_offset, float* dev_out_vals, int32_t* dev_out_ids, void* stream);
/* lm_head followed by sampling's first step (src/backend/engine.rs:528-529 single request,
 * :810-824 batched: logits of the last position -> LogitsProcessor::sample, tokenizer.rs:9-29):
 * the head's product and the k best (logit, token id) pairs per row in one call; greedy decoding
 * is k = 1. The logits stay in context memory unless dev_logits ([m, n_rows] f32) is given.
 * id_offset is the first vocabulary row of a sharded head. */
int32_t turq_lm_head_topk(turq_ctx* ctx, const turq_qtensor* qt, const void* dev_x, int32_t x_dtype, int64_t m,
                          int32_t k, int32_t id_offset, float* dev_out_vals, int32_t* dev_out_ids,
                          float* dev_logits, int32_t mode, void* stream);

/* ---- Tensor parallelism inside one node (no counterpart in the reference, which is
 * single-device: src/models/layers/norm.rs:50 passes Shard::default() everywhere).
 *
 * One process per GPU. Every rank creates a group handle, exports an opaque blob, the host
 * exchanges the blobs by whatever channel it has (the ranks' process group, a pipe, a file) and
 * hands all of them, in rank order, to turq_tp_connect. After that the row-parallel linears
 * (attn_output, ffn_down: each rank holds a range of input columns) and the gathers behind
 * column-parallel ones (the vocabulary-sharded head) exchange their data with kernels of this
 * library over peer memory (NVLink): plain peer loads in rank order, so sums are deterministic,
 * and no NCCL call, so a whole sharded decode pass can be captured in one CUDA graph.
 *
 * All ranks must issue the same sequence of group calls with the same sizes. A peer that does
 * not arrive within the wait limit makes the kernel give up: the exchange is skipped, the
 * context's status word becomes TURQ_E_TIMEOUT (turq_ctx_poll_status) and the group is out of
 * step until every rank has called turq_tp_reset. max_bytes is the largest m * n * 4 of any
 * exchanged tensor (per rank for gathers); the group holds twice that on the device. */
typedef struct turq_tp turq_tp;
#define TURQ_TP_HANDLE_BYTES 64
int32_t turq_tp_create(turq_ctx* ctx, int32_t rank, int32_t world, size_t max_bytes, turq_tp** out);
int32_t turq_tp_export(const turq_tp* tp, void* handle_out /* TURQ_TP_HANDLE_BYTES */);
int32_t turq_tp_connect(turq_tp* tp, const void* handles /* world * TURQ_TP_HANDLE_BYTES, rank order */);
int32_t turq_tp_destroy(turq_tp* tp);
/* Upper bound of every device-side wait for a peer, in SM clock cycles (default 2e9, about 1 s). */
int32_t turq_tp_set_wait_limit(turq_tp* tp, int64_t cycles);
/* Largest result (m * n * 4 bytes) turq_qmatmul_rowparallel exchanges inside the matmul kernel
 * itself (default 64 KB); 0 = always use the separate exchange launch. Same value on every rank. */
int32_t turq_tp_set_fuse_limit(turq_tp* tp, int64_t bytes);
/* Smallest result (bytes) that takes the two-shot exchange on three or more ranks: every rank
 * reduces one slice, then copies the others (default 4 MB). Same value on every rank. */
int32_t turq_tp_set_twoshot_limit(turq_tp* tp, int64_t bytes);
/* Rows per chunk of a prefill-sized turq_qmatmul_rowparallel in the dequantizing modes: the
 * exchange of a chunk then runs on a second stream while the next chunk is computed, and an
 * exchange slot only has to hold one chunk (0 = default: the product is not cut; products of
 * fewer than two chunks never are). Same value on every rank. */
int32_t turq_tp_set_chunk_rows(turq_tp* tp, int64_t rows);
/* Clears this rank's flags and call counter. Collective in effect: call it on every rank, with
 * no group call in flight (the host synchronizes the ranks around it). */
int32_t turq_tp_reset(turq_tp* tp);
/* dev_out[i] = sum over ranks of dev_in[i], i < count, added in rank order on every rank. */
int32_t turq_tp_allreduce(turq_tp* tp, const float* dev_in, float* dev_out, int64_t count, void* stream);
/* dev_out[r, col0(p) + j] = rank p's dev_in[r, j]: rank p contributes [m, widths[p]], the result
 * is [m, sum(widths)] on every rank. */
int32_t turq_tp_allgather(turq_tp* tp, const float* dev_in, int64_t m, const int64_t* widths, float* dev_out,
                          void* stream);
/* Row-parallel LinearX::forward: qt holds this rank's range of input columns, dev_x the matching
 * activation columns [m, n_cols of the shard]; dev_y [m, n_rows] receives the sum over the ranks
 * (+ bias) on every rank. In the integer scheme the GEMV's epilogue writes its partial result
 * straight into the exchange memory. For results up to 64 KB (decode) the CTAs of that launch
 * that finish last then signal the peers, wait and add: compute and all-reduce are ONE kernel. Larger results get a multi-CTA exchange launch behind the matmul. */
int32_t turq_qmatmul_rowparallel(turq_tp* tp, const turq_qtensor* qt, const void* dev_x, int32_t x_dtype,
                                 int64_t m, float* dev_y, int32_t mode, const float* dev_bias, void* stream);
/* Column-parallel LinearX::forward with gathered output (the vocabulary-sharded head): qt holds
 * this rank's rows, dev_x the full activations; dev_out [m, sum(widths)] receives every rank's
 * columns on every rank, widths[p] = out-features of rank p's shard. The product lands straight
 * in the exchange memory. dev_bias: this shard's bias rows or NULL. */
int32_t turq_qmatmul_gather(turq_tp* tp, const turq_qtensor* qt, const void* dev_x, int32_t x_dtype, int64_t m,
                            const int64_t* widths, float* dev_out, int32_t mode, const float* dev_bias,
                            void* stream);
/* Test support on a single GPU: connects the group to local stand-ins for the other ranks, which
 * never signal by themselves (a call then runs into its wait limit), and lets the host play a
 * peer's part for the next call: its data (count floats, may be NULL / 0) and, with signal != 0,
 * its "ready" flags (signal = k: the stand-in has arrived at the next k calls). */
int32_t turq_tp_connect_loopback(turq_tp* tp);
int32_t turq_tp_loopback_fill(turq_tp* tp, int32_t peer, const float* dev_src, int64_t count, int32_t signal,
                              void* stream);

#ifdef __cplusplus
}
#endif
#endif
