/*
 * CPU oracle for the GGUF quantized-linear path (TEST INFRASTRUCTURE, not product code).
 *
 * A plain-C restatement of the arithmetic that tur reaches through
 * candle_core::quantized::{QTensor::dequantize, QMatMul::forward}
 * (call sites: src/models/layers/linear.rs:24,66,69; src/weights/mod.rs:150,161).
 * The implementation lives in crates.io candle-core 0.10.2 (Cargo.lock:316-320), which is
 * not vendored in the reference tree, so this file restates the published GGUF/GGML block
 * formats and the CPU "quantize the activation row, integer block dot, f32 scale" scheme.
 *
 * Pinning status:
 *   - dequantize Q8_0/Q4_K/Q5_K/Q6_K and quantize Q8_0: pinned bit-exact against the
 *     independent numpy codec of the `gguf` 0.19.0 package (golden vectors in tests/golden).
 *   - Q8_K activation quantizer, K-quant weight quantizers, vec_dot summation order:
 *     PARITY UNPINNED against candle 0.10.2 (no source, no toolchain). The Q8_K quantizer
 *     restates candle-core's published one (iscale = -128/max, ties away from zero, clamp
 *     127); divisor, scale sign and rounding are compile-time switches (TQO_Q8K_*).
 *
 * Only tests, the smoke check and the benchmark's CPU-baseline leg may link or call this.
 */
#ifndef TURQ_ORACLE_H
#define TURQ_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* GGUF wire-format type ids (same numbering as the GGUF tensor-info `type` field). */
enum {
  TQO_F32 = 0,
  TQO_F16 = 1,
  TQO_Q8_0 = 8,
  TQO_Q4_K = 12,
  TQO_Q5_K = 13,
  TQO_Q6_K = 14,
  TQO_Q8_K = 15,
  TQO_BF16 = 30
};

/* elements per block / bytes per block; 0 for an unknown type */
int tqo_block_elems(int dtype);
int tqo_block_bytes(int dtype);
/* bytes of one row of k elements; 0 if k is not a multiple of the block size */
size_t tqo_row_bytes(int dtype, int64_t k);

float tqo_f16_to_f32(uint16_t h);
uint16_t tqo_f32_to_f16(float f);
float tqo_bf16_to_f32(uint16_t h);
uint16_t tqo_f32_to_bf16(float f);

/* GGUF blocks -> f32, nrows rows of k elements each. Returns 0 on success. */
int tqo_dequantize(int dtype, const void* blocks, float* out, int64_t nrows, int64_t k);

/* f32 -> GGUF blocks (Q8_0, Q4_K, Q5_K, Q6_K weight quantizers; Q8_K activation quantizer). */
int tqo_quantize(int dtype, const float* x, void* blocks, int64_t nrows, int64_t k);

/* One block-row dot product in the CPU scheme: weight row (dtype) . activation row
 * (Q8_0 blocks for Q8_0 weights, Q8_K blocks for K-quant weights). */
float tqo_vec_dot(int dtype, const void* wrow, const void* arow, int64_t k);

/* y[m,n] = sum_k x[m,k] * W[n,k], CPU quantized scheme (activation rows quantized first).
 * nthreads <= 0 uses all OpenMP threads. */
int tqo_qmatmul(int dtype, const void* w, int64_t n, int64_t k, const float* x, int64_t m,
                float* y, int nthreads);

/* y = x . dequantize(W)^T with f64 accumulation (the "f32 dequantize-then-matmul" oracle). */
int tqo_matmul_f64(int dtype, const void* w, int64_t n, int64_t k, const float* x, int64_t m,
                   float* y, int nthreads);

int tqo_num_threads(void);
/* Q8_K quantizer build switches: divisor | 0x100 (negative-scale convention) | 0x200 (ties to even) */
int tqo_q8k_variant(void);

#ifdef __cplusplus
}
#endif
#endif
