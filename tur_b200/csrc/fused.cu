// Fused neighbours of the quantized linears (what tur does between and after them):
//   * ffn_gate | ffn_up -> silu(g) * u   (src/models/qwen3.rs:160-166: x.apply(gate).apply(act) *
//     x.apply(up)): one interleaved GEMV launch whose epilogue applies SiLU and the product, so
//     the two [m, inter] intermediates are never written;
//   * RMSNorm -> activation quantization -> attn_q|k|v or ffn_gate|up (qwen3.rs:633-638: ln1 /
//     ln2 feed the projections): one prologue launch normalises the rows and emits the Q8_K /
//     Q8_0 planes the GEMV reads, instead of a normalisation pass, a write of h, and a
//     quantization pass (or every CTA quantizing h again);
//   * lm_head -> arg-max / top-k (src/backend/engine.rs:528-529, 810-824 sample from the last
//     row's logits): the k largest logits and their ids per row, ties to the lowest id, so a
//     host (or a vocabulary-sharded head) moves k pairs per row instead of the whole vocabulary.
#include <cfloat>
#include <cstdio>

#include "../../include/turq.h"
#include "actquant.cuh"
#include "handles.h"
#include "turq_internal.h"

namespace turq {

__global__ void __launch_bounds__(256) silu_mul_kernel(const float* __restrict__ g, const float* __restrict__ u,
                                                        float* __restrict__ out, int64_t total) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const float gv = g[i];
    out[i] = (gv / (1.f + expf(-gv))) * u[i];
  }
}

// One CTA per row: h = x / sqrt(mean(x^2) + eps) * weight (f32, the order candle's CPU rms-norm
// uses), optionally written out, and quantized block by block into the GEMV's activation planes.
// 256 threads = 8 warps; a warp owns whole 256-element blocks (Q8_K) or groups of 8 32-element
// blocks (Q8_0), so the block arithmetic is the stand-alone quantizer's.
struct NormQuantArgs {
  const void* x;
  int x_is_bf16;
  const float* weight;
  float eps;
  int64_t k;
  float* h_out;  // nullable
  int fmt;       // TQ_Q8_K or TQ_Q8_0
  int8_t* qs;
  float* dsc;
  int16_t* bs16;
  int16_t* bs32;
};

__global__ void __launch_bounds__(256) rmsnorm_quant_kernel(const NormQuantArgs a) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  __shared__ float wsum[8];
  const int64_t row = blockIdx.x, k = a.k;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float ss = 0.f;
  for (int64_t i = threadIdx.x * 8; i < k; i += 256 * 8) {
    float v[8];
    load8(a.x, a.x_is_bf16, row * k + i, v);
#pragma unroll
    for (int e = 0; e < 8; e++) ss += v[e] * v[e];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
  if (lane == 0) wsum[warp] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int w = 0; w < 8; w++) tot += wsum[w];
  const float denom = sqrtf(tot / (float)k + a.eps);
  if (a.fmt == TQ_Q8_K) {
    const int64_t nblk = k >> 8;
    for (int64_t blk = warp; blk < nblk; blk += 8) {
      float v[8];
      load8(a.x, a.x_is_bf16, row * k + blk * 256 + lane * 8, v);
      const float4 w0 = *reinterpret_cast<const float4*>(a.weight + blk * 256 + lane * 8);
      const float4 w1 = *reinterpret_cast<const float4*>(a.weight + blk * 256 + lane * 8 + 4);
      const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
      for (int e = 0; e < 8; e++) v[e] = __fmul_rn(__fdiv_rn(v[e], denom), wv[e]);
      if (a.h_out) {
        float* dst = a.h_out + row * k + blk * 256 + lane * 8;
        *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4*>(dst + 4) = make_float4(v[4], v[5], v[6], v[7]);
      }
      uint32_t q0, q1;
      float d;
      int s16, s32;
      quant_block_q8k(v, lane, q0, q1, d, s16, s32);
      *reinterpret_cast<uint2*>(a.qs + row * k + blk * 256 + lane * 8) = make_uint2(q0, q1);
      if (lane == 0) a.dsc[row * nblk + blk] = d;
      if ((lane & 1) == 0) a.bs16[row * (k >> 4) + blk * 16 + (lane >> 1)] = (int16_t)s16;
      if ((lane & 3) == 0) a.bs32[row * (k >> 5) + blk * 8 + (lane >> 2)] = (int16_t)s32;
    }
  } else {
    const int64_t nblk = k >> 5, groups = (nblk + 7) >> 3;
    for (int64_t grp = warp; grp < groups; grp += 8) {
      const int64_t blk = grp * 8 + (lane >> 2);
      const bool live = blk < nblk;
      float v[8];
      if (live) {
        const int64_t off = blk * 32 + (lane & 3) * 8;
        load8(a.x, a.x_is_bf16, row * k + off, v);
        const float4 w0 = *reinterpret_cast<const float4*>(a.weight + off);
        const float4 w1 = *reinterpret_cast<const float4*>(a.weight + off + 4);
        const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
        for (int e = 0; e < 8; e++) v[e] = __fmul_rn(__fdiv_rn(v[e], denom), wv[e]);
        if (a.h_out) {
          float* dst = a.h_out + row * k + off;
          *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
          *reinterpret_cast<float4*>(dst + 4) = make_float4(v[4], v[5], v[6], v[7]);
        }
      } else {
#pragma unroll
        for (int e = 0; e < 8; e++) v[e] = 0.f;
      }
      uint32_t q0, q1;
      __half dh;
      quant_block_q8_0(v, q0, q1, dh);
      if (live) {
        *reinterpret_cast<uint2*>(a.qs + row * k + blk * 32 + (lane & 3) * 8) = make_uint2(q0, q1);
        if ((lane & 3) == 0) a.dsc[row * nblk + blk] = __half2float(dh);
      }
    }
  }
}

}  // namespace turq

namespace turq {

constexpr int TOPK_CHUNK = 2048;   // candidates one CTA sorts
constexpr int TOPK_THREADS = 256;
constexpr int TOPK_MAX_K = 64;

// "a ranks before b": larger value first, equal values by lower id (the arg-max convention of a
// sequential scan); NaN counts as the smallest value.
__device__ __forceinline__ bool ranks_before(float av, int ai, float bv, int bi) { return av > bv || (av == bv && ai < bi); }

// grid (chunks, m). Row r of the input holds n candidates (values, and ids when ids_in is given,
// else id = position + id_offset). Every CTA sorts one chunk of up to 2048 of them in shared
// memory (bitonic network) and writes its k best to out[r][chunk][0..k).
__global__ void __launch_bounds__(TOPK_THREADS) topk_chunk_kernel(const float* __restrict__ vals_in, const int32_t* __restrict__ ids_in,
                                                                   int64_t n, int64_t row_stride, int32_t id_offset, int k,
                                                                   float* __restrict__ vals_out, int32_t* __restrict__ ids_out) {
  __shared__ float sv[TOPK_CHUNK];
  __shared__ int si[TOPK_CHUNK];
  const int64_t row = blockIdx.y, base = (int64_t)blockIdx.x * TOPK_CHUNK;
  for (int t = threadIdx.x; t < TOPK_CHUNK; t += TOPK_THREADS) {
    const int64_t pos = base + t;
    float v = -INFINITY;
    int id = INT32_MAX;
    if (pos < n) {
      v = vals_in[row * row_stride + pos];
      if (v != v) v = -INFINITY;
      id = ids_in ? ids_in[row * row_stride + pos] : (int)(pos + id_offset);
    }
    sv[t] = v;
    si[t] = id;
  }
  __syncthreads();
  for (int size = 2; size <= TOPK_CHUNK; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int t = threadIdx.x; t < TOPK_CHUNK / 2; t += TOPK_THREADS) {
        const int lo = 2 * t - (t & (stride - 1));  // index with bit `stride` clear
        const int hi = lo + stride;
        const bool descending = (lo & size) == 0;   // final pass (size = CHUNK): everything descending
        const float av = sv[lo], bv = sv[hi];
        const int ai = si[lo], bi = si[hi];
        const bool in_order = ranks_before(av, ai, bv, bi);
        if (in_order != descending && !(av == bv && ai == bi)) {
          sv[lo] = bv; sv[hi] = av;
          si[lo] = bi; si[hi] = ai;
        }
      }
      __syncthreads();
    }
  }
  const int64_t out_base = (row * gridDim.x + blockIdx.x) * k;
  for (int t = threadIdx.x; t < k; t += TOPK_THREADS) {
    vals_out[out_base + t] = sv[t];
    ids_out[out_base + t] = si[t];
  }
}

// k best of every row of (vals, ids) into out_vals / out_ids [m, k]; work = 2 x m x chunks x k
// pairs of ping-pong space. Rows with fewer than k candidates are padded with (-inf, INT32_MAX).
static cudaError_t launch_topk(const float* vals, const int32_t* ids, int64_t m, int64_t n, int64_t row_stride, int k,
                               int32_t id_offset, float* out_vals, int32_t* out_ids, uint8_t* work, size_t work_bytes,
                               cudaStream_t s, int* launches) {
  int64_t chunks = (n + TOPK_CHUNK - 1) / TOPK_CHUNK;
  const size_t pair_elems = (size_t)m * (size_t)chunks * (size_t)k;
  if (work_bytes < 2 * pair_elems * 8) return cudaErrorInvalidValue;
  float* wv[2] = {reinterpret_cast<float*>(work), reinterpret_cast<float*>(work + pair_elems * 8)};
  int32_t* wi[2] = {reinterpret_cast<int32_t*>(work + pair_elems * 4), reinterpret_cast<int32_t*>(work + pair_elems * 12)};
  int cur = 0;
  const float* in_v = vals;
  const int32_t* in_i = ids;
  for (;;) {
    const bool last = chunks == 1;
    dim3 grid((unsigned)chunks, (unsigned)m);
    topk_chunk_kernel<<<grid, TOPK_THREADS, 0, s>>>(in_v, in_i, n, row_stride, id_offset, k, last ? out_vals : wv[cur],
                                                    last ? out_ids : wi[cur]);
    if (launches) (*launches)++;
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess || last) return e;
    in_v = wv[cur];
    in_i = wi[cur];
    n = chunks * k;
    row_stride = n;
    id_offset = 0;
    chunks = (n + TOPK_CHUNK - 1) / TOPK_CHUNK;
    cur ^= 1;
  }
}

size_t topk_work_bytes(int64_t m, int64_t n, int k) {
  const size_t chunks = (size_t)((n + TOPK_CHUNK - 1) / TOPK_CHUNK);
  return 2 * (size_t)m * chunks * (size_t)k * 8 + 256;
}

}  // namespace turq

using turq::api_cuda_fail;
using turq::api_fail;

extern "C" {

int32_t turq_qmatmul_swiglu(turq_ctx* ctx, const turq_qtensor* gate, const turq_qtensor* up, const void* dev_x, int32_t x_dtype,
                            int64_t m, float* dev_out, int32_t mode, void* stream) {
  if (!ctx || !gate || !up || !dev_x || !dev_out) return api_fail(ctx, TURQ_E_INVALID_ARG, "null argument");
  if (gate->n_rows != up->n_rows || gate->n_cols != up->n_cols) return api_fail(ctx, TURQ_E_SHAPE, "ffn_gate and ffn_up must have the same shape");
  if (x_dtype != TURQ_F32 && x_dtype != TURQ_BF16) return api_fail(ctx, TURQ_E_DTYPE, "activations must be F32 or BF16");
  if (m <= 0 || m > INT32_MAX / 2) return api_fail(ctx, TURQ_E_SHAPE, "m out of range");
  if (gate->device != ctx->device || up->device != ctx->device) return api_fail(ctx, TURQ_E_INVALID_ARG, "tensors and context must live on the same device");
  if ((uintptr_t)dev_x % 16 != 0 || (uintptr_t)dev_out % 4 != 0) return api_fail(ctx, TURQ_E_ALIGN, "dev_x must be 16-byte aligned");
  cudaError_t e = cudaSetDevice(ctx->device);
  if (e != cudaSuccess) return api_cuda_fail(ctx, e, "cudaSetDevice");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t n = gate->n_rows, k = gate->n_cols;
  const int32_t eff = mode == TURQ_MODE_AUTO ? turq::api_auto_mode(ctx, 2 * n, k, m) : mode;
  if (eff == TURQ_MODE_INT8_ACT && gate->dtype == up->dtype) {
    const int fmt = gate->dtype == TURQ_Q8_0 ? TQ_Q8_0 : TQ_Q8_K;
    int32_t st = turq::api_ensure_scratch(ctx, turq::plan_act_pack(fmt, m, k).total);
    if (st != TURQ_OK) return st;
    int launches = 0;
    e = turq::launch_gemv_int8_swiglu(gate->dtype, gate->tiles, up->tiles, n, k, dev_x, x_dtype, ctx->scratch, m, dev_out,
                                      ctx->gemv_ws, ctx->dev_status, ctx->sm_count, s, &launches);
    ctx->launches += launches;
    if (e == cudaSuccess) return TURQ_OK;
    if (e != cudaErrorNotSupported) return api_cuda_fail(ctx, e, "swiglu launch");
  }
  // General route: both products into context memory, then one elementwise pass.
  int32_t st = turq::api_ensure_tmp(ctx, 2 * (size_t)m * n * 4);
  if (st != TURQ_OK) return st;
  float* g = reinterpret_cast<float*>(ctx->tmp);
  float* u = g + (size_t)m * n;
  const turq_qtensor* qts[2] = {gate, up};
  float* ys[2] = {g, u};
  st = turq_qmatmul_multi(ctx, 2, qts, dev_x, x_dtype, m, ys, mode, nullptr, stream);
  if (st != TURQ_OK) return st;
  const int64_t total = m * n;
  int64_t blocks = (total + 255) / 256;
  if (blocks > 8 * (int64_t)ctx->sm_count) blocks = 8 * (int64_t)ctx->sm_count;
  turq::silu_mul_kernel<<<(unsigned)blocks, 256, 0, s>>>(g, u, dev_out, total);
  ctx->launches++;
  e = cudaGetLastError();
  if (e != cudaSuccess) return api_cuda_fail(ctx, e, "silu-mul launch");
  return TURQ_OK;
}

int32_t turq_rmsnorm_qmatmul_multi(turq_ctx* ctx, int32_t count, const turq_qtensor* const* qts, const void* dev_x,
                                   int32_t x_dtype, int64_t m, const float* dev_norm_weight, float eps, float* dev_h_out,
                                   float* const* dev_ys, int32_t mode, const float* const* dev_biases, void* stream) {
  if (!ctx || !qts || !dev_x || !dev_norm_weight || !dev_ys) return api_fail(ctx, TURQ_E_INVALID_ARG, "null argument");
  if (count < 1 || count > 4) return api_fail(ctx, TURQ_E_INVALID_ARG, "count outside 1..4");
  if (x_dtype != TURQ_F32 && x_dtype != TURQ_BF16) return api_fail(ctx, TURQ_E_DTYPE, "activations must be F32 or BF16");
  if (m <= 0 || m > INT32_MAX / 2) return api_fail(ctx, TURQ_E_SHAPE, "m out of range");
  bool k_quant = false, q8_0 = false;
  int64_t rows_all = 0;
  for (int i = 0; i < count; i++) {
    if (!qts[i] || !dev_ys[i]) return api_fail(ctx, TURQ_E_INVALID_ARG, "null argument");
    if (qts[i]->n_cols != qts[0]->n_cols) return api_fail(ctx, TURQ_E_SHAPE, "weights of one call must share the in-feature count");
    if (qts[i]->device != ctx->device) return api_fail(ctx, TURQ_E_INVALID_ARG, "tensors and context must live on the same device");
    (qts[i]->dtype == TURQ_Q8_0 ? q8_0 : k_quant) = true;
    rows_all += qts[i]->n_rows;
  }
  const int64_t k = qts[0]->n_cols;
  if ((uintptr_t)dev_x % 16 != 0 || (uintptr_t)dev_norm_weight % 16 != 0 || (dev_h_out && (uintptr_t)dev_h_out % 16 != 0))
    return api_fail(ctx, TURQ_E_ALIGN, "dev_x, dev_norm_weight and dev_h_out must be 16-byte aligned");
  cudaError_t e = cudaSetDevice(ctx->device);
  if (e != cudaSuccess) return api_cuda_fail(ctx, e, "cudaSetDevice");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int32_t eff = mode == TURQ_MODE_AUTO ? turq::api_auto_mode(ctx, rows_all, k, m) : mode;
  const bool direct = eff == TURQ_MODE_INT8_ACT && !(k_quant && q8_0);
  const int fmt = q8_0 && !k_quant ? TQ_Q8_0 : TQ_Q8_K;
  const turq::ActPackPlan plan = turq::plan_act_pack(fmt, m, k);
  int32_t st = turq::api_ensure_scratch(ctx, plan.total);
  if (st != TURQ_OK) return st;
  float* h = dev_h_out;
  if (!direct && !h) {  // the other schemes read h itself
    st = turq::api_ensure_tmp(ctx, (size_t)m * k * 4);
    if (st != TURQ_OK) return st;
    h = reinterpret_cast<float*>(ctx->tmp);
  }
  turq::NormQuantArgs a{};
  a.x = dev_x;
  a.x_is_bf16 = x_dtype == TURQ_BF16;
  a.weight = dev_norm_weight;
  a.eps = eps;
  a.k = k;
  a.h_out = h;
  a.fmt = fmt;
  a.qs = reinterpret_cast<int8_t*>(ctx->scratch + plan.off_qs);
  a.dsc = reinterpret_cast<float*>(ctx->scratch + plan.off_dsc);
  a.bs16 = reinterpret_cast<int16_t*>(ctx->scratch + plan.off_bs16);
  a.bs32 = reinterpret_cast<int16_t*>(ctx->scratch + plan.off_bs32);
  turq::rmsnorm_quant_kernel<<<(unsigned)m, 256, 0, s>>>(a);
  ctx->launches++;
  e = cudaGetLastError();
  if (e != cudaSuccess) return api_cuda_fail(ctx, e, "rmsnorm launch");
  if (!direct) return turq_qmatmul_multi(ctx, count, qts, h, TURQ_F32, m, dev_ys, mode, dev_biases, stream);
  turq::GemvPart parts[4];
  for (int i = 0; i < count; i++)
    parts[i] = turq::GemvPart{qts[i]->tiles, qts[i]->n_rows, dev_ys[i], dev_biases ? dev_biases[i] : nullptr, qts[i]->dtype, nullptr};
  int launches = 0;
  // the GEMV only ever reads the planes; x is passed for completeness
  e = turq::launch_gemv_int8_multi(qts[0]->dtype, parts, count, k, dev_x, x_dtype, ctx->scratch, m, ctx->gemv_ws, ctx->dev_status,
                                   ctx->sm_count, s, &launches, false, nullptr, true);
  ctx->launches += launches;
  if (e != cudaSuccess) return api_cuda_fail(ctx, e, "rmsnorm + qmatmul launch");
  return TURQ_OK;
}

int32_t turq_topk(turq_ctx* ctx, const float* dev_vals, const int32_t* dev_ids, int64_t m, int64_t n, int32_t k,
                  int32_t id_offset, float* dev_out_vals, int32_t* dev_out_ids, void* stream) {
  if (!ctx || !dev_vals || !dev_out_vals || !dev_out_ids) return api_fail(ctx, TURQ_E_INVALID_ARG, "null argument");
  if (m <= 0 || n <= 0 || m > 65535) return api_fail(ctx, TURQ_E_SHAPE, "m must be in 1..65535 and n positive");
  if (k < 1 || k > turq::TOPK_MAX_K) return api_fail(ctx, TURQ_E_LIMIT, "k must be in 1..64");
  cudaError_t e = cudaSetDevice(ctx->device);
  if (e != cudaSuccess) return api_cuda_fail(ctx, e, "cudaSetDevice");
  const size_t work = turq::topk_work_bytes(m, n, k);
  int32_t st = turq::api_ensure_tmp(ctx, work);
  if (st != TURQ_OK) return st;
  int launches = 0;
  e = turq::launch_topk(dev_vals, dev_ids, m, n, n, k, id_offset, dev_out_vals, dev_out_ids, ctx->tmp, work,
                        static_cast<cudaStream_t>(stream), &launches);
  ctx->launches += launches;
  if (e != cudaSuccess) return api_cuda_fail(ctx, e, "top-k launch");
  return TURQ_OK;
}

int32_t turq_lm_head_topk(turq_ctx* ctx, const turq_qtensor* qt, const void* dev_x, int32_t x_dtype, int64_t m, int32_t k,
                          int32_t id_offset, float* dev_out_vals, int32_t* dev_out_ids, float* dev_logits, int32_t mode,
                          void* stream) {
  if (!ctx || !qt || !dev_x || !dev_out_vals || !dev_out_ids) return api_fail(ctx, TURQ_E_INVALID_ARG, "null argument");
  if (m <= 0 || m > 65535) return api_fail(ctx, TURQ_E_SHAPE, "m must be in 1..65535");
  if (k < 1 || k > turq::TOPK_MAX_K) return api_fail(ctx, TURQ_E_LIMIT, "k must be in 1..64");
  cudaError_t e = cudaSetDevice(ctx->device);
  if (e != cudaSuccess) return api_cuda_fail(ctx, e, "cudaSetDevice");
  const int64_t n = qt->n_rows;
  const size_t work = turq::topk_work_bytes(m, n, k);
  const size_t logits_bytes = dev_logits ? 0 : (((size_t)m * n * 4 + 255) & ~(size_t)255);
  int32_t st = turq::api_ensure_tmp(ctx, logits_bytes + work);
  if (st != TURQ_OK) return st;
  float* logits = dev_logits ? dev_logits : reinterpret_cast<float*>(ctx->tmp);
  st = turq_qmatmul(ctx, qt, dev_x, x_dtype, m, logits, mode, nullptr, stream);
  if (st != TURQ_OK) return st;
  int launches = 0;
  e = turq::launch_topk(logits, nullptr, m, n, n, k, id_offset, dev_out_vals, dev_out_ids, ctx->tmp + logits_bytes, work,
                        static_cast<cudaStream_t>(stream), &launches);
  ctx->launches += launches;
  if (e != cudaSuccess) return api_cuda_fail(ctx, e, "top-k launch");
  return TURQ_OK;
}

}  // extern "C"
