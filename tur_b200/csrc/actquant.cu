// Activation quantization of QMatMul::forward's CPU scheme: rows of x -> Q8_K blocks (paired
// with Q4_K/Q5_K/Q6_K weights) or Q8_0 blocks (paired with Q8_0 weights). Two output forms:
// GGUF wire blocks (public entry, parity-tested bit-exact) and the plane layout the GEMV
// kernels read (same integers and scales, produced by the same device code).
//
// Q8_K (defaults; the three choices are compile-time switches, see actquant.cuh): the element of
// largest magnitude (first one on ties) maps to -128 before the clamp at 127, ties round away
// from zero, d = 1/iscale.
// Q8_0: d = amax/127 in f32, stored as f16; q = round-half-away(x * (1/d)).
#include "actquant.cuh"
#include "turq_internal.h"

namespace turq {

int q8k_variant() { return TURQ_Q8K_DIVISOR | (TURQ_Q8K_NEG_SCALE ? 0x100 : 0) | (TURQ_Q8K_ROUND_HALF_EVEN ? 0x200 : 0); }

ActPackPlan plan_act_pack(int fmt, int64_t m, int64_t k) {
  auto up = [](size_t v) { return (v + 255) & ~(size_t)255; };
  ActPackPlan p{};
  p.off_qs = 0;
  p.off_dsc = up((size_t)m * k);
  int bs = fmt == TQ_Q8_0 ? 32 : 256;
  p.off_bs16 = up(p.off_dsc + (size_t)m * (k / bs) * 4);
  if (fmt == TQ_Q8_0) {
    p.off_bs32 = p.off_bs16;
    p.total = p.off_bs16;
  } else {
    p.off_bs32 = up(p.off_bs16 + (size_t)m * (k / 16) * 2);
    p.total = up(p.off_bs32 + (size_t)m * (k / 32) * 2);
  }
  return p;
}

struct ActOut {
  uint8_t* wire;   // wire blocks or nullptr
  int8_t* qs;      // planes (when wire == nullptr)
  float* dsc;
  int16_t* bs16;
  int16_t* bs32;
};

// One warp per 256-element block: lane owns elements 8*lane .. 8*lane+7.
__global__ void __launch_bounds__(128) quant_q8k_kernel(const void* __restrict__ x, int is_bf16, int64_t m,
                                                        int64_t k, ActOut out) {
  // Both this launch and the GEMV behind it carry the programmatic-stream-serialization
  // attribute. Trigger first: the GEMV may become resident and stream weights at once (it waits
  // for this grid's completion before it reads the planes). Then wait: the preceding kernel may
  // still be reading the planes this grid is about to overwrite, and may be producing x.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int lane = threadIdx.x & 31;
  const int64_t nblk = k >> 8;
  const int64_t total = m * nblk;
  int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t wb = warp; wb < total; wb += nwarps) {
    int64_t row = wb / nblk, blk = wb - row * nblk;
    float v[8];
    load8(x, is_bf16, row * k + blk * 256 + lane * 8, v);
    uint32_t w0, w1;
    float d;
    int s16, s32;
    quant_block_q8k(v, lane, w0, w1, d, s16, s32);
    if (out.wire) {
      uint8_t* b = out.wire + wb * 292;  // 292 = 4 * 73: every field stays 4-byte aligned
      if (lane == 0) *reinterpret_cast<float*>(b) = d;
      uint32_t* qs = reinterpret_cast<uint32_t*>(b + 4 + lane * 8);
      qs[0] = w0;
      qs[1] = w1;
      if ((lane & 1) == 0) *reinterpret_cast<int16_t*>(b + 260 + lane) = (int16_t)s16;
    } else {
      *reinterpret_cast<uint2*>(out.qs + row * k + blk * 256 + lane * 8) = make_uint2(w0, w1);
      if (lane == 0) out.dsc[wb] = d;
      if ((lane & 1) == 0) out.bs16[row * (k >> 4) + blk * 16 + (lane >> 1)] = (int16_t)s16;
      if ((lane & 3) == 0) out.bs32[row * (k >> 5) + blk * 8 + (lane >> 2)] = (int16_t)s32;
    }
  }
}

// Four lanes per 32-element block; a warp covers 8 consecutive blocks of one row.
__global__ void __launch_bounds__(128) quant_q8_0_kernel(const void* __restrict__ x, int is_bf16, int64_t m,
                                                         int64_t k, ActOut out) {
  // Both this launch and the GEMV behind it carry the programmatic-stream-serialization
  // attribute. Trigger first: the GEMV may become resident and stream weights at once (it waits
  // for this grid's completion before it reads the planes). Then wait: the preceding kernel may
  // still be reading the planes this grid is about to overwrite, and may be producing x.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int lane = threadIdx.x & 31;
  const int64_t nblk = k >> 5;
  const int64_t groups = (nblk + 7) >> 3;  // warp-sized groups of 8 blocks per row
  const int64_t total = m * groups;
  int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t wg = warp; wg < total; wg += nwarps) {
    int64_t row = wg / groups, grp = wg - row * groups;
    int64_t blk = grp * 8 + (lane >> 2);
    bool live = blk < nblk;
    float v[8];
    if (live) {
      load8(x, is_bf16, row * k + blk * 32 + (lane & 3) * 8, v);
    } else {
#pragma unroll
      for (int e = 0; e < 8; e++) v[e] = 0.f;
    }
    uint32_t w0, w1;
    __half dh;
    quant_block_q8_0(v, w0, w1, dh);
    if (!live) continue;
    if (out.wire) {
      uint8_t* b = out.wire + (row * nblk + blk) * 34;  // 2-byte aligned only
      if ((lane & 3) == 0) *reinterpret_cast<__half*>(b) = dh;
      uint16_t* qs = reinterpret_cast<uint16_t*>(b + 2 + (lane & 3) * 8);
      qs[0] = (uint16_t)(w0 & 0xFFFF);
      qs[1] = (uint16_t)(w0 >> 16);
      qs[2] = (uint16_t)(w1 & 0xFFFF);
      qs[3] = (uint16_t)(w1 >> 16);
    } else {
      *reinterpret_cast<uint2*>(out.qs + row * k + blk * 32 + (lane & 3) * 8) = make_uint2(w0, w1);
      if ((lane & 3) == 0) out.dsc[row * nblk + blk] = __half2float(dh);
    }
  }
}

// Launch that may be scheduled while the preceding kernel of the stream still runs (the kernels
// order themselves with griddepcontrol.wait).
template <class... Args>
static cudaError_t launch_pdl(void (*kernel)(Args...), unsigned blocks, int threads, cudaStream_t s, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(blocks);
  cfg.blockDim = dim3((unsigned)threads);
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, args...);
}

static cudaError_t launch_act(int fmt, const void* x, int x_dtype, int64_t m, int64_t k, ActOut out,
                              cudaStream_t s) {
  if (m == 0 || k == 0) return cudaSuccess;
  int is_bf16 = x_dtype == TQ_BF16;
  int threads = 128;
  if (fmt == TQ_Q8_K) {
    int64_t warps = m * (k >> 8);
    int64_t blocks = (warps + 3) / 4;
    if (blocks > (int64_t)device_sm_count() * 16) blocks = (int64_t)device_sm_count() * 16;
    return launch_pdl(quant_q8k_kernel, (unsigned)blocks, threads, s, x, is_bf16, m, k, out);
  } else if (fmt == TQ_Q8_0) {
    int64_t warps = m * (((k >> 5) + 7) >> 3);
    int64_t blocks = (warps + 3) / 4;
    if (blocks > (int64_t)device_sm_count() * 16) blocks = (int64_t)device_sm_count() * 16;
    return launch_pdl(quant_q8_0_kernel, (unsigned)blocks, threads, s, x, is_bf16, m, k, out);
  } else {
    return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

cudaError_t launch_quantize_act_wire(int fmt, const void* x, int x_dtype, int64_t m, int64_t k, void* blocks,
                                     cudaStream_t s) {
  ActOut out{};
  out.wire = reinterpret_cast<uint8_t*>(blocks);
  return launch_act(fmt, x, x_dtype, m, k, out, s);
}

cudaError_t launch_quantize_act_pack(int fmt, const void* x, int x_dtype, int64_t m, int64_t k,
                                     uint8_t* scratch, cudaStream_t s) {
  ActPackPlan p = plan_act_pack(fmt, m, k);
  ActOut out{};
  out.wire = nullptr;
  out.qs = reinterpret_cast<int8_t*>(scratch + p.off_qs);
  out.dsc = reinterpret_cast<float*>(scratch + p.off_dsc);
  out.bs16 = reinterpret_cast<int16_t*>(scratch + p.off_bs16);
  out.bs32 = reinterpret_cast<int16_t*>(scratch + p.off_bs32);
  return launch_act(fmt, x, x_dtype, m, k, out, s);
}

}  // namespace turq
