// Device side of the tensor-parallel exchange over peer memory, shared by the stand-alone
// exchange kernels (tp.cu) and the decode GEMV whose last CTA performs the exchange itself
// (gemv_stream.cu). Protocol and memory layout are described at the top of tp.cu.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/turq.h"

namespace turq {

constexpr int TP_MAX_RANKS = 8;
constexpr int TP_MAX_BLOCKS = 128;
constexpr int TP_THREADS = 256;
constexpr size_t TP_FLAGS_BYTES = (size_t)TP_MAX_BLOCKS * TP_MAX_RANKS * 4;  // 4 KB
constexpr size_t TP_HEADER_BYTES = TP_FLAGS_BYTES + 256;                     // + counter words, 256-byte aligned

struct TpArgs {
  const float* peer_data[TP_MAX_RANKS];  // slot 0 of every rank's region, in rank order (own: local pointer)
  unsigned* peer_flags[TP_MAX_RANKS];    // flag array of every rank's region
  unsigned* counter;                     // own region: [0] calls completed, [1] CTA ticket, [2] GEMV CTAs done (fused launches)
  size_t slot_elems;                     // floats per slot
  int rank, world;
  long long wait_cycles;
  int* status;
  // reduce: out[i] = sum_p peer[p][i] (+ bias[i % n]) for i < count
  int64_t count, n;
  const float* bias;
  // gather: out[r, col0[p] + j] = peer[p][r * width[p] + j]
  int64_t m, n_total;
  int64_t col0[TP_MAX_RANKS + 1];
  float* out;
};

__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// peer data: system-scope loads that do not linger in this SM's L1 across calls
__device__ __forceinline__ float4 ld_peer_v4(const float* p) {
  float4 v;
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float ld_peer_f32(const float* p) {
  float v;
  asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
  return v;
}

// Signals this CTA's peers, waits for theirs. Returns false when the wait ran out.
// `b` = which row of flags this CTA pairs on with the same CTA of the peers.
// A call has up to two meeting points (`phase` 0: "my slot is complete", 1: "my share of the
// result is in my slot"); the flag value of call `seq`, phase `phase` is 2 * seq + phase.
__device__ __forceinline__ bool tp_rendezvous(const TpArgs& a, unsigned seq, int* s_ok, int b, unsigned phase = 0u) {
  if (threadIdx.x == 0) *s_ok = 1;
  __syncthreads();
  if (threadIdx.x < a.world) {
    const int p = threadIdx.x;
    const unsigned value = 2u * seq + phase;
    // everything this rank put into its slot was written by kernels that completed before this
    // one started (phase 0) or by this CTA before the barrier above (phase 1); the release store
    // publishes it to the peer together with the flag
    st_release_sys(a.peer_flags[p] + b * TP_MAX_RANKS + a.rank, value);
    const unsigned* mine = a.peer_flags[a.rank] + b * TP_MAX_RANKS + p;
    const long long t0 = clock64();
    for (;;) {
      if ((int)(ld_acquire_sys(mine) - value) >= 0) break;
      if (clock64() - t0 > a.wait_cycles) {
        *s_ok = 0;
        break;
      }
      __nanosleep(40);
    }
  }
  __syncthreads();
  return *s_ok != 0;
}

// out[i] = sum over ranks (rank order) of their slot's element i (+ bias[i % n]), for the float4
// groups first_vec, first_vec + vec_stride, ... and - by the caller's thread set with first_vec <
// vec_stride covering the tail - the last count % 4 elements.
__device__ __forceinline__ void tp_reduce_range(const TpArgs& a, size_t slot_off, int64_t first_vec, int64_t vec_stride, bool do_tail) {
  const int64_t nvec = a.count >> 2;
  const bool vec_bias = a.bias && (a.n & 3) == 0;
  for (int64_t v = first_vec; v < nvec; v += vec_stride) {
    // all ranks' loads go out before the first add: one peer round trip per group, not one per rank
    float4 t[TP_MAX_RANKS];
#pragma unroll
    for (int p = 0; p < TP_MAX_RANKS; p++)
      if (p < a.world) t[p] = ld_peer_v4(a.peer_data[p] + slot_off + 4 * v);
    float4 acc = t[0];
#pragma unroll
    for (int p = 1; p < TP_MAX_RANKS; p++)
      if (p < a.world) { acc.x += t[p].x; acc.y += t[p].y; acc.z += t[p].z; acc.w += t[p].w; }
    if (a.bias) {
      if (vec_bias) {
        const float4 bb = *reinterpret_cast<const float4*>(a.bias + (4 * v) % a.n);
        acc.x += bb.x; acc.y += bb.y; acc.z += bb.z; acc.w += bb.w;
      } else {
        acc.x += a.bias[(4 * v) % a.n]; acc.y += a.bias[(4 * v + 1) % a.n];
        acc.z += a.bias[(4 * v + 2) % a.n]; acc.w += a.bias[(4 * v + 3) % a.n];
      }
    }
    *reinterpret_cast<float4*>(a.out + 4 * v) = acc;
  }
  if (do_tail) {
    for (int64_t i = (nvec << 2) + first_vec; i < a.count; i += vec_stride) {
      float acc = ld_peer_f32(a.peer_data[0] + slot_off + i);
      for (int p = 1; p < a.world; p++) acc += ld_peer_f32(a.peer_data[p] + slot_off + i);
      if (a.bias) acc += a.bias[i % a.n];
      a.out[i] = acc;
    }
  }
}

// Two-shot all-reduce of one CTA's share (count % 4 == 0). The float4 groups are cut into `world`
// equal slices; slice r is reduced by rank r alone - in rank order, so every rank ends with the
// same bits - written to out and, in place, into rank r's own slot; after the second meeting
// point every rank copies the other slices from their owners. A rank moves 2 (world - 1) / world
// of the result over the links instead of (world - 1) times the result. CTA b of every rank walks
// the same offsets of every slice, so what it copies from a peer is what CTA b of that peer wrote.
__device__ __forceinline__ bool tp_twoshot(const TpArgs& a, unsigned seq, size_t slot_off, int* s_ok, int b, int nblocks) {
  const int64_t nvec = a.count >> 2;
  const int64_t per = (nvec + a.world - 1) / a.world;
  const bool vec_bias = a.bias && (a.n & 3) == 0;
  float* own = const_cast<float*>(a.peer_data[a.rank]) + slot_off;
  const int64_t stride = (int64_t)nblocks * blockDim.x;
  for (int64_t off = (int64_t)b * blockDim.x + threadIdx.x; off < per; off += stride) {
    const int64_t v = (int64_t)a.rank * per + off;
    if (v >= nvec) break;
    float4 t[TP_MAX_RANKS];
#pragma unroll
    for (int p = 0; p < TP_MAX_RANKS; p++)
      if (p < a.world) t[p] = ld_peer_v4(a.peer_data[p] + slot_off + 4 * v);
    float4 acc = t[0];
#pragma unroll
    for (int p = 1; p < TP_MAX_RANKS; p++)
      if (p < a.world) { acc.x += t[p].x; acc.y += t[p].y; acc.z += t[p].z; acc.w += t[p].w; }
    if (a.bias) {
      if (vec_bias) {
        const float4 bb = *reinterpret_cast<const float4*>(a.bias + (4 * v) % a.n);
        acc.x += bb.x; acc.y += bb.y; acc.z += bb.z; acc.w += bb.w;
      } else {
        acc.x += a.bias[(4 * v) % a.n]; acc.y += a.bias[(4 * v + 1) % a.n];
        acc.z += a.bias[(4 * v + 2) % a.n]; acc.w += a.bias[(4 * v + 3) % a.n];
      }
    }
    *reinterpret_cast<float4*>(a.out + 4 * v) = acc;
    *reinterpret_cast<float4*>(own + 4 * v) = acc;
  }
  __threadfence_system();
  if (!tp_rendezvous(a, seq, s_ok, b, 1u)) return false;
  for (int64_t off = (int64_t)b * blockDim.x + threadIdx.x; off < per; off += stride) {
    float4 t[TP_MAX_RANKS];
#pragma unroll
    for (int i = 1; i < TP_MAX_RANKS; i++) {
      if (i < a.world) {
        const int q = (a.rank + i) % a.world;  // every rank starts at another owner
        const int64_t v = (int64_t)q * per + off;
        if (v < nvec) t[i] = ld_peer_v4(a.peer_data[q] + slot_off + 4 * v);
      }
    }
#pragma unroll
    for (int i = 1; i < TP_MAX_RANKS; i++) {
      if (i < a.world) {
        const int q = (a.rank + i) % a.world;
        const int64_t v = (int64_t)q * per + off;
        if (v < nvec) *reinterpret_cast<float4*>(a.out + 4 * v) = t[i];
      }
    }
  }
  return true;
}

// The last CTA to finish advances the call number (every CTA read it at its start).
__device__ __forceinline__ void tp_finish(const TpArgs& a, unsigned seq, bool ok) {
  __syncthreads();
  if (threadIdx.x == 0) {
    if (!ok) {
      *reinterpret_cast<volatile int*>(a.status) = TURQ_E_TIMEOUT;  // the word may be mapped host memory
      __threadfence_system();
    }
    __threadfence();
    const unsigned ticket = atomicAdd(a.counter + 1, 1u);
    if (ticket == gridDim.x - 1) {
      a.counter[1] = 0;
      __threadfence();
      *reinterpret_cast<volatile unsigned*>(a.counter) = seq;
    }
  }
}

}  // namespace turq
