// Definitions of the opaque handle types of the C ABI (shared by the translation units that
// implement entry points).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

struct turq_ctx {
  int device = 0;
  int sm_count = 0;
  uint8_t* scratch = nullptr;  // activation planes / f16 operand for the current call
  size_t scratch_bytes = 0;
  uint8_t* io = nullptr;  // device staging for the host-buffer entry (x, y, bias)
  size_t io_bytes = 0;
  uint8_t* tmp = nullptr;  // results on their way to a tensor-parallel exchange slot / fused epilogues
  size_t tmp_bytes = 0;
  int* host_status = nullptr;  // status word in mapped pinned host memory, written by kernels with bounded waits
  int* dev_status = nullptr;   // the same word's device address
  // completion word of bound host calls: the last kernel of a call stores the call number into
  // mapped host memory (word 16 of the status allocation); the host waits on that word instead
  // of synchronizing the stream
  volatile unsigned* host_done = nullptr;
  unsigned* dev_done = nullptr;       // the same word's device address
  unsigned* done_count = nullptr;     // device memory: calls signalled so far
  unsigned done_expected = 0;         // host: calls launched so far
  uint8_t* gemv_ws = nullptr;  // split row-tile workspace of the streaming GEMV (zeroed once)
  cudaStream_t own_stream = nullptr;
  int auto_policy = 0;  // what TURQ_MODE_AUTO resolves to: 0 = by row count, else a fixed turq_mode
  int64_t launches = 0;
  std::string err;
};

struct turq_qtensor {
  int device = 0;
  int dtype = 0;
  int64_t n_rows = 0, n_cols = 0;
  size_t wire_bytes = 0;
  uint8_t* tiles = nullptr;
  size_t tile_bytes = 0;
};

// A host-buffer matmul call with everything resolved up front (turq_host_call_*): the device
// aliases of the caller's page-locked buffers, a planes buffer of its own, and the launches
// recorded as an executable graph.
struct turq_host_call {
  turq_ctx* ctx = nullptr;
  uint8_t* scratch = nullptr;
  cudaGraphExec_t exec = nullptr;
};
