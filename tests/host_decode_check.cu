// CPU execution of the device layout code: repacks GGUF wire blocks into fragment tiles with the
// word map of layout.h and decodes every lane of every tile with decode.cuh (the code the
// dequantize kernel and the exact-f32 GEMV run on the GPU), then compares with the expected f32
// values bit for bit. Usage: host_decode_check <dtype> <n_rows> <k> <blocks.bin> <f32.bin>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "decode.cuh"

using namespace turq;

static std::vector<uint8_t> read_file(const char* path) {
  std::vector<uint8_t> v;
  FILE* f = std::fopen(path, "rb");
  if (!f) return v;
  std::fseek(f, 0, SEEK_END);
  long n = std::ftell(f);
  std::fseek(f, 0, SEEK_SET);
  v.resize((size_t)n);
  if (std::fread(v.data(), 1, (size_t)n, f) != (size_t)n) v.clear();
  std::fclose(f);
  return v;
}

template <int DT>
static long run(int64_t n, int64_t k, const std::vector<uint8_t>& wire, const float* want) {
  const int ke = tq_block_elems(DT), bb = tq_block_bytes(DT), tb = tq_tile_bytes(DT);
  const int64_t kt_n = k / ke, rt_n = (n + 15) / 16;
  const size_t rb = (size_t)kt_n * bb;
  std::vector<uint8_t> tiles((size_t)rt_n * kt_n * tb + 16);
  for (int64_t rt = 0; rt < rt_n; rt++)
    for (int64_t kt = 0; kt < kt_n; kt++) {
      uint32_t* dst = reinterpret_cast<uint32_t*>(tiles.data() + (rt * kt_n + kt) * tb);
      auto blk = [&](int r) -> const uint8_t* {
        const int64_t row = rt * 16 + r;
        return row < n ? wire.data() + row * rb + kt * bb : nullptr;
      };
      for (int w = 0; w < tb / 4; w++) dst[w] = tq_tile_word(DT, w, blk);
    }
  std::vector<float> got((size_t)n * k, -12345.f);
  for (int64_t rt = 0; rt < rt_n; rt++)
    for (int64_t kt = 0; kt < kt_n; kt++)
      for (int lane = 0; lane < 32; lane++)
        decode_tile<DT>(tiles.data() + (rt * kt_n + kt) * tb, lane, [&](int hr, int off, const auto& v) {
          const int64_t row = rt * 16 + (lane >> 2) + 8 * hr;
          if (row >= n) return;
          for (unsigned e = 0; e < sizeof(v) / 4; e++) got[row * k + kt * ke + off + e] = v[e];
        });
  long bad = 0;
  for (size_t i = 0; i < got.size(); i++)
    if (std::memcmp(&want[i], &got[i], 4) != 0) {
      if (bad < 5) std::printf("mismatch at %zu: want %a got %a\n", i, want[i], got[i]);
      bad++;
    }
  return bad;
}

int main(int argc, char** argv) {
  if (argc != 6) return 2;
  const int dt = std::atoi(argv[1]);
  const int64_t n = std::atoll(argv[2]), k = std::atoll(argv[3]);
  const std::vector<uint8_t> wire = read_file(argv[4]), f32 = read_file(argv[5]);
  if (wire.size() != (size_t)n * (k / tq_block_elems(dt)) * tq_block_bytes(dt) || f32.size() != (size_t)n * k * 4) {
    std::printf("size mismatch\n");
    return 2;
  }
  const float* want = reinterpret_cast<const float*>(f32.data());
  long bad = -1;
  switch (dt) {
    case TQ_Q8_0: bad = run<TQ_Q8_0>(n, k, wire, want); break;
    case TQ_Q4_K: bad = run<TQ_Q4_K>(n, k, wire, want); break;
    case TQ_Q5_K: bad = run<TQ_Q5_K>(n, k, wire, want); break;
    case TQ_Q6_K: bad = run<TQ_Q6_K>(n, k, wire, want); break;
    default: return 2;
  }
  std::printf("dtype %d n %lld k %lld mismatches %ld\n", dt, (long long)n, (long long)k, bad);
  return bad == 0 ? 0 : 1;
}
