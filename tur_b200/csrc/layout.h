// Device-resident weight layout ("fragment tiles") and its mapping to the GGUF wire format.
//
// A QTensor [N rows, K cols] is stored on the GPU as row-tiles of 16 rows; each row-tile is a
// run of K-tiles (256 elements for Q4_K/Q5_K/Q6_K, one 32-element block for Q8_0). Inside a
// K-tile the quants are interleaved so that lane l = 4*g + c of a warp (g = 0..7, c = 0..3)
// finds, in consecutive 16-byte chunks, exactly the bytes of rows g and g+8 it owns in an
// m16n8k32 / m16n8k16 integer MMA A-fragment. One coalesced 128-bit load per lane brings a
// fragment pair straight into registers; no shared-memory staging or byte shuffling is
// needed, and every chunk is 16-byte aligned although the wire blocks (34 B, 210 B) are not.
// The repack is a bijection on the block bits, so dequantisation stays bit-exact with the
// wire format and the stored size equals the GGUF size (rows padded up to a multiple of 16
// with zero blocks).
//
// Element ownership (the "k permutation" shared by weights and activations):
//   32-element sub-block (Q4_K, Q5_K, Q8_0): lane column c owns elements 8c .. 8c+7
//   16-element sub-block (Q6_K):             lane column c owns elements 4c .. 4c+3
//
// Tile byte maps (row r = 0..15, lane l, g = l>>2, c = l&3):
//   Q8_0 (544 B):  [0,32)    d[r] f16
//                  [32,544)  lane l: 8 B of row g (wire qs[8c..8c+7]) | 8 B of row g+8
//   Q4_K (2304 B): [0,256)   header[r] = wire bytes 0..15 (d, dmin, 12 scale bytes)
//                  [256,..)  chunk i=0..3, lane l at 256+512i+16l:
//                            row g wire qs[32i+8c .. +7] | row g+8 same   (low nibble =
//                            sub-block 2i, high nibble = sub-block 2i+1)
//   Q5_K (2816 B): [0,256) header; [256,768) lane l: row g wire qh[8c..8c+7] | row g+8;
//                  [768,..) as Q4_K qs
//   Q6_K (3360 B): [0,256) scales[r][16] int8; [256,288) d[r] f16;
//                  [288,2336) ql chunk i=0..3 lane l: words (row g: t=2i, 2i+1 | row g+8: same)
//                             word t byte e: low nibble  = low 4 bits of element 32t+4c+e
//                                            high nibble = low 4 bits of element 32t+16+4c+e
//                  [2336,3360) qh chunk h=0..1 lane l: words (row g: u=2h, 2h+1 | row g+8: same)
//                             word u byte e bits 2s..2s+1 = high 2 bits of element 16(4u+s)+4c+e
//
// Wire formats: gguf-py quants.py (Q8_0 395-401, Q4_K 503-522, Q5_K 527-549, Q6_K 554-572).
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define TQ_HD __host__ __device__ __forceinline__
#else
#define TQ_HD inline
#endif

// GGUF wire-format type ids
enum : int32_t {
  TQ_F32 = 0,
  TQ_F16 = 1,
  TQ_Q8_0 = 8,
  TQ_Q4_K = 12,
  TQ_Q5_K = 13,
  TQ_Q6_K = 14,
  TQ_Q8_K = 15,
  TQ_BF16 = 30
};

constexpr int TQ_TILE_ROWS = 16;

TQ_HD int tq_block_elems(int dtype) {
  switch (dtype) {
    case TQ_Q8_0: return 32;
    case TQ_Q4_K: case TQ_Q5_K: case TQ_Q6_K: case TQ_Q8_K: return 256;
    case TQ_F32: case TQ_F16: case TQ_BF16: return 1;
    default: return 0;
  }
}
TQ_HD int tq_block_bytes(int dtype) {
  switch (dtype) {
    case TQ_Q8_0: return 34;
    case TQ_Q4_K: return 144;
    case TQ_Q5_K: return 176;
    case TQ_Q6_K: return 210;
    case TQ_Q8_K: return 292;
    case TQ_F32: return 4;
    case TQ_F16: case TQ_BF16: return 2;
    default: return 0;
  }
}
TQ_HD bool tq_is_weight_type(int dtype) {
  return dtype == TQ_Q8_0 || dtype == TQ_Q4_K || dtype == TQ_Q5_K || dtype == TQ_Q6_K;
}
// K-tile = one wire block; 16 rows of it make one device tile.
TQ_HD int tq_tile_bytes(int dtype) { return tq_block_bytes(dtype) * TQ_TILE_ROWS; }

constexpr int TQ_Q8_0_QS = 32;
constexpr int TQ_Q4K_QS = 256;
constexpr int TQ_Q5K_QH = 256;
constexpr int TQ_Q5K_QS = 768;
constexpr int TQ_Q6K_D = 256;
constexpr int TQ_Q6K_QL = 288;
constexpr int TQ_Q6K_QH = 2336;

// Source of one 32-bit word of a device tile.
//   word index w in [0, tile_bytes/4); returns the word assembled from wire bytes.
//   `blk(r)` must return a pointer to the wire block of tile row r (or nullptr for a padded
//   row, which reads as zero).
template <class BlockOf>
TQ_HD uint32_t tq_tile_word(int dtype, int w, BlockOf blk) {
  auto byte_at = [&](int r, int off) -> uint32_t {
    const uint8_t* p = blk(r);
    return p ? (uint32_t)p[off] : 0u;
  };
  auto word_at = [&](int r, int off) -> uint32_t {
    return byte_at(r, off) | (byte_at(r, off + 1) << 8) | (byte_at(r, off + 2) << 16) |
           (byte_at(r, off + 3) << 24);
  };
  const int b = w * 4;  // byte offset in tile
  // chunk decoding helper: byte offset inside a [lane][16 B] region -> (row, 8-byte half offset)
  auto lane_piece = [&](int rel, int* row, int* c, int* off8) {
    int l = (rel >> 4) & 31, in = rel & 15;
    *row = (l >> 2) + (in >= 8 ? 8 : 0);
    *c = l & 3;
    *off8 = in & 7;
  };
  switch (dtype) {
    case TQ_Q8_0: {
      if (b < TQ_Q8_0_QS) {  // two f16 scales per word
        int r = b >> 1;
        return byte_at(r, 0) | (byte_at(r, 1) << 8) | (byte_at(r + 1, 0) << 16) | (byte_at(r + 1, 1) << 24);
      }
      int row, c, o;
      lane_piece(b - TQ_Q8_0_QS, &row, &c, &o);
      return word_at(row, 2 + 8 * c + o);
    }
    case TQ_Q4_K:
    case TQ_Q5_K: {
      if (b < 256) return word_at(b >> 4, b & 15);
      int row, c, o;
      if (dtype == TQ_Q5_K && b < TQ_Q5K_QS) {
        lane_piece(b - TQ_Q5K_QH, &row, &c, &o);
        return word_at(row, 16 + 8 * c + o);
      }
      int qs_tile = dtype == TQ_Q4_K ? TQ_Q4K_QS : TQ_Q5K_QS;
      int qs_wire = dtype == TQ_Q4_K ? 16 : 48;
      int rel = b - qs_tile;
      int i = rel >> 9;
      lane_piece(rel & 511, &row, &c, &o);
      return word_at(row, qs_wire + 32 * i + 8 * c + o);
    }
    case TQ_Q6_K: {
      if (b < 256) return word_at(b >> 4, 192 + (b & 15));
      if (b < TQ_Q6K_QL) {
        int r = (b - TQ_Q6K_D) >> 1;
        return byte_at(r, 208) | (byte_at(r, 209) << 8) | (byte_at(r + 1, 208) << 16) | (byte_at(r + 1, 209) << 24);
      }
      // 6-bit value of element E of row r, straight from the wire block
      auto q6 = [&](int r, int E) -> uint32_t {
        int h = E >> 7, rr = E & 127, l = rr & 31, grp = rr >> 5;
        uint32_t ql = byte_at(r, 64 * h + 32 * (grp & 1) + l);
        uint32_t qh = byte_at(r, 128 + 32 * h + l);
        uint32_t lo = (grp >> 1) ? (ql >> 4) : (ql & 0x0F);
        return lo | (((qh >> (2 * grp)) & 3) << 4);
      };
      int row, c, o;
      uint32_t out = 0;
      if (b < TQ_Q6K_QH) {
        int rel = b - TQ_Q6K_QL;
        int i = rel >> 9;
        lane_piece(rel & 511, &row, &c, &o);
        int t = 2 * i + (o >> 2);
        for (int e = 0; e < 4; e++) {
          uint32_t lo = q6(row, 32 * t + 4 * c + e) & 0x0F;
          uint32_t hi = q6(row, 32 * t + 16 + 4 * c + e) & 0x0F;
          out |= (lo | (hi << 4)) << (8 * e);
        }
        return out;
      }
      int rel = b - TQ_Q6K_QH;
      int h = rel >> 9;
      lane_piece(rel & 511, &row, &c, &o);
      int u = 2 * h + (o >> 2);
      for (int e = 0; e < 4; e++) {
        uint32_t byte = 0;
        for (int s = 0; s < 4; s++) byte |= (q6(row, 16 * (4 * u + s) + 4 * c + e) >> 4) << (2 * s);
        out |= byte << (8 * e);
      }
      return out;
    }
    default: return 0;
  }
}

// 6-bit scale / min of sub-block j from the 12 packed bytes held as three words
// (gguf-py quants.py:479-500).
TQ_HD void tq_k4_scale_min(uint32_t s0, uint32_t s1, uint32_t s2, int j, int* sc, int* mn) {
  if (j < 4) {
    *sc = (s0 >> (8 * j)) & 63;
    *mn = (s1 >> (8 * j)) & 63;
  } else {
    int jj = j - 4;
    uint32_t hi = (s2 >> (8 * jj)) & 0xFF;
    *sc = (hi & 0x0F) | (((s0 >> (8 * jj + 6)) & 3) << 4);
    *mn = (hi >> 4) | (((s1 >> (8 * jj + 6)) & 3) << 4);
  }
}
