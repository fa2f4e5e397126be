// Host-side conversion between the reference's row-major block arrays
// (include/lutmac/types.hpp:126-465, the same bytes src/format.cpp:463-496 reads from a
// .lutmac file) and the device tile layout described in common.cuh.  Pure integer/byte
// shuffling: lossless, and checked bit-exact by the round-trip tests.
#include <algorithm>
#include <cstring>
#include <thread>
#include <vector>

#include "common.cuh"

namespace lmb {

namespace {

inline unsigned stream_get(const uint8_t *data, size_t nbytes, size_t idx, unsigned bits) {
  // MSB-first bit stream read through a 16-bit window (types.hpp:255-266, :302-314, :350-362)
  size_t bit = idx * bits, byte = bit / 8;
  unsigned off = unsigned(bit % 8);
  unsigned word = unsigned(data[byte]) << 8;
  if (byte + 1 < nbytes) word |= data[byte + 1];
  return (word >> (16 - bits - off)) & ((1u << bits) - 1u);
}

inline void stream_set(uint8_t *data, size_t nbytes, size_t idx, unsigned bits, unsigned val) {
  size_t bit = idx * bits, byte = bit / 8;
  unsigned off = unsigned(bit % 8), sh = 16 - bits - off, m = (1u << bits) - 1u;
  unsigned word = unsigned(data[byte]) << 8;
  if (byte + 1 < nbytes) word |= data[byte + 1];
  word = ((word & ~(m << sh)) | ((val & m) << sh)) & 0xFFFFu;
  data[byte] = uint8_t(word >> 8);
  if (byte + 1 < nbytes) data[byte + 1] = uint8_t(word & 0xFF);
}

inline void plane_set(uint8_t *plane, size_t i, unsigned bit) {  // MSB-first, like pack_to_bitplanes
  if (bit) plane[i / 8] |= uint8_t(1u << (7 - (i % 8)));
}
inline unsigned plane_get(const uint8_t *plane, size_t i) { return (plane[i / 8] >> (7 - (i % 8))) & 1u; }

// One reference block -> the lane's payload (chunks*16 bytes) and scales.
void block_to_lane(int kind, const uint8_t *blk, uint8_t *pay, float *sc) {
  switch (kind) {
  case LMB_TERNARY: {
    const uint8_t *sign = blk, *zero = blk + 32;
    for (int c = 0; c < 4; ++c)
      for (int j = 0; j < 8; ++j) {
        uint8_t s = sign[8 * c + j], z = zero[8 * c + j];
        pay[16 * c + j] = uint8_t(~z & ~s);
        pay[16 * c + 8 + j] = uint8_t(~z & s);
      }
    std::memcpy(sc, blk + 64, 4);
    break;
  }
  case DK_TERNARY_MMA: {  // row-major 2-bit codes t+1 (column c in byte c/4, bits 2(c%4)); permuted per tile later
    const uint8_t *sign = blk, *zero = blk + 32;
    std::memset(pay, 0, 64);
    for (size_t i = 0; i < 256; ++i) {
      const unsigned z = plane_get(zero, i), sg = plane_get(sign, i);
      const unsigned code = z ? 1u : (sg ? 0u : 2u);
      pay[i / 4] |= uint8_t(code << (2 * (i % 4)));
    }
    std::memcpy(sc, blk + 64, 4);
    break;
  }
  case LMB_BINARY:
  case DK_BINARY_MMA:  // row-major sign bits; permuted per tile later
    std::memcpy(pay, blk, 32);
    std::memcpy(sc, blk + 32, 4);
    break;
  case DK_INT2_MMA: {  // row-major 2-bit fields b1 | b2 << 1 (column c in byte c/4, bits 2(c%4)); permuted per tile later
    std::memset(pay, 0, 64);
    for (size_t i = 0; i < 256; ++i) {
      const unsigned code = (blk[i / 4] >> (6 - 2 * (i % 4))) & 3u;  // (b1 << 1) | b2, types.hpp Int2Block
      pay[i / 4] |= uint8_t(((code >> 1) | ((code & 1u) << 1)) << (2 * (i % 4)));
    }
    std::memcpy(sc, blk + 64, 8);
    break;
  }
  case LMB_INT2: {
    uint8_t b1[32] = {0}, b2[32] = {0};
    for (size_t i = 0; i < 256; ++i) {
      unsigned code = (blk[i / 4] >> (6 - 2 * (i % 4))) & 3u;
      plane_set(b1, i, code >> 1);
      plane_set(b2, i, code & 1u);
    }
    for (int c = 0; c < 4; ++c) {
      std::memcpy(pay + 16 * c, b1 + 8 * c, 8);
      std::memcpy(pay + 16 * c + 8, b2 + 8 * c, 8);
    }
    std::memcpy(sc, blk + 64, 8);
    break;
  }
  case LMB_INT3: {
    uint8_t q[3][32];
    std::memset(q, 0, sizeof q);
    for (size_t i = 0; i < 256; ++i) {
      unsigned code = stream_get(blk, 96, i, 3);
      for (int p = 0; p < 3; ++p) plane_set(q[p], i, (code >> p) & 1u);
    }
    for (int j = 0; j < 2; ++j)
      for (int p = 0; p < 3; ++p) std::memcpy(pay + 16 * (3 * j + p), q[2 - p] + 16 * j, 16);
    std::memcpy(sc, blk + 96, 4);
    break;
  }
  case DK_INT3_MMA: {  // three row-major MSB-first bit planes, least significant first; permuted per tile later
    std::memset(pay, 0, 96);
    for (size_t i = 0; i < 256; ++i) {
      unsigned code = stream_get(blk, 96, i, 3);
      for (int p = 0; p < 3; ++p) plane_set(pay + 32 * p, i, (code >> p) & 1u);
    }
    std::memcpy(sc, blk + 96, 4);
    break;
  }
  case LMB_INT4:
    std::memcpy(pay, blk, 128);
    std::memcpy(sc, blk + 128, 4);
    break;
  case LMB_INT5:
  case LMB_INT6: {
    const unsigned bits = unsigned(kind);
    const size_t nbytes = 32 * bits;
    std::memset(pay, 0, 16 * size_t(kind_info(kind).chunks));
    for (size_t i = 0; i < 256; ++i) {
      unsigned code = stream_get(blk, nbytes, i, bits);
      unsigned nib = code & 15u;
      pay[i / 2] |= uint8_t((i % 2 == 0) ? (nib << 4) : nib);
      plane_set(pay + 128, i, (code >> 4) & 1u);
      if (bits == 6) plane_set(pay + 160, i, (code >> 5) & 1u);
    }
    std::memcpy(sc, blk + nbytes, 4);
    break;
  }
  case LMB_INT8:
  case DK_INT8_MMA:  // row-major bytes; permuted per tile later
    std::memcpy(sc, blk, 4);
    std::memcpy(pay, blk + 4, 256);
    break;
  }
}

void lane_to_block(int kind, const uint8_t *pay, const float *sc, uint8_t *blk) {
  switch (kind) {
  case LMB_TERNARY:
    for (int c = 0; c < 4; ++c)
      for (int j = 0; j < 8; ++j) {
        uint8_t p = pay[16 * c + j], n = pay[16 * c + 8 + j];
        blk[8 * c + j] = n;                      // sign plane
        blk[32 + 8 * c + j] = uint8_t(~(p | n));  // zero plane
      }
    std::memcpy(blk + 64, sc, 4);
    break;
  case DK_TERNARY_MMA: {
    std::memset(blk, 0, 64);
    for (size_t i = 0; i < 256; ++i) {
      const unsigned code = (pay[i / 4] >> (2 * (i % 4))) & 3u;
      if (code == 0) plane_set(blk, i, 1);       // sign plane
      if (code == 1) plane_set(blk + 32, i, 1);  // zero plane
    }
    std::memcpy(blk + 64, sc, 4);
    break;
  }
  case LMB_BINARY:
  case DK_BINARY_MMA:
    std::memcpy(blk, pay, 32);
    std::memcpy(blk + 32, sc, 4);
    break;
  case DK_INT2_MMA: {
    std::memset(blk, 0, 64);
    for (size_t i = 0; i < 256; ++i) {
      const unsigned f = (pay[i / 4] >> (2 * (i % 4))) & 3u;  // b1 | b2 << 1
      blk[i / 4] |= uint8_t((((f & 1u) << 1) | (f >> 1)) << (6 - 2 * (i % 4)));
    }
    std::memcpy(blk + 64, sc, 8);
    break;
  }
  case LMB_INT2: {
    uint8_t b1[32], b2[32];
    for (int c = 0; c < 4; ++c) {
      std::memcpy(b1 + 8 * c, pay + 16 * c, 8);
      std::memcpy(b2 + 8 * c, pay + 16 * c + 8, 8);
    }
    std::memset(blk, 0, 64);
    for (size_t i = 0; i < 256; ++i) {
      unsigned code = (plane_get(b1, i) << 1) | plane_get(b2, i);
      blk[i / 4] |= uint8_t(code << (6 - 2 * (i % 4)));
    }
    std::memcpy(blk + 64, sc, 8);
    break;
  }
  case LMB_INT3: {
    uint8_t q[3][32];
    for (int j = 0; j < 2; ++j)
      for (int p = 0; p < 3; ++p) std::memcpy(q[2 - p] + 16 * j, pay + 16 * (3 * j + p), 16);
    std::memset(blk, 0, 96);
    for (size_t i = 0; i < 256; ++i) {
      unsigned code = plane_get(q[0], i) | (plane_get(q[1], i) << 1) | (plane_get(q[2], i) << 2);
      stream_set(blk, 96, i, 3, code);
    }
    std::memcpy(blk + 96, sc, 4);
    break;
  }
  case DK_INT3_MMA: {
    std::memset(blk, 0, 96);
    for (size_t i = 0; i < 256; ++i) {
      unsigned code = plane_get(pay, i) | (plane_get(pay + 32, i) << 1) | (plane_get(pay + 64, i) << 2);
      stream_set(blk, 96, i, 3, code);
    }
    std::memcpy(blk + 96, sc, 4);
    break;
  }
  case LMB_INT4:
    std::memcpy(blk, pay, 128);
    std::memcpy(blk + 128, sc, 4);
    break;
  case LMB_INT5:
  case LMB_INT6: {
    const unsigned bits = unsigned(kind);
    const size_t nbytes = 32 * bits;
    std::memset(blk, 0, nbytes);
    for (size_t i = 0; i < 256; ++i) {
      unsigned nib = (i % 2 == 0) ? (pay[i / 2] >> 4) : (pay[i / 2] & 15u);
      unsigned code = nib | (plane_get(pay + 128, i) << 4);
      if (bits == 6) code |= plane_get(pay + 160, i) << 5;
      stream_set(blk, nbytes, i, bits, code);
    }
    std::memcpy(blk + nbytes, sc, 4);
    break;
  }
  case LMB_INT8:
  case DK_INT8_MMA:
    std::memcpy(blk, sc, 4);
    std::memcpy(blk + 4, pay, 256);
    break;
  }
}

// INT4 and DK_TERNARY_MMA tiles are stored in the operand order of the 8-bit integer MMA
// (m16n8k32).  Lane (g, tid) of a warp owns, for k-step s (columns 32s..32s+31), a word WA whose
// byte j belongs to column 32s+4tid+j and a word WB whose byte j belongs to column 32s+16+4tid+j;
// inside every byte several ROWS share the bits:
//   INT4     low nibble = row 16h+g, high nibble = row 16h+g+8; chunk h*4+q = {WA(2q), WB(2q), WA(2q+1), WB(2q+1)}
//   ternary  2-bit field m = row g+8m;                         chunk q     = {WA(2q), WB(2q), WA(2q+1), WB(2q+1)}
// so `word & field_mask` is an A-operand register of that row (scaled by the field's power of
// two) without a shift.  A pure permutation of the codes of the 32 row-blocks of a tile.  The
// scales of these kinds are stored in the matching order: float 4g+m = scale of row g+8m.
inline unsigned int4_code(const uint8_t *rowmajor, size_t row, size_t col) {
  const size_t jb = col / 2;
  const uint8_t byte = rowmajor[(jb / 16) * 512 + row * 16 + jb % 16];
  return (col % 2 == 0) ? (byte >> 4) : (byte & 15u);
}
inline void int4_set(uint8_t *rowmajor, size_t row, size_t col, unsigned code) {
  const size_t jb = col / 2;
  uint8_t &byte = rowmajor[(jb / 16) * 512 + row * 16 + jb % 16];
  byte = (col % 2 == 0) ? uint8_t((byte & 0x0F) | (code << 4)) : uint8_t((byte & 0xF0) | code);
}
// fn(index of the byte in the tile, row of the low nibble (the high nibble is row + 8), column)
template <class Fn> inline void int4_fragment_walk(Fn &&fn) {
  for (size_t h = 0; h < 2; ++h)
    for (size_t q = 0; q < 4; ++q)
      for (size_t g = 0; g < 8; ++g)
        for (size_t tid = 0; tid < 4; ++tid)
          for (size_t wi = 0; wi < 4; ++wi)
            for (size_t j = 0; j < 4; ++j) {
              const size_t s = 2 * q + wi / 2, col = 32 * s + 16 * (wi % 2) + 4 * tid + j;
              fn(((h * 4 + q) * 32 + g * 4 + tid) * 16 + wi * 4 + j, 16 * h + g, col);
            }
}
void int4_to_fragments(uint8_t *payload) {  // 4096 bytes, in place
  uint8_t src[4096];
  std::memcpy(src, payload, 4096);
  int4_fragment_walk([&](size_t idx, size_t row, size_t col) {
    payload[idx] = uint8_t((int4_code(src, row + 8, col) << 4) | int4_code(src, row, col));
  });
}
void int4_from_fragments(uint8_t *payload) {
  uint8_t src[4096];
  std::memcpy(src, payload, 4096);
  std::memset(payload, 0, 4096);
  int4_fragment_walk([&](size_t idx, size_t row, size_t col) {
    int4_set(payload, row, col, src[idx] & 15u);
    int4_set(payload, row + 8, col, src[idx] >> 4);
  });
}

// fn(index of the byte in the tile, bit offset of the field, row, column)
template <class Fn> inline void tern_fragment_walk(Fn &&fn) {
  for (size_t q = 0; q < 4; ++q)
    for (size_t g = 0; g < 8; ++g)
      for (size_t tid = 0; tid < 4; ++tid)
        for (size_t wi = 0; wi < 4; ++wi)
          for (size_t j = 0; j < 4; ++j)
            for (size_t m = 0; m < 4; ++m) {
              const size_t s = 2 * q + wi / 2, col = 32 * s + 16 * (wi % 2) + 4 * tid + j;
              fn((q * 32 + g * 4 + tid) * 16 + wi * 4 + j, 2 * m, g + 8 * m, col);
            }
}
inline unsigned tern_code(const uint8_t *rowmajor, size_t row, size_t col) {
  const size_t jb = col / 4;
  return (rowmajor[(jb / 16) * 512 + row * 16 + jb % 16] >> (2 * (col % 4))) & 3u;
}
void tern_to_fragments(uint8_t *payload) {  // 2048 bytes, in place
  uint8_t src[2048];
  std::memcpy(src, payload, 2048);
  std::memset(payload, 0, 2048);
  tern_fragment_walk([&](size_t idx, size_t shift, size_t row, size_t col) {
    payload[idx] |= uint8_t(tern_code(src, row, col) << shift);
  });
}
void tern_from_fragments(uint8_t *payload) {
  uint8_t src[2048];
  std::memcpy(src, payload, 2048);
  std::memset(payload, 0, 2048);
  tern_fragment_walk([&](size_t idx, size_t shift, size_t row, size_t col) {
    const unsigned code = (src[idx] >> shift) & 3u;
    const size_t jb = col / 4;
    payload[(jb / 16) * 512 + row * 16 + jb % 16] |= uint8_t(code << (2 * (col % 4)));
  });
}

// fn(index of the byte in the tile, bit, row, column)
template <class Fn> inline void bin_fragment_walk(Fn &&fn) {
  for (size_t wi = 0; wi < 8; ++wi)
    for (size_t g = 0; g < 8; ++g)
      for (size_t tid = 0; tid < 4; ++tid)
        for (size_t j = 0; j < 4; ++j)
          for (size_t m = 0; m < 4; ++m)
            for (size_t kh = 0; kh < 2; ++kh) {
              const size_t sp = wi / 2, ab = wi % 2, col = 32 * (2 * sp + kh) + 16 * ab + 4 * tid + j;
              fn(((wi / 4) * 32 + g * 4 + tid) * 16 + (wi % 4) * 4 + j, m + 4 * kh, g + 8 * m, col);
            }
}
void bin_to_fragments(uint8_t *payload) {  // 1024 bytes, in place
  uint8_t src[1024];
  std::memcpy(src, payload, 1024);
  std::memset(payload, 0, 1024);
  bin_fragment_walk([&](size_t idx, size_t bit, size_t row, size_t col) {
    const size_t jb = col / 8;
    const unsigned v = (src[(jb / 16) * 512 + row * 16 + jb % 16] >> (7 - col % 8)) & 1u;
    payload[idx] |= uint8_t(v << bit);
  });
}
void bin_from_fragments(uint8_t *payload) {
  uint8_t src[1024];
  std::memcpy(src, payload, 1024);
  std::memset(payload, 0, 1024);
  bin_fragment_walk([&](size_t idx, size_t bit, size_t row, size_t col) {
    const size_t jb = col / 8;
    const unsigned v = (src[idx] >> bit) & 1u;
    payload[(jb / 16) * 512 + row * 16 + jb % 16] |= uint8_t(v << (7 - col % 8));
  });
}

// fn(index of the byte in the tile, row, column)
template <class Fn> inline void int8_fragment_walk(Fn &&fn) {
  for (size_t h = 0; h < 2; ++h)
    for (size_t st = 0; st < 8; ++st)
      for (size_t g = 0; g < 8; ++g)
        for (size_t tid = 0; tid < 4; ++tid)
          for (size_t a = 0; a < 4; ++a)
            for (size_t j = 0; j < 4; ++j)
              fn(((h * 8 + st) * 32 + g * 4 + tid) * 16 + a * 4 + j, 16 * h + g + 8 * (a % 2), 32 * st + 16 * (a / 2) + 4 * tid + j);
}
void int8_to_fragments(uint8_t *payload) {  // 8192 bytes, in place
  std::vector<uint8_t> src(payload, payload + 8192);
  int8_fragment_walk([&](size_t idx, size_t row, size_t col) { payload[idx] = src[(col / 16) * 512 + row * 16 + col % 16]; });
}
void int8_from_fragments(uint8_t *payload) {
  std::vector<uint8_t> src(payload, payload + 8192);
  int8_fragment_walk([&](size_t idx, size_t row, size_t col) { payload[(col / 16) * 512 + row * 16 + col % 16] = src[idx]; });
}

// scale of row l of a tile: index into the tile's scale array
inline size_t scale_slot(int kind, size_t l) { return kind_is_mma(kind) ? 4 * (l % 8) + l / 8 : l; }

template <class F> void parallel_tiles(size_t n, F &&f) {
  unsigned hw = std::max(1u, std::thread::hardware_concurrency());
  size_t nt = std::min<size_t>(hw, std::max<size_t>(1, n / 64));
  if (nt <= 1) {
    for (size_t i = 0; i < n; ++i) f(i);
    return;
  }
  std::vector<std::thread> th;
  for (size_t t = 0; t < nt; ++t)
    th.emplace_back([&, t] {
      for (size_t i = n * t / nt; i < n * (t + 1) / nt; ++i) f(i);
    });
  for (auto &x : th) x.join();
}

}  // namespace

// Re-tile rows [row0,row1) x block-columns [blk0,blk1) of a reference block array with
// src_bpr block-columns per row.
void retile(int kind, const uint8_t *blocks, size_t src_bpr, size_t row0, size_t row1, size_t blk0,
            size_t blk1, uint8_t *tiled) {
  const KindInfo ki = kind_info(kind);
  const size_t M = row1 - row0, bpr = blk1 - blk0, row_tiles = (M + TILE_ROWS - 1) / TILE_ROWS;
  const size_t tb = tile_bytes(kind);
  parallel_tiles(row_tiles, [&](size_t rt) {
    std::vector<uint8_t> pay(size_t(ki.chunks) * 16);
    float sc[2];
    for (size_t b = 0; b < bpr; ++b) {
      uint8_t *tile = tiled + (rt * bpr + b) * tb;
      std::memset(tile, 0, tb);  // rows beyond M: zero payload, zero scales
      for (size_t l = 0; l < TILE_ROWS; ++l) {
        size_t r = rt * TILE_ROWS + l;
        if (r >= M) break;
        const uint8_t *blk = blocks + ((row0 + r) * src_bpr + blk0 + b) * size_t(ki.ref_bytes);
        sc[0] = sc[1] = 0.0f;
        block_to_lane(kind, blk, pay.data(), sc);
        for (int c = 0; c < ki.chunks; ++c) std::memcpy(tile + (size_t(c) * TILE_ROWS + l) * 16, pay.data() + 16 * c, 16);
        float *ts = reinterpret_cast<float *>(tile + size_t(ki.chunks) * TILE_ROWS * 16);
        for (int s = 0; s < ki.nscales; ++s) ts[size_t(s) * TILE_ROWS + scale_slot(kind, l)] = sc[s];
      }
      if (kind == LMB_INT4 || kind == LMB_INT5 || kind == LMB_INT6) int4_to_fragments(tile);
      if (kind == LMB_INT5 || kind == LMB_INT6) bin_to_fragments(tile + 4096);
      if (kind == LMB_INT6) bin_to_fragments(tile + 5120);
      if (kind == DK_INT8_MMA) int8_to_fragments(tile);
      if (kind == DK_INT3_MMA)
        for (size_t pl = 0; pl < 3; ++pl) bin_to_fragments(tile + 1024 * pl);
      if (kind == DK_TERNARY_MMA || kind == DK_INT2_MMA) tern_to_fragments(tile);
      if (kind == DK_BINARY_MMA) bin_to_fragments(tile);
    }
  });
}

void untile(int kind, const uint8_t *tiled, size_t M, size_t bpr, uint8_t *blocks) {
  const KindInfo ki = kind_info(kind);
  const size_t row_tiles = (M + TILE_ROWS - 1) / TILE_ROWS, tb = tile_bytes(kind);
  parallel_tiles(row_tiles, [&](size_t rt) {
    std::vector<uint8_t> pay(size_t(ki.chunks) * 16);
    float sc[2];
    for (size_t b = 0; b < bpr; ++b) {
      const uint8_t *tile = tiled + (rt * bpr + b) * tb;
      uint8_t rowmajor[8192];
      if (kind == LMB_INT4 || kind == LMB_INT5 || kind == LMB_INT6) {
        std::memcpy(rowmajor, tile, size_t(ki.chunks) * 512);
        int4_from_fragments(rowmajor);
        if (kind != LMB_INT4) bin_from_fragments(rowmajor + 4096);
        if (kind == LMB_INT6) bin_from_fragments(rowmajor + 5120);
      } else if (kind == DK_INT3_MMA) {
        std::memcpy(rowmajor, tile, 3072);
        for (size_t pl = 0; pl < 3; ++pl) bin_from_fragments(rowmajor + 1024 * pl);
      } else if (kind == DK_INT8_MMA) {
        std::memcpy(rowmajor, tile, 8192);
        int8_from_fragments(rowmajor);
      } else if (kind == DK_TERNARY_MMA || kind == DK_INT2_MMA) {
        std::memcpy(rowmajor, tile, 2048);
        tern_from_fragments(rowmajor);
      } else if (kind == DK_BINARY_MMA) {
        std::memcpy(rowmajor, tile, 1024);
        bin_from_fragments(rowmajor);
      }
      const uint8_t *paysrc = kind_is_mma(kind) ? rowmajor : tile;
      for (size_t l = 0; l < TILE_ROWS; ++l) {
        size_t r = rt * TILE_ROWS + l;
        if (r >= M) break;
        for (int c = 0; c < ki.chunks; ++c) std::memcpy(pay.data() + 16 * c, paysrc + (size_t(c) * TILE_ROWS + l) * 16, 16);
        const float *ts = reinterpret_cast<const float *>(tile + size_t(ki.chunks) * TILE_ROWS * 16);
        for (int s = 0; s < ki.nscales; ++s) sc[s] = ts[size_t(s) * TILE_ROWS + scale_slot(kind, l)];
        lane_to_block(kind, pay.data(), sc, blocks + (r * bpr + b) * size_t(ki.ref_bytes));
      }
    }
  });
}

}  // namespace lmb

extern "C" {

size_t lmb_block_bytes(int kind) { return size_t(lmb::kind_info(kind).ref_bytes); }

size_t lmb_tiled_bytes(int kind, size_t M, size_t K) {
  if (!lmb::kind_valid(kind)) return 0;
  size_t bpr = (K + lmb::BLK - 1) / lmb::BLK, rt = (M + lmb::TILE_ROWS - 1) / lmb::TILE_ROWS;
  return rt * bpr * lmb::tile_bytes(kind);
}

int lmb_retile_host(int kind, const void *blocks, size_t M, size_t K, void *tiled) {
  LMB_REQUIRE(lmb::kind_valid(kind), "lmb_retile_host: unknown block kind");
  LMB_REQUIRE(blocks && tiled && M > 0 && K > 0, "lmb_retile_host: null pointer or empty shape");
  size_t bpr = (K + lmb::BLK - 1) / lmb::BLK;
  lmb::retile(kind, static_cast<const uint8_t *>(blocks), bpr, 0, M, 0, bpr, static_cast<uint8_t *>(tiled));
  return LMB_OK;
}

int lmb_untile_host(int kind, const void *tiled, size_t M, size_t K, void *blocks_out) {
  LMB_REQUIRE(lmb::kind_valid(kind), "lmb_untile_host: unknown block kind");
  LMB_REQUIRE(blocks_out && tiled && M > 0 && K > 0, "lmb_untile_host: null pointer or empty shape");
  size_t bpr = (K + lmb::BLK - 1) / lmb::BLK;
  lmb::untile(kind, static_cast<const uint8_t *>(tiled), M, bpr, static_cast<uint8_t *>(blocks_out));
  return LMB_OK;
}

}  // extern "C"
