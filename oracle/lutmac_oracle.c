/*
 * TEST INFRASTRUCTURE ONLY -- see lutmac_oracle.h.  Plain-C restatement of the LutMac
 * decode hot path.  Each function names the reference file:line it follows.
 * Built without -ffast-math so that its results do not depend on the compiler.
 */
#include "lutmac_oracle.h"

#include <math.h>
#include <pthread.h>
#include <stdlib.h>
#include <string.h>

#define BLK 256

size_t orc_block_bytes(int kind) {
  switch (kind) {
  case ORC_TERNARY: return sizeof(orc_ternary_block);
  case ORC_BINARY: return sizeof(orc_binary_block);
  case ORC_INT2: return sizeof(orc_int2_block);
  case ORC_INT3: return sizeof(orc_int3_block);
  case ORC_INT4: return sizeof(orc_int4_block);
  case ORC_INT5: return sizeof(orc_int5_block);
  case ORC_INT6: return sizeof(orc_int6_block);
  case ORC_INT8: return sizeof(orc_int8_block);
  default: return 0;
  }
}

/* ---------------------------------------------------------------------------------------
 * LUT helpers
 * ------------------------------------------------------------------------------------- */

/* include/lutmac/lut_gemm.hpp:30-44 -- entry bit 3 selects a0 ... bit 0 selects a3; the
 * additions happen in the order a0, a1, a2, a3. */
void orc_precompute_lut(const float *a, float *lut) {
  lut[0] = 0.0f;
  for (int i = 1; i < 16; ++i) {
    float s = 0.0f;
    if (i & 8) s += a[0];
    if (i & 4) s += a[1];
    if (i & 2) s += a[2];
    if (i & 1) s += a[3];
    lut[i] = s;
  }
}

/* include/lutmac/lut_gemm.hpp:53-58 */
void orc_precompute_luts(const float *act, size_t n, float *luts) {
  for (size_t g = 0; g < n / 4; ++g) orc_precompute_lut(act + 4 * g, luts + 16 * g);
}

/* include/lutmac/lut_gemm.hpp:79-99 -- group g lives in byte g/2, high nibble when g is
 * even; pos = ~zero & ~sign, neg = ~zero & sign. */
void orc_extract_indices(const uint8_t *sign_plane, const uint8_t *zero_plane, size_t g,
                         uint8_t *pos_idx, uint8_t *neg_idx) {
  size_t byte_idx = g / 2;
  unsigned shift = (g % 2) ? 0u : 4u;
  uint8_t s = (uint8_t)((sign_plane[byte_idx] >> shift) & 0x0F);
  uint8_t z = (uint8_t)((zero_plane[byte_idx] >> shift) & 0x0F);
  uint8_t nz = (uint8_t)((~z) & 0x0F);
  *pos_idx = (uint8_t)(nz & (uint8_t)(~s));
  *neg_idx = (uint8_t)(nz & s);
}

/* ---------------------------------------------------------------------------------------
 * FWHT -- src/kernels/transform_simd.cpp:14-23 (stride 1,2 passes), :33-36,57-64 (generic
 * butterfly for strides 4..128), :82,95-97 (multiply by 1/16).  The AVX2 branch of that
 * file (:46-55) overlaps its own operands at stride 4 and is not the parity target.
 * ------------------------------------------------------------------------------------- */
void orc_fwht_256(float *d) {
  for (size_t h = 1; h < BLK; h <<= 1)
    for (size_t i = 0; i < BLK; i += 2 * h)
      for (size_t j = i; j < i + h; ++j) {
        float x = d[j], y = d[j + h];
        d[j] = x + y;
        d[j + h] = x - y;
      }
  for (size_t i = 0; i < BLK; ++i) d[i] *= (1.0f / 16.0f);
}

/* src/kernels/transform_simd.cpp:101-110 -- a trailing partial block is left untouched */
void orc_apply_hadamard_rotation(float *d, size_t n) {
  for (size_t i = 0; i + BLK <= n; i += BLK) orc_fwht_256(d + i);
}

/* ---------------------------------------------------------------------------------------
 * Weight accessors (Block::get without the scale), include/lutmac/types.hpp
 * ------------------------------------------------------------------------------------- */
static inline unsigned bitstream_get(const uint8_t *data, size_t nbytes, size_t idx, unsigned bits) {
  /* types.hpp:255-266 (3-bit), :302-314 (5-bit), :350-362 (6-bit): MSB-first stream read
   * through a 16-bit window whose low byte is 0 past the end of the array. */
  size_t bit_idx = idx * bits;
  size_t byte_idx = bit_idx / 8;
  unsigned off = (unsigned)(bit_idx % 8);
  unsigned word = (unsigned)data[byte_idx] << 8;
  if (byte_idx + 1 < nbytes) word |= data[byte_idx + 1];
  return (word >> (16 - bits - off)) & ((1u << bits) - 1u);
}

static inline int ternary_at(const orc_ternary_block *b, size_t i) { /* types.hpp:140-148 */
  unsigned bit = 7u - (unsigned)(i % 8);
  if ((b->zero_plane[i / 8] >> bit) & 1) return 0;
  return ((b->sign_plane[i / 8] >> bit) & 1) ? -1 : 1;
}
static inline int binary_at(const orc_binary_block *b, size_t i) { /* types.hpp:404-411 */
  return ((b->data[i / 8] >> (7u - (unsigned)(i % 8))) & 1) ? 1 : -1;
}
static inline unsigned int2_code(const orc_int2_block *b, size_t i) { /* types.hpp:217-221 */
  return (b->data[i / 4] >> (6u - 2u * (unsigned)(i % 4))) & 3u;
}
static inline int int4_at(const orc_int4_block *b, size_t i) { /* types.hpp:184-190 */
  uint8_t byte = b->data[i / 2];
  unsigned nib = (i % 2 == 0) ? (byte >> 4) : (byte & 0x0F);
  return (int)nib - 8;
}

float orc_block_get(int kind, const void *block, size_t i) {
  switch (kind) {
  case ORC_TERNARY: { const orc_ternary_block *b = block; return (float)ternary_at(b, i) * b->scale; }
  case ORC_BINARY: { const orc_binary_block *b = block; return (float)binary_at(b, i) * b->scale; }
  case ORC_INT2: { /* types.hpp:217-234: +-scale +- scale2, bit1 = primary, bit0 = residual */
    const orc_int2_block *b = block;
    unsigned c = int2_code(b, i);
    return ((c & 2) ? b->scale : -b->scale) + ((c & 1) ? b->scale2 : -b->scale2);
  }
  case ORC_INT3: { const orc_int3_block *b = block; return (float)((int)bitstream_get(b->data, 96, i, 3) - 4) * b->scale; }
  case ORC_INT4: { const orc_int4_block *b = block; return (float)int4_at(b, i) * b->scale; }
  case ORC_INT5: { const orc_int5_block *b = block; return (float)((int)bitstream_get(b->data, 160, i, 5) - 16) * b->scale; }
  case ORC_INT6: { const orc_int6_block *b = block; return (float)((int)bitstream_get(b->data, 192, i, 6) - 32) * b->scale; }
  case ORC_INT8: { const orc_int8_block *b = block; return (float)b->data[i] * b->scale; }
  default: return 0.0f;
  }
}

/* ---------------------------------------------------------------------------------------
 * GEMV kernels.  All share the loop nest of src/kernels/lut_gemm_scalar.cpp: for each row,
 * for each of ceil(K/256) blocks, a left-to-right fp32 sum over the block's 256 weights,
 * then acc += block_sum * scale.  The activation vector is read for ceil(K/256)*256
 * entries.  num_blocks is ignored by every reference kernel and is not a parameter here.
 * ------------------------------------------------------------------------------------- */
#define ROW_LOOP_BEGIN(T)                                                   \
  const size_t bpr = (K + BLK - 1) / BLK;                                   \
  for (size_t row = 0; row < M; ++row) {                                    \
    ACC acc = 0;                                                            \
    for (size_t b = 0; b < bpr; ++b) {                                      \
      const T *blk = (const T *)blocks + row * bpr + b;                     \
      const XT *x = act + b * BLK;                                          \
      ACC s = 0;
#define ROW_LOOP_END(scale_expr)                                            \
      acc += s * (ACC)(scale_expr);                                         \
    }                                                                       \
    out[row] = acc;                                                         \
  }

#define DEFINE_GEMVS(SUFFIX, ACCTYPE, XTYPE)                                                             \
  /* lut_gemm_scalar.cpp:7-61 */                                                                   \
  static void gemv_ternary_##SUFFIX(const void *blocks, const XTYPE *act, ACCTYPE *out, size_t M, size_t K) { \
    typedef ACCTYPE ACC; typedef XTYPE XT;                                                                         \
    ROW_LOOP_BEGIN(orc_ternary_block)                                                              \
    for (size_t i = 0; i < BLK; ++i) { int t = ternary_at(blk, i); if (t > 0) s += x[i]; else if (t < 0) s -= x[i]; } \
    ROW_LOOP_END(blk->scale)                                                                       \
  }                                                                                                \
  /* lut_gemm_scalar.cpp:228-259 */                                                                \
  static void gemv_binary_##SUFFIX(const void *blocks, const XTYPE *act, ACCTYPE *out, size_t M, size_t K) { \
    typedef ACCTYPE ACC; typedef XTYPE XT;                                                                         \
    ROW_LOOP_BEGIN(orc_binary_block)                                                               \
    for (size_t i = 0; i < BLK; ++i) s += (binary_at(blk, i) > 0) ? x[i] : -x[i];                  \
    ROW_LOOP_END(blk->scale)                                                                       \
  }                                                                                                \
  /* lut_gemm_scalar.cpp:298-321: sum of get(i)*x/scale, times scale.  Restated in the     */      \
  /* algebraically equal RRQ form of lut_gemm_simd.cpp:326-328 (primary sum * scale +      */      \
  /* residual sum * scale2), which is also defined when scale == 0.                        */      \
  static void gemv_int2_##SUFFIX(const void *blocks, const XTYPE *act, ACCTYPE *out, size_t M, size_t K) { \
    typedef ACCTYPE ACC;                                                                                           \
    const size_t bpr = (K + BLK - 1) / BLK;                                                        \
    for (size_t row = 0; row < M; ++row) {                                                         \
      ACC acc = 0;                                                                                 \
      for (size_t b = 0; b < bpr; ++b) {                                                           \
        const orc_int2_block *blk = (const orc_int2_block *)blocks + row * bpr + b;                \
        const XTYPE *x = act + b * BLK;                                                            \
        ACC p = 0, r = 0;                                                                          \
        for (size_t i = 0; i < BLK; ++i) {                                                         \
          unsigned c = int2_code(blk, i);                                                          \
          p += (c & 2) ? x[i] : -x[i];                                                             \
          r += (c & 1) ? x[i] : -x[i];                                                             \
        }                                                                                          \
        acc += p * (ACC)blk->scale + r * (ACC)blk->scale2;                                         \
      }                                                                                            \
      out[row] = acc;                                                                              \
    }                                                                                              \
  }                                                                                                \
  /* lut_gemm_scalar.cpp:327-350 */                                                                \
  static void gemv_int3_##SUFFIX(const void *blocks, const XTYPE *act, ACCTYPE *out, size_t M, size_t K) { \
    typedef ACCTYPE ACC; typedef XTYPE XT;                                                                         \
    ROW_LOOP_BEGIN(orc_int3_block)                                                                 \
    for (size_t i = 0; i < BLK; ++i) s += (ACC)((int)bitstream_get(blk->data, 96, i, 3) - 4) * x[i]; \
    ROW_LOOP_END(blk->scale)                                                                       \
  }                                                                                                \
  /* lut_gemm_scalar.cpp:186-222 */                                                                \
  static void gemv_int4_##SUFFIX(const void *blocks, const XTYPE *act, ACCTYPE *out, size_t M, size_t K) { \
    typedef ACCTYPE ACC; typedef XTYPE XT;                                                                         \
    ROW_LOOP_BEGIN(orc_int4_block)                                                                 \
    for (size_t i = 0; i < BLK; ++i) s += (ACC)int4_at(blk, i) * x[i];                             \
    ROW_LOOP_END(blk->scale)                                                                       \
  }                                                                                                \
  /* lut_gemm_scalar.cpp:356-389 */                                                                \
  static void gemv_int5_##SUFFIX(const void *blocks, const XTYPE *act, ACCTYPE *out, size_t M, size_t K) { \
    typedef ACCTYPE ACC; typedef XTYPE XT;                                                                         \
    ROW_LOOP_BEGIN(orc_int5_block)                                                                 \
    for (size_t i = 0; i < BLK; ++i) s += (ACC)((int)bitstream_get(blk->data, 160, i, 5) - 16) * x[i]; \
    ROW_LOOP_END(blk->scale)                                                                       \
  }                                                                                                \
  /* lut_gemm_scalar.cpp:395-428 */                                                                \
  static void gemv_int6_##SUFFIX(const void *blocks, const XTYPE *act, ACCTYPE *out, size_t M, size_t K) { \
    typedef ACCTYPE ACC; typedef XTYPE XT;                                                                         \
    ROW_LOOP_BEGIN(orc_int6_block)                                                                 \
    for (size_t i = 0; i < BLK; ++i) s += (ACC)((int)bitstream_get(blk->data, 192, i, 6) - 32) * x[i]; \
    ROW_LOOP_END(blk->scale)                                                                       \
  }                                                                                                \
  /* lut_gemm_scalar.cpp:265-292 */                                                                \
  static void gemv_int8_##SUFFIX(const void *blocks, const XTYPE *act, ACCTYPE *out, size_t M, size_t K) { \
    typedef ACCTYPE ACC; typedef XTYPE XT;                                                                         \
    ROW_LOOP_BEGIN(orc_int8_block)                                                                 \
    for (size_t i = 0; i < BLK; ++i) s += (ACC)blk->data[i] * x[i];                                \
    ROW_LOOP_END(blk->scale)                                                                       \
  }                                                                                                \
  static void gemv_dispatch_##SUFFIX(int kind, const void *blocks, const XTYPE *act, ACCTYPE *out, size_t M, size_t K) { \
    switch (kind) {                                                                                \
    case ORC_TERNARY: gemv_ternary_##SUFFIX(blocks, act, out, M, K); break;                        \
    case ORC_BINARY: gemv_binary_##SUFFIX(blocks, act, out, M, K); break;                          \
    case ORC_INT2: gemv_int2_##SUFFIX(blocks, act, out, M, K); break;                              \
    case ORC_INT3: gemv_int3_##SUFFIX(blocks, act, out, M, K); break;                              \
    case ORC_INT4: gemv_int4_##SUFFIX(blocks, act, out, M, K); break;                              \
    case ORC_INT5: gemv_int5_##SUFFIX(blocks, act, out, M, K); break;                              \
    case ORC_INT6: gemv_int6_##SUFFIX(blocks, act, out, M, K); break;                              \
    case ORC_INT8: gemv_int8_##SUFFIX(blocks, act, out, M, K); break;                              \
    default: break;                                                                                \
    }                                                                                              \
  }

DEFINE_GEMVS(f32, float, float)
DEFINE_GEMVS(f64, double, float)
DEFINE_GEMVS(d64, double, double) /* double activations too: the fp64 evaluation of a whole decode step */

void orc_gemv(int kind, const void *blocks, const float *act, float *out, size_t M, size_t K) {
  gemv_dispatch_f32(kind, blocks, act, out, M, K);
}
void orc_gemv_f64(int kind, const void *blocks, const float *act, double *out, size_t M, size_t K) {
  gemv_dispatch_f64(kind, blocks, act, out, M, K);
}

/* ---------------------------------------------------------------------------------------
 * LUT-form evaluation: the same products, obtained by table lookups with the reference's
 * group-of-4 index convention.  Used to check LUT indices and lookup-accumulate kernels.
 * ------------------------------------------------------------------------------------- */
static unsigned plane_index4(const unsigned q[4], unsigned p) {
  /* lut_gemm_simd.cpp:356-361: plane-p bits of (q0,q1,q2,q3), q0 at bit 3 */
  return (((q[0] >> p) & 1u) << 3) | (((q[1] >> p) & 1u) << 2) | (((q[2] >> p) & 1u) << 1) | ((q[3] >> p) & 1u);
}

void orc_gemv_lutform(int kind, const void *blocks, const float *act, float *out, size_t M, size_t K) {
  const size_t bpr = (K + BLK - 1) / BLK;
  float *luts = (float *)malloc(sizeof(float) * bpr * 64 * 16);
  orc_precompute_luts(act, bpr * BLK, luts);
  for (size_t row = 0; row < M; ++row) {
    float acc = 0.0f;
    for (size_t b = 0; b < bpr; ++b) {
      const float *L = luts + b * 64 * 16;
      if (kind == ORC_TERNARY) { /* lut_gemm_simd.cpp:196-221 */
        const orc_ternary_block *blk = (const orc_ternary_block *)blocks + row * bpr + b;
        float s = 0.0f;
        for (size_t g = 0; g < 64; ++g) {
          uint8_t p, n;
          orc_extract_indices(blk->sign_plane, blk->zero_plane, g, &p, &n);
          s += L[g * 16 + p] - L[g * 16 + n];
        }
        acc += s * blk->scale;
      } else if (kind == ORC_BINARY) { /* one sign plane: sum(+-x) = 2*L[idx] - L[15] */
        const orc_binary_block *blk = (const orc_binary_block *)blocks + row * bpr + b;
        float s = 0.0f;
        for (size_t g = 0; g < 64; ++g) {
          unsigned idx = (g % 2 == 0) ? (blk->data[g / 2] >> 4) : (blk->data[g / 2] & 0x0F);
          s += 2.0f * L[g * 16 + idx] - L[g * 16 + 15];
        }
        acc += s * blk->scale;
      } else if (kind == ORC_INT2) { /* lut_gemm_simd.cpp:228-333 epilogue :326-328 */
        const orc_int2_block *blk = (const orc_int2_block *)blocks + row * bpr + b;
        float p = 0.0f, r = 0.0f;
        for (size_t g = 0; g < 64; ++g) {
          unsigned q[4];
          for (int j = 0; j < 4; ++j) q[j] = int2_code(blk, 4 * g + j);
          p += 2.0f * L[g * 16 + plane_index4(q, 1)] - L[g * 16 + 15];
          r += 2.0f * L[g * 16 + plane_index4(q, 0)] - L[g * 16 + 15];
        }
        acc += p * blk->scale + r * blk->scale2;
      } else if (kind == ORC_INT3 || kind == ORC_INT4) { /* lut_gemm_simd.cpp:335-371 */
        const unsigned bits = (kind == ORC_INT3) ? 3u : 4u;
        const float zero_point = (kind == ORC_INT3) ? 4.0f : 8.0f;
        float scale, s = 0.0f, xs = 0.0f;
        const void *blkv;
        if (kind == ORC_INT3) { const orc_int3_block *blk = (const orc_int3_block *)blocks + row * bpr + b; blkv = blk; scale = blk->scale; }
        else { const orc_int4_block *blk = (const orc_int4_block *)blocks + row * bpr + b; blkv = blk; scale = blk->scale; }
        for (size_t g = 0; g < 64; ++g) {
          unsigned q[4];
          for (int j = 0; j < 4; ++j)
            q[j] = (kind == ORC_INT3) ? bitstream_get(((const orc_int3_block *)blkv)->data, 96, 4 * g + j, 3)
                                      : (unsigned)(int4_at((const orc_int4_block *)blkv, 4 * g + j) + 8);
          for (unsigned p = 0; p < bits; ++p) s += (float)(1u << p) * L[g * 16 + plane_index4(q, p)];
          xs += L[g * 16 + 15];
        }
        acc += (s - zero_point * xs) * scale;
      }
    }
    out[row] = acc;
  }
  free(luts);
}

/* ---------------------------------------------------------------------------------------
 * Layer API -- src/kernels/lut_gemm_scalar.cpp:68-180
 * ------------------------------------------------------------------------------------- */
void orc_lut_linear(int kind, int quant_bits, const void *blocks, size_t M, size_t K,
                    const float *bias, const float *input, float *output, size_t batch) {
  const size_t k_aligned = (K + 255) / 256 * 256; /* :90 */
  /* :92-93 rotation iff 0 < quant_bits <= 2, or the ternary block vector is non-empty */
  const int rotate = (quant_bits <= 2 && quant_bits > 0) || (kind == ORC_TERNARY);
  float *buf = (float *)malloc(sizeof(float) * k_aligned);
  for (size_t b = 0; b < batch; ++b) {
    const float *x = input + b * K;
    float *y = output + b * M;
    memcpy(buf, x, K * sizeof(float));                           /* :101 */
    memset(buf + K, 0, (k_aligned - K) * sizeof(float));         /* :103-106 */
    if (rotate) orc_apply_hadamard_rotation(buf, k_aligned);     /* :108-110 */
    orc_gemv(kind, blocks, buf, y, M, K);                        /* :115-156 */
    if (bias) for (size_t i = 0; i < M; ++i) y[i] += bias[i];    /* :174-178 */
  }
  free(buf);
}

/* ---------------------------------------------------------------------------------------
 * Quantizers (2-D tensors), include/lutmac/quantize.hpp
 * ------------------------------------------------------------------------------------- */
size_t orc_num_blocks_2d(int kind, size_t M, size_t K) {
  (void)kind;
  return M * ((K + BLK - 1) / BLK);
}

/* quantize.hpp:135-154 */
void orc_pack_to_bitplanes(const int8_t *t, size_t n, uint8_t *sign_plane, uint8_t *zero_plane) {
  for (size_t i = 0; i < n; i += 8) {
    uint8_t s = 0, z = 0;
    for (size_t j = 0; j < 8; ++j)
      if (i + j < n) {
        if (t[i + j] < 0) s |= (uint8_t)(1u << (7 - j));
        if (t[i + j] == 0) z |= (uint8_t)(1u << (7 - j));
      }
    sign_plane[i / 8] = s;
    zero_plane[i / 8] = z;
  }
}

/* quantize.hpp:158-181 */
void orc_unpack_from_bitplanes(const uint8_t *sign_plane, const uint8_t *zero_plane, size_t n, int8_t *t) {
  for (size_t i = 0; i < n; ++i) {
    unsigned bit = 7u - (unsigned)(i % 8);
    int neg = (sign_plane[i / 8] >> bit) & 1, zero = (zero_plane[i / 8] >> bit) & 1;
    t[i] = zero ? 0 : (neg ? -1 : 1);
  }
}

static void bitstream_set(uint8_t *data, size_t nbytes, size_t idx, unsigned bits, unsigned val) {
  /* types.hpp:268-288 (3-bit) and the 5/6-bit twins */
  size_t bit_idx = idx * bits, byte_idx = bit_idx / 8;
  unsigned off = (unsigned)(bit_idx % 8), sh = 16 - bits - off, m = (1u << bits) - 1u;
  unsigned word = (unsigned)data[byte_idx] << 8;
  if (byte_idx + 1 < nbytes) word |= data[byte_idx + 1];
  word = (word & ~(m << sh)) | ((val & m) << sh);
  word &= 0xFFFFu;
  data[byte_idx] = (uint8_t)(word >> 8);
  if (byte_idx + 1 < nbytes) data[byte_idx + 1] = (uint8_t)(word & 0xFF);
}

static int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }

size_t orc_quantize(int kind, const float *data, size_t M, size_t K, void *out) {
  const size_t bpr = (K + BLK - 1) / BLK, n = M * K;
  const size_t nblocks = M * bpr;
  memset(out, 0, nblocks * orc_block_bytes(kind));

  if (kind == ORC_TERNARY) { /* quantize.hpp:193-287 */
    double abs_sum = 0.0;
    for (size_t i = 0; i < n; ++i) abs_sum += fabsf(data[i]);
    const float threshold = (float)(abs_sum / (double)n); /* :96-102 */
    const float zero_thr = 0.5f * threshold;              /* :211,271 */
    for (size_t r = 0; r < M; ++r)
      for (size_t b = 0; b < bpr; ++b) {
        orc_ternary_block *blk = (orc_ternary_block *)out + r * bpr + b;
        size_t start = b * BLK, valid = start < K ? (K - start < BLK ? K - start : BLK) : 0;
        int8_t t[BLK];
        memset(t, 0, sizeof t);
        float scale_sum = 0.0f; /* float accumulator, :268 */
        size_t count = 0;
        for (size_t i = 0; i < valid; ++i) {
          float v = data[r * K + start + i];
          t[i] = (fabsf(v) < zero_thr) ? 0 : (v > 0 ? 1 : -1); /* :83-88 */
          if (fabsf(v) >= threshold) { scale_sum += fabsf(v); count++; }
        }
        orc_pack_to_bitplanes(t, BLK, blk->sign_plane, blk->zero_plane);
        blk->scale = count > 0 ? (float)(scale_sum / (float)count) : 1.0f;
      }
    return nblocks;
  }

  if (kind == ORC_INT2 || kind == ORC_INT3) {
    /* quantize.hpp:918-975 / :982-1039: these two quantizers walk the FLAT element
     * stream in 256-element chunks (no per-row padding), unlike the others. */
    const size_t flat_blocks = nblocks;
    for (size_t b = 0; b < flat_blocks; ++b) {
      size_t start = b * BLK, valid = start < n ? (n - start < BLK ? n - start : BLK) : 0;
      float absmax = 0.0f;
      for (size_t i = 0; i < valid; ++i) absmax = fmaxf(absmax, fabsf(data[start + i]));
      if (kind == ORC_INT2) {
        orc_int2_block *blk = (orc_int2_block *)out + b;
        blk->scale = absmax / 2.0f;
        float inv = blk->scale > 1e-10f ? 1.0f / blk->scale : 0.0f;
        for (size_t i = 0; i < BLK; ++i) {
          float v = i < valid ? data[start + i] : 0.0f;
          int q = clampi((int)roundf(v * inv), -2, 1);
          unsigned sh = 6u - 2u * (unsigned)(i % 4);
          blk->data[i / 4] = (uint8_t)((blk->data[i / 4] & ~(3u << sh)) | ((unsigned)(q + 2) << sh));
        }
      } else {
        orc_int3_block *blk = (orc_int3_block *)out + b;
        blk->scale = absmax / 4.0f;
        float inv = blk->scale > 1e-10f ? 1.0f / blk->scale : 0.0f;
        for (size_t i = 0; i < BLK; ++i) {
          float v = i < valid ? data[start + i] : 0.0f;
          int q = clampi((int)roundf(v * inv), -4, 3);
          bitstream_set(blk->data, 96, i, 3, (unsigned)(q + 4));
        }
      }
    }
    return flat_blocks;
  }

  for (size_t r = 0; r < M; ++r)
    for (size_t b = 0; b < bpr; ++b) {
      size_t start = b * BLK, valid = start < K ? (K - start < BLK ? K - start : BLK) : 0;
      const float *src = data + r * K + start;
      if (kind == ORC_INT4) { /* quantize.hpp:387-461 */
        orc_int4_block *blk = (orc_int4_block *)out + r * bpr + b;
        float absmax = 0.0f;
        for (size_t i = 0; i < valid; ++i) absmax = fmaxf(absmax, fabsf(src[i]));
        blk->scale = absmax / 7.0f;
        float inv = blk->scale > 1e-10f ? 1.0f / blk->scale : 0.0f;
        for (size_t i = 0; i < BLK; ++i) {
          float v = i < valid ? src[i] : 0.0f;
          unsigned uq = (unsigned)(clampi((int)roundf(v * inv), -7, 7) + 8);
          if (i % 2 == 0) blk->data[i / 2] = (uint8_t)((blk->data[i / 2] & 0x0F) | (uq << 4));
          else blk->data[i / 2] = (uint8_t)((blk->data[i / 2] & 0xF0) | (uq & 0x0F));
        }
      } else if (kind == ORC_BINARY) { /* quantize.hpp:725-796 */
        orc_binary_block *blk = (orc_binary_block *)out + r * bpr + b;
        double sum_abs = 0.0;
        for (size_t i = 0; i < valid; ++i) sum_abs += fabsf(src[i]);
        blk->scale = valid > 0 ? (float)(sum_abs / (double)valid) : 0.0f;
        for (size_t i = 0; i < BLK; ++i) {
          float v = i < valid ? src[i] : 0.0f;
          if (v >= 0.0f) blk->data[i / 8] |= (uint8_t)(1u << (7 - (i % 8)));
        }
      } else if (kind == ORC_INT8) { /* quantize.hpp:833-911 via Int8Block::set, types.hpp:441-461 */
        orc_int8_block *blk = (orc_int8_block *)out + r * bpr + b;
        float w[BLK];
        for (size_t i = 0; i < BLK; ++i) w[i] = i < valid ? src[i] : 0.0f;
        float max_abs = 0.0f;
        for (size_t i = 0; i < BLK; ++i) max_abs = fmaxf(max_abs, fabsf(w[i]));
        blk->scale = max_abs / 127.0f;
        if (blk->scale == 0.0f) continue;
        float inv = 1.0f / blk->scale;
        for (size_t i = 0; i < BLK; ++i) {
          float v = w[i] * inv;
          v = fmaxf(-127.0f, fminf(127.0f, v));
          blk->data[i] = (int8_t)roundf(v);
        }
      }
    }
  return nblocks;
}

/* ---------------------------------------------------------------------------------------
 * Glue ops
 * ------------------------------------------------------------------------------------- */
/* src/layers/norm.cpp:18-34 */
void orc_rms_norm(const float *in, const float *w, float *out, size_t n, float eps) {
  float ss = 0.0f;
  for (size_t i = 0; i < n; ++i) ss += in[i] * in[i];
  float inv = 1.0f / sqrtf(ss / (float)n + eps);
  for (size_t i = 0; i < n; ++i) out[i] = in[i] * inv * w[i];
}

/* src/layers/norm.cpp:40-53: the weights are offsets from one */
void orc_gemma_rms_norm(const float *in, const float *w, float *out, size_t n, float eps) {
  float ss = 0.0f;
  for (size_t i = 0; i < n; ++i) ss += in[i] * in[i];
  float rms = sqrtf(ss / (float)n + eps);
  float inv = 1.0f / rms;
  for (size_t i = 0; i < n; ++i) out[i] = in[i] * inv * (1.0f + w[i]);
}

/* src/layers/embedding.cpp:36-75: pairs (d, d + head_dim/2); angle = (pos/factor)*freq,
 * freq = 1/pow(theta, 2d/head_dim), all in float. */
void orc_apply_rope(float *q, float *k, size_t position, size_t nh, size_t nkv, size_t hd,
                    float theta, float factor) {
  size_t half = hd / 2;
  for (int pass = 0; pass < 2; ++pass) {
    float *base = pass == 0 ? q : k;
    size_t heads = pass == 0 ? nh : nkv;
    for (size_t h = 0; h < heads; ++h) {
      float *v = base + h * hd;
      for (size_t d = 0; d < half; ++d) {
        float freq = 1.0f / powf(theta, (2.0f * (float)d) / (float)hd);
        float angle = ((float)position / factor) * freq;
        float c = cosf(angle), s = sinf(angle);
        float a = v[d], b = v[d + half];
        v[d] = a * c - b * s;
        v[d + half] = a * s + b * c;
      }
    }
  }
}

/* src/layers/attention.cpp:23-42 */
void orc_softmax(float *d, size_t n) {
  float mx = d[0];
  for (size_t i = 1; i < n; ++i) mx = fmaxf(mx, d[i]);
  float sum = 0.0f;
  for (size_t i = 0; i < n; ++i) { d[i] = expf(d[i] - mx); sum += d[i]; }
  float inv = 1.0f / sum;
  for (size_t i = 0; i < n; ++i) d[i] *= inv;
}

/* ---------------------------------------------------------------------------------------
 * One decode step -- src/model.cpp:47-453 for the llama-type path (rms_norm, SiLU).
 * Rows of each GEMV may be split over threads; that does not change any row's arithmetic.
 * ------------------------------------------------------------------------------------- */
typedef struct {
  int kind; const void *blocks; const float *act; float *out; size_t M, K;
} gemv_job;

static void *gemv_thread(void *p) {
  gemv_job *j = (gemv_job *)p;
  orc_gemv(j->kind, j->blocks, j->act, j->out, j->M, j->K);
  return NULL;
}

static void gemv_mt(int kind, const void *blocks, const float *act, float *out, size_t M, size_t K, int nt) {
  if (nt <= 1 || M < (size_t)nt * 4) { orc_gemv(kind, blocks, act, out, M, K); return; }
  const size_t bpr = (K + BLK - 1) / BLK, bb = orc_block_bytes(kind);
  pthread_t *th = (pthread_t *)malloc(sizeof(pthread_t) * (size_t)nt);
  gemv_job *jobs = (gemv_job *)malloc(sizeof(gemv_job) * (size_t)nt);
  for (int t = 0; t < nt; ++t) {
    size_t r0 = M * (size_t)t / (size_t)nt, r1 = M * (size_t)(t + 1) / (size_t)nt;
    jobs[t] = (gemv_job){kind, (const char *)blocks + r0 * bpr * bb, act, out + r0, r1 - r0, K};
    pthread_create(&th[t], NULL, gemv_thread, &jobs[t]);
  }
  for (int t = 0; t < nt; ++t) pthread_join(th[t], NULL);
  free(th);
  free(jobs);
}

static void linear_mt(const orc_tensor *w, const float *in, float *out, int nt) {
  /* lut_linear for batch 1, no bias (model.cpp passes nullptr) */
  const size_t k_aligned = (w->K + 255) / 256 * 256;
  const int rotate = (w->quant_bits <= 2 && w->quant_bits > 0) || (w->kind == ORC_TERNARY);
  float *buf = (float *)malloc(sizeof(float) * k_aligned);
  memcpy(buf, in, w->K * sizeof(float));
  memset(buf + w->K, 0, (k_aligned - w->K) * sizeof(float));
  if (rotate) orc_apply_hadamard_rotation(buf, k_aligned);
  gemv_mt(w->kind, w->blocks, buf, out, w->M, w->K, nt);
  free(buf);
}

static inline float silu(float x) { return x / (1.0f + expf(-x)); } /* model.cpp:36 */
/* model.cpp:38-42: the constant and the tanh are evaluated in double (M_PI is a double) */
static inline float gelu(float x) {
  return (float)(0.5f * x * (1.0f + tanh(sqrt(2.0f / 3.14159265358979323846) * (x + 0.044715f * x * x * x))));
}

void orc_model_forward(const orc_model *m, int token_id, size_t position, float *logits) {
  const size_t h = m->hidden, nh = m->n_heads, nkv = m->n_kv_heads, hd = m->head_dim, inter = m->inter;
  const size_t attn_dim = nh * hd, kv_dim = nkv * hd;
  const int nt = m->n_threads > 0 ? m->n_threads : 1;
  float *hidden = (float *)calloc(h, sizeof(float));
  float *normed = (float *)calloc(h, sizeof(float));
  float *q = (float *)calloc(attn_dim, sizeof(float));
  float *k = (float *)calloc(kv_dim, sizeof(float));
  float *v = (float *)calloc(kv_dim, sizeof(float));
  float *att = (float *)calloc(attn_dim, sizeof(float));
  float *w = (float *)calloc(m->max_seq, sizeof(float));
  float *proj = (float *)calloc(h, sizeof(float));
  float *gate = (float *)calloc(inter, sizeof(float));
  float *up = (float *)calloc(inter, sizeof(float));

  /* embedding row: model.cpp:58-252 (per-row block lookup, Block::get) */
  {
    const size_t bpr = (h + BLK - 1) / BLK, bb = orc_block_bytes(m->embed.kind);
    for (size_t i = 0; i < h; ++i) {
      const char *blk = (const char *)m->embed.blocks + ((size_t)token_id * bpr + i / BLK) * bb;
      hidden[i] = orc_block_get(m->embed.kind, blk, i % BLK);
    }
    if (m->gemma) { /* model.cpp:255-260 */
      float scale = sqrtf((float)h);
      for (size_t i = 0; i < h; ++i) hidden[i] *= scale;
    }
  }
  void (*norm)(const float *, const float *, float *, size_t, float) = m->gemma ? orc_gemma_rms_norm : orc_rms_norm;

  for (size_t l = 0; l < m->n_layers; ++l) {
    const orc_layer *L = &m->layers[l];
    norm(hidden, L->input_norm, normed, h, m->eps); /* model.cpp:294-301 */
    linear_mt(&L->q, normed, q, nt);                       /* :307-309 */
    linear_mt(&L->k, normed, k, nt);
    linear_mt(&L->v, normed, v, nt);
    if (L->q_bias) for (size_t j = 0; j < attn_dim; ++j) q[j] += L->q_bias[j]; /* :312-323 */
    if (L->k_bias) for (size_t j = 0; j < kv_dim; ++j) k[j] += L->k_bias[j];
    if (L->v_bias) for (size_t j = 0; j < kv_dim; ++j) v[j] += L->v_bias[j];
    orc_apply_rope(q, k, position, nh, nkv, hd, m->rope_theta, m->rope_factor); /* :326-327 */

    float *kc = m->kv_cache + (l * 2) * m->max_seq * kv_dim;     /* types.hpp:617-624 */
    float *vc = m->kv_cache + (l * 2 + 1) * m->max_seq * kv_dim;
    memcpy(kc + position * kv_dim, k, kv_dim * sizeof(float));    /* :330-335 */
    memcpy(vc + position * kv_dim, v, kv_dim * sizeof(float));

    const size_t seq = position + 1, group = nh / nkv;            /* :338-341 */
    const float scale = 1.0f / sqrtf((float)hd);
    memset(att, 0, attn_dim * sizeof(float));
    for (size_t head = 0; head < nh; ++head) {                    /* :345-372 */
      const size_t kvh = head / group;
      const float *qh = q + head * hd;
      for (size_t t = 0; t < seq; ++t) {
        const float *kt = kc + t * kv_dim + kvh * hd;
        float s = 0.0f;
        for (size_t d = 0; d < hd; ++d) s += qh[d] * kt[d];
        w[t] = s * scale;
      }
      orc_softmax(w, seq);
      float *oh = att + head * hd;
      for (size_t t = 0; t < seq; ++t) {
        const float *vt = vc + t * kv_dim + kvh * hd;
        for (size_t d = 0; d < hd; ++d) oh[d] += w[t] * vt[d];
      }
    }
    linear_mt(&L->o, att, proj, nt);                              /* :380-381 */
    for (size_t j = 0; j < h; ++j) hidden[j] += proj[j];          /* :385-387 */
    norm(hidden, L->post_norm, normed, h, m->eps);                /* :390-399 */
    linear_mt(&L->gate, normed, gate, nt);                        /* :402-403 */
    linear_mt(&L->up, normed, up, nt);
    if (m->gelu) for (size_t j = 0; j < inter; ++j) gate[j] = gelu(gate[j]) * up[j]; /* :409-412 */
    else for (size_t j = 0; j < inter; ++j) gate[j] = silu(gate[j]) * up[j];          /* :414-416 */
    linear_mt(&L->down, gate, proj, nt);                          /* :419-420 */
    for (size_t j = 0; j < h; ++j) hidden[j] += proj[j];          /* :424-426 */
  }
  norm(hidden, m->final_norm, normed, h, m->eps);                 /* :436-442 */
  linear_mt(&m->lm_head, normed, logits, nt);                     /* :447 */

  free(hidden); free(normed); free(q); free(k); free(v); free(att); free(w); free(proj); free(gate); free(up);
}


/* ---------------------------------------------------------------------------------------
 * The same decode step evaluated in fp64 throughout (weights are the exact real values of the
 * codes and scales, activations, norms, softmax and sums in double; cos/sin of the float angle
 * the reference forms).  Not a restatement of reference code: the arbiter for "how far is an
 * fp32 implementation from the exact result" when two fp32 implementations disagree.
 * The KV cache (fp32, shared layout) is read as given and NOT updated.
 * ------------------------------------------------------------------------------------- */
typedef struct {
  int kind; const void *blocks; const double *act; double *out; size_t M, K;
} gemv_job_d;

static void *gemv_thread_d(void *p) {
  gemv_job_d *j = (gemv_job_d *)p;
  gemv_dispatch_d64(j->kind, j->blocks, j->act, j->out, j->M, j->K);
  return NULL;
}

static void linear_d(const orc_tensor *w, const double *in, double *out, int nt) {
  const size_t k_aligned = (w->K + 255) / 256 * 256, bpr = k_aligned / 256, bb = orc_block_bytes(w->kind);
  const int rotate = (w->quant_bits <= 2 && w->quant_bits > 0) || (w->kind == ORC_TERNARY);
  double *buf = (double *)calloc(k_aligned, sizeof(double));
  memcpy(buf, in, w->K * sizeof(double));
  if (rotate)
    for (size_t b = 0; b < bpr; ++b) {
      double *d = buf + b * 256;
      for (size_t h = 1; h < 256; h <<= 1)
        for (size_t i = 0; i < 256; i += 2 * h)
          for (size_t j = i; j < i + h; ++j) { double x = d[j], y = d[j + h]; d[j] = x + y; d[j + h] = x - y; }
      for (size_t i = 0; i < 256; ++i) d[i] *= 0.0625;
    }
  if (nt < 1) nt = 1;
  if ((size_t)nt > w->M) nt = (int)w->M;
  pthread_t *th = (pthread_t *)malloc(sizeof(pthread_t) * (size_t)nt);
  gemv_job_d *jobs = (gemv_job_d *)malloc(sizeof(gemv_job_d) * (size_t)nt);
  for (int t = 0; t < nt; ++t) {
    size_t r0 = w->M * (size_t)t / (size_t)nt, r1 = w->M * (size_t)(t + 1) / (size_t)nt;
    jobs[t] = (gemv_job_d){w->kind, (const char *)w->blocks + r0 * bpr * bb, buf, out + r0, r1 - r0, w->K};
    pthread_create(&th[t], NULL, gemv_thread_d, &jobs[t]);
  }
  for (int t = 0; t < nt; ++t) pthread_join(th[t], NULL);
  free(th); free(jobs); free(buf);
}

static void norm_d(const double *in, const float *w, double *out, size_t n, float eps, int gemma) {
  double ss = 0.0;
  for (size_t i = 0; i < n; ++i) ss += in[i] * in[i];
  double inv = 1.0 / sqrt(ss / (double)n + (double)eps);
  for (size_t i = 0; i < n; ++i) out[i] = in[i] * inv * (gemma ? 1.0 + (double)w[i] : (double)w[i]);
}

void orc_model_forward_f64(const orc_model *m, int token_id, size_t position, double *logits) {
  const size_t h = m->hidden, nh = m->n_heads, nkv = m->n_kv_heads, hd = m->head_dim, inter = m->inter;
  const size_t attn_dim = nh * hd, kv_dim = nkv * hd, half = hd / 2;
  const int nt = m->n_threads > 0 ? m->n_threads : 1;
  double *hidden = calloc(h, 8), *normed = calloc(h, 8), *q = calloc(attn_dim, 8), *k = calloc(kv_dim, 8), *v = calloc(kv_dim, 8);
  double *att = calloc(attn_dim, 8), *w = calloc(m->max_seq, 8), *proj = calloc(h, 8), *gate = calloc(inter, 8), *up = calloc(inter, 8);
  {
    const size_t bpr = (h + BLK - 1) / BLK, bb = orc_block_bytes(m->embed.kind);
    for (size_t i = 0; i < h; ++i) {
      const char *blk = (const char *)m->embed.blocks + ((size_t)token_id * bpr + i / BLK) * bb;
      hidden[i] = (double)orc_block_get(m->embed.kind, blk, i % BLK); /* int8 embedding: code * scale, exact enough in float */
    }
    if (m->gemma) { double scale = sqrt((double)h); for (size_t i = 0; i < h; ++i) hidden[i] *= scale; }
  }
  for (size_t l = 0; l < m->n_layers; ++l) {
    const orc_layer *L = &m->layers[l];
    norm_d(hidden, L->input_norm, normed, h, m->eps, m->gemma);
    linear_d(&L->q, normed, q, nt); linear_d(&L->k, normed, k, nt); linear_d(&L->v, normed, v, nt);
    if (L->q_bias) for (size_t j = 0; j < attn_dim; ++j) q[j] += (double)L->q_bias[j];
    if (L->k_bias) for (size_t j = 0; j < kv_dim; ++j) k[j] += (double)L->k_bias[j];
    if (L->v_bias) for (size_t j = 0; j < kv_dim; ++j) v[j] += (double)L->v_bias[j];
    for (int pass = 0; pass < 2; ++pass) { /* rotary embedding on the float angle of embedding.cpp:45-46 */
      double *base = pass == 0 ? q : k;
      size_t heads = pass == 0 ? nh : nkv;
      for (size_t hh = 0; hh < heads; ++hh)
        for (size_t d = 0; d < half; ++d) {
          float freq = 1.0f / powf(m->rope_theta, (2.0f * (float)d) / (float)hd);
          float angle = ((float)position / m->rope_factor) * freq;
          double c = cos((double)angle), s = sin((double)angle), a = base[hh * hd + d], b = base[hh * hd + d + half];
          base[hh * hd + d] = a * c - b * s;
          base[hh * hd + d + half] = a * s + b * c;
        }
    }
    const float *kc = m->kv_cache + (l * 2) * m->max_seq * kv_dim, *vc = m->kv_cache + (l * 2 + 1) * m->max_seq * kv_dim;
    const size_t seq = position + 1, group = nh / nkv;
    const double scale = 1.0 / sqrt((double)hd);
    memset(att, 0, attn_dim * 8);
    for (size_t head = 0; head < nh; ++head) {
      const size_t kvh = head / group;
      const double *qh = q + head * hd;
      double mx = -1e300, sum = 0.0;
      for (size_t t = 0; t < seq; ++t) {
        double s = 0.0;
        for (size_t d = 0; d < hd; ++d) s += qh[d] * (t == position ? k[kvh * hd + d] : (double)kc[t * kv_dim + kvh * hd + d]);
        w[t] = s * scale;
        if (w[t] > mx) mx = w[t];
      }
      for (size_t t = 0; t < seq; ++t) { w[t] = exp(w[t] - mx); sum += w[t]; }
      for (size_t t = 0; t < seq; ++t)
        for (size_t d = 0; d < hd; ++d)
          att[head * hd + d] += w[t] / sum * (t == position ? v[kvh * hd + d] : (double)vc[t * kv_dim + kvh * hd + d]);
    }
    linear_d(&L->o, att, proj, nt);
    for (size_t j = 0; j < h; ++j) hidden[j] += proj[j];
    norm_d(hidden, L->post_norm, normed, h, m->eps, m->gemma);
    linear_d(&L->gate, normed, gate, nt); linear_d(&L->up, normed, up, nt);
    for (size_t j = 0; j < inter; ++j) {
      double g = gate[j];
      gate[j] = (m->gelu ? 0.5 * g * (1.0 + tanh(sqrt(2.0 / 3.14159265358979323846) * (g + 0.044715 * g * g * g))) : g / (1.0 + exp(-g))) * up[j];
    }
    linear_d(&L->down, gate, proj, nt);
    for (size_t j = 0; j < h; ++j) hidden[j] += proj[j];
  }
  norm_d(hidden, m->final_norm, normed, h, m->eps, m->gemma);
  linear_d(&m->lm_head, normed, logits, nt);
  free(hidden); free(normed); free(q); free(k); free(v); free(att); free(w); free(proj); free(gate); free(up);
}
