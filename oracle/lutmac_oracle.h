/*
 * TEST INFRASTRUCTURE ONLY.  CPU restatement (plain C11) of the LutMac decode hot path,
 * used as the parity checker for the CUDA library.  Nothing in the shipped product may
 * link, import or execute this file; only the test-suite, the smoke check and the
 * benchmark's CPU-baseline leg do.
 *
 * Parity status: PINNED.  Every function below is checked (a) against the known-answer
 * vectors held by the reference's own tests (tests/test_lut_gemm.cpp,
 * tests/test_tmac_correctness.cpp, tests/test_quantization.cpp) and (b) against the
 * reference's own C++ sources compiled on the build machine (oracle/_ref), with the
 * resulting input/output vectors committed as fixtures under tests/golden/.
 *
 * Citations are file:line inside the reference project (YASSERRMD/lutmac).
 */
#ifndef LUTMAC_ORACLE_H
#define LUTMAC_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Block kinds.  The value is the reference's PackedTensor::quant_bits for that block
 * vector, except ternary (the reference leaves quant_bits at its default for ternary,
 * include/lutmac/types.hpp:483) which gets 0 here. */
enum {
  ORC_TERNARY = 0, /* BitPlaneBlock  68 B  include/lutmac/types.hpp:126-137 */
  ORC_BINARY = 1,  /* BinaryBlock    36 B  include/lutmac/types.hpp:394-401 */
  ORC_INT2 = 2,    /* Int2Block      72 B  include/lutmac/types.hpp:209-215 */
  ORC_INT3 = 3,    /* Int3Block     100 B  include/lutmac/types.hpp:249-254 */
  ORC_INT4 = 4,    /* Int4Block     132 B  include/lutmac/types.hpp:174-181 */
  ORC_INT5 = 5,    /* Int5Block     164 B  include/lutmac/types.hpp:296-301 */
  ORC_INT6 = 6,    /* Int6Block     196 B  include/lutmac/types.hpp:344-349 */
  ORC_INT8 = 8     /* Int8Block     260 B  include/lutmac/types.hpp:434-438 (scale first) */
};

#pragma pack(push, 1)
typedef struct { uint8_t sign_plane[32]; uint8_t zero_plane[32]; float scale; } orc_ternary_block;
typedef struct { uint8_t data[32]; float scale; } orc_binary_block;
typedef struct { uint8_t data[64]; float scale; float scale2; } orc_int2_block;
typedef struct { uint8_t data[96]; float scale; } orc_int3_block;
typedef struct { uint8_t data[128]; float scale; } orc_int4_block;
typedef struct { uint8_t data[160]; float scale; } orc_int5_block;
typedef struct { uint8_t data[192]; float scale; } orc_int6_block;
typedef struct { float scale; int8_t data[256]; } orc_int8_block;
#pragma pack(pop)

size_t orc_block_bytes(int kind);

/* --- LUT helpers ------------------------------------------------------------------- */
void orc_precompute_lut(const float *act4, float *lut16);
void orc_precompute_luts(const float *act, size_t n, float *luts);
void orc_extract_indices(const uint8_t *sign_plane, const uint8_t *zero_plane,
                         size_t group_idx, uint8_t *pos_idx, uint8_t *neg_idx);

/* --- FWHT ---------------------------------------------------------------------------- */
void orc_fwht_256(float *data);
void orc_apply_hadamard_rotation(float *data, size_t n);

/* --- GEMV kernels (scalar semantics of src/kernels/lut_gemm_scalar.cpp) -------------- */
void orc_gemv(int kind, const void *blocks, const float *act, float *out, size_t M, size_t K);
/* Same GEMV evaluated in double precision (error budgeting only). */
void orc_gemv_f64(int kind, const void *blocks, const float *act, double *out, size_t M, size_t K);
/* LUT-form evaluation (table lookups with the reference's index convention):
 * ternary as lut_gemv_neon, n-bit planes as int3_gemv_neon, RRQ as int2_gemv_neon. */
void orc_gemv_lutform(int kind, const void *blocks, const float *act, float *out, size_t M, size_t K);
/* Dequantise one weight (Block::get). */
float orc_block_get(int kind, const void *block, size_t idx);

/* --- Layer API ------------------------------------------------------------------------ */
/* quant_bits is the PackedTensor field; has_ternary_blocks says whether `blocks` is the
 * ternary vector (the reference rotates whenever that vector is non-empty). */
void orc_lut_linear(int kind, int quant_bits, const void *blocks, size_t M, size_t K,
                    const float *bias, const float *input, float *output, size_t batch);

/* --- Quantizers (2-D tensors) ---------------------------------------------------------- */
size_t orc_quantize(int kind, const float *data, size_t M, size_t K, void *blocks_out);
size_t orc_num_blocks_2d(int kind, size_t M, size_t K);
void orc_pack_to_bitplanes(const int8_t *ternary, size_t n, uint8_t *sign_plane, uint8_t *zero_plane);
void orc_unpack_from_bitplanes(const uint8_t *sign_plane, const uint8_t *zero_plane, size_t n, int8_t *ternary);

/* --- Glue ops --------------------------------------------------------------------------- */
void orc_rms_norm(const float *in, const float *w, float *out, size_t n, float eps);
void orc_apply_rope(float *q, float *k, size_t position, size_t num_heads, size_t num_kv_heads,
                    size_t head_dim, float theta, float factor);
void orc_softmax(float *data, size_t n);

/* --- One decode step -------------------------------------------------------------------- */
typedef struct {
  int kind;
  int quant_bits;
  const void *blocks;
  size_t M, K;
} orc_tensor;

typedef struct {
  const float *input_norm, *post_norm;
  orc_tensor q, k, v, o, gate, up, down;
  const float *q_bias, *k_bias, *v_bias; /* may be NULL (= all zero) */
} orc_layer;

typedef struct {
  size_t vocab, hidden, inter, n_layers, n_heads, n_kv_heads, head_dim, max_seq;
  float rope_theta, rope_factor, eps;
  orc_tensor embed, lm_head;
  const float *final_norm;
  const orc_layer *layers;
  float *kv_cache; /* [layer][2][max_seq][n_kv_heads][head_dim] fp32 */
  int n_threads;   /* rows of each GEMV are split over this many threads (1 = as shipped) */
  int gemma;       /* model_type "gemma": embedding x sqrt(hidden), norms scale by (1 + weight) */
  int gelu;        /* ActivationType::GELU: gelu(gate) * up instead of silu(gate) * up */
} orc_model;

void orc_model_forward(const orc_model *m, int token_id, size_t position, float *logits);
/* The same step in fp64 throughout (exact weight values, double activations); reads the KV cache
 * without updating it.  Not reference arithmetic: the yardstick for two fp32 implementations. */
void orc_model_forward_f64(const orc_model *m, int token_id, size_t position, double *logits);

#ifdef __cplusplus
}
#endif
#endif
