// TEST INFRASTRUCTURE ONLY.  extern "C" access to the UNMODIFIED reference (YASSERRMD/lutmac)
// for oracle validation, fixture generation and the benchmark's CPU-baseline leg.  It is
// compiled together with the reference's own sources where they lie (see oracle/Makefile);
// nothing from the reference is copied into this repository.  The product never links it.
#include "lutmac/format.hpp"
#include "lutmac/lut_gemm.hpp"
#include "lutmac/model.hpp"
#include "lutmac/quantize.hpp"
#include "lutmac/transform.hpp"
#include "lutmac/types.hpp"

#include <cstring>
#include <memory>
#include <string>
#include <vector>

using namespace lutmac;

namespace {

// Same kind numbering as oracle/lutmac_oracle.h.
enum { K_TERNARY = 0, K_BINARY = 1, K_INT2 = 2, K_INT3 = 3, K_INT4 = 4, K_INT5 = 5, K_INT6 = 6, K_INT8 = 8 };

size_t kind_bytes(int kind) {
  switch (kind) {
  case K_TERNARY: return sizeof(BitPlaneBlock);
  case K_BINARY: return sizeof(BinaryBlock);
  case K_INT2: return sizeof(Int2Block);
  case K_INT3: return sizeof(Int3Block);
  case K_INT4: return sizeof(Int4Block);
  case K_INT5: return sizeof(Int5Block);
  case K_INT6: return sizeof(Int6Block);
  case K_INT8: return sizeof(Int8Block);
  default: return 0;
  }
}

template <class B> void fill(std::vector<B> &v, const void *blocks, size_t n) {
  v.resize(n);
  std::memcpy(static_cast<void *>(v.data()), blocks, n * sizeof(B));
}

void fill_tensor(PackedTensor &t, int kind, int quant_bits, const void *blocks, size_t M, size_t K) {
  size_t n = M * ((K + 255) / 256);
  t.shape = {M, K};
  t.is_quantized = true;
  t.quant_bits = quant_bits;
  switch (kind) {
  case K_TERNARY: fill(t.blocks, blocks, n); break;
  case K_BINARY: fill(t.binary_blocks, blocks, n); break;
  case K_INT2: fill(t.int2_blocks, blocks, n); break;
  case K_INT3: fill(t.int3_blocks, blocks, n); break;
  case K_INT4: fill(t.int4_blocks, blocks, n); break;
  case K_INT5: fill(t.int5_blocks, blocks, n); break;
  case K_INT6: fill(t.int6_blocks, blocks, n); break;
  case K_INT8: fill(t.int8_blocks, blocks, n); break;
  }
}

} // namespace

extern "C" {

size_t ref_block_bytes(int kind) { return kind_bytes(kind); }

void ref_precompute_lut(const float *a, float *lut) { precompute_lut(a, lut); }
void ref_precompute_luts(const float *a, size_t n, float *luts) { precompute_luts(a, n, luts); }
void ref_extract_indices(const uint8_t *s, const uint8_t *z, size_t g, uint8_t *p, uint8_t *n) {
  extract_indices(s, z, g, *p, *n);
}
void ref_fwht_256(float *d) { fwht_256(d); }
void ref_apply_hadamard_rotation(float *d, size_t n) { apply_hadamard_rotation(d, n); }

// Kernel API, through the reference's own compile-time dispatchers (lut_gemm.hpp:172-408).
void ref_gemv(int kind, const void *blocks, size_t num_blocks, const float *act, float *out, size_t M, size_t K) {
  switch (kind) {
  case K_TERNARY: lut_gemv(static_cast<const BitPlaneBlock *>(blocks), num_blocks, act, out, M, K); break;
  case K_BINARY: lut_gemv_binary(static_cast<const BinaryBlock *>(blocks), num_blocks, act, out, M, K); break;
  case K_INT2: int2_gemv(static_cast<const Int2Block *>(blocks), num_blocks, act, out, M, K); break;
  case K_INT3: int3_gemv(static_cast<const Int3Block *>(blocks), num_blocks, act, out, M, K); break;
  case K_INT4: int4_gemv(static_cast<const Int4Block *>(blocks), num_blocks, act, out, M, K); break;
  case K_INT5: int5_gemv(static_cast<const Int5Block *>(blocks), num_blocks, act, out, M, K); break;
  case K_INT6: int6_gemv(static_cast<const Int6Block *>(blocks), num_blocks, act, out, M, K); break;
  case K_INT8: int8_gemv(static_cast<const Int8Block *>(blocks), num_blocks, act, out, M, K); break;
  }
}

float ref_block_get(int kind, const void *b, size_t i) {
  switch (kind) {
  case K_TERNARY: return static_cast<const BitPlaneBlock *>(b)->get(i);
  case K_BINARY: return static_cast<const BinaryBlock *>(b)->get(i);
  case K_INT2: return static_cast<const Int2Block *>(b)->get(i);
  case K_INT3: return static_cast<const Int3Block *>(b)->get(i);
  case K_INT4: return static_cast<const Int4Block *>(b)->get(i);
  case K_INT5: return static_cast<const Int5Block *>(b)->get(i);
  case K_INT6: return static_cast<const Int6Block *>(b)->get(i);
  case K_INT8: return static_cast<const Int8Block *>(b)->get(static_cast<int>(i));
  }
  return 0.0f;
}

// Layer API.  A PackedTensor is assembled per call (copies the blocks).
void *ref_tensor_create(int kind, int quant_bits, const void *blocks, size_t M, size_t K) {
  auto *t = new PackedTensor();
  fill_tensor(*t, kind, quant_bits, blocks, M, K);
  return t;
}
void ref_tensor_free(void *t) { delete static_cast<PackedTensor *>(t); }
void ref_lut_linear_t(const void *t, const float *bias, const float *in, float *out, size_t batch) {
  lut_linear(*static_cast<const PackedTensor *>(t), bias, in, out, batch);
}
void ref_lut_linear(int kind, int quant_bits, const void *blocks, size_t M, size_t K, const float *bias,
                    const float *in, float *out, size_t batch) {
  PackedTensor t;
  fill_tensor(t, kind, quant_bits, blocks, M, K);
  lut_linear(t, bias, in, out, batch);
}

// Quantizers.  Returns the number of blocks written; quant_bits_out receives the
// PackedTensor::quant_bits the reference leaves on the result.
size_t ref_quantize(int kind, const float *data, size_t M, size_t K, void *out, int *quant_bits_out) {
  PackedTensor t;
  std::vector<size_t> shape = {M, K};
  const void *src = nullptr;
  size_t n = 0;
  switch (kind) {
  case K_TERNARY: t = quantize_tensor(data, shape, "t"); src = t.blocks.data(); n = t.blocks.size(); break;
  case K_BINARY: t = quantize_tensor_binary(data, shape, "t"); src = t.binary_blocks.data(); n = t.binary_blocks.size(); break;
  case K_INT2: t = quantize_tensor_int2(data, shape, "t"); src = t.int2_blocks.data(); n = t.int2_blocks.size(); break;
  case K_INT3: t = quantize_tensor_int3(data, shape, "t"); src = t.int3_blocks.data(); n = t.int3_blocks.size(); break;
  case K_INT4: t = quantize_tensor_int4(data, shape, "t"); src = t.int4_blocks.data(); n = t.int4_blocks.size(); break;
  case K_INT8: t = quantize_tensor_int8(data, shape, "t"); src = t.int8_blocks.data(); n = t.int8_blocks.size(); break;
  default: return 0;
  }
  if (out) std::memcpy(out, src, n * kind_bytes(kind));
  if (quant_bits_out) *quant_bits_out = t.quant_bits;
  return n;
}

void ref_pack_to_bitplanes(const int8_t *t, size_t n, uint8_t *s, uint8_t *z) {
  pack_to_bitplanes(reinterpret_cast<const TernaryValue *>(t), n, s, z);
}
void ref_unpack_from_bitplanes(const uint8_t *s, const uint8_t *z, size_t n, int8_t *t) {
  unpack_from_bitplanes(s, z, n, reinterpret_cast<TernaryValue *>(t));
}

} // extern "C"

// Glue ops are free functions without a header (declared in src/model.cpp:20-30).
namespace lutmac {
void rms_norm(const float *, const float *, float *, size_t, float);
void apply_rope(float *, float *, size_t, size_t, size_t, size_t, float, float);
void softmax(float *, size_t);
} // namespace lutmac

extern "C" {

void ref_rms_norm(const float *in, const float *w, float *out, size_t n, float eps) { rms_norm(in, w, out, n, eps); }
void ref_apply_rope(float *q, float *k, size_t pos, size_t nh, size_t nkv, size_t hd, float theta, float factor) {
  apply_rope(q, k, pos, nh, nkv, hd, theta, factor);
}
void ref_softmax(float *d, size_t n) { softmax(d, n); }

// ---- Model (built in memory, include/lutmac/model.hpp:53-142) -------------------------
void *ref_model_create(size_t vocab, size_t hidden, size_t inter, size_t n_layers, size_t n_heads,
                       size_t n_kv_heads, size_t head_dim, size_t max_seq, float rope_theta,
                       float rope_factor, float eps) {
  auto *m = new Model();
  m->config.model_type = "llama";
  m->config.vocab_size = vocab;
  m->config.hidden_size = hidden;
  m->config.intermediate_size = inter;
  m->config.num_hidden_layers = n_layers;
  m->config.num_attention_heads = n_heads;
  m->config.num_key_value_heads = n_kv_heads;
  m->config.head_dim_val = head_dim;
  m->config.max_position_embeddings = max_seq;
  m->config.rope_theta = rope_theta;
  m->config.rope_scaling_factor = rope_factor;
  m->config.rms_norm_eps = eps;
  m->config.activation = ActivationType::SILU;
  m->allocate();
  return m;
}
// model_type "gemma" (embedding scale, (1 + w) norms) and / or ActivationType::GELU
void ref_model_set_variant(void *mp, int gemma, int gelu) {
  auto *m = static_cast<Model *>(mp);
  m->config.model_type = gemma ? "gemma" : "llama";
  m->config.activation = gelu ? ActivationType::GELU : ActivationType::SILU;
}
void ref_model_free(void *m) { delete static_cast<Model *>(m); }

// slot: 0 embed, 1 lm_head, 2 q, 3 k, 4 v, 5 o, 6 gate, 7 up, 8 down
void ref_model_set_tensor(void *mp, int layer, int slot, int kind, int quant_bits, const void *blocks, size_t M, size_t K) {
  auto *m = static_cast<Model *>(mp);
  PackedTensor *t = nullptr;
  if (slot == 0) t = &m->embed_tokens;
  else if (slot == 1) t = &m->lm_head;
  else {
    TransformerLayer &L = m->layers[static_cast<size_t>(layer)];
    PackedTensor *slots[] = {&L.q_proj, &L.k_proj, &L.v_proj, &L.o_proj, &L.gate_proj, &L.up_proj, &L.down_proj};
    t = slots[slot - 2];
  }
  *t = PackedTensor();
  fill_tensor(*t, kind, quant_bits, blocks, M, K);
}

// which: 0 input_layernorm, 1 post_attention_layernorm, 2 q_bias, 3 k_bias, 4 v_bias, 5 final norm
void ref_model_set_vector(void *mp, int layer, int which, const float *data, size_t n) {
  auto *m = static_cast<Model *>(mp);
  AlignedVector<float> *v = nullptr;
  if (which == 5) v = &m->norm_weight;
  else {
    TransformerLayer &L = m->layers[static_cast<size_t>(layer)];
    AlignedVector<float> *vs[] = {&L.input_layernorm_weight, &L.post_attention_layernorm_weight, &L.q_bias, &L.k_bias, &L.v_bias};
    v = vs[which];
  }
  v->assign(data, data + n);
}

void ref_model_forward(void *mp, int token, size_t position) { static_cast<Model *>(mp)->forward(token, position); }
const float *ref_model_logits(void *mp) { return static_cast<Model *>(mp)->get_logits(); }
float *ref_model_kv(void *mp, size_t *n_floats) {
  auto *m = static_cast<Model *>(mp);
  if (n_floats) *n_floats = m->kv_cache.cache.size();
  return m->kv_cache.cache.data();
}
void ref_model_reset(void *mp) { static_cast<Model *>(mp)->reset_cache(); }

// ---- .lutmac files (src/format.cpp:146-290, :292-505) ------------------------------------
// Writes a file with one tensor per entry, through the reference's own save_lutmac.
struct ref_file_tensor {
  const char *name;
  int kind;       // block kind, or -1 for raw fp32
  int quant_bits;
  const void *data;
  size_t M, K;    // raw 1-D vectors: M = length, K = 0
};

int ref_save_lutmac(const char *path, size_t vocab, size_t hidden, size_t inter, size_t n_layers,
                    size_t n_heads, size_t n_kv_heads, size_t head_dim, float rope_theta, float rope_factor,
                    float eps, const ref_file_tensor *tensors, size_t n_tensors, int gemma, int gelu) {
  ModelConfig c;
  c.model_type = gemma ? "gemma" : "llama";
  c.activation = gelu ? ActivationType::GELU : ActivationType::SILU;
  c.vocab_size = vocab;
  c.hidden_size = hidden;
  c.intermediate_size = inter;
  c.num_hidden_layers = n_layers;
  c.num_attention_heads = n_heads;
  c.num_key_value_heads = n_kv_heads;
  c.head_dim_val = head_dim;
  c.rope_theta = rope_theta;
  c.rope_scaling_factor = rope_factor;
  c.rms_norm_eps = eps;
  std::vector<PackedTensor> ts(n_tensors);
  for (size_t i = 0; i < n_tensors; ++i) {
    const ref_file_tensor &f = tensors[i];
    ts[i].name = f.name;
    if (f.kind < 0) {
      ts[i].is_quantized = false;
      ts[i].quant_bits = 32;
      size_t n = f.K ? f.M * f.K : f.M;
      ts[i].shape = f.K ? std::vector<size_t>{f.M, f.K} : std::vector<size_t>{f.M};
      ts[i].raw_data.assign(static_cast<const float *>(f.data), static_cast<const float *>(f.data) + n);
    } else {
      fill_tensor(ts[i], f.kind, f.quant_bits, f.data, f.M, f.K);
      ts[i].name = f.name;
    }
  }
  return save_lutmac(path, c, ts) ? 0 : 1;
}

void *ref_load_model(const char *path) { return load_model(path).release(); }

} // extern "C"
