// Drop-in definitions of the reference's kernel, layer and transform API on top of the
// lutmac_b200 C ABI.
//
// Built against the REFERENCE'S OWN headers (include/lutmac/lut_gemm.hpp, transform.hpp, types.hpp):
// this file defines every non-inline function those headers declare for the path -- the
// X_gemv_scalar / _avx2 / _avx512 kernels behind the inline dispatchers lut_gemv, lut_gemv_binary,
// int2_gemv ... int8_gemv (lut_gemm.hpp:172-408), lut_linear (lut_gemm.hpp:419) and fwht_256 /
// apply_hadamard_rotation (transform.hpp:14,19) -- so that callers written against the reference
// (its tests, tools/lutmac-bench.cpp, src/model.cpp) link unchanged and run on the GPU.  Link this
// file INSTEAD OF src/kernels/lut_gemm_scalar.cpp, lut_gemm_simd.cpp and transform_simd.cpp, and
// add liblutmac_b200.so.
//
// Errors: the reference's functions return void; a failing C-ABI call throws std::runtime_error
// with the library's message (reference callers do not catch: the process ends with the message).
#include <cstdint>
#include <cstring>
#include <map>
#include <mutex>
#include <stdexcept>
#include <string>
#include <tuple>

#include "lutmac/lut_gemm.hpp"
#include "lutmac/transform.hpp"
#include "lutmac_b200.h"

namespace {

[[noreturn]] void fail(int st, const char *where) {
  throw std::runtime_error(std::string("lutmac_b200 (") + where + "): " + lmb_strerror(st) + ": " + lmb_last_error());
}

void gemv(int kind, const void *blocks, size_t num_blocks, const float *activations, float *output, size_t M, size_t K,
          const char *where) {
  const int st = lmb_gemv_host(kind, blocks, num_blocks, activations, output, M, K);
  if (st != LMB_OK) fail(st, where);
}

lmb_ctx *context() {
  static lmb_ctx *ctx = [] {
    lmb_ctx *c = nullptr;
    const int st = lmb_ctx_create(0, &c);
    if (st != LMB_OK) fail(st, "lmb_ctx_create");
    return c;
  }();
  return ctx;
}

// Device copies of the tensors lut_linear has seen.  The reference's signature gives no hook for
// a tensor's lifetime, so an entry is keyed by the address and size of the host array, the shape
// and a fingerprint of sampled content: an array freed and reallocated at the same address with
// other weights gets a new device copy instead of silently reusing the old one.
// lutmac_b200_dropin_clear() drops all copies.
struct Key {
  const void *data;
  size_t bytes, M, K;
  int kind;
  uint64_t print;
  bool operator<(const Key &o) const {
    return std::tie(data, bytes, M, K, kind, print) < std::tie(o.data, o.bytes, o.M, o.K, o.kind, o.print);
  }
};
std::map<Key, lmb_weight *> g_cache;
std::mutex g_mu;

uint64_t fingerprint(const void *data, size_t bytes) {
  const unsigned char *p = static_cast<const unsigned char *>(data);
  uint64_t h = 1469598103934665603ull;
  auto mix = [&](size_t at, size_t n) {
    for (size_t i = 0; i < n && at + i < bytes; ++i) h = (h ^ p[at + i]) * 1099511628211ull;
  };
  const size_t samples = 256, span = 64;
  for (size_t s = 0; s < samples; ++s) mix(bytes / samples * s, span);
  mix(bytes > span ? bytes - span : 0, span);
  return h;
}

lmb_weight *resident(int kind, const void *data, size_t bytes, size_t M, size_t K) {
  const Key key{data, bytes, M, K, kind, fingerprint(data, bytes)};
  std::lock_guard<std::mutex> lk(g_mu);
  auto it = g_cache.find(key);
  if (it != g_cache.end()) return it->second;
  lmb_weight *w = nullptr;
  const int st = lmb_weight_upload(context(), kind, data, M, K, &w);
  if (st != LMB_OK) fail(st, "lmb_weight_upload");
  g_cache[key] = w;
  return w;
}

}  // namespace

extern "C" void lutmac_b200_dropin_clear(void) {
  std::lock_guard<std::mutex> lk(g_mu);
  for (auto &e : g_cache) lmb_weight_free(e.second);
  g_cache.clear();
}

namespace lutmac {

#define LMB_DROPIN_GEMV(NAME, BLOCK, KIND)                                                                          \
  void NAME(const BLOCK *blocks, size_t num_blocks, const float *activations, float *output, size_t M, size_t K) {  \
    gemv(KIND, blocks, num_blocks, activations, output, M, K, #NAME);                                              \
  }

// src/kernels/lut_gemm_scalar.cpp:7-61, 186-428
LMB_DROPIN_GEMV(lut_gemv_scalar, BitPlaneBlock, LMB_TERNARY)
LMB_DROPIN_GEMV(lut_gemv_binary_scalar, BinaryBlock, LMB_BINARY)
LMB_DROPIN_GEMV(int2_gemv_scalar, Int2Block, LMB_INT2)
LMB_DROPIN_GEMV(int3_gemv_scalar, Int3Block, LMB_INT3)
LMB_DROPIN_GEMV(int4_gemv_scalar, Int4Block, LMB_INT4)
LMB_DROPIN_GEMV(int5_gemv_scalar, Int5Block, LMB_INT5)
LMB_DROPIN_GEMV(int6_gemv_scalar, Int6Block, LMB_INT6)
LMB_DROPIN_GEMV(int8_gemv_scalar, Int8Block, LMB_INT8)

#if defined(LUTMAC_HAS_AVX2) || defined(LUTMAC_AVX2)  // src/kernels/lut_gemm_simd.cpp:35-71
LMB_DROPIN_GEMV(lut_gemv_avx2, BitPlaneBlock, LMB_TERNARY)
LMB_DROPIN_GEMV(lut_gemv_binary_avx2, BinaryBlock, LMB_BINARY)
LMB_DROPIN_GEMV(int2_gemv_avx2, Int2Block, LMB_INT2)
LMB_DROPIN_GEMV(int3_gemv_avx2, Int3Block, LMB_INT3)
LMB_DROPIN_GEMV(int4_gemv_avx2, Int4Block, LMB_INT4)
LMB_DROPIN_GEMV(int8_gemv_avx2, Int8Block, LMB_INT8)
#endif

#if defined(LUTMAC_HAS_AVX512) || defined(LUTMAC_AVX512)  // src/kernels/lut_gemm_simd.cpp:73-160
LMB_DROPIN_GEMV(lut_gemv_avx512, BitPlaneBlock, LMB_TERNARY)
LMB_DROPIN_GEMV(lut_gemv_binary_avx512, BinaryBlock, LMB_BINARY)
LMB_DROPIN_GEMV(int2_gemv_avx512, Int2Block, LMB_INT2)
LMB_DROPIN_GEMV(int3_gemv_avx512, Int3Block, LMB_INT3)
LMB_DROPIN_GEMV(int4_gemv_avx512, Int4Block, LMB_INT4)
LMB_DROPIN_GEMV(int8_gemv_avx512, Int8Block, LMB_INT8)
#endif

#if defined(LUTMAC_HAS_NEON) || defined(LUTMAC_NEON)  // src/kernels/lut_gemm_simd.cpp:178-725
LMB_DROPIN_GEMV(lut_gemv_neon, BitPlaneBlock, LMB_TERNARY)
LMB_DROPIN_GEMV(lut_gemv_binary_neon, BinaryBlock, LMB_BINARY)
LMB_DROPIN_GEMV(int2_gemv_neon, Int2Block, LMB_INT2)
LMB_DROPIN_GEMV(int3_gemv_neon, Int3Block, LMB_INT3)
LMB_DROPIN_GEMV(int4_gemv_neon, Int4Block, LMB_INT4)
LMB_DROPIN_GEMV(int8_gemv_neon, Int8Block, LMB_INT8)
#endif

// src/kernels/lut_gemm_scalar.cpp:68-180.  The dispatch ladder is the reference's: quant_bits and
// a non-empty block vector select the kind, everything else that is quantised is ternary, an
// unquantised tensor takes the fp32 dot product.  Padding to 256 columns, the rotation of the
// input for quant_bits <= 2 and ternary tensors, the bias and the batch loop happen on the device.
void lut_linear(const PackedTensor &weight, const float *bias, const float *input, float *output, size_t batch_size) {
  if (weight.shape.size() != 2) return;  // :70-71
  const size_t M = weight.shape[0], K = weight.shape[1];
  int kind = LMB_TERNARY;
  const void *data = weight.blocks.data();
  size_t bytes = weight.blocks.size() * sizeof(BitPlaneBlock);
  auto pick = [&](int k, const auto &vec) {
    kind = k;
    data = vec.data();
    bytes = vec.size() * sizeof(vec[0]);
  };
  if (!weight.is_quantized) pick(LMB_RAW_F32, weight.raw_data);
  else if (weight.quant_bits == 4 && !weight.int4_blocks.empty()) pick(LMB_INT4, weight.int4_blocks);
  else if (weight.quant_bits == 8 && !weight.int8_blocks.empty()) pick(LMB_INT8, weight.int8_blocks);
  else if (weight.quant_bits == 1 && !weight.binary_blocks.empty()) pick(LMB_BINARY, weight.binary_blocks);
  else if (weight.quant_bits == 2 && !weight.int2_blocks.empty()) pick(LMB_INT2, weight.int2_blocks);
  else if (weight.quant_bits == 3 && !weight.int3_blocks.empty()) pick(LMB_INT3, weight.int3_blocks);
  else if (weight.quant_bits == 5 && !weight.int5_blocks.empty()) pick(LMB_INT5, weight.int5_blocks);
  else if (weight.quant_bits == 6 && !weight.int6_blocks.empty()) pick(LMB_INT6, weight.int6_blocks);
  if (bytes == 0) throw std::runtime_error("lutmac_b200 (lut_linear): the tensor has no data for the kind its quant_bits select");
  // :92-93 -- not for the unquantised branch, which reads the caller's input as it is (:166-168)
  const bool rotate = kind != LMB_RAW_F32 && ((weight.quant_bits <= 2 && weight.quant_bits > 0) || !weight.blocks.empty());
  lmb_weight *w = resident(kind, data, bytes, M, K);
  const int st = lmb_linear_host(context(), w, bias, input, output, batch_size, rotate ? LMB_ROTATE : 0u);
  if (st != LMB_OK) fail(st, "lut_linear");
}

// src/kernels/transform_simd.cpp:26-110
void fwht_256(float *data) {
  const int st = lmb_apply_hadamard_rotation_host(data, 256);
  if (st != LMB_OK) fail(st, "fwht_256");
}

void apply_hadamard_rotation(float *data, size_t n) {
  const int st = lmb_apply_hadamard_rotation_host(data, n);
  if (st != LMB_OK) fail(st, "apply_hadamard_rotation");
}

}  // namespace lutmac
