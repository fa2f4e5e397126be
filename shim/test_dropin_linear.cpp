// lut_linear through the drop-in (the reference's own tests never call it): every branch of its
// dispatch ladder -- ternary and 2-bit with the rotated input, 4-bit and 8-bit without, the
// unquantised fp32 dot product -- with a K that needs zero padding, a bias and a batch of 3,
// against an fp64 evaluation of  W_dequantised * rot?(pad(x)) + bias  built from the reference's
// own block accessors (Block::get) and a textbook 256-point Walsh-Hadamard transform / 16.
// Built against the reference's headers; exits non-zero on the first mismatch above 1e-5 rel L2.
#include <cmath>
#include <cstdio>
#include <random>
#include <vector>

#include "lutmac/lut_gemm.hpp"
#include "lutmac/quantize.hpp"
#include "lutmac/transform.hpp"

using namespace lutmac;

static void fwht256_f64(double *d) {
  for (int h = 1; h < 256; h <<= 1)
    for (int i = 0; i < 256; i += 2 * h)
      for (int j = i; j < i + h; ++j) {
        const double a = d[j], b = d[j + h];
        d[j] = a + b;
        d[j + h] = a - b;
      }
  for (int i = 0; i < 256; ++i) d[i] /= 16.0;
}

template <class Get>
static int check(const char *name, const PackedTensor &t, bool rotate, Get get, std::mt19937 &rng) {
  const size_t M = t.shape[0], K = t.shape[1], kp = (K + 255) / 256 * 256, batch = 3;
  std::normal_distribution<float> nd(0.0f, 1.0f);
  std::vector<float> x(batch * K), bias(M), y(batch * M, -1.0f);
  for (auto &v : x) v = nd(rng);
  for (auto &v : bias) v = 0.1f * nd(rng);
  lut_linear(t, bias.data(), x.data(), y.data(), batch);
  double num = 0.0, den = 0.0;
  for (size_t b = 0; b < batch; ++b) {
    std::vector<double> xp(kp, 0.0);
    for (size_t k = 0; k < K; ++k) xp[k] = x[b * K + k];
    if (rotate)
      for (size_t k = 0; k < kp; k += 256) fwht256_f64(xp.data() + k);
    for (size_t r = 0; r < M; ++r) {
      double acc = bias[r];
      for (size_t k = 0; k < (rotate ? kp : K); ++k) acc += double(get(r, k)) * xp[k];
      const double d = double(y[b * M + r]) - acc;
      num += d * d;
      den += acc * acc;
    }
  }
  const double err = std::sqrt(num / den);
  std::printf("%-10s M=%zu K=%zu batch=%zu rotate=%d  rel L2 %.3e  %s\n", name, M, K, batch, int(rotate), err, err < 1e-5 ? "ok" : "FAIL");
  return err < 1e-5 ? 0 : 1;
}

int main() {
  std::mt19937 rng(7);
  const size_t M = 96, K = 600;  // K pads to 768
  const size_t bpr = (K + 255) / 256;
  std::uniform_real_distribution<float> ud(-1.0f, 1.0f);
  std::vector<float> w(M * K);
  for (auto &v : w) v = ud(rng);
  int bad = 0;
  {
    PackedTensor t = quantize_tensor(w.data(), {M, K});  // ternary: rotates (non-empty block vector)
    bad += check("ternary", t, true, [&](size_t r, size_t k) { return t.blocks[r * bpr + k / 256].get(k % 256); }, rng);
  }
  {
    PackedTensor t = quantize_tensor_int2(w.data(), {M, K});  // quant_bits 2: rotates
    for (auto &blk : t.int2_blocks) blk.scale2 = 0.3f * blk.scale;  // a residual plane the quantizer never writes
    bad += check("int2 (RRQ)", t, true, [&](size_t r, size_t k) { return t.int2_blocks[r * bpr + k / 256].get(k % 256); }, rng);
  }
  {
    PackedTensor t = quantize_tensor_int4(w.data(), {M, K});
    bad += check("int4", t, false, [&](size_t r, size_t k) { return t.int4_blocks[r * bpr + k / 256].get(k % 256); }, rng);
  }
  {
    PackedTensor t = quantize_tensor_int8(w.data(), {M, K});
    bad += check("int8", t, false, [&](size_t r, size_t k) { return t.int8_blocks[r * bpr + k / 256].get(k % 256); }, rng);
  }
  {
    PackedTensor t;  // unquantised: the fp32 dot product
    t.shape = {M, K};
    t.is_quantized = false;
    t.quant_bits = 32;
    t.raw_data = w;
    bad += check("raw fp32", t, false, [&](size_t r, size_t k) { return w[r * K + k]; }, rng);
  }
  {
    PackedTensor t = quantize_tensor_int4(w.data(), {M, K});  // a 1-D "shape": returns without touching the output
    t.shape = {M * K};
    float out = 42.0f, in = 1.0f;
    lut_linear(t, nullptr, &in, &out, 1);
    if (out != 42.0f) {
      std::printf("non-2-D tensor: output touched  FAIL\n");
      ++bad;
    }
  }
  std::printf("%s\n", bad ? "FAILED" : "all lut_linear branches ok");
  return bad;
}
