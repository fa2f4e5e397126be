// Quantize + pack on the device: fp32 weights -> the reference's block structs, code for code.
//
// Replaces quantize_tensor (ternary, include/lutmac/quantize.hpp:193-336 with quantize_ternary
// :83-88, compute_absmean_threshold :93-102 and pack_to_bitplanes :135-154), quantize_tensor_binary
// (:725-823), quantize_tensor_int2 (:918-975), quantize_tensor_int3 (:982-1039),
// quantize_tensor_int4 (:387-495) and quantize_tensor_int8 (:833-911, Int8Block::set
// types.hpp:441-461) for 2-D tensors.  The Hadamard rotation the reference's quantize tool applies
// to the weights of its <= 2-bit formats (tools/lutmac-quantize.cpp:423-453: apply_hadamard_rotation
// over the flat array) is lmb_fwht256 on the same buffer, called first.
//
// One warp per 256-weight block, lane l holding weights 8l..8l+7 -- which is exactly one byte of a
// ternary / binary plane, two bytes of 2-bit codes, three bytes of the 3-bit stream, four bytes
// of nibbles or eight int8 codes, so every lane packs and stores its own bytes.  Arithmetic that
// decides a code follows the reference operation for operation (absmax / 7, v * (1 / scale),
// round half away from zero, clamp), so the codes are bit-exact; block maxima are order-free;
// the one order-dependent float sum (the ternary block scale, a left-to-right float sum of the
// large weights) is added by one lane in the reference's order.
#include <cstring>

#include "common.cuh"
#include "device_utils.cuh"

namespace lmb {

namespace {

constexpr int QT_WARPS = 8;

__device__ __forceinline__ int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }

// sum over the tensor of |w| in double: per-CTA partial sums (a fixed tree per CTA), added in CTA order afterwards
__global__ void __launch_bounds__(256) k_abs_sum_partials(const float *w, size_t n, double *partials) {
  __shared__ double red[256];
  double s = 0.0;
  for (size_t i = size_t(blockIdx.x) * 256 + threadIdx.x; i < n; i += size_t(gridDim.x) * 256) s += double(fabsf(w[i]));
  red[threadIdx.x] = s;
  __syncthreads();
  for (int m = 128; m > 0; m >>= 1) {
    if (int(threadIdx.x) < m) red[threadIdx.x] += red[threadIdx.x + m];
    __syncthreads();
  }
  if (threadIdx.x == 0) partials[blockIdx.x] = red[0];
}

// threshold = mean |w| as a float (quantize.hpp:93-102); thr[0] = threshold, thr[1] = 0.5 * threshold (:211,271)
__global__ void k_abs_mean(const double *partials, int n_partials, size_t n, float *thr) {
  double s = 0.0;
  for (int i = 0; i < n_partials; ++i) s += partials[i];
  const float t = float(s / double(n));
  thr[0] = t;
  thr[1] = 0.5f * t;
}

// Blocks of a 2-D tensor: row-blocks (every row padded to whole blocks) for ternary, binary, 4- and
// 8-bit; the 2- and 3-bit quantizers walk the FLAT element stream in chunks of 256 instead
// (quantize.hpp:918-975, :982-1039).
template <int KIND>
__global__ void __launch_bounds__(QT_WARPS * 32) k_quantize(const float *w, size_t M, size_t K, const float *thr, uint8_t *out) {
  __shared__ float stage[QT_WARPS][BLK];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const size_t bpr = (K + BLK - 1) / BLK, nblocks = M * bpr;
  const size_t blk = size_t(blockIdx.x) * QT_WARPS + warp;
  if (blk >= nblocks) return;
  constexpr bool FLAT = (KIND == LMB_INT2 || KIND == LMB_INT3);
  size_t base, valid;
  if (FLAT) {
    const size_t n = M * K, start = blk * BLK;
    base = start;
    valid = start < n ? (n - start < size_t(BLK) ? n - start : size_t(BLK)) : 0;
  } else {
    const size_t r = blk / bpr, b = blk - r * bpr, start = b * BLK;
    base = r * K + start;
    valid = start < K ? (K - start < size_t(BLK) ? K - start : size_t(BLK)) : 0;
  }
  float v[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const size_t i = size_t(lane) * 8 + j;
    v[j] = i < valid ? w[base + i] : 0.0f;
  }
  uint8_t *dst = out + blk * size_t(kind_info(KIND).ref_bytes);

  if constexpr (KIND == LMB_TERNARY) {
    const float threshold = thr[0], zero_thr = thr[1];
    unsigned sign = 0, zero = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const bool in = size_t(lane) * 8 + j < valid;
      const float a = fabsf(v[j]);
      const int t = (!in || a < zero_thr) ? 0 : (v[j] > 0.0f ? 1 : -1);  // quantize.hpp:83-88; padding is zero
      if (t < 0) sign |= 1u << (7 - j);
      if (t == 0) zero |= 1u << (7 - j);
      stage[warp][lane * 8 + j] = (in && a >= threshold) ? a : -1.0f;  // -1: not part of the scale
    }
    dst[lane] = uint8_t(sign);        // sign_plane[32]
    dst[32 + lane] = uint8_t(zero);   // zero_plane[32]
    __syncwarp();
    if (lane == 0) {  // the reference's float accumulator, left to right (quantize.hpp:268-287)
      float scale_sum = 0.0f;
      unsigned count = 0;
      for (int i = 0; i < BLK; ++i) {
        const float a = stage[warp][i];
        if (a >= 0.0f) {
          scale_sum += a;
          ++count;
        }
      }
      const float scale = count > 0 ? scale_sum / float(count) : 1.0f;
      memcpy(dst + 64, &scale, 4);
    }
  } else if constexpr (KIND == LMB_BINARY) {
    double s = 0.0;
#pragma unroll
    for (int j = 0; j < 8; ++j) s += double(fabsf(v[j]));  // padding adds zero
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) s += __shfl_xor_sync(0xffffffffu, s, m);
    unsigned bits = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (v[j] >= 0.0f) bits |= 1u << (7 - j);  // padding (0.0) packs as +1, like the reference
    dst[lane] = uint8_t(bits);
    if (lane == 0) {
      const float scale = valid > 0 ? float(s / double(valid)) : 0.0f;
      memcpy(dst + 32, &scale, 4);
    }
  } else {
    float amax = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
    if constexpr (KIND == LMB_INT4) {
      const float scale = amax / 7.0f, inv = scale > 1e-10f ? 1.0f / scale : 0.0f;
      unsigned q[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) q[j] = unsigned(clampi(int(roundf(v[j] * inv)), -7, 7) + 8);
#pragma unroll
      for (int j = 0; j < 4; ++j) dst[lane * 4 + j] = uint8_t((q[2 * j] << 4) | q[2 * j + 1]);  // even weight in the high nibble
      if (lane == 0) memcpy(dst + 128, &scale, 4);
    } else if constexpr (KIND == LMB_INT8) {
      const float scale = amax / 127.0f;
      if (lane == 0) memcpy(dst, &scale, 4);  // scale first (types.hpp:434-438)
      const float inv = scale != 0.0f ? 1.0f / scale : 0.0f;  // an all-zero block keeps zero codes (types.hpp:447-449)
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float x = fmaxf(-127.0f, fminf(127.0f, v[j] * inv));
        dst[4 + lane * 8 + j] = uint8_t(int8_t(roundf(x)));
      }
    } else if constexpr (KIND == LMB_INT2) {
      const float scale = amax / 2.0f, inv = scale > 1e-10f ? 1.0f / scale : 0.0f;
      unsigned b0 = 0, b1 = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        b0 |= unsigned(clampi(int(roundf(v[j] * inv)), -2, 1) + 2) << (6 - 2 * j);
        b1 |= unsigned(clampi(int(roundf(v[4 + j] * inv)), -2, 1) + 2) << (6 - 2 * j);
      }
      dst[lane * 2] = uint8_t(b0);
      dst[lane * 2 + 1] = uint8_t(b1);
      if (lane == 0) {
        const float zero = 0.0f;
        memcpy(dst + 64, &scale, 4);
        memcpy(dst + 68, &zero, 4);  // the residual scale is never written by the reference's quantizer
      }
    } else {  // LMB_INT3: eight 3-bit codes = three bytes, most significant bit first (types.hpp:268-288)
      const float scale = amax / 4.0f, inv = scale > 1e-10f ? 1.0f / scale : 0.0f;
      unsigned bits = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) bits |= unsigned(clampi(int(roundf(v[j] * inv)), -4, 3) + 4) << (21 - 3 * j);
      dst[lane * 3] = uint8_t(bits >> 16);
      dst[lane * 3 + 1] = uint8_t(bits >> 8);
      dst[lane * 3 + 2] = uint8_t(bits);
      if (lane == 0) memcpy(dst + 96, &scale, 4);
    }
  }
}

}  // namespace

}  // namespace lmb

using namespace lmb;

extern "C" {

int lmb_quantize(lmb_ctx *ctx, int kind, const float *d_weights, size_t M, size_t K, void *d_blocks_out) {
  LMB_REQUIRE(ctx && d_weights && d_blocks_out && M > 0 && K > 0, "lmb_quantize: bad argument");
  const size_t bpr = (K + BLK - 1) / BLK, nblocks = M * bpr;
  const unsigned grid = unsigned((nblocks + QT_WARPS - 1) / QT_WARPS);
  uint8_t *out = static_cast<uint8_t *>(d_blocks_out);
  switch (kind) {
  case LMB_TERNARY: {
    const int n_part = 1024;
    double *partials = nullptr;
    float *thr = nullptr;
    LMB_CUDA(cudaMalloc(&partials, n_part * sizeof(double)));
    cudaError_t e = cudaMalloc(&thr, 2 * sizeof(float));
    if (e != cudaSuccess) {
      cudaFree(partials);
      return cuda_fail(e, "lmb_quantize");
    }
    k_abs_sum_partials<<<n_part, 256, 0, ctx->stream>>>(d_weights, M * K, partials);
    k_abs_mean<<<1, 1, 0, ctx->stream>>>(partials, n_part, M * K, thr);
    k_quantize<LMB_TERNARY><<<grid, QT_WARPS * 32, 0, ctx->stream>>>(d_weights, M, K, thr, out);
    ctx->launches += 3;
    e = cudaStreamSynchronize(ctx->stream);
    cudaFree(partials);
    cudaFree(thr);
    if (e != cudaSuccess) return cuda_fail(e, "lmb_quantize");
    break;
  }
  case LMB_BINARY: k_quantize<LMB_BINARY><<<grid, QT_WARPS * 32, 0, ctx->stream>>>(d_weights, M, K, nullptr, out); ctx->launches++; break;
  case LMB_INT2: k_quantize<LMB_INT2><<<grid, QT_WARPS * 32, 0, ctx->stream>>>(d_weights, M, K, nullptr, out); ctx->launches++; break;
  case LMB_INT3: k_quantize<LMB_INT3><<<grid, QT_WARPS * 32, 0, ctx->stream>>>(d_weights, M, K, nullptr, out); ctx->launches++; break;
  case LMB_INT4: k_quantize<LMB_INT4><<<grid, QT_WARPS * 32, 0, ctx->stream>>>(d_weights, M, K, nullptr, out); ctx->launches++; break;
  case LMB_INT8: k_quantize<LMB_INT8><<<grid, QT_WARPS * 32, 0, ctx->stream>>>(d_weights, M, K, nullptr, out); ctx->launches++; break;
  default: set_last_error("lmb_quantize: ternary, binary, 2-, 3-, 4- and 8-bit blocks are quantised on the device"); return LMB_ERR_ARG;
  }
  LMB_CUDA(cudaGetLastError());
  return LMB_OK;
}

int lmb_quantize_host(lmb_ctx *ctx, int kind, const float *weights, size_t M, size_t K, int rotate_first, void *blocks_out) {
  LMB_REQUIRE(ctx && weights && blocks_out && M > 0 && K > 0, "lmb_quantize_host: bad argument");
  LMB_REQUIRE(kind_valid(kind) && kind != LMB_INT5 && kind != LMB_INT6, "lmb_quantize_host: unsupported block kind");
  const size_t n = M * K, nblocks = M * ((K + BLK - 1) / BLK), bytes = nblocks * size_t(kind_info(kind).ref_bytes);
  float *d_w = nullptr;
  uint8_t *d_b = nullptr;
  LMB_CUDA(cudaSetDevice(ctx->device));
  LMB_CUDA(cudaMalloc(&d_w, n * sizeof(float)));
  cudaError_t e = cudaMalloc(&d_b, bytes);
  if (e == cudaSuccess) e = cudaMemcpyAsync(d_w, weights, n * sizeof(float), cudaMemcpyHostToDevice, ctx->stream);
  int st = e == cudaSuccess ? LMB_OK : cuda_fail(e, "lmb_quantize_host");
  // the reference's tool rotates the FLAT array in chunks of 256 before its <= 2-bit quantizers
  if (st == LMB_OK && rotate_first) st = launch_fwht256(ctx, d_w, n);
  if (st == LMB_OK) st = lmb_quantize(ctx, kind, d_w, M, K, d_b);
  if (st == LMB_OK) {
    e = cudaMemcpyAsync(blocks_out, d_b, bytes, cudaMemcpyDeviceToHost, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) st = cuda_fail(e, "lmb_quantize_host");
  }
  cudaFree(d_w);
  if (d_b) cudaFree(d_b);
  return st;
}

}  // extern "C"
