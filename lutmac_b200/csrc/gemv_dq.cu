// Dequantise-and-FMA GEMV for the byte/nibble kinds (4-bit, 8-bit).
//
// Replaces int4_gemv / int8_gemv (include/lutmac/lut_gemm.hpp:238-250, 396-408; scalar loops
// src/kernels/lut_gemm_scalar.cpp:186-222, 265-292) and the zero padding (and optional
// rotation) of lut_linear (lut_gemm_scalar.cpp:85-113), fused into the prologue.
//
// Same decomposition as the LUT kernel: a CTA of 8 warps owns R row-tiles, one row per lane,
// 128-bit coalesced weight loads; the activations of a K-slice sit in shared memory and are
// read as broadcast float4.  Codes become fp32 without integer-to-float conversions: a
// nibble (or byte) is OR-ed into the mantissa of 2^23, and one exact subtraction removes
// 2^23 together with the code's zero point (8 for 4-bit, 128 after the sign flip for 8-bit).
// A nibble that sits p bits up in its word is not shifted down: it yields (q-8)*2^p, is
// accumulated in a slot of its own, and the slot is rescaled by 2^-p once per row-block
// (both scalings are exact).  Subtract and multiply-add run as packed fp32 pairs.
#include "common.cuh"
#include "device_utils.cuh"

namespace lmb {

namespace {

constexpr int WARPS = 8;
constexpr int THREADS = WARPS * 32;

struct DqParams {
  const uint8_t *tiles;
  const float *x;
  float *y;
  const float *bias;
  int M, bpr, row_tiles;
  int R, S;
  size_t x_len, x_stride, y_stride;
  int rotate;
};

__device__ __forceinline__ float as_f(uint32_t u) { return __uint_as_float(u); }

constexpr uint32_t MAGIC = 0x4B000000u;  // 2^23

// -(2^23 + 8 * 2^p): removes the magic and the zero point 8 of a nibble sitting at bit p.
__device__ __forceinline__ constexpr float nib_bias(int p) { return -(8388608.0f + 8.0f * float(1 << p)); }

// 8 weights of one 32-bit word of 4-bit codes (byte j: weight 2j in the high nibble, 2j+1 in
// the low nibble, types.hpp:184-190) times 8 activations {xa, xb}.
__device__ __forceinline__ void int4_word(uint32_t w, const float4 xa, const float4 xb, float2 acc[4]) {
  const uint32_t h = w >> 12;  // brings bits 20..31 down to 8..19
  float2 g;
  g = add2(make_float2(as_f((w & 0x000000F0u) | MAGIC), as_f((w & 0x0000000Fu) | MAGIC)),
           make_float2(nib_bias(4), nib_bias(0)));
  fma2(acc[0], g, make_float2(xa.x, xa.y));
  g = add2(make_float2(as_f((w & 0x0000F000u) | MAGIC), as_f((w & 0x00000F00u) | MAGIC)),
           make_float2(nib_bias(12), nib_bias(8)));
  fma2(acc[1], g, make_float2(xa.z, xa.w));
  g = add2(make_float2(as_f((h & 0x00000F00u) | MAGIC), as_f((w & 0x000F0000u) | MAGIC)),
           make_float2(nib_bias(8), nib_bias(16)));
  fma2(acc[2], g, make_float2(xb.x, xb.y));
  g = add2(make_float2(as_f((h & 0x000F0000u) | MAGIC), as_f((h & 0x0000F000u) | MAGIC)),
           make_float2(nib_bias(16), nib_bias(12)));
  fma2(acc[3], g, make_float2(xb.z, xb.w));
}

__device__ __forceinline__ float int4_finish(const float2 acc[4]) {
  // slot scalings: acc0 (2^4, 1), acc1 (2^12, 2^8), acc2 (2^8, 2^16), acc3 (2^16, 2^12)
  const float s0 = acc[0].y + acc[0].x * 0.0625f;
  const float s8 = (acc[1].y + acc[2].x) * (1.0f / 256.0f);
  const float s12 = (acc[1].x + acc[3].y) * (1.0f / 4096.0f);
  const float s16 = (acc[2].y + acc[3].x) * (1.0f / 65536.0f);
  return (s0 + s8) + (s12 + s16);
}

// 4 weights of one word of int8 codes times 4 activations.
__device__ __forceinline__ void int8_word(uint32_t w, const float4 xv, float2 acc[2]) {
  const uint32_t u = w ^ 0x80808080u;  // q + 128 in every byte
  const float2 c = make_float2(-(8388608.0f + 128.0f), -(8388608.0f + 128.0f));
  float2 g;
  g = add2(make_float2(as_f(__byte_perm(u, MAGIC, 0x7540)), as_f(__byte_perm(u, MAGIC, 0x7541))), c);
  fma2(acc[0], g, make_float2(xv.x, xv.y));
  g = add2(make_float2(as_f(__byte_perm(u, MAGIC, 0x7542)), as_f(__byte_perm(u, MAGIC, 0x7543))), c);
  fma2(acc[1], g, make_float2(xv.z, xv.w));
}

template <int KIND> struct DqUnit;

template <> struct DqUnit<LMB_INT4> {
  uint4 v[8];
  float sc = 0.0f;
  __device__ __forceinline__ void load(const uint8_t *tile, int lane) {
#pragma unroll
    for (int c = 0; c < 8; ++c) v[c] = ld_stream_v4(tile + (size_t(c) * TILE_ROWS + lane) * 16);
    sc = ld_stream_f32(tile + size_t(8) * TILE_ROWS * 16 + size_t(lane) * 4);
  }
  __device__ __forceinline__ float eval(const float *xs) const {
    const float4 *x4 = reinterpret_cast<const float4 *>(xs);
    float2 acc[4] = {{0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}};
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      int4_word(v[c].x, x4[8 * c + 0], x4[8 * c + 1], acc);
      int4_word(v[c].y, x4[8 * c + 2], x4[8 * c + 3], acc);
      int4_word(v[c].z, x4[8 * c + 4], x4[8 * c + 5], acc);
      int4_word(v[c].w, x4[8 * c + 6], x4[8 * c + 7], acc);
    }
    return int4_finish(acc) * sc;
  }
};

// An 8-bit row-block is 256 B per lane; it is streamed in two halves to bound registers.
template <> struct DqUnit<LMB_INT8> {
  uint4 v[8];
  float sc = 0.0f;
  __device__ __forceinline__ void load_half(const uint8_t *tile, int lane, int half) {
#pragma unroll
    for (int c = 0; c < 8; ++c) v[c] = ld_stream_v4(tile + (size_t(8 * half + c) * TILE_ROWS + lane) * 16);
  }
  __device__ __forceinline__ void load_scale(const uint8_t *tile, int lane) {
    sc = ld_stream_f32(tile + size_t(16) * TILE_ROWS * 16 + size_t(lane) * 4);
  }
  __device__ __forceinline__ float eval_half(const float *xs_half) const {
    const float4 *x4 = reinterpret_cast<const float4 *>(xs_half);
    float2 acc[2] = {{0.f, 0.f}, {0.f, 0.f}};
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      int8_word(v[c].x, x4[4 * c + 0], acc);
      int8_word(v[c].y, x4[4 * c + 1], acc);
      int8_word(v[c].z, x4[4 * c + 2], acc);
      int8_word(v[c].w, x4[4 * c + 3], acc);
    }
    return (acc[0].x + acc[0].y) + (acc[1].x + acc[1].y);
  }
};

template <int KIND>
__global__ void __launch_bounds__(THREADS) k_gemv_dq(const DqParams p) {
  extern __shared__ __align__(16) float smem[];
  float *xs = smem;                              // [S][256]
  float *part = xs + size_t(p.S) * 256;          // [WARPS][32]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rt0 = blockIdx.x * p.R;
  const int nrt = min(p.R, p.row_tiles - rt0);
  const int wpr = WARPS / p.R;
  const int rtl = warp / wpr, sub = warp - rtl * wpr;
  const float *x = p.x + size_t(blockIdx.y) * p.x_stride;
  constexpr size_t TB = tile_bytes(KIND);

  float acc = 0.0f;
  for (int b0 = 0; b0 < p.bpr; b0 += p.S) {
    const int ns = min(p.S, p.bpr - b0);
    if (b0 > 0) __syncthreads();
    for (int bl = warp; bl < ns; bl += WARPS) {
      float v[8];
      load_x8(x, p.x_len, size_t(b0 + bl), lane, v);
      if (p.rotate) fwht256_warp(v, lane);
      float4 *o = reinterpret_cast<float4 *>(xs + size_t(bl) * 256 + lane * 8);
      o[0] = make_float4(v[0], v[1], v[2], v[3]);
      o[1] = make_float4(v[4], v[5], v[6], v[7]);
    }
    __syncthreads();
    if (rtl < nrt) {
      const uint8_t *row_tiles = p.tiles + (size_t(rt0 + rtl) * p.bpr + b0) * TB;
      if constexpr (KIND == LMB_INT4) {
        DqUnit<LMB_INT4> cur;
        if (sub < ns) cur.load(row_tiles + size_t(sub) * TB, lane);
        for (int bl = sub; bl < ns; bl += wpr) {
          DqUnit<LMB_INT4> nxt;
          const bool more = bl + wpr < ns;
          if (more) nxt.load(row_tiles + size_t(bl + wpr) * TB, lane);
          acc += cur.eval(xs + size_t(bl) * 256);
          if (more) cur = nxt;
        }
      } else {
        // half-blocks: h = 2*bl + half
        DqUnit<LMB_INT8> cur;
        if (sub < ns) {
          cur.load_half(row_tiles + size_t(sub) * TB, lane, 0);
          cur.load_scale(row_tiles + size_t(sub) * TB, lane);
        }
        for (int bl = sub; bl < ns; bl += wpr) {
          const uint8_t *tile = row_tiles + size_t(bl) * TB;
          DqUnit<LMB_INT8> nxt;
          nxt.load_half(tile, lane, 1);
          float s = cur.eval_half(xs + size_t(bl) * 256);
          const float scale = cur.sc;
          cur = nxt;
          const bool more = bl + wpr < ns;
          if (more) {
            nxt.load_half(tile + size_t(wpr) * TB, lane, 0);
            nxt.load_scale(tile + size_t(wpr) * TB, lane);
          }
          s += cur.eval_half(xs + size_t(bl) * 256 + 128);
          acc += s * scale;
          if (more) cur = nxt;
        }
      }
    }
  }
  part[warp * 32 + lane] = acc;
  __syncthreads();
  if (sub == 0 && rtl < nrt) {
    float s = part[warp * 32 + lane];
    for (int k = 1; k < wpr; ++k) s += part[(warp + k) * 32 + lane];
    const int row = (rt0 + rtl) * TILE_ROWS + lane;
    if (row < p.M) {
      if (p.bias) s += p.bias[row];
      p.y[size_t(blockIdx.y) * p.y_stride + row] = s;
    }
  }
}

template <int KIND> int launch_kind(lmb_ctx *ctx, const LinearArgs &a) {
  const lmb_weight *w = a.w;
  DqParams p;
  p.tiles = w->d_tiles;
  p.x = a.x;
  p.y = a.y;
  p.bias = a.bias;
  p.M = int(w->M);
  p.bpr = int(w->bpr);
  p.row_tiles = int(w->row_tiles);
  p.x_len = a.x_len;
  p.x_stride = a.x_stride;
  p.y_stride = a.y_stride;
  p.rotate = a.rotate ? 1 : 0;
  int R = 8;
  while (R > 1 && (p.row_tiles + R - 1) / R < 2 * ctx->sm_count) R >>= 1;
  p.R = R;
  const int s_max = 64;  // 64 KB of activations per slice
  const int nslices = (p.bpr + s_max - 1) / s_max;
  p.S = (p.bpr + nslices - 1) / nslices;
  const size_t smem = (size_t(p.S) * 256 + WARPS * 32) * sizeof(float);
  dim3 grid((p.row_tiles + R - 1) / R, unsigned(a.batch));
  k_gemv_dq<KIND><<<grid, THREADS, smem, ctx->stream>>>(p);
  ctx->launches++;
  LMB_CUDA(cudaGetLastError());
  return LMB_OK;
}

}  // namespace

int configure_gemv_dq(lmb_ctx *ctx) {
  const int bytes = int(ctx->smem_optin);
  LMB_CUDA(cudaFuncSetAttribute(k_gemv_dq<LMB_INT4>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  LMB_CUDA(cudaFuncSetAttribute(k_gemv_dq<LMB_INT8>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  return LMB_OK;
}

int launch_gemv_dq(lmb_ctx *ctx, const LinearArgs &a) {
  switch (a.w->kind) {
  case LMB_INT4: return launch_kind<LMB_INT4>(ctx, a);
  case LMB_INT8: return launch_kind<LMB_INT8>(ctx, a);
  default: set_last_error("launch_gemv_dq: kind has no dequantise kernel"); return LMB_ERR_ARG;
  }
}

}  // namespace lmb
