// LUT GEMV for the bit-plane kinds (ternary, binary, RRQ 2-bit, 3-bit).
//
// Replaces lut_gemv / lut_gemv_binary / int2_gemv / int3_gemv
// (include/lutmac/lut_gemm.hpp:172-334; scalar loops src/kernels/lut_gemm_scalar.cpp:7-61,
// 228-259, 298-350) and, fused into the prologue, the padding + FWHT rotation of lut_linear
// (lut_gemm_scalar.cpp:85-113) and precompute_luts (lut_gemm.hpp:53-58).  The lookup
// formulation follows the reference's table kernels: ternary L[pos] - L[neg]
// (lut_gemm_simd.cpp:203-221), n-bit planes sum_p 2^p L[idx_p] - zero_point * L[15]
// (lut_gemm_simd.cpp:352-366), RRQ primary*scale + residual*scale2 (lut_gemm_simd.cpp:326-328).
//
// Work decomposition.  A CTA of 8 warps owns R row-tiles (32 rows each) and walks the K
// dimension in slices of S block-columns.  Per slice it (1) builds the 16-entry group tables
// of the slice in shared memory, one warp per 256-block, (2) streams the weight tiles: a warp
// handles a (row-tile, block-column) unit with one row per lane, 128-bit coalesced loads, and
// one shared-memory lookup per group and bit plane.  All lanes of a warp look into the same
// 64-byte table at lane-specific entries: 16 entries fall into 16 distinct banks, so the
// lookups are bank-conflict free by construction.
#include "common.cuh"
#include "device_utils.cuh"

namespace lmb {

namespace {

constexpr int WARPS = 8;
constexpr int THREADS = WARPS * 32;

struct LutParams {
  const uint8_t *tiles;
  const float *x;
  float *y;
  const float *bias;
  int M, bpr, row_tiles;
  int R;  // row-tiles per CTA: 1, 2, 4 or 8
  int S;  // block-columns per K-slice
  size_t x_len, x_stride, y_stride;
  int rotate;
};

// Sum of the 8 lookups addressed by the 8 nibbles of `w` (4 plane bytes, little endian) into
// 8 consecutive group tables starting at `t`.  Byte k holds groups 2k (high nibble) and 2k+1.
__device__ __forceinline__ float lut_word(uint32_t w, const float *t) {
  float s0 = 0.0f, s1 = 0.0f;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const uint32_t hi = (w >> (8 * k + 4)) & 15u, lo = (w >> (8 * k)) & 15u;
    s0 += t[(2 * k) * 16 + hi];
    s1 += t[(2 * k + 1) * 16 + lo];
  }
  return s0 + s1;
}

// 8 plane bytes {lo, hi} = 16 groups.
__device__ __forceinline__ float lut_8bytes(uint32_t lo, uint32_t hi, const float *t) {
  return lut_word(lo, t) + lut_word(hi, t + 8 * 16);
}
// 16 plane bytes = 32 groups.
__device__ __forceinline__ float lut_16bytes(const uint4 v, const float *t) {
  return (lut_word(v.x, t) + lut_word(v.y, t + 8 * 16)) + (lut_word(v.z, t + 16 * 16) + lut_word(v.w, t + 24 * 16));
}

template <int KIND> struct Unit {
  static constexpr int C = kind_info(KIND).chunks;
  static constexpr int NS = kind_info(KIND).nscales;
  uint4 v[C];
  float sc[NS];

  __device__ __forceinline__ void load(const uint8_t *tile, int lane) {
#pragma unroll
    for (int c = 0; c < C; ++c) v[c] = ld_stream_v4(tile + (size_t(c) * TILE_ROWS + lane) * 16);
#pragma unroll
    for (int s = 0; s < NS; ++s) sc[s] = ld_stream_f32(tile + size_t(C) * TILE_ROWS * 16 + (size_t(s) * TILE_ROWS + lane) * 4);
  }

  // Contribution of this row-block: scale * sum_i w_i x_i.
  __device__ __forceinline__ float eval(const float *tab, float xsum) const {
    if constexpr (KIND == LMB_TERNARY) {
      float p = 0.0f, n = 0.0f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        p += lut_8bytes(v[c].x, v[c].y, tab + c * 256);
        n += lut_8bytes(v[c].z, v[c].w, tab + c * 256);
      }
      return (p - n) * sc[0];
    } else if constexpr (KIND == LMB_BINARY) {
      const float a = lut_16bytes(v[0], tab) + lut_16bytes(v[1], tab + 512);
      return (2.0f * a - xsum) * sc[0];
    } else if constexpr (KIND == LMB_INT2) {
      float a1 = 0.0f, a2 = 0.0f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        a1 += lut_8bytes(v[c].x, v[c].y, tab + c * 256);
        a2 += lut_8bytes(v[c].z, v[c].w, tab + c * 256);
      }
      return (2.0f * a1 - xsum) * sc[0] + (2.0f * a2 - xsum) * sc[1];
    } else {  // LMB_INT3: chunk 3j+p holds plane 2-p of weights 128j..128j+127
      float q2 = lut_16bytes(v[0], tab) + lut_16bytes(v[3], tab + 512);
      float q1 = lut_16bytes(v[1], tab) + lut_16bytes(v[4], tab + 512);
      float q0 = lut_16bytes(v[2], tab) + lut_16bytes(v[5], tab + 512);
      return ((4.0f * q2 + 2.0f * q1 + q0) - 4.0f * xsum) * sc[0];
    }
  }
};

template <int KIND>
__global__ void __launch_bounds__(THREADS) k_gemv_lut(const LutParams p) {
  extern __shared__ __align__(16) float smem[];
  float *tab = smem;                         // [S][64][16]
  float *xsum = tab + size_t(p.S) * 1024;    // [S]
  float *part = xsum + ((p.S + 31) & ~31);   // [WARPS][32]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rt0 = blockIdx.x * p.R;
  const int nrt = min(p.R, p.row_tiles - rt0);
  const int wpr = WARPS / p.R;  // warps sharing one row-tile
  const int rtl = warp / wpr, sub = warp - rtl * wpr;
  const float *x = p.x + size_t(blockIdx.y) * p.x_stride;
  constexpr size_t TB = tile_bytes(KIND);

  float acc = 0.0f;
  for (int b0 = 0; b0 < p.bpr; b0 += p.S) {
    const int ns = min(p.S, p.bpr - b0);
    if (b0 > 0) __syncthreads();  // the previous slice's tables are still being read
    for (int bl = warp; bl < ns; bl += WARPS)
      build_block_tables(x, p.x_len, size_t(b0 + bl), p.rotate != 0, lane, tab + size_t(bl) * 1024, xsum + bl);
    __syncthreads();
    if (rtl < nrt) {
      const uint8_t *row_tiles = p.tiles + (size_t(rt0 + rtl) * p.bpr + b0) * TB;
      Unit<KIND> cur;
      if (sub < ns) cur.load(row_tiles + size_t(sub) * TB, lane);
      for (int bl = sub; bl < ns; bl += wpr) {
        Unit<KIND> nxt;
        const bool more = bl + wpr < ns;
        if (more) nxt.load(row_tiles + size_t(bl + wpr) * TB, lane);
        acc += cur.eval(tab + size_t(bl) * 1024, xsum[bl]);
        if (more) cur = nxt;
      }
    }
  }
  // Combine the partial sums of the warps that share a row-tile, in warp order.
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

// Tables only (debug view used by the parity tests): one warp per 256-block.
__global__ void k_debug_luts(const float *x, size_t x_len, int nblocks, int rotate, float *out) {
  __shared__ __align__(16) float tab[WARPS][1024];
  __shared__ float xs[WARPS];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.x * WARPS + warp;
  if (b < nblocks) {
    build_block_tables(x, x_len, size_t(b), rotate != 0, lane, tab[warp], &xs[warp]);
    __syncwarp();
    for (int i = lane; i < 1024; i += 32) out[size_t(b) * 1024 + i] = tab[warp][i];
  }
}

template <int KIND> int launch_kind(lmb_ctx *ctx, const LinearArgs &a) {
  const lmb_weight *w = a.w;
  LutParams p;
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
  // Row-tiles per CTA: as many as keep at least two CTAs per SM in flight.
  int R = 8;
  while (R > 1 && (p.row_tiles + R - 1) / R < 2 * ctx->sm_count) R >>= 1;
  p.R = R;
  // K-slice: whole K if its tables fit in ~96 KB, else equal slices.
  const int s_max = 24;
  const int nslices = (p.bpr + s_max - 1) / s_max;
  p.S = (p.bpr + nslices - 1) / nslices;
  const size_t smem = (size_t(p.S) * 1024 + ((p.S + 31) & ~31) + WARPS * 32) * sizeof(float);
  dim3 grid((p.row_tiles + R - 1) / R, unsigned(a.batch));
  k_gemv_lut<KIND><<<grid, THREADS, smem, ctx->stream>>>(p);
  ctx->launches++;
  LMB_CUDA(cudaGetLastError());
  return LMB_OK;
}

}  // namespace

// Opt every instantiation into the device's full dynamic shared memory (once per context).
int configure_gemv_lut(lmb_ctx *ctx) {
  const int bytes = int(ctx->smem_optin);
  LMB_CUDA(cudaFuncSetAttribute(k_gemv_lut<LMB_TERNARY>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  LMB_CUDA(cudaFuncSetAttribute(k_gemv_lut<LMB_BINARY>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  LMB_CUDA(cudaFuncSetAttribute(k_gemv_lut<LMB_INT2>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  LMB_CUDA(cudaFuncSetAttribute(k_gemv_lut<LMB_INT3>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  return LMB_OK;
}

int launch_gemv_lut(lmb_ctx *ctx, const LinearArgs &a) {
  switch (a.w->kind) {
  case LMB_TERNARY: return launch_kind<LMB_TERNARY>(ctx, a);
  case LMB_BINARY: return launch_kind<LMB_BINARY>(ctx, a);
  case LMB_INT2: return launch_kind<LMB_INT2>(ctx, a);
  case LMB_INT3: return launch_kind<LMB_INT3>(ctx, a);
  default: set_last_error("launch_gemv_lut: kind is not a bit-plane kind"); return LMB_ERR_ARG;
  }
}

int launch_debug_luts(lmb_ctx *ctx, const float *d_x, size_t x_len, bool rotate, float *d_out) {
  const int nblocks = int((x_len + BLK - 1) / BLK);
  k_debug_luts<<<(nblocks + WARPS - 1) / WARPS, THREADS, 0, ctx->stream>>>(d_x, x_len, nblocks, rotate ? 1 : 0, d_out);
  ctx->launches++;
  LMB_CUDA(cudaGetLastError());
  return LMB_OK;
}

}  // namespace lmb
