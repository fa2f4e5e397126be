// Device helpers shared by the GEMV kernels: streaming loads, the in-register 256-point FWHT,
// the group-of-4 LUT construction and packed-fp32 arithmetic.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

namespace lmb {

// 128-bit streaming load of weight payload: read-only path, no L1 allocation (each byte is
// used once).
__device__ __forceinline__ uint4 ld_stream_v4(const void *p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ float4 ld_stream_v4f(const void *p) {
  float4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ float ld_stream_f32(const void *p) {
  float v;
  asm volatile("ld.global.nc.L1::no_allocate.f32 %0, [%1];" : "=f"(v) : "l"(p));
  return v;
}

// Packed fp32 pairs (sm_100 FFMA2 / FADD2): one instruction, two IEEE fp32 results.
__device__ __forceinline__ void fma2(float2 &acc, const float2 a, const float2 b) {
  unsigned long long &c = reinterpret_cast<unsigned long long &>(acc);
  asm("fma.rn.f32x2 %0, %1, %2, %0;"
      : "+l"(c)
      : "l"(reinterpret_cast<const unsigned long long &>(a)), "l"(reinterpret_cast<const unsigned long long &>(b)));
}
__device__ __forceinline__ float2 add2(const float2 a, const float2 b) {
  float2 r;
  asm("add.rn.f32x2 %0, %1, %2;"
      : "=l"(reinterpret_cast<unsigned long long &>(r))
      : "l"(reinterpret_cast<const unsigned long long &>(a)), "l"(reinterpret_cast<const unsigned long long &>(b)));
  return r;
}

// gelu(x) of src/model.cpp:38-42 (tanh form)
__device__ __forceinline__ float gelu_tanh(float x) {
  return 0.5f * x * (1.0f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x)));
}

// Loads the lane's 8 consecutive activations of 256-block `b` (elements b*256 + lane*8 + j);
// positions at or beyond x_len read as zero, which is lut_linear's zero padding
// (lut_gemm_scalar.cpp:101-106).
__device__ __forceinline__ void load_x8(const float *__restrict__ x, size_t x_len, size_t b, int lane, float v[8]) {
  const size_t i0 = b * 256 + size_t(lane) * 8;
  if (i0 + 8 <= x_len && ((reinterpret_cast<uintptr_t>(x + i0) & 15) == 0)) {
    const float4 a = *reinterpret_cast<const float4 *>(x + i0);
    const float4 c = *reinterpret_cast<const float4 *>(x + i0 + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    v[4] = c.x; v[5] = c.y; v[6] = c.z; v[7] = c.w;
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = (i0 + j < x_len) ? x[i0 + j] : 0.0f;
  }
}

// 256-point Walsh-Hadamard transform scaled by 1/16 across one warp, lane l holding elements
// 8l..8l+7.  Butterfly stages run in the reference's order h = 1,2,...,128
// (transform_simd.cpp:14-23,57-64) with the same operand pairing, so the result is
// bit-identical to the reference's generic branch; strides 1,2,4 stay inside the lane,
// strides 8..128 cross lanes by shuffle.
__device__ __forceinline__ void fwht256_warp(float v[8], int lane) {
#pragma unroll
  for (int h = 1; h < 8; h <<= 1) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if ((j & h) == 0) {
        const float a = v[j], b = v[j + h];
        v[j] = a + b;
        v[j + h] = a - b;
      }
    }
  }
#pragma unroll
  for (int m = 1; m < 32; m <<= 1) {
    const float sgn = (lane & m) ? -1.0f : 1.0f;  // upper half of a butterfly: other - own (exact as an FMA by +-1)
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float o = __shfl_xor_sync(0xffffffffu, v[j], m);
      v[j] = fmaf(v[j], sgn, o);
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) v[j] *= 0.0625f;
}

// The 16 subset sums of 4 activations with the reference's index convention (entry bit 3
// selects a0 ... bit 0 selects a3) and its left-to-right order of additions
// (lut_gemm.hpp:30-44), written as four float4 to `t` (16 floats, 16-byte aligned).
__device__ __forceinline__ void lut16_store(float a0, float a1, float a2, float a3, float *t) {
  const float t12 = a0 + a1;
  const float t10 = a0 + a2, t6 = a1 + a2, t14 = t12 + a2;
  float4 *o = reinterpret_cast<float4 *>(t);
  o[0] = make_float4(0.0f, a3, a2, a2 + a3);
  o[1] = make_float4(a1, a1 + a3, t6, t6 + a3);
  o[2] = make_float4(a0, a0 + a3, t10, t10 + a3);
  o[3] = make_float4(t12, t12 + a3, t14, t14 + a3);
}

// Prologue for one 256-block: load (zero padded), optionally rotate, build the 64 group
// tables into tab[64][16] and the block total into *xsum.  One warp per block.
__device__ __forceinline__ void build_block_tables(const float *__restrict__ x, size_t x_len, size_t b, bool rotate,
                                                   int lane, float *tab, float *xsum) {
  float v[8];
  load_x8(x, x_len, b, lane, v);
  if (rotate) fwht256_warp(v, lane);
  lut16_store(v[0], v[1], v[2], v[3], tab + (2 * lane) * 16);
  lut16_store(v[4], v[5], v[6], v[7], tab + (2 * lane + 1) * 16);
  float s = (((v[0] + v[1]) + v[2]) + v[3]) + (((v[4] + v[5]) + v[6]) + v[7]);
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) s += __shfl_xor_sync(0xffffffffu, s, m);
  if (lane == 0) *xsum = s;
}


// Launch timeline (debugging): word 0 first CTA start, 1 / 2 first / last CTA past the wait for the
// preceding kernel, 3 last CTA with its activations ready, 4 last CTA through its main loop,
// 5 / 6 last / first CTA done.  Called by one thread per CTA; dbg null: off.
__device__ __forceinline__ unsigned long long tl_now() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void tl_min(unsigned long long *dbg, int w) {
  if (dbg) atomicMin(dbg + w, tl_now());
}
__device__ __forceinline__ void tl_max(unsigned long long *dbg, int w) {
  if (dbg) atomicMax(dbg + w, tl_now());
}


// Range-checking build (-DLMB_DEBUG_BOUNDS, liblutmac_b200_dbg.so): LMB_IN_BOUNDS(cond, code, value)
// is `cond`, and a false one records the first violation of this translation unit -- code, value,
// block and thread -- instead of letting the access run: the caller skips it, nothing traps.  In
// the ordinary build the macro is `true` and the checks cost nothing.
enum BoundsCode : unsigned { BOUNDS_WEIGHT_TILE = 1, BOUNDS_OUTPUT = 2, BOUNDS_SCRATCH = 3, BOUNDS_KV_SLICE = 4, BOUNDS_PREP = 5 };
#ifdef LMB_DEBUG_BOUNDS
namespace {
__device__ unsigned long long tu_bounds[4];  // {code (0: clean), value, block | thread << 32, count}
}
__device__ __forceinline__ bool bounds_ok(bool ok, unsigned code, unsigned long long value) {
  if (!ok) {
    if (atomicCAS(&tu_bounds[0], 0ull, static_cast<unsigned long long>(code)) == 0ull) {
      tu_bounds[1] = value;
      tu_bounds[2] = static_cast<unsigned long long>(blockIdx.x) | (static_cast<unsigned long long>(threadIdx.x) << 32);
    }
    atomicAdd(&tu_bounds[3], 1ull);
  }
  return ok;
}
#define LMB_IN_BOUNDS(cond, code, value) (::lmb::bounds_ok((cond), (code), static_cast<unsigned long long>(value)))
#else
#define LMB_IN_BOUNDS(cond, code, value) (true)
#endif

}  // namespace lmb

#ifdef LMB_DEBUG_BOUNDS
// every translation unit with checked kernels registers a reader of its record (see api.cu)
namespace lmb {
using BoundsReader = int (*)(unsigned long long out[4], bool clear);
void register_bounds_reader(BoundsReader fn);
namespace {
inline int read_tu_bounds(unsigned long long out[4], bool clear) {
  cudaError_t e = cudaMemcpyFromSymbol(out, tu_bounds, 4 * sizeof(unsigned long long));
  if (e == cudaSuccess && clear) {
    const unsigned long long zero[4] = {0, 0, 0, 0};
    e = cudaMemcpyToSymbol(tu_bounds, zero, sizeof(zero));
  }
  return int(e);
}
const struct BoundsRegistrar {
  BoundsRegistrar() { register_bounds_reader(&read_tu_bounds); }
} bounds_registrar;
}  // namespace
}  // namespace lmb
#endif
