// The per-kind evaluation units of the GEMV kernels: what a warp lane loads of one (row-tile,
// 256-column block) and how it is multiplied with the prepared activations.  Shared by the
// one-GEMV-per-launch kernel (gemv.cu) and the persistent decode-step kernel (persist.cu).
//   * integer tensor-core units (default for every kind): the weight tile is stored in the
//     operand order of the 8-bit integer MMA with several rows sharing the bits of a byte, so an
//     `and` with a mask yields an operand register; the activations of a 256-block become 32-bit
//     fixed point with one exponent, cut into four signed base-256 digits (the B operand);
//     sums are exact integers, the code's zero point is removed with the digit sums;
//   * table-lookup units (the reference's own formulation, selectable): ternary L[pos]-L[neg]
//     (lut_gemm_simd.cpp:203-221), n-bit planes sum_p 2^p L[idx_p] - zero_point*L[15]
//     (lut_gemm_simd.cpp:352-366), RRQ primary*scale + residual*scale2 (lut_gemm_simd.cpp:
//     326-328), with 16-entry group tables in shared memory; 8-bit as dequantise + FMA.
#pragma once

#include "common.cuh"
#include "device_utils.cuh"

namespace lmb {

namespace {

__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Thread-block clusters: the shared memory of the other CTAs of the cluster (distributed shared memory).
__device__ __forceinline__ uint32_t smem_addr(const void *p) { return uint32_t(__cvta_generic_to_shared(p)); }
// address of the same shared-memory location in the CTA of rank `rank` of this cluster
__device__ __forceinline__ uint32_t cluster_addr(const void *p, unsigned rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr(p)), "r"(rank));
  return r;
}
__device__ __forceinline__ void st_cluster_v4(uint32_t addr, uint4 v) {
  asm volatile("st.shared::cluster.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void st_cluster_f32(uint32_t addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ float ld_cluster_f32(uint32_t addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
  return v;
}
// all threads of all CTAs of the cluster; writes before it (own and remote shared memory) are visible after it
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

template <int IMM> __device__ __forceinline__ float lds_f32(uint32_t addr) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1+%2];" : "=f"(v) : "r"(addr), "n"(IMM) : "memory");
  return v;
}
// (a & b) | c in one LOP3
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
  return r;
}

// ---------------------------------------------------------------------------------------------
// Bit-plane kinds: table lookups
// ---------------------------------------------------------------------------------------------

// Sum of the 8 lookups addressed by the 8 nibbles of `w` (4 plane bytes, little endian; byte k
// holds group 2k in its high nibble and group 2k+1 in its low nibble) into 8 consecutive group
// tables; `tb` is the shared-memory byte address of the block's tables (1 KiB aligned) and G0
// the first group.  Index extraction is one shift and one LOP3 that masks the nibble (already
// scaled by 4) and ORs in the table base; the group offset rides in the load's immediate.
template <int G0> __device__ __forceinline__ float lut_word(uint32_t w, uint32_t tb) {
  float s0, s1;
  s0 = lds_f32<(G0 + 0) * 64>(and_or(w >> 2, 0x3Cu, tb));
  s1 = lds_f32<(G0 + 1) * 64>(and_or(w << 2, 0x3Cu, tb));
  s0 += lds_f32<(G0 + 2) * 64>(and_or(w >> 10, 0x3Cu, tb));
  s1 += lds_f32<(G0 + 3) * 64>(and_or(w >> 6, 0x3Cu, tb));
  s0 += lds_f32<(G0 + 4) * 64>(and_or(w >> 18, 0x3Cu, tb));
  s1 += lds_f32<(G0 + 5) * 64>(and_or(w >> 14, 0x3Cu, tb));
  s0 += lds_f32<(G0 + 6) * 64>(and_or(w >> 26, 0x3Cu, tb));
  s1 += lds_f32<(G0 + 7) * 64>(and_or(w >> 22, 0x3Cu, tb));
  return s0 + s1;
}
template <int G0> __device__ __forceinline__ float lut_8bytes(uint32_t lo, uint32_t hi, uint32_t tb) {
  return lut_word<G0>(lo, tb) + lut_word<G0 + 8>(hi, tb);
}
template <int G0> __device__ __forceinline__ float lut_16bytes(const uint4 v, uint32_t tb) {
  return (lut_word<G0>(v.x, tb) + lut_word<G0 + 8>(v.y, tb)) + (lut_word<G0 + 16>(v.z, tb) + lut_word<G0 + 24>(v.w, tb));
}

template <int KIND> struct Unit;  // one (row-tile, 256-column block): a lane's payload + scales

template <int KIND> struct LutUnit {
  static constexpr int C = kind_info(KIND).chunks;
  static constexpr int NS = kind_info(KIND).nscales;
  static constexpr int FPB = 1024;  // shared-memory floats per 256-column block: 64 tables x 16
  uint4 v[C];
  float sc[NS];

  __device__ __forceinline__ void load(const uint8_t *tile, int lane) {
#pragma unroll
    for (int c = 0; c < C; ++c) v[c] = ld_stream_v4(tile + (size_t(c) * TILE_ROWS + lane) * 16);
#pragma unroll
    for (int s = 0; s < NS; ++s) sc[s] = ld_stream_f32(tile + size_t(C) * TILE_ROWS * 16 + (size_t(s) * TILE_ROWS + lane) * 4);
  }

  using Acc = float;  // one row per lane
  static __device__ __forceinline__ void acc_init(Acc &a) { a = 0.0f; }
  static __device__ __forceinline__ float acc_row(const Acc &a, int) { return a; }
  __device__ __forceinline__ void eval(const float *blk, float xsum, const int *, Acc &acc) const {
    acc += value(blk, xsum);
  }

  // scale * sum_i w_i x_i of this row-block
  __device__ __forceinline__ float value(const float *blk, float xsum) const {
    const uint32_t tb = smem_u32(blk);
    if constexpr (KIND == LMB_TERNARY) {
      const float p = (lut_8bytes<0>(v[0].x, v[0].y, tb) + lut_8bytes<16>(v[1].x, v[1].y, tb)) +
                      (lut_8bytes<32>(v[2].x, v[2].y, tb) + lut_8bytes<48>(v[3].x, v[3].y, tb));
      const float n = (lut_8bytes<0>(v[0].z, v[0].w, tb) + lut_8bytes<16>(v[1].z, v[1].w, tb)) +
                      (lut_8bytes<32>(v[2].z, v[2].w, tb) + lut_8bytes<48>(v[3].z, v[3].w, tb));
      return (p - n) * sc[0];
    } else if constexpr (KIND == LMB_BINARY) {
      const float a = lut_16bytes<0>(v[0], tb) + lut_16bytes<32>(v[1], tb);
      return (2.0f * a - xsum) * sc[0];
    } else if constexpr (KIND == LMB_INT2) {
      const float a1 = (lut_8bytes<0>(v[0].x, v[0].y, tb) + lut_8bytes<16>(v[1].x, v[1].y, tb)) +
                       (lut_8bytes<32>(v[2].x, v[2].y, tb) + lut_8bytes<48>(v[3].x, v[3].y, tb));
      const float a2 = (lut_8bytes<0>(v[0].z, v[0].w, tb) + lut_8bytes<16>(v[1].z, v[1].w, tb)) +
                       (lut_8bytes<32>(v[2].z, v[2].w, tb) + lut_8bytes<48>(v[3].z, v[3].w, tb));
      return (2.0f * a1 - xsum) * sc[0] + (2.0f * a2 - xsum) * sc[1];
    } else {  // LMB_INT3: chunk 3j+p holds plane 2-p of weights 128j..128j+127
      const float q2 = lut_16bytes<0>(v[0], tb) + lut_16bytes<32>(v[3], tb);
      const float q1 = lut_16bytes<0>(v[1], tb) + lut_16bytes<32>(v[4], tb);
      const float q0 = lut_16bytes<0>(v[2], tb) + lut_16bytes<32>(v[5], tb);
      return ((4.0f * q2 + 2.0f * q1 + q0) - 4.0f * xsum) * sc[0];
    }
  }

  // Prologue for one 256-block by one warp: load (zero padded), optionally rotate, stage the
  // 256 values in the block's table area, then build the 64 tables with one (group,
  // quarter-table) pair per lane and pass, so that the 128-bit table stores are contiguous
  // across the warp (no bank conflicts).  Addition order per entry is the reference's
  // (a0, a1, a2, a3 left to right, lut_gemm.hpp:30-44).
  static __device__ __forceinline__ void prologue(const float (&v)[8], int lane, float *blk, float *xsum, int *) {
    float s = (((v[0] + v[1]) + v[2]) + v[3]) + (((v[4] + v[5]) + v[6]) + v[7]);
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) s += __shfl_xor_sync(0xffffffffu, s, m);
    if (lane == 0) *xsum = s;
    float *stage = blk + 768;  // read back in full before any table is stored
    reinterpret_cast<float4 *>(stage)[2 * lane] = make_float4(v[0], v[1], v[2], v[3]);
    reinterpret_cast<float4 *>(stage)[2 * lane + 1] = make_float4(v[4], v[5], v[6], v[7]);
    __syncwarp();
    const int q = lane & 3;
    float4 a[8];
#pragma unroll
    for (int pass = 0; pass < 8; ++pass) a[pass] = reinterpret_cast<const float4 *>(stage)[pass * 8 + (lane >> 2)];
    __syncwarp();
#pragma unroll
    for (int pass = 0; pass < 8; ++pass) {
      const int g = pass * 8 + (lane >> 2);
      const float a0 = a[pass].x, a1 = a[pass].y, a2 = a[pass].z, a3 = a[pass].w;
      const float base = (q == 0) ? 0.0f : (q == 1) ? a1 : (q == 2) ? a0 : (a0 + a1);
      const float e2 = base + a2;
      reinterpret_cast<float4 *>(blk + g * 16)[q] = make_float4(base, base + a3, e2, e2 + a3);
    }
  }
};

template <> struct Unit<LMB_TERNARY> : LutUnit<LMB_TERNARY> {};
template <> struct Unit<LMB_BINARY> : LutUnit<LMB_BINARY> {};
template <> struct Unit<LMB_INT2> : LutUnit<LMB_INT2> {};
template <> struct Unit<LMB_INT3> : LutUnit<LMB_INT3> {};

// ---------------------------------------------------------------------------------------------
// Nibble / byte kinds: dequantise + FMA.  Codes become fp32 without integer-to-float
// conversions: a nibble (or byte) is OR-ed into the mantissa of 2^23 and one exact subtraction
// removes 2^23 together with the code's zero point (8 for 4-bit; 128 after the sign flip for
// 8-bit).  A nibble that sits p bits up in its word is not shifted down: it yields (q-8)*2^p,
// is accumulated in a slot of its own, and the slot is rescaled by 2^-p once per row-block
// (both scalings are exact).  Subtract and multiply-add run as packed fp32 pairs.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float as_f(uint32_t u) { return __uint_as_float(u); }
constexpr uint32_t MAGIC = 0x4B000000u;  // 2^23

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

// Shared prologue of the dequantise kinds: the (padded, optionally rotated) block itself.
__device__ __forceinline__ void dq_prologue(const float (&v)[8], int lane, float *blk) {
  reinterpret_cast<float4 *>(blk)[2 * lane] = make_float4(v[0], v[1], v[2], v[3]);
  reinterpret_cast<float4 *>(blk)[2 * lane + 1] = make_float4(v[4], v[5], v[6], v[7]);
}

// ---------------------------------------------------------------------------------------------
// Integer tensor-core path.  A dequantise+FMA form of the 4-bit kernel cost about four
// issue slots per weight and is bound by instruction issue at 0.3 of HBM bandwidth (ncu), so
// the 4-bit codes are fed to the 8-bit integer MMA as they are (two masks per 8 codes) and the
// activations are turned, once per 256-block, into 32-bit fixed point with a shared exponent,
// split into four signed base-256 digits (the MMA's 8 output columns hold the digits).  All
// products and sums are exact integers; the only rounding is the fixed-point conversion of x
// (absolute error <= 2^-31 of the block's largest |x|) and two int->float conversions per row
// and block.  The zero point 8 is removed in integers with the per-block digit sums.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void mma_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void mma_s8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void mma_prologue(const float (&v)[8], int lane, float *blk, float *bscale, int *aux2);

// Where a warp finds the prepared activations of its sequences (see the kernel's prologue).
struct MmaX {
  const float *dig;  // digits of block 0 of the first sequence, [seq][block][FPB]
  const float *bs;   // block scales, [seq][64]
  const int *aux;    // digit-pair sums, [pair][64][4] = {seq 2p: d01, d23; seq 2p+1: d01, d23}
  int seq_stride;    // floats between the digits of consecutive sequences
};

// Shared by the integer-MMA units.  The activations of a block are 32-bit fixed point with one
// exponent per block, cut into four signed base-256 digits.  The B operand of one MMA carries
// the digits of two sequences: columns 0..3 the first, columns 4..7 the second (with a single
// sequence they repeat the first and their results are ignored).  Several rows share one weight
// word: row g + 8m sits in a bit-field of every byte, so `word & mask` IS the A operand of that
// row, scaled by 2^(field offset); the power of two is folded into the row's scale.
// Accumulators are exact integers; the zero point is removed with the digit sums.
struct MmaAcc { float r[4]; };  // rows g, g+8, g+16, g+24; lanes tid 0,1: first sequence (digits 0,1 / 2,3), tid 2,3: second
__device__ __forceinline__ void mma_acc_init(MmaAcc &a) { a.r[0] = a.r[1] = a.r[2] = a.r[3] = 0.0f; }
// value of row `lane` of the tile for the first (half = 0) or second sequence of the pair
__device__ __forceinline__ float mma_acc_row(const MmaAcc &a, int lane, int half = 0) {
  const int src = 4 * (lane & 7) + 2 * half;
  float r[4];
#pragma unroll
  for (int k = 0; k < 4; ++k)
    r[k] = __shfl_sync(0xffffffffu, a.r[k], src) + 65536.0f * __shfl_sync(0xffffffffu, a.r[k], src + 1);
  const int k = lane >> 3;
  return k == 0 ? r[0] : (k == 1 ? r[1] : (k == 2 ? r[2] : r[3]));
}
// c0,c1: digit pair of a row; dz = zero point * digit-pair sum, already shifted to the row's field
__device__ __forceinline__ float mma_row_value(int c0, int c1, uint32_t dz) {
  return float(int(uint32_t(c0) + 256u * uint32_t(c1) - dz));
}
// the same for a +-1 bit plane: sum((2b-1) x) = 2 sum(b x) - sum(x); modular arithmetic, the result fits
__device__ __forceinline__ float mma_plane_value(uint32_t c0, uint32_t c1, uint32_t dz) {
  return float(int(2u * c0 + 512u * c1 - dz));
}
__device__ __forceinline__ float4 as_float4(uint4 u) {
  return make_float4(__uint_as_float(u.x), __uint_as_float(u.y), __uint_as_float(u.z), __uint_as_float(u.w));
}

// Common frame of the MMA units: Derived supplies the payload, `mma_block` (all MMAs of one
// row-tile-block for PG sequence pairs) and `finish` (integer sums -> scaled floats).
template <class Derived, int PG_> struct MmaUnitBase {
  static constexpr int FPB = 256;  // 1 KiB per block and sequence: 256 activations x 4 digit bytes, in B-operand order
  static constexpr int PG = PG_;   // sequence pairs evaluated per pass over the A operands
  using Acc = MmaAcc;
  static __device__ __forceinline__ void acc_init(Acc &a) { mma_acc_init(a); }
  static __device__ __forceinline__ float acc_row(const Acc &a, int lane, int half = 0) { return mma_acc_row(a, lane, half); }
  // One warp per 256-block and sequence: convert to fixed point with the block's exponent, split
  // into signed base-256 digits and store them in B-operand order; *bscale = 2^(E-30),
  // aux2[0..1] = sums over the block of digit 0 + 256 digit 1 and digit 2 + 256 digit 3.
  static __device__ __forceinline__ void prologue(const float (&v)[8], int lane, float *blk, float *bscale, int *aux2) {
    mma_prologue(v, lane, blk, bscale, aux2);
  }
  // MULTI: more than one sequence (the second half of every B operand is a real sequence)
  template <int NP, bool MULTI> __device__ __forceinline__ void eval(const MmaX &xo, int bl, Acc (&acc)[NP]) const {
    const int lane = threadIdx.x & 31, g = lane >> 2, tid = lane & 3;
    const uint4 *dig = reinterpret_cast<const uint4 *>(xo.dig + size_t(bl) * FPB + (MULTI ? size_t(g >> 2) * xo.seq_stride : 0)) +
                       ((g & 3) * 4 + tid);
    const int ps = MULTI ? xo.seq_stride >> 1 : 0;  // uint4 between consecutive pairs
    constexpr int STEP = NP < PG ? NP : PG;
#pragma unroll
    for (int p0 = 0; p0 < NP; p0 += STEP) {
      typename Derived::template Sums<STEP> c;
      static_cast<const Derived *>(this)->template mma_block<STEP>(dig + size_t(p0) * ps, ps, c);
#pragma unroll
      for (int p = 0; p < STEP; ++p) {
        const uint32_t d = uint32_t(xo.aux[((p0 + p) * 64 + bl) * 4 + tid]);
        const float bs = MULTI ? xo.bs[(2 * (p0 + p) + (tid >> 1)) * 64 + bl] : xo.bs[bl];
        static_cast<const Derived *>(this)->finish(c, p, d, bs, acc[p0 + p]);
      }
    }
  }
};

template <> struct Unit<LMB_INT4> : MmaUnitBase<Unit<LMB_INT4>, 4> {
  uint4 v[8];
  float4 sc;  // scales of rows g, g+8, g+16, g+24
  template <int N> struct Sums { int c[N][2][4]; };
  __device__ __forceinline__ void load(const uint8_t *tile, int lane) {
#pragma unroll
    for (int c = 0; c < 8; ++c) v[c] = ld_stream_v4(tile + (size_t(c) * TILE_ROWS + lane) * 16);
    sc = as_float4(ld_stream_v4(tile + size_t(8) * TILE_ROWS * 16 + size_t(lane >> 2) * 16));
  }
  template <int N> __device__ __forceinline__ void mma_block(const uint4 *dig, int ps, Sums<N> &s) const {
    constexpr uint32_t LO = 0x0F0F0F0Fu, HI = 0xF0F0F0F0u;
#pragma unroll
    for (int p = 0; p < N; ++p)
#pragma unroll
      for (int h = 0; h < 2; ++h) s.c[p][h][0] = s.c[p][h][1] = s.c[p][h][2] = s.c[p][h][3] = 0;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      uint4 b[N];  // {k-step 2q: b0, b1; k-step 2q+1: b0, b1}
#pragma unroll
      for (int p = 0; p < N; ++p) b[p] = dig[q * 16 + p * ps];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const uint4 w = v[h * 4 + q];  // rows 16h+g (low nibbles) and 16h+g+8 (high nibbles)
        const uint32_t a0 = w.x & LO, a1 = w.x & HI, a2 = w.y & LO, a3 = w.y & HI;
        const uint32_t e0 = w.z & LO, e1 = w.z & HI, e2 = w.w & LO, e3 = w.w & HI;
#pragma unroll
        for (int p = 0; p < N; ++p) {
          mma_u8s8(s.c[p][h], a0, a1, a2, a3, b[p].x, b[p].y);
          mma_u8s8(s.c[p][h], e0, e1, e2, e3, b[p].z, b[p].w);
        }
      }
    }
  }
  template <int N> __device__ __forceinline__ void finish(const Sums<N> &s, int p, uint32_t d, float bs, Acc &acc) const {
    const uint32_t d8 = 8u * d;  // zero point 8
    const float b16 = bs * 0.0625f;
    acc.r[0] += mma_row_value(s.c[p][0][0], s.c[p][0][1], d8) * (bs * sc.x);
    acc.r[1] += mma_row_value(s.c[p][0][2], s.c[p][0][3], d8 << 4) * (b16 * sc.y);
    acc.r[2] += mma_row_value(s.c[p][1][0], s.c[p][1][1], d8) * (bs * sc.z);
    acc.r[3] += mma_row_value(s.c[p][1][2], s.c[p][1][3], d8 << 4) * (b16 * sc.w);
  }
};

// (definition of the shared MMA prologue)
__device__ __forceinline__ void mma_prologue(const float (&v)[8], int lane, float *blk, float *bscale, int *aux2) {
  float amax = 0.0f;
#pragma unroll
  for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
  // non-negative floats order like their bit patterns
  const uint32_t am = __reduce_max_sync(0xffffffffu, __float_as_uint(amax));
  int e = int((am >> 23) & 0xFFu) - 126;  // amax < 2^e
  e = max(e, -90);                        // keeps 2^(30-e) finite for vanishing blocks
  const float inv = __uint_as_float(uint32_t(127 + 30 - e) << 23);
  // q = round(v * 2^(30-e)), |q| <= 2^30.  Adding 0x808080 and flipping the same bits turns the
  // four bytes of q into its signed base-256 digits (the top byte is the signed top digit).
  uint32_t w[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) w[j] = (uint32_t(__float2int_rn(v[j] * inv)) + 0x00808080u) ^ 0x00808080u;
  // 4x4 byte transposes: words[d][h] = digit d of elements 4h..4h+3
  uint32_t words[4][2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const uint32_t t0 = __byte_perm(w[4 * h], w[4 * h + 1], 0x5140), t1 = __byte_perm(w[4 * h + 2], w[4 * h + 3], 0x5140);
    const uint32_t t2 = __byte_perm(w[4 * h], w[4 * h + 1], 0x7362), t3 = __byte_perm(w[4 * h + 2], w[4 * h + 3], 0x7362);
    words[0][h] = __byte_perm(t0, t1, 0x5410);
    words[1][h] = __byte_perm(t0, t1, 0x7632);
    words[2][h] = __byte_perm(t2, t3, 0x5410);
    words[3][h] = __byte_perm(t2, t3, 0x7632);
  }
  // element j of lane l is column 8l+j: k-step s = l/4, position kk = 8(l%4)+j inside it
  const int s = lane >> 2, reg = (lane & 3) >> 1, tidb = 2 * (lane & 1);
  uint32_t *dst = reinterpret_cast<uint32_t *>(blk) + ((s >> 1) * 16 + tidb) * 4 + (s & 1) * 2 + reg;
#pragma unroll
  for (int d = 0; d < 4; ++d) {
    dst[d * 16] = words[d][0];
    dst[d * 16 + 4] = words[d][1];
  }
  int ds[4];
#pragma unroll
  for (int d = 0; d < 4; ++d) ds[d] = __dp4a(int(words[d][0]), 0x01010101, __dp4a(int(words[d][1]), 0x01010101, 0));
  const int d01 = __reduce_add_sync(0xffffffffu, ds[0] + 256 * ds[1]);
  const int d23 = __reduce_add_sync(0xffffffffu, ds[2] + 256 * ds[3]);
  if (lane == 0) {
    *bscale = (am != 0u) ? __uint_as_float(uint32_t(127 + e - 30) << 23) : 0.0f;
    aux2[0] = d01;
    aux2[1] = d23;
  }
}

// Ternary weights as 2-bit codes t+1 on the same integer MMA path (zero point 1): the four
// 2-bit fields of a byte belong to rows g, g+8, g+16, g+24 of the tile.
template <> struct Unit<DK_TERNARY_MMA> : MmaUnitBase<Unit<DK_TERNARY_MMA>, 4> {
  uint4 v[4];
  float4 sc;
  template <int N> struct Sums { int c[N][2][4]; };
  __device__ __forceinline__ void load(const uint8_t *tile, int lane) {
#pragma unroll
    for (int c = 0; c < 4; ++c) v[c] = ld_stream_v4(tile + (size_t(c) * TILE_ROWS + lane) * 16);
    sc = as_float4(ld_stream_v4(tile + size_t(4) * TILE_ROWS * 16 + size_t(lane >> 2) * 16));
  }
  template <int N> __device__ __forceinline__ void mma_block(const uint4 *dig, int ps, Sums<N> &s) const {
    constexpr uint32_t F0 = 0x03030303u, F1 = 0x0C0C0C0Cu, F2 = 0x30303030u, F3 = 0xC0C0C0C0u;
#pragma unroll
    for (int p = 0; p < N; ++p)
#pragma unroll
      for (int h = 0; h < 2; ++h) s.c[p][h][0] = s.c[p][h][1] = s.c[p][h][2] = s.c[p][h][3] = 0;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const uint4 w = v[q];  // {k-step 2q: columns +0..15, +16..31; k-step 2q+1: the same}
#pragma unroll
      for (int p = 0; p < N; ++p) {
        const uint4 b = dig[q * 16 + p * ps];
        mma_u8s8(s.c[p][0], w.x & F0, w.x & F1, w.y & F0, w.y & F1, b.x, b.y);
        mma_u8s8(s.c[p][1], w.x & F2, w.x & F3, w.y & F2, w.y & F3, b.x, b.y);
        mma_u8s8(s.c[p][0], w.z & F0, w.z & F1, w.w & F0, w.w & F1, b.z, b.w);
        mma_u8s8(s.c[p][1], w.z & F2, w.z & F3, w.w & F2, w.w & F3, b.z, b.w);
      }
    }
  }
  template <int N> __device__ __forceinline__ void finish(const Sums<N> &s, int p, uint32_t d1, float bs, Acc &acc) const {
    acc.r[0] += mma_row_value(s.c[p][0][0], s.c[p][0][1], d1) * (bs * sc.x);  // zero point 1
    acc.r[1] += mma_row_value(s.c[p][0][2], s.c[p][0][3], d1 << 2) * ((bs * 0.25f) * sc.y);
    acc.r[2] += mma_row_value(s.c[p][1][0], s.c[p][1][1], d1 << 4) * ((bs * 0.0625f) * sc.z);
    acc.r[3] += mma_row_value(s.c[p][1][2], s.c[p][1][3], d1 << 6) * ((bs * 0.015625f) * sc.w);
  }
};

// INT2 (residual binary, w = +-s1 +- s2) as two +-1 bit planes on the integer MMA path: the
// ternary arrangement with bit 2m = b1 and bit 2m+1 = b2 of row g+8m; one accumulator per plane.
template <> struct Unit<DK_INT2_MMA> : MmaUnitBase<Unit<DK_INT2_MMA>, 2> {
  uint4 v[4];
  float4 sc[2];
  template <int N> struct Sums { int c[N][2][2][4]; };  // [pair][row half][plane]
  __device__ __forceinline__ void load(const uint8_t *tile, int lane) {
#pragma unroll
    for (int c = 0; c < 4; ++c) v[c] = ld_stream_v4(tile + (size_t(c) * TILE_ROWS + lane) * 16);
#pragma unroll
    for (int p = 0; p < 2; ++p)
      sc[p] = as_float4(ld_stream_v4(tile + size_t(4) * TILE_ROWS * 16 + size_t(p) * TILE_ROWS * 4 + size_t(lane >> 2) * 16));
  }
  template <int N> __device__ __forceinline__ void mma_block(const uint4 *dig, int ps, Sums<N> &s) const {
    constexpr uint32_t M1 = 0x01010101u;
#pragma unroll
    for (int p = 0; p < N; ++p)
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int pl = 0; pl < 2; ++pl) s.c[p][h][pl][0] = s.c[p][h][pl][1] = s.c[p][h][pl][2] = s.c[p][h][pl][3] = 0;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const uint4 w = v[q];
      uint4 b[N];
#pragma unroll
      for (int p = 0; p < N; ++p) b[p] = dig[q * 16 + p * ps];
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int pl = 0; pl < 2; ++pl) {
          const int sh = 4 * h + pl;  // rows g+16h (bit 4h+pl) and g+16h+8 (bit 4h+2+pl)
          const uint32_t a0 = w.x & (M1 << sh), a1 = w.x & (M1 << (sh + 2)), a2 = w.y & (M1 << sh), a3 = w.y & (M1 << (sh + 2));
          const uint32_t e0 = w.z & (M1 << sh), e1 = w.z & (M1 << (sh + 2)), e2 = w.w & (M1 << sh), e3 = w.w & (M1 << (sh + 2));
#pragma unroll
          for (int p = 0; p < N; ++p) {
            mma_u8s8(s.c[p][h][pl], a0, a1, a2, a3, b[p].x, b[p].y);
            mma_u8s8(s.c[p][h][pl], e0, e1, e2, e3, b[p].z, b[p].w);
          }
        }
    }
  }
  template <int N> __device__ __forceinline__ void finish(const Sums<N> &s, int p, uint32_t d, float bs, Acc &acc) const {
    const float s1[4] = {sc[0].x, sc[0].y, sc[0].z, sc[0].w}, s2[4] = {sc[1].x, sc[1].y, sc[1].z, sc[1].w};
#pragma unroll
    for (int m = 0; m < 4; ++m) {
      const int h = m >> 1, j = m & 1;
      const float f1 = bs * (1.0f / float(1 << (2 * m))), f2 = bs * (1.0f / float(2 << (2 * m)));
      float t = mma_plane_value(uint32_t(s.c[p][h][0][2 * j]), uint32_t(s.c[p][h][0][2 * j + 1]), d << (2 * m)) * (f1 * s1[m]);
      t = fmaf(mma_plane_value(uint32_t(s.c[p][h][1][2 * j]), uint32_t(s.c[p][h][1][2 * j + 1]), d << (2 * m + 1)), f2 * s2[m], t);
      acc.r[m] += t;
    }
  }
};

// BINARY (w = +-s) as one +-1 bit plane: bit m + 4kh of a byte is row g+8m of the first (kh = 0)
// or second (kh = 1) k-step of the word's pair; one accumulator per kh, merged by an exact shift.
template <> struct Unit<DK_BINARY_MMA> : MmaUnitBase<Unit<DK_BINARY_MMA>, 2> {
  uint4 v[2];
  float4 sc;
  template <int N> struct Sums { int c[N][2][2][4]; };  // [pair][row half][kh]
  __device__ __forceinline__ void load(const uint8_t *tile, int lane) {
#pragma unroll
    for (int c = 0; c < 2; ++c) v[c] = ld_stream_v4(tile + (size_t(c) * TILE_ROWS + lane) * 16);
    sc = as_float4(ld_stream_v4(tile + size_t(2) * TILE_ROWS * 16 + size_t(lane >> 2) * 16));
  }
  template <int N> __device__ __forceinline__ void mma_block(const uint4 *dig, int ps, Sums<N> &s) const {
    constexpr uint32_t M1 = 0x01010101u;
#pragma unroll
    for (int p = 0; p < N; ++p)
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int kh = 0; kh < 2; ++kh) s.c[p][h][kh][0] = s.c[p][h][kh][1] = s.c[p][h][kh][2] = s.c[p][h][kh][3] = 0;
    const uint32_t wa[4] = {v[0].x, v[0].z, v[1].x, v[1].z}, wb[4] = {v[0].y, v[0].w, v[1].y, v[1].w};
#pragma unroll
    for (int sp = 0; sp < 4; ++sp) {
      uint4 b[N];  // {k-step 2sp: b0, b1; k-step 2sp+1: b0, b1}
#pragma unroll
      for (int p = 0; p < N; ++p) b[p] = dig[sp * 16 + p * ps];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int s0 = 2 * h, s1 = 2 * h + 4;
        const uint32_t a0 = wa[sp] & (M1 << s0), a1 = wa[sp] & (M1 << (s0 + 1)), a2 = wb[sp] & (M1 << s0), a3 = wb[sp] & (M1 << (s0 + 1));
        const uint32_t e0 = wa[sp] & (M1 << s1), e1 = wa[sp] & (M1 << (s1 + 1)), e2 = wb[sp] & (M1 << s1), e3 = wb[sp] & (M1 << (s1 + 1));
#pragma unroll
        for (int p = 0; p < N; ++p) {
          mma_u8s8(s.c[p][h][0], a0, a1, a2, a3, b[p].x, b[p].y);
          mma_u8s8(s.c[p][h][1], e0, e1, e2, e3, b[p].z, b[p].w);
        }
      }
    }
  }
  template <int N> __device__ __forceinline__ void finish(const Sums<N> &s, int p, uint32_t d, float bs, Acc &acc) const {
    const float sv[4] = {sc.x, sc.y, sc.z, sc.w};
#pragma unroll
    for (int m = 0; m < 4; ++m) {
      const int h = m >> 1, j = m & 1;
      // the kh = 1 sums carry 16 times the field's power of two: an exact shift brings them back
      const uint32_t c0 = uint32_t(s.c[p][h][0][2 * j] + (s.c[p][h][1][2 * j] >> 4));
      const uint32_t c1 = uint32_t(s.c[p][h][0][2 * j + 1] + (s.c[p][h][1][2 * j + 1] >> 4));
      acc.r[m] += mma_plane_value(c0, c1, d << m) * ((bs * (1.0f / float(1 << m))) * sv[m]);
    }
  }
};

// Codes made of bit planes on the DK_BINARY_MMA arrangement, optionally on top of low nibbles on
// the INT4 arrangement: 3-bit = planes 0..2; 5- and 6-bit = nibbles + planes 4 (and 5).  The
// partial sums are put back on a common scale by exact shifts and the zero point 2^(BITS-1) is
// removed with the digit sums.
template <int KIND, int BITS, bool NIB> struct PlanesUnit : MmaUnitBase<Unit<KIND>, 1> {
  static constexpr int NPL = NIB ? BITS - 4 : BITS;  // bit planes
  static constexpr int P0 = NIB ? 4 : 0;             // weight of the first plane: 2^P0
  static constexpr int NC = NIB ? 8 : 0;             // nibble chunks
  using Acc = MmaAcc;
  uint4 v[NC + 2 * NPL];
  float4 sc;
  template <int N> struct Sums {
    int n[N][2][4];            // nibbles, [row half]
    int pl[N][NPL][2][2][4];   // planes, [plane][row half][kh]
  };
  __device__ __forceinline__ void load(const uint8_t *tile, int lane) {
#pragma unroll
    for (int c = 0; c < NC + 2 * NPL; ++c) v[c] = ld_stream_v4(tile + (size_t(c) * TILE_ROWS + lane) * 16);
    sc = as_float4(ld_stream_v4(tile + size_t(NC + 2 * NPL) * TILE_ROWS * 16 + size_t(lane >> 2) * 16));
  }
  template <int N> __device__ __forceinline__ void mma_block(const uint4 *dig, int ps, Sums<N> &s) const {
    constexpr uint32_t LO = 0x0F0F0F0Fu, HI = 0xF0F0F0F0u, M1 = 0x01010101u;
#pragma unroll
    for (int p = 0; p < N; ++p)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        s.n[p][h][0] = s.n[p][h][1] = s.n[p][h][2] = s.n[p][h][3] = 0;
#pragma unroll
        for (int pl = 0; pl < NPL; ++pl)
#pragma unroll
          for (int kh = 0; kh < 2; ++kh) s.pl[p][pl][h][kh][0] = s.pl[p][pl][h][kh][1] = s.pl[p][pl][h][kh][2] = s.pl[p][pl][h][kh][3] = 0;
      }
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      uint4 b[N];  // {k-step 2q: b0, b1; k-step 2q+1: b0, b1}
#pragma unroll
      for (int p = 0; p < N; ++p) b[p] = dig[q * 16 + p * ps];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        if constexpr (NIB) {
          const uint4 w = v[h * 4 + q];
#pragma unroll
          for (int p = 0; p < N; ++p) {
            mma_u8s8(s.n[p][h], w.x & LO, w.x & HI, w.y & LO, w.y & HI, b[p].x, b[p].y);
            mma_u8s8(s.n[p][h], w.z & LO, w.z & HI, w.w & LO, w.w & HI, b[p].z, b[p].w);
          }
        }
#pragma unroll
        for (int pl = 0; pl < NPL; ++pl) {
          const uint4 pv = v[NC + 2 * pl + (q >> 1)];
          const uint32_t wa = (q & 1) ? pv.z : pv.x, wb = (q & 1) ? pv.w : pv.y;
          const int s0 = 2 * h, s1 = 2 * h + 4;
#pragma unroll
          for (int p = 0; p < N; ++p) {
            mma_u8s8(s.pl[p][pl][h][0], wa & (M1 << s0), wa & (M1 << (s0 + 1)), wb & (M1 << s0), wb & (M1 << (s0 + 1)), b[p].x, b[p].y);
            mma_u8s8(s.pl[p][pl][h][1], wa & (M1 << s1), wa & (M1 << (s1 + 1)), wb & (M1 << s1), wb & (M1 << (s1 + 1)), b[p].z, b[p].w);
          }
        }
      }
    }
  }
  template <int N> __device__ __forceinline__ void finish(const Sums<N> &s, int p, uint32_t d, float bs, Acc &acc) const {
    const float sv[4] = {sc.x, sc.y, sc.z, sc.w};
#pragma unroll
    for (int m = 0; m < 4; ++m) {
      const int h = m >> 1, j = m & 1;
      int i0 = 0, i1 = 0;
      if constexpr (NIB) {  // exact: multiples of 16 in the high-nibble rows
        i0 = s.n[p][h][2 * j] >> (4 * j);
        i1 = s.n[p][h][2 * j + 1] >> (4 * j);
      }
#pragma unroll
      for (int pl = 0; pl < NPL; ++pl) {
        i0 += ((s.pl[p][pl][h][0][2 * j] + (s.pl[p][pl][h][1][2 * j] >> 4)) >> m) << (P0 + pl);
        i1 += ((s.pl[p][pl][h][0][2 * j + 1] + (s.pl[p][pl][h][1][2 * j + 1] >> 4)) >> m) << (P0 + pl);
      }
      acc.r[m] += mma_row_value(i0, i1, d << (BITS - 1)) * (bs * sv[m]);  // zero point 2^(BITS-1)
    }
  }
};
template <> struct Unit<LMB_INT5> : PlanesUnit<LMB_INT5, 5, true> {};
template <> struct Unit<LMB_INT6> : PlanesUnit<LMB_INT6, 6, true> {};
template <> struct Unit<DK_INT3_MMA> : PlanesUnit<DK_INT3_MMA, 3, false> {};

// 8-bit weights on the signed 8-bit MMA: the tile's words are the A operands as they are.
template <> struct Unit<DK_INT8_MMA> : MmaUnitBase<Unit<DK_INT8_MMA>, 2> {
  uint4 v[16];
  float4 sc;
  template <int N> struct Sums { int c[N][2][4]; };
  __device__ __forceinline__ void load(const uint8_t *tile, int lane) {
#pragma unroll
    for (int c = 0; c < 16; ++c) v[c] = ld_stream_v4(tile + (size_t(c) * TILE_ROWS + lane) * 16);
    sc = as_float4(ld_stream_v4(tile + size_t(16) * TILE_ROWS * 16 + size_t(lane >> 2) * 16));
  }
  template <int N> __device__ __forceinline__ void mma_block(const uint4 *dig, int ps, Sums<N> &s) const {
#pragma unroll
    for (int p = 0; p < N; ++p)
#pragma unroll
      for (int h = 0; h < 2; ++h) s.c[p][h][0] = s.c[p][h][1] = s.c[p][h][2] = s.c[p][h][3] = 0;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      uint4 b[N];
#pragma unroll
      for (int p = 0; p < N; ++p) b[p] = dig[q * 16 + p * ps];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const uint4 w0 = v[h * 8 + 2 * q], w1 = v[h * 8 + 2 * q + 1];
#pragma unroll
        for (int p = 0; p < N; ++p) {
          mma_s8s8(s.c[p][h], w0.x, w0.y, w0.z, w0.w, b[p].x, b[p].y);
          mma_s8s8(s.c[p][h], w1.x, w1.y, w1.z, w1.w, b[p].z, b[p].w);
        }
      }
    }
  }
  template <int N> __device__ __forceinline__ void finish(const Sums<N> &s, int p, uint32_t, float bs, Acc &acc) const {
    acc.r[0] += mma_row_value(s.c[p][0][0], s.c[p][0][1], 0u) * (bs * sc.x);
    acc.r[1] += mma_row_value(s.c[p][0][2], s.c[p][0][3], 0u) * (bs * sc.y);
    acc.r[2] += mma_row_value(s.c[p][1][0], s.c[p][1][1], 0u) * (bs * sc.z);
    acc.r[3] += mma_row_value(s.c[p][1][2], s.c[p][1][3], 0u) * (bs * sc.w);
  }
};

template <> struct Unit<LMB_INT8> {
  static constexpr int FPB = 256;
  uint4 v[16];
  float sc;
  __device__ __forceinline__ void load(const uint8_t *tile, int lane) {
#pragma unroll
    for (int c = 0; c < 16; ++c) v[c] = ld_stream_v4(tile + (size_t(c) * TILE_ROWS + lane) * 16);
    sc = ld_stream_f32(tile + size_t(16) * TILE_ROWS * 16 + size_t(lane) * 4);
  }
  using Acc = float;
  static __device__ __forceinline__ void acc_init(Acc &a) { a = 0.0f; }
  static __device__ __forceinline__ float acc_row(const Acc &a, int) { return a; }
  __device__ __forceinline__ void eval(const float *blk, float, const int *, Acc &out) const {
    const float4 *x4 = reinterpret_cast<const float4 *>(blk);
    float2 acc[2] = {{0.f, 0.f}, {0.f, 0.f}};
#pragma unroll
    for (int c = 0; c < 16; ++c) {
      int8_word(v[c].x, x4[4 * c + 0], acc);
      int8_word(v[c].y, x4[4 * c + 1], acc);
      int8_word(v[c].z, x4[4 * c + 2], acc);
      int8_word(v[c].w, x4[4 * c + 3], acc);
    }
    out += ((acc[0].x + acc[0].y) + (acc[1].x + acc[1].y)) * sc;
  }
  static __device__ __forceinline__ void prologue(const float (&v)[8], int lane, float *blk, float *, int *) {
    dq_prologue(v, lane, blk);
  }
};

// ---------------------------------------------------------------------------------------------
// The kernel
// ---------------------------------------------------------------------------------------------
// Row-blocks a warp keeps in flight (in registers) besides the one it evaluates: small units
// need more of them to cover the HBM latency with the two or three CTAs an SM holds.
__host__ __device__ constexpr int prefetch_depth(int kind) {
  return kind == DK_TERNARY_MMA ? 3 : kind == DK_INT2_MMA ? 2 : kind == DK_BINARY_MMA ? 5 : kind == LMB_TERNARY ? 2
       : (kind == LMB_INT5 || kind == LMB_INT6 || kind == DK_INT8_MMA) ? 0 : kind == DK_INT3_MMA ? 1 : kind == LMB_INT2 ? 2 : kind == LMB_BINARY ? 3
       : kind == LMB_INT8 ? 0 : 1;
}

// Resident CTAs per SM the kernel is compiled for (128 or 255 registers per thread).
__host__ __device__ constexpr bool kind_is_wide(int kind) { return kind == LMB_INT5 || kind == LMB_INT6 || kind == DK_INT8_MMA; }
__host__ __device__ constexpr int min_ctas(int kind, int nseq) {
  return (kind == LMB_INT8 || nseq == 8 || (nseq == 4 && kind_is_wide(kind))) ? 1 : 2;
}
// Most sequences one pass over the weights serves.
__host__ __device__ constexpr int max_seqs_per_pass(int kind) {
  return !kind_is_mma(kind) ? 1 : (kind == LMB_INT5 || kind == LMB_INT6 || kind == DK_INT3_MMA) ? 2 : 8;
}

}  // namespace

}  // namespace lmb
