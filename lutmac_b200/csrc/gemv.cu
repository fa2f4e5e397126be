// GEMV kernels for every block kind, with the lut_linear prologue (zero padding, block-wise
// FWHT rotation, optional RMSNorm or SiLU*up of the input) and epilogue (block scales, RRQ
// residual plane, bias, residual add) fused in.
//
// Replaces lut_gemv / lut_gemv_binary / int2_gemv ... int8_gemv (include/lutmac/lut_gemm.hpp:
// 172-408, scalar loops src/kernels/lut_gemm_scalar.cpp:7-61,186-428) and lut_linear
// (lut_gemm_scalar.cpp:85-113,174-178) with precompute_luts (lut_gemm.hpp:53-58) and
// apply_hadamard_rotation (transform_simd.cpp:101-110).  Two formulations:
//   * integer tensor-core units (default for every kind): the weight tile is stored in the
//     operand order of the 8-bit integer MMA with several rows sharing the bits of a byte, so an
//     `and` with a mask yields an operand register; the activations of a 256-block become 32-bit
//     fixed point with one exponent, cut into four signed base-256 digits (the B operand);
//     sums are exact integers, the code's zero point is removed with the digit sums;
//   * table-lookup units (the reference's own formulation, selectable): ternary L[pos]-L[neg]
//     (lut_gemm_simd.cpp:203-221), n-bit planes sum_p 2^p L[idx_p] - zero_point*L[15]
//     (lut_gemm_simd.cpp:352-366), RRQ primary*scale + residual*scale2 (lut_gemm_simd.cpp:
//     326-328), with 16-entry group tables in shared memory; 8-bit as dequantise + FMA.
//
// Work decomposition.  One launch serves up to MAX_JOBS independent GEMVs of one kind (q/k/v
// or gate/up of a layer share a launch), any number through a prepared group.  A CTA of 8
// warps owns a work item = (job, group of R row-tiles of 32 rows, slice of S consecutive
// 256-column blocks).  A warp streams weight tiles with 128-bit coalesced loads through a ring
// of register slots.  When K is split over several CTAs, partial sums go to a scratch buffer
// and the last CTA to arrive for a row group adds them in slice order (deterministic).
// Batches: 2, 4 or 8 sequences share one pass over the weights on the tensor-core units.
//
// Programmatic dependent launch: a kernel lets its successor start at once, the successor
// prefetches its first weight tiles (weights never depend on a predecessor) and only then
// waits for the predecessor's results before touching activations or writing anything.
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <new>
#include <vector>

#include "gemv_units.cuh"

namespace lmb {

namespace {

constexpr int WARPS = 8;
constexpr int THREADS = WARPS * 32;
constexpr int MAX_JOBS = 4;
constexpr int MAX_CLUSTER_BLOCKS = 384;  // longest input (in 256-blocks) of a launch that uses thread-block clusters
constexpr int MAX_CLUSTER = 8;           // portable cluster size

struct Job {
  const uint8_t *tiles;
  const float *x;
  float *y;
  const float *bias;
  const float *x2;        // second prologue operand: norm weight (XMODE_RMSNORM) or up vector (XMODE_SILU_MUL)
  const float *residual;  // added to the output, laid out like y (may alias y); null for none
  float *scratch;       // [batch][n_ks][mp] partial sums (n_ks > 1 only)
  unsigned *counters;   // [batch][n_rg] arrival counters (n_ks > 1 only)
  int M, mp, bpr, row_tiles;
  int R, S, n_rg, n_ks;
  int cta_end;          // exclusive prefix of CTAs over the jobs of the launch
  unsigned x_len, x_stride, y_stride;
  // Hand-off to the next projection (batch 1, R = 8: a row group is one 256-block of the output):
  // the CTA that completes a row group also prepares that block as the NEXT GEMV's activation --
  // times the next norm's weight, rotated, as fixed-point digits -- so that the consumer's CTAs copy
  // records instead of each converting the whole vector.  next_prep null: off.
  uint32_t *next_prep;      // [block] records of PREP_WORDS words
  float *next_sumsq;        // [block] sum of squares of the block's outputs (the consumer's RMSNorm statistic)
  const float *next_w;      // weight of the norm between this projection and the next (null: none)
  int next_rotate;
#ifdef LMB_DEBUG_BOUNDS
  size_t tiles_bytes;   // extent of `tiles`
  size_t y_floats;      // extent of `y`
  size_t scratch_floats;  // extent of `scratch`
#endif
};

// One prepared (sequence, block): 256 words of digits in B-operand order, block scale, two digit-pair sums, pad.
constexpr int PREP_WORDS = PREP_RECORD_WORDS;

struct GemvParams {
  Job job[MAX_JOBS];
  int njobs;
  int rotate;
  int xmode;   // how the activations are formed in the prologue (XMODE_*)
  int batch;   // sequences of the launch
  float eps;   // XMODE_RMSNORM
  // a prepared group of any number of jobs: job table and per-CTA (job, first CTA of the job)
  // pairs in device memory; null for ordinary launches
  const Job *jobs_dev;
  const int2 *cta_map;
  PeerOut peer;  // peer.n > 0: job 0's output goes to every rank's exchange block
  // activations already converted by k_prepare_x (batched launches whose jobs share one input):
  // [sequence][block] records of PREP_WORDS words; null: every CTA converts its own slice
  const uint32_t *prep;
  // with `prep` from a producer's hand-off: the partial sums of squares whose total normalises the
  // prepared vector (RMSNorm is linear in that scalar, so it is applied to the block scales); null: none
  const float *prep_sumsq;
  int prep_sumsq_n;
  unsigned long long *dbg;  // this launch's slot of the launch timeline (debugging), or null
  // Thread-block clusters (batch 1, integer-MMA kinds): cl_size consecutive CTAs = the n_ks K slices of
  // cl_size / n_ks consecutive row groups of one job.  The CTAs that read the same K slice convert
  // its activations together (each a share, written into the shared memory of all of them), and the
  // K slices of a row group are added up through distributed shared memory instead of a scratch
  // buffer and an arrival counter.  0 or 1: no clusters.
  int cl_size;
};

// CLUSTERED: the instantiation launched with thread-block clusters (GemvParams::cl_size); kept apart so
// that the ordinary kernel carries none of its code.
template <int KIND, int NSEQ, bool CLUSTERED = false>
__global__ void __launch_bounds__(THREADS, min_ctas(KIND, NSEQ)) k_gemv(const __grid_constant__ GemvParams p) {
  static_assert(!CLUSTERED || (NSEQ == 1 && kind_is_mma(KIND)), "clusters: batch 1, integer-MMA kinds");
  // NSEQ sequences share one pass over the weights (integer-MMA kinds only: two sequences per
  // MMA); the other kinds run one sequence per CTA, blockIdx.y selecting it.
  static_assert(NSEQ == 1 || kind_is_mma(KIND), "several sequences per pass need an integer-MMA kind");
  using U = Unit<KIND>;
  constexpr int FPB = U::FPB;
  constexpr size_t TB = tile_bytes(KIND);
  constexpr int NP = (NSEQ + 1) / 2;
  extern __shared__ __align__(1024) float smem[];
  __shared__ float part[NSEQ][THREADS];
  __shared__ float xsum[NSEQ * 64];
  __shared__ __align__(16) int xaux[NP * 64 * 4];
  __shared__ int is_last;
  __shared__ float xss[CLUSTERED ? MAX_CLUSTER_BLOCKS : 1];  // cluster mode: sum of squares of every 256-block of the input

  pdl_launch_dependents();
  if (threadIdx.x == 0) tl_min(p.dbg, 0);

  // work item of this CTA
  int j = 0, first = 0;
  if (p.jobs_dev) {
    const int2 m = p.cta_map[blockIdx.x];
    j = m.x;
    first = m.y;
  } else {
    while (j + 1 < p.njobs && int(blockIdx.x) >= p.job[j].cta_end) ++j;
    first = j ? p.job[j - 1].cta_end : 0;
  }
  const Job &job = p.jobs_dev ? p.jobs_dev[j] : p.job[j];
  const int local = int(blockIdx.x) - first;
  const int rg = local / job.n_ks, ks = local - rg * job.n_ks;
  const int batch0 = blockIdx.y * NSEQ;               // first sequence of this CTA
  const int nb = min(NSEQ, p.batch - batch0);         // sequences of this CTA
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rt0 = rg * job.R;
  const int nrt = min(job.R, job.row_tiles - rt0);
  const int wpr = WARPS / job.R;  // warps sharing one row-tile
  const int rtl = warp / wpr, sub = warp - rtl * wpr;
  const int b0 = ks * job.S;
  const int ns = min(job.S, job.bpr - b0);
  const bool active = rtl < nrt && sub < ns;
  const uint8_t *row_tiles = job.tiles + (size_t(rt0 + rtl) * job.bpr + b0) * TB;
  constexpr bool clustered = CLUSTERED;
  const int crank = clustered ? local % p.cl_size : 0;                    // rank in the cluster (job starts are multiples of cl_size)

  // weights do not depend on the preceding kernel: fetch the first units before waiting for it
  constexpr int NSLOT = (NSEQ > 2 ? 1 : prefetch_depth(KIND)) + 1;  // a ring of row-blocks held in registers
  U slot[NSLOT];
#ifdef LMB_DEBUG_BOUNDS
  auto tile_ok = [&](const uint8_t *tp) { return LMB_IN_BOUNDS(size_t(tp - job.tiles) + TB <= job.tiles_bytes, BOUNDS_WEIGHT_TILE, tp - job.tiles); };
#else
  auto tile_ok = [](const uint8_t *) { return true; };
#endif
  if (active) {
#pragma unroll
    for (int sl = 0; sl < NSLOT; ++sl)
      if (sub + sl * wpr < ns && tile_ok(row_tiles + size_t(sub + sl * wpr) * TB)) slot[sl].load(row_tiles + size_t(sub + sl * wpr) * TB, lane);
  }

  pdl_wait();
  if (threadIdx.x == 0) {
    tl_min(p.dbg, 1);
    tl_max(p.dbg, 2);
  }

  // tensor-parallel output: the epoch selects the parity of the exchange slot
  const unsigned epoch = p.peer.n ? *reinterpret_cast<volatile unsigned *>(p.peer.epoch) : 0u;
  const float *x = job.x + size_t(batch0) * job.x_stride;
  float *inv_rms = part[0];  // [sequence] after the block below (XMODE_RMSNORM)
  if (p.xmode == XMODE_RMSNORM && !p.prep && !clustered) {
    // RMSNorm of the whole input vectors (src/layers/norm.cpp:18-34), recomputed by every CTA
    float ss[NSEQ];
#pragma unroll
    for (int q = 0; q < NSEQ; ++q) ss[q] = 0.0f;
    for (unsigned i = threadIdx.x; i < job.x_len; i += THREADS) {
#pragma unroll
      for (int q = 0; q < NSEQ; ++q) {
        const float v = (q < nb) ? x[size_t(q) * job.x_stride + i] : 0.0f;
        ss[q] += v * v;
      }
    }
#pragma unroll
    for (int q = 0; q < NSEQ; ++q) {
#pragma unroll
      for (int m = 16; m > 0; m >>= 1) ss[q] += __shfl_xor_sync(0xffffffffu, ss[q], m);
      if (lane == 0) xsum[q * WARPS + warp] = ss[q];  // xsum is free until the prologue below
    }
    __syncthreads();
    if (threadIdx.x < NSEQ) {
      float t = 0.0f;
#pragma unroll
      for (int k = 0; k < WARPS; ++k) t += xsum[threadIdx.x * WARPS + k];
      inv_rms[threadIdx.x] = 1.0f / sqrtf(t / float(job.x_len) + p.eps);
    }
    __syncthreads();
  }
  if constexpr (kind_is_mma(KIND)) {
    if (p.prep) {
      float prep_scale = 1.0f;
      if (p.prep_sumsq) {  // src/layers/norm.cpp:18-34 with the sum of squares from the producer's per-block partials
        // all partials in one round trip: lane l of every warp takes l, l + 32, ... (a loop of dependent
        // loads here cost 17 us per launch)
        float tot = 0.0f;
        for (int i = lane; i < p.prep_sumsq_n; i += 32) tot += __ldcg(p.prep_sumsq + i);
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, m);
        prep_scale = 1.0f / sqrtf(tot / float(job.x_len) + p.eps);
      }
      // the launch's activations were converted once (k_prepare_x, or the producing GEMV): copy this CTA's slice
      const int items = ns * nb;
      for (int it = warp; it < items; it += WARPS) {
        const int q = NSEQ == 1 ? 0 : it / ns, bl = it - q * ns;
        const uint32_t *src = p.prep + (size_t(batch0 + q) * job.bpr + b0 + bl) * PREP_WORDS;
        uint4 *dst = reinterpret_cast<uint4 *>(smem + (size_t(q) * job.S + bl) * FPB);
        const uint4 *s4 = reinterpret_cast<const uint4 *>(src);
        dst[lane] = __ldcg(s4 + lane);
        dst[lane + 32] = __ldcg(s4 + lane + 32);
        if (lane == 0) {
          const uint4 tail = __ldcg(s4 + 64);  // {block scale, d01, d23, -}
          int *aux = xaux + ((q >> 1) * 64 + bl) * 4;
          xsum[q * 64 + bl] = __uint_as_float(tail.x) * prep_scale;
          aux[2 * (q & 1)] = int(tail.y);
          aux[2 * (q & 1) + 1] = int(tail.z);
          if ((q | 1) >= nb) aux[2] = aux[3] = 0;
        }
      }
    }
  }
  if constexpr (CLUSTERED) {
    {
      // The cr-th of the Cr CTAs that read this K slice converts blocks cr, cr + Cr, ... and writes each
      // record into all Cr of them.  RMSNorm (src/layers/norm.cpp:18-34) is linear in 1 / rms: the
      // digits are those of x * w, every converter publishes its blocks' sums of squares to the whole
      // cluster (which covers all of K), and the block scales are multiplied by 1 / rms afterwards.
      const int Cr = p.cl_size / job.n_ks, cr = crank / job.n_ks;
      const int mine = ns > cr ? (ns - cr + Cr - 1) / Cr : 0;
      float v[8], w8[8], nv[8];
      if (warp < mine) load_x8(x, job.x_len, size_t(b0 + cr + warp * Cr), lane, nv);
      for (int it = warp; it < mine; it += WARPS) {
        const int bl = cr + it * Cr;
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = nv[e];
        if (p.xmode == XMODE_RMSNORM) load_x8(job.x2, job.x_len, size_t(b0 + bl), lane, w8);
        if (p.xmode == XMODE_SILU_MUL || p.xmode == XMODE_GELU_MUL) load_x8(job.x2 + size_t(batch0) * job.x_stride, job.x_len, size_t(b0 + bl), lane, w8);
        if (it + WARPS < mine) load_x8(x, job.x_len, size_t(b0 + cr + (it + WARPS) * Cr), lane, nv);
        if (p.xmode == XMODE_RMSNORM) {
          float ss = 0.0f;
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            ss += v[e] * v[e];
            v[e] *= w8[e];
          }
#pragma unroll
          for (int m = 16; m > 0; m >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, m);
          if (lane < p.cl_size) st_cluster_f32(cluster_addr(&xss[b0 + bl], unsigned(lane)), ss);
        } else if (p.xmode == XMODE_SILU_MUL) {
#pragma unroll
          for (int e = 0; e < 8; ++e) v[e] = (v[e] / (1.0f + expf(-v[e]))) * w8[e];  // silu(gate) * up, model.cpp:36,414-416
        } else if (p.xmode == XMODE_GELU_MUL) {
#pragma unroll
          for (int e = 0; e < 8; ++e) v[e] = gelu_tanh(v[e]) * w8[e];  // gelu(gate) * up, model.cpp:38-42,409-412
        }
        if (p.rotate) fwht256_warp(v, lane);
        float *blk = smem + size_t(bl) * FPB;
        int *aux = xaux + bl * 4;
        U::prologue(v, lane, blk, xsum + bl, aux);
        if (lane == 0) aux[2] = aux[3] = 0;  // no second sequence
        __syncwarp();
        if (Cr > 1) {
          const uint4 *src = reinterpret_cast<const uint4 *>(blk);
          const uint4 d0 = src[lane], d1 = src[lane + 32];
          const float bs = xsum[bl];
          const uint4 ax = *reinterpret_cast<const uint4 *>(aux);
          for (int c2 = 0; c2 < Cr; ++c2) {
            if (c2 == cr) continue;
            const unsigned peer = unsigned(c2 * job.n_ks + ks);
            st_cluster_v4(cluster_addr(src + lane, peer), d0);
            st_cluster_v4(cluster_addr(src + lane + 32, peer), d1);
            if (lane == 0) {
              st_cluster_f32(cluster_addr(xsum + bl, peer), bs);
              st_cluster_v4(cluster_addr(aux, peer), ax);
            }
          }
        }
      }
      cluster_sync_all();
      if (p.xmode == XMODE_RMSNORM) {
        float tot = 0.0f;
        for (int i = lane; i < job.bpr; i += 32) tot += xss[i];
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, m);
        const float ir = 1.0f / sqrtf(tot / float(job.x_len) + p.eps);
        if (int(threadIdx.x) < ns) xsum[threadIdx.x] *= ir;
      }
    }
  }
  if (!(kind_is_mma(KIND) && p.prep) && !clustered) {
    // one warp per (sequence, block); the next item's activations are fetched while this one is converted
    float v[8], w8[8], nv[8];
    const int items = ns * nb;
    if (warp < items) load_x8(x + size_t(NSEQ == 1 ? 0 : warp / ns) * job.x_stride, job.x_len, size_t(b0 + (NSEQ == 1 ? warp : warp % ns)), lane, nv);
    for (int it = warp; it < items; it += WARPS) {
      const int q = NSEQ == 1 ? 0 : it / ns, bl = it - q * ns;
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] = nv[e];
      if (p.xmode == XMODE_RMSNORM) load_x8(job.x2, job.x_len, size_t(b0 + bl), lane, w8);
      if (p.xmode == XMODE_SILU_MUL || p.xmode == XMODE_GELU_MUL) load_x8(job.x2 + size_t(batch0 + q) * job.x_stride, job.x_len, size_t(b0 + bl), lane, w8);
      if (it + WARPS < items) {
        const int nq = NSEQ == 1 ? 0 : (it + WARPS) / ns;
        load_x8(x + size_t(nq) * job.x_stride, job.x_len, size_t(b0 + (it + WARPS) - nq * ns), lane, nv);
      }
      if (p.xmode == XMODE_RMSNORM) {
        const float ir = inv_rms[q];
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = v[e] * ir * w8[e];
      } else if (p.xmode == XMODE_SILU_MUL) {
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = (v[e] / (1.0f + expf(-v[e]))) * w8[e];  // silu(gate) * up, model.cpp:36,414-416
      } else if (p.xmode == XMODE_GELU_MUL) {
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = gelu_tanh(v[e]) * w8[e];  // gelu(gate) * up, model.cpp:38-42,409-412
      }
      if (p.rotate) fwht256_warp(v, lane);
      if constexpr (kind_is_mma(KIND)) {
        int *aux = xaux + ((q >> 1) * 64 + bl) * 4;
        U::prologue(v, lane, smem + (size_t(q) * job.S + bl) * FPB, xsum + q * 64 + bl, aux + 2 * (q & 1));
        if ((q | 1) >= nb && lane == 0) aux[2] = aux[3] = 0;  // no second sequence in this pair
      } else {
        U::prologue(v, lane, smem + size_t(bl) * FPB, xsum + bl, xaux + 4 * bl);
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) tl_max(p.dbg, 3);

  // each slot is evaluated and at once refilled with the row-block NSLOT steps ahead, so that
  // NSLOT-1 loads are in flight during every evaluation
  float acc[NSEQ];
  if constexpr (kind_is_mma(KIND)) {
    typename U::Acc accs[NP];
#pragma unroll
    for (int q = 0; q < NP; ++q) U::acc_init(accs[q]);
    const MmaX xo{smem, xsum, xaux, job.S * FPB};
    if (active) {
      for (int base = sub; base < ns; base += NSLOT * wpr) {
#pragma unroll
        for (int sl = 0; sl < NSLOT; ++sl) {
          const int bl = base + sl * wpr;
          if (bl < ns) {
            slot[sl].template eval<NP, (NSEQ > 1)>(xo, bl, accs);
            if (bl + NSLOT * wpr < ns && tile_ok(row_tiles + size_t(bl + NSLOT * wpr) * TB)) slot[sl].load(row_tiles + size_t(bl + NSLOT * wpr) * TB, lane);
          }
        }
      }
    }
#pragma unroll
    for (int q = 0; q < NSEQ; ++q) acc[q] = U::acc_row(accs[q >> 1], lane, q & 1);  // warp-uniform: every lane takes part
  } else {
    typename U::Acc accs;
    U::acc_init(accs);
    if (active) {
      for (int base = sub; base < ns; base += NSLOT * wpr) {
#pragma unroll
        for (int sl = 0; sl < NSLOT; ++sl) {
          const int bl = base + sl * wpr;
          if (bl < ns) {
            slot[sl].eval(smem + size_t(bl) * FPB, xsum[bl], xaux + 4 * bl, accs);
            if (bl + NSLOT * wpr < ns && tile_ok(row_tiles + size_t(bl + NSLOT * wpr) * TB)) slot[sl].load(row_tiles + size_t(bl + NSLOT * wpr) * TB, lane);
          }
        }
      }
    }
    acc[0] = U::acc_row(accs, lane);
  }

  // combine the warps that share a row-tile, in warp order: thread t ends up with row rt0*32 + t
  if (threadIdx.x == 0) tl_max(p.dbg, 4);
  if (p.xmode == XMODE_RMSNORM && !p.prep && !clustered) __syncthreads();  // inv_rms (in part[0]) has been read by everyone
#pragma unroll
  for (int q = 0; q < NSEQ; ++q) part[q][threadIdx.x] = acc[q];
  __syncthreads();
  const int t = threadIdx.x;
  const bool owns_row = t < nrt * TILE_ROWS;
  float s[NSEQ];
#pragma unroll
  for (int q = 0; q < NSEQ; ++q) {
    s[q] = 0.0f;
    if (owns_row) {
      const int r = t >> 5;
      for (int k = 0; k < wpr; ++k) s[q] += part[q][(r * wpr + k) * 32 + (t & 31)];
    }
  }
  const int row = rt0 * TILE_ROWS + t;
  // one output element; with tensor parallelism it goes to this rank's slot in every rank's block
  auto emit = [&](int q, float o) {
    const size_t at = size_t(batch0 + q) * job.y_stride + row;
#ifdef LMB_DEBUG_BOUNDS
    if (!LMB_IN_BOUNDS(at < job.y_floats, BOUNDS_OUTPUT, at)) return;
#endif
    if (p.peer.n == 0) {
      job.y[at] = o;
    } else {
      // value and tag travel in one 8-byte store: the reader needs no fence and no separate flag
      const size_t slot = (size_t(epoch & 1u) * p.peer.n + p.peer.rank) * p.peer.cap + at;
      const unsigned long long word = (static_cast<unsigned long long>(epoch + 1u) << 32) | __float_as_uint(o);
      for (int r = 0; r < p.peer.n; ++r) *reinterpret_cast<volatile unsigned long long *>(p.peer.data[r] + slot) = word;
    }
  };
  // Hand-off (see Job::next_prep): thread t of the CTA that completes the row group holds output
  // 256 * rg + t; one warp turns the block into the next GEMV's prepared activation record.
  float handoff = 0.0f;  // this thread's finished output (first sequence), 0 beyond M
  auto hand_off = [&]() {
    if (NSEQ != 1 || !job.next_prep) return;  // uniform over the CTA
    __syncthreads();
    part[0][t] = handoff;
    __syncthreads();
    if (warp == 0) {
      float v[8];
      float ss = 0.0f;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        v[e] = part[0][lane * 8 + e];
        ss += v[e] * v[e];
      }
#pragma unroll
      for (int m = 16; m > 0; m >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, m);
      if (job.next_w) {
        float w8[8];
        load_x8(job.next_w, size_t(job.M), size_t(rg), lane, w8);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] *= w8[e];
      }
      if (job.next_rotate) fwht256_warp(v, lane);
      float *stage = smem;  // the activation digits of this launch are no longer needed by this CTA
      mma_prologue(v, lane, stage, &xsum[0], &xaux[0]);
      __syncwarp();
      uint4 *dst = reinterpret_cast<uint4 *>(job.next_prep + size_t(rg) * PREP_WORDS);
      const uint4 *src = reinterpret_cast<const uint4 *>(stage);
      dst[lane] = src[lane];
      dst[lane + 32] = src[lane + 32];
      if (lane == 0) {
        dst[64] = make_uint4(__float_as_uint(xsum[0]), uint32_t(xaux[0]), uint32_t(xaux[1]), 0u);
        job.next_sumsq[rg] = ss;
      }
    }
  };
  if (job.n_ks == 1) {
    if (owns_row && row < job.M) {
      const float bias = job.bias ? job.bias[row] : 0.0f;
#pragma unroll
      for (int q = 0; q < NSEQ; ++q)
        if (q < nb) {
          float o = s[q];
          if (job.bias) o += bias;
          if (job.residual) o += job.residual[size_t(batch0 + q) * job.y_stride + row];
          emit(q, o);
          if (q == 0) handoff = o;
        }
    }
    if (rg < job.n_rg) hand_off();
    if (t == 0) {
      tl_max(p.dbg, 5);
      tl_min(p.dbg, 6);
    }
    return;
  }
  if constexpr (CLUSTERED) {
    // split K inside a cluster: slice 0 of the row group adds the partial sums of the others, in slice
    // order, out of their shared memory
    __syncthreads();  // part[] has been read
    if (owns_row) part[0][t] = s[0];
    cluster_sync_all();
    if (ks == 0 && owns_row && row < job.M) {
      float tot = s[0];
      for (int k = 1; k < job.n_ks; ++k) tot += ld_cluster_f32(cluster_addr(&part[0][t], unsigned(crank + k)));
      if (job.bias) tot += job.bias[row];
      if (job.residual) tot += job.residual[size_t(batch0) * job.y_stride + row];
      emit(0, tot);
      handoff = tot;
    }
    cluster_sync_all();  // the other slices' shared memory stays alive until it has been read
    if (ks == 0 && rg < job.n_rg) hand_off();
    if (t == 0) {
      tl_max(p.dbg, 5);
      tl_min(p.dbg, 6);
    }
    return;
  }
  // split K: publish the partial sums, the last slice to arrive adds them in slice order
  if (owns_row) {
#pragma unroll
    for (int q = 0; q < NSEQ; ++q)
      if (q < nb) {
        const size_t at = (size_t(batch0 + q) * job.n_ks + ks) * job.mp + row;
#ifdef LMB_DEBUG_BOUNDS
        if (!LMB_IN_BOUNDS(at < job.scratch_floats, BOUNDS_SCRATCH, at)) continue;
#endif
        job.scratch[at] = s[q];
      }
  }
  __syncthreads();
  unsigned *ctr = job.counters + size_t(blockIdx.y) * job.n_rg + rg;
  if (t == 0) {
    // release: this CTA's partial sums (ordered before the atomic by the barrier above, and release is
    // cumulative); acquire: the partial sums of the slices that arrived earlier
    unsigned before;
    asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(before) : "l"(ctr) : "memory");
    is_last = (before == unsigned(job.n_ks - 1));
  }
  __syncthreads();
  if (!is_last) {  // uniform over the CTA
    if (t == 0) tl_min(p.dbg, 6);
    return;
  }
  if (owns_row && row < job.M) {
    const float bias = job.bias ? job.bias[row] : 0.0f;
#pragma unroll
    for (int q = 0; q < NSEQ; ++q)
      if (q < nb) {
        const float *scr = job.scratch + size_t(batch0 + q) * job.n_ks * job.mp;
        float tot = 0.0f;
        for (int k = 0; k < job.n_ks; ++k) tot += __ldcg(scr + size_t(k) * job.mp + row);
        if (job.bias) tot += bias;
        if (job.residual) tot += job.residual[size_t(batch0 + q) * job.y_stride + row];
        emit(q, tot);
        if (q == 0) handoff = tot;
      }
  }
  if (t == 0) *ctr = 0u;  // ready for the next launch
  hand_off();
  if (t == 0) tl_max(p.dbg, 5);
}

// Conversion pass for batched launches: the activations of every (sequence, block) of the shared
// input are normalised / gated / rotated and turned into fixed-point digits ONCE, instead of by
// every CTA of the GEMV.  One warp per (sequence, block); grid = (ceil(bpr / 8), sequences).
__global__ void __launch_bounds__(THREADS) k_prepare_x(const float *x, const float *x2, unsigned x_len, unsigned x_stride, int bpr,
                                                       int xmode, int rotate, float eps, uint32_t *out) {
  pdl_launch_dependents();
  __shared__ float red[WARPS];
  __shared__ __align__(16) float stage[WARPS][256];
  __shared__ float bsc[WARPS];
  __shared__ int aux2[WARPS][2];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, q = blockIdx.y;
  const float *xq = x + size_t(q) * x_stride;
  float inv_rms = 1.0f;
  if (xmode == XMODE_RMSNORM) {
    float ss = 0.0f;
    for (unsigned i = threadIdx.x; i < x_len; i += THREADS) {
      const float v = xq[i];
      ss += v * v;
    }
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, m);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    ss = 0.0f;
#pragma unroll
    for (int k = 0; k < WARPS; ++k) ss += red[k];
    inv_rms = 1.0f / sqrtf(ss / float(x_len) + eps);
  }
  const int bl = blockIdx.x * WARPS + warp;
  if (bl >= bpr) return;
  float v[8], w8[8];
  load_x8(xq, x_len, size_t(bl), lane, v);
  if (xmode == XMODE_RMSNORM) {
    load_x8(x2, x_len, size_t(bl), lane, w8);
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = v[e] * inv_rms * w8[e];
  } else if (xmode == XMODE_SILU_MUL || xmode == XMODE_GELU_MUL) {
    load_x8(x2 + size_t(q) * x_stride, x_len, size_t(bl), lane, w8);
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = (xmode == XMODE_GELU_MUL ? gelu_tanh(v[e]) : v[e] / (1.0f + expf(-v[e]))) * w8[e];
  }
  if (rotate) fwht256_warp(v, lane);
  mma_prologue(v, lane, stage[warp], &bsc[warp], aux2[warp]);
  __syncwarp();
  uint4 *dst = reinterpret_cast<uint4 *>(out + (size_t(q) * bpr + bl) * PREP_WORDS);
  const uint4 *src = reinterpret_cast<const uint4 *>(stage[warp]);
  dst[lane] = src[lane];
  dst[lane + 32] = src[lane + 32];
  if (lane == 0) dst[64] = make_uint4(__float_as_uint(bsc[warp]), uint32_t(aux2[warp][0]), uint32_t(aux2[warp][1]), 0u);
}

// Tables only (debug view used by the parity tests): the same prologue, one warp per block.
__global__ void k_debug_luts(const float *x, size_t x_len, int nblocks, int rotate, float *out) {
  __shared__ __align__(1024) float tab[WARPS][1024];
  __shared__ float xs[WARPS];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.x * WARPS + warp;
  if (b < nblocks) {
    float v[8];
    load_x8(x, x_len, size_t(b), lane, v);
    if (rotate) fwht256_warp(v, lane);
    LutUnit<LMB_TERNARY>::prologue(v, lane, tab[warp], &xs[warp], nullptr);
    __syncwarp();
    for (int i = lane; i < 1024; i += 32) out[size_t(b) * 1024 + i] = tab[warp][i];
  }
}

// Tensor-parallel sum as a producer of prepared activations (batch 1, integer-MMA consumers): one CTA
// per 256-block of the hidden state adds the ranks' partial vectors out of this rank's exchange block
// (words {value, epoch tag}, polled with a bound: all ranks' words of an element are requested at once)
// and the residual, writes the new hidden state, and leaves the block as the next GEMV's activation
// record -- times the norm weight, rotated, as fixed-point digits -- with its sum of squares; the
// consumers normalise by the total (src/layers/norm.cpp:18-34 is linear in 1 / rms).  Replaces
// k_tp_sum_add_rmsnorm plus the conversion in every consumer CTA.
__global__ void __launch_bounds__(BLK) k_tp_sum_prepare(float *hidden, XchgHeader *hdr, const unsigned long long *data, int tp, unsigned cap,
                                                        const float *w, int rotate, uint32_t *prep, float *sumsq, unsigned spin_limit) {
  pdl_launch_dependents();
  __shared__ __align__(16) float vals[BLK];
  __shared__ __align__(16) float stage[BLK];
  __shared__ float red[BLK / 32];
  __shared__ float xs[1];
  __shared__ __align__(16) int xa[4];
  pdl_wait();  // the epoch below is advanced by the previous consumer of the exchange block, the residual written by earlier kernels
  const int t = threadIdx.x, warp = t >> 5, lane = t & 31, blk = blockIdx.x;
  const size_t i = size_t(blk) * BLK + t;
  const unsigned epoch = *reinterpret_cast<volatile unsigned *>(&hdr->epoch), tag = epoch + 1u;
  const unsigned long long *part = data + size_t(epoch & 1u) * tp * cap + i;
  unsigned long long word[MAX_TP];
#pragma unroll
  for (int r = 0; r < MAX_TP; ++r)
    if (r < tp) asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(word[r]) : "l"(part + size_t(r) * cap));
  bool gave_up = *reinterpret_cast<volatile unsigned *>(&hdr->timed_out) != 0u;
  float add = 0.0f;
#pragma unroll
  for (int r = 0; r < MAX_TP; ++r) {
    if (r < tp) {
      unsigned spins = 0;
      while (unsigned(word[r] >> 32) != tag && !gave_up) {
        if (++spins > spin_limit) {  // give up, report, carry on with what is there
          hdr->timed_out = 1u;
          gave_up = true;
          break;
        }
        __nanosleep(40);
        asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(word[r]) : "l"(part + size_t(r) * cap));
      }
      add += __uint_as_float(unsigned(word[r]));  // rank order: every rank computes the same bits
    }
  }
  const float v = hidden[i] + add;
  hidden[i] = v;
  float ss = v * v;
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, m);
  if (lane == 0) red[warp] = ss;
  vals[t] = v * w[i];
  __syncthreads();
  if (warp == 0) {
    float tot = lane < BLK / 32 ? red[lane] : 0.0f;
#pragma unroll
    for (int m = 4; m > 0; m >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, m);
    const float4 a = *reinterpret_cast<const float4 *>(vals + 8 * lane), c = *reinterpret_cast<const float4 *>(vals + 8 * lane + 4);
    float v8[8] = {a.x, a.y, a.z, a.w, c.x, c.y, c.z, c.w};
    if (rotate) fwht256_warp(v8, lane);
    mma_prologue(v8, lane, stage, &xs[0], &xa[0]);
    __syncwarp();
    uint4 *dst = reinterpret_cast<uint4 *>(prep + size_t(blk) * PREP_WORDS);
    const uint4 *src = reinterpret_cast<const uint4 *>(stage);
    dst[lane] = src[lane];
    dst[lane + 32] = src[lane + 32];
    if (lane == 0) {
      dst[64] = make_uint4(__float_as_uint(xs[0]), uint32_t(xa[0]), uint32_t(xa[1]), 0u);
      sumsq[blk] = tot;
    }
  }
  __syncthreads();
  if (t == 0 && atomicAdd(&hdr->done, 1u) == gridDim.x - 1u) {
    hdr->done = 0u;
    *reinterpret_cast<volatile unsigned *>(&hdr->epoch) = tag;  // read by the next producer, a later kernel
  }
}

struct Plan {
  int R, S, n_rg, n_ks, ctas;
  int cr;  // thread-block clusters: row groups per cluster (cluster size = cr * n_ks); 0: no cluster
};

// LMB_PLAN_FORCE="R,n_ks,cr" or lmb_debug_force_plan (experiments and tests): every batch-1 plan
// that can take these values does.
struct PlanForce {
  bool on = false;
  int R = 0, n_ks = 0, cr = 0;
  PlanForce() {
    const char *e = std::getenv("LMB_PLAN_FORCE");
    on = e && std::sscanf(e, "%d,%d,%d", &R, &n_ks, &cr) == 3;
  }
};
PlanForce g_plan_force;
// LMB_GEMV_CLUSTER=1: the planner may choose thread-block clusters (a plan forced with
// lmb_debug_force_plan may use them either way).  Off by default: a cluster starts only when all its
// CTAs find room at once, which costs part of the overlap with the preceding kernel's tail (1.5 to
// 5 us measured on the 70B-shaped decode step), and with the hand-off of prepared activations the
// conversion work they would share is gone; on the 1B / 1.5B-shaped steps they measured 5 % slower.
inline bool clusters_allowed() {
  static const bool ok = [] {
    const char *e = std::getenv("LMB_GEMV_CLUSTER");
    return e && e[0] == '1';
  }();
  return ok;
}

// Resident CTAs per SM of k_gemv<kind> (register limited), used to count waves.
int ctas_per_sm(int kind) { return kind_info(kind).lut ? 3 : 2; }

// Chooses R (row-tiles per CTA: 8, 4, 2 or 1; the 8 warps of a CTA then share a row-tile
// 1, 2, 4 or 8 ways along K, which costs only a shared-memory reduction), the K split over CTAs
// and whether the CTAs form thread-block clusters (K slices added up through distributed shared
// memory, and the conversion of the activations shared by the row groups of a cluster) or pass
// their partial sums through global scratch, by minimising a makespan estimate in units of "one
// warp evaluates one 256-column block":
//     waves of CTAs x (blocks per warp + prologue share + fixed CTA cost [+ split-K hand-off]).
// `other_row_tiles` are the row-tiles of the other jobs of the same launch.
// Work split of one GEMV.  `cluster`: -1 free choice (none or 2 / 4 / 8 CTAs), 0 none, else exactly this
// cluster size (the other jobs of the launch use it).
Plan make_plan(int kind, size_t row_tiles, size_t bpr, size_t batch, int sm_count, size_t other_row_tiles = 0, int nseq = 1,
               bool whole_blocks = false, int cluster = 0) {
  const PlanForce force = g_plan_force;
  const bool lut = kind_info(kind).lut;
  // 48 KiB of tables / activations per CTA (96 KiB when 4 or 8 sequences share a pass)
  const size_t s_cap = lut ? 12 : nseq == 1 ? 48 : nseq == 8 ? 12 : 24;
  const size_t slots = size_t(sm_count) * (min_ctas(kind, nseq) == 1 ? 1 : ctas_per_sm(kind));
  const double prologue_per_block = 1.5 * nseq, fixed = 1.5, split_cost = 2.5, cluster_sync = 3.0, cluster_split = 0.8;
  const bool throughput = (other_row_tiles + 7) / 8 * batch >= 2 * slots;
  const bool may_cluster = cluster != 0 && kind_is_mma(kind) && nseq == 1 && batch == 1 && bpr <= size_t(MAX_CLUSTER_BLOCKS) &&
                           (clusters_allowed() || (force.on && force.cr > 0));
  Plan best{};
  if (force.on && batch == 1 && nseq == 1 && force.n_ks >= 1 && size_t(force.n_ks) <= bpr) {
    const size_t fS = (bpr + size_t(force.n_ks) - 1) / size_t(force.n_ks), fc = size_t(force.cr) * size_t(force.n_ks);
    const bool shape_ok = fS <= s_cap && (bpr + fS - 1) / fS == size_t(force.n_ks) &&
                          (force.R == 8 || force.R == 4 || force.R == 2 || force.R == 1) && (size_t(force.R) <= row_tiles || force.R == 1) &&
                          (!whole_blocks || force.R == 8);
    const bool cluster_ok = force.cr == 0 ? cluster <= 0
                                          : (may_cluster && fc >= 2 && fc <= size_t(MAX_CLUSTER) && !(fc & (fc - 1)) &&
                                             (cluster < 0 || fc == size_t(cluster)));
    if (shape_ok && cluster_ok) {
      const size_t n_rg = (row_tiles + size_t(force.R) - 1) / size_t(force.R);
      const size_t n_rgp = force.cr ? (n_rg + size_t(force.cr) - 1) / size_t(force.cr) * size_t(force.cr) : n_rg;
      return Plan{force.R, int(fS), int(n_rg), force.n_ks, int(n_rgp) * force.n_ks, force.cr};
    }
  }
  double best_cost = 1e30;
  for (int R = 8; R >= 1; R >>= 1) {
    if (whole_blocks && R != 8) break;  // a row group must be one 256-block of the output (hand-off to the next GEMV)
    if (size_t(R) > row_tiles && R > 1 && !whole_blocks) continue;
    const size_t n_rg = (row_tiles + R - 1) / R, wpr = size_t(8 / R);
    for (size_t n_ks = 1; n_ks <= bpr; ++n_ks) {
      const size_t S = (bpr + n_ks - 1) / n_ks;
      if (S > s_cap) continue;
      if ((bpr + S - 1) / S != n_ks) continue;  // not a distinct split
      for (int cr = 0; cr <= MAX_CLUSTER; cr = cr ? cr * 2 : 1) {
        const size_t csize = size_t(cr) * n_ks;  // 0: no cluster
        if (cr && (!may_cluster || csize < 2 || csize > size_t(MAX_CLUSTER) || (csize & (csize - 1)))) continue;
        if (cluster > 0 && may_cluster && csize != size_t(cluster)) continue;
        if (cluster > 0 && !may_cluster) continue;
        const size_t n_rgp = cr ? (n_rg + size_t(cr) - 1) / size_t(cr) * size_t(cr) : n_rg;
        const size_t own = n_rgp * n_ks * batch;
        // other jobs of the launch are assumed to be cut the same way
        const size_t other_ctas = (other_row_tiles + R - 1) / R * n_ks * batch;
        const double per_warp = double((S + wpr - 1) / wpr);
        const size_t converted = cr ? (S + size_t(cr) - 1) / size_t(cr) : S;  // blocks this CTA converts itself
        const double cta_time = per_warp + prologue_per_block * double((converted + 7) / 8) + fixed + (cr ? cluster_sync : 0.0) +
                                (n_ks > 1 ? (cr ? cluster_split : split_cost) : 0.0);
        // with plenty of work from other jobs (even cut 8 row-tiles per CTA) the GPU is busy anyway:
        // minimise this job's total CTA time; otherwise minimise the time until its last CTA finishes
        const double cost = (throughput ? double(own) * cta_time / double(slots)
                                        : double((own + other_ctas + slots - 1) / slots) * cta_time) +
                            1e-3 * double(n_ks) + 1e-4 * double(8 / R);
        if (cost < best_cost) {
          best_cost = cost;
          best.R = R;
          best.S = int(S);
          best.n_rg = int(n_rg);
          best.n_ks = int(n_ks);
          best.cr = cr;
          best.ctas = int(n_rgp * n_ks);
        }
      }
    }
  }
  return best;
}

// Sequences that share one pass over the weights (template parameter NSEQ of k_gemv).
int seqs_per_pass(int kind, size_t batch) {
  if (!kind_is_mma(kind) || batch <= 1) return 1;
  const int n = batch == 2 ? 2 : batch <= 4 ? 4 : 8;
  return n < max_seqs_per_pass(kind) ? n : max_seqs_per_pass(kind);
}

// Plans every job of a launch and fills the job descriptors (scratch regions are carved out of
// the context's scratch buffer, which is grown here when the stream is not capturing).
int prepare_jobs(lmb_ctx *ctx, int kind, const LinearArgs *args, int njobs, Job *jobs, int *ctas_out, int *s_max_out,
                 std::vector<int2> *cta_map, bool allow_cluster, int *cluster_out) {
  const size_t batch = args[0].batch;
  const int nseq = seqs_per_pass(kind, batch);
  const size_t ny = (batch + size_t(nseq) - 1) / size_t(nseq);  // grid.y
  std::vector<Plan> plans(static_cast<size_t>(njobs));
  size_t scratch_need = 0, counter_need = 0;
  size_t total_rt = 0;
  for (int j = 0; j < njobs; ++j) total_rt += args[j].w->row_tiles;
  // One cluster size per launch: the job with the most rows chooses (clusters only for direct batch-1
  // launches whose CTAs convert their own activations), the others follow.
  int cluster = 0;
  if (allow_cluster && !cta_map && batch == 1 && !args[0].prep_in) {
    int big = 0;
    for (int j = 1; j < njobs; ++j)
      if (args[j].w->row_tiles > args[big].w->row_tiles) big = j;
    const Plan lead = make_plan(kind, args[big].w->row_tiles, args[big].w->bpr, ny, ctx->sm_count, total_rt - args[big].w->row_tiles, nseq,
                                args[big].next_prep != nullptr, -1);
    cluster = lead.cr * lead.n_ks;
    for (int j = 0; j < njobs && cluster; ++j)  // every job must be able to follow
      if (make_plan(kind, args[j].w->row_tiles, args[j].w->bpr, ny, ctx->sm_count, total_rt - args[j].w->row_tiles, nseq,
                    args[j].next_prep != nullptr, cluster).ctas == 0)
        cluster = 0;
  }
  *cluster_out = cluster;
  for (int j = 0; j < njobs; ++j) {
    const lmb_weight *w = args[j].w;
    const size_t others = total_rt - w->row_tiles;
    plans[size_t(j)] = make_plan(kind, w->row_tiles, w->bpr, ny, ctx->sm_count, others, nseq, args[j].next_prep != nullptr, cluster);
    static const bool print_plans = std::getenv("LMB_PLAN_PRINT") != nullptr;  // debugging: the work split of every launch
    if (print_plans)
      std::fprintf(stderr, "lmb plan: kind %d job %d/%d rows %zu blocks/row %zu batch %zu: R %d S %d K slices %d, row groups per cluster %d, %d CTAs\n",
                   kind, j, njobs, size_t(w->M), size_t(w->bpr), batch, plans[size_t(j)].R, plans[size_t(j)].S, plans[size_t(j)].n_ks,
                   plans[size_t(j)].cr, plans[size_t(j)].ctas);
    if (plans[size_t(j)].n_ks > 1 && !cluster) {
      scratch_need += batch * plans[size_t(j)].n_ks * w->row_tiles * TILE_ROWS;
      counter_need += ny * plans[size_t(j)].n_rg;
    }
  }
  if (scratch_need > ctx->scratch_floats || counter_need > ctx->n_counters) {
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    LMB_CUDA(cudaStreamIsCapturing(ctx->stream, &cs));
    if (cs != cudaStreamCaptureStatusNone) {
      set_last_error("split-K scratch too small while the stream is capturing; run the call once outside capture");
      return LMB_ERR_STATE;
    }
    LMB_CUDA(cudaStreamSynchronize(ctx->stream));
    int st = ensure_scratch(ctx, scratch_need, counter_need);
    if (st != LMB_OK) return st;
  }
  size_t scratch_off = 0, counter_off = 0;
  int ctas = 0, s_max = 1;
  for (int j = 0; j < njobs; ++j) {
    const lmb_weight *w = args[j].w;
    const Plan &pl = plans[size_t(j)];
    Job &jb = jobs[j];
    jb.tiles = w->d_tiles;
    jb.x = args[j].x;
    jb.y = args[j].y;
    jb.bias = args[j].bias;
    jb.x2 = args[j].x2;
    jb.residual = args[j].residual;
    jb.M = int(w->M);
    jb.mp = int(w->row_tiles * TILE_ROWS);
    jb.bpr = int(w->bpr);
    jb.row_tiles = int(w->row_tiles);
    jb.R = pl.R;
    jb.S = pl.S;
    jb.n_rg = pl.n_rg;
    jb.n_ks = pl.n_ks;
    jb.x_len = unsigned(args[j].x_len);
    jb.x_stride = unsigned(args[j].x_stride);
    jb.y_stride = unsigned(args[j].y_stride);
    jb.scratch = ctx->scratch + scratch_off;
    jb.counters = ctx->counters + counter_off;
    jb.next_prep = args[j].next_prep;
    jb.next_sumsq = args[j].next_sumsq;
    jb.next_w = args[j].next_w;
    jb.next_rotate = args[j].next_rotate ? 1 : 0;
#ifdef LMB_DEBUG_BOUNDS
    jb.tiles_bytes = w->bytes > g_bounds_shrink ? w->bytes - g_bounds_shrink : 0;
    jb.y_floats = (batch - 1) * args[j].y_stride + w->M;
    jb.scratch_floats = pl.n_ks > 1 && !cluster ? batch * size_t(pl.n_ks) * size_t(jb.mp) : 0;
#endif
    if (pl.n_ks > 1 && !cluster) {
      scratch_off += batch * pl.n_ks * jb.mp;
      counter_off += ny * pl.n_rg;
    }
    ctas += pl.ctas;
    jb.cta_end = ctas;
    s_max = pl.S > s_max ? pl.S : s_max;
  }
  if (cta_map) {
    // prepared groups: the jobs with the longest CTAs get the lowest block indices, so that
    // they start first and the short ones fill the tail of the launch
    std::vector<int> order(static_cast<size_t>(njobs));
    for (int j = 0; j < njobs; ++j) order[size_t(j)] = j;
    std::stable_sort(order.begin(), order.end(), [&](int a, int b) {
      const Plan &pa = plans[size_t(a)], &pb = plans[size_t(b)];
      return pa.R * pa.S > pb.R * pb.S;
    });
    int first = 0;
    for (int j : order) {
      for (int c = 0; c < plans[size_t(j)].ctas; ++c) cta_map->push_back(make_int2(j, first));
      first += plans[size_t(j)].ctas;
    }
  }
  *ctas_out = ctas;
  *s_max_out = s_max;
  return LMB_OK;
}

template <int KIND, int NSEQ> int launch_params(lmb_ctx *ctx, GemvParams &p, int ctas, int s_max, size_t batch) {
  p.batch = int(batch);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(unsigned(ctas), unsigned((batch + NSEQ - 1) / NSEQ));
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = size_t(s_max) * Unit<KIND>::FPB * sizeof(float) * NSEQ;
  cfg.stream = ctx->stream;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (ctx->pdl) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  if (NSEQ == 1 && p.cl_size > 1) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = unsigned(p.cl_size);
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = 1;
    ++na;
  } else {
    p.cl_size = 0;
  }
  cfg.attrs = attr;
  cfg.numAttrs = unsigned(na);
  p.dbg = timeline_slot(ctx);
  if constexpr (NSEQ == 1 && kind_is_mma(KIND)) {
    if (p.cl_size > 1) {
      LMB_CUDA(cudaLaunchKernelEx(&cfg, k_gemv<KIND, 1, true>, p));
      ctx->launches++;
      return LMB_OK;
    }
  }
  LMB_CUDA(cudaLaunchKernelEx(&cfg, k_gemv<KIND, NSEQ>, p));
  ctx->launches++;
  return LMB_OK;
}

template <int KIND> int launch_params_mma(lmb_ctx *ctx, GemvParams &p, int ctas, int s_max, size_t batch) {
  switch (seqs_per_pass(KIND, batch)) {
  case 1: return launch_params<KIND, 1>(ctx, p, ctas, s_max, batch);
  case 2: return launch_params<KIND, 2>(ctx, p, ctas, s_max, batch);
  case 4:
    if constexpr (max_seqs_per_pass(KIND) >= 4) return launch_params<KIND, 4>(ctx, p, ctas, s_max, batch);
    return LMB_ERR_STATE;
  default:
    if constexpr (max_seqs_per_pass(KIND) >= 8) return launch_params<KIND, 8>(ctx, p, ctas, s_max, batch);
    return LMB_ERR_STATE;
  }
}

int launch_params_kind(lmb_ctx *ctx, int kind, GemvParams &p, int ctas, int s_max, size_t batch) {
  switch (kind) {
  case LMB_TERNARY: return launch_params<LMB_TERNARY, 1>(ctx, p, ctas, s_max, batch);
  case LMB_BINARY: return launch_params<LMB_BINARY, 1>(ctx, p, ctas, s_max, batch);
  case LMB_INT2: return launch_params<LMB_INT2, 1>(ctx, p, ctas, s_max, batch);
  case LMB_INT3: return launch_params<LMB_INT3, 1>(ctx, p, ctas, s_max, batch);
  case LMB_INT8: return launch_params<LMB_INT8, 1>(ctx, p, ctas, s_max, batch);
  case LMB_INT4: return launch_params_mma<LMB_INT4>(ctx, p, ctas, s_max, batch);
  case DK_TERNARY_MMA: return launch_params_mma<DK_TERNARY_MMA>(ctx, p, ctas, s_max, batch);
  case DK_INT2_MMA: return launch_params_mma<DK_INT2_MMA>(ctx, p, ctas, s_max, batch);
  case DK_BINARY_MMA: return launch_params_mma<DK_BINARY_MMA>(ctx, p, ctas, s_max, batch);
  case LMB_INT5: return launch_params_mma<LMB_INT5>(ctx, p, ctas, s_max, batch);
  case LMB_INT6: return launch_params_mma<LMB_INT6>(ctx, p, ctas, s_max, batch);
  case DK_INT8_MMA: return launch_params_mma<DK_INT8_MMA>(ctx, p, ctas, s_max, batch);
  case DK_INT3_MMA: return launch_params_mma<DK_INT3_MMA>(ctx, p, ctas, s_max, batch);
  default: set_last_error("launch_gemv: kind has no device kernel"); return LMB_ERR_ARG;
  }
}

}  // namespace

template <int KIND> int configure_mma() {
  const int small = 64 * 1024, large = 100 * 1024;
  LMB_CUDA(cudaFuncSetAttribute(k_gemv<KIND, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, small));
  LMB_CUDA(cudaFuncSetAttribute(k_gemv<KIND, 1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, small));
  LMB_CUDA(cudaFuncSetAttribute(k_gemv<KIND, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, small));
  if constexpr (max_seqs_per_pass(KIND) >= 4)
    LMB_CUDA(cudaFuncSetAttribute(k_gemv<KIND, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, large));
  if constexpr (max_seqs_per_pass(KIND) >= 8)
    LMB_CUDA(cudaFuncSetAttribute(k_gemv<KIND, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, large));
  return LMB_OK;
}

int configure_gemv(lmb_ctx *ctx) {
  (void)ctx;
  const int bytes = 64 * 1024;
  LMB_CUDA(cudaFuncSetAttribute(k_gemv<LMB_TERNARY, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  LMB_CUDA(cudaFuncSetAttribute(k_gemv<LMB_BINARY, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  LMB_CUDA(cudaFuncSetAttribute(k_gemv<LMB_INT2, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  LMB_CUDA(cudaFuncSetAttribute(k_gemv<LMB_INT3, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  LMB_CUDA(cudaFuncSetAttribute(k_gemv<LMB_INT8, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  int st = configure_mma<LMB_INT4>();
  if (st == LMB_OK) st = configure_mma<DK_TERNARY_MMA>();
  if (st == LMB_OK) st = configure_mma<DK_INT2_MMA>();
  if (st == LMB_OK) st = configure_mma<DK_BINARY_MMA>();
  if (st == LMB_OK) st = configure_mma<LMB_INT5>();
  if (st == LMB_OK) st = configure_mma<LMB_INT6>();
  if (st == LMB_OK) st = configure_mma<DK_INT8_MMA>();
  if (st == LMB_OK) st = configure_mma<DK_INT3_MMA>();
  return st;
}

// See k_tp_sum_prepare.  h must be a multiple of 256; prep holds h / 256 records, sumsq h / 256 floats.
int launch_tp_sum_prepare(lmb_ctx *ctx, float *d_hidden, const float *d_w, bool rotate, uint32_t *prep, float *sumsq, size_t h) {
  if (!ctx->xchg.ready || h % BLK != 0 || h > ctx->xchg.cap) {
    set_last_error("launch_tp_sum_prepare: no exchange block, or hidden size not a multiple of 256 within its capacity");
    return LMB_ERR_STATE;
  }
  XchgHeader *hdr = static_cast<XchgHeader *>(ctx->xchg.local);
  const unsigned long long *data =
      reinterpret_cast<const unsigned long long *>(static_cast<const char *>(ctx->xchg.local) + XCHG_HEADER_BYTES);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(unsigned(h / BLK));
  cfg.blockDim = dim3(BLK);
  cfg.stream = ctx->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = ctx->pdl ? 1 : 0;
  LMB_CUDA(cudaLaunchKernelEx(&cfg, k_tp_sum_prepare, d_hidden, hdr, data, ctx->tp_size, unsigned(ctx->xchg.cap), d_w, rotate ? 1 : 0, prep,
                              sumsq, ctx->xchg.spin_limit));
  ctx->launches++;
  return LMB_OK;
}

// Up to MAX_JOBS independent GEMVs of one kind and one batch size in a single launch.
int launch_gemv(lmb_ctx *ctx, const LinearArgs *args, int njobs, bool rotate, int xmode, float eps) {
  if (njobs < 1 || njobs > MAX_JOBS) {
    set_last_error("launch_gemv: between 1 and 4 jobs per launch");
    return LMB_ERR_ARG;
  }
  const int kind = args[0].w->kind;
  for (int j = 1; j < njobs; ++j)
    if (args[j].w->kind != kind || args[j].batch != args[0].batch) {
      set_last_error("launch_gemv: jobs of one launch must share block kind and batch size");
      return LMB_ERR_ARG;
    }
  GemvParams p;
  p.njobs = njobs;
  p.rotate = rotate ? 1 : 0;
  p.xmode = xmode;
  p.eps = eps;
  p.jobs_dev = nullptr;
  p.cta_map = nullptr;
  p.peer.n = 0;
  if (args[0].to_peers) {
    if (njobs != 1 || !ctx->xchg.ready || args[0].batch * args[0].y_stride > ctx->xchg.cap) {
      set_last_error("launch_gemv: peer output needs one job, an opened exchange block and batch x rows within its capacity");
      return LMB_ERR_STATE;
    }
    p.peer.n = ctx->tp_size;
    p.peer.rank = ctx->tp_rank;
    p.peer.cap = unsigned(ctx->xchg.cap);
    XchgHeader *mine = static_cast<XchgHeader *>(ctx->xchg.local);
    p.peer.epoch = &mine->epoch;
    for (int r = 0; r < ctx->tp_size; ++r)
      p.peer.data[r] = reinterpret_cast<unsigned long long *>(static_cast<char *>(ctx->xchg.peer[r]) + XCHG_HEADER_BYTES);
  }
  int ctas = 0, s_max = 1;
  int cluster = 0;
  int st = prepare_jobs(ctx, kind, args, njobs, p.job, &ctas, &s_max, nullptr, true, &cluster);
  if (st != LMB_OK) return st;
  p.cl_size = cluster;
  p.prep_sumsq = nullptr;
  p.prep_sumsq_n = 0;
  if (args[0].prep_in) {  // the producing GEMV prepared the activations (batch 1)
    if (args[0].batch != 1 || !kind_is_mma(kind)) {
      set_last_error("launch_gemv: prepared activations need batch 1 and an integer tensor-core layout");
      return LMB_ERR_ARG;
    }
    p.prep = args[0].prep_in;
    p.prep_sumsq = args[0].prep_sumsq_in;
    p.prep_sumsq_n = args[0].prep_sumsq_n;
    return launch_params_kind(ctx, kind, p, ctas, s_max, 1);
  }
  // Batches of three or more sequences whose jobs read one input: convert the activations once
  // for the whole launch instead of once per CTA.
  p.prep = nullptr;
  bool shared_x = seqs_per_pass(kind, args[0].batch) >= 4;
  for (int j = 1; j < njobs && shared_x; ++j)
    shared_x = args[j].x == args[0].x && args[j].x2 == args[0].x2 && args[j].x_len == args[0].x_len &&
               args[j].x_stride == args[0].x_stride && args[j].w->bpr == args[0].w->bpr;
  if (shared_x) {
    const size_t bpr = args[0].w->bpr, need = args[0].batch * bpr;
    if (need > ctx->xprep_blocks) {
      cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
      LMB_CUDA(cudaStreamIsCapturing(ctx->stream, &cs));
      if (cs == cudaStreamCaptureStatusNone) {
        LMB_CUDA(cudaStreamSynchronize(ctx->stream));
        if (ctx->xprep) LMB_CUDA(cudaFree(ctx->xprep));
        ctx->xprep = nullptr;
        ctx->xprep_blocks = 0;
        LMB_CUDA(cudaMalloc(&ctx->xprep, need * PREP_WORDS * sizeof(uint32_t)));
        ctx->xprep_blocks = need;
        ctx->scratch_gen++;
      }
    }
    if (need <= ctx->xprep_blocks) {
      dim3 grid(unsigned((bpr + WARPS - 1) / WARPS), unsigned(args[0].batch));
      k_prepare_x<<<grid, THREADS, 0, ctx->stream>>>(args[0].x, args[0].x2, unsigned(args[0].x_len), unsigned(args[0].x_stride),
                                                     int(bpr), xmode, rotate ? 1 : 0, eps, ctx->xprep);
      ctx->launches++;
      LMB_CUDA(cudaGetLastError());
      p.prep = ctx->xprep;
    }
  }
  return launch_params_kind(ctx, kind, p, ctas, s_max, args[0].batch);
}

}  // namespace lmb

// ---- prepared groups: any number of independent batch-1 GEMVs of one kind in one launch ---------
struct lmb_group {
  int kind = 0, ctas = 0, s_max = 1, njobs = 0;
  bool rotate = false;
  // the job table holds pointers into the context's split-K scratch: it is rebuilt when the
  // scratch has been reallocated since (lmb_ctx::scratch_gen)
  uint64_t scratch_gen = 0;
  std::vector<lmb::LinearArgs> args;
  size_t map_entries = 0;
  lmb::Job *d_jobs = nullptr;
  int2 *d_map = nullptr;
  // host-buffer form (lmb_group_create_host): the group owns contiguous device and pinned
  // host buffers for all inputs and all outputs
  float *d_io = nullptr, *h_io = nullptr;
  size_t in_floats = 0, out_floats = 0;
  std::vector<size_t> in_off, out_off, in_len, out_len;
};

extern "C" {

int lmb_group_create(lmb_ctx *ctx, size_t n, const lmb_weight *const *ws, const float *const *d_xs, float *const *d_ys,
                     unsigned flags, lmb_group **out) {
  using namespace lmb;
  LMB_REQUIRE(ctx && ws && d_xs && d_ys && out && n > 0, "lmb_group_create: null argument");
  *out = nullptr;
  std::vector<LinearArgs> args(n);
  for (size_t i = 0; i < n; ++i) {
    LMB_REQUIRE(ws[i] && d_xs[i] && d_ys[i], "lmb_group_create: null entry");
    LMB_REQUIRE(ws[i]->kind == ws[0]->kind, "lmb_group_create: all weights of a group must share a block kind");
    args[i] = LinearArgs{ws[i], nullptr, d_xs[i], ws[i]->K, ws[i]->K, d_ys[i], ws[i]->M, 1, false, nullptr, nullptr};
  }
  const int kind = ws[0]->kind;
  const bool auto_rot = (kind == LMB_TERNARY || kind == DK_TERNARY_MMA || kind == LMB_BINARY || kind == LMB_INT2 ||
                         kind == DK_INT2_MMA || kind == DK_BINARY_MMA);
  std::vector<Job> jobs(n);
  std::vector<int2> map;
  lmb_group *g = new (std::nothrow) lmb_group();
  if (!g) return LMB_ERR_ALLOC;
  g->kind = kind;
  g->njobs = int(n);
  g->rotate = (flags & LMB_ROTATE) || ((flags & LMB_AUTO_ROTATE) && auto_rot);
  int no_cluster = 0;
  int st = prepare_jobs(ctx, kind, args.data(), int(n), jobs.data(), &g->ctas, &g->s_max, &map, false, &no_cluster);
  g->scratch_gen = ctx->scratch_gen;
  g->args = args;
  g->map_entries = map.size();
  if (st == LMB_OK) {
    cudaError_t e = cudaMalloc(&g->d_jobs, n * sizeof(Job));
    if (e == cudaSuccess) e = cudaMalloc(&g->d_map, map.size() * sizeof(int2));
    if (e == cudaSuccess) e = cudaMemcpy(g->d_jobs, jobs.data(), n * sizeof(Job), cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemcpy(g->d_map, map.data(), map.size() * sizeof(int2), cudaMemcpyHostToDevice);
    if (e != cudaSuccess) st = cuda_fail(e, "lmb_group_create");
  }
  if (st != LMB_OK) {
    lmb_group_destroy(g);
    return st;
  }
  *out = g;
  return LMB_OK;
}

int lmb_group_launch(lmb_ctx *ctx, lmb_group *g) {
  using namespace lmb;
  LMB_REQUIRE(ctx && g, "lmb_group_launch: null argument");
  if (g->scratch_gen != ctx->scratch_gen) {
    // same shapes, same plan: only the scratch addresses inside the job table change
    std::vector<Job> jobs(g->args.size());
    std::vector<int2> map;
    int ctas = 0, s_max = 1;
    int no_cluster = 0;
    int st = prepare_jobs(ctx, g->kind, g->args.data(), g->njobs, jobs.data(), &ctas, &s_max, &map, false, &no_cluster);
    if (st != LMB_OK) return st;
    if (ctas != g->ctas || map.size() != g->map_entries) {
      set_last_error("lmb_group_launch: the group's plan changed; create the group again");
      return LMB_ERR_STATE;
    }
    LMB_CUDA(cudaStreamSynchronize(ctx->stream));
    LMB_CUDA(cudaMemcpy(g->d_jobs, jobs.data(), jobs.size() * sizeof(Job), cudaMemcpyHostToDevice));
    LMB_CUDA(cudaMemcpy(g->d_map, map.data(), map.size() * sizeof(int2), cudaMemcpyHostToDevice));
    g->s_max = s_max;
    g->scratch_gen = ctx->scratch_gen;
  }
  GemvParams p;
  p.njobs = g->njobs;
  p.rotate = g->rotate ? 1 : 0;
  p.xmode = XMODE_PLAIN;
  p.eps = 0.0f;
  p.jobs_dev = g->d_jobs;
  p.cta_map = g->d_map;
  p.peer.n = 0;
  p.prep = nullptr;
  p.prep_sumsq = nullptr;
  p.prep_sumsq_n = 0;
  p.cl_size = 0;
  return launch_params_kind(ctx, g->kind, p, g->ctas, g->s_max, 1);
}

int lmb_group_destroy(lmb_group *g) {
  if (!g) return LMB_OK;
  if (g->d_jobs) cudaFree(g->d_jobs);
  if (g->d_map) cudaFree(g->d_map);
  if (g->d_io) cudaFree(g->d_io);
  if (g->h_io) cudaFreeHost(g->h_io);
  delete g;
  return LMB_OK;
}

int lmb_group_create_host(lmb_ctx *ctx, size_t n, const lmb_weight *const *ws, unsigned flags, lmb_group **out) {
  using namespace lmb;
  LMB_REQUIRE(ctx && ws && out && n > 0, "lmb_group_create_host: null argument");
  *out = nullptr;
  std::vector<size_t> in_off(n), out_off(n), in_len(n), out_len(n);
  size_t in_f = 0, out_f = 0;
  for (size_t i = 0; i < n; ++i) {
    LMB_REQUIRE(ws[i], "lmb_group_create_host: null entry");
    in_off[i] = in_f;
    in_len[i] = ws[i]->K;
    in_f += (ws[i]->K + 3) / 4 * 4;  // keeps every input 16-byte aligned
  }
  for (size_t i = 0; i < n; ++i) {
    out_off[i] = in_f + out_f;
    out_len[i] = ws[i]->M;
    out_f += (ws[i]->M + 3) / 4 * 4;
  }
  float *d_io = nullptr, *h_io = nullptr;
  LMB_CUDA(cudaMalloc(&d_io, (in_f + out_f) * sizeof(float)));
  cudaError_t e = cudaMallocHost(&h_io, (in_f + out_f) * sizeof(float));
  if (e != cudaSuccess) {
    cudaFree(d_io);
    return cuda_fail(e, "lmb_group_create_host");
  }
  std::vector<const float *> xs(n);
  std::vector<float *> ys(n);
  for (size_t i = 0; i < n; ++i) {
    xs[i] = d_io + in_off[i];
    ys[i] = d_io + out_off[i];
  }
  int st = lmb_group_create(ctx, n, ws, xs.data(), ys.data(), flags, out);
  if (st != LMB_OK) {
    cudaFree(d_io);
    cudaFreeHost(h_io);
    return st;
  }
  lmb_group *g = *out;
  g->d_io = d_io;
  g->h_io = h_io;
  g->in_floats = in_f;
  g->out_floats = out_f;
  g->in_off = in_off;
  g->out_off = out_off;
  g->in_len = in_len;
  g->out_len = out_len;
  return LMB_OK;
}

int lmb_group_run_host(lmb_ctx *ctx, lmb_group *g, const float *const *inputs, float *const *outputs) {
  using namespace lmb;
  LMB_REQUIRE(ctx && g && inputs && outputs, "lmb_group_run_host: null argument");
  LMB_REQUIRE(g->d_io, "lmb_group_run_host: the group was not made by lmb_group_create_host");
  const size_t n = size_t(g->njobs);
  // inputs that already live in the group's pinned buffer (lmb_group_host_io) need no staging copy
  for (size_t i = 0; i < n; ++i)
    if (inputs[i] != g->h_io + g->in_off[i]) std::memcpy(g->h_io + g->in_off[i], inputs[i], g->in_len[i] * sizeof(float));
  LMB_CUDA(cudaMemcpyAsync(g->d_io, g->h_io, g->in_floats * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
  int st = lmb_group_launch(ctx, g);
  if (st != LMB_OK) return st;
  LMB_CUDA(cudaMemcpyAsync(g->h_io + g->in_floats, g->d_io + g->in_floats, g->out_floats * sizeof(float),
                           cudaMemcpyDeviceToHost, ctx->stream));
  LMB_CUDA(cudaStreamSynchronize(ctx->stream));
  for (size_t i = 0; i < n; ++i)
    if (outputs[i] != g->h_io + g->out_off[i]) std::memcpy(outputs[i], g->h_io + g->out_off[i], g->out_len[i] * sizeof(float));
  return LMB_OK;
}

int lmb_debug_plan(int kind, size_t M, size_t K, size_t batch, size_t other_rows, int sm_count, int out5[5]) {
  using namespace lmb;
  LMB_REQUIRE(kind_valid(kind) && M > 0 && K > 0 && batch > 0 && sm_count > 0 && out5, "lmb_debug_plan: bad argument");
  const int nseq = seqs_per_pass(kind, batch);
  const size_t ny = (batch + size_t(nseq) - 1) / size_t(nseq);
  const Plan pl = make_plan(kind, (M + TILE_ROWS - 1) / TILE_ROWS, (K + BLK - 1) / BLK, ny, sm_count,
                            (other_rows + TILE_ROWS - 1) / TILE_ROWS, nseq);
  out5[0] = pl.R;
  out5[1] = pl.S;
  out5[2] = pl.n_rg;
  out5[3] = pl.n_ks;
  out5[4] = nseq;
  return LMB_OK;
}

int lmb_debug_force_plan(int R, int n_ks, int cr) {
  using namespace lmb;
  g_plan_force.on = R > 0;
  g_plan_force.R = R;
  g_plan_force.n_ks = n_ks;
  g_plan_force.cr = cr;
  return LMB_OK;
}

int lmb_debug_plan_weight(const lmb_weight *w, int sm_count, int out5[5]) {
  using namespace lmb;
  LMB_REQUIRE(w && out5 && sm_count > 0, "lmb_debug_plan_weight: bad argument");
  return lmb_debug_plan(w->kind, w->M, w->K, 1, 0, sm_count, out5);
}

int lmb_group_host_io(lmb_group *g, size_t i, float **h_in, float **h_out) {
  using namespace lmb;
  LMB_REQUIRE(g && g->d_io && i < size_t(g->njobs), "lmb_group_host_io: not a host group, or index out of range");
  if (h_in) *h_in = g->h_io + g->in_off[i];
  if (h_out) *h_out = g->h_io + g->out_off[i];
  return LMB_OK;
}

// ---- lmb_linear_static_scratch ---------------------------------------------------------------------
// Split-K scratch that belongs to the library image instead of the heap: every GPU that loads the
// library carries these two arrays until the process exits.
#define LMB_STATIC_SCRATCH_FLOATS (size_t(1) << 17)  /* 512 KiB of partial sums */
#define LMB_STATIC_COUNTERS 1024                     /* row-group arrival counters */
static __device__ __align__(256) float g_static_scratch[LMB_STATIC_SCRATCH_FLOATS];
static __device__ __align__(256) unsigned g_static_counters[LMB_STATIC_COUNTERS];

namespace {
struct StaticSetup {
  bool ready = false;
  float *scratch = nullptr;      // device address of g_static_scratch on this device
  unsigned *counters = nullptr;  // device address of g_static_counters on this device
  int sm_count = 0;
};
StaticSetup g_static_setup[64];  // per device ordinal
std::mutex g_static_setup_mu;    // two host threads may make their first call at once
}  // namespace

int lmb_linear_static_scratch(const lmb_weight *w, const float *d_bias, const float *d_x, size_t x_len, float *d_y,
                              unsigned flags, void *cuda_stream) {
  using namespace lmb;
  LMB_REQUIRE(w && d_x && d_y, "lmb_linear_static_scratch: null argument");
  LMB_REQUIRE(x_len <= w->bpr * size_t(BLK), "lmb_linear_static_scratch: x_len exceeds the padded input width");
  int dev = -1;
  LMB_CUDA(cudaGetDevice(&dev));
  LMB_REQUIRE(dev == w->device, "lmb_linear_static_scratch: the weight's device is not the current device");
  LMB_REQUIRE(dev >= 0 && dev < 64, "lmb_linear_static_scratch: device ordinal beyond 63");
  StaticSetup &su = g_static_setup[dev];
  {
  std::lock_guard<std::mutex> setup_lock(g_static_setup_mu);  // first calls from several host threads set up once
  if (!su.ready) {
    // Once per device, with that device current.  In host code the array names are only handles:
    // the device addresses the kernel needs come from cudaGetSymbolAddress.
    void *ps = nullptr, *pc = nullptr;
    LMB_CUDA(cudaGetSymbolAddress(&ps, g_static_scratch));
    LMB_CUDA(cudaGetSymbolAddress(&pc, g_static_counters));
    LMB_CUDA(cudaDeviceGetAttribute(&su.sm_count, cudaDevAttrMultiProcessorCount, dev));
    lmb_ctx probe;  // only carries the device for configure_gemv; nothing is allocated
    probe.device = dev;
    int st = configure_gemv(&probe);
    if (st != LMB_OK) return st;
    su.scratch = static_cast<float *>(ps);
    su.counters = static_cast<unsigned *>(pc);
    su.ready = true;
  }
  }
  const int kind = w->kind;
  const Plan pl = make_plan(kind, w->row_tiles, w->bpr, 1, su.sm_count);
  const size_t mp = w->row_tiles * TILE_ROWS;
  if (pl.n_ks > 1 && (size_t(pl.n_ks) * mp > LMB_STATIC_SCRATCH_FLOATS || size_t(pl.n_rg) > LMB_STATIC_COUNTERS)) {
    set_last_error("lmb_linear_static_scratch: this shape needs more than the built-in 512 KiB of split-K scratch "
                   "(K slices x padded rows > 131072 floats, or more than 1024 row groups); use lmb_linear");
    return LMB_ERR_LIMIT;
  }
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  // The array keeps whatever the last call left.  Partial sums are fully overwritten before they
  // are read; the counters must start at zero, so they are cleared on the caller's stream.
  if (pl.n_ks > 1) LMB_CUDA(cudaMemsetAsync(su.counters, 0, size_t(pl.n_rg) * sizeof(unsigned), stream));
  GemvParams p;
  p.njobs = 1;
  p.xmode = XMODE_PLAIN;
  p.eps = 0.0f;
  const bool auto_rot = (kind == LMB_TERNARY || kind == DK_TERNARY_MMA || kind == LMB_BINARY || kind == LMB_INT2 ||
                         kind == DK_INT2_MMA || kind == DK_BINARY_MMA);
  p.rotate = ((flags & LMB_ROTATE) || ((flags & LMB_AUTO_ROTATE) && auto_rot)) ? 1 : 0;
  p.jobs_dev = nullptr;
  p.cta_map = nullptr;
  p.peer.n = 0;
  p.prep = nullptr;
  p.prep_sumsq = nullptr;
  p.prep_sumsq_n = 0;
  p.cl_size = 0;
  Job &jb = p.job[0];
  jb.tiles = w->d_tiles;
  jb.x = d_x;
  jb.y = d_y;
  jb.bias = d_bias;
  jb.x2 = nullptr;
  jb.residual = nullptr;
  jb.next_prep = nullptr;
  jb.next_sumsq = nullptr;
  jb.next_w = nullptr;
  jb.next_rotate = 0;
  jb.scratch = su.scratch;
  jb.counters = su.counters;
  jb.M = int(w->M);
  jb.mp = int(mp);
  jb.bpr = int(w->bpr);
  jb.row_tiles = int(w->row_tiles);
  jb.R = pl.R;
  jb.S = pl.S;
  jb.n_rg = pl.n_rg;
  jb.n_ks = pl.n_ks;
  jb.cta_end = pl.ctas;
  jb.x_len = unsigned(x_len);
  jb.x_stride = unsigned(x_len);
  jb.y_stride = unsigned(w->M);
#ifdef LMB_DEBUG_BOUNDS
  jb.tiles_bytes = w->bytes;
  jb.y_floats = w->M;
  jb.scratch_floats = LMB_STATIC_SCRATCH_FLOATS;
#endif
  lmb_ctx launch_ctx;  // plain launch on the caller's stream, no programmatic dependent launch
  launch_ctx.device = dev;
  launch_ctx.stream = stream;
  launch_ctx.pdl = false;
  return launch_params_kind(&launch_ctx, kind, p, pl.ctas, pl.S, 1);
}

}  // extern "C"

namespace lmb {

int launch_debug_luts(lmb_ctx *ctx, const float *d_x, size_t x_len, bool rotate, float *d_out) {
  const int nblocks = int((x_len + BLK - 1) / BLK);
  k_debug_luts<<<(nblocks + WARPS - 1) / WARPS, THREADS, 0, ctx->stream>>>(d_x, x_len, nblocks, rotate ? 1 : 0, d_out);
  ctx->launches++;
  LMB_CUDA(cudaGetLastError());
  return LMB_OK;
}

}  // namespace lmb
