// One batch-1 decode step (embedding row and every layer of Model::forward, src/model.cpp:58-433)
// as ONE persistent kernel.
//
// The launch-per-projection step spends most of its time between kernels: five dependent
// launches per layer, each with its own ramp, activation prologue and tail, while the bytes a
// launch moves are worth a few microseconds of HBM time.  Here a grid of exactly (resident CTAs
// per SM) x (SMs) CTAs stays on the GPU for the whole step and walks a list of phases prepared
// on the host:
//     embedding row | per layer: q/k/v GEMVs | attention | o GEMV | gate/up GEMVs | down GEMV
// (tensor parallel: o and down deliver their partial vectors to every rank's exchange block and a
// short reduce phase after each adds the ranks' vectors in rank order).  Phases are ordered by
// arrival counters in device memory; every wait is bounded and on expiry records the phase in a
// status word and ends the kernel (no trap, no endless spin).  Design points:
//   * weights never depend on a predecessor, so every warp issues the loads of its first
//     row-blocks of the NEXT phase into its register ring BEFORE it waits for the current phase
//     to finish everywhere (about 140 KB per SM in flight across every dependency);
//   * the work of a GEMV phase is cut by SM, not by CTA slot: K slices x row groups = grid size
//     exactly, row groups differ by at most one row-tile, and the warps of a CTA split its
//     (row-tile, block) units evenly;
//   * the activations of a K slice arrive by ONE bulk asynchronous copy (cp.async.bulk + mbarrier)
//     and are converted in place from shared memory; attention fetches a slice's keys and values
//     the same way;
//   * RMSNorm statistics are computed once by the phase that produces the hidden state (one
//     partial sum of squares per row group) instead of by every CTA of the consuming phase.
// Measured on B200 the step is not faster than the launch-per-projection step on one GPU (the
// spread of the CTAs' arrivals at each wait, 6 to 14 us, costs more than a kernel boundary under
// programmatic dependent launch), so models take this path only on request.
// The evaluation units (weights x fixed-point digits on the integer MMA) are those of the
// one-GEMV kernels; only the integer tensor-core layouts take this path, and only models whose
// seven projections per layer share one layout.  Cooperative launch guarantees co-residency.
#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <new>
#include <vector>

#include "decode_device.cuh"
#include "gemv_units.cuh"
#include "model.cuh"

namespace lmb {

namespace {

constexpr int PS_THREADS = 256;
constexpr int PS_WARPS = PS_THREADS / 32;
constexpr int PS_MAX_JOBS = 3;
constexpr int PS_S_MAX = 48;     // 256-column blocks of activations a CTA prepares (1 KiB of digits each)
constexpr int PS_MAX_SEG = 160;  // (row-tile, contributing warp) partial rows a CTA can hold (128 B each)
constexpr int PS_NRT_MAX = 80;   // row-tiles per CTA and phase
// digits of the CTA's K slice, then either the staged second operand of the prologue (norm weight
// or `up` slice, as large as the digits) or, later, the warps' partial rows
constexpr size_t PS_SMEM = size_t(PS_S_MAX) * 1024 * 2;
static_assert(size_t(PS_MAX_SEG) * 128 <= size_t(PS_S_MAX) * 1024, "partial rows must fit behind the digits");

enum { PH_EMBED = 0, PH_GEMV = 1, PH_ATTN = 2, PH_REDUCE = 3 };

struct PsJob {
  const uint8_t *tiles;
  float *y;
  int M, rt_begin;  // rows; first row-tile in the phase's concatenated row-tile space
};

struct PsPhase {
  int type;
  // PH_GEMV: up to three projections that read the same input
  int njobs, rt_total, bpr, n_ks, n_rg;
  int xmode, rotate, to_peers, xchg_seq;
  unsigned x_len;
  int n_sumsq_in;
  PsJob job[PS_MAX_JOBS];
  const float *x, *x2, *residual, *sumsq_in;
  float *sumsq_out;  // one partial sum of squares of the output per row group (PH_GEMV), per CTA (PH_EMBED, PH_REDUCE)
  // PH_ATTN
  AttnArgs at;
  RopeDims rd;
  int attn_per;  // 0: one item per (query head, split); 2 or 4: group form, head_dim / 32
  // PH_EMBED (tokens, embed_*) and PH_REDUCE (hidden += sum over ranks of exchange xchg_seq)
  const int *tokens;
  const uint8_t *embed_tiles;
  int embed_kind;
  unsigned embed_bpr, vocab, h;
  float embed_scale;  // 1, or sqrt(hidden size) for gemma-type models (model.cpp:255-260)
  float *hidden;
};

struct PsParams {
  const PsPhase *phases;
  int n_phases, n_xchg;
  unsigned *barrier;   // [n_phases] arrival counters, zeroed before the launch
  unsigned *counters;  // [grid] split-K arrival counters, zeroed before the launch
  float *scratch;      // split-K partial sums [K slice][row of the phase]
  unsigned *status;    // 0, or 1 + the phase whose wait expired
  unsigned spin_limit, extra_arrivals;
  float eps;
  PeerOut peer;  // peer.n > 0: tensor parallel
  XchgHeader *hdr;
  const unsigned long long *xchg_data;  // this rank's exchange block
  // optional (null: off): nanosecond timestamps of CTA 0 and of the last CTA at five points of every
  // phase -- descriptor read, dependency met, activations prepared, main loop done, phase done --
  // then per phase the last arrival and the complement of the first arrival over all CTAs
  unsigned long long *timeline;  // [2][n_phases][5] + [n_phases][2]
};

__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned *p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned ld_volatile_u32(const unsigned *p) {
  unsigned v;
  asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// This CTA has finished phase `ph`: one release-ordered reduction (the CTA's global writes, ordered
// before it by the block barrier, become visible to whoever observes the count with an acquire).
__device__ __forceinline__ void ps_arrive(const PsParams &p, int ph) {
  __syncthreads();
  if (threadIdx.x == 0) {
    if (p.timeline) {
      const unsigned long long now = global_ns();
      unsigned long long *skew = p.timeline + size_t(2) * p.n_phases * 5 + size_t(ph) * 2;
      atomicMax(skew, now);       // last arrival
      atomicMax(skew + 1, ~now);  // first arrival, complemented
    }
    asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(p.barrier + ph) : "memory");
  }
}

// Waits (bounded) until every CTA has finished phase `ph`.  False when this wait, or any wait
// anywhere before it, ran out: the caller leaves the kernel.
__device__ __forceinline__ bool ps_wait(const PsParams &p, int ph, int *flag) {
  if (threadIdx.x == 0) {
    const unsigned target = gridDim.x + p.extra_arrivals;
    unsigned spins = 0;
    int ok = 1;
    while (ld_acquire_u32(p.barrier + ph) < target) {
      ++spins;
      if ((spins & 63u) == 0u && ld_volatile_u32(p.status) != 0u) {  // somebody else gave up
        ok = 0;
        break;
      }
      if (spins > p.spin_limit) {
        atomicCAS(p.status, 0u, unsigned(ph) + 1u);
        ok = 0;
        break;
      }
    }
    *flag = ok;
  }
  __syncthreads();
  const bool ok = *flag != 0;
  __syncthreads();
  return ok;
}

// load_x8 for vectors written earlier in the same launch: around the (incoherent) L1
__device__ __forceinline__ void load_x8_cg(const float *x, size_t x_len, size_t b, int lane, float v[8]) {
  const size_t i0 = b * 256 + size_t(lane) * 8;
  if (i0 + 8 <= x_len && ((reinterpret_cast<uintptr_t>(x + i0) & 15) == 0)) {
    const float4 a = __ldcg(reinterpret_cast<const float4 *>(x + i0));
    const float4 c = __ldcg(reinterpret_cast<const float4 *>(x + i0 + 4));
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    v[4] = c.x; v[5] = c.y; v[6] = c.z; v[7] = c.w;
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = (i0 + j < x_len) ? __ldcg(x + i0 + j) : 0.0f;
  }
}

__device__ __forceinline__ int job_of(const PsPhase &P, int vrt) {
  int j = 0;
  if (P.njobs > 1 && vrt >= P.job[1].rt_begin) j = 1;
  if (P.njobs > 2 && vrt >= P.job[2].rt_begin) j = 2;
  return j;
}

// warp that evaluates unit u when N units are dealt to 8 warps as [w*N/8, (w+1)*N/8)
__device__ __forceinline__ int warp_of_unit(int u, int N) { return ((u + 1) * PS_WARPS - 1) / N; }

template <int KIND>
__global__ void __launch_bounds__(PS_THREADS, 2) k_decode_step(const __grid_constant__ PsParams p) {
  using U = Unit<KIND>;
  static_assert(kind_is_mma(KIND), "the persistent step runs the integer tensor-core layouts only");
  constexpr int FPB = U::FPB;
  constexpr size_t TB = tile_bytes(KIND);
  constexpr int NSLOT = prefetch_depth(KIND) + 1;
  extern __shared__ __align__(1024) float smem[];
  __shared__ PsPhase P;
  __shared__ float xsum[64];
  __shared__ __align__(16) int xaux[64 * 4];
  __shared__ float red[32];
  __shared__ int flag;
  __shared__ __align__(8) uint64_t bar;  // completion of the attention phase's bulk copies
  unsigned bar_parity = 0;
  if (threadIdx.x == 0) mbar_init(&bar, 1);
  __syncthreads();
  const int G = int(gridDim.x), c = int(blockIdx.x);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, t = threadIdx.x;
  const unsigned epoch0 = p.peer.n ? ld_volatile_u32(&p.hdr->epoch) : 0u;
  unsigned long long *tl = nullptr;
  if (p.timeline && t == 0 && (c == 0 || c == G - 1)) tl = p.timeline + size_t(c == 0 ? 0 : 1) * p.n_phases * 5;
  auto stamp = [&](int ph, int k) {
    if (tl) tl[ph * 5 + k] = global_ns();
  };

  for (int ph = 0; ph < p.n_phases; ++ph) {
    stamp(ph, 0);
    {  // the phase descriptor: constant for the launch, so it can be read ahead of the dependency
      const uint32_t *src = reinterpret_cast<const uint32_t *>(p.phases + ph);
      uint32_t *dst = reinterpret_cast<uint32_t *>(&P);
      for (int i = t; i < int(sizeof(PsPhase) / 4); i += PS_THREADS) dst[i] = __ldg(src + i);
    }
    __syncthreads();

    if (P.type == PH_GEMV) {
      // ---- this CTA's share: K slice ks, row-tiles [rt_a, rt_b) of the concatenated jobs -----------------
      const int ks = c % P.n_ks, rg = c / P.n_ks;
      const int rt_a = int((long long)(rg)*P.rt_total / P.n_rg), rt_b = int((long long)(rg + 1) * P.rt_total / P.n_rg);
      const int nrt = rg < P.n_rg ? rt_b - rt_a : 0;
      const int b0 = ks * P.bpr / P.n_ks, S = (ks + 1) * P.bpr / P.n_ks - b0;
      const int N = nrt * S;
      const int u0 = warp * N / PS_WARPS, u1 = (warp + 1) * N / PS_WARPS;
      const int seg_slots = N > 0 ? min(PS_WARPS, (S * PS_WARPS + N - 1) / N + 1) : 1;
      float *seg = smem + size_t(S) * FPB;

      auto tile_ptr = [&](int rtl, int b) {
        const int vrt = rt_a + rtl, j = job_of(P, vrt);
        return P.job[j].tiles + (size_t(vrt - P.job[j].rt_begin) * P.bpr + b0 + b) * TB;
      };
      // load cursor (runs NSLOT units ahead of the evaluation)
      int l_rtl = 0, l_b = 0;
      const uint8_t *l_ptr = nullptr;
      if (u0 < u1) {
        l_rtl = u0 / S;
        l_b = u0 - l_rtl * S;
        l_ptr = tile_ptr(l_rtl, l_b);
      }
      auto advance_load = [&]() {
        l_ptr += TB;
        if (++l_b == S) {
          l_b = 0;
          ++l_rtl;
          if (l_rtl < nrt) l_ptr = tile_ptr(l_rtl, 0);
        }
      };
      U slot[NSLOT];
#pragma unroll
      for (int sl = 0; sl < NSLOT; ++sl)
        if (u0 + sl < u1) {
          slot[sl].load(l_ptr, lane);
          advance_load();
        }

      // ---- the activations exist once every CTA has finished the previous phase --------------------------
      if (ph > 0 && !ps_wait(p, ph - 1, &flag)) return;
      stamp(ph, 1);

      // Activations of the K slice.  Whole 256-blocks (every decoder shape): ONE bulk asynchronous
      // copy brings the slice into shared memory (a second one the norm weights or the `up` slice)
      // while the RMSNorm statistics are summed; each warp then converts its blocks in place, from
      // shared memory, instead of paying a global-memory round trip per block.
      const bool staged = (P.x_len % BLK == 0) && S > 0;
      float *stage2 = smem + size_t(S) * FPB;
      if (staged && t == 0) {
        asm volatile("fence.proxy.async;" ::: "memory");  // the producers' writes, acquired above, precede the asynchronous reads
        const unsigned bytes = unsigned(S) * BLK * 4u;
        mbar_arrive_expect_tx(&bar, P.xmode == XMODE_PLAIN ? bytes : 2u * bytes);
        bulk_copy_g2s(smem, P.x + size_t(b0) * BLK, bytes, &bar);
        if (P.xmode != XMODE_PLAIN) bulk_copy_g2s(stage2, P.x2 + size_t(b0) * BLK, bytes, &bar);
      }
      float inv_rms = 1.0f;
      if (P.xmode == XMODE_RMSNORM) {  // src/layers/norm.cpp:18-34, the sum of squares from the producer's partials
        float ss = 0.0f;
        for (int i = t; i < P.n_sumsq_in; i += PS_THREADS) ss += __ldcg(P.sumsq_in + i);
        ss = block_sum(ss, red);
        inv_rms = 1.0f / sqrtf(ss / float(P.x_len) + p.eps);
      }
      if (staged) {  // bounded wait for the copies
        unsigned spins = 0;
        bool ok = true;
        while (!mbar_try_wait(&bar, bar_parity)) {
          if (++spins > p.spin_limit) {
            ok = false;
            break;
          }
        }
        bar_parity ^= 1u;
        if (!ok) atomicCAS(p.status, 0u, unsigned(ph) + 1u);
        if (__syncthreads_or(!ok)) return;
      }
      for (int it = warp; it < S; it += PS_WARPS) {
        float v[8], w8[8];
        if (staged) {
          const float4 a0 = reinterpret_cast<const float4 *>(smem + size_t(it) * FPB)[2 * lane];
          const float4 a1 = reinterpret_cast<const float4 *>(smem + size_t(it) * FPB)[2 * lane + 1];
          v[0] = a0.x; v[1] = a0.y; v[2] = a0.z; v[3] = a0.w; v[4] = a1.x; v[5] = a1.y; v[6] = a1.z; v[7] = a1.w;
          if (P.xmode != XMODE_PLAIN) {
            const float4 c0 = reinterpret_cast<const float4 *>(stage2 + size_t(it) * BLK)[2 * lane];
            const float4 c1 = reinterpret_cast<const float4 *>(stage2 + size_t(it) * BLK)[2 * lane + 1];
            w8[0] = c0.x; w8[1] = c0.y; w8[2] = c0.z; w8[3] = c0.w; w8[4] = c1.x; w8[5] = c1.y; w8[6] = c1.z; w8[7] = c1.w;
          }
          __syncwarp();  // the block is overwritten with its digits below
        } else {
          load_x8_cg(P.x, P.x_len, size_t(b0 + it), lane, v);
          if (P.xmode == XMODE_RMSNORM) load_x8(P.x2, P.x_len, size_t(b0 + it), lane, w8);
          else if (P.xmode != XMODE_PLAIN) load_x8_cg(P.x2, P.x_len, size_t(b0 + it), lane, w8);
        }
        if (P.xmode == XMODE_RMSNORM) {
#pragma unroll
          for (int e = 0; e < 8; ++e) v[e] = v[e] * inv_rms * w8[e];
        } else if (P.xmode == XMODE_SILU_MUL) {
#pragma unroll
          for (int e = 0; e < 8; ++e) v[e] = (v[e] / (1.0f + expf(-v[e]))) * w8[e];  // silu(gate) * up, model.cpp:36,414-416
        } else if (P.xmode == XMODE_GELU_MUL) {
#pragma unroll
          for (int e = 0; e < 8; ++e) v[e] = gelu_tanh(v[e]) * w8[e];  // gelu(gate) * up, model.cpp:38-42,409-412
        }
        if (P.rotate) fwht256_warp(v, lane);
        int *aux = xaux + 4 * it;
        U::prologue(v, lane, smem + size_t(it) * FPB, xsum + it, aux);
        if (lane == 0) aux[2] = aux[3] = 0;
      }
      __syncthreads();
      stamp(ph, 2);

      // ---- main loop: evaluate a slot, refill it with the unit NSLOT ahead ------------------------------
      typename U::Acc accs[1];
      U::acc_init(accs[0]);
      const MmaX xo{smem, xsum, xaux, S * FPB};
      if (u0 < u1) {
        int e_rtl = u0 / S, e_b = u0 - e_rtl * S;
        for (int base = u0; base < u1; base += NSLOT) {
#pragma unroll
          for (int sl = 0; sl < NSLOT; ++sl) {
            const int u = base + sl;
            if (u < u1) {
              slot[sl].template eval<1, false>(xo, e_b, accs);
              if (u + NSLOT < u1) {
                slot[sl].load(l_ptr, lane);
                advance_load();
              }
              if (e_b == S - 1 || u == u1 - 1) {  // this warp's part of the row-tile is complete
                const float v = U::acc_row(accs[0], lane);
                const int k = warp - warp_of_unit(e_rtl * S, N);
                seg[(e_rtl * seg_slots + k) * 32 + lane] = v;
                U::acc_init(accs[0]);
              }
              if (++e_b == S) {
                e_b = 0;
                ++e_rtl;
              }
            }
          }
        }
      }
      __syncthreads();
      stamp(ph, 3);

      // ---- rows: add the warps' parts in warp order; split K goes through scratch ------------------------
      const unsigned epoch = epoch0 + unsigned(P.xchg_seq);
      float my_ss = 0.0f;
      auto finish_row = [&](int rtl, int l, float val) {
        const int vrt = rt_a + rtl, j = job_of(P, vrt);
        const int row = (vrt - P.job[j].rt_begin) * TILE_ROWS + l;
        if (row >= P.job[j].M) return;
        float o = val;
        if (P.residual) o += __ldcg(P.residual + row);
        if (P.to_peers) {  // value and tag in one 8-byte store per rank: the reader needs no fence and no flag
          const size_t at = (size_t(epoch & 1u) * p.peer.n + p.peer.rank) * p.peer.cap + row;
          const unsigned long long word = (static_cast<unsigned long long>(epoch + 1u) << 32) | __float_as_uint(o);
          for (int r = 0; r < p.peer.n; ++r) *reinterpret_cast<volatile unsigned long long *>(p.peer.data[r] + at) = word;
        } else {
          P.job[j].y[row] = o;
        }
        my_ss += o * o;
      };
      const int nrows = nrt * TILE_ROWS;
      const int mp = P.rt_total * TILE_ROWS;
      bool final_writer = (P.n_ks == 1);
      for (int r = t; r < nrows; r += PS_THREADS) {
        const int rtl = r >> 5, l = r & 31;
        const int wf = warp_of_unit(rtl * S, N), wl = warp_of_unit(rtl * S + S - 1, N);
        float s = 0.0f;
        for (int k = 0; k <= wl - wf; ++k) {  // warps without a unit of this row-tile (fewer units than warps) wrote nothing
          const int w = wf + k;
          if (max(w * N / PS_WARPS, rtl * S) < min((w + 1) * N / PS_WARPS, (rtl + 1) * S)) s += seg[(rtl * seg_slots + k) * 32 + l];
        }
        if (P.n_ks == 1) finish_row(rtl, l, s);
        else p.scratch[size_t(ks) * mp + (rt_a + rtl) * TILE_ROWS + l] = s;
      }
      if (P.n_ks > 1 && nrt > 0) {
        __syncthreads();
        if (t == 0) {
          // release: publishes the CTA's partial sums (ordered before it by the block barrier);
          // acquire: the last arriver sees the other slices' sums
          unsigned before;
          asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(before) : "l"(p.counters + rg) : "memory");
          flag = (before == unsigned(P.n_ks - 1));
        }
        __syncthreads();
        final_writer = flag != 0;
        if (final_writer) {  // the last slice to arrive adds all slices in slice order
          for (int r = t; r < nrows; r += PS_THREADS) {
            const int rtl = r >> 5, l = r & 31;
            const float *scr = p.scratch + (rt_a + rtl) * TILE_ROWS + l;
            float tot = 0.0f;
            for (int k = 0; k < P.n_ks; ++k) tot += __ldcg(scr + size_t(k) * mp);
            finish_row(rtl, l, tot);
          }
          if (t == 0) p.counters[rg] = 0u;
        }
        __syncthreads();
      }
      if (P.sumsq_out && nrt > 0 && final_writer) {  // uniform over the CTA
        my_ss = block_sum(my_ss, red);
        if (t == 0) P.sumsq_out[rg] = my_ss;
      } else if (P.sumsq_out && nrt == 0 && ks == 0 && t == 0) {
        P.sumsq_out[rg] = 0.0f;  // a row group without rows (fewer row-tiles than groups): the slot may hold an older phase's value
      }
    } else {
      if (ph > 0 && !ps_wait(p, ph - 1, &flag)) return;
      stamp(ph, 1);
      if (P.type == PH_ATTN) {
        // model.cpp:312-372
        if (P.attn_per) {  // one (KV head, KV split) item at a time, all query heads of the group together
          const int items = int(P.rd.nkv) * P.at.n_splits;
          for (int it = c; it < items; it += G) {
            const size_t kvh = size_t(it % int(P.rd.nkv)), split = size_t(it / int(P.rd.nkv));
            unsigned long long *dbg = tl ? tl + ph * 5 + 2 : nullptr;  // timeline slots 2 and 3 of the phase
            const bool ok = P.attn_per == 4 ? attn_group_item<true, 4>(P.at, P.rd, kvh, split, 0, smem, &bar, bar_parity, p.spin_limit, &flag, dbg)
                                            : attn_group_item<true, 2>(P.at, P.rd, kvh, split, 0, smem, &bar, bar_parity, p.spin_limit, &flag, dbg);
            if (!ok) {
              if (t == 0) atomicCAS(p.status, 0u, unsigned(ph) + 1u);
              return;
            }
            __syncthreads();
          }
        } else {  // one (query head, KV split) item at a time
          const int items = int(P.rd.nh) * P.at.n_splits;
          for (int it = c; it < items; it += G) {
            attn_item<true>(P.at, P.rd, size_t(it % int(P.rd.nh)), size_t(it / int(P.rd.nh)), 0, smem, &flag);
            __syncthreads();
          }
        }
      } else if (P.type == PH_EMBED) {
        // model.cpp:58-252: the token's embedding row, and the sum of squares of this CTA's part
        const int i0 = int((long long)(c)*P.h / G), i1 = int((long long)(c + 1) * P.h / G);
        const int tok = P.tokens[0];
        float ss = 0.0f;
        for (int i = i0 + t; i < i1; i += PS_THREADS) {
          const float v = (tok >= 0 && unsigned(tok) < P.vocab) ? tile_elem(P.embed_kind, P.embed_tiles, P.embed_bpr, size_t(tok), size_t(i)) * P.embed_scale : 0.0f;
          P.hidden[i] = v;
          ss += v * v;
        }
        ss = block_sum(ss, red);
        if (t == 0) P.sumsq_out[c] = ss;
      } else if (P.type == PH_REDUCE) {
        // tensor parallel: hidden += the ranks' partial vectors of exchange xchg_seq, in rank order
        const unsigned epoch = epoch0 + unsigned(P.xchg_seq), tag = epoch + 1u;
        const unsigned long long *part = p.xchg_data + size_t(epoch & 1u) * p.peer.n * p.peer.cap;
        const int i0 = int((long long)(c)*P.h / G), i1 = int((long long)(c + 1) * P.h / G);
        float ss = 0.0f;
        bool gave_up = ld_volatile_u32(&p.hdr->timed_out) != 0u;
        for (int i = i0 + t; i < i1; i += PS_THREADS) {
          float add = 0.0f;
          for (int r = 0; r < p.peer.n; ++r) {
            const unsigned long long *src = part + size_t(r) * p.peer.cap + i;
            unsigned long long word = *reinterpret_cast<const volatile unsigned long long *>(src);
            unsigned spins = 0;
            while (unsigned(word >> 32) != tag && !gave_up) {
              if (++spins > p.spin_limit) {  // give up, report, carry on with what is there
                p.hdr->timed_out = 1u;
                atomicCAS(p.status, 0u, unsigned(ph) + 1u);
                gave_up = true;
                break;
              }
              __nanosleep(40);
              word = *reinterpret_cast<const volatile unsigned long long *>(src);
            }
            add += __uint_as_float(unsigned(word));
          }
          const float v = __ldcg(P.hidden + i) + add;
          P.hidden[i] = v;
          ss += v * v;
        }
        ss = block_sum(ss, red);
        if (t == 0) P.sumsq_out[c] = ss;
      }
    }
    ps_arrive(p, ph);
    stamp(ph, 4);
  }
  // tensor parallel: the exchange block's epoch advances once every CTA is past its last use of it
  if (p.peer.n && c == 0 && p.n_phases > 0) {
    if (!ps_wait(p, p.n_phases - 1, &flag)) return;
    if (t == 0) *reinterpret_cast<volatile unsigned *>(&p.hdr->epoch) = epoch0 + unsigned(p.n_xchg);
  }
}

// ---- host side ------------------------------------------------------------------------------------------

// K slices of a GEMV phase: a divisor of the grid size (so that K slices x row groups = grid),
// chosen by a cost estimate in microseconds: prologue of the slice + the longest warp's units at
// an SM's share of the HBM bandwidth + the trip through scratch when K is split.
int choose_k_slices(int grid, int rt_total, int bpr, size_t tile_b) {
  int best = 0;
  double best_cost = 1e30;
  const char *force = std::getenv("LMB_PERSIST_KSLICES");  // tuning: largest K split allowed
  const int cap = force ? std::max(1, std::atoi(force)) : 16;
  for (int n_ks = 1; n_ks <= 16 && n_ks <= bpr; ++n_ks) {
    if (grid % n_ks) continue;
    if (n_ks > cap && best > 0) continue;
    const int S = (bpr + n_ks - 1) / n_ks;
    if (S > PS_S_MAX) continue;
    const int n_rg = grid / n_ks;
    const int nrt = (rt_total + n_rg - 1) / n_rg;
    if (nrt > PS_NRT_MAX) continue;
    const int slots = std::min(PS_WARPS, (PS_WARPS + std::max(1, rt_total / n_rg) - 1) / std::max(1, rt_total / n_rg) + 1);
    if (nrt * slots > PS_MAX_SEG) continue;
    const double per_warp = double((nrt * S + PS_WARPS - 1) / PS_WARPS);
    const double cost = 0.4 + 0.35 * double((S + PS_WARPS - 1) / PS_WARPS) + per_warp * 0.79 * double(tile_b) / 2176.0 +
                        (n_ks > 1 ? 1.5 : 0.0) + 0.01 * n_ks;
    if (cost < best_cost) {
      best_cost = cost;
      best = n_ks;
    }
  }
  return best;
}

template <int KIND> int launch_step(lmb_ctx *ctx, int grid, const PsParams &prm) {
  PsParams p = prm;
  void *args[] = {&p};
  LMB_CUDA(cudaLaunchCooperativeKernel(reinterpret_cast<const void *>(&k_decode_step<KIND>), dim3(unsigned(grid)), dim3(PS_THREADS),
                                       args, PS_SMEM, ctx->stream));
  ctx->launches++;
  return LMB_OK;
}

template <int KIND> int configure_step(int *ctas_per_sm) {
  LMB_CUDA(cudaFuncSetAttribute(k_decode_step<KIND>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(PS_SMEM)));
  LMB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(ctas_per_sm, k_decode_step<KIND>, PS_THREADS, PS_SMEM));
  return LMB_OK;
}

#define PS_FOR_KIND(kind, CALL)                                                       \
  switch (kind) {                                                                     \
  case LMB_INT4: return CALL(LMB_INT4);                                               \
  case DK_TERNARY_MMA: return CALL(DK_TERNARY_MMA);                                   \
  case DK_INT2_MMA: return CALL(DK_INT2_MMA);                                         \
  case DK_BINARY_MMA: return CALL(DK_BINARY_MMA);                                     \
  case DK_INT8_MMA: return CALL(DK_INT8_MMA);                                         \
  case DK_INT3_MMA: return CALL(DK_INT3_MMA);                                         \
  case LMB_INT5: return CALL(LMB_INT5);                                               \
  case LMB_INT6: return CALL(LMB_INT6);                                               \
  default: set_last_error("persistent step: kind has no kernel"); return LMB_ERR_ARG; \
  }

int launch_step_kind(int kind, lmb_ctx *ctx, int grid, const PsParams &prm) {
#define PS_LAUNCH(K) launch_step<K>(ctx, grid, prm)
  PS_FOR_KIND(kind, PS_LAUNCH)
#undef PS_LAUNCH
}
int configure_step_kind(int kind, int *ctas_per_sm) {
#define PS_CONFIGURE(K) configure_step<K>(ctas_per_sm)
  PS_FOR_KIND(kind, PS_CONFIGURE)
#undef PS_CONFIGURE
}

}  // namespace

struct PersistPlan {
  int kind = -1, grid = 0, n_phases = 0, n_xchg = 0;
  PsPhase *d_phases = nullptr;
  // [status | barrier[n_phases] | split-K counters[grid]]; everything but the status word is zeroed
  // before each launch.  The status word stays set until the host has read it: steps launched in
  // between leave at their first wait.
  unsigned *d_sync = nullptr;
  size_t sync_words = 0;
  float *d_scratch = nullptr, *d_sumsq = nullptr;
  unsigned *h_status = nullptr;  // pinned copy of the status word of the last step
  bool status_pending = false;
  unsigned long long *d_timeline = nullptr;  // debug timeline (persist_timeline), allocated on first request
  ~PersistPlan() {
    if (d_phases) cudaFree(d_phases);
    if (d_sync) cudaFree(d_sync);
    if (d_scratch) cudaFree(d_scratch);
    if (d_sumsq) cudaFree(d_sumsq);
    if (h_status) cudaFreeHost(h_status);
    if (d_timeline) cudaFree(d_timeline);
  }
};

bool persist_eligible(const lmb_model *m) {
  if (!m->persistent || m->layers.empty()) return false;
  const lmb_model_config &c = m->cfg;
  if (c.tp_size > 1 && !(m->ctx->xchg.ready && m->tp_peers && c.hidden_size <= m->ctx->xchg.cap)) return false;
  int kind = -1;
  for (const LayerW &L : m->layers) {
    for (int i = 0; i < 7; ++i) {
      if (!L.w[i]) return false;
      if (kind < 0) kind = L.w[i]->kind;
      if (L.w[i]->kind != kind) return false;
    }
    if (L.rot[0] != L.rot[1] || L.rot[0] != L.rot[2] || L.rot[4] != L.rot[5]) return false;
  }
  if (!kind_is_mma(kind) || !m->embed) return false;
  if (c.hidden_size >= (size_t(1) << 24) || c.intermediate_size >= (size_t(1) << 24)) return false;
  return true;
}

void persist_invalidate(lmb_model *m) {
  if (m->ps) {
    cudaStreamSynchronize(m->ctx->stream);
    delete m->ps;
    m->ps = nullptr;
  }
}

static int build_plan(lmb_model *m) {
  lmb_ctx *ctx = m->ctx;
  const lmb_model_config &c = m->cfg;
  PersistPlan *pl = new (std::nothrow) PersistPlan();
  if (!pl) return LMB_ERR_ALLOC;
  auto fail = [&](int st) {
    delete pl;
    return st;
  };
  pl->kind = m->layers[0].w[0]->kind;
  int coop = 0, per_sm = 0;
  LMB_CUDA(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, ctx->device));
  int st = configure_step_kind(pl->kind, &per_sm);
  if (st != LMB_OK) return fail(st);
  if (!coop || per_sm < 1) {
    set_last_error("persistent step: cooperative launch unavailable or the kernel does not fit an SM");
    return fail(LMB_ERR_STATE);
  }
  const int grid = pl->grid = std::min(per_sm, 2) * ctx->sm_count;
  const bool tp = c.tp_size > 1;
  const size_t h = c.hidden_size, hd = c.head_dim;
  const size_t TB = tile_bytes(pl->kind);
  std::vector<PsPhase> ph;
  size_t scratch_floats = 1;
  LMB_CUDA(cudaMalloc(&pl->d_sumsq, size_t(2) * grid * sizeof(float)));
  LMB_CUDA(cudaMemset(pl->d_sumsq, 0, size_t(2) * grid * sizeof(float)));
  float *ss[2] = {pl->d_sumsq, pl->d_sumsq + grid};
  int cur = 0;  // sumsq buffer that describes the current hidden state
  int n_cur = grid;
  bool ok = true;

  PsPhase e;
  std::memset(&e, 0, sizeof e);
  e.type = PH_EMBED;
  e.tokens = m->d_tokens;
  e.embed_tiles = m->embed->d_tiles;
  e.embed_kind = m->embed->kind;
  e.embed_bpr = unsigned(m->embed->bpr);
  e.vocab = unsigned(c.vocab_size);
  e.h = unsigned(h);
  e.embed_scale = c.gemma ? std::sqrt(float(h)) : 1.0f;
  e.hidden = m->hidden;
  e.sumsq_out = ss[cur];
  ph.push_back(e);

  auto gemv = [&](int njobs, lmb_weight *const *ws, float *const *ys, const float *x, size_t x_len, int xmode, const float *x2,
                  bool rotate, const float *residual, bool hidden_out) {
    PsPhase g;
    std::memset(&g, 0, sizeof g);
    g.type = PH_GEMV;
    g.njobs = njobs;
    int rt = 0;
    for (int j = 0; j < njobs; ++j) {
      g.job[j] = PsJob{ws[j]->d_tiles, ys[j], int(ws[j]->M), rt};
      rt += int(ws[j]->row_tiles);
      if (ws[j]->bpr != ws[0]->bpr) ok = false;
    }
    g.rt_total = rt;
    g.bpr = int(ws[0]->bpr);
    g.n_ks = choose_k_slices(grid, rt, g.bpr, TB);
    if (g.n_ks < 1) {
      ok = false;
      g.n_ks = 1;
    }
    g.n_rg = grid / g.n_ks;
    g.xmode = xmode;
    g.rotate = rotate ? 1 : 0;
    g.x = x;
    g.x2 = x2;
    g.x_len = unsigned(x_len);
    g.residual = residual;
    if (xmode == XMODE_RMSNORM) {
      g.sumsq_in = ss[cur];
      g.n_sumsq_in = n_cur;
    }
    if (g.n_ks > 1) scratch_floats = std::max(scratch_floats, size_t(g.n_ks) * rt * TILE_ROWS);
    if (hidden_out && tp) {  // partial vector to every rank; the reduce phase makes the hidden state
      g.to_peers = 1;
      g.xchg_seq = pl->n_xchg;
      g.residual = nullptr;
      ph.push_back(g);
      PsPhase r;
      std::memset(&r, 0, sizeof r);
      r.type = PH_REDUCE;
      r.xchg_seq = pl->n_xchg++;
      r.hidden = m->hidden;
      r.h = unsigned(h);
      cur ^= 1;
      r.sumsq_out = ss[cur];
      n_cur = grid;
      ph.push_back(r);
      return;
    }
    if (hidden_out) {
      cur ^= 1;
      g.sumsq_out = ss[cur];
      n_cur = g.n_rg;
    }
    ph.push_back(g);
  };

  // Attention: the group form where the shape allows it (every (KV head, split) item gets a CTA of
  // its own: a second round of a few left-over items would double the phase's time), else one item
  // per (query head, split).
  RopeDims rd{m->nh, m->nkv, hd, c.max_seq_len, m->seq_stride, 0};
  int n_splits = 1, attn_per = 0;
  // as many items as fit the grid in one round (more only when the context needs that many slices)
  const AttnGroupPlan agp = m->attn_group ? plan_attn_group(m->nh, m->nkv, hd, c.max_seq_len, 1, (size_t(grid) / m->nkv) * m->nkv, PS_SMEM)
                                          : AttnGroupPlan{false, 1, 0, 0, 0};
  if (agp.ok) {
    n_splits = agp.n_splits;
    attn_per = agp.per;
    rd.split_len = agp.split_len;
  } else {
    n_splits = std::max(1, std::min(decode_attn_splits(ctx, m->nh, 1, c.max_seq_len), grid / int(m->nh)));
    rd.split_len = ((c.max_seq_len + n_splits - 1) / n_splits + 15) / 16 * 16;
    if ((rd.split_len + 3 * hd + 32 + ATT_THREADS) * sizeof(float) > PS_SMEM || hd > size_t(ATT_THREADS) || ATT_THREADS % hd != 0) ok = false;
  }

  for (size_t l = 0; l < m->layers.size(); ++l) {
    LayerW &L = m->layers[l];
    float *qkv[3] = {m->q, m->k, m->v};
    gemv(3, &L.w[0], qkv, m->hidden, h, XMODE_RMSNORM, L.in_norm, L.rot[0], nullptr, false);
    PsPhase a;
    std::memset(&a, 0, sizeof a);
    a.type = PH_ATTN;
    a.at = AttnArgs{m->q, m->k, m->v, L.qb, L.kb, L.vb, m->cs_table, m->d_pos, m->kv, m->att, m->att_partial, m->att_counters, n_splits, l};
#ifdef LMB_DEBUG_BOUNDS
    a.at.kv_floats = m->seq_stride * m->cfg.max_batch;
#endif
    a.rd = rd;
    a.attn_per = attn_per;
    ph.push_back(a);
    float *o[1] = {tp ? m->proj : m->hidden};
    gemv(1, &L.w[3], o, m->att, m->nh * hd, XMODE_PLAIN, nullptr, L.rot[3], m->hidden, true);
    float *gu[2] = {m->gate, m->up};
    gemv(2, &L.w[4], gu, m->hidden, h, XMODE_RMSNORM, L.post_norm, L.rot[4], nullptr, false);
    float *d[1] = {tp ? m->proj : m->hidden};
    gemv(1, &L.w[6], d, m->gate, m->inter, c.activation == LMB_ACT_GELU ? XMODE_GELU_MUL : XMODE_SILU_MUL, m->up, L.rot[6], m->hidden, true);
  }
  if (!ok) {
    set_last_error("persistent step: a projection shape does not fit the kernel's per-CTA limits");
    return fail(LMB_ERR_STATE);
  }
  pl->n_phases = int(ph.size());
  pl->sync_words = 1 + size_t(pl->n_phases) + size_t(grid);
  cudaError_t err = cudaMalloc(&pl->d_phases, ph.size() * sizeof(PsPhase));
  if (err == cudaSuccess) err = cudaMemcpy(pl->d_phases, ph.data(), ph.size() * sizeof(PsPhase), cudaMemcpyHostToDevice);
  if (err == cudaSuccess) err = cudaMalloc(&pl->d_sync, pl->sync_words * sizeof(unsigned));
  if (err == cudaSuccess) err = cudaMemset(pl->d_sync, 0, pl->sync_words * sizeof(unsigned));
  if (err == cudaSuccess) err = cudaMalloc(&pl->d_scratch, scratch_floats * sizeof(float));
  if (err == cudaSuccess) err = cudaMallocHost(&pl->h_status, sizeof(unsigned));
  if (err != cudaSuccess) return fail(cuda_fail(err, "persistent step: allocation"));
  *pl->h_status = 0;
  m->ps = pl;
  return LMB_OK;
}

int persist_forward(lmb_model *m) {
  if (!persist_eligible(m)) return LMB_ERR_STATE;
  lmb_ctx *ctx = m->ctx;
  if (!m->ps) {
    int st = build_plan(m);
    if (st != LMB_OK) return st;
  }
  PersistPlan *pl = m->ps;
  LMB_CUDA(cudaMemsetAsync(pl->d_sync + 1, 0, (pl->sync_words - 1) * sizeof(unsigned), ctx->stream));
  PsParams p;
  std::memset(&p, 0, sizeof p);
  p.phases = pl->d_phases;
  p.n_phases = pl->n_phases;
  p.n_xchg = pl->n_xchg;
  p.status = pl->d_sync;
  p.barrier = pl->d_sync + 1;
  p.counters = pl->d_sync + 1 + pl->n_phases;
  p.scratch = pl->d_scratch;
  p.spin_limit = ctx->xchg.spin_limit;
  p.extra_arrivals = unsigned(m->debug_extra_arrivals);
  p.eps = m->cfg.rms_norm_eps;
  p.timeline = pl->d_timeline;
  if (m->cfg.tp_size > 1) {
    p.peer.n = ctx->tp_size;
    p.peer.rank = ctx->tp_rank;
    p.peer.cap = unsigned(ctx->xchg.cap);
    p.hdr = static_cast<XchgHeader *>(ctx->xchg.local);
    p.peer.epoch = &p.hdr->epoch;
    p.xchg_data = reinterpret_cast<const unsigned long long *>(static_cast<const char *>(ctx->xchg.local) + XCHG_HEADER_BYTES);
    for (int r = 0; r < ctx->tp_size; ++r)
      p.peer.data[r] = reinterpret_cast<unsigned long long *>(static_cast<char *>(ctx->xchg.peer[r]) + XCHG_HEADER_BYTES);
  }
  if (pl->d_timeline)
    LMB_CUDA(cudaMemsetAsync(pl->d_timeline + size_t(2) * pl->n_phases * 5, 0, size_t(pl->n_phases) * 2 * sizeof(unsigned long long), ctx->stream));
  return launch_step_kind(pl->kind, ctx, pl->grid, p);
}

// Queues the copy of the step's status word to the host (after the kernels that follow the step,
// so that it does not sit between the step and the head's GEMV).
int persist_record_status(lmb_model *m) {
  PersistPlan *pl = m->ps;
  if (!pl) return LMB_OK;
  LMB_CUDA(cudaMemcpyAsync(pl->h_status, pl->d_sync, sizeof(unsigned), cudaMemcpyDeviceToHost, m->ctx->stream));
  pl->status_pending = true;
  return LMB_OK;
}

// Debug view: turns the per-phase timestamps on (first call) and returns those of the last step:
// out[2][n_phases][5] nanoseconds, phase types in types[n_phases], K slices in kslices[n_phases].
int persist_timeline(lmb_model *m, unsigned long long *out, int *types, int *kslices, size_t cap_phases, size_t *n_phases) {
  PersistPlan *pl = m->ps;
  if (!pl) {
    set_last_error("persistent step: no plan yet (run one batch-1 step first)");
    return LMB_ERR_STATE;
  }
  *n_phases = size_t(pl->n_phases);
  const size_t words = size_t(2) * pl->n_phases * 5 + size_t(pl->n_phases) * 2;
  LMB_CUDA(cudaStreamSynchronize(m->ctx->stream));
  if (!pl->d_timeline) {
    LMB_CUDA(cudaMalloc(&pl->d_timeline, words * sizeof(unsigned long long)));
    LMB_CUDA(cudaMemset(pl->d_timeline, 0, words * sizeof(unsigned long long)));
    return LMB_OK;  // recorded from the next step on
  }
  if (cap_phases < size_t(pl->n_phases)) return LMB_OK;
  LMB_CUDA(cudaMemcpy(out, pl->d_timeline, words * sizeof(unsigned long long), cudaMemcpyDeviceToHost));
  std::vector<PsPhase> ph(size_t(pl->n_phases));
  LMB_CUDA(cudaMemcpy(ph.data(), pl->d_phases, ph.size() * sizeof(PsPhase), cudaMemcpyDeviceToHost));
  for (int i = 0; i < pl->n_phases; ++i) {
    types[i] = ph[size_t(i)].type;
    kslices[i] = ph[size_t(i)].n_ks;
  }
  return LMB_OK;
}

int persist_take_status(lmb_model *m, unsigned *status) {
  *status = 0;
  if (!m->ps || !m->ps->status_pending) return LMB_OK;
  LMB_CUDA(cudaStreamSynchronize(m->ctx->stream));
  *status = *m->ps->h_status;
  m->ps->status_pending = false;
  if (*status) LMB_CUDA(cudaMemsetAsync(m->ps->d_sync, 0, sizeof(unsigned), m->ctx->stream));  // reported: steps may run again
  return LMB_OK;
}

}  // namespace lmb
