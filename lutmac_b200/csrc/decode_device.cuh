// Device code shared by the decode-step kernels (decode_ops.cu launches each piece on its own,
// persist.cu runs them as phases of one persistent kernel): a dequantised weight element out of
// the tile layout (embedding rows), block-wide reductions and one (head, KV split) item of the
// split-KV decode attention.
#pragma once

#include "common.cuh"
#include "decode_ops.cuh"
#include "device_utils.cuh"

namespace lmb {

namespace {

// Dequantised weight (row, col) out of the device tile layout: Block::get of types.hpp.
__device__ float tile_elem(int kind, const uint8_t *tiles, size_t bpr, size_t row, size_t col) {
  const size_t rt = row / TILE_ROWS, l = row % TILE_ROWS, b = col / BLK, j = col % BLK;
  const KindInfo ki = kind_info(kind);
  const uint8_t *tile = tiles + (rt * bpr + b) * (size_t(TILE_ROWS) * ki.ref_bytes);
  const float *sc = reinterpret_cast<const float *>(tile + size_t(ki.chunks) * TILE_ROWS * 16);
  const float s0 = sc[l];
  auto pay = [&](size_t chunk, size_t byte) { return tile[(chunk * TILE_ROWS + l) * 16 + byte]; };
  const unsigned bit = 7u - unsigned(j % 8);
  switch (kind) {
  case LMB_INT8: return float(int8_t(pay(j / 16, j % 16))) * s0;
  case LMB_INT4:
  case LMB_INT5:
  case LMB_INT6: {  // MMA operand order, see common.cuh
    const size_t h = l / 16, g = l % 8, m = l / 8, s = j / 32, kk = j % 32, tid = (kk % 16) / 4;
    const size_t lane = g * 4 + tid, chunk = h * 4 + s / 2, word = (s % 2) * 2 + kk / 16;
    const uint8_t byte = tile[(chunk * TILE_ROWS + lane) * 16 + word * 4 + kk % 4];
    int code = ((l % 16) >= 8) ? (byte >> 4) : (byte & 15);
    for (int pl = 0; pl < kind - 4; ++pl) {  // bit planes 4 (and 5) in the binary arrangement
      const size_t wi = (s / 2) * 2 + kk / 16;
      const uint8_t pb = tile[4096 + 1024 * pl + ((wi / 4) * TILE_ROWS + lane) * 16 + (wi % 4) * 4 + kk % 4];
      code |= int((pb >> (m + 4 * (s % 2))) & 1u) << (4 + pl);
    }
    return float(code - (8 << (kind - 4))) * sc[4 * g + m];
  }
  case DK_INT3_MMA: {
    const size_t m = l / 8, g = l % 8, s = j / 32, kk = j % 32, tid = (kk % 16) / 4;
    const size_t lane = g * 4 + tid, wi = (s / 2) * 2 + kk / 16;
    int code = 0;
    for (int pl = 0; pl < 3; ++pl) {
      const uint8_t pb = tile[1024 * pl + ((wi / 4) * TILE_ROWS + lane) * 16 + (wi % 4) * 4 + kk % 4];
      code |= int((pb >> (m + 4 * (s % 2))) & 1u) << pl;
    }
    return float(code - 4) * sc[4 * g + m];
  }
  case DK_INT8_MMA: {
    const size_t h = l / 16, g = l % 8, s = j / 32, kk = j % 32, tid = (kk % 16) / 4;
    const size_t a = 2 * (kk / 16) + (l % 16) / 8;
    return float(int8_t(tile[((h * 8 + s) * TILE_ROWS + g * 4 + tid) * 16 + a * 4 + kk % 4])) * sc[4 * g + l / 8];
  }
  case DK_TERNARY_MMA: {  // 2-bit codes t+1 in MMA operand order, see common.cuh
    const size_t m = l / 8, g = l % 8, s = j / 32, kk = j % 32, tid = (kk % 16) / 4;
    const size_t lane = g * 4 + tid, chunk = s / 2, word = (s % 2) * 2 + kk / 16;
    const unsigned code = (tile[(chunk * TILE_ROWS + lane) * 16 + word * 4 + kk % 4] >> (2 * m)) & 3u;
    return (float(int(code)) - 1.0f) * sc[4 * g + m];
  }
  case DK_INT2_MMA: {
    const size_t m = l / 8, g = l % 8, s = j / 32, kk = j % 32, tid = (kk % 16) / 4;
    const size_t lane = g * 4 + tid, chunk = s / 2, word = (s % 2) * 2 + kk / 16;
    const unsigned f = (tile[(chunk * TILE_ROWS + lane) * 16 + word * 4 + kk % 4] >> (2 * m)) & 3u;
    const float s1 = sc[4 * g + m], s2 = sc[TILE_ROWS + 4 * g + m];
    return ((f & 1u) ? s1 : -s1) + ((f & 2u) ? s2 : -s2);
  }
  case DK_BINARY_MMA: {
    const size_t m = l / 8, g = l % 8, s = j / 32, kk = j % 32, tid = (kk % 16) / 4;
    const size_t lane = g * 4 + tid, wi = (s / 2) * 2 + kk / 16;
    const unsigned v = (tile[((wi / 4) * TILE_ROWS + lane) * 16 + (wi % 4) * 4 + kk % 4] >> (m + 4 * (s % 2))) & 1u;
    return v ? sc[4 * g + m] : -sc[4 * g + m];
  }
  case LMB_TERNARY: {
    const size_t jb = j / 8;
    const unsigned p = (pay(jb / 8, jb % 8) >> bit) & 1u, n = (pay(jb / 8, 8 + jb % 8) >> bit) & 1u;
    return p ? s0 : (n ? -s0 : 0.0f);
  }
  case LMB_INT2: {
    const size_t jb = j / 8;
    const unsigned b1 = (pay(jb / 8, jb % 8) >> bit) & 1u, b2 = (pay(jb / 8, 8 + jb % 8) >> bit) & 1u;
    const float s1 = sc[TILE_ROWS + l];
    return (b1 ? s0 : -s0) + (b2 ? s1 : -s1);
  }
  case LMB_INT3: {
    const size_t jb = j / 8, jj = jb / 16;
    unsigned code = 0;
    for (unsigned q = 0; q < 3; ++q) code |= ((pay(3 * jj + (2 - q), jb % 16) >> bit) & 1u) << q;
    return float(int(code) - 4) * s0;
  }
  case LMB_BINARY: return (((pay((j / 8) / 16, (j / 8) % 16)) >> bit) & 1u) ? s0 : -s0;
  default: return 0.0f;
  }
}

__device__ __forceinline__ float block_sum(float v, float *red) {
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : 0.0f;
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) t += __shfl_xor_sync(0xffffffffu, t, m);
  return t;
}

__device__ __forceinline__ float block_max(float v, float *red) {
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, m));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : -INFINITY;
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) t = fmaxf(t, __shfl_xor_sync(0xffffffffu, t, m));
  return t;
}

// Split-KV decode attention with the q/k/v bias, the rotary embedding and the KV-cache write of
// the new position folded in (model.cpp:312-372, embedding.cpp:36-75, attention.cpp:23-42).
// One CTA per (query head, KV split, sequence).  Every CTA rotates its own query head; the split
// that contains the new position takes that position's key/value from the fresh projections
// (and, for the first query head of a KV group, stores them in the cache) instead of reading
// the cache.  Scores of the slice (four timesteps in flight per warp), a local softmax, the
// weighted values (eight loads in flight per thread); partial (max, sum, vector) go to scratch
// and the last split to arrive for a head merges them in split order and normalises.
constexpr int ATT_THREADS = 256;

struct AttnArgs {
  const float *q, *k, *v;          // fresh projections [batch][heads*hd]
  const float *qb, *kb, *vb;       // biases or null
  const float *cs_table;           // [max_seq][hd/2 cos | hd/2 sin]
  const size_t *positions;
  float *kv;                       // cache
  float *out;                      // [batch][nh*hd]
  float *partial;
  unsigned *counters;
  int n_splits;
  size_t layer;
#ifdef LMB_DEBUG_BOUNDS
  size_t kv_floats;  // extent of `kv`
#endif
};

// FRESH_CG: the fresh projections were written earlier in the SAME kernel launch (persistent
// decode step) and must be read around the L1 cache, which is not coherent within a launch.
template <bool FRESH_CG> __device__ __forceinline__ float ld_fresh(const float *p) { return FRESH_CG ? __ldcg(p) : *p; }

template <bool FRESH_CG>
__device__ __forceinline__ void attn_item(const AttnArgs &a, const RopeDims &d, size_t head, size_t split, size_t b, float *sm,
                                          int *is_last_p) {
  float *sc = sm;                    // [split_len]
  float *qs = sc + d.split_len;      // [hd] rotated query
  float *kn = qs + d.hd;             // [hd] rotated key of the new position
  float *vn = kn + d.hd;             // [hd] value of the new position
  float *red = vn + d.hd;            // [32]
  float *acc = red + 32;             // [ATT_THREADS]
  const size_t pos = a.positions[b], seq = pos + 1;
  const size_t group = d.nh / d.nkv, kvh = head / group, kv_dim = d.nkv * d.hd, half = d.hd / 2;
  // cache layout on the device: [sequence][layer][K|V][kv head][position][head_dim]
  float *kc_w = a.kv + b * d.seq_stride + (a.layer * 2) * d.max_seq * kv_dim + kvh * d.max_seq * d.hd;
  float *vc_w = kc_w + d.max_seq * kv_dim;
  const size_t rs = d.hd;  // floats between consecutive positions of one head
  const float *kc = kc_w, *vc = vc_w;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = ATT_THREADS / 32;
  const int n_splits = a.n_splits;
  size_t len = (seq + n_splits - 1) / n_splits;
  len = (len + 15) / 16 * 16;
  const size_t t0 = min(split * len, seq), t1 = min(t0 + len, seq), n = t1 - t0;
  const bool has_new = (pos >= t0 && pos < t1);
  const float *cs = a.cs_table + pos * d.hd;
  // rotate the query head (and the new key), pairs (i, i + hd/2)
  for (size_t i = threadIdx.x; i < half; i += ATT_THREADS) {
    const float c = cs[i], sn = cs[half + i];
    const size_t i0 = (b * d.nh + head) * d.hd + i, i1 = i0 + half;
    float x0 = ld_fresh<FRESH_CG>(a.q + i0), x1 = ld_fresh<FRESH_CG>(a.q + i1);
    if (a.qb) {
      x0 += a.qb[head * d.hd + i];
      x1 += a.qb[head * d.hd + i + half];
    }
    qs[i] = x0 * c - x1 * sn;
    qs[i + half] = x0 * sn + x1 * c;
    if (has_new) {
      const size_t k0 = (b * d.nkv + kvh) * d.hd + i, k1 = k0 + half;
      float y0 = ld_fresh<FRESH_CG>(a.k + k0), y1 = ld_fresh<FRESH_CG>(a.k + k1), v0 = ld_fresh<FRESH_CG>(a.v + k0), v1 = ld_fresh<FRESH_CG>(a.v + k1);
      if (a.kb) {
        y0 += a.kb[kvh * d.hd + i];
        y1 += a.kb[kvh * d.hd + i + half];
      }
      if (a.vb) {
        v0 += a.vb[kvh * d.hd + i];
        v1 += a.vb[kvh * d.hd + i + half];
      }
      const float r0 = y0 * c - y1 * sn, r1 = y0 * sn + y1 * c;
      kn[i] = r0;
      kn[i + half] = r1;
      vn[i] = v0;
      vn[i + half] = v1;
      if (head % group == 0) {  // one writer per KV head
        kc_w[pos * rs + i] = r0;
        kc_w[pos * rs + i + half] = r1;
        vc_w[pos * rs + i] = v0;
        vc_w[pos * rs + i + half] = v1;
      }
    }
  }
  __syncthreads();
  const float scale = 1.0f / sqrtf(float(d.hd));
  const size_t per = d.hd / 32;  // 2 or 4 (head_dim 64 or 128); other head dims take the generic loop
  const size_t tnew = has_new ? pos - t0 : ~size_t(0);  // slice-local index of the new position
  constexpr int TS = 8;  // timesteps per warp and iteration: eight key loads in flight per lane
  for (size_t tb = warp * TS; tb < n; tb += nw * TS) {
    float s[TS];
#pragma unroll
    for (int i = 0; i < TS; ++i) s[i] = 0.0f;
    if (per == 4) {
      float4 kk[TS];
      const float4 qv = reinterpret_cast<const float4 *>(qs)[lane];
#pragma unroll
      for (int i = 0; i < TS; ++i) {
        const size_t t = tb + i;
        kk[i] = (t >= n) ? make_float4(0, 0, 0, 0)
                : (t == tnew) ? reinterpret_cast<const float4 *>(kn)[lane]
                              : reinterpret_cast<const float4 *>(kc + (t0 + t) * rs)[lane];
      }
#pragma unroll
      for (int i = 0; i < TS; ++i) s[i] = qv.x * kk[i].x + qv.y * kk[i].y + qv.z * kk[i].z + qv.w * kk[i].w;
    } else if (per == 2) {
      float2 kk[TS];
      const float2 qv = reinterpret_cast<const float2 *>(qs)[lane];
#pragma unroll
      for (int i = 0; i < TS; ++i) {
        const size_t t = tb + i;
        kk[i] = (t >= n) ? make_float2(0, 0)
                : (t == tnew) ? reinterpret_cast<const float2 *>(kn)[lane]
                              : reinterpret_cast<const float2 *>(kc + (t0 + t) * rs)[lane];
      }
#pragma unroll
      for (int i = 0; i < TS; ++i) s[i] = qv.x * kk[i].x + qv.y * kk[i].y;
    } else {
#pragma unroll
      for (int i = 0; i < TS; ++i) {
        const size_t t = tb + i;
        if (t < n)
          for (size_t c = lane; c < d.hd; c += 32) s[i] += qs[c] * (t == tnew ? kn[c] : kc[(t0 + t) * rs + c]);
      }
    }
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) {
#pragma unroll
      for (int i = 0; i < TS; ++i) s[i] += __shfl_xor_sync(0xffffffffu, s[i], m);
    }
#pragma unroll
    for (int i = 0; i < TS; ++i)
      if (lane == i && tb + i < n) sc[tb + i] = s[i] * scale;
  }
  __syncthreads();
  float mx = -INFINITY;
  for (size_t t = threadIdx.x; t < n; t += ATT_THREADS) mx = fmaxf(mx, sc[t]);
  mx = block_max(mx, red);
  float sum = 0.0f;
  for (size_t t = threadIdx.x; t < n; t += ATT_THREADS) {
    const float e = expf(sc[t] - mx);
    sc[t] = e;
    sum += e;
  }
  sum = block_sum(sum, red);
  __syncthreads();
  // weighted values: thread = (group, dim); groups stride over the slice, 16 loads in flight.
  // The new position (if in this slice) is left out here and added from shared memory below.
  const size_t groups = ATT_THREADS / d.hd, g = threadIdx.x / d.hd, dd = threadIdx.x % d.hd;
  const size_t n_old = has_new ? n - 1 : n;  // the new position is always the last of its slice
  float av = 0.0f;
  {
    size_t t = g;
    for (; t + 15 * groups < n_old; t += 16 * groups) {
      float vv[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) vv[i] = vc[(t0 + t + i * groups) * rs + dd];
#pragma unroll
      for (int i = 0; i < 16; ++i) av += sc[t + i * groups] * vv[i];
    }
    for (; t + 3 * groups < n_old; t += 4 * groups) {
      float vv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) vv[i] = vc[(t0 + t + i * groups) * rs + dd];
#pragma unroll
      for (int i = 0; i < 4; ++i) av += sc[t + i * groups] * vv[i];
    }
    for (; t < n_old; t += groups) av += sc[t] * vc[(t0 + t) * rs + dd];
    if (has_new && g == 0) av += sc[n - 1] * vn[dd];
  }
  acc[threadIdx.x] = av;
  __syncthreads();
  // partial record of this split: [hd values | max | sum]
  const size_t rec = d.hd + 2;
  float *prt = a.partial + ((b * d.nh + head) * n_splits + split) * rec;
  if (threadIdx.x < d.hd) {
    float v = 0.0f;
    for (size_t k2 = 0; k2 < groups; ++k2) v += acc[k2 * d.hd + threadIdx.x];
    prt[threadIdx.x] = v;
  }
  if (threadIdx.x == 0) {
    prt[d.hd] = mx;
    prt[d.hd + 1] = sum;
  }
  __syncthreads();
  unsigned *ctr = a.counters + b * d.nh + head;
  if (threadIdx.x == 0) {
    __threadfence();
    *is_last_p = (atomicAdd(ctr, 1u) == unsigned(n_splits - 1));
    __threadfence();
  }
  __syncthreads();
  if (!*is_last_p) return;
  // merge of the splits by the last CTA of the head: the (max, sum) pairs first, one thread per
  // split, then the vectors with the splits dealt over the thread groups and four loads in flight
  const float *all = a.partial + ((b * d.nh + head) * n_splits) * rec;
  float *wk = sc;  // [n_splits] weights, reusing the score buffer (n_splits <= 32 <= split_len)
  if (threadIdx.x < unsigned(n_splits)) {
    red[threadIdx.x] = __ldcg(all + threadIdx.x * rec + d.hd);
    wk[threadIdx.x] = __ldcg(all + threadIdx.x * rec + d.hd + 1);
  }
  __syncthreads();
  float gmx = -INFINITY, den = 0.0f;
  for (int k2 = 0; k2 < n_splits; ++k2) gmx = fmaxf(gmx, red[k2]);
  for (int k2 = 0; k2 < n_splits; ++k2) den += (wk[k2] > 0.0f) ? expf(red[k2] - gmx) * wk[k2] : 0.0f;
  __syncthreads();
  if (threadIdx.x < unsigned(n_splits)) wk[threadIdx.x] = (wk[threadIdx.x] > 0.0f) ? expf(red[threadIdx.x] - gmx) : 0.0f;
  __syncthreads();
  {
    float tot = 0.0f;
    int k2 = int(g);
    for (; k2 + 3 * int(groups) < n_splits; k2 += 4 * int(groups)) {
      float pv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) pv[i] = __ldcg(all + (k2 + i * int(groups)) * rec + dd);
#pragma unroll
      for (int i = 0; i < 4; ++i) tot += wk[k2 + i * int(groups)] * pv[i];
    }
    for (; k2 < n_splits; k2 += int(groups)) tot += wk[k2] * __ldcg(all + k2 * rec + dd);
    acc[threadIdx.x] = tot;
  }
  __syncthreads();
  if (threadIdx.x < d.hd) {
    float tot = 0.0f;
    for (size_t k2 = 0; k2 < groups; ++k2) tot += acc[k2 * d.hd + threadIdx.x];
    a.out[(b * d.nh + head) * d.hd + threadIdx.x] = tot * (1.0f / den);
  }
  if (threadIdx.x == 0) *ctr = 0u;
}


// ---------------------------------------------------------------------------------------------
// Group attention: one CTA per (KV head, KV split, sequence) serves ALL query heads of the KV
// group, so the keys and values of the slice are read once instead of once per query head
// (grouped-query attention, model.cpp:338-372, reads the same cache rows for every head of a
// group).  The slice's keys and its values are each fetched with ONE bulk asynchronous copy
// (cp.async.bulk, completion on an mbarrier): the whole slice is in flight at once instead of a
// few loads per thread, which is what bounds a latency-limited decode attention.  The new position's
// key / value come from the fresh projections (bias and rotary embedding applied here) and are
// written to the cache by this CTA.  Partial (max, sum, vector) records go to scratch; the last
// split of a KV head to arrive merges the records of the group's heads in split order.
// ---------------------------------------------------------------------------------------------
constexpr int ATT_MAX_GROUP = 8;    // query heads per KV head the group form handles
constexpr int ATT_MAX_SPLITS = 64;  // KV splits the merge handles
constexpr int ATT_REC_PAD = 4;      // a partial record is head_dim + 4 floats: {vector, max, sum, -, -} (16-byte aligned)

__host__ __device__ inline size_t attn_group_smem_floats(size_t split_len, size_t hd, size_t group) {
  return 2 * split_len * hd + group * hd + group * split_len + size_t(ATT_MAX_GROUP) * ATT_MAX_SPLITS + 2 * ATT_MAX_GROUP;
}

__device__ __forceinline__ uint32_t smem_addr_u32(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(uint64_t *bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr_u32(bar)), "r"(count) : "memory");
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, unsigned parity) {
  unsigned ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_addr_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Plain (not multicast) bulk copy from this GPU's global memory into this CTA's shared memory:
// both addresses 16-byte aligned, the size a multiple of 16.
__device__ __forceinline__ void bulk_copy_g2s(void *dst, const void *src, unsigned bytes, uint64_t *bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_addr_u32(dst)),
               "l"(src), "r"(bytes), "r"(smem_addr_u32(bar))
               : "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

template <int PER> struct LaneVec { float v[PER]; };
template <int PER> __device__ __forceinline__ LaneVec<PER> ld_lane_vec(const float *row, int lane) {
  LaneVec<PER> r;
  if constexpr (PER == 4) {
    const float4 x = reinterpret_cast<const float4 *>(row)[lane];
    r.v[0] = x.x; r.v[1] = x.y; r.v[2] = x.z; r.v[3] = x.w;
  } else {
    const float2 x = reinterpret_cast<const float2 *>(row)[lane];
    r.v[0] = x.x; r.v[1] = x.y;
  }
  return r;
}
template <int PER> __device__ __forceinline__ void st_lane_vec(float *row, int lane, const LaneVec<PER> &r) {
  if constexpr (PER == 4) reinterpret_cast<float4 *>(row)[lane] = make_float4(r.v[0], r.v[1], r.v[2], r.v[3]);
  else reinterpret_cast<float2 *>(row)[lane] = make_float2(r.v[0], r.v[1]);
}
template <int PER> __device__ __forceinline__ LaneVec<PER> ldcg_lane_vec(const float *row, int lane) {
  LaneVec<PER> r;
  if constexpr (PER == 4) {
    const float4 x = __ldcg(reinterpret_cast<const float4 *>(row) + lane);
    r.v[0] = x.x; r.v[1] = x.y; r.v[2] = x.z; r.v[3] = x.w;
  } else {
    const float2 x = __ldcg(reinterpret_cast<const float2 *>(row) + lane);
    r.v[0] = x.x; r.v[1] = x.y;
  }
  return r;
}

// One (KV head, split, sequence) item.  head_dim = 32 * PER.  `parity` is the phase of `bar` this
// item waits for (flipped here).  False when the bounded wait for the copies ran out (*timed_out
// is then set): the caller leaves the kernel.  All ATT_THREADS threads of the CTA take part.
// `dbg` (profiling aid, usually null): thread 0 records the device's nanosecond timer after the wait
// for the copies (dbg[0]) and after the partial records are written (dbg[1]).
// WIDE: the form for batch 1, where the kernel is one wave of CTAs and bound by their latency: queries
// kept in registers, the value pass by timestep with all heads per lane, merge statistics in one round
// trip and 16 partial records in flight.  With several sequences (many waves) the plain form is faster.
template <bool FRESH_CG, int PER, bool WIDE = false>
__device__ __forceinline__ bool attn_group_item(const AttnArgs &a, const RopeDims &d, size_t kvh, size_t split, size_t b, float *sm,
                                                uint64_t *bar, unsigned &parity, unsigned spin_limit, int *flag,
                                                unsigned long long *dbg = nullptr, unsigned long long *tl = nullptr) {
  const size_t hd = d.hd, g = d.nh / d.nkv, kv_dim = d.nkv * hd, half = hd / 2, sl = d.split_len;
  float *Ks = sm, *Vs = Ks + sl * hd, *qs = Vs + sl * hd, *sc = qs + g * hd, *wk = sc + g * sl, *stat = wk + ATT_MAX_GROUP * ATT_MAX_SPLITS;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, nw = ATT_THREADS / 32;
  const size_t pos = a.positions[b], seq = pos + 1;
  const int n_splits = a.n_splits;
  size_t len = (seq + n_splits - 1) / n_splits;
  len = (len + 7) / 8 * 8;  // <= split_len, which was sized for the longest context
  const size_t t0 = min(split * len, seq), t1 = min(t0 + len, seq), n = t1 - t0;
  const bool has_new = (pos >= t0 && pos < t1);  // the new position is the last one of its slice
  const size_t n_old = has_new ? n - 1 : n;
  // cache layout on the device: [sequence][layer][K|V][kv head][position][head_dim]: the slice of one
  // head is contiguous, so it takes ONE bulk copy for the keys and one for the values
  float *kc = a.kv + b * d.seq_stride + (a.layer * 2) * d.max_seq * kv_dim + kvh * d.max_seq * hd;
  float *vc = kc + d.max_seq * kv_dim;
  const unsigned row_bytes = unsigned(hd * sizeof(float));

  __syncthreads();  // whatever used this shared memory before is done
  // cached rows of the slice: all in flight at once
  if (tid == 0) {
    fence_proxy_async_smem();  // earlier generic-proxy accesses of this memory precede the asynchronous writes
#ifdef LMB_DEBUG_BOUNDS
    const bool slice_ok = LMB_IN_BOUNDS(size_t(vc - a.kv) + (t0 + n_old) * hd <= a.kv_floats, BOUNDS_KV_SLICE, size_t(vc - a.kv) + (t0 + n_old) * hd);
#else
    const bool slice_ok = true;
#endif
    mbar_arrive_expect_tx(bar, slice_ok ? unsigned(2 * n_old) * row_bytes : 0u);  // a refused slice is not copied
    if (n_old && slice_ok) {
      bulk_copy_g2s(Ks, kc + t0 * hd, unsigned(n_old) * row_bytes, bar);
      bulk_copy_g2s(Vs, vc + t0 * hd, unsigned(n_old) * row_bytes, bar);
    }
  }
  if constexpr (!FRESH_CG) {
    // a kernel of its own: the cached rows do not depend on the preceding kernel (they were written by
    // earlier steps), the fresh projections do
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (tid == 0) {
      tl_min(tl, 1);
      tl_max(tl, 2);
    }
  }
  // meanwhile: the group's rotated queries, and the new position's key / value (pairs (i, i + hd/2))
  const float *cs = a.cs_table + pos * hd;
  for (size_t i = tid; i < g * half; i += ATT_THREADS) {
    const size_t h = i / half, j = i - h * half, head = kvh * g + h;
    const float c = cs[j], sn = cs[half + j];
    const size_t i0 = (b * d.nh + head) * hd + j;
    float x0 = ld_fresh<FRESH_CG>(a.q + i0), x1 = ld_fresh<FRESH_CG>(a.q + i0 + half);
    if (a.qb) {
      x0 += a.qb[head * hd + j];
      x1 += a.qb[head * hd + j + half];
    }
    qs[h * hd + j] = x0 * c - x1 * sn;
    qs[h * hd + j + half] = x0 * sn + x1 * c;
  }
  if (has_new) {
    for (size_t j = tid; j < half; j += ATT_THREADS) {
      const float c = cs[j], sn = cs[half + j];
      const size_t k0 = (b * d.nkv + kvh) * hd + j;
      float y0 = ld_fresh<FRESH_CG>(a.k + k0), y1 = ld_fresh<FRESH_CG>(a.k + k0 + half);
      float v0 = ld_fresh<FRESH_CG>(a.v + k0), v1 = ld_fresh<FRESH_CG>(a.v + k0 + half);
      if (a.kb) {
        y0 += a.kb[kvh * hd + j];
        y1 += a.kb[kvh * hd + j + half];
      }
      if (a.vb) {
        v0 += a.vb[kvh * hd + j];
        v1 += a.vb[kvh * hd + j + half];
      }
      const float r0 = y0 * c - y1 * sn, r1 = y0 * sn + y1 * c;
      float *kr = Ks + n_old * hd, *vr = Vs + n_old * hd;
      kr[j] = r0; kr[j + half] = r1;
      vr[j] = v0; vr[j + half] = v1;
      kc[pos * hd + j] = r0; kc[pos * hd + j + half] = r1;  // this CTA is the only one that holds the position
      vc[pos * hd + j] = v0; vc[pos * hd + j + half] = v1;
    }
  }
  {  // bounded wait for the copies
    unsigned spins = 0;
    bool ok = true;
    while (!mbar_try_wait(bar, parity)) {
      if (++spins > spin_limit) {
        ok = false;
        break;
      }
    }
    parity ^= 1u;
    if (tid == 0) *flag = 1;
    __syncthreads();
    if (!ok) *flag = 0;  // any thread that gave up
    __syncthreads();
    if (*flag == 0) return false;
  }
  if (dbg && tid == 0) asm volatile("mov.u64 %0, %globaltimer;" : "=l"(dbg[0]));
  if (tid == 0) tl_max(tl, 3);
  // scores: a warp per timestep, a lane per PER dimensions
  const float scale = 1.0f / sqrtf(float(hd));
  LaneVec<PER> qreg[WIDE ? ATT_MAX_GROUP : 1];
  if constexpr (WIDE) {
#pragma unroll
    for (int h = 0; h < ATT_MAX_GROUP; ++h) {
      if (size_t(h) < g) {
        qreg[h] = ld_lane_vec<PER>(qs + h * hd, lane);
      } else {
#pragma unroll
        for (int e = 0; e < PER; ++e) qreg[h].v[e] = 0.0f;
      }
    }
  }
  for (size_t t = warp; t < n; t += nw) {
    const LaneVec<PER> kk = ld_lane_vec<PER>(Ks + t * hd, lane);
    float s[ATT_MAX_GROUP];
#pragma unroll
    for (int h = 0; h < ATT_MAX_GROUP; ++h) {
      s[h] = 0.0f;
      if constexpr (WIDE) {
#pragma unroll
        for (int e = 0; e < PER; ++e) s[h] += qreg[h].v[e] * kk.v[e];
      } else if (size_t(h) < g) {
        const LaneVec<PER> qv = ld_lane_vec<PER>(qs + h * hd, lane);
#pragma unroll
        for (int e = 0; e < PER; ++e) s[h] += qv.v[e] * kk.v[e];
      }
    }
    // Eight sums per lane to reduce over the 32 lanes: each step halves the values a lane carries
    // (it keeps one half of the heads and hands the other half to its partner), 4 + 2 + 1 + 1 + 1
    // shuffles instead of 8 x 5.  Lane l ends with the total of head 4*bit4(l) + 2*bit3(l) + bit2(l).
    float a4[4], a2[2];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float keep = (lane & 16) ? s[4 + i] : s[i], give = (lane & 16) ? s[i] : s[4 + i];
      a4[i] = keep + __shfl_xor_sync(0xffffffffu, give, 16);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const float keep = (lane & 8) ? a4[2 + i] : a4[i], give = (lane & 8) ? a4[i] : a4[2 + i];
      a2[i] = keep + __shfl_xor_sync(0xffffffffu, give, 8);
    }
    float a1 = ((lane & 4) ? a2[1] : a2[0]) + __shfl_xor_sync(0xffffffffu, (lane & 4) ? a2[0] : a2[1], 4);
    a1 += __shfl_xor_sync(0xffffffffu, a1, 2);
    a1 += __shfl_xor_sync(0xffffffffu, a1, 1);
    const int hsel = ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1);
    if ((lane & 3) == 0 && size_t(hsel) < g) sc[hsel * sl + t] = a1 * scale;
  }
  __syncthreads();
  // softmax of the slice (attention.cpp:23-42 per head), a warp per head
  for (size_t h = warp; h < g; h += nw) {
    float mx = -INFINITY;
    for (size_t t = lane; t < n; t += 32) mx = fmaxf(mx, sc[h * sl + t]);
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, m));
    float sum = 0.0f;
    for (size_t t = lane; t < n; t += 32) {
      const float e = expf(sc[h * sl + t] - mx);
      sc[h * sl + t] = e;
      sum += e;
    }
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, m);
    if (lane == 0) {
      stat[2 * h] = mx;
      stat[2 * h + 1] = sum;
    }
  }
  __syncthreads();
  // weighted values; the partial record of (head, split)
  const size_t rec = hd + ATT_REC_PAD;
  if (WIDE && sl >= size_t(nw - 1) * g && nw == 8) {
    // A warp per timestep (w, w + 8, ...), every lane keeping its dimensions of all heads: a value row is
    // read once for the whole group.  The eight warps' sums meet in the key area, which is free now:
    // warp w keeps head w for itself and leaves the other heads where their warps add them up.
    LaneVec<PER> acc[ATT_MAX_GROUP];
#pragma unroll
    for (int h = 0; h < ATT_MAX_GROUP; ++h)
#pragma unroll
      for (int e = 0; e < PER; ++e) acc[h].v[e] = 0.0f;
    for (size_t t = warp; t < n; t += nw) {
      const LaneVec<PER> vv = ld_lane_vec<PER>(Vs + t * hd, lane);
#pragma unroll
      for (int h = 0; h < ATT_MAX_GROUP; ++h) {
        if (size_t(h) < g) {
          const float pt = sc[h * sl + t];
#pragma unroll
          for (int e = 0; e < PER; ++e) acc[h].v[e] += pt * vv.v[e];
        }
      }
    }
    float *red = Ks;  // [head][7 other warps][hd]
#pragma unroll
    for (int h = 0; h < ATT_MAX_GROUP; ++h)
      if (size_t(h) < g && h != warp) st_lane_vec<PER>(red + (size_t(h) * (nw - 1) + size_t(warp - (warp > h ? 1 : 0))) * hd, lane, acc[h]);
    __syncthreads();
    if (size_t(warp) < g) {
      LaneVec<PER> tot;
#pragma unroll
      for (int h = 0; h < ATT_MAX_GROUP; ++h)
        if (h == warp) tot = acc[h];
      // warps in index order, as a sequential sum over the timesteps of each warp would give
      LaneVec<PER> sum;
#pragma unroll
      for (int e = 0; e < PER; ++e) sum.v[e] = 0.0f;
      for (int w = 0; w < nw; ++w) {
        const LaneVec<PER> part = w == warp ? tot : ld_lane_vec<PER>(red + (size_t(warp) * (nw - 1) + size_t(w - (w > warp ? 1 : 0))) * hd, lane);
#pragma unroll
        for (int e = 0; e < PER; ++e) sum.v[e] += part.v[e];
      }
      float *prt = a.partial + ((b * d.nh + kvh * g + size_t(warp)) * n_splits + split) * rec;
      st_lane_vec<PER>(prt, lane, sum);
      if (lane == 0) {
        prt[hd] = stat[2 * warp];
        prt[hd + 1] = stat[2 * warp + 1];
      }
    }
  } else {
    // short slices: a warp per head walks the timesteps
    for (size_t h = warp; h < g; h += nw) {
      LaneVec<PER> acc;
#pragma unroll
      for (int e = 0; e < PER; ++e) acc.v[e] = 0.0f;
      for (size_t t = 0; t < n; ++t) {
        const float pt = sc[h * sl + t];
        const LaneVec<PER> vv = ld_lane_vec<PER>(Vs + t * hd, lane);
#pragma unroll
        for (int e = 0; e < PER; ++e) acc.v[e] += pt * vv.v[e];
      }
      float *prt = a.partial + ((b * d.nh + kvh * g + h) * n_splits + split) * rec;
      st_lane_vec<PER>(prt, lane, acc);
      if (lane == 0) {
        prt[hd] = stat[2 * h];
        prt[hd + 1] = stat[2 * h + 1];
      }
    }
  }
  __syncthreads();
  if (dbg && tid == 0) asm volatile("mov.u64 %0, %globaltimer;" : "=l"(dbg[1]));
  if (tid == 0) tl_max(tl, 4);
  unsigned *ctr = a.counters + b * d.nkv + kvh;
  if (tid == 0) {
    unsigned before;  // release: this CTA's partial records; acquire: the other splits' records
    asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(before) : "l"(ctr) : "memory");
    *flag = (before == unsigned(n_splits - 1));
  }
  __syncthreads();
  if (*flag == 0) {
    if (tid == 0) tl_min(tl, 6);
    return true;
  }
  // merge by the last split of the KV head: a warp per query head of the group
  for (size_t h = warp; h < g; h += nw) {
    const size_t head = kvh * g + h;
    const float *all = a.partial + ((b * d.nh + head) * n_splits) * rec;
    float *w = wk + h * ATT_MAX_SPLITS;
    float den;
    LaneVec<PER> tot;
#pragma unroll
    for (int e = 0; e < PER; ++e) tot.v[e] = 0.0f;
    if constexpr (WIDE) {
      // statistics of all slices in one round trip: lane l holds slices l and l + 32 (ATT_MAX_SPLITS = 64)
      const bool h0 = lane < n_splits, h1 = lane + 32 < n_splits;
      const float2 st0 = h0 ? __ldcg(reinterpret_cast<const float2 *>(all + lane * rec + hd)) : make_float2(-INFINITY, 0.0f);
      const float2 st1 = h1 ? __ldcg(reinterpret_cast<const float2 *>(all + (lane + 32) * rec + hd)) : make_float2(-INFINITY, 0.0f);
      float gmx = fmaxf(st0.x, st1.x);
#pragma unroll
      for (int m = 16; m > 0; m >>= 1) gmx = fmaxf(gmx, __shfl_xor_sync(0xffffffffu, gmx, m));
      const float w0 = st0.y > 0.0f ? expf(st0.x - gmx) : 0.0f;  // empty slices (short contexts) weigh nothing
      const float w1 = st1.y > 0.0f ? expf(st1.x - gmx) : 0.0f;
      if (h0) w[lane] = w0;
      if (h1) w[lane + 32] = w1;
      den = w0 * st0.y + w1 * st1.y;
#pragma unroll
      for (int m = 16; m > 0; m >>= 1) den += __shfl_xor_sync(0xffffffffu, den, m);
      __syncwarp();
      int s2 = 0;
      constexpr int FLY = PER == 4 ? 16 : 24;  // records in flight per lane
      for (; s2 < n_splits; s2 += FLY) {  // the last round is partly empty: its loads are skipped, not serialised
        LaneVec<PER> pv[FLY];
#pragma unroll
        for (int i = 0; i < FLY; ++i)
          if (s2 + i < n_splits) pv[i] = ldcg_lane_vec<PER>(all + (s2 + i) * rec, lane);
#pragma unroll
        for (int i = 0; i < FLY; ++i)
          if (s2 + i < n_splits) {
#pragma unroll
            for (int e = 0; e < PER; ++e) tot.v[e] += w[s2 + i] * pv[i].v[e];
          }
      }
    } else {
      float gmx = -INFINITY;
      for (int s2 = lane; s2 < n_splits; s2 += 32) gmx = fmaxf(gmx, __ldcg(all + s2 * rec + hd));
#pragma unroll
      for (int m = 16; m > 0; m >>= 1) gmx = fmaxf(gmx, __shfl_xor_sync(0xffffffffu, gmx, m));
      den = 0.0f;
      for (int s2 = lane; s2 < n_splits; s2 += 32) {
        const float sm2 = __ldcg(all + s2 * rec + hd + 1);
        const float ws = sm2 > 0.0f ? expf(__ldcg(all + s2 * rec + hd) - gmx) : 0.0f;  // empty slices (short contexts) weigh nothing
        w[s2] = ws;
        den += ws * sm2;
      }
#pragma unroll
      for (int m = 16; m > 0; m >>= 1) den += __shfl_xor_sync(0xffffffffu, den, m);
      __syncwarp();
      int s2 = 0;
      for (; s2 + 7 < n_splits; s2 += 8) {  // eight records in flight per lane
        LaneVec<PER> pv[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) pv[i] = ldcg_lane_vec<PER>(all + (s2 + i) * rec, lane);
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
          for (int e = 0; e < PER; ++e) tot.v[e] += w[s2 + i] * pv[i].v[e];
      }
      for (; s2 < n_splits; ++s2) {
        const LaneVec<PER> pv = ldcg_lane_vec<PER>(all + s2 * rec, lane);
#pragma unroll
        for (int e = 0; e < PER; ++e) tot.v[e] += w[s2] * pv.v[e];
      }
    }
    const float inv = 1.0f / den;
#pragma unroll
    for (int e = 0; e < PER; ++e) tot.v[e] *= inv;
    st_lane_vec<PER>(a.out + (b * d.nh + head) * hd, lane, tot);
  }
  if (tid == 0) *ctr = 0u;
  if (tid == 0) tl_max(tl, 5);
  return true;
}

}  // namespace

}  // namespace lmb
