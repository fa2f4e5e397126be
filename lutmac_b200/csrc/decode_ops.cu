// Glue kernels of one decode step, all fp32 like the reference: embedding-row dequantisation
// (src/model.cpp:58-252), RMSNorm with fused residual add (src/layers/norm.cpp:18-34,
// model.cpp:385-399), GQA decode attention with bias + RoPE + KV-cache write folded in
// (model.cpp:312-372, src/layers/embedding.cpp:36-75, src/layers/attention.cpp:23-42) and SiLU(gate)*up (model.cpp:36,414-416).
#include "decode_device.cuh"
#include "device_utils.cuh"

#include <algorithm>
#include <cstdlib>

namespace lmb {

namespace {

__global__ void k_embed_rows(const int *tokens, int kind, const uint8_t *tiles, size_t bpr, size_t vocab, size_t h,
                             float scale, float *hidden) {
  asm volatile("griddepcontrol.launch_dependents;");  // a following GEMV may prefetch its weights
  const size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= h) return;
  const int tok = tokens[blockIdx.y];
  // rows beyond the table read as zero (model.cpp:95-104)
  // gemma-type models scale the row by sqrt(hidden size) (model.cpp:255-260); scale = 1 otherwise
  hidden[size_t(blockIdx.y) * h + i] = (tok >= 0 && size_t(tok) < vocab) ? tile_elem(kind, tiles, bpr, size_t(tok), i) * scale : 0.0f;
}

// hidden += add (if given); out = hidden * rsqrt(mean(hidden^2) + eps) * w.  One CTA per sequence.
__global__ void __launch_bounds__(1024) k_add_rmsnorm(float *hidden, const float *add, const float *w, float *out,
                                                      size_t h, float eps) {
  asm volatile("griddepcontrol.launch_dependents;");  // a following GEMV may prefetch its weights
  __shared__ float red[32];
  float *x = hidden + size_t(blockIdx.x) * h;
  const float *a = add ? add + size_t(blockIdx.x) * h : nullptr;
  float *o = out + size_t(blockIdx.x) * h;
  float ss = 0.0f;
  for (size_t i = threadIdx.x; i < h; i += blockDim.x) {
    float v = x[i];
    if (a) {
      v += a[i];
      x[i] = v;
    }
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / float(h) + eps);
  for (size_t i = threadIdx.x; i < h; i += blockDim.x) o[i] = x[i] * inv * w[i];
}

// Tensor-parallel form of k_add_rmsnorm: the vector to add is the sum over ranks of the partial
// vectors in this rank's exchange block.  Every element is an 8-byte word {value, epoch tag}
// written by its producer with one store; the reader polls the word (bounded) until the tag is
// the expected one, adds the partials in rank order (so that every rank computes the same bits),
// then normalises.  One CTA per sequence; the last CTA to finish advances the epoch.
__device__ __forceinline__ unsigned long long ld_volatile_u64(const unsigned long long *p) {
  unsigned long long v;
  asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(1024) k_tp_sum_add_rmsnorm(float *hidden, XchgHeader *hdr, const unsigned long long *data, int tp,
                                                             unsigned cap, const float *w, float *out, size_t h, float eps,
                                                             unsigned spin_limit) {
  asm volatile("griddepcontrol.launch_dependents;");
  __shared__ float red[32];
  const unsigned epoch = *reinterpret_cast<volatile unsigned *>(&hdr->epoch);
  const unsigned tag = epoch + 1u;
  const unsigned long long *part = data + size_t(epoch & 1u) * tp * cap + size_t(blockIdx.x) * h;
  float *x = hidden + size_t(blockIdx.x) * h;
  float *o = out + size_t(blockIdx.x) * h;
  float ss = 0.0f;
  bool gave_up = *reinterpret_cast<volatile unsigned *>(&hdr->timed_out) != 0u;
  for (size_t i = threadIdx.x; i < h; i += blockDim.x) {
    float add = 0.0f;
    for (int r = 0; r < tp; ++r) {
      const unsigned long long *src = part + size_t(r) * cap + i;
      unsigned long long word = ld_volatile_u64(src);
      unsigned spins = 0;
      while (unsigned(word >> 32) != tag && !gave_up) {
        if (++spins > spin_limit) {  // give up, report, carry on with what is there
          hdr->timed_out = 1u;
          gave_up = true;
          break;
        }
        __nanosleep(40);
        word = ld_volatile_u64(src);
      }
      add += __uint_as_float(unsigned(word));
    }
    const float v = x[i] + add;
    x[i] = v;
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / float(h) + eps);
  for (size_t i = threadIdx.x; i < h; i += blockDim.x) o[i] = x[i] * inv * w[i];
  __syncthreads();
  if (threadIdx.x == 0 && atomicAdd(&hdr->done, 1u) == gridDim.x - 1u) {
    hdr->done = 0u;
    *reinterpret_cast<volatile unsigned *>(&hdr->epoch) = tag;  // read by the next producer, a later kernel
  }
}

__global__ void __launch_bounds__(ATT_THREADS) k_decode_attn(const AttnArgs a, const RopeDims d) {
  asm volatile("griddepcontrol.launch_dependents;");  // a following GEMV may prefetch its weights
  extern __shared__ float sm[];
  __shared__ int is_last;
  attn_item<false>(a, d, blockIdx.x, blockIdx.y, blockIdx.z, sm, &is_last);
}

// Group attention as a kernel of its own: grid = (KV heads x splits, sequences).
template <int PER, bool WIDE>
__global__ void __launch_bounds__(ATT_THREADS) k_decode_attn_group(const AttnArgs a, const RopeDims d, unsigned spin_limit,
                                                                    unsigned *timed_out, unsigned long long *tl) {
  asm volatile("griddepcontrol.launch_dependents;");
  if (threadIdx.x == 0) tl_min(tl, 0);
  extern __shared__ __align__(16) float sm[];
  __shared__ __align__(8) uint64_t bar;
  __shared__ int flag;
  if (threadIdx.x == 0) mbar_init(&bar, 1);
  __syncthreads();
  unsigned parity = 0;
  const size_t kvh = blockIdx.x % d.nkv, split = blockIdx.x / d.nkv;
  if (!attn_group_item<false, PER, WIDE>(a, d, kvh, split, blockIdx.y, sm, &bar, parity, spin_limit, &flag, nullptr, tl) && threadIdx.x == 0 &&
      timed_out)
    *timed_out = 1u;
}

__global__ void k_interleave_rows(const float *src, float *dst, size_t ranks, size_t batch, size_t n) {
  const size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x, total = ranks * batch * n;
  if (i >= total) return;
  const size_t r = i / (batch * n), b = (i / n) % batch, j = i % n;
  dst[b * ranks * n + r * n + j] = src[i];
}

__global__ void k_silu_mul(const float *gate, const float *up, float *out, size_t n, int gelu) {
  asm volatile("griddepcontrol.launch_dependents;");  // a following GEMV may prefetch its weights
  const size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) {
    const float g = gate[i];
    out[i] = (gelu ? gelu_tanh(g) : g / (1.0f + expf(-g))) * up[i];
  }
}

}  // namespace

int launch_embed_rows(lmb_ctx *ctx, const int *d_tokens, const lmb_weight *embed, size_t vocab, size_t h, size_t batch,
                      float scale, float *d_hidden) {
  dim3 grid(unsigned((h + 255) / 256), unsigned(batch));
  k_embed_rows<<<grid, 256, 0, ctx->stream>>>(d_tokens, embed->kind, embed->d_tiles, embed->bpr, vocab, h, scale, d_hidden);
  ctx->launches++;
  LMB_CUDA(cudaGetLastError());
  return LMB_OK;
}

int launch_add_rmsnorm(lmb_ctx *ctx, float *d_hidden, const float *d_add, const float *d_w, float *d_out, size_t h,
                       size_t batch, float eps) {
  const int threads = h >= 4096 ? 1024 : (h >= 1024 ? 512 : 256);
  k_add_rmsnorm<<<unsigned(batch), threads, 0, ctx->stream>>>(d_hidden, d_add, d_w, d_out, h, eps);
  ctx->launches++;
  LMB_CUDA(cudaGetLastError());
  return LMB_OK;
}

int launch_tp_sum_add_rmsnorm(lmb_ctx *ctx, float *d_hidden, const float *d_w, float *d_out, size_t h, size_t batch, float eps) {
  if (!ctx->xchg.ready || batch * h > ctx->xchg.cap) {
    set_last_error("tensor-parallel sum: exchange block missing or too small");
    return LMB_ERR_STATE;
  }
  const int threads = h >= 4096 ? 1024 : (h >= 1024 ? 512 : 256);
  XchgHeader *hdr = static_cast<XchgHeader *>(ctx->xchg.local);
  const unsigned long long *data =
      reinterpret_cast<const unsigned long long *>(static_cast<const char *>(ctx->xchg.local) + XCHG_HEADER_BYTES);
  k_tp_sum_add_rmsnorm<<<unsigned(batch), threads, 0, ctx->stream>>>(d_hidden, hdr, data, ctx->tp_size, unsigned(ctx->xchg.cap),
                                                                     d_w, d_out, h, eps, ctx->xchg.spin_limit);
  ctx->launches++;
  LMB_CUDA(cudaGetLastError());
  return LMB_OK;
}

int decode_attn_splits(const lmb_ctx *ctx, size_t nh, size_t batch, size_t max_seq) {
  size_t n = (size_t(2) * ctx->sm_count + nh * batch - 1) / (nh * batch);
  const size_t most = (max_seq + 63) / 64;  // no slice shorter than 64 timesteps at full context
  n = n < 1 ? 1 : (n > 32 ? 32 : n);
  return int(n > most ? most : n);
}

// q/k/v are the fresh projections of this step; the kernel applies bias and RoPE, writes the new
// position into the cache and attends over positions 0..pos.
int launch_decode_attn(lmb_ctx *ctx, const float *q, const float *k, const float *v, const float *qb, const float *kb,
                       const float *vb, const float *cs_table, const size_t *positions, float *kv, float *out,
                       float *partial, unsigned *counters, int n_splits, size_t layer, const RopeDims &d0, size_t batch) {
  RopeDims d = d0;
  if (d.hd > ATT_THREADS || d.hd == 0 || ATT_THREADS % d.hd != 0 || d.hd % 2 != 0) {
    set_last_error("decode attention: head_dim must be even and divide 256");
    return LMB_ERR_ARG;
  }
  size_t len = (d.max_seq + n_splits - 1) / n_splits;
  d.split_len = (len + 15) / 16 * 16;
  const size_t smem = (d.split_len + 3 * d.hd + 32 + ATT_THREADS) * sizeof(float);
  AttnArgs a{q, k, v, qb, kb, vb, cs_table, positions, kv, out, partial, counters, n_splits, layer};
  dim3 grid(unsigned(d.nh), unsigned(n_splits), unsigned(batch));
  k_decode_attn<<<grid, ATT_THREADS, smem, ctx->stream>>>(a, d);
  ctx->launches++;
  LMB_CUDA(cudaGetLastError());
  return LMB_OK;
}

size_t attn_partial_floats(size_t batch, size_t nh, size_t hd) { return batch * nh * ATT_MAX_SPLITS * (hd + ATT_REC_PAD); }

AttnGroupPlan plan_attn_group(size_t nh, size_t nkv, size_t hd, size_t max_seq, size_t batch, size_t want_items, size_t smem_bytes) {
  AttnGroupPlan pl{false, 1, 0, 0, 0};
  if (nkv == 0 || nh % nkv != 0) return pl;
  const size_t g = nh / nkv;
  if (g > size_t(ATT_MAX_GROUP) || (hd != 64 && hd != 128)) return pl;
  pl.per = int(hd / 32);
  // longest slice whose rows, queries and scores fit
  const size_t fixed = g * hd + size_t(ATT_MAX_GROUP) * ATT_MAX_SPLITS + 2 * ATT_MAX_GROUP, budget = smem_bytes / sizeof(float);
  if (budget <= fixed + 8 * (2 * hd + g)) return pl;
  const size_t cap = (budget - fixed) / (2 * hd + g) / 8 * 8;
  const size_t min_splits = (max_seq + cap - 1) / cap;
  size_t want = (want_items + nkv * batch - 1) / (nkv * batch);
  size_t n = std::max(min_splits, std::max<size_t>(want, 1));
  n = std::min<size_t>(n, ATT_MAX_SPLITS);
  n = std::min<size_t>(n, std::max<size_t>(1, (max_seq + 7) / 8));  // no slice shorter than 8 positions at full context
  if (n < min_splits) return pl;
  pl.n_splits = int(n);
  pl.split_len = ((max_seq + n - 1) / n + 7) / 8 * 8;
  if (pl.split_len > cap) return pl;
  pl.smem_bytes = attn_group_smem_floats(pl.split_len, hd, g) * sizeof(float);
  pl.ok = true;
  return pl;
}

int launch_decode_attn_group(lmb_ctx *ctx, const float *q, const float *k, const float *v, const float *qb, const float *kb,
                             const float *vb, const float *cs_table, const size_t *positions, float *kv, float *out,
                             float *partial, unsigned *counters, const AttnGroupPlan &plan, size_t layer, const RopeDims &d0,
                             size_t batch) {
  RopeDims d = d0;
  d.split_len = plan.split_len;
  AttnArgs a{q, k, v, qb, kb, vb, cs_table, positions, kv, out, partial, counters, plan.n_splits, layer};
#ifdef LMB_DEBUG_BOUNDS
  a.kv_floats = d.seq_stride * batch;  // the cache holds at least the sequences of this launch
#endif
  dim3 grid(unsigned(d.nkv * size_t(plan.n_splits)), unsigned(batch));
  unsigned *flag = ctx->d_fault;  // set when a bounded wait for the bulk copies runs out
  // programmatic dependent launch: the CTAs start fetching their cache slices while the q/k/v
  // projections finish, and wait for those only before they read the fresh vectors
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(ATT_THREADS);
  cfg.dynamicSmemBytes = plan.smem_bytes;
  cfg.stream = ctx->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  static const bool attn_pdl = [] {  // LMB_ATTN_PDL=0: the attention kernel starts only when the q/k/v projections have finished
    const char *e = std::getenv("LMB_ATTN_PDL");
    return !(e && e[0] == '0');
  }();
  cfg.numAttrs = ctx->pdl && attn_pdl ? 1 : 0;
  unsigned long long *tl = timeline_slot(ctx);
  // one sequence: one wave of CTAs, bound by their latency (the WIDE form); several: many waves, bound by throughput
  if (batch == 1) {
    if (plan.per == 4) LMB_CUDA(cudaLaunchKernelEx(&cfg, k_decode_attn_group<4, true>, a, d, ctx->xchg.spin_limit, flag, tl));
    else LMB_CUDA(cudaLaunchKernelEx(&cfg, k_decode_attn_group<2, true>, a, d, ctx->xchg.spin_limit, flag, tl));
  } else {
    if (plan.per == 4) LMB_CUDA(cudaLaunchKernelEx(&cfg, k_decode_attn_group<4, false>, a, d, ctx->xchg.spin_limit, flag, tl));
    else LMB_CUDA(cudaLaunchKernelEx(&cfg, k_decode_attn_group<2, false>, a, d, ctx->xchg.spin_limit, flag, tl));
  }
  ctx->launches++;
  return LMB_OK;
}

int launch_interleave_rows(lmb_ctx *ctx, const float *src, float *dst, size_t ranks, size_t batch, size_t n) {
  const size_t total = ranks * batch * n;
  k_interleave_rows<<<unsigned((total + 255) / 256), 256, 0, ctx->stream>>>(src, dst, ranks, batch, n);
  ctx->launches++;
  LMB_CUDA(cudaGetLastError());
  return LMB_OK;
}

int launch_silu_mul(lmb_ctx *ctx, const float *gate, const float *up, float *out, size_t n, bool gelu) {
  k_silu_mul<<<unsigned((n + 255) / 256), 256, 0, ctx->stream>>>(gate, up, out, n, gelu ? 1 : 0);
  ctx->launches++;
  LMB_CUDA(cudaGetLastError());
  return LMB_OK;
}

int configure_decode_ops(lmb_ctx *ctx) {
  LMB_CUDA(cudaFuncSetAttribute(k_decode_attn, cudaFuncAttributeMaxDynamicSharedMemorySize, int(ctx->smem_optin) - 1024));
  LMB_CUDA(cudaFuncSetAttribute(k_decode_attn_group<4, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(ATTN_GROUP_SMEM)));
  LMB_CUDA(cudaFuncSetAttribute(k_decode_attn_group<2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(ATTN_GROUP_SMEM)));
  LMB_CUDA(cudaFuncSetAttribute(k_decode_attn_group<4, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(ATTN_GROUP_SMEM)));
  LMB_CUDA(cudaFuncSetAttribute(k_decode_attn_group<2, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(ATTN_GROUP_SMEM)));
  return LMB_OK;
}

}  // namespace lmb
