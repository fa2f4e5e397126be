// Launchers of the decode-step glue kernels (decode_ops.cu).
#pragma once

#include "common.cuh"

namespace lmb {

struct RopeDims {
  size_t nh, nkv, hd;   // local query heads, local KV heads, head dim
  size_t max_seq;       // cache slots per sequence
  size_t seq_stride;    // floats between the caches of consecutive sequences
  size_t split_len;     // longest KV slice of one attention CTA (set by the launcher)
};

int configure_decode_ops(lmb_ctx *ctx);
int launch_embed_rows(lmb_ctx *ctx, const int *d_tokens, const lmb_weight *embed, size_t vocab, size_t h, size_t batch,
                      float scale, float *d_hidden);
int launch_add_rmsnorm(lmb_ctx *ctx, float *d_hidden, const float *d_add, const float *d_w, float *d_out, size_t h,
                       size_t batch, float eps);
// hidden += sum over ranks of the partial vectors in the exchange block; out = RMSNorm(hidden) * w
int launch_tp_sum_add_rmsnorm(lmb_ctx *ctx, float *d_hidden, const float *d_w, float *d_out, size_t h, size_t batch, float eps);
int decode_attn_splits(const lmb_ctx *ctx, size_t nh, size_t batch, size_t max_seq);
int launch_decode_attn(lmb_ctx *ctx, const float *q, const float *k, const float *v, const float *qb, const float *kb,
                       const float *vb, const float *cs_table, const size_t *positions, float *kv, float *out,
                       float *partial, unsigned *counters, int n_splits, size_t layer, const RopeDims &d, size_t batch);
// Group form of the decode attention (one CTA per KV head, split and sequence; keys and values of a
// slice fetched once with bulk asynchronous copies).  plan_attn_group sizes the KV splits so that a
// slice's rows fit `smem_bytes` of shared memory and about `want_items` CTAs result; ok = false
// when the shape is outside what the group form handles (more than 8 query heads per KV head, a
// head_dim other than 64 or 128, a context that needs more than 64 splits).
constexpr size_t ATTN_GROUP_SMEM = 72 * 1024;  // shared memory a group-attention CTA may use (two CTAs per SM)
struct AttnGroupPlan {
  bool ok;
  int n_splits, per;  // per = head_dim / 32
  size_t split_len, smem_bytes;
};
AttnGroupPlan plan_attn_group(size_t nh, size_t nkv, size_t hd, size_t max_seq, size_t batch, size_t want_items, size_t smem_bytes);
int launch_decode_attn_group(lmb_ctx *ctx, const float *q, const float *k, const float *v, const float *qb, const float *kb,
                             const float *vb, const float *cs_table, const size_t *positions, float *kv, float *out,
                             float *partial, unsigned *counters, const AttnGroupPlan &plan, size_t layer, const RopeDims &d,
                             size_t batch);
size_t attn_partial_floats(size_t batch, size_t nh, size_t hd);  // scratch both attention forms fit in
// dst[b][r * n + i] = src[r][b][i]: the gathered per-rank logits slabs into rows of the full vocabulary
int launch_interleave_rows(lmb_ctx *ctx, const float *src, float *dst, size_t ranks, size_t batch, size_t n);
int launch_silu_mul(lmb_ctx *ctx, const float *gate, const float *up, float *out, size_t n, bool gelu = false);

}  // namespace lmb
