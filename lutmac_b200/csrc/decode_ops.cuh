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
int launch_silu_mul(lmb_ctx *ctx, const float *gate, const float *up, float *out, size_t n, bool gelu = false);

}  // namespace lmb
