// Device-resident decoder: replaces Model::allocate / Model::forward / get_logits / reset_cache
// (include/lutmac/model.hpp:88-141, src/model.cpp:47-453) for the llama-type path (RMSNorm,
// RoPE half-split pairs, GQA attention over an fp32 KV cache, SwiGLU FFN, quantised lm_head).
// Only token ids and positions go in and logits come out; weights, activations and the KV
// cache stay in HBM.  Batched decode runs `batch` independent sequences through the same
// weights; tensor parallelism keeps a shard per rank and adds two all-reduces per layer.
#include <dlfcn.h>

#include <cmath>
#include <cstdlib>
#include <cstring>
#include <new>
#include <vector>

#include "model.cuh"

namespace lmb {

// ---- NCCL, bound at run time (the process may already hold a libnccl.so.2 of its own) ----------
struct Nccl {
  typedef struct { char internal[128]; } UniqueId;
  int (*GetUniqueId)(UniqueId *) = nullptr;
  int (*CommInitRank)(void **, int, UniqueId, int) = nullptr;
  int (*CommDestroy)(void *) = nullptr;
  int (*AllReduce)(const void *, void *, size_t, int, int, void *, cudaStream_t) = nullptr;
  int (*AllGather)(const void *, void *, size_t, int, void *, cudaStream_t) = nullptr;
  const char *(*GetErrorString)(int) = nullptr;
  bool ok = false;
};

static Nccl &nccl() {
  static Nccl n;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void *h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (h) {
      n.GetUniqueId = reinterpret_cast<decltype(n.GetUniqueId)>(dlsym(h, "ncclGetUniqueId"));
      n.CommInitRank = reinterpret_cast<decltype(n.CommInitRank)>(dlsym(h, "ncclCommInitRank"));
      n.CommDestroy = reinterpret_cast<decltype(n.CommDestroy)>(dlsym(h, "ncclCommDestroy"));
      n.AllReduce = reinterpret_cast<decltype(n.AllReduce)>(dlsym(h, "ncclAllReduce"));
      n.AllGather = reinterpret_cast<decltype(n.AllGather)>(dlsym(h, "ncclAllGather"));
      n.GetErrorString = reinterpret_cast<decltype(n.GetErrorString)>(dlsym(h, "ncclGetErrorString"));
      n.ok = n.GetUniqueId && n.CommInitRank && n.CommDestroy && n.AllReduce && n.AllGather && n.GetErrorString;
    }
  }
  return n;
}

static int nccl_fail(int rc, const char *what) {
  set_last_error(std::string(what) + ": " + (nccl().GetErrorString ? nccl().GetErrorString(rc) : "NCCL error"));
  return LMB_ERR_CUDA;
}

constexpr int NCCL_FLOAT = 7, NCCL_SUM = 0;

}  // namespace lmb

using namespace lmb;

// Whether batch-1 steps run as the persistent kernel when the environment does not say.  Measured
// on B200 (Llama-3-70B-shaped ternary stack, 2048 positions): on one GPU the waits between its
// phases cost about what the kernel boundaries of the launch-per-projection step cost, so it is
// opt-in there.
static constexpr bool PERSISTENT_BY_DEFAULT = false;

static int dev_alloc(float **p, size_t n) {
  LMB_CUDA(cudaMalloc(p, (n ? n : 1) * sizeof(float)));
  LMB_CUDA(cudaMemset(*p, 0, (n ? n : 1) * sizeof(float)));
  return LMB_OK;
}

extern "C" {

int lmb_tp_unique_id(void *id128_out) {
  LMB_REQUIRE(id128_out, "lmb_tp_unique_id: null argument");
  if (!nccl().ok) {
    set_last_error("lmb_tp_unique_id: libnccl.so.2 could not be loaded");
    return LMB_ERR_STATE;
  }
  Nccl::UniqueId id;
  int rc = nccl().GetUniqueId(&id);
  if (rc != 0) return nccl_fail(rc, "ncclGetUniqueId");
  std::memcpy(id128_out, &id, 128);
  return LMB_OK;
}

int lmb_tp_init(lmb_ctx *ctx, const void *id128, int rank, int size) {
  LMB_REQUIRE(ctx && id128 && size >= 1 && rank >= 0 && rank < size, "lmb_tp_init: bad argument");
  if (!nccl().ok) {
    set_last_error("lmb_tp_init: libnccl.so.2 could not be loaded");
    return LMB_ERR_STATE;
  }
  LMB_CUDA(cudaSetDevice(ctx->device));
  Nccl::UniqueId id;
  std::memcpy(&id, id128, 128);
  int rc = nccl().CommInitRank(&ctx->comm, size, id, rank);
  if (rc != 0) return nccl_fail(rc, "ncclCommInitRank");
  ctx->tp_rank = rank;
  ctx->tp_size = size;
  return LMB_OK;
}

int lmb_tp_peer_create(lmb_ctx *ctx, size_t max_floats, void *handle64_out) {
  LMB_REQUIRE(ctx && handle64_out && max_floats > 0, "lmb_tp_peer_create: bad argument");
  LMB_REQUIRE(ctx->tp_size > 1 && ctx->tp_size <= MAX_TP, "lmb_tp_peer_create: call lmb_tp_init first (2 to 8 ranks)");
  LMB_REQUIRE(!ctx->xchg.local, "lmb_tp_peer_create: the exchange block exists already");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  static_assert(sizeof(XchgHeader) <= XCHG_HEADER_BYTES, "exchange header size");
  LMB_CUDA(cudaSetDevice(ctx->device));
  const size_t cap = (max_floats + 63) / 64 * 64;
  const size_t bytes = XCHG_HEADER_BYTES + size_t(2) * ctx->tp_size * cap * sizeof(unsigned long long);
  void *blk = nullptr;
  LMB_CUDA(cudaMalloc(&blk, bytes));
  cudaError_t e = cudaMemset(blk, 0, bytes);
  cudaIpcMemHandle_t hnd;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&hnd, blk);
  if (e != cudaSuccess) {
    cudaFree(blk);
    return cuda_fail(e, "lmb_tp_peer_create");
  }
  std::memcpy(handle64_out, &hnd, 64);
  ctx->xchg.local = blk;
  ctx->xchg.cap = cap;
  return LMB_OK;
}

int lmb_tp_peer_open(lmb_ctx *ctx, const void *handles) {
  LMB_REQUIRE(ctx && handles && ctx->xchg.local && !ctx->xchg.ready, "lmb_tp_peer_open: create the local block first (once)");
  LMB_CUDA(cudaSetDevice(ctx->device));
  for (int r = 0; r < ctx->tp_size; ++r) {
    if (r == ctx->tp_rank) {
      ctx->xchg.peer[r] = ctx->xchg.local;
      continue;
    }
    cudaIpcMemHandle_t hnd;
    std::memcpy(&hnd, static_cast<const char *>(handles) + size_t(r) * 64, 64);
    LMB_CUDA(cudaIpcOpenMemHandle(&ctx->xchg.peer[r], hnd, cudaIpcMemLazyEnablePeerAccess));
  }
  if (const char *e = std::getenv("LMB_TP_WAIT_POLLS")) {  // polls per word before a consumer gives up (default 1 << 22: seconds)
    const long v = std::atol(e);
    if (v > 0 && v < (1l << 31)) ctx->xchg.spin_limit = unsigned(v);
  }
  ctx->xchg.ready = true;
  return LMB_OK;
}

int lmb_tp_peer_status(lmb_ctx *ctx, int *timed_out) {
  LMB_REQUIRE(ctx && timed_out, "lmb_tp_peer_status: null argument");
  *timed_out = 0;
  if (!ctx->xchg.local) return LMB_OK;
  unsigned v = 0;
  LMB_CUDA(cudaStreamSynchronize(ctx->stream));
  LMB_CUDA(cudaMemcpy(&v, &static_cast<XchgHeader *>(ctx->xchg.local)->timed_out, sizeof v, cudaMemcpyDeviceToHost));
  *timed_out = int(v);
  return LMB_OK;
}

static int tp_wait_selftest(lmb_ctx *ctx, int ranks, int posted, size_t h, unsigned spin_limit, int out4[4], bool prepare) {
  LMB_REQUIRE(ctx && out4 && ranks >= 2 && ranks <= MAX_TP && posted >= 0 && posted <= ranks && h > 0 && spin_limit > 0,
              "lmb_debug_tp_wait: bad argument");
  LMB_REQUIRE(!ctx->xchg.local, "lmb_debug_tp_wait: the context already has an exchange block");
  LMB_CUDA(cudaSetDevice(ctx->device));
  const size_t cap = (h + 63) / 64 * 64;
  const size_t bytes = XCHG_HEADER_BYTES + size_t(2) * ranks * cap * sizeof(unsigned long long);
  void *blk = nullptr;
  float *hidden = nullptr, *w = nullptr, *out = nullptr;
  std::vector<unsigned long long> words(size_t(2) * ranks * cap, 0ull);
  for (int r = 0; r < posted; ++r)  // epoch 0: parity 0, tag 1; value r + 1
    for (size_t i = 0; i < h; ++i) {
      const float v = float(r + 1);
      unsigned bits;
      std::memcpy(&bits, &v, 4);
      words[size_t(r) * cap + i] = (1ull << 32) | bits;
    }
  std::vector<float> ones(h, 1.0f), res(h, 0.0f);
  XchgHeader hdr;
  cudaError_t e = cudaMalloc(&blk, bytes);
  if (e == cudaSuccess) e = cudaMemset(blk, 0, XCHG_HEADER_BYTES);
  if (e == cudaSuccess) e = cudaMemcpy(static_cast<char *>(blk) + XCHG_HEADER_BYTES, words.data(), words.size() * 8, cudaMemcpyHostToDevice);
  if (e == cudaSuccess) e = cudaMalloc(&hidden, h * 4);
  if (e == cudaSuccess) e = cudaMalloc(&w, h * 4);
  if (e == cudaSuccess) e = cudaMalloc(&out, (h + h / BLK * (PREP_RECORD_WORDS + 1) + 64) * 4);
  if (e == cudaSuccess) e = cudaMemset(hidden, 0, h * 4);
  if (e == cudaSuccess) e = cudaMemcpy(w, ones.data(), h * 4, cudaMemcpyHostToDevice);
  int st = e == cudaSuccess ? LMB_OK : cuda_fail(e, "lmb_debug_tp_wait setup");
  if (st == LMB_OK) {
    // the context stands in for one rank of `ranks`; every "peer" block is the local one
    const PeerXchg saved = ctx->xchg;
    const int saved_size = ctx->tp_size;
    ctx->xchg.local = blk;
    ctx->xchg.cap = cap;
    ctx->xchg.ready = true;
    ctx->xchg.spin_limit = spin_limit;
    ctx->tp_size = ranks;
    // the prepared form writes h / 256 records and as many sums of squares into `out` (it is large enough: 260 + 1 words per 256)
    st = prepare ? launch_tp_sum_prepare(ctx, hidden, w, false, reinterpret_cast<uint32_t *>(out), out + h / BLK * PREP_RECORD_WORDS, h)
                 : launch_tp_sum_add_rmsnorm(ctx, hidden, w, out, h, 1, 1e-5f);
    ctx->xchg = saved;
    ctx->tp_size = saved_size;
    if (st == LMB_OK) e = cudaStreamSynchronize(ctx->stream);
    if (st == LMB_OK && e == cudaSuccess) e = cudaMemcpy(&hdr, blk, sizeof hdr, cudaMemcpyDeviceToHost);
    if (st == LMB_OK && e == cudaSuccess) e = cudaMemcpy(res.data(), hidden, h * 4, cudaMemcpyDeviceToHost);
    if (st == LMB_OK && e != cudaSuccess) st = cuda_fail(e, "lmb_debug_tp_wait");
  }
  if (st == LMB_OK) {
    const float want = float(posted * (posted + 1) / 2);  // sum of the posted partial vectors
    bool ok = true;
    for (size_t i = 0; i < h; ++i) ok = ok && res[i] == want;
    out4[0] = int(hdr.timed_out);
    out4[1] = int(hdr.epoch);
    out4[2] = int(hdr.done);
    out4[3] = ok ? 1 : 0;
  }
  if (blk) cudaFree(blk);
  if (hidden) cudaFree(hidden);
  if (w) cudaFree(w);
  if (out) cudaFree(out);
  return st;
}

int lmb_debug_tp_wait(lmb_ctx *ctx, int ranks, int posted, size_t h, unsigned spin_limit, int out4[4]) {
  return tp_wait_selftest(ctx, ranks, posted, h, spin_limit, out4, false);
}

int lmb_debug_tp_wait_prepare(lmb_ctx *ctx, int ranks, int posted, size_t h, unsigned spin_limit, int out4[4]) {
  LMB_REQUIRE(h % lmb::BLK == 0, "lmb_debug_tp_wait_prepare: h must be a multiple of 256");
  return tp_wait_selftest(ctx, ranks, posted, h, spin_limit, out4, true);
}

int lmb_tp_destroy(lmb_ctx *ctx) {
  LMB_REQUIRE(ctx, "lmb_tp_destroy: null context");
  if (ctx->xchg.local) {
    cudaStreamSynchronize(ctx->stream);
    for (int r = 0; r < ctx->tp_size; ++r)
      if (r != ctx->tp_rank && ctx->xchg.peer[r]) cudaIpcCloseMemHandle(ctx->xchg.peer[r]);
    cudaFree(ctx->xchg.local);
    ctx->xchg = PeerXchg();
  }
  if (ctx->comm) {
    cudaStreamSynchronize(ctx->stream);
    nccl().CommDestroy(ctx->comm);
    ctx->comm = nullptr;
  }
  ctx->tp_rank = 0;
  ctx->tp_size = 1;
  return LMB_OK;
}

int lmb_allreduce_sum(lmb_ctx *ctx, float *d_buf, size_t n) {
  LMB_REQUIRE(ctx && d_buf, "lmb_allreduce_sum: null argument");
  if (ctx->tp_size <= 1) return LMB_OK;
  int rc = nccl().AllReduce(d_buf, d_buf, n, NCCL_FLOAT, NCCL_SUM, ctx->comm, ctx->stream);
  if (rc != 0) return nccl_fail(rc, "ncclAllReduce");
  return LMB_OK;
}

int lmb_allgather(lmb_ctx *ctx, const float *d_send, float *d_recv, size_t n_per_rank) {
  LMB_REQUIRE(ctx && d_send && d_recv, "lmb_allgather: null argument");
  if (ctx->tp_size <= 1) {
    if (d_send != d_recv) LMB_CUDA(cudaMemcpyAsync(d_recv, d_send, n_per_rank * 4, cudaMemcpyDeviceToDevice, ctx->stream));
    return LMB_OK;
  }
  int rc = nccl().AllGather(d_send, d_recv, n_per_rank, NCCL_FLOAT, ctx->comm, ctx->stream);
  if (rc != 0) return nccl_fail(rc, "ncclAllGather");
  return LMB_OK;
}

}  // extern "C"

// ---- model ---------------------------------------------------------------------------------------
extern "C" {

int lmb_model_create(lmb_ctx *ctx, const lmb_model_config *c, lmb_model **out) {
  LMB_REQUIRE(ctx && c && out, "lmb_model_create: null argument");
  *out = nullptr;
  const int g = c->tp_size > 0 ? c->tp_size : 1;
  LMB_REQUIRE(c->tp_rank >= 0 && c->tp_rank < g, "lmb_model_create: tp_rank out of range");
  LMB_REQUIRE(g == 1 || (ctx->comm && ctx->tp_size == g && ctx->tp_rank == c->tp_rank),
              "lmb_model_create: tensor-parallel model needs lmb_tp_init on its context first");
  LMB_REQUIRE(c->vocab_size > 0 && c->hidden_size > 0 && c->intermediate_size > 0 && c->num_attention_heads > 0 &&
                  c->num_key_value_heads > 0,
              "lmb_model_create: vocab, hidden, intermediate sizes and head counts must be positive");
  LMB_REQUIRE(c->num_attention_heads % c->num_key_value_heads == 0, "lmb_model_create: heads not divisible by kv heads");
  LMB_REQUIRE(c->head_dim > 0 && c->head_dim % 2 == 0 && 256 % c->head_dim == 0, "lmb_model_create: head_dim must divide 256");
  LMB_REQUIRE(c->num_attention_heads % g == 0 && c->num_key_value_heads % g == 0 && c->intermediate_size % g == 0 &&
                  c->vocab_size % g == 0,
              "lmb_model_create: heads, kv heads, intermediate and vocab sizes must divide by tp_size");
  if (g > 1)
    LMB_REQUIRE((c->num_attention_heads / g * c->head_dim) % 256 == 0 && (c->intermediate_size / g) % 256 == 0,
                "lmb_model_create: o/down shards must be whole 256-column blocks");
  LMB_REQUIRE(c->max_batch >= 1 && c->max_seq_len >= 1, "lmb_model_create: max_batch and max_seq_len must be >= 1");
  LMB_CUDA(cudaSetDevice(ctx->device));
  lmb_model *m = new (std::nothrow) lmb_model();
  if (!m) return LMB_ERR_ALLOC;
  m->ctx = ctx;
  m->cfg = *c;
  m->cfg.tp_size = g;
  m->nh = c->num_attention_heads / g;
  m->nkv = c->num_key_value_heads / g;
  m->inter = c->intermediate_size / g;
  m->vocab_local = c->vocab_size / g;
  m->layers.resize(c->num_hidden_layers);
  {
    const char *gv = getenv("LMB_MODEL_GRAPH");
    m->use_graph = !(gv && gv[0] == '0');
    const char *fv = getenv("LMB_MODEL_FUSED");
    m->fused = !(fv && fv[0] == '0');
    const char *pv = std::getenv("LMB_TP_PEERS");
    m->tp_peers = !(pv && pv[0] == '0');
    // LMB_MODEL_PERSISTENT=1 / 0 forces the persistent batch-1 step on / off; unset: the default below
    const char *sv = std::getenv("LMB_MODEL_PERSISTENT");
    m->persistent = sv ? (sv[0] != '0') : PERSISTENT_BY_DEFAULT;
    const char *av = std::getenv("LMB_ATTN_GROUP");
    m->attn_group = !(av && av[0] == '0');
    const char *hv = std::getenv("LMB_MODEL_HANDOFF");
    m->handoff = !(hv && hv[0] == '0');  // LMB_MODEL_HANDOFF=0: every consumer CTA converts its own activations
    m->handoff_forced = hv && hv[0] == '1' ? 1 : 0;  // LMB_MODEL_HANDOFF=1: also for narrow models
  }
  const size_t B = c->max_batch, h = c->hidden_size, hd = c->head_dim;
  m->seq_stride = c->num_hidden_layers * 2 * c->max_seq_len * m->nkv * hd;
  int st = LMB_OK;
  auto A = [&](float **p, size_t n) { if (st == LMB_OK) st = dev_alloc(p, n); };
  A(&m->hidden, B * h); A(&m->normed, B * h); A(&m->q, B * m->nh * hd); A(&m->k, B * m->nkv * hd);
  A(&m->v, B * m->nkv * hd); A(&m->att, B * m->nh * hd); A(&m->proj, B * h); A(&m->gate, B * m->inter);
  A(&m->up, B * m->inter); A(&m->act, B * m->inter); A(&m->logits, B * c->vocab_size);
  if (g > 1) A(&m->logits_local, B * m->vocab_local);
  if (g > 1 && B > 1) A(&m->logits_gather, B * c->vocab_size);
  A(&m->att_partial, attn_partial_floats(B, m->nh, hd));
  for (int i = 0; i < 2; ++i) {  // hand-off records of the hidden state (batch 1) and their per-block sums of squares
    A(reinterpret_cast<float **>(&m->prep[i]), (h + BLK - 1) / BLK * PREP_RECORD_WORDS);
    A(&m->prep_ss[i], (h + BLK - 1) / BLK);
  }
  A(reinterpret_cast<float **>(&m->att_counters), B * m->nh);
  A(&m->kv, B * m->seq_stride); A(&m->final_norm, h); A(&m->cs_table, c->max_seq_len * hd);
  for (auto &L : m->layers) { A(&L.in_norm, h); A(&L.post_norm, h); }
  if (st == LMB_OK) {
    cudaError_t e = cudaMalloc(&m->d_tokens, B * sizeof(int));
    if (e == cudaSuccess) e = cudaMalloc(&m->d_pos, B * sizeof(size_t));
    if (e == cudaSuccess) e = cudaMallocHost(&m->h_io, B * (sizeof(int) + sizeof(size_t)));
    if (e == cudaSuccess) e = cudaMallocHost(&m->h_status, 4 * sizeof(unsigned));
    if (e != cudaSuccess) st = cuda_fail(e, "lmb_model_create");
  }
  if (st == LMB_OK) {
    // cos/sin with the reference's float arithmetic (src/layers/embedding.cpp:45-49):
    // freq = 1/pow(theta, 2d/head_dim), angle = (position / factor) * freq.
    const size_t half = hd / 2;
    std::vector<float> cs(c->max_seq_len * hd);
    for (size_t pos = 0; pos < c->max_seq_len; ++pos)
      for (size_t d = 0; d < half; ++d) {
        const float freq = 1.0f / std::pow(c->rope_theta, (2.0f * d) / hd);
        const float angle = (pos / c->rope_scaling_factor) * freq;
        cs[pos * hd + d] = std::cos(angle);
        cs[pos * hd + half + d] = std::sin(angle);
      }
    // norm weights default to one (model.hpp:96-104).  For gemma-type models the device keeps the
    // multiplier 1 + weight of gemma_rms_norm (norm.cpp:40-53), so every norm kernel stays x * inv * w.
    std::vector<float> ones(h, c->gemma ? 2.0f : 1.0f);
    cudaError_t e = cudaMemcpy(m->cs_table, cs.data(), cs.size() * 4, cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemcpy(m->final_norm, ones.data(), h * 4, cudaMemcpyHostToDevice);
    for (auto &L : m->layers) {
      if (e == cudaSuccess) e = cudaMemcpy(L.in_norm, ones.data(), h * 4, cudaMemcpyHostToDevice);
      if (e == cudaSuccess) e = cudaMemcpy(L.post_norm, ones.data(), h * 4, cudaMemcpyHostToDevice);
    }
    if (e != cudaSuccess) st = cuda_fail(e, "lmb_model_create init");
  }
  if (st == LMB_OK) st = configure_decode_ops(ctx);
  if (st != LMB_OK) {
    lmb_model_destroy(m);
    return st;
  }
  *out = m;
  return LMB_OK;
}

int lmb_model_destroy(lmb_model *m) {
  if (!m) return LMB_OK;
  cudaSetDevice(m->ctx->device);
  cudaStreamSynchronize(m->ctx->stream);
  float *bufs[] = {m->hidden, m->normed, m->q, m->k, m->v, m->att, m->proj, m->gate, m->up, m->act, m->logits,
                   m->logits_local, m->logits_gather, m->kv, m->final_norm, m->cs_table, m->att_partial,
                   reinterpret_cast<float *>(m->att_counters), reinterpret_cast<float *>(m->prep[0]),
                   reinterpret_cast<float *>(m->prep[1]), m->prep_ss[0], m->prep_ss[1]};
  for (float *b : bufs) if (b) cudaFree(b);
  for (auto &L : m->layers) {
    for (auto *w : L.w) lmb_weight_free(w);
    float *vs[] = {L.in_norm, L.post_norm, L.qb, L.kb, L.vb};
    for (float *b : vs) if (b) cudaFree(b);
  }
  if (m->lm_head && !m->head_tied) lmb_weight_free(m->lm_head);
  lmb_weight_free(m->embed);
  for (auto g : m->graphs) if (g) cudaGraphExecDestroy(g);
  persist_invalidate(m);
  if (m->d_tokens) cudaFree(m->d_tokens);
  if (m->d_pos) cudaFree(m->d_pos);
  if (m->h_io) cudaFreeHost(m->h_io);
  if (m->h_status) cudaFreeHost(m->h_status);
  delete m;
  return LMB_OK;
}

int lmb_model_set_weight(lmb_model *m, int layer, int slot, int kind, int quant_bits, const void *blocks, size_t M, size_t K) {
  LMB_REQUIRE(m && blocks, "lmb_model_set_weight: null argument");
  LMB_REQUIRE(slot >= LMB_SLOT_EMBED && slot <= LMB_SLOT_DOWN, "lmb_model_set_weight: unknown slot");
  LMB_REQUIRE(kind != LMB_RAW_F32, "lmb_model_set_weight: the device decoder takes quantised tensors only "
                                   "(unquantised matrices go through lmb_linear)");
  for (auto &g : m->graphs) {  // captured steps hold the old pointers
    if (g) cudaGraphExecDestroy(g);
    g = nullptr;
  }
  persist_invalidate(m);
  const lmb_model_config &c = m->cfg;
  const size_t g = size_t(c.tp_size), r = size_t(c.tp_rank), bpr = (K + BLK - 1) / BLK;
  const size_t h = c.hidden_size, hd = c.head_dim;
  // lut_linear rotates iff 0 < quant_bits <= 2 or the tensor is ternary (lut_gemm_scalar.cpp:92-93)
  const bool rot = (quant_bits > 0 && quant_bits <= 2) || kind == LMB_TERNARY;
  lmb_weight **dst = nullptr;
  size_t r0 = 0, r1 = M, b0 = 0, b1 = bpr, wantM = 0, wantK = 0;
  if (slot == LMB_SLOT_EMBED) {
    dst = &m->embed; wantM = c.vocab_size; wantK = h; m->embed_rot = rot;
    if (m->head_tied) {  // the tied head shares the device copy that is about to be replaced
      m->lm_head = nullptr;
      m->head_tied = false;
    }
  } else if (slot == LMB_SLOT_LM_HEAD) {
    dst = &m->lm_head; wantM = c.vocab_size; wantK = h; r0 = M * r / g; r1 = M * (r + 1) / g; m->head_rot = rot;
  } else {
    LMB_REQUIRE(layer >= 0 && size_t(layer) < m->layers.size(), "lmb_model_set_weight: layer out of range");
    LayerW &L = m->layers[size_t(layer)];
    const int i = slot - LMB_SLOT_Q;
    dst = &L.w[i];
    L.rot[i] = rot;
    const size_t qd = c.num_attention_heads * hd, kvd = c.num_key_value_heads * hd, it = c.intermediate_size;
    switch (slot) {
    case LMB_SLOT_Q: wantM = qd; wantK = h; r0 = M * r / g; r1 = M * (r + 1) / g; break;
    case LMB_SLOT_K: case LMB_SLOT_V: wantM = kvd; wantK = h; r0 = M * r / g; r1 = M * (r + 1) / g; break;
    case LMB_SLOT_O: wantM = h; wantK = qd; b0 = bpr * r / g; b1 = bpr * (r + 1) / g; break;
    case LMB_SLOT_GATE: case LMB_SLOT_UP: wantM = it; wantK = h; r0 = M * r / g; r1 = M * (r + 1) / g; break;
    case LMB_SLOT_DOWN: wantM = h; wantK = it; b0 = bpr * r / g; b1 = bpr * (r + 1) / g; break;
    }
  }
  LMB_REQUIRE(M == wantM && K == wantK, "lmb_model_set_weight: tensor shape does not match the model config");
  if (*dst && !(slot == LMB_SLOT_LM_HEAD && m->head_tied)) lmb_weight_free(*dst);
  if (slot == LMB_SLOT_LM_HEAD) m->head_tied = false;
  *dst = nullptr;
  return lmb_weight_upload_shard(m->ctx, kind, blocks, M, K, r0, r1, b0, b1, dst);
}

int lmb_model_tie_head(lmb_model *m) {
  LMB_REQUIRE(m, "lmb_model_tie_head: null model");
  return model_tie_head(m);
}

int lmb_model_set_vector(lmb_model *m, int layer, int which, const float *data, size_t n) {
  LMB_REQUIRE(m && data, "lmb_model_set_vector: null argument");
  const lmb_model_config &c = m->cfg;
  const size_t g = size_t(c.tp_size), r = size_t(c.tp_rank), hd = c.head_dim;
  float **dst = nullptr;
  size_t want = c.hidden_size, off = 0, keep = c.hidden_size;
  if (which == LMB_VEC_FINAL_NORM) dst = &m->final_norm;
  else {
    LMB_REQUIRE(layer >= 0 && size_t(layer) < m->layers.size(), "lmb_model_set_vector: layer out of range");
    LayerW &L = m->layers[size_t(layer)];
    switch (which) {
    case LMB_VEC_INPUT_NORM: dst = &L.in_norm; break;
    case LMB_VEC_POST_NORM: dst = &L.post_norm; break;
    case LMB_VEC_Q_BIAS: dst = &L.qb; want = c.num_attention_heads * hd; keep = want / g; off = keep * r; break;
    case LMB_VEC_K_BIAS: dst = &L.kb; want = c.num_key_value_heads * hd; keep = want / g; off = keep * r; break;
    case LMB_VEC_V_BIAS: dst = &L.vb; want = c.num_key_value_heads * hd; keep = want / g; off = keep * r; break;
    default: set_last_error("lmb_model_set_vector: unknown vector slot"); return LMB_ERR_ARG;
    }
  }
  LMB_REQUIRE(n == want, "lmb_model_set_vector: length does not match the model config");
  std::vector<float> plus_one;
  if (c.gemma && (which == LMB_VEC_FINAL_NORM || which == LMB_VEC_INPUT_NORM || which == LMB_VEC_POST_NORM)) {
    plus_one.resize(n);
    for (size_t i = 0; i < n; ++i) plus_one[i] = 1.0f + data[i];  // gemma_rms_norm's (1.0f + weight[i]), same fp32 rounding
    data = plus_one.data();
  }
  if (!*dst) {
    for (auto &gr : m->graphs) {  // a bias that did not exist when a step was captured or planned
      if (gr) cudaGraphExecDestroy(gr);
      gr = nullptr;
    }
    persist_invalidate(m);
    LMB_CUDA(cudaMalloc(dst, keep * sizeof(float)));
  }
  LMB_CUDA(cudaMemcpy(*dst, data + off, keep * sizeof(float), cudaMemcpyHostToDevice));
  return LMB_OK;
}

}  // extern "C"

namespace lmb {
// lm_head = embed_tokens without a second device copy (load_model's tied head, model.cpp:667-689).
int model_tie_head(lmb_model *m) {
  if (m->cfg.tp_size != 1 || !m->embed) {
    set_last_error("lmb_model_tie_head: needs an unsharded model whose embedding is set");
    return LMB_ERR_STATE;
  }
  for (auto &g : m->graphs) {  // captured steps hold the old head
    if (g) cudaGraphExecDestroy(g);
    g = nullptr;
  }
  persist_invalidate(m);
  if (m->lm_head && !m->head_tied) lmb_weight_free(m->lm_head);
  m->lm_head = m->embed;
  m->head_tied = true;
  m->head_rot = m->embed_rot;
  return LMB_OK;
}
}  // namespace lmb

namespace {

struct Fuse {
  int xmode = XMODE_PLAIN;
  const float *x2 = nullptr;        // norm weight / multiplied-in vector
  const float *residual = nullptr;  // added to the output
  // hand-off of prepared activations (LinearArgs): producer side, consumer side
  uint32_t *next_prep = nullptr;
  float *next_sumsq = nullptr;
  const float *next_w = nullptr;
  bool next_rotate = false;
  const uint32_t *prep_in = nullptr;
  const float *prep_sumsq_in = nullptr;
  int prep_sumsq_n = 0;
};

void apply_handoff(LinearArgs &a, const Fuse &f) {
  a.next_prep = f.next_prep;
  a.next_sumsq = f.next_sumsq;
  a.next_w = f.next_w;
  a.next_rotate = f.next_rotate;
  a.prep_in = f.prep_in;
  a.prep_sumsq_in = f.prep_sumsq_in;
  a.prep_sumsq_n = f.prep_sumsq_n;
}

int gemv1(lmb_model *m, const lmb_weight *w, bool rot, const float *x, size_t x_len, float *y, size_t batch,
          const Fuse &f = Fuse()) {
  LinearArgs a{w, nullptr, x, x_len, x_len, y, w->M, batch, rot, f.x2, f.residual};
  apply_handoff(a, f);
  return launch_gemv(m->ctx, &a, 1, rot, f.xmode, m->cfg.rms_norm_eps);
}

// Several projections that read the same input: one launch when kinds and rotation agree.
int gemv_group(lmb_model *m, int n, lmb_weight *const *ws, const bool *rot, const float *x, size_t x_len, float *const *ys,
               size_t batch, const Fuse &f = Fuse()) {
  bool same = true;
  for (int i = 1; i < n; ++i) same = same && ws[i]->kind == ws[0]->kind && rot[i] == rot[0];
  if (same) {
    LinearArgs a[4];
    for (int i = 0; i < n; ++i) {
      a[i] = LinearArgs{ws[i], nullptr, x, x_len, x_len, ys[i], ws[i]->M, batch, rot[0], f.x2, nullptr};
      apply_handoff(a[i], f);
    }
    return launch_gemv(m->ctx, a, n, rot[0], f.xmode, m->cfg.rms_norm_eps);
  }
  for (int i = 0; i < n; ++i) {
    int st = gemv1(m, ws[i], rot[i], x, x_len, ys[i], batch, f);
    if (st != LMB_OK) return st;
  }
  return LMB_OK;
}

// Whether the tensor-parallel sum may leave the hidden state as prepared activations: whole 256-blocks,
// integer tensor-core layouts in every consumer, one rotation setting per group of consumers.
bool tp_prepare_possible(const lmb_model *m) {
  if (!m->handoff || m->cfg.hidden_size % BLK != 0 || !m->lm_head || !kind_is_mma(m->lm_head->kind)) return false;
  for (const LayerW &L : m->layers) {
    for (int i : {0, 1, 2, 4, 5})
      if (!L.w[i] || !kind_is_mma(L.w[i]->kind)) return false;
    if (L.rot[0] != L.rot[1] || L.rot[0] != L.rot[2] || L.rot[4] != L.rot[5]) return false;
  }
  return true;
}

// Whether the producing projections of a batch-1 step may prepare the next projection's
// activations: whole 256-blocks of hidden state, integer tensor-core layouts everywhere.
bool handoff_possible(const lmb_model *m) {
  if (!m->handoff || m->cfg.tp_size != 1 || m->cfg.hidden_size % BLK != 0 || !m->lm_head || !kind_is_mma(m->lm_head->kind)) return false;
  // The producers must cut their rows into groups of 256 (8 row tiles per CTA): with fewer than 16
  // such groups they cannot fill the GPU without many K slices, which costs more than the consumers
  // save (1B / 1.5B-shaped steps measured 10 to 15 % slower; the 70B-shaped step 9 % faster).
  if (m->cfg.hidden_size < 16 * BLK && m->handoff_forced == 0) return false;
  for (const LayerW &L : m->layers) {
    for (int i = 0; i < 7; ++i)
      if (!L.w[i] || !kind_is_mma(L.w[i]->kind)) return false;
    if (L.rot[0] != L.rot[1] || L.rot[0] != L.rot[2] || L.rot[4] != L.rot[5]) return false;
  }
  return true;
}

}  // namespace

extern "C" {

int lmb_model_forward(lmb_model *m, const int *token_ids, const size_t *positions, size_t batch, float *h_logits) {
  LMB_REQUIRE(m && token_ids && positions, "lmb_model_forward: null argument");
  const lmb_model_config &c = m->cfg;
  LMB_REQUIRE(batch >= 1 && batch <= c.max_batch, "lmb_model_forward: batch exceeds max_batch");
  LMB_REQUIRE(m->embed && m->lm_head, "lmb_model_forward: embedding or lm_head not set");
  for (auto &L : m->layers)
    for (auto *w : L.w) LMB_REQUIRE(w, "lmb_model_forward: a layer weight is not set");
  for (size_t b = 0; b < batch; ++b)
    LMB_REQUIRE(positions[b] < c.max_seq_len, "lmb_model_forward: position beyond the KV cache");
  lmb_ctx *ctx = m->ctx;
  ctx->timeline_cursor = 0;  // launch timeline (debugging): slots are counted from the start of a step
  const size_t h = c.hidden_size, hd = c.head_dim;
  const RopeDims rd{m->nh, m->nkv, hd, c.max_seq_len, m->seq_stride, 0};
  const int n_splits = decode_attn_splits(ctx, m->nh, batch, c.max_seq_len);
  // attention of one layer: the group form (keys / values of a slice read once for all query heads of
  // a KV head, bulk asynchronous copies) where the shape allows it, else one CTA per query head
  const AttnGroupPlan agp = m->attn_group ? plan_attn_group(m->nh, m->nkv, hd, c.max_seq_len, batch, size_t(2) * ctx->sm_count, ATTN_GROUP_SMEM)
                                          : AttnGroupPlan{false, 1, 0, 0, 0};
  auto attention = [&](LayerW &L, size_t l) {
    if (agp.ok)
      return launch_decode_attn_group(ctx, m->q, m->k, m->v, L.qb, L.kb, L.vb, m->cs_table, m->d_pos, m->kv, m->att, m->att_partial,
                                      m->att_counters, agp, l, rd, batch);
    return launch_decode_attn(ctx, m->q, m->k, m->v, L.qb, L.kb, L.vb, m->cs_table, m->d_pos, m->kv, m->att, m->att_partial,
                              m->att_counters, n_splits, l, rd, batch);
  };

  int *ht = static_cast<int *>(m->h_io);
  size_t *hp = reinterpret_cast<size_t *>(static_cast<char *>(m->h_io) + c.max_batch * sizeof(int));
  if (!m->capturing) {
    LMB_CUDA(cudaStreamSynchronize(ctx->stream));  // the staging buffer may still be in use by the previous step
    std::memcpy(ht, token_ids, batch * sizeof(int));
    std::memcpy(hp, positions, batch * sizeof(size_t));
    LMB_CUDA(cudaMemcpyAsync(m->d_tokens, ht, batch * sizeof(int), cudaMemcpyHostToDevice, ctx->stream));
    LMB_CUDA(cudaMemcpyAsync(m->d_pos, hp, batch * sizeof(size_t), cudaMemcpyHostToDevice, ctx->stream));
  }

  int st = LMB_OK;
  bool graphed = false;
  if (batch == 1 && !m->capturing && persist_eligible(m)) {
    // embedding and all layers as one persistent kernel, then the final norm inside the head's launch
    st = persist_forward(m);
    if (st == LMB_OK) {
      Fuse fin;
      fin.xmode = XMODE_RMSNORM;
      fin.x2 = m->final_norm;
      if (c.tp_size > 1) {
        st = gemv1(m, m->lm_head, m->head_rot, m->hidden, h, m->logits_local, 1, fin);
        if (st == LMB_OK) st = lmb_allgather(ctx, m->logits_local, m->logits, m->vocab_local);
      } else {
        st = gemv1(m, m->lm_head, m->head_rot, m->hidden, h, m->logits, 1, fin);
      }
      if (st == LMB_OK) st = persist_record_status(m);
      if (st != LMB_OK) return st;
      goto fetch;
    }
    if (st != LMB_ERR_STATE) return st;  // LMB_ERR_STATE: the model does not fit the persistent kernel's limits
    m->persistent = false;
    st = LMB_OK;
  }
  graphed = m->use_graph;
  if (graphed) {
    if (m->graphs.size() <= batch) {
      m->graphs.resize(batch + 1, nullptr);
      m->graph_launches.resize(batch + 1, 0);
      m->graph_gen.resize(batch + 1, 0);
    }
    if (m->graphs[batch] && m->graph_gen[batch] != ctx->scratch_gen) {
      // the context's scratch buffers were reallocated since (a larger batch, another model or an
      // lmb_linear call on this context): the graph's pointers are stale, capture it again
      cudaGraphExecDestroy(m->graphs[batch]);
      m->graphs[batch] = nullptr;
    }
    if (m->graphs[batch]) {
      LMB_CUDA(cudaGraphLaunch(m->graphs[batch], ctx->stream));
      ctx->launches += m->graph_launches[batch];
      goto fetch;
    }
    {
      // size the split-K scratch outside capture: one eager step first (it also is this step)
      const uint64_t before = ctx->launches;
      m->use_graph = false;
      st = lmb_model_forward(m, token_ids, positions, batch, nullptr);
      m->use_graph = true;
      if (st != LMB_OK) return st;
      // capture the same step (it rewrites the same KV slots with the same values)
      const uint64_t base = ctx->launches;
      LMB_CUDA(cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
      m->use_graph = false;
      m->capturing = true;
      st = lmb_model_forward(m, token_ids, positions, batch, nullptr);
      m->capturing = false;
      m->use_graph = true;
      cudaGraph_t g = nullptr;
      cudaError_t e = cudaStreamEndCapture(ctx->stream, &g);
      if (st != LMB_OK) {
        if (g) cudaGraphDestroy(g);
        return st;
      }
      if (e != cudaSuccess) return cuda_fail(e, "cudaStreamEndCapture(decode step)");
      e = cudaGraphInstantiate(&m->graphs[batch], g, 0);
      cudaGraphDestroy(g);
      if (e != cudaSuccess) return cuda_fail(e, "cudaGraphInstantiate(decode step)");
      m->graph_launches[batch] = ctx->launches - base;
      m->graph_gen[batch] = ctx->scratch_gen;
      ctx->launches = base;
      (void)before;
      goto fetch;
    }
  }
  st = launch_embed_rows(ctx, m->d_tokens, m->embed, c.vocab_size, h, batch, c.gemma ? std::sqrt(float(h)) : 1.0f, m->hidden);
  {
  if (c.tp_size == 1 && m->fused) {
    // Fused form: RMSNorm rides in the prologue of the projections that consume it, SiLU*up in
    // the prologue of down_proj, the residual adds in the epilogues of o_proj and down_proj
    // (which write the hidden state in place): 6 launches per layer instead of 9.
    // Hand-off (batch 1): o_proj and down_proj, which complete the hidden state, also prepare it --
    // block by block, in the CTA that finishes the block -- as the next projections' activations, so
    // that the CTAs of q/k/v, gate/up and the head copy 1 KiB records instead of each normalising,
    // rotating and converting the whole vector.
    const bool ho = batch == 1 && handoff_possible(m);
    const int hb = int(h / BLK);
    bool have = false;  // prep[1] holds the prepared hidden state left by the previous layer's down_proj
    for (size_t l = 0; l < m->layers.size() && st == LMB_OK; ++l) {
      LayerW &L = m->layers[l];
      Fuse norm1, norm2, res, act;
      norm1.xmode = XMODE_RMSNORM; norm1.x2 = L.in_norm;
      norm2.xmode = XMODE_RMSNORM; norm2.x2 = L.post_norm;
      res.residual = m->hidden;
      act.xmode = c.activation == LMB_ACT_GELU ? XMODE_GELU_MUL : XMODE_SILU_MUL; act.x2 = m->up; act.residual = m->hidden;
      if (ho) {
        if (have) { norm1.prep_in = m->prep[1]; norm1.prep_sumsq_in = m->prep_ss[1]; norm1.prep_sumsq_n = hb; }
        res.next_prep = m->prep[0]; res.next_sumsq = m->prep_ss[0]; res.next_w = L.post_norm; res.next_rotate = L.rot[4];
        norm2.prep_in = m->prep[0]; norm2.prep_sumsq_in = m->prep_ss[0]; norm2.prep_sumsq_n = hb;
        const bool last = l + 1 == m->layers.size();
        act.next_prep = m->prep[1]; act.next_sumsq = m->prep_ss[1];
        act.next_w = last ? m->final_norm : m->layers[l + 1].in_norm;
        act.next_rotate = last ? m->head_rot : m->layers[l + 1].rot[0];
        have = true;
      }
      float *qkv[3] = {m->q, m->k, m->v};
      st = gemv_group(m, 3, &L.w[0], &L.rot[0], m->hidden, h, qkv, batch, norm1);
      if (st != LMB_OK) break;
      st = attention(L, l);
      if (st != LMB_OK) break;
      st = gemv1(m, L.w[3], L.rot[3], m->att, m->nh * hd, m->hidden, batch, res);
      if (st != LMB_OK) break;
      float *gu[2] = {m->gate, m->up};
      st = gemv_group(m, 2, &L.w[4], &L.rot[4], m->hidden, h, gu, batch, norm2);
      if (st != LMB_OK) break;
      st = gemv1(m, L.w[6], L.rot[6], m->gate, m->inter, m->hidden, batch, act);
    }
    if (st != LMB_OK) return st;
    Fuse fin;
    fin.xmode = XMODE_RMSNORM; fin.x2 = m->final_norm;
    if (ho && have) { fin.prep_in = m->prep[1]; fin.prep_sumsq_in = m->prep_ss[1]; fin.prep_sumsq_n = hb; }
    st = gemv1(m, m->lm_head, m->head_rot, m->hidden, h, m->logits, batch, fin);
    if (st != LMB_OK) return st;
  } else {
  const float *pending = nullptr;  // residual branch not yet added to hidden
  // Tensor parallelism over peer memory: o_proj and down_proj store their partial vectors straight
  // into every rank's exchange block; the next normalisation waits for all ranks and adds them.
  const bool peers = c.tp_size > 1 && ctx->xchg.ready && batch * h <= ctx->xchg.cap && m->tp_peers;
  bool in_flight = false;  // a partial vector is on its way through the exchange block
  // Batch 1 with integer tensor-core layouts everywhere: the kernel that adds the ranks' partial vectors
  // also leaves the hidden state as the next projections' prepared activations (k_tp_sum_prepare), one
  // CTA per 256-block, instead of one CTA normalising the whole vector and every consumer CTA converting it.
  const bool prepare = peers && batch == 1 && tp_prepare_possible(m);
  Fuse consumer;  // how the projections after the latest `norm` read their input
  auto norm = [&](const float *w, bool rot) {
    int r;
    consumer = Fuse();
    if (in_flight && prepare) {
      r = launch_tp_sum_prepare(ctx, m->hidden, w, rot, m->prep[0], m->prep_ss[0], h);
      consumer.xmode = XMODE_RMSNORM;
      consumer.prep_in = m->prep[0];
      consumer.prep_sumsq_in = m->prep_ss[0];
      consumer.prep_sumsq_n = int(h / BLK);
    } else {
      r = in_flight ? launch_tp_sum_add_rmsnorm(ctx, m->hidden, w, m->normed, h, batch, c.rms_norm_eps)
                    : launch_add_rmsnorm(ctx, m->hidden, pending, w, m->normed, h, batch, c.rms_norm_eps);
    }
    in_flight = false;
    pending = nullptr;
    return r;
  };
  auto row_reduce = [&](const lmb_weight *w, bool rot, const float *x, size_t x_len, const Fuse &f) {
    if (peers) {
      LinearArgs a{w, nullptr, x, x_len, x_len, m->proj, w->M, batch, rot, f.x2, nullptr, true};
      in_flight = true;
      return launch_gemv(ctx, &a, 1, rot, f.xmode, c.rms_norm_eps);
    }
    int r = gemv1(m, w, rot, x, x_len, m->proj, batch, f);
    if (r == LMB_OK && c.tp_size > 1) r = lmb_allreduce_sum(ctx, m->proj, batch * h);
    pending = m->proj;
    return r;
  };
  for (size_t l = 0; l < m->layers.size() && st == LMB_OK; ++l) {
    LayerW &L = m->layers[l];
    st = norm(L.in_norm, L.rot[0]);
    if (st != LMB_OK) break;
    float *qkv[3] = {m->q, m->k, m->v};
    st = gemv_group(m, 3, &L.w[0], &L.rot[0], m->normed, h, qkv, batch, consumer);
    if (st != LMB_OK) break;
    st = attention(L, l);
    if (st != LMB_OK) break;
    st = row_reduce(L.w[3], L.rot[3], m->att, m->nh * hd, Fuse());
    if (st != LMB_OK) break;
    st = norm(L.post_norm, L.rot[4]);
    if (st != LMB_OK) break;
    float *gu[2] = {m->gate, m->up};
    st = gemv_group(m, 2, &L.w[4], &L.rot[4], m->normed, h, gu, batch, consumer);
    if (st != LMB_OK) break;
    Fuse act;  // SiLU(gate) * up in the prologue of down_proj (element-wise, so a column shard needs no exchange)
    act.xmode = c.activation == LMB_ACT_GELU ? XMODE_GELU_MUL : XMODE_SILU_MUL;
    act.x2 = m->up;
    st = row_reduce(L.w[6], L.rot[6], m->gate, m->inter, act);
  }
  if (st != LMB_OK) return st;
  st = norm(m->final_norm, m->head_rot);
  if (st != LMB_OK) return st;
  if (c.tp_size > 1) {
    st = gemv1(m, m->lm_head, m->head_rot, m->normed, h, m->logits_local, batch, consumer);
    if (st == LMB_OK && batch == 1) {
      st = lmb_allgather(ctx, m->logits_local, m->logits, m->vocab_local);
    } else if (st == LMB_OK) {
      // ONE all-gather per step: every rank's [batch][vocab / ranks] slab into [rank][batch][vocab / ranks],
      // then the rows are put in place ([batch][vocab]) by a copy kernel
      st = lmb_allgather(ctx, m->logits_local, m->logits_gather, batch * m->vocab_local);
      if (st == LMB_OK) st = launch_interleave_rows(ctx, m->logits_gather, m->logits, size_t(c.tp_size), batch, m->vocab_local);
    }
  } else {
    st = gemv1(m, m->lm_head, m->head_rot, m->normed, h, m->logits, batch);
  }
  if (st != LMB_OK) return st;
  }
  }
fetch:
  if (h_logits) {
    // the logits and, behind them in the same stream, the three status words a step can leave: the
    // context's fault flag, the exchange block's time-out flag, the persistent step's status
    unsigned *hs = static_cast<unsigned *>(m->h_status);
    hs[0] = hs[1] = 0;
    LMB_CUDA(cudaMemcpyAsync(h_logits, m->logits, batch * c.vocab_size * sizeof(float), cudaMemcpyDeviceToHost, ctx->stream));
    LMB_CUDA(cudaMemcpyAsync(&hs[0], ctx->d_fault, sizeof(unsigned), cudaMemcpyDeviceToHost, ctx->stream));
    if (c.tp_size > 1 && ctx->xchg.ready)
      LMB_CUDA(cudaMemcpyAsync(&hs[1], &static_cast<XchgHeader *>(ctx->xchg.local)->timed_out, sizeof(unsigned),
                               cudaMemcpyDeviceToHost, ctx->stream));
    LMB_CUDA(cudaStreamSynchronize(ctx->stream));
    if (hs[0]) {  // a kernel's bounded wait for its own asynchronous copies ran out
      LMB_CUDA(cudaMemset(ctx->d_fault, 0, sizeof(unsigned)));
      set_last_error("lmb_model_forward: a bounded wait for asynchronous copies expired in the attention kernel");
      return LMB_ERR_TIMEOUT;
    }
    unsigned expired = 0;
    int ps = persist_take_status(m, &expired);
    if (ps != LMB_OK) return ps;
    if (expired) {
      set_last_error("lmb_model_forward: a bounded wait between the phases of the decode step expired (phase " +
                     std::to_string(expired - 1) + ")");
      return LMB_ERR_TIMEOUT;
    }
    if (hs[1]) {
      // a consumer that gave up waiting for another rank's partial vector has produced garbage:
      // the step reports it instead of returning the logits as if nothing had happened
      set_last_error("lmb_model_forward: a bounded wait for another rank's partial vector expired");
      return LMB_ERR_TIMEOUT;
    }
  }
  return LMB_OK;
}

int lmb_debug_model_timeline(lmb_model *m, unsigned long long *out, int *types, int *kslices, size_t cap_phases, size_t *n_phases) {
  LMB_REQUIRE(m && n_phases && (cap_phases == 0 || (out && types && kslices)), "lmb_debug_model_timeline: null argument");
  return persist_timeline(m, out, types, kslices, cap_phases, n_phases);
}

int lmb_debug_model_waits(lmb_model *m, int extra_arrivals, unsigned spin_limit) {
  LMB_REQUIRE(m && extra_arrivals >= 0, "lmb_debug_model_waits: bad argument");
  m->debug_extra_arrivals = extra_arrivals;
  m->ctx->xchg.spin_limit = spin_limit ? spin_limit : (1u << 22);
  return LMB_OK;
}

int lmb_model_logits_dev(lmb_model *m, const float **d_logits) {
  LMB_REQUIRE(m && d_logits, "lmb_model_logits_dev: null argument");
  *d_logits = m->logits;
  return LMB_OK;
}

int lmb_model_reset(lmb_model *m) {
  LMB_REQUIRE(m, "lmb_model_reset: null model");
  LMB_CUDA(cudaMemsetAsync(m->kv, 0, m->cfg.max_batch * m->seq_stride * sizeof(float), m->ctx->stream));
  return LMB_OK;
}

// The host side always sees the reference layout of the WHOLE model, [layer][2][max_seq][kv_heads][head_dim]
// (types.hpp:599-627).  On the device a sequence's cache is [layer][2][local kv head][max_seq][head_dim]
// (the positions of one head contiguous); a tensor-parallel rank holds kv_heads / tp_size consecutive
// heads.  One strided copy per (layer, K|V, head).
static int kv_transfer(lmb_model *m, size_t seq, float *h, bool to_host) {
  const lmb_model_config &c = m->cfg;
  const size_t hd = c.head_dim, full = c.num_key_value_heads * hd, S = c.max_seq_len;
  for (size_t lk = 0; lk < c.num_hidden_layers * 2; ++lk)
    for (size_t kh = 0; kh < m->nkv; ++kh) {
      float *dev = m->kv + seq * m->seq_stride + (lk * m->nkv + kh) * S * hd;
      float *host = h + lk * S * full + (size_t(c.tp_rank) * m->nkv + kh) * hd;
      if (to_host)
        LMB_CUDA(cudaMemcpy2DAsync(host, full * sizeof(float), dev, hd * sizeof(float), hd * sizeof(float), S, cudaMemcpyDeviceToHost,
                                   m->ctx->stream));
      else
        LMB_CUDA(cudaMemcpy2DAsync(dev, hd * sizeof(float), host, full * sizeof(float), hd * sizeof(float), S, cudaMemcpyHostToDevice,
                                   m->ctx->stream));
    }
  LMB_CUDA(cudaStreamSynchronize(m->ctx->stream));
  return LMB_OK;
}

int lmb_model_kv_export(lmb_model *m, size_t seq, float *h_out) {
  LMB_REQUIRE(m && h_out && seq < m->cfg.max_batch, "lmb_model_kv_export: bad argument");
  return kv_transfer(m, seq, h_out, true);
}

int lmb_model_kv_import(lmb_model *m, size_t seq, const float *h_in) {
  LMB_REQUIRE(m && h_in && seq < m->cfg.max_batch, "lmb_model_kv_import: bad argument");
  return kv_transfer(m, seq, const_cast<float *>(h_in), false);
}

int lmb_model_step_bytes(lmb_model *m, size_t position, uint64_t *bytes_out) {
  LMB_REQUIRE(m && bytes_out, "lmb_model_step_bytes: null argument");
  auto wb = [](const lmb_weight *w) -> uint64_t {
    return w ? uint64_t(w->M) * w->bpr * kind_info(w->kind).ref_bytes + 4 * w->bpr * BLK + 4 * w->M : 0;
  };
  uint64_t n = wb(m->lm_head) + 4 * m->cfg.hidden_size;
  for (auto &L : m->layers)
    for (auto *w : L.w) n += wb(w);
  n += uint64_t(2) * m->layers.size() * (position + 1) * m->nkv * m->cfg.head_dim * 4;
  *bytes_out = n;
  return LMB_OK;
}

}  // extern "C"
