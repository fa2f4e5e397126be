// The device-resident decoder object shared by model.cu (the C ABI and the launch-per-projection
// decode step) and persist.cu (the decode step as one persistent kernel).
#pragma once

#include <vector>

#include "decode_ops.cuh"

namespace lmb {
struct PersistPlan;  // persist.cu
}

struct LayerW {
  lmb_weight *w[7] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};  // q k v o gate up down
  bool rot[7] = {false, false, false, false, false, false, false};
  float *in_norm = nullptr, *post_norm = nullptr, *qb = nullptr, *kb = nullptr, *vb = nullptr;
};

struct lmb_model {
  lmb_ctx *ctx = nullptr;
  lmb_model_config cfg;
  size_t nh = 0, nkv = 0, inter = 0, vocab_local = 0;  // this rank's share
  lmb_weight *embed = nullptr, *lm_head = nullptr;
  bool head_tied = false, head_rot = false, embed_rot = false;
  float *final_norm = nullptr;
  std::vector<LayerW> layers;
  // activations [max_batch][...]
  float *hidden = nullptr, *normed = nullptr, *q = nullptr, *k = nullptr, *v = nullptr, *att = nullptr, *proj = nullptr,
        *gate = nullptr, *up = nullptr, *act = nullptr, *logits = nullptr, *logits_local = nullptr, *logits_gather = nullptr;
  float *att_partial = nullptr;      // [max_batch][nh][32 splits][hd + 2]
  unsigned *att_counters = nullptr;  // [max_batch][nh]
  float *kv = nullptr;        // [max_batch][L][2][nkv][max_seq][hd]: the positions of one head contiguous
  float *cs_table = nullptr;  // [max_seq][hd/2 cos | hd/2 sin]
  int *d_tokens = nullptr;
  size_t *d_pos = nullptr;
  void *h_io = nullptr;  // pinned staging for tokens + positions
  void *h_status = nullptr;  // pinned: status words copied back with the logits
  size_t seq_stride = 0;
  // one instantiated CUDA graph of the whole step per batch size (token ids and positions are
  // read from device buffers, so the graph never changes)
  bool use_graph = true, capturing = false;
  bool fused = true;  // norm / activation / residual fused into the GEMV launches (unsharded models)
  bool tp_peers = true;  // tensor parallelism: partial vectors through peer memory (else NCCL all-reduce)
  std::vector<cudaGraphExec_t> graphs;      // index = batch
  std::vector<uint64_t> graph_launches;
  std::vector<uint64_t> graph_gen;  // lmb_ctx::scratch_gen each graph was captured under
  // batch-1 steps of models whose layer projections share one integer-MMA kind run as one
  // persistent kernel over all layers (persist.cu); LMB_MODEL_PERSISTENT=0 disables it
  bool persistent = true;
  bool handoff = true;  // LMB_MODEL_HANDOFF=0: every consumer CTA converts its own activations (batch 1, fused step)
  int handoff_forced = 0;  // hand-off requested explicitly: also for models narrower than 16 blocks
  uint32_t *prep[2] = {nullptr, nullptr};  // prepared hidden state after o_proj / after down_proj
  float *prep_ss[2] = {nullptr, nullptr};
  bool attn_group = true;  // LMB_ATTN_GROUP=0: one attention CTA per query head instead of per KV head
  lmb::PersistPlan *ps = nullptr;
  int debug_extra_arrivals = 0;  // failure-path test: every grid barrier waits for this many arrivals that never come
};


namespace lmb {
// One batch-1 decode step up to (not including) the final norm and lm_head: embedding, all layers.
// LMB_ERR_STATE (without touching anything) when the model does not qualify.
bool persist_eligible(const lmb_model *m);
int persist_forward(lmb_model *m);
int persist_record_status(lmb_model *m);  // after the launches that follow the step
void persist_invalidate(lmb_model *m);  // weights or vectors changed: plan again at the next step
// whether a bounded wait of a persistent step expired since the last call (the flag is cleared)
int persist_take_status(lmb_model *m, unsigned *status);
int persist_timeline(lmb_model *m, unsigned long long *out, int *types, int *kslices, size_t cap_phases, size_t *n_phases);
}  // namespace lmb
