/*
 * lutmac_b200 -- C ABI of the B200 (sm_100a) implementation of LutMac's LUT-GEMV decode path.
 *
 * Every entry point is extern "C", takes plain pointers / sizes / opaque handles and returns
 * an int status (0 = LMB_OK).  There is no CPU fallback: every compute call needs a CUDA
 * device and fails with LMB_ERR_CUDA otherwise.
 *
 * Each declaration cites the reference interface (YASSERRMD/lutmac, file:line) it replaces.
 */
#ifndef LUTMAC_B200_H
#define LUTMAC_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes --------------------------------------------------------------------- */
enum {
  LMB_OK = 0,
  LMB_ERR_ARG = 1,      /* bad argument (null pointer, unknown kind, bad shape)            */
  LMB_ERR_CUDA = 2,     /* a CUDA runtime call failed; see lmb_last_error()                 */
  LMB_ERR_ALLOC = 3,    /* host or device allocation failed                                */
  LMB_ERR_TIMEOUT = 4,  /* a bounded device-side wait expired                              */
  LMB_ERR_FORMAT = 5,   /* malformed .lutmac file                                          */
  LMB_ERR_LIMIT = 6,    /* size beyond a documented limit of the entry point               */
  LMB_ERR_STATE = 7     /* call not valid in the handle's current state                    */
};
const char *lmb_strerror(int status);
/* Text of the most recent failure on the calling thread (CUDA error string etc.). */
const char *lmb_last_error(void);

/* ---- block kinds ------------------------------------------------------------------------
 * One per block struct of include/lutmac/types.hpp; the value is PackedTensor::quant_bits
 * for that block vector (types.hpp:470-484), ternary = 0.  256 weights per block. */
enum {
  LMB_TERNARY = 0, /* BitPlaneBlock  68 B  types.hpp:126-137 */
  LMB_BINARY = 1,  /* BinaryBlock    36 B  types.hpp:394-401 */
  LMB_INT2 = 2,    /* Int2Block      72 B  types.hpp:209-215 (RRQ: scale, scale2) */
  LMB_INT3 = 3,    /* Int3Block     100 B  types.hpp:249-254 */
  LMB_INT4 = 4,    /* Int4Block     132 B  types.hpp:174-181 */
  LMB_INT5 = 5,    /* Int5Block     164 B  types.hpp:296-301 */
  LMB_INT6 = 6,    /* Int6Block     196 B  types.hpp:344-349 */
  LMB_INT8 = 8,    /* Int8Block     260 B  types.hpp:434-438 */
  /* PackedTensor::raw_data of an unquantised tensor (is_quantized == false, types.hpp:470-492):
   * `blocks` is then the row-major fp32 matrix [M][K] and lut_linear takes its plain dot-product
   * branch (lut_gemm_scalar.cpp:157-171: no rotation, no padding).  lmb_linear* only. */
  LMB_RAW_F32 = 32
};
/* sizeof the reference block struct of a kind (0 for an unknown kind). */
size_t lmb_block_bytes(int kind);

/* ---- flags for lmb_linear* ---------------------------------------------------------------- */
enum {
  LMB_ROTATE = 1u,      /* apply the block-wise 256-point FWHT/16 to the (zero-padded) input   */
  LMB_AUTO_ROTATE = 2u  /* rotate iff the reference's lut_linear would (lut_gemm_scalar.cpp:92-93) */
};

typedef struct lmb_ctx lmb_ctx;       /* one device + one stream + scratch                   */
typedef struct lmb_weight lmb_weight; /* a weight matrix resident on the device              */
typedef struct lmb_model lmb_model;   /* a device-resident decoder (weights, KV cache, scratch) */

/* ---- context ---------------------------------------------------------------------------------
 * Not thread-safe per context; independent contexts may be used from different threads.  */
int lmb_ctx_create(int device, lmb_ctx **out);
int lmb_ctx_destroy(lmb_ctx *ctx);
/* Run all later work of this context on an existing CUDA stream (a cudaStream_t passed as a
 * pointer); NULL returns to the context's own stream. */
int lmb_ctx_set_stream(lmb_ctx *ctx, void *cuda_stream);
int lmb_ctx_sync(lmb_ctx *ctx);
/* Options.  LMB_OPT_TERNARY_LUT = 1: ternary, INT2, INT3 and binary weights uploaded afterwards
 * use the table-lookup kernel (16-entry group tables, the reference's LUT formulation), INT8
 * weights the dequantise+FMA kernel, instead of the default integer tensor-core kernels.  LMB_OPT_PDL = 0: plain stream order instead of programmatic dependent
 * launch between consecutive kernels.
 * LMB_OPT_SCRATCH_FLOATS = n: reallocate the split-K scratch at n floats (it starts at 4 Mi floats
 * and grows on demand; graphs and groups made earlier notice the reallocation and are rebuilt). */
enum { LMB_OPT_TERNARY_LUT = 1, LMB_OPT_PDL = 2, LMB_OPT_SCRATCH_FLOATS = 3 };
int lmb_ctx_set_option(lmb_ctx *ctx, int option, int value);
int lmb_device_count(int *out);
/* Number of kernels this library has launched on the context since creation. */
int lmb_ctx_launch_count(lmb_ctx *ctx, uint64_t *out);

/* Device memory helpers for hosts that have no CUDA binding of their own. */
int lmb_malloc(lmb_ctx *ctx, size_t bytes, void **d_ptr);
int lmb_free(lmb_ctx *ctx, void *d_ptr);
int lmb_memcpy_h2d(lmb_ctx *ctx, void *d_dst, const void *h_src, size_t bytes);
int lmb_memcpy_d2h(lmb_ctx *ctx, void *h_dst, const void *d_src, size_t bytes);
int lmb_memset(lmb_ctx *ctx, void *d_dst, int value, size_t bytes);
int lmb_host_alloc_pinned(size_t bytes, void **h_ptr);
int lmb_host_free_pinned(void *h_ptr);

/* CUDA-event timing on the context's stream. */
int lmb_timer_start(lmb_ctx *ctx);
int lmb_timer_stop(lmb_ctx *ctx, float *ms_out); /* records, synchronises, returns elapsed ms */

/* CUDA-graph capture of the work a context issues (kernel launches only; no host-pointer entry
 * point may be called while capturing).  lmb_graph_end returns an executable graph that
 * lmb_graph_launch replays on the context's stream. */
typedef struct lmb_graph lmb_graph;
int lmb_graph_begin(lmb_ctx *ctx);
int lmb_graph_end(lmb_ctx *ctx, lmb_graph **out);
int lmb_graph_launch(lmb_ctx *ctx, lmb_graph *g);
int lmb_graph_destroy(lmb_graph *g);

/* ---- weights: replaces the host block vectors of PackedTensor (types.hpp:470-492) and the
 * raw struct reads of load_lutmac (src/format.cpp:463-496) --------------------------------------
 * `blocks` is the reference's row-major block array: row r starts at blocks + r*ceil(K/256).
 * The array is re-tiled once into the device layout and may be freed after the call.
 * lmb_weight_upload_shard keeps rows [row0,row1) and 256-column blocks [blk0,blk1) of every
 * kept row (tensor-parallel shards); the shard behaves as an (row1-row0) x ((blk1-blk0)*256)
 * matrix. */
int lmb_weight_upload(lmb_ctx *ctx, int kind, const void *blocks, size_t M, size_t K, lmb_weight **out);
int lmb_weight_upload_shard(lmb_ctx *ctx, int kind, const void *blocks, size_t M, size_t K,
                            size_t row0, size_t row1, size_t blk0, size_t blk1, lmb_weight **out);
int lmb_weight_free(lmb_weight *w);
int lmb_weight_info(const lmb_weight *w, int *kind, size_t *M, size_t *K, size_t *device_bytes);
/* Reads the device copy back and converts it to the reference block layout (the inverse of
 * the upload re-tiling; bit-exact for blocks in the canonical form the reference's own
 * quantizers emit). `blocks_out` holds M*ceil(K/256) blocks. */
int lmb_weight_download(lmb_ctx *ctx, const lmb_weight *w, void *blocks_out);
/* The same two conversions on the host only (no device needed). `tiled` holds
 * lmb_tiled_bytes(kind, M, K) bytes. */
size_t lmb_tiled_bytes(int kind, size_t M, size_t K);
int lmb_retile_host(int kind, const void *blocks, size_t M, size_t K, void *tiled);
int lmb_untile_host(int kind, const void *tiled, size_t M, size_t K, void *blocks_out);

/* ---- quantize + pack on the device: replaces quantize_tensor (ternary), quantize_tensor_binary,
 * _int2, _int3, _int4, _int8 (include/lutmac/quantize.hpp:193-336, 725-823, 918-975, 982-1039,
 * 387-495, 833-911) for a row-major fp32 matrix [M][K] -----------------------------------------------
 * d_blocks_out receives M*ceil(K/256) blocks in the reference's struct layout (what a .lutmac file
 * stores and lmb_weight_upload takes, from host memory).  Codes and bit planes are bit-exact with
 * the reference's quantizers; scales agree to the last ulp or two of a -ffast-math build.  The
 * Hadamard rotation the reference's quantize tool applies to the weights of its <= 2-bit formats
 * (tools/lutmac-quantize.cpp:423-453) is lmb_fwht256 over the same buffer, called first;
 * lmb_quantize_host does that when rotate_first is non-zero.  5- and 6-bit blocks are not
 * produced on the device. */
int lmb_quantize(lmb_ctx *ctx, int kind, const float *d_weights, size_t M, size_t K, void *d_blocks_out);
int lmb_quantize_host(lmb_ctx *ctx, int kind, const float *weights, size_t M, size_t K, int rotate_first, void *blocks_out);

/* ---- layer API on device pointers: replaces lut_linear (include/lutmac/lut_gemm.hpp:419,
 * src/kernels/lut_gemm_scalar.cpp:68-180) ---------------------------------------------------------
 * y[b] = W * rot?(pad(x[b])) + bias for b < batch.  d_x holds batch rows of x_stride floats of
 * which the first x_len are read (the rest of each 256-block counts as zero, which is the
 * reference's zero padding); d_y holds batch rows of M floats.  d_bias is NULL or M floats. */
int lmb_linear(lmb_ctx *ctx, const lmb_weight *w, const float *d_bias, const float *d_x, size_t x_len,
               size_t x_stride, float *d_y, size_t batch, unsigned flags);

/* lut_linear for hosts that must not allocate device memory.  No counterpart in the reference.
 *
 * Some callers cannot reach cudaMalloc at all: a plugin running inside a serving process whose
 * framework has already claimed the whole GPU for its own memory pool, a host thread with a
 * hard latency bound that may not enter the driver's allocator, or code issued while a stream
 * is being captured.  For them this entry point runs the same kernel as lmb_linear (batch 1)
 * but takes the split-K scratch from an array built into the library image instead of from a
 * context: it needs no lmb_ctx and calls no allocating routine.  The caller passes the resident
 * weight, the input and output device pointers and the stream to run on.
 *
 * Limit: the built-in scratch holds 131,072 floats (512 KiB) and 1024 row-group counters per
 * GPU (every GPU that loads the library carries them until the process exits).  A shape whose
 * split needs more -- (K slices) x (rows padded to 32) floats -- is refused with LMB_ERR_LIMIT;
 * every projection of the 1B, 1.5B and 70B decoder shapes fits.
 * All calls on one GPU share that array: calls that overlap on the device (different streams)
 * race with each other; issue them on one stream or order them with events.
 * The first call on each device looks up the array's device address and configures the kernel;
 * make that first call before any stream capture begins. */
int lmb_linear_static_scratch(const lmb_weight *w, const float *d_bias, const float *d_x, size_t x_len, float *d_y,
                              unsigned flags, void *cuda_stream);

/* Prepared group: n independent batch-1 lut_linear calls of one block kind (inputs d_xs[i] of K_i
 * floats, outputs d_ys[i] of M_i floats, device pointers) planned once and issued as a single
 * kernel launch.  The reference issues them one by one (e.g. q/k/v at src/model.cpp:307-309). */
typedef struct lmb_group lmb_group;
int lmb_group_create(lmb_ctx *ctx, size_t n, const lmb_weight *const *ws, const float *const *d_xs, float *const *d_ys,
                     unsigned flags, lmb_group **out);
int lmb_group_launch(lmb_ctx *ctx, lmb_group *g);
/* Host-buffer form: the group owns its device and pinned staging buffers; one call copies all
 * inputs in (inputs[i] = K_i floats), runs the single launch and copies all outputs back
 * (outputs[i] = M_i floats). */
int lmb_group_create_host(lmb_ctx *ctx, size_t n, const lmb_weight *const *ws, unsigned flags, lmb_group **out);
int lmb_group_run_host(lmb_ctx *ctx, lmb_group *g, const float *const *inputs, float *const *outputs);
/* The pinned host buffers of job i of a host group: an input written there and an output read
 * from there need no staging copy (pass the same pointers to lmb_group_run_host). */
int lmb_group_host_io(lmb_group *g, size_t i, float **h_in, float **h_out);
int lmb_group_destroy(lmb_group *g);

/* ---- kernel API on host pointers: replaces the dispatchers lut_gemv, lut_gemv_binary,
 * int2_gemv ... int8_gemv (include/lutmac/lut_gemm.hpp:172-408) -----------------------------------
 * Same arguments as the reference: activations are read for ceil(K/256)*256 floats, num_blocks is
 * ignored, output receives M floats.  One difference in the padding columns of the last block:
 * a value there that is not finite, or more than 4096 times larger than every activation of the
 * block's first K % 256 columns, is taken as zero (the reference's own tests pass arrays of exactly
 * K floats and rely on the zero weights of the padding to hide whatever follows them in memory).
 * Each call uploads the blocks, runs the CUDA kernel on the default context of the current device
 * and copies the result back. */
int lmb_gemv_host(int kind, const void *blocks, size_t num_blocks, const float *activations, float *output,
                  size_t M, size_t K);
/* Layer API on host pointers: lut_linear for a weight already resident (lmb_weight_upload),
 * host input/output, host<->device copies included. */
int lmb_linear_host(lmb_ctx *ctx, const lmb_weight *w, const float *bias, const float *input, float *output,
                    size_t batch, unsigned flags);
/* Several independent lut_linear calls (batch 1 each) issued together: one staged input
 * copy, the kernels, one staged output copy.  inputs[i] holds K_i floats, outputs[i] M_i. */
int lmb_linear_host_multi(lmb_ctx *ctx, size_t n, const lmb_weight *const *ws, const float *const *inputs,
                          float *const *outputs, unsigned flags);

/* ---- transform API: replaces fwht_256 / apply_hadamard_rotation
 * (include/lutmac/transform.hpp:14,19; src/kernels/transform_simd.cpp:26-110) --------------------- */
int lmb_fwht256(lmb_ctx *ctx, float *d_x, size_t n);                 /* in place, device pointer */
int lmb_apply_hadamard_rotation_host(float *data, size_t n);         /* in place, host pointer   */

/* ---- debug views used by the parity tests ----------------------------------------------------------
 * LUT tables exactly as the kernel prologue builds them: ceil(x_len/256)*64 groups x 16 entries
 * (precompute_luts, lut_gemm.hpp:53-58), after optional rotation. */
/* How a GEMV of this shape would be cut into CTAs on a GPU with sm_count SMs (no GPU needed):
 * out5 = {row-tiles per CTA, blocks per K slice, row groups, K slices, sequences per pass}.
 * kind is a device layout kind as reported by lmb_weight_info; other_rows = rows of the other
 * jobs of the same launch. */
int lmb_debug_plan(int kind, size_t M, size_t K, size_t batch, size_t other_rows, int sm_count, int out5[5]);
/* The same for a batch-1 launch of a resident weight alone (uses the weight's device layout kind). */
int lmb_debug_plan_weight(const lmb_weight *w, int sm_count, int out5[5]);
/* Tests and experiments: from now on every batch-1 launch whose shape can take this work split uses it
 * (R row tiles per CTA, n_ks K slices, cr row groups per thread-block cluster -- cluster size
 * cr * n_ks in {2, 4, 8}, cr = 0: no cluster); launches that cannot, plan as usual.  R = 0: off.
 * Process-wide; graphs captured earlier keep their plans. */
int lmb_debug_force_plan(int R, int n_ks, int cr);
/* Range-checking build (liblutmac_b200_dbg.so, compiled with -DLMB_DEBUG_BOUNDS; the reference has no
 * sanitizer set-up to mirror): the GEMV kernels check every weight-tile load, output store and
 * split-K scratch store against the extent of its buffer, the attention kernel its cache slices; an
 * access that would leave its buffer is skipped and recorded, nothing traps.  lmb_debug_bounds
 * synchronises, returns the first violation since the last call -- out4 = {code (0: none; 1 weight
 * tile, 2 output, 3 scratch, 4 KV slice), offending offset, block | thread << 32, number of
 * violations} -- and clears the record.  lmb_debug_bounds_shrink makes later launches claim their
 * weight buffers `bytes` shorter than they are (a test hook: the check trips, every access that does
 * run is inside the real buffer).  In the ordinary library both return LMB_ERR_STATE. */
int lmb_debug_bounds(lmb_ctx *ctx, unsigned long long out4[4]);
int lmb_debug_bounds_shrink(size_t bytes);
/* Launch timeline (debugging; no counterpart in the reference).  cap_launches > 0 on the first call
 * switches recording on for the GEMV and attention launches issued (or captured into a graph) from
 * then on, up to cap_launches per decode step.  Every call synchronises, copies the slots recorded
 * since the previous call to `out` (8 words per launch, *n_launches of them, device global-timer
 * nanoseconds: 0 first CTA started, 1 / 2 first / last CTA past the wait for the preceding kernel,
 * 3 last CTA with its activations ready, 4 last CTA through its main loop, 5 / 6 last / first CTA
 * done, 7 last CTA with its activations fetched into shared memory, GEMV only) and clears them; minima and maxima accumulate over the steps run in between,
 * so run one step between two calls.  out may be null. */
int lmb_debug_launch_timeline(lmb_ctx *ctx, size_t cap_launches, unsigned long long *out, size_t *n_launches);
int lmb_debug_luts(lmb_ctx *ctx, const float *d_x, size_t x_len, unsigned flags, float *d_luts_out);
/* Ternary LUT indices as the kernel consumes them: for every row and group of 4 weights the
 * (pos, neg) nibbles of extract_indices (lut_gemm.hpp:79-99); out = M*ceil(K/256)*64*2 bytes. */
int lmb_debug_ternary_indices(lmb_ctx *ctx, const lmb_weight *w, uint8_t *h_out);

/* ---- model API: replaces Model::allocate / Model::forward / get_logits / reset_cache
 * (include/lutmac/model.hpp:88-141, src/model.cpp:47-453) ------------------------------------------- */
typedef struct {
  size_t vocab_size, hidden_size, intermediate_size, num_hidden_layers;
  size_t num_attention_heads, num_key_value_heads, head_dim, max_seq_len;
  float rope_theta, rope_scaling_factor, rms_norm_eps;
  size_t max_batch;  /* sequences decoded together (the reference decodes one) */
  int tp_rank, tp_size; /* tensor-parallel position of this process (0,1 = unsharded) */
  /* model_type "gemma" (src/model.cpp:255-260,294-301,390-399,436-442): the embedding row is scaled
   * by sqrt(hidden_size) and every RMSNorm multiplies by (1 + weight) (gemma_rms_norm,
   * src/layers/norm.cpp:40-53).  0 = the llama-type path. */
  int gemma;
  /* FFN activation: LMB_ACT_SILU = silu(gate) * up (the reference's default branch,
   * src/model.cpp:414-416), LMB_ACT_GELU = gelu(gate) * up with the tanh form of src/model.cpp:38-42
   * (ActivationType::GELU, :409-412). */
  int activation;
} lmb_model_config;
enum { LMB_ACT_SILU = 0, LMB_ACT_GELU = 1 };

enum { /* tensor slots of lmb_model_set_weight */
  LMB_SLOT_EMBED = 0, LMB_SLOT_LM_HEAD = 1, LMB_SLOT_Q = 2, LMB_SLOT_K = 3, LMB_SLOT_V = 4,
  LMB_SLOT_O = 5, LMB_SLOT_GATE = 6, LMB_SLOT_UP = 7, LMB_SLOT_DOWN = 8
};
enum { /* vector slots of lmb_model_set_vector */
  LMB_VEC_INPUT_NORM = 0, LMB_VEC_POST_NORM = 1, LMB_VEC_Q_BIAS = 2, LMB_VEC_K_BIAS = 3,
  LMB_VEC_V_BIAS = 4, LMB_VEC_FINAL_NORM = 5
};

int lmb_model_create(lmb_ctx *ctx, const lmb_model_config *cfg, lmb_model **out);
int lmb_model_destroy(lmb_model *m);
/* Full (unsharded) reference block arrays; the model keeps only its tensor-parallel shard. */
int lmb_model_set_weight(lmb_model *m, int layer, int slot, int kind, int quant_bits, const void *blocks,
                         size_t M, size_t K);
/* lm_head = embed_tokens without a second device copy: what load_model does when the file has
 * no lm_head tensor (src/model.cpp:667-689).  Unsharded models only; a sharded model keeps its
 * vocabulary rows of the head through lmb_model_set_weight(LMB_SLOT_LM_HEAD). */
int lmb_model_tie_head(lmb_model *m);
int lmb_model_set_vector(lmb_model *m, int layer, int which, const float *data, size_t n);
/* One decode step for `batch` sequences: token_ids[b] at positions[b].  h_logits is NULL or
 * batch*vocab floats on the host.  Batch 1 of a model whose seven projections per layer share
 * one block kind runs embedding and all layers as ONE persistent kernel (LMB_MODEL_PERSISTENT=0 in
 * the environment at lmb_model_create selects the launch-per-projection step instead). */
int lmb_model_forward(lmb_model *m, const int *token_ids, const size_t *positions, size_t batch, float *h_logits);
int lmb_model_logits_dev(lmb_model *m, const float **d_logits);
/* Failure-path test of the bounded waits between the phases of the persistent decode step (batch 1
 * runs embedding and all layers as one kernel whose CTAs wait for each other through arrival
 * counters): every wait expects `extra_arrivals` arrivals more than there are CTAs and polls at
 * most `spin_limit` times (0 = the default, about a second).  With extra_arrivals > 0 the first
 * wait runs out, the kernel records the phase and returns by itself, and the lmb_model_forward
 * call that fetches logits returns LMB_ERR_TIMEOUT; (0, 0) restores normal operation. */
int lmb_debug_model_waits(lmb_model *m, int extra_arrivals, unsigned spin_limit);
/* Per-phase timestamps of the persistent decode step (profiling aid).  The first call switches
 * the recording on (and returns only *n_phases); later calls return the last step's record:
 * out[2][n_phases][5] nanoseconds of the device's global timer for CTA 0 and for the last CTA at
 * {phase descriptor read, dependency met, activations prepared, main loop done, phase done},
 * followed by out[10 n_phases + 2 i] = the last CTA's arrival at the end of phase i and
 * out[10 n_phases + 2 i + 1] = the bitwise complement of the first CTA's arrival
 * (so `out` holds 12 * n_phases words),
 * types[i] = 0 embedding, 1 GEMV, 2 attention, 3 tensor-parallel reduce, kslices[i] = K split. */
int lmb_debug_model_timeline(lmb_model *m, unsigned long long *out, int *types, int *kslices, size_t cap_phases,
                             size_t *n_phases);
int lmb_model_reset(lmb_model *m);
/* KV cache exchange in the reference layout [layer][2][max_seq][kv_heads][head_dim]
 * (types.hpp:599-627) for sequence `seq`.  The host buffer always has the layout of the whole
 * model; a tensor-parallel rank reads / fills only the columns of its own KV heads. */
int lmb_model_kv_export(lmb_model *m, size_t seq, float *h_out);
int lmb_model_kv_import(lmb_model *m, size_t seq, const float *h_in);
/* Algorithmic bytes one decode step reads at the given context length (weights + KV + embedding row). */
int lmb_model_step_bytes(lmb_model *m, size_t position, uint64_t *bytes_out);

/* ---- .lutmac files: replaces load_lutmac (src/format.cpp:292-505) and load_model
 * (include/lutmac/model.hpp:147, src/model.cpp:576-699) -------------------------------------------
 * lmb_file_* expose the parsed header (kind = block kind or -1 for raw fp32 tensors) and read one
 * tensor's bytes; lmb_model_load builds the device-resident model: tensor names are mapped to
 * slots like the reference does, the head is tied to the embedding when the file has none.
 * max_seq = 0 keeps the reference's 2048 cache positions. */
typedef struct lmb_file lmb_file;
int lmb_file_open(const char *path, lmb_file **out);
int lmb_file_close(lmb_file *f);
int lmb_file_config(const lmb_file *f, lmb_model_config *cfg_out);
int lmb_file_tensor_count(const lmb_file *f, size_t *n);
int lmb_file_tensor_info(const lmb_file *f, size_t i, const char **name, int *kind, int *quant_bits, size_t *dim0,
                         size_t *dim1, size_t *num_blocks);
int lmb_file_read_tensor(lmb_file *f, size_t i, void *dst, size_t dst_bytes);
int lmb_model_load(lmb_ctx *ctx, const char *path, size_t max_batch, size_t max_seq, int tp_rank, int tp_size,
                   lmb_model **out);

/* ---- tensor parallelism (no counterpart in the reference, which is single-process) ---------------
 * One process per GPU.  Rank 0 obtains a 128-byte NCCL unique id, the host distributes it by
 * whatever means it has, every rank calls lmb_tp_init with it.  Collectives run on the
 * context's stream.  A model created on a context with tp_size > 1 in its config keeps only
 * its shard: q/k/v/gate/up by output rows (whole heads), o/down by 256-column blocks, lm_head
 * by vocabulary rows; it all-reduces after o_proj and down_proj and all-gathers the logits. */
int lmb_tp_unique_id(void *id128_out);
int lmb_tp_init(lmb_ctx *ctx, const void *id128, int rank, int size);
int lmb_tp_destroy(lmb_ctx *ctx);
/* One-shot all-reduce over peer memory for the decode step (no counterpart in the single-process
 * reference).  After lmb_tp_init every rank creates its exchange block (room for max_floats =
 * max batch x hidden size per partial vector) and gets a 64-byte inter-process handle; the host
 * gathers the handles of all ranks in rank order and every rank opens them.  From then on the
 * o_proj / down_proj kernels of lmb_model_forward store their partial outputs (tagged with an
 * epoch) straight into every rank's block and the following normalisation kernel waits (at most
 * about a second) for the words of all ranks before it adds them; lmb_tp_peer_status reports whether a wait ever ran out.
 * lmb_model_forward returns LMB_ERR_TIMEOUT for a step whose logits it fetched after a wait ran out.
 * Without the block (or with LMB_TP_PEERS=0) the step uses lmb_allreduce_sum (NCCL). */
int lmb_tp_peer_create(lmb_ctx *ctx, size_t max_floats, void *handle64_out);
int lmb_tp_peer_open(lmb_ctx *ctx, const void *handles_rank_order);
int lmb_tp_peer_status(lmb_ctx *ctx, int *timed_out);
/* Self-test of that bounded wait on ONE GPU, without NCCL and without a second process: builds a
 * local exchange block for `ranks` ranks, posts the tagged partial vectors of the first `posted`
 * ranks only (rank r contributes the value r + 1 in every element), runs the consumer kernel once
 * with `spin_limit` polls per word and reports out4 = {timed_out flag, epoch afterwards, CTA
 * counter afterwards, 1 if the hidden vector equals the sum of the posted partials}.  With
 * posted < ranks the wait runs out and the kernel returns by itself: nothing faults or hangs. */
int lmb_debug_tp_wait(lmb_ctx *ctx, int ranks, int posted, size_t h, unsigned spin_limit, int out4[4]);
/* The same for the consumer kernel of batch-1 steps with integer tensor-core layouts, which also leaves
 * the hidden state as the next projections' prepared activations (h a multiple of 256). */
int lmb_debug_tp_wait_prepare(lmb_ctx *ctx, int ranks, int posted, size_t h, unsigned spin_limit, int out4[4]);
int lmb_allreduce_sum(lmb_ctx *ctx, float *d_buf, size_t n_floats);
int lmb_allgather(lmb_ctx *ctx, const float *d_send, float *d_recv, size_t n_floats_per_rank);

#ifdef __cplusplus
}
#endif
#endif /* LUTMAC_B200_H */
