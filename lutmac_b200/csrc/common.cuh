// Shared definitions of the lutmac_b200 CUDA library: block kinds, the device tile layout,
// error plumbing and the context object.
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <string>

#include "../../include/lutmac_b200.h"

namespace lmb {

constexpr int BLK = 256;       // weights per block (every reference block struct)
constexpr int TILE_ROWS = 32;  // rows per device tile: one warp lane per row
constexpr int SM_COUNT_HINT = 148;

// ---------------------------------------------------------------------------------------------
// Device tile layout
//
// A weight matrix of M rows and bpr = ceil(K/256) block-columns is stored as tiles of 32 rows
// x 1 block-column, row-tile major: tile (rt, b) starts at ((rt * bpr) + b) * tile_bytes.
// Inside a tile:
//     payload  [chunk c][lane l][16 bytes]     c < chunks(kind), l = row within the tile
//     scales   [scale s][lane l] float          s < nscales(kind)
// so that lane l of a warp reads its row with 128-bit loads that are contiguous across the
// warp (512 B per load).  tile_bytes = 32 * sizeof(reference block): the device copy has
// exactly the reference's bytes.  Rows beyond M are padded with zero-weight blocks.
//
// What a lane's chunks hold, per kind (256 weights w0..w255 of one reference block):
//   TERNARY  (table-lookup layout; the default device layout of ternary weights is
//            DK_TERNARY_MMA below) 4 chunks; chunk c = { P[8c..8c+7], N[8c..8c+7] } where P = ~zero & ~sign and
//            N = ~zero & sign are the positive / negative masks of extract_indices
//            (lut_gemm.hpp:79-99), same byte order and MSB-first bit order as the planes.
//   BINARY   2 chunks; chunk c = data[16c..16c+15] unchanged.
//   INT2     4 chunks; chunk c = { B1[8c..8c+7], B2[8c..8c+7] }: the primary and residual
//            bits of the interleaved (b1,b2) pairs split into two MSB-first bit planes.
//   INT3     6 chunks; chunk 3j+p = Q_{2-p}[16j..16j+15] (j < 2): bit planes of the 3-bit
//            code, most significant plane first.
//   INT4     8 chunks in the operand order of the 8-bit integer MMA (m16n8k32) instead of one
//            row per lane: chunk h*4+q of lane (g = lane/4, tid = lane%4) = four words
//            {WA(2q), WB(2q), WA(2q+1), WB(2q+1)}; byte j of WA(s) is column 32s+4tid+j, of WB(s)
//            column 32s+16+4tid+j; the low nibble is row 16h+g, the high nibble row 16h+g+8.
//            Scales: float 4g+m = scale of row g+8m.
//   INT5     10 chunks; 0..7 = low nibbles of the 5-bit codes in the INT4 arrangement, 8..9 = the
//            bit-4 plane in the DK_BINARY_MMA arrangement.
//   INT6     12 chunks; as INT5 plus 10..11 = the bit-5 plane.
//   INT8     16 chunks; chunk c = data[16c..16c+15] unchanged.
//   DK_TERNARY_MMA  4 chunks of 2-bit codes t+1 in MMA operand order: chunk q of lane (g, tid) =
//            {WA(2q), WB(2q), WA(2q+1), WB(2q+1)} with the same columns per byte as INT4; the
//            2-bit field m (bits 2m, 2m+1) of every byte is row g+8m.  Scales as for INT4.
//   DK_INT2_MMA  the DK_TERNARY_MMA arrangement with the field holding b1 (bit 2m) and b2
//            (bit 2m+1) of the residual-binary pair; scales [plane][4g+m].
//   DK_INT3_MMA  6 chunks: chunks 2p, 2p+1 = bit plane p (p = 0 the least significant bit of the
//            3-bit code) in the DK_BINARY_MMA arrangement.
//   DK_INT8_MMA  16 chunks: chunk 8h+s of lane (g, tid) = the four A-operand registers of k-step s
//            for rows 16h+g / 16h+g+8: {row g: columns 32s+4tid..+3, row g+8: the same, row g:
//            columns 32s+16+4tid..+3, row g+8: the same}.
//   DK_BINARY_MMA  2 chunks: words W(sp, ab), sp < 4, ab < 2, word index 2sp+ab; byte j, bit
//            m+4kh of W(sp, ab) is row g+8m, column 32(2sp+kh) + 16ab + 4tid + j.
// ---------------------------------------------------------------------------------------------
// Device-only layout kind: ternary weights as 2-bit codes (t+1) in the operand order of the
// 8-bit integer MMA.  lmb_weight::kind holds the device layout, lmb_weight::ref_kind the
// reference block kind it was made from.
constexpr int DK_TERNARY_MMA = 16;
// The same for INT2 (residual binary) and BINARY blocks.
constexpr int DK_INT2_MMA = 17;
constexpr int DK_BINARY_MMA = 18;
// INT8 blocks in the operand order of the signed 8-bit MMA (the tile's words are the operands).
constexpr int DK_INT8_MMA = 19;
// INT3 blocks as three bit planes in the DK_BINARY_MMA arrangement.
constexpr int DK_INT3_MMA = 20;

__host__ __device__ constexpr bool kind_is_mma(int kind) {
  return kind == LMB_INT4 || kind == LMB_INT5 || kind == LMB_INT6 || kind == DK_TERNARY_MMA || kind == DK_INT2_MMA ||
         kind == DK_BINARY_MMA || kind == DK_INT8_MMA || kind == DK_INT3_MMA;
}

struct KindInfo {
  int ref_bytes;   // sizeof the reference block struct
  int chunks;      // 16-byte payload chunks per row-block
  int nscales;     // floats per row-block
  bool lut;        // evaluated by group-of-4 table lookups (else dequantise + FMA)
};

__host__ __device__ constexpr KindInfo kind_info(int kind) {
  return kind == LMB_TERNARY ? KindInfo{68, 4, 1, true}
       : kind == LMB_BINARY  ? KindInfo{36, 2, 1, true}
       : kind == LMB_INT2    ? KindInfo{72, 4, 2, true}
       : kind == LMB_INT3    ? KindInfo{100, 6, 1, true}
       : kind == LMB_INT4    ? KindInfo{132, 8, 1, false}
       : kind == LMB_INT5    ? KindInfo{164, 10, 1, false}
       : kind == LMB_INT6    ? KindInfo{196, 12, 1, false}
       : kind == LMB_INT8    ? KindInfo{260, 16, 1, false}
       : kind == DK_TERNARY_MMA ? KindInfo{68, 4, 1, false}
       : kind == DK_INT2_MMA ? KindInfo{72, 4, 2, false}
       : kind == DK_BINARY_MMA ? KindInfo{36, 2, 1, false}
       : kind == DK_INT8_MMA ? KindInfo{260, 16, 1, false}
       : kind == DK_INT3_MMA ? KindInfo{100, 6, 1, false}
                             : KindInfo{0, 0, 0, false};
}

__host__ __device__ constexpr size_t tile_bytes(int kind) { return size_t(TILE_ROWS) * kind_info(kind).ref_bytes; }

inline bool kind_valid(int kind) { return kind_info(kind).ref_bytes != 0; }

// ---------------------------------------------------------------------------------------------
// Errors
// ---------------------------------------------------------------------------------------------
void set_last_error(const std::string &msg);
int cuda_fail(cudaError_t e, const char *what);

#define LMB_CUDA(call)                                              \
  do {                                                              \
    cudaError_t _e = (call);                                        \
    if (_e != cudaSuccess) return ::lmb::cuda_fail(_e, #call);      \
  } while (0)

#define LMB_REQUIRE(cond, msg)                                      \
  do {                                                              \
    if (!(cond)) {                                                  \
      ::lmb::set_last_error(msg);                                   \
      return LMB_ERR_ARG;                                           \
    }                                                               \
  } while (0)

}  // namespace lmb

// ---------------------------------------------------------------------------------------------
// Opaque handles of the C ABI
// ---------------------------------------------------------------------------------------------
namespace lmb {
// One-shot all-reduce over peer memory (tensor parallelism, one process per GPU).  Every rank
// owns one exchange block, mapped by all ranks: a header (epoch, CTA counter, time-out flag) and
// the partial vectors [2 parities][ranks][cap] as 8-byte words {value, epoch tag}.  The kernel
// that produces a partial vector stores every element, tagged, into every rank's block with one
// 8-byte store (no fence, no separate flag); the kernel that consumes the sum reads each word
// until its tag is the expected one and adds the partials in rank order.
constexpr int MAX_TP = 8;
constexpr size_t XCHG_HEADER_BYTES = 1024;
struct XchgHeader {
  unsigned reserved[MAX_TP];
  unsigned pad0[24];
  unsigned epoch;          // all-reduces this rank has consumed; the next vector carries the tag epoch + 1
  unsigned pad1[15];
  unsigned done;           // CTAs of the running consumer kernel that have finished
  unsigned pad2[15];
  unsigned timed_out;      // set when a consumer gave up waiting
};
struct PeerXchg {
  bool ready = false;
  unsigned spin_limit = 1u << 22;  // polls (a 40 ns sleep and a load each) before a consumer gives up: a few seconds; LMB_TP_WAIT_POLLS
  size_t cap = 0;            // floats per (parity, rank) slot
  void *local = nullptr;     // this rank's block
  void *peer[MAX_TP] = {};   // every rank's block as mapped here (own block included)
};
// What a GEMV launch needs to deliver its output to all ranks (n = 0: ordinary output).
struct PeerOut {
  unsigned long long *data[MAX_TP];  // tagged words: value in the low half, epoch tag in the high half
  unsigned *epoch;
  int n, rank;
  unsigned cap;
};
}  // namespace lmb

struct lmb_ctx {
  int device = 0;
  lmb::PeerXchg xchg;
  cudaStream_t own_stream = nullptr;
  cudaStream_t stream = nullptr;  // the stream work is issued on (own_stream unless overridden)
  cudaEvent_t ev0 = nullptr, ev1 = nullptr;
  int sm_count = lmb::SM_COUNT_HINT;
  size_t smem_optin = 0;  // max dynamic shared memory per block
  uint64_t launches = 0;
  uint64_t capture_base = 0;
  void *comm = nullptr;  // NCCL communicator (tensor parallelism)
  int tp_rank = 0, tp_size = 1;
  bool pdl = true;
  bool ternary_lut = false;  // upload ternary weights for the table-lookup kernel instead of the MMA kernel  // programmatic dependent launch between consecutive kernels
  // scratch for split-K partial sums and its arrival counters (grown on demand)
  // scratch_gen counts reallocations of scratch / counters / xprep: a captured graph holds the raw
  // pointers and must be captured again when the generation it was captured under is gone
  uint64_t scratch_gen = 0;
  float *scratch = nullptr;
  size_t scratch_floats = 0;
  unsigned *counters = nullptr;
  size_t n_counters = 0;
  // activations prepared once per launch for batched GEMVs (digits, block scales, digit sums)
  uint32_t *xprep = nullptr;
  size_t xprep_blocks = 0;  // capacity in (sequence, block) pairs
  // set by a kernel whose bounded wait (for its own asynchronous copies) ran out; read with the logits
  unsigned *d_fault = nullptr;
  // launch timeline (debugging, lmb_debug_launch_timeline): 8 time stamps per launch, null when off
  unsigned long long *d_timeline = nullptr;
  int timeline_cap = 0, timeline_cursor = 0, timeline_used = 0;  // used: most slots any step has taken (graph replays launch nothing)
  void *h_upload = nullptr;  // pinned staging of lmb_weight_upload
  size_t h_upload_bytes = 0;
  // staging buffers of the host-pointer entry points
  void *h_stage = nullptr;
  size_t h_stage_bytes = 0;
  float *d_stage = nullptr;
  size_t d_stage_bytes = 0;
};

// The next launch's slot of the launch timeline, or null (off / full).
inline unsigned long long *timeline_slot(lmb_ctx *ctx) {
  if (!ctx->d_timeline || ctx->timeline_cursor >= ctx->timeline_cap) return nullptr;
  unsigned long long *slot = ctx->d_timeline + size_t(8) * size_t(ctx->timeline_cursor++);
  if (ctx->timeline_cursor > ctx->timeline_used) ctx->timeline_used = ctx->timeline_cursor;
  return slot;
}

#ifdef LMB_DEBUG_BOUNDS
namespace lmb {
// test hook of the range-checking build: launches claim their weight buffers this many bytes shorter
// than they are, so that the check of the last tiles trips (and skips the loads) while every access
// that does run stays inside the real buffer
extern size_t g_bounds_shrink;
}
#endif

struct lmb_weight {
  int kind = 0;      // device layout kind (a reference kind, or DK_TERNARY_MMA)
  int ref_kind = 0;  // reference block kind
  int device = 0;
  size_t M = 0, K = 0;   // logical shape (of the shard, if sharded)
  size_t bpr = 0;        // block-columns
  size_t row_tiles = 0;  // ceil(M / 32)
  uint8_t *d_tiles = nullptr;
  size_t bytes = 0;
};

namespace lmb {

// Launchers (implemented in the kernel files).  All pointers are device pointers.
struct LinearArgs {
  const lmb_weight *w;
  const float *bias;
  const float *x;
  size_t x_len, x_stride;
  float *y;
  size_t y_stride;
  size_t batch;
  bool rotate;
  const float *x2 = nullptr;        // norm weight (XMODE_RMSNORM) or the vector multiplied in (XMODE_SILU_MUL, XMODE_GELU_MUL)
  const float *residual = nullptr;  // added to the output (same layout as y; may alias y)
  bool to_peers = false;            // deliver y into every rank's exchange block instead (single-job launches)
  // Hand-off of prepared activations between two batch-1 GEMVs (integer tensor-core kinds).  Producer
  // side: next_prep / next_sumsq receive, per 256-block of this GEMV's output, the record the next
  // GEMV's CTAs would otherwise each compute (output x next_w, rotated if next_rotate, as fixed-point
  // digits) and the block's sum of squares.  Consumer side: prep_in / prep_sumsq_in (prep_sumsq_n
  // blocks) replace x; with prep_sumsq_in the vector is RMS-normalised by the total.
  uint32_t *next_prep = nullptr;
  float *next_sumsq = nullptr;
  const float *next_w = nullptr;
  bool next_rotate = false;
  const uint32_t *prep_in = nullptr;
  const float *prep_sumsq_in = nullptr;
  int prep_sumsq_n = 0;
};
constexpr int PREP_RECORD_WORDS = 256 + 4;  // one prepared 256-block: digits, block scale, two digit-pair sums, pad
// How the GEMV prologue forms its activations from x.
enum { XMODE_PLAIN = 0, XMODE_RMSNORM = 1, XMODE_SILU_MUL = 2, XMODE_GELU_MUL = 3 };
int configure_gemv(lmb_ctx *ctx);
int launch_tp_sum_prepare(lmb_ctx *ctx, float *d_hidden, const float *d_w, bool rotate, uint32_t *prep, float *sumsq, size_t h);
int launch_gemv(lmb_ctx *ctx, const LinearArgs *args, int njobs, bool rotate, int xmode = XMODE_PLAIN, float eps = 0.0f);
int launch_fwht256(lmb_ctx *ctx, float *d_x, size_t n);
int launch_debug_luts(lmb_ctx *ctx, const float *d_x, size_t x_len, bool rotate, float *d_out);

int model_tie_head(lmb_model *m);  // definition of lmb_model_tie_head
int ensure_scratch(lmb_ctx *ctx, size_t floats, size_t counters);
int ensure_stage(lmb_ctx *ctx, size_t bytes);

}  // namespace lmb
