// C ABI: context, device memory helpers, weight upload, the layer / kernel / transform entry
// points.  Declarations and the reference interfaces they replace: include/lutmac_b200.h.
#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <new>
#include <vector>

#include "common.cuh"
#include "device_utils.cuh"

namespace lmb {

void retile(int kind, const uint8_t *blocks, size_t src_bpr, size_t row0, size_t row1, size_t blk0, size_t blk1,
            uint8_t *tiled);
void untile(int kind, const uint8_t *tiled, size_t M, size_t bpr, uint8_t *blocks);

static thread_local std::string g_last_error;

void set_last_error(const std::string &msg) { g_last_error = msg; }

int cuda_fail(cudaError_t e, const char *what) {
  g_last_error = std::string(what) + ": " + cudaGetErrorName(e) + " (" + cudaGetErrorString(e) + ")";
  return LMB_ERR_CUDA;
}

int ensure_scratch(lmb_ctx *ctx, size_t floats, size_t counters) {
  if (floats > ctx->scratch_floats) {
    if (ctx->scratch) LMB_CUDA(cudaFree(ctx->scratch));
    ctx->scratch = nullptr;
    ctx->scratch_floats = 0;
    LMB_CUDA(cudaMalloc(&ctx->scratch, floats * sizeof(float)));
    ctx->scratch_floats = floats;
    ctx->scratch_gen++;
  }
  if (counters > ctx->n_counters) {
    if (ctx->counters) LMB_CUDA(cudaFree(ctx->counters));
    ctx->counters = nullptr;
    ctx->n_counters = 0;
    LMB_CUDA(cudaMalloc(&ctx->counters, counters * sizeof(unsigned)));
    LMB_CUDA(cudaMemsetAsync(ctx->counters, 0, counters * sizeof(unsigned), ctx->stream));
    ctx->n_counters = counters;
    ctx->scratch_gen++;
  }
  return LMB_OK;
}

int ensure_stage(lmb_ctx *ctx, size_t bytes) {
  if (bytes > ctx->h_stage_bytes) {
    if (ctx->h_stage) LMB_CUDA(cudaFreeHost(ctx->h_stage));
    ctx->h_stage = nullptr;
    ctx->h_stage_bytes = 0;
    LMB_CUDA(cudaMallocHost(&ctx->h_stage, bytes));
    ctx->h_stage_bytes = bytes;
  }
  if (bytes > ctx->d_stage_bytes) {
    if (ctx->d_stage) LMB_CUDA(cudaFree(ctx->d_stage));
    ctx->d_stage = nullptr;
    ctx->d_stage_bytes = 0;
    LMB_CUDA(cudaMalloc(&ctx->d_stage, bytes));
    ctx->d_stage_bytes = bytes;
  }
  return LMB_OK;
}

// --- standalone FWHT (one warp per 256-block, in place) ------------------------------------------
__global__ void k_fwht256(float *x, size_t nblocks) {
  const int lane = threadIdx.x & 31;
  const size_t b = size_t(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (b >= nblocks) return;
  float v[8];
  load_x8(x, (b + 1) * 256, b, lane, v);
  fwht256_warp(v, lane);
  float *o = x + b * 256 + size_t(lane) * 8;
#pragma unroll
  for (int j = 0; j < 8; ++j) o[j] = v[j];
}

int launch_fwht256(lmb_ctx *ctx, float *d_x, size_t n) {
  const size_t nblocks = n / 256;  // a trailing partial block stays untouched (transform_simd.cpp:104-108)
  if (nblocks == 0) return LMB_OK;
  const unsigned grid = unsigned((nblocks + 7) / 8);
  k_fwht256<<<grid, 256, 0, ctx->stream>>>(d_x, nblocks);
  ctx->launches++;
  LMB_CUDA(cudaGetLastError());
  return LMB_OK;
}

// Unquantised weights: the raw fp32 branch of lut_linear (lut_gemm_scalar.cpp:157-171), y = W x + bias
// with W row-major [M][K].  One warp per row, 128-bit loads where the row is 16-byte aligned.
__global__ void __launch_bounds__(256) k_gemv_raw(const float *__restrict__ W, const float *x, const float *bias, float *y, size_t M,
                                                  size_t K, size_t x_len, size_t x_stride) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const size_t row = size_t(blockIdx.x) * 8 + warp;
  if (row >= M) return;
  const float *w = W + row * K, *xb = x + size_t(blockIdx.y) * x_stride;
  const size_t n = x_len < K ? x_len : K;  // columns at or beyond x_len read as zero
  float acc = 0.0f;
  if ((K & 3) == 0 && ((reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(xb)) & 15) == 0) {
    const size_t n4 = n / 4;
    for (size_t i = lane; i < n4; i += 32) {
      const float4 a = ld_stream_v4f(w + 4 * i), b = *reinterpret_cast<const float4 *>(xb + 4 * i);
      acc += (a.x * b.x + a.y * b.y) + (a.z * b.z + a.w * b.w);
    }
    for (size_t i = 4 * n4 + lane; i < n; i += 32) acc += w[i] * xb[i];
  } else {
    for (size_t i = lane; i < n; i += 32) acc += w[i] * xb[i];
  }
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, m);
  if (lane == 0) y[size_t(blockIdx.y) * M + row] = acc + (bias ? bias[row] : 0.0f);
}

static int linear_impl(lmb_ctx *ctx, const lmb_weight *w, const float *d_bias, const float *d_x, size_t x_len,
                       size_t x_stride, float *d_y, size_t batch, unsigned flags) {
  LMB_REQUIRE(ctx && w && d_x && d_y, "lmb_linear: null argument");
  LMB_REQUIRE(batch > 0 && batch <= 65535, "lmb_linear: batch must be in 1..65535");
  LMB_REQUIRE(w->device == ctx->device, "lmb_linear: weight lives on another device");
  LMB_REQUIRE(x_len <= w->bpr * size_t(BLK), "lmb_linear: x_len exceeds the padded input width");
  if (w->kind == LMB_RAW_F32) {
    LMB_REQUIRE(!(flags & LMB_ROTATE), "lmb_linear: the unquantised branch of lut_linear never rotates its input");
    dim3 grid(unsigned((w->M + 7) / 8), unsigned(batch));
    k_gemv_raw<<<grid, 256, 0, ctx->stream>>>(reinterpret_cast<const float *>(w->d_tiles), d_x, d_bias, d_y, w->M, w->K, x_len, x_stride);
    ctx->launches++;
    LMB_CUDA(cudaGetLastError());
    return LMB_OK;
  }
  LinearArgs a;
  a.w = w;
  a.bias = d_bias;
  a.x = d_x;
  a.x_len = x_len;
  a.x_stride = x_stride;
  a.y = d_y;
  a.y_stride = w->M;
  a.batch = batch;
  // lut_linear rotates iff 0 < quant_bits <= 2 or the ternary block vector is non-empty
  // (lut_gemm_scalar.cpp:92-93): ternary, binary and 2-bit tensors.
  const bool auto_rot = (w->ref_kind == LMB_TERNARY || w->ref_kind == LMB_BINARY || w->ref_kind == LMB_INT2);
  a.rotate = (flags & LMB_ROTATE) || ((flags & LMB_AUTO_ROTATE) && auto_rot);
  return launch_gemv(ctx, &a, 1, a.rotate);
}

static std::mutex g_default_mu;
static std::vector<lmb_ctx *> g_default_ctx;  // per device, for the host-pointer kernel API

static int default_ctx(lmb_ctx **out) {
  int dev = 0;
  LMB_CUDA(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lk(g_default_mu);
  if (g_default_ctx.size() <= size_t(dev)) g_default_ctx.resize(size_t(dev) + 1, nullptr);
  if (!g_default_ctx[size_t(dev)]) {
    int st = lmb_ctx_create(dev, &g_default_ctx[size_t(dev)]);
    if (st != LMB_OK) return st;
  }
  *out = g_default_ctx[size_t(dev)];
  return LMB_OK;
}

}  // namespace lmb

using namespace lmb;

#ifdef LMB_DEBUG_BOUNDS
namespace lmb {
size_t g_bounds_shrink = 0;
namespace {
std::vector<BoundsReader> &bounds_readers() {
  static std::vector<BoundsReader> v;
  return v;
}
}  // namespace
void register_bounds_reader(BoundsReader fn) { bounds_readers().push_back(fn); }
}  // namespace lmb
#endif

extern "C" {

const char *lmb_strerror(int status) {
  switch (status) {
  case LMB_OK: return "ok";
  case LMB_ERR_ARG: return "invalid argument";
  case LMB_ERR_CUDA: return "CUDA error";
  case LMB_ERR_ALLOC: return "allocation failed";
  case LMB_ERR_TIMEOUT: return "bounded device wait expired";
  case LMB_ERR_FORMAT: return "malformed .lutmac file";
  case LMB_ERR_LIMIT: return "size beyond the entry point's limit";
  case LMB_ERR_STATE: return "call not valid in this state";
  default: return "unknown status";
  }
}

const char *lmb_last_error(void) { return g_last_error.c_str(); }

int lmb_device_count(int *out) {
  LMB_REQUIRE(out, "lmb_device_count: null argument");
  *out = 0;
  LMB_CUDA(cudaGetDeviceCount(out));
  return LMB_OK;
}

int lmb_ctx_create(int device, lmb_ctx **out) {
  LMB_REQUIRE(out, "lmb_ctx_create: null argument");
  *out = nullptr;
  int n = 0;
  LMB_CUDA(cudaGetDeviceCount(&n));
  LMB_REQUIRE(device >= 0 && device < n, "lmb_ctx_create: no such CUDA device");
  LMB_CUDA(cudaSetDevice(device));
  cudaDeviceProp prop;
  LMB_CUDA(cudaGetDeviceProperties(&prop, device));
  if (prop.major < 10) {
    set_last_error("lmb_ctx_create: this library contains sm_100a code only (Blackwell B200 required)");
    return LMB_ERR_CUDA;
  }
  lmb_ctx *ctx = new (std::nothrow) lmb_ctx();
  if (!ctx) return LMB_ERR_ALLOC;
  ctx->device = device;
  ctx->sm_count = prop.multiProcessorCount;
  ctx->smem_optin = prop.sharedMemPerBlockOptin;
  cudaError_t e = cudaStreamCreateWithFlags(&ctx->own_stream, cudaStreamNonBlocking);
  if (e == cudaSuccess) e = cudaEventCreate(&ctx->ev0);
  if (e == cudaSuccess) e = cudaEventCreate(&ctx->ev1);
  if (e != cudaSuccess) {
    delete ctx;
    return cuda_fail(e, "lmb_ctx_create");
  }
  ctx->stream = ctx->own_stream;
  const char *pdl_env = getenv("LMB_PDL");
  ctx->pdl = !(pdl_env && pdl_env[0] == '0');
  int st = configure_gemv(ctx);
  if (st == LMB_OK) st = ensure_scratch(ctx, size_t(4) << 20, size_t(1) << 16);
  if (st == LMB_OK) {
    e = cudaMalloc(&ctx->d_fault, sizeof(unsigned));
    if (e == cudaSuccess) e = cudaMemset(ctx->d_fault, 0, sizeof(unsigned));
    if (e != cudaSuccess) st = cuda_fail(e, "lmb_ctx_create");
  }
  if (st != LMB_OK) {
    lmb_ctx_destroy(ctx);
    return st;
  }
  *out = ctx;
  return LMB_OK;
}

int lmb_debug_bounds(lmb_ctx *ctx, unsigned long long out4[4]) {
  LMB_REQUIRE(ctx && out4, "lmb_debug_bounds: null argument");
#ifdef LMB_DEBUG_BOUNDS
  LMB_CUDA(cudaSetDevice(ctx->device));
  LMB_CUDA(cudaStreamSynchronize(ctx->stream));
  out4[0] = out4[1] = out4[2] = out4[3] = 0;
  for (lmb::BoundsReader fn : lmb::bounds_readers()) {
    unsigned long long r[4] = {0, 0, 0, 0};
    LMB_CUDA(static_cast<cudaError_t>(fn(r, true)));
    if (r[0] && !out4[0]) {
      out4[0] = r[0];
      out4[1] = r[1];
      out4[2] = r[2];
    }
    out4[3] += r[3];
  }
  return LMB_OK;
#else
  set_last_error("lmb_debug_bounds: this library was built without -DLMB_DEBUG_BOUNDS (python -m lutmac_b200.build --debug-bounds)");
  return LMB_ERR_STATE;
#endif
}

int lmb_debug_bounds_shrink(size_t bytes) {
#ifdef LMB_DEBUG_BOUNDS
  lmb::g_bounds_shrink = bytes;
  return LMB_OK;
#else
  (void)bytes;
  set_last_error("lmb_debug_bounds_shrink: this library was built without -DLMB_DEBUG_BOUNDS");
  return LMB_ERR_STATE;
#endif
}

int lmb_debug_launch_timeline(lmb_ctx *ctx, size_t cap_launches, unsigned long long *out, size_t *n_launches) {
  LMB_REQUIRE(ctx && n_launches, "lmb_debug_launch_timeline: null argument");
  LMB_CUDA(cudaSetDevice(ctx->device));
  LMB_CUDA(cudaStreamSynchronize(ctx->stream));
  if (!ctx->d_timeline) {
    LMB_REQUIRE(cap_launches > 0 && cap_launches < (size_t(1) << 20), "lmb_debug_launch_timeline: recording is off and no capacity was given");
    LMB_CUDA(cudaMalloc(&ctx->d_timeline, cap_launches * 8 * sizeof(unsigned long long)));
    ctx->timeline_cap = int(cap_launches);
    ctx->timeline_cursor = 0;
  }
  const size_t n = size_t(ctx->timeline_used), words = size_t(ctx->timeline_cap) * 8;
  if (out && n) LMB_CUDA(cudaMemcpy(out, ctx->d_timeline, n * 8 * sizeof(unsigned long long), cudaMemcpyDeviceToHost));
  *n_launches = n;
  std::vector<unsigned long long> init(words, 0ull);  // minima start at the largest value, maxima at 0
  for (size_t i = 0; i < words; i += 8) init[i] = init[i + 1] = init[i + 6] = ~0ull;
  LMB_CUDA(cudaMemcpy(ctx->d_timeline, init.data(), words * sizeof(unsigned long long), cudaMemcpyHostToDevice));
  return LMB_OK;
}

int lmb_ctx_destroy(lmb_ctx *ctx) {
  if (!ctx) return LMB_OK;
  cudaSetDevice(ctx->device);
  if (ctx->own_stream) cudaStreamSynchronize(ctx->own_stream);
  if (ctx->scratch) cudaFree(ctx->scratch);
  if (ctx->counters) cudaFree(ctx->counters);
  if (ctx->xprep) cudaFree(ctx->xprep);
  if (ctx->d_fault) cudaFree(ctx->d_fault);
  if (ctx->d_timeline) cudaFree(ctx->d_timeline);
  if (ctx->h_upload) cudaFreeHost(ctx->h_upload);
  if (ctx->h_stage) cudaFreeHost(ctx->h_stage);
  if (ctx->d_stage) cudaFree(ctx->d_stage);
  if (ctx->ev0) cudaEventDestroy(ctx->ev0);
  if (ctx->ev1) cudaEventDestroy(ctx->ev1);
  if (ctx->own_stream) cudaStreamDestroy(ctx->own_stream);
  delete ctx;
  return LMB_OK;
}

int lmb_ctx_set_stream(lmb_ctx *ctx, void *cuda_stream) {
  LMB_REQUIRE(ctx, "lmb_ctx_set_stream: null context");
  ctx->stream = cuda_stream ? static_cast<cudaStream_t>(cuda_stream) : ctx->own_stream;
  return LMB_OK;
}

int lmb_ctx_set_option(lmb_ctx *ctx, int option, int value) {
  LMB_REQUIRE(ctx, "lmb_ctx_set_option: null context");
  switch (option) {
  case LMB_OPT_TERNARY_LUT: ctx->ternary_lut = value != 0; return LMB_OK;
  case LMB_OPT_PDL: ctx->pdl = value != 0; return LMB_OK;
  case LMB_OPT_SCRATCH_FLOATS: {
    LMB_REQUIRE(value > 0, "lmb_ctx_set_option: the scratch size must be positive");
    LMB_CUDA(cudaStreamSynchronize(ctx->stream));
    if (ctx->scratch) LMB_CUDA(cudaFree(ctx->scratch));
    ctx->scratch = nullptr;
    ctx->scratch_floats = 0;
    ctx->scratch_gen++;
    return ensure_scratch(ctx, size_t(value), 0);
  }
  default: set_last_error("lmb_ctx_set_option: unknown option"); return LMB_ERR_ARG;
  }
}

int lmb_ctx_sync(lmb_ctx *ctx) {
  LMB_REQUIRE(ctx, "lmb_ctx_sync: null context");
  LMB_CUDA(cudaStreamSynchronize(ctx->stream));
  return LMB_OK;
}

int lmb_ctx_launch_count(lmb_ctx *ctx, uint64_t *out) {
  LMB_REQUIRE(ctx && out, "lmb_ctx_launch_count: null argument");
  *out = ctx->launches;
  return LMB_OK;
}

int lmb_malloc(lmb_ctx *ctx, size_t bytes, void **d_ptr) {
  LMB_REQUIRE(ctx && d_ptr, "lmb_malloc: null argument");
  LMB_CUDA(cudaSetDevice(ctx->device));
  LMB_CUDA(cudaMalloc(d_ptr, bytes ? bytes : 1));
  return LMB_OK;
}

int lmb_free(lmb_ctx *ctx, void *d_ptr) {
  LMB_REQUIRE(ctx, "lmb_free: null context");
  if (d_ptr) {
    LMB_CUDA(cudaStreamSynchronize(ctx->stream));
    LMB_CUDA(cudaFree(d_ptr));
  }
  return LMB_OK;
}

int lmb_memcpy_h2d(lmb_ctx *ctx, void *d_dst, const void *h_src, size_t bytes) {
  LMB_REQUIRE(ctx && (bytes == 0 || (d_dst && h_src)), "lmb_memcpy_h2d: null argument");
  LMB_CUDA(cudaMemcpyAsync(d_dst, h_src, bytes, cudaMemcpyHostToDevice, ctx->stream));
  LMB_CUDA(cudaStreamSynchronize(ctx->stream));
  return LMB_OK;
}

int lmb_memcpy_d2h(lmb_ctx *ctx, void *h_dst, const void *d_src, size_t bytes) {
  LMB_REQUIRE(ctx && (bytes == 0 || (h_dst && d_src)), "lmb_memcpy_d2h: null argument");
  LMB_CUDA(cudaMemcpyAsync(h_dst, d_src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
  LMB_CUDA(cudaStreamSynchronize(ctx->stream));
  return LMB_OK;
}

int lmb_memset(lmb_ctx *ctx, void *d_dst, int value, size_t bytes) {
  LMB_REQUIRE(ctx && (bytes == 0 || d_dst), "lmb_memset: null argument");
  LMB_CUDA(cudaMemsetAsync(d_dst, value, bytes, ctx->stream));
  return LMB_OK;
}

int lmb_host_alloc_pinned(size_t bytes, void **h_ptr) {
  LMB_REQUIRE(h_ptr, "lmb_host_alloc_pinned: null argument");
  LMB_CUDA(cudaMallocHost(h_ptr, bytes ? bytes : 1));
  return LMB_OK;
}

int lmb_host_free_pinned(void *h_ptr) {
  if (h_ptr) LMB_CUDA(cudaFreeHost(h_ptr));
  return LMB_OK;
}

int lmb_timer_start(lmb_ctx *ctx) {
  LMB_REQUIRE(ctx, "lmb_timer_start: null context");
  LMB_CUDA(cudaEventRecord(ctx->ev0, ctx->stream));
  return LMB_OK;
}

int lmb_timer_stop(lmb_ctx *ctx, float *ms_out) {
  LMB_REQUIRE(ctx && ms_out, "lmb_timer_stop: null argument");
  LMB_CUDA(cudaEventRecord(ctx->ev1, ctx->stream));
  LMB_CUDA(cudaEventSynchronize(ctx->ev1));
  LMB_CUDA(cudaEventElapsedTime(ms_out, ctx->ev0, ctx->ev1));
  return LMB_OK;
}

// ---- CUDA graphs ------------------------------------------------------------------------------------
struct lmb_graph {
  cudaGraphExec_t exec = nullptr;
  uint64_t launches = 0;  // kernels captured in the graph
  uint64_t scratch_gen = 0;  // lmb_ctx::scratch_gen at capture: the graph holds the scratch pointers of that generation
};

int lmb_graph_begin(lmb_ctx *ctx) {
  LMB_REQUIRE(ctx, "lmb_graph_begin: null context");
  ctx->capture_base = ctx->launches;
  LMB_CUDA(cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
  return LMB_OK;
}

int lmb_graph_end(lmb_ctx *ctx, lmb_graph **out) {
  LMB_REQUIRE(ctx && out, "lmb_graph_end: null argument");
  *out = nullptr;
  cudaGraph_t g = nullptr;
  LMB_CUDA(cudaStreamEndCapture(ctx->stream, &g));
  lmb_graph *h = new (std::nothrow) lmb_graph();
  if (!h) {
    cudaGraphDestroy(g);
    return LMB_ERR_ALLOC;
  }
  cudaError_t e = cudaGraphInstantiate(&h->exec, g, 0);
  cudaGraphDestroy(g);
  if (e != cudaSuccess) {
    delete h;
    return cuda_fail(e, "cudaGraphInstantiate");
  }
  h->launches = ctx->launches - ctx->capture_base;
  h->scratch_gen = ctx->scratch_gen;
  ctx->launches = ctx->capture_base;  // captured launches have not run yet
  *out = h;
  return LMB_OK;
}

int lmb_graph_launch(lmb_ctx *ctx, lmb_graph *g) {
  LMB_REQUIRE(ctx && g && g->exec, "lmb_graph_launch: null argument");
  if (g->scratch_gen != ctx->scratch_gen) {
    set_last_error("lmb_graph_launch: the context's split-K scratch was reallocated after this graph was captured "
                   "(a later call needed more); capture the graph again");
    return LMB_ERR_STATE;
  }
  LMB_CUDA(cudaGraphLaunch(g->exec, ctx->stream));
  ctx->launches += g->launches;
  return LMB_OK;
}

int lmb_graph_destroy(lmb_graph *g) {
  if (!g) return LMB_OK;
  if (g->exec) cudaGraphExecDestroy(g->exec);
  delete g;
  return LMB_OK;
}

// ---- weights ---------------------------------------------------------------------------------------
int lmb_weight_upload_shard(lmb_ctx *ctx, int kind, const void *blocks, size_t M, size_t K, size_t row0,
                            size_t row1, size_t blk0, size_t blk1, lmb_weight **out) {
  LMB_REQUIRE(ctx && blocks && out, "lmb_weight_upload: null argument");
  if (kind == LMB_RAW_F32) {  // row-major fp32, kept as it is (rows [row0,row1) only; no column shards)
    LMB_REQUIRE(M > 0 && K > 0 && row0 < row1 && row1 <= M && blk0 == 0 && blk1 == (K + BLK - 1) / BLK,
                "lmb_weight_upload: an unquantised matrix can be sharded by rows only");
    *out = nullptr;
    lmb_weight *w = new (std::nothrow) lmb_weight();
    if (!w) return LMB_ERR_ALLOC;
    w->kind = w->ref_kind = LMB_RAW_F32;
    w->device = ctx->device;
    w->M = row1 - row0;
    w->K = K;
    w->bpr = blk1;
    w->row_tiles = (w->M + TILE_ROWS - 1) / TILE_ROWS;
    w->bytes = w->M * K * sizeof(float);
    cudaError_t e = cudaSetDevice(ctx->device);
    if (e == cudaSuccess) e = cudaMalloc(&w->d_tiles, w->bytes);
    if (e == cudaSuccess) e = cudaMemcpyAsync(w->d_tiles, static_cast<const float *>(blocks) + row0 * K, w->bytes, cudaMemcpyHostToDevice, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) {
      if (w->d_tiles) cudaFree(w->d_tiles);
      delete w;
      return cuda_fail(e, "lmb_weight_upload(raw)");
    }
    *out = w;
    return LMB_OK;
  }
  LMB_REQUIRE(kind_valid(kind), "lmb_weight_upload: unknown block kind");
  const size_t src_bpr = (K + BLK - 1) / BLK;
  LMB_REQUIRE(M > 0 && K > 0, "lmb_weight_upload: empty shape");
  LMB_REQUIRE(row0 < row1 && row1 <= M && blk0 < blk1 && blk1 <= src_bpr, "lmb_weight_upload: bad shard range");
  LMB_REQUIRE(M < (size_t(1) << 31) && K < (size_t(1) << 31), "lmb_weight_upload: dimension too large");
  *out = nullptr;
  lmb_weight *w = new (std::nothrow) lmb_weight();
  if (!w) return LMB_ERR_ALLOC;
  w->ref_kind = kind;
  w->kind = kind;
  if (!ctx->ternary_lut) {  // the integer-MMA layouts are the default for these kinds
    if (kind == LMB_TERNARY) w->kind = DK_TERNARY_MMA;
    if (kind == LMB_INT2) w->kind = DK_INT2_MMA;
    if (kind == LMB_BINARY) w->kind = DK_BINARY_MMA;
    if (kind == LMB_INT8) w->kind = DK_INT8_MMA;
    if (kind == LMB_INT3) w->kind = DK_INT3_MMA;
  }
  w->device = ctx->device;
  w->M = row1 - row0;
  w->bpr = blk1 - blk0;
  // The last block-column of an unsharded matrix may be partial; a shard's width is whole blocks
  // except when it includes that last column.
  w->K = (blk1 == src_bpr) ? (K - blk0 * BLK) : (w->bpr * BLK);
  w->row_tiles = (w->M + TILE_ROWS - 1) / TILE_ROWS;
  w->bytes = w->row_tiles * w->bpr * tile_bytes(w->kind);
  // re-tile into the context's pinned upload buffer (kept and grown on demand: allocating pinned
  // memory per tensor costs more than the copy it serves)
  cudaError_t e = cudaSuccess;
  if (w->bytes > ctx->h_upload_bytes) {
    if (ctx->h_upload) cudaFreeHost(ctx->h_upload);
    ctx->h_upload = nullptr;
    ctx->h_upload_bytes = 0;
    e = cudaMallocHost(&ctx->h_upload, w->bytes);
    if (e != cudaSuccess) {
      delete w;
      return cuda_fail(e, "cudaMallocHost(weight staging)");
    }
    ctx->h_upload_bytes = w->bytes;
  }
  void *h = ctx->h_upload;
  retile(w->kind, static_cast<const uint8_t *>(blocks), src_bpr, row0, row1, blk0, blk1, static_cast<uint8_t *>(h));
  e = cudaSetDevice(ctx->device);
  if (e == cudaSuccess) e = cudaMalloc(&w->d_tiles, w->bytes);
  if (e == cudaSuccess) e = cudaMemcpyAsync(w->d_tiles, h, w->bytes, cudaMemcpyHostToDevice, ctx->stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
  if (e != cudaSuccess) {
    if (w->d_tiles) cudaFree(w->d_tiles);
    delete w;
    return cuda_fail(e, "lmb_weight_upload");
  }
  *out = w;
  return LMB_OK;
}

int lmb_weight_upload(lmb_ctx *ctx, int kind, const void *blocks, size_t M, size_t K, lmb_weight **out) {
  return lmb_weight_upload_shard(ctx, kind, blocks, M, K, 0, M, 0, (K + BLK - 1) / BLK, out);
}

int lmb_weight_free(lmb_weight *w) {
  if (!w) return LMB_OK;
  cudaSetDevice(w->device);
  if (w->d_tiles) LMB_CUDA(cudaFree(w->d_tiles));
  delete w;
  return LMB_OK;
}

int lmb_weight_info(const lmb_weight *w, int *kind, size_t *M, size_t *K, size_t *device_bytes) {
  LMB_REQUIRE(w, "lmb_weight_info: null weight");
  if (kind) *kind = w->ref_kind;
  if (M) *M = w->M;
  if (K) *K = w->K;
  if (device_bytes) *device_bytes = w->bytes;
  return LMB_OK;
}

int lmb_weight_download(lmb_ctx *ctx, const lmb_weight *w, void *blocks_out) {
  LMB_REQUIRE(ctx && w && blocks_out, "lmb_weight_download: null argument");
  if (w->kind == LMB_RAW_F32) {
    LMB_CUDA(cudaMemcpyAsync(blocks_out, w->d_tiles, w->bytes, cudaMemcpyDeviceToHost, ctx->stream));
    LMB_CUDA(cudaStreamSynchronize(ctx->stream));
    return LMB_OK;
  }
  std::vector<uint8_t> h(w->bytes);
  LMB_CUDA(cudaMemcpyAsync(h.data(), w->d_tiles, w->bytes, cudaMemcpyDeviceToHost, ctx->stream));
  LMB_CUDA(cudaStreamSynchronize(ctx->stream));
  untile(w->kind, h.data(), w->M, w->bpr, static_cast<uint8_t *>(blocks_out));
  return LMB_OK;
}

// ---- layer / kernel / transform API -----------------------------------------------------------------
int lmb_linear(lmb_ctx *ctx, const lmb_weight *w, const float *d_bias, const float *d_x, size_t x_len,
               size_t x_stride, float *d_y, size_t batch, unsigned flags) {
  return linear_impl(ctx, w, d_bias, d_x, x_len, x_stride, d_y, batch, flags);
}

int lmb_linear_host(lmb_ctx *ctx, const lmb_weight *w, const float *bias, const float *input, float *output,
                    size_t batch, unsigned flags) {
  LMB_REQUIRE(ctx && w && input && output && batch > 0, "lmb_linear_host: null argument");
  const size_t K = w->K, M = w->M;
  const size_t in_f = batch * K, out_f = batch * M, bias_f = bias ? M : 0;
  int st = ensure_stage(ctx, (in_f + out_f + bias_f) * sizeof(float));
  if (st != LMB_OK) return st;
  float *h = static_cast<float *>(ctx->h_stage), *d = ctx->d_stage;
  std::memcpy(h, input, in_f * sizeof(float));
  if (bias) std::memcpy(h + in_f, bias, bias_f * sizeof(float));
  LMB_CUDA(cudaMemcpyAsync(d, h, (in_f + bias_f) * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
  float *d_y = d + in_f + bias_f;
  st = linear_impl(ctx, w, bias ? d + in_f : nullptr, d, K, K, d_y, batch, flags);
  if (st != LMB_OK) return st;
  float *h_y = h + in_f + bias_f;
  LMB_CUDA(cudaMemcpyAsync(h_y, d_y, out_f * sizeof(float), cudaMemcpyDeviceToHost, ctx->stream));
  LMB_CUDA(cudaStreamSynchronize(ctx->stream));
  std::memcpy(output, h_y, out_f * sizeof(float));
  return LMB_OK;
}

int lmb_linear_host_multi(lmb_ctx *ctx, size_t n, const lmb_weight *const *ws, const float *const *inputs,
                          float *const *outputs, unsigned flags) {
  LMB_REQUIRE(ctx && ws && inputs && outputs && n > 0, "lmb_linear_host_multi: null argument");
  size_t in_f = 0, out_f = 0;
  for (size_t i = 0; i < n; ++i) {
    LMB_REQUIRE(ws[i] && inputs[i] && outputs[i], "lmb_linear_host_multi: null entry");
    in_f += (ws[i]->K + 3) / 4 * 4;  // keep every input 16-byte aligned
    out_f += ws[i]->M;
  }
  int st = ensure_stage(ctx, (in_f + out_f) * sizeof(float));
  if (st != LMB_OK) return st;
  float *h = static_cast<float *>(ctx->h_stage), *d = ctx->d_stage;
  size_t off = 0;
  for (size_t i = 0; i < n; ++i) {
    std::memcpy(h + off, inputs[i], ws[i]->K * sizeof(float));
    off += (ws[i]->K + 3) / 4 * 4;
  }
  LMB_CUDA(cudaMemcpyAsync(d, h, in_f * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
  size_t xo = 0, yo = in_f;
  for (size_t i = 0; i < n; ++i) {
    st = linear_impl(ctx, ws[i], nullptr, d + xo, ws[i]->K, ws[i]->K, d + yo, 1, flags);
    if (st != LMB_OK) return st;
    xo += (ws[i]->K + 3) / 4 * 4;
    yo += ws[i]->M;
  }
  LMB_CUDA(cudaMemcpyAsync(h + in_f, d + in_f, out_f * sizeof(float), cudaMemcpyDeviceToHost, ctx->stream));
  LMB_CUDA(cudaStreamSynchronize(ctx->stream));
  yo = in_f;
  for (size_t i = 0; i < n; ++i) {
    std::memcpy(outputs[i], h + yo, ws[i]->M * sizeof(float));
    yo += ws[i]->M;
  }
  return LMB_OK;
}

int lmb_gemv_host(int kind, const void *blocks, size_t num_blocks, const float *activations, float *output, size_t M,
                  size_t K) {
  (void)num_blocks;  // ignored by every reference kernel (lut_gemm_scalar.cpp:15-16)
  LMB_REQUIRE(blocks && activations && output, "lmb_gemv_host: null argument");
  lmb_ctx *ctx = nullptr;
  int st = default_ctx(&ctx);
  if (st != LMB_OK) return st;
  lmb_weight *w = nullptr;
  st = lmb_weight_upload(ctx, kind, blocks, M, K, &w);
  if (st != LMB_OK) return st;
  // The reference kernels read whole 256-blocks of the activation vector, and so does this call.
  // What lies beyond column K normally meets the zero weights the quantizers pad a row's last
  // block with, and the reference's own tests pass arrays of exactly K floats
  // (tests/test_lut_gemm.cpp:108-118,150-158), i.e. whatever the heap holds behind them.  In the
  // reference such values are multiplied by zero; here they would also enter the block's shared
  // fixed-point exponent.  So a padding value that is not finite, or more than 4096 times larger than
  // every activation of the block's valid part, is taken as zero (a genuine activation vector never
  // looks like that; at most 12 of the 31 fixed-point bits are given up to the padding).
  const size_t kp = w->bpr * BLK;
  st = ensure_stage(ctx, (kp + M) * sizeof(float));
  if (st == LMB_OK) {
    float *h = static_cast<float *>(ctx->h_stage), *d = ctx->d_stage;
    std::memcpy(h, activations, kp * sizeof(float));
    if (K < kp) {
      const size_t b0 = (w->bpr - 1) * BLK;
      float amax = 0.0f;
      for (size_t i = b0; i < K; ++i) amax = std::max(amax, std::fabs(h[i]));
      const float lim = 4096.0f * std::max(amax, 1e-30f);
      for (size_t i = K; i < kp; ++i)
        if (!(std::fabs(h[i]) <= lim)) h[i] = 0.0f;  // also catches NaN
    }
    cudaError_t e = cudaMemcpyAsync(d, h, kp * sizeof(float), cudaMemcpyHostToDevice, ctx->stream);
    if (e != cudaSuccess) st = cuda_fail(e, "lmb_gemv_host h2d");
    if (st == LMB_OK) st = linear_impl(ctx, w, nullptr, d, kp, kp, d + kp, 1, 0);
    if (st == LMB_OK) {
      e = cudaMemcpyAsync(h + kp, d + kp, M * sizeof(float), cudaMemcpyDeviceToHost, ctx->stream);
      if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
      if (e != cudaSuccess) st = cuda_fail(e, "lmb_gemv_host d2h");
      else std::memcpy(output, h + kp, M * sizeof(float));
    }
  }
  lmb_weight_free(w);
  return st;
}

int lmb_fwht256(lmb_ctx *ctx, float *d_x, size_t n) {
  LMB_REQUIRE(ctx && d_x, "lmb_fwht256: null argument");
  return launch_fwht256(ctx, d_x, n);
}

int lmb_apply_hadamard_rotation_host(float *data, size_t n) {
  LMB_REQUIRE(data, "lmb_apply_hadamard_rotation_host: null argument");
  lmb_ctx *ctx = nullptr;
  int st = default_ctx(&ctx);
  if (st != LMB_OK) return st;
  st = ensure_stage(ctx, n * sizeof(float));
  if (st != LMB_OK) return st;
  std::memcpy(ctx->h_stage, data, n * sizeof(float));
  LMB_CUDA(cudaMemcpyAsync(ctx->d_stage, ctx->h_stage, n * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
  st = launch_fwht256(ctx, ctx->d_stage, n);
  if (st != LMB_OK) return st;
  LMB_CUDA(cudaMemcpyAsync(ctx->h_stage, ctx->d_stage, n * sizeof(float), cudaMemcpyDeviceToHost, ctx->stream));
  LMB_CUDA(cudaStreamSynchronize(ctx->stream));
  std::memcpy(data, ctx->h_stage, n * sizeof(float));
  return LMB_OK;
}

// ---- debug views ------------------------------------------------------------------------------------------
int lmb_debug_luts(lmb_ctx *ctx, const float *d_x, size_t x_len, unsigned flags, float *d_luts_out) {
  LMB_REQUIRE(ctx && d_x && d_luts_out, "lmb_debug_luts: null argument");
  return launch_debug_luts(ctx, d_x, x_len, (flags & LMB_ROTATE) != 0, d_luts_out);
}

int lmb_debug_ternary_indices(lmb_ctx *ctx, const lmb_weight *w, uint8_t *h_out) {
  LMB_REQUIRE(ctx && w && h_out, "lmb_debug_ternary_indices: null argument");
  LMB_REQUIRE(w->kind == LMB_TERNARY,
              "lmb_debug_ternary_indices: only for ternary weights uploaded in the table-lookup layout (LMB_OPT_TERNARY_LUT)");
  // The kernel's LUT indices are the nibbles of the P / N planes held in the device tiles.
  std::vector<uint8_t> h(w->bytes);
  LMB_CUDA(cudaMemcpyAsync(h.data(), w->d_tiles, w->bytes, cudaMemcpyDeviceToHost, ctx->stream));
  LMB_CUDA(cudaStreamSynchronize(ctx->stream));
  const size_t tb = tile_bytes(LMB_TERNARY);
  for (size_t r = 0; r < w->M; ++r)
    for (size_t b = 0; b < w->bpr; ++b) {
      const uint8_t *tile = h.data() + ((r / TILE_ROWS) * w->bpr + b) * tb;
      const size_t l = r % TILE_ROWS;
      uint8_t *o = h_out + (r * w->bpr + b) * 128;
      for (size_t g = 0; g < 64; ++g) {
        const size_t byte = g / 2, c = byte / 8, j = byte % 8;
        const uint8_t p = tile[(c * TILE_ROWS + l) * 16 + j], n = tile[(c * TILE_ROWS + l) * 16 + 8 + j];
        o[2 * g] = (g % 2 == 0) ? (p >> 4) : (p & 15);
        o[2 * g + 1] = (g % 2 == 0) ? (n >> 4) : (n & 15);
      }
    }
  return LMB_OK;
}

}  // extern "C"
