// C ABI, workspace management, tensor maps and the launch sequence of the MoE layer.
//
// Host-side counterpart of the reference's run_impl and Workspace
// (moe/solution/cuda/moe.cu:2832-3258).  Unlike the reference there is no host
// synchronisation inside a call (its tile schedule is built on the host after a
// device->host copy, moe.cu:3127-3186): the tile table is built on the device and the
// persistent GEMM kernels read their work count from device memory.
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <new>
#include <string>

#include "../../include/syfi_moe.h"
#include "moe_internal.h"

using namespace syfi;

struct syfi_moe_ctx {
  Workspace ws;
  int num_sms = 0;
  int launches = 0;
  // staging buffers of syfi_moe_forward_host
  void* stage = nullptr;
  size_t stage_bytes = 0;
  // tensor maps of the last call: they only depend on the operand addresses, the expert count and
  // the token tile, which rarely change between calls (re-encoding costs a few microseconds of host time)
  GemmLaunch g1, g2;
  PairGemmLaunch p1, p2;             // tensor maps of the CTA-pair kernels (large batches)
  const void* map_w13 = nullptr;
  const void* map_w2 = nullptr;
  const void* map_ws = nullptr;      // workspace generation the maps were built for (a_perm pointer)
  int map_e_local = 0, map_token_tile = 0;
  bool map_packed = false;
  // true while the row counters of the workspace are known to be zero at the point of the next launch
  bool counters_clean = false;
  // second stream of syfi_moe_forward_host: the hidden states travel while the router runs
  cudaStream_t copy_stream = nullptr;
  cudaEvent_t ev_copy_begin = nullptr, ev_copy_done = nullptr;
  // third stream of syfi_moe_forward_host for large batches: finished output slices travel back while the next
  // slice is computed
  cudaStream_t out_stream = nullptr;
  cudaEvent_t ev_slice_done = nullptr, ev_out_done = nullptr;
  cudaEvent_t wait_before_gather = nullptr;   // set by forward_host for one call
  // host -> device copies forward_host wants on the second stream; run_layer issues them right after it has
  // launched the router, so that the GPU starts on the router while the host is still queueing the copies
  struct PendingCopy { void* dst; const void* src; size_t bytes; };
  PendingCopy pending[2] = {};
  int n_pending = 0;
  // gathered token-side tensors of the peer-memory expert-parallel path
  void* ep_gather = nullptr;
  size_t ep_gather_bytes = 0;
  // set by the expert-parallel entry points for one run_layer: GEMM2 stores its rows straight into the token
  // owners' receive slots of this region (step ep_rows_seq) instead of the local row buffer
  const syfi_moe_ep_desc* ep_rows = nullptr;
  uint32_t ep_rows_seq = 0;
  // one-shot test hook (syfi_moe_debug_fault): applies to the next forward, then clears itself
  int64_t reserved_rows = 0;          // syfi_moe_reserve: row capacity the caller asked for (0 = the default rule)
  int fault_mask = 0;
  long long fault_wait_limit = 0;
  // optional per-kernel timing
  bool timing = false;
  bool timing_valid = false;
  cudaEvent_t ev[7] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  std::mutex mu;
};

namespace {

thread_local std::string g_err;

int fail(int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  g_err = buf;
  return code;
}

#define CU_TRY(expr)                                                                                 \
  do {                                                                                               \
    cudaError_t _e = (expr);                                                                         \
    if (_e != cudaSuccess)                                                                           \
      return fail(SYFI_MOE_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__, __LINE__); \
  } while (0)

struct DeviceGuard {
  int prev = -1;
  bool ok = false;
  explicit DeviceGuard(int dev) {
    if (cudaGetDevice(&prev) == cudaSuccess && cudaSetDevice(dev) == cudaSuccess) ok = true;
  }
  ~DeviceGuard() {
    if (prev >= 0) cudaSetDevice(prev);
  }
};

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// 2-D byte tensor [rows, cols] (cols contiguous), box [box_rows, 128 bytes], 128-byte swizzle.
int make_map(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return fail(SYFI_MOE_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols};
  const cuuint32_t box[2] = {128, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(SYFI_MOE_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return SYFI_MOE_OK;
}

void free_workspace(Workspace& ws) {
  void* ptrs[] = {ws.topk_idx, ws.topk_w, ws.local_mask, ws.counts, ws.meta, ws.status, ws.trace, ws.row_token, ws.route_row,
                  ws.work, ws.a_perm, ws.a_scale, ws.c_hi, ws.c_lo, ws.c_scale, ws.o_rows, ws.ep_ticket, ws.row_out};
  for (void* p : ptrs)
    if (p) cudaFree(p);
  const int dev = ws.device;
  ws = Workspace();
  ws.device = dev;
}

template <typename T>
cudaError_t dev_alloc(T** p, size_t count, size_t* total) {
  const size_t bytes = (count * sizeof(T) + 255) / 256 * 256;
  *total += bytes;
  return cudaMalloc(reinterpret_cast<void**>(p), bytes);
}

// Rows of the permuted row space (one per (token, local expert) route, plus per-expert padding) the workspace is
// sized for.  A token can in theory send all 8 of its routes to the local experts (8 T rows), but with at most
// 32 of 256 experts local it sends about one; the f32 per-route output rows are 28 KB each, so sizing for the
// worst case costs 2.5 GB at 8192 tokens.  Up to 2048 tokens the worst case is kept (it is small); beyond,
// 3 rows per token unless the caller reserved more (syfi_moe_reserve).  A call that needs more rows than there
// are writes nothing out of bounds: the row-list kernel reports status 104 and the call's output is undefined.
int64_t default_rows(int64_t T) { return T <= 2048 ? 8 * T : (3 * T > 16384 ? 3 * T : 16384); }

int alloc_workspace(Workspace& ws, int64_t max_tokens, int64_t max_rows = 0) {
  if (max_tokens < 1) max_tokens = 1;
  free_workspace(ws);
  const int64_t T = max_tokens;
  int64_t rows = max_rows > 0 ? max_rows : default_rows(T);
  if (rows > 8 * T) rows = 8 * T;
  const int64_t row_cap = (rows + kRowPad * kMaxLocalExperts + 256 + kMaxTokenTile - 1) / kMaxTokenTile * kMaxTokenTile;
  if (row_cap * (int64_t)kHidden > (int64_t)1 << 40) return fail(SYFI_MOE_ERR_INVALID, "max_tokens too large");
  size_t total = 0;
  CU_TRY(dev_alloc(&ws.topk_idx, T * kTopK, &total));
  CU_TRY(dev_alloc(&ws.topk_w, T * kTopK, &total));
  CU_TRY(dev_alloc(&ws.local_mask, T, &total));
  CU_TRY(dev_alloc(&ws.counts, 3 * kMaxLocalExperts, &total));
  ws.ready = ws.counts + kMaxLocalExperts;
  ws.counts_last = ws.counts + 2 * kMaxLocalExperts;
  CU_TRY(cudaMemset(ws.counts, 0, 3 * kMaxLocalExperts * sizeof(int)));
  CU_TRY(dev_alloc(&ws.meta, kMetaInts, &total));
  CU_TRY(dev_alloc(&ws.status, 4, &total));
  CU_TRY(dev_alloc(&ws.trace, 8 * 4096, &total));
  CU_TRY(dev_alloc(&ws.row_token, row_cap, &total));
  CU_TRY(dev_alloc(&ws.route_row, T * kTopK, &total));
  CU_TRY(dev_alloc(&ws.work, kMaxLocalExperts, &total));
  CU_TRY(cudaMemset(ws.work, 0, kMaxLocalExperts * sizeof(ExpertWork)));
  CU_TRY(dev_alloc(&ws.a_perm, row_cap * kHidden, &total));
  CU_TRY(dev_alloc(&ws.a_scale, row_cap * kHBlocks, &total));
  CU_TRY(dev_alloc(&ws.c_hi, row_cap * kInter, &total));
  CU_TRY(dev_alloc(&ws.c_lo, row_cap * kInter, &total));
  CU_TRY(dev_alloc(&ws.c_scale, row_cap * kIBlocks, &total));
  CU_TRY(dev_alloc(&ws.o_rows, row_cap * kHidden, &total));
  CU_TRY(dev_alloc(&ws.ep_ticket, 4, &total));
  CU_TRY(dev_alloc(&ws.row_out, row_cap, &total));
  CU_TRY(cudaMemset(ws.row_out, 0, row_cap * sizeof(float*)));
  CU_TRY(cudaMemset(ws.ep_ticket, 0, 4 * sizeof(int)));
  CU_TRY(cudaMemset(ws.status, 0, 4 * sizeof(int)));
  CU_TRY(cudaMemset(ws.meta, 0, kMetaInts * sizeof(int)));
  ws.max_tokens = (int)T;
  ws.row_cap = (int)row_cap;
  ws.bytes = total;
  return SYFI_MOE_OK;
}

// Device-side alias of a page-locked host buffer, or nullptr for pageable memory.  Asked on every call
// (about a microsecond each): an address can change hands between a pinned and a pageable allocation.
const void* mapped_alias(const void* host) {
  cudaPointerAttributes attr;
  if (cudaPointerGetAttributes(&attr, host) == cudaSuccess) {
    if (attr.type == cudaMemoryTypeHost && attr.devicePointer != nullptr) return attr.devicePointer;
  } else {
    cudaGetLastError();   // unregistered memory is reported as an error by some drivers: not ours to keep
  }
  return nullptr;
}

constexpr int64_t kPairMinTokens = 6144;   // batches from this size on use the CTA-pair GEMM kernels (measured: even at 4096, 8 % faster at 8192, 17 % at 16384)
constexpr int kFlagOutF32 = 1;      // run_layer flags
constexpr int kFlagPrepacked = 2;
constexpr int kFlagRoutingGiven = 4;   // the workspace already holds routes, masks and row counters of all tokens (token dispatch)

// f32 matrix [rows, cols] (cols contiguous), box [rows, box_cols], no swizzle: the per-K-block scales of a
// token tile, fetched with one load.
int make_scale_map(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint32_t box_cols) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return fail(SYFI_MOE_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols * 4};
  const cuuint32_t box[2] = {box_cols, (cuuint32_t)rows};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(SYFI_MOE_ERR_CUDA, "cuTensorMapEncodeTiled (scales) failed with CUresult %d", (int)r);
  return SYFI_MOE_OK;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int validate(syfi_moe_ctx* ctx, const void* const* ptrs, int nptrs, int64_t T, int32_t e_local, int64_t offset,
             double scaling) {
  if (!ctx) return fail(SYFI_MOE_ERR_INVALID, "context is null");
  if (T < 0 || T > (1 << 24)) return fail(SYFI_MOE_ERR_INVALID, "num_tokens %lld out of range", (long long)T);
  if (e_local < 1 || e_local > kMaxLocalExperts)
    return fail(SYFI_MOE_ERR_INVALID, "num_local_experts %d must be in [1, %d]", e_local, kMaxLocalExperts);
  if (offset < 0 || offset + e_local > kExpertsGlobal)
    return fail(SYFI_MOE_ERR_INVALID, "local experts [%lld, %lld) outside [0, %d)", (long long)offset,
                (long long)(offset + e_local), kExpertsGlobal);
  if (!(scaling == scaling) || scaling > 3.0e38 || scaling < -3.0e38)
    return fail(SYFI_MOE_ERR_INVALID, "routed_scaling_factor is not a finite float");
  if (T == 0) return SYFI_MOE_OK;
  for (int i = 0; i < nptrs; ++i) {
    if (!ptrs[i]) return fail(SYFI_MOE_ERR_INVALID, "tensor argument %d is null", i);
    if (!aligned16(ptrs[i])) return fail(SYFI_MOE_ERR_INVALID, "tensor argument %d is not 16-byte aligned", i);
  }
  return SYFI_MOE_OK;
}

int ensure_capacity(syfi_moe_ctx* ctx, int64_t T) {
  if (T <= ctx->ws.max_tokens && (ctx->reserved_rows > 0 || ctx->ws.row_cap >= default_rows(T))) return SYFI_MOE_OK;
  // growing frees buffers that earlier calls may still be using
  CU_TRY(cudaDeviceSynchronize());
  ctx->map_w13 = nullptr;   // cached tensor maps point into the old workspace
  ctx->counters_clean = false;
  return alloc_workspace(ctx->ws, T > ctx->ws.max_tokens ? T : ctx->ws.max_tokens, ctx->reserved_rows);
}

int run_layer(syfi_moe_ctx* ctx, const void* logits, const void* bias, const void* hs, const void* hs_scale,
              const void* w13, const void* w13_scale, const void* w2, const void* w2_scale, int64_t T64,
              int32_t e_local, int64_t offset, double scaling, void* out, int flags, cudaStream_t st) {
  Workspace& ws = ctx->ws;
  const int out_is_f32 = flags & kFlagOutF32;
  const bool packed = (flags & kFlagPrepacked) != 0;   // w13 / w2 point at pre-packed weights
  const int T = (int)T64;
  GemmLaunch& g1 = ctx->g1;
  GemmLaunch& g2 = ctx->g2;
  int rc;
  // Token tile (MMA N) of this call's GEMMs, chosen from the batch size because the per-expert counts
  // only exist on the device: 32 rows while the layer is bound by streaming weights (measured faster up
  // to 1024 tokens: 8 accumulator slots in flight, two K blocks per barrier round), 64 rows beyond.
  // Large batches (experts with hundreds of rows each) run the CTA-pair kernels, which cut their own
  // token tiles (256 rows in GEMM1, 128 in GEMM2); token_tile 256 stands for that configuration here.
  int token_tile = (T64 <= 1024) ? 32 : (T64 < kPairMinTokens || packed) ? 64 : 256;
  if (const char* ov = getenv("SYFI_MOE_TOKEN_TILE")) {   // tuning knob: force 32, 64, 128 or (pair kernels) 256
    const int v = atoi(ov);
    if (v == 32 || v == 64 || v == 128 || (v == 256 && !packed)) token_tile = v;
  }
  const bool pair = token_tile == 256;
  const bool maps_valid = ctx->map_w13 == w13 && ctx->map_w2 == w2 && ctx->map_ws == ws.a_perm &&
                          ctx->map_e_local == e_local && ctx->map_token_tile == token_tile &&
                          ctx->map_packed == packed;
  if (!maps_valid) {
  ctx->map_w13 = nullptr;
  g1.token_tile = g2.token_tile = token_tile;
  g1.w_packed = packed ? static_cast<const uint8_t*>(w13) : nullptr;
  g2.w_packed = packed ? static_cast<const uint8_t*>(w2) : nullptr;
  if (packed) {   // the producer fetches packed tiles with untiled copies: no weight tensor map
    memset(&g1.tm_w, 0, sizeof(g1.tm_w));
    memset(&g2.tm_w, 0, sizeof(g2.tm_w));
  } else {
    if ((rc = make_map(&g1.tm_w, w13, (uint64_t)e_local * 2 * kInter, kHidden, 128))) return rc;
    if ((rc = make_map(&g2.tm_w, w2, (uint64_t)e_local * kHidden, kInter, 128))) return rc;
  }
  if (pair) {
    ctx->p1.tm_w = g1.tm_w;
    ctx->p2.tm_w = g2.tm_w;
    if ((rc = make_map(&ctx->p1.tm_b0, ws.a_perm, ws.row_cap, kHidden, 32))) return rc;
    ctx->p1.tm_b1 = ctx->p1.tm_b0;
    if ((rc = make_map(&ctx->p2.tm_b0, ws.c_hi, ws.row_cap, kInter, 32))) return rc;
    if ((rc = make_map(&ctx->p2.tm_b1, ws.c_lo, ws.row_cap, kInter, 32))) return rc;
    if ((rc = make_map(&ctx->p1.tm_b0w, ws.a_perm, ws.row_cap, kHidden, 128))) return rc;
    ctx->p1.tm_b1w = ctx->p1.tm_b0w;
    if ((rc = make_map(&ctx->p2.tm_b0w, ws.c_hi, ws.row_cap, kInter, 128))) return rc;
    if ((rc = make_map(&ctx->p2.tm_b1w, ws.c_lo, ws.row_cap, kInter, 128))) return rc;
  } else {
  if ((rc = make_map(&g1.tm_b0, ws.a_perm, ws.row_cap, kHidden, token_tile))) return rc;
  g1.tm_b1 = g1.tm_b0;
  if ((rc = make_map(&g1.tm_b0s, ws.a_perm, ws.row_cap, kHidden, 16))) return rc;
  g1.tm_b1s = g1.tm_b0s;
  if ((rc = make_map(&g2.tm_b0, ws.c_hi, ws.row_cap, kInter, token_tile))) return rc;
  if ((rc = make_map(&g2.tm_b1, ws.c_lo, ws.row_cap, kInter, token_tile))) return rc;
  if ((rc = make_map(&g2.tm_b0s, ws.c_hi, ws.row_cap, kInter, 16))) return rc;
  if ((rc = make_map(&g2.tm_b1s, ws.c_lo, ws.row_cap, kInter, 16))) return rc;
  if ((rc = make_scale_map(&g2.tm_sc, ws.c_scale, kIBlocks, ws.row_cap, token_tile))) return rc;
  g1.tm_sc = g2.tm_sc;
  }
  ctx->map_w13 = w13;
  ctx->map_w2 = w2;
  ctx->map_ws = ws.a_perm;
  ctx->map_e_local = e_local;
  ctx->map_token_tile = token_tile;
  ctx->map_packed = packed;
  }

  const int grid = ctx->num_sms < kMaxGrid ? ctx->num_sms : kMaxGrid;
  ctx->launches = 0;
  const bool timed = ctx->timing && ctx->ev[0] != nullptr;
  ctx->timing_valid = false;
#define STAGE_MARK(i) do { if (timed) CU_TRY(cudaEventRecord(ctx->ev[i], st)); } while (0)
  STAGE_MARK(0);
  // counters_clean: the previous chain on this workspace was enqueued completely, so its gather kernel
  // has left (or will have left, in stream order) the row counters at zero
  const bool clean = ctx->counters_clean;
  ctx->counters_clean = false;
  if (!(flags & kFlagRoutingGiven)) {
    CU_TRY(launch_router(static_cast<const float*>(logits), bias, T, e_local, (int)offset, (float)scaling, ws, clean, st));
    ctx->launches += 1;
  }
  STAGE_MARK(1);
  if (ctx->n_pending > 0) {         // forward_host: the hidden states travel while the router runs
    for (int i = 0; i < ctx->n_pending; ++i)
      CU_TRY(cudaMemcpyAsync(ctx->pending[i].dst, ctx->pending[i].src, ctx->pending[i].bytes, cudaMemcpyHostToDevice,
                             ctx->copy_stream));
    ctx->n_pending = 0;
    CU_TRY(cudaEventRecord(ctx->ev_copy_done, ctx->copy_stream));
    ctx->wait_before_gather = ctx->ev_copy_done;
  }
  CU_TRY(launch_build_rows(T, e_local, (int)offset, pair ? 128 : token_tile, ws, st));
  ctx->launches += 1;
  const syfi_moe_ep_desc* ep_rows = ctx->ep_rows;
  ctx->ep_rows = nullptr;
  g2.rows_to_targets = ctx->p2.rows_to_targets = ep_rows != nullptr ? 1 : 0;
  if (ep_rows != nullptr) {          // where GEMM2 will store every row: the token owners' memory
    CU_TRY(launch_ep_row_targets(*ep_rows, ctx->ep_rows_seq, ws, st));
    ctx->launches += 1;
  }
  STAGE_MARK(2);
  if (ctx->wait_before_gather) {    // hidden states still on their way from the host (forward_host)
    CU_TRY(cudaStreamWaitEvent(st, ctx->wait_before_gather, 0));
    ctx->wait_before_gather = nullptr;
  }
  CU_TRY(launch_gather(static_cast<const uint8_t*>(hs), static_cast<const float*>(hs_scale), T, ws, ctx->num_sms, st));
  ctx->launches += 1;
  STAGE_MARK(3);
  // test hook: short wait limit and roles / kernels left out for this one call (see syfi_moe_debug_fault)
  const int fault = ctx->fault_mask;
  const long long wl = ctx->fault_wait_limit > 0 ? ctx->fault_wait_limit : (1ll << 32);
  ctx->fault_mask = 0;
  ctx->fault_wait_limit = 0;
  g1.wait_limit = g2.wait_limit = ctx->p1.wait_limit = ctx->p2.wait_limit = wl;
  g1.silent_producer = ctx->p1.silent_producer = (fault & 1) ? 1 : 0;
  g2.silent_producer = ctx->p2.silent_producer = (fault & 8) ? 1 : 0;
  if (!(fault & 2)) {
    if (pair) CU_TRY(launch_pair_gemm1(ctx->p1, static_cast<const float*>(w13_scale), e_local, ws, grid, st));
    else CU_TRY(launch_gemm1(g1, static_cast<const float*>(w13_scale), e_local, ws, grid, st));
    ctx->launches += 1;
  }
  STAGE_MARK(4);
  if (!(fault & 4)) {
    if (pair) CU_TRY(launch_pair_gemm2(ctx->p2, static_cast<const float*>(w2_scale), e_local, ws, grid, st));
    else CU_TRY(launch_gemm2(g2, static_cast<const float*>(w2_scale), e_local, ws, grid, st));
    ctx->launches += 1;
  }
  STAGE_MARK(5);
  if (out != nullptr) {   // the expert-parallel path combines straight into the owners' memory instead
    CU_TRY(launch_combine(T, ws, out, out_is_f32, st));
    ctx->launches += 1;
  }
  STAGE_MARK(6);
#undef STAGE_MARK
  ctx->timing_valid = timed;
  ctx->counters_clean = true;
  return SYFI_MOE_OK;
}

int forward_common(syfi_moe_ctx* ctx, const void* logits, const void* bias, const void* hs, const void* hs_scale,
                   const void* w13, const void* w13_scale, const void* w2, const void* w2_scale, int64_t T,
                   int32_t e_local, int64_t offset, double scaling, void* out, int flags, void* stream) {
  const void* ptrs[] = {logits, bias, hs, hs_scale, w13, w13_scale, w2, w2_scale, out};
  int rc = validate(ctx, ptrs, 9, T, e_local, offset, scaling);
  if (rc) return rc;
  if (T == 0) return SYFI_MOE_OK;
  std::lock_guard<std::mutex> lock(ctx->mu);
  DeviceGuard guard(ctx->ws.device);
  if (!guard.ok) return fail(SYFI_MOE_ERR_CUDA, "cannot select device %d", ctx->ws.device);
  if ((rc = ensure_capacity(ctx, T))) return rc;
  return run_layer(ctx, logits, bias, hs, hs_scale, w13, w13_scale, w2, w2_scale, T, e_local, offset, scaling, out,
                   flags, static_cast<cudaStream_t>(stream));
}

}  // namespace

namespace syfi {
int set_last_error(int code, const char* msg) {
  g_err = msg ? msg : "";
  return code;
}
}  // namespace syfi

extern "C" {

const char* syfi_moe_last_error(void) { return g_err.c_str(); }

int syfi_moe_create(int device, int64_t max_tokens, syfi_moe_ctx** out_ctx) {
  if (!out_ctx) return fail(SYFI_MOE_ERR_INVALID, "out_ctx is null");
  *out_ctx = nullptr;
  if (max_tokens < 0 || max_tokens > (1 << 24)) return fail(SYFI_MOE_ERR_INVALID, "max_tokens out of range");
  int ndev = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0)
    return fail(SYFI_MOE_ERR_CUDA, "no CUDA device: this library has no CPU path");
  if (device < 0 || device >= ndev) return fail(SYFI_MOE_ERR_INVALID, "device %d out of range [0, %d)", device, ndev);
  DeviceGuard guard(device);
  if (!guard.ok) return fail(SYFI_MOE_ERR_CUDA, "cannot select device %d", device);
  cudaDeviceProp prop;
  CU_TRY(cudaGetDeviceProperties(&prop, device));
  if (prop.major != 10)
    return fail(SYFI_MOE_ERR_CUDA, "device %d is sm_%d%d; this library is built for sm_100a only", device, prop.major,
                prop.minor);
  CU_TRY(gemm_set_attributes());
  CU_TRY(pair_gemm_set_attributes());
  syfi_moe_ctx* ctx = new (std::nothrow) syfi_moe_ctx();
  if (!ctx) return fail(SYFI_MOE_ERR_INVALID, "out of host memory");
  ctx->ws.device = device;
  ctx->num_sms = prop.multiProcessorCount;
  int rc = alloc_workspace(ctx->ws, max_tokens);
  if (rc) {
    free_workspace(ctx->ws);
    delete ctx;
    return rc;
  }
  *out_ctx = ctx;
  return SYFI_MOE_OK;
}

int syfi_moe_reserve(syfi_moe_ctx* ctx, int64_t max_tokens, int64_t max_rows) {
  if (!ctx) return fail(SYFI_MOE_ERR_INVALID, "context is null");
  if (max_tokens < 1 || max_tokens > (1 << 24)) return fail(SYFI_MOE_ERR_INVALID, "max_tokens out of range");
  if (max_rows < 0 || max_rows > 8 * max_tokens) return fail(SYFI_MOE_ERR_INVALID, "max_rows must be in [0, 8 * max_tokens]");
  std::lock_guard<std::mutex> lock(ctx->mu);
  DeviceGuard guard(ctx->ws.device);
  if (!guard.ok) return fail(SYFI_MOE_ERR_CUDA, "cannot select device %d", ctx->ws.device);
  CU_TRY(cudaDeviceSynchronize());       // earlier calls may still be using the buffers that are replaced
  ctx->map_w13 = nullptr;
  ctx->counters_clean = false;
  ctx->reserved_rows = max_rows;
  return alloc_workspace(ctx->ws, max_tokens, max_rows);
}

int syfi_moe_destroy(syfi_moe_ctx* ctx) {
  if (!ctx) return SYFI_MOE_OK;
  {
    DeviceGuard guard(ctx->ws.device);
    cudaDeviceSynchronize();
    free_workspace(ctx->ws);
    if (ctx->stage) cudaFree(ctx->stage);
    if (ctx->ep_gather) cudaFree(ctx->ep_gather);
    if (ctx->out_stream) cudaStreamDestroy(ctx->out_stream);
    if (ctx->ev_slice_done) cudaEventDestroy(ctx->ev_slice_done);
    if (ctx->ev_out_done) cudaEventDestroy(ctx->ev_out_done);
    for (cudaEvent_t e : ctx->ev)
      if (e) cudaEventDestroy(e);
    if (ctx->ev_copy_begin) cudaEventDestroy(ctx->ev_copy_begin);
    if (ctx->ev_copy_done) cudaEventDestroy(ctx->ev_copy_done);
    if (ctx->copy_stream) cudaStreamDestroy(ctx->copy_stream);
  }
  delete ctx;
  return SYFI_MOE_OK;
}

int syfi_moe_forward(syfi_moe_ctx* ctx, const void* routing_logits, const void* routing_bias,
                     const void* hidden_states, const void* hidden_states_scale, const void* gemm1_weights,
                     const void* gemm1_weights_scale, const void* gemm2_weights, const void* gemm2_weights_scale,
                     int64_t num_tokens, int32_t num_local_experts, int64_t local_expert_offset,
                     double routed_scaling_factor, void* output, void* stream) {
  return forward_common(ctx, routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights,
                        gemm1_weights_scale, gemm2_weights, gemm2_weights_scale, num_tokens, num_local_experts,
                        local_expert_offset, routed_scaling_factor, output, 0, stream);
}

int syfi_moe_prepack_weights(syfi_moe_ctx* ctx, const void* gemm1_weights, const void* gemm2_weights,
                             int32_t num_local_experts, void* gemm1_packed, void* gemm2_packed, void* stream) {
  if (!ctx) return fail(SYFI_MOE_ERR_INVALID, "context is null");
  if (num_local_experts < 1 || num_local_experts > kMaxLocalExperts)
    return fail(SYFI_MOE_ERR_INVALID, "num_local_experts %d must be in [1, %d]", num_local_experts, kMaxLocalExperts);
  const void* ptrs[] = {gemm1_weights, gemm2_weights, gemm1_packed, gemm2_packed};
  for (int i = 0; i < 4; ++i) {
    if (!ptrs[i]) return fail(SYFI_MOE_ERR_INVALID, "tensor argument %d is null", i);
    if (!aligned16(ptrs[i])) return fail(SYFI_MOE_ERR_INVALID, "tensor argument %d is not 16-byte aligned", i);
  }
  if (gemm1_weights == gemm1_packed || gemm2_weights == gemm2_packed)
    return fail(SYFI_MOE_ERR_INVALID, "packing in place is not supported");
  DeviceGuard guard(ctx->ws.device);
  if (!guard.ok) return fail(SYFI_MOE_ERR_CUDA, "cannot select device %d", ctx->ws.device);
  CU_TRY(launch_prepack(static_cast<const uint8_t*>(gemm1_weights), static_cast<const uint8_t*>(gemm2_weights),
                        num_local_experts, static_cast<uint8_t*>(gemm1_packed), static_cast<uint8_t*>(gemm2_packed),
                        ctx->num_sms, static_cast<cudaStream_t>(stream)));
  return SYFI_MOE_OK;
}

int syfi_moe_forward_prepacked(syfi_moe_ctx* ctx, const void* routing_logits, const void* routing_bias,
                               const void* hidden_states, const void* hidden_states_scale,
                               const void* gemm1_packed, const void* gemm1_weights_scale, const void* gemm2_packed,
                               const void* gemm2_weights_scale, int64_t num_tokens, int32_t num_local_experts,
                               int64_t local_expert_offset, double routed_scaling_factor, void* output,
                               void* stream) {
  return forward_common(ctx, routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_packed,
                        gemm1_weights_scale, gemm2_packed, gemm2_weights_scale, num_tokens, num_local_experts,
                        local_expert_offset, routed_scaling_factor, output, kFlagPrepacked, stream);
}

int syfi_moe_forward_partial_f32(syfi_moe_ctx* ctx, const void* routing_logits, const void* routing_bias,
                                 const void* hidden_states, const void* hidden_states_scale,
                                 const void* gemm1_weights, const void* gemm1_weights_scale,
                                 const void* gemm2_weights, const void* gemm2_weights_scale, int64_t num_tokens,
                                 int32_t num_local_experts, int64_t local_expert_offset,
                                 double routed_scaling_factor, void* output_f32, void* stream) {
  return forward_common(ctx, routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights,
                        gemm1_weights_scale, gemm2_weights, gemm2_weights_scale, num_tokens, num_local_experts,
                        local_expert_offset, routed_scaling_factor, output_f32, 1, stream);
}

int syfi_moe_forward_host(syfi_moe_ctx* ctx, const void* routing_logits_host, const void* routing_bias_host,
                          const void* hidden_states_host, const void* hidden_states_scale_host,
                          const void* gemm1_weights, const void* gemm1_weights_scale, const void* gemm2_weights,
                          const void* gemm2_weights_scale, int64_t num_tokens, int32_t num_local_experts,
                          int64_t local_expert_offset, double routed_scaling_factor, void* output_host,
                          void* stream) {
  const int64_t T = num_tokens;
  {
    const void* hp[] = {routing_logits_host, routing_bias_host, hidden_states_host, hidden_states_scale_host,
                        output_host};
    if (!ctx) return fail(SYFI_MOE_ERR_INVALID, "context is null");
    if (T < 0 || T > (1 << 24)) return fail(SYFI_MOE_ERR_INVALID, "num_tokens %lld out of range", (long long)T);
    if (T == 0) return SYFI_MOE_OK;
    for (int i = 0; i < 5; ++i)
      if (!hp[i]) return fail(SYFI_MOE_ERR_INVALID, "host tensor argument %d is null", i);
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t b_logits = (size_t)T * kExpertsGlobal * 4, b_bias = kExpertsGlobal * 2;
  const size_t b_hs = (size_t)T * kHidden, b_hss = (size_t)T * kHBlocks * 4, b_out = (size_t)T * kHidden * 2;
  auto up = [](size_t v) { return (v + 255) / 256 * 256; };
  const size_t o_logits = 0, o_bias = o_logits + up(b_logits), o_hs = o_bias + up(b_bias), o_hss = o_hs + up(b_hs),
               o_out = o_hss + up(b_hss), need = o_out + up(b_out);
  {
    std::lock_guard<std::mutex> lock(ctx->mu);
    DeviceGuard guard(ctx->ws.device);
    if (!guard.ok) return fail(SYFI_MOE_ERR_CUDA, "cannot select device %d", ctx->ws.device);
    if (need > ctx->stage_bytes) {
      CU_TRY(cudaDeviceSynchronize());
      if (ctx->stage) cudaFree(ctx->stage);
      ctx->stage = nullptr;
      ctx->stage_bytes = 0;
      CU_TRY(cudaMalloc(&ctx->stage, need));
      ctx->stage_bytes = need;
    }
  }
  DeviceGuard guard(ctx->ws.device);
  char* base = static_cast<char*>(ctx->stage);
  if (!ctx->copy_stream) {
    CU_TRY(cudaStreamCreateWithFlags(&ctx->copy_stream, cudaStreamNonBlocking));
    CU_TRY(cudaEventCreateWithFlags(&ctx->ev_copy_begin, cudaEventDisableTiming));
    CU_TRY(cudaEventCreateWithFlags(&ctx->ev_copy_done, cudaEventDisableTiming));
  }
  // Large batches are cut into slices of kHostSlice tokens that move through a three-stage pipeline: slice
  // s + 1 travels to the device while slice s is computed and slice s - 1 travels back (PCIe carries both
  // directions at once).  Tokens are independent and a token's result does not depend on the batch it is
  // computed in, so the output is bit-identical to the unsliced call; each slice re-reads the active experts'
  // weights from HBM (about 0.2 ms per 1024-token slice), which is less than a slice's output needs on the
  // link (0.26 ms), so the call as a whole runs at the speed of the device-to-host copy.
  constexpr int64_t kHostSlice = 1024;
  if (T >= 2 * kHostSlice) {
    if (!ctx->out_stream) {
      CU_TRY(cudaStreamCreateWithFlags(&ctx->out_stream, cudaStreamNonBlocking));
      CU_TRY(cudaEventCreateWithFlags(&ctx->ev_slice_done, cudaEventDisableTiming));
      CU_TRY(cudaEventCreateWithFlags(&ctx->ev_out_done, cudaEventDisableTiming));
    }
    // both copy streams start after whatever the caller's stream did before
    CU_TRY(cudaEventRecord(ctx->ev_copy_begin, st));
    CU_TRY(cudaStreamWaitEvent(ctx->copy_stream, ctx->ev_copy_begin, 0));
    CU_TRY(cudaStreamWaitEvent(ctx->out_stream, ctx->ev_copy_begin, 0));
    CU_TRY(cudaMemcpyAsync(base + o_bias, routing_bias_host, b_bias, cudaMemcpyHostToDevice, ctx->copy_stream));
    int rc = SYFI_MOE_OK;
    for (int64_t t0 = 0; t0 < T && rc == SYFI_MOE_OK; t0 += kHostSlice) {
      const int64_t c = T - t0 < kHostSlice ? T - t0 : kHostSlice;
      char* d_logits = base + o_logits + (size_t)t0 * kExpertsGlobal * 4;
      char* d_hs = base + o_hs + (size_t)t0 * kHidden;
      char* d_hss = base + o_hss + (size_t)t0 * kHBlocks * 4;       // the slice's scales as a [56, c] block of its own
      char* d_out = base + o_out + (size_t)t0 * kHidden * 2;
      CU_TRY(cudaMemcpyAsync(d_logits, static_cast<const char*>(routing_logits_host) + (size_t)t0 * kExpertsGlobal * 4,
                             (size_t)c * kExpertsGlobal * 4, cudaMemcpyHostToDevice, ctx->copy_stream));
      CU_TRY(cudaMemcpyAsync(d_hs, static_cast<const char*>(hidden_states_host) + (size_t)t0 * kHidden,
                             (size_t)c * kHidden, cudaMemcpyHostToDevice, ctx->copy_stream));
      CU_TRY(cudaMemcpy2DAsync(d_hss, (size_t)c * 4, static_cast<const char*>(hidden_states_scale_host) + (size_t)t0 * 4,
                               (size_t)T * 4, (size_t)c * 4, kHBlocks, cudaMemcpyHostToDevice, ctx->copy_stream));
      CU_TRY(cudaEventRecord(ctx->ev_copy_done, ctx->copy_stream));
      CU_TRY(cudaStreamWaitEvent(st, ctx->ev_copy_done, 0));
      ctx->n_pending = 0;
      rc = forward_common(ctx, d_logits, base + o_bias, d_hs, d_hss, gemm1_weights, gemm1_weights_scale, gemm2_weights,
                          gemm2_weights_scale, c, num_local_experts, local_expert_offset, routed_scaling_factor, d_out,
                          0, stream);
      if (rc) break;
      CU_TRY(cudaEventRecord(ctx->ev_slice_done, st));
      CU_TRY(cudaStreamWaitEvent(ctx->out_stream, ctx->ev_slice_done, 0));
      CU_TRY(cudaMemcpyAsync(static_cast<char*>(output_host) + (size_t)t0 * kHidden * 2, d_out, (size_t)c * kHidden * 2,
                             cudaMemcpyDeviceToHost, ctx->out_stream));
    }
    // keep the caller's stream ordered behind both copy streams, whatever happened
    cudaEventRecord(ctx->ev_copy_done, ctx->copy_stream);
    cudaStreamWaitEvent(st, ctx->ev_copy_done, 0);
    cudaEventRecord(ctx->ev_out_done, ctx->out_stream);
    cudaStreamWaitEvent(st, ctx->ev_out_done, 0);
    if (rc) return rc;
    CU_TRY(cudaStreamSynchronize(st));
    return SYFI_MOE_OK;
  }
  // Pinned (page-locked) host buffers are mapped into the device's address space: the router then reads
  // its 64 KB of logits straight from them and the combine kernel writes the output rows straight into
  // them, which saves two copy operations (and their launch latency) on the critical stream.  Pageable
  // buffers go through the staging area.
  const void* logits_dev = mapped_alias(routing_logits_host);
  const void* bias_dev = mapped_alias(routing_bias_host);
  void* out_dev = const_cast<void*>(mapped_alias(output_host));
  const bool direct_in = logits_dev != nullptr && bias_dev != nullptr;
  // router inputs on the caller's stream; hidden states and their scales on a second stream, ordered
  // after whatever the caller's stream did before, and awaited just before the gather kernel
  CU_TRY(cudaEventRecord(ctx->ev_copy_begin, st));
  CU_TRY(cudaStreamWaitEvent(ctx->copy_stream, ctx->ev_copy_begin, 0));
  if (!direct_in) {
    CU_TRY(cudaMemcpyAsync(base + o_logits, routing_logits_host, b_logits, cudaMemcpyHostToDevice, st));
    CU_TRY(cudaMemcpyAsync(base + o_bias, routing_bias_host, b_bias, cudaMemcpyHostToDevice, st));
  }
  ctx->pending[0] = {base + o_hs, hidden_states_host, b_hs};
  ctx->pending[1] = {base + o_hss, hidden_states_scale_host, b_hss};
  ctx->n_pending = 2;
  int rc = forward_common(ctx, direct_in ? logits_dev : base + o_logits, direct_in ? bias_dev : base + o_bias,
                          base + o_hs, base + o_hss, gemm1_weights, gemm1_weights_scale, gemm2_weights,
                          gemm2_weights_scale, T, num_local_experts, local_expert_offset, routed_scaling_factor,
                          out_dev ? out_dev : base + o_out, 0, stream);
  if (rc) {
    if (ctx->n_pending == 0) cudaStreamWaitEvent(st, ctx->ev_copy_done, 0);   // copies were issued: keep the streams ordered
    ctx->n_pending = 0;
    ctx->wait_before_gather = nullptr;
    return rc;
  }
  if (!out_dev) CU_TRY(cudaMemcpyAsync(output_host, base + o_out, b_out, cudaMemcpyDeviceToHost, st));
  CU_TRY(cudaStreamSynchronize(st));
  return SYFI_MOE_OK;
}

int64_t syfi_moe_ep_region_bytes(int32_t world_size, int64_t tokens_per_rank) {
  if (world_size < 1 || world_size > SYFI_MOE_EP_MAX_RANKS || tokens_per_rank < 1 || tokens_per_rank > (1 << 20)) return 0;
  return (int64_t)ep_region_bytes(world_size, tokens_per_rank);
}

namespace {
// The return leg of the expert-parallel entry points.  Default: GEMM2 stores its rows straight into the token
// owners' memory and the owners sum them (launch_ep_row_targets / launch_ep_raise_final).  SYFI_MOE_EP_RETURN=push
// selects the earlier scheme for comparison: rows stay local, a combine kernel after GEMM2 sums each token's local
// routes and pushes the partial row, the owners add the partials in rank order.  All ranks must choose alike.
bool ep_rows_in_gemm2() {
  const char* v = getenv("SYFI_MOE_EP_RETURN");
  return !(v != nullptr && strcmp(v, "push") == 0);
}

int ep_layer_and_return(syfi_moe_ctx* ctx, const syfi_moe_ep_desc* ep, uint32_t seq, const void* logits,
                        const void* bias, const void* hs, const void* hs_scale, const void* w13,
                        const void* w13_scale, const void* w2, const void* w2_scale, int64_t tokens_all,
                        int32_t e_local, int64_t offset, double scaling, void* output, int flags, cudaStream_t st) {
  const bool fused = ep_rows_in_gemm2();
  // test hook (syfi_moe_debug_fault, bits 16 and 32): a step cut in two, so that a test can walk several ranks
  // through one step on ONE GPU, one after the other — all ranks up to their flags, then all owners' sums —
  // without any kernel waiting for a kernel launched later
  const int phase = fused ? (ctx->fault_mask & (16 | 32)) : 0;
  ctx->fault_mask &= ~(16 | 32);
  if (!(phase & 32)) {
    if (fused) { ctx->ep_rows = ep; ctx->ep_rows_seq = seq; }
    int rc = run_layer(ctx, logits, bias, hs, hs_scale, w13, w13_scale, w2, w2_scale, tokens_all, e_local, offset,
                       scaling, nullptr, flags, st);
    ctx->ep_rows = nullptr;
    if (rc) return rc;
    if (!fused) {
      CU_TRY(launch_ep_push_final(*ep, seq, ctx->ws, output, ctx->ws.ep_ticket, st));
      ctx->launches += 2;
      return SYFI_MOE_OK;
    }
    CU_TRY(launch_ep_raise(*ep, seq, ctx->ws, st));
    ctx->launches += 1;
  }
  if (!(phase & 16)) {
    CU_TRY(launch_ep_final_rows(*ep, seq, ctx->ws, output, st));
    ctx->launches += 1;
  }
  return SYFI_MOE_OK;
}

int validate_ep(const syfi_moe_ep_desc* ep, int64_t step) {
  if (!ep) return fail(SYFI_MOE_ERR_INVALID, "ep descriptor is null");
  const int W = ep->world_size;
  const int64_t T = ep->tokens_per_rank;
  if (W < 1 || W > SYFI_MOE_EP_MAX_RANKS) return fail(SYFI_MOE_ERR_INVALID, "world_size %d outside [1, %d]", W, SYFI_MOE_EP_MAX_RANKS);
  if (ep->rank < 0 || ep->rank >= W) return fail(SYFI_MOE_ERR_INVALID, "rank %d outside the world of %d", ep->rank, W);
  if (T < 1 || T * W > (1 << 24)) return fail(SYFI_MOE_ERR_INVALID, "tokens_per_rank %lld out of range", (long long)T);
  if (step < 1 || step > 0x7fffffff) return fail(SYFI_MOE_ERR_INVALID, "step must count up from 1");
  if (ep->wait_limit_cycles < 0) return fail(SYFI_MOE_ERR_INVALID, "wait_limit_cycles must not be negative");
  for (int r = 0; r < W; ++r)
    if (!ep->region[r] || !aligned16(ep->region[r])) return fail(SYFI_MOE_ERR_INVALID, "region[%d] is null or misaligned", r);
  return SYFI_MOE_OK;
}

// gathered token-side tensors of the sharded layout: logits [W*T, 256] f32 | hidden [W*T, 7168] e4m3 | scales [56, W*T] f32
int ensure_ep_gather(syfi_moe_ctx* ctx, size_t need) {
  if (need <= ctx->ep_gather_bytes) return SYFI_MOE_OK;
  CU_TRY(cudaDeviceSynchronize());
  if (ctx->ep_gather) cudaFree(ctx->ep_gather);
  ctx->ep_gather = nullptr;
  ctx->ep_gather_bytes = 0;
  CU_TRY(cudaMalloc(&ctx->ep_gather, need));
  ctx->ep_gather_bytes = need;
  return SYFI_MOE_OK;
}
size_t up256(size_t v) { return (v + 255) / 256 * 256; }
}  // namespace

int syfi_moe_ep_prepare(syfi_moe_ctx* ctx, const syfi_moe_ep_desc* ep) {
  if (!ctx) return fail(SYFI_MOE_ERR_INVALID, "context is null");
  int rc = validate_ep(ep, 1);
  if (rc) return rc;
  std::lock_guard<std::mutex> lock(ctx->mu);
  DeviceGuard guard(ctx->ws.device);
  if (!guard.ok) return fail(SYFI_MOE_ERR_CUDA, "cannot select device %d", ctx->ws.device);
  const size_t NT = (size_t)ep->tokens_per_rank * ep->world_size;
  if ((rc = ensure_capacity(ctx, (int64_t)NT))) return rc;
  const size_t need = up256(NT * kExpertsGlobal * 4) + up256(NT * kHidden) + up256(NT * kHBlocks * 4);
  return ensure_ep_gather(ctx, need);
}

int syfi_moe_ep_forward(syfi_moe_ctx* ctx, const syfi_moe_ep_desc* ep, int64_t step, const void* routing_logits,
                        const void* routing_bias, const void* hidden_states, const void* hidden_states_scale,
                        const void* gemm1_weights, const void* gemm1_weights_scale, const void* gemm2_weights,
                        const void* gemm2_weights_scale, int32_t num_local_experts, int64_t local_expert_offset,
                        double routed_scaling_factor, void* output, void* stream) {
  int rc = validate_ep(ep, step);
  if (rc) return rc;
  const int W = ep->world_size;
  const int64_t T = ep->tokens_per_rank;
  const void* ptrs[] = {routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights,
                        gemm1_weights_scale, gemm2_weights, gemm2_weights_scale, output};
  rc = validate(ctx, ptrs, 9, T * W, num_local_experts, local_expert_offset, routed_scaling_factor);
  if (rc) return rc;
  std::lock_guard<std::mutex> lock(ctx->mu);
  DeviceGuard guard(ctx->ws.device);
  if (!guard.ok) return fail(SYFI_MOE_ERR_CUDA, "cannot select device %d", ctx->ws.device);
  if ((rc = ensure_capacity(ctx, T * W))) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t NT = (size_t)T * W;
  const size_t o_hs = up256(NT * kExpertsGlobal * 4), o_sc = o_hs + up256(NT * kHidden), need = o_sc + up256(NT * kHBlocks * 4);
  if ((rc = ensure_ep_gather(ctx, need))) return rc;
  char* g = static_cast<char*>(ctx->ep_gather);
  const uint32_t seq = (uint32_t)step;
  CU_TRY(launch_ep_publish_gather(*ep, seq, routing_logits, hidden_states, hidden_states_scale, g, g + o_hs, g + o_sc,
                                  ctx->ws.ep_ticket, ctx->ws.status, st));
  rc = ep_layer_and_return(ctx, ep, seq, g, routing_bias, g + o_hs, g + o_sc, gemm1_weights, gemm1_weights_scale,
                           gemm2_weights, gemm2_weights_scale, (int64_t)NT, num_local_experts, local_expert_offset,
                           routed_scaling_factor, output, 0, st);
  if (rc) return rc;
  ctx->launches += 2;
  return SYFI_MOE_OK;
}

int syfi_moe_ep_forward_dispatch(syfi_moe_ctx* ctx, const syfi_moe_ep_desc* ep, int64_t step,
                                 const void* routing_logits, const void* routing_bias, const void* hidden_states,
                                 const void* hidden_states_scale, const void* gemm1_weights,
                                 const void* gemm1_weights_scale, const void* gemm2_weights,
                                 const void* gemm2_weights_scale, int32_t num_local_experts,
                                 int64_t local_expert_offset, double routed_scaling_factor, void* output,
                                 void* stream) {
  int rc = validate_ep(ep, step);
  if (rc) return rc;
  const int W = ep->world_size;
  const int64_t T = ep->tokens_per_rank;
  const void* ptrs[] = {routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights,
                        gemm1_weights_scale, gemm2_weights, gemm2_weights_scale, output};
  rc = validate(ctx, ptrs, 9, T * W, num_local_experts, local_expert_offset, routed_scaling_factor);
  if (rc) return rc;
  std::lock_guard<std::mutex> lock(ctx->mu);
  DeviceGuard guard(ctx->ws.device);
  if (!guard.ok) return fail(SYFI_MOE_ERR_CUDA, "cannot select device %d", ctx->ws.device);
  if ((rc = ensure_capacity(ctx, T * W))) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t NT = (size_t)T * W;
  const size_t o_hs = up256(NT * kExpertsGlobal * 4), o_sc = o_hs + up256(NT * kHidden), need = o_sc + up256(NT * kHBlocks * 4);
  if ((rc = ensure_ep_gather(ctx, need))) return rc;
  char* g = static_cast<char*>(ctx->ep_gather);
  const uint32_t seq = (uint32_t)step;
  // test hook (syfi_moe_debug_fault, bits 64 and 128): the step may stop after the publication or start behind
  // it, so that a test can walk several ranks through a step on one GPU
  const int dphase = ctx->fault_mask & (64 | 128);
  ctx->fault_mask &= ~(64 | 128);
  if (!(dphase & 128)) {
    // 1. route this rank's own tokens; ids and weights go straight into the step's in-buffer of the region
    //    (no expert counts as local here: masks and row counters are made by the pull, per destination)
    Workspace own = ctx->ws;
    ep_dispatch_route_targets(*ep, seq, &own.topk_idx, &own.topk_w);
    CU_TRY(launch_router(static_cast<const float*>(routing_logits), routing_bias, (int)T, 0, 0,
                         (float)routed_scaling_factor, own, true, st));
    // 2. publish rows and scales
    CU_TRY(launch_ep_dispatch_publish(*ep, seq, hidden_states, hidden_states_scale, ctx->ws, ctx->num_sms, st));
    ctx->launches = 2;
  }
  if (dphase & 64) return SYFI_MOE_OK;
  // 3. pull the rows routed to this rank's experts from every rank (the pull counts rows per expert)
  if (!(ctx->fault_mask & 32)) {   // (bit 32 of the test hook: only the owners' sum is wanted)
    if (!ctx->counters_clean) CU_TRY(cudaMemsetAsync(ctx->ws.counts, 0, sizeof(int) * 2 * kMaxLocalExperts, st));
    ctx->counters_clean = false;
    CU_TRY(launch_ep_dispatch_pull(*ep, seq, num_local_experts, (int)local_expert_offset, ctx->ws, g + o_hs, g + o_sc,
                                   ctx->num_sms, st));
  }
  // 4. the layer from the row lists on, rows back to the tokens' owners, summed there
  rc = ep_layer_and_return(ctx, ep, seq, nullptr, routing_bias, g + o_hs, g + o_sc, gemm1_weights,
                           gemm1_weights_scale, gemm2_weights, gemm2_weights_scale, (int64_t)NT, num_local_experts,
                           local_expert_offset, routed_scaling_factor, output, kFlagRoutingGiven, st);
  if (rc) return rc;
  ctx->launches += 3;   // router, publish, pull
  return SYFI_MOE_OK;
}

int syfi_moe_ep_forward_replicated(syfi_moe_ctx* ctx, const syfi_moe_ep_desc* ep, int64_t step,
                                   const void* routing_logits, const void* routing_bias, const void* hidden_states,
                                   const void* hidden_states_scale, const void* gemm1_weights,
                                   const void* gemm1_weights_scale, const void* gemm2_weights,
                                   const void* gemm2_weights_scale, int32_t num_local_experts,
                                   int64_t local_expert_offset, double routed_scaling_factor, void* output,
                                   void* stream) {
  int rc = validate_ep(ep, step);
  if (rc) return rc;
  const int64_t NT = ep->tokens_per_rank * ep->world_size;
  const void* ptrs[] = {routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights,
                        gemm1_weights_scale, gemm2_weights, gemm2_weights_scale, output};
  rc = validate(ctx, ptrs, 9, NT, num_local_experts, local_expert_offset, routed_scaling_factor);
  if (rc) return rc;
  std::lock_guard<std::mutex> lock(ctx->mu);
  DeviceGuard guard(ctx->ws.device);
  if (!guard.ok) return fail(SYFI_MOE_ERR_CUDA, "cannot select device %d", ctx->ws.device);
  if ((rc = ensure_capacity(ctx, NT))) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // every rank already holds all tokens: the layer for this rank's experts, then the combine that pushes each
  // token's partial row to the token's owner and the final sum of the owners
  return ep_layer_and_return(ctx, ep, (uint32_t)step, routing_logits, routing_bias, hidden_states,
                             hidden_states_scale, gemm1_weights, gemm1_weights_scale, gemm2_weights,
                             gemm2_weights_scale, NT, num_local_experts, local_expert_offset, routed_scaling_factor,
                             output, 0, st);
}

int syfi_moe_route(syfi_moe_ctx* ctx, const void* routing_logits, const void* routing_bias, int64_t num_tokens,
                   int32_t num_local_experts, int64_t local_expert_offset, double routed_scaling_factor,
                   int32_t* topk_idx, float* topk_weights, void* stream) {
  const void* ptrs[] = {routing_logits, routing_bias, topk_idx, topk_weights};
  int rc = validate(ctx, ptrs, 4, num_tokens, num_local_experts, local_expert_offset, routed_scaling_factor);
  if (rc) return rc;
  if (num_tokens == 0) return SYFI_MOE_OK;
  std::lock_guard<std::mutex> lock(ctx->mu);
  DeviceGuard guard(ctx->ws.device);
  if (!guard.ok) return fail(SYFI_MOE_ERR_CUDA, "cannot select device %d", ctx->ws.device);
  if ((rc = ensure_capacity(ctx, num_tokens))) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int T = (int)num_tokens;
  // the router alone leaves its histogram behind: zero it before and after, so that a captured graph
  // of the whole layer (which relies on finding zeros) stays valid
  ctx->counters_clean = false;
  CU_TRY(launch_router(static_cast<const float*>(routing_logits), routing_bias, T, num_local_experts,
                       (int)local_expert_offset, (float)routed_scaling_factor, ctx->ws, false, st));
  CU_TRY(cudaMemsetAsync(ctx->ws.counts, 0, sizeof(int) * kMaxLocalExperts, st));
  ctx->counters_clean = true;
  CU_TRY(cudaMemcpyAsync(topk_idx, ctx->ws.topk_idx, sizeof(int) * T * kTopK, cudaMemcpyDeviceToDevice, st));
  CU_TRY(cudaMemcpyAsync(topk_weights, ctx->ws.topk_w, sizeof(float) * T * kTopK, cudaMemcpyDeviceToDevice, st));
  ctx->launches = 1;
  return SYFI_MOE_OK;
}

int syfi_moe_last_routing(syfi_moe_ctx* ctx, int64_t num_tokens, int32_t* topk_idx_host, float* topk_weights_host,
                          void* stream) {
  if (!ctx) return fail(SYFI_MOE_ERR_INVALID, "context is null");
  if (num_tokens < 0 || num_tokens > ctx->ws.max_tokens)
    return fail(SYFI_MOE_ERR_INVALID, "num_tokens %lld exceeds the workspace (%d)", (long long)num_tokens,
                ctx->ws.max_tokens);
  DeviceGuard guard(ctx->ws.device);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (topk_idx_host)
    CU_TRY(cudaMemcpyAsync(topk_idx_host, ctx->ws.topk_idx, sizeof(int) * num_tokens * kTopK, cudaMemcpyDeviceToHost, st));
  if (topk_weights_host)
    CU_TRY(cudaMemcpyAsync(topk_weights_host, ctx->ws.topk_w, sizeof(float) * num_tokens * kTopK, cudaMemcpyDeviceToHost, st));
  CU_TRY(cudaStreamSynchronize(st));
  return SYFI_MOE_OK;
}

int syfi_moe_check(syfi_moe_ctx* ctx, int32_t* stats4, void* stream) {
  if (!ctx) return fail(SYFI_MOE_ERR_INVALID, "context is null");
  DeviceGuard guard(ctx->ws.device);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int status[4] = {0, 0, 0, 0};
  int meta[kMetaInts] = {0};
  CU_TRY(cudaMemcpyAsync(status, ctx->ws.status, sizeof(status), cudaMemcpyDeviceToHost, st));
  CU_TRY(cudaMemcpyAsync(meta, ctx->ws.meta, sizeof(meta), cudaMemcpyDeviceToHost, st));
  CU_TRY(cudaStreamSynchronize(st));
  if (stats4)
    for (int i = 0; i < 4; ++i) stats4[i] = meta[i];
  if (status[0] != kStatusOk) {
    cudaMemsetAsync(ctx->ws.status, 0, sizeof(status), st);
    cudaMemsetAsync(ctx->ws.counts, 0, kMaxLocalExperts * sizeof(int), st);
    return fail(SYFI_MOE_ERR_DEVICE, "a kernel reported status %d (101/102/103: bounded wait expired in the TMA / MMA / "
                "epilogue role of a grouped GEMM; 104: more routed rows than the workspace holds, reserve more with syfi_moe_reserve; 105: a peer rank's flag did not arrive; "
                "106: GEMM2 waited in vain for GEMM1 to finish an expert)", status[0]);
  }
  return SYFI_MOE_OK;
}

int syfi_moe_debug_read(syfi_moe_ctx* ctx, const char* name, void* dst_host, int64_t max_bytes, int64_t* bytes,
                        int32_t* row_cap) {
  if (!ctx || !name || !bytes) return fail(SYFI_MOE_ERR_INVALID, "null argument");
  DeviceGuard guard(ctx->ws.device);
  const Workspace& ws = ctx->ws;
  const int64_t T = ws.max_tokens, R = ws.row_cap;
  struct Entry { const char* name; void* ptr; int64_t bytes; };
  const Entry table[] = {
      {"row_token", ws.row_token, R * 4},        {"route_row", ws.route_row, T * kTopK * 4},
      {"expert_work", ws.work, (int64_t)kMaxLocalExperts * (int64_t)sizeof(ExpertWork)},
      {"meta", ws.meta, kMetaInts * 4},          {"counts", ws.counts_last, kMaxLocalExperts * 4},
      {"a_perm", ws.a_perm, R * kHidden},        {"a_scale", ws.a_scale, R * kHBlocks * 4},
      {"c_hi", ws.c_hi, R * kInter},             {"c_lo", ws.c_lo, R * kInter},
      {"c_scale", ws.c_scale, R * kIBlocks * 4}, {"o_rows", ws.o_rows, R * kHidden * 4},
      {"trace", ws.trace, 8 * 4096 * 8},
      {"topk_idx", ws.topk_idx, T * kTopK * 4},  {"topk_w", ws.topk_w, T * kTopK * 4},
  };
  for (const Entry& e : table) {
    if (strcmp(e.name, name) == 0) {
      *bytes = e.bytes;
      if (row_cap) *row_cap = ws.row_cap;
      if (dst_host && max_bytes > 0) {
        CU_TRY(cudaDeviceSynchronize());
        CU_TRY(cudaMemcpy(dst_host, e.ptr, (size_t)(e.bytes < max_bytes ? e.bytes : max_bytes), cudaMemcpyDeviceToHost));
      }
      return SYFI_MOE_OK;
    }
  }
  return fail(SYFI_MOE_ERR_INVALID, "unknown workspace buffer '%s'", name);
}

int syfi_moe_debug_fault(syfi_moe_ctx* ctx, int32_t mask, int64_t wait_limit_cycles) {
  if (!ctx) return fail(SYFI_MOE_ERR_INVALID, "context is null");
  if (mask < 0 || mask > 255 || (mask & 48) == 48 || (mask & 192) == 192)
    return fail(SYFI_MOE_ERR_INVALID, "mask must be a combination of 1, 2, 4, 8, one of 16 / 32 and one of 64 / 128");
  if (wait_limit_cycles < 0) return fail(SYFI_MOE_ERR_INVALID, "wait_limit_cycles must not be negative");
  std::lock_guard<std::mutex> lock(ctx->mu);
  ctx->fault_mask = mask;
  ctx->fault_wait_limit = wait_limit_cycles;
  return SYFI_MOE_OK;
}

int syfi_moe_set_stage_timing(syfi_moe_ctx* ctx, int32_t enable) {
  if (!ctx) return fail(SYFI_MOE_ERR_INVALID, "context is null");
  std::lock_guard<std::mutex> lock(ctx->mu);
  DeviceGuard guard(ctx->ws.device);
  if (enable && ctx->ev[0] == nullptr)
    for (cudaEvent_t& e : ctx->ev) CU_TRY(cudaEventCreate(&e));
  ctx->timing = enable != 0;
  ctx->timing_valid = false;
  return SYFI_MOE_OK;
}

int syfi_moe_last_stage_ms(syfi_moe_ctx* ctx, float* ms6) {
  if (!ctx || !ms6) return fail(SYFI_MOE_ERR_INVALID, "null argument");
  if (!ctx->timing_valid) return fail(SYFI_MOE_ERR_INVALID, "no timed forward has run (enable stage timing first)");
  DeviceGuard guard(ctx->ws.device);
  CU_TRY(cudaEventSynchronize(ctx->ev[6]));
  for (int i = 0; i < 6; ++i) CU_TRY(cudaEventElapsedTime(&ms6[i], ctx->ev[i], ctx->ev[i + 1]));
  return SYFI_MOE_OK;
}

int syfi_moe_last_launch_count(syfi_moe_ctx* ctx) { return ctx ? ctx->launches : 0; }

int64_t syfi_moe_workspace_bytes(syfi_moe_ctx* ctx) { return ctx ? (int64_t)ctx->ws.bytes : 0; }

}  // extern "C"
