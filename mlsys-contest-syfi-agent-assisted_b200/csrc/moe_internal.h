// Internal declarations shared by the translation units of the MoE library:
// problem constants, the device workspace layout and the per-stage launchers.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace syfi {

constexpr int kHidden = 7168;       // H
constexpr int kInter = 2048;        // I
constexpr int kBlock = 128;         // quantisation block
constexpr int kExpertsGlobal = 256;
constexpr int kGroups = 8;
constexpr int kGroupSize = 32;
constexpr int kTopKGroups = 4;
constexpr int kTopK = 8;
constexpr int kMaxLocalExperts = 32;
constexpr int kHBlocks = kHidden / kBlock;   // 56
constexpr int kIBlocks = kInter / kBlock;    // 16
constexpr int kRowPad = 16;                  // each expert's row range is padded to this
constexpr int kMaxTokenTile = 128;           // largest token tile (MMA N) any GEMM variant uses
constexpr int kMaxGrid = 256;                // upper bound of the GEMM kernels' persistent grid
constexpr float kLoRatio = 28.0f;            // scale(hi) / scale(lo) of the two-term e4m3 intermediate

// status codes written by kernels into Workspace::status[0]
enum : int {
  kStatusOk = 0,
  kStatusWaitTimeoutProducer = 101,
  kStatusWaitTimeoutMma = 102,
  kStatusWaitTimeoutEpilogue = 103,
  kStatusBadIndex = 104,
  kStatusPeerTimeout = 105,   // a flag another rank should have raised did not arrive in time
  kStatusDependencyTimeout = 106,   // GEMM2 waited in vain for GEMM1 to finish an expert
};

// Device-side control block (one int array); the GEMM kernels read the tile count from it.
//   meta[0] = number of token tiles, meta[1] = padded row total, meta[2] = routed (token, local expert) rows,
//   meta[3] = active local experts
constexpr int kMetaInts = 8;

// Per local expert: its rows [row_off, row_off + rows_pad) of the permuted row space
// (rows_pad is a multiple of 16) cut into `tiles` token tiles of the launch's tile size;
// tile_off is the number of token tiles of all earlier experts.  A GEMM work item is
// (expert, feature tile, token tile); items are numbered expert-major, then feature tile,
// then token tile, so the CTAs that run side by side share a weight tile through L2.
struct ExpertWork {
  int row_off;
  int rows_pad;
  int tile_off;
  int tiles;
};

struct Workspace {
  int device = -1;
  int max_tokens = 0;
  int row_cap = 0;        // capacity of the permuted row space
  // routing
  int* topk_idx = nullptr;        // [T, 8] global expert ids
  float* topk_w = nullptr;        // [T, 8]
  uint32_t* local_mask = nullptr; // [T] bit e set when local expert e was selected
  int* counts = nullptr;          // [32] rows per local expert
  int* ready = nullptr;           // [32] GEMM1 work items finished per local expert (counts + 32: zeroed together)
  int* counts_last = nullptr;     // [32] copy of counts kept after the call (counts itself is re-zeroed for the next)
  int* meta = nullptr;            // [kMetaInts]
  int* status = nullptr;          // [4]
  long long* trace = nullptr;     // [2][3][4096] GEMM1 / GEMM2 timeline of CTA 0 (only written by SYFI_TRACE builds)
  // permutation
  int* row_token = nullptr;       // [row_cap] token of each row, -1 for padding
  int* route_row = nullptr;       // [T, 8] row of each (token, k) route, -1 when the expert is not local
  ExpertWork* work = nullptr;     // [32]
  // operands
  uint8_t* a_perm = nullptr;      // [row_cap, 7168] e4m3 gathered activations
  float* a_scale = nullptr;       // [56, row_cap]
  uint8_t* c_hi = nullptr;        // [row_cap, 2048] e4m3 SwiGLU output, leading term
  uint8_t* c_lo = nullptr;        // [row_cap, 2048] e4m3 residual term (scale = c_scale / 28)
  float* c_scale = nullptr;       // [16, row_cap]
  float* o_rows = nullptr;        // [row_cap, 7168] f32 per-route expert outputs
  float** row_out = nullptr;      // [row_cap] expert parallelism: where GEMM2 stores each row (a peer's memory), null = nowhere
  int* ep_ticket = nullptr;       // last-CTA ticket of the expert-parallel exchange kernels (self-resetting)
  size_t bytes = 0;
};

struct GemmLaunch {
  CUtensorMap tm_w;    // weights, 2-D [E * rows_per_expert, K], box 128 x 128
  CUtensorMap tm_b0;   // token-side operand, box token_tile x 128 (GEMM1: a_perm; GEMM2: c_hi)
  CUtensorMap tm_b1;   // GEMM2: c_lo (unused by GEMM1)
  CUtensorMap tm_b0s;  // same tensors with a 16-row box: tiles of <= 16 rows pull half the bytes
  CUtensorMap tm_b1s;
  CUtensorMap tm_sc;   // GEMM2: c_scale as f32 [16, row_cap], box 16 x token_tile (one load per work item)
  const uint8_t* w_packed = nullptr;   // pre-packed weights (tm_w unused) or nullptr
  int token_tile;      // 32, 64 or 128: token rows per work item, must match the row-list kernel's
  long long wait_limit = 1ll << 32;   // SM clocks a device-side wait may take (about two seconds)
  int silent_producer = 0;            // test hook, see syfi_moe_debug_fault
  int rows_to_targets = 0;            // GEMM2 stores row r at Workspace::row_out[r] instead of o_rows
};

// Tensor maps of the CTA-pair GEMM kernels (grouped_gemm_pair.cu): token-side operands use 32-row boxes.
struct PairGemmLaunch {
  CUtensorMap tm_w;    // weights, 2-D [E * rows_per_expert, K], box 128 x 128
  CUtensorMap tm_b0;   // GEMM1: a_perm; GEMM2: c_hi; box 32 x 128
  CUtensorMap tm_b1;   // GEMM2: c_lo (unused by GEMM1)
  CUtensorMap tm_b0w;  // the same tensors with 128-row boxes (tiles of more than 64 rows: one load instead of four)
  CUtensorMap tm_b1w;
  long long wait_limit = 1ll << 32;   // SM clocks a device-side wait may take (about two seconds)
  int silent_producer = 0;            // test hook, see syfi_moe_debug_fault
  int rows_to_targets = 0;            // GEMM2 stores row r at Workspace::row_out[r] instead of o_rows
};

// Programmatic dependent launch: the kernel may be scheduled while its predecessor in the stream is
// still running (its CTAs take whatever SM resources are free and run their prologue); it must
// execute griddepcontrol.wait (pdl_wait() in ptx.cuh) before it touches anything the predecessor
// wrote.  Hides the launch latency and the prologue of every kernel after the first.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                    Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// launchers (each returns the cudaGetLastError() of its launches)
cudaError_t launch_router(const float* logits, const void* bias_bf16, int T, int e_local, int expert_offset,
                          float scaling, const Workspace& ws, bool counters_are_zero, cudaStream_t st);
cudaError_t launch_build_rows(int T, int e_local, int expert_offset, int token_tile, const Workspace& ws,
                              cudaStream_t st);
cudaError_t launch_gather(const uint8_t* hidden, const float* hidden_scale, int T, const Workspace& ws, int num_sms,
                          cudaStream_t st);
cudaError_t launch_gemm1(const GemmLaunch& g, const float* w13_scale, int e_local, const Workspace& ws, int num_sms,
                         cudaStream_t st);
cudaError_t launch_gemm2(const GemmLaunch& g, const float* w2_scale, int e_local, const Workspace& ws, int num_sms,
                         cudaStream_t st);
// CTA-pair variants for large batches (grouped_gemm_pair.cu); they recompute the token-tile table from
// ExpertWork::rows_pad, so the row-list kernel's tile size does not matter to them.
cudaError_t pair_gemm_set_attributes();
cudaError_t launch_pair_gemm1(const PairGemmLaunch& g, const float* w13_scale, int e_local, const Workspace& ws,
                              int num_sms, cudaStream_t st);
cudaError_t launch_pair_gemm2(const PairGemmLaunch& g, const float* w2_scale, int e_local, const Workspace& ws,
                              int num_sms, cudaStream_t st);
// Weight pre-packing (prepack.cu): [E, rows, K] row-major e4m3 -> per (expert, 128-row feature tile, 128-byte K
// block) one 16 KB tile holding the rows' 128 bytes with the 128-byte shared-memory swizzle already applied;
// GEMM1's up and gate tiles of the same features interleave per K block.
cudaError_t launch_prepack(const uint8_t* w13, const uint8_t* w2, int e_local, uint8_t* w13_packed,
                           uint8_t* w2_packed, int num_sms, cudaStream_t st);
cudaError_t launch_combine(int T, const Workspace& ws, void* out, int out_is_f32, cudaStream_t st);
cudaError_t gemm_set_attributes();

// expert-parallel exchange over peer memory (ep_exchange.cu)
}  // namespace syfi
struct syfi_moe_ep_desc;
namespace syfi {
size_t ep_region_bytes(int world, int64_t tokens_per_rank);
cudaError_t launch_ep_publish_gather(const syfi_moe_ep_desc& d, uint32_t seq, const void* logits, const void* hs,
                                     const void* hs_scale, void* g_logits, void* g_hs, void* g_scale, int* ticket,
                                     int* status, cudaStream_t st);
// token dispatch: where the router of this rank's own tokens must write (inside the step's in-buffer), and the
// publish + sparse pull that fills ws.topk_idx / topk_w / local_mask / route_row / counts for all W*T tokens
void ep_dispatch_route_targets(const syfi_moe_ep_desc& d, uint32_t seq, int** topk_idx, float** topk_w);
cudaError_t launch_ep_dispatch_publish(const syfi_moe_ep_desc& d, uint32_t seq, const void* hs, const void* hs_scale,
                                       const Workspace& ws, int num_sms, cudaStream_t st);
cudaError_t launch_ep_dispatch_pull(const syfi_moe_ep_desc& d, uint32_t seq, int e_local, int expert_offset,
                                    const Workspace& ws, void* g_hs, void* g_scale, int num_sms, cudaStream_t st);
// GEMM2 rows stored straight into the owners' memory: per-row target pointers (ws.row_out) before the GEMMs,
// flags and the owners' sum over route slots after them
cudaError_t launch_ep_row_targets(const syfi_moe_ep_desc& d, uint32_t seq, const Workspace& ws, cudaStream_t st);
cudaError_t launch_ep_raise(const syfi_moe_ep_desc& d, uint32_t seq, const Workspace& ws, cudaStream_t st);
cudaError_t launch_ep_final_rows(const syfi_moe_ep_desc& d, uint32_t seq, const Workspace& ws, void* out_bf16,
                                 cudaStream_t st);
cudaError_t launch_ep_push_final(const syfi_moe_ep_desc& d, uint32_t seq, const Workspace& ws, void* out_bf16,
                                 int* ticket, cudaStream_t st);

// Records `msg` as the calling thread's last error (what syfi_moe_last_error() returns) and returns `code`.
int set_last_error(int code, const char* msg);

}  // namespace syfi
