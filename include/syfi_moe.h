/*
 * C ABI of the B200-native fused FP8 block-scale DeepSeek-V3 MoE layer
 * (definition moe_fp8_block_scale_ds_routing_topk8_ng8_kg4_e32_h7168_i2048).
 *
 * This is the drop-in boundary for the reference's single exported function,
 *   TVM_FFI_DLL_EXPORT_TYPED_FUNC(run_moe, run_impl)      moe/solution/cuda/moe.cu:3260
 * whose typed signature is at moe/solution/cuda/moe.cu:2987-2998.  All pointers are
 * DEVICE pointers to contiguous row-major tensors on the context's device unless a
 * function says otherwise; nothing is owned by the library except its workspace.
 * Every function returns 0 on success and a non-zero code on failure;
 * syfi_moe_last_error() then returns a message for the calling thread.
 * There is no CPU path: without a CUDA device every call fails.
 */
#ifndef SYFI_MOE_H_
#define SYFI_MOE_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct syfi_moe_ctx syfi_moe_ctx;

enum {
  SYFI_MOE_OK = 0,
  SYFI_MOE_ERR_INVALID = 1,   /* bad argument (null pointer, shape, expert range, alignment) */
  SYFI_MOE_ERR_CUDA = 2,      /* a CUDA runtime / driver call failed */
  SYFI_MOE_ERR_DEVICE = 3     /* a kernel reported a failure through the status word (bounded wait expired, bad index) */
};

/* Fixed problem sizes of the definition (reference constants: moe/solution/cuda/moe.cu:40-53). */
#define SYFI_MOE_HIDDEN 7168
#define SYFI_MOE_INTER 2048
#define SYFI_MOE_EXPERTS_GLOBAL 256
#define SYFI_MOE_TOP_K 8
#define SYFI_MOE_MAX_LOCAL_EXPERTS 32

/* Creates the per-device context and its workspace, sized for max_tokens tokens per call
 * (it grows on demand).  Replaces the reference's file-static Workspace g_ws and its
 * ensure_singletons / ensure_per_token / ensure_schedule (moe.cu:2832-2926). */
int syfi_moe_create(int device, int64_t max_tokens, syfi_moe_ctx** out_ctx);

/* Sizes the workspace explicitly: for calls of up to max_tokens tokens that route up to max_rows (token, local
 * expert) pairs to this rank's experts (0 = the worst case, 8 * max_tokens).  Without it the workspace holds
 * 8 rows per token up to 2048 tokens and 3 rows per token beyond (a token sends about one of its 8 routes to 32
 * of 256 experts; the per-route f32 output rows are 28 KB each, so the worst case costs 2.5 GB at 8192 tokens
 * against 1 GB for three rows per token).  A call that routes more rows than the workspace holds writes nothing
 * out of bounds: syfi_moe_check reports status 104 and the output of that call is undefined.  Synchronises the
 * device.  The reference sizes for 8 T rows always (moe.cu:2896-2926) but bounds its small-batch grids by
 * min(8 T, 2 T + 4) rows (moe.cu:3069). */
int syfi_moe_reserve(syfi_moe_ctx* ctx, int64_t max_tokens, int64_t max_rows);

/* Frees the workspace (the reference never frees, moe.cu:2896-2926). */
int syfi_moe_destroy(syfi_moe_ctx* ctx);

/* The layer.  Replaces run_impl / run_moe (moe.cu:2987-3258, exported at :3260), same argument
 * order and meaning:
 *   routing_logits       f32  [T, 256]
 *   routing_bias         bf16 [256]
 *   hidden_states        e4m3 [T, 7168]
 *   hidden_states_scale  f32  [56, T]
 *   gemm1_weights        e4m3 [E_local, 4096, 7168]   gemm1_weights_scale f32 [E_local, 32, 56]
 *   gemm2_weights        e4m3 [E_local, 7168, 2048]   gemm2_weights_scale f32 [E_local, 56, 16]
 *   local_expert_offset  first global expert owned by this call; experts [offset, offset + E_local)
 *   routed_scaling_factor
 *   output               bf16 [T, 7168] (destination-passing, moe/config.toml:10)
 * Differences from the reference, all deliberate: E_local (1..32) is an argument so an
 * expert-parallel rank can own a slice; work is enqueued on `stream` (a cudaStream_t; the
 * reference uses stream 0, moe.cu:3005) and the call never synchronises with the host (the
 * reference blocks on a device->host copy for T >= 128, moe.cu:3127-3131); arguments are
 * validated.  T == 0 is a no-op, as in the reference (moe.cu:3001).
 * Calls on one context must not overlap on the GPU (they share the workspace). */
int syfi_moe_forward(syfi_moe_ctx* ctx, const void* routing_logits, const void* routing_bias,
                     const void* hidden_states, const void* hidden_states_scale, const void* gemm1_weights,
                     const void* gemm1_weights_scale, const void* gemm2_weights, const void* gemm2_weights_scale,
                     int64_t num_tokens, int32_t num_local_experts, int64_t local_expert_offset,
                     double routed_scaling_factor, void* output, void* stream);

/* One-off weight pre-packing, the layout neighbour of the GEMM loaders (the reference reads the weights
 * as given through raw pointers, moe.cu:3045-3053, with its GEMM1 tensor map over that layout,
 * moe.cu:2941-2978).  Rewrites gemm1_weights [E_local, 4096, 7168] and gemm2_weights [E_local, 7168, 2048]
 * (e4m3, row-major) into buffers of the same sizes in which the 128 x 128-byte tile a work item needs per
 * K block is 16 KB of consecutive memory, already in the swizzled shared-memory order, and the tiles of a
 * work item follow each other in consumption order:
 *   gemm1_packed: [expert][feature tile 0..15][K block 0..55][up tile, gate tile]
 *   gemm2_packed: [expert][feature tile 0..55][K block 0..15][tile]
 *   inside a tile: byte b of row r at  r * 128 + (((b >> 4) ^ (r & 7)) << 4) + (b & 15)
 * Enqueued on `stream`; in-place packing is rejected.  The scales are not touched. */
int syfi_moe_prepack_weights(syfi_moe_ctx* ctx, const void* gemm1_weights, const void* gemm2_weights,
                             int32_t num_local_experts, void* gemm1_packed, void* gemm2_packed, void* stream);

/* syfi_moe_forward on weights packed by syfi_moe_prepack_weights (same arguments otherwise, same
 * results bit for bit): the weight stream becomes sequential, which HBM and L2 serve faster. */
int syfi_moe_forward_prepacked(syfi_moe_ctx* ctx, const void* routing_logits, const void* routing_bias,
                               const void* hidden_states, const void* hidden_states_scale,
                               const void* gemm1_packed, const void* gemm1_weights_scale, const void* gemm2_packed,
                               const void* gemm2_weights_scale, int64_t num_tokens, int32_t num_local_experts,
                               int64_t local_expert_offset, double routed_scaling_factor, void* output,
                               void* stream);

/* Same, but writes the un-rounded f32 [T, 7168] partial sum of this rank's experts instead of
 * bf16 — what an expert-parallel rank feeds to the cross-rank reduction (the reference has no
 * multi-GPU path; its only hook is local_expert_offset, moe.cu:182-185, 250-256). */
int syfi_moe_forward_partial_f32(syfi_moe_ctx* ctx, const void* routing_logits, const void* routing_bias,
                                 const void* hidden_states, const void* hidden_states_scale,
                                 const void* gemm1_weights, const void* gemm1_weights_scale,
                                 const void* gemm2_weights, const void* gemm2_weights_scale, int64_t num_tokens,
                                 int32_t num_local_experts, int64_t local_expert_offset,
                                 double routed_scaling_factor, void* output_f32, void* stream);

/* Same as syfi_moe_forward but every tensor argument except the four weight tensors is a HOST
 * pointer: inputs travel to the device, the layer runs, the bf16 output travels back and the stream is
 * synchronised before returning.  Page-locked (pinned) buffers are used through their device mapping where
 * that saves a copy (the router reads logits and bias from them, the last kernel writes the output rows
 * into them) and make the remaining copies asynchronous; pageable buffers are staged.
 * The reference's harness does these copies outside the kernel (moe/scripts/debug_correctness.py:35-55). */
int syfi_moe_forward_host(syfi_moe_ctx* ctx, const void* routing_logits_host, const void* routing_bias_host,
                          const void* hidden_states_host, const void* hidden_states_scale_host,
                          const void* gemm1_weights, const void* gemm1_weights_scale, const void* gemm2_weights,
                          const void* gemm2_weights_scale, int64_t num_tokens, int32_t num_local_experts,
                          int64_t local_expert_offset, double routed_scaling_factor, void* output_host,
                          void* stream);

/* Router only (replaces route_kernel, moe.cu:62-188): writes topk_idx int32 [T, 8] (global expert
 * ids, best first) and topk_weights f32 [T, 8] to DEVICE buffers supplied by the caller. */
int syfi_moe_route(syfi_moe_ctx* ctx, const void* routing_logits, const void* routing_bias, int64_t num_tokens,
                   int32_t num_local_experts, int64_t local_expert_offset, double routed_scaling_factor,
                   int32_t* topk_idx, float* topk_weights, void* stream);

/* Expert parallelism over peer memory: one step of the serving layout (every rank brings its own
 * tokens_per_rank tokens and owns num_local_experts experts starting at local_expert_offset), with the
 * token all-gather and the reduce-scatter of the partial outputs done by this library's own kernels
 * through plain loads and stores on NVLink-mapped peer memory instead of NCCL (the reference has no
 * multi-GPU path at all; its only hook is local_expert_offset, moe.cu:182-185, 250-256).
 *   region[r]   rank r's symmetric region as mapped into THIS process (region[rank] is the local one);
 *               every rank allocates syfi_moe_ep_region_bytes(world_size, tokens_per_rank) bytes,
 *               zero-fills them and exchanges the mappings before the first step (the Python mirror
 *               uses torch's symmetric memory for that).
 *   step        1, 2, 3, ... — the same on every rank, increased by one per call; it tags the flags the
 *               ranks raise for each other and selects one of two buffer sets, so consecutive steps need
 *               no barrier.
 * Inputs are this rank's OWN token-side tensors (device pointers, shapes as in syfi_moe_forward with
 * T = tokens_per_rank) and its expert weights; output is bf16 [tokens_per_rank, 7168]: this rank's tokens
 * summed over all ranks' experts, rounded once.
 * Waits on other ranks are bounded: wait_limit_cycles SM clocks per wait (0 = the default, 2^35, about
 * 17 s: a serving process may stall for seconds in an allocation or a module load; tests use short
 * limits).  A rank whose wait runs out records status 105 and marks the step as failed for everybody:
 * it sends a failure mark instead of rows, and every output row that depends on a failed rank is
 * written as NaN, so a stalled peer can never turn into plausible numbers.  The status word is only read
 * by syfi_moe_check (which synchronises): poll it at some cadence, e.g. once per model step.
 * Call syfi_moe_ep_prepare on every rank and put a barrier of your own behind it before step 1, so that no
 * rank allocates (and stalls) inside its first step. */
#define SYFI_MOE_EP_MAX_RANKS 8
typedef struct syfi_moe_ep_desc {
  int32_t world_size;
  int32_t rank;
  int64_t tokens_per_rank;
  void* region[SYFI_MOE_EP_MAX_RANKS];
  int64_t wait_limit_cycles;
} syfi_moe_ep_desc;
int64_t syfi_moe_ep_region_bytes(int32_t world_size, int64_t tokens_per_rank);
/* Allocates everything the expert-parallel entry points below need for this descriptor (workspace for
 * world_size * tokens_per_rank tokens, the gathered-token buffers), so that the steps themselves do not
 * allocate.  No counterpart in the reference. */
int syfi_moe_ep_prepare(syfi_moe_ctx* ctx, const syfi_moe_ep_desc* ep);
int syfi_moe_ep_forward(syfi_moe_ctx* ctx, const syfi_moe_ep_desc* ep, int64_t step, const void* routing_logits,
                        const void* routing_bias, const void* hidden_states, const void* hidden_states_scale,
                        const void* gemm1_weights, const void* gemm1_weights_scale, const void* gemm2_weights,
                        const void* gemm2_weights_scale, int32_t num_local_experts, int64_t local_expert_offset,
                        double routed_scaling_factor, void* output, void* stream);
/* Token dispatch: same inputs, output, region and step rules as syfi_moe_ep_forward, and bit-identical
 * results, but the tokens are not all-gathered.  Each rank routes only its OWN tokens and publishes their
 * eight (expert, weight) pairs, hidden rows and scales; each rank then pulls from every rank only the rows
 * that selected one of its experts (with DeepSeek's group-limited routing a token reaches at most four of
 * the eight expert groups, so at most half of the rows travel to a rank that owns one group), derives the
 * masks and row counts of its experts from the received routes, and runs the layer from the row lists on.
 * Against the all-gather layout: the router runs on tokens_per_rank instead of world_size * tokens_per_rank
 * tokens, no logits cross the link, and only routed rows do.  The return leg (GEMM2 storing each expert row
 * into the memory of the token's owner, see below) is the same.  The two layouts may share a region as long as every
 * rank makes the same sequence of calls.  No counterpart in the reference (moe.cu:182-185 is its only
 * multi-GPU hook). */
int syfi_moe_ep_forward_dispatch(syfi_moe_ctx* ctx, const syfi_moe_ep_desc* ep, int64_t step,
                                 const void* routing_logits, const void* routing_bias, const void* hidden_states,
                                 const void* hidden_states_scale, const void* gemm1_weights,
                                 const void* gemm1_weights_scale, const void* gemm2_weights,
                                 const void* gemm2_weights_scale, int32_t num_local_experts,
                                 int64_t local_expert_offset, double routed_scaling_factor, void* output,
                                 void* stream);
/* The same exchange for REPLICATED tokens (the large-prefill layout: every rank holds the same
 * world_size * tokens_per_rank tokens and owns a slice of the experts; the reference's
 * local_expert_offset hook, moe.cu:182-185, used as expert parallelism).  No inbound exchange: each rank runs
 * the layer for its experts on all tokens.
 * Return leg of all three expert-parallel entry points: the reduce-scatter is fused into GEMM2.  GEMM2's
 * epilogue stores every f32 expert row straight into the receive slot [token][k] of the rank that owns the
 * token (rank t / tokens_per_rank; k = the route's position among the token's eight) with plain stores over
 * NVLink, so the transfer overlaps the GEMM tile by tile and the rows never make a round trip through local
 * memory; after GEMM2 a flag goes up on every rank, and each owner computes sum_k weight[k] * row[k] over the
 * slots that arrived, in route order, and rounds once.  That is the order of the single-GPU combine, so the
 * result equals the single-GPU layer over the union of the ranks' experts bit for bit, however the experts
 * are spread.  (The environment variable SYFI_MOE_EP_RETURN=push, set alike on all ranks, selects the earlier
 * scheme for comparison: rows stay local, a kernel after GEMM2 sums each token's local routes and pushes one
 * partial row per token, the owners add the partials in rank order.)
 * Inputs: token-side tensors of ALL world_size * tokens_per_rank tokens (identical on every rank);
 * output: bf16 [tokens_per_rank, 7168], the rows of this rank's tokens.  Same step / region / wait rules as
 * syfi_moe_ep_forward; the entry points may share a region as long as every rank makes the same sequence of
 * calls. */
int syfi_moe_ep_forward_replicated(syfi_moe_ctx* ctx, const syfi_moe_ep_desc* ep, int64_t step,
                                   const void* routing_logits, const void* routing_bias, const void* hidden_states,
                                   const void* hidden_states_scale, const void* gemm1_weights,
                                   const void* gemm1_weights_scale, const void* gemm2_weights,
                                   const void* gemm2_weights_scale, int32_t num_local_experts,
                                   int64_t local_expert_offset, double routed_scaling_factor, void* output,
                                   void* stream);

/* Router for callers that cannot allocate device memory (no counterpart in the reference, which
 * allocates its workspace with cudaMalloc on first use, moe.cu:2863-2926).  Same result as
 * syfi_moe_route, but it needs no context and calls no cudaMalloc / cudaFree or any other allocating
 * routine: the scratch it needs sits in a fixed array inside the library image (about 145 KB of device
 * memory on every GPU that loads the library, held until the process exits), which limits a call to
 * SYFI_MOE_NOALLOC_MAX_TOKENS tokens; larger batches are rejected with SYFI_MOE_ERR_INVALID.
 * It works on the CURRENT device.  The first call on a device looks up the array's device address
 * (one cudaGetSymbolAddress) and keeps it for the life of the process: after cudaDeviceReset on that
 * device the kept address is stale, so a process that resets a device must not call this again for it.
 * Make that first call during start-up, outside any stream capture.  All calls on a
 * device share the array, so calls that overlap on the GPU (different streams, no dependency) race;
 * keep them on one stream or order them with events.  Outputs are caller-supplied DEVICE buffers:
 * topk_idx int32 [T, 8], topk_weights f32 [T, 8]. */
#define SYFI_MOE_NOALLOC_MAX_TOKENS 4096
int syfi_moe_route_noalloc(const void* routing_logits, const void* routing_bias, int64_t num_tokens,
                           int32_t num_local_experts, int64_t local_expert_offset, double routed_scaling_factor,
                           int32_t* topk_idx, float* topk_weights, void* stream);

/* Copies the routing result of the most recent forward on this context into HOST buffers
 * (either may be null): topk_idx int32 [T, 8], topk_weights f32 [T, 8].  Synchronises `stream`. */
int syfi_moe_last_routing(syfi_moe_ctx* ctx, int64_t num_tokens, int32_t* topk_idx_host, float* topk_weights_host,
                          void* stream);

/* Synchronises `stream`, then reads the device status word and the work counters of the most
 * recent forward: stats[0] = token tiles, [1] = padded rows, [2] = routed (token, local expert)
 * rows, [3] = active local experts (stats may be null).  Returns SYFI_MOE_ERR_DEVICE when a
 * kernel gave up on a bounded wait (the reference's mbarrier waits spin for ever, moe.cu:1298-1305);
 * the message names the status word: 101/102/103 = a GEMM kernel's producer/MMA/epilogue wait expired,
 * 104 = more routed rows than the workspace holds (syfi_moe_reserve), 105 = a peer rank's flag did not arrive, 106 = GEMM2 waited in vain for
 * GEMM1 to finish an expert. */
int syfi_moe_check(syfi_moe_ctx* ctx, int32_t* stats4, void* stream);

/* Test hook: copies a named workspace buffer of the most recent forward into HOST memory
 * ("row_token", "route_row", "expert_work", "meta", "counts", "a_perm", "a_scale", "c_hi", "c_lo",
 * "c_scale", "o_rows", "topk_idx", "topk_w").  *bytes receives the buffer's size; at most
 * max_bytes are copied (dst_host may be null to query the size); *row_cap receives the row
 * capacity, the leading dimension of the k-block-major scale arrays.  Synchronises the device.
 * The reference exposes no intermediates; its debug script only compares the final output
 * (moe/scripts/debug_correctness.py:58-91). */
int syfi_moe_debug_read(syfi_moe_ctx* ctx, const char* name, void* dst_host, int64_t max_bytes, int64_t* bytes,
                        int32_t* row_cap);

/* Test hook for the bounded device-side waits (the reference's waits spin for ever, moe.cu:1298-1305, so it
 * has nothing to test).  Applies to the NEXT forward on this context only, then clears itself:
 *   wait_limit_cycles  SM clocks any wait inside the GEMM kernels may take (0 = the normal limit, 2^32);
 *   mask               1 = GEMM1's TMA producer issues nothing (its MMA / epilogue waits run out: status
 *                      102 / 103), 2 = GEMM1 is not launched (GEMM2's wait for GEMM1's experts runs out:
 *                      106), 4 = GEMM2 is not launched, 8 = GEMM2's TMA producer issues nothing;
 *                      expert-parallel entry points only: 16 = the step stops after this rank has raised its
 *                      flags (no owners' sum), 32 = only the owners' sum of the step runs (the routing of the
 *                      previous call on this context is used) — with these a test walks several ranks through
 *                      a step on one GPU, rank after rank, with no kernel waiting for a later launch;
 *                      syfi_moe_ep_forward_dispatch only: 64 = the step stops after the rank has published its
 *                      tokens, 128 = the step starts behind the publication (at the pull).
 * Nothing faults, traps or spins without limit: the roles give up, the kernel frees its tensor memory and
 * returns, syfi_moe_check reports the status, and the context stays usable.  The output of such a call is
 * undefined. */
int syfi_moe_debug_fault(syfi_moe_ctx* ctx, int32_t mask, int64_t wait_limit_cycles);

/* Per-kernel timing.  When enabled, every forward brackets each of its six kernels (router,
 * row lists, gather, GEMM1, GEMM2, combine — in that order) with CUDA events on the stream it is
 * enqueued on; syfi_moe_last_stage_ms() synchronises on the last event and writes the six
 * durations in milliseconds.  Off by default.  (The reference has no timing hooks; its
 * profiling script wraps whole calls, moe/scripts/profile_single.py:50-56.) */
int syfi_moe_set_stage_timing(syfi_moe_ctx* ctx, int32_t enable);
int syfi_moe_last_stage_ms(syfi_moe_ctx* ctx, float* ms6);

/* Number of kernels the most recent forward enqueued (for launch accounting). */
int syfi_moe_last_launch_count(syfi_moe_ctx* ctx);

/* Bytes of device workspace currently held. */
int64_t syfi_moe_workspace_bytes(syfi_moe_ctx* ctx);

/* Message for the last failure on the calling thread ("" if none). */
const char* syfi_moe_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* SYFI_MOE_H_ */
