// Expert-parallel exchange over peer memory (NVLink), fused with the layer's own kernels.
//
// Return leg (default): GEMM2 stores each expert row into the token owner's memory; see "GEMM2 rows straight
// into the owners' memory" below (targets / raise / final).  The push / final pair described next is the earlier
// return leg, kept selectable for comparison.
//
// The reference has no multi-GPU path (its only hook is local_expert_offset,
// moe/solution/cuda/moe.cu:182-185, 250-256).  In the serving layout every rank brings its own T
// tokens and owns 32 experts; a step is
//     all-gather token-side tensors -> layer on W*T tokens (partial rows) -> reduce-scatter -> bf16.
// Instead of two NCCL collectives plus glue kernels, four small kernels work directly on a
// symmetric memory region every rank maps from every other rank (plain peer loads and stores, no
// multicast of any kind):
//   publish : copy this rank's logits / hidden states / scales into its region, then raise
//             in_flag[me] = seq on every rank
//   gather  : per source rank, wait for its flag, PULL its block into the local gathered tensors
//             (the scales land directly in the [56, W*T] layout the layer wants)
//   push    : the weighted combine of the layer, but the f32 row of a token goes straight into the
//             receive slot [me][token] of the rank that owns the token; tokens with no local route
//             send nothing (a one-word presence mark); then raise out_flag[me] = seq on every rank
//   final   : wait for all out flags, add the present slots in rank order, round to bf16 once
// Flags carry the caller's monotonically increasing step number, buffers are double buffered by its
// parity, so no barrier is needed between steps: a rank can only be one step ahead of a peer because
// its own next final depends on that peer's push.  Every flag wait is bounded (the descriptor carries the
// limit); on expiry the kernel records status 105, the rank sends failure marks instead of rows, and every
// output row that depends on a failed rank is written as NaN.
// With replicated tokens (every rank holds all W*T tokens, syfi_moe_ep_forward_replicated) only push and
// final run: the reduce-scatter is the combine kernel itself.
// Token dispatch (syfi_moe_ep_forward_dispatch) replaces publish + gather by
//   route   : the router runs on this rank's own T tokens and writes ids and weights into the in-buffer
//   publish : hidden rows and token-major scales beside them, then the same in_flag
//   pull    : per source rank, wait for its flag, read the routes of its tokens (64 bytes each), keep the
//             ones that name a local expert (mask, row counters), and pull only those tokens' rows
// so the layer starts at the row lists; push and final are shared with the other layouts.
#include <cuda_bf16.h>

#include "../../include/syfi_moe.h"
#include "moe_internal.h"
#include "ptx.cuh"

namespace syfi {

namespace {

constexpr int kMaxRanks = SYFI_MOE_EP_MAX_RANKS;
constexpr long long kDefaultFlagWaitCycles = 1ll << 35;   // about 17 s: a serving process may stall for seconds
constexpr uint32_t kHasRow = 1u, kHasNothing = 0u, kHasFailed = 2u;   // presence words of a (source rank, token) slot

struct EpView {
  uint8_t* base[kMaxRanks];   // every rank's region, as mapped into this process
  int world, rank, T;
  long long wait_cycles;
  size_t in_off[2], recv_off[2], has_off[2], flag_off;
};

__host__ __device__ inline size_t align256(size_t v) { return (v + 255) / 256 * 256; }

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// true once *flag >= seq (step numbers only grow); false after the cycle budget
__device__ __forceinline__ bool wait_flag(const uint32_t* flag, uint32_t seq, long long limit) {
  const long long t0 = clock64();
  while (static_cast<int>(ld_acquire_sys(flag) - seq) < 0) {
    if (clock64() - t0 > limit) return false;
    __nanosleep(100);
  }
  return true;
}

__device__ __forceinline__ uint32_t* in_flag(const EpView& v, int on_rank, int src) {
  return reinterpret_cast<uint32_t*>(v.base[on_rank] + v.flag_off) + src;
}
__device__ __forceinline__ uint32_t* out_flag(const EpView& v, int on_rank, int src) {
  return reinterpret_cast<uint32_t*>(v.base[on_rank] + v.flag_off) + kMaxRanks + src;
}

__device__ __forceinline__ uint32_t* fail_word(const EpView& v, int on_rank, int src) {
  return reinterpret_cast<uint32_t*>(v.base[on_rank] + v.flag_off) + 2 * kMaxRanks + src;
}

// ------------------------------------------------------------------------------ publish
__global__ void __launch_bounds__(256)
ep_publish_kernel(EpView v, uint32_t seq, const uint4* __restrict__ logits, const uint4* __restrict__ hs,
                  const uint4* __restrict__ scale, int* __restrict__ ticket) {
  const int T = v.T;
  uint4* dst = reinterpret_cast<uint4*>(v.base[v.rank] + v.in_off[seq & 1]);
  const size_t n_logits = static_cast<size_t>(T) * 64, n_hs = static_cast<size_t>(T) * 448, n_sc = static_cast<size_t>(T) * 14;
  const size_t total = n_logits + n_hs + n_sc;
  for (size_t i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    uint4 x;
    if (i < n_logits) x = __ldg(logits + i);
    else if (i < n_logits + n_hs) x = __ldg(hs + (i - n_logits));
    else x = __ldg(scale + (i - n_logits - n_hs));
    dst[i] = x;
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    if (atomicAdd(ticket, 1) == static_cast<int>(gridDim.x) - 1) {   // last CTA: everything is written
      *ticket = 0;
      __threadfence_system();
      for (int r = 0; r < v.world; ++r) st_release_sys(in_flag(v, r, v.rank), seq);
    }
  }
}

// ------------------------------------------------------------------------------- gather
// grid = (chunks, world): blockIdx.y is the source rank
__global__ void __launch_bounds__(256)
ep_gather_kernel(EpView v, uint32_t seq, uint4* __restrict__ g_logits, uint4* __restrict__ g_hs,
                 float* __restrict__ g_scale, int* __restrict__ status) {
  __shared__ int s_ok;
  const int src = blockIdx.y, T = v.T, W = v.world;
  if (threadIdx.x == 0) {
    s_ok = wait_flag(in_flag(v, v.rank, src), seq, v.wait_cycles) ? 1 : 0;
    if (!s_ok) atomicExch(status, kStatusPeerTimeout);
  }
  __syncthreads();
  if (!s_ok) return;
  const uint4* in = reinterpret_cast<const uint4*>(v.base[src] + v.in_off[seq & 1]);
  const size_t n_logits = static_cast<size_t>(T) * 64, n_hs = static_cast<size_t>(T) * 448;
  const size_t n_sc = static_cast<size_t>(T) * 56;   // floats
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n_logits; i += stride)
    g_logits[static_cast<size_t>(src) * n_logits + i] = in[i];
  for (size_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n_hs; i += stride)
    g_hs[static_cast<size_t>(src) * n_hs + i] = in[n_logits + i];
  const float* sc = reinterpret_cast<const float*>(in + n_logits + n_hs);   // [56][T] on the source
  for (size_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n_sc; i += stride) {
    const int kb = static_cast<int>(i / T), t = static_cast<int>(i % T);
    g_scale[static_cast<size_t>(kb) * (static_cast<size_t>(W) * T) + static_cast<size_t>(src) * T + t] = sc[i];
  }
}

// ------------------------------------------------------------------- token dispatch: publish
// Token dispatch: a rank routes its OWN tokens (the router writes the eight expert ids and weights of every
// token straight into this rank's in-buffer), publishes hidden rows and token-major scales beside them, and
// every rank then pulls only the rows that selected one of its experts.  In-buffer of a step:
//   topk_idx int32 [T, 8] | topk_w f32 [T, 8] | hidden e4m3 [T, 7168] | scales f32 [T, 56]
// (7456 bytes per token: fits the in-buffer of the all-gather layout, so both layouts share one region).
__host__ __device__ inline size_t disp_w_off(size_t T) { return T * 32; }
__host__ __device__ inline size_t disp_hs_off(size_t T) { return T * 64; }
__host__ __device__ inline size_t disp_sc_off(size_t T) { return T * 64 + T * kHidden; }

__global__ void __launch_bounds__(256)
ep_publish_tokens_kernel(EpView v, uint32_t seq, const uint4* __restrict__ hs, const float* __restrict__ scale,
                         int* __restrict__ ticket) {
  const size_t T = v.T;
  uint8_t* in = v.base[v.rank] + v.in_off[seq & 1];
  uint4* dst_hs = reinterpret_cast<uint4*>(in + disp_hs_off(T));
  float* dst_sc = reinterpret_cast<float*>(in + disp_sc_off(T));
  const size_t n_hs = T * (kHidden / 16), n_sc = T * kHBlocks;
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n_hs; i += stride) dst_hs[i] = __ldg(hs + i);
  // scales arrive [56, T]; a puller wants the 56 scales of a token side by side (one 224-byte read)
  for (size_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n_sc; i += stride) {
    const size_t kb = i / T, t = i % T;
    dst_sc[t * kHBlocks + kb] = __ldg(scale + i);
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    if (atomicAdd(ticket, 1) == static_cast<int>(gridDim.x) - 1) {   // last CTA: everything is written
      *ticket = 0;
      __threadfence_system();
      for (int r = 0; r < v.world; ++r) st_release_sys(in_flag(v, r, v.rank), seq);
    }
  }
}

// ---------------------------------------------------------------------- token dispatch: pull
// grid = (chunks, world): blockIdx.y is the source rank; a CTA takes 32 tokens of that rank at a time.
// Warp 0 reads the tokens' routes from the source, keeps a copy for the row-list and combine kernels,
// derives the mask of this rank's experts and counts rows per expert; then the eight warps pull the rows
// of the tokens whose mask is not empty (7168 + 224 bytes each) into the slot [source rank][token] of the
// gathered tensors.  Rows nobody here needs never cross the link.
constexpr int kPullTokens = 32;
constexpr int kPullThreads = 256;

__global__ void __launch_bounds__(kPullThreads)
ep_dispatch_pull_kernel(EpView v, uint32_t seq, int e_local, int expert_offset, int* __restrict__ topk_idx,
                        float* __restrict__ topk_w, uint32_t* __restrict__ local_mask, int* __restrict__ route_row,
                        int* __restrict__ counts, uint4* __restrict__ g_hs, float* __restrict__ g_scale,
                        int* __restrict__ status) {
  __shared__ int s_ok, s_n;
  __shared__ int s_list[kPullTokens];
  __shared__ int s_cnt[kMaxLocalExperts];
  const int src = blockIdx.y, T = v.T, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const size_t NT = static_cast<size_t>(v.world) * T;
  if (tid == 0) {
    s_ok = wait_flag(in_flag(v, v.rank, src), seq, v.wait_cycles) ? 1 : 0;
    if (!s_ok) atomicExch(status, kStatusPeerTimeout);
  }
  __syncthreads();
  const bool ok = s_ok != 0;
  const uint8_t* in = v.base[src] + v.in_off[seq & 1];
  const int4* r_idx = reinterpret_cast<const int4*>(in);
  const float4* r_w = reinterpret_cast<const float4*>(in + disp_w_off(T));
  const uint4* r_hs = reinterpret_cast<const uint4*>(in + disp_hs_off(T));
  const float4* r_sc = reinterpret_cast<const float4*>(in + disp_sc_off(T));
  const int chunks = (T + kPullTokens - 1) / kPullTokens;
  for (int c = blockIdx.x; c < chunks; c += gridDim.x) {
    if (tid < kMaxLocalExperts) s_cnt[tid] = 0;
    if (tid == 0) s_n = 0;
    __syncthreads();
    if (warp == 0) {
      const int t = c * kPullTokens + lane;
      uint32_t mask = 0;
      if (t < T) {
        const size_t g = static_cast<size_t>(src) * T + t;
        int4 i0 = make_int4(-1, -1, -1, -1), i1 = i0;
        float4 w0 = make_float4(0.f, 0.f, 0.f, 0.f), w1 = w0;
        if (ok) {   // a source that never published contributes no rows (and the step is marked failed)
          i0 = r_idx[2 * t]; i1 = r_idx[2 * t + 1];
          w0 = r_w[2 * t]; w1 = r_w[2 * t + 1];
        }
        reinterpret_cast<int4*>(topk_idx)[2 * g] = i0;
        reinterpret_cast<int4*>(topk_idx)[2 * g + 1] = i1;
        reinterpret_cast<float4*>(topk_w)[2 * g] = w0;
        reinterpret_cast<float4*>(topk_w)[2 * g + 1] = w1;
        const int4 none = make_int4(-1, -1, -1, -1);
        reinterpret_cast<int4*>(route_row)[2 * g] = none;
        reinterpret_cast<int4*>(route_row)[2 * g + 1] = none;
        const int ids[kTopK] = {i0.x, i0.y, i0.z, i0.w, i1.x, i1.y, i1.z, i1.w};
#pragma unroll
        for (int k = 0; k < kTopK; ++k) {
          const int le = ids[k] - expert_offset;
          if (ids[k] >= 0 && le >= 0 && le < e_local) { mask |= 1u << le; atomicAdd(&s_cnt[le], 1); }
        }
        local_mask[g] = mask;
      }
      const unsigned hit = __ballot_sync(0xffffffffu, mask != 0);
      if (mask != 0) s_list[__popc(hit & ((1u << lane) - 1u))] = t;
      if (lane == 0) s_n = __popc(hit);
    }
    __syncthreads();
    if (tid < e_local && s_cnt[tid] != 0) atomicAdd(&counts[tid], s_cnt[tid]);
    const int n = s_n;
    for (int j = warp; j < n; j += kPullThreads / 32) {
      const int t = s_list[j];
      const size_t g = static_cast<size_t>(src) * T + t;
      const uint4* rs = r_hs + static_cast<size_t>(t) * (kHidden / 16);
      uint4* rd = g_hs + g * (kHidden / 16);
      uint4 x[14];                       // 448 x 16 bytes per row: all of a lane's loads in flight together
#pragma unroll
      for (int i = 0; i < 14; ++i) x[i] = rs[i * 32 + lane];
      float4 sc = make_float4(0.f, 0.f, 0.f, 0.f);
      if (lane < kHBlocks / 4) sc = r_sc[static_cast<size_t>(t) * (kHBlocks / 4) + lane];
#pragma unroll
      for (int i = 0; i < 14; ++i) rd[i * 32 + lane] = x[i];
      if (lane < kHBlocks / 4) {         // the layer wants scales k-block-major: [56, W*T]
        g_scale[(4 * lane + 0) * NT + g] = sc.x;
        g_scale[(4 * lane + 1) * NT + g] = sc.y;
        g_scale[(4 * lane + 2) * NT + g] = sc.z;
        g_scale[(4 * lane + 3) * NT + g] = sc.w;
      }
    }
    __syncthreads();
  }
}

// --------------------------------------------------------------------------------- push
constexpr int kPushThreads = 256;
constexpr int kVec = kHidden / (kPushThreads * 4);   // 7 float4 per thread

__global__ void __launch_bounds__(kPushThreads)
ep_combine_push_kernel(EpView v, uint32_t seq, const int* __restrict__ route_row, const float* __restrict__ topk_w,
                       const float* __restrict__ o_rows, int row_cap, int* __restrict__ ticket,
                       const int* __restrict__ status) {
  const int t = blockIdx.x;                      // token index over all ranks' tokens, 0 .. W*T-1
  const int owner = t / v.T, tl = t % v.T;
  const int tid = threadIdx.x;
  // a step that already failed on this rank (a gather wait ran out: the layer worked on stale tokens; a GEMM
  // wait ran out) sends a failure mark instead of rows, so the owners write NaN rather than plausible numbers
  const bool failed = *reinterpret_cast<const volatile int*>(status) != 0;
  int rows[kTopK];
  float w[kTopK];
  bool any = false;
#pragma unroll
  for (int k = 0; k < kTopK; ++k) {
    rows[k] = route_row[t * kTopK + k];
    w[k] = topk_w[t * kTopK + k];
    if (rows[k] >= row_cap) rows[k] = -1;
    any = any || rows[k] >= 0;
  }
  uint32_t* has = reinterpret_cast<uint32_t*>(v.base[owner] + v.has_off[seq & 1]) + v.rank * v.T + tl;
  if (any && !failed) {
    float4 acc[kVec];
#pragma unroll
    for (int i = 0; i < kVec; ++i) acc[i] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 1
    for (int k = 0; k < kTopK; ++k) {
      if (rows[k] < 0) continue;
      const float4* src = reinterpret_cast<const float4*>(o_rows + static_cast<size_t>(rows[k]) * kHidden);
#pragma unroll
      for (int i = 0; i < kVec; ++i) {
        const float4 x = __ldg(src + i * kPushThreads + tid);
        acc[i].x = fmaf(w[k], x.x, acc[i].x);
        acc[i].y = fmaf(w[k], x.y, acc[i].y);
        acc[i].z = fmaf(w[k], x.z, acc[i].z);
        acc[i].w = fmaf(w[k], x.w, acc[i].w);
      }
    }
    float4* dst = reinterpret_cast<float4*>(v.base[owner] + v.recv_off[seq & 1]) +
                  (static_cast<size_t>(v.rank) * v.T + tl) * (kHidden / 4);
#pragma unroll
    for (int i = 0; i < kVec; ++i) dst[i * kPushThreads + tid] = acc[i];
  }
  if (tid == 0) *has = failed ? kHasFailed : (any ? kHasRow : kHasNothing);
  __threadfence_system();
  __syncthreads();
  if (tid == 0) {
    if (atomicAdd(ticket, 1) == static_cast<int>(gridDim.x) - 1) {
      *ticket = 0;
      __threadfence_system();
      for (int r = 0; r < v.world; ++r) st_release_sys(out_flag(v, r, v.rank), seq);
    }
  }
}

// -------------------------------------------------------------------------------- final
__global__ void __launch_bounds__(kPushThreads)
ep_final_kernel(EpView v, uint32_t seq, __nv_bfloat16* __restrict__ out, int* __restrict__ status) {
  __shared__ int s_ok;
  const int tl = blockIdx.x, tid = threadIdx.x;
  if (tid == 0) {
    int ok = 1;
    for (int q = 0; q < v.world && ok; ++q) ok = wait_flag(out_flag(v, v.rank, q), seq, v.wait_cycles) ? 1 : 0;
    if (!ok) atomicExch(status, kStatusPeerTimeout);
    s_ok = ok;
  }
  __syncthreads();
  const uint32_t* has = reinterpret_cast<const uint32_t*>(v.base[v.rank] + v.has_off[seq & 1]);
  const float4* recv = reinterpret_cast<const float4*>(v.base[v.rank] + v.recv_off[seq & 1]);
  bool poisoned = !s_ok;
  float4 acc[kVec];
#pragma unroll
  for (int i = 0; i < kVec; ++i) acc[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int q = 0; q < v.world && !poisoned; ++q) {
    const uint32_t h = __ldcg(has + q * v.T + tl);
    if (h == kHasFailed) { poisoned = true; break; }
    if (h == kHasNothing) continue;
    const float4* src = recv + (static_cast<size_t>(q) * v.T + tl) * (kHidden / 4);
#pragma unroll
    for (int i = 0; i < kVec; ++i) {
      const float4 x = __ldcg(src + i * kPushThreads + tid);
      acc[i].x += x.x; acc[i].y += x.y; acc[i].z += x.z; acc[i].w += x.w;
    }
  }
  if (poisoned) {   // a peer never answered, or told us its step failed: no number is better than a wrong one
    const float nan = __int_as_float(0x7fc00000);
#pragma unroll
    for (int i = 0; i < kVec; ++i) acc[i] = make_float4(nan, nan, nan, nan);
  }
  uint2* dst = reinterpret_cast<uint2*>(out + static_cast<size_t>(tl) * kHidden);
#pragma unroll
  for (int i = 0; i < kVec; ++i) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(acc[i].x, acc[i].y);
    const __nv_bfloat162 hi = __floats2bfloat162_rn(acc[i].z, acc[i].w);
    uint2 p;
    p.x = *reinterpret_cast<const uint32_t*>(&lo);
    p.y = *reinterpret_cast<const uint32_t*>(&hi);
    dst[i * kPushThreads + tid] = p;
  }
}

// ------------------------------------------------- GEMM2 rows straight into the owners' memory
// The exchange fused into GEMM2: instead of storing an expert's output rows locally, summing a token's local
// routes and pushing the partial row, GEMM2's epilogue stores every row where the token's OWNER will read it:
// slot [token][k] of the owner's receive area, k = the route's position among the token's eight.  The transfer
// then overlaps the GEMM tile by tile, the f32 rows never make a round trip through local memory, and the owner
// adds the rows that arrived in route order k = 0..7 — the order of the single-GPU combine, so the result does
// not depend on how the experts are spread over the ranks.
//   targets : one pointer per permuted row (null for padding rows) + a presence word = step number in the
//             owner's table for every routed (token, k)
//   raise   : after GEMM2 (an ordinary launch: all of GEMM2's stores have been performed), out_flag[me] = seq
//             on every rank, preceded by a failure word when this rank's step failed
//   final   : wait for all ranks, sum_k w[k] * slot[token][k] over the present slots, round once
__global__ void __launch_bounds__(256)
ep_row_targets_kernel(EpView v, uint32_t seq, int tokens_all, const int* __restrict__ route_row,
                      const int* __restrict__ row_token, const int* __restrict__ meta, int row_cap,
                      float** __restrict__ row_out) {
  pdl_wait();
  pdl_trigger();
  const int rows_total = meta[1];
  const int stride = gridDim.x * blockDim.x;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < tokens_all * kTopK; i += stride) {
    const int row = route_row[i];
    if (row < 0 || row >= row_cap) continue;
    const int t = i / kTopK, k = i % kTopK;
    const int owner = t / v.T, tl = t % v.T;
    const size_t slot = static_cast<size_t>(tl) * kTopK + k;
    row_out[row] = reinterpret_cast<float*>(v.base[owner] + v.recv_off[seq & 1]) + slot * kHidden;
    reinterpret_cast<uint32_t*>(v.base[owner] + v.has_off[seq & 1])[slot] = seq;
  }
  for (int r = blockIdx.x * blockDim.x + threadIdx.x; r < rows_total && r < row_cap; r += stride)
    if (row_token[r] < 0) row_out[r] = nullptr;
}

__global__ void __launch_bounds__(32)
ep_raise_kernel(EpView v, uint32_t seq, const int* __restrict__ status) {
  const bool failed = *reinterpret_cast<const volatile int*>(status) != 0;
  __threadfence_system();
  const int r = threadIdx.x;
  if (r < v.world) {
    if (failed) *fail_word(v, r, v.rank) = seq;   // same thread, same destination: ordered before the release below
    st_release_sys(out_flag(v, r, v.rank), seq);
  }
}

__global__ void __launch_bounds__(kPushThreads)
ep_final_rows_kernel(EpView v, uint32_t seq, const float* __restrict__ topk_w, __nv_bfloat16* __restrict__ out,
                     int* __restrict__ status) {
  __shared__ int s_state;     // 0 = fine, 1 = poisoned
  const int tl = blockIdx.x, tid = threadIdx.x;
  if (tid == 0) {
    int bad = 0;
    for (int q = 0; q < v.world && !bad; ++q) bad = wait_flag(out_flag(v, v.rank, q), seq, v.wait_cycles) ? 0 : 1;
    if (bad) atomicExch(status, kStatusPeerTimeout);
    for (int q = 0; q < v.world && !bad; ++q)
      if (*reinterpret_cast<const volatile uint32_t*>(fail_word(v, v.rank, q)) == seq) bad = 1;
    if (!bad && *reinterpret_cast<const volatile int*>(status) != 0) bad = 1;
    s_state = bad;
  }
  __syncthreads();
  const bool poisoned = s_state != 0;
  const uint32_t* has = reinterpret_cast<const uint32_t*>(v.base[v.rank] + v.has_off[seq & 1]) + static_cast<size_t>(tl) * kTopK;
  const float4* recv = reinterpret_cast<const float4*>(v.base[v.rank] + v.recv_off[seq & 1]) +
                       static_cast<size_t>(tl) * kTopK * (kHidden / 4);
  const float* w = topk_w + (static_cast<size_t>(v.rank) * v.T + tl) * kTopK;
  float4 acc[kVec];
#pragma unroll
  for (int i = 0; i < kVec; ++i) acc[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  if (!poisoned) {
#pragma unroll 1
    for (int k = 0; k < kTopK; ++k) {
      if (__ldcg(has + k) != seq) continue;
      const float wk = w[k];
      const float4* src = recv + static_cast<size_t>(k) * (kHidden / 4);
#pragma unroll
      for (int i = 0; i < kVec; ++i) {
        const float4 x = __ldcg(src + i * kPushThreads + tid);
        acc[i].x = fmaf(wk, x.x, acc[i].x);
        acc[i].y = fmaf(wk, x.y, acc[i].y);
        acc[i].z = fmaf(wk, x.z, acc[i].z);
        acc[i].w = fmaf(wk, x.w, acc[i].w);
      }
    }
  } else {   // a peer never answered, or a rank's step failed: no number is better than a wrong one
    const float nan = __int_as_float(0x7fc00000);
#pragma unroll
    for (int i = 0; i < kVec; ++i) acc[i] = make_float4(nan, nan, nan, nan);
  }
  uint2* dst = reinterpret_cast<uint2*>(out + static_cast<size_t>(tl) * kHidden);
#pragma unroll
  for (int i = 0; i < kVec; ++i) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(acc[i].x, acc[i].y);
    const __nv_bfloat162 hi = __floats2bfloat162_rn(acc[i].z, acc[i].w);
    uint2 pk;
    pk.x = *reinterpret_cast<const uint32_t*>(&lo);
    pk.y = *reinterpret_cast<const uint32_t*>(&hi);
    dst[i * kPushThreads + tid] = pk;
  }
}

EpView make_view(const syfi_moe_ep_desc& d) {
  EpView v;
  for (int r = 0; r < kMaxRanks; ++r) v.base[r] = r < d.world_size ? static_cast<uint8_t*>(d.region[r]) : nullptr;
  v.world = d.world_size;
  v.rank = d.rank;
  v.T = static_cast<int>(d.tokens_per_rank);
  v.wait_cycles = d.wait_limit_cycles > 0 ? d.wait_limit_cycles : kDefaultFlagWaitCycles;
  const size_t T = v.T, W = v.world;
  size_t off = 0;
  for (int b = 0; b < 2; ++b) { v.in_off[b] = off; off += align256(T * (kExpertsGlobal * 4 + kHidden + kHBlocks * 4)); }
  // receive area of a step: either one f32 partial row per (source rank, token) or one f32 expert row per
  // (token, route k); the second is the larger (world_size <= 8 = routes per token) and sizes both
  const size_t slots = (W > static_cast<size_t>(kTopK) ? W : static_cast<size_t>(kTopK)) * T;
  for (int b = 0; b < 2; ++b) { v.recv_off[b] = off; off += align256(slots * kHidden * 4); }
  for (int b = 0; b < 2; ++b) { v.has_off[b] = off; off += align256(slots * 4); }
  v.flag_off = off;
  return v;
}

}  // namespace

size_t ep_region_bytes(int world, int64_t tokens_per_rank) {
  syfi_moe_ep_desc d{};
  d.world_size = world;
  d.tokens_per_rank = tokens_per_rank;
  return make_view(d).flag_off + align256(3 * kMaxRanks * sizeof(uint32_t));   // in flags, out flags, failure words
}

cudaError_t launch_ep_publish_gather(const syfi_moe_ep_desc& d, uint32_t seq, const void* logits, const void* hs,
                                     const void* hs_scale, void* g_logits, void* g_hs, void* g_scale, int* ticket,
                                     int* status, cudaStream_t st) {
  const EpView v = make_view(d);
  // grids sized for large batches (tens of MB per rank); the grid-stride loops make small ones cheap
  ep_publish_kernel<<<256, 256, 0, st>>>(v, seq, static_cast<const uint4*>(logits), static_cast<const uint4*>(hs),
                                        static_cast<const uint4*>(hs_scale), ticket);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  ep_gather_kernel<<<dim3(1024 / d.world_size, d.world_size), 256, 0, st>>>(v, seq, static_cast<uint4*>(g_logits),
                                                           static_cast<uint4*>(g_hs), static_cast<float*>(g_scale),
                                                           status);
  return cudaGetLastError();
}

void ep_dispatch_route_targets(const syfi_moe_ep_desc& d, uint32_t seq, int** topk_idx, float** topk_w) {
  const EpView v = make_view(d);
  uint8_t* in = v.base[v.rank] + v.in_off[seq & 1];
  *topk_idx = reinterpret_cast<int*>(in);
  *topk_w = reinterpret_cast<float*>(in + disp_w_off(v.T));
}

cudaError_t launch_ep_dispatch_publish(const syfi_moe_ep_desc& d, uint32_t seq, const void* hs, const void* hs_scale,
                                       const Workspace& ws, int num_sms, cudaStream_t st) {
  const EpView v = make_view(d);
  const long long vecs = static_cast<long long>(v.T) * (kHidden / 16);
  int pub = static_cast<int>((vecs + 256 * 4 - 1) / (256 * 4));       // about four 16-byte vectors per thread
  if (pub > num_sms * 8) pub = num_sms * 8;
  if (pub < 1) pub = 1;
  ep_publish_tokens_kernel<<<pub, 256, 0, st>>>(v, seq, static_cast<const uint4*>(hs),
                                               static_cast<const float*>(hs_scale), ws.ep_ticket);
  return cudaGetLastError();
}

cudaError_t launch_ep_dispatch_pull(const syfi_moe_ep_desc& d, uint32_t seq, int e_local, int expert_offset,
                                    const Workspace& ws, void* g_hs, void* g_scale, int num_sms, cudaStream_t st) {
  const EpView v = make_view(d);
  const int chunks = (v.T + kPullTokens - 1) / kPullTokens;
  int per_src = (num_sms * 8 + d.world_size - 1) / d.world_size;   // about eight CTAs per SM over all sources
  if (per_src > chunks) per_src = chunks;
  if (per_src < 1) per_src = 1;
  ep_dispatch_pull_kernel<<<dim3(per_src, d.world_size), kPullThreads, 0, st>>>(
      v, seq, e_local, expert_offset, ws.topk_idx, ws.topk_w, ws.local_mask, ws.route_row, ws.counts,
      static_cast<uint4*>(g_hs), static_cast<float*>(g_scale), ws.status);
  return cudaGetLastError();
}

cudaError_t launch_ep_row_targets(const syfi_moe_ep_desc& d, uint32_t seq, const Workspace& ws, cudaStream_t st) {
  const EpView v = make_view(d);
  const int tokens = d.world_size * static_cast<int>(d.tokens_per_rank);
  int grid = (tokens * kTopK + 255) / 256;
  if (grid > 1184) grid = 1184;
  return launch_dependent(ep_row_targets_kernel, dim3(grid), dim3(256), 0, st, v, seq, tokens, ws.route_row,
                          ws.row_token, ws.meta, ws.row_cap, ws.row_out);
}

cudaError_t launch_ep_raise(const syfi_moe_ep_desc& d, uint32_t seq, const Workspace& ws, cudaStream_t st) {
  const EpView v = make_view(d);
  ep_raise_kernel<<<1, 32, 0, st>>>(v, seq, ws.status);
  return cudaGetLastError();
}

cudaError_t launch_ep_final_rows(const syfi_moe_ep_desc& d, uint32_t seq, const Workspace& ws, void* out_bf16,
                                 cudaStream_t st) {
  const EpView v = make_view(d);
  ep_final_rows_kernel<<<static_cast<int>(d.tokens_per_rank), kPushThreads, 0, st>>>(
      v, seq, ws.topk_w, static_cast<__nv_bfloat16*>(out_bf16), ws.status);
  return cudaGetLastError();
}

cudaError_t launch_ep_push_final(const syfi_moe_ep_desc& d, uint32_t seq, const Workspace& ws, void* out_bf16,
                                 int* ticket, cudaStream_t st) {
  const EpView v = make_view(d);
  const int tokens = d.world_size * static_cast<int>(d.tokens_per_rank);
  ep_combine_push_kernel<<<tokens, kPushThreads, 0, st>>>(v, seq, ws.route_row, ws.topk_w, ws.o_rows, ws.row_cap,
                                                         ticket, ws.status);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  ep_final_kernel<<<static_cast<int>(d.tokens_per_rank), kPushThreads, 0, st>>>(
      v, seq, static_cast<__nv_bfloat16*>(out_bf16), ws.status);
  return cudaGetLastError();
}

}  // namespace syfi
