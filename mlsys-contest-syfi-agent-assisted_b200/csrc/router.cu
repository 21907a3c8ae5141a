// DeepSeek-V3 no-aux router, one warp per token.
//
// Replaces the reference's route_kernel (moe/solution/cuda/moe.cu:62-188: one CTA of
// 256 threads per token, eight block-wide argmax rounds).  Here a warp owns a token:
// lane l holds experts [8l, 8l+8), so a routing group (32 experts) is four adjacent
// lanes and every reduction is a handful of shuffles.
//
// Numerics follow the definition's reference (flashinfer/trace/templates/moe.py:139-170):
// s = 1 / (1 + exp(-x)) with accurate expf and IEEE division (this file must not be
// compiled with fast-math), biased = s + bias, group score = sum of the two largest
// biased scores of the group, ties resolved towards the lower index, weights from the
// un-biased s, normalised with +1e-20 and multiplied by the scaling factor.
#include <cuda_bf16.h>
#include <math_constants.h>

#include <cstdio>
#include <mutex>

#include "../../include/syfi_moe.h"
#include "moe_internal.h"
#include "ptx.cuh"

namespace syfi {

namespace {

constexpr int kWarpsPerBlock = 4;

__global__ void __launch_bounds__(kWarpsPerBlock * 32)
route_kernel(const float* __restrict__ logits, const __nv_bfloat16* __restrict__ bias, int T, int e_local,
             int expert_offset, float scaling, int* __restrict__ topk_idx, float* __restrict__ topk_w,
             uint32_t* __restrict__ local_mask, int* __restrict__ route_row, int* __restrict__ counts) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  pdl_trigger();
  if (t >= T) return;
  const unsigned full = 0xffffffffu;

  float x[8];
  {
    const float4* lp = reinterpret_cast<const float4*>(logits + static_cast<size_t>(t) * kExpertsGlobal + lane * 8);
    const float4 a = __ldg(lp), b = __ldg(lp + 1);
    x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w;
    x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
  }
  float bf[8];
  {
    const uint4 bv = __ldg(reinterpret_cast<const uint4*>(bias + lane * 8));
    const uint32_t w[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      bf[2 * i] = __uint_as_float(w[i] << 16);
      bf[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  float s[8], v[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    s[i] = 1.0f / (1.0f + expf(-x[i]));
    v[i] = s[i] + bf[i];
  }

  // two largest biased scores of the group (4 lanes x 8 values)
  float m1 = -CUDART_INF_F, m2 = -CUDART_INF_F;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    if (v[i] > m1) { m2 = m1; m1 = v[i]; }
    else if (v[i] > m2) { m2 = v[i]; }
  }
#pragma unroll
  for (int d = 1; d <= 2; d <<= 1) {
    const float o1 = __shfl_xor_sync(full, m1, d);
    const float o2 = __shfl_xor_sync(full, m2, d);
    const float n1 = fmaxf(m1, o1);
    const float n2 = fmaxf(fminf(m1, o1), fmaxf(m2, o2));
    m1 = n1; m2 = n2;
  }
  const float gscore = m1 + m2;
  const int g = lane >> 2;
  int rank = 0;
#pragma unroll
  for (int gg = 0; gg < kGroups; ++gg) {
    const float o = __shfl_sync(full, gscore, gg * 4);
    rank += (o > gscore || (o == gscore && gg < g)) ? 1 : 0;
  }
  const bool keep = rank < kTopKGroups;
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = keep ? v[i] : -CUDART_MAX_NORMAL_F;

  // eight rounds of warp-wide argmax over the kept experts
  int my_idx = 0;
  float my_s = 0.0f;
#pragma unroll 1
  for (int r = 0; r < kTopK; ++r) {
    float bv = v[0];
    int bi = 0;
#pragma unroll
    for (int i = 1; i < 8; ++i)
      if (v[i] > bv) { bv = v[i]; bi = i; }
    bi += lane * 8;
    // Warp-wide maximum of the lanes' best values through an order-preserving integer key (one redux
    // instead of five shuffle steps); ties go to the lowest lane, i.e. the lowest expert index, and
    // inside a lane the strict '>' above already kept the lowest slot.  (+ 0.0f folds -0 into +0 so
    // that equal floats have equal keys.)
    const uint32_t fb = __float_as_uint(bv + 0.0f);
    const uint32_t key = (fb & 0x80000000u) ? ~fb : (fb | 0x80000000u);
    const uint32_t kmax = __reduce_max_sync(full, key);
    const int owner = __ffs(__ballot_sync(full, key == kmax)) - 1;
    bi = __shfl_sync(full, bi, owner);
    const int slot = bi & 7;
    float sel = s[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) sel = (slot == i) ? s[i] : sel;
    sel = __shfl_sync(full, sel, owner);
    if (lane == owner) {
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (slot == i) v[i] = -CUDART_INF_F;
    }
    if (lane == r) { my_idx = bi; my_s = sel; }
  }

  float sum = (lane < kTopK) ? my_s : 0.0f;
#pragma unroll
  for (int d = 4; d >= 1; d >>= 1) sum += __shfl_xor_sync(full, sum, d);
  sum = __shfl_sync(full, sum, 0);
  const float w = (my_s / (sum + 1e-20f)) * scaling;

  const int le = my_idx - expert_offset;
  const bool local = (lane < kTopK) && le >= 0 && le < e_local;
  const uint32_t mask = __reduce_or_sync(full, local ? (1u << le) : 0u);
  if (lane < kTopK) {
    topk_idx[t * kTopK + lane] = my_idx;
    topk_w[t * kTopK + lane] = w;
    route_row[t * kTopK + lane] = -1;
    if (local) atomicAdd(&counts[le], 1);
  }
  if (lane == 0) local_mask[t] = mask;
}

}  // namespace

cudaError_t launch_router(const float* logits, const void* bias_bf16, int T, int e_local, int expert_offset,
                          float scaling, const Workspace& ws, bool counters_are_zero, cudaStream_t st) {
  // The per-expert row counters must start at zero.  Inside the layer the kernels further down the
  // chain leave them zeroed for the next call (gather_rows_kernel, build_rows_kernel), which saves a
  // memset node in front of every call; any other caller zeroes them here.
  if (!counters_are_zero) {
    cudaError_t e = cudaMemsetAsync(ws.counts, 0, sizeof(int) * 2 * kMaxLocalExperts, st);
    if (e != cudaSuccess) return e;
  }
  const int blocks = (T + kWarpsPerBlock - 1) / kWarpsPerBlock;
  route_kernel<<<blocks, kWarpsPerBlock * 32, 0, st>>>(logits, static_cast<const __nv_bfloat16*>(bias_bf16), T,
                                                      e_local, expert_offset, scaling, ws.topk_idx, ws.topk_w,
                                                      ws.local_mask, ws.route_row, ws.counts);
  return cudaGetLastError();
}

}  // namespace syfi

// ---------------------------------------------------------------------------------------------
// Router entry point for callers that must not allocate.
//
// Some hosts of this library cannot call cudaMalloc on the path that runs the router: a serving
// process whose memory pool owns the whole device, a plugin loaded into a framework that forbids
// allocation inside its execution callbacks, or code that runs while other threads capture CUDA
// graphs (an allocation there would invalidate the capture).  For them the router's scratch (the
// per-token expert mask, the per-route row slots and the per-expert counters that the context-based
// entry point keeps in its cudaMalloc'ed workspace) lives in a fixed array inside the library image.
// The array costs kNoAllocScratchBytes of device memory on every GPU that loads the library, until
// the process exits, and bounds the batch at SYFI_MOE_NOALLOC_MAX_TOKENS tokens per call.
// ---------------------------------------------------------------------------------------------
namespace {

constexpr int kNoAllocMaxTokens = SYFI_MOE_NOALLOC_MAX_TOKENS;
constexpr size_t kNoAllocMaskBytes = sizeof(uint32_t) * kNoAllocMaxTokens;               // local_mask
constexpr size_t kNoAllocRowBytes = sizeof(int) * kNoAllocMaxTokens * syfi::kTopK;       // route_row
constexpr size_t kNoAllocCountBytes = 256;                                               // counts (32 ints, padded)
constexpr size_t kNoAllocScratchBytes = kNoAllocMaskBytes + kNoAllocRowBytes + kNoAllocCountBytes;

// In host code this name is only a handle for the runtime, never an address to hand to a kernel:
// the device address is looked up once per device with cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_noalloc_mu;
unsigned char* g_noalloc_ptr[kMaxDevices] = {nullptr};

}  // namespace

extern "C" int syfi_moe_route_noalloc(const void* routing_logits, const void* routing_bias, int64_t num_tokens,
                                      int32_t num_local_experts, int64_t local_expert_offset,
                                      double routed_scaling_factor, int32_t* topk_idx, float* topk_weights,
                                      void* stream) {
  using namespace syfi;
  char msg[256];
  if (num_tokens < 0 || num_tokens > kNoAllocMaxTokens) {
    snprintf(msg, sizeof(msg),
             "syfi_moe_route_noalloc handles at most %d tokens per call (its scratch is a fixed array); got %lld",
             kNoAllocMaxTokens, (long long)num_tokens);
    return set_last_error(SYFI_MOE_ERR_INVALID, msg);
  }
  if (num_local_experts < 1 || num_local_experts > kMaxLocalExperts || local_expert_offset < 0 ||
      local_expert_offset + num_local_experts > kExpertsGlobal)
    return set_last_error(SYFI_MOE_ERR_INVALID, "local expert range outside [0, 256) or more than 32 experts");
  if (!(routed_scaling_factor == routed_scaling_factor) || routed_scaling_factor > 3.0e38 ||
      routed_scaling_factor < -3.0e38)
    return set_last_error(SYFI_MOE_ERR_INVALID, "routed_scaling_factor is not a finite float");
  if (num_tokens == 0) return SYFI_MOE_OK;
  if (!routing_logits || !routing_bias || !topk_idx || !topk_weights)
    return set_last_error(SYFI_MOE_ERR_INVALID, "null tensor argument");
  if ((reinterpret_cast<uintptr_t>(routing_logits) | reinterpret_cast<uintptr_t>(routing_bias)) & 15u)
    return set_last_error(SYFI_MOE_ERR_INVALID, "routing_logits and routing_bias must be 16-byte aligned");

  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    snprintf(msg, sizeof(msg), "cannot identify the current device: %s", cudaGetErrorString(e));
    return set_last_error(SYFI_MOE_ERR_CUDA, msg);
  }
  unsigned char* base = nullptr;
  {
    // Set-up, once per device, with that device current: resolve the device address of the array.
    std::lock_guard<std::mutex> lock(g_noalloc_mu);
    if (g_noalloc_ptr[dev] == nullptr) {
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
      if (e != cudaSuccess || p == nullptr) {
        snprintf(msg, sizeof(msg), "cudaGetSymbolAddress(scratch) failed on device %d: %s", dev,
                 cudaGetErrorString(e));
        return set_last_error(SYFI_MOE_ERR_CUDA, msg);
      }
      g_noalloc_ptr[dev] = static_cast<unsigned char*>(p);
    }
    base = g_noalloc_ptr[dev];
  }
  uint32_t* local_mask = reinterpret_cast<uint32_t*>(base);
  int* route_row = reinterpret_cast<int*>(base + kNoAllocMaskBytes);
  int* counts = reinterpret_cast<int*>(base + kNoAllocMaskBytes + kNoAllocRowBytes);

  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int T = static_cast<int>(num_tokens);
  // The array keeps whatever the previous call left; only the counters must start at zero.
  e = cudaMemsetAsync(counts, 0, sizeof(int) * kMaxLocalExperts, st);
  if (e == cudaSuccess) {
    const int blocks = (T + kWarpsPerBlock - 1) / kWarpsPerBlock;
    route_kernel<<<blocks, kWarpsPerBlock * 32, 0, st>>>(
        static_cast<const float*>(routing_logits), static_cast<const __nv_bfloat16*>(routing_bias), T,
        num_local_experts, static_cast<int>(local_expert_offset), static_cast<float>(routed_scaling_factor),
        topk_idx, topk_weights, local_mask, route_row, counts);
    e = cudaGetLastError();
  }
  if (e != cudaSuccess) {
    snprintf(msg, sizeof(msg), "router launch failed: %s", cudaGetErrorString(e));
    return set_last_error(SYFI_MOE_ERR_CUDA, msg);
  }
  return SYFI_MOE_OK;
}

