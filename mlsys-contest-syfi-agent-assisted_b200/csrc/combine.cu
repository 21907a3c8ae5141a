// Weighted un-permute / combine: out[t, :] = sum_k w[t, k] * O_rows[row(t, k), :].
//
// Replaces the reference's fp32 atomic scatter in the GEMM2 epilogue plus
// fin_cast_kernel (moe/solution/cuda/moe.cu:1879-1884, 2758-2779) and its small-T
// finalize_rows_bf16_kernel (moe.cu:2781-2817).  The sum runs over the token's eight
// routes in a fixed order, in f32, with a single rounding to bf16 at the end, so the
// result is deterministic; tokens with no local route get zeros.  With out_is_f32 the
// un-rounded f32 row is written instead (the partial an expert-parallel rank hands to
// the cross-rank reduction).
#include <cuda_bf16.h>

#include "moe_internal.h"
#include "ptx.cuh"

namespace syfi {

namespace {

constexpr int kCombineThreads = 256;
constexpr int kSegments = kHidden / (kCombineThreads * 4);  // 7 segments of 1024 features per row
static_assert(kSegments * kCombineThreads * 4 == kHidden, "row must split evenly");

// One CTA per (token, 1024-feature segment), one float4 per thread and route: the eight routes' loads are
// all in flight at once (a loop over the routes with the whole row per thread pays eight dependent
// round trips to memory, which is what this kernel's duration consists of at small batches).
__global__ void __launch_bounds__(kCombineThreads)
combine_segments_kernel(int T, const int* __restrict__ route_row, const float* __restrict__ topk_w,
               const float* __restrict__ o_rows, void* __restrict__ out, int out_is_f32, int row_cap) {
  const int t = blockIdx.x, seg = blockIdx.y;
  pdl_wait();
  pdl_trigger();
  if (t >= T) return;
  const int col4 = seg * kCombineThreads + threadIdx.x;        // float4 index inside the row
  int rows[kTopK];
  float w[kTopK];
#pragma unroll
  for (int k = 0; k < kTopK; ++k) {
    rows[k] = route_row[t * kTopK + k];
    w[k] = topk_w[t * kTopK + k];
  }
  float4 v[kTopK];
#pragma unroll
  for (int k = 0; k < kTopK; ++k) {
    const bool valid = rows[k] >= 0 && rows[k] < row_cap;
    v[k] = valid ? __ldg(reinterpret_cast<const float4*>(o_rows + static_cast<size_t>(rows[k]) * kHidden) + col4)
                 : make_float4(0.f, 0.f, 0.f, 0.f);
    if (!valid) w[k] = 0.0f;
  }
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int k = 0; k < kTopK; ++k) {                            // fixed order: deterministic sum
    if (rows[k] >= 0 && rows[k] < row_cap) {
      acc.x = fmaf(w[k], v[k].x, acc.x);
      acc.y = fmaf(w[k], v[k].y, acc.y);
      acc.z = fmaf(w[k], v[k].z, acc.z);
      acc.w = fmaf(w[k], v[k].w, acc.w);
    }
  }
  if (out_is_f32) {
    reinterpret_cast<float4*>(static_cast<float*>(out) + static_cast<size_t>(t) * kHidden)[col4] = acc;
  } else {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y);
    const __nv_bfloat162 hi = __floats2bfloat162_rn(acc.z, acc.w);
    uint2 pk;
    pk.x = *reinterpret_cast<const uint32_t*>(&lo);
    pk.y = *reinterpret_cast<const uint32_t*>(&hi);
    reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(out) + static_cast<size_t>(t) * kHidden)[col4] = pk;
  }
}

constexpr int kVecPerThread = kHidden / (kCombineThreads * 4);  // 7
static_assert(kVecPerThread * kCombineThreads * 4 == kHidden, "row must split evenly");

// One CTA per token, seven float4 per thread and route, the routes one after the other: fewer, fatter CTAs
// for large batches, where the kernel is bound by HBM and not by its chain of dependent reads.
__global__ void __launch_bounds__(kCombineThreads)
combine_rows_kernel(int T, const int* __restrict__ route_row, const float* __restrict__ topk_w,
               const float* __restrict__ o_rows, void* __restrict__ out, int out_is_f32, int row_cap) {
  const int t = blockIdx.x;
  pdl_wait();
  pdl_trigger();
  if (t >= T) return;
  const int tid = threadIdx.x;
  float4 acc[kVecPerThread];
#pragma unroll
  for (int i = 0; i < kVecPerThread; ++i) acc[i] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 1
  for (int k = 0; k < kTopK; ++k) {
    const int row = route_row[t * kTopK + k];
    if (row < 0 || row >= row_cap) continue;
    const float w = topk_w[t * kTopK + k];
    const float4* src = reinterpret_cast<const float4*>(o_rows + static_cast<size_t>(row) * kHidden);
#pragma unroll
    for (int i = 0; i < kVecPerThread; ++i) {
      const float4 v = __ldg(src + i * kCombineThreads + tid);
      acc[i].x = fmaf(w, v.x, acc[i].x);
      acc[i].y = fmaf(w, v.y, acc[i].y);
      acc[i].z = fmaf(w, v.z, acc[i].z);
      acc[i].w = fmaf(w, v.w, acc[i].w);
    }
  }
  if (out_is_f32) {
    float4* dst = reinterpret_cast<float4*>(static_cast<float*>(out) + static_cast<size_t>(t) * kHidden);
#pragma unroll
    for (int i = 0; i < kVecPerThread; ++i) dst[i * kCombineThreads + tid] = acc[i];
  } else {
    uint2* dst = reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(out) + static_cast<size_t>(t) * kHidden);
#pragma unroll
    for (int i = 0; i < kVecPerThread; ++i) {
      const __nv_bfloat162 lo = __floats2bfloat162_rn(acc[i].x, acc[i].y);
      const __nv_bfloat162 hi = __floats2bfloat162_rn(acc[i].z, acc[i].w);
      uint2 p;
      p.x = *reinterpret_cast<const uint32_t*>(&lo);
      p.y = *reinterpret_cast<const uint32_t*>(&hi);
      dst[i * kCombineThreads + tid] = p;
    }
  }
}

}  // namespace

cudaError_t launch_combine(int T, const Workspace& ws, void* out, int out_is_f32, cudaStream_t st) {
  if (T <= 512)   // latency-bound sizes: 7 CTAs per token, all eight routes' loads in flight
    return launch_dependent(combine_segments_kernel, dim3(T, kSegments), dim3(kCombineThreads), 0, st, T,
                            ws.route_row, ws.topk_w, ws.o_rows, out, out_is_f32, ws.row_cap);
  return launch_dependent(combine_rows_kernel, dim3(T), dim3(kCombineThreads), 0, st, T, ws.route_row, ws.topk_w,
                          ws.o_rows, out, out_is_f32, ws.row_cap);
}

}  // namespace syfi
