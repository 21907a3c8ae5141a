// DSA top-k indexer (definition dsa_topk_indexer_fp8_h64_d128_topk2048_ps64), the sibling operator of the MoE
// layer that shares its building blocks: FP8 scoring on the tensor cores and a selection of the best tokens.
//
// Replaces the reference's score_kernel (dsa_indexer/solution/cuda/dsa_topk_indexer.cu:78-250: e4m3 unpacked
// to bf16 in shared memory, wmma 16x16x16) and topk_kernel_radix (:251-395: one 8-bit histogram, tokens of the
// threshold byte in arbitrary order), and computes what the definition's configured entry point computes
// (dsa_indexer/solution/python/dsa_topk_indexer.py:64-112, pure torch):
//     score[t] = sum_h weights[b, h] * relu(q[b, h, :] . (k8[t, :] * kscale[t])),   best 2048 tokens, best first.
//
//   score kernel : one CTA per (sequence, 128 tokens = two cache pages).  The pages' 64 x 128 e4m3 bytes are
//                  contiguous in the cache (a page is 64 rows of 128 bytes followed by 64 f32 scales = 66 rows of
//                  128 bytes), so one tensor map over the cache as rows of 128 bytes fetches a page with one TMA
//                  box; the query's 64 heads are a second box.  tcgen05.mma kind::f8f6f4, M = 128 tokens,
//                  N = 64 heads, K = 128 in four steps, accumulator in tensor memory; the raw e4m3 products are
//                  exact, so the token's scale is applied once, after the sum over K.  Each thread then owns a
//                  token: relu, times the head weight, summed over the 64 heads in head order.
//   select kernel: one CTA per sequence.  Exact radix select of the k-th largest score over an order-preserving
//                  32-bit key (four 8-bit passes), compaction of the k winners (ties at the cut by lower position),
//                  bitonic sort of the 2048 (key, position) pairs in shared memory: best first, ties by position.
// Every wait is bounded; a failure is recorded in the status word the host entry point reads back.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdio>
#include <mutex>

#include "../../include/syfi_dsa.h"
#include "moe_internal.h"
#include "ptx.cuh"

namespace syfi {

namespace {

constexpr int kHeads = 64;
constexpr int kDim = 128;
constexpr int kPage = 64;
constexpr int kPageRows = 66;                 // 128-byte rows per cache page: 64 key rows + 2 rows of scales
constexpr int kPageBytes = kPageRows * 128;   // 8448
constexpr int kTopK = SYFI_DSA_TOPK;
constexpr int kTokTile = 128;                 // tokens per score CTA
constexpr int kScoreThreads = 128;
constexpr int kScoreSmem = 1024 + kTokTile * kDim + kHeads * kDim;   // alignment slack + key tile + query tile
constexpr int kSelectThreads = 1024;
constexpr long long kWaitLimit = 1ll << 31;   // SM clocks (about a second)
constexpr int kStatusScoreTimeout = 201;

__global__ void __launch_bounds__(kScoreThreads)
dsa_score_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                 const uint8_t* __restrict__ cache, const float* __restrict__ weights,
                 const int32_t* __restrict__ seq_lens, const int32_t* __restrict__ block_table, int max_pages,
                 float* __restrict__ scores, int max_ls, int* __restrict__ status) {
  const int b = blockIdx.y, t0 = blockIdx.x * kTokTile;
  const int n = seq_lens[b];
  if (t0 >= n) return;                         // the whole CTA leaves before any barrier or allocation

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t* s_k = smem;                         // [128 tokens][128 B], 128-byte swizzle (two page boxes)
  uint8_t* s_q = smem + kTokTile * kDim;       // [64 heads][128 B]
  __shared__ uint64_t bar_tma, bar_mma;
  __shared__ uint32_t s_tmem;
  __shared__ float s_w[kHeads];
  __shared__ int s_page[2];
  __shared__ volatile int s_abort;

  const int tid = threadIdx.x, warp = tid >> 5;
  if (tid < kHeads) s_w[tid] = weights[b * kHeads + tid];
  if (tid < 2) s_page[tid] = (t0 + tid * kPage < n) ? block_table[b * max_pages + (t0 / kPage) + tid] : -1;
  if (tid == 0) {
    mbar_init(&bar_tma, 1);
    mbar_init(&bar_mma, 1);
    s_abort = 0;
    fence_barrier_init();
  }
  if (warp == 0) {
    tmem_alloc(&s_tmem, kHeads);               // 64 columns: one f32 per head and token lane
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = s_tmem;

  if (tid == 0) {
    const int pages = s_page[1] >= 0 ? 2 : 1;
    mbar_arrive_expect_tx(&bar_tma, kHeads * kDim + pages * kPage * kDim);
    const uint64_t pol = l2_policy_evict_normal();
    tma_load_2d(s_q, &tm_q, &bar_tma, 0, b * kHeads, pol);
    for (int p = 0; p < pages; ++p) tma_load_2d(s_k + p * kPage * kDim, &tm_k, &bar_tma, 0, s_page[p] * kPageRows, pol);
    if (mbar_wait_bounded(&bar_tma, 0, &s_abort, kStatusScoreTimeout, kWaitLimit)) {
      tc_fence_after();
      const uint64_t a0 = umma_smem_desc_sw128(smem_u32(s_k));
      const uint64_t b0 = umma_smem_desc_sw128(smem_u32(s_q));
      const uint32_t idesc = umma_idesc_e4m3_m128(kHeads);
#pragma unroll
      for (int k4 = 0; k4 < 4; ++k4) umma_f8(tmem_base, a0 + 2 * k4, b0 + 2 * k4, idesc, k4 > 0 ? 1u : 0u);
      umma_commit(&bar_mma);
    }
  }
  __syncwarp();
  const bool ok = mbar_wait_bounded(&bar_mma, 0, &s_abort, kStatusScoreTimeout, kWaitLimit);
  tc_fence_after();
  if (ok) {
    // this thread's token: lane `tid` of tensor memory (a warp reads its own lane quarter)
    const int t = t0 + tid;
    const int page = s_page[tid >> 6];
    const bool valid = t < n && page >= 0;
    const float scale = valid ? *reinterpret_cast<const float*>(cache + static_cast<size_t>(page) * kPageBytes +
                                                                kPage * kDim + (tid & (kPage - 1)) * 4)
                              : 0.0f;
    const uint32_t taddr = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
    float acc = 0.0f;
#pragma unroll
    for (int c = 0; c < kHeads / 16; ++c) {
      uint32_t r[16];
      tmem_ld16(taddr + c * 16, r);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 16; ++j) acc = fmaf(s_w[c * 16 + j], fmaxf(__uint_as_float(r[j]) * scale, 0.0f), acc);
    }
    if (valid) scores[static_cast<size_t>(b) * max_ls + t] = acc;
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kHeads);
  }
  if (tid == 0 && s_abort != 0) atomicExch(status, s_abort);
}

// larger float <-> larger key (NaN aside); key 0 is below every score
__device__ __forceinline__ uint32_t score_key(float s) {
  const uint32_t u = __float_as_uint(s);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__global__ void __launch_bounds__(kSelectThreads)
dsa_select_kernel(const float* __restrict__ scores, int max_ls, const int32_t* __restrict__ seq_lens,
                  const int32_t* __restrict__ block_table, int max_pages, int32_t* __restrict__ out) {
  __shared__ unsigned long long s_item[kTopK];   // (key << 32) | ~position: descending order = best first, ties by position
  __shared__ int s_hist[256];
  __shared__ int s_pick, s_above, s_fill, s_eq;
  const int b = blockIdx.x, tid = threadIdx.x;
  const int n = min(seq_lens[b], max_ls);
  const int k = min(kTopK, n);
  int32_t* o = out + static_cast<size_t>(b) * kTopK;
  const float* sc = scores + static_cast<size_t>(b) * max_ls;
  for (int i = tid; i < kTopK; i += kSelectThreads) s_item[i] = 0ull;
  if (k == 0) {
    for (int i = tid; i < kTopK; i += kSelectThreads) o[i] = -1;
    return;
  }
  // ---- the k-th largest key, byte by byte from the top: `prefix` holds the bytes found so far, `want` how
  // many of the keys that match the prefix are still to be taken from the top
  uint32_t prefix = 0, mask = 0;
  int want = k;
  for (int shift = 24; shift >= 0; shift -= 8) {
    if (tid < 256) s_hist[tid] = 0;
    __syncthreads();
    for (int i = tid; i < n; i += kSelectThreads) {
      const uint32_t key = score_key(sc[i]);
      if ((key & mask) == prefix) atomicAdd(&s_hist[(key >> shift) & 255u], 1);
    }
    __syncthreads();
    if (tid == 0) {
      int seen = 0, pick = 0;
      for (int v = 255; v >= 0; --v) {
        if (seen + s_hist[v] >= want) { pick = v; break; }
        seen += s_hist[v];
      }
      s_pick = pick;
      s_above = seen;
    }
    __syncthreads();
    prefix |= static_cast<uint32_t>(s_pick) << shift;
    mask |= 255u << shift;
    want -= s_above;
    __syncthreads();
  }
  // prefix = the key of the last place; `want` of the keys equal to it are kept (the lowest positions)
  const uint32_t cut = prefix;
  if (tid == 0) { s_fill = 0; s_eq = 0; }
  __syncthreads();
  for (int i0 = 0; i0 < n; i0 += kSelectThreads) {
    const int i = i0 + tid;
    const uint32_t key = i < n ? score_key(sc[i]) : 0u;
    if (i < n && key > cut) s_item[atomicAdd(&s_fill, 1)] = (static_cast<unsigned long long>(key) << 32) | (~static_cast<uint32_t>(i));
    // ties at the cut are admitted in position order: count the ones before this position, pass by pass
    const bool tie = i < n && key == cut;
    const unsigned bal = __ballot_sync(0xffffffffu, tie);
    __shared__ int s_wtie[kSelectThreads / 32];
    if ((tid & 31) == 0) s_wtie[tid >> 5] = __popc(bal);
    __syncthreads();
    int before = s_eq;
    for (int w = 0; w < (tid >> 5); ++w) before += s_wtie[w];
    before += __popc(bal & ((1u << (tid & 31)) - 1u));
    if (tie && before < want)
      s_item[atomicAdd(&s_fill, 1)] = (static_cast<unsigned long long>(key) << 32) | (~static_cast<uint32_t>(i));
    __syncthreads();
    if (tid == 0) {
      int tot = 0;
      for (int w = 0; w < kSelectThreads / 32; ++w) tot += s_wtie[w];
      s_eq += tot;
    }
    __syncthreads();
  }
  // ---- bitonic sort of the 2048 items, descending (empty places are 0 and sink to the end)
  for (int size = 2; size <= kTopK; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      __syncthreads();
      for (int i = tid; i < kTopK / 2; i += kSelectThreads) {
        const int lo = 2 * i - (i & (stride - 1));
        const int hi = lo + stride;
        const bool desc = (lo & size) == 0;
        const unsigned long long a = s_item[lo], c = s_item[hi];
        if ((a < c) == desc) { s_item[lo] = c; s_item[hi] = a; }
      }
    }
  }
  __syncthreads();
  for (int i = tid; i < kTopK; i += kSelectThreads) {
    int32_t tok = -1;
    if (i < k) {
      const int pos = static_cast<int>(~static_cast<uint32_t>(s_item[i] & 0xffffffffull));
      tok = block_table[b * max_pages + pos / kPage] * kPage + pos % kPage;
    }
    o[i] = tok;
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
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

// rows of 128 bytes, boxes of 64 rows, 128-byte swizzle
bool rows128_map(CUtensorMap* m, const void* base, uint64_t rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {128, rows};
  const cuuint64_t strides[1] = {128};
  const cuuint32_t box[2] = {128, 64};
  const cuuint32_t estr[2] = {1, 1};
  return fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// per-device scratch: the scores of every token of every sequence, and a status word
struct Scratch {
  float* scores = nullptr;
  size_t floats = 0;
  int* status = nullptr;
  bool checked = false;
};
std::mutex g_mu;
Scratch g_scratch[64];

int fail(int code, const char* msg) { return set_last_error(code, msg); }

}  // namespace

}  // namespace syfi

using namespace syfi;

extern "C" int syfi_dsa_topk_indexer(const void* q_index_fp8, const void* k_index_cache_fp8, const float* weights,
                                     const int32_t* seq_lens, const int32_t* block_table, int32_t batch,
                                     int64_t num_pages, int32_t max_pages, int32_t* topk_indices, void* stream) {
  if (batch < 0 || batch > (1 << 20)) return fail(SYFI_DSA_ERR_INVALID, "batch out of range");
  if (batch == 0) return SYFI_DSA_OK;
  if (num_pages < 1 || num_pages > (1ll << 24)) return fail(SYFI_DSA_ERR_INVALID, "num_pages out of range");
  if (max_pages < 1 || max_pages > (1 << 20)) return fail(SYFI_DSA_ERR_INVALID, "max_pages (block table width) out of range");
  const void* ptrs[] = {q_index_fp8, k_index_cache_fp8, weights, seq_lens, block_table, topk_indices};
  for (const void* p : ptrs)
    if (!p || (reinterpret_cast<uintptr_t>(p) & 15u)) return fail(SYFI_DSA_ERR_INVALID, "a tensor argument is null or not 16-byte aligned");
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return fail(SYFI_DSA_ERR_CUDA, "no current CUDA device: this library has no CPU path");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int max_ls = max_pages * kPage;
  std::lock_guard<std::mutex> lock(g_mu);
  Scratch& s = g_scratch[dev];
  if (!s.checked) {     // once per device: the attribute queries cost more than the kernels
    int major = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess || major != 10)
      return fail(SYFI_DSA_ERR_CUDA, "this library is built for sm_100a (B200) only");
    s.checked = true;
  }
  const size_t need = static_cast<size_t>(batch) * max_ls;
  if (need > s.floats) {
    if (cudaDeviceSynchronize() != cudaSuccess) return fail(SYFI_DSA_ERR_CUDA, "device synchronisation failed");
    if (s.scores) cudaFree(s.scores);
    s.scores = nullptr;
    s.floats = 0;
    if (cudaMalloc(&s.scores, need * sizeof(float)) != cudaSuccess) return fail(SYFI_DSA_ERR_CUDA, "out of device memory for the scores");
    s.floats = need;
  }
  if (!s.status) {
    if (cudaMalloc(&s.status, 16) != cudaSuccess) return fail(SYFI_DSA_ERR_CUDA, "out of device memory");
    cudaMemset(s.status, 0, 16);
    if (cudaFuncSetAttribute(dsa_score_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kScoreSmem) != cudaSuccess)
      return fail(SYFI_DSA_ERR_CUDA, "cannot raise the shared-memory limit of the score kernel");
  }
  CUtensorMap tm_q, tm_k;
  if (!rows128_map(&tm_q, q_index_fp8, static_cast<uint64_t>(batch) * kHeads) ||
      !rows128_map(&tm_k, k_index_cache_fp8, static_cast<uint64_t>(num_pages) * kPageRows))
    return fail(SYFI_DSA_ERR_CUDA, "cuTensorMapEncodeTiled failed");
  const int tiles = (max_ls + kTokTile - 1) / kTokTile;
  dsa_score_kernel<<<dim3(tiles, batch), kScoreThreads, kScoreSmem, st>>>(
      tm_q, tm_k, static_cast<const uint8_t*>(k_index_cache_fp8), weights, seq_lens, block_table, max_pages, s.scores,
      max_ls, s.status);
  if (cudaGetLastError() != cudaSuccess) return fail(SYFI_DSA_ERR_CUDA, "score kernel launch failed");
  dsa_select_kernel<<<batch, kSelectThreads, 0, st>>>(s.scores, max_ls, seq_lens, block_table, max_pages, topk_indices);
  if (cudaGetLastError() != cudaSuccess) return fail(SYFI_DSA_ERR_CUDA, "select kernel launch failed");
  return SYFI_DSA_OK;
}

extern "C" int syfi_dsa_check(void* stream) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return fail(SYFI_DSA_ERR_CUDA, "no current CUDA device");
  if (cudaStreamSynchronize(static_cast<cudaStream_t>(stream)) != cudaSuccess)
    return fail(SYFI_DSA_ERR_CUDA, "stream synchronisation failed");
  std::lock_guard<std::mutex> lock(g_mu);
  Scratch& s = g_scratch[dev];
  if (!s.status) return SYFI_DSA_OK;
  int status = 0;
  if (cudaMemcpy(&status, s.status, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return fail(SYFI_DSA_ERR_CUDA, "cannot read the status word");
  if (status != 0) {
    cudaMemset(s.status, 0, sizeof(int));
    char msg[128];
    snprintf(msg, sizeof(msg), "a kernel reported status %d (201: a bounded wait in the score kernel ran out)", status);
    return fail(SYFI_DSA_ERR_DEVICE, msg);
  }
  return SYFI_DSA_OK;
}
