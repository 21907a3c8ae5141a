// DSA top-k indexer (definition dsa_topk_indexer_fp8_h64_d128_topk2048_ps64), the sibling operator of the MoE
// layer that shares its building blocks: FP8 scoring on the tensor cores and a selection of the best tokens.
//
// Replaces the reference's score_kernel (dsa_indexer/solution/cuda/dsa_topk_indexer.cu:78-250: e4m3 unpacked
// to bf16 in shared memory, wmma 16x16x16) and topk_kernel_radix (:251-395: one 8-bit histogram, tokens of the
// threshold byte in arbitrary order), and computes what the definition's configured entry point computes
// (dsa_indexer/solution/python/dsa_topk_indexer.py:64-112, pure torch):
//     score[t] = sum_h weights[b, h] * relu(q[b, h, :] . (k8[t, :] * kscale[t])),   best 2048 tokens, best first.
//
//   score kernel : one CTA per (sequence, 1024 tokens), 128 tokens = two cache pages per MMA, key tiles and
//                  accumulators double-buffered.  The pages' 64 x 128 e4m3 bytes are
//                  contiguous in the cache (a page is 64 rows of 128 bytes followed by 64 f32 scales = 66 rows of
//                  128 bytes), so one tensor map over the cache as rows of 128 bytes fetches a page with one TMA
//                  box; the query's 64 heads are a second box.  tcgen05.mma kind::f8f6f4, M = 128 tokens,
//                  N = 64 heads, K = 128 in four steps, accumulator in tensor memory; the raw e4m3 products are
//                  exact, so the token's scale is applied once, after the sum over K.  Each thread then owns a
//                  token: relu, times the head weight, summed over the 64 heads in head order.
//   select kernels: items (order-preserving key of the score, position) are distinct, so the cut is one exact item:
//                  an 8-pass radix select, compaction of the winners, bitonic sort of 2048 items in shared memory
//                  (best first, ties by position).  Two levels: a CTA per 16384 positions keeps its best 2048 (a
//                  sequence of one chunk is finished there), a CTA per longer sequence merges the chunks' candidates.
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
constexpr int kKeep = SYFI_DSA_TOPK;          // tokens kept per sequence
constexpr int kTokTile = 128;                 // tokens per MMA: two cache pages
constexpr int kTilesPerCta = 8;               // a score CTA walks 1024 tokens of one sequence
constexpr int kScoreThreads = 160;            // four epilogue warps (one tensor-memory lane quarter each) + a producer / MMA warp
constexpr int kScoreStages = 2;
constexpr int kScoreSmem = 1024 + kScoreStages * kTokTile * kDim + kHeads * kDim;   // slack + key tiles + query tile
constexpr int kSelectThreads = 1024;
constexpr long long kWaitLimit = 1ll << 31;   // SM clocks (about a second)
constexpr int kStatusScoreTimeout = 201;

// Score kernel: CTA (x, b) scores tokens [1024 x, 1024 x + 1024) of sequence b, 128 at a time, through a two-deep
// ring of key tiles in shared memory and two accumulators in tensor memory: while the four epilogue warps turn
// tile i into scores, the tensor core works on tile i + 1 and TMA fetches tile i + 2.
__global__ void __launch_bounds__(kScoreThreads)
dsa_score_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                 const uint8_t* __restrict__ cache, const float* __restrict__ weights,
                 const int32_t* __restrict__ seq_lens, const int32_t* __restrict__ block_table, int max_pages,
                 float* __restrict__ scores, int max_ls, int* __restrict__ status) {
  const int b = blockIdx.y, t_begin = blockIdx.x * kTilesPerCta * kTokTile;
  const int n = min(seq_lens[b], max_ls);
  if (t_begin >= n) return;                    // the whole CTA leaves before any barrier or allocation
  const int tiles = min(kTilesPerCta, (n - t_begin + kTokTile - 1) / kTokTile);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t* s_k = smem;                                     // [2 stages][128 tokens][128 B], 128-byte swizzle
  uint8_t* s_q = smem + kScoreStages * kTokTile * kDim;    // [64 heads][128 B]
  __shared__ uint64_t full[kScoreStages], empty[kScoreStages], tfull[kScoreStages], tempty[kScoreStages], qfull;
  __shared__ uint32_t s_tmem;
  __shared__ float s_w[kHeads];
  __shared__ int s_page[2 * kTilesPerCta];
  __shared__ volatile int s_abort;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid < kHeads) s_w[tid] = weights[b * kHeads + tid];
  if (tid < 2 * kTilesPerCta)
    s_page[tid] = (t_begin + tid * kPage < n) ? block_table[b * max_pages + t_begin / kPage + tid] : -1;
  if (tid == 0) {
    for (int i = 0; i < kScoreStages; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
      mbar_init(&tfull[i], 1);
      mbar_init(&tempty[i], 4);                // one arrival per epilogue warp
    }
    mbar_init(&qfull, 1);
    s_abort = 0;
    fence_barrier_init();
  }
  if (warp == 4) {
    tmem_alloc(&s_tmem, kScoreStages * kHeads);            // two accumulators of 64 columns
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = s_tmem;

  if (warp == 4) {
    if (lane == 0) {
      // ---------------------------------------------------------- producer and MMA issuer (one thread)
      const uint64_t pol = l2_policy_evict_first();        // the cache is streamed once
      auto load_tile = [&](int i) {
        const int st = i % kScoreStages;
        const int pages = s_page[2 * i + 1] >= 0 ? 2 : 1;
        mbar_arrive_expect_tx(&full[st], pages * kPage * kDim);
        for (int p = 0; p < pages; ++p)
          tma_load_2d(s_k + st * kTokTile * kDim + p * kPage * kDim, &tm_k, &full[st], 0, s_page[2 * i + p] * kPageRows, pol);
      };
      mbar_arrive_expect_tx(&qfull, kHeads * kDim);
      tma_load_2d(s_q, &tm_q, &qfull, 0, b * kHeads, l2_policy_evict_last());
      load_tile(0);
      if (tiles > 1) load_tile(1);
      bool alive = mbar_wait_bounded(&qfull, 0, &s_abort, kStatusScoreTimeout, kWaitLimit);
      const uint64_t b0 = umma_smem_desc_sw128(smem_u32(s_q));
      const uint32_t idesc = umma_idesc_e4m3_m128(kHeads);
      for (int i = 0; i < tiles && alive; ++i) {
        const int st = i % kScoreStages;
        const uint32_t ph = (i / kScoreStages) & 1u;
        if (!mbar_wait_bounded(&full[st], ph, &s_abort, kStatusScoreTimeout, kWaitLimit)) break;
        if (!mbar_wait_bounded(&tempty[st], ph ^ 1u, &s_abort, kStatusScoreTimeout, kWaitLimit)) break;
        tc_fence_after();
        const uint64_t a0 = umma_smem_desc_sw128(smem_u32(s_k + st * kTokTile * kDim));
#pragma unroll
        for (int k4 = 0; k4 < 4; ++k4) umma_f8(tmem_base + st * kHeads, a0 + 2 * k4, b0 + 2 * k4, idesc, k4 > 0 ? 1u : 0u);
        umma_commit(&empty[st]);               // the key tile may be overwritten once these MMAs have read it
        umma_commit(&tfull[st]);
        if (i + kScoreStages < tiles) {
          if (!mbar_wait_bounded(&empty[st], ph, &s_abort, kStatusScoreTimeout, kWaitLimit)) break;
          load_tile(i + kScoreStages);
        }
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ epilogue: thread = token lane of the tile
    const int tl = tid;                        // 0..127
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
    for (int i = 0; i < tiles; ++i) {
      const int st = i % kScoreStages;
      const uint32_t ph = (i / kScoreStages) & 1u;
      const int t = t_begin + i * kTokTile + tl;
      const int page = s_page[2 * i + (tl >> 6)];
      const bool valid = t < n && page >= 0;
      // the token's scale sits behind the page's 64 x 128 key bytes; requested before the wait
      const float scale = valid ? __ldg(reinterpret_cast<const float*>(cache + static_cast<size_t>(page) * kPageBytes +
                                                                       kPage * kDim + (tl & (kPage - 1)) * 4))
                                : 0.0f;
      if (!mbar_wait_bounded(&tfull[st], ph, &s_abort, kStatusScoreTimeout, kWaitLimit)) break;
      tc_fence_after();
      float acc = 0.0f;
#pragma unroll
      for (int c = 0; c < kHeads / 16; ++c) {
        uint32_t r[16];
        tmem_ld16(lane_addr + st * kHeads + c * 16, r);
        tmem_ld_wait();
        if (c == kHeads / 16 - 1) {            // the accumulator is in registers: hand it back
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tempty[st]);
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) acc = fmaf(s_w[c * 16 + j], fmaxf(__uint_as_float(r[j]) * scale, 0.0f), acc);
      }
      if (valid) scores[static_cast<size_t>(b) * max_ls + t] = acc;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 4) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kScoreStages * kHeads);
  }
  if (tid == 0 && s_abort != 0) atomicExch(status, s_abort);
}

// larger float <-> larger key (NaN aside); key 0 is below every score
__device__ __forceinline__ uint32_t score_key(float s) {
  const uint32_t u = __float_as_uint(s);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

constexpr int kSelectChunk = 16 * kSelectThreads;   // 16384 positions per select CTA of the first level

// The best min(2048, n) of n items, best first, left in s_item[0 .. 2047] (zeros behind them).  An item is
// (order-preserving key of the score << 32) | ~position, so items are distinct, "larger" means "better score, then
// lower position", and the cut is one exact item value: an 8-pass radix select over the 64 bits (one byte per
// pass, a histogram in shared memory filled through warp-aggregated increments, since most scores of a sequence
// share their top bytes), a compaction of the items at or above the cut, and a bitonic sort.
// get(j) returns the calling thread's j-th item (j < per_thread), 0 where it has none; without `sorted` the winners
// are left in arbitrary order.
template <typename Get>
__device__ __forceinline__ void select_best(Get get, int per_thread, int k, bool sorted, unsigned long long* s_item,
                                            unsigned long long* s_swap, int* s_hist, int* s_misc) {
  const int tid = threadIdx.x, lane = tid & 31;
  for (int i = tid; i < kKeep; i += kSelectThreads) s_item[i] = 0ull;
  unsigned long long prefix = 0ull, mask = 0ull;
  int want = k;
  for (int shift = 56; shift >= 0; shift -= 8) {
    if (tid < 256) s_hist[tid] = 0;
    __syncthreads();
    for (int j = 0; j < per_thread; ++j) {
      const unsigned long long it = get(j);
      const int bin = (it != 0ull && (it & mask) == prefix) ? static_cast<int>((it >> shift) & 255ull) : 256;
      if (shift >= 48) {      // sign and exponent: a handful of values, so the warp adds up its lanes first
        const unsigned peers = __match_any_sync(0xffffffffu, bin);
        if (bin < 256 && lane == __ffs(peers) - 1) atomicAdd(&s_hist[bin], __popc(peers));
      } else if (bin < 256) { // mantissa and position bytes: spread out, and fewer items match the prefix each pass
        atomicAdd(&s_hist[bin], 1);
      }
    }
    __syncthreads();
    // the byte value at which the count from the top reaches `want`: thread t < 256 owns value 255 - t, an
    // inclusive scan in thread order counts the items with that byte or a larger one
    int h = 0, incl = 0;
    if (tid < 256) {
      h = s_hist[255 - tid];
      incl = h;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += up;
      }
      if (lane == 31) s_misc[4 + (tid >> 5)] = incl;
    }
    __syncthreads();
    if (tid < 256) {
      for (int w = 0; w < (tid >> 5); ++w) incl += s_misc[4 + w];
      if (incl >= want && incl - h < want) {
        s_misc[0] = 255 - tid;
        s_misc[1] = incl - h;
        s_misc[3] = h;
      }
    }
    __syncthreads();
    prefix |= static_cast<unsigned long long>(s_misc[0]) << shift;
    mask |= 255ull << shift;
    want -= s_misc[1];
    const bool all_taken = s_misc[3] == want;   // every item that still matches the prefix is wanted: no more passes
    __syncthreads();
    if (all_taken) break;
  }
  const unsigned long long cut = prefix;       // the k-th best item (its leading bytes, when the passes stopped early)
  if (tid == 0) s_misc[2] = 0;
  __syncthreads();
  for (int j = 0; j < per_thread; ++j) {     // one counter increment per warp and round, not per winner
    const unsigned long long it = get(j);
    const bool win = it != 0ull && it >= cut;
    const unsigned winners = __ballot_sync(0xffffffffu, win);
    int base = 0;
    if (lane == 0 && winners != 0u) base = atomicAdd(&s_misc[2], __popc(winners));
    base = __shfl_sync(0xffffffffu, base, 0);
    if (win) s_item[base + __popc(winners & ((1u << lane) - 1u))] = it;
  }
  __syncthreads();
  if (sorted) {
    // Bitonic sort, descending, two adjacent items per thread in registers.  A compare-exchange at distance d pairs
    // item i with item i ^ d: d = 1 is inside the thread, d = 2 .. 32 pairs this thread with lane ^ (d / 2) of its
    // warp (shuffles, no barrier), d >= 64 goes through shared memory (two buffers in turn: one barrier per stage,
    // 15 stages instead of 66 barriers).  The first of a pair keeps the larger item where the block of `size`
    // items it lies in is sorted downwards ((i & size) == 0), the smaller one otherwise.
    unsigned long long e0 = s_item[2 * tid], e1 = s_item[2 * tid + 1];
    unsigned long long* buf = s_swap;
    unsigned long long* other = s_item;
    auto pick = [](unsigned long long a, unsigned long long c, bool keep_max) {
      return keep_max ? (a > c ? a : c) : (a < c ? a : c);
    };
    for (int size = 2; size <= kKeep; size <<= 1) {
      const bool desc = ((2 * tid) & size) == 0;
      for (int stride = size >> 1; stride >= 64; stride >>= 1) {
        buf[2 * tid] = e0;
        buf[2 * tid + 1] = e1;
        __syncthreads();
        const int half = stride >> 1;
        const int pt = tid ^ half;
        const bool keep_max = ((tid & half) == 0) == desc;
        e0 = pick(e0, buf[2 * pt], keep_max);
        e1 = pick(e1, buf[2 * pt + 1], keep_max);
        unsigned long long* t = buf; buf = other; other = t;
      }
      for (int stride = (size >> 1) < 32 ? (size >> 1) : 32; stride >= 2; stride >>= 1) {
        const int half = stride >> 1;
        const bool keep_max = ((tid & half) == 0) == desc;
        e0 = pick(e0, __shfl_xor_sync(0xffffffffu, e0, half), keep_max);
        e1 = pick(e1, __shfl_xor_sync(0xffffffffu, e1, half), keep_max);
      }
      const unsigned long long hi = e0 > e1 ? e0 : e1, lo = e0 > e1 ? e1 : e0;
      e0 = desc ? hi : lo;
      e1 = desc ? lo : hi;
    }
    __syncthreads();                             // every reader of either buffer is through
    s_item[2 * tid] = e0;
    s_item[2 * tid + 1] = e1;
  }
  __syncthreads();
}

__device__ __forceinline__ void write_tokens(const unsigned long long* s_item, int k, const int32_t* table_row,
                                             int32_t* o) {
  for (int i = threadIdx.x; i < kKeep; i += kSelectThreads) {
    int32_t tok = -1;
    if (i < k) {
      const int pos = static_cast<int>(~static_cast<uint32_t>(s_item[i] & 0xffffffffull));
      tok = table_row[pos / kPage] * kPage + pos % kPage;
    }
    o[i] = tok;
  }
}

// First level: CTA (c, b) takes positions [16384 c, 16384 c + 16384) of sequence b, 16 per thread in registers.
// A sequence of one chunk is finished here; of a longer one, each chunk's best 2048 items go to `cand` (every token
// of the sequence's best 2048 is among the best 2048 of its chunk).
__global__ void __launch_bounds__(kSelectThreads)
dsa_select_kernel(const float* __restrict__ scores, int max_ls, const int32_t* __restrict__ seq_lens,
                  const int32_t* __restrict__ block_table, int max_pages, unsigned long long* __restrict__ cand,
                  int32_t* __restrict__ out) {
  __shared__ unsigned long long s_item[kKeep];
  __shared__ unsigned long long s_swap[kKeep];   // second buffer of the sort
  __shared__ int s_hist[256];
  __shared__ int s_misc[12];
  const int b = blockIdx.y, c = blockIdx.x, tid = threadIdx.x;
  const int n = min(seq_lens[b], max_ls);
  const int chunks = (n + kSelectChunk - 1) / kSelectChunk;
  if (c >= max(chunks, 1)) return;
  int32_t* o = out + static_cast<size_t>(b) * kKeep;
  if (n == 0) {
    for (int i = tid; i < kKeep; i += kSelectThreads) o[i] = -1;
    return;
  }
  const int begin = c * kSelectChunk, len = min(kSelectChunk, n - begin);
  const float* sc = scores + static_cast<size_t>(b) * max_ls;
  unsigned long long mine[16];
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    const int i = begin + j * kSelectThreads + tid;
    mine[j] = (j * kSelectThreads + tid < len)
                  ? (static_cast<unsigned long long>(score_key(sc[i])) << 32) | (~static_cast<uint32_t>(i))
                  : 0ull;
  }
  const int k = min(kKeep, len);
  select_best([&](int j) { return mine[j]; }, 16, k, chunks == 1, s_item, s_swap, s_hist, s_misc);
  if (chunks == 1) {
    write_tokens(s_item, k, block_table + static_cast<size_t>(b) * max_pages, o);
  } else {
    unsigned long long* dst = cand + (static_cast<size_t>(b) * gridDim.x + c) * kKeep;
    for (int i = tid; i < kKeep; i += kSelectThreads) dst[i] = s_item[i];
  }
}

// Second level, sequences of more than one chunk: the best 2048 of the chunks' candidates.
__global__ void __launch_bounds__(kSelectThreads)
dsa_merge_kernel(const unsigned long long* __restrict__ cand, int max_chunks, int max_ls,
                 const int32_t* __restrict__ seq_lens, const int32_t* __restrict__ block_table, int max_pages,
                 int32_t* __restrict__ out) {
  __shared__ unsigned long long s_item[kKeep];
  __shared__ unsigned long long s_swap[kKeep];   // second buffer of the sort
  __shared__ int s_hist[256];
  __shared__ int s_misc[12];
  const int b = blockIdx.x, tid = threadIdx.x;
  const int n = min(seq_lens[b], max_ls);
  const int chunks = (n + kSelectChunk - 1) / kSelectChunk;
  if (chunks <= 1) return;                     // finished by the first level
  const unsigned long long* src = cand + static_cast<size_t>(b) * max_chunks * kKeep;
  const int total = chunks * kKeep;
  const int per_thread = (total + kSelectThreads - 1) / kSelectThreads;
  if (per_thread <= 16) {   // up to 8 chunks (131072 tokens): the candidates stay in registers over the eight passes
    unsigned long long mine[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const int i = j * kSelectThreads + tid;
      mine[j] = i < total ? src[i] : 0ull;
    }
    select_best([&](int j) { return mine[j]; }, 16, kKeep, true, s_item, s_swap, s_hist, s_misc);
  } else {
    select_best([&](int j) { const int i = j * kSelectThreads + tid; return i < total ? src[i] : 0ull; }, per_thread,
                kKeep, true, s_item, s_swap, s_hist, s_misc);
  }
  write_tokens(s_item, kKeep, block_table + static_cast<size_t>(b) * max_pages, out + static_cast<size_t>(b) * kKeep);
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
  unsigned long long* cand = nullptr;   // [batch][chunks][2048] items of the first selection level
  size_t cand_items = 0;
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
  {
    const size_t chunks_all = static_cast<size_t>((max_ls + kSelectChunk - 1) / kSelectChunk);
    const size_t need_items = chunks_all > 1 ? static_cast<size_t>(batch) * chunks_all * kKeep : 0;
    if (need_items > s.cand_items) {
      if (cudaDeviceSynchronize() != cudaSuccess) return fail(SYFI_DSA_ERR_CUDA, "device synchronisation failed");
      if (s.cand) cudaFree(s.cand);
      s.cand = nullptr;
      s.cand_items = 0;
      if (cudaMalloc(&s.cand, need_items * sizeof(unsigned long long)) != cudaSuccess)
        return fail(SYFI_DSA_ERR_CUDA, "out of device memory for the selection candidates");
      s.cand_items = need_items;
    }
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
  const int tiles = (max_ls + kTilesPerCta * kTokTile - 1) / (kTilesPerCta * kTokTile);
  dsa_score_kernel<<<dim3(tiles, batch), kScoreThreads, kScoreSmem, st>>>(
      tm_q, tm_k, static_cast<const uint8_t*>(k_index_cache_fp8), weights, seq_lens, block_table, max_pages, s.scores,
      max_ls, s.status);
  if (cudaGetLastError() != cudaSuccess) return fail(SYFI_DSA_ERR_CUDA, "score kernel launch failed");
  const int chunks = (max_ls + kSelectChunk - 1) / kSelectChunk;
  dsa_select_kernel<<<dim3(chunks, batch), kSelectThreads, 0, st>>>(s.scores, max_ls, seq_lens, block_table, max_pages,
                                                                    s.cand, topk_indices);
  if (cudaGetLastError() != cudaSuccess) return fail(SYFI_DSA_ERR_CUDA, "select kernel launch failed");
  if (chunks > 1) {
    dsa_merge_kernel<<<batch, kSelectThreads, 0, st>>>(s.cand, chunks, max_ls, seq_lens, block_table, max_pages,
                                                       topk_indices);
    if (cudaGetLastError() != cudaSuccess) return fail(SYFI_DSA_ERR_CUDA, "merge kernel launch failed");
  }
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
