// Grouped FP8 block-scale GEMMs of the MoE layer on CTA PAIRS (tcgen05 cta_group::2) for large batches.
//
// Same arithmetic and the same operands as grouped_gemm.cu (GEMM1 + SwiGLU + two-term requantisation
// replaces gemm_fp8_fp8_tcgen05_grouped_kernel / gemm_fp8_fp8_grouped_kernel / swiglu_quant_fp8_kernel
// of the reference, moe/solution/cuda/moe.cu:2194-2350, 1461-1627, 1631-1714; GEMM2 replaces
// gemm_fp8_fp8_fused_acc_grouped_kernel, moe.cu:1718-1887), with a work split made for experts that own
// hundreds of rows: the kernel is launched as clusters of two CTAs and every MMA spans the pair
// (M = 256, N up to 256), so one instruction issue feeds both tensor cores for 128 cycles and a K block
// costs each CTA 32 KB of operand traffic per 4.2 M MACs (the single-CTA kernel with 64-row token tiles
// moves 40 KB per 2.1 M MACs and is bound by the L2-to-SM rate).  Each CTA loads only its own operand
// halves; nothing is multicast.
//
//   mode 1, work item = (expert, 128 intermediate features, up to 256 token rows):
//     CTA 0 holds the up rows of W13, CTA 1 the gate rows of the same features (A operand, 128 rows
//     each); each CTA loads half of the token rows (B operand).  After the K loop CTA 0 owns
//     up[feature, token] and CTA 1 gate[feature, token]; the CTAs swap halves through distributed shared
//     memory so that each ends up with both values for half of the tokens, then SwiGLU, the per-row amax
//     over the 128 features and the two-term e4m3 requantisation run exactly as in the single-CTA kernel.
//   mode 2, work item = (expert, 256 output features, up to 128 token rows):
//     CTA r holds the W2 rows of feature tile 2 * pair + r; CTA 0 loads the hi term of the token rows,
//     CTA 1 the lo term, so the accumulator columns [0, n) are hi products and [n, 2n) lo products.
//
// Per K block (128 bytes of K) the raw e4m3 products accumulate in tensor memory (4 MMAs of K = 32) and
// are then promoted into f32 registers with activation scale x weight scale; tensor memory holds two
// accumulator slots of 256 columns, so the MMAs of block k + 1 run while block k is promoted.
//
// Roles per CTA: warp 0 = TMA producer (one thread), warp 1 = tensor memory owner and, in the pair's
// first CTA, the MMA issuer, warp 2 = scale warp (multiplies the block's activation scales with its
// weight scale into a small shared-memory ring, which takes a multiply per element off the promotion
// loop), warp 3 = cross-kernel bookkeeping (as in grouped_gemm.cu), warps 4..19 = promotion / epilogue
// (a warp reads one tensor-memory lane quarter; four warps share a quarter and split the columns).
// Barriers another CTA signals: full[] lives in the first CTA and counts the bytes of both CTAs' loads;
// empty[] and tfull[] exist in both CTAs and are signalled by one tcgen05.commit each; tempty[] lives
// in the first CTA and collects the arrivals of both CTAs' epilogue warps.
// Every wait is bounded; a CTA that gives up also raises the abort flag of its partner.
#include <cuda_fp16.h>

#include "moe_internal.h"
#include "ptx.cuh"

namespace syfi {

namespace {

constexpr int kWTile = 128 * 128;            // weight tile: 128 rows x 128 bytes of K
constexpr int kBox = 32 * 128;               // token-side TMA box: 32 rows x 128 bytes
constexpr int kStageBytes = 2 * kWTile;      // one K block: weight tile + up to 128 token-side rows
constexpr int kScaleRing = 8;                // K blocks of scale products in flight
constexpr int kScaleEntry = 256;             // floats per ring entry (one per accumulator token column)
constexpr int kEpiWarps = 16;
constexpr int kEpiThreads = 32 * kEpiWarps;
constexpr int kPairThreads = 128 + kEpiThreads;
constexpr int kSlotCols = 256;               // tensor-memory columns of one accumulator slot
constexpr int kSlots = 2;
constexpr int kPairTmemCols = 512;
constexpr long long kWaitLimit = 1ll << 31;  // cycles before a wait gives up (about a second)

template <int MODE> struct PairCfg {
  static constexpr int kKBlocks = MODE == 1 ? kHBlocks : kIBlocks;          // 56 / 16
  static constexpr int kFeatItems = MODE == 1 ? kInter / 128 : kHidden / 256;   // 16 / 28 per expert and token tile
  static constexpr int kTokTile = MODE == 1 ? 256 : 128;
  static constexpr int kStages = MODE == 1 ? 4 : 6;
  static constexpr int kXchgBytes = MODE == 1 ? 128 * 128 * 4 : 0;          // half of a CTA's accumulators
  static constexpr int kSmemBytes = 1024 + kStages * kStageBytes + kXchgBytes + kScaleRing * kScaleEntry * 4 +
                                    (MODE == 1 ? 4 * 128 * 4 + 2 * 128 * 4 : 0) + 8 * 48 +
                                    kMaxLocalExperts * static_cast<int>(sizeof(ExpertWork)) + 64;
  static_assert(kSmemBytes <= 232448, "exceeds the 227 KB of shared memory a CTA may use");
  static_assert(kStages % 2 == 0 && kKBlocks % 2 == 0, "stages are filled in K-adjacent pairs");
};

struct PairArgs {
  const ExpertWork* work;   // per expert: row_off, rows_pad (tile fields are recomputed for this kernel's tile)
  const int* meta;
  const float* act_scale;   // [K blocks][row_cap] scales of the token-side operand
  const float* w_scale;     // mode 1: [E][32][56], mode 2: [E][56][16]
  uint8_t* c_hi;            // mode 1 outputs
  uint8_t* c_lo;
  float* c_scale;           // [16][row_cap]
  float* o_rows;            // mode 2 output [row_cap][7168]
  int row_cap;
  int e_local;
  int* ready;               // [32] GEMM1 (CTA, item) completions per expert: mode 1 increments, mode 2 waits
  int* status;
  long long* stats;         // [grid][16] cycle counters per CTA (only written by SYFI_PAIR_STATS builds)
};

// Optional per-CTA cycle accounting (compile with -DSYFI_PAIR_STATS): where each role spends its time.
#ifdef SYFI_PAIR_STATS
#define ST_DECL long long st_t0 = 0; long long st_acc[4] = {0, 0, 0, 0}; (void)st_t0
#define ST_BEGIN() st_t0 = clock64()
#define ST_END(k) st_acc[k] += clock64() - st_t0
#define ST_WRITE(base, cond)                                                                     \
  do {                                                                                           \
    if ((cond) && p.stats != nullptr)                                                            \
      for (int k_ = 0; k_ < 4; ++k_) p.stats[blockIdx.x * 16 + (base) + k_] = st_acc[k_];        \
  } while (0)
#else
#define ST_DECL do { } while (0)
#define ST_BEGIN() do { } while (0)
#define ST_END(k) do { } while (0)
#define ST_WRITE(base, cond) do { } while (0)
#endif

struct PItem {
  int expert, ft, row_start, n;
};

// Work item w -> (expert, feature item, token tile): expert-major, then feature item, then token tile, so
// the clusters running side by side share weight tiles and token tiles through L2.
template <int FI, int NT>
__device__ __forceinline__ PItem decode_pair_item(const ExpertWork* s_work, int e_local, int w, int& e_hint) {
  PItem it{0, 0, 0, 0};
  for (int e = e_hint; e < e_local; ++e) {
    const ExpertWork ew = s_work[e];
    const int base = ew.tile_off * FI;
    if (w < base + ew.tiles * FI) {
      const int local = w - base;
      const int ti = local % ew.tiles;
      it.expert = e;
      it.ft = local / ew.tiles;
      it.row_start = ew.row_off + ti * NT;
      it.n = min(NT, ew.rows_pad - ti * NT);
      e_hint = e;
      return it;
    }
  }
  return it;
}

template <int MODE>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPairThreads, 1)
pair_gemm_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_b0,
                 const __grid_constant__ CUtensorMap tm_b1, const PairArgs p) {
  using C = PairCfg<MODE>;
  constexpr int G = C::kStages;
  constexpr int KB = C::kKBlocks;
  constexpr int FI = C::kFeatItems;
  constexpr int NT = C::kTokTile;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  float* s_xchg = reinterpret_cast<float*>(smem + G * kStageBytes);            // [128 cols][128 features] (mode 1)
  float* s_scale = reinterpret_cast<float*>(smem + G * kStageBytes + C::kXchgBytes);   // [kScaleRing][256]
  float* s_red = s_scale + kScaleRing * kScaleEntry;                           // [4][128] (mode 1)
  float* s_cs = s_red + (MODE == 1 ? 4 * 128 : 0);                             // [128] scale (mode 1)
  float* s_inv = s_cs + (MODE == 1 ? 128 : 0);                                 // [128] 1 / scale (mode 1)
  uint64_t* full = reinterpret_cast<uint64_t*>(s_inv + (MODE == 1 ? 128 : 0)); // [G]   first CTA's are used
  uint64_t* empty = full + G;                                                  // [G/2] per CTA
  uint64_t* tfull = empty + G / 2;                                             // [2]   per CTA
  uint64_t* tempty = tfull + kSlots;                                           // [2]   first CTA's are used
  uint64_t* sfull = tempty + kSlots;                                           // [8]   per CTA
  uint64_t* sempty = sfull + kScaleRing;                                       // [8]   per CTA
  uint64_t* xfull = sempty + kScaleRing;                                       // the partner's halves have arrived
  uint64_t* xfree = xfull + 1;                                                 // the partner has read what this CTA sent
  ExpertWork* s_work = reinterpret_cast<ExpertWork*>(xfree + 1);
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(s_work + kMaxLocalExperts);
  volatile int* s_abort = reinterpret_cast<volatile int*>(s_tmem + 1);
  int* s_done = reinterpret_cast<int*>(s_tmem + 2);   // mode 1: epilogue warps done with an item (running total); mode 2: items cleared
  int* s_meta = reinterpret_cast<int*>(s_tmem + 3);   // [2] token tiles, active experts

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const uint32_t peer = rank ^ 1u;
  const uint32_t peer_abort = mapa_u32(smem_u32(const_cast<int*>(s_abort)), peer);

  if (threadIdx.x == 0) {
    for (int i = 0; i < G; ++i) mbar_init(&full[i], 1);
    for (int i = 0; i < G / 2; ++i) mbar_init(&empty[i], 1);
    for (int i = 0; i < kSlots; ++i) { mbar_init(&tfull[i], 1); mbar_init(&tempty[i], 2 * kEpiWarps); }
    for (int i = 0; i < kScaleRing; ++i) { mbar_init(&sfull[i], 1); mbar_init(&sempty[i], kEpiWarps); }
    mbar_init(xfull, kEpiWarps);
    mbar_init(xfree, kEpiWarps);
    *s_abort = 0;
    *s_done = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tm_w);
    tma_prefetch_desc(&tm_b0);
    if (MODE == 2) tma_prefetch_desc(&tm_b1);
  }
  // both CTAs' barriers exist before anyone signals across the pair
  cluster_sync_all();
  if (warp == 1) {
    tmem_alloc_pair(s_tmem, kPairTmemCols);
    tmem_relinquish_pair();
  }
  // See grouped_gemm.cu: mode 1 waits for the kernels before it as a whole; mode 2 is released expert by
  // expert through p.ready (its CTAs only exist once every GEMM1 CTA has started, and GEMM1 waits for
  // nothing, so the overlap cannot deadlock).
  if (MODE == 1) pdl_wait();
  pdl_trigger();
  if (warp == 3) {
    // this kernel's own tile table: token tiles of NT rows per expert and their prefix sums
    ExpertWork ew = (lane < p.e_local) ? p.work[lane] : ExpertWork{0, 0, 0, 0};
    const int tiles = (ew.rows_pad + NT - 1) / NT;
    int incl = tiles;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d) incl += v;
    }
    ew.tiles = tiles;
    ew.tile_off = incl - tiles;
    s_work[lane] = ew;
    if (lane == 31) s_meta[0] = incl;
    if (lane == 0) s_meta[1] = p.meta[3];
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // the partner's tensor memory is allocated too
  tc_fence_after();
  const uint32_t tmem_base = *s_tmem;
  const int total = s_meta[0] * FI;                 // work items (per cluster)
  const int n_clusters = static_cast<int>(gridDim.x >> 1);
  const int cluster_id = static_cast<int>(blockIdx.x >> 1);
  const int my_items = cluster_id < total ? (total - cluster_id + n_clusters - 1) / n_clusters : 0;
  auto item_of = [&](int i) { return cluster_id + i * n_clusters; };

  if (warp < 4) {
    if (warp == 0) {
      // ------------------------------------------------------------ TMA producer (one thread per CTA)
      if (lane == 0) {
        const uint64_t pol_w = s_meta[0] > s_meta[1] ? l2_policy_evict_last() : l2_policy_evict_first();
        const uint64_t pol_b = l2_policy_evict_last();
        uint32_t full0[G];                     // the first CTA's full barriers as cluster addresses
#pragma unroll
        for (int i = 0; i < G; ++i) full0[i] = mapa_u32(smem_u32(&full[i]), 0);
        uint32_t it = 0, g = 0, ph = 0;        // stage pairs armed, next stage, phase of its empty barrier
        uint32_t n_items = 0;
        int e_hint = 0;
        bool alive = true;
        ST_DECL;
        const long long st_start = clock64();
        (void)st_start;
        for (int i = 0; i < my_items && alive; ++i) {
          const PItem im = decode_pair_item<FI, NT>(s_work, p.e_local, item_of(i), e_hint);
          int nh, my_row, wrow;
          const CUtensorMap* mb;
          if (MODE == 1) {
            nh = im.n >> 1;                                      // this CTA's half of the token rows
            my_row = im.row_start + static_cast<int>(rank) * nh;
            wrow = im.expert * 2 * kInter + static_cast<int>(rank) * kInter + im.ft * 128;
            mb = &tm_b0;
          } else {
            nh = im.n;                                           // all rows of one term
            my_row = im.row_start;
            wrow = im.expert * kHidden + (2 * im.ft + static_cast<int>(rank)) * 128;
            mb = rank == 0 ? &tm_b0 : &tm_b1;
          }
          const int boxes = (nh + 31) >> 5;
          const uint32_t stage_tx = 2u * static_cast<uint32_t>(kWTile + boxes * kBox);   // both CTAs' bytes
          if (MODE == 2) {
            // the item's expert must have left GEMM1 (the helper warp checks and counts cleared items)
            if (*reinterpret_cast<volatile int*>(s_done) <= static_cast<int>(n_items)) {
              const long long t0 = clock64();
              while (*reinterpret_cast<volatile int*>(s_done) <= static_cast<int>(n_items)) {
                if (*s_abort != 0) { alive = false; break; }
                if (clock64() - t0 > kWaitLimit) {
                  *s_abort = kStatusDependencyTimeout;
                  st_cluster_u32(peer_abort, kStatusDependencyTimeout);
                  alive = false;
                  break;
                }
              }
              if (!alive) break;
            }
            __threadfence_block();
            ++n_items;
          }
          for (int kb = 0; kb < KB; kb += 2) {
            ST_BEGIN();
            if (!mbar_wait_bounded_tell(&empty[g >> 1], ph ^ 1u, s_abort, peer_abort, kStatusWaitTimeoutProducer,
                                        kWaitLimit)) { alive = false; break; }
            ST_END(0);
            if (rank == 0) {
              mbar_arrive_expect_tx(&full[g], stage_tx);
              mbar_arrive_expect_tx(&full[g + 1], stage_tx);
            }
            // boxes that continue each other along K are issued back to back (a row's 256 contiguous
            // bytes are served by L2 far faster than two separate 128-byte visits)
            uint8_t* st0 = smem + g * kStageBytes;
            uint8_t* st1 = st0 + kStageBytes;
            const int x0 = kb * 128;
            tma_load_2d_pair(st0, &tm_w, full0[g], x0, wrow, pol_w);
            tma_load_2d_pair(st1, &tm_w, full0[g + 1], x0 + 128, wrow, pol_w);
            for (int b = 0; b < boxes; ++b) {
              tma_load_2d_pair(st0 + kWTile + b * kBox, mb, full0[g], x0, my_row + 32 * b, pol_b);
              tma_load_2d_pair(st1 + kWTile + b * kBox, mb, full0[g + 1], x0 + 128, my_row + 32 * b, pol_b);
            }
            ++it;
            g += 2;
            if (g == G) { g = 0; ph ^= 1u; }
          }
        }
#ifdef SYFI_PAIR_STATS
        st_acc[1] = clock64() - st_start;
#endif
        ST_WRITE(0, true);
        // drain: the first CTA's full barriers count both CTAs' bytes, and no CTA of the pair leaves
        // before the final cluster barrier, so waiting there covers the partner's loads as well
        if (rank == 0) {
          const uint32_t armed = 2 * it;
          const uint32_t first = armed > static_cast<uint32_t>(G) ? armed - G : 0;
          for (uint32_t i = first; i < armed; ++i)
            mbar_wait_bounded_tell(&full[i % G], (i / G) & 1, s_abort, peer_abort, kStatusWaitTimeoutProducer, 1ll << 28);
        }
      }
      __syncwarp();
    } else if (warp == 1) {
      // --------------------------------------------------------------- MMA issuer (one thread of the pair)
      if (lane == 0 && rank == 0) {
        uint32_t g = 0, ph = 0, sl = 0, sph = 0;   // stage / phase, accumulator slot / phase
        int e_hint = 0;
        bool alive = true;
        ST_DECL;
        const long long st_start = clock64();
        (void)st_start;
        for (int i = 0; i < my_items && alive; ++i) {
          const PItem im = decode_pair_item<FI, NT>(s_work, p.e_local, item_of(i), e_hint);
          const uint32_t idesc = umma_idesc_e4m3_m256(MODE == 1 ? static_cast<uint32_t>(im.n) : 2u * im.n);
          for (int kb = 0; kb < KB; ++kb) {
            ST_BEGIN();
            if (!mbar_wait_bounded_tell(&full[g], ph, s_abort, peer_abort, kStatusWaitTimeoutMma, kWaitLimit)) { alive = false; break; }
            ST_END(0);
            ST_BEGIN();
            if (!mbar_wait_bounded_tell(&tempty[sl], sph ^ 1u, s_abort, peer_abort, kStatusWaitTimeoutMma, kWaitLimit)) { alive = false; break; }
            ST_END(1);
            tc_fence_after();
            const uint32_t sb = smem_u32(smem + g * kStageBytes);
            const uint64_t a0 = umma_smem_desc_sw128(sb);
            const uint64_t b0 = umma_smem_desc_sw128(sb + kWTile);
            const uint32_t d0 = tmem_base + sl * kSlotCols;
#pragma unroll
            for (int k4 = 0; k4 < 4; ++k4) umma_f8_pair(d0, a0 + 2 * k4, b0 + 2 * k4, idesc, k4 > 0 ? 1u : 0u);
            if (g & 1u) umma_commit_pair(&empty[g >> 1], 3);
            umma_commit_pair(&tfull[sl], 3);
            if (++g == G) { g = 0; ph ^= 1u; }
            if (++sl == kSlots) { sl = 0; sph ^= 1u; }
          }
        }
#ifdef SYFI_PAIR_STATS
        st_acc[2] = clock64() - st_start;
#endif
        ST_WRITE(4, true);
      }
      __syncwarp();
    } else if (warp == 2) {
      // --------------------------------------------------------------- scale warp
      // entry s of the ring holds, for one K block, act_scale[row, kb] * w_scale[kb] of every token column
      // of the item; lane l serves columns 4 l .. 4 l + 3 (and 128 + 4 l .. in mode 1)
      constexpr int kBatch = 4;
      uint32_t s = 0, sp = 0;
      uint32_t n_items = 0;
      int e_hint = 0;
      bool alive = true;
      for (int i = 0; i < my_items && alive; ++i) {
        const PItem im = decode_pair_item<FI, NT>(s_work, p.e_local, item_of(i), e_hint);
        if (MODE == 2) {
          if (*reinterpret_cast<volatile int*>(s_done) <= static_cast<int>(n_items)) {
            const long long t0 = clock64();
            while (*reinterpret_cast<volatile int*>(s_done) <= static_cast<int>(n_items)) {
              if (*s_abort != 0 || clock64() - t0 > kWaitLimit) { alive = false; break; }
            }
          }
          alive = __all_sync(0xffffffffu, alive);
          if (!alive) break;
          __threadfence_block();
          ++n_items;
        }
        const float* wsp = MODE == 1
            ? p.w_scale + (static_cast<size_t>(im.expert) * 32 + rank * 16 + im.ft) * kHBlocks
            : p.w_scale + (static_cast<size_t>(im.expert) * kHBlocks + 2 * im.ft + rank) * kIBlocks;
        const float ws_a = lane < KB ? __ldg(wsp + lane) : 0.0f;
        const float ws_b = (MODE == 1 && 32 + lane < KB) ? __ldg(wsp + 32 + lane) : 0.0f;
        const int col = 4 * lane;
        const bool v0 = col < im.n, v1 = MODE == 1 && 128 + col < im.n;
        const float* src = p.act_scale + im.row_start + col;
        for (int kb0 = 0; kb0 < KB && alive; kb0 += kBatch) {
          float4 a[kBatch], b[kBatch];
#pragma unroll
          for (int k = 0; k < kBatch; ++k) {
            const float* sp0 = src + static_cast<size_t>(kb0 + k) * p.row_cap;
            // plain loads: in mode 2 these scales were written by GEMM1, which may still be running
            a[k] = v0 ? ld_global_f32x4(sp0) : make_float4(0.f, 0.f, 0.f, 0.f);
            if (MODE == 1) b[k] = v1 ? ld_global_f32x4(sp0 + 128) : make_float4(0.f, 0.f, 0.f, 0.f);
          }
#pragma unroll
          for (int k = 0; k < kBatch; ++k) {
            const int kb = kb0 + k;
            const float ws = __shfl_sync(0xffffffffu, kb < 32 ? ws_a : ws_b, kb & 31);
            bool ok = mbar_wait_bounded_tell(&sempty[s], sp ^ 1u, s_abort, peer_abort, kStatusWaitTimeoutProducer, kWaitLimit);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) { alive = false; break; }
            float* dst = s_scale + s * kScaleEntry + col;
            *reinterpret_cast<float4*>(dst) = make_float4(a[k].x * ws, a[k].y * ws, a[k].z * ws, a[k].w * ws);
            if (MODE == 1)
              *reinterpret_cast<float4*>(dst + 128) = make_float4(b[k].x * ws, b[k].y * ws, b[k].z * ws, b[k].w * ws);
            __syncwarp();
            if (lane == 0) mbar_arrive(&sfull[s]);
            if (++s == kScaleRing) { s = 0; sp ^= 1u; }
          }
        }
      }
    } else {
      // ------------------------------------------------ publisher (mode 1) / dependency helper (mode 2)
      // Same hand-off as in grouped_gemm.cu.  Every CTA of a pair counts its own half of an item, so an
      // expert is complete at 2 * 16 * (its 256-row token tiles).
      if (MODE == 1 && lane == 0) {
        int done_target = 0, e_hint = 0;
        for (int i = 0; i < my_items; ++i) {
          const PItem im = decode_pair_item<FI, NT>(s_work, p.e_local, item_of(i), e_hint);
          done_target += kEpiWarps;
          const long long t0 = clock64();
          bool seen = true;
          while (*reinterpret_cast<volatile int*>(s_done) < done_target) {
            if (*s_abort != 0 || clock64() - t0 > (1ll << 33)) { seen = false; break; }
            __nanosleep(200);
          }
          if (!seen || *s_abort != 0) break;          // a failed item is never published
          __threadfence();
          fence_proxy_async_all();
          red_release_gpu_add(p.ready + im.expert, 1);
        }
      }
      if (MODE == 2 && lane == 0) {
        int cleared = 0, ready_expert = -1, e_hint = 0;
        for (int i = 0; i < my_items; ++i) {
          const PItem im = decode_pair_item<FI, NT>(s_work, p.e_local, item_of(i), e_hint);
          if (im.expert != ready_expert) {
            const int rows_pad = s_work[im.expert].rows_pad;
            const int need = 2 * (kInter / 128) * ((rows_pad + PairCfg<1>::kTokTile - 1) / PairCfg<1>::kTokTile);
            const long long t0 = clock64();
            bool seen = true;
            while (ld_acquire_gpu(p.ready + im.expert) < need) {
              if (*s_abort != 0) { seen = false; break; }
              if (clock64() - t0 > kWaitLimit) {
                *s_abort = kStatusDependencyTimeout;
                st_cluster_u32(peer_abort, kStatusDependencyTimeout);
                seen = false;
                break;
              }
              __nanosleep(100);
            }
            if (!seen) break;
            fence_proxy_async_all();
            ready_expert = im.expert;
          }
          ++cleared;
          __threadfence_block();
          *reinterpret_cast<volatile int*>(s_done) = cleared;
        }
      }
      __syncwarp();
    }
  } else {
    // ------------------------------------------------ promotion + epilogue warps
    // A thread owns one feature (tensor-memory lane) and CN token columns of every accumulator slot.
    constexpr int CN = MODE == 1 ? 64 : 32;       // token columns per thread
    const int q = warp & 3;                       // lane quarter this warp may read
    const int grp = (warp - 4) >> 2;              // which quarter of the columns
    const int c0 = grp * CN;                      // first token column of this thread
    const int f = q * 32 + lane;                  // feature inside the CTA's 128-row tile
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    const uint32_t tempty0[kSlots] = {mapa_u32(smem_u32(&tempty[0]), 0), mapa_u32(smem_u32(&tempty[1]), 0)};
    const uint32_t peer_xfull = mapa_u32(smem_u32(xfull), peer);
    const uint32_t peer_xfree = mapa_u32(smem_u32(xfree), peer);
    const uint32_t peer_xchg = mapa_u32(smem_u32(s_xchg), peer);
    uint32_t sl = 0, sph = 0;                     // accumulator slot and its phase
    uint32_t s = 0, sp = 0;                       // scale ring entry and its phase
    uint32_t xph = 0;                             // phase of the exchange barriers (mode 1)
    bool ok = true;
    int e_hint = 0;
    const uint64_t inv_ratio = f32x2_pack(1.0f / kLoRatio, 1.0f / kLoRatio);
    ST_DECL;
    const long long st_start = clock64();
    (void)st_start;
    (void)inv_ratio; (void)xph; (void)peer_xfull; (void)peer_xfree; (void)peer_xchg; (void)f;

    for (int i = 0; i < my_items; ++i) {
      const PItem im = decode_pair_item<FI, NT>(s_work, p.e_local, item_of(i), e_hint);
      const int n = ok ? im.n : 0;
      uint64_t acc[CN / 2];
#pragma unroll
      for (int j = 0; j < CN / 2; ++j) acc[j] = 0ull;

      for (int kb = 0; kb < KB && ok; ++kb) {
        ST_BEGIN();
        if (!mbar_wait_bounded_tell(&tfull[sl], sph, s_abort, peer_abort, kStatusWaitTimeoutEpilogue, kWaitLimit)) { ok = false; break; }
        ST_END(0);
        tc_fence_after();
        if (!mbar_wait_bounded_tell(&sfull[s], sp, s_abort, peer_abort, kStatusWaitTimeoutEpilogue, kWaitLimit)) { ok = false; break; }
#ifdef SYFI_PAIR_STATS
        const long long st_p0 = clock64();
#endif
        const float* sc = s_scale + s * kScaleEntry + c0;
        const uint32_t t0 = lane_addr + sl * kSlotCols + c0;
#pragma unroll
        for (int ch = 0; ch < CN / 16; ++ch) {
          if (c0 + ch * 16 < n) {
            const ulonglong2* sp4 = reinterpret_cast<const ulonglong2*>(sc + ch * 16);
            if (MODE == 1) {
              uint32_t r[16];
              ST_BEGIN();
#ifndef PAIR_NO_LD
              tmem_ld16(t0 + ch * 16, r);
#else
#pragma unroll
              for (int z = 0; z < 16; ++z) r[z] = t0 + z;
#endif
              const ulonglong2 s0 = sp4[0], s1 = sp4[1], s2 = sp4[2], s3 = sp4[3];
              tmem_ld_wait();
              ST_END(1);
#ifdef PAIR_NO_FMA
              if (r[0] == 0x12345678u) acc[ch * 8] = s0.x;
#else
              acc[ch * 8 + 0] = f32x2_fma(f32x2_pack_bits(r[0], r[1]), s0.x, acc[ch * 8 + 0]);
              acc[ch * 8 + 1] = f32x2_fma(f32x2_pack_bits(r[2], r[3]), s0.y, acc[ch * 8 + 1]);
              acc[ch * 8 + 2] = f32x2_fma(f32x2_pack_bits(r[4], r[5]), s1.x, acc[ch * 8 + 2]);
              acc[ch * 8 + 3] = f32x2_fma(f32x2_pack_bits(r[6], r[7]), s1.y, acc[ch * 8 + 3]);
              acc[ch * 8 + 4] = f32x2_fma(f32x2_pack_bits(r[8], r[9]), s2.x, acc[ch * 8 + 4]);
              acc[ch * 8 + 5] = f32x2_fma(f32x2_pack_bits(r[10], r[11]), s2.y, acc[ch * 8 + 5]);
              acc[ch * 8 + 6] = f32x2_fma(f32x2_pack_bits(r[12], r[13]), s3.x, acc[ch * 8 + 6]);
              acc[ch * 8 + 7] = f32x2_fma(f32x2_pack_bits(r[14], r[15]), s3.y, acc[ch * 8 + 7]);
#endif
            } else {
              uint32_t r[16], l[16];
              tmem_ld16(t0 + ch * 16, r);                 // hi products
              tmem_ld16(t0 + im.n + ch * 16, l);          // lo products of the same token columns
              const ulonglong2 s0 = sp4[0], s1 = sp4[1], s2 = sp4[2], s3 = sp4[3];
              tmem_ld_wait();
              const uint64_t sv[8] = {s0.x, s0.y, s1.x, s1.y, s2.x, s2.y, s3.x, s3.y};
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const uint64_t v = f32x2_fma(f32x2_pack_bits(l[2 * j], l[2 * j + 1]), inv_ratio,
                                             f32x2_pack_bits(r[2 * j], r[2 * j + 1]));
                acc[ch * 8 + j] = f32x2_fma(v, sv[j], acc[ch * 8 + j]);
              }
            }
          }
        }
        // the slot and the scale entry go back (the values are in registers)
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
#ifdef PAIR_RELEASE_ARRIVE
          mbar_arrive_cluster(tempty0[sl]);
#else
          mbar_arrive_cluster_relaxed(sl == 0 ? tempty0[0] : tempty0[1]);
#endif
          mbar_arrive(&sempty[s]);
        }
        if (++sl == kSlots) { sl = 0; sph ^= 1u; }
        if (++s == kScaleRing) { s = 0; sp ^= 1u; }
#ifdef SYFI_PAIR_STATS
        st_acc[2] += clock64() - st_p0;
#endif
      }
      const int n_out = ok ? n : 0;               // a failed item stores nothing
      ST_BEGIN();

      if (MODE == 1) {
        // ---- swap halves with the partner: this CTA keeps columns c0 + 32 rank .. + 31 of every thread's
        // 64 and sends the other 32; the same thread of the partner CTA does the opposite, so each CTA
        // ends up with up AND gate of 128 features x (its 128 of the 256 token columns).
        if (rank == 1) {
#pragma unroll
          for (int j = 0; j < 16; ++j) { const uint64_t t = acc[j]; acc[j] = acc[j + 16]; acc[j + 16] = t; }
        }
        // now acc[0..15] = kept columns, acc[16..31] = columns to send
        const int keep0 = c0 + 32 * static_cast<int>(rank);      // first kept token column of the item
        const int send0 = c0 + 32 * static_cast<int>(peer);
        float mine[32], other[32];
#pragma unroll
        for (int j = 0; j < 16; ++j) f32x2_unpack(acc[j], mine[2 * j], mine[2 * j + 1]);
        if (ok && !mbar_wait_bounded_pair(xfree, xph ^ 1u, s_abort, peer_abort, kStatusWaitTimeoutEpilogue, kWaitLimit)) ok = false;
        if (ok) {
          const uint32_t dst = peer_xchg + static_cast<uint32_t>((grp * 32) * 128 + f) * 4u;
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if (send0 + ((2 * j) & ~15) < n_out) {
              float a, b;
              f32x2_unpack(acc[16 + j], a, b);
              st_cluster_f32(dst + static_cast<uint32_t>(2 * j) * 512u, a);
              st_cluster_f32(dst + static_cast<uint32_t>(2 * j + 1) * 512u, b);
            }
          }
          fence_acq_rel_cluster();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(peer_xfull);
          if (!mbar_wait_bounded_pair(xfull, xph, s_abort, peer_abort, kStatusWaitTimeoutEpilogue, kWaitLimit)) ok = false;
        }
        const int n_keep = ok ? n_out : 0;
#pragma unroll
        for (int j = 0; j < 32; ++j)
          other[j] = (keep0 + (j & ~15) < n_keep) ? s_xchg[(grp * 32 + j) * 128 + f] : 0.0f;
        if (ok) {
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(peer_xfree);
        }
        xph ^= 1u;

        // ---- SwiGLU, per-row amax over the 128 features, two-term requantisation (as in grouped_gemm.cu)
        const int slot0 = grp * 32;               // this thread's columns in the CTA's 128 kept columns
        const int bar_id = 1 + grp;
#pragma unroll
        for (int jb = 0; jb < 32; jb += 16) {
          if (keep0 + jb < n_keep) {
            float mx[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const float up = rank == 0 ? mine[jb + j] : other[jb + j];
              const float gt = rank == 0 ? other[jb + j] : mine[jb + j];
              const float cv = gt * __fdividef(1.0f, 1.0f + __expf(-gt)) * up;
              mine[jb + j] = cv;
              mx[j] = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(fabsf(cv))));
            }
            if (lane == 0) {
              float4* dst = reinterpret_cast<float4*>(s_red + q * 128 + slot0 + jb);
#pragma unroll
              for (int j = 0; j < 4; ++j) dst[j] = make_float4(mx[4 * j], mx[4 * j + 1], mx[4 * j + 2], mx[4 * j + 3]);
            }
          }
        }
        named_bar_sync(bar_id, 128);
        if (q == 0 && keep0 + lane < n_keep) {
          const int sl_i = slot0 + lane;
          const float amax = fmaxf(fmaxf(s_red[sl_i], s_red[128 + sl_i]), fmaxf(s_red[256 + sl_i], s_red[384 + sl_i]));
          const float scv = fmaxf(amax * (1.0f / 448.0f), 1e-12f);
          s_cs[sl_i] = scv;
          s_inv[sl_i] = 1.0f / scv;
          p.c_scale[static_cast<size_t>(im.ft) * p.row_cap + im.row_start + keep0 + lane] = scv;
        }
        named_bar_sync(bar_id, 128);
        const int qrow = lane & 3;                // which of four rows this lane stores after the transpose
        const size_t qoff = static_cast<size_t>(im.ft) * 128 + q * 32 + (lane >> 2) * 4;
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
          if (keep0 + (j & ~15) < n_keep) {
            uint32_t hp = 0, lp = 0;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const int c = j + 2 * h;
              const float sc0 = s_cs[slot0 + c], sc1 = s_cs[slot0 + c + 1];
              const float in0 = s_inv[slot0 + c], in1 = s_inv[slot0 + c + 1];
              const float v0 = mine[c], v1 = mine[c + 1];
              const uint16_t hh = cvt_e4m3x2(v0 * in0, v1 * in1);
              const float2 hb = e4m3x2_to_float2(hh);
              const float r0 = fmaf(-hb.x, sc0, v0), r1 = fmaf(-hb.y, sc1, v1);
              const uint16_t ll = cvt_e4m3x2(r0 * in0 * kLoRatio, r1 * in1 * kLoRatio);
              hp |= static_cast<uint32_t>(hh) << (16 * h);
              lp |= static_cast<uint32_t>(ll) << (16 * h);
            }
            hp = quad_transpose_bytes(hp, lane);
            lp = quad_transpose_bytes(lp, lane);
            const size_t off = static_cast<size_t>(im.row_start + keep0 + j + qrow) * kInter + qoff;
            *reinterpret_cast<uint32_t*>(p.c_hi + off) = hp;
            *reinterpret_cast<uint32_t*>(p.c_lo + off) = lp;
          }
        }
        named_bar_sync(bar_id, 128);              // s_red / s_cs of this group are free for the next item
        __threadfence_block();
        __syncwarp();
        if (lane == 0) atomicAdd(s_done, 1);
      } else {
        float out[CN];
#pragma unroll
        for (int j = 0; j < CN / 2; ++j) f32x2_unpack(acc[j], out[2 * j], out[2 * j + 1]);
        const int qrow = lane & 3;
        float* o = p.o_rows + static_cast<size_t>(im.row_start + c0 + qrow) * kHidden +
                   (2 * im.ft + static_cast<int>(rank)) * 128 + q * 32 + (lane >> 2) * 4;
#pragma unroll
        for (int j = 0; j < CN; j += 4) {
          if (c0 + j < n_out) {
            float a0 = out[j], a1 = out[j + 1], a2 = out[j + 2], a3 = out[j + 3];
            quad_transpose_f32(a0, a1, a2, a3, lane);   // now: row c0 + j + qrow, four adjacent features
            *reinterpret_cast<float4*>(o + static_cast<size_t>(j) * kHidden) = make_float4(a0, a1, a2, a3);
          }
        }
      }
      ST_END(3);
    }
    ST_WRITE(8, warp == 4 && lane == 0);
#ifdef SYFI_PAIR_STATS
    if (warp == 4 && lane == 0 && p.stats != nullptr) p.stats[blockIdx.x * 16 + 12] = clock64() - st_start;
#endif
  }

  // no CTA of the pair may leave (or free tensor memory the partner's MMAs write) before both are done
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kPairTmemCols);
  }
  if (threadIdx.x == 0 && *s_abort != 0) atomicExch(p.status, *s_abort);
}

template <int MODE>
cudaError_t launch_pair(const PairGemmLaunch& g, const PairArgs& a, int num_sms, cudaStream_t st) {
  const int grid = num_sms & ~1;   // whole pairs
  return launch_dependent(pair_gemm_kernel<MODE>, dim3(grid), dim3(kPairThreads),
                          static_cast<size_t>(PairCfg<MODE>::kSmemBytes), st, g.tm_w, g.tm_b0, g.tm_b1, a);
}

}  // namespace

cudaError_t pair_gemm_set_attributes() {
  cudaError_t e = cudaFuncSetAttribute(pair_gemm_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       PairCfg<1>::kSmemBytes);
  if (e != cudaSuccess) return e;
  return cudaFuncSetAttribute(pair_gemm_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              PairCfg<2>::kSmemBytes);
}

cudaError_t launch_pair_gemm1(const PairGemmLaunch& g, const float* w13_scale, int e_local, const Workspace& ws,
                              int num_sms, cudaStream_t st) {
  PairArgs a{ws.work, ws.meta, ws.a_scale, w13_scale, ws.c_hi, ws.c_lo, ws.c_scale, nullptr, ws.row_cap, e_local,
             ws.ready, ws.status, ws.trace};
  return launch_pair<1>(g, a, num_sms, st);
}

cudaError_t launch_pair_gemm2(const PairGemmLaunch& g, const float* w2_scale, int e_local, const Workspace& ws,
                              int num_sms, cudaStream_t st) {
  PairArgs a{ws.work, ws.meta, ws.c_scale, w2_scale, nullptr, nullptr, nullptr, ws.o_rows, ws.row_cap, e_local,
             ws.ready, ws.status, ws.trace + 4096};
  return launch_pair<2>(g, a, num_sms, st);
}

}  // namespace syfi
