// Grouped FP8 block-scale GEMMs of the MoE layer on CTA PAIRS (tcgen05 cta_group::2) for large batches.
//
// Same arithmetic and the same operands as grouped_gemm.cu (GEMM1 + SwiGLU + two-term requantisation
// replaces gemm_fp8_fp8_tcgen05_grouped_kernel / gemm_fp8_fp8_grouped_kernel / swiglu_quant_fp8_kernel
// of the reference, moe/solution/cuda/moe.cu:2194-2350, 1461-1627, 1631-1714; GEMM2 replaces
// gemm_fp8_fp8_fused_acc_grouped_kernel, moe.cu:1718-1887), with a work split made for experts that own
// hundreds of rows: the kernel is launched as clusters of two CTAs and every MMA spans the pair
// (M = 256, N = 256), so one instruction issue feeds both tensor cores for 128 cycles and a K block
// costs each CTA 32 KB of operand traffic per 4.2 M MACs (the single-CTA kernel with 64-row token tiles
// moves 40 KB per 2.1 M MACs and is bound by the L2-to-SM rate).  Each CTA loads only its own operand
// halves; nothing is multicast.
//
//   mode 1 (GEMM1), work item = (expert, 128 intermediate features, up to 256 token rows), TOKEN-MAJOR:
//     the token rows are the M operand (CTA r holds rows 128 r .. 128 r + 127 of the tile), the weights
//     the N operand (CTA 0 loads the 128 up rows of W13, CTA 1 the 128 gate rows of the same features).
//     A tensor-memory lane is a token, columns 0..127 are its up values and 128..255 its gate values:
//     the block scale of a lane is ONE number per K block (activation scale of the token x weight scale),
//     SwiGLU needs no exchange, and the row's amax over the 128 features is a reduction inside four
//     threads.  (With features on the lanes, as in grouped_gemm.cu, every thread needs the scale of each
//     of its 64 token columns per K block; filling registers with those through the shared-memory pipe,
//     128 bytes per clock, costs ~1000 cycles per K block and SM against 512 cycles of MMA.)
//   mode 2 (GEMM2), work item = (expert, 256 output features, up to 128 token rows), feature-major:
//     CTA r holds the W2 rows of feature tile 2 * pair + r (M operand); CTA 0 loads the hi term of the
//     token rows, CTA 1 the lo term (N operand), so accumulator columns [0, n) are hi products and
//     [n, 2n) lo products.
//
// Per K block (128 bytes of K) the raw e4m3 products accumulate in tensor memory (4 MMAs of K = 32) and
// are then promoted into f32 registers with activation scale x weight scale; tensor memory holds two
// accumulator slots of 256 columns, so the MMAs of block k + 1 run while block k is promoted.
//
// Roles per CTA: warp 0 = TMA producer (one thread), warp 1 = tensor memory owner and, in the pair's
// first CTA, the MMA issuer, warp 2 = scale warp (mode 1: fetches the weight scales of the next item;
// mode 2: multiplies a K block's activation scales with its weight scale into a shared-memory ring),
// warp 3 = cross-kernel bookkeeping (as in grouped_gemm.cu), warps 4..19 = promotion / epilogue
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

constexpr int kTile = 128 * 128;             // operand tile: 128 rows x 128 bytes of K
constexpr int kBox = 32 * 128;               // token-side TMA box: 32 rows x 128 bytes
constexpr int kStageBytes = 2 * kTile;       // one K block: M-side tile, then N-side tile
constexpr int kScaleRing = 16;               // K blocks of scales in flight
constexpr int kEpiWarps = 16;
constexpr int kEpiThreads = 32 * kEpiWarps;
constexpr int kPairThreads = 128 + kEpiThreads;
constexpr int kMaxSlots = 4;
constexpr int kPairTmemCols = 512;

template <int MODE> struct PairCfg {
  static constexpr int kKBlocks = MODE == 1 ? kHBlocks : kIBlocks;              // 56 / 16
  static constexpr int kFeatItems = MODE == 1 ? kInter / 128 : kHidden / 256;   // 16 / 28 per expert and token tile
  static constexpr int kTokTile = MODE == 1 ? 256 : 128;
  static constexpr int kStages = 6;
  // Two accumulator slots of 256 tensor-memory columns: the MMAs of K block k + 1 run while block k is
  // promoted.  (Four slots of 128 columns, a K block issued as two MMA groups of N = 128, doubled the
  // hand-offs between the MMA thread and the promotion warps and were slower.)
  static constexpr int kSlots = 2;
  static constexpr int kSlotCols = kPairTmemCols / kSlots;
  static constexpr int kScaleEntry = 128;   // floats per ring entry: one per token lane (mode 1) / token column (mode 2)
  // mode 1: the activation scales of a whole item, [56][128]; mode 2: a ring of K blocks of scale products
  static constexpr int kScaleFloats = MODE == 1 ? kHBlocks * 128 : kScaleRing * kScaleEntry;
  static constexpr int kSmemBytes = 1024 + kStages * kStageBytes + kScaleFloats * 4 +
                                    (MODE == 1 ? 4 * 128 * 4 + 2 * 128 * 4 : 0) + 8 * 64 +
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
  long long wait_limit;     // SM clocks a wait may take before the CTA gives up (tests make it short)
  int silent_producer;      // test hook: the TMA producer issues nothing, so that the other roles' waits run out
  float* const* row_out;    // mode 2, expert parallelism: row r goes to row_out[r] (a peer's memory; null = padding row, not stored) instead of o_rows
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

// bytes the token-side loads of `rows` rows bring in: one 128-row box above 64 rows, else 32-row boxes
__device__ __forceinline__ int box_bytes(int rows) {
  return rows > 64 ? kTile : ((rows + 31) >> 5) * kBox;
}

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
                 const __grid_constant__ CUtensorMap tm_b1, const __grid_constant__ CUtensorMap tm_b0w,
                 const __grid_constant__ CUtensorMap tm_b1w, const PairArgs p) {
  using C = PairCfg<MODE>;
  constexpr int G = C::kStages;
  constexpr int KB = C::kKBlocks;
  constexpr int FI = C::kFeatItems;
  constexpr int NT = C::kTokTile;
  constexpr int SE = C::kScaleEntry;
  constexpr int kSlots = C::kSlots;
  constexpr int kSlotCols = C::kSlotCols;
  constexpr int kIssuers = MODE == 1 ? 2 : 1;   // MMA-issuing threads (see mma_role)

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  float* s_scale = reinterpret_cast<float*>(smem + G * kStageBytes);           // mode 1: [56][128]; mode 2: [kScaleRing][SE]
  float* s_red = s_scale + C::kScaleFloats;                                    // [4][128] partial amax (mode 1)
  float* s_ws = s_red + (MODE == 1 ? 4 * 128 : 0);                             // [2][128] weight scales of an item (mode 1)
  uint64_t* full = reinterpret_cast<uint64_t*>(s_ws + (MODE == 1 ? 2 * 128 : 0));   // [G]   first CTA's are used
  uint64_t* empty = full + G;                                                  // [G/2] per CTA
  uint64_t* tfull = empty + G / 2;                                             // [4]   per CTA
  uint64_t* tempty = tfull + kMaxSlots;                                        // [4]   first CTA's are used
  uint64_t* sfull = tempty + kMaxSlots;                                         // [16]  per CTA
  uint64_t* sempty = sfull + kScaleRing;                                       // [16]  per CTA
  uint64_t* wfull = sempty + kScaleRing;                                       // [2]   mode 1: an item's weight scales are there
  uint64_t* wempty = wfull + 2;                                                // [2]
  ExpertWork* s_work = reinterpret_cast<ExpertWork*>(wempty + 2);
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
    for (int i = 0; i < G / 2; ++i) mbar_init(&empty[i], kIssuers);   // one commit per MMA issuer
    for (int i = 0; i < kMaxSlots; ++i) { mbar_init(&tfull[i], 1); mbar_init(&tempty[i], 2 * kEpiWarps); }
    for (int i = 0; i < kScaleRing; ++i) { mbar_init(&sfull[i], 1); mbar_init(&sempty[i], kEpiWarps); }
    for (int i = 0; i < 2; ++i) { mbar_init(&wfull[i], 1); mbar_init(&wempty[i], kEpiWarps); }
    *s_abort = 0;
    *s_done = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tm_w);
    tma_prefetch_desc(&tm_b0);
    tma_prefetch_desc(&tm_b0w);
    if (MODE == 2) { tma_prefetch_desc(&tm_b1); tma_prefetch_desc(&tm_b1w); }
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
    // (meta[1] = 0: the row-list kernel refused the call, its work table is stale)
    ExpertWork ew = (lane < p.e_local && p.meta[1] > 0) ? p.work[lane] : ExpertWork{0, 0, 0, 0};
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

  // MMA issue, one thread of the pair's first CTA per K-block parity.  Two issuers (even K blocks -> slot 0,
  // odd -> slot 1) because an issuer is tied up for the whole execution time of its MMAs (the queue behind
  // tcgen05.mma is shallow) and then pays its commits and the wait for its slot: with one issuer the tensor
  // pipe idles during those; with two, one's waits overlap the other's MMAs.  MMAs of different slots are
  // independent, and tcgen05.commit tracks the MMAs of the committing thread only, so each issuer commits its
  // own slot and its own half of the stage pair (empty[] counts two arrivals).
  auto mma_role = [&](const uint32_t par) {
    uint32_t g = par, ph = 0, sph = 0;      // this issuer's next stage and its phase, phase of its slot
    uint32_t slot = par;                    // mode 2 (one issuer): alternates between the two slots
    int e_hint = 0;
    bool alive = true;
    ST_DECL;
    const long long st_start = clock64();
    (void)st_start;
    for (int i = 0; i < my_items && alive; ++i) {
      const PItem im = decode_pair_item<FI, NT>(s_work, p.e_local, item_of(i), e_hint);
      const uint32_t idesc = umma_idesc_e4m3_m256(MODE == 1 ? 256u : 2u * im.n);
      for (int kb = static_cast<int>(par); kb < KB; kb += kIssuers) {
        ST_BEGIN();
        if (!mbar_wait_bounded_tell(&full[g], ph, s_abort, peer_abort, kStatusWaitTimeoutMma, p.wait_limit)) { alive = false; break; }
        ST_END(0);
        const uint32_t sb = smem_u32(smem + g * kStageBytes);
        const uint64_t a0 = umma_smem_desc_sw128(sb);
        const uint64_t b0 = umma_smem_desc_sw128(sb + kTile);
        ST_BEGIN();
        if (!mbar_wait_bounded_tell(&tempty[slot], sph ^ 1u, s_abort, peer_abort, kStatusWaitTimeoutMma, p.wait_limit)) { alive = false; break; }
        ST_END(1);
        tc_fence_after();
        const uint32_t d0 = tmem_base + slot * kSlotCols;
#pragma unroll
        for (int k4 = 0; k4 < 4; ++k4) umma_f8_pair(d0, a0 + 2 * k4, b0 + 2 * k4, idesc, k4 > 0 ? 1u : 0u);
        if (kIssuers == 2 || (g & 1u)) umma_commit_pair(&empty[g >> 1], 3);
        umma_commit_pair(&tfull[slot], 3);
        if (kIssuers == 2) {
          sph ^= 1u;
        } else {
          slot ^= 1u;
          if (slot == 0) sph ^= 1u;
        }
        g += kIssuers;
        if (g >= static_cast<uint32_t>(G)) { g -= G; ph ^= 1u; }
      }
    }
#ifdef SYFI_PAIR_STATS
    st_acc[2] = clock64() - st_start;
#endif
    ST_WRITE(4, par == 0);
  };

  if (warp < 4) {
    if (warp == 0) {
      // ------------------------------------------------------------ TMA producer (one thread per CTA)
      if (lane == 0 && !p.silent_producer) {
        const uint64_t pol_w = s_meta[0] > s_meta[1] ? l2_policy_evict_last() : l2_policy_evict_first();
        const uint64_t pol_b = l2_policy_evict_last();
        uint32_t full0[G];                     // the first CTA's full barriers as cluster addresses
#pragma unroll
        for (int i = 0; i < G; ++i) full0[i] = mapa_u32(smem_u32(&full[i]), 0);
        uint32_t it = 0, g = 0, ph = 0;        // stage pairs armed, next stage, phase of its empty barrier
        uint32_t s = 0, sp = 0;                // scale ring entry and phase (mode 1)
        uint32_t wp = 0;                       // phase bits of wempty[0..1] (mode 1)
        uint32_t n_items = 0;
        int e_hint = 0;
        bool alive = true;
        ST_DECL;
        const long long st_start = clock64();
        (void)st_start; (void)s; (void)sp; (void)wp;
        for (int i = 0; i < my_items && alive; ++i) {
          const PItem im = decode_pair_item<FI, NT>(s_work, p.e_local, item_of(i), e_hint);
          int my_rows, my_row, wrow, tok_off, w_off;
          uint32_t stage_tx;
          const CUtensorMap* mb;
          if (MODE == 1) {
            // token tile on the M side: this CTA's rows 128 rank .. of the tile (none when the tile is short)
            const int cnt0 = min(im.n, 128), cnt1 = im.n - cnt0;
            my_rows = rank == 0 ? cnt0 : cnt1;
            my_row = im.row_start + 128 * static_cast<int>(rank);
            wrow = im.expert * 2 * kInter + static_cast<int>(rank) * kInter + im.ft * 128;
            mb = my_rows > 64 ? &tm_b0w : &tm_b0;
            tok_off = 0;
            w_off = kTile;
            stage_tx = static_cast<uint32_t>(2 * kTile + box_bytes(cnt0) + box_bytes(cnt1));
          } else {
            my_rows = im.n;                                      // all rows of one term
            my_row = im.row_start;
            wrow = im.expert * kHidden + (2 * im.ft + static_cast<int>(rank)) * 128;
            mb = my_rows > 64 ? (rank == 0 ? &tm_b0w : &tm_b1w) : (rank == 0 ? &tm_b0 : &tm_b1);
            tok_off = kTile;
            w_off = 0;
            stage_tx = 2u * static_cast<uint32_t>(kTile + box_bytes(im.n));
          }
          // more than 64 rows: one 128-row box (fewer TMA instructions); else 32-row boxes
          if (MODE == 1) {
            // weight scales of the item, [0..55] up block and [64..119] gate block, into the buffer the
            // epilogue released two items ago
            const int par = i & 1;
            if (!mbar_wait_bounded_tell(&wempty[par], ((wp >> par) & 1u) ^ 1u, s_abort, peer_abort,
                                        kStatusWaitTimeoutProducer, p.wait_limit)) { alive = false; break; }
            wp ^= 1u << par;
            mbar_arrive_expect_tx(&wfull[par], 2u * kHBlocks * 4u);
            bulk_load(s_ws + par * 128, p.w_scale + (static_cast<size_t>(im.expert) * 32 + im.ft) * kHBlocks,
                      kHBlocks * 4, &wfull[par], pol_b);
            bulk_load(s_ws + par * 128 + 64, p.w_scale + (static_cast<size_t>(im.expert) * 32 + 16 + im.ft) * kHBlocks,
                      kHBlocks * 4, &wfull[par], pol_b);
          }
          const int boxes = my_rows > 64 ? 1 : (my_rows + 31) >> 5;
          const int box_pitch = my_rows > 64 ? kTile : kBox;
          const int box_rows = my_rows > 64 ? 128 : 32;
          if (MODE == 2) {
            // the item's expert must have left GEMM1 (the helper warp checks and counts cleared items)
            if (*reinterpret_cast<volatile int*>(s_done) <= static_cast<int>(n_items)) {
              const long long t0 = clock64();
              while (*reinterpret_cast<volatile int*>(s_done) <= static_cast<int>(n_items)) {
                if (*s_abort != 0) { alive = false; break; }
                if (clock64() - t0 > p.wait_limit) {
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
                                        p.wait_limit)) { alive = false; break; }
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
            tma_load_2d_pair(st0 + w_off, &tm_w, full0[g], x0, wrow, pol_w);
            tma_load_2d_pair(st1 + w_off, &tm_w, full0[g + 1], x0 + 128, wrow, pol_w);
            for (int b = 0; b < boxes; ++b) {
              tma_load_2d_pair(st0 + tok_off + b * box_pitch, mb, full0[g], x0, my_row + box_rows * b, pol_b);
              tma_load_2d_pair(st1 + tok_off + b * box_pitch, mb, full0[g + 1], x0 + 128, my_row + box_rows * b, pol_b);
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
      // --------------------------------------------------------------- MMA issuer for the even K blocks
      if (lane == 0 && rank == 0) mma_role(0);
      __syncwarp();
    } else if (warp == 2) {
      // --------------------------------------------------------------- scale warp
      if (MODE == 1) {
        // ------------------------------------------------------------- MMA issuer for the odd K blocks
        if (lane == 0 && rank == 0) mma_role(1);
        __syncwarp();
      } else {
        // entry s of the ring holds, for one K block, act_scale[row, kb] * w_scale[kb] of every token column
        // of the item; lane l serves columns 4 l .. 4 l + 3
        constexpr int kBatch = 4;
        uint32_t s = 0, sp = 0;
        uint32_t n_items = 0;
        int e_hint = 0;
        bool alive = true;
        for (int i = 0; i < my_items && alive; ++i) {
          const PItem im = decode_pair_item<FI, NT>(s_work, p.e_local, item_of(i), e_hint);
          if (*reinterpret_cast<volatile int*>(s_done) <= static_cast<int>(n_items)) {
            const long long t0 = clock64();
            while (*reinterpret_cast<volatile int*>(s_done) <= static_cast<int>(n_items)) {
              if (*s_abort != 0 || clock64() - t0 > p.wait_limit) { alive = false; break; }
            }
          }
          alive = __all_sync(0xffffffffu, alive);
          if (!alive) break;
          __threadfence_block();
          ++n_items;
          const float* wsp = p.w_scale + (static_cast<size_t>(im.expert) * kHBlocks + 2 * im.ft + rank) * kIBlocks;
          const float ws_a = lane < KB ? __ldg(wsp + lane) : 0.0f;
          const int col = 4 * lane;
          const bool v0 = col < im.n;
          const float* src = p.act_scale + im.row_start + col;
          for (int kb0 = 0; kb0 < KB && alive; kb0 += kBatch) {
            float4 a[kBatch];
#pragma unroll
            for (int k = 0; k < kBatch; ++k) {
              // plain loads: these scales were written by GEMM1, which may still be running
              a[k] = v0 ? ld_global_f32x4(src + static_cast<size_t>(kb0 + k) * p.row_cap) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int k = 0; k < kBatch; ++k) {
              const float ws = __shfl_sync(0xffffffffu, ws_a, kb0 + k);
              bool ok = mbar_wait_bounded_tell(&sempty[s], sp ^ 1u, s_abort, peer_abort, kStatusWaitTimeoutProducer, p.wait_limit);
              ok = __all_sync(0xffffffffu, ok);
              if (!ok) { alive = false; break; }
              *reinterpret_cast<float4*>(s_scale + s * SE + col) =
                  make_float4(a[k].x * ws, a[k].y * ws, a[k].z * ws, a[k].w * ws);
              __syncwarp();
              if (lane == 0) mbar_arrive(&sfull[s]);
              if (++s == kScaleRing) { s = 0; sp ^= 1u; }
            }
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
          // same ordering chain as the single-CTA kernel's publisher (grouped_gemm.cu): stores -> CTA-scope
          // count -> gpu-scope fence + proxy fence + release here; acquire + proxy fence in GEMM2's helper
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
              if (clock64() - t0 > (p.wait_limit >> 1)) {   // half the other roles' limit: this wait reports first
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
    const int q = warp & 3;                       // lane quarter this warp may read
    const int grp = (warp - 4) >> 2;              // which quarter of the columns
    const int tl = q * 32 + lane;                 // tensor-memory lane: mode 1 token of this CTA, mode 2 feature
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    const uint32_t mapa_tempty = mapa_u32(smem_u32(&tempty[0]), 0);   // the first CTA's tempty[0]; the others follow at 8 bytes each
    uint32_t sl = 0, sph = 0;                     // accumulator slot and its phase
    uint32_t s = 0, sp = 0;                       // scale ring entry and its phase
    uint32_t wp = 0;                              // phase bits of wfull[0..1] (mode 1)
    bool ok = true;
    int e_hint = 0;
    const uint64_t inv_ratio = f32x2_pack(1.0f / kLoRatio, 1.0f / kLoRatio);
    ST_DECL;
    const long long st_start = clock64();
    (void)st_start; (void)inv_ratio; (void)wp;

    if (MODE == 1 && my_items > 0) {
      // activation scales of the first item (later items: fetched during the previous item's epilogue)
      int eh = 0;
      const PItem f = decode_pair_item<FI, NT>(s_work, p.e_local, item_of(0), eh);
      const int nrows = rank == 0 ? min(f.n, 128) : max(f.n - 128, 0);
      const float* src = p.act_scale + static_cast<size_t>(grp) * (kHBlocks / 4) * p.row_cap + f.row_start + 128 * rank + tl;
#pragma unroll
      for (int k = 0; k < kHBlocks / 4; ++k)
        s_scale[(grp * (kHBlocks / 4) + k) * 128 + tl] = tl < nrows ? __ldg(src + static_cast<size_t>(k) * p.row_cap) : 0.0f;
      named_bar_sync(1 + q, 128);
    }
    for (int i = 0; i < my_items; ++i) {
      const PItem im = decode_pair_item<FI, NT>(s_work, p.e_local, item_of(i), e_hint);

      if (MODE == 1) {
        // ===== token-major: lane = token, columns [32 grp, +32) = up, [128 + 32 grp, +32) = gate
        const int par = i & 1;
        const float* ws = s_ws + par * 128;
        if (ok && !mbar_wait_bounded_tell(&wfull[par], (wp >> par) & 1u, s_abort, peer_abort,
                                          kStatusWaitTimeoutEpilogue, p.wait_limit)) ok = false;
        wp ^= 1u << par;
        float up[32], gt[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) { up[j] = 0.0f; gt[j] = 0.0f; }
        for (int kb = 0; kb < KB && ok; ++kb) {
          // block scale of this thread's token: its activation scale (staged in shared memory for the whole
          // item, see the end of the previous item) times the weight scales of the up and the gate block
          const float a = s_scale[kb * 128 + tl];
          const float su = a * ws[kb], sg = a * ws[64 + kb];
          ST_BEGIN();
          if (!mbar_wait_bounded_tell(&tfull[sl], sph, s_abort, peer_abort, kStatusWaitTimeoutEpilogue, p.wait_limit)) { ok = false; break; }
          ST_END(0);
          tc_fence_after();
#ifdef SYFI_PAIR_STATS
          const long long st_p0 = clock64();
#endif
          const uint32_t t0 = lane_addr + sl * kSlotCols + grp * 32;
          // scalar FMAs (measured faster here than packed f32x2 ones, whose operand pairs cost extra moves);
          // the slot goes back to the MMA thread as soon as its last values are in registers
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const bool is_gate = c >= 2;
            const int cc = c & 1;
            uint32_t r[16];
            tmem_ld16(t0 + (is_gate ? 128 : 0) + cc * 16, r);
            tmem_ld_wait();
            if (c == 3) {
              tc_fence_before();
              __syncwarp();
              if (lane == 0) mbar_arrive_cluster_relaxed(mapa_tempty + 8u * sl);
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              if (!is_gate) up[cc * 16 + j] = fmaf(__uint_as_float(r[j]), su, up[cc * 16 + j]);
              else gt[cc * 16 + j] = fmaf(__uint_as_float(r[j]), sg, gt[cc * 16 + j]);
            }
          }
          if (++sl == kSlots) { sl = 0; sph ^= 1u; }
#ifdef SYFI_PAIR_STATS
          st_acc[2] += clock64() - st_p0;
#endif
        }
        if (ok) {   // the weight scales go back to the producer
          __syncwarp();
          if (lane == 0) mbar_arrive(&wempty[par]);
        }
        ST_BEGIN();
        // ---- SwiGLU of this token's 32 features, amax over the token's 128 features (four threads, one per
        // column quarter), two-term requantisation; the fast exp and divide are a few ulp off the exact ones,
        // far below the 8-bit requantisation that follows
        const int my_rows = ok ? (rank == 0 ? min(im.n, 128) : max(im.n - 128, 0)) : 0;
        // the next item's activation scales are requested now (this thread: 14 K blocks of its token) and
        // stored once every warp of this lane quarter has left the K loop (the barrier below)
        float nxt[kHBlocks / 4];
        {
          const bool more = i + 1 < my_items;
          int eh = e_hint;
          const PItem nx = more ? decode_pair_item<FI, NT>(s_work, p.e_local, item_of(i + 1), eh) : PItem{0, 0, 0, 0};
          const int nrows = rank == 0 ? min(nx.n, 128) : max(nx.n - 128, 0);
          const float* src = p.act_scale + static_cast<size_t>(grp) * (kHBlocks / 4) * p.row_cap + nx.row_start + 128 * rank + tl;
#pragma unroll
          for (int k = 0; k < kHBlocks / 4; ++k)
            nxt[k] = (more && tl < nrows) ? __ldg(src + static_cast<size_t>(k) * p.row_cap) : 0.0f;
        }
        float c[32];
        float amax = 0.0f;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const float g = gt[j];
          c[j] = g * __fdividef(1.0f, 1.0f + __expf(-g)) * up[j];
          amax = fmaxf(amax, fabsf(c[j]));
        }
        float* red = s_red;
        red[grp * 128 + tl] = amax;
        named_bar_sync(1 + q, 128);             // the four warps that share this lane quarter
        amax = fmaxf(fmaxf(red[tl], red[128 + tl]), fmaxf(red[256 + tl], red[384 + tl]));
#pragma unroll
        for (int k = 0; k < kHBlocks / 4; ++k) s_scale[(grp * (kHBlocks / 4) + k) * 128 + tl] = nxt[k];
        if (tl < my_rows) {
          const float scv = fmaxf(amax * (1.0f / 448.0f), 1e-12f);
          const float inv = 1.0f / scv;
          const size_t row = static_cast<size_t>(im.row_start) + 128 * rank + tl;
          if (grp == 0) p.c_scale[static_cast<size_t>(im.ft) * p.row_cap + row] = scv;
          uint32_t hw[8], lw[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            uint32_t hp = 0, lp = 0;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const float v0 = c[4 * j + 2 * h], v1 = c[4 * j + 2 * h + 1];
              const uint16_t hh = cvt_e4m3x2(v0 * inv, v1 * inv);
              const float2 hb = e4m3x2_to_float2(hh);
              const float r0 = fmaf(-hb.x, scv, v0), r1 = fmaf(-hb.y, scv, v1);
              const uint16_t ll = cvt_e4m3x2(r0 * inv * kLoRatio, r1 * inv * kLoRatio);
              hp |= static_cast<uint32_t>(hh) << (16 * h);
              lp |= static_cast<uint32_t>(ll) << (16 * h);
            }
            hw[j] = hp;
            lw[j] = lp;
          }
          const size_t off = row * kInter + static_cast<size_t>(im.ft) * 128 + grp * 32;
          *reinterpret_cast<uint4*>(p.c_hi + off) = make_uint4(hw[0], hw[1], hw[2], hw[3]);
          *reinterpret_cast<uint4*>(p.c_hi + off + 16) = make_uint4(hw[4], hw[5], hw[6], hw[7]);
          *reinterpret_cast<uint4*>(p.c_lo + off) = make_uint4(lw[0], lw[1], lw[2], lw[3]);
          *reinterpret_cast<uint4*>(p.c_lo + off + 16) = make_uint4(lw[4], lw[5], lw[6], lw[7]);
        }
        named_bar_sync(1 + q, 128);             // the next item's scales are in place, the amax exchange is free
        // hand the item to the publisher warp (see grouped_gemm.cu)
        __threadfence_block();
        __syncwarp();
        if (lane == 0) atomicAdd(s_done, 1);
        ST_END(3);
      } else {
        // ===== feature-major: lane = output feature, columns [32 grp, +32) = hi, [n + 32 grp, +32) = lo
        constexpr int CN = 32;
        const int c0 = grp * CN;
        const int n = ok ? im.n : 0;
        uint64_t acc[CN / 2];
#pragma unroll
        for (int j = 0; j < CN / 2; ++j) acc[j] = 0ull;
        for (int kb = 0; kb < KB && ok; ++kb) {
          ST_BEGIN();
          if (!mbar_wait_bounded_tell(&tfull[sl], sph, s_abort, peer_abort, kStatusWaitTimeoutEpilogue, p.wait_limit)) { ok = false; break; }
          ST_END(0);
          tc_fence_after();
          if (!mbar_wait_bounded_tell(&sfull[s], sp, s_abort, peer_abort, kStatusWaitTimeoutEpilogue, p.wait_limit)) { ok = false; break; }
#ifdef SYFI_PAIR_STATS
          const long long st_p0 = clock64();
#endif
          const float* sc = s_scale + s * SE + c0;
          const uint32_t t0 = lane_addr + sl * kSlotCols + c0;
          // (handing the slot back before the arithmetic of the last chunk, as mode 1 does, costs registers
          // here and was slower: 400 us against 359 us)
#pragma unroll
          for (int ch = 0; ch < CN / 16; ++ch) {
            if (c0 + ch * 16 < n) {
              const ulonglong2* sp4 = reinterpret_cast<const ulonglong2*>(sc + ch * 16);
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
          tc_fence_before();
          __syncwarp();
          if (lane == 0) {
            mbar_arrive_cluster_relaxed(mapa_tempty + 8u * sl);
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
        float out[CN];
#pragma unroll
        for (int j = 0; j < CN / 2; ++j) f32x2_unpack(acc[j], out[2 * j], out[2 * j + 1]);
        const int qrow = lane & 3;
        const int row0 = im.row_start + c0 + qrow;
        const int col = (2 * im.ft + static_cast<int>(rank)) * 128 + q * 32 + (lane >> 2) * 4;
#pragma unroll
        for (int j = 0; j < CN; j += 4) {
          if (c0 + j < n_out) {
            float a0 = out[j], a1 = out[j + 1], a2 = out[j + 2], a3 = out[j + 3];
            quad_transpose_f32(a0, a1, a2, a3, lane);   // now: row c0 + j + qrow, four adjacent features
            // expert parallelism: the row's place in its token owner's memory (plain stores over NVLink)
            float* o = p.row_out != nullptr ? p.row_out[row0 + j] : p.o_rows + static_cast<size_t>(row0 + j) * kHidden;
            if (o != nullptr) *reinterpret_cast<float4*>(o + col) = make_float4(a0, a1, a2, a3);
          }
        }
        ST_END(3);
      }
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
                          static_cast<size_t>(PairCfg<MODE>::kSmemBytes), st, g.tm_w, g.tm_b0, g.tm_b1, g.tm_b0w, g.tm_b1w,
                          a);
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
             ws.ready, ws.status, ws.trace, g.wait_limit, g.silent_producer, nullptr};
  return launch_pair<1>(g, a, num_sms, st);
}

cudaError_t launch_pair_gemm2(const PairGemmLaunch& g, const float* w2_scale, int e_local, const Workspace& ws,
                              int num_sms, cudaStream_t st) {
  PairArgs a{ws.work, ws.meta, ws.c_scale, w2_scale, nullptr, nullptr, nullptr, ws.o_rows, ws.row_cap, e_local,
             ws.ready, ws.status, ws.trace + 4096, g.wait_limit, g.silent_producer,
             g.rows_to_targets ? ws.row_out : nullptr};
  return launch_pair<2>(g, a, num_sms, st);
}

}  // namespace syfi
