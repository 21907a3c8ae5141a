// Grouped FP8 block-scale GEMMs of the MoE layer on tcgen05 (sm_100a).
//
// GEMM1 (mode 1) replaces gemm_fp8_fp8_tcgen05_grouped_kernel / gemm_fp8_fp8_grouped_kernel
// plus swiglu_quant_fp8_kernel of the reference (moe/solution/cuda/moe.cu:2194-2350,
// 1461-1627, 1631-1714); GEMM2 (mode 2) replaces gemm_fp8_fp8_fused_acc_grouped_kernel
// (moe.cu:1718-1887).
//
// Orientation ("swap-AB"): the WEIGHT tile is the 128-row M operand of the MMA and the
// expert's token rows are the N operand (16..NT columns, NT = 32 or 64 chosen per launch), so an expert with a handful of
// rows still issues full-height MMAs and the kernel streams weights at HBM speed.  In the
// TMEM accumulator a lane is an output feature and a column is a token row.
//
//   mode 1, work item = (token tile, 128 intermediate features f0..f0+127):
//       up[f, r]   = sum_k W13[e, f0 + f, k]        * A[r, k]
//       gate[f, r] = sum_k W13[e, 2048 + f0 + f, k] * A[r, k]
//     per 128-wide K block the raw e4m3 x e4m3 products are accumulated in TMEM (4 MMAs of
//     K = 32 per operand pair) and then promoted into f32 registers with the product of
//     the activation scale (per row, per K block) and the weight scale (per 128x128 block).
//     Epilogue: c = silu(gate) * up, quantised along the 128 features of this tile (one
//     1x128 block of GEMM2's K) into TWO e4m3 terms that share one scale:
//       hi = e4m3(c / s),  lo = e4m3((c - hi * s) * 28 / s),   s = max(amax / 448, 1e-12)
//     (|c - hi*s| <= 16 s because the e4m3 spacing below 448 is 32, and 16 * 28 = 448, so
//     lo never saturates); c ~= s * (hi + lo / 28) carries about 8 mantissa bits, which a
//     single e4m3 term does not and the output tolerance needs.
//   mode 2, work item = (token tile, 128 output features h0..h0+127):
//       o[h, r] = sum_k W2[e, h0 + h, k] * (hi[r, k] + lo[r, k] / 28) * s[r, kb] * w2s[e, hb, kb]
//     two accumulators (hi and lo) share the weight tile in shared memory.
//
// Pipeline per CTA (persistent over work items): warp 0 = TMA producer (weights with an
// evict-first L2 policy when streamed once, token-side tiles evict-last), warp 1 = MMA issuer
// and TMEM owner, then the promotion/epilogue warps (a warp reads one TMEM lane quarter; the
// tile's columns are split between two or four warps per quarter), and a last warp that keeps
// the cross-kernel bookkeeping off everybody else's path (mode 1: publishes finished items to
// GEMM2; mode 2: waits for GEMM1 to finish an item's expert).  Shared-memory stages form a
// ring guarded by full/empty mbarriers; the 512 TMEM columns form a ring of 512 / (2 NT)
// accumulator-pair slots (tfull/tempty), so the MMAs of several K blocks are in flight while
// earlier blocks are promoted: the issue -> commit -> tcgen05.ld -> release round trip costs
// about 1.5 us and has to be hidden behind 4 to 8 K blocks to keep up with HBM.
// Every wait is bounded: on expiry the CTA raises an abort flag, all roles leave their
// loops, TMEM is released and the status word reports the failure to the host.
#include <cuda_fp16.h>

#include "moe_internal.h"
#include "ptx.cuh"

namespace syfi {

namespace {

constexpr int kATile = 128 * 128;         // weight tile: 128 rows x 128 bytes of K
constexpr int kTmemCols = 512;

template <int MODE, int NT> struct Cfg {
  static constexpr int kKBlocks = MODE == 1 ? kHBlocks : kIBlocks;              // 56 / 16
  static constexpr int kFeatTiles = MODE == 1 ? kInter / 128 : kHidden / 128;   // 16 / 56
  static constexpr int kRowsPerExpert = MODE == 1 ? 2 * kInter : kHidden;       // weight rows per expert
  static constexpr int kBTile = NT * 128;                                       // token-side tile bytes
  static constexpr int kStageBytes = MODE == 1 ? 2 * kATile + kBTile : kATile + 2 * kBTile;  // one K block
  // K blocks per pipeline step.  One thread issues every MMA (about 50 cycles each) and every
  // tcgen05.commit (about 90 cycles), so with small N the issue loop, not the tensor pipe, sets
  // the pace; handing over two K blocks per barrier round halves the waits and commits per byte.
  static constexpr int kKps = 2;
  static constexpr int kGroups = NT == 128 ? 2 : MODE == 1 ? (NT == 32 ? 3 : 2) : (NT == 32 ? 4 : 3);   // smem ring depth
  static constexpr int kGroupBytes = kKps * kStageBytes;
  static constexpr int kSlots = kTmemCols / (2 * NT);                           // accumulator-pair slots
  // K blocks per TMEM ring entry.  The 128-row token tile fills half of TMEM with one K block's
  // accumulator pair, so there the MMA thread and the epilogue hand slots over one K block at a time
  // (the shared-memory ring still moves two, for the K-adjacent request pattern).
  static constexpr int kTKps = NT == 128 ? 1 : kKps;
  static constexpr int kPairs = kSlots / kTKps;                                 // TMEM ring entries
  static constexpr int kScaleBufs = MODE == 2 ? 3 : 1;   // mode 2 prefetches the scales two items ahead
  // Epilogue warps per TMEM lane quarter: each owns 16 token columns (32 at the 128-row tile, where the
  // thread limit of a CTA caps the split).  Two or more warps per scheduler hide the latency of the
  // promotion chain and of the SwiGLU / requantisation epilogue, which a single warp runs back to back:
  // measured 3-8 % faster per call than 32 columns per warp; 8 columns per warp was no better than 16.
  static constexpr int kColSplit = NT == 128 ? 4 : NT / 16;
  static constexpr int kThreads = 64 + 128 * kColSplit + 32;   // producer, MMA, epilogue warps, publisher warp
  static constexpr int kSmemBytes = 1024 /* alignment slack */ + kGroups * kGroupBytes +
                                    4 * (kScaleBufs * (kKBlocks * NT + 128) + 4 * NT + 2 * NT) +
                                    8 * (2 * kGroups + 2 * kPairs + 6) +
                                    kMaxLocalExperts * static_cast<int>(sizeof(ExpertWork)) + 32;
  static_assert(kSmemBytes <= 232448, "exceeds the 227 KB of shared memory a CTA may use");
  static_assert(kKBlocks % kKps == 0 && kSlots % kTKps == 0 && kKps % kTKps == 0,
                "steps must tile the K blocks and the slots");
  static_assert(kThreads <= 1024, "too many epilogue warps");
};

struct GemmArgs {
  // Pre-packed weights (see prepack.cu) or nullptr.  When set, the weight tiles of a work item are
  // consecutive 16 KB images of what the tiled loads would have written to shared memory, and the
  // producer fetches them with untiled bulk copies instead of going through the weight tensor map.
  const uint8_t* w_packed;
  const ExpertWork* work;
  const int* meta;
  const float* act_scale;   // [K blocks][row_cap] scales of the token-side operand
  const float* w_scale;     // mode 1: [E][32][56], mode 2: [E][56][16]
  uint8_t* c_hi;            // mode 1 outputs
  uint8_t* c_lo;
  float* c_scale;           // [16][row_cap]
  float* o_rows;            // mode 2 output [row_cap][7168]
  int row_cap;
  int e_local;
  int* ready;               // [32] GEMM1 items finished per expert: mode 1 increments, mode 2 waits on it
  int* status;
  long long* trace;         // [3][4096] timeline of CTA 0 when built with SYFI_TRACE, else unused
  long long* trace_cta;     // [grid][5] per-CTA start/end (globaltimer, clock64) and SM id, SYFI_TRACE only
  long long wait_limit;     // SM clocks a wait may take before the CTA gives up (tests make it short)
  int silent_producer;      // test hook: the TMA producer issues nothing, so that the other roles' waits run out
  float* const* row_out;    // mode 2, expert parallelism: row r goes to row_out[r] (a peer's memory; null = padding row, not stored) instead of o_rows
};

// Optional timeline trace of CTA 0 (compile with -DSYFI_TRACE): role r appends (tag, clock) pairs.
#ifdef SYFI_TRACE
#define TRACE(role, tag)                                                                       \
  do {                                                                                         \
    if (blockIdx.x == 0 && p.trace != nullptr && trace_n < 2040) {                             \
      p.trace[(role) * 4096 + 2 * trace_n] = (tag);                                            \
      p.trace[(role) * 4096 + 2 * trace_n + 1] = clock64();                                    \
      ++trace_n;                                                                               \
    }                                                                                          \
  } while (0)
#else
#define TRACE(role, tag) do { } while (0)
#endif

struct Item {
  int expert, ft, row_start, n;
};

// Work item w -> (expert, feature tile, token tile); see ExpertWork for the numbering.  A CTA's items
// come in increasing order, so each role resumes the search at the expert of its previous item
// (`e_hint`, start at 0): scanning the table from the front costs over a thousand cycles per item and
// role once the later experts are reached, which the short GEMM2 items do not hide.
template <int FT, int NT>
__device__ __forceinline__ Item decode_item(const ExpertWork* s_work, int e_local, int w, int& e_hint) {
  Item it{0, 0, 0, 0};
  for (int e = e_hint; e < e_local; ++e) {
    const ExpertWork ew = s_work[e];
    const int base = ew.tile_off * FT;
    if (w < base + ew.tiles * FT) {
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

// Schedule: whole work items are dealt round-robin over the persistent grid (CTA b takes items b,
// b + grid, ...).  With the item numbering above, the CTAs running side by side work on the token
// tiles of the SAME weight tile, so all but one of them find it in L2.  Splitting items across CTAs
// at K-step granularity (stream-K, static or with a dynamically claimed tail) was measured and
// bought nothing at any batch size: the kernels are bound by aggregate HBM bandwidth, not by the
// last wave, and the hand-off of partial sums costs what the better balance gains.

template <int MODE, int NT>
__global__ void __launch_bounds__((Cfg<MODE, NT>::kThreads), 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_b0,
                    const __grid_constant__ CUtensorMap tm_b1, const __grid_constant__ CUtensorMap tm_b0s,
                    const __grid_constant__ CUtensorMap tm_b1s, const __grid_constant__ CUtensorMap tm_sc,
                    const GemmArgs p) {
  using C = Cfg<MODE, NT>;
  constexpr int G = C::kGroups;           // smem ring entries, each kKps K blocks
  constexpr int KPS = C::kKps;
  constexpr int KB = C::kKBlocks;
  constexpr int STEPS = KB / KPS;
  constexpr int FT = C::kFeatTiles;
  constexpr int TKPS = C::kTKps;
  constexpr int PAIRS = C::kPairs;        // TMEM ring entries, each kTKps accumulator-pair slots
  constexpr int kBTile = C::kBTile;
  // Layout of one ring entry (KPS K blocks).  Mode 1: per K block [up tile][gate tile][token tile].
  // Mode 2: the weight tiles of all K blocks first (adjacent, so pre-packed weights arrive as one
  // copy), then per K block [hi tile][lo tile].
  auto w_off = [](int k) { return MODE == 1 ? k * C::kStageBytes : k * kATile; };
  auto b_off = [](int k) { return MODE == 1 ? k * C::kStageBytes + 2 * kATile : KPS * kATile + k * 2 * kBTile; };

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  constexpr int kScaleStride = KB * NT + 128;                           // one buffer: [KB][NT] + [2][64]
  float* s_scales = reinterpret_cast<float*>(smem + G * C::kGroupBytes);
  float* s_red = s_scales + C::kScaleBufs * kScaleStride;               // [4][NT]
  float* s_cs = s_red + 4 * NT;                                         // [NT] scale
  float* s_inv = s_cs + NT;                                             // [NT] 1 / scale
  uint64_t* full = reinterpret_cast<uint64_t*>(s_inv + NT);
  uint64_t* empty = full + G;
  uint64_t* tfull = empty + G;
  uint64_t* tempty = tfull + PAIRS;
  uint64_t* sfull = tempty + PAIRS;       // [3] mode 2: a scale buffer has landed
  uint64_t* sempty = sfull + 3;           // [3] mode 2: the epilogue is done with a scale buffer
  ExpertWork* s_work = reinterpret_cast<ExpertWork*>(sempty + 3);
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(s_work + kMaxLocalExperts);
  volatile int* s_abort = reinterpret_cast<volatile int*>(s_tmem + 1);
  int* s_meta = reinterpret_cast<int*>(s_tmem + 3);   // [2] token tiles, active experts (copied from p.meta)
  int* s_done = reinterpret_cast<int*>(s_tmem + 2);   // mode 1: epilogue warps that finished storing an item (running total); mode 2: items cleared for loading

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int trace_n = 0;
  (void)trace_n;
#ifdef SYFI_TRACE
  if (threadIdx.x == 0 && p.trace_cta != nullptr) {
    unsigned long long gt; unsigned smid;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(gt));
    asm volatile("mov.u32 %0, %smid;" : "=r"(smid));
    p.trace_cta[blockIdx.x * 5 + 0] = static_cast<long long>(gt);
    p.trace_cta[blockIdx.x * 5 + 2] = clock64();
    p.trace_cta[blockIdx.x * 5 + 4] = smid;
  }
#endif

  if (threadIdx.x == 0) {
    for (int i = 0; i < G; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
    for (int i = 0; i < PAIRS; ++i) { mbar_init(&tfull[i], 1); mbar_init(&tempty[i], 4 * C::kColSplit); }
    for (int i = 0; i < 3; ++i) { mbar_init(&sfull[i], 1); mbar_init(&sempty[i], 4 * C::kColSplit); }
    *s_abort = 0;
    *s_done = 0;
    fence_barrier_init();
    if (p.w_packed == nullptr) tma_prefetch_desc(&tm_w);
    tma_prefetch_desc(&tm_b0);
    if (MODE == 2) tma_prefetch_desc(&tm_b1);
    tma_prefetch_desc(&tm_b0s);
    if (MODE == 2) tma_prefetch_desc(&tm_b1s);
    if (MODE == 2) tma_prefetch_desc(&tm_sc);
  }
  if (warp == 1) {
    tmem_alloc(s_tmem, kTmemCols);
    tmem_relinquish();
  }
  // Everything above touched only this CTA's own resources; from here on the kernel reads what the
  // kernels before it in the stream produced.  Mode 1 waits for them as a whole.  Mode 2 does not wait
  // for GEMM1 as a whole: its CTAs start on the SMs GEMM1 has already left and its producer waits, per
  // work item, until GEMM1 has finished that item's expert (p.ready), so the tail of GEMM1 and the head
  // of GEMM2 overlap.  This cannot deadlock: a GEMM2 CTA only exists once every GEMM1 CTA has started
  // (that is when GEMM1 triggers its dependents), and GEMM1 CTAs wait for nothing.  The row tables and
  // counters GEMM2 reads here were complete before GEMM1 passed its own wait.
  if (MODE == 1) pdl_wait();
  pdl_trigger();
  // the work table and the two counters every role needs, fetched in one round trip
  if (threadIdx.x >= 64 && threadIdx.x < 64 + kMaxLocalExperts) {
    const int e = threadIdx.x - 64;
    s_work[e] = (e < p.e_local) ? p.work[e] : ExpertWork{0, 0, 0, 0};
  } else if (threadIdx.x == 64 + kMaxLocalExperts) {
    s_meta[0] = p.meta[0];                          // token tiles
    s_meta[1] = p.meta[3];                          // active experts
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *s_tmem;
  const int total = s_meta[0] * FT;                 // work items
  // Effective grid: the launch always has one CTA per SM, but when the items do not fill the last
  // round, fewer CTAs with equally many items each finish sooner than a last round that keeps only a
  // handful of SMs busy (a single SM cannot pull more than about 1.4x its fair share of HBM).  Only
  // taken when it costs at most a fifth of the SMs; the rest of the CTAs exit at once.
  int eff_grid = static_cast<int>(gridDim.x);
  {
    const int rounds = (total + eff_grid - 1) / eff_grid;
    const int even = rounds > 0 ? (total + rounds - 1) / rounds : eff_grid;   // CTAs needed for `rounds` each
    if (even * 5 >= eff_grid * 4) eff_grid = even;
  }
  const int my_items = (static_cast<int>(blockIdx.x) < eff_grid && static_cast<int>(blockIdx.x) < total)
                           ? (total - blockIdx.x + eff_grid - 1) / eff_grid : 0;
  auto item_of = [&](int i) { return static_cast<int>(blockIdx.x) + i * eff_grid; };   // this CTA's i-th item

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (one thread)
    if (lane == 0 && !p.silent_producer) {
      // a weight tile is re-read by the other token tiles of its expert (from L2) only when the
      // expert has several tiles; with a single tile per expert it is streamed exactly once
      const uint64_t pol_w = s_meta[0] > s_meta[1] ? l2_policy_evict_last() : l2_policy_evict_first();
      const uint64_t pol_b = l2_policy_evict_last();
      uint32_t it = 0, g = 0, ph = 0;      // step counter, ring entry, its phase
      uint32_t n_items = 0;                // items started (mode 2: selects the scale buffer)
      int e_hint = 0;
      bool alive = true;
      for (int i = 0; i < my_items && alive; ++i) {
        const Item im = decode_item<FT, NT>(s_work, p.e_local, item_of(i), e_hint);
        const int wrow = im.expert * C::kRowsPerExpert + im.ft * 128;
        // Tiles of at most 16 rows use the 16-row box: the token-side tiles come from L2 through the
        // same SM port as the weights, so every byte not fetched is bandwidth for the weight stream.
        const bool small = im.n <= 16;
        const CUtensorMap* mb0 = small ? &tm_b0s : &tm_b0;
        const CUtensorMap* mb1 = small ? &tm_b1s : &tm_b1;
        const uint32_t b_bytes = small ? 16 * 128 : kBTile;
        const uint32_t group_tx = KPS * (MODE == 1 ? 2 * kATile + b_bytes : kATile + 2 * b_bytes);
        if (MODE == 2) {
          // This item's expert must have left GEMM1 before its rows and scales are read; the helper
          // warp checks that (see there) and counts cleared items in shared memory, so the producer
          // itself never waits for a round trip to L2 nor executes a proxy fence with its ring in flight.
          if (*reinterpret_cast<volatile int*>(s_done) <= static_cast<int>(n_items)) {
            const long long t0 = clock64();
            while (*reinterpret_cast<volatile int*>(s_done) <= static_cast<int>(n_items)) {
              if (*s_abort != 0) { alive = false; break; }
              if (clock64() - t0 > p.wait_limit) { *s_abort = kStatusDependencyTimeout; alive = false; break; }
            }
            if (!alive) break;
          }
          __threadfence_block();
          // scales of the item: [16 K blocks x NT rows] activation scales through a tensor map and the
          // 16 weight scales as a 64-byte bulk copy, into the buffer the epilogue released three items ago
          const uint32_t sb = n_items % 3u, sp = (n_items / 3u) & 1u;
          if (!mbar_wait_bounded(&sempty[sb], sp ^ 1u, s_abort, kStatusWaitTimeoutProducer, p.wait_limit)) { alive = false; break; }
          float* d_act = s_scales + sb * kScaleStride;
          mbar_arrive_expect_tx(&sfull[sb], (KB * NT + KB) * 4);
          tma_load_2d(d_act, &tm_sc, &sfull[sb], im.row_start, 0, pol_b);
          bulk_load(d_act + KB * NT, p.w_scale + (static_cast<size_t>(im.expert) * kHBlocks + im.ft) * kIBlocks,
                    KB * 4, &sfull[sb], pol_b);
          ++n_items;
        }
        for (int step = 0; step < STEPS; ++step) {
          if (!mbar_wait_bounded(&empty[g], ph ^ 1u, s_abort, kStatusWaitTimeoutProducer, p.wait_limit)) { alive = false; break; }
          TRACE(0, step);
          mbar_arrive_expect_tx(&full[g], group_tx);
          // The boxes that continue each other along K (same rows, next 128 bytes) are issued back to
          // back: L2 serves a row's 256 contiguous bytes far faster than two separate 128-byte visits.
          uint8_t* st0 = smem + g * C::kGroupBytes;
          const int x0 = step * KPS * 128;
          if (p.w_packed != nullptr) {
            if (MODE == 1) {            // 32 KB per K block: up tile, gate tile
              const uint8_t* src = p.w_packed + (static_cast<size_t>(im.expert * FT + im.ft) * KB + step * KPS) * (2 * kATile);
#pragma unroll
              for (int k = 0; k < KPS; ++k)
                bulk_load(st0 + w_off(k), src + static_cast<size_t>(k) * 2 * kATile, 2 * kATile, &full[g], pol_w);
            } else {                    // the K blocks of a step are adjacent: one copy
              const uint8_t* src = p.w_packed + (static_cast<size_t>(im.expert * FT + im.ft) * KB + step * KPS) * kATile;
              bulk_load(st0, src, KPS * kATile, &full[g], pol_w);
            }
          } else {
#pragma unroll
            for (int k = 0; k < KPS; ++k) tma_load_2d(st0 + w_off(k), &tm_w, &full[g], x0 + k * 128, wrow, pol_w);
            if (MODE == 1) {
#pragma unroll
              for (int k = 0; k < KPS; ++k)
                tma_load_2d(st0 + w_off(k) + kATile, &tm_w, &full[g], x0 + k * 128, wrow + kInter, pol_w);
            }
          }
#pragma unroll
          for (int k = 0; k < KPS; ++k) tma_load_2d(st0 + b_off(k), mb0, &full[g], x0 + k * 128, im.row_start, pol_b);
          if (MODE == 2) {
#pragma unroll
            for (int k = 0; k < KPS; ++k)
              tma_load_2d(st0 + b_off(k) + kBTile, mb1, &full[g], x0 + k * 128, im.row_start, pol_b);
          }
          ++it;
          if (++g == G) { g = 0; ph ^= 1u; }
        }
      }
      // drain: every ring entry this thread armed must have landed before the CTA may exit
      const uint32_t first = it > static_cast<uint32_t>(G) ? it - G : 0;
      for (uint32_t i = first; i < it; ++i)
        mbar_wait_bounded(&full[i % G], (i / G) & 1, s_abort, kStatusWaitTimeoutProducer, 1ll << 28);
    }
    __syncwarp();
  } else if (warp == 1) {
    // --------------------------------------------------------------- MMA issuer (one thread)
    if (lane == 0) {
      uint32_t g = 0, ph = 0, pr = 0, pph = 0;   // smem ring entry / phase, TMEM ring entry / phase
      int e_hint = 0;
      bool alive = true;
      for (int i = 0; i < my_items && alive; ++i) {
        const Item im = decode_item<FT, NT>(s_work, p.e_local, item_of(i), e_hint);
        // Mode 2 issues ONE MMA of N = 2 NT per 32 bytes of K over the adjacent hi and lo tiles
        // (the columns past the tile's n rows hold other rows' data and are never read back)
        // instead of one per term; mode 1 needs two because up and gate are different A tiles.
        const uint32_t idesc = umma_idesc_e4m3_m128(MODE == 1 ? static_cast<uint32_t>(im.n) : 2u * NT);
        for (int step = 0; step < STEPS; ++step) {
          if (!mbar_wait_bounded(&full[g], ph, s_abort, kStatusWaitTimeoutMma, p.wait_limit)) { alive = false; break; }
          TRACE(1, step);
#pragma unroll
          for (int tk = 0; tk < KPS / TKPS && alive; ++tk) {
            if (!mbar_wait_bounded(&tempty[pr], pph ^ 1u, s_abort, kStatusWaitTimeoutMma, p.wait_limit)) { alive = false; break; }
            tc_fence_after();
#pragma unroll
            for (int k2 = 0; k2 < TKPS; ++k2) {
              const int k = tk * TKPS + k2;
              const uint32_t gb = smem_u32(smem + g * C::kGroupBytes);
              const uint32_t d0 = tmem_base + (pr * TKPS + k2) * (2 * NT);
              if (MODE == 1) {
                const uint64_t a0 = umma_smem_desc_sw128(gb + w_off(k));
                const uint64_t a1 = umma_smem_desc_sw128(gb + w_off(k) + kATile);
                const uint64_t b0 = umma_smem_desc_sw128(gb + b_off(k));
#pragma unroll
                for (int k4 = 0; k4 < 4; ++k4) {
                  // 32 bytes of K per MMA: +2 in the 16-byte-unit address field
                  umma_f8(d0, a0 + 2 * k4, b0 + 2 * k4, idesc, k4 > 0 ? 1u : 0u);
                  umma_f8(d0 + NT, a1 + 2 * k4, b0 + 2 * k4, idesc, k4 > 0 ? 1u : 0u);
                }
              } else {
                const uint64_t a0 = umma_smem_desc_sw128(gb + w_off(k));
                const uint64_t b0 = umma_smem_desc_sw128(gb + b_off(k));   // hi rows, then lo rows
#pragma unroll
                for (int k4 = 0; k4 < 4; ++k4) umma_f8(d0, a0 + 2 * k4, b0 + 2 * k4, idesc, k4 > 0 ? 1u : 0u);
              }
            }
            if (tk == KPS / TKPS - 1) umma_commit(&empty[g]);
            umma_commit(&tfull[pr]);
            if (++pr == PAIRS) { pr = 0; pph ^= 1u; }
          }
          if (!alive) break;
          if (++g == G) { g = 0; ph ^= 1u; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 2 + 4 * C::kColSplit) {
    // ------------------------------------------------ publisher (mode 1, one thread)
    // GEMM2 reads an expert's rows once p.ready[expert] has counted all of the expert's GEMM1 items.
    // An item counts when every epilogue warp has issued its stores (s_done) and a gpu-scope fence has
    // made them visible; that fence waits for the stores to be acknowledged (microseconds while HBM is
    // saturated), which is why it runs here and not in an epilogue warp.
    //
    // The ordering chain from GEMM1's stores to GEMM2's TMA loads, link by link:
    //   1. epilogue threads: generic-proxy stores of c_hi / c_lo / c_scale, then __threadfence_block(),
    //      then one atomicAdd on s_done per warp (CTA scope: stores before the count);
    //   2. this lane: volatile read of s_done (observes the counts, hence the stores, by causality at
    //      CTA scope), __threadfence() (cumulative: lifts what it observed to gpu scope),
    //      fence.proxy.async (generic-proxy writes ordered before later async-proxy accesses),
    //      red.release.gpu on ready[expert];
    //   3. GEMM2's helper lane: ld.acquire.gpu of ready[expert] (synchronises with every release of 2),
    //      fence.proxy.async, __threadfence_block(), volatile store of the cleared-item count to s_done;
    //   4. GEMM2's producer lane: volatile read of that count, __threadfence_block(), then the TMA loads.
    // Links 2 and 3 put a proxy fence on both sides of the release/acquire pair; links 1 and 4 are plain
    // CTA-scope causality, which the fences of 2 and 3 extend because fences are cumulative.  The fences
    // are executed by the publishing / acquiring lanes, not by the threads that store or that issue the
    // loads; the back-to-back bit-identity test exercises exactly this hand-off.
    if (MODE == 1 && lane == 0) {
      int done_target = 0, e_hint = 0;
      for (int i = 0; i < my_items; ++i) {
        const Item im = decode_item<FT, NT>(s_work, p.e_local, item_of(i), e_hint);
        done_target += 4 * C::kColSplit;
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
    // ------------------------------------------------ dependency helper (mode 2, one thread)
    // Clears this CTA's items one by one: item i may be loaded once GEMM1 has counted all items of its
    // expert.  The acquire load and the proxy fence (generic-proxy stores of GEMM1 before async-proxy
    // loads of this kernel) run here; the producer only reads the count of cleared items (s_done).
    if (MODE == 2 && lane == 0) {
      int cleared = 0, ready_expert = -1, e_hint = 0;
      for (int i = 0; i < my_items; ++i) {
        const Item im = decode_item<FT, NT>(s_work, p.e_local, item_of(i), e_hint);
        if (im.expert != ready_expert) {
          const int need = (kInter / 128) * s_work[im.expert].tiles;
          const long long t0 = clock64();
          bool seen = true;
          while (ld_acquire_gpu(p.ready + im.expert) < need) {
            if (*s_abort != 0) { seen = false; break; }
            if (clock64() - t0 > (p.wait_limit >> 1)) { *s_abort = kStatusDependencyTimeout; seen = false; break; }   // half the other roles' limit: this wait reports first
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
  } else {
    // ------------------------------------------------ promotion + epilogue warps
    // CS warps share each TMEM lane quarter and split the tile's columns between them, so a thread
    // owns one feature and CN = NT / CS token columns.
    constexpr int CS = C::kColSplit;
    constexpr int CN = NT / CS;
    constexpr int kEpi = 128 * CS;          // epilogue threads
    static_assert(CN == 16 || CN == 32, "the drain below moves 16 or 32 columns per thread and step");
    const int q = warp & 3;                 // TMEM lane quarter this warp may read
    const int c0 = ((warp - 2) >> 2) * CN;  // first column of this thread's share
    const int et = threadIdx.x - 64;        // 0..kEpi-1 among the epilogue threads
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    uint32_t pr = 0, pph = 0;               // TMEM ring entry and its phase
    bool ok = true;
    int sbuf = 0;
    int cached_row_start = -1;              // token tile whose activation scales sit in shared memory (mode 1)
    int e_hint = 0;
    uint32_t sph = 0;                       // phase bits of sfull[0..2] (mode 2)
    // After a failed wait a warp keeps walking the work list and still joins every named
    // barrier below (doing no other work), so the epilogue warps can never strand each other.
    for (int i = 0; i < my_items; ++i) {
      const Item im = decode_item<FT, NT>(s_work, p.e_local, item_of(i), e_hint);
      const int ft = im.ft;
      const int n = ok ? im.n : 0;
      if (et == 0) TRACE(2, 1000);
      float* s_act;
      float* s_ws;
      if (MODE == 1) {
        s_act = s_scales;
        s_ws = s_scales + KB * NT;
        named_bar_sync(1, kEpi);            // previous item's readers of the staging arrays are done
        // the activation scales depend on the token tile only: consecutive items of a CTA mostly
        // share it (same expert, next feature tile), so they are reloaded only when it changes
        if (im.row_start != cached_row_start) {
          constexpr int kIters = (KB * NT + kEpi - 1) / kEpi;
          float tmp[kIters];
#pragma unroll
          for (int r = 0; r < kIters; ++r) {   // all loads in flight before the first store
            const int i = et + r * kEpi;
            const int kb = i / NT, j = i % NT;
            tmp[r] = (i < KB * NT && j < n) ? __ldg(p.act_scale + static_cast<size_t>(kb) * p.row_cap + im.row_start + j) : 0.0f;
          }
#pragma unroll
          for (int r = 0; r < kIters; ++r)
            if (et + r * kEpi < KB * NT) s_act[et + r * kEpi] = tmp[r];
          cached_row_start = ok ? im.row_start : -1;
        }
        if (et < KB && ok) {
          s_ws[et] = __ldg(p.w_scale + (static_cast<size_t>(im.expert) * 32 + ft) * kHBlocks + et);
          s_ws[64 + et] = __ldg(p.w_scale + (static_cast<size_t>(im.expert) * 32 + 16 + ft) * kHBlocks + et);
        }
        named_bar_sync(1, kEpi);
      } else {
        // The producer requested this item's scales when it started the item (it runs about one item
        // ahead of the epilogue); the buffer goes back to it after the K loop.  Columns >= n hold other
        // rows' scales and are never read.
        s_act = s_scales + sbuf * kScaleStride;
        s_ws = s_act + KB * NT;
        if (ok && !mbar_wait_bounded(&sfull[sbuf], (sph >> sbuf) & 1u, s_abort, kStatusWaitTimeoutEpilogue, p.wait_limit)) ok = false;
        sph ^= 1u << sbuf;
      }
      if (et == 0) TRACE(2, 1001);

      // accumulators as packed f32 pairs (columns 2i, 2i + 1) while the K loop runs
      uint64_t acc0p[CN / 2];                   // mode 1: up,   mode 2: output
      uint64_t acc1p[MODE == 1 ? CN / 2 : 1];   // mode 1: gate
#pragma unroll
      for (int j = 0; j < CN / 2; ++j) acc0p[j] = 0ull;
      if (MODE == 1) {
#pragma unroll
        for (int j = 0; j < CN / 2; ++j) acc1p[j] = 0ull;
      }

      // One promotion step: sixteen columns of one or both accumulators of a K block into the registers,
      // two columns per instruction.  `sa` points at the sixteen activation scales (16-byte aligned).
      auto promote16 = [&](const uint32_t (&r0)[16], const uint32_t (&r1)[16], int cbase, const float* sa,
                           uint64_t ws0, uint64_t ws1, int sel) {   // mode 1: sel 0 = up, 1 = gate, 2 = both
        const ulonglong2* sp = reinterpret_cast<const ulonglong2*>(sa);
        const uint64_t inv_ratio = f32x2_pack(1.0f / kLoRatio, 1.0f / kLoRatio);
#pragma unroll
        for (int j4 = 0; j4 < 4; ++j4) {
          const ulonglong2 a4 = sp[j4];         // scales of four columns
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int j = j4 * 4 + h * 2, ai = (cbase + j) / 2;
            const uint64_t a = h == 0 ? a4.x : a4.y;
            const uint64_t v0 = f32x2_pack_bits(r0[j], r0[j + 1]);
            if (MODE == 1) {
              if (sel != 1) acc0p[ai] = f32x2_fma(v0, f32x2_mul(a, ws0), acc0p[ai]);
              if (sel != 0) acc1p[ai] = f32x2_fma(f32x2_pack_bits(r1[j], r1[j + 1]), f32x2_mul(a, ws1), acc1p[ai]);
            } else {
              const uint64_t v = f32x2_fma(f32x2_pack_bits(r1[j], r1[j + 1]), inv_ratio, v0);
              acc0p[ai] = f32x2_fma(v, f32x2_mul(a, ws0), acc0p[ai]);
            }
          }
        }
      };
      for (int ts = 0; ts < STEPS * (KPS / TKPS) && ok; ++ts) {
        if (!mbar_wait_bounded(&tfull[pr], pph, s_abort, kStatusWaitTimeoutEpilogue, p.wait_limit)) { ok = false; break; }
        tc_fence_after();
        if (et == 0) TRACE(2, ts);
#pragma unroll
        for (int k = 0; k < TKPS; ++k) {
          const int kb = ts * TKPS + k;
          const uint32_t t0 = lane_addr + (pr * TKPS + k) * (2 * NT) + c0;
          const uint64_t ws0 = f32x2_pack(s_ws[kb], s_ws[kb]);
          const uint64_t ws1 = (MODE == 1) ? f32x2_pack(s_ws[64 + kb], s_ws[64 + kb]) : 0ull;
          const float* sa = s_act + kb * NT + c0;
          if (c0 < n) {
            if constexpr (CN == 16) {         // both accumulators of this thread's 16 columns in flight
              uint32_t r0[16], r1[16];
              tmem_ld16(t0, r0);
              tmem_ld16(t0 + NT, r1);
              tmem_ld_wait();
              promote16(r0, r1, 0, sa, ws0, ws1, 2);
            } else if constexpr (NT == 128 && MODE == 1) {
              // 18 warps share the register file and 64 registers of a thread hold accumulators: eight
              // columns of one accumulator at a time
#pragma unroll
              for (int c = 0; c < 4; ++c) {
                if (c0 + c * 8 < n) {
                  const ulonglong2* sp = reinterpret_cast<const ulonglong2*>(sa + c * 8);
                  const ulonglong2 s03 = sp[0], s47 = sp[1];
                  uint32_t r[8];
                  tmem_ld8(t0 + c * 8, r);
                  tmem_ld_wait();
                  acc0p[c * 4 + 0] = f32x2_fma(f32x2_pack_bits(r[0], r[1]), f32x2_mul(s03.x, ws0), acc0p[c * 4 + 0]);
                  acc0p[c * 4 + 1] = f32x2_fma(f32x2_pack_bits(r[2], r[3]), f32x2_mul(s03.y, ws0), acc0p[c * 4 + 1]);
                  acc0p[c * 4 + 2] = f32x2_fma(f32x2_pack_bits(r[4], r[5]), f32x2_mul(s47.x, ws0), acc0p[c * 4 + 2]);
                  acc0p[c * 4 + 3] = f32x2_fma(f32x2_pack_bits(r[6], r[7]), f32x2_mul(s47.y, ws0), acc0p[c * 4 + 3]);
                  tmem_ld8(t0 + NT + c * 8, r);
                  tmem_ld_wait();
                  acc1p[c * 4 + 0] = f32x2_fma(f32x2_pack_bits(r[0], r[1]), f32x2_mul(s03.x, ws1), acc1p[c * 4 + 0]);
                  acc1p[c * 4 + 1] = f32x2_fma(f32x2_pack_bits(r[2], r[3]), f32x2_mul(s03.y, ws1), acc1p[c * 4 + 1]);
                  acc1p[c * 4 + 2] = f32x2_fma(f32x2_pack_bits(r[4], r[5]), f32x2_mul(s47.x, ws1), acc1p[c * 4 + 2]);
                  acc1p[c * 4 + 3] = f32x2_fma(f32x2_pack_bits(r[6], r[7]), f32x2_mul(s47.y, ws1), acc1p[c * 4 + 3]);
                }
              }
            } else if constexpr (NT == 128) {
#pragma unroll
              for (int c = 0; c < 2; ++c) {
                if (c0 + c * 16 < n) {
                  uint32_t r0[16], r1[16];
                  tmem_ld16(t0 + c * 16, r0);
                  tmem_ld16(t0 + NT + c * 16, r1);
                  tmem_ld_wait();
                  promote16(r0, r1, c * 16, sa + c * 16, ws0, ws1, 2);
                }
              }
            } else {                          // this thread's 32 columns: four loads in flight, one wait
              uint32_t v0[2][16], v1[2][16];
              tmem_ld16(t0, v0[0]);
              tmem_ld16(t0 + NT, v1[0]);
              if (c0 + 16 < n) {
                tmem_ld16(t0 + 16, v0[1]);
                tmem_ld16(t0 + NT + 16, v1[1]);
              }
              tmem_ld_wait();
              promote16(v0[0], v1[0], 0, sa, ws0, ws1, 2);
              if (c0 + 16 < n) promote16(v0[1], v1[1], 16, sa + 16, ws0, ws1, 2);
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty[pr]);
        if (++pr == PAIRS) { pr = 0; pph ^= 1u; }
      }
      if (et == 0) TRACE(2, 1002);
      if (MODE == 2) {                        // the scale buffer goes back to the producer
        __syncwarp();
        if (lane == 0) mbar_arrive(&sempty[sbuf]);
        sbuf = sbuf == 2 ? 0 : sbuf + 1;
      }
      const int n_out = ok ? n : 0;           // a failed item stores nothing
      float acc0[CN];
      float acc1[MODE == 1 ? CN : 1];
#pragma unroll
      for (int j = 0; j < CN / 2; ++j) f32x2_unpack(acc0p[j], acc0[2 * j], acc0[2 * j + 1]);
      if (MODE == 1) {
#pragma unroll
        for (int j = 0; j < CN / 2; ++j) f32x2_unpack(acc1p[j], acc1[2 * j], acc1[2 * j + 1]);
      }

      if (MODE == 1) {
        // SwiGLU, then the per-row amax over the 128 features of this tile.  The fast exp and
        // divide are a few ulp off the exact ones, far below the 8-bit requantisation that follows.
        // (n is a multiple of 16, so validity is decided per block of sixteen columns and the
        // sixteen columns inside a block run without branches between them)
#pragma unroll
        for (int jb = 0; jb < CN; jb += 16) {
          if (c0 + jb < n_out) {
            float mx[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const float gt = acc1[jb + j];
              const float cv = gt * __fdividef(1.0f, 1.0f + __expf(-gt)) * acc0[jb + j];
              acc0[jb + j] = cv;
              mx[j] = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(fabsf(cv))));
            }
            if (lane == 0) {
              float4* dst = reinterpret_cast<float4*>(s_red + q * NT + c0 + jb);
#pragma unroll
              for (int j = 0; j < 4; ++j) dst[j] = make_float4(mx[4 * j], mx[4 * j + 1], mx[4 * j + 2], mx[4 * j + 3]);
            }
          }
        }
        named_bar_sync(2, kEpi);
        if (et < n_out) {
          const float amax = fmaxf(fmaxf(s_red[et], s_red[NT + et]), fmaxf(s_red[2 * NT + et], s_red[3 * NT + et]));
          const float sc = fmaxf(amax * (1.0f / 448.0f), 1e-12f);
          s_cs[et] = sc;
          s_inv[et] = 1.0f / sc;
          p.c_scale[static_cast<size_t>(ft) * p.row_cap + im.row_start + et] = sc;
        }
        named_bar_sync(2, kEpi);
        // Quantise four token rows at a time into packed bytes, transpose across the lane quad so a
        // lane holds four adjacent features of ONE row, and store 4 bytes per lane: n/4 store
        // instructions per tensor instead of n byte stores.
        const int qrow = lane & 3;              // which of the four rows this lane stores
        const size_t qoff = static_cast<size_t>(ft) * 128 + q * 32 + (lane >> 2) * 4;
#pragma unroll
        for (int j = 0; j < CN; j += 4) {
          if (c0 + (j & ~15) < n_out) {
            uint32_t hp = 0, lp = 0;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const int c = j + 2 * h;
              const float sc0 = s_cs[c0 + c], sc1 = s_cs[c0 + c + 1];
              const float in0 = s_inv[c0 + c], in1 = s_inv[c0 + c + 1];
              const float v0 = acc0[c], v1 = acc0[c + 1];
              const uint16_t hh = cvt_e4m3x2(v0 * in0, v1 * in1);
              const float2 hb = e4m3x2_to_float2(hh);
              const float r0 = fmaf(-hb.x, sc0, v0), r1 = fmaf(-hb.y, sc1, v1);
              const uint16_t ll = cvt_e4m3x2(r0 * in0 * kLoRatio, r1 * in1 * kLoRatio);
              hp |= static_cast<uint32_t>(hh) << (16 * h);
              lp |= static_cast<uint32_t>(ll) << (16 * h);
            }
            hp = quad_transpose_bytes(hp, lane);
            lp = quad_transpose_bytes(lp, lane);
            const size_t off = static_cast<size_t>(im.row_start + c0 + j + qrow) * kInter + qoff;
            *reinterpret_cast<uint32_t*>(p.c_hi + off) = hp;
            *reinterpret_cast<uint32_t*>(p.c_lo + off) = lp;
          }
        }
        // Hand the item to the publisher warp, which makes it visible to GEMM2 (see there): waiting
        // here for the stores to be acknowledged would stall the promotion of the next item.
        __threadfence_block();
        __syncwarp();
        if (lane == 0) atomicAdd(s_done, 1);
      } else {
        const int qrow = lane & 3;
        const int row0 = im.row_start + c0 + qrow;
        const int col = ft * 128 + q * 32 + (lane >> 2) * 4;
#pragma unroll
        for (int j = 0; j < CN; j += 4) {
          if (c0 + j < n_out) {
            float a0 = acc0[j], a1 = acc0[j + 1], a2 = acc0[j + 2], a3 = acc0[j + 3];
            quad_transpose_f32(a0, a1, a2, a3, lane);   // now: row c0 + j + qrow, four adjacent features
            // expert parallelism: the row's place in its token owner's memory (plain stores over NVLink)
            float* o = p.row_out != nullptr ? p.row_out[row0 + j] : p.o_rows + static_cast<size_t>(row0 + j) * kHidden;
            if (o != nullptr) *reinterpret_cast<float4*>(o + col) = make_float4(a0, a1, a2, a3);
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
  if (threadIdx.x == 0 && *s_abort != 0) atomicExch(p.status, *s_abort);
#ifdef SYFI_TRACE
  if (threadIdx.x == 0 && p.trace_cta != nullptr) {
    unsigned long long gt;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(gt));
    p.trace_cta[blockIdx.x * 5 + 1] = static_cast<long long>(gt);
    p.trace_cta[blockIdx.x * 5 + 3] = clock64();
  }
#endif
}

template <int MODE, int NT>
cudaError_t launch_gemm(const GemmLaunch& g, const GemmArgs& a, int num_sms, cudaStream_t st) {
  return launch_dependent(grouped_gemm_kernel<MODE, NT>, dim3(num_sms), dim3(Cfg<MODE, NT>::kThreads),
                          static_cast<size_t>(Cfg<MODE, NT>::kSmemBytes), st, g.tm_w, g.tm_b0, g.tm_b1, g.tm_b0s,
                          g.tm_b1s, g.tm_sc, a);
}

template <int MODE, int NT>
cudaError_t set_smem_attr() {
  return cudaFuncSetAttribute(grouped_gemm_kernel<MODE, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              Cfg<MODE, NT>::kSmemBytes);
}

}  // namespace

cudaError_t gemm_set_attributes() {
  cudaError_t e;
  if ((e = set_smem_attr<1, 32>()) != cudaSuccess) return e;
  if ((e = set_smem_attr<1, 64>()) != cudaSuccess) return e;
  if ((e = set_smem_attr<1, 128>()) != cudaSuccess) return e;
  if ((e = set_smem_attr<2, 32>()) != cudaSuccess) return e;
  if ((e = set_smem_attr<2, 64>()) != cudaSuccess) return e;
  return set_smem_attr<2, 128>();
}

cudaError_t launch_gemm1(const GemmLaunch& g, const float* w13_scale, int e_local, const Workspace& ws, int num_sms,
                         cudaStream_t st) {
  GemmArgs a{g.w_packed, ws.work, ws.meta, ws.a_scale, w13_scale, ws.c_hi, ws.c_lo, ws.c_scale, nullptr, ws.row_cap, e_local,
             ws.ready, ws.status, ws.trace, ws.trace + 6 * 4096, g.wait_limit, g.silent_producer, nullptr};
  if (g.token_tile == 128) return launch_gemm<1, 128>(g, a, num_sms, st);
  return g.token_tile == 32 ? launch_gemm<1, 32>(g, a, num_sms, st) : launch_gemm<1, 64>(g, a, num_sms, st);
}

cudaError_t launch_gemm2(const GemmLaunch& g, const float* w2_scale, int e_local, const Workspace& ws, int num_sms,
                         cudaStream_t st) {
  GemmArgs a{g.w_packed, ws.work, ws.meta, ws.c_scale, w2_scale, nullptr, nullptr, nullptr, ws.o_rows, ws.row_cap, e_local,
             ws.ready, ws.status, ws.trace + 3 * 4096, ws.trace + 7 * 4096, g.wait_limit, g.silent_producer,
             g.rows_to_targets ? ws.row_out : nullptr};
  if (g.token_tile == 128) return launch_gemm<2, 128>(g, a, num_sms, st);
  return g.token_tile == 32 ? launch_gemm<2, 32>(g, a, num_sms, st) : launch_gemm<2, 64>(g, a, num_sms, st);
}

}  // namespace syfi
