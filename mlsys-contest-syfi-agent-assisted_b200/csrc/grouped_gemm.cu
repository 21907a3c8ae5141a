// Grouped FP8 block-scale GEMMs of the MoE layer on tcgen05 (sm_100a).
//
// GEMM1 (mode 1) replaces gemm_fp8_fp8_tcgen05_grouped_kernel / gemm_fp8_fp8_grouped_kernel
// plus swiglu_quant_fp8_kernel of the reference (moe/solution/cuda/moe.cu:2194-2350,
// 1461-1627, 1631-1714); GEMM2 (mode 2) replaces gemm_fp8_fp8_fused_acc_grouped_kernel
// (moe.cu:1718-1887).
//
// Orientation ("swap-AB"): the WEIGHT tile is the 128-row M operand of the MMA and the
// expert's token rows are the N operand (16..64 columns), so an expert with a handful of
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
// Pipeline per CTA (persistent over work items, 6 warps): warp 0 = TMA producer (weights
// with an evict-first L2 policy, token-side tiles evict-last), warp 1 = MMA issuer and TMEM
// owner, warps 2-5 = promotion/epilogue (one TMEM lane quarter each).  Shared-memory stages
// form a ring guarded by full/empty mbarriers; the TMEM accumulator pair is double
// buffered (tfull/tempty) so the MMAs of K block k+1 overlap the promotion of block k.
// Every wait is bounded: on expiry the CTA raises an abort flag, all roles leave their
// loops, TMEM is released and the status word reports the failure to the host.
#include <cuda_fp16.h>

#include "moe_internal.h"
#include "ptx.cuh"

namespace syfi {

namespace {

constexpr int NT = kTokenTile;            // token columns per work item
constexpr int kGemmThreads = 192;
constexpr int kEpiThreads = 128;
constexpr int kATile = 128 * 128;         // weight tile: 128 rows x 128 bytes of K
constexpr int kBTile = NT * 128;          // token-side tile
constexpr int kTmemCols = 4 * NT;         // two accumulators x two buffers

template <int MODE> struct Cfg;
template <> struct Cfg<1> {
  static constexpr int kKBlocks = kHBlocks;            // 56
  static constexpr int kFeatTiles = kInter / 128;      // 16
  static constexpr int kRowsPerExpert = 2 * kInter;    // rows of W13 per expert
  static constexpr int kStages = 5;
  static constexpr int kStageBytes = 2 * kATile + kBTile;
};
template <> struct Cfg<2> {
  static constexpr int kKBlocks = kIBlocks;            // 16
  static constexpr int kFeatTiles = kHidden / 128;     // 56
  static constexpr int kRowsPerExpert = kHidden;
  static constexpr int kStages = 6;
  static constexpr int kStageBytes = kATile + 2 * kBTile;
};

template <int MODE>
constexpr int smem_bytes() {
  using C = Cfg<MODE>;
  return 1024 /* alignment slack */ + C::kStages * C::kStageBytes + 4 * (C::kKBlocks * NT + 128 + 4 * NT + 2 * NT) +
         8 * (2 * C::kStages + 4) + 16;
}

struct GemmArgs {
  const TokenTile* tiles;
  const int* meta;
  const float* act_scale;   // [K blocks][row_cap] scales of the token-side operand
  const float* w_scale;     // mode 1: [E][32][56], mode 2: [E][56][16]
  uint8_t* c_hi;            // mode 1 outputs
  uint8_t* c_lo;
  float* c_scale;           // [16][row_cap]
  float* o_rows;            // mode 2 output [row_cap][7168]
  int row_cap;
  int* status;
};

template <int MODE>
__global__ void __launch_bounds__(kGemmThreads, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_b0,
                    const __grid_constant__ CUtensorMap tm_b1, const GemmArgs p) {
  using C = Cfg<MODE>;
  constexpr int S = C::kStages;
  constexpr int KB = C::kKBlocks;
  constexpr int FT = C::kFeatTiles;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  float* s_act = reinterpret_cast<float*>(smem + S * C::kStageBytes);   // [KB][NT]
  float* s_ws = s_act + KB * NT;                                        // [2][64]
  float* s_red = s_ws + 128;                                            // [4][NT]
  float* s_cs = s_red + 4 * NT;                                         // [NT] scale
  float* s_inv = s_cs + NT;                                             // [NT] 1 / scale
  uint64_t* full = reinterpret_cast<uint64_t*>(s_inv + NT);
  uint64_t* empty = full + S;
  uint64_t* tfull = empty + S;
  uint64_t* tempty = tfull + 2;
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* s_abort = reinterpret_cast<volatile int*>(s_tmem + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < S; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&tfull[i], 1); mbar_init(&tempty[i], 4); }
    *s_abort = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tm_w);
    tma_prefetch_desc(&tm_b0);
    if (MODE == 2) tma_prefetch_desc(&tm_b1);
  }
  if (warp == 1) {
    tmem_alloc(s_tmem, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *s_tmem;
  const int total = p.meta[0] * FT;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    const uint64_t pol_w = l2_policy_evict_first();
    const uint64_t pol_b = l2_policy_evict_last();
    uint32_t it = 0;
    for (int w = blockIdx.x; w < total; w += gridDim.x) {
      const TokenTile tt = p.tiles[w / FT];
      const int ft = w % FT;
      const int wrow = tt.expert * C::kRowsPerExpert + ft * 128;
      for (int kb = 0; kb < KB; ++kb) {
        if (lane == 0) {
          const int s = it % S;
          if (mbar_wait_bounded(&empty[s], ((it / S) & 1) ^ 1, s_abort, kStatusWaitTimeoutProducer)) {
            uint8_t* st = smem + s * C::kStageBytes;
            mbar_arrive_expect_tx(&full[s], C::kStageBytes);
            if (MODE == 1) {
              tma_load_2d(st, &tm_w, &full[s], kb * 128, wrow, pol_w);
              tma_load_2d(st + kATile, &tm_w, &full[s], kb * 128, wrow + kInter, pol_w);
              tma_load_2d(st + 2 * kATile, &tm_b0, &full[s], kb * 128, tt.row_start, pol_b);
            } else {
              tma_load_2d(st, &tm_w, &full[s], kb * 128, wrow, pol_w);
              tma_load_2d(st + kATile, &tm_b0, &full[s], kb * 128, tt.row_start, pol_b);
              tma_load_2d(st + kATile + kBTile, &tm_b1, &full[s], kb * 128, tt.row_start, pol_b);
            }
            ++it;
          }
        }
        __syncwarp();
        if (*s_abort) break;
      }
      if (*s_abort) break;
    }
    // drain: every stage this warp armed must have landed before the CTA may exit
    if (lane == 0) {
      const uint32_t first = it > static_cast<uint32_t>(S) ? it - S : 0;
      for (uint32_t i = first; i < it; ++i)
        mbar_wait_bounded(&full[i % S], (i / S) & 1, s_abort, kStatusWaitTimeoutProducer, 1ll << 28);
    }
    __syncwarp();
  } else if (warp == 1) {
    // --------------------------------------------------------------- MMA issuer
    uint32_t it = 0, ab = 0;
    for (int w = blockIdx.x; w < total; w += gridDim.x) {
      const TokenTile tt = p.tiles[w / FT];
      const uint32_t idesc = umma_idesc_e4m3_m128(static_cast<uint32_t>(tt.n));
      for (int kb = 0; kb < KB; ++kb, ++it, ++ab) {
        if (lane == 0) {
          const int s = it % S;
          const uint32_t buf = ab & 1u;
          if (mbar_wait_bounded(&full[s], (it / S) & 1, s_abort, kStatusWaitTimeoutMma) &&
              mbar_wait_bounded(&tempty[buf], ((ab >> 1) & 1u) ^ 1u, s_abort, kStatusWaitTimeoutMma)) {
            tc_fence_after();
            const uint32_t st = smem_u32(smem + s * C::kStageBytes);
            const uint32_t d0 = tmem_base + buf * (2 * NT);
            const uint32_t d1 = d0 + NT;
            uint64_t a0, a1, b0, b1;
            if (MODE == 1) {
              a0 = umma_smem_desc_sw128(st);
              a1 = umma_smem_desc_sw128(st + kATile);
              b0 = umma_smem_desc_sw128(st + 2 * kATile);
              b1 = b0;
            } else {
              a0 = umma_smem_desc_sw128(st);
              a1 = a0;
              b0 = umma_smem_desc_sw128(st + kATile);
              b1 = umma_smem_desc_sw128(st + kATile + kBTile);
            }
#pragma unroll
            for (int k4 = 0; k4 < 4; ++k4) {
              // 32 bytes of K per MMA: +2 in the 16-byte-unit address field
              umma_f8(d0, a0 + 2 * k4, b0 + 2 * k4, idesc, k4 > 0 ? 1u : 0u);
              umma_f8(d1, a1 + 2 * k4, b1 + 2 * k4, idesc, k4 > 0 ? 1u : 0u);
            }
            umma_commit(&empty[s]);
            umma_commit(&tfull[buf]);
          }
        }
        __syncwarp();
        if (*s_abort) break;
      }
      if (*s_abort) break;
    }
  } else {
    // ------------------------------------------------ promotion + epilogue warps
    const int q = warp & 3;                 // TMEM lane quarter this warp may read
    const int feat = q * 32 + lane;         // feature (row of the weight tile) of this thread
    const int et = threadIdx.x - 64;        // 0..127 among the epilogue threads
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    uint32_t ab = 0;
    bool ok = true;
    // After a failed wait a warp keeps walking the work list and still joins every named
    // barrier below (doing no other work), so the four warps can never strand each other.
    for (int w = blockIdx.x; w < total; w += gridDim.x) {
      const TokenTile tt = p.tiles[w / FT];
      const int ft = w % FT;
      const int n = ok ? tt.n : 0;
      named_bar_sync(1, kEpiThreads);       // previous item's readers of the staging arrays are done
      for (int i = et; i < KB * NT && ok; i += kEpiThreads) {
        const int kb = i / NT, j = i % NT;
        s_act[i] = (j < n) ? __ldg(p.act_scale + static_cast<size_t>(kb) * p.row_cap + tt.row_start + j) : 0.0f;
      }
      if (et < KB && ok) {
        if (MODE == 1) {
          s_ws[et] = __ldg(p.w_scale + (static_cast<size_t>(tt.expert) * 32 + ft) * kHBlocks + et);
          s_ws[64 + et] = __ldg(p.w_scale + (static_cast<size_t>(tt.expert) * 32 + 16 + ft) * kHBlocks + et);
        } else {
          s_ws[et] = __ldg(p.w_scale + (static_cast<size_t>(tt.expert) * kHBlocks + ft) * kIBlocks + et);
        }
      }
      named_bar_sync(1, kEpiThreads);

      float acc0[NT];                        // mode 1: up,   mode 2: output
      float acc1[MODE == 1 ? NT : 1];        // mode 1: gate
#pragma unroll
      for (int j = 0; j < NT; ++j) acc0[j] = 0.0f;
      if (MODE == 1) {
#pragma unroll
        for (int j = 0; j < NT; ++j) acc1[j] = 0.0f;
      }

      for (int kb = 0; kb < KB && ok; ++kb, ++ab) {
        const uint32_t buf = ab & 1u;
        if (!mbar_wait_bounded(&tfull[buf], (ab >> 1) & 1u, s_abort, kStatusWaitTimeoutEpilogue)) { ok = false; break; }
        tc_fence_after();
        const uint32_t t0 = lane_addr + buf * (2 * NT);
        const float ws0 = s_ws[kb];
        const float ws1 = (MODE == 1) ? s_ws[64 + kb] : 0.0f;
        const float* sa = s_act + kb * NT;
#pragma unroll
        for (int c = 0; c < NT / 16; ++c) {
          if (c * 16 < n) {
            uint32_t v0[16], v1[16];
            tmem_ld16(t0 + c * 16, v0);
            tmem_ld16(t0 + NT + c * 16, v1);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const float a = sa[c * 16 + j];
              if (MODE == 1) {
                acc0[c * 16 + j] = fmaf(__uint_as_float(v0[j]), a * ws0, acc0[c * 16 + j]);
                acc1[c * 16 + j] = fmaf(__uint_as_float(v1[j]), a * ws1, acc1[c * 16 + j]);
              } else {
                const float v = fmaf(__uint_as_float(v1[j]), 1.0f / kLoRatio, __uint_as_float(v0[j]));
                acc0[c * 16 + j] = fmaf(v, a * ws0, acc0[c * 16 + j]);
              }
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty[buf]);
      }
      const int n_out = ok ? n : 0;           // a failed item stores nothing

      if (MODE == 1) {
        // SwiGLU, then the per-row amax over the 128 features of this tile
#pragma unroll
        for (int j = 0; j < NT; ++j) {
          if (j < n_out) {
            const float gt = acc1[j];
            const float cv = (gt / (1.0f + expf(-gt))) * acc0[j];
            acc0[j] = cv;
            const uint32_t m = __reduce_max_sync(0xffffffffu, __float_as_uint(fabsf(cv)));
            if (lane == 0) s_red[q * NT + j] = __uint_as_float(m);
          }
        }
        named_bar_sync(2, kEpiThreads);
        if (et < n_out) {
          const float amax = fmaxf(fmaxf(s_red[et], s_red[NT + et]), fmaxf(s_red[2 * NT + et], s_red[3 * NT + et]));
          const float sc = fmaxf(amax * (1.0f / 448.0f), 1e-12f);
          s_cs[et] = sc;
          s_inv[et] = 1.0f / sc;
          p.c_scale[static_cast<size_t>(ft) * p.row_cap + tt.row_start + et] = sc;
        }
        named_bar_sync(2, kEpiThreads);
        uint8_t* hi = p.c_hi + static_cast<size_t>(tt.row_start) * kInter + ft * 128 + feat;
        uint8_t* lo = p.c_lo + static_cast<size_t>(tt.row_start) * kInter + ft * 128 + feat;
#pragma unroll
        for (int j = 0; j < NT; j += 2) {
          if (j < n_out) {
            const float sc0 = s_cs[j], sc1 = s_cs[j + 1];
            const float in0 = s_inv[j], in1 = s_inv[j + 1];
            const float c0 = acc0[j], c1 = acc0[j + 1];
            const uint16_t h = cvt_e4m3x2(c0 * in0, c1 * in1);
            const float2 hb = e4m3x2_to_float2(h);
            const float r0 = fmaf(-hb.x, sc0, c0), r1 = fmaf(-hb.y, sc1, c1);
            const uint16_t l = cvt_e4m3x2(r0 * in0 * kLoRatio, r1 * in1 * kLoRatio);
            hi[static_cast<size_t>(j) * kInter] = static_cast<uint8_t>(h & 0xff);
            hi[static_cast<size_t>(j + 1) * kInter] = static_cast<uint8_t>(h >> 8);
            lo[static_cast<size_t>(j) * kInter] = static_cast<uint8_t>(l & 0xff);
            lo[static_cast<size_t>(j + 1) * kInter] = static_cast<uint8_t>(l >> 8);
          }
        }
      } else {
        float* o = p.o_rows + static_cast<size_t>(tt.row_start) * kHidden + ft * 128 + feat;
#pragma unroll
        for (int j = 0; j < NT; ++j)
          if (j < n_out) o[static_cast<size_t>(j) * kHidden] = acc0[j];
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
}

template <int MODE>
cudaError_t launch_gemm(const GemmLaunch& g, const GemmArgs& a, int num_sms, cudaStream_t st) {
  grouped_gemm_kernel<MODE><<<num_sms, kGemmThreads, smem_bytes<MODE>(), st>>>(g.tm_w, g.tm_b0, g.tm_b1, a);
  return cudaGetLastError();
}

}  // namespace

cudaError_t gemm_set_attributes() {
  cudaError_t e = cudaFuncSetAttribute(grouped_gemm_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       smem_bytes<1>());
  if (e != cudaSuccess) return e;
  return cudaFuncSetAttribute(grouped_gemm_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              smem_bytes<2>());
}

cudaError_t launch_gemm1(const GemmLaunch& g, const float* w13_scale, const Workspace& ws, int num_sms,
                         cudaStream_t st) {
  GemmArgs a{ws.tiles, ws.meta, ws.a_scale, w13_scale, ws.c_hi, ws.c_lo, ws.c_scale, nullptr, ws.row_cap,
             ws.status};
  return launch_gemm<1>(g, a, num_sms, st);
}

cudaError_t launch_gemm2(const GemmLaunch& g, const float* w2_scale, const Workspace& ws, int num_sms,
                         cudaStream_t st) {
  GemmArgs a{ws.tiles, ws.meta, ws.c_scale, w2_scale, nullptr, nullptr, nullptr, ws.o_rows, ws.row_cap, ws.status};
  return launch_gemm<2>(g, a, num_sms, st);
}

}  // namespace syfi
