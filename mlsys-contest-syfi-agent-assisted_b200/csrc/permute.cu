// Per-expert row lists, the token-tile table, and the gathered activation operand.
//
// Replaces the reference's scan_offsets_kernel / perm_fill_kernel /
// scan_fill_small_kernel (moe/solution/cuda/moe.cu:214-303), its host-side tile
// schedule (moe.cu:3127-3186, a device->host->device round trip) and
// gather_hs_fp8_kernel (moe.cu:2356-2399).
//
// Row order is deterministic: inside an expert, rows are sorted by token.  The router
// leaves one 32-bit word per token with a bit per selected local expert, so the row of
// token t in expert e is the number of earlier tokens with bit e set; CTA e computes
// that with ballots.  Every expert's row range is padded to a multiple of 16 rows
// (the tcgen05 N granularity), padding rows carry token -1 and zero data.
#include "moe_internal.h"
#include "ptx.cuh"

namespace syfi {

namespace {

// kBuildThreads tokens are ranked per pass; a pass costs two dependent round trips to memory (the
// masks, then the routes of the tokens that hit), so large batches use the largest CTA.
template <int kBuildThreads>
__global__ void __launch_bounds__(kBuildThreads)
build_rows_kernel(int T, int e_local, int expert_offset, const uint32_t* __restrict__ local_mask,
                  const int* __restrict__ counts, const int* __restrict__ topk_idx, int* __restrict__ row_token,
                  int* __restrict__ route_row, ExpertWork* __restrict__ work, int* __restrict__ meta, int row_cap,
                  int token_tile, int* __restrict__ status, int* __restrict__ ready, int* __restrict__ counts_last) {
  __shared__ int s_warp[kBuildThreads / 32];
  const int e = blockIdx.x;
  // large batches: gridDim.y CTAs share an expert, each ranks one contiguous range of the tokens
  const int split = blockIdx.y, splits = gridDim.y;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  pdl_wait();
  pdl_trigger();

  // lane i of every warp owns expert i: padded rows, token tiles, and their prefix sums by warp scans
  // (a serial loop over the experts with its integer divisions costs microseconds at the head of the chain)
  const unsigned full = 0xffffffffu;
  const int c_lane = (lane < e_local) ? counts[lane] : 0;
  const int cp_lane = (c_lane + kRowPad - 1) / kRowPad * kRowPad;
  const int nt_lane = (cp_lane + token_tile - 1) / token_tile;
  int rows_incl = cp_lane, tiles_incl = nt_lane;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int r = __shfl_up_sync(full, rows_incl, d), tl = __shfl_up_sync(full, tiles_incl, d);
    if (lane >= d) { rows_incl += r; tiles_incl += tl; }
  }
  const int rows_total = __shfl_sync(full, rows_incl, 31), tiles_total = __shfl_sync(full, tiles_incl, 31);
  const int routed = __reduce_add_sync(full, c_lane);
  const int active = __popc(__ballot_sync(full, c_lane > 0));
  const int row_off = __shfl_sync(full, rows_incl - cp_lane, e);
  const int tile_off = __shfl_sync(full, tiles_incl - nt_lane, e);
  const int cnt = __shfl_sync(full, c_lane, e);
  const int cnt_pad = (cnt + kRowPad - 1) / kRowPad * kRowPad;
  // the GEMM1 -> GEMM2 readiness counters start every call at zero (nothing of the previous call is
  // still running: the router in front of this kernel is an ordinary launch)
  if (split == 0) {
    if (tid == 0) { ready[e] = 0; counts_last[e] = cnt; }
    if (e == 0 && tid >= e_local && tid < kMaxLocalExperts) { ready[tid] = 0; counts_last[tid] = 0; }
  }
  if (rows_total > row_cap) {  // sizing bug: refuse to write out of bounds
    if (tid == 0 && split == 0) { atomicExch(status, kStatusBadIndex); if (e == 0) { meta[0] = 0; meta[1] = 0; meta[2] = 0; meta[3] = 0; } }
    return;
  }

  // this CTA's token range, and the expert's rows among the tokens before it: one coalesced sweep over their
  // masks (4 bytes per token) and a block-wide sum, instead of ranking them pass by pass
  const int per = ((T + splits * kBuildThreads - 1) / (splits * kBuildThreads)) * kBuildThreads;
  const int t_begin = min(T, split * per), t_end = min(T, t_begin + per);
  int base = 0;
  if (split > 0) {
    int mine = 0;
    for (int t = tid; t < t_begin; t += kBuildThreads) mine += (local_mask[t] >> e) & 1u;
    mine = __reduce_add_sync(full, mine);
    if (lane == 0) s_warp[warp] = mine;
    __syncthreads();
#pragma unroll
    for (int w = 0; w < kBuildThreads / 32; ++w) base += s_warp[w];
    __syncthreads();
  }

  // The token's mask and its eight routes are requested together (the routes are only needed when the mask
  // hits, but asking afterwards costs a second dependent round trip per pass), and one pass ahead: a pass is
  // a round trip to L2 plus two barriers, and with the next pass's loads already in flight only the barriers
  // remain on the critical path.
  uint32_t m_nx = 0;
  int4 r0_nx = make_int4(-1, -1, -1, -1), r1_nx = r0_nx;
  auto request = [&](int t) {
    m_nx = 0;
    r0_nx = make_int4(-1, -1, -1, -1);
    r1_nx = r0_nx;
    if (t < T) {
      m_nx = local_mask[t];
      const int4* rp = reinterpret_cast<const int4*>(topk_idx + t * kTopK);
      r0_nx = __ldg(rp);
      r1_nx = __ldg(rp + 1);
    }
  };
  request(t_begin + tid);
  for (int t0 = t_begin; t0 < t_end; t0 += kBuildThreads) {
    const int t = t0 + tid;
    const uint32_t m = m_nx;
    const int4 r0 = r0_nx, r1 = r1_nx;
    request(t + kBuildThreads);
    const bool has = (m >> e) & 1u;
    const unsigned b = __ballot_sync(0xffffffffu, has);
    if (lane == 0) s_warp[warp] = __popc(b);
    __syncthreads();
    int before = 0, block_total = 0;
#pragma unroll
    for (int w = 0; w < kBuildThreads / 32; ++w) {
      const int c = s_warp[w];
      before += (w < warp) ? c : 0;
      block_total += c;
    }
    if (has) {
      const int row = row_off + base + before + __popc(b & ((1u << lane) - 1u));
      row_token[row] = t;
      const int ge = e + expert_offset;
      const int routes[kTopK] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
#pragma unroll
      for (int k = 0; k < kTopK; ++k)
        if (routes[k] == ge) route_row[t * kTopK + k] = row;
    }
    base += block_total;
    __syncthreads();
  }
  if (split != 0) return;
  for (int r = cnt + tid; r < cnt_pad; r += kBuildThreads) row_token[row_off + r] = -1;
  if (tid == 0) {
    ExpertWork ew;
    ew.row_off = row_off;
    ew.rows_pad = cnt_pad;
    ew.tile_off = tile_off;
    ew.tiles = (cnt_pad + token_tile - 1) / token_tile;
    work[e] = ew;
  }
  if (e == 0 && tid == 0) {
    meta[0] = tiles_total; meta[1] = rows_total; meta[2] = routed; meta[3] = active;
  }
}

constexpr int kGatherThreads = 224;  // 7168 B per row = 448 x 16 B = 2 per thread

__global__ void __launch_bounds__(kGatherThreads)
gather_rows_kernel(const uint8_t* __restrict__ hidden, const float* __restrict__ hidden_scale, int T,
                   const int* __restrict__ row_token, const int* __restrict__ meta, uint8_t* __restrict__ a_perm,
                   float* __restrict__ a_scale, int row_cap, int* __restrict__ counts) {
  pdl_wait();
  pdl_trigger();
  // every reader of the per-expert row counters (the row-list kernel) has finished: zero them for the
  // router of the next call
  if (blockIdx.x == 0 && threadIdx.x < kMaxLocalExperts) counts[threadIdx.x] = 0;
  const int rows_total = meta[1];
  const int tid = threadIdx.x;
  for (int r = blockIdx.x; r < rows_total; r += gridDim.x) {
    const int t = row_token[r];
    uint4* dst = reinterpret_cast<uint4*>(a_perm + static_cast<size_t>(r) * kHidden);
    if (t >= 0 && t < T) {
      const uint4* src = reinterpret_cast<const uint4*>(hidden + static_cast<size_t>(t) * kHidden);
      const uint4 v0 = __ldg(src + tid), v1 = __ldg(src + tid + kGatherThreads);
      dst[tid] = v0;
      dst[tid + kGatherThreads] = v1;
      if (tid < kHBlocks) a_scale[static_cast<size_t>(tid) * row_cap + r] = __ldg(hidden_scale + static_cast<size_t>(tid) * T + t);
    } else {
      const uint4 z = make_uint4(0, 0, 0, 0);
      dst[tid] = z;
      dst[tid + kGatherThreads] = z;
      if (tid < kHBlocks) a_scale[static_cast<size_t>(tid) * row_cap + r] = 0.0f;
    }
  }
}

}  // namespace

cudaError_t launch_build_rows(int T, int e_local, int expert_offset, int token_tile, const Workspace& ws,
                              cudaStream_t st) {
  if (T <= 256)
    return launch_dependent(build_rows_kernel<256>, dim3(e_local), dim3(256), 0, st, T, e_local, expert_offset,
                            ws.local_mask, ws.counts, ws.topk_idx, ws.row_token, ws.route_row, ws.work, ws.meta,
                            ws.row_cap, token_tile, ws.status, ws.ready, ws.counts_last);
  // from 4096 tokens on, four CTAs per expert (each ranks a quarter of the tokens after counting the expert's
  // rows in the quarters before it): 18 -> about 8 us at 8192 tokens
  const int splits = T >= 4096 ? 4 : 1;
  return launch_dependent(build_rows_kernel<1024>, dim3(e_local, splits), dim3(1024), 0, st, T, e_local, expert_offset,
                          ws.local_mask, ws.counts, ws.topk_idx, ws.row_token, ws.route_row, ws.work, ws.meta,
                          ws.row_cap, token_tile, ws.status, ws.ready, ws.counts_last);
}

cudaError_t launch_gather(const uint8_t* hidden, const float* hidden_scale, int T, const Workspace& ws, int num_sms,
                          cudaStream_t st) {
  const int max_rows = 8 * T + kRowPad * kMaxLocalExperts;
  const int grid = max_rows < num_sms * 8 ? max_rows : num_sms * 8;
  return launch_dependent(gather_rows_kernel, dim3(grid), dim3(kGatherThreads), 0, st, hidden, hidden_scale, T,
                          ws.row_token, ws.meta, ws.a_perm, ws.a_scale, ws.row_cap, ws.counts);
}

}  // namespace syfi
