// One-off weight pre-packing: the layout neighbour of the GEMM loaders.
//
// The reference reads its weights as given, [E, rows, K] row-major (moe/solution/cuda/moe.cu:3045-3053
// takes the raw pointers; its GEMM1 tensor map is built over that layout at moe.cu:2941-2978).  In that
// layout the 128 x 128-byte tile a GEMM work item needs per K block is 128 separate 128-byte pieces,
// K bytes apart.  Packed, the same tile is 16 KB of consecutive memory that already holds the
// shared-memory image the MMA descriptors expect (rows of 128 bytes, 16-byte chunk c of row r stored at
// chunk c ^ (r & 7)), and a work item's tiles follow each other in the order the kernel consumes them:
//
//   gemm1 packed: [expert][feature tile 0..15][K block 0..55][up tile, gate tile]     32 KB per K block
//   gemm2 packed: [expert][feature tile 0..55][K block 0..15][tile]                   16 KB per K block
//
// so the producer streams one work item as a single sequential read.  Sizes equal the unpacked ones.
#include "moe_internal.h"

namespace syfi {

namespace {

constexpr int kPackThreads = 256;

// One thread moves one 16-byte chunk.  K16 = K / 16 chunks per row.
template <int ROWS, int K, bool UP_GATE>
__global__ void __launch_bounds__(kPackThreads)
prepack_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, long long total_chunks) {
  constexpr int K16 = K / 16;
  constexpr int KB = K / 128;
  for (long long i = static_cast<long long>(blockIdx.x) * kPackThreads + threadIdx.x; i < total_chunks;
       i += static_cast<long long>(gridDim.x) * kPackThreads) {
    const int c = static_cast<int>(i % K16);
    const long long er = i / K16;
    const int row = static_cast<int>(er % ROWS);
    const long long e = er / ROWS;
    const int kb = c >> 3, cc = c & 7;
    long long tile;      // index of the 16 KB tile
    int r;               // row inside the tile
    if (UP_GATE) {
      const int half = row / kInter, f = row % kInter;
      r = f & 127;
      tile = (((e * (kInter / 128) + (f >> 7)) * KB + kb) * 2 + half);
    } else {
      r = row & 127;
      tile = (e * (ROWS / 128) + (row >> 7)) * KB + kb;
    }
    dst[tile * 1024 + r * 8 + (cc ^ (r & 7))] = __ldg(src + i);
  }
}

}  // namespace

cudaError_t launch_prepack(const uint8_t* w13, const uint8_t* w2, int e_local, uint8_t* w13_packed,
                           uint8_t* w2_packed, int num_sms, cudaStream_t st) {
  const long long c13 = static_cast<long long>(e_local) * 2 * kInter * (kHidden / 16);
  const long long c2 = static_cast<long long>(e_local) * kHidden * (kInter / 16);
  const int grid = num_sms * 16;
  prepack_kernel<2 * kInter, kHidden, true><<<grid, kPackThreads, 0, st>>>(
      reinterpret_cast<const uint4*>(w13), reinterpret_cast<uint4*>(w13_packed), c13);
  prepack_kernel<kHidden, kInter, false><<<grid, kPackThreads, 0, st>>>(
      reinterpret_cast<const uint4*>(w2), reinterpret_cast<uint4*>(w2_packed), c2);
  return cudaGetLastError();
}

}  // namespace syfi
