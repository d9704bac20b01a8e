// Stable least-significant-digit radix sort of (64-bit key, 32-bit value) pairs, 8 bits per pass.
// Used to put GPU-side events in order of their start timestamp before sizes are scanned, so the
// emit pass still writes every event straight to its final offset.  Per pass: per-tile digit
// histograms, one exclusive scan over the digit-major histogram, and a stable scatter.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace k2j {

constexpr int kSortThreads = 256;
constexpr int kSortRounds = 8;
constexpr int kSortTile = kSortThreads * kSortRounds;  // keys per block

// hist[digit * n_tiles + tile] = number of keys of the tile with that digit
__global__ void __launch_bounds__(kSortThreads) k_rs_hist(const uint64_t* keys, uint64_t n, int shift, uint32_t* hist, uint32_t n_tiles) {
  __shared__ uint32_t s_h[256];
  s_h[threadIdx.x] = 0;
  __syncthreads();
  const uint64_t base = (uint64_t)blockIdx.x * kSortTile;
#pragma unroll
  for (int r = 0; r < kSortRounds; r++) {
    const uint64_t i = base + (uint64_t)r * kSortThreads + threadIdx.x;
    if (i < n) atomicAdd(&s_h[(uint32_t)(keys[i] >> shift) & 255u], 1u);
  }
  __syncthreads();
  hist[(uint64_t)threadIdx.x * n_tiles + blockIdx.x] = s_h[threadIdx.x];
}

// base[digit * n_tiles + tile] = global position of the tile's first key with that digit
__global__ void __launch_bounds__(kSortThreads) k_rs_scatter(const uint64_t* keys, const uint32_t* vals, uint64_t n, int shift,
                                                             const uint64_t* base, uint32_t n_tiles, uint64_t* keys_out,
                                                             uint32_t* vals_out) {
  __shared__ uint32_t s_cnt[kSortThreads / 32][256];  // per warp and digit: count, then offset within the round
  __shared__ uint32_t s_run[256];                      // keys of each digit placed by earlier rounds
  const uint32_t lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  s_run[threadIdx.x] = 0;
  const uint64_t tile0 = (uint64_t)blockIdx.x * kSortTile;
  for (int r = 0; r < kSortRounds; r++) {
    for (int i = threadIdx.x; i < (kSortThreads / 32) * 256; i += kSortThreads) (&s_cnt[0][0])[i] = 0;
    __syncthreads();
    const uint64_t i = tile0 + (uint64_t)r * kSortThreads + threadIdx.x;
    const bool in = i < n;
    const uint64_t key = in ? keys[i] : 0;
    const uint32_t val = in ? vals[i] : 0;
    const uint32_t dg = (uint32_t)(key >> shift) & 255u;
    // lanes of this warp with the same digit (out-of-range lanes form their own group)
    const uint32_t peers = __match_any_sync(0xffffffffu, in ? dg : 256u + 0u);
    const uint32_t rank_in_warp = __popc(peers & ((1u << lane) - 1u));
    if (in && rank_in_warp == 0) s_cnt[w][dg] = __popc(peers);
    __syncthreads();
    {  // thread d: exclusive prefix over warps of digit d, on top of what earlier rounds placed
      const uint32_t d = threadIdx.x;
      uint32_t acc = s_run[d];
#pragma unroll
      for (int ww = 0; ww < kSortThreads / 32; ww++) { const uint32_t t = s_cnt[ww][d]; s_cnt[ww][d] = acc; acc += t; }
      s_run[d] = acc;
    }
    __syncthreads();
    if (in) {
      const uint64_t pos = base[(uint64_t)dg * n_tiles + blockIdx.x] + s_cnt[w][dg] + rank_in_warp;
      keys_out[pos] = key;
      vals_out[pos] = val;
    }
    __syncthreads();
  }
}

// rank[vals_sorted[pos]] = pos
__global__ void k_rs_invert(const uint32_t* vals_sorted, uint64_t n, uint32_t* rank) {
  const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) rank[vals_sorted[i]] = (uint32_t)i;
}

}  // namespace k2j
