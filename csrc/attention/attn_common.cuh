// Masking shared by the attention kernels.  Every query token i may attend to the inclusive key range
// [k_lo[i], k_hi[i]] of the key / value buffer (empty when k_lo > k_hi).  Causal self-attention over packed sequences
// is k_lo[i] = first token of i's sequence, k_hi[i] = i; passing k_hi == nullptr selects exactly that without
// materialising the second array.  Other masks of the same shape are the steps of context-parallel ring attention
// (queries of one rank against the keys of another: prefixes, no diagonal) and non-causal attention over packed
// sequences.
#pragma once
#include <climits>

#include "../common/ptx.cuh"

namespace mcb {

__device__ __forceinline__ void attn_row_range(const int* __restrict__ k_lo, const int* __restrict__ k_hi, int i, int Tq,
                                               int& lo, int& hi) {
  if (i < Tq) {
    lo = k_lo[i];
    hi = k_hi ? k_hi[i] : i;
  } else {
    lo = 1;
    hi = 0;
  }
}

// The first four warps reduce, over the 128 rows starting at `row0` of a table of inclusive ranges, the smallest
// lower bound and the largest upper bound of the non-empty ones into `s_rng[0..3]` / `s_rng[4..7]` (one entry per
// warp).  Call before a __syncthreads(); afterwards use tile_range_min / tile_range_max.
__device__ __forceinline__ void tile_range_partial(const int* __restrict__ lo_tab, const int* __restrict__ hi_tab,
                                                   int row0, int rows, int* s_rng) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp < 4) {
    int lo, hi;
    attn_row_range(lo_tab, hi_tab, row0 + warp * 32 + lane, rows, lo, hi);
    int mn = lo <= hi ? lo : INT_MAX, mx = lo <= hi ? hi : -1;
#pragma unroll
    for (int s = 16; s; s >>= 1) {
      mn = min(mn, __shfl_xor_sync(0xffffffffu, mn, s));
      mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, s));
    }
    if (lane == 0) {
      s_rng[warp] = mn;
      s_rng[4 + warp] = mx;
    }
  }
}
__device__ __forceinline__ int tile_range_min(const int* s_rng) {
  return min(min(s_rng[0], s_rng[1]), min(s_rng[2], s_rng[3]));
}
__device__ __forceinline__ int tile_range_max(const int* s_rng) {
  return max(max(s_rng[4], s_rng[5]), max(s_rng[6], s_rng[7]));
}

}  // namespace mcb
