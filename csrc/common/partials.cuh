// Fixed-order column sums of per-CTA partial rows: out[c] += sum_b partials[b][c].
//
// A 32 x 32 thread block takes 32 columns; thread (tx, ty) adds the rows ty, ty + 32, ... of column tx in ascending
// order, then one thread per column adds the 32 row-group sums in ascending order.  The association of the sum
// depends only on the number of rows, never on which CTA or warp finished first, so the result repeats bit for bit.
#pragma once
#include <cuda_runtime.h>

namespace mcb {

// `out_hi` (optional) receives the columns >= split (written at index c - split); columns < split go to `out_lo`.
static __global__ void __launch_bounds__(1024) reduce_partials_kernel(const float* __restrict__ partials, int nparts, int ncols,
                                                               float* __restrict__ out_lo, float* __restrict__ out_hi,
                                                               int split) {
  __shared__ float s[32][33];
  const int tx = threadIdx.x, ty = threadIdx.y;
  const int c = blockIdx.x * 32 + tx;
  float acc = 0.f;
  if (c < ncols)
    for (int b = ty; b < nparts; b += 32) acc += partials[(long long)b * ncols + c];
  s[ty][tx] = acc;
  __syncthreads();
  if (ty == 0 && c < ncols) {
    float total = 0.f;
#pragma unroll
    for (int g = 0; g < 32; ++g) total += s[g][tx];
    float* dst = c < split ? (out_lo ? out_lo + c : nullptr) : (out_hi ? out_hi + (c - split) : nullptr);
    if (dst) *dst += total;
  }
}

static inline void launch_reduce_partials(const float* partials, int nparts, int ncols, float* out_lo, float* out_hi, int split,
                                   cudaStream_t s) {
  reduce_partials_kernel<<<(ncols + 31) / 32, dim3(32, 32), 0, s>>>(partials, nparts, ncols, out_lo, out_hi, split);
}

}  // namespace mcb
