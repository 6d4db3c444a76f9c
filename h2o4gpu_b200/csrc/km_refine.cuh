// Exact re-evaluation of ambiguous rows (tensor-core path for small centroid tables).
//
// The fast kernel hands over every row that has more than one score within the rounding
// error bound of its best score, together with the bit mask of those columns (128 bits, one
// per centroid).  The true nearest centroid is one of them - every other score is farther
// than the bound - so one warp per row recomputes just those few scores, |c|^2 - 2 x.c, in
// double precision (lanes split the columns, butterfly sum) and takes the smallest, lowest
// index first on a tie.  Labels then agree with exact arithmetic on the float inputs.
// Double-precision arithmetic is slow on this part (the re-evaluation of all k scores of a
// row, as first built, cost as much as a tenth of the whole E-step), which is why only the
// candidates are touched.
#pragma once

#include "km_common.cuh"

namespace km {

constexpr int kRefineThreads = 256;

template <typename T>
__global__ void __launch_bounds__(kRefineThreads)
refine_near_kernel(const T* __restrict__ X, int d, const T* __restrict__ C, int k,
                   const unsigned int* __restrict__ amb_rows, const uint4* __restrict__ amb_near, IterState* st,
                   int* __restrict__ labels, int count_changes, unsigned int* __restrict__ moved_bits) {
  const unsigned int cnt = st->amb_count;
  const int lane = threadIdx.x & 31;
  const unsigned int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const unsigned int nwarp = (gridDim.x * blockDim.x) >> 5;
  unsigned int changed = 0;
  for (unsigned int e = warp; e < cnt; e += nwarp) {
    const size_t row = amb_rows[e];
    const uint4 nm = amb_near[e];
    const unsigned int near[4] = {nm.x, nm.y, nm.z, nm.w};
    const T* x = X + row * (size_t)d;
    const int old_label = labels[row];
    double best = __longlong_as_double(0x7ff0000000000000LL);
    int bi = 0x7fffffff;
#pragma unroll
    for (int ch = 0; ch < 4; ++ch) {
      unsigned int m = near[ch];
      while (m) {
        const int c = ch * 32 + __ffs(m) - 1;
        m &= m - 1;
        if (c >= k) continue;
        const T* cr = C + (size_t)c * d;
        double s = 0.0;
        for (int t = lane; t < d; t += 32) {
          const double cv = (double)cr[t];
          s = fma(cv, cv - 2.0 * (double)x[t], s);
        }
        s = warp_sum(s);
        if (s < best || (s == best && c < bi)) { best = s; bi = c; }
      }
    }
    if (lane == 0 && bi != 0x7fffffff) {
      changed += (old_label != bi);
      labels[row] = bi;
      // the moved-rows map of the fast kernel has a zero for this row
      if (moved_bits != nullptr && count_changes && old_label != bi)
        atomicOr(&moved_bits[row >> 5], 1u << (unsigned int)(row & 31));
    }
  }
  if (count_changes && lane == 0 && changed) atomicAdd(&st->changed, (unsigned long long)changed);
}

}  // namespace km
