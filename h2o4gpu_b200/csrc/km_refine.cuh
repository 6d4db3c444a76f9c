// Exact re-evaluation of ambiguous rows.  The fast distance kernels hand over the
// rows whose best and second-best scores are closer than their rounding error
// bound; one warp per such row recomputes |c|^2 - 2 x.c for every centroid in
// double precision and takes the argmin (first minimum wins), so labels agree
// with exact arithmetic on the float inputs.  The list is short (a fraction of
// a percent of the rows), bounded by the shard size in the worst case.
#pragma once

#include "km_common.cuh"

namespace km {

template <typename T>
__global__ void __launch_bounds__(256)
refine_kernel(const T* __restrict__ X, int d, const T* __restrict__ C, int k,
              const unsigned int* __restrict__ amb_rows, IterState* st, int* __restrict__ labels,
              int count_changes) {
  const unsigned int cnt = st->amb_count;
  const int lane = threadIdx.x & 31;
  const unsigned int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const unsigned int nwarp = (gridDim.x * blockDim.x) >> 5;
  unsigned int changed = 0;
  for (unsigned int e = warp; e < cnt; e += nwarp) {
    const size_t row = amb_rows[e];
    const T* x = X + row * (size_t)d;
    double best = __longlong_as_double(0x7ff0000000000000LL);
    int bi = 0x7fffffff;
    for (int c = lane; c < k; c += 32) {
      const T* cv = C + (size_t)c * d;
      double dot = 0.0, cn = 0.0;
      for (int t = 0; t < d; ++t) {
        const double cc = (double)cv[t];
        dot = fma((double)x[t], cc, dot);
        cn = fma(cc, cc, cn);
      }
      const double s = cn - 2.0 * dot;
      if (s < best) { best = s; bi = c; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const double ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob < best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    if (lane == 0) {
      changed += (labels[row] != bi);
      labels[row] = bi;
    }
  }
  if (count_changes && lane == 0 && changed) atomicAdd(&st->changed, (unsigned long long)changed);
}

}  // namespace km
