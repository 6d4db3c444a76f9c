// Exact re-evaluation of ambiguous rows.  The fast distance kernels hand over the
// rows whose best and second-best scores are closer than their rounding error
// bound; one warp per such row recomputes |c|^2 - 2 x.c for every centroid in
// double precision and takes the argmin (first minimum wins), so labels agree
// with exact arithmetic on the float inputs.  The list is short (a fraction of
// a percent of the rows), bounded by the shard size in the worst case.
//
// The centroid table is staged once per CTA in shared memory, transposed
// ([d][k], so the lanes of a warp read consecutive centroids of one column), with
// |c|^2 in double; each lane carries up to kRefineCpl centroids as independent
// FMA chains.  A row is fetched with one coalesced load per 32 columns (XR of them,
// d <= 32 * XR), the next row's fetch is issued before the current row's arithmetic,
// and the column values are handed round the warp with shuffles.
#pragma once

#include "km_common.cuh"

namespace km {

constexpr int kRefineThreads = 256;
constexpr int kRefineCpl = 4;  // centroids per lane: k <= 32 * kRefineCpl

template <typename T>
inline size_t refine_smem_bytes(int k, int d) {
  const int kp = (k + 31) / 32 * 32;
  return (size_t)d * (kp + 1) * sizeof(T) + (size_t)kp * sizeof(double) + 16;
}

template <typename T, int XR>
__global__ void __launch_bounds__(kRefineThreads)
refine_kernel(const T* __restrict__ X, int d, const T* __restrict__ C, int k,
              const unsigned int* __restrict__ amb_rows, IterState* st, int* __restrict__ labels,
              int count_changes) {
  const unsigned int cnt = st->amb_count;
  const int lane = threadIdx.x & 31;
  const unsigned int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const unsigned int nwarp = (gridDim.x * blockDim.x) >> 5;
  if (blockIdx.x * (kRefineThreads / 32) >= cnt) return;  // no row for this CTA (uniform)

  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int kp = (k + 31) / 32 * 32;
  const int kps = kp + 1;                                        // odd row stride: conflict-free transposed stores
  double* cn_s = reinterpret_cast<double*>(smem_raw);            // [kp]
  T* Ct = reinterpret_cast<T*>(cn_s + kp);                       // [d][kps]
  for (int i = threadIdx.x; i < d * kp; i += kRefineThreads) {
    const int c = i / d, t = i - c * d;                          // coalesced read of C, transposed store
    Ct[t * kps + c] = (c < k) ? C[(size_t)c * d + t] : (T)0;
  }
  __syncthreads();
  for (int c = threadIdx.x; c < kp; c += kRefineThreads) {
    double s = 0.0;
    for (int t = 0; t < d; ++t) {
      const double v = (double)Ct[t * kps + c];
      s = fma(v, v, s);
    }
    cn_s[c] = s;
  }
  __syncthreads();

  unsigned int changed = 0;
  T xn[XR];
  size_t row_n = 0;
  int old_n = 0;
  auto fetch = [&](unsigned int e) {
    row_n = amb_rows[e];
    const T* x = X + row_n * (size_t)d;
#pragma unroll
    for (int j = 0; j < XR; ++j) xn[j] = (j * 32 + lane < d) ? x[j * 32 + lane] : (T)0;
    old_n = labels[row_n];
  };
  if (warp < cnt) fetch(warp);
  for (unsigned int e = warp; e < cnt; e += nwarp) {
    T xr[XR];
#pragma unroll
    for (int j = 0; j < XR; ++j) xr[j] = xn[j];
    const size_t row = row_n;
    const int old_label = old_n;
    if (e + nwarp < cnt) fetch(e + nwarp);
    double dot[kRefineCpl];
#pragma unroll
    for (int u = 0; u < kRefineCpl; ++u) dot[u] = 0.0;
#pragma unroll
    for (int j = 0; j < XR; ++j) {
      const int tn = min(32, d - j * 32);
      for (int tt = 0; tt < tn; ++tt) {
        const double xv = (double)__shfl_sync(0xffffffffu, xr[j], tt);
        const T* ct = Ct + (j * 32 + tt) * kps + lane;
#pragma unroll
        for (int u = 0; u < kRefineCpl; ++u)
          if (u * 32 < kp) dot[u] = fma(xv, (double)ct[u * 32], dot[u]);
      }
    }
    double best = __longlong_as_double(0x7ff0000000000000LL);
    int bi = 0x7fffffff;
#pragma unroll
    for (int u = 0; u < kRefineCpl; ++u) {
      const int c = u * 32 + lane;
      if (c < k) {
        const double s = cn_s[c] - 2.0 * dot[u];
        if (s < best) { best = s; bi = c; }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const double ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob < best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    if (lane == 0) {
      changed += (old_label != bi);
      labels[row] = bi;
    }
  }
  if (count_changes && lane == 0 && changed) atomicAdd(&st->changed, (unsigned long long)changed);
}

}  // namespace km
