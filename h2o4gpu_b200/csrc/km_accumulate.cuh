// Centroid sums and counts of a labelled shard: the M-step's reduction.
// Replaces the reference's per-iteration radix sort of (label, row) pairs plus
// the 30-CTA gather/atomic kernel (find_centroids / calculate_centroids,
// src/gpu/kmeans/kmeans_centroids.h:40-75, 108-189).
//
// X is streamed once with 128-bit coalesced loads.  Each CTA owns a slice of
// clusters [c0, c0 + kc) whose fixed-point sums fit its shared memory and a
// partition of at most 32768 rows; it adds the rows of its partition whose
// label falls in its slice with integer shared-memory atomics and drains the
// result into the int64 global sums.  Integer addition makes the result
// independent of the order of additions, so it is deterministic without sorting.
// With one slice (k*d small) the CTA streams its partition as a flat array; with
// several slices each warp compacts the in-slice rows of 32-row blocks first.
//
// Sample weights (W != null; the sklearn-style fit(X, sample_weight=w) of the wrapper,
// src/interface_py/h2o4gpu/solvers/kmeans.py:800-804, which the reference hands to the CPU):
// a row adds w * x to the sums and its weight to the count.  The weight enters the count as a
// two-piece fixed-point number (30 bits below the largest weight), so weighted counts are
// integers too and stay order-independent; `scale` then covers |w * x|.
#pragma once

#include "km_common.cuh"
#include "km_tiles.cuh"

namespace km {

constexpr int kAccThreads = 512;

template <typename T>
inline size_t accumulate_smem_bytes(int kc, int d) {
  return (size_t)Fixed<T>::NP * kc * d * sizeof(int) + (size_t)2 * kc * sizeof(int) + 16;
}

// divisor for idx / dv with idx * dv < 2^40: q = (idx * magic) >> 40
inline unsigned long long fastdiv_magic(unsigned int dv) { return ((1ULL << 40) / dv) + 1ULL; }

template <typename T, int V>
__global__ void __launch_bounds__(kAccThreads)
accumulate_kernel(const T* __restrict__ X, size_t n, int d, const int* __restrict__ labels, int k,
                  int kc, int n_slices, long long* __restrict__ gsums,
                  unsigned long long* __restrict__ gcounts, T scale, unsigned int rows_per_part,
                  unsigned long long dv_magic,
                  const unsigned long long* gate_changed, unsigned long long gate_limit,
                  const T* __restrict__ W, T wscale) {
  constexpr int NP = Fixed<T>::NP;
  if (delta_turn(gate_changed, gate_limit)) return;   // the incremental branch has this iteration
  extern __shared__ __align__(16) unsigned char smem_raw[];
  int* acc = reinterpret_cast<int*>(smem_raw);   // [NP][kc][d]
  int* cnt = acc + (size_t)NP * kc * d;          // [2][kc]: units, then units * 2^15

  const int tid = threadIdx.x;
  const int slice = blockIdx.x % n_slices;
  const size_t part = blockIdx.x / n_slices;
  const int c0 = slice * kc;
  const int c1 = min(k, c0 + kc);
  const size_t r0 = part * (size_t)rows_per_part;
  size_t r1 = r0 + rows_per_part;
  if (r1 > n) r1 = n;
  if (r0 >= n || c0 >= k) return;
  const unsigned int nrows = (unsigned int)(r1 - r0);
  const int dv = d / V;
  const size_t pstride = (size_t)kc * d;

  for (int i = tid; i < NP * kc * d; i += kAccThreads) acc[i] = 0;
  for (int i = tid; i < 2 * kc; i += kAccThreads) cnt[i] = 0;
  __syncthreads();

  const T* Xp = X + r0 * (size_t)d;
  const int* Lp = labels + r0;
  const T* Wp = W ? W + r0 : nullptr;
  auto count_row = [&](int c, T w) {
    if (Wp) {
      int p[2];
      split_pieces<2>(w, wscale, p);
      if (p[1]) atomicAdd(&cnt[c], p[1]);
      if (p[0]) atomicAdd(&cnt[kc + c], p[0]);
    } else {
      atomicAdd(&cnt[c], 1);
    }
  };

  if (n_slices == 1) {
    // flat stream over the partition: item = one vector of V elements
    const unsigned int items = nrows * (unsigned int)dv;
    constexpr int UNROLL = 4;
    for (unsigned int base = tid; base < items; base += kAccThreads * UNROLL) {
      T x[UNROLL][V];
      int lab[UNROLL];
      unsigned int col[UNROLL], rowu[UNROLL];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        unsigned int idx = base + u * kAccThreads;
        lab[u] = -1;
        if (idx < items) {
          unsigned int row = (unsigned int)(((unsigned long long)idx * dv_magic) >> 40);
          col[u] = idx - row * dv;  // vector index within the row
          rowu[u] = row;
          VecLoad<T, V>::ld(Xp + (size_t)idx * V, x[u]);
          lab[u] = Lp[row];
          const T w = Wp ? Wp[row] : (T)1;
          if ((unsigned)lab[u] >= (unsigned)k) lab[u] = -1;  // cannot come from the E-step kernels; skipped
          else if (col[u] == 0) count_row(lab[u], w);
          if (Wp) {
#pragma unroll
            for (int e = 0; e < V; ++e) x[u][e] *= w;
          }
        }
      }
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        if (lab[u] < 0) continue;
        add_vec_fixed<T, V, NP>(acc + (size_t)lab[u] * d, pstride, dv, (int)col[u], (int)rowu[u] & (V - 1), x[u], scale);
      }
    }
  } else {
    const int lane = tid & 31;
    const int warp = tid >> 5;
    constexpr int NWARP = kAccThreads / 32;
    int lpr = 1;
    while (lpr < dv && lpr < 32) lpr <<= 1;
    const int groups = 32 / lpr;
    const int g = lane / lpr;
    const int l = lane % lpr;
    for (unsigned int b = warp * 32; b < nrows; b += NWARP * 32) {
      unsigned int r = b + lane;
      int my = (r < nrows) ? Lp[r] : -1;
      bool in = (my >= c0 && my < c1);
      unsigned int mask = __ballot_sync(0xffffffffu, in);
      const T myw = (Wp && r < nrows) ? Wp[r] : (T)1;
      if (in) count_row(my - c0, myw);
      while (mask) {
        unsigned int src = __fns(mask, 0, g + 1);  // lane of the (g+1)-th in-slice row
        bool have = (src != 0xffffffffu);
        int lab = __shfl_sync(0xffffffffu, my, have ? src : 0);
        const T w = __shfl_sync(0xffffffffu, myw, have ? src : 0);
        if (have) {
          const T* xr = Xp + (size_t)(b + src) * d;
          int* a = acc + (size_t)(lab - c0) * d;
          for (int idx = l; idx < dv; idx += lpr) {
            T x[V];
            VecLoad<T, V>::ld(xr + (size_t)idx * V, x);
            if (Wp) {
#pragma unroll
              for (int e = 0; e < V; ++e) x[e] *= w;
            }
            add_vec_fixed<T, V, NP>(a, pstride, dv, idx, g & (V - 1), x, scale);
          }
        }
        for (int i = 0; i < groups && mask; ++i) mask &= mask - 1;
      }
    }
  }
  __syncthreads();

  const int kloc = c1 - c0;
  for (int i = tid; i < kloc * d; i += kAccThreads) {
    const int c = i / d;
    const int col = pos_to_col(i - c * d, dv, V);
#pragma unroll
    for (int q = 0; q < NP / 2; ++q) {
      long long v = (long long)acc[(size_t)(2 * q) * pstride + i] * (1LL << kPieceBits) +
                    (long long)acc[(size_t)(2 * q + 1) * pstride + i];
      if (v) atomicAdd(reinterpret_cast<unsigned long long*>(gsums + (size_t)q * k * d + (size_t)(c0 + c) * d + col),
                       (unsigned long long)v);
    }
  }
  for (int i = tid; i < kloc; i += kAccThreads) {
    const long long v = (long long)cnt[kc + i] * (1LL << kPieceBits) + (long long)cnt[i];
    if (v) atomicAdd(gcounts + c0 + i, (unsigned long long)v);
  }
}

}  // namespace km
