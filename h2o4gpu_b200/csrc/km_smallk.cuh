// Fused single-pass Lloyd step for k <= 16 (the bandwidth-bound regime): every
// row of X is read from HBM once per iteration.  A group of lanes owns a row,
// forms the k dot products against the centroids held in shared memory,
// reduces them with shuffles, takes the argmin and immediately adds the row
// (re-read from L1/L2) into fixed-point per-CTA sums in shared memory, which are
// drained into the int64 global sums at the end.  Replaces, for small k, the
// reference's distance matrix + relabel + sort + calculate_centroids sequence
// (src/gpu/kmeans/kmeans_labels.cu:115-244, kmeans_labels.h:360-392,
// kmeans_centroids.h:108-189).
#pragma once

#include "km_common.cuh"
#include "km_tiles.cuh"

namespace km {

constexpr int kSmallKThreads = 256;
constexpr int kSmallKRpw = 2;        // rows per lane group processed together (shares centroid loads): fused step
constexpr int kSmallKRpwAssign = 4;  // the same for the E-step alone, which has the registers for it

template <typename T>
inline size_t smallk_smem_bytes(int K, int d, bool update) {
  size_t b = (size_t)K * d * sizeof(T) + (size_t)K * sizeof(T);
  if (update) b += (size_t)Fixed<T>::NP * K * d * sizeof(int) + (size_t)K * sizeof(int);
  return b + 16;
}

// K: compile-time bound on the number of centroids (k <= K).  V: elements per
// global load.  rows [blockIdx.x * rows_per_cta, ...) belong to this CTA.
template <typename T, int K, int V, int RPW>
__global__ void __launch_bounds__(kSmallKThreads, 2)
smallk_kernel(const T* __restrict__ X, size_t n, int d, const T* __restrict__ C, int k,
              const T* __restrict__ cnorm, int* __restrict__ labels, IterState* st,
              long long* __restrict__ gsums, unsigned long long* __restrict__ gcounts, T scale,
              int update, unsigned int rows_per_cta) {
  constexpr int NP = Fixed<T>::NP;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* Cs = reinterpret_cast<T*>(smem_raw);                 // [K][d]
  T* cns = Cs + (size_t)K * d;                            // [K]
  int* acc = reinterpret_cast<int*>(cns + K);             // [NP][K][d]
  int* cnt = acc + (size_t)NP * K * d;                    // [K]
  __shared__ unsigned int s_changed;

  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  constexpr int NWARP = kSmallKThreads / 32;
  const int dv = d / V;

  for (int i = tid; i < K * d; i += kSmallKThreads) {
    int c = i / d;
    Cs[i] = (c < k) ? C[i] : (T)0;
  }
  for (int i = tid; i < K; i += kSmallKThreads) cns[i] = (i < k) ? cnorm[i] : (T)0;
  if (update) {
    for (int i = tid; i < NP * K * d; i += kSmallKThreads) acc[i] = 0;
    for (int i = tid; i < K; i += kSmallKThreads) cnt[i] = 0;
  }
  if (tid == 0) s_changed = 0;
  __syncthreads();

  // lanes per row: smallest power of two covering dv, at most 32
  int lpr = 1;
  while (lpr < dv && lpr < 32) lpr <<= 1;
  const int groups = 32 / lpr;
  const int g = lane / lpr;
  const int l = lane % lpr;

  const size_t r0 = (size_t)blockIdx.x * rows_per_cta;
  size_t r1 = r0 + rows_per_cta;
  if (r1 > n) r1 = n;
  unsigned int changed = 0;

  const int step_rows = groups * RPW;
  for (size_t base = r0 + (size_t)warp * step_rows; base < r1; base += (size_t)NWARP * step_rows) {
    size_t row[RPW];
    bool valid[RPW];
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
      row[r] = base + (size_t)r * groups + g;
      valid[r] = row[r] < r1;
    }
    T dot[RPW][K];
#pragma unroll
    for (int r = 0; r < RPW; ++r)
#pragma unroll
      for (int c = 0; c < K; ++c) dot[r][c] = 0;

#pragma unroll 2
    for (int idx = l; idx < dv; idx += lpr) {
      T x[RPW][V];
#pragma unroll
      for (int r = 0; r < RPW; ++r) {
#pragma unroll
        for (int e = 0; e < V; ++e) x[r][e] = 0;
        if (valid[r]) VecLoad<T, V>::ld(X + row[r] * (size_t)d + (size_t)idx * V, x[r]);
      }
#pragma unroll
      for (int c = 0; c < K; ++c) {
        T cv[V];
        VecLoad<T, V>::ld(Cs + (size_t)c * d + (size_t)idx * V, cv);
#pragma unroll
        for (int r = 0; r < RPW; ++r)
#pragma unroll
          for (int e = 0; e < V; ++e) dot[r][c] = fma(x[r][e], cv[e], dot[r][c]);
      }
    }
    // reduce over the lanes of a row
#pragma unroll
    for (int r = 0; r < RPW; ++r)
#pragma unroll
      for (int c = 0; c < K; ++c) {
        T v = dot[r][c];
        for (int o = lpr >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        dot[r][c] = v;
      }
    int lab[RPW];
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
      T m = Inf<T>::v();
      int mi = 0;
#pragma unroll
      for (int c = 0; c < K; ++c) {
        T s = cns[c] - (T)2 * dot[r][c];
        if (c < k && s < m) { m = s; mi = c; }
      }
      lab[r] = mi;
      if (valid[r] && l == 0) {
        changed += (labels[row[r]] != mi);
        labels[row[r]] = mi;
        if (update) atomicAdd(&cnt[mi], 1);
      }
    }
    if (update) {
#pragma unroll
      for (int r = 0; r < RPW; ++r) {
        if (!valid[r]) continue;
        int* a = acc + (size_t)lab[r] * d;
        for (int idx = l; idx < dv; idx += lpr) {
          T x[V];
          VecLoad<T, V>::ld(X + row[r] * (size_t)d + (size_t)idx * V, x);
          add_vec_fixed<T, V, NP>(a, (size_t)K * d, dv, idx, g & (V - 1), x, scale);
        }
      }
    }
  }

  if (changed) atomicAdd(&s_changed, changed);
  __syncthreads();
  if (tid == 0 && s_changed && st) atomicAdd(&st->changed, (unsigned long long)s_changed);

  if (update) {
    // drain: pair q of the global sums = piece(2q) * 2^15 + piece(2q+1)
    for (int i = tid; i < k * d; i += kSmallKThreads) {
      const int c = i / d;
      const int col = pos_to_col(i - c * d, dv, V);
#pragma unroll
      for (int q = 0; q < NP / 2; ++q) {
        long long v = (long long)acc[(size_t)(2 * q) * K * d + i] * (1LL << kPieceBits) +
                      (long long)acc[(size_t)(2 * q + 1) * K * d + i];
        if (v) atomicAdd(reinterpret_cast<unsigned long long*>(gsums + (size_t)q * k * d + (size_t)c * d + col),
                         (unsigned long long)v);
      }
    }
    for (int i = tid; i < k; i += kSmallKThreads)
      if (cnt[i]) atomicAdd(gcounts + i, (unsigned long long)cnt[i]);
  }
}

}  // namespace km
