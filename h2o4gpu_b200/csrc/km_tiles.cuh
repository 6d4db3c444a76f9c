// SIMT register-tiled distance kernel: scores = |c|^2 - 2 X.C^T are formed tile
// by tile in registers and consumed in the epilogue, so the rows x k matrix is
// never stored unless the caller asks for it (transform).
//
//   MODE_ASSIGN     running (min, argmin) over the k tiles, first minimum wins
//                   (tie rule of make_new_labels, src/gpu/kmeans/kmeans_labels.h:360-377);
//                   replaces calculate_distances + relabel
//                   (src/gpu/kmeans/kmeans_labels.cu:115-244, kmeans_labels.h:360-392).
//   MODE_TRANSFORM  writes |xn + cn - 2 x.c| column-major (kmeans_labels.cu:173-176).
//
// This is the general path: any k, any d, float or double.  float inputs with
// 32-column-aligned d take the tensor-core kernel instead; k <= 16 takes the
// fused single-pass kernel.
#pragma once

#include "km_common.cuh"

namespace km {

enum { MODE_ASSIGN = 0, MODE_TRANSFORM = 1 };

template <typename T> struct VecOf;
template <> struct VecOf<float> { using type = float4; static constexpr int N = 4; };
template <> struct VecOf<double> { using type = double2; static constexpr int N = 2; };

template <typename T, int N> struct VecLoad;
template <> struct VecLoad<float, 4> {
  __device__ static void ld(const float* p, float (&v)[4]) {
    float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  }
};
template <> struct VecLoad<double, 2> {
  __device__ static void ld(const double* p, double (&v)[2]) {
    double2 t = *reinterpret_cast<const double2*>(p);
    v[0] = t.x; v[1] = t.y;
  }
};
template <typename T> struct VecLoad<T, 1> {
  __device__ static void ld(const T* p, T (&v)[1]) { v[0] = *p; }
};
// The same loads marked streaming (evict first): for one-pass reads of X beside a small table
// that should stay in L1.
template <typename T, int N> struct VecLoadStream;
template <> struct VecLoadStream<float, 4> {
  __device__ static void ld(const float* p, float (&v)[4]) {
    float4 t = __ldcs(reinterpret_cast<const float4*>(p));
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  }
};
template <> struct VecLoadStream<double, 2> {
  __device__ static void ld(const double* p, double (&v)[2]) {
    double2 t = __ldcs(reinterpret_cast<const double2*>(p));
    v[0] = t.x; v[1] = t.y;
  }
};
template <typename T> struct VecLoadStream<T, 1> {
  __device__ static void ld(const T* p, T (&v)[1]) { v[0] = __ldcs(p); }
};

// BM x BN output tile per CTA, BK columns of d per stage, TM x TN per thread.
// VEC: elements per global load (needs d % VEC == 0 and 16-byte aligned rows).
template <typename T, int BM, int BN, int BK, int TM, int TN, int VEC, int MODE>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
tile_kernel(const T* __restrict__ X, size_t n, int d, const T* __restrict__ C, int k,
            const T* __restrict__ cnorm, int* __restrict__ labels, IterState* st,
            T* __restrict__ out, size_t ld_out) {
  constexpr int NTX = BN / TN;
  constexpr int NTY = BM / TM;
  constexpr int NT = NTX * NTY;
  constexpr int PAD = 4;
  static_assert((NTX & (NTX - 1)) == 0 && NTX <= 32, "NTX must be a power of two <= 32");
  static_assert(BK % VEC == 0, "BK % VEC");
  constexpr int A_LD = (BM * BK / VEC + NT - 1) / NT;  // vector loads per thread per stage
  constexpr int B_LD = (BN * BK / VEC + NT - 1) / NT;

  __shared__ T As[BK][BM + PAD];
  __shared__ T Bs[BK][BN + PAD];
  __shared__ unsigned int s_changed;

  const int tid = threadIdx.x;
  const int tx = tid % NTX;
  const int ty = tid / NTX;
  const size_t row0 = (size_t)blockIdx.x * BM;

  if (tid == 0) s_changed = 0;

  T best[TM];
  int bidx[TM];
  T xn[TM];
#pragma unroll
  for (int i = 0; i < TM; ++i) { best[i] = Inf<T>::v(); bidx[i] = 0; xn[i] = 0; }

  for (int n0 = 0; n0 < k; n0 += BN) {
    T acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
      for (int j = 0; j < TN; ++j) acc[i][j] = 0;
    if (MODE == MODE_TRANSFORM) {
#pragma unroll
      for (int i = 0; i < TM; ++i) xn[i] = 0;
    }

    for (int k0 = 0; k0 < d; k0 += BK) {
      // ---- global -> registers ----
      T ra[A_LD][VEC], rb[B_LD][VEC];
#pragma unroll
      for (int u = 0; u < A_LD; ++u) {
        int i = tid + u * NT;
        int r = i / (BK / VEC), q = i % (BK / VEC);
        size_t row = row0 + r;
        int col = k0 + q * VEC;
#pragma unroll
        for (int e = 0; e < VEC; ++e) ra[u][e] = 0;
        if (i < BM * BK / VEC && row < n && col < d) VecLoad<T, VEC>::ld(X + row * (size_t)d + col, ra[u]);
      }
#pragma unroll
      for (int u = 0; u < B_LD; ++u) {
        int i = tid + u * NT;
        int r = i / (BK / VEC), q = i % (BK / VEC);
        int c = n0 + r;
        int col = k0 + q * VEC;
#pragma unroll
        for (int e = 0; e < VEC; ++e) rb[u][e] = 0;
        if (i < BN * BK / VEC && c < k && col < d) VecLoad<T, VEC>::ld(C + (size_t)c * d + col, rb[u]);
      }
      __syncthreads();  // previous stage fully consumed
#pragma unroll
      for (int u = 0; u < A_LD; ++u) {
        int i = tid + u * NT;
        int r = i / (BK / VEC), q = i % (BK / VEC);
        if (i < BM * BK / VEC) {
#pragma unroll
          for (int e = 0; e < VEC; ++e) As[q * VEC + e][r] = ra[u][e];
        }
      }
#pragma unroll
      for (int u = 0; u < B_LD; ++u) {
        int i = tid + u * NT;
        int r = i / (BK / VEC), q = i % (BK / VEC);
        if (i < BN * BK / VEC) {
#pragma unroll
          for (int e = 0; e < VEC; ++e) Bs[q * VEC + e][r] = rb[u][e];
        }
      }
      __syncthreads();
      // ---- registers x shared ----
#pragma unroll
      for (int kk = 0; kk < BK; ++kk) {
        T a[TM], b[TN];
#pragma unroll
        for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
        for (int j = 0; j < TN; ++j) b[j] = Bs[kk][tx * TN + j];
#pragma unroll
        for (int i = 0; i < TM; ++i) {
#pragma unroll
          for (int j = 0; j < TN; ++j) acc[i][j] = fma(a[i], b[j], acc[i][j]);
          if (MODE == MODE_TRANSFORM) xn[i] = fma(a[i], a[i], xn[i]);
        }
      }
    }

    // ---- epilogue of this k tile ----
    T cn[TN];
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      int c = n0 + tx * TN + j;
      cn[j] = (c < k) ? cnorm[c] : (T)0;
    }
    if (MODE == MODE_ASSIGN) {
#pragma unroll
      for (int i = 0; i < TM; ++i) {
        T m = Inf<T>::v();
        int mi = 0x7fffffff;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
          int c = n0 + tx * TN + j;
          T s = cn[j] - (T)2 * acc[i][j];
          if (c < k && s < m) { m = s; mi = c; }
        }
#pragma unroll
        for (int o = NTX / 2; o > 0; o >>= 1) {
          T om = __shfl_xor_sync(0xffffffffu, m, o);
          int oi = __shfl_xor_sync(0xffffffffu, mi, o);
          if (om < m || (om == m && oi < mi)) { m = om; mi = oi; }
        }
        if (m < best[i]) { best[i] = m; bidx[i] = mi; }
      }
    } else {
#pragma unroll
      for (int j = 0; j < TN; ++j) {
        int c = n0 + tx * TN + j;
        if (c < k) {
#pragma unroll
          for (int i = 0; i < TM; ++i) {
            size_t row = row0 + ty * TM + i;
            if (row < n) out[(size_t)c * ld_out + row] = fabs(xn[i] + cn[j] - (T)2 * acc[i][j]);
          }
        }
      }
    }
  }

  if (MODE == MODE_ASSIGN) {
    unsigned int changed = 0;
    if (tx == 0) {
#pragma unroll
      for (int i = 0; i < TM; ++i) {
        size_t row = row0 + ty * TM + i;
        if (row < n) {
          changed += (labels[row] != bidx[i]);
          labels[row] = bidx[i];
        }
      }
      if (changed) atomicAdd(&s_changed, changed);
    }
    __syncthreads();
    if (tid == 0 && s_changed && st) atomicAdd(&st->changed, (unsigned long long)s_changed);
  }
}

}  // namespace km
