// The small kernels that close an M-step: empty-cluster bookkeeping and
// relocation, averaging, norms, shift.  Replaces revert_zeroed_centroids /
// scale_centroids (src/gpu/kmeans/kmeans_centroids.h:77-105), the host-staged
// multi-GPU divide (src/gpu/kmeans/kmeans_impl.h:140-188), self_dots on the
// centroids (src/gpu/kmeans/kmeans_labels.h:187-214) and the inner_product
// convergence test (kmeans_impl.h:191-208).  The empty-cluster rule is the CPU
// path's (relocate to the farthest points; a cluster still empty copies the
// largest cluster), not the GPU reference's keep-the-old-centroid rule.
#pragma once

#include <cooperative_groups.h>
#include <cuda_fp16.h>

#include "km_common.cuh"
#include "km_tiles.cuh"

namespace km {

namespace cg = cooperative_groups;

// ---- max |x| and finiteness of a shard (once per upload) ----------------------
template <typename T, int V>
__global__ void __launch_bounds__(256)
absmax_kernel(const T* __restrict__ X, size_t count, double* __restrict__ out_max,
              int* __restrict__ out_nonfinite) {
  __shared__ double smax[8];
  double m = 0;
  int bad = 0;
  const size_t nv = count / V;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nv;
       i += (size_t)gridDim.x * blockDim.x) {
    T x[V];
    VecLoad<T, V>::ld(X + i * V, x);
#pragma unroll
    for (int e = 0; e < V; ++e) {
      double a = fabs((double)x[e]);
      bad |= !(a <= 1.7976931348623157e308);
      m = fmax(m, a);
    }
  }
  // tail (count % V) handled by block 0
  if (blockIdx.x == 0 && threadIdx.x < (count % V)) {
    double a = fabs((double)X[nv * V + threadIdx.x]);
    bad |= !(a <= 1.7976931348623157e308);
    m = fmax(m, a);
  }
  m = warp_max(m);
  bad = __any_sync(0xffffffffu, bad);
  if ((threadIdx.x & 31) == 0) smax[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x < 32) {
    m = (threadIdx.x < 8) ? smax[threadIdx.x] : 0.0;
    m = warp_max(m);
    if (threadIdx.x == 0) {
      // order-independent: max of non-negative doubles compared as integers
      atomicMax(reinterpret_cast<unsigned long long*>(out_max), (unsigned long long)__double_as_longlong(m));
    }
  }
  if (bad && (threadIdx.x & 31) == 0) atomicOr(out_nonfinite, 1);
}

// ---- |c|^2 of a centroid table -------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128)
cnorm_kernel(const T* __restrict__ C, int k, int d, T* __restrict__ cnorm, double* __restrict__ C_double = nullptr) {
  __shared__ double red[4];
  int j = blockIdx.x;
  double s = 0;
  for (int t = threadIdx.x; t < d; t += blockDim.x) {
    double v = (double)C[(size_t)j * d + t];
    if (C_double) C_double[(size_t)j * d + t] = v;
    s += v * v;
  }
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) cnorm[j] = (T)(red[0] + red[1] + red[2] + red[3]);
}

// ---- per-iteration bookkeeping: empties, largest cluster ----------------------
// `empties` receives the ids of the empty clusters in ascending order.
__global__ void __launch_bounds__(256)
prepare_kernel(const unsigned long long* __restrict__ gcounts, int k, IterState* st,
               int* __restrict__ empties, int* __restrict__ host_n_empty, int* __restrict__ host_seq, int seq) {
  __shared__ int s_n;
  __shared__ unsigned long long s_best[256];
  __shared__ int s_idx[256];
  if (threadIdx.x == 0) s_n = 0;
  __syncthreads();
  unsigned long long best = 0;
  int bi = 0x7fffffff;
  int local = 0;
  for (int j = threadIdx.x; j < k; j += 256) {
    unsigned long long c = gcounts[j];
    if (c == 0) ++local;
    if (c > best || (c == best && j < bi)) { best = c; bi = j; }
  }
  if (local) atomicAdd(&s_n, local);
  s_best[threadIdx.x] = best;
  s_idx[threadIdx.x] = bi;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if (threadIdx.x < o) {
      const unsigned long long ob = s_best[threadIdx.x + o];
      const int oi = s_idx[threadIdx.x + o];
      if (ob > s_best[threadIdx.x] || (ob == s_best[threadIdx.x] && oi < s_idx[threadIdx.x])) {
        s_best[threadIdx.x] = ob;
        s_idx[threadIdx.x] = oi;
      }
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    st->argmax_count = s_idx[0];
    st->n_empty = s_n;
    st->relocated = 0;
    if (s_n) {
      int e = 0;
      for (int j = 0; j < k; ++j)
        if (gcounts[j] == 0) empties[e++] = j;
    }
    if (host_n_empty) *host_n_empty = s_n;
    if (host_seq) {
      // the host polls this word (pinned memory) instead of synchronising the stream
      __threadfence_system();
      *reinterpret_cast<volatile int*>(host_seq) = seq;
    }
  }
}

// ---- squared distance of every row to its assigned (old) centre ---------------
// Direct differences in double.  Runs only when the M-step found empty clusters (and for
// inertia).  A row is shared by lpr lanes (a power of two, at most 32) that load V elements
// each; a warp works on 32 / lpr rows at a time and on eight adjacent such sets per loop trip
// (4 KB of contiguous rows for d = 64), so that enough loads are in flight to stream X at
// HBM speed.
// The centroid table arrives in double (kept beside the T table by the kernels that write
// centroids) and x is widened with integer operations: float -> double conversions run at a
// small fraction of the FMA rate and were the limit of this kernel (measured again with the table in
// shared memory: 1e7 x 64 in 0.94 ms with conversions, 0.73 ms with the integer form).
// SM = true: the whole table (k_smem * d doubles, dynamic shared memory) is copied into shared memory
// first and the gather by label reads it there - 8 bytes of centroid per 4 bytes of X otherwise go
// through L1, which then is the limit of the kernel.
template <typename T, int V, bool SM = false>
__global__ void __launch_bounds__(256)
rowdist_kernel(const T* __restrict__ X, size_t n, int d, const int* __restrict__ labels,
               const double* __restrict__ C_old, double* __restrict__ dist, const IterState* st,
               int force, int k_smem = 0) {
  if (!force && st->n_empty == 0) return;
  extern __shared__ __align__(16) double rowdist_table[];
  if (SM) {
    // element planes: coordinate idx * V + e of a centroid sits at e * (d / V) + idx, so that the lanes of
    // a row read consecutive doubles (a lane's own V doubles side by side would collide on the banks)
    const int total = k_smem * d, dvs = d / V;
    for (int i = threadIdx.x; i < total; i += blockDim.x) {
      const int c = i / d, col = i - c * d;
      rowdist_table[c * d + (col % V) * dvs + col / V] = C_old[i];
    }
    __syncthreads();
  }
  constexpr int U = 8;
  const int lane = threadIdx.x & 31;
  const size_t warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const size_t nwarp = ((size_t)gridDim.x * blockDim.x) >> 5;
  const int dv = d / V;
  int lpr = 1;
  while (lpr < dv && lpr < 32) lpr <<= 1;
  const int gpw = 32 / lpr;
  const int g = lane / lpr, l = lane % lpr;
  const size_t stride = nwarp * gpw;
  if (dv <= 32) {
    // one vector per lane and row: labels, then rows, are all requested before any arithmetic
    for (size_t base = warp * gpw * U; base < n; base += stride * U) {
      int lab[U];
      T xv[U][V];
      double s[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const size_t row = base + (size_t)u * gpw + g;
        lab[u] = (row < n) ? labels[row] : 0;
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const size_t row = base + (size_t)u * gpw + g;
        if (row < n && l < dv) {
          VecLoadStream<T, V>::ld(X + row * (size_t)d + (size_t)l * V, xv[u]);
        } else {
#pragma unroll
          for (int e = 0; e < V; ++e) xv[u][e] = (T)0;
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const size_t row = base + (size_t)u * gpw + g;
        s[u] = 0;
        if (row < n && l < dv) {
          const double* c = SM ? rowdist_table + (size_t)lab[u] * d + l : C_old + (size_t)lab[u] * d + (size_t)l * V;
#pragma unroll
          for (int e = 0; e < V; ++e) {
            const double q = widen_exact(xv[u][e]) - (SM ? c[e * dv] : c[e]);
            s[u] = fma(q, q, s[u]);
          }
        }
      }
      // The eight partial sums of a lane belong to eight rows.  Instead of eight butterflies over the lpr
      // lanes of a row, the lanes first trade halves (xor 1: rows 0-3 against 4-7, xor 2, xor 4), which
      // leaves every lane one row's sum over eight lanes after 7 instead of 24 exchanges; a plain butterfly
      // finishes rows wider than eight lanes.  The additions of a row form the same tree whichever lane
      // ends up with it, so its value does not depend on where in a shard the row sits.
      int ubase = 0, cnt = U;
      if (lpr > 1) {
        const bool up = (l & 1) != 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const double keep = up ? s[i + 4] : s[i], send = up ? s[i] : s[i + 4];
          s[i] = keep + __shfl_xor_sync(0xffffffffu, send, 1);
        }
        ubase += up ? 4 : 0;
        cnt = 4;
      }
      if (lpr > 2) {
        const bool up = (l & 2) != 0;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const double keep = up ? s[i + 2] : s[i], send = up ? s[i] : s[i + 2];
          s[i] = keep + __shfl_xor_sync(0xffffffffu, send, 2);
        }
        ubase += up ? 2 : 0;
        cnt = 2;
      }
      if (lpr > 4) {
        const bool up = (l & 4) != 0;
        const double keep = up ? s[1] : s[0], send = up ? s[0] : s[1];
        s[0] = keep + __shfl_xor_sync(0xffffffffu, send, 4);
        ubase += up ? 1 : 0;
        cnt = 1;
      }
      for (int o = 8; o < lpr; o <<= 1) s[0] += __shfl_xor_sync(0xffffffffu, s[0], o);
      if (l < 8) {
#pragma unroll
        for (int i = 0; i < U; ++i) {
          const size_t row = base + (size_t)(ubase + i) * gpw + g;
          if (i < cnt && row < n) dist[row] = s[i];
        }
      }
    }
    return;
  }
  for (size_t base = warp * gpw * U; base < n; base += stride * U) {
    double s[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      s[u] = 0;
      const size_t row = base + (size_t)u * gpw + g;
      if (row < n) {
        const T* x = X + row * (size_t)d;
        const double* c = (SM ? rowdist_table : C_old) + (size_t)labels[row] * d;
        for (int idx = l; idx < dv; idx += lpr) {
          T xv[V];
          VecLoadStream<T, V>::ld(x + (size_t)idx * V, xv);
#pragma unroll
          for (int e = 0; e < V; ++e) {
            const double q = widen_exact(xv[e]) - (SM ? c[e * dv + idx] : c[(size_t)idx * V + e]);
            s[u] = fma(q, q, s[u]);
          }
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      for (int o = lpr >> 1; o > 0; o >>= 1) s[u] += __shfl_xor_sync(0xffffffffu, s[u], o);
      const size_t row = base + (size_t)u * gpw + g;
      if (l == 0 && row < n) dist[row] = s[u];
    }
  }
}

// Sum of dist (inertia; weighted by W when given), deterministic two-stage tree: per-CTA partials
// then CTA 0.
template <typename T>
__global__ void __launch_bounds__(256)
sum_partials_kernel(const double* __restrict__ v, size_t n, double* __restrict__ partials,
                    const T* __restrict__ W = nullptr) {
  __shared__ double red[8];
  double s = 0;
  for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (size_t)gridDim.x * 256)
    s += W ? v[i] * (double)W[i] : v[i];
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0;
    for (int w = 0; w < 8; ++w) t += red[w];
    partials[blockIdx.x] = t;
  }
}
// One warp: lane l adds partials [l * per, (l + 1) * per) in order, then a butterfly over the lanes.
__global__ void sum_final_kernel(const double* __restrict__ partials, int m, double* out) {
  if (blockIdx.x != 0 || threadIdx.x >= 32) return;
  const int per = (m + 31) / 32;
  const int b = threadIdx.x * per, e = min(m, b + per);
  double t = 0;
  for (int i = b; i < e; ++i) t += partials[i];
  t = warp_sum(t);
  if (threadIdx.x == 0) *out = t;
}

// ---- the E farthest rows of a shard in two passes over the distances ------------------
// The empty-cluster rule needs the E rows with the largest distance to their centre, in
// descending order (ties: lowest row).  Taking them one at a time costs E passes over the shard's
// distances and 2 E grid-wide barriers (48 empty clusters on 2.5e7 rows: 10 ms).  Here: pass 1,
// every thread keeps the largest distance among its rows; the E-th largest of these thread maxima
// is a lower bound T of the E-th largest distance of the shard (they belong to E different rows);
// pass 2 collects the rows with distance >= T - the E farthest are among them - into a candidate
// list that one CTA then orders.  Returns false when the list overflows (very many rows tied at the
// threshold); the caller then falls back to one pass per row.
constexpr int kFarDirectMax = 4;   // up to this many empty clusters are served one pass at a time
struct FarScratch {
  double* tmax;                  // [grid * 256] thread maxima
  unsigned long long* trow;
  double* cval;                  // [cap] candidates
  unsigned long long* crow;
  double* oval;                  // [>= E] result, descending
  unsigned long long* orow;
  unsigned int* counters;        // [0] candidates, [1] overflow
  double* thr;                   // threshold T
  int cap;
};

// block-wide arg-max over (v, r) pairs with an index payload; ties: lowest row.  256 threads.
__device__ __forceinline__ void block_argmax(double& bv, unsigned long long& br, int& bi, double* s_v,
                                             unsigned long long* s_r, int* s_i) {
  s_v[threadIdx.x] = bv;
  s_r[threadIdx.x] = br;
  s_i[threadIdx.x] = bi;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if (threadIdx.x < o) {
      const double ov = s_v[threadIdx.x + o];
      const unsigned long long orow = s_r[threadIdx.x + o];
      if (ov > s_v[threadIdx.x] || (ov == s_v[threadIdx.x] && orow < s_r[threadIdx.x])) {
        s_v[threadIdx.x] = ov;
        s_r[threadIdx.x] = orow;
        s_i[threadIdx.x] = s_i[threadIdx.x + o];
      }
    }
    __syncthreads();
  }
  bv = s_v[0];
  br = s_r[0];
  bi = s_i[0];
  __syncthreads();
}

// Called by every thread of a cooperative grid of 256-thread CTAs.  On success oval / orow hold the
// min(E, rows) farthest rows in descending order and *n_out their number.
__device__ bool top_far(cg::grid_group& grid, const double* __restrict__ dist, size_t n, int E, const FarScratch& fs,
                        double* s_v, unsigned long long* s_r, int* s_i, int* n_out) {
  const size_t per = (n + gridDim.x - 1) / gridDim.x;
  const size_t b0 = (size_t)blockIdx.x * per;
  const size_t b1 = (b0 + per < n) ? b0 + per : n;
  const size_t gtid = (size_t)blockIdx.x * 256 + threadIdx.x;
  const int M = (int)gridDim.x * 256;
  {
    double bv = -1.0;
    unsigned long long br = ~0ULL;
    for (size_t i = b0 + threadIdx.x; i < b1; i += 256) {
      const double v = dist[i];
      if (v > bv) { bv = v; br = i; }
    }
    fs.tmax[gtid] = bv;
    fs.trow[gtid] = br;
    if (gtid == 0) { fs.counters[0] = 0; fs.counters[1] = 0; }
  }
  grid.sync();
  if (blockIdx.x == 0) {
    // E-th largest thread maximum (removing one maximum per round)
    double T = 0.0;
    for (int e = 0; e < E; ++e) {
      double bv = -1.0;
      unsigned long long br = ~0ULL;
      int bi = -1;
      for (int c = threadIdx.x; c < M; c += 256) {
        const double v = __ldcg(fs.tmax + c);
        const unsigned long long r = __ldcg(fs.trow + c);
        if (v > bv || (v == bv && r < br)) { bv = v; br = r; bi = c; }
      }
      block_argmax(bv, br, bi, s_v, s_r, s_i);
      if (bv < 0.0) { T = 0.0; break; }      // fewer than E rows: every row is a candidate
      T = bv;
      if (threadIdx.x == 0) fs.tmax[bi] = -3.0;
      __syncthreads();
    }
    if (threadIdx.x == 0) *fs.thr = T;
  }
  grid.sync();
  {
    const double T = __ldcg(fs.thr);
    for (size_t i = b0 + threadIdx.x; i < b1; i += 256) {
      const double v = dist[i];
      if (v >= T) {
        const unsigned int pos = atomicAdd(&fs.counters[0], 1u);
        if (pos < (unsigned int)fs.cap) { fs.cval[pos] = v; fs.crow[pos] = i; }
        else fs.counters[1] = 1u;
      }
    }
  }
  grid.sync();
  if (__ldcg(fs.counters + 1) != 0u) return false;
  const int C = (int)__ldcg(fs.counters);
  const int take = E < C ? E : C;
  if (blockIdx.x == 0) {
    for (int e = 0; e < take; ++e) {
      double bv = -4.0;
      unsigned long long br = ~0ULL;
      int bi = -1;
      for (int c = threadIdx.x; c < C; c += 256) {
        const double v = __ldcg(fs.cval + c);
        const unsigned long long r = __ldcg(fs.crow + c);
        if (v > bv || (v == bv && r < br)) { bv = v; br = r; bi = c; }
      }
      block_argmax(bv, br, bi, s_v, s_r, s_i);
      if (threadIdx.x == 0) {
        fs.oval[e] = bv;
        fs.orow[e] = br;
        fs.cval[bi] = -5.0;
      }
      __syncthreads();
    }
  }
  *n_out = take;
  return true;
}

// ---- relocation of empty clusters (cooperative launch, single shard) ----------
// For each empty cluster, lowest id first: take the remaining row with the
// largest distance to its assigned centre (ties: lowest row), remove it from its
// donor's sums and make it the sole member of the empty cluster.  Nothing moves
// when the largest distance is zero.  `cand_*` hold one candidate per CTA.
template <typename T>
__global__ void __launch_bounds__(256)
relocate_kernel(const T* __restrict__ X, size_t n, int d, const int* __restrict__ labels, int k,
                double* __restrict__ dist, long long* __restrict__ gsums,
                unsigned long long* __restrict__ gcounts, const int* __restrict__ empties,
                IterState* st, double* __restrict__ cand_val, unsigned long long* __restrict__ cand_row,
                T scale, const T* __restrict__ W, T wscale, FarScratch fs) {
  constexpr int NP = Fixed<T>::NP;
  const int E = st->n_empty;
  if (E == 0) return;
  cg::grid_group grid = cg::this_grid();
  __shared__ double s_v[256];
  __shared__ unsigned long long s_r[256];
  __shared__ int s_i[256];
  const size_t per = (n + gridDim.x - 1) / gridDim.x;
  const size_t b0 = (size_t)blockIdx.x * per;
  const size_t b1 = (b0 + per < n) ? b0 + per : n;

  int n_far = 0;
  // (a handful of empty clusters: one pass per cluster is cheaper than the two passes and the ordering)
  if (E > kFarDirectMax && top_far(grid, dist, n, E, fs, s_v, s_r, s_i, &n_far)) {
    // the farthest rows are known and ordered: one CTA moves them, lowest empty cluster first
    if (blockIdx.x != 0) return;
    for (int e = 0; e < n_far; ++e) {
      const double bv = fs.oval[e];
      const unsigned long long br = fs.orow[e];
      if (bv < 0.0 || (e == 0 && bv == 0.0)) break;
      const int cid = empties[e];
      const int old = labels[br];
      const T* x = X + (size_t)br * d;
      const T w = W ? W[br] : (T)1;
      long long units = 1;
      if (W) {
        int pw[2];
        split_pieces<2>(w, wscale, pw);
        units = (long long)pw[0] * (1LL << kPieceBits) + (long long)pw[1];
      }
      for (int t = threadIdx.x; t < d; t += 256) {
        int p[NP];
        split_pieces<NP>(W ? x[t] * w : x[t], scale, p);
#pragma unroll
        for (int q = 0; q < NP / 2; ++q) {
          long long v = (long long)p[2 * q] * (1LL << kPieceBits) + (long long)p[2 * q + 1];
          gsums[(size_t)q * k * d + (size_t)old * d + t] -= v;
          gsums[(size_t)q * k * d + (size_t)cid * d + t] = v;
        }
      }
      __syncthreads();   // two relocated rows may share a donor cluster: one row's updates at a time
      if (threadIdx.x == 0) {
        gcounts[cid] = (unsigned long long)units;
        gcounts[old] -= (unsigned long long)units;
        st->relocated += 1;
      }
      __syncthreads();
    }
    return;
  }

  // (candidate list overflowed: one pass over the distances per empty cluster)
  for (int e = 0; e < E; ++e) {
    double bv = -1.0;
    unsigned long long br = ~0ULL;
    for (size_t i = b0 + threadIdx.x; i < b1; i += 256) {
      double v = dist[i];
      if (v > bv) { bv = v; br = i; }  // ascending i: first maximum kept
    }
    s_v[threadIdx.x] = bv;
    s_r[threadIdx.x] = br;
    __syncthreads();
    for (int o = 128; o > 0; o >>= 1) {
      if (threadIdx.x < o) {
        double ov = s_v[threadIdx.x + o];
        unsigned long long orow = s_r[threadIdx.x + o];
        if (ov > s_v[threadIdx.x] || (ov == s_v[threadIdx.x] && orow < s_r[threadIdx.x])) {
          s_v[threadIdx.x] = ov;
          s_r[threadIdx.x] = orow;
        }
      }
      __syncthreads();
    }
    if (threadIdx.x == 0) { cand_val[blockIdx.x] = s_v[0]; cand_row[blockIdx.x] = s_r[0]; }
    grid.sync();
    // every CTA takes the same decision from the candidate table
    bv = -1.0;
    br = ~0ULL;
    for (unsigned int c = threadIdx.x; c < gridDim.x; c += 256) {
      double v = cand_val[c];
      unsigned long long r = cand_row[c];
      if (v > bv || (v == bv && r < br)) { bv = v; br = r; }
    }
    s_v[threadIdx.x] = bv;
    s_r[threadIdx.x] = br;
    __syncthreads();
    for (int o = 128; o > 0; o >>= 1) {
      if (threadIdx.x < o) {
        double ov = s_v[threadIdx.x + o];
        unsigned long long orow = s_r[threadIdx.x + o];
        if (ov > s_v[threadIdx.x] || (ov == s_v[threadIdx.x] && orow < s_r[threadIdx.x])) {
          s_v[threadIdx.x] = ov;
          s_r[threadIdx.x] = orow;
        }
      }
      __syncthreads();
    }
    bv = s_v[0];
    br = s_r[0];
    __syncthreads();
    bool stop = (bv < 0.0) || (e == 0 && bv == 0.0);
    if (stop) break;  // uniform over the grid
    if (blockIdx.x == 0) {
      const int cid = empties[e];
      const int old = labels[br];
      const T* x = X + (size_t)br * d;
      // with sample weights the row carries w * x in the sums and its fixed-point weight in the counts
      const T w = W ? W[br] : (T)1;
      long long units = 1;
      if (W) {
        int pw[2];
        split_pieces<2>(w, wscale, pw);
        units = (long long)pw[0] * (1LL << kPieceBits) + (long long)pw[1];
      }
      for (int t = threadIdx.x; t < d; t += 256) {
        int p[NP];
        split_pieces<NP>(W ? x[t] * w : x[t], scale, p);
#pragma unroll
        for (int q = 0; q < NP / 2; ++q) {
          long long v = (long long)p[2 * q] * (1LL << kPieceBits) + (long long)p[2 * q + 1];
          gsums[(size_t)q * k * d + (size_t)old * d + t] -= v;
          gsums[(size_t)q * k * d + (size_t)cid * d + t] = v;
        }
      }
      if (threadIdx.x == 0) {
        gcounts[cid] = (unsigned long long)units;
        gcounts[old] -= (unsigned long long)units;
        dist[br] = -2.0;
        st->relocated += 1;
      }
    }
    grid.sync();
  }
}

// ---- averaging, norms, shift, logs and the tensor-core operands in one kernel ----------
// Where the split centroid table of the tensor-core distance kernels goes (null bhi: not used):
// bhi / blo = fp16 halves of -2 c * sb, rows of `dp` halves (columns >= d zero), `npad` rows
// (rows >= k zero); cn_pad[j] = |c_j|^2 * sxsb (+inf for padding rows), cn_pad[npad] = max |c_j|^2.
struct SplitTable {
  __half* bhi;
  __half* blo;
  float* cn_pad;
  int npad, dp;
  float sb, sxsb;
};

template <typename T>
__device__ __forceinline__ void split_table_row(const SplitTable& tp, int j, int d, const T* c_row, T cn) {}
template <>
__device__ __forceinline__ void split_table_row<float>(const SplitTable& tp, int j, int d, const float* c_row,
                                                       float cn) {
  for (int t = threadIdx.x; t < tp.dp; t += blockDim.x) {
    const float v = (t < d) ? -2.0f * c_row[t] * tp.sb : 0.0f;
    const __half h = __float2half_rn(v);
    tp.bhi[(size_t)j * tp.dp + t] = h;
    tp.blo[(size_t)j * tp.dp + t] = __float2half_rn(v - __half2float(h));
  }
  if (threadIdx.x == 0) tp.cn_pad[j] = cn * tp.sxsb;
}

// One CTA per cluster closes an M-step: mean of the cluster in double -> T (inv = 2^-(sa+15) turns
// the int64 pairs back into sums), |c|^2, the cluster's squared shift, and - for the tensor-core
// distance kernels - the cluster's row of the split operand table.  A cluster without members
// copies the largest cluster's row as the CPU path leaves it at that moment: already averaged if
// its id is lower, raw sums if not.  The CTA that finishes last (a ticket counter) adds the
// per-cluster shifts in a fixed order, logs the iteration, re-arms the label-change counter and
// writes the padding rows and the largest |c|^2 of the operand table.
// run_if: 0 = only when the M-step found no empty cluster, 1 = only when it found one (queued
// behind the repair kernels), 2 = always.  The pair (0, 1) around the gated repair kernels lets the
// stream decide on the device, so the host never waits for the count of empty clusters.
template <typename T>
__global__ void __launch_bounds__(128)
close_kernel(const long long* __restrict__ gsums, const unsigned long long* __restrict__ gcounts,
             int k, int d, double inv, const T* __restrict__ C_old, T* __restrict__ C_new,
             T* __restrict__ cnorm, double* __restrict__ shift_k, IterState* st,
             double* __restrict__ C_new_double, int run_if, double count_unit,
             double* __restrict__ shift_log, unsigned long long* __restrict__ changed_log,
             int* __restrict__ reloc_log, unsigned int* __restrict__ amb_log, int it,
             double* __restrict__ host_shift, unsigned long long* __restrict__ host_changed,
             unsigned int* __restrict__ ticket, SplitTable tp) {
  constexpr int NP = Fixed<T>::NP;
  // count_unit: weight of one unit of gcounts (1 for plain counts, a power of two for sample weights)
  const int n_empty = st->n_empty;
  if ((run_if == 0 && n_empty != 0) || (run_if == 1 && n_empty == 0)) return;
  __shared__ double red_n[4], red_s[4];
  __shared__ int s_src, s_last;
  const int j = blockIdx.x;
  unsigned long long cnt = gcounts[j];
  int src = j;
  double a;
  if (cnt > 0) {
    a = 1.0 / ((double)cnt * count_unit);
  } else {
    // still empty after the relocation (no row left to take, or a row of weight zero): the
    // largest cluster as the counts stand now, lowest id on ties
    if (threadIdx.x == 0) {
      unsigned long long best = 0;
      int bi = 0;
      for (int c = 0; c < k; ++c) {
        const unsigned long long v = gcounts[c];
        if (v > best) { best = v; bi = c; }
      }
      s_src = bi;
    }
    __syncthreads();
    src = s_src;
    unsigned long long cb = gcounts[src];
    a = (src < j && cb > 0) ? 1.0 / ((double)cb * count_unit) : 1.0;
  }
  double sn = 0, ss = 0;
  for (int t = threadIdx.x; t < d; t += blockDim.x) {
    long long g[NP / 2];
#pragma unroll
    for (int q = 0; q < NP / 2; ++q) g[q] = gsums[(size_t)q * k * d + (size_t)src * d + t];
    T v = (T)(fixed_to_double<NP>(g, inv) * a);
    C_new[(size_t)j * d + t] = v;
    double dv = (double)v;
    if (C_new_double) C_new_double[(size_t)j * d + t] = dv;
    double df = dv - (double)C_old[(size_t)j * d + t];
    sn += dv * dv;
    ss += df * df;
  }
  sn = warp_sum(sn);
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) { red_n[threadIdx.x >> 5] = sn; red_s[threadIdx.x >> 5] = ss; }
  __syncthreads();
  const T cn = (T)(red_n[0] + red_n[1] + red_n[2] + red_n[3]);
  if (threadIdx.x == 0) {
    cnorm[j] = cn;
    shift_k[j] = red_s[0] + red_s[1] + red_s[2] + red_s[3];
  }
  if (tp.bhi != nullptr) {
    __syncthreads();   // the row of C_new written above is read back by other threads
    split_table_row<T>(tp, j, d, C_new + (size_t)j * d, cn);
  }
  // ---- the last CTA closes the iteration ----
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_last = (atomicAdd(ticket, 1u) == gridDim.x - 1) ? 1 : 0;
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  __shared__ double red[128];
  __shared__ float redm[128];
  double s = 0;
  float m = 0.f;
  for (int c = threadIdx.x; c < k; c += 128) {
    s += __ldcg(shift_k + c);
    if (tp.bhi != nullptr) m = fmaxf(m, (float)__ldcg(cnorm + c));
  }
  red[threadIdx.x] = s;
  redm[threadIdx.x] = m;
  __syncthreads();
  for (int o = 64; o > 0; o >>= 1) {
    if (threadIdx.x < o) {
      red[threadIdx.x] += red[threadIdx.x + o];
      redm[threadIdx.x] = fmaxf(redm[threadIdx.x], redm[threadIdx.x + o]);
    }
    __syncthreads();
  }
  if (tp.bhi != nullptr) {
    for (int r = k; r < tp.npad; ++r) {
      for (int t = threadIdx.x; t < tp.dp; t += 128) {
        tp.bhi[(size_t)r * tp.dp + t] = __float2half_rn(0.f);
        tp.blo[(size_t)r * tp.dp + t] = __float2half_rn(0.f);
      }
      if (threadIdx.x == 0) tp.cn_pad[r] = __int_as_float(0x7f800000);
    }
    if (threadIdx.x == 0) tp.cn_pad[tp.npad] = redm[0];
  }
  if (threadIdx.x == 0) {
    *ticket = 0;
    st->shift_sq = red[0];
    shift_log[it] = red[0];
    changed_log[it] = st->changed;
    reloc_log[it] = st->relocated;
    amb_log[it] = st->amb_count;
    st->amb_count = 0;
    if (host_shift) { *host_shift = red[0]; *host_changed = st->changed; }
    st->changed = 0;
  }
}

}  // namespace km

namespace km {

// ---- relocation across several shards / ranks ----------------------------------
// Each shard lists its E farthest rows (descending distance, ties lowest row) as
// one packed record: [E double val][E u64 id][E i64 label][E double weight][E*d T row].  The
// records of all ranks are all-gathered and every rank applies the same E-way
// choice to its (already all-reduced, hence identical) sums.
template <typename T>
__global__ void __launch_bounds__(256)
select_far_kernel(const T* __restrict__ X, size_t n, int d, const int* __restrict__ labels,
                  double* __restrict__ dist, int E, unsigned long long id_base,
                  double* __restrict__ cand_val, unsigned long long* __restrict__ cand_row,
                  unsigned char* __restrict__ rec, const T* __restrict__ W, const IterState* gate, FarScratch fs) {
  // with a gate the number of empty clusters is read on the device (the same on every rank: the
  // counts were all-reduced) and the kernel returns at once when there is none
  if (gate != nullptr) {
    E = gate->n_empty;
    if (E == 0) return;
  }
  cg::grid_group grid = cg::this_grid();
  __shared__ double s_v[256];
  __shared__ unsigned long long s_r[256];
  __shared__ int s_i[256];
  double* r_val = reinterpret_cast<double*>(rec);
  unsigned long long* r_id = reinterpret_cast<unsigned long long*>(rec + (size_t)E * 8);
  long long* r_lab = reinterpret_cast<long long*>(rec + (size_t)E * 16);
  double* r_w = reinterpret_cast<double*>(rec + (size_t)E * 24);
  T* r_vec = reinterpret_cast<T*>(rec + (size_t)E * 32);
  const size_t per = (n + gridDim.x - 1) / gridDim.x;
  const size_t b0 = (size_t)blockIdx.x * per;
  const size_t b1 = (b0 + per < n) ? b0 + per : n;
  int n_far = 0;
  if (E > kFarDirectMax && top_far(grid, dist, n, E, fs, s_v, s_r, s_i, &n_far)) {
    if (blockIdx.x != 0) return;
    for (int e = 0; e < E; ++e) {
      const bool have = e < n_far && fs.oval[e] >= 0.0;
      const unsigned long long br = have ? fs.orow[e] : 0ULL;
      if (threadIdx.x == 0) {
        r_val[e] = have ? fs.oval[e] : -1.0;
        r_id[e] = have ? (id_base + br) : ~0ULL;
        r_lab[e] = have ? (long long)labels[br] : -1;
        r_w[e] = (have && W) ? (double)W[br] : 1.0;
      }
      for (int t = threadIdx.x; t < d; t += 256) r_vec[(size_t)e * d + t] = have ? X[(size_t)br * d + t] : (T)0;
    }
    return;
  }
  for (int e = 0; e < E; ++e) {
    double bv = -1.0;
    unsigned long long br = ~0ULL;
    for (size_t i = b0 + threadIdx.x; i < b1; i += 256) {
      double v = dist[i];
      if (v > bv) { bv = v; br = i; }
    }
    s_v[threadIdx.x] = bv;
    s_r[threadIdx.x] = br;
    __syncthreads();
    for (int o = 128; o > 0; o >>= 1) {
      if (threadIdx.x < o) {
        double ov = s_v[threadIdx.x + o];
        unsigned long long orow = s_r[threadIdx.x + o];
        if (ov > s_v[threadIdx.x] || (ov == s_v[threadIdx.x] && orow < s_r[threadIdx.x])) {
          s_v[threadIdx.x] = ov;
          s_r[threadIdx.x] = orow;
        }
      }
      __syncthreads();
    }
    if (threadIdx.x == 0) { cand_val[blockIdx.x] = s_v[0]; cand_row[blockIdx.x] = s_r[0]; }
    grid.sync();
    if (blockIdx.x == 0) {
      bv = -1.0;
      br = ~0ULL;
      for (unsigned int c = threadIdx.x; c < gridDim.x; c += 256) {
        double v = cand_val[c];
        unsigned long long r = cand_row[c];
        if (v > bv || (v == bv && r < br)) { bv = v; br = r; }
      }
      s_v[threadIdx.x] = bv;
      s_r[threadIdx.x] = br;
      __syncthreads();
      for (int o = 128; o > 0; o >>= 1) {
        if (threadIdx.x < o) {
          double ov = s_v[threadIdx.x + o];
          unsigned long long orow = s_r[threadIdx.x + o];
          if (ov > s_v[threadIdx.x] || (ov == s_v[threadIdx.x] && orow < s_r[threadIdx.x])) {
            s_v[threadIdx.x] = ov;
            s_r[threadIdx.x] = orow;
          }
        }
        __syncthreads();
      }
      bv = s_v[0];
      br = s_r[0];
      __syncthreads();
      const bool have = (bv >= 0.0) && (br != ~0ULL);
      if (threadIdx.x == 0) {
        r_val[e] = have ? bv : -1.0;
        r_id[e] = have ? (id_base + br) : ~0ULL;
        r_lab[e] = have ? (long long)labels[br] : -1;
        r_w[e] = (have && W) ? (double)W[br] : 1.0;
        if (have) dist[br] = -2.0;
      }
      for (int t = threadIdx.x; t < d; t += 256) r_vec[(size_t)e * d + t] = have ? X[(size_t)br * d + t] : (T)0;
    }
    grid.sync();
  }
}

// The E-way choice among the gathered records, applied to this rank's (all-reduced, hence
// identical) sums: one CTA of 256 threads.  FRESH: the records were written by other GPUs into
// memory this SM may have cached from an earlier exchange, so they are read past L1.
template <typename V, bool FRESH>
__device__ __forceinline__ V rec_load(const V* p) { return FRESH ? __ldcv(p) : *p; }

template <typename T, bool FRESH>
__device__ __forceinline__ void apply_far_body(const unsigned char* rec_all, int world, int E, size_t rec_stride, int k,
                                               int d, long long* gsums, unsigned long long* gcounts,
                                               const int* empties, IterState* st, T scale, int weighted, T wscale) {
  constexpr int NP = Fixed<T>::NP;
  __shared__ int head[64];
  __shared__ int s_w;
  __shared__ int s_stop;
  if (threadIdx.x < 64) head[threadIdx.x] = 0;
  __syncthreads();
  for (int e = 0; e < E; ++e) {
    if (threadIdx.x == 0) {
      double bv = -1.0;
      unsigned long long bid = ~0ULL;
      int bw = -1;
      for (int w = 0; w < world; ++w) {
        if (head[w] >= E) continue;
        const unsigned char* rec = rec_all + (size_t)w * rec_stride;
        double v = rec_load<double, FRESH>(reinterpret_cast<const double*>(rec) + head[w]);
        unsigned long long id =
            rec_load<unsigned long long, FRESH>(reinterpret_cast<const unsigned long long*>(rec + (size_t)E * 8) + head[w]);
        if (v > bv || (v == bv && id < bid)) { bv = v; bid = id; bw = w; }
      }
      s_w = bw;
      s_stop = (bw < 0) || (bv < 0.0) || (e == 0 && bv == 0.0);
    }
    __syncthreads();
    if (s_stop) break;
    const int w = s_w;
    const unsigned char* rec = rec_all + (size_t)w * rec_stride;
    const int h = head[w];
    const int old = (int)rec_load<long long, FRESH>(reinterpret_cast<const long long*>(rec + (size_t)E * 16) + h);
    const T* x = reinterpret_cast<const T*>(rec + (size_t)E * 32) + (size_t)h * d;
    const T wt = (T)rec_load<double, FRESH>(reinterpret_cast<const double*>(rec + (size_t)E * 24) + h);
    long long units = 1;
    if (weighted) {
      int pw[2];
      split_pieces<2>(wt, wscale, pw);
      units = (long long)pw[0] * (1LL << kPieceBits) + (long long)pw[1];
    }
    const int cid = empties[e];
    for (int t = threadIdx.x; t < d; t += 256) {
      int p[NP];
      const T xv = rec_load<T, FRESH>(x + t);
      split_pieces<NP>(weighted ? xv * wt : xv, scale, p);
#pragma unroll
      for (int q = 0; q < NP / 2; ++q) {
        long long v = (long long)p[2 * q] * (1LL << kPieceBits) + (long long)p[2 * q + 1];
        gsums[(size_t)q * k * d + (size_t)old * d + t] -= v;
        gsums[(size_t)q * k * d + (size_t)cid * d + t] = v;
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      gcounts[cid] = (unsigned long long)units;
      gcounts[old] -= (unsigned long long)units;
      st->relocated += 1;
      head[w] = h + 1;
    }
    __syncthreads();
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
apply_far_kernel(const unsigned char* __restrict__ rec_all, int world, int E, size_t rec_bytes, int k, int d,
                 long long* __restrict__ gsums, unsigned long long* __restrict__ gcounts,
                 const int* __restrict__ empties, IterState* st, T scale, int weighted, T wscale) {
  apply_far_body<T, false>(rec_all, world, E, rec_bytes, k, d, gsums, gcounts, empties, st, scale, weighted, wscale);
}

// Several ranks, decided on the device: when the M-step left empty clusters (st->n_empty, the same on
// every rank) this one CTA stores the rank's candidate record into slot `rank` of every peer's gather
// mailbox (plain peer stores), raises its flag there, waits - bounded by `spin_limit` polls - for all
// ranks' flags in its own mailbox and applies the common choice.  No empty cluster: returns at once,
// nothing is sent.  One mailbox generation is enough: two exchanges are always separated by an
// all-reduce of the sums, which no rank passes before every rank has finished the earlier exchange.
//   gmail[world][slot_bytes], gflags[world] (sequence number of the last record a rank delivered)
template <typename T>
__global__ void __launch_bounds__(256)
gather_apply_kernel(const unsigned char* __restrict__ rec, size_t slot_bytes, int rank, int world,
                    unsigned char* const* __restrict__ peer_gmail, unsigned int* const* __restrict__ peer_gflags,
                    const unsigned char* my_gmail, const unsigned int* my_gflags, unsigned int seq,
                    unsigned int spin_limit, int k, int d, long long* __restrict__ gsums,
                    unsigned long long* __restrict__ gcounts, const int* __restrict__ empties, IterState* st,
                    T scale, int weighted, T wscale) {
  const int E = st->n_empty;
  if (E == 0) return;
  __shared__ int s_bad;
  if (threadIdx.x == 0) s_bad = 0;
  const size_t words = ((size_t)E * 32 + (size_t)E * d * sizeof(T)) / 4;
  const unsigned int* src = reinterpret_cast<const unsigned int*>(rec);
  for (int p = 0; p < world; ++p) {
    unsigned int* dst = reinterpret_cast<unsigned int*>(peer_gmail[p] + (size_t)rank * slot_bytes);
    for (size_t i = threadIdx.x; i < words; i += 256) dst[i] = src[i];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < world) {
    *reinterpret_cast<volatile unsigned int*>(peer_gflags[threadIdx.x] + rank) = seq;
    __threadfence_system();
    const volatile unsigned int* f = my_gflags + threadIdx.x;
    unsigned int spins = 0;
    while (*f != seq) {
      if (++spins > spin_limit) { s_bad = 1; break; }
      __nanosleep(40);
    }
  }
  __syncthreads();
  if (s_bad) {
    if (threadIdx.x == 0) atomicMax(&st->error, 12);
    return;
  }
  __threadfence();
  apply_far_body<T, true>(my_gmail, world, E, slot_bytes, k, d, gsums, gcounts, empties, st, scale, weighted, wscale);
}

}  // namespace km
