// E-step for float64 shards on the double-precision tensor-core path (DMMA).
//
// Replaces calculate_distances + relabel (src/gpu/kmeans/kmeans_labels.cu:115-244,
// kmeans_labels.h:360-392) for double data with more than a few centroids.  tcgen05 has no
// float64 kind; the float64 matrix unit of this part is reached through
// mma.sync.m8n8k4.f64, and a dense float64 GEMM of the vendor library runs about three times
// faster on it than the register-tiled FMA kernel of km_tiles.cuh runs on the vector pipe.
// The products are exact and every accumulation rounds once, like an FMA chain, so the scores
// are float64-accurate; they are |c|^2 - 2 x.c, first minimum wins, as in the other kernels.
//
//   CTA: 128 rows x 64 centroids, 8 warps as 4 (rows) x 2 (centroids), warp tile 32 x 32
//        = 4 x 4 fragments of 8 x 8, 32 accumulator doubles per lane; two CTAs per SM, so that
//        one computes while the other sits at its barrier (one CTA of 16 warps and a 128 x 128
//        tile left the unit idle a quarter of the time);
//   d in chunks of 16 columns: X chunk (128 x 16) and centroid chunk (64 x 16) through a
//        three-stage cp.async pipeline; rows of 16 doubles are padded to 20 in shared memory,
//        which makes the fragment loads (lane = (row in 0..7, column in 0..3)) conflict-free;
//   the pipeline runs over the flattened (centroid tile, chunk) pairs, the running
//        (min, argmin) of a row stays in registers across centroid tiles.
// The instruction rate of the unit is low (one m8n8k4 every few cycles per SM), so the kernel is
// bound by it and not by shared memory or L2: 8 fragment loads feed 16 MMAs.
#pragma once

#include "km_common.cuh"

namespace km {
namespace dmma {

constexpr int BM = 128, BN = 64, BK = 16;
constexpr int kPitch = BK + 4;          // doubles per padded row
constexpr int kWarpsN = BN / 32;        // warps side by side over the centroids
constexpr int kThreads = (BM / 32) * kWarpsN * 32;
constexpr int kStages = 3;
constexpr int kVecPerThread = (BM + BN) * (BK / 2) / kThreads;
static_assert((BM + BN) * (BK / 2) % kThreads == 0, "whole vectors per thread");
constexpr size_t kStageDoubles = (size_t)(BM + BN) * kPitch;
constexpr size_t kSmemBytes = kStages * kStageDoubles * sizeof(double);

inline bool shape_ok(int k, int d) { return k > 32 && d % 2 == 0 && d >= 4; }

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, int src_bytes) {
  const unsigned int s = (unsigned int)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// D (8 x 8) += A (8 x 4, row-major) * B (4 x 8, column-major).  Lane l = 4 g + t holds A[g][t],
// B[t][g] and the accumulator pair (g, 2 t), (g, 2 t + 1).
__device__ __forceinline__ void mma884(double (&c)[2], double a, double b) {
  asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};"
               : "+d"(c[0]), "+d"(c[1])
               : "d"(a), "d"(b));
}

__global__ void __launch_bounds__(kThreads, 2)
assign_kernel(const double* __restrict__ X, size_t n, int d, const double* __restrict__ C, int k,
              const double* __restrict__ cnorm, int* __restrict__ labels, IterState* st) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  double* stage = reinterpret_cast<double*>(smem_raw);   // [kStages][(BM + BN)][kPitch]
  __shared__ double s_best[kWarpsN][BM];
  __shared__ int s_idx[kWarpsN][BM];
  __shared__ unsigned int s_changed;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int wm = warp / kWarpsN, wn = warp % kWarpsN;   // warp's place in the grid of warp tiles
  const int g = lane >> 2, t = lane & 3;
  const size_t row0 = (size_t)blockIdx.x * BM;
  const int n_chunks = (d + BK - 1) / BK;
  const int n_ctiles = (k + BN - 1) / BN;
  const int total = n_ctiles * n_chunks;
  if (tid == 0) s_changed = 0;

  // one pair = X chunk + centroid chunk: (BM + BN) rows x 8 vectors of 16 bytes
  auto issue = [&](int pair) {
    if (pair < total) {
      const int ct = pair / n_chunks, kc = pair - ct * n_chunks;
      double* dst = stage + (size_t)(pair % kStages) * kStageDoubles;
#pragma unroll
      for (int j = 0; j < kVecPerThread; ++j) {
        const int v = tid + j * kThreads;
        const int r = v >> 3, q = v & 7;           // row of the stage (X rows first), vector of the row
        const int col = kc * BK + q * 2;
        const bool is_x = r < BM;
        const size_t grow = is_x ? row0 + r : (size_t)ct * BN + (r - BM);
        const bool in = col < d && (is_x ? grow < n : grow < (size_t)k);
        const double* src = (is_x ? X : C) + (in ? grow * (size_t)d + col : 0);
        cp_async16(dst + (size_t)r * kPitch + q * 2, src, in ? 16 : 0);
      }
    }
    cp_async_commit();
  };

  double acc[4][4][2];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j][0] = acc[i][j][1] = 0.0;
  double best[4];
  int bidx[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) { best[i] = Inf<double>::v(); bidx[i] = 0x7fffffff; }

#pragma unroll
  for (int s = 0; s < kStages - 1; ++s) issue(s);

  for (int pair = 0; pair < total; ++pair) {
    cp_async_wait<kStages - 2>();   // this thread's copies of the pair have landed
    __syncthreads();                // ... everybody's; the stage refilled next was read in the last round
    issue(pair + kStages - 1);
    const double* As = stage + (size_t)(pair % kStages) * kStageDoubles + (size_t)(wm * 32 + g) * kPitch + t;
    const double* Bs = stage + (size_t)(pair % kStages) * kStageDoubles + (size_t)(BM + wn * 32 + g) * kPitch + t;
#pragma unroll
    for (int kk = 0; kk < BK / 4; ++kk) {
      double a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[(size_t)i * 8 * kPitch + kk * 4];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[(size_t)j * 8 * kPitch + kk * 4];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) mma884(acc[i][j], a[i], b[j]);
    }
    const int ct = pair / n_chunks, kc = pair - ct * n_chunks;
    if (kc == n_chunks - 1) {
      // ---- scores of this centroid tile: columns ascend with j, then with the pair element ----
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int c0 = ct * BN + wn * 32 + j * 8 + t * 2;
        const double cn0 = (c0 < k) ? cnorm[c0] : 0.0;
        const double cn1 = (c0 + 1 < k) ? cnorm[c0 + 1] : 0.0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const double s0 = cn0 - 2.0 * acc[i][j][0];
          const double s1 = cn1 - 2.0 * acc[i][j][1];
          if (c0 < k && s0 < best[i]) { best[i] = s0; bidx[i] = c0; }
          if (c0 + 1 < k && s1 < best[i]) { best[i] = s1; bidx[i] = c0 + 1; }
          acc[i][j][0] = 0.0;
          acc[i][j][1] = 0.0;
        }
      }
    }
  }
  cp_async_wait<0>();

  // ---- the four lanes of a row group, then the four warps that share the rows ----
#pragma unroll
  for (int i = 0; i < 4; ++i) {
#pragma unroll
    for (int o = 1; o <= 2; o <<= 1) {
      const double ob = __shfl_xor_sync(0xffffffffu, best[i], o);
      const int oi = __shfl_xor_sync(0xffffffffu, bidx[i], o);
      if (ob < best[i] || (ob == best[i] && oi < bidx[i])) { best[i] = ob; bidx[i] = oi; }
    }
    if (t == 0) {
      s_best[wn][wm * 32 + i * 8 + g] = best[i];
      s_idx[wn][wm * 32 + i * 8 + g] = bidx[i];
    }
  }
  __syncthreads();
  if (tid < BM) {
    double m = s_best[0][tid];
    int mi = s_idx[0][tid];
#pragma unroll
    for (int w = 1; w < kWarpsN; ++w) {
      const double om = s_best[w][tid];
      const int oi = s_idx[w][tid];
      if (om < m || (om == m && oi < mi)) { m = om; mi = oi; }
    }
    const size_t row = row0 + tid;
    unsigned int changed = 0;
    if (row < n) {
      if (mi == 0x7fffffff) mi = 0;   // every score NaN-free by the input check; kept for safety
      changed = (labels[row] != mi);
      labels[row] = mi;
    }
    changed = __reduce_add_sync(0xffffffffu, changed);
    if (lane == 0 && changed && st) atomicAdd(&s_changed, changed);
  }
  __syncthreads();
  if (tid == 0 && s_changed && st) atomicAdd(&st->changed, (unsigned long long)s_changed);
}

inline int launch(const double* X, size_t n, int d, const double* C, int k, const double* cnorm, int* labels,
                  IterState* st, cudaStream_t stream) {
  // per device, so set on every launch (cheap)
  KM_CUDA(cudaFuncSetAttribute(assign_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes));
  // without this the driver sizes the shared-memory carve-out for one CTA and only one is resident
  cudaFuncSetAttribute(assign_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
  const size_t grid = (n + BM - 1) / BM;
  if (grid == 0) return KM_OK;
  if (grid > 0x7fffffffULL) KM_FAIL(KM_EINVAL, "shard too large for one launch");
  assign_kernel<<<(unsigned)grid, kThreads, kSmemBytes, stream>>>(X, n, d, C, k, cnorm, labels, st);
  KM_CUDA(cudaGetLastError());
  return KM_OK;
}

}  // namespace dmma
}  // namespace km
