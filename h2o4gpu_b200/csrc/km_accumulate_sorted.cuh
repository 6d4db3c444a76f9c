// Centroid sums of a labelled float32 shard, run-length version.
//
// The plain kernel (km_accumulate.cuh) spends two shared-memory atomics and about
// twenty instructions on every element and is issue-bound.  Here each CTA takes a
// tile of rows, counting-sorts the tile's row indices by label in shared memory
// (two atomics per ROW), and then lets every group of threads walk a contiguous
// piece of the sorted list: rows with the same label arrive back to back, so the
// group keeps the running sum of its columns in registers - one multiply, one
// float->int conversion and a 64-bit integer add per element - and touches the
// shared accumulators only when the label changes.  X is still read exactly once
// (each row is a contiguous 16-byte-per-thread gather inside the tile's window).
//
// Arithmetic is the same fixed point as everywhere else: v = rint(x * 2^(30-e)) for
// max|x| < 2^e, summed as integers, so the result is identical, bit for bit, to the
// two-piece scheme of km_common.cuh and independent of any ordering.  A run sum
// (< 2^30 * run length) is cut into three non-overlapping pieces (bits 30.., 15..29,
// 0..14) that are added to int32 shared accumulators; a CTA drains them into the
// int64 global sums at least every 65536 rows.  When k * d is too large for shared
// accumulators, run sums go straight to the global sums with 64-bit reductions and
// the tile is made as large as shared memory allows so that runs stay long.
#pragma once

#include "km_common.cuh"

namespace km {

constexpr int kSortThreads = 512;
constexpr int kSortMaxK = 4096;        // histogram / offsets in shared memory
constexpr int kSortDrainRows = 65536;  // int32 headroom of the shared accumulators

struct SortPlan {
  int tile_rows;     // rows per tile (multiple of 32, <= 65536)
  int smem_acc;      // 1: shared accumulators, 0: run sums go to global memory
  size_t smem_bytes;
  int grid;
};

inline bool sorted_accumulate_plan(size_t rows, int d, int k, int num_sms, size_t max_smem, SortPlan* p) {
  if (d % 4 != 0 || d / 4 > kSortThreads || k > kSortMaxK || k < 1) return false;
  const size_t fixed = (size_t)2 * k * sizeof(int) + 64;            // histogram + running offsets
  const size_t acc_bytes = (size_t)3 * k * d * sizeof(int);
  size_t budget = max_smem - 2048;
  p->smem_acc = (acc_bytes + fixed + 4096 * sizeof(unsigned) <= budget / 2) ? 1 : 0;
  size_t avail = (p->smem_acc ? budget / 2 : budget) - fixed - (p->smem_acc ? acc_bytes : 0);
  size_t tile = avail / sizeof(unsigned);
  tile = std::min<size_t>(tile, p->smem_acc ? 8192 : 32768);
  tile = tile / 32 * 32;
  if (tile < 1024) return false;
  // whole waves of equal tiles: with the largest tile the last wave is ragged (C2: 4.1 waves cost
  // five) and a small shard leaves most SMs without a tile (250,000 rows of 784 columns: 56 tiles)
  const size_t slots = (size_t)num_sms * (p->smem_acc ? 2 : 1);
  const size_t waves = std::max<size_t>(1, (rows + slots * tile - 1) / (slots * tile));
  size_t even = (rows + waves * slots - 1) / (waves * slots);
  even = std::max<size_t>((even + 31) / 32 * 32, 256);
  tile = std::min(tile, even);
  p->tile_rows = (int)tile;
  p->smem_bytes = fixed + (p->smem_acc ? acc_bytes : 0) + tile * sizeof(unsigned);
  size_t tiles = (rows + tile - 1) / tile;
  p->grid = (int)std::min<size_t>(tiles, (size_t)num_sms * (p->smem_acc ? 2 : 1));
  return true;
}

// Out of line on purpose: label changes are rare, and inlined (if-converted) copies of
// this code would be issued for every row.
__device__ __noinline__ void flush_run(long long s, int* a0, size_t pstride, long long* g, int smem_acc) {
  if (s == 0) return;
  if (smem_acc) {
    const long long s0 = s >> 30;                       // arithmetic shift: floor
    const int rem = (int)(s - s0 * (1LL << 30));        // 0 .. 2^30-1
    atomicAdd(a0, (int)s0);
    atomicAdd(a0 + pstride, rem >> 15);
    atomicAdd(a0 + 2 * pstride, rem & 0x7fff);
  } else {
    atomicAdd(reinterpret_cast<unsigned long long*>(g), (unsigned long long)s);
  }
}

// GS = threads per row, VPT = float4 vectors per thread and row (GS * VPT >= d / 4, GS a power of two):
// with two vectors per thread the per-row bookkeeping (list entry, label compare, address) is spread
// over eight elements instead of four.  scale30 = 2^(30 - e).
template <int GS, int VPT>
__global__ void __launch_bounds__(kSortThreads, 2)
sorted_accumulate_kernel(const float* __restrict__ X, size_t n, int d, const int* __restrict__ labels, int k,
                         long long* __restrict__ gsums, unsigned long long* __restrict__ gcounts,
                         float scale30, int tile_rows, int smem_acc,
                         const unsigned long long* gate_changed, unsigned long long gate_limit) {
  if (delta_turn(gate_changed, gate_limit)) return;   // the incremental branch has this iteration
  extern __shared__ __align__(16) unsigned char smem_raw[];
  int* hist = reinterpret_cast<int*>(smem_raw);        // [k]   per-tile label counts
  int* offs = hist + k;                                // [k]   scatter cursors
  unsigned* sorted = reinterpret_cast<unsigned*>(offs + k);   // [tile_rows] (label << 16 | row) or two-word form
  int* acc = reinterpret_cast<int*>(sorted + tile_rows);      // [3][k][d] when smem_acc
  const size_t pstride = (size_t)k * d;
  const int tid = threadIdx.x;
  const int dv = d >> 2;
  constexpr int G = kSortThreads / GS;                 // groups walking the sorted list
  const int grp = tid / GS;
  const int l = tid % GS;
  bool active[VPT];
#pragma unroll
  for (int j = 0; j < VPT; ++j) active[j] = (l + j * GS) < dv;

  if (smem_acc)
    for (int i = tid; i < 3 * k * d; i += kSortThreads) acc[i] = 0;
  size_t since_drain = 0;
  const size_t n_tiles = (n + tile_rows - 1) / tile_rows;

  for (size_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
    const size_t r0 = tile * (size_t)tile_rows;
    const int nr = (int)min((size_t)tile_rows, n - r0);
    // ---- counting sort of the tile's rows by label ----
    for (int i = tid; i < k; i += kSortThreads) hist[i] = 0;
    __syncthreads();
    // (labels outside [0, k) cannot come from the E-step kernels; such rows are skipped)
    for (int i = tid; i < nr; i += kSortThreads) {
      const int lab = labels[r0 + i];
      if ((unsigned)lab < (unsigned)k) atomicAdd(&hist[lab], 1);
    }
    __syncthreads();
    // exclusive scan of hist into offs (k <= 4096: each thread owns a contiguous chunk)
    {
      const int per = (k + kSortThreads - 1) / kSortThreads;
      const int b = tid * per;
      int sum = 0;
      for (int j = 0; j < per; ++j)
        if (b + j < k) sum += hist[b + j];
      // block scan of the per-thread sums through shared memory (offs reused as scratch tail-safe: k >= 1)
      __shared__ int s_part[kSortThreads];
      s_part[tid] = sum;
      __syncthreads();
      for (int o = 1; o < kSortThreads; o <<= 1) {
        int v = (tid >= o) ? s_part[tid - o] : 0;
        __syncthreads();
        s_part[tid] += v;
        __syncthreads();
      }
      int run = s_part[tid] - sum;
      for (int j = 0; j < per; ++j)
        if (b + j < k) { offs[b + j] = run; run += hist[b + j]; }
    }
    __syncthreads();
    for (int i = tid; i < nr; i += kSortThreads) {
      const int lab = labels[r0 + i];
      if ((unsigned)lab >= (unsigned)k) continue;
      const int pos = atomicAdd(&offs[lab], 1);
      sorted[pos] = ((unsigned)lab << 16) | (unsigned)i;     // tile_rows <= 65536, k <= 4096
    }

    // per-cluster counts of this tile
    for (int i = tid; i < k; i += kSortThreads)
      if (hist[i]) atomicAdd(gcounts + i, (unsigned long long)hist[i]);
    __syncthreads();

    // ---- walk the sorted list: group `grp` owns positions [p0, p1) ----
    const int nsorted = offs[k - 1];  // rows with a valid label (all of them in normal operation)
    const int per_grp = (nsorted + G - 1) / G;
    const int p0 = grp * per_grp;
    const int p1 = min(nsorted, p0 + per_grp);
    long long s[VPT][4];
#pragma unroll
    for (int j = 0; j < VPT; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0;
    int cur = -1;
    const float* Xt = X + r0 * (size_t)d;
    constexpr int U = 4 / VPT;   // rows in flight: four 16-byte loads per thread either way
    auto flush_all = [&](int c) {
#pragma unroll
      for (int j = 0; j < VPT; ++j) {
        if (active[j]) {
          int* a0 = acc + (size_t)c * d + (l + j * GS) * 4;
          long long* g = gsums + (size_t)c * d + (l + j * GS) * 4;
#pragma unroll
          for (int e = 0; e < 4; ++e) flush_run(s[j][e], a0 + e, pstride, g + e, smem_acc);
        }
        s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0;
      }
    };
    for (int p = p0; p < p1; p += U) {
      unsigned ent[U];
      float4 x[U][VPT];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        ent[u] = (p + u < p1) ? sorted[p + u] : 0xffffffffu;
#pragma unroll
        for (int j = 0; j < VPT; ++j)
          if (ent[u] != 0xffffffffu && active[j])
            x[u][j] = *reinterpret_cast<const float4*>(Xt + (size_t)(ent[u] & 0xffffu) * d + (l + j * GS) * 4);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (ent[u] == 0xffffffffu) continue;
        const int lab = (int)(ent[u] >> 16);
        if (lab != cur) {
          if (cur >= 0) flush_all(cur);
          cur = lab;
        }
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
          if (active[j]) {
            s[j][0] += (long long)__float2int_rn(x[u][j].x * scale30);
            s[j][1] += (long long)__float2int_rn(x[u][j].y * scale30);
            s[j][2] += (long long)__float2int_rn(x[u][j].z * scale30);
            s[j][3] += (long long)__float2int_rn(x[u][j].w * scale30);
          }
        }
      }
    }
    if (cur >= 0) flush_all(cur);
    since_drain += nr;
    __syncthreads();
    if (smem_acc && (since_drain + tile_rows > (size_t)kSortDrainRows || tile + gridDim.x >= n_tiles)) {
      for (int i = tid; i < k * d; i += kSortThreads) {
        const long long v = (long long)acc[i] * (1LL << 30) + (long long)acc[pstride + i] * (1LL << 15) +
                            (long long)acc[2 * pstride + i];
        if (v) atomicAdd(reinterpret_cast<unsigned long long*>(gsums + i), (unsigned long long)v);
        acc[i] = 0;
        acc[pstride + i] = 0;
        acc[2 * pstride + i] = 0;
      }
      since_drain = 0;
      __syncthreads();
    }
  }
}

}  // namespace km
