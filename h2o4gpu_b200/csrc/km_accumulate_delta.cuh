// Incremental centroid sums.
//
// The fixed-point sums of km_common.cuh are exact integers, so the sums of the
// new labelling can be had from those of the previous one without rounding:
// for every row whose label moved from a to b, subtract the row's integers from
// cluster a and add them to cluster b.  The result is, bit for bit, what a full
// pass over the shard produces, whatever the order of the updates.  Once Lloyd's
// iteration has settled only a small fraction of the rows move per step, and the
// M-step's traffic drops from the whole shard (4d + 4 bytes per row) to the two
// label arrays (8 bytes per row) plus the rows that moved.
//
// The choice between the full pass and the incremental one is made on the
// device, from the label-change counter the E-step kernels have just written:
// every kernel of either branch is launched in every iteration and returns at
// once when it is not its turn, so the host never waits for the counter.
//
// `pure` holds the sums and counts that follow from the labels alone; the
// iteration copies (or all-reduces) it into the working array before empty
// clusters are repaired there, so repairs never leak into the next step.
#pragma once

#include "km_common.cuh"
#include "km_tiles.cuh"

namespace km {

// Full branch, first kernel: clears the pure sums and snapshots the labels.
__global__ void __launch_bounds__(256)
full_prologue_kernel(long long* __restrict__ pure, size_t count, const int* __restrict__ labels,
                     int* __restrict__ prev, size_t n, const unsigned long long* changed, unsigned long long limit) {
  if (delta_turn(changed, limit)) return;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const size_t t = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (size_t i = t; i < count; i += stride) pure[i] = 0;
  const size_t n4 = n / 4;
  const int4* l4 = reinterpret_cast<const int4*>(labels);
  int4* p4 = reinterpret_cast<int4*>(prev);
  for (size_t i = t; i < n4; i += stride) p4[i] = l4[i];
  for (size_t i = n4 * 4 + t; i < n; i += stride) prev[i] = labels[i];
}

// Incremental branch: one warp per block of 32 rows; rows whose label differs from
// the snapshot are moved between clusters with 64-bit integer reductions.
template <typename T, int V>
__global__ void __launch_bounds__(256)
delta_accumulate_kernel(const T* __restrict__ X, size_t n, int d, const int* __restrict__ labels,
                        int* __restrict__ prev, int k, long long* __restrict__ psums,
                        unsigned long long* __restrict__ pcounts, T scale,
                        const unsigned long long* changed, unsigned long long limit,
                        const T* __restrict__ W, T wscale) {
  constexpr int NP = Fixed<T>::NP;
  if (!delta_turn(changed, limit)) return;
  const int lane = threadIdx.x & 31;
  const size_t warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const size_t n_warps = ((size_t)gridDim.x * blockDim.x) >> 5;
  const int dv = d / V;
  const size_t plane = (size_t)k * d;
  for (size_t b = warp * 32; b < n; b += n_warps * 32) {
    const size_t r = b + lane;
    int nw = -1, od = -1;
    if (r < n) { nw = labels[r]; od = prev[r]; }
    const bool moved = nw != od;
    unsigned int mask = __ballot_sync(0xffffffffu, moved);
    if (moved) prev[r] = nw;
    while (mask) {
      const int src = __ffs(mask) - 1;
      mask &= mask - 1;
      const int to = __shfl_sync(0xffffffffu, nw, src);
      const int from = __shfl_sync(0xffffffffu, od, src);
      const bool to_ok = (unsigned)to < (unsigned)k, from_ok = (unsigned)from < (unsigned)k;
      const T* xr = X + (b + src) * (size_t)d;
      // sample weights: the row moves w * x and its fixed-point weight (see accumulate_kernel)
      const T w = W ? W[b + src] : (T)1;
      unsigned long long units = 1;
      if (W) {
        int pw[2];
        split_pieces<2>(w, wscale, pw);
        units = (unsigned long long)((long long)pw[0] * (1LL << kPieceBits) + (long long)pw[1]);
      }
      for (int idx = lane; idx < dv; idx += 32) {
        T x[V];
        VecLoad<T, V>::ld(xr + (size_t)idx * V, x);
#pragma unroll
        for (int e = 0; e < V; ++e) {
          int p[NP];
          split_pieces<NP>(W ? x[e] * w : x[e], scale, p);
          const int col = idx * V + e;
#pragma unroll
          for (int q = 0; q < NP / 2; ++q) {
            const long long v = (long long)p[2 * q] * (1LL << kPieceBits) + (long long)p[2 * q + 1];
            if (v == 0) continue;
            if (to_ok)
              atomicAdd(reinterpret_cast<unsigned long long*>(psums + q * plane + (size_t)to * d + col),
                        (unsigned long long)v);
            if (from_ok)
              atomicAdd(reinterpret_cast<unsigned long long*>(psums + q * plane + (size_t)from * d + col),
                        (unsigned long long)(-v));
          }
        }
      }
      if (lane == 0) {
        if (to_ok) atomicAdd(pcounts + to, units);
        if (from_ok) atomicAdd(pcounts + from, 0ULL - units);   // minus, modulo 2^64
      }
    }
  }
}

// Incremental branch for centroid tables whose fixed-point pieces fit shared memory.
// Moves between a few clusters hit the same few lines of the global sums, and 64-bit
// reductions on one line serialise in the L2; here a CTA nets the moves of its rows in
// int32 shared accumulators first (same layout and arithmetic as accumulate_kernel) and
// sends each non-zero total to the global sums once.  Subtracting a row is adding its
// negation: rint is odd, so the pieces of -x are minus the pieces of x.
// The netting kernels drain into a padded copy of the sums, one int64 per 128-byte line:
// several hundred CTAs send their totals to the same k * d addresses, and 64-bit reductions
// on one L2 line are served one after the other (about 13 ns each measured), so with the
// dense layout (16 sums per line) the drain alone took longer than the netting.
// fold_flush_kernel adds the padded array into the dense sums and clears it.
constexpr int kFlushPad = 16;
constexpr int kDeltaThreads = 512;    // two CTAs per SM
constexpr int kDeltaChunk = 32768;   // rows between two drains: the int32 accumulators hold 2^15 rows of 2^15-sized pieces
constexpr int kDeltaStepRows = (kDeltaThreads / 32) * 128;   // rows a CTA scans in one step
constexpr int kDeltaListCap = 2 * kDeltaStepRows;            // entries of the moved-row list

template <typename T>
inline size_t delta_smem_bytes(int k, int d) {
  const size_t acc = (size_t)Fixed<T>::NP * k * d * sizeof(int) + (size_t)2 * k * sizeof(int);
  return (acc + 15) / 16 * 16 + (size_t)kDeltaListCap * sizeof(uint2);
}

// A CTA scans its rows in steps of kDeltaStepRows.  Scan: every warp compares the two label arrays
// for 128 rows (one 16-byte load per lane and array, the next step's loads already in flight) and
// appends the rows that moved - offset, new and old label - to a list in shared memory.  Apply, once
// the list could not take another step's rows or the accumulators are due to be drained: the list is
// cut into items of one row segment each (the lpr lanes of a group times V columns) that the warps
// take in turn, two items per group in flight; a wide row is thus spread over several warps, and the
// moved rows over all of them, wherever they sat.  (Before, a warp worked through the moved rows of
// its own 256 rows one after the other: with 784 columns and 8 % of the labels moving that was
// 0.15 ms for 250,000 rows.  Applying after every step cost a memory latency per step: with 0.1 % of
// 1e7 x 64 rows moving the kernel took 43 us, the label scan alone needs 15.)
template <typename T, int V>
__global__ void __launch_bounds__(kDeltaThreads, 2)
delta_accumulate_smem_kernel(const T* __restrict__ X, size_t n, int d, const int* __restrict__ labels,
                             int* __restrict__ prev, int k, long long* __restrict__ psums,
                             unsigned long long* __restrict__ pcounts, T scale,
                             const unsigned long long* changed, unsigned long long limit,
                             const T* __restrict__ W, T wscale) {
  constexpr int NP = Fixed<T>::NP;
  if (!delta_turn(changed, limit)) return;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  int* acc = reinterpret_cast<int*>(smem_raw);      // [NP][k][d]
  int* cnt = acc + (size_t)NP * k * d;              // [2][k]: units, then units * 2^15 (sample weights)
  uint2* list = reinterpret_cast<uint2*>(smem_raw + (((size_t)NP * k * d + 2 * k) * sizeof(int) + 15) / 16 * 16);
  __shared__ int s_touched;                         // rows netted since the last drain
  __shared__ int s_list_n;                          // entries of the list
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  constexpr int NWARP = kDeltaThreads / 32;
  static_assert(kDeltaChunk % kDeltaStepRows == 0, "whole steps per chunk");
  const int dv = d / V;
  const size_t pstride = (size_t)k * d;
  int lpr = 1;
  while (lpr < dv && lpr < 32) lpr <<= 1;
  const int groups = 32 / lpr;
  const int g = lane / lpr;
  const int l = lane % lpr;
  const int nseg = (dv + lpr - 1) / lpr;

  size_t per = (n + gridDim.x - 1) / gridDim.x;
  per = (per + 31) / 32 * 32;
  const size_t r_begin = min(n, (size_t)blockIdx.x * per);
  const size_t r_end = min(n, r_begin + per);

  for (int i = tid; i < NP * k * d; i += kDeltaThreads) acc[i] = 0;
  for (int i = tid; i < 2 * k; i += kDeltaThreads) cnt[i] = 0;
  if (tid == 0) { s_touched = 0; s_list_n = 0; }
  __syncthreads();

  // labels of this lane's four rows of a step (r_begin is a multiple of 32 rows: aligned 16-byte loads)
  auto load_step = [&](size_t sb, int (&nw)[4], int (&od)[4]) {
    const size_t r4 = sb + (size_t)warp * 128 + lane * 4;
    if (r4 + 3 < r_end) {
      const int4 a = *reinterpret_cast<const int4*>(labels + r4);
      const int4 b = *reinterpret_cast<const int4*>(prev + r4);
      nw[0] = a.x; nw[1] = a.y; nw[2] = a.z; nw[3] = a.w;
      od[0] = b.x; od[1] = b.y; od[2] = b.z; od[3] = b.w;
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const bool in = r4 + j < r_end;
        nw[j] = in ? labels[r4 + j] : -1;
        od[j] = in ? prev[r4 + j] : -1;
      }
    }
  };
  int nwn[4], odn[4];
  if (r_begin < r_end) load_step(r_begin, nwn, odn);
  int since_drain = 0;

  for (size_t sb = r_begin; sb < r_end; sb += kDeltaStepRows) {
    // ---- scan ----
    int nw[4], od[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) { nw[j] = nwn[j]; od[j] = odn[j]; }
    if (sb + kDeltaStepRows < r_end) load_step(sb + kDeltaStepRows, nwn, odn);
    const unsigned int off0 = (unsigned int)(sb - r_begin) + (unsigned int)(warp * 128 + lane * 4);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const bool moved = nw[j] != od[j];
      const unsigned int mask = __ballot_sync(0xffffffffu, moved);
      if (mask == 0) continue;
      int base = 0;
      if (lane == 0) base = atomicAdd(&s_list_n, __popc(mask));
      base = __shfl_sync(0xffffffffu, base, 0);
      if (moved) {
        const unsigned int to = (unsigned)nw[j] < (unsigned)k ? (unsigned)nw[j] : 0xffffu;
        const unsigned int from = (unsigned)od[j] < (unsigned)k ? (unsigned)od[j] : 0xffffu;
        list[base + __popc(mask & ((1u << lane) - 1u))] = make_uint2(off0 + j, (to << 16) | from);
        prev[r_begin + off0 + j] = nw[j];
      }
    }
    __syncthreads();
    const int n_list = s_list_n;
    since_drain += kDeltaStepRows;
    // every piece is at most 2^15 in magnitude: drain after 2^15 rows at the latest, and at the end
    const bool drain_due = since_drain >= kDeltaChunk || sb + kDeltaStepRows >= r_end;
    const bool apply = n_list > 0 && (drain_due || n_list > kDeltaListCap - kDeltaStepRows);
    __syncthreads();   // everybody has read the count before the next scan can add to it
    if (apply) {
      const int items = n_list * nseg;
      for (int it0 = warp * groups; it0 < items; it0 += 2 * NWARP * groups) {
        T x[2][V];
        uint2 en[2];
        int idx[2];
        bool have[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int it = it0 + u * NWARP * groups + g;
          have[u] = it < items;
          idx[u] = 0;
          en[u] = make_uint2(0u, 0u);
          if (have[u]) {
            const int e = (nseg == 1) ? it : it / nseg;
            idx[u] = (it - e * nseg) * lpr + l;
            en[u] = list[e];
            have[u] = idx[u] < dv;
          }
          if (have[u]) VecLoad<T, V>::ld(X + (r_begin + en[u].x) * (size_t)d + (size_t)idx[u] * V, x[u]);
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          if (!have[u]) continue;
          const unsigned int to = en[u].y >> 16, from = en[u].y & 0xffffu;
          const bool to_ok = to != 0xffffu, from_ok = from != 0xffffu;
          const T w = W ? W[r_begin + en[u].x] : (T)1;
          T y[V];
          if (W) {
#pragma unroll
            for (int e = 0; e < V; ++e) x[u][e] *= w;
          }
#pragma unroll
          for (int e = 0; e < V; ++e) y[e] = -x[u][e];
          if (to_ok) add_vec_fixed<T, V, NP>(acc + (size_t)to * d, pstride, dv, idx[u], g & (V - 1), x[u], scale);
          if (from_ok) add_vec_fixed<T, V, NP>(acc + (size_t)from * d, pstride, dv, idx[u], g & (V - 1), y, scale);
          if (idx[u] == 0) {
            int pw[2] = {0, 1};
            if (W) split_pieces<2>(w, wscale, pw);
            if (to_ok) { atomicAdd(&cnt[to], pw[1]); if (pw[0]) atomicAdd(&cnt[k + to], pw[0]); }
            if (from_ok) { atomicAdd(&cnt[from], -pw[1]); if (pw[0]) atomicAdd(&cnt[k + from], -pw[0]); }
          }
        }
      }
      __syncthreads();
      if (tid == 0) { s_touched += n_list; s_list_n = 0; }
      __syncthreads();
    }
    if (drain_due) {
      since_drain = 0;
      if (s_touched > 0) {
        for (int i = tid; i < k * d; i += kDeltaThreads) {
          const int c = i / d;
          const int col = pos_to_col(i - c * d, dv, V);
#pragma unroll
          for (int q = 0; q < NP / 2; ++q) {
            const long long v = (long long)acc[(size_t)(2 * q) * pstride + i] * (1LL << kPieceBits) +
                                (long long)acc[(size_t)(2 * q + 1) * pstride + i];
            if (v) atomicAdd(reinterpret_cast<unsigned long long*>(psums + ((size_t)q * k * d + (size_t)c * d + col) * kFlushPad),
                             (unsigned long long)v);
            acc[(size_t)(2 * q) * pstride + i] = 0;
            acc[(size_t)(2 * q + 1) * pstride + i] = 0;
          }
        }
        for (int i = tid; i < k; i += kDeltaThreads) {
          const long long v = (long long)cnt[k + i] * (1LL << kPieceBits) + (long long)cnt[i];
          if (v) atomicAdd(pcounts + (size_t)i * kFlushPad, (unsigned long long)v);
          cnt[i] = 0;
          cnt[k + i] = 0;
        }
      }
      __syncthreads();
      if (tid == 0) s_touched = 0;
      __syncthreads();
    }
  }
}

// The same netting, fed by the moved-rows bit map the tensor-core E-step writes (one bit per
// row, one word per 32 rows): the scan reads rows / 8 bytes instead of 8 bytes per row, and
// the two labels are fetched only for the 32-row blocks that have a bit set.
template <typename T, int V>
__global__ void __launch_bounds__(kDeltaThreads, 2)
delta_accumulate_bitmap_kernel(const T* __restrict__ X, size_t n, int d, const int* __restrict__ labels,
                               int* __restrict__ prev, const unsigned int* __restrict__ moved_bits, int k,
                               long long* __restrict__ psums, unsigned long long* __restrict__ pcounts, T scale,
                               const unsigned long long* changed, unsigned long long limit) {
  constexpr int NP = Fixed<T>::NP;
  if (!delta_turn(changed, limit)) return;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  int* acc = reinterpret_cast<int*>(smem_raw);      // [NP][k][d]
  int* cnt = acc + (size_t)NP * k * d;              // [k]
  __shared__ int s_touched;
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  constexpr int NWARP = kDeltaThreads / 32;
  const int dv = d / V;
  const size_t pstride = (size_t)k * d;
  int lpr = 1;
  while (lpr < dv && lpr < 32) lpr <<= 1;
  const int groups = 32 / lpr;
  const int g = lane / lpr;
  const int l = lane % lpr;

  // partitions in whole chunks of 32768 rows (1024 words), so a word never straddles two CTAs
  const size_t n_chunks = (n + kDeltaChunk - 1) / kDeltaChunk;
  const size_t n_words = (n + 31) / 32;

  for (int i = tid; i < NP * k * d; i += kDeltaThreads) acc[i] = 0;
  for (int i = tid; i < k; i += kDeltaThreads) cnt[i] = 0;
  if (tid == 0) s_touched = 0;
  __syncthreads();

  for (size_t chunk = blockIdx.x; chunk < n_chunks; chunk += gridDim.x) {
    const size_t w0 = chunk * (kDeltaChunk / 32);
    const size_t w1 = min(n_words, w0 + kDeltaChunk / 32);
    for (size_t wb = w0 + (size_t)warp * 32; wb < w1; wb += (size_t)NWARP * 32) {
      const size_t wi = wb + lane;
      const unsigned int my_word = (wi < w1) ? moved_bits[wi] : 0u;
      unsigned int nonzero = __ballot_sync(0xffffffffu, my_word != 0u);
      while (nonzero) {
        const int wsrc = __ffs(nonzero) - 1;
        nonzero &= nonzero - 1;
        unsigned int mask = __shfl_sync(0xffffffffu, my_word, wsrc);
        const size_t b = (wb + wsrc) * 32;            // first row of this 32-row block
        const size_t r = b + lane;
        int nw = -1, od = -1;
        if (r < n && ((mask >> lane) & 1u)) { nw = labels[r]; od = prev[r]; prev[r] = nw; }
        if (lane == 0) atomicAdd(&s_touched, __popc(mask));
        while (mask) {
          const unsigned int src = __fns(mask, 0, g + 1);   // lane of this group's row
          const bool have = (src != 0xffffffffu);
          const int to = __shfl_sync(0xffffffffu, nw, have ? src : 0);
          const int from = __shfl_sync(0xffffffffu, od, have ? src : 0);
          if (have && to != from) {
            const bool to_ok = (unsigned)to < (unsigned)k, from_ok = (unsigned)from < (unsigned)k;
            const T* xr = X + (b + src) * (size_t)d;
            for (int idx = l; idx < dv; idx += lpr) {
              T x[V], y[V];
              VecLoad<T, V>::ld(xr + (size_t)idx * V, x);
#pragma unroll
              for (int e = 0; e < V; ++e) y[e] = -x[e];
              if (to_ok) add_vec_fixed<T, V, NP>(acc + (size_t)to * d, pstride, dv, idx, g & (V - 1), x, scale);
              if (from_ok) add_vec_fixed<T, V, NP>(acc + (size_t)from * d, pstride, dv, idx, g & (V - 1), y, scale);
            }
            if (l == 0) {
              if (to_ok) atomicAdd(&cnt[to], 1);
              if (from_ok) atomicAdd(&cnt[from], -1);
            }
          }
          for (int i = 0; i < groups && mask; ++i) mask &= mask - 1;
        }
      }
    }
    __syncthreads();
    // a chunk has 2^15 rows and every piece is at most 2^15 in magnitude: drain after each
    if (s_touched > 0) {
      for (int i = tid; i < k * d; i += kDeltaThreads) {
        const int c = i / d;
        const int col = pos_to_col(i - c * d, dv, V);
#pragma unroll
        for (int q = 0; q < NP / 2; ++q) {
          const long long v = (long long)acc[(size_t)(2 * q) * pstride + i] * (1LL << kPieceBits) +
                              (long long)acc[(size_t)(2 * q + 1) * pstride + i];
          if (v) atomicAdd(reinterpret_cast<unsigned long long*>(psums + ((size_t)q * k * d + (size_t)c * d + col) * kFlushPad),
                           (unsigned long long)v);
          acc[(size_t)(2 * q) * pstride + i] = 0;
          acc[(size_t)(2 * q + 1) * pstride + i] = 0;
        }
      }
      for (int i = tid; i < k; i += kDeltaThreads) {
        if (cnt[i]) atomicAdd(pcounts + (size_t)i * kFlushPad, (unsigned long long)(long long)cnt[i]);
        cnt[i] = 0;
      }
    }
    __syncthreads();
    if (tid == 0) s_touched = 0;
    __syncthreads();
  }
}

// pure[i] += flush[i * kFlushPad] (then cleared); work[i] = pure[i] when work is given.
__global__ void __launch_bounds__(256)
fold_flush_kernel(long long* __restrict__ flush, long long* __restrict__ pure, long long* __restrict__ work,
                  size_t count) {
  for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < count; i += (size_t)gridDim.x * 256) {
    long long v = pure[i];
    if (flush != nullptr) {
      const long long f = flush[i * kFlushPad];
      if (f != 0) {
        v += f;
        flush[i * kFlushPad] = 0;
        pure[i] = v;
      }
    }
    if (work != nullptr) work[i] = v;
  }
}

}  // namespace km
