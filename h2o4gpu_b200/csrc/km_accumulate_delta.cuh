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
constexpr int kDeltaThreads = 512;    // two CTAs per SM: room for the registers of a prefetched step
constexpr int kDeltaChunk = 32768;   // rows between two drains: the int32 accumulators hold 2^15 rows of 2^15-sized pieces

template <typename T>
inline size_t delta_smem_bytes(int k, int d) {
  return (size_t)Fixed<T>::NP * k * d * sizeof(int) + (size_t)2 * k * sizeof(int) + 16;
}

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
  __shared__ int s_touched;                         // rows netted since the last drain
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  constexpr int NWARP = kDeltaThreads / 32;
  static_assert(kDeltaChunk % (NWARP * 256) == 0, "whole 256-row steps per warp and chunk");
  const int dv = d / V;
  const size_t pstride = (size_t)k * d;
  int lpr = 1;
  while (lpr < dv && lpr < 32) lpr <<= 1;
  const int groups = 32 / lpr;
  const int g = lane / lpr;
  const int l = lane % lpr;

  size_t per = (n + gridDim.x - 1) / gridDim.x;
  per = (per + 31) / 32 * 32;
  const size_t r_begin = min(n, (size_t)blockIdx.x * per);
  const size_t r_end = min(n, r_begin + per);

  for (int i = tid; i < NP * k * d; i += kDeltaThreads) acc[i] = 0;
  for (int i = tid; i < 2 * k; i += kDeltaThreads) cnt[i] = 0;
  if (tid == 0) s_touched = 0;
  __syncthreads();

  for (size_t c0 = r_begin; c0 < r_end; c0 += kDeltaChunk) {
    const size_t c1 = min(r_end, c0 + (size_t)kDeltaChunk);
    // a warp takes 256 rows per step, eight per lane, all label loads in flight together
    // (c0 is a multiple of 32 rows, so the 16-byte loads are aligned); between two drains the
    // warps run free of one another
    auto load_step = [&](size_t wb, int (&nw)[8], int (&od)[8]) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const size_t r4 = wb + h * 128 + lane * 4;
        if (r4 + 3 < c1) {
          const int4 a = *reinterpret_cast<const int4*>(labels + r4);
          const int4 b = *reinterpret_cast<const int4*>(prev + r4);
          nw[4 * h + 0] = a.x; nw[4 * h + 1] = a.y; nw[4 * h + 2] = a.z; nw[4 * h + 3] = a.w;
          od[4 * h + 0] = b.x; od[4 * h + 1] = b.y; od[4 * h + 2] = b.z; od[4 * h + 3] = b.w;
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const bool in = r4 + j < c1;
            nw[4 * h + j] = in ? labels[r4 + j] : -1;
            od[4 * h + j] = in ? prev[r4 + j] : -1;
          }
        }
      }
    };
    int nwn[8], odn[8];
    {
      const size_t wb0 = c0 + (size_t)warp * 256;
      if (wb0 < c1) load_step(wb0, nwn, odn);
    }
    for (size_t wb = c0 + (size_t)warp * 256; wb < c1; wb += (size_t)NWARP * 256) {
    int nw[8], od[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) { nw[j] = nwn[j]; od[j] = odn[j]; }
    {
      // the next step's labels are requested before this step's rows are worked on
      const size_t wbn = wb + (size_t)NWARP * 256;
      if (wbn < c1) load_step(wbn, nwn, odn);
    }
    // which of the eight label pairs of every lane moved: lane j keeps the ballot of pair j, so
    // that the loop over the pairs below need not be unrolled (its body is long, and eight copies
    // of it made the kernel wait for instruction fetches more than for memory)
    unsigned int my_ballot = 0;
    bool any = false;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const unsigned int m = __ballot_sync(0xffffffffu, nw[j] != od[j]);
      if (lane == j) my_ballot = m;
      any |= (m != 0);
    }
    if (any) {
#pragma unroll 1
      for (int j = 0; j < 8; ++j) {
        unsigned int mask = __shfl_sync(0xffffffffu, my_ballot, j);
        if (mask == 0) continue;
        const size_t jb = wb + (j >> 2) * 128 + (j & 3);   // row of lane 0 for this pair; lane s holds jb + 4 s
        if (lane == 0) atomicAdd(&s_touched, __popc(mask));
        while (mask) {
          const unsigned int src = __fns(mask, 0, g + 1);   // lane of this group's row
          const bool have = (src != 0xffffffffu);
          if (have) {
            // the two labels are read again (they are in L1) rather than indexed out of registers
            const size_t row = jb + (size_t)src * 4;
            const int to = labels[row], from = prev[row];
            const bool to_ok = (unsigned)to < (unsigned)k, from_ok = (unsigned)from < (unsigned)k;
            const T* xr = X + row * (size_t)d;
            const T w = W ? W[row] : (T)1;
            for (int idx = l; idx < dv; idx += lpr) {
              T x[V], y[V];
              VecLoad<T, V>::ld(xr + (size_t)idx * V, x);
              if (W) {
#pragma unroll
                for (int e = 0; e < V; ++e) x[e] *= w;
              }
#pragma unroll
              for (int e = 0; e < V; ++e) y[e] = -x[e];
              if (to_ok) add_vec_fixed<T, V, NP>(acc + (size_t)to * d, pstride, dv, idx, g & (V - 1), x, scale);
              if (from_ok) add_vec_fixed<T, V, NP>(acc + (size_t)from * d, pstride, dv, idx, g & (V - 1), y, scale);
            }
            if (l == 0) {
              int pw[2] = {0, 1};
              if (W) split_pieces<2>(w, wscale, pw);
              if (to_ok) { atomicAdd(&cnt[to], pw[1]); if (pw[0]) atomicAdd(&cnt[k + to], pw[0]); }
              if (from_ok) { atomicAdd(&cnt[from], -pw[1]); if (pw[0]) atomicAdd(&cnt[k + from], -pw[0]); }
            }
          }
          for (int i = 0; i < groups && mask; ++i) mask &= mask - 1;
        }
      }
      // the snapshot follows once every group has read the old labels
      __syncwarp();
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (nw[j] != od[j]) prev[wb + (j >> 2) * 128 + lane * 4 + (j & 3)] = nw[j];
    }
    }
    __syncthreads();
    // every piece is at most 2^15 in magnitude and a chunk has 2^15 rows: drain after each
    {
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
