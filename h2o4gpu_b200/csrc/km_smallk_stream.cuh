// E-step for few centroids and wide rows (k <= 16, float32, d % 4 == 0): the
// bandwidth-bound corner of the path (image-like data, d in the hundreds).
//
// Replaces calculate_distances + relabel (src/gpu/kmeans/kmeans_labels.cu:115-244,
// kmeans_labels.h:360-392) for that shape.  The register-tiled kernels waste most of
// their arithmetic on a 64-wide centroid tile here, and a warp that loads its rows straight
// from global memory cannot keep enough bytes in flight.  So X goes through shared memory
// in a four-stage cp.async pipeline of 64-row x 128-column pieces (memory latency is hidden
// by the pipeline, not by occupancy) and the whole centroid table stays in shared memory:
//   warp w owns rows 8w .. 8w+7 of the piece, lane l owns columns 4l .. 4l+3;
//   per piece a lane reads 8 row vectors and K centroid vectors (conflict-free 16-byte
//   loads) for 32 K multiply-adds, issued as 16 K packed ones (fma.rn.f32x2 over pairs of
//   centroids, whose table is interleaved for that): 8 x K accumulators per lane (sixteen
//   warps of four rows each measured 8 % slower, a fifth pipeline stage changed nothing);
//   after the last piece of a row tile the 8 K partial sums of the 32 lanes are combined by
//   recursive halving (every shuffle step halves the values a lane still holds: 8 K / 4
//   shuffles instead of 40 K), the four lanes that end up with a quarter of a row's scores
//   finish the argmin with two more steps.
// Scores are |c|^2 - 2 x.c in float, ties to the lowest index, like the other SIMT kernels.
#pragma once

#include "km_common.cuh"

namespace km {
namespace sks {

constexpr int kRows = 64;      // rows per tile
constexpr int kCols = 128;     // columns per piece
constexpr int kStages = 4;
constexpr int kThreads = 256;  // 8 warps x 8 rows
constexpr int kRpw = 8;        // rows per warp

inline int padded_cols(int d) { return (d + kCols - 1) / kCols * kCols; }
inline size_t smem_bytes(int K, int d) {
  return (size_t)K * padded_cols(d) * sizeof(float) + (size_t)kStages * kRows * kCols * sizeof(float) +
         (size_t)K * sizeof(float) + 16;
}

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, int src_bytes) {
  const unsigned int s = (unsigned int)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// K: centroid slots (multiple of 4, k <= K <= 16).  Persistent CTAs, tiles strided over the grid.
template <int K>
__global__ void __launch_bounds__(kThreads, 1)
assign_stream_kernel(const float* __restrict__ X, size_t n, int d, const float* __restrict__ C, int k,
                     const float* __restrict__ cnorm, int* __restrict__ labels, IterState* st) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int dp = (d + kCols - 1) / kCols * kCols;
  const int n_pieces = dp / kCols;
  // Centroids 2p, 2p+1 interleaved for the packed multiply-add: [K/2][2][dp/4][4], where the 16-byte
  // chunk (p, h, g) holds (c0, c1) of column 4g + 2h and (c0, c1) of column 4g + 2h + 1.  Consecutive lanes
  // (consecutive g) read consecutive chunks: no bank conflicts.  Zero beyond k rows / d columns.
  float* Cs = reinterpret_cast<float*>(smem_raw);
  float* stage = Cs + (size_t)K * dp;                              // [kStages][kRows][kCols]
  float* cns = stage + (size_t)kStages * kRows * kCols;            // [K]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  for (int i = tid; i < K * dp; i += kThreads) {
    const int c = i / dp, t = i - c * dp;
    const int g4 = t >> 2, j = t & 3;
    Cs[(((size_t)(c >> 1) * 2 + (j >> 1)) * (dp >> 2) + g4) * 4 + (j & 1) * 2 + (c & 1)] =
        (c < k && t < d) ? C[(size_t)c * d + t] : 0.f;
  }
  for (int i = tid; i < K; i += kThreads) cns[i] = (i < k) ? cnorm[i] : 0.f;

  const size_t n_tiles = (n + kRows - 1) / kRows;
  const size_t my_tiles = (blockIdx.x < n_tiles) ? (n_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  const size_t total = my_tiles * (size_t)n_pieces;               // (tile, piece) pairs of this CTA, in order

  // one pair = 64 rows x 128 columns = 2048 16-byte vectors: eight per thread, at fixed places of
  // the piece (vector v = tid + 256 j sits in row v / 32, columns 4 (v % 32) ..): only the tile
  // and the piece change from one pair to the next
  constexpr int kVec = (kRows * kCols / 4) / kThreads;
  const int my_c = (tid & 31) * 4;               // first column of this thread's vectors within a piece
  const int my_r = tid >> 5;                     // row of vector j: my_r + 8 j
  auto issue = [&](size_t pair) {
    if (pair < total) {
      const size_t tile = blockIdx.x + (pair / n_pieces) * gridDim.x;
      const int piece = (int)(pair % n_pieces);
      float* dst = stage + (size_t)(pair % kStages) * kRows * kCols + my_r * kCols + my_c;
      const int col = piece * kCols + my_c;
      const bool col_in = col < d;                                 // d % 4 == 0: a vector is inside or outside
      const size_t row0 = tile * kRows + my_r;
      const float* src = X + row0 * (size_t)d + col;
#pragma unroll
      for (int j = 0; j < kVec; ++j) {
        const bool in = col_in && (row0 + (size_t)j * (kThreads / 32) < n);
        cp_async16(dst + j * (kThreads / 32) * kCols, in ? (const void*)(src + (size_t)j * (kThreads / 32) * d) : (const void*)X,
                   in ? 16 : 0);
      }
    }
    cp_async_commit();
  };

#pragma unroll
  for (int s = 0; s < kStages - 1; ++s) issue(s);
  __syncthreads();   // centroid table in place

  // accumulators in pairs (centroids 2p, 2p+1): one packed fused multiply-add serves both
  float2 acc[kRpw][K / 2];
  unsigned int changed = 0;
  for (size_t pair = 0; pair < total; ++pair) {
    const int piece = (int)(pair % n_pieces);
    if (piece == 0) {
#pragma unroll
      for (int r = 0; r < kRpw; ++r)
#pragma unroll
        for (int c = 0; c < K / 2; ++c) acc[r][c] = make_float2(0.f, 0.f);
    }
    cp_async_wait<kStages - 2>();   // this pair's copies (of this thread) have landed
    __syncthreads();                // ... and everybody else's; the stage refilled below was read in the last round
    issue(pair + kStages - 1);
    const float* sx = stage + (size_t)(pair % kStages) * kRows * kCols + (size_t)(warp * kRpw) * kCols + lane * 4;
    const float* sc = Cs + (size_t)(piece * (kCols / 4) + lane) * 4;   // chunk g = piece * 32 + lane of plane (p, 0)
    float4 xv[kRpw];
#pragma unroll
    for (int r = 0; r < kRpw; ++r) xv[r] = *reinterpret_cast<const float4*>(sx + r * kCols);
#pragma unroll
    for (int c = 0; c < K / 2; ++c) {
      // columns 4l, 4l+1 and 4l+2, 4l+3 of the centroid pair: (c0, c1) per column
      const float4 ca = *reinterpret_cast<const float4*>(sc + (size_t)(2 * c) * dp);
      const float4 cb = *reinterpret_cast<const float4*>(sc + (size_t)(2 * c + 1) * dp);
#pragma unroll
      for (int r = 0; r < kRpw; ++r) {
        float2 a = acc[r][c];
        a = __ffma2_rn(make_float2(xv[r].x, xv[r].x), make_float2(ca.x, ca.y), a);
        a = __ffma2_rn(make_float2(xv[r].y, xv[r].y), make_float2(ca.z, ca.w), a);
        a = __ffma2_rn(make_float2(xv[r].z, xv[r].z), make_float2(cb.x, cb.y), a);
        a = __ffma2_rn(make_float2(xv[r].w, xv[r].w), make_float2(cb.z, cb.w), a);
        acc[r][c] = a;
      }
    }
    if (piece == n_pieces - 1) {
      // ---- combine the 32 lanes' partial sums: recursive halving over v[r * K + c] ----
      float v[kRpw * K];
#pragma unroll
      for (int r = 0; r < kRpw; ++r)
#pragma unroll
        for (int c = 0; c < K / 2; ++c) { v[r * K + 2 * c] = acc[r][c].x; v[r * K + 2 * c + 1] = acc[r][c].y; }
      int cur = kRpw * K;
#pragma unroll
      for (int s = 16; s >= 1; s >>= 1) {
        const int half = cur >> 1;
        const bool upper = (lane & s) != 0;
#pragma unroll
        for (int i = 0; i < kRpw * K / 2; ++i) {
          if (i < half) {
            const float send = upper ? v[i] : v[i + half];
            const float keep = upper ? v[i + half] : v[i];
            v[i] = keep + __shfl_xor_sync(0xffffffffu, send, s);
          }
        }
        cur = half;
      }
      // five halvings of 8 K values leave K / 4 per lane.  Index of v[0]: the halves taken
      // (lane bits 4, 3, 2 pick the row, bits 1, 0 the quarter of it)
      constexpr int Q = K / 4;
      const int r = ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1);
      const int c0 = ((lane >> 1) & 1) * (K / 2) + (lane & 1) * (K / 4);
      float best = __int_as_float(0x7f800000);
      int bi = 0x7fffffff;
#pragma unroll
      for (int j = 0; j < Q; ++j) {
        const int c = c0 + j;
        const float sscore = cns[c] - 2.f * v[j];
        if (c < k && sscore < best) { best = sscore; bi = c; }
      }
      // the quarters of a row sit in lanes that differ in bits 1 and 0
#pragma unroll
      for (int o = 2; o >= 1; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ob < best || (ob == best && oi < bi)) { best = ob; bi = oi; }
      }
      const size_t tile = blockIdx.x + (pair / n_pieces) * gridDim.x;
      const size_t row = tile * kRows + warp * kRpw + r;
      if ((lane & 3) == 0 && row < n) {
        if (st) changed += (labels[row] != bi);
        labels[row] = bi;
      }
    }
  }
  cp_async_wait<0>();
  if (st) {
    changed = __reduce_add_sync(0xffffffffu, changed);
    if (lane == 0 && changed) atomicAdd(&st->changed, (unsigned long long)changed);
  }
}

}  // namespace sks
}  // namespace km
