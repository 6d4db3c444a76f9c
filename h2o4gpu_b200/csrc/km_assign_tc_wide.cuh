// Tensor-core distance + argmin (and transform) for few centroids and wide rows:
// float32, k <= 16, d % 4 == 0 (image-like data, d in the hundreds): the
// bandwidth-bound corner of the path.  Replaces calculate_distances + relabel
// (src/gpu/kmeans/kmeans_labels.cu:115-244, kmeans_labels.h:360-392) and the
// distance block of kmeans_transform (src/gpu/kmeans/kmeans_h2o4gpu.cu:891-975)
// for that shape.
//
// 2 k d flops per row are nothing for the tensor pipe, but on the FMA pipe they
// take longer than the row takes to arrive from HBM; with the products on the
// tensor cores the SM only converts and streams.  Same split-fp16 arithmetic as
// km_assign_tc.cuh (x sx = xh + xl, -2 c sb = bh + bl, acc = xh.bh + xl.bh + xh.bl,
// fp32 accumulation in TMEM).  A row tile of 128 rows is walked in chunks of 64
// columns: the chunk arrives by TMA (two 128B-swizzled panels of 32 columns; columns
// beyond d are zero-filled by the copy engine), converter warps split it into one of
// four TMEM A buffers, the issuer adds 12 MMAs (M = 128, N = 16, K = 16) per chunk to
// the tile's accumulator, and after the last chunk the epilogue reads 16 columns per
// row: label (or all k squared distances for transform).  The split centroid table
// stays in shared memory for the life of the CTA.
//
// Warps: 0 TMA producer, 1 MMA issuer, 2-3 spare, 4-11 converters (two groups of
// four, alternating chunks), 12-15 epilogue.  Every mbarrier wait is bounded.
#pragma once

#include "km_assign_tc.cuh"

namespace km {
namespace tcw {

using namespace km::tc;

constexpr int kWThreads = 512;
constexpr int kNPad = 16;        // centroid slots = MMA N
constexpr int kChunk = 64;       // fp32 columns per chunk
constexpr int kNA = 4;           // A buffers in TMEM
constexpr int kMaxStages = 5;
constexpr uint32_t kStageBytes = kBM * kChunk * 4;          // 32 KB
constexpr uint32_t kPanelBytes = kNPad * 128;               // one fp16 panel of the centroid table: 16 rows x 64 halves

enum WBar { W_FULL = 0, W_EMPTY = kMaxStages, W_ARDY = 2 * kMaxStages, W_AEMP = 2 * kMaxStages + kNA,
            W_ACF = 2 * kMaxStages + 2 * kNA, W_ACE = 2 * kMaxStages + 2 * kNA + 2, W_BFUL = 2 * kMaxStages + 2 * kNA + 4,
            W_DRAIN = 2 * kMaxStages + 2 * kNA + 5, W_NBARS = 2 * kMaxStages + 2 * kNA + 6 };

inline size_t wide_smem_bytes(int n_chunks, int stages) {
  return 1024 + (size_t)2 * n_chunks * kPanelBytes + (size_t)stages * kStageBytes + kNPad * 4 + W_NBARS * 8 + 64;
}

// n_chunks = ceil(d / 64); stages: X ring depth, even (4 or 2: a stage always serves the same converter group)
// out != nullptr: transform - out[j * ld_out + (row - row0)] = |xn + score_j|, labels untouched
__global__ void __launch_bounds__(kWThreads, 1)
assign_tc_wide_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmBhi,
                      const __grid_constant__ CUtensorMap tmBlo, const float* __restrict__ cn_pad,
                      const float* __restrict__ xnorm, int* __restrict__ labels, size_t n, int tile0, int n_tiles,
                      int n_chunks, int stages, int k, IterState* st, int count_changes,
                      unsigned int* __restrict__ amb_rows, float tol_rel, float tol_floor, float sx, float sxsb,
                      unsigned int wait_iters, float* __restrict__ out, size_t ld_out) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_u32 = smem_u32(smem_raw);
  const uint32_t base = (raw_u32 + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - raw_u32);

  const uint32_t off_blo = (uint32_t)n_chunks * kPanelBytes;
  const uint32_t off_stage = (2u * off_blo + 1023u) & ~1023u;
  const uint32_t off_cn = off_stage + (uint32_t)stages * kStageBytes;
  const uint32_t off_bar = (off_cn + kNPad * 4u + 7u) & ~7u;
  const uint32_t off_misc = off_bar + W_NBARS * 8;
  float* cn_s = reinterpret_cast<float*>(sm + off_cn);
  volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(sm + off_misc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + off_misc + 4);
  auto bar = [&](int i) { return base + off_bar + (uint32_t)i * 8u; };

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  if (tid == 0) {
    for (int s = 0; s < kMaxStages; ++s) { mbar_init(bar(W_FULL + s), 1); mbar_init(bar(W_EMPTY + s), 128); }
    for (int b = 0; b < kNA; ++b) { mbar_init(bar(W_ARDY + b), 128); mbar_init(bar(W_AEMP + b), 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(bar(W_ACF + a), 1); mbar_init(bar(W_ACE + a), 128); }
    mbar_init(bar(W_BFUL), 1);
    mbar_init(bar(W_DRAIN), 1);
    *abort_flag = 0;
    abort_flag[3] = (int)wait_iters;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (tid < kNPad) cn_s[tid] = cn_pad[tid];
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(base + off_misc),
                 "r"((uint32_t)kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const float cn_max = cn_pad[kNPad];
  // TMEM columns: accumulator a at 32 a (16 used); A buffer b at 64 + 64 b: xh in 32 columns, xl in the next 32
  constexpr uint32_t kACol = 64u;
  const uint32_t idesc = (1u << 4) | ((uint32_t)(kNPad >> 3) << 17) | ((128u >> 4) << 24);

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      mbar_expect_tx(bar(W_BFUL), 2u * off_blo);
      for (int c = 0; c < n_chunks; ++c) {
        tma_load_2d(base + c * kPanelBytes, &tmBhi, c * 64, 0, bar(W_BFUL));
        tma_load_2d(base + off_blo + c * kPanelBytes, &tmBlo, c * 64, 0, bar(W_BFUL));
      }
      int c = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
        for (int ch = 0; ch < n_chunks && ok; ++ch, ++c) {
          const int s = c % stages;
          if (c >= stages) ok = mbar_wait(bar(W_EMPTY + s), (uint32_t)(c / stages - 1) & 1u, abort_flag, 1, c);
          if (!ok) break;
          mbar_expect_tx(bar(W_FULL + s), kStageBytes);
          const uint32_t dst = base + off_stage + (uint32_t)s * kStageBytes;
          tma_load_2d(dst, &tmX, ch * kChunk, (tile0 + tile) * kBM, bar(W_FULL + s));
          tma_load_2d(dst + 16384u, &tmX, ch * kChunk + 32, (tile0 + tile) * kBM, bar(W_FULL + s));
        }
      }
      if (!ok) {
        // aborting: let the copies already issued land before the CTA exits
        mbar_wait(bar(W_BFUL), 0, abort_flag, 0);
        const int lo = (c > stages) ? c - stages : 0;
        for (int j = lo; j < c; ++j) {
          mbar_drain(bar(W_FULL + j % stages), (uint32_t)(j / stages) & 1u);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0) {
      bool ok = mbar_wait(bar(W_BFUL), 0, abort_flag, 2);
      int c = 0, i = 0;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++i) {
        const int a = i & 1;
        if (i >= 2) ok = mbar_wait(bar(W_ACE + a), (uint32_t)((i >> 1) - 1) & 1u, abort_flag, 4, i);
        const uint32_t acc = tmem_base + (uint32_t)a * 32u;
        for (int ch = 0; ch < n_chunks && ok; ++ch, ++c) {
          const int b = c % kNA;
          ok = mbar_wait(bar(W_ARDY + b), (uint32_t)(c / kNA) & 1u, abort_flag, 3, c);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_hi = tmem_base + kACol + (uint32_t)b * 64u;
          const uint32_t bh = base + (uint32_t)ch * kPanelBytes;
          const uint32_t bl = base + off_blo + (uint32_t)ch * kPanelBytes;
#pragma unroll
          for (int term = 0; term < 3; ++term) {
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
              const uint32_t a_col = a_hi + (term == 1 ? 32u : 0u) + kk * 8u;
              const uint64_t bd = smem_desc_sw128((term == 2 ? bl : bh) + kk * 32u);
              tc_mma_ts(acc, a_col, bd, idesc, (ch | term | kk) ? 1u : 0u);
            }
          }
          tc_commit(bar(W_AEMP + b));
        }
        if (!ok) break;
        tc_commit(bar(W_ACF + a));
      }
      if (!ok) {
        // aborting, possibly in the middle of a tile: every MMA issued so far must retire before TMEM is
        // freed and the CTA's shared memory goes away
        tc_commit(bar(W_DRAIN));
        mbar_drain(bar(W_DRAIN), 0);
      }
    }
  } else if (warp < 4) {
    // spare warps (keep the role warps aligned to the four TMEM lane quadrants)
  } else if (warp < 12) {
    // ------------------------------ converters --------------------------------
    // group g takes the chunks with running index c % 2 == g; thread = row of the tile
    const int grp = (warp - 4) >> 2;
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    // chunks of this CTA: tiles x n_chunks, in the producer's order
    int my_tiles = 0;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) ++my_tiles;
    const long long total = (long long)my_tiles * n_chunks;
    bool ok = true;
    for (long long c = grp; c < total && ok; c += 2) {
      const int s = (int)(c % stages);
      const int b = (int)(c % kNA);
      ok = mbar_wait(bar(W_FULL + s), (uint32_t)(c / stages) & 1u, abort_flag, 5, (int)c);
      if (ok && c >= kNA) ok = mbar_wait(bar(W_AEMP + b), (uint32_t)(c / kNA - 1) & 1u, abort_flag, 6, (int)c);
      ok = __all_sync(0xffffffffu, ok);  // the tcgen05.st below needs the whole warp
      if (!ok) break;
      tc_fence_after();
      const uint32_t a_hi = tmem_base + lane_addr + kACol + (uint32_t)b * 64u;
      const uint8_t* stage = sm + off_stage + (size_t)s * kStageBytes;
#pragma unroll
      for (int p = 0; p < 2; ++p) {
        const uint8_t* rowp = stage + p * 16384 + row * 128;
        float4 xv[8];
#pragma unroll
        for (int cc = 0; cc < 8; ++cc) xv[cc] = *reinterpret_cast<const float4*>(rowp + ((cc ^ (row & 7)) << 4));
        uint32_t hi[16], lo[16];
#pragma unroll
        for (int cc = 0; cc < 8; ++cc) {
          const float y0 = xv[cc].x * sx, y1 = xv[cc].y * sx, y2 = xv[cc].z * sx, y3 = xv[cc].w * sx;
          const __half2 h01 = __floats2half2_rn(y0, y1);
          const __half2 h23 = __floats2half2_rn(y2, y3);
          const float2 f01 = __half22float2(h01);
          const float2 f23 = __half22float2(h23);
          const __half2 l01 = __floats2half2_rn(y0 - f01.x, y1 - f01.y);
          const __half2 l23 = __floats2half2_rn(y2 - f23.x, y3 - f23.y);
          hi[cc * 2 + 0] = *reinterpret_cast<const uint32_t*>(&h01);
          hi[cc * 2 + 1] = *reinterpret_cast<const uint32_t*>(&h23);
          lo[cc * 2 + 0] = *reinterpret_cast<const uint32_t*>(&l01);
          lo[cc * 2 + 1] = *reinterpret_cast<const uint32_t*>(&l23);
        }
        tmem_st16(a_hi + p * 16u, hi);
        tmem_st16(a_hi + 32u + p * 16u, lo);
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(bar(W_EMPTY + s));
      mbar_arrive(bar(W_ARDY + b));
    }
  } else {
    // ------------------------------ epilogue ----------------------------------
    const int q = warp & 3;
    const int row_in_tile = q * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    const float kInf = __int_as_float(0x7f800000);
    const float inv_sxsb = 1.0f / sxsb;
    unsigned int changed = 0;
    bool ok = true;
    int i = 0;
    for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++i) {
      const int a = i & 1;
      const size_t row = (size_t)(tile0 + tile) * kBM + row_in_tile;
      int old_label = -1;
      float xn = 0.f;
      if (row < n) {
        xn = xnorm[row];
        if (count_changes && out == nullptr) old_label = labels[row];
      }
      ok = mbar_wait(bar(W_ACF + a), (uint32_t)(i >> 1) & 1u, abort_flag, 7, i);
      ok = __all_sync(0xffffffffu, ok);  // the tcgen05.ld below needs the whole warp
      if (!ok) break;
      tc_fence_after();
      uint32_t v[32];
      tmem_ld16(tmem_base + lane_addr + (uint32_t)a * 32u, v, 0);
#pragma unroll
      for (int j = 16; j < 32; ++j) v[j] = 0u;
      tmem_wait_ld(v);
      tc_fence_before();
      mbar_arrive(bar(W_ACE + a));
      if (out != nullptr) {
        if (row < n) {
          const size_t r = row - (size_t)tile0 * kBM;
#pragma unroll
          for (int j = 0; j < kNPad; ++j)
            if (j < k) out[(size_t)j * ld_out + r] = fabsf(xn + (__uint_as_float(v[j]) + cn_s[j]) * inv_sxsb);
        }
        continue;
      }
      float best = kInf, second = kInf;
      int bidx = 0;
#pragma unroll
      for (int j = 0; j < kNPad; ++j) {
        const float sc = __uint_as_float(v[j]) + cn_s[j];   // +inf for the padding slots
        second = fminf(second, fmaxf(sc, best));
        const bool lt = sc < best;                          // strict: ties keep the lowest index
        best = lt ? sc : best;
        bidx = lt ? j : bidx;
      }
      if (row < n) {
        const float tol = split_tolerance(tol_rel, tol_floor, xn, cn_max, sx, sxsb);
        if (amb_rows != nullptr && !(second - best > tol)) {
          const unsigned int pos = atomicAdd(&st->amb_count, 1u);
          // (a row is listed at most once per launch, so the list cannot pass n entries; checked all the
          // same: an entry beyond the list's end would be a write outside the buffer)
          if (pos < n) amb_rows[pos] = (unsigned int)row;
          else atomicMax(&st->error, 31);
        } else {
          changed += (old_label != bidx);
          labels[row] = bidx;
        }
      }
    }
    if (count_changes && out == nullptr) {
      changed = __reduce_add_sync(0xffffffffu, changed);
      if (lane == 0 && changed) atomicAdd(&st->changed, (unsigned long long)changed);
    }
  }

  __syncthreads();
  if (tid == 0 && *abort_flag) atomicMax(&st->error, *abort_flag);
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)kTmemCols)
                 : "memory");
  }
}

}  // namespace tcw
}  // namespace km
