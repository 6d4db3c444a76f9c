// Tensor-core distance + argmin (and transform) with BOTH operands streamed: float32 rows of any
// width (d % 4 == 0) against more than 16 centroids.  Serves the shapes the other tensor-core kernels
// do not - rows wider than 256 columns with many centroids (d = 784, k = 100: the row does not fit
// tensor memory beside the accumulators) - and the n x k distance block of transform for every shape
// with more than 16 centroids.  Replaces calculate_distances + relabel
// (src/gpu/kmeans/kmeans_labels.cu:115-244, kmeans_labels.h:360-392) and the distance block of
// kmeans_transform (src/gpu/kmeans/kmeans_h2o4gpu.cu:891-975) there; the reference sends these
// shapes through cublasSgemm (kmeans_labels.cu:221-228).
//
// Same split-fp16 arithmetic as km_assign_tc.cuh (x sx = xh + xl, -2 c sb = bh + bl,
// acc = xh.bh + xl.bh + xh.bl, fp32 accumulation in TMEM).  A tile of 128 rows is walked in chunks of
// 64 columns, once per pass over NPAD centroids (NPAD = 128 or 256 = the MMA's N):
//   X chunk   TMA (two 128B-swizzled panels of 32 columns, zero fill beyond d) into a ring; converter
//             warps split it into one of four TMEM A buffers (as in km_assign_tc_wide.cuh)
//   B chunk   the pass's NPAD rows x 64 columns of the split centroid table, upper and lower halves,
//             TMA from L2 into a ring of three stages (N = 128) or two (N = 256)
//   MMA       12 instructions (M = 128, N = NPAD, K = 16) per chunk into the pass's accumulator
//   epilogue  after the last chunk: NPAD scores per row, folded into the row's running
//             (best, second best, index) - or stored as squared distances for transform
// With NPAD = 256 a chunk's MMAs take as long as its 32 KB of X take to arrive from HBM, so up to
// 256 centroids cost one pass at memory speed; more centroids re-read the tile from L2 once per pass.
// NPAD = 128 keeps two accumulators (the epilogue of one pass overlaps the next tile's MMAs).
//
// Warps: 0 X producer, 1 MMA issuer, 2 B producer, 3 spare, 4-11 converters (two groups of four,
// alternating chunks), 12-15 epilogue.  The X ring and the A buffers have even depths, so a stage always
// serves the same converter group (a barrier shared by two groups that are not ordered against each other cannot be
// waited for with a one-bit parity).  Every mbarrier wait is bounded.
#pragma once

#include "km_assign_tc.cuh"

namespace km {
namespace tcs {

using namespace km::tc;

constexpr int kSThreads = 512;
constexpr int kSChunk = 64;        // fp32 columns per chunk
constexpr int kSNA = 4;            // A buffers in TMEM
constexpr int kSMaxBStages = 3;    // ring of centroid chunks: three stages with N = 128, two with N = 256
constexpr int kSMaxXStages = 4;
constexpr uint32_t kSXStageBytes = kBM * kSChunk * 4;   // 32 KB

template <int NPAD> struct StreamCfg {
  static_assert(NPAD == 128 || NPAD == 256, "MMA N of the streaming kernel");
  static constexpr int kNAcc = 256 / NPAD;                       // accumulators of NPAD columns in TMEM columns 0..255
  static constexpr int kXStages = NPAD == 128 ? 4 : 2;           // even on purpose
  static constexpr uint32_t kBHalfBytes = (uint32_t)NPAD * 128u;  // one half (hi or lo) of a centroid chunk
  static constexpr uint32_t kBStageBytes = 2u * kBHalfBytes;
  // one consumer (the issuer), so an odd depth is fine here; a third stage covers the L2 latency of a
  // chunk while the two before it are multiplied (N = 128: 768 clocks of MMA per chunk)
  static constexpr int kBStages = NPAD == 128 ? 3 : 2;
};

enum SBar { S_XFUL = 0, S_XEMP = kSMaxXStages, S_ARDY = 2 * kSMaxXStages, S_AEMP = 2 * kSMaxXStages + kSNA,
            S_ACF = 2 * kSMaxXStages + 2 * kSNA, S_ACE = S_ACF + 2, S_BFUL = S_ACE + 2, S_BEMP = S_BFUL + kSMaxBStages,
            S_DRAIN = S_BEMP + kSMaxBStages, S_NBARS = S_DRAIN + 1 };

template <int NPAD>
inline size_t stream_smem_bytes() {
  using Cf = StreamCfg<NPAD>;
  return 1024 + (size_t)Cf::kBStages * Cf::kBStageBytes + (size_t)Cf::kXStages * kSXStageBytes + S_NBARS * 8 + 64;
}

// n_chunks = ceil(d / 64); n_pass = ceil(k / NPAD); cn_pad[n_pass * NPAD + 1]: |c|^2 sx sb (+inf in the
// padding), then max |c|^2.  out != nullptr: transform - out[j * ld_out + (row - row0)] = |xn + score_j|.
template <int NPAD>
__global__ void __launch_bounds__(kSThreads, 1)
assign_tc_stream_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmBhi,
                        const __grid_constant__ CUtensorMap tmBlo, const float* __restrict__ cn_pad,
                        const float* __restrict__ xnorm, int* __restrict__ labels, size_t n, int tile0, int n_tiles,
                        int n_chunks, int n_pass, int k, IterState* st, int count_changes,
                        unsigned int* __restrict__ amb_rows, float tol_rel, float tol_floor, float sx, float sxsb,
                        unsigned int wait_iters, float* __restrict__ out, size_t ld_out) {
  using Cf = StreamCfg<NPAD>;
  constexpr int kXS = Cf::kXStages;
  constexpr int kNAcc = Cf::kNAcc;
  constexpr int kSBStages = Cf::kBStages;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_u32 = smem_u32(smem_raw);
  const uint32_t base = (raw_u32 + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - raw_u32);

  constexpr uint32_t off_x = (uint32_t)kSBStages * Cf::kBStageBytes;
  constexpr uint32_t off_bar = off_x + (uint32_t)kXS * kSXStageBytes;
  constexpr uint32_t off_misc = off_bar + S_NBARS * 8;
  volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(sm + off_misc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + off_misc + 4);
  auto bar = [&](int i) { return base + off_bar + (uint32_t)i * 8u; };

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  if (tid == 0) {
    for (int s = 0; s < kSMaxXStages; ++s) { mbar_init(bar(S_XFUL + s), 1); mbar_init(bar(S_XEMP + s), 128); }
    for (int b = 0; b < kSNA; ++b) { mbar_init(bar(S_ARDY + b), 128); mbar_init(bar(S_AEMP + b), 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(bar(S_ACF + a), 1); mbar_init(bar(S_ACE + a), 128); }
    for (int t = 0; t < kSMaxBStages; ++t) { mbar_init(bar(S_BFUL + t), 1); mbar_init(bar(S_BEMP + t), 1); }
    mbar_init(bar(S_DRAIN), 1);
    *abort_flag = 0;
    abort_flag[3] = (int)wait_iters;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
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
  // TMEM columns: accumulator a at NPAD a (columns 0..255); A buffer b at 256 + 64 b: xh in 32 columns, xl in the next 32
  constexpr uint32_t kACol = 256u;
  const uint32_t idesc = (1u << 4) | ((uint32_t)(NPAD >> 3) << 17) | ((128u >> 4) << 24);

  // this CTA's work, in the order every role walks it: tiles x passes x chunks
  int my_tiles = 0;
  for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) ++my_tiles;
  const long long total = (long long)my_tiles * n_pass * n_chunks;

  if (warp == 0) {
    // ------------------------------ X producer --------------------------------
    if (lane == 0) {
      long long c = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
        for (int p = 0; p < n_pass && ok; ++p) {
          for (int ch = 0; ch < n_chunks && ok; ++ch, ++c) {
            const int s = (int)(c % kXS);
            if (c >= kXS) ok = mbar_wait(bar(S_XEMP + s), (uint32_t)(c / kXS - 1) & 1u, abort_flag, 1, (int)c);
            if (!ok) break;
            mbar_expect_tx(bar(S_XFUL + s), kSXStageBytes);
            const uint32_t dst = base + off_x + (uint32_t)s * kSXStageBytes;
            tma_load_2d(dst, &tmX, ch * kSChunk, (tile0 + tile) * kBM, bar(S_XFUL + s));
            tma_load_2d(dst + 16384u, &tmX, ch * kSChunk + 32, (tile0 + tile) * kBM, bar(S_XFUL + s));
          }
        }
      }
      if (!ok) {
        // aborting: let the copies already issued land before the CTA exits
        const long long lo = (c > kXS) ? c - kXS : 0;
        for (long long j = lo; j < c; ++j) mbar_drain(bar(S_XFUL + (int)(j % kXS)), (uint32_t)(j / kXS) & 1u);
      }
    }
  } else if (warp == 2) {
    // ------------------------------ B producer --------------------------------
    if (lane == 0) {
      long long c = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
        for (int p = 0; p < n_pass && ok; ++p) {
          for (int ch = 0; ch < n_chunks && ok; ++ch, ++c) {
            const int t = (int)(c % kSBStages);
            if (c >= kSBStages)
              ok = mbar_wait(bar(S_BEMP + t), (uint32_t)(c / kSBStages - 1) & 1u, abort_flag, 2, (int)c);
            if (!ok) break;
            mbar_expect_tx(bar(S_BFUL + t), Cf::kBStageBytes);
            const uint32_t dst = base + (uint32_t)t * Cf::kBStageBytes;
            tma_load_2d(dst, &tmBhi, ch * kSChunk, p * NPAD, bar(S_BFUL + t));
            tma_load_2d(dst + Cf::kBHalfBytes, &tmBlo, ch * kSChunk, p * NPAD, bar(S_BFUL + t));
          }
        }
      }
      if (!ok) {
        const long long lo = (c > kSBStages) ? c - kSBStages : 0;
        for (long long j = lo; j < c; ++j)
          mbar_drain(bar(S_BFUL + (int)(j % kSBStages)), (uint32_t)(j / kSBStages) & 1u);
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0) {
      bool ok = true;
      long long c = 0;
      int i = 0;   // running (tile, pass) index = use of an accumulator
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
        for (int p = 0; p < n_pass && ok; ++p, ++i) {
          const int a = i % kNAcc;
          if (i >= kNAcc) ok = mbar_wait(bar(S_ACE + a), (uint32_t)(i / kNAcc - 1) & 1u, abort_flag, 4, i);
          const uint32_t acc = tmem_base + (uint32_t)a * NPAD;
          for (int ch = 0; ch < n_chunks && ok; ++ch, ++c) {
            const int b = (int)(c % kSNA);
            const int t = (int)(c % kSBStages);
            ok = mbar_wait(bar(S_ARDY + b), (uint32_t)(c / kSNA) & 1u, abort_flag, 3, (int)c);
            if (ok) ok = mbar_wait(bar(S_BFUL + t), (uint32_t)(c / kSBStages) & 1u, abort_flag, 12, (int)c);
            if (!ok) break;
            tc_fence_after();
            const uint32_t a_hi = tmem_base + kACol + (uint32_t)b * 64u;
            const uint32_t bh = base + (uint32_t)t * Cf::kBStageBytes;
            const uint32_t bl = bh + Cf::kBHalfBytes;
#pragma unroll
            for (int term = 0; term < 3; ++term) {
#pragma unroll
              for (int kk = 0; kk < 4; ++kk) {
                const uint32_t a_col = a_hi + (term == 1 ? 32u : 0u) + kk * 8u;
                const uint64_t bd = smem_desc_sw128((term == 2 ? bl : bh) + kk * 32u);
                tc_mma_ts(acc, a_col, bd, idesc, (ch | term | kk) ? 1u : 0u);
              }
            }
            tc_commit(bar(S_AEMP + b));
            tc_commit(bar(S_BEMP + t));
          }
          if (!ok) break;
          tc_commit(bar(S_ACF + a));
        }
      }
      if (!ok) {
        // aborting, possibly in the middle of a tile: every MMA issued so far must retire before TMEM is
        // freed and the CTA's shared memory goes away
        tc_commit(bar(S_DRAIN));
        mbar_drain(bar(S_DRAIN), 0);
      }
    }
  } else if (warp < 4) {
    // spare warp (keeps the role warps aligned to the four TMEM lane quadrants)
  } else if (warp < 12) {
    // ------------------------------ converters --------------------------------
    // group g takes the chunks with running index c % 2 == g; thread = row of the tile
    const int grp = (warp - 4) >> 2;
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    bool ok = true;
    for (long long c = grp; c < total && ok; c += 2) {
      const int s = (int)(c % kXS);
      const int b = (int)(c % kSNA);
      ok = mbar_wait(bar(S_XFUL + s), (uint32_t)(c / kXS) & 1u, abort_flag, 5, (int)c);
      if (ok && c >= kSNA) ok = mbar_wait(bar(S_AEMP + b), (uint32_t)(c / kSNA - 1) & 1u, abort_flag, 6, (int)c);
      ok = __all_sync(0xffffffffu, ok);  // the tcgen05.st below needs the whole warp
      if (!ok) break;
      tc_fence_after();
      const uint32_t a_hi = tmem_base + lane_addr + kACol + (uint32_t)b * 64u;
      const uint8_t* stage = sm + off_x + (size_t)s * kSXStageBytes;
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
      mbar_arrive(bar(S_XEMP + s));
      mbar_arrive(bar(S_ARDY + b));
    }
  } else {
    // ------------------------------ epilogue ----------------------------------
    const int q = warp & 3;
    const int row_in_tile = q * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    const float kInf = __int_as_float(0x7f800000);
    const float inv_sxsb = 1.0f / sxsb;
    const float cn_max = cn_pad[n_pass * NPAD];
    unsigned int changed = 0;
    bool ok = true;
    int i = 0;
    for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
      const size_t row = (size_t)(tile0 + tile) * kBM + row_in_tile;
      int old_label = -1;
      float xn = 0.f;
      if (row < n) {
        xn = xnorm[row];
        if (count_changes && out == nullptr) old_label = labels[row];
      }
      float rbest = kInf, rsecond = kInf;
      int ridx = 0x7fffffff;
      for (int p = 0; p < n_pass && ok; ++p, ++i) {
        const int a = i % kNAcc;
        ok = mbar_wait(bar(S_ACF + a), (uint32_t)(i / kNAcc) & 1u, abort_flag, 7, i);
        ok = __all_sync(0xffffffffu, ok);  // the tcgen05.ld below needs the whole warp
        if (!ok) break;
        tc_fence_after();
        const uint32_t acc = tmem_base + lane_addr + (uint32_t)a * NPAD;
        const float* cnp = cn_pad + (size_t)p * NPAD;
        float bst[4] = {kInf, kInf, kInf, kInf}, sec[4] = {kInf, kInf, kInf, kInf};
        int bix[4] = {0, 0, 0, 0};
#pragma unroll 1
        for (int ch = 0; ch < NPAD / 32; ++ch) {
          const int c0 = ch * 32;
          uint32_t v[32];
          tmem_ld16(acc + c0, v, 0);
          tmem_ld16(acc + c0 + 16, v, 16);
          tmem_wait_ld(v);
          if (out != nullptr) {
            if (row < n) {
              const int col0 = p * NPAD + c0;
              float* op = out + (size_t)col0 * ld_out + (row - (size_t)tile0 * kBM);
#pragma unroll
              for (int j4 = 0; j4 < 8; ++j4) {
                const float4 cn4 = __ldg(reinterpret_cast<const float4*>(cnp + c0 + j4 * 4));
                const float cn[4] = {cn4.x, cn4.y, cn4.z, cn4.w};
#pragma unroll
                for (int qq = 0; qq < 4; ++qq) {
                  const int j = j4 * 4 + qq;
                  if (col0 + j < k) op[(size_t)j * ld_out] = fabsf(fmaf(__uint_as_float(v[j]) + cn[qq], inv_sxsb, xn));
                }
              }
            }
            continue;
          }
#pragma unroll
          for (int j4 = 0; j4 < 8; ++j4) {
            const float4 cn4 = __ldg(reinterpret_cast<const float4*>(cnp + c0 + j4 * 4));
            const float cn[4] = {cn4.x, cn4.y, cn4.z, cn4.w};
#pragma unroll
            for (int qq = 0; qq < 4; ++qq) {
              const float sc = __uint_as_float(v[j4 * 4 + qq]) + cn[qq];   // +inf for the padding slots
              sec[qq] = fminf(sec[qq], fmaxf(sc, bst[qq]));
              const bool lt = sc < bst[qq];                                // strict: ties keep the lowest index
              bst[qq] = lt ? sc : bst[qq];
              bix[qq] = lt ? (c0 + j4 * 4 + qq) : bix[qq];
            }
          }
        }
        tc_fence_before();
        mbar_arrive(bar(S_ACE + a));
        if (out != nullptr) continue;
        // fold the four chains, then this pass into the row's running result (ties: lowest index)
        float tb = bst[0], ts = sec[0];
        int ti = bix[0];
#pragma unroll
        for (int qq = 1; qq < 4; ++qq) {
          if (bst[qq] < tb || (bst[qq] == tb && bix[qq] < ti)) { ts = fminf(ts, tb); tb = bst[qq]; ti = bix[qq]; }
          else ts = fminf(ts, bst[qq]);
          ts = fminf(ts, sec[qq]);
        }
        ti += p * NPAD;
        if (tb < rbest || (tb == rbest && ti < ridx)) { rsecond = fminf(rbest, ts); rbest = tb; ridx = ti; }
        else rsecond = fminf(rsecond, tb);
        rsecond = fminf(rsecond, ts);
      }
      if (!ok) break;
      if (out != nullptr || row >= n) continue;
      const float tol = split_tolerance(tol_rel, tol_floor, xn, cn_max, sx, sxsb);
      if (amb_rows != nullptr && !(rsecond - rbest > tol)) {
        const unsigned int pos = atomicAdd(&st->amb_count, 1u);
        // (a row is listed at most once per launch, so the list cannot pass n entries; checked all the same)
        if (pos < n) amb_rows[pos] = (unsigned int)row;
        else atomicMax(&st->error, 31);
      } else {
        changed += (old_label != ridx);
        labels[row] = ridx;
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

}  // namespace tcs
}  // namespace km
