// Tensor-core distance + argmin for large centroid tables (k > 128; d = 32, 64, 128
// or 256): the contraction-bound regime.  Same split-fp16 arithmetic as
// km_assign_tc.cuh, but the centroid table no longer fits shared memory, so it is
// streamed: for every 128-row tile of X (converted once into TMEM) the CTA walks the
// centroid table in tiles of 128 centroids; each tile's (bh, bl) panels arrive by TMA
// through a ring of shared-memory stages of up to 128 K-columns, the MMAs of one
// centroid tile fill one of two TMEM accumulators, and the epilogue warps keep a
// running (min, second-min, argmin) per row across the centroid tiles while the next
// tile's MMAs run.  The rows x k matrix never exists.
//
// Per row tile: 3 * (d/16) * (k/128) MMAs of 128x128x16.  The kernel is bound by
// the tensor pipe; the X tile (<= 64 KB per chunk) and its conversion are a few
// percent of a row tile's time and overlap the previous tile's MMAs when the A
// operand is double-buffered (d <= 128).
//
// Warps: 0 X producer, 1 MMA issuer, 2 B producer, 3 spare, 4-7 converters,
// 8-11 epilogue of accumulator 0, 12-15 epilogue of accumulator 1.
#pragma once

#include "km_assign_tc.cuh"

namespace km {
namespace tcb {

using namespace km::tc;

constexpr int kNT = 128;        // centroids per tile = accumulator columns
constexpr int kBigThreads = 512;
constexpr int kBStages = 2;

// barriers
enum BBar { X_FULL = 0, X_EMPTY = 1, A_RDY = 2, A_EMP = 4, B_FUL = 6, B_EMP = 6 + kBStages,
            AC_FUL = 6 + 2 * kBStages, AC_EMP = 8 + 2 * kBStages, PT_FUL = 10 + 2 * kBStages,
            PT_EMP = 11 + 2 * kBStages, DRAIN = 12 + 2 * kBStages, NBARS = 13 + 2 * kBStages };

template <int D> struct BigCfg {
  static constexpr int DP = D < 64 ? 64 : D;          // fp16 columns of the centroid panels (padded to 64)
  static constexpr int KC = DP < 128 ? DP : 128;      // K columns per B stage
  static constexpr int NKC = DP / KC;                 // B stages per centroid tile
  static constexpr int XC = D < 128 ? D : 128;        // fp32 columns per X chunk
  static constexpr int NXC = D / XC;                  // X chunks per row tile
  static constexpr int NA = D <= 128 ? 2 : 1;         // A buffers in TMEM
  static constexpr int ACOLS = DP;                    // TMEM columns per A buffer (xh DP/2 + xl DP/2)
  static constexpr uint32_t kXBytes = XC * kBM * 4;   // one X chunk
  static constexpr uint32_t kBBytes = 2u * kNT * KC * 2;  // one B stage: hi + lo panels
  static constexpr uint32_t kAccCol = NA * ACOLS;     // accumulators behind the A buffers
};

template <int D>
inline size_t big_smem_bytes(int kpad) {
  using Cf = BigCfg<D>;
  return 1024 + Cf::kXBytes + (size_t)kBStages * Cf::kBBytes + (size_t)kpad * 4 + 3 * kBM * 4 + NBARS * 8 + 64;
}

// bh/bl: [kpad][DP] halves of -2 c * sb (zero padded), cn_pad[kpad] scaled |c|^2 (+inf padding),
// cn_pad[kpad] = max |c|^2 (zeroed before the launch)
__global__ void __launch_bounds__(256)
big_prep_kernel(const float* __restrict__ C, const float* __restrict__ cnorm, int k, int d, int dp, int kpad,
                float sb, float sxsb, __half* __restrict__ bhi, __half* __restrict__ blo,
                float* __restrict__ cn_pad) {
  const int j = blockIdx.x;
  for (int t = threadIdx.x; t < dp; t += blockDim.x) {
    float v = (j < k && t < d) ? -2.0f * C[(size_t)j * d + t] * sb : 0.0f;
    const __half h = __float2half_rn(v);
    bhi[(size_t)j * dp + t] = h;
    blo[(size_t)j * dp + t] = __float2half_rn(v - __half2float(h));
  }
  if (threadIdx.x == 0) {
    cn_pad[j] = (j < k) ? cnorm[j] * sxsb : __int_as_float(0x7f800000);
    if (j < k) atomicMax(reinterpret_cast<int*>(cn_pad + kpad), __float_as_int(cnorm[j]));
  }
}

__device__ __forceinline__ void tc_mma_ts2(uint32_t d_tmem, uint32_t a_tmem, uint32_t desc_lo, uint32_t desc_hi,
                                           uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 bd;\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "mov.b64 bd, {%2, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], bd, %4, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "r"(desc_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}

template <int D>
__global__ void __launch_bounds__(kBigThreads, 1)
assign_tc_big_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmBhi,
                     const __grid_constant__ CUtensorMap tmBlo, const float* __restrict__ cn_pad,
                     const float* __restrict__ xnorm, int* __restrict__ labels, size_t n, int n_tiles, int kpad,
                     IterState* st, int count_changes, unsigned int* __restrict__ amb_rows, float tol_rel,
                     float tol_floor, float sx, float sxsb, unsigned int wait_iters) {
  using Cf = BigCfg<D>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_u32 = smem_u32(smem_raw);
  const uint32_t base = (raw_u32 + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - raw_u32);

  constexpr uint32_t off_x = 0;
  constexpr uint32_t off_b = Cf::kXBytes;
  constexpr uint32_t off_cn = off_b + kBStages * Cf::kBBytes;
  const uint32_t off_part = off_cn + (uint32_t)kpad * 4u;      // [3][128] partial result of epilogue group 1
  const uint32_t off_bar = (off_part + 3u * kBM * 4u + 7u) & ~7u;
  const uint32_t off_misc = off_bar + NBARS * 8;
  float* cn_s = reinterpret_cast<float*>(sm + off_cn);
  float* part = reinterpret_cast<float*>(sm + off_part);
  volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(sm + off_misc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + off_misc + 4);
  auto bar = [&](int i) { return base + off_bar + (uint32_t)i * 8u; };

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int n_ct = kpad / kNT;  // centroid tiles per row tile

  if (tid == 0) {
    mbar_init(bar(X_FULL), 1);
    mbar_init(bar(X_EMPTY), 128);
    for (int a = 0; a < 2; ++a) {
      mbar_init(bar(A_RDY + a), 128);
      mbar_init(bar(A_EMP + a), 1);
      mbar_init(bar(AC_FUL + a), 1);
      mbar_init(bar(AC_EMP + a), 128);
    }
    for (int s = 0; s < kBStages; ++s) { mbar_init(bar(B_FUL + s), 1); mbar_init(bar(B_EMP + s), 1); }
    mbar_init(bar(PT_FUL), 128);
    mbar_init(bar(PT_EMP), 128);
    mbar_init(bar(DRAIN), 1);
    *abort_flag = 0;
    abort_flag[3] = (int)wait_iters;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  for (int i = tid; i < kpad; i += kBigThreads) cn_s[i] = cn_pad[i];
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
  const float cn_max = cn_pad[kpad];
  const uint32_t idesc = (1u << 4) | ((uint32_t)(kNT >> 3) << 17) | ((128u >> 4) << 24);

  if (warp == 0) {
    // ------------------------------ X producer --------------------------------
    if (lane == 0) {
      int xi = 0;  // chunk counter
      bool ok = true;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
        for (int xc = 0; xc < Cf::NXC && ok; ++xc, ++xi) {
          if (xi >= 1) ok = mbar_wait(bar(X_EMPTY), (uint32_t)(xi - 1) & 1u, abort_flag, 1);
          if (!ok) break;
          mbar_expect_tx(bar(X_FULL), Cf::kXBytes);
#pragma unroll
          for (int p = 0; p < Cf::XC / 32; ++p)
            tma_load_2d(base + off_x + p * 16384u, &tmX, xc * Cf::XC + p * 32, tile * kBM, bar(X_FULL));
        }
      }
      if (!ok && xi > 0) {
        mbar_drain(bar(X_FULL), (uint32_t)(xi - 1) & 1u);
      }
    }
  } else if (warp == 2) {
    // ------------------------------ B producer --------------------------------
    if (lane == 0) {
      int bs = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
        for (int ct = 0; ct < n_ct && ok; ++ct) {
          for (int kc = 0; kc < Cf::NKC && ok; ++kc, ++bs) {
            const int s = bs % kBStages;
            if (bs >= kBStages) ok = mbar_wait(bar(B_EMP + s), (uint32_t)(bs / kBStages - 1) & 1u, abort_flag, 2);
            if (!ok) break;
            mbar_expect_tx(bar(B_FUL + s), Cf::kBBytes);
            const uint32_t sb0 = base + off_b + s * Cf::kBBytes;
#pragma unroll
            for (int p = 0; p < Cf::KC / 64; ++p) {
              tma_load_2d(sb0 + p * (kNT * 128u), &tmBhi, kc * Cf::KC + p * 64, ct * kNT, bar(B_FUL + s));
              tma_load_2d(sb0 + (Cf::KC / 64 + p) * (kNT * 128u), &tmBlo, kc * Cf::KC + p * 64, ct * kNT,
                          bar(B_FUL + s));
            }
          }
        }
      }
      if (!ok) {
        const int lo = (bs > kBStages) ? bs - kBStages : 0;
        for (int j = lo; j < bs; ++j) {
          mbar_drain(bar(B_FUL + j % kBStages), (uint32_t)(j / kBStages) & 1u);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0) {
      bool ok = true;
      int it = 0, bs = 0, j = 0;
      // constant upper word of every centroid-panel descriptor
      const uint32_t desc_hi = (uint32_t)(smem_desc_sw128(0) >> 32);
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++it) {
        const int a = it % Cf::NA;
        ok = mbar_wait(bar(A_RDY + a), (uint32_t)(it / Cf::NA) & 1u, abort_flag, 3);
        const uint32_t a_base = tmem_base + (uint32_t)a * Cf::ACOLS;
        for (int ct = 0; ct < n_ct && ok; ++ct, ++j) {
          const int ac = j & 1;
          if (j >= 2) ok = mbar_wait(bar(AC_EMP + ac), (uint32_t)((j >> 1) - 1) & 1u, abort_flag, 4);
          const uint32_t acc = tmem_base + Cf::kAccCol + (uint32_t)ac * kNT;
          for (int kc = 0; kc < Cf::NKC && ok; ++kc, ++bs) {
            const int s = bs % kBStages;
            ok = mbar_wait(bar(B_FUL + s), (uint32_t)(bs / kBStages) & 1u, abort_flag, 5);
            if (!ok) break;
            tc_fence_after();
            const uint32_t sb0 = base + off_b + s * Cf::kBBytes;
            const uint32_t lo_hi = (uint32_t)smem_desc_sw128(sb0);                               // hi panels
            const uint32_t lo_lo = (uint32_t)smem_desc_sw128(sb0 + (Cf::KC / 64) * (kNT * 128u));  // lo panels
#pragma unroll
            for (int term = 0; term < 3; ++term) {
#pragma unroll
              for (int kk = 0; kk < Cf::KC / 16; ++kk) {
                // k-step kk of this stage: panel kk / 4 (16 KB apart), 32 bytes per step inside it
                const uint32_t boff = ((kk >> 2) * (kNT * 128u) + (kk & 3) * 32u) >> 4;
                const uint32_t a_col = a_base + (term == 1 ? Cf::ACOLS / 2 : 0) + (kc * (Cf::KC / 16) + kk) * 8u;
                tc_mma_ts2(acc, a_col, ((term == 2) ? lo_lo : lo_hi) + boff, desc_hi, idesc,
                           (kc | term | kk) ? 1u : 0u);
              }
            }
            tc_commit(bar(B_EMP + s));
          }
          if (!ok) break;
          tc_commit(bar(AC_FUL + ac));
        }
        if (ok) tc_commit(bar(A_EMP + a));
      }
      if (!ok) {
        // aborting, possibly in the middle of a centroid tile: every MMA issued so far must retire before
        // TMEM is freed
        tc_commit(bar(DRAIN));
        mbar_drain(bar(DRAIN), 0);
      }

    }
  } else if (warp == 3) {
    // spare
  } else if (warp < 8) {
    // ------------------------------ converters --------------------------------
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    bool ok = true;
    int it = 0, xi = 0;
    for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++it) {
      const int a = it % Cf::NA;
      const uint32_t a_hi = tmem_base + lane_addr + (uint32_t)a * Cf::ACOLS;
      for (int xc = 0; xc < Cf::NXC && ok; ++xc, ++xi) {
        ok = mbar_wait(bar(X_FULL), (uint32_t)xi & 1u, abort_flag, 6);
        if (ok && xc == 0 && it >= Cf::NA)
          ok = mbar_wait(bar(A_EMP + a), (uint32_t)(it / Cf::NA - 1) & 1u, abort_flag, 7);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int p = 0; p < Cf::XC / 32; ++p) {
          const uint8_t* rowp = sm + off_x + p * 16384 + row * 128;
          float4 xv[8];
#pragma unroll
          for (int c = 0; c < 8; ++c) xv[c] = *reinterpret_cast<const float4*>(rowp + ((c ^ (row & 7)) << 4));
          uint32_t hi[16], lo[16];
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            const float y0 = xv[c].x * sx, y1 = xv[c].y * sx, y2 = xv[c].z * sx, y3 = xv[c].w * sx;
            const __half2 h01 = __floats2half2_rn(y0, y1);
            const __half2 h23 = __floats2half2_rn(y2, y3);
            const float2 f01 = __half22float2(h01);
            const float2 f23 = __half22float2(h23);
            const __half2 l01 = __floats2half2_rn(y0 - f01.x, y1 - f01.y);
            const __half2 l23 = __floats2half2_rn(y2 - f23.x, y3 - f23.y);
            hi[c * 2 + 0] = *reinterpret_cast<const uint32_t*>(&h01);
            hi[c * 2 + 1] = *reinterpret_cast<const uint32_t*>(&h23);
            lo[c * 2 + 0] = *reinterpret_cast<const uint32_t*>(&l01);
            lo[c * 2 + 1] = *reinterpret_cast<const uint32_t*>(&l23);
          }
          const uint32_t col = (uint32_t)(xc * (Cf::XC / 2) + p * 16);
          tmem_st16(a_hi + col, hi);
          tmem_st16(a_hi + Cf::ACOLS / 2 + col, lo);
        }
        if (D < 64 && xc == Cf::NXC - 1) {
          // d = 32: the centroid panels are padded to 64 columns; the matching A columns are zero
          uint32_t z[16];
#pragma unroll
          for (int c = 0; c < 16; ++c) z[c] = 0u;
          tmem_st16(a_hi + 16u, z);
          tmem_st16(a_hi + Cf::ACOLS / 2 + 16u, z);
        }
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(bar(X_EMPTY));
      }
      if (ok) mbar_arrive(bar(A_RDY + a));
    }
  } else {
    // ------------------------------ epilogue ----------------------------------
    // group g drains accumulator g, i.e. the centroid tiles whose running index is g mod 2
    const int grp = (warp - 8) >> 2;
    const int q = warp & 3;
    const int row_in_tile = q * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    const uint32_t acc = tmem_base + lane_addr + Cf::kAccCol + (uint32_t)grp * kNT;
    const float kInf = __int_as_float(0x7f800000);
    unsigned int changed = 0;
    bool ok = true;
    int it = 0;
    long long j0 = 0;  // running index of this row tile's first centroid tile
    int uses = 0;      // how often this group has used its accumulator
    for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++it, j0 += n_ct) {
      const size_t row = (size_t)tile * kBM + row_in_tile;
      int old_label = -1;
      float xn = 0.f;
      if (grp == 0 && row < n) {
        xn = xnorm[row];
        if (count_changes) old_label = labels[row];
      }
      float rbest = kInf, rsecond = kInf;
      int ridx = 0x7fffffff;
      for (int ct = (int)((grp - j0) & 1); ct < n_ct && ok; ct += 2, ++uses) {
        ok = mbar_wait(bar(AC_FUL + grp), (uint32_t)uses & 1u, abort_flag, 8);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        float bst[4] = {kInf, kInf, kInf, kInf}, sec[4] = {kInf, kInf, kInf, kInf};
        int bix[4] = {0, 0, 0, 0};
        const float* cnp = cn_s + ct * kNT;
#pragma unroll
        for (int ch = 0; ch < kNT / 32; ++ch) {
          const int c0 = ch * 32;
          uint32_t v[32];
          tmem_ld16(acc + c0, v, 0);
          tmem_ld16(acc + c0 + 16, v, 16);
          tmem_wait_ld(v);
#pragma unroll
          for (int j4 = 0; j4 < 8; ++j4) {
            const float4 cn4 = *reinterpret_cast<const float4*>(cnp + c0 + j4 * 4);
            const float cn[4] = {cn4.x, cn4.y, cn4.z, cn4.w};
#pragma unroll
            for (int qq = 0; qq < 4; ++qq) {
              const float sc = __uint_as_float(v[j4 * 4 + qq]) + cn[qq];
              sec[qq] = fminf(sec[qq], fmaxf(sc, bst[qq]));
              const bool lt = sc < bst[qq];
              bst[qq] = lt ? sc : bst[qq];
              bix[qq] = lt ? (c0 + j4 * 4 + qq) : bix[qq];
            }
          }
        }
        tc_fence_before();
        mbar_arrive(bar(AC_EMP + grp));
        // fold the four chains, then this tile into the row's running result
        float tb = bst[0], ts = sec[0];
        int ti = bix[0];
#pragma unroll
        for (int qq = 1; qq < 4; ++qq) {
          if (bst[qq] < tb || (bst[qq] == tb && bix[qq] < ti)) { ts = fminf(ts, tb); tb = bst[qq]; ti = bix[qq]; }
          else ts = fminf(ts, bst[qq]);
          ts = fminf(ts, sec[qq]);
        }
        ti += ct * kNT;
        if (tb < rbest || (tb == rbest && ti < ridx)) { rsecond = fminf(rbest, ts); rbest = tb; ridx = ti; }
        else rsecond = fminf(rsecond, tb);
        rsecond = fminf(rsecond, ts);
      }
      if (!ok) break;
      // group 1 hands its partial result to group 0, which finishes the row
      const uint32_t phx = (uint32_t)it & 1u;
      if (grp == 1) {
        if (it >= 1) ok = mbar_wait(bar(PT_EMP), phx ^ 1u, abort_flag, 9);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        part[row_in_tile] = rbest;
        part[kBM + row_in_tile] = rsecond;
        part[2 * kBM + row_in_tile] = __int_as_float(ridx);
        mbar_arrive(bar(PT_FUL));
      } else {
        ok = mbar_wait(bar(PT_FUL), phx, abort_flag, 10);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        const float ob = part[row_in_tile];
        const float os = part[kBM + row_in_tile];
        const int oi = __float_as_int(part[2 * kBM + row_in_tile]);
        mbar_arrive(bar(PT_EMP));
        if (ob < rbest || (ob == rbest && oi < ridx)) { rsecond = fminf(rbest, os); rbest = ob; ridx = oi; }
        else rsecond = fminf(rsecond, ob);
        rsecond = fminf(rsecond, os);
        if (row < n) {
          const float tol = split_tolerance(tol_rel, tol_floor, xn, cn_max, sx, sxsb);
          if (amb_rows != nullptr && !(rsecond - rbest > tol)) {
            const unsigned int pos = atomicAdd(&st->amb_count, 1u);
            amb_rows[pos] = (unsigned int)row;
          } else {
            changed += (old_label != ridx);
            labels[row] = ridx;
          }
        }
      }
    }
    if (count_changes && grp == 0) {
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

// Exact re-evaluation of the listed rows against all k centroids: direct differences in double on
// the double copy of the centroid table, lowest index on ties.  A CTA takes two rows at a time: it
// widens them into shared memory once (integer operations - no float -> double conversion
// instructions: the first version converted x and c for every pair and spent most of its time
// there), and its eight warps share the centroids, four per warp and step, so that a centroid element
// fetched from L1 / L2 serves two rows and a short list still fills the GPU (one warp per row left
// most SMs idle when a few thousand rows were listed).  The eight partial sums of a step are reduced
// by trading halves between lanes (9 exchanges instead of 40), which leaves each group of four lanes
// with one (row, centroid) total; every lane keeps the running minimum of its own slot, the four
// slots of a row are merged at the end of the warp's share and the eight warps' results in shared
// memory.  Dynamic shared memory: 16 d bytes.
// Tried instead: the table transposed so that the lanes of a warp own 32 centroids and walk the columns
// together (no cross-lane sums at all, one argmin per 32 centroids): equal on C3, 3 % faster on C5
// (k = 4096), 8-16 % slower with 10 or 100 centroids and 784 columns - not kept.
constexpr int kRefineBigThreads = 256;
__global__ void __launch_bounds__(kRefineBigThreads)
refine_big_kernel(const float* __restrict__ X, int d, const double* __restrict__ Cd, int k,
                  const unsigned int* __restrict__ amb_rows, IterState* st, int* __restrict__ labels,
                  int count_changes) {
  extern __shared__ __align__(16) double refine_xs[];   // [2][d]
  __shared__ double s_best[2][kRefineBigThreads / 32];
  __shared__ int s_idx[2][kRefineBigThreads / 32];
  const unsigned int cnt = st->amb_count;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  constexpr int NW = kRefineBigThreads / 32;
  const double kInf = __longlong_as_double(0x7ff0000000000000LL);
  // this lane's slot after the reduction: row (bit 4), centroid of the step (bits 3 and 2)
  const int my_r = (lane >> 4) & 1;
  const int my_u = ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1);
  const double* xs0 = refine_xs;
  const double* xs1 = refine_xs + d;
  unsigned int changed = 0;
  for (unsigned int e = blockIdx.x * 2; e < cnt; e += gridDim.x * 2) {
    const bool two = e + 1 < cnt;
    const size_t r0 = amb_rows[e];
    const size_t r1 = two ? amb_rows[e + 1] : r0;
    __syncthreads();   // the previous pair's rows are no longer read
    for (int t = threadIdx.x; t < d; t += kRefineBigThreads) {
      refine_xs[t] = widen_exact(X[r0 * (size_t)d + t]);
      refine_xs[d + t] = widen_exact(X[r1 * (size_t)d + t]);
    }
    __syncthreads();
    double best = kInf;
    int bi = 0x7fffffff;
    for (int c0 = warp * 4; c0 < k; c0 += NW * 4) {
      double v[8] = {0, 0, 0, 0, 0, 0, 0, 0};   // [row][centroid of the step]
      for (int t0 = 0; t0 < d; t0 += 256) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int t = t0 + lane + 32 * i;
          if (t < d) {
            const double xa = xs0[t], xb = xs1[t];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              if (c0 + u < k) {
                const double cv = Cd[(size_t)(c0 + u) * d + t];
                const double q0 = xa - cv, q1 = xb - cv;
                v[u] = fma(q0, q0, v[u]);
                v[4 + u] = fma(q1, q1, v[4 + u]);
              }
            }
          }
        }
      }
      // trade halves: xor 16 separates the rows, xor 8 and xor 4 the centroids; then a butterfly over the quad
      {
        const bool up = (lane & 16) != 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const double keep = up ? v[i + 4] : v[i], send = up ? v[i] : v[i + 4];
          v[i] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
        }
      }
      {
        const bool up = (lane & 8) != 0;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const double keep = up ? v[i + 2] : v[i], send = up ? v[i] : v[i + 2];
          v[i] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
        }
      }
      {
        const bool up = (lane & 4) != 0;
        const double keep = up ? v[1] : v[0], send = up ? v[0] : v[1];
        v[0] = keep + __shfl_xor_sync(0xffffffffu, send, 4);
      }
      v[0] += __shfl_xor_sync(0xffffffffu, v[0], 2);
      v[0] += __shfl_xor_sync(0xffffffffu, v[0], 1);
      const int c = c0 + my_u;
      if (c < k && v[0] < best) { best = v[0]; bi = c; }   // ascending c within a slot: strict < keeps the lowest
    }
    // merge the four slots of each row (lanes that differ in bits 3 and 2): smaller distance, then lower index
#pragma unroll
    for (int o = 8; o >= 4; o >>= 1) {
      const double ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob < best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    if ((lane & 15) == 0) { s_best[my_r][warp] = best; s_idx[my_r][warp] = bi; }
    __syncthreads();
    if (warp == 0 && (lane & 15) == 0 && (my_r == 0 || two)) {
      double b = s_best[my_r][0];
      int id = s_idx[my_r][0];
#pragma unroll
      for (int w = 1; w < NW; ++w) {
        const double ob = s_best[my_r][w];
        const int oi = s_idx[my_r][w];
        if (ob < b || (ob == b && oi < id)) { b = ob; id = oi; }
      }
      const size_t row = my_r ? r1 : r0;
      changed += (labels[row] != id);
      labels[row] = id;
    }
  }
  if (count_changes && changed) atomicAdd(&st->changed, (unsigned long long)changed);
}

}  // namespace tcb
}  // namespace km
