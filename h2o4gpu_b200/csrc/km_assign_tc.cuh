// Tensor-core distance + argmin kernel for sm_100a (tcgen05 / TMEM / TMA).
//
// Scores |c|^2 - 2 x.c for a 128-row tile of X against all centroids are formed
// on the 5th-generation tensor cores as a 3xTF32 product so that fp32 accuracy
// is kept:   x = xh + xl,  -2c = bh + bl  (h = nearest TF32 value, l = rounded rest)
//            acc = xh.bh + xl.bh + xh.bl          (fp32 accumulation in TMEM)
// and the epilogue adds |c|^2 and takes the running argmin, so the rows x k
// distance matrix never exists.  Replaces calculate_distances + relabel
// (src/gpu/kmeans/kmeans_labels.cu:115-244, kmeans_labels.h:360-392) for
// float32, d in {32, 64}, 16 < k <= 128.
//
// Persistent CTAs (one per SM), warp-specialised:
//   warp 0      TMA producer: raw fp32 X tiles (128 x d, 128B-swizzled panels of
//               32 columns) into a 4-stage shared-memory ring; the split
//               centroid table (bh, bl) is loaded once per CTA and stays resident.
//   warps 4-11  converters (two groups of four, alternating tiles): thread r reads row r of the tile (conflict-free
//               thanks to the swizzle), splits it and writes xh / xl into TMEM
//               with tcgen05.st - the A operand of the MMA lives in TMEM, so
//               the tensor core reads only the centroid panels from shared memory.
//   warps 1-2   MMA issuers, one per A buffer / accumulator: 3 * d/8 tcgen05.mma
//               (M=128, N=kpad, K=8) per tile; tcgen05.commit releases the A
//               buffer and publishes the accumulator.
//   warps 12-19 epilogue (two groups of four, one per accumulator): tcgen05.ld, + |c|^2, argmin (first minimum wins),
//               label store, changed-label count.
// Every mbarrier wait is bounded (wall-clock limit); on a timeout the CTA sets an
// error word, drains its copies, frees its TMEM and returns.
#pragma once

#include <cuda.h>

#include "km_common.cuh"

namespace km {
namespace tc {



constexpr int kBM = 128;
constexpr int kThreads = 640;  // producer, 2 MMA issuers, spare, 2 x 4 converter warps, 2 x 4 epilogue warps
constexpr int kStages = 4;
constexpr int kMaxD = 64;
constexpr int kMaxNPad = 128;
constexpr int kTmemCols = 512;
constexpr unsigned long long kWaitLimitNs = 2000000000ULL;  // 2 s (abort drain loops)
constexpr long long kWaitLimitClk = 6000000000LL;          // about 3 s of SM clocks

enum Bar { FULL = 0, EMPTY = kStages, A_READY = 2 * kStages, A_EMPTY = 2 * kStages + 2,
           ACC_FULL = 2 * kStages + 4, ACC_EMPTY = 2 * kStages + 6, B_FULL = 2 * kStages + 8,
           NUM_BARS = 2 * kStages + 9 };

inline size_t smem_bytes(int d, int npad) {
  size_t P = d / 32;
  return 1024 + 2 * P * (size_t)npad * 128 + (size_t)kStages * P * 16384 + (size_t)npad * 4 + 2 * kBM * 4 +
         NUM_BARS * 8 + 64;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ unsigned long long gtime_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait.  Returns false when the CTA is aborting (this wait or another
// one gave up); the caller leaves its loop.
// try_wait that lets the hardware park the warp for up to `ns` nanoseconds (it wakes
// as soon as the phase completes), so waiting costs no issue slots.
__device__ __forceinline__ bool mbar_try_hint(uint32_t bar, uint32_t parity, uint32_t ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(ns)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code) {
  // 150000 parked waits of at most 20 us each: gives up after about 3 s
  for (unsigned int it = 0; it < 150000u; ++it) {
    if (mbar_try_hint(bar, parity, 20000u)) return true;
    if (*abort_flag) return false;
  }
  *abort_flag = code;
  return false;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem desc], kind::tf32, M=128
__device__ __forceinline__ void tc_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// K-major, 128-byte swizzle, dense 8-row groups (1024 B apart)
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
  uint64_t desc = (uint64_t)((addr & 0x3FFFFu) >> 4);
  desc |= (uint64_t)1 << 16;             // leading byte offset (unused for swizzled K-major)
  desc |= (uint64_t)(1024 >> 4) << 32;   // stride byte offset between 8-row groups
  desc |= (uint64_t)1 << 46;             // descriptor version (sm_100)
  desc |= (uint64_t)2 << 61;             // SWIZZLE_128B
  return desc;
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[32], int o) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(v[o + 0]), "=r"(v[o + 1]), "=r"(v[o + 2]), "=r"(v[o + 3]), "=r"(v[o + 4]), "=r"(v[o + 5]),
        "=r"(v[o + 6]), "=r"(v[o + 7]), "=r"(v[o + 8]), "=r"(v[o + 9]), "=r"(v[o + 10]), "=r"(v[o + 11]),
        "=r"(v[o + 12]), "=r"(v[o + 13]), "=r"(v[o + 14]), "=r"(v[o + 15])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&v)[16]) {
  const int o = 0;
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(v[o + 0]), "r"(v[o + 1]), "r"(v[o + 2]), "r"(v[o + 3]), "r"(v[o + 4]), "r"(v[o + 5]),
        "r"(v[o + 6]), "r"(v[o + 7]), "r"(v[o + 8]), "r"(v[o + 9]), "r"(v[o + 10]), "r"(v[o + 11]), "r"(v[o + 12]),
        "r"(v[o + 13]), "r"(v[o + 14]), "r"(v[o + 15])
      : "memory");
}
// The loaded registers are operands of the wait so that no use of them can be
// scheduled ahead of it.
__device__ __forceinline__ void tmem_wait_ld(uint32_t (&v)[32]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]), "+r"(v[7]),
                 "+r"(v[8]), "+r"(v[9]), "+r"(v[10]), "+r"(v[11]), "+r"(v[12]), "+r"(v[13]), "+r"(v[14]), "+r"(v[15]),
                 "+r"(v[16]), "+r"(v[17]), "+r"(v[18]), "+r"(v[19]), "+r"(v[20]), "+r"(v[21]), "+r"(v[22]), "+r"(v[23]),
                 "+r"(v[24]), "+r"(v[25]), "+r"(v[26]), "+r"(v[27]), "+r"(v[28]), "+r"(v[29]), "+r"(v[30]), "+r"(v[31])
               :
               : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// x rounded to the nearest TF32 value (11 significand bits, ties away from zero);
// the low 13 bits of the result are zero, so the tensor core reads it exactly.
__device__ __forceinline__ float tf32_rn(float x) {
  return __uint_as_float((__float_as_uint(x) + 0x00001000u) & 0xffffe000u);
}

// Split centroid table for the tensor-core kernel: bh/bl = split(-2 c), rows
// k..npad-1 zero with |c|^2 = +inf so that padding never wins the argmin.
__global__ void __launch_bounds__(64)
prep_kernel(const float* __restrict__ C, const float* __restrict__ cnorm, int k, int d, int npad,
            float* __restrict__ bhi, float* __restrict__ blo, float* __restrict__ cnorm_pad) {
  const int j = blockIdx.x;
  for (int t = threadIdx.x; t < d; t += blockDim.x) {
    float v = (j < k) ? -2.0f * C[(size_t)j * d + t] : 0.0f;
    float h = tf32_rn(v);
    bhi[(size_t)j * d + t] = h;
    blo[(size_t)j * d + t] = tf32_rn(v - h);
  }
  if (threadIdx.x == 0) {
    cnorm_pad[j] = (j < k) ? cnorm[j] : __int_as_float(0x7f800000);
    // slot npad (zeroed before the launch) receives max |c|^2; non-negative floats order as ints
    if (j < k) atomicMax(reinterpret_cast<int*>(cnorm_pad + npad), __float_as_int(cnorm[j]));
  }
}

// Operand halves: xh is x itself (the tensor core ignores the low 13 bits of an
// fp32 operand - measured on B200 - so it sees x truncated to TF32), xl is
// x - trunc(x) rounded to TF32; -2c is split by rounding on both halves.
// dbg: bit 1 (2) = do not issue the MMAs, bit 2 (4) = skip the epilogue arithmetic,
// bit 3 (8) = skip the TMEM stores (timing experiments only).
template <int D>
__global__ void __launch_bounds__(kThreads, 1)
assign_tc_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmBhi,
                 const __grid_constant__ CUtensorMap tmBlo, const float* __restrict__ cnorm_pad,
                 int* __restrict__ labels, size_t n, int n_tiles, int npad, IterState* st,
                 int count_changes, unsigned int* __restrict__ amb_rows, float tol_rel, int dbg) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_u32 = smem_u32(smem_raw);
  const uint32_t base = (raw_u32 + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - raw_u32);

  constexpr int P = D / 32;  // 32-column panels per row tile
  const uint32_t b_panel = (uint32_t)npad * 128u;
  const uint32_t off_blo = (uint32_t)P * b_panel;
  const uint32_t off_stage = 2u * P * b_panel;
  constexpr uint32_t stage_bytes = (uint32_t)P * 16384u;
  const uint32_t off_cn = off_stage + kStages * stage_bytes;
  const uint32_t off_xn = off_cn + (uint32_t)npad * 4u;
  const uint32_t off_bar = (off_xn + 2u * kBM * 4u + 7u) & ~7u;
  const uint32_t off_misc = off_bar + NUM_BARS * 8;
  float* cn_s = reinterpret_cast<float*>(sm + off_cn);
  float* xn_s = reinterpret_cast<float*>(sm + off_xn);  // [2][128] |x|^2 of the rows in A buffer b
  volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(sm + off_misc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + off_misc + 4);
  auto bar = [&](int i) { return base + off_bar + (uint32_t)i * 8u; };

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(bar(FULL + s), 1); mbar_init(bar(EMPTY + s), 128); }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar(A_READY + b), 128);
      mbar_init(bar(A_EMPTY + b), 1);
      mbar_init(bar(ACC_FULL + b), 1);
      mbar_init(bar(ACC_EMPTY + b), 128);
    }
    mbar_init(bar(B_FULL), 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  for (int i = tid; i < npad; i += kThreads) cn_s[i] = cnorm_pad[i];
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
  const float cn_max = cnorm_pad[npad];  // largest |c|^2, stored behind the padded table
  // TMEM columns: accumulators at 0 and 128; A buffers b at 256 + 128 b (xh) and + 64 (xl)
  const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(npad >> 3) << 17) | ((128u >> 4) << 24);

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      mbar_expect_tx(bar(B_FULL), 2u * P * b_panel);
      for (int p = 0; p < P; ++p) {
        tma_load_2d(base + p * b_panel, &tmBhi, p * 32, 0, bar(B_FULL));
        tma_load_2d(base + off_blo + p * b_panel, &tmBlo, p * 32, 0, bar(B_FULL));
      }
      int i = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++i) {
        const int s = i % kStages;
        const uint32_t ph = (uint32_t)(i / kStages) & 1u;
        if (i >= kStages) ok = mbar_wait(bar(EMPTY + s), ph ^ 1u, abort_flag, 1);
        if (!ok) break;
        mbar_expect_tx(bar(FULL + s), stage_bytes);
#pragma unroll
        for (int p = 0; p < P; ++p)
          tma_load_2d(base + off_stage + s * stage_bytes + p * 16384u, &tmX, p * 32, tile * kBM, bar(FULL + s));
      }
      if (!ok) {
        // aborting: let the copies already issued land before the CTA exits
        mbar_wait(bar(B_FULL), 0, abort_flag, 0);
        const int lo = (i > kStages) ? i - kStages : 0;
        for (int j = lo; j < i; ++j) {
          const unsigned long long t0 = gtime_ns();
          while (!mbar_try(bar(FULL + j % kStages), (uint32_t)(j / kStages) & 1u))
            if (gtime_ns() - t0 > kWaitLimitNs) break;
        }
      }
    }
  } else if (warp == 1 || warp == 2) {
    // ------------------------------ MMA issuers -------------------------------
    // Two issuing threads on two schedulers, one per A buffer / accumulator: the
    // issue rate of a single thread (about ten scalar instructions per MMA) would
    // otherwise cap the tensor pipe below its rate for these short K = 8 MMAs.
    const int grp = warp - 1;
    if (lane == 0) {
      bool ok = mbar_wait(bar(B_FULL), 0, abort_flag, 2);
      // the centroid panels never move: one shared-memory descriptor per (panel, k-step)
      uint64_t bdesc_hi[P * 4], bdesc_lo[P * 4];
#pragma unroll
      for (int p = 0; p < P; ++p)
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          bdesc_hi[p * 4 + kk] = smem_desc_sw128(base + p * b_panel + kk * 32u);
          bdesc_lo[p * 4 + kk] = smem_desc_sw128(base + off_blo + p * b_panel + kk * 32u);
        }
      const uint32_t acc = tmem_base + (uint32_t)grp * 128u;
      const uint32_t a_hi = tmem_base + 256u + (uint32_t)grp * 128u;
      int i = grp;
      for (int tile = blockIdx.x + grp * gridDim.x; tile < n_tiles && ok; tile += 2 * gridDim.x, i += 2) {
        const uint32_t phb = (uint32_t)(i >> 1) & 1u;
        ok = mbar_wait(bar(A_READY + grp), phb, abort_flag, 3);
        if (ok && i >= 2) ok = mbar_wait(bar(ACC_EMPTY + grp), phb ^ 1u, abort_flag, 4);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int term = 0; term < 3; ++term) {
#pragma unroll
          for (int p = 0; p < P; ++p) {
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
              const uint32_t a_col = a_hi + (term == 1 ? 64u : 0u) + p * 32u + kk * 8u;
              const uint64_t bd = (term == 2) ? bdesc_lo[p * 4 + kk] : bdesc_hi[p * 4 + kk];
              if (!(dbg & 2) && !((dbg & 64) && term > 0))
                tc_mma_ts((dbg & 128) ? (acc ^ ((uint32_t)(kk & 1) << 6)) : acc, a_col, bd, idesc, (term | p | kk) ? 1u : 0u);
            }
          }
        }
        tc_commit(bar(A_EMPTY + grp));
        tc_commit(bar(ACC_FULL + grp));
      }
      if (!ok && i >= 2 + grp) {
        // aborting: the MMAs already issued must retire before TMEM is freed
        const int j = i - 2;
        const unsigned long long t0 = gtime_ns();
        while (!mbar_try(bar(ACC_FULL + grp), (uint32_t)(j >> 1) & 1u))
          if (gtime_ns() - t0 > kWaitLimitNs) break;
      }
    }
  } else if (warp == 3) {
    // spare warp (keeps the role warps aligned to the four TMEM lane quadrants)
  } else if (warp < 12) {
    // ------------------------------ converters --------------------------------
    // two groups of four warps; group g serves the tiles with i % 2 == g, i.e. A buffer g
    const int grp = (warp - 4) >> 2;
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    const uint32_t a_hi = tmem_base + lane_addr + 256u + (uint32_t)grp * 128u;
    bool ok = true;
    int i = grp;
    for (int tile = blockIdx.x + grp * gridDim.x; tile < n_tiles && ok; tile += 2 * gridDim.x, i += 2) {
      const int s = i % kStages;
      const uint32_t ph = (uint32_t)(i / kStages) & 1u;
      const uint32_t phb = (uint32_t)(i >> 1) & 1u;
      ok = mbar_wait(bar(FULL + s), ph, abort_flag, 5);
      if (ok && i >= 2) ok = mbar_wait(bar(A_EMPTY + grp), phb ^ 1u, abort_flag, 6);
      ok = __all_sync(0xffffffffu, ok);  // the tcgen05.st below needs the whole warp
      if (!ok) break;
      tc_fence_after();
      const uint8_t* stage = sm + off_stage + s * stage_bytes;
      float xn = 0.0f;
#pragma unroll
      for (int p = 0; p < P; ++p) {
        const uint8_t* rowp = stage + p * 16384 + row * 128;
        float4 xv[8];
#pragma unroll
        for (int c = 0; c < 8; ++c)
          xv[c] = (dbg & 32) ? make_float4(1.f, 2.f, 3.f, 4.f)
                             : *reinterpret_cast<const float4*>(rowp + ((c ^ (row & 7)) << 4));
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t hi[16], lo[16];
#pragma unroll
          for (int cc = 0; cc < 4; ++cc) {
            const float4 x = xv[half * 4 + cc];
            const float xs[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const uint32_t bits = __float_as_uint(xs[e]);
              const float h = __uint_as_float(bits & 0xffffe000u);
              xn = fmaf(xs[e], xs[e], xn);
              hi[cc * 4 + e] = bits;
              lo[cc * 4 + e] = __float_as_uint(tf32_rn(xs[e] - h));
            }
          }
          if (!(dbg & 8)) {
            tmem_st16(a_hi + p * 32u + half * 16u, hi);
            tmem_st16(a_hi + 64u + p * 32u + half * 16u, lo);
          } else if (hi[3] == 0x12345u && lo[7] == 0x54321u) {
            labels[0] = 0;  // keeps the loads alive
          }
        }
      }
      xn_s[grp * kBM + row] = xn;
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(bar(EMPTY + s));
      mbar_arrive(bar(A_READY + grp));
    }
  } else {
    // ------------------------------ epilogue ----------------------------------
    // two groups of four warps; group g drains accumulator g
    const int grp = (warp - 12) >> 2;
    const int q = warp & 3;
    const int row_in_tile = q * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    const uint32_t acc = tmem_base + lane_addr + (uint32_t)grp * 128u;
    const float kInf = __int_as_float(0x7f800000);
    unsigned int changed = 0;
    bool ok = true;
    int i = grp;
    for (int tile = blockIdx.x + grp * gridDim.x; tile < n_tiles && ok; tile += 2 * gridDim.x, i += 2) {
      const uint32_t phb = (uint32_t)(i >> 1) & 1u;
      // the previous label is only needed for the change count at the very end: fetch
      // it now so that its DRAM round trip hides behind the wait and the arithmetic
      const size_t row = (size_t)tile * kBM + row_in_tile;
      int old_label = -1;
      if (count_changes && row < n) old_label = labels[row];
      ok = mbar_wait(bar(ACC_FULL + grp), phb, abort_flag, 7);
      ok = __all_sync(0xffffffffu, ok);  // the tcgen05.ld below needs the whole warp
      if (!ok) break;
      tc_fence_after();
      // four interleaved (best, second, index) chains keep the compare/select
      // dependency short; chain q sees columns j with j % 4 == q in ascending order
      float bst[4] = {kInf, kInf, kInf, kInf}, sec[4] = {kInf, kInf, kInf, kInf};
      int bix[4] = {0, 0, 0, 0};
      // The load of chunk ch+1 is issued before the arithmetic on chunk ch, so its
      // latency overlaps the compare/select work (tcgen05.wait::ld waits for all loads
      // in flight, hence "wait, issue next, compute").
      uint32_t va[32], vb[32];
      if (!(dbg & 4)) {
        tmem_ld16(acc, va, 0);
        if (16 < npad) tmem_ld16(acc + 16, va, 16);
      }
#pragma unroll
      for (int ch = 0; ch < kMaxNPad / 32; ++ch) {
        const int c0 = ch * 32;  // compile-time after unrolling: column indices are immediates
        if (c0 < npad && !(dbg & 4)) {
          uint32_t(&v)[32] = (ch & 1) ? vb : va;
          uint32_t(&vn)[32] = (ch & 1) ? va : vb;
          const bool two = (c0 + 16 < npad);
          tmem_wait_ld(v);
          if (c0 + 32 < npad) {
            tmem_ld16(acc + c0 + 32, vn, 0);
            if (c0 + 48 < npad) tmem_ld16(acc + c0 + 48, vn, 16);
          }
#pragma unroll
          for (int j4 = 0; j4 < 8; ++j4) {
            if (j4 < 4 || two) {
              const float4 cn4 = *reinterpret_cast<const float4*>(cn_s + c0 + j4 * 4);
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
        }
      }
      const float xn = xn_s[grp * kBM + row_in_tile];
      tc_fence_before();
      mbar_arrive(bar(ACC_EMPTY + grp));
      float best = bst[0], second = sec[0];
      int bidx = bix[0];
#pragma unroll
      for (int qq = 1; qq < 4; ++qq) {
        if (bst[qq] < best || (bst[qq] == best && bix[qq] < bidx)) {
          second = fminf(second, best);
          best = bst[qq];
          bidx = bix[qq];
        } else {
          second = fminf(second, bst[qq]);
        }
        second = fminf(second, sec[qq]);
      }
      if (row < n && !(dbg & 16)) {
        // rows whose two best scores are closer than the error bound of the 3xTF32
        // product are left to the exact re-evaluation pass
        const float tol = tol_rel * (xn + cn_max);
        if (amb_rows != nullptr && !(second - best > tol)) {
          const unsigned int pos = atomicAdd(&st->amb_count, 1u);
          amb_rows[pos] = (unsigned int)row;
        } else {
          changed += (old_label != bidx);
          labels[row] = bidx;
        }
      }
    }
    if (count_changes) {
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

}  // namespace tc
}  // namespace km
