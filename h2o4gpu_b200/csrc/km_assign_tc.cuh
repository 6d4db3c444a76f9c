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
//   warps 2-9   converters (two groups of four, alternating tiles): thread r reads row r of the tile (conflict-free
//               thanks to the swizzle), splits it and writes xh / xl into TMEM
//               with tcgen05.st - the A operand of the MMA lives in TMEM, so
//               the tensor core reads only the centroid panels from shared memory.
//   warp 1      MMA issuer: 3 * d/8 tcgen05.mma (M=128, N=kpad, K=8) per tile into
//               one of two TMEM accumulators; tcgen05.commit releases the A
//               buffer and publishes the accumulator.
//   warps 10-25 epilogue (two groups of eight, one group per accumulator; two warps share a
//               row block and split the columns): tcgen05.ld, + |c|^2, argmin (first minimum wins),
//               label store, changed-label count.
// Every mbarrier wait is bounded (wall-clock limit); on a timeout the CTA sets an
// error word, drains its copies, frees its TMEM and returns.
#pragma once

#include <cuda.h>

#include "km_common.cuh"

namespace km {
namespace tc {

#ifdef KM_TC_PROFILE
// debug build only: per-CTA clock totals of the waits of each role
__device__ long long g_tc_prof[160][24];
__device__ long long g_tc_trace[64][12];
#define KM_TRACE(ev) do { if (blockIdx.x == 0 && i < 64) g_tc_trace[i][ev] = clock64(); } while (0)
#define KM_PROF_T0() const long long _pt0 = clock64()
#define KM_PROF_ADD(slot) do { if (lane == 0) g_tc_prof[blockIdx.x][slot] += clock64() - _pt0; } while (0)
#ifdef KM_TC_TRACE_ONLY
#define KM_PROF_SCOPE(slot, stmt) do { stmt; } while (0)
#else
#define KM_PROF_SCOPE(slot, stmt) do { const long long _t = clock64(); stmt; if (lane == 0) g_tc_prof[blockIdx.x][slot] += clock64() - _t; } while (0)
#endif
#else
#define KM_PROF_SCOPE(slot, stmt) do { stmt; } while (0)
#define KM_TRACE(ev) do { } while (0)
#endif

constexpr int kBM = 128;
constexpr int kThreads = 832;  // producer, MMA issuer, 2 x 4 converter warps, 2 x 8 epilogue warps
constexpr int kStages = 4;
constexpr int kMaxD = 64;
constexpr int kMaxNPad = 128;
constexpr int kTmemCols = 512;
constexpr unsigned long long kWaitLimitNs = 2000000000ULL;  // 2 s (abort drain loops)
constexpr long long kWaitLimitClk = 6000000000LL;          // about 3 s of SM clocks

enum Bar { FULL = 0, EMPTY = kStages, A_READY = 2 * kStages, A_EMPTY = 2 * kStages + 2,
           ACC_FULL = 2 * kStages + 4, ACC_EMPTY = 2 * kStages + 6, B_FULL = 2 * kStages + 8,
           PART_FULL = 2 * kStages + 9, PART_EMPTY = 2 * kStages + 11, NUM_BARS = 2 * kStages + 13 };

inline size_t smem_bytes(int d, int npad) {
  size_t P = d / 32;
  return 1024 + 2 * P * (size_t)npad * 128 + (size_t)kStages * P * 16384 + (size_t)npad * 4 + 2 * kBM * 4 +
         2 * kBM * 12 + NUM_BARS * 8 + 64;
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
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code) {
  if (mbar_try(bar, parity)) return true;
  // Back off between polls: a spinning warp would otherwise take issue slots from
  // the warps doing the arithmetic on the same scheduler.
  long long t0 = 0;
  for (unsigned int it = 1;; ++it) {
    __nanosleep(it < 64 ? 20 : 100);
    if (mbar_try(bar, parity)) return true;
    if ((it & 4095u) == 0) {
      if (*abort_flag) return false;
      const long long now = clock64();
      if (t0 == 0) t0 = now;
      if (now - t0 > kWaitLimitClk) {
        *abort_flag = code;
        return false;
      }
    }
  }
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

// Both halves of every operand are rounded to TF32 before they reach the tensor
// core, so the result does not depend on how the hardware treats the low 13 bits
// (measured on B200: it ignores them).  mask_hi is kept for experiments.
template <int D>
__global__ void __launch_bounds__(kThreads, 1)
assign_tc_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmBhi,
                 const __grid_constant__ CUtensorMap tmBlo, const float* __restrict__ cnorm_pad,
                 int* __restrict__ labels, size_t n, int n_tiles, int npad, IterState* st,
                 int count_changes, unsigned int* __restrict__ amb_rows, float tol_rel, int mask_hi) {
#ifdef KM_TC_PROFILE
  const long long _kstart = clock64();
#endif
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_u32 = smem_u32(smem_raw);
  const uint32_t base = (raw_u32 + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - raw_u32);

  constexpr int P = D / 32;  // 32-column panels per row tile
  const uint32_t b_panel = (uint32_t)npad * 128u;
  const uint32_t off_blo = (uint32_t)P * b_panel;
  const uint32_t off_stage = 2u * P * b_panel;
  const uint32_t stage_bytes = (uint32_t)P * 16384u;
  const uint32_t off_cn = off_stage + kStages * stage_bytes;
  const uint32_t off_xn = off_cn + (uint32_t)npad * 4u;
  const uint32_t off_part = off_xn + 2u * kBM * 4u;  // [2 groups][3][128] partial argmin of the upper columns
  const uint32_t off_bar = (off_part + 2u * kBM * 12u + 7u) & ~7u;
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
      mbar_init(bar(ACC_EMPTY + b), 256);
      mbar_init(bar(PART_FULL + b), 128);
      mbar_init(bar(PART_EMPTY + b), 128);
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
        if (i >= kStages) KM_PROF_SCOPE(0, ok = mbar_wait(bar(EMPTY + s), ph ^ 1u, abort_flag, 1));
        if (!ok) break;
        mbar_expect_tx(bar(FULL + s), stage_bytes);
        for (int p = 0; p < P; ++p)
          tma_load_2d(base + off_stage + s * stage_bytes + p * 16384u, &tmX, p * 32, tile * kBM, bar(FULL + s));
        KM_TRACE(8);
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
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
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
      int i = 0;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++i) {
        const int b = i & 1;
        const uint32_t phb = (uint32_t)(i >> 1) & 1u;
        KM_PROF_SCOPE(1, ok = mbar_wait(bar(A_READY + b), phb, abort_flag, 3));
        KM_TRACE(2);
        if (ok && i >= 2) KM_PROF_SCOPE(2, ok = mbar_wait(bar(ACC_EMPTY + b), phb ^ 1u, abort_flag, 4));
        KM_TRACE(3);
        if (!ok) break;
        KM_PROF_SCOPE(16, tc_fence_after());
#ifdef KM_TC_PROFILE
        const long long _m0 = clock64();
#endif
        const uint32_t acc = tmem_base + (uint32_t)b * 128u;
        const uint32_t a_hi = tmem_base + 256u + (uint32_t)b * 128u;
        // straight-line issue: descriptors were built once, operand addresses are immediates
#pragma unroll
        for (int term = 0; term < 3; ++term) {
#pragma unroll
          for (int p = 0; p < P; ++p) {
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
              const uint32_t a_col = a_hi + (term == 1 ? 64u : 0u) + p * 32u + kk * 8u;
              const uint64_t bd = (term == 2) ? bdesc_lo[p * 4 + kk] : bdesc_hi[p * 4 + kk];
              if (!(mask_hi & 2)) tc_mma_ts(acc, a_col, bd, idesc, (term | p | kk) ? 1u : 0u);
            }
          }
        }
#ifdef KM_TC_PROFILE
        g_tc_prof[blockIdx.x][17] += clock64() - _m0;
#endif
        KM_PROF_SCOPE(18, tc_commit(bar(A_EMPTY + b)));
        KM_PROF_SCOPE(19, tc_commit(bar(ACC_FULL + b)));
        KM_TRACE(4);
      }
      if (!ok && i > 0) {
        // aborting: the MMAs already issued must retire before TMEM is freed
        const int j = i - 1;
        const unsigned long long t0 = gtime_ns();
        while (!mbar_try(bar(ACC_FULL + (j & 1)), (uint32_t)(j >> 1) & 1u))
          if (gtime_ns() - t0 > kWaitLimitNs) break;
      }
    }
  } else if (warp < 10) {
    // ------------------------------ converters --------------------------------
    // two groups of four warps; group g serves the tiles with i % 2 == g, i.e. A buffer g
    const int grp = (warp - 2) >> 2;
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    bool ok = true;
    int i = 0;
    for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++i) {
      if ((i & 1) != grp) continue;
      const int s = i % kStages;
      const uint32_t ph = (uint32_t)(i / kStages) & 1u;
      const int b = i & 1;
      const uint32_t phb = (uint32_t)(i >> 1) & 1u;
      KM_PROF_SCOPE(3 + grp * 4, ok = mbar_wait(bar(FULL + s), ph, abort_flag, 5));
      if (q == 0 && lane == 0) KM_TRACE(9);
      if (ok && i >= 2) KM_PROF_SCOPE(4 + grp * 4, ok = mbar_wait(bar(A_EMPTY + b), phb ^ 1u, abort_flag, 6));
#ifdef KM_TC_PROFILE
      const long long _cw0 = clock64();
      if (q == 0 && lane == 0) KM_TRACE(0);
#endif
      ok = __all_sync(0xffffffffu, ok);  // the tcgen05.st below needs the whole warp
      if (!ok) break;
      tc_fence_after();
      const uint8_t* stage = sm + off_stage + s * stage_bytes;
      const uint32_t a_hi = tmem_base + lane_addr + 256u + (uint32_t)b * 128u;
      float xn = 0.0f;
#pragma unroll
      for (int p = 0; p < P; ++p) {
        const uint8_t* rowp = stage + p * 16384 + row * 128;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t hi[16], lo[16];
#pragma unroll
          for (int cc = 0; cc < 4; ++cc) {
            const int c = half * 4 + cc;
            const float4 x = *reinterpret_cast<const float4*>(rowp + ((c ^ (row & 7)) << 4));
            const float xs[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float h = tf32_rn(xs[e]);
              xn = fmaf(xs[e], xs[e], xn);
              hi[cc * 4 + e] = __float_as_uint(h);
              lo[cc * 4 + e] = __float_as_uint(tf32_rn(xs[e] - h));
            }
          }
          if (!(mask_hi & 8)) {
            tmem_st16(a_hi + p * 32u + half * 16u, hi);
            tmem_st16(a_hi + 64u + p * 32u + half * 16u, lo);
          } else if (hi[3] == 0x12345u && lo[7] == 0x54321u) {
            labels[0] = 0;  // keeps the loads alive
          }
        }
      }
      xn_s[b * kBM + row] = xn;
#ifdef KM_TC_PROFILE
      if (lane == 0 && q == 0) g_tc_prof[blockIdx.x][5 + grp * 4] += clock64() - _cw0;
#endif
      KM_PROF_SCOPE(6 + grp * 4, tmem_wait_st());
      tc_fence_before();
      if (q == 0 && lane == 0) KM_TRACE(1);
      mbar_arrive(bar(EMPTY + s));
      mbar_arrive(bar(A_READY + b));
    }
  } else {
    // ------------------------------ epilogue ----------------------------------
    // Two groups of eight warps; group g drains accumulator g.  Within a group the
    // warps with hsel = 0 scan columns [0, 64) and those with hsel = 1 the rest; the
    // upper half hands its (best, second, index) to the lower half through shared
    // memory, which finishes the row.
    const int ew = warp - 10;
    const int grp = ew >> 3;
    const int hsel = (ew >> 2) & 1;
    const int q = warp & 3;
    const int row_in_tile = q * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    float* part = reinterpret_cast<float*>(sm + off_part) + grp * 3 * kBM;
    const float kInf = __int_as_float(0x7f800000);
    unsigned int changed = 0;
    bool ok = true;
    int i = 0;
    for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++i) {
      if ((i & 1) != grp) continue;
      const int b = i & 1;
      const uint32_t phb = (uint32_t)(i >> 1) & 1u;
      KM_PROF_SCOPE(11 + grp * 2, ok = mbar_wait(bar(ACC_FULL + b), phb, abort_flag, 7));
#ifdef KM_TC_PROFILE
      const long long _ew0 = clock64();
      if (ew == grp * 8 && lane == 0) KM_TRACE(5);
#endif
      ok = __all_sync(0xffffffffu, ok);  // the tcgen05.ld below needs the whole warp
      if (!ok) break;
      tc_fence_after();
      const uint32_t acc = tmem_base + lane_addr + (uint32_t)b * 128u;
      // four interleaved (best, second, index) chains keep the compare/select
      // dependency short; chain q sees columns j with j % 4 == q in ascending order
      float bst[4] = {kInf, kInf, kInf, kInf}, sec[4] = {kInf, kInf, kInf, kInf};
      int bix[4] = {0, 0, 0, 0};
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        if (hh != hsel) continue;
#pragma unroll
        for (int ch = 0; ch < 2; ++ch) {
          const int c0 = hh * 64 + ch * 32;  // compile-time after unrolling: column indices are immediates
          if (c0 < npad && !(mask_hi & 4)) {
            uint32_t v[32];
            const bool two = (c0 + 16 < npad);
            tmem_ld16(acc + c0, v, 0);
            if (two) tmem_ld16(acc + c0 + 16, v, 16);
            tmem_wait_ld(v);
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
      }
      tc_fence_before();
      if (ew == grp * 8 && lane == 0) KM_TRACE(6);
      mbar_arrive(bar(ACC_EMPTY + b));
#ifdef KM_TC_PROFILE
      if (lane == 0 && ew == grp * 8) g_tc_prof[blockIdx.x][12 + grp * 2] += clock64() - _ew0;
#endif
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
      const uint32_t pht = phb;  // this group's tile counter is i >> 1
      if (hsel == 1) {
        // (bounded waits instead of a named barrier: a warp that aborts must not strand its partners)
        if (i >= 2) ok = mbar_wait(bar(PART_EMPTY + grp), pht ^ 1u, abort_flag, 8);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        part[row_in_tile] = best;
        part[kBM + row_in_tile] = second;
        part[2 * kBM + row_in_tile] = __int_as_float(bidx);
        mbar_arrive(bar(PART_FULL + grp));
      } else {
        ok = mbar_wait(bar(PART_FULL + grp), pht, abort_flag, 9);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        const float ub = part[row_in_tile];
        const float us = part[kBM + row_in_tile];
        const int ui = __float_as_int(part[2 * kBM + row_in_tile]);
        if (ub < best) {  // upper columns have larger indices: they win only when strictly smaller
          second = fminf(best, us);
          best = ub;
          bidx = ui;
        } else {
          second = fminf(second, ub);
        }
        const float xn = xn_s[b * kBM + row_in_tile];
        const size_t row = (size_t)tile * kBM + row_in_tile;
        if (row < n) {
          // rows whose two best scores are closer than the error bound of the 3xTF32
          // product are left to the exact re-evaluation pass
          const float tol = tol_rel * (xn + cn_max);
          if (amb_rows != nullptr && !(second - best > tol)) {
            const unsigned int pos = atomicAdd(&st->amb_count, 1u);
            amb_rows[pos] = (unsigned int)row;
          } else {
            changed += (labels[row] != bidx);
            labels[row] = bidx;
          }
        }
        if (ew == grp * 8 && lane == 0) KM_TRACE(7);
        mbar_arrive(bar(PART_EMPTY + grp));  // `part` has been read
      }
    }
    if (count_changes) {
      changed = __reduce_add_sync(0xffffffffu, changed);
      if (lane == 0 && changed) atomicAdd(&st->changed, (unsigned long long)changed);
    }
  }

  __syncthreads();
#ifdef KM_TC_PROFILE
  if (tid == 0) g_tc_prof[blockIdx.x][15] += clock64() - _kstart;
#endif
  if (tid == 0 && *abort_flag) atomicMax(&st->error, *abort_flag);
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)kTmemCols)
                 : "memory");
  }
}

}  // namespace tc
}  // namespace km
