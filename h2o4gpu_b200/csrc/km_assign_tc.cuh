// Tensor-core distance + argmin kernel for sm_100a (tcgen05 / TMEM / TMA).
//
// Scores |c|^2 - 2 x.c for a 128-row tile of X against all centroids are formed
// on the 5th-generation tensor cores as a three-term split product so that fp32
// accuracy is kept:
//      x * Sx = xh + xl,   -2c * Sb = bh + bl      (Sx, Sb powers of two)
//      acc    = xh.bh + xl.bh + xh.bl              (fp32 accumulation in TMEM)
// where every half is an IEEE half-precision number (11 significant bits, the
// same as TF32): products of two halves are exact in fp32, so the split loses
// only xl.bl (2^-22 relative) and the rounding of the low halves (2^-23).  The
// power-of-two scales keep every operand inside the fp16 range; they cancel in
// the comparison because |c|^2 is scaled by the same Sx*Sb.  Using kind::f16
// (K = 16 per instruction) instead of kind::tf32 (K = 8) halves the number of
// MMA instructions per tile (3 * d/16), which matters because for N = 112 the
// tensor pipe is bound by a per-instruction cost, not by N.  Every accumulator is
// handed to the MMAs already holding |c_j|^2 in column j, so the finished score is
// what the epilogue reads, and the rows x k distance matrix never exists.  Replaces calculate_distances + relabel
// (src/gpu/kmeans/kmeans_labels.cu:115-244, kmeans_labels.h:360-392) for
// float32, d in {32, 64}, 16 < k <= 128.
//
// Persistent CTAs (one per SM), warp-specialised:
//   warp 0      TMA producer: raw fp32 X tiles (128 x d, 128B-swizzled panels of
//               32 columns) into a 5-stage shared-memory ring; the split centroid
//               table (bh, bl; fp16, one swizzled panel each) is loaded once per
//               CTA and stays resident.
//   warps 4-11  converters (two groups of four, alternating tiles): thread r
//               reads row r of the tile (conflict-free thanks to the swizzle),
//               splits it and writes packed xh / xl into TMEM with tcgen05.st -
//               the A operand of the MMA lives in TMEM, so the tensor core reads
//               only the centroid panels from shared memory.
//   warps 1-2   MMA issuers, one per A buffer: 3 * d/16 tcgen05.mma.kind::f16
//               (M=128, N=kpad, K=16) per tile into one of three TMEM
//               accumulators; tcgen05.commit releases the A buffer and publishes
//               the accumulator.
//   warps 12-23 epilogue (three groups of four, one per accumulator), two passes of
//               tcgen05.ld over the row: the minimum (three-input min, half an
//               instruction per column), then one bit per column whose score lies
//               within the error bound of it (compare + predicated OR).  One bit:
//               that column is the label; more: the row goes to the exact
//               re-evaluation list.  The group then refills the accumulator with
//               the norms (tcgen05.st) and releases it.
// Every mbarrier wait is bounded; on a timeout the CTA sets an error word, drains
// its copies, frees its TMEM and returns.
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>

#include "km_common.cuh"

namespace km {
namespace tc {

constexpr int kBM = 128;
constexpr int kThreads = 768;  // producer, 2 MMA issuers, spare, 2 x 4 converter warps, 3 x 4 epilogue warps
constexpr int kStages = 5;
constexpr int kAcc = 3;        // TMEM accumulators
constexpr int kMaxD = 64;
constexpr int kMaxNPad = 128;
constexpr int kTmemCols = 512;

enum Bar { FULL = 0, EMPTY = kStages, A_READY = 2 * kStages, A_EMPTY = 2 * kStages + 2,
           ACC_FULL = 2 * kStages + 4, ACC_EMPTY = 2 * kStages + 4 + kAcc, B_FULL = 2 * kStages + 4 + 2 * kAcc,
           NUM_BARS = 2 * kStages + 5 + 2 * kAcc };

// shared memory: [bh panel][bl panel][stages][cn][barriers][misc]; d is 32 or 64
inline size_t smem_bytes(int d, int npad) {
  size_t P = d / 32;
  return 1024 + 2 * (size_t)npad * 128 + (size_t)kStages * P * 16384 + (size_t)npad * 4 + NUM_BARS * 8 + 64;
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
// Bounded wait.  Returns false when the CTA is aborting (this wait or another one
// gave up); the caller leaves its loop.  The poll is mbarrier.try_wait without a suspend-time
// hint: the hardware parks the warp for a short, implementation-defined time and wakes it when
// the phase completes.  With a 20 us hint the wake-up was slow enough to cost the streamed-table
// kernel a tenth of its time (accumulator hand-overs between the issuer and the epilogue warps are
// on its critical path); spinning on test_wait instead took issue slots from the working warps.
// Where the waits of an aborting CTA stood, one record per wait site (code): CTA, the
// caller's tile counter, the parity waited for, 1 = this wait gave up / 2 = it saw the abort.
// Read back by the host only to word the error message.
__device__ int g_wait_diag[16][4];

__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code,
                                          int info = -1) {
  // the limit (150000 units of 20 us by default: gives up after about 3 s) sits in the CTA's shared
  // memory behind the abort word, written by the kernel's first thread
  int why = 1;
  // The limit (units of 20 us, kmeans_set_wait_limits) is measured on the SM's own cycle counter
  // (at most 2 GHz: 40,000 cycles per unit) every 32 polls, and a wait only gives up after a minimum
  // number of polls as well (40 per unit: a tenth of the limit even if a poll took only 50 ns), so
  // that a single odd timer reading cannot end a wait that has barely begun.
  if (mbar_try(bar, parity)) return true;
  const unsigned int units = (unsigned int)abort_flag[3];
  const long long lim_cycles = (long long)units * 40000ll;
  const unsigned int min_polls = units < 0x1ffffffu ? units * 40u : 0x7ffffff0u;
  const long long c0 = clock64();
  for (unsigned int it = 0; it < 0x7fffffffu; ++it) {
    if (mbar_try(bar, parity)) return true;
    if ((it & 31u) == 31u) {
      if (*abort_flag) { why = 2; break; }
      if (it > min_polls && clock64() - c0 > lim_cycles) break;
    }
  }
  if (why == 1) *abort_flag = code;
  g_wait_diag[code & 15][0] = (int)blockIdx.x;
  g_wait_diag[code & 15][1] = info;
  g_wait_diag[code & 15][2] = (int)parity;
  g_wait_diag[code & 15][3] = why;
  return false;
}

// Wait of an aborting CTA for work it has already issued (TMA copies, MMAs) to land: that work signals
// the barrier on its own, so this only returns early after about two seconds of SM cycles.
__device__ __forceinline__ void mbar_drain(uint32_t bar, uint32_t parity) {
  const long long c0 = clock64();
  for (unsigned int it = 0; it < 0x7fffffffu; ++it) {
    if (mbar_try(bar, parity)) return;
    if ((it & 1023u) == 1023u && it > 4000000u && clock64() - c0 > 4000000000ll) return;
  }
}

// One warp waits on an mbarrier that nothing ever arrives at: the give-up path of mbar_wait,
// run on its own (kmeans_selftest_wait_timeout).  The wait returns false after `wait_iters` parked
// polls, the error word takes the wait's code, the kernel ends normally.
__global__ void mbar_timeout_probe_kernel(int* error_word, unsigned int wait_iters) {
  __shared__ __align__(8) unsigned long long bar_mem;
  __shared__ int abort_words[4];
  if (threadIdx.x == 0) {
    abort_words[0] = 0;
    abort_words[3] = (int)wait_iters;
    mbar_init((uint32_t)__cvta_generic_to_shared(&bar_mem), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const bool ok = mbar_wait((uint32_t)__cvta_generic_to_shared(&bar_mem), 0, abort_words, 9, 0);
    if (!ok) atomicMax(error_word, abort_words[0]);
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

// D[tmem] (+)= A[tmem] * B[smem desc], kind::f16 (fp16 inputs, fp32 accumulate), M=128, K=16
__device__ __forceinline__ void tc_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// the same with A from shared memory (descriptor)
__device__ __forceinline__ void tc_mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
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
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
        "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
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
// three-input minimum (one instruction on sm_100)
__device__ __forceinline__ float fmin3(float a, float b, float c) {
  float d;
  asm("min.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Bound on the error of the difference of two scores of one row, in the scaled units of the
// accumulator (scores carry the factor sx * sb).  Two parts:
//  * relative: tol_rel * (|x|^2 + max|c|^2) covers the dropped xl.bl term, the 11-bit rounding of
//    the low halves and the fp32 accumulation;
//  * absolute: a low half whose magnitude falls below fp16's smallest normal number (2^-14) is a
//    subnormal with a fixed quantum of 2^-24, so an element of x * sx (or of -2c * sb) is only
//    known to 2^-25 whatever its size; the product error is then at most
//    2^-25 * (|y|_1 + |b|_1) per score with y = x * sx, b = -2c * sb, and
//    |y|_1 <= sqrt(d) * sx * |x|, |b|_1 <= sqrt(d) * 2 sb * max|c|.  tol_floor = 2^-23 sqrt(d)
//    (two scores, and a factor two of margin).  This term matters only when the data spans many
//    orders of magnitude (an element 1e5 times the typical one); it then widens the band of rows
//    handed to the exact pass instead of letting a wrong label through.
__device__ __forceinline__ float split_tolerance(float tol_rel, float tol_floor, float xn, float cn_max, float sx,
                                                 float sxsb) {
  const float sb2 = 2.0f * sxsb / sx;
  return tol_rel * (xn + cn_max) * sxsb + tol_floor * (sx * sqrtf(xn) + sb2 * sqrtf(cn_max));
}

// |x|^2 of every row (float), once per upload: the error bound of a row's scores.  The
// tensor-core paths have d % 4 == 0 and 16-byte aligned rows: a row is shared by lpr lanes
// loading a float4 each, four sets of rows per loop trip.
__global__ void __launch_bounds__(256)
rownorm_kernel(const float* __restrict__ X, size_t n, int d, float* __restrict__ xn) {
  constexpr int U = 8;
  const int lane = threadIdx.x & 31;
  const size_t warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const size_t nwarp = ((size_t)gridDim.x * blockDim.x) >> 5;
  const int dv = d >> 2;
  int lpr = 1;
  while (lpr < dv && lpr < 32) lpr <<= 1;
  const int gpw = 32 / lpr;
  const int g = lane / lpr, l = lane % lpr;
  const size_t stride = nwarp * gpw;
  for (size_t base = warp * gpw * U; base < n; base += stride * U) {
    float s[U];
    if (dv <= 32) {
      // one float4 per lane and row: all of them requested before any arithmetic
      float4 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const size_t row = base + (size_t)u * gpw + g;
        v[u] = (row < n && l < dv) ? reinterpret_cast<const float4*>(X + row * (size_t)d)[l] : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int u = 0; u < U; ++u)
        s[u] = fmaf(v[u].x, v[u].x, fmaf(v[u].y, v[u].y, fmaf(v[u].z, v[u].z, v[u].w * v[u].w)));
    } else {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        s[u] = 0.f;
        const size_t row = base + (size_t)u * gpw + g;
        if (row < n) {
          const float4* x = reinterpret_cast<const float4*>(X + row * (size_t)d);
          for (int idx = l; idx < dv; idx += lpr) {
            const float4 v = x[idx];
            s[u] = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, s[u]))));
          }
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      for (int o = lpr >> 1; o > 0; o >>= 1) s[u] += __shfl_xor_sync(0xffffffffu, s[u], o);
      const size_t row = base + (size_t)u * gpw + g;
      if (l == 0 && row < n) xn[row] = s[u];
    }
  }
}

// Split centroid table: bh/bl = fp16 halves of (-2 c * sb), one row of 64 halves per
// centroid (columns >= d and rows >= k zero); cn_pad[j] = |c_j|^2 * sx * sb, +inf for
// padding rows; cn_pad[npad] = max_j |c_j|^2 (unscaled; zeroed before the launch).
__global__ void __launch_bounds__(64)
prep_kernel(const float* __restrict__ C, const float* __restrict__ cnorm, int k, int d, int npad, float sb,
            float sxsb, __half* __restrict__ bhi, __half* __restrict__ blo, float* __restrict__ cn_pad) {
  const int j = blockIdx.x;
  const int t = threadIdx.x;  // 64 threads = 64 columns
  float v = (j < k && t < d) ? -2.0f * C[(size_t)j * d + t] * sb : 0.0f;
  const __half h = __float2half_rn(v);
  bhi[(size_t)j * 64 + t] = h;
  blo[(size_t)j * 64 + t] = __float2half_rn(v - __half2float(h));
  if (t == 0) {
    cn_pad[j] = (j < k) ? cnorm[j] * sxsb : __int_as_float(0x7f800000);
    // non-negative floats order as ints
    if (j < k) atomicMax(reinterpret_cast<int*>(cn_pad + npad), __float_as_int(cnorm[j]));
  }
}

// The rows of X split once into the two fp16 operands of the product (the arithmetic of the
// converter warps below: y = x * sx, upper half = fp16(y), lower half = fp16(y - upper)), so that
// the E-step can read them with TMA straight into the layout the MMA consumes and needs no
// conversion per iteration.  Same bytes per element as the float32 matrix (2 + 2).
__global__ void __launch_bounds__(256)
split_rows_kernel(const float* __restrict__ X, size_t count, float sx, __half* __restrict__ xh,
                  __half* __restrict__ xl) {
  const size_t nvec = count / 8;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (size_t)gridDim.x * blockDim.x) {
    const float4 a = __ldcs(reinterpret_cast<const float4*>(X) + 2 * i);
    const float4 b = __ldcs(reinterpret_cast<const float4*>(X) + 2 * i + 1);
    const float y[8] = {a.x * sx, a.y * sx, a.z * sx, a.w * sx, b.x * sx, b.y * sx, b.z * sx, b.w * sx};
    uint32_t hi[4], lo[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const __half2 h = __floats2half2_rn(y[2 * c], y[2 * c + 1]);
      const float2 f = __half22float2(h);
      const __half2 l = __floats2half2_rn(y[2 * c] - f.x, y[2 * c + 1] - f.y);
      hi[c] = *reinterpret_cast<const uint32_t*>(&h);
      lo[c] = *reinterpret_cast<const uint32_t*>(&l);
    }
    reinterpret_cast<uint4*>(xh)[i] = make_uint4(hi[0], hi[1], hi[2], hi[3]);
    reinterpret_cast<uint4*>(xl)[i] = make_uint4(lo[0], lo[1], lo[2], lo[3]);
  }
}

template <int D, bool PRE>
__global__ void __launch_bounds__(kThreads, 1)
assign_tc_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmXl,
                 const __grid_constant__ CUtensorMap tmBhi,
                 const __grid_constant__ CUtensorMap tmBlo, const float* __restrict__ cn_pad,
                 const float* __restrict__ xnorm, int* __restrict__ labels, size_t n, int n_tiles, int npad,
                 IterState* st, int count_changes, unsigned int* __restrict__ amb_rows, float tol_rel, float tol_floor,
                 float sx, float sxsb, unsigned int* __restrict__ moved_bits, uint4* __restrict__ amb_near,
                 unsigned int wait_iters) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_u32 = smem_u32(smem_raw);
  const uint32_t base = (raw_u32 + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - raw_u32);

  constexpr int P = D / 32;    // 32-column fp32 panels per row tile
  constexpr int KS = D / 16;   // K = 16 steps per term
  const uint32_t b_panel = (uint32_t)npad * 128u;       // one fp16 panel: npad rows x 64 halves
  const uint32_t off_blo = b_panel;
  const uint32_t off_stage = 2u * b_panel;
  constexpr uint32_t stage_bytes = (uint32_t)P * 16384u;
  const uint32_t off_cn = off_stage + kStages * stage_bytes;
  const uint32_t off_bar = (off_cn + (uint32_t)npad * 4u + 7u) & ~7u;
  const uint32_t off_misc = off_bar + NUM_BARS * 8;
  float* cn_s = reinterpret_cast<float*>(sm + off_cn);
  volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(sm + off_misc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + off_misc + 4);
  volatile int* issued_upto = reinterpret_cast<volatile int*>(sm + off_misc + 8);  // [2]: last tile counter issued by each issuer
  auto bar = [&](int i) { return base + off_bar + (uint32_t)i * 8u; };

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(bar(FULL + s), 1); mbar_init(bar(EMPTY + s), PRE ? 1 : 128); }
    for (int b = 0; b < 2; ++b) { mbar_init(bar(A_READY + b), 128); mbar_init(bar(A_EMPTY + b), 1); }
    for (int a = 0; a < kAcc; ++a) { mbar_init(bar(ACC_FULL + a), 1); mbar_init(bar(ACC_EMPTY + a), 128); }
    mbar_init(bar(B_FULL), 1);
    *abort_flag = 0;
    abort_flag[3] = (int)wait_iters;
    issued_upto[0] = -1;
    issued_upto[1] = -1;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  for (int i = tid; i < npad; i += kThreads) cn_s[i] = cn_pad[i];
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
  const float cn_max = cn_pad[npad];  // largest |c|^2 (unscaled), stored behind the padded table
  // TMEM columns: accumulators at 0, 128, 256; A buffer b at 384 + 64 b: xh in 32 columns
  // (two halves per column), xl in the next 32
  constexpr uint32_t kACol = 384u;
  // instruction descriptor: D = f32, A = B = f16, K-major, N = npad, M = 128
  const uint32_t idesc = (1u << 4) | ((uint32_t)(npad >> 3) << 17) | ((128u >> 4) << 24);

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      mbar_expect_tx(bar(B_FULL), 2u * b_panel);
      tma_load_2d(base, &tmBhi, 0, 0, bar(B_FULL));
      tma_load_2d(base + off_blo, &tmBlo, 0, 0, bar(B_FULL));
      int i = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++i) {
        const int s = i % kStages;
        const uint32_t ph = (uint32_t)(i / kStages) & 1u;
        if (i >= kStages) ok = mbar_wait(bar(EMPTY + s), ph ^ 1u, abort_flag, 1, i);
        if (!ok) break;
        mbar_expect_tx(bar(FULL + s), stage_bytes);
        if (PRE) {
          // the row tile arrives split already: upper halves, then lower halves, each 128 rows x 64 halves in
          // the layout the MMA reads
          tma_load_2d(base + off_stage + s * stage_bytes, &tmX, 0, tile * kBM, bar(FULL + s));
          tma_load_2d(base + off_stage + s * stage_bytes + 16384u, &tmXl, 0, tile * kBM, bar(FULL + s));
        } else {
#pragma unroll
          for (int p = 0; p < P; ++p)
            tma_load_2d(base + off_stage + s * stage_bytes + p * 16384u, &tmX, p * 32, tile * kBM, bar(FULL + s));
        }
      }
      if (!ok) {
        // aborting: let the copies already issued land before the CTA exits
        mbar_wait(bar(B_FULL), 0, abort_flag, 0);
        const int lo = (i > kStages) ? i - kStages : 0;
        for (int j = lo; j < i; ++j) {
          mbar_drain(bar(FULL + j % kStages), (uint32_t)(j / kStages) & 1u);
        }
      }
    }
  } else if (warp == 1 || warp == 2) {
    // ------------------------------ MMA issuers -------------------------------
    // Two issuing threads on two schedulers, one per A buffer: a single thread's
    // issue rate (about ten scalar instructions per MMA) would otherwise cap the
    // tensor pipe for these short MMAs.
    const int grp = warp - 1;
    if (lane == 0) {
      bool ok = mbar_wait(bar(B_FULL), 0, abort_flag, 2);
      // the centroid panels never move: one shared-memory descriptor per k-step
      uint64_t bdesc_hi[KS], bdesc_lo[KS];
#pragma unroll
      for (int kk = 0; kk < KS; ++kk) {
        bdesc_hi[kk] = smem_desc_sw128(base + kk * 32u);
        bdesc_lo[kk] = smem_desc_sw128(base + off_blo + kk * 32u);
      }
      const uint32_t a_hi = tmem_base + kACol + (uint32_t)grp * 64u;
      int i = grp;
      int last_acc = 0;
      uint32_t last_ph = 0;
      for (int tile = blockIdx.x + grp * gridDim.x; tile < n_tiles && ok; tile += 2 * gridDim.x, i += 2) {
        const uint32_t phb = (uint32_t)(i >> 1) & 1u;
        const int a = i % kAcc;
        const uint32_t pha = (uint32_t)(i / kAcc) & 1u;
        const int s = i % kStages;
        if (PRE) ok = mbar_wait(bar(FULL + s), (uint32_t)(i / kStages) & 1u, abort_flag, 3, i);
        else ok = mbar_wait(bar(A_READY + grp), phb, abort_flag, 3, i);
        // Consecutive uses of an accumulator (tile counters i - 3 and i) belong to different
        // issuers, and a parity wait cannot tell "two phases behind" from "done": an issuer
        // that ran ahead of the other (a slow epilogue group is enough) could take the
        // accumulator one use early.  So the previous use must have been issued first.
        for (unsigned int spins = 0; ok && issued_upto[grp ^ 1] < i - 3; ++spins) {
          if (*abort_flag) ok = false;
          else if (spins > 40000000u) { *abort_flag = 8; ok = false; }
          else __nanosleep(32);
        }
        // phase u of ACC_EMPTY completes when the accumulator holds |c|^2 again: after the
        // epilogue's initial fill (u = 0) or after it has consumed use u - 1
        if (ok) ok = mbar_wait(bar(ACC_EMPTY + a), pha, abort_flag, 4, i);
        if (!ok) break;
        tc_fence_after();
        const uint32_t acc = tmem_base + (uint32_t)a * 128u;
#pragma unroll
        for (int term = 0; term < 3; ++term) {
#pragma unroll
          for (int kk = 0; kk < KS; ++kk) {
            const uint32_t a_col = a_hi + (term == 1 ? 32u : 0u) + kk * 8u;
            const uint64_t bd = (term == 2) ? bdesc_lo[kk] : bdesc_hi[kk];
            if (PRE) {
              const uint32_t a_smem = base + off_stage + (uint32_t)s * stage_bytes + (term == 1 ? 16384u : 0u) + kk * 32u;
              tc_mma_ss(acc, smem_desc_sw128(a_smem), bd, idesc, 1u);
            } else {
              tc_mma_ts(acc, a_col, bd, idesc, 1u);
            }
          }
        }
        tc_commit(bar(PRE ? EMPTY + s : A_EMPTY + grp));
        tc_commit(bar(ACC_FULL + a));
        __threadfence_block();
        issued_upto[grp] = i;
        last_acc = a;
        last_ph = pha;
      }
      if (!ok && i >= 2 + grp) {
        // aborting: the MMAs already issued must retire before TMEM is freed
        mbar_drain(bar(ACC_FULL + last_acc), last_ph);
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
    const uint32_t a_hi = tmem_base + lane_addr + kACol + (uint32_t)grp * 64u;
    bool ok = true;
    int i = grp;
    // (nothing to convert when the rows arrive split)
    for (int tile = blockIdx.x + grp * gridDim.x; !PRE && tile < n_tiles && ok; tile += 2 * gridDim.x, i += 2) {
      const int s = i % kStages;
      const uint32_t ph = (uint32_t)(i / kStages) & 1u;
      const uint32_t phb = (uint32_t)(i >> 1) & 1u;
      // The A buffer first: its release (MMAs of this group's tile i - 2 retired) implies that tile i - 5,
      // the previous user of this stage and a tile of the OTHER group, has been consumed, so the stage's
      // barrier has left that phase - a one-bit parity could not tell it from the one waited for here.
      if (i >= 2) ok = mbar_wait(bar(A_EMPTY + grp), phb ^ 1u, abort_flag, 6, i);
      if (ok) ok = mbar_wait(bar(FULL + s), ph, abort_flag, 5, i);
      ok = __all_sync(0xffffffffu, ok);  // the tcgen05.st below needs the whole warp
      if (!ok) break;
      tc_fence_after();
      const uint8_t* stage = sm + off_stage + s * stage_bytes;
#pragma unroll
      for (int p = 0; p < P; ++p) {
        const uint8_t* rowp = stage + p * 16384 + row * 128;
        float4 xv[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) xv[c] = *reinterpret_cast<const float4*>(rowp + ((c ^ (row & 7)) << 4));
        // 32 floats -> 16 words of packed xh pairs and 16 words of packed xl pairs
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
        tmem_st16(a_hi + p * 16u, hi);
        tmem_st16(a_hi + 32u + p * 16u, lo);
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(bar(EMPTY + s));
      mbar_arrive(bar(A_READY + grp));
    }
  } else {
    // ------------------------------ epilogue ----------------------------------
    // three groups of four warps; group g owns accumulator g and takes the tiles with i % 3 == g
    const int grp = (warp - 12) >> 2;
    const int q = warp & 3;
    const int row_in_tile = q * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    unsigned int changed = 0;
    bool ok = true;
    // The accumulator starts every tile holding |c_j|^2 (scaled) in column j of every row, so
    // the MMAs leave the finished score there and the epilogue never adds the norms itself.
    auto fill_norms = [&](uint32_t acc) {
#pragma unroll
      for (int c0 = 0; c0 < kMaxNPad; c0 += 16) {
        if (c0 < npad) {
          uint32_t c[16];
#pragma unroll
          for (int j4 = 0; j4 < 4; ++j4) {
            const uint4 q4 = *reinterpret_cast<const uint4*>(cn_s + c0 + j4 * 4);
            c[j4 * 4 + 0] = q4.x; c[j4 * 4 + 1] = q4.y; c[j4 * 4 + 2] = q4.z; c[j4 * 4 + 3] = q4.w;
          }
          tmem_st16(acc + c0, c);
        }
      }
      tmem_wait_st();
    };
    fill_norms(tmem_base + lane_addr + (uint32_t)grp * 128u);
    tc_fence_before();
    mbar_arrive(bar(ACC_EMPTY + grp));
    int i = grp;
    for (int tile = blockIdx.x + grp * gridDim.x; tile < n_tiles && ok; tile += kAcc * gridDim.x, i += kAcc) {
      const int a = grp;
      const uint32_t pha = (uint32_t)(i / kAcc) & 1u;
      // the previous label and |x|^2 are only needed at the very end: fetch them now so
      // that their DRAM round trip hides behind the wait and the arithmetic
      const size_t row = (size_t)tile * kBM + row_in_tile;
      int old_label = -1;
      float xn = 0.f;
      if (row < n) {
        xn = xnorm[row];
        if (count_changes) old_label = labels[row];
      }
      ok = mbar_wait(bar(ACC_FULL + a), pha, abort_flag, 7, i);
      ok = __all_sync(0xffffffffu, ok);  // the tcgen05.ld below needs the whole warp
      if (!ok) break;
      tc_fence_after();
      const uint32_t acc = tmem_base + lane_addr + (uint32_t)a * 128u;
      // pass 1: the smallest score of the row, two three-input minima per four columns
      float m0 = __int_as_float(0x7f800000), m1 = m0;
#pragma unroll
      for (int ch = 0; ch < kMaxNPad / 32; ++ch) {
        const int c0 = ch * 32;
        if (c0 < npad) {
          uint32_t v[32];
          const bool two = (c0 + 16 < npad);
          tmem_ld16(acc + c0, v, 0);
          if (two) tmem_ld16(acc + c0 + 16, v, 16);
          tmem_wait_ld(v);
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            if (j < 16 || two) {
              m0 = fmin3(m0, __uint_as_float(v[j]), __uint_as_float(v[j + 1]));
              m1 = fmin3(m1, __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
            }
          }
        }
      }
      const float best = fminf(m0, m1);
      // rows with a second score within the error bound of the split product (scores carry the
      // factor sx*sb) go to the exact re-evaluation pass; without that pass only exact ties count
      const float tol = (amb_rows != nullptr) ? split_tolerance(tol_rel, tol_floor, xn, cn_max, sx, sxsb) : 0.f;
      const float thr = best + tol;
      // pass 2: one bit per column whose score is within the bound of the best
      uint32_t near[kMaxNPad / 32];
#pragma unroll
      for (int ch = 0; ch < kMaxNPad / 32; ++ch) {
        const int c0 = ch * 32;
        uint32_t mk = 0;
        if (c0 < npad) {
          uint32_t v[32];
          const bool two = (c0 + 16 < npad);
          tmem_ld16(acc + c0, v, 0);
          if (two) tmem_ld16(acc + c0 + 16, v, 16);
          tmem_wait_ld(v);
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if ((j < 16 || two) && __uint_as_float(v[j]) <= thr) mk |= (1u << j);
        }
        near[ch] = mk;
      }
      // hand the accumulator back with the norms in place
      fill_norms(acc);
      tc_fence_before();
      mbar_arrive(bar(ACC_EMPTY + a));
      int n_near = 0, bidx = 0;
#pragma unroll
      for (int ch = kMaxNPad / 32 - 1; ch >= 0; --ch) {
        n_near += __popc(near[ch]);
        if (near[ch]) bidx = ch * 32 + __ffs(near[ch]) - 1;   // lowest column wins
      }
      bool moved = false;
      if (row < n) {
        if (amb_rows != nullptr && n_near != 1) {
          const unsigned int pos = atomicAdd(&st->amb_count, 1u);
          amb_rows[pos] = (unsigned int)row;
          amb_near[pos] = make_uint4(near[0], near[1], near[2], near[3]);   // the candidates of the exact pass
        } else {
          moved = (old_label != bidx);
          changed += moved;
          labels[row] = bidx;
        }
      }
      // one bit per row whose label moved (the warp's 32 rows are one word): the incremental
      // M-step reads this map instead of comparing two label arrays.  Rows left to the exact
      // pass get their bit there.
      if (moved_bits != nullptr) {
        const unsigned int word = __ballot_sync(0xffffffffu, moved);
        if (lane == 0) moved_bits[(size_t)tile * (kBM / 32) + q] = word;
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
