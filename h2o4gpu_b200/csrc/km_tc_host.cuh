// Host side of the tensor-core distance kernel: eligibility, the split centroid
// buffers, TMA tensor maps (encoded through the driver entry point, so the
// library has no link-time dependency on libcuda) and the launch.
#pragma once

#include "km_assign_tc.cuh"
#include "km_push.cuh"

namespace km {
namespace tc {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// rows x cols row-major matrix of fp32 (elem 4) or fp16 (elem 2), boxes of box_rows rows x
// 128 bytes, 128-byte swizzle
inline int make_map(CUtensorMap* map, const void* base, size_t rows, int cols, int box_rows, int elem) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) KM_FAIL(KM_ECUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t gdim[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t gstride[1] = {(cuuint64_t)cols * elem};
  cuuint32_t box[2] = {(cuuint32_t)(128 / elem), (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1u, 1u};
  CUresult r = fn(map, elem == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                  const_cast<void*>(base), gdim, gstride, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) KM_FAIL(KM_ECUDA, "cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
  return KM_OK;
}

struct Plan {
  __half* bhi = nullptr;   // [npad][64] upper halves of -2 c * sb
  __half* blo = nullptr;   // [npad][64] lower halves
  float* cn = nullptr;     // [npad] |c|^2 * sx * sb (+inf padding), [npad] max |c|^2
  float* xnorm = nullptr;  // [rows] |x|^2
  size_t xnorm_cap = 0;
  const float* xnorm_of = nullptr;
  size_t xnorm_rows = 0;
  int npad = 0, k = 0, d = 0;
  const float* x_base = nullptr;
  size_t x_rows = 0;
  float sx = 1.f, sb = 1.f;
  CUtensorMap tmX, tmBhi, tmBlo;
  bool ready = false;
  // the rows split once into fp16 halves (d = 64): [rows][64] upper, then [rows][64] lower
  __half* xsplit = nullptr;
  size_t xsplit_cap = 0;
  const float* xsplit_of = nullptr;
  size_t xsplit_rows = 0;
  float xsplit_sx = 0.f;
  bool xsplit_failed = false;   // no memory for it: stay with the converting kernel
  CUtensorMap tmXh, tmXl;

  void release() {
    km_free(bhi); km_free(blo); km_free(cn); km_free(xnorm); km_free(xsplit);
    bhi = blo = nullptr;
    cn = xnorm = nullptr;
    xsplit = nullptr;
    xnorm_cap = xsplit_cap = 0;
    xnorm_of = xsplit_of = nullptr;
    ready = false;
  }
};

// Power-of-two scales that put x * sx and 2 c * sb below 2^14 (fp16 overflows at 65504):
// xmax bounds |x|, cbound bounds |c| (centroids are means of rows, or the caller's
// initial table).  Returns false when the magnitudes cannot be scaled into range.
inline bool pick_scales(double xmax, double cbound, float* sx, float* sb) {
  int ex = 0, ec = 0;
  if (xmax > 0) std::frexp(xmax, &ex);
  if (cbound > 0) std::frexp(cbound, &ec);
  const int px = 14 - ex, pb = 13 - ec;
  if (px < -100 || px > 100 || pb < -100 || pb > 100 || px + pb < -120 || px + pb > 120) return false;
  *sx = (float)std::ldexp(1.0, px);
  *sb = (float)std::ldexp(1.0, pb);
  return true;
}

inline bool shape_ok(int k, int d) { return (d == 32 || d == 64) && k > 16 && k <= kMaxNPad; }

// |x|^2 per row, once per attached matrix
inline int ensure_xnorm(Plan& pl, const float* X, size_t rows, int d, int num_sms, cudaStream_t stream) {
  if (pl.xnorm_of != X || pl.xnorm_rows != rows) {
    if (pl.xnorm_cap < rows) {
      km_free(pl.xnorm);
      pl.xnorm = nullptr;
      KM_CUDA(km_malloc(&pl.xnorm, rows * sizeof(float)));
      pl.xnorm_cap = rows;
    }
    rownorm_kernel<<<num_sms * 8, 256, 0, stream>>>(X, rows, d, pl.xnorm);
    KM_CUDA(cudaGetLastError());
    pl.xnorm_of = X;
    pl.xnorm_rows = rows;
  }
  return KM_OK;
}

// The split copy of X for the kernel variant without converter warps (d = 64): made when the
// matrix, its size or the scale changed; costs one pass over X and as much memory again.
inline bool presplit_enabled() {
  static const bool on = [] {
    const char* e = std::getenv("H2O4GPU_KM_TC_PRESPLIT");
    return !(e && e[0] == '0');
  }();
  return on;
}
inline bool ensure_xsplit(Plan& pl, const float* X, size_t rows, int d, float sx, int num_sms, cudaStream_t stream,
                          bool allow_build) {
  if (d != 64 || !presplit_enabled() || pl.xsplit_failed) return false;
  if (pl.xsplit && pl.xsplit_of == X && pl.xsplit_rows == rows && pl.xsplit_sx == sx) return true;
  if (!allow_build) return false;   // a single pass (predict) does not pay for the split
  if (pl.xsplit_cap < rows) {
    km_free(pl.xsplit);
    pl.xsplit = nullptr;
    pl.xsplit_cap = 0;
    if (km_malloc(&pl.xsplit, rows * 64 * 2 * sizeof(__half)) != cudaSuccess) {
      cudaGetLastError();
      pl.xsplit_failed = true;
      return false;
    }
    pl.xsplit_cap = rows;
  }
  __half* xh = pl.xsplit;
  __half* xl = pl.xsplit + rows * 64;
  split_rows_kernel<<<num_sms * 8, 256, 0, stream>>>(X, rows * 64, sx, xh, xl);
  if (cudaGetLastError() != cudaSuccess || make_map(&pl.tmXh, xh, rows, 64, kBM, 2) != KM_OK ||
      make_map(&pl.tmXl, xl, rows, 64, kBM, 2) != KM_OK) {
    pl.xsplit_failed = true;
    return false;
  }
  pl.xsplit_of = X;
  pl.xsplit_rows = rows;
  pl.xsplit_sx = sx;
  return true;
}

inline int setup(Plan& pl, const float* X, size_t rows, int k, int d, int num_sms, cudaStream_t stream) {
  const int npad = (k + 15) / 16 * 16;
  KM_TRY(ensure_xnorm(pl, X, rows, d, num_sms, stream));
  if (pl.ready && pl.k == k && pl.d == d && pl.x_base == X && pl.x_rows == rows) return KM_OK;
  if (!(pl.bhi && pl.k == k && pl.d == d)) {
    km_free(pl.bhi); km_free(pl.blo); km_free(pl.cn);
    pl.bhi = pl.blo = nullptr;
    pl.cn = nullptr;
    KM_CUDA(km_malloc(&pl.bhi, (size_t)npad * 64 * sizeof(__half)));
    KM_CUDA(km_malloc(&pl.blo, (size_t)npad * 64 * sizeof(__half)));
    KM_CUDA(km_malloc(&pl.cn, (size_t)(npad + 1) * sizeof(float)));
  }
  pl.npad = npad; pl.k = k; pl.d = d; pl.x_base = X; pl.x_rows = rows;
  KM_TRY(make_map(&pl.tmX, X, rows, d, kBM, 4));
  KM_TRY(make_map(&pl.tmBhi, pl.bhi, npad, 64, npad, 2));
  KM_TRY(make_map(&pl.tmBlo, pl.blo, npad, 64, npad, 2));
  if (d == 32) {
    KM_CUDA(cudaFuncSetAttribute(assign_tc_kernel<32, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem_bytes(d, npad)));
  } else {
    KM_CUDA(cudaFuncSetAttribute(assign_tc_kernel<64, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem_bytes(d, npad)));
    KM_CUDA(cudaFuncSetAttribute(assign_tc_kernel<64, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem_bytes(d, npad)));
  }
  pl.ready = true;
  return KM_OK;
}

inline int prep(Plan& pl, const float* C, const float* cnorm, cudaStream_t stream) {
  KM_CUDA(cudaMemsetAsync(pl.cn + pl.npad, 0, sizeof(float), stream));
  prep_kernel<<<pl.npad, 64, 0, stream>>>(C, cnorm, pl.k, pl.d, pl.npad, pl.sb, pl.sx * pl.sb, pl.bhi, pl.blo, pl.cn);
  KM_CUDA(cudaGetLastError());
  return KM_OK;
}

// A row goes to the exact pass when second - best <= split_tolerance(...) (km_assign_tc.cuh):
// kTolRel * (|x|^2 + max|c|^2) plus an absolute floor.  Error of the split product with
// y = x sx = xh + xl + ex, b = -2c sb = bh + bl + eb: the kernel forms xh.bh + xl.bh + xh.bl, so a
// score misses xl.bl + ex.b + y.eb per element.  While the low halves are normal fp16 numbers
// |ex| <= 2^-22 |y|, |eb| <= 2^-22 |b|, |xl.bl| <= 2^-22 |y||b|: 3 * 2^-22 sum|y||b|
// <= 3 * 2^-22 (|x|^2 + |c|^2) sx sb per score; with the fp32 accumulation of the 3 d / 16 partial
// sums that is below 2^-20.4 (|x|^2 + |c|^2), twice that for a difference: kTolRel = 2^-19.
// A low half below 2^-14 is an fp16 subnormal (quantum 2^-24): |ex|, |eb| <= 2^-25 absolute,
// which adds 2^-25 (|y|_1 + |b|_1) per score; tol_floor_of(d) = 2^-23 sqrt(d) bounds twice that
// for a difference through |v|_1 <= sqrt(d) |v|_2.
// The accumulation term grows with the row width: the tensor core adds every K = 16 slice into the fp32
// accumulator with truncation, a one-sided error per step that is proportional to the accumulator's
// magnitude.  Measured on the worst case for it (all coordinates near a common offset, so that
// |x.c| = |x||c| and the accumulator reaches |x|^2 + |c|^2), the largest error of a single score was
// (0.38 + d / 210) * 2^-19 (|x|^2 + |c|^2): 2^-19.5 at d = 64, 2^-18.4 at 256, 2^-17.1 at 784, 2^-15.6 at 2048
// - the constant is the split error above (two-sided), the slope the truncation - and with the flat 2^-19
// rows of 2048 columns were mislabelled (3 of 40,000, gaps up to 3e-4 relative; none seen up to 784
// columns).  For the difference of two nearly tied scores the split errors add (2 * 0.38); the truncation
// errors have the sign of their accumulators: equal signs cancel in part, opposite signs mean
// |acc_j| + |acc_l| = | |c_l|^2 - |c_j|^2 | <= max|c|^2, so their sum stays below the single-score
// figure.  tol_rel_of(d) = 2^-19 (0.8 + d / 200) keeps 5 % above 2^-19 (0.76 + d / 210).
constexpr float kTolRel = 1.9073486328125e-06f;
inline float tol_rel_of(int d) { return kTolRel * (0.8f + (float)d / 200.0f); }
inline float tol_floor_of(int d) { return 1.1920928955078125e-07f * std::sqrt((float)d); }

inline int launch(Plan& pl, int* labels, IterState* st, bool count_changes, unsigned int* amb_rows, float tol_rel,
                  int num_sms, cudaStream_t stream, unsigned int* moved_bits, uint4* amb_near,
                  bool allow_split_build) {
  const size_t tiles = (pl.x_rows + kBM - 1) / kBM;
  if (tiles > 0x7fffffffULL / kBM) KM_FAIL(KM_EINVAL, "shard too large for the tensor-core kernel");
  const int grid = (int)std::min<size_t>(tiles, (size_t)num_sms);
  const bool pre = ensure_xsplit(pl, pl.x_base, pl.x_rows, pl.d, pl.sx, num_sms, stream, allow_split_build);
  if (pl.d == 32)
    assign_tc_kernel<32, false><<<grid, kThreads, smem_bytes(pl.d, pl.npad), stream>>>(
        pl.tmX, pl.tmX, pl.tmBhi, pl.tmBlo, pl.cn, pl.xnorm, labels, pl.x_rows, (int)tiles, pl.npad, st,
        count_changes ? 1 : 0, amb_rows, tol_rel, tol_floor_of(pl.d), pl.sx, pl.sx * pl.sb, count_changes ? moved_bits : nullptr,
        amb_near, wait_limits().mbar_iters);
  else if (pre)
    assign_tc_kernel<64, true><<<grid, kThreads, smem_bytes(pl.d, pl.npad), stream>>>(
        pl.tmXh, pl.tmXl, pl.tmBhi, pl.tmBlo, pl.cn, pl.xnorm, labels, pl.x_rows, (int)tiles, pl.npad, st,
        count_changes ? 1 : 0, amb_rows, tol_rel, tol_floor_of(pl.d), pl.sx, pl.sx * pl.sb, count_changes ? moved_bits : nullptr,
        amb_near, wait_limits().mbar_iters);
  else
    assign_tc_kernel<64, false><<<grid, kThreads, smem_bytes(pl.d, pl.npad), stream>>>(
        pl.tmX, pl.tmX, pl.tmBhi, pl.tmBlo, pl.cn, pl.xnorm, labels, pl.x_rows, (int)tiles, pl.npad, st,
        count_changes ? 1 : 0, amb_rows, tol_rel, tol_floor_of(pl.d), pl.sx, pl.sx * pl.sb, count_changes ? moved_bits : nullptr,
        amb_near, wait_limits().mbar_iters);
  KM_CUDA(cudaGetLastError());
  return KM_OK;
}

}  // namespace tc
}  // namespace km

#include "km_assign_tc_big.cuh"

namespace km {
namespace tcb {

struct BigPlan {
  __half* bhi = nullptr;
  __half* blo = nullptr;
  float* cn = nullptr;
  int kpad = 0, k = 0, d = 0, dp = 0;
  const float* x_base = nullptr;
  size_t x_rows = 0;
  float sx = 1.f, sb = 1.f;
  CUtensorMap tmX, tmBhi, tmBlo;
  bool ready = false;
  void release() {
    km_free(bhi); km_free(blo); km_free(cn);
    bhi = blo = nullptr;
    cn = nullptr;
    ready = false;
  }
};

// float32, rows of at most 256 columns with 16-byte alignment (d % 4 == 0); the |c|^2 table of all
// centroids must fit shared memory.  The kernel is compiled for 32, 64, 128 and 256 columns; other
// widths run the next larger variant: the copy engine zero-fills the columns of an X tile that lie
// beyond d and the split centroid table is zero there too, so the products are unchanged.
inline bool big_shape_ok(int k, int d) { return d >= 32 && d <= 256 && d % 4 == 0 && k > 16 && k <= 6144; }
inline int big_variant(int d) { return d <= 32 ? 32 : (d <= 64 ? 64 : (d <= 128 ? 128 : 256)); }

template <int D>
inline int big_set_attr(int kpad) {
  KM_CUDA(cudaFuncSetAttribute(assign_tc_big_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               (int)big_smem_bytes<D>(kpad)));
  return KM_OK;
}

// ldx: row pitch of X in elements (d, or d rounded up to four for the padded copy of unaligned rows)
inline int big_setup(BigPlan& pl, const float* X, size_t rows, int k, int d, int ldx) {
  const int kpad = (k + kNT - 1) / kNT * kNT;
  const int dv = big_variant(d);
  const int dp = dv < 64 ? 64 : dv;
  if (pl.ready && pl.k == k && pl.d == d && pl.x_base == X && pl.x_rows == rows) return KM_OK;
  if (!(pl.bhi && pl.k == k && pl.d == d)) {
    pl.release();
    KM_CUDA(km_malloc(&pl.bhi, (size_t)kpad * dp * sizeof(__half)));
    KM_CUDA(km_malloc(&pl.blo, (size_t)kpad * dp * sizeof(__half)));
    KM_CUDA(km_malloc(&pl.cn, (size_t)(kpad + 1) * sizeof(float)));
  }
  pl.kpad = kpad; pl.k = k; pl.d = d; pl.dp = dp; pl.x_base = X; pl.x_rows = rows;
  KM_TRY(tc::make_map(&pl.tmX, X, rows, ldx, kBM, 4));
  KM_TRY(tc::make_map(&pl.tmBhi, pl.bhi, kpad, dp, kNT, 2));
  KM_TRY(tc::make_map(&pl.tmBlo, pl.blo, kpad, dp, kNT, 2));
  if (dv == 32) KM_TRY(big_set_attr<32>(kpad));
  else if (dv == 64) KM_TRY(big_set_attr<64>(kpad));
  else if (dv == 128) KM_TRY(big_set_attr<128>(kpad));
  else KM_TRY(big_set_attr<256>(kpad));
  pl.ready = true;
  return KM_OK;
}

inline int big_prep(BigPlan& pl, const float* C, const float* cnorm, cudaStream_t stream) {
  KM_CUDA(cudaMemsetAsync(pl.cn + pl.kpad, 0, sizeof(float), stream));
  big_prep_kernel<<<pl.kpad, 256, 0, stream>>>(C, cnorm, pl.k, pl.d, pl.dp, pl.kpad, pl.sb, pl.sx * pl.sb, pl.bhi,
                                               pl.blo, pl.cn);
  KM_CUDA(cudaGetLastError());
  return KM_OK;
}

template <int D>
inline void big_launch_d(BigPlan& pl, const float* xnorm, int* labels, IterState* st, int count_changes,
                         unsigned int* amb_rows, float tol_rel, int grid, int tiles, cudaStream_t stream) {
  assign_tc_big_kernel<D><<<grid, kBigThreads, big_smem_bytes<D>(pl.kpad), stream>>>(
      pl.tmX, pl.tmBhi, pl.tmBlo, pl.cn, xnorm, labels, pl.x_rows, tiles, pl.kpad, st, count_changes, amb_rows,
      tol_rel, tc::tol_floor_of(pl.d), pl.sx, pl.sx * pl.sb, wait_limits().mbar_iters);
}

inline int big_launch(BigPlan& pl, const float* xnorm, int* labels, IterState* st, bool count_changes,
                      unsigned int* amb_rows, float tol_rel, int num_sms, cudaStream_t stream) {
  const size_t tiles = (pl.x_rows + kBM - 1) / kBM;
  if (tiles > 0x7fffffffULL / kBM) KM_FAIL(KM_EINVAL, "shard too large for the tensor-core kernel");
  const int grid = (int)std::min<size_t>(tiles, (size_t)num_sms);
  const int cc = count_changes ? 1 : 0;
  const int dv = big_variant(pl.d);
  if (dv == 32) big_launch_d<32>(pl, xnorm, labels, st, cc, amb_rows, tol_rel, grid, (int)tiles, stream);
  else if (dv == 64) big_launch_d<64>(pl, xnorm, labels, st, cc, amb_rows, tol_rel, grid, (int)tiles, stream);
  else if (dv == 128) big_launch_d<128>(pl, xnorm, labels, st, cc, amb_rows, tol_rel, grid, (int)tiles, stream);
  else big_launch_d<256>(pl, xnorm, labels, st, cc, amb_rows, tol_rel, grid, (int)tiles, stream);
  KM_CUDA(cudaGetLastError());
  return KM_OK;
}

}  // namespace tcb
}  // namespace km

#include "km_assign_tc_wide.cuh"

namespace km {
namespace tcw {

struct WidePlan {
  __half* bhi = nullptr;
  __half* blo = nullptr;
  float* cn = nullptr;
  int k = 0, d = 0, dp = 0, n_chunks = 0, stages = 0;
  const float* x_base = nullptr;
  size_t x_rows = 0;
  float sx = 1.f, sb = 1.f;
  CUtensorMap tmX, tmBhi, tmBlo;
  bool ready = false;
  void release() {
    km_free(bhi); km_free(blo); km_free(cn);
    bhi = blo = nullptr;
    cn = nullptr;
    ready = false;
  }
};

// Ring depth for d columns: four stages, or two when shared memory is short.  EVEN on purpose: chunks
// alternate between the two converter groups, so with an even depth a stage always serves the same
// group and every "stage full" barrier has one waiter that takes its phases in order.  With an odd
// depth the two groups would share a stage's barrier without being ordered against each other, and a
// one-bit phase parity cannot tell "the phase I wait for" from "the phase before the previous one":
// a group that ran ahead of a late copy took the stage early (a device fault at 2e6 rows x 784).
inline int wide_stages(int d) {
  const int n_chunks = (d + kChunk - 1) / kChunk;
  for (int s = 4; s >= 2; s -= 2)
    if (wide_smem_bytes(n_chunks, s) <= (size_t)227 * 1024) return s;
  return 0;
}
// float32, at most 16 centroids, rows of 128 or more columns (16-byte aligned rows: d % 4 == 0)
inline bool wide_shape_ok(int k, int d) { return k >= 1 && k <= kNPad && d >= 128 && d % 4 == 0 && wide_stages(d) > 0; }

inline int wide_setup(WidePlan& pl, const float* X, size_t rows, int k, int d, int ldx) {
  if (pl.ready && pl.k == k && pl.d == d && pl.x_base == X && pl.x_rows == rows) return KM_OK;
  const int n_chunks = (d + kChunk - 1) / kChunk;
  const int dp = n_chunks * kChunk;
  if (!(pl.bhi && pl.k == k && pl.d == d)) {
    pl.release();
    KM_CUDA(km_malloc(&pl.bhi, (size_t)kNPad * dp * sizeof(__half)));
    KM_CUDA(km_malloc(&pl.blo, (size_t)kNPad * dp * sizeof(__half)));
    KM_CUDA(km_malloc(&pl.cn, (size_t)(kNPad + 1) * sizeof(float)));
  }
  pl.k = k; pl.d = d; pl.dp = dp; pl.n_chunks = n_chunks; pl.stages = wide_stages(d);
  pl.x_base = X; pl.x_rows = rows;
  KM_TRY(tc::make_map(&pl.tmX, X, rows, ldx, kBM, 4));
  KM_TRY(tc::make_map(&pl.tmBhi, pl.bhi, kNPad, dp, kNPad, 2));
  KM_TRY(tc::make_map(&pl.tmBlo, pl.blo, kNPad, dp, kNPad, 2));
  KM_CUDA(cudaFuncSetAttribute(assign_tc_wide_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               (int)wide_smem_bytes(n_chunks, pl.stages)));
  pl.ready = true;
  return KM_OK;
}

inline int wide_prep(WidePlan& pl, const float* C, const float* cnorm, cudaStream_t stream) {
  KM_CUDA(cudaMemsetAsync(pl.cn + kNPad, 0, sizeof(float), stream));
  tcb::big_prep_kernel<<<kNPad, 256, 0, stream>>>(C, cnorm, pl.k, pl.d, pl.dp, kNPad, pl.sb, pl.sx * pl.sb, pl.bhi,
                                                  pl.blo, pl.cn);
  KM_CUDA(cudaGetLastError());
  return KM_OK;
}

// labels of rows [row0, row0 + nrows) (row0 a multiple of 128), or - with `out` - their squared distances to
// the k centroids as a column-major block with leading dimension ld_out
inline int wide_launch(WidePlan& pl, const float* xnorm, int* labels, IterState* st, bool count_changes,
                       unsigned int* amb_rows, float tol_rel, int num_sms, cudaStream_t stream, size_t row0 = 0,
                       size_t nrows = 0, float* out = nullptr, size_t ld_out = 0) {
  if (nrows == 0) nrows = pl.x_rows - row0;
  const size_t tiles = (nrows + kBM - 1) / kBM;
  if ((pl.x_rows + kBM - 1) / kBM > 0x7fffffffULL / kBM) KM_FAIL(KM_EINVAL, "shard too large for the tensor-core kernel");
  const int grid = (int)std::min<size_t>(tiles, (size_t)num_sms);
  assign_tc_wide_kernel<<<grid, kWThreads, wide_smem_bytes(pl.n_chunks, pl.stages), stream>>>(
      pl.tmX, pl.tmBhi, pl.tmBlo, pl.cn, xnorm, labels, std::min(pl.x_rows, row0 + nrows), (int)(row0 / kBM), (int)tiles,
      pl.n_chunks, pl.stages, pl.k, st, count_changes ? 1 : 0, amb_rows, tol_rel, tc::tol_floor_of(pl.d), pl.sx,
      pl.sx * pl.sb, wait_limits().mbar_iters, out, ld_out);
  KM_CUDA(cudaGetLastError());
  return KM_OK;
}

}  // namespace tcw
}  // namespace km

#include "km_assign_tc_stream.cuh"

namespace km {
namespace tcs {

struct StreamPlan {
  __half* bhi = nullptr;
  __half* blo = nullptr;
  float* cn = nullptr;
  int k = 0, d = 0, dp = 0, n_chunks = 0, npad = 0, n_pass = 0, kpad = 0;
  const float* x_base = nullptr;
  size_t x_rows = 0;
  float sx = 1.f, sb = 1.f;
  CUtensorMap tmX, tmBhi, tmBlo;
  bool ready = false;
  void release() {
    km_free(bhi); km_free(blo); km_free(cn);
    bhi = blo = nullptr;
    cn = nullptr;
    ready = false;
  }
};

// float32, more than 16 centroids, 16-byte aligned rows of 32 to 4096 columns.  Up to 128 centroids run
// with N = 128 and two accumulators, more with N = 256 (one pass per 256 centroids).
inline bool stream_shape_ok(int k, int d) { return k > 16 && k <= 6144 && d >= 32 && d <= 4096 && d % 4 == 0; }
inline int stream_npad(int k) { return k <= 128 ? 128 : 256; }

inline int stream_setup(StreamPlan& pl, const float* X, size_t rows, int k, int d, int ldx) {
  if (pl.ready && pl.k == k && pl.d == d && pl.x_base == X && pl.x_rows == rows) return KM_OK;
  const int n_chunks = (d + kSChunk - 1) / kSChunk;
  const int dp = n_chunks * kSChunk;
  const int npad = stream_npad(k);
  const int n_pass = (k + npad - 1) / npad;
  const int kpad = n_pass * npad;
  if (!(pl.bhi && pl.k == k && pl.d == d)) {
    pl.release();
    KM_CUDA(km_malloc(&pl.bhi, (size_t)kpad * dp * sizeof(__half)));
    KM_CUDA(km_malloc(&pl.blo, (size_t)kpad * dp * sizeof(__half)));
    KM_CUDA(km_malloc(&pl.cn, (size_t)(kpad + 1) * sizeof(float)));
  }
  pl.k = k; pl.d = d; pl.dp = dp; pl.n_chunks = n_chunks; pl.npad = npad; pl.n_pass = n_pass; pl.kpad = kpad;
  pl.x_base = X; pl.x_rows = rows;
  KM_TRY(tc::make_map(&pl.tmX, X, rows, ldx, kBM, 4));
  KM_TRY(tc::make_map(&pl.tmBhi, pl.bhi, kpad, dp, npad, 2));
  KM_TRY(tc::make_map(&pl.tmBlo, pl.blo, kpad, dp, npad, 2));
  if (npad == 128)
    KM_CUDA(cudaFuncSetAttribute(assign_tc_stream_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)stream_smem_bytes<128>()));
  else
    KM_CUDA(cudaFuncSetAttribute(assign_tc_stream_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)stream_smem_bytes<256>()));
  pl.ready = true;
  return KM_OK;
}

inline int stream_prep(StreamPlan& pl, const float* C, const float* cnorm, cudaStream_t stream) {
  KM_CUDA(cudaMemsetAsync(pl.cn + pl.kpad, 0, sizeof(float), stream));
  tcb::big_prep_kernel<<<pl.kpad, 256, 0, stream>>>(C, cnorm, pl.k, pl.d, pl.dp, pl.kpad, pl.sb, pl.sx * pl.sb, pl.bhi,
                                                   pl.blo, pl.cn);
  KM_CUDA(cudaGetLastError());
  return KM_OK;
}

// labels of rows [row0, row0 + nrows) (row0 a multiple of 128), or - with `out` - their squared distances to
// the k centroids as a column-major block with leading dimension ld_out
inline int stream_launch(StreamPlan& pl, const float* xnorm, int* labels, IterState* st, bool count_changes,
                         unsigned int* amb_rows, float tol_rel, int num_sms, cudaStream_t stream, size_t row0 = 0,
                         size_t nrows = 0, float* out = nullptr, size_t ld_out = 0) {
  if (nrows == 0) nrows = pl.x_rows - row0;
  const size_t tiles = (nrows + kBM - 1) / kBM;
  if ((pl.x_rows + kBM - 1) / kBM > 0x7fffffffULL / kBM) KM_FAIL(KM_EINVAL, "shard too large for the tensor-core kernel");
  const int grid = (int)std::min<size_t>(tiles, (size_t)num_sms);
  const size_t n_end = std::min(pl.x_rows, row0 + nrows);
  if (pl.npad == 128)
    assign_tc_stream_kernel<128><<<grid, kSThreads, stream_smem_bytes<128>(), stream>>>(
        pl.tmX, pl.tmBhi, pl.tmBlo, pl.cn, xnorm, labels, n_end, (int)(row0 / kBM), (int)tiles, pl.n_chunks, pl.n_pass,
        pl.k, st, count_changes ? 1 : 0, amb_rows, tol_rel, tc::tol_floor_of(pl.d), pl.sx, pl.sx * pl.sb,
        wait_limits().mbar_iters, out, ld_out);
  else
    assign_tc_stream_kernel<256><<<grid, kSThreads, stream_smem_bytes<256>(), stream>>>(
        pl.tmX, pl.tmBhi, pl.tmBlo, pl.cn, xnorm, labels, n_end, (int)(row0 / kBM), (int)tiles, pl.n_chunks, pl.n_pass,
        pl.k, st, count_changes ? 1 : 0, amb_rows, tol_rel, tc::tol_floor_of(pl.d), pl.sx, pl.sx * pl.sb,
        wait_limits().mbar_iters, out, ld_out);
  KM_CUDA(cudaGetLastError());
  return KM_OK;
}

}  // namespace tcs
}  // namespace km
