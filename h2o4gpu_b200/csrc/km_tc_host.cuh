// Host side of the tensor-core distance kernel: eligibility, the split centroid
// buffers, TMA tensor maps (encoded through the driver entry point, so the
// library has no link-time dependency on libcuda) and the launch.
#pragma once

#include "km_assign_tc.cuh"

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

// rows x cols fp32 row-major, boxes of box_rows x 32 columns, 128-byte swizzle
inline int make_map(CUtensorMap* map, const float* base, size_t rows, int cols, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) KM_FAIL(KM_ECUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t gdim[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t gstride[1] = {(cuuint64_t)cols * sizeof(float)};
  cuuint32_t box[2] = {32u, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1u, 1u};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), gdim, gstride, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) KM_FAIL(KM_ECUDA, "cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
  return KM_OK;
}

struct Plan {
  float* bhi = nullptr;
  float* blo = nullptr;
  float* cn = nullptr;
  int npad = 0, k = 0, d = 0;
  const float* x_base = nullptr;
  size_t x_rows = 0;
  CUtensorMap tmX, tmBhi, tmBlo;
  bool ready = false;

  void release() {
    cudaFree(bhi); cudaFree(blo); cudaFree(cn);
    bhi = blo = cn = nullptr;
    ready = false;
  }
};

inline bool shape_ok(int k, int d) { return (d == 32 || d == 64) && k > 16 && k <= kMaxNPad; }

inline int setup(Plan& pl, const float* X, size_t rows, int k, int d) {
  const int npad = (k + 15) / 16 * 16;
  if (pl.ready && pl.k == k && pl.d == d && pl.x_base == X && pl.x_rows == rows) return KM_OK;
  if (!(pl.bhi && pl.k == k && pl.d == d)) {
    pl.release();
    KM_CUDA(cudaMalloc(&pl.bhi, (size_t)npad * d * sizeof(float)));
    KM_CUDA(cudaMalloc(&pl.blo, (size_t)npad * d * sizeof(float)));
    KM_CUDA(cudaMalloc(&pl.cn, (size_t)(npad + 1) * sizeof(float)));
  }
  pl.npad = npad; pl.k = k; pl.d = d; pl.x_base = X; pl.x_rows = rows;
  KM_TRY(make_map(&pl.tmX, X, rows, d, kBM));
  KM_TRY(make_map(&pl.tmBhi, pl.bhi, npad, d, npad));
  KM_TRY(make_map(&pl.tmBlo, pl.blo, npad, d, npad));
  if (d == 32)
    KM_CUDA(cudaFuncSetAttribute(assign_tc_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem_bytes(d, npad)));
  else
    KM_CUDA(cudaFuncSetAttribute(assign_tc_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem_bytes(d, npad)));
  pl.ready = true;
  return KM_OK;
}

inline int prep(Plan& pl, const float* C, const float* cnorm, cudaStream_t stream) {
  KM_CUDA(cudaMemsetAsync(pl.cn + pl.npad, 0, sizeof(float), stream));
  prep_kernel<<<pl.npad, 64, 0, stream>>>(C, cnorm, pl.k, pl.d, pl.npad, pl.bhi, pl.blo, pl.cn);
  KM_CUDA(cudaGetLastError());
  return KM_OK;
}

// tol_rel: a row goes to the exact pass when second - best <= tol_rel * (|x|^2 + max|c|^2).
// Error of the 3xTF32 product: xh truncated (exact residual), xl and both halves of
// -2c rounded to TF32 (2^-12 relative each), xl.bl dropped (2^-21 |x||b|): about
// 2^-20.4 (|x|^2 + |c|^2) per score, twice that for a difference -> 2^-19.
constexpr float kTolRel = 1.9073486328125e-06f;

inline int launch(Plan& pl, int* labels, IterState* st, bool count_changes, unsigned int* amb_rows, float tol_rel,
                  int num_sms, int mask_hi, cudaStream_t stream) {
  const size_t tiles = (pl.x_rows + kBM - 1) / kBM;
  if (tiles > 0x7fffffffULL / kBM) KM_FAIL(KM_EINVAL, "shard too large for the tensor-core kernel");
  const int grid = (int)std::min<size_t>(tiles, (size_t)num_sms);
  if (pl.d == 32)
    assign_tc_kernel<32><<<grid, kThreads, smem_bytes(pl.d, pl.npad), stream>>>(
        pl.tmX, pl.tmBhi, pl.tmBlo, pl.cn, labels, pl.x_rows, (int)tiles, pl.npad, st, count_changes ? 1 : 0,
        amb_rows, tol_rel, mask_hi);
  else
    assign_tc_kernel<64><<<grid, kThreads, smem_bytes(pl.d, pl.npad), stream>>>(
        pl.tmX, pl.tmBhi, pl.tmBlo, pl.cn, labels, pl.x_rows, (int)tiles, pl.npad, st, count_changes ? 1 : 0,
        amb_rows, tol_rel, mask_hi);
  KM_CUDA(cudaGetLastError());
  return KM_OK;
}

}  // namespace tc
}  // namespace km
