// Shared helpers of the k-means kernels: error plumbing, the fixed-point
// representation of the centroid sums, small device utilities.
#pragma once

#include <algorithm>
#include <cstdlib>
#include <mutex>

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <string>

#include "../../include/h2o4gpu_kmeans.h"

// Named ranges for timeline tools (NVTX, header-only; without a tool attached a call costs a few
// nanoseconds).  The reference marks nothing; these make upload / check / init / fit / iteration /
// assign / transform visible next to the kernels.
#if defined(__has_include)
#if __has_include(<nvtx3/nvToolsExt.h>)
#include <nvtx3/nvToolsExt.h>
#define KM_HAVE_NVTX 1
#endif
#endif

namespace km {

struct TraceRange {
  explicit TraceRange(const char* name) {
#ifdef KM_HAVE_NVTX
    nvtxRangePushA(name);
#else
    (void)name;
#endif
  }
  ~TraceRange() {
#ifdef KM_HAVE_NVTX
    nvtxRangePop();
#endif
  }
  TraceRange(const TraceRange&) = delete;
  TraceRange& operator=(const TraceRange&) = delete;
};


// ---- error plumbing -----------------------------------------------------------
void set_error(const std::string& msg);

struct Status {
  int code;
  Status(int c = KM_OK) : code(c) {}
  bool ok() const { return code == KM_OK; }
};

#define KM_CUDA(expr)                                                                   \
  do {                                                                                  \
    cudaError_t _e = (expr);                                                            \
    if (_e != cudaSuccess) {                                                            \
      ::km::set_error(std::string(#expr) + ": " + cudaGetErrorString(_e) + " (" +       \
                      __FILE__ + ":" + std::to_string(__LINE__) + ")");                 \
      return (_e == cudaErrorMemoryAllocation) ? KM_ENOMEM : KM_ECUDA;                  \
    }                                                                                   \
  } while (0)

#define KM_TRY(expr)                   \
  do {                                 \
    int _s = (expr);                   \
    if (_s != KM_OK) return _s;        \
  } while (0)

#define KM_FAIL(code, msg)             \
  do {                                 \
    ::km::set_error(msg);              \
    return (code);                     \
  } while (0)

// ---- device memory ------------------------------------------------------------
// Every buffer of the library comes from one stream-ordered memory pool per device that
// keeps what is freed (release threshold: unlimited).  A fit through the host-pointer entry
// points creates and destroys some twenty-five buffers, one of them the whole matrix;
// with cudaMalloc / cudaFree that costs 5-20 ms per call in mapping and unmapping alone,
// with the pool a later call finds the memory in place.  kmeans_trim_memory() hands the
// cached memory back to the driver; H2O4GPU_KM_POOL=0 turns the pool off.
// km_malloc returns memory that any stream may use at once (the allocation is made on a
// stream of its own, which is then waited for); km_free waits for the device to go idle
// first, as cudaFree does.  Both act on the current device.
struct DevicePools {
  static constexpr int kMaxDev = 64;
  cudaMemPool_t pool[kMaxDev] = {};
  cudaStream_t stream[kMaxDev] = {};
  int state[kMaxDev] = {};        // 0 untried, 1 pool in use, -1 plain cudaMalloc
  std::mutex m;
  static DevicePools& get() {
    static DevicePools* p = new DevicePools();   // outlives the CUDA runtime's own teardown
    return *p;
  }
  int mode(int dev) {
    if (dev < 0 || dev >= kMaxDev) return -1;
    std::lock_guard<std::mutex> lock(m);
    if (state[dev] != 0) return state[dev];
    state[dev] = -1;
    const char* e = std::getenv("H2O4GPU_KM_POOL");
    if (e && e[0] == '0') return -1;
    int supported = 0;
    if (cudaDeviceGetAttribute(&supported, cudaDevAttrMemoryPoolsSupported, dev) != cudaSuccess || !supported) {
      cudaGetLastError();
      return -1;
    }
    cudaMemPoolProps props = {};
    props.allocType = cudaMemAllocationTypePinned;
    props.handleTypes = cudaMemHandleTypeNone;
    props.location.type = cudaMemLocationTypeDevice;
    props.location.id = dev;
    if (cudaMemPoolCreate(&pool[dev], &props) != cudaSuccess) { cudaGetLastError(); return -1; }
    unsigned long long keep = ~0ULL;
    cudaMemPoolSetAttribute(pool[dev], cudaMemPoolAttrReleaseThreshold, &keep);
    if (cudaStreamCreateWithFlags(&stream[dev], cudaStreamNonBlocking) != cudaSuccess) {
      cudaGetLastError();
      cudaMemPoolDestroy(pool[dev]);
      return -1;
    }
    state[dev] = 1;
    return 1;
  }
};

inline cudaError_t km_malloc_bytes(void** p, size_t bytes) {
  int dev = 0;
  cudaError_t ce = cudaGetDevice(&dev);
  if (ce != cudaSuccess) return ce;
  DevicePools& dp = DevicePools::get();
  if (dp.mode(dev) != 1) return cudaMalloc(p, bytes);
  ce = cudaMallocFromPoolAsync(p, std::max<size_t>(bytes, 1), dp.pool[dev], dp.stream[dev]);
  if (ce != cudaSuccess) return ce;
  return cudaStreamSynchronize(dp.stream[dev]);
}
template <typename P>
inline cudaError_t km_malloc(P** p, size_t bytes) { return km_malloc_bytes(reinterpret_cast<void**>(p), bytes); }

inline cudaError_t km_free(void* p) {
  if (!p) return cudaSuccess;
  int dev = 0;
  cudaError_t ce = cudaGetDevice(&dev);
  if (ce != cudaSuccess) return ce;
  DevicePools& dp = DevicePools::get();
  if (dp.mode(dev) != 1) return cudaFree(p);
  ce = cudaDeviceSynchronize();      // nothing in flight may still use the buffer
  if (ce != cudaSuccess) return ce;
  return cudaFreeAsync(p, dp.stream[dev]);
}

inline void km_trim_pools() {
  DevicePools& dp = DevicePools::get();
  std::lock_guard<std::mutex> lock(dp.m);
  for (int dev = 0; dev < DevicePools::kMaxDev; ++dev)
    if (dp.state[dev] == 1) {
      cudaStreamSynchronize(dp.stream[dev]);
      cudaMemPoolTrimTo(dp.pool[dev], 0);
    }
}

// ---- fixed-point centroid sums ------------------------------------------------
// A value x (|x| <= xmax < 2^e) is cut into NP signed pieces of 15 bits:
//   p0 = rint(x * 2^sa), sa = 15 - e, |p0| <= 2^15
//   r0 = x * 2^sa - p0 (exact), p1 = rint(r0 * 2^15), r1 = r0 * 2^15 - p1, ...
// Pieces are summed as integers, so the sum does not depend on the order of
// additions: any CTA schedule, any number of GPUs and any reduction tree give
// the same bits.  int32 accumulators in shared memory hold up to 2^15 rows;
// int64 accumulators in global memory hold pairs p(2q) * 2^15 + p(2q+1) and are
// exact for up to 2^32 rows.  float uses 2 pieces (quantum xmax * 2^-30, below
// half an ulp of any |x| >= xmax * 2^-7), double 4 pieces (quantum xmax * 2^-60).
template <typename T> struct Fixed;
template <> struct Fixed<float> { static constexpr int NP = 2; };
template <> struct Fixed<double> { static constexpr int NP = 4; };
constexpr int kPieceBits = 15;
constexpr int kFlushRows = 32768;  // rows a CTA may add before its int32 accumulators are drained

// Splits x * scale into NP 15-bit pieces.  `scale` = 2^sa.
template <int NP>
__device__ __forceinline__ void split_pieces(float x, float scale, int (&p)[NP]) {
  // rint via the 1.5*2^23 trick: exact for |v| < 2^22, all full-rate ops.
  const float magic = 12582912.0f;
  float v = x * scale;
#pragma unroll
  for (int q = 0; q < NP; ++q) {
    float t = v + magic;
    p[q] = __float_as_int(t) - __float_as_int(magic);
    float pf = t - magic;
    v = (v - pf) * 32768.0f;
  }
}
template <int NP>
__device__ __forceinline__ void split_pieces(double x, double scale, int (&p)[NP]) {
  const double magic = 6755399441055744.0;  // 1.5 * 2^52
  double v = x * scale;
#pragma unroll
  for (int q = 0; q < NP; ++q) {
    double t = v + magic;
    p[q] = (int)(__double2loint(t));  // low word of the mantissa holds rint(v) (two's complement)
    double pf = t - magic;
    v = (v - pf) * 32768.0;
  }
}

// Shared-memory accumulators of one cluster hold column `col` at position
//   pos = (col % V) * dv + col / V        (dv = d / V, V = elements per vector load)
// so that the lanes of a warp, which own consecutive vectors of a row, hit
// consecutive banks.  When several rows share a warp step, row r starts with
// element (r % V) of its vector, which spreads the rows over different banks.
// adds x[0..V) (vector c4 of its row) into the cluster whose piece-0 base is a0.
template <typename T, int V, int NP>
__device__ __forceinline__ void add_vec_fixed(int* a0, size_t pstride, int dv, int c4, int rot, const T (&x)[V],
                                              T scale) {
  T y[V];
#pragma unroll
  for (int e = 0; e < V; ++e) y[e] = x[e];
  if (V == 4) {
    if (rot & 1) { T t = y[0]; y[0] = y[1]; y[1] = y[2]; y[2] = y[3]; y[3] = t; }
    if (rot & 2) { T t = y[0]; y[0] = y[2]; y[2] = t; t = y[1]; y[1] = y[3]; y[3] = t; }
  } else if (V == 2) {
    if (rot & 1) { T t = y[0]; y[0] = y[1]; y[1] = t; }
  }
#pragma unroll
  for (int ee = 0; ee < V; ++ee) {
    const int e = (ee + rot) & (V - 1);
    int p[NP];
    split_pieces<NP>(y[ee], scale, p);
    int* a = a0 + e * dv + c4;
#pragma unroll
    for (int q = 0; q < NP; ++q) atomicAdd(a + q * pstride, p[q]);
  }
}
// column of position `pos`
__device__ __forceinline__ int pos_to_col(int pos, int dv, int V) { return (pos % dv) * V + pos / dv; }

// Value of NP/2 int64 pairs back as a double.  inv = 2^-(sa + 15).
template <int NP>
__device__ __host__ __forceinline__ double fixed_to_double(const long long* g, double inv) {
  // pair q weighs inv * 2^(-30 q); the small pair is added first
  if (NP == 2) return (double)g[0] * inv;
  return (double)g[1] * (inv * (1.0 / 1073741824.0)) + (double)g[0] * inv;
}

// float -> double without cvt.f64.f32, which runs at a small fraction of the FMA rate on this part.
__device__ __forceinline__ double widen_exact(double x) { return x; }
__device__ __forceinline__ double widen_exact(float x) {
  // normal numbers exactly; zero and denormals (below 1.2e-38) become zero; the data has
  // been checked for Inf / NaN
  const unsigned int u = __float_as_uint(x);
  const unsigned int hi = (u & 0x80000000u) | (((u & 0x7fffffffu) >> 3) + 0x38000000u);
  return (u & 0x7f800000u) ? __hiloint2double((int)hi, (int)(u << 29)) : 0.0;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ double warp_max(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmax(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <typename T> struct Inf;
template <> struct Inf<float> { __device__ static float v() { return __int_as_float(0x7f800000); } };
template <> struct Inf<double> { __device__ static double v() { return __longlong_as_double(0x7ff0000000000000LL); } };

// Device-side scalars of one shard, shared by the kernels of an iteration.
struct IterState {
  unsigned long long changed;   // labels that changed in the current E-step
  int n_empty;                  // empty clusters found by the current M-step
  int argmax_count;             // index of the largest cluster
  int relocated;                // relocations done in the current M-step
  int error;                    // sticky device-side error word (0 = none)
  unsigned int amb_count;       // rows handed to the exact re-evaluation pass in the current E-step
  unsigned int pad0;
  double shift_sq;              // summed squared centroid shift of the current M-step
  double inertia;               // scratch for the inertia pass
};

// Gate of the M-step's two branches (km_accumulate_delta.cuh): true when the incremental
// branch handles this iteration.  `changed` is the E-step's label-change counter.
__device__ __forceinline__ bool delta_turn(const unsigned long long* changed, unsigned long long limit) {
  return changed != nullptr && *changed <= limit;
}

}  // namespace km
