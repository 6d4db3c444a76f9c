// Centroid sums for callers that must not allocate.
//
// Some callers cannot call cudaMalloc where they call this library: serving loops
// whose device-memory budget is fixed after start-up (an allocation could fail or
// evict what the budget promised to others), and hosts that forbid the implicit
// device-wide synchronisation a cudaMalloc / cudaFree may cause in the middle of
// their pipeline.  For them this file offers the M-step reduction (per-cluster sums
// and counts of a labelled shard) with every byte of working memory in one
// file-scope device array: the call takes device pointers for its inputs and
// outputs, enqueues five small operations on the caller's stream and returns;
// it never calls cudaMalloc, cudaFree or any library routine that allocates.
//
// Limits and rules (also in include/h2o4gpu_kmeans.h):
//   * k * cols <= 24576 and k <= 4096; larger problems are refused with KM_EINVAL.
//     The array is 229,440 bytes and every GPU that loads the library holds it
//     until the process exits.
//   * The first call on a device looks up the array's device address and raises
//     the kernel's shared-memory limit; that first call should come before any
//     stream capture.  Later calls do no set-up.
//   * All calls on a device share the array.  It still holds the previous call's
//     numbers, so each call clears the part it uses first; two calls whose work
//     overlaps on the GPU (different streams) race on it and must be serialised
//     by the caller.
#include <atomic>
#include <mutex>

#include "km_common.cuh"
#include "km_tiles.cuh"

namespace {

constexpr int kNaMaxKD = 24576;   // k * cols
constexpr int kNaMaxK = 4096;
constexpr int kNaHeader = 8;      // [0] max|x| (double bits) [2] scale (float bits) [3] 2^-(sa+15) (double bits)
constexpr int kNaEntries = kNaHeader + kNaMaxKD + kNaMaxK;
constexpr int kNaThreads = 512;

// The scratch: fixed-point sums (int64) and counts of the call in flight.  In host
// code this name is only a handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) unsigned long long g_na_scratch[kNaEntries];

// max |x| of the shard into scratch[0] (as double bits; non-negative doubles order as integers)
template <int V>
__global__ void __launch_bounds__(256)
na_absmax_kernel(const float* __restrict__ X, size_t count, unsigned long long* __restrict__ scratch) {
  double m = 0;
  const size_t nv = count / V;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += (size_t)gridDim.x * blockDim.x) {
    float x[V];
    km::VecLoad<float, V>::ld(X + i * V, x);
#pragma unroll
    for (int e = 0; e < V; ++e) m = fmax(m, fabs((double)x[e]));
  }
  if (blockIdx.x == 0 && threadIdx.x < (count % V)) m = fmax(m, fabs((double)X[nv * V + threadIdx.x]));
  m = km::warp_max(m);
  if ((threadIdx.x & 31) == 0) atomicMax(scratch, (unsigned long long)__double_as_longlong(m));
}

__global__ void na_scale_kernel(unsigned long long* scratch) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  const double xmax = __longlong_as_double((long long)scratch[0]);
  int e = 0;
  if (xmax > 0.0) e = ilogb(xmax) + 1;  // xmax < 2^e
  const int sa = km::kPieceBits - e;
  scratch[2] = (unsigned long long)__float_as_uint((float)ldexp(1.0, sa));
  scratch[3] = (unsigned long long)__double_as_longlong(ldexp(1.0, -(sa + km::kPieceBits)));
}

// Variant of the centroid-sum kernel (km_accumulate.cuh, single-slice path) whose
// scale and global accumulators live in the static scratch.  Rows with a label
// outside [0, k) are skipped.
template <int V>
__global__ void __launch_bounds__(kNaThreads)
na_accumulate_kernel(const float* __restrict__ X, size_t n, int d, const int* __restrict__ labels, int k,
                     unsigned long long* __restrict__ scratch, unsigned int rows_per_part,
                     unsigned long long dv_magic) {
  constexpr int NP = km::Fixed<float>::NP;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  int* acc = reinterpret_cast<int*>(smem_raw);   // [NP][k][d]
  int* cnt = acc + (size_t)NP * k * d;           // [k]
  const int tid = threadIdx.x;
  const size_t r0 = (size_t)blockIdx.x * rows_per_part;
  size_t r1 = r0 + rows_per_part;
  if (r1 > n) r1 = n;
  if (r0 >= n) return;
  const unsigned int nrows = (unsigned int)(r1 - r0);
  const int dv = d / V;
  const size_t pstride = (size_t)k * d;
  const float scale = __uint_as_float((unsigned int)scratch[2]);
  for (int i = tid; i < NP * k * d; i += kNaThreads) acc[i] = 0;
  for (int i = tid; i < k; i += kNaThreads) cnt[i] = 0;
  __syncthreads();
  const float* Xp = X + r0 * (size_t)d;
  const int* Lp = labels + r0;
  const unsigned int items = nrows * (unsigned int)dv;
  for (unsigned int idx = tid; idx < items; idx += kNaThreads) {
    const unsigned int row = (unsigned int)(((unsigned long long)idx * dv_magic) >> 40);
    const unsigned int c4 = idx - row * dv;
    const int lab = Lp[row];
    if (lab < 0 || lab >= k) continue;
    float x[V];
    km::VecLoad<float, V>::ld(Xp + (size_t)idx * V, x);
    if (c4 == 0) atomicAdd(&cnt[lab], 1);
    km::add_vec_fixed<float, V, NP>(acc + (size_t)lab * d, pstride, dv, (int)c4, (int)row & (V - 1), x, scale);
  }
  __syncthreads();
  unsigned long long* gs = scratch + kNaHeader;
  for (int i = tid; i < k * d; i += kNaThreads) {
    const int c = i / d;
    const int col = km::pos_to_col(i - c * d, dv, V);
    const long long v = (long long)acc[i] * (1LL << km::kPieceBits) + (long long)acc[pstride + i];
    if (v) atomicAdd(gs + (size_t)c * d + col, (unsigned long long)v);
  }
  for (int i = tid; i < k; i += kNaThreads)
    if (cnt[i]) atomicAdd(gs + (size_t)k * d + i, (unsigned long long)cnt[i]);
}

__global__ void na_export_kernel(const unsigned long long* __restrict__ scratch, int kd, int k,
                                 double* __restrict__ sums, long long* __restrict__ counts) {
  const double inv = __longlong_as_double((long long)scratch[3]);
  const unsigned long long* gs = scratch + kNaHeader;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < kd + k; i += gridDim.x * blockDim.x) {
    if (i < kd) sums[i] = (double)(long long)gs[i] * inv;
    else counts[i - kd] = (long long)gs[i];
  }
}

struct NaDevice {
  unsigned long long* scratch = nullptr;  // device address of g_na_scratch on this device
  int num_sms = 0;
  std::atomic<bool> ready{false};
};
NaDevice g_na_dev[64];
std::mutex g_na_mutex;

// Once per device, with that device current; later calls only read the flag.
int na_setup(int dev, NaDevice** out) {
  NaDevice& nd = g_na_dev[dev];
  *out = &nd;
  if (nd.ready.load(std::memory_order_acquire)) return KM_OK;
  std::lock_guard<std::mutex> lock(g_na_mutex);
  if (!nd.ready.load(std::memory_order_relaxed)) {
    unsigned long long* ptr = nullptr;
    KM_CUDA(cudaGetSymbolAddress((void**)&ptr, g_na_scratch));
    KM_CUDA(cudaDeviceGetAttribute(&nd.num_sms, cudaDevAttrMultiProcessorCount, dev));
    const int smem_max = 2 * (int)sizeof(int) * kNaMaxKD + (int)sizeof(int) * kNaMaxK + 16;
    KM_CUDA(cudaFuncSetAttribute(na_accumulate_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_max));
    KM_CUDA(cudaFuncSetAttribute(na_accumulate_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_max));
    nd.scratch = ptr;
    nd.ready.store(true, std::memory_order_release);
  }
  return KM_OK;
}

}  // namespace

extern "C" int kmeans_centroid_sums_noalloc_f32(const float* dX, const int32_t* dLabels, size_t rows, size_t cols,
                                                int k, double* dSums, long long* dCounts, void* stream_) {
  if (!dX || !dLabels || !dSums || !dCounts || rows == 0 || cols == 0 || k < 1)
    KM_FAIL(KM_EINVAL, "kmeans_centroid_sums_noalloc_f32: bad argument");
  if (k > kNaMaxK || (unsigned long long)k * cols > (unsigned long long)kNaMaxKD)
    KM_FAIL(KM_EINVAL, "kmeans_centroid_sums_noalloc_f32: k * cols = " + std::to_string((unsigned long long)k * cols) +
                           " exceeds the static scratch (k * cols <= 24576, k <= 4096); use kmeans_centroid_sums_f32");
  int dev = 0;
  KM_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) KM_FAIL(KM_ENODEV, "kmeans_centroid_sums_noalloc_f32: device index out of range");
  NaDevice* nd = nullptr;
  KM_TRY(na_setup(dev, &nd));
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int d = (int)cols;
  const int kd = k * d;
  unsigned long long* scratch = nd->scratch;  // the looked-up device address, not the symbol
  KM_CUDA(cudaMemsetAsync(scratch, 0, (size_t)(kNaHeader + kd + k) * sizeof(unsigned long long), stream));
  const size_t count = rows * cols;
  const bool vec = (d % 4 == 0) && ((reinterpret_cast<uintptr_t>(dX) & 15) == 0);
  if (vec)
    na_absmax_kernel<4><<<nd->num_sms * 8, 256, 0, stream>>>(dX, count, scratch);
  else
    na_absmax_kernel<1><<<nd->num_sms * 8, 256, 0, stream>>>(dX, count, scratch);
  na_scale_kernel<<<1, 32, 0, stream>>>(scratch);
  const size_t smem = (size_t)2 * kd * sizeof(int) + (size_t)k * sizeof(int) + 16;
  size_t rpp = (rows + (size_t)nd->num_sms * 2 - 1) / ((size_t)nd->num_sms * 2);
  rpp = rpp < 1024 ? 1024 : rpp;
  rpp = rpp > (size_t)km::kFlushRows ? (size_t)km::kFlushRows : rpp;
  const int dv = vec ? d / 4 : d;
  // the row index comes from a multiply-shift division that is exact while items * dv < 2^40
  const size_t div_cap = ((1ULL << 40) - 1) / ((size_t)dv * dv);
  if (div_cap < 1) KM_FAIL(KM_EINVAL, "kmeans_centroid_sums_noalloc_f32: cols too large");
  rpp = rpp > div_cap ? div_cap : rpp;
  const size_t grid = (rows + rpp - 1) / rpp;
  if (grid > 0x7fffffffULL) KM_FAIL(KM_EINVAL, "kmeans_centroid_sums_noalloc_f32: too many rows for one launch");
  const unsigned long long magic = ((1ULL << 40) / (unsigned)dv) + 1ULL;
  if (vec)
    na_accumulate_kernel<4><<<(unsigned)grid, kNaThreads, smem, stream>>>(dX, rows, d, dLabels, k, scratch, (unsigned)rpp, magic);
  else
    na_accumulate_kernel<1><<<(unsigned)grid, kNaThreads, smem, stream>>>(dX, rows, d, dLabels, k, scratch, (unsigned)rpp, magic);
  na_export_kernel<<<(kd + k + 255) / 256, 256, 0, stream>>>(scratch, kd, k, dSums, dCounts);
  KM_CUDA(cudaGetLastError());
  return KM_OK;
}
