// Host side of the engine: row shards resident on the local devices, the Lloyd
// loop, kernel dispatch.  Replaces kmeans_fit / kmeans_predict / kmeans_transform
// and kmeans::kmeans (src/gpu/kmeans/kmeans_h2o4gpu.cu:617-975,
// src/gpu/kmeans/kmeans_impl.h:45-247).  One host thread drives all local
// devices asynchronously (the reference uses one OpenMP thread per GPU); the
// per-iteration exchange is one NCCL all-reduce of the int64 sums and counts
// instead of the reference's device->host->device staging (kmeans_impl.h:140-188).
#pragma once

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstring>
#include <map>
#include <memory>
#include <atomic>
#include <mutex>
#include <thread>
#include <vector>

#include <cuda_fp16.h>

#include "km_accumulate.cuh"
#include "km_accumulate_sorted.cuh"
#include "km_accumulate_delta.cuh"
#include "km_assign_dmma.cuh"
#include "km_common.cuh"
#include "km_finalize.cuh"
#include "km_nccl.h"
#include "km_push.cuh"
#include "km_refine.cuh"
#include "km_smallk.cuh"
#include "km_smallk_stream.cuh"
#include "km_tc_host.cuh"
#include "km_tiles.cuh"

#include <type_traits>

namespace km {

void log_msg(int verbose, int level, const char* fmt, ...);

struct DevGuard {
  int prev = -1;
  explicit DevGuard(int dev) {
    cudaGetDevice(&prev);
    if (dev != prev) cudaSetDevice(dev);
  }
  ~DevGuard() {
    if (prev >= 0) cudaSetDevice(prev);
  }
};

// Small pinned host blocks (64 bytes: the words the closing kernels publish to the host), kept for
// the life of the process: pinning and unpinning memory costs about a millisecond per engine, a
// visible share of a host-pointer call that builds and tears down an engine around one fit.
struct PinnedWords {
  std::mutex m;
  std::vector<double*> free_list;
  static PinnedWords& get() {
    static PinnedWords* p = new PinnedWords();   // never destroyed: the CUDA runtime may be gone at exit
    return *p;
  }
  double* take() {
    {
      std::lock_guard<std::mutex> lock(m);
      if (!free_list.empty()) {
        double* b = free_list.back();
        free_list.pop_back();
        return b;
      }
    }
    double* b = nullptr;
    if (cudaHostAlloc(&b, 8 * sizeof(double), cudaHostAllocPortable) != cudaSuccess) {
      cudaGetLastError();
      return nullptr;
    }
    return b;
  }
  void give(double* b) {
    if (!b) return;
    std::lock_guard<std::mutex> lock(m);
    free_list.push_back(b);
  }
};

inline double now_s() {
  return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

constexpr size_t kMaxDynSmem = 227 * 1024;

template <typename T>
struct Shard {
  int dev = -1;
  int num_sms = 0;
  int cc_major = 0;
  tc::Plan tcp;  // tensor-core path (float only)
  tcb::BigPlan tcbp;  // tensor-core path for large centroid tables
  tcw::WidePlan tcwp; // tensor-core path for few centroids and wide rows
  tcs::StreamPlan tcsp;  // tensor-core path with both operands streamed: wide rows and many centroids, transform
  unsigned int* amb_rows = nullptr;  // rows handed to the exact re-evaluation pass
  T* xpad = nullptr;                 // rows padded to a multiple of four columns (d % 4 != 0): what TMA can address
  size_t xpad_cap = 0;               // elements
  const T* xpad_of = nullptr;
  size_t xpad_rows = 0;
  size_t amb_cap = 0;
  uint4* amb_near = nullptr;         // per listed row: bit mask of the candidate centroids (small tables)
  size_t amb_near_cap = 0;
  unsigned int* amb_log = nullptr;
  cudaStream_t stream = nullptr;
  const T* X = nullptr;
  T* X_owned = nullptr;
  T* w = nullptr;             // sample weights of the shard's rows (weighted fits), or null
  size_t w_cap = 0;
  void* raw = nullptr;        // bytes of an upload in another element type, until they are converted
  int raw_dtype = -1;
  size_t rows = 0, row0 = 0;
  int* labels = nullptr;
  size_t labels_cap = 0;
  double* dist = nullptr;
  size_t dist_cap = 0;
  // buffers that depend on (k, d)
  int k_cap = 0, d_cap = 0;
  long long* gacc = nullptr;  // [NP/2][k][d] sums followed by [k] counts: one all-reduce covers both
  long long* pacc = nullptr;  // same layout: sums that follow from the labels alone (incremental M-step)
  long long* pflush = nullptr;  // padded drain target of the netting kernels (kFlushPad int64 per entry), or null
  int* labels_prev = nullptr; // labelling pacc corresponds to
  unsigned int* moved_bits = nullptr;  // one bit per row whose label the last E-step moved (tensor-core path)
  bool moved_bits_valid = false;
  size_t labels_prev_cap = 0;
  T* C[2] = {nullptr, nullptr};
  double* Cd[2] = {nullptr, nullptr};  // the same tables in double (float shards; the row-distance kernel reads them)
  T* cnorm = nullptr;
  double* shift_k = nullptr;
  int* empties = nullptr;
  IterState* st = nullptr;
  double* cand_val = nullptr;
  unsigned long long* cand_row = nullptr;
  unsigned int* ticket = nullptr;     // CTAs of the running close_kernel that have finished (zero between launches)
  FarScratch far{};                   // two-pass selection of the farthest rows (empty-cluster repair)
  int far_out_cap = 0;
  unsigned char* reloc_rec = nullptr; // several ranks without the push path: this rank's candidate record ...
  unsigned char* reloc_all = nullptr; // ... and the all-gathered ones (host-driven repair)
  size_t reloc_cap = 0;
  double* sum_partials = nullptr;
  double* shift_log = nullptr;
  unsigned long long* changed_log = nullptr;
  int* reloc_log = nullptr;
  int log_cap = 0;
  double* xstat = nullptr;  // device: [0] max|x| ; int flag behind it
  double* host_pin = nullptr;  // pinned: [0] shift, [1] changed (as u64), [2] n_empty etc.
  ncclComm_t comm = nullptr;
  PushState push;   // one-shot push all-reduce over peer memory (several ranks, small tables)
  bool x_checked = false;
  double xmax = 0;

  long long* sums() const { return gacc; }
  unsigned long long* counts(int k, int d) const {
    return reinterpret_cast<unsigned long long*>(gacc + (size_t)(Fixed<T>::NP / 2) * k * d);
  }
  size_t gacc_count(int k, int d) const { return (size_t)(Fixed<T>::NP / 2) * k * d + k; }
};

struct EngineBase {
  int dtype = 0;
  virtual ~EngineBase() {}
};

template <typename T>
struct Engine : EngineBase {
  std::vector<Shard<T>> shards;
  int world_rank0 = 0, world_size = 1;
  bool comm_cached = false;
  // Communicators of a one-process device set are shared by every engine made for that set; NCCL
  // communicators must not be used from two host threads at once, so an engine holds the set's
  // lock from init() to destroy(): multi-GPU calls on the same devices from several threads
  // run one after the other.
  std::unique_lock<std::mutex> comm_lock;
  size_t n_total = 0;
  int d = 0, k = 0;
  int cur = 0;  // index of the current centroid buffer
  bool have_centroids = false;
  int verbose = 0;
  kmeans_stats stats{};
  int launches = 0;

  ~Engine() { destroy(); }

  int init(int n_local, const int* devs, int rank0, int world, const void* nccl_id);
  void destroy();
  int attach_device(int local, const T* dX, size_t rows, size_t cols, size_t ntot);
  // wait = false: the copies may still be in flight on return (host threads staging a pageable
  // matrix, or DMA from a pinned one); upload_wait() completes them
  int upload_host(const T* X, size_t rows, size_t cols, char order, bool wait = true) {
    return upload_host_typed(X, sizeof(T) == 8 ? KM_DTYPE_F64 : KM_DTYPE_F32, rows, cols, order, wait);
  }
  // the same for a host matrix of any supported element type: the bytes go down as they are
  // and a kernel converts them into T
  int upload_host_typed(const void* X, int src_dtype, size_t rows, size_t cols, char order, bool wait = true);
  int upload_wait();
  // Sample weights of all local rows, shard after shard (null: back to unit weights).  They must
  // be finite and non-negative with a positive maximum.  Attaching other data drops them.
  int set_sample_weight(const T* host_w, size_t count);
  bool weighted = false;
  double wmax = 0;          // largest weight over all ranks
  double w_scale = 1;       // 2^(15 - e), wmax < 2^e: a weight counts as rint(w * w_scale * 2^15) units
  double count_unit = 1;    // weight of one unit of the counts (1 without weights)
  int preallocate(int k_, int max_iter);
  std::vector<std::thread> upload_threads;
  std::atomic<int> upload_error{0};
  double upload_t0 = 0;
  bool upload_pool_locked = false;
  int ensure_buffers(int k_);
  int check_data();
  int set_centroids(int k_, const T* host_c);
  int fit(int k_, int max_iter, double threshold, const T* init, int flags);
  int assign_all(int flags);
  int transform_shard(int local, T* out_host, size_t ld);
  int inertia(double* out);
  int inertia_launch();
  int inertia_collect(double* out);
  int allreduce_acc();
  int relocate_multi(double scale, int seq, int* n_empty);
  // operand table of the tensor-core kernels as close_kernel fills it (null members: not in use)
  SplitTable split_table(Shard<T>& s, bool use_tc);
  int launch_close(Shard<T>& s, int run_if, int it, double inv, bool use_tc);
  int poll_seq = 0;   // sequence number the finalize kernels publish to pinned memory
  bool tc_ok(int flags) const;
  // which tensor-core distance kernel labels this shape: 1 table resident (d 32/64, k <= 128), 2 table streamed
  // (d <= 256), 3 few centroids and wide rows, 4 both operands streamed (wider rows, many centroids), 0 none
  int tc_kind() const {
    if (tcw::wide_shape_ok(k, dtc())) return 3;
    if (d % 4 == 0 && tc::shape_ok(k, d)) return 1;
    if (tcb::big_shape_ok(k, dtc())) return 2;
    if (tcs::stream_shape_ok(k, dtc())) return 4;
    return 0;
  }
  // Rows that are not a multiple of 16 bytes cannot be addressed by TMA: the tensor-core kernels then read a
  // copy of the shard padded with zero columns to dtc() columns (built once per attached matrix; the exact pass,
  // the sums and everything else keep reading the rows as they are).
  int dtc() const { return (d + 3) / 4 * 4; }
  int ensure_xpad(Shard<T>& s);
  const T* xtc(const Shard<T>& s) const { return d % 4 == 0 ? s.X : s.xpad; }
  int stream_refresh(Shard<T>& s);   // operand table and plan of the streaming kernel for the current centroids
  int tc_refresh(Shard<T>& s);  // split the current centroids for the tensor-core kernel
  int launch_assign(Shard<T>& s, bool use_tc, bool count_changes);
  bool tc_split_build = false;   // the running fit has enough iterations to pay for the split copy of X
  float tc_sx = 1.f, tc_sb = 1.f;   // operand scales of the tensor-core kernel
  double cbound = 0;                // bound on |centroid coordinate|: max(|x|, |initial centroids|)

  // launch helpers (device of the shard must be current)
  int launch_tiles(Shard<T>& s, const T* Xp, size_t nrows, int* labels, int mode, T* out, size_t ld_out,
                   bool count_changes);
  int launch_smallk(Shard<T>& s, bool update, T scale);
  // sums of the current labels into dst (default: the working array); with a gate the
  // kernels return at once when the incremental branch has the iteration
  int launch_accumulate(Shard<T>& s, T scale, long long* dst = nullptr, const unsigned long long* gate = nullptr,
                        unsigned long long limit = 0);
  int launch_delta(Shard<T>& s, T scale, const unsigned long long* gate, unsigned long long limit);
  // exact squared distance of every row to its labelled centroid into s.dist
  void launch_rowdist(Shard<T>& s, int force) {
    constexpr int V = VecOf<T>::N;
    const double* cd = std::is_same<T, double>::value ? reinterpret_cast<const double*>(s.C[cur]) : s.Cd[cur];
    const size_t table_bytes = (size_t)k * d * sizeof(double);
    if (vec_ok(s) && table_bytes <= (size_t)96 * 1024) {
      // small tables: gather from a copy in shared memory, as many CTAs per SM as fit beside it
      cudaFuncSetAttribute(rowdist_kernel<T, V, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
      int per_sm = (int)((size_t)200 * 1024 / (table_bytes + 1024));
      per_sm = per_sm > 8 ? 8 : (per_sm < 1 ? 1 : per_sm);
      rowdist_kernel<T, V, true><<<s.num_sms * per_sm, 256, table_bytes, s.stream>>>(s.X, s.rows, d, s.labels, cd,
                                                                                    s.dist, s.st, force, k);
    } else if (vec_ok(s))
      rowdist_kernel<T, V><<<s.num_sms * 8, 256, 0, s.stream>>>(s.X, s.rows, d, s.labels, cd, s.dist, s.st, force);
    else
      rowdist_kernel<T, 1><<<s.num_sms * 8, 256, 0, s.stream>>>(s.X, s.rows, d, s.labels, cd, s.dist, s.st, force);
  }
  // exact pass of the tensor-core kernels that keep no candidate list (all centroids of every listed row)
  int launch_refine_big(Shard<T>& s, bool count_changes) {
    if constexpr (std::is_same<T, float>::value) {
      const size_t smem = (size_t)16 * d;
      if (smem > 48 * 1024)
        KM_CUDA(cudaFuncSetAttribute(tcb::refine_big_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      tcb::refine_big_kernel<<<s.num_sms * 8, tcb::kRefineBigThreads, smem, s.stream>>>(
          s.X, d, s.Cd[cur], k, s.amb_rows, s.st, s.labels, count_changes ? 1 : 0);
      KM_CUDA(cudaGetLastError());
    }
    return KM_OK;
  }
  int allreduce_from(bool from_pure);
  int push_setup(size_t count);
  void push_release();
  bool push_failed = false;   // set-up was tried and is not available: stay with NCCL
  bool smallk_ok(bool update) const;
  bool vec_ok(const Shard<T>& s) const {
    constexpr int V = VecOf<T>::N;
    return (d % V == 0) && ((reinterpret_cast<uintptr_t>(s.X) & 15) == 0);
  }
};

// -------------------------------------------------------------------------------
template <typename T>
int Engine<T>::init(int n_local, const int* devs, int rank0, int world, const void* nccl_id) {
  dtype = sizeof(T) == 8;
  int visible = 0;
  if (cudaGetDeviceCount(&visible) != cudaSuccess || visible == 0) KM_FAIL(KM_ENODEV, "no CUDA device visible");
  if (n_local < 1 || world < n_local || rank0 < 0 || rank0 + n_local > world)
    KM_FAIL(KM_EINVAL, "kmeans_create: bad device / rank layout");
  world_rank0 = rank0;
  world_size = world;
  shards.resize(n_local);
  for (int i = 0; i < n_local; ++i) {
    Shard<T>& s = shards[i];
    s.dev = devs[i];
    if (s.dev < 0 || s.dev >= visible) KM_FAIL(KM_ENODEV, "kmeans_create: device id out of range");
    DevGuard g(s.dev);
    KM_CUDA(cudaDeviceGetAttribute(&s.num_sms, cudaDevAttrMultiProcessorCount, s.dev));
    KM_CUDA(cudaDeviceGetAttribute(&s.cc_major, cudaDevAttrComputeCapabilityMajor, s.dev));
    KM_CUDA(cudaStreamCreateWithFlags(&s.stream, cudaStreamNonBlocking));
    KM_CUDA(km_malloc(&s.st, sizeof(IterState)));
    KM_CUDA(cudaMemset(s.st, 0, sizeof(IterState)));
    KM_CUDA(km_malloc(&s.xstat, 2 * sizeof(double)));
    s.host_pin = PinnedWords::get().take();
    if (!s.host_pin) KM_FAIL(KM_ENOMEM, "kmeans_create: no pinned host memory");
    std::memset(s.host_pin, 0, 8 * sizeof(double));
    KM_CUDA(km_malloc(&s.cand_val, 1024 * sizeof(double)));
    KM_CUDA(km_malloc(&s.cand_row, 2048 * sizeof(unsigned long long)));   // also the exchange buffer of push_setup
    KM_CUDA(km_malloc(&s.sum_partials, 1024 * sizeof(double)));
    KM_CUDA(km_malloc(&s.ticket, sizeof(unsigned int)));
    KM_CUDA(cudaMemset(s.ticket, 0, sizeof(unsigned int)));
    s.far.cap = 32768;
    KM_CUDA(km_malloc(&s.far.tmax, (size_t)s.num_sms * 256 * sizeof(double)));
    KM_CUDA(km_malloc(&s.far.trow, (size_t)s.num_sms * 256 * sizeof(unsigned long long)));
    KM_CUDA(km_malloc(&s.far.cval, (size_t)s.far.cap * sizeof(double)));
    KM_CUDA(km_malloc(&s.far.crow, (size_t)s.far.cap * sizeof(unsigned long long)));
    KM_CUDA(km_malloc(&s.far.counters, 2 * sizeof(unsigned int)));
    KM_CUDA(km_malloc(&s.far.thr, sizeof(double)));
  }
  if (world > 1) {
    NcclApi* api = NcclApi::get();
    if (!api) KM_FAIL(KM_ENCCL, "more than one GPU requested but libnccl.so.2 could not be loaded");
    if (world == n_local) {
      // Communicators of a one-process device set are kept for the life of the process:
      // creating them costs far more than a whole fit, and the reference's entry points
      // are called once per fit / predict.
      struct CommSet { std::vector<ncclComm_t> comms; std::mutex in_use; };
      static std::mutex cache_mutex;
      static std::map<std::vector<int>, std::unique_ptr<CommSet>> cache;   // entries are never removed
      std::vector<int> dl(devs, devs + n_local);
      CommSet* set = nullptr;
      {
        std::lock_guard<std::mutex> lock(cache_mutex);
        auto it = cache.find(dl);
        if (it == cache.end()) it = cache.emplace(dl, std::unique_ptr<CommSet>(new CommSet())).first;
        set = it->second.get();
      }
      comm_lock = std::unique_lock<std::mutex>(set->in_use);
      if (set->comms.empty()) {
        std::vector<ncclComm_t> comms(n_local);
        KM_NCCL(api, api->CommInitAll(comms.data(), n_local, dl.data()));
        set->comms = comms;
      }
      for (int i = 0; i < n_local; ++i) shards[i].comm = set->comms[i];
      comm_cached = true;
    } else {
      if (!nccl_id) KM_FAIL(KM_EINVAL, "kmeans_create: nccl_id required when world_size > n_local");
      ncclUniqueId id;
      std::memcpy(&id, nccl_id, sizeof(id));
      KM_NCCL(api, api->GroupStart());
      for (int i = 0; i < n_local; ++i) {
        DevGuard g(shards[i].dev);
        KM_NCCL(api, api->CommInitRank(&shards[i].comm, world, id, rank0 + i));
      }
      KM_NCCL(api, api->GroupEnd());
    }
  }
  return KM_OK;
}

template <typename T>
void Engine<T>::destroy() {
  upload_wait();
  push_release();
  for (auto& s : shards) {
    if (s.dev < 0) continue;
    DevGuard g(s.dev);
    if (s.stream) cudaStreamSynchronize(s.stream);
    if (s.comm && !comm_cached) {
      NcclApi* api = NcclApi::get();
      if (api) api->CommDestroy(s.comm);
    }
    s.tcp.release();
    s.tcbp.release();
    s.tcwp.release();
    s.tcsp.release();
    km_free(s.amb_rows); km_free(s.amb_near); km_free(s.amb_log); km_free(s.xpad);
    km_free(s.X_owned); km_free(s.raw); km_free(s.w); km_free(s.labels); km_free(s.dist); km_free(s.gacc);
    km_free(s.pacc); km_free(s.pflush); km_free(s.labels_prev); km_free(s.moved_bits);
    km_free(s.C[0]); km_free(s.C[1]); km_free(s.Cd[0]); km_free(s.Cd[1]); km_free(s.cnorm); km_free(s.shift_k); km_free(s.empties);
    km_free(s.st); km_free(s.cand_val); km_free(s.cand_row); km_free(s.sum_partials);
    km_free(s.ticket); km_free(s.reloc_rec); km_free(s.reloc_all);
    km_free(s.far.tmax); km_free(s.far.trow); km_free(s.far.cval); km_free(s.far.crow); km_free(s.far.counters);
    km_free(s.far.thr); km_free(s.far.oval); km_free(s.far.orow);
    km_free(s.shift_log); km_free(s.changed_log); km_free(s.reloc_log); km_free(s.xstat);
    PinnedWords::get().give(s.host_pin);
    s.host_pin = nullptr;
    if (s.stream) cudaStreamDestroy(s.stream);
    s.dev = -1;
  }
  shards.clear();
  if (comm_lock.owns_lock()) comm_lock.unlock();
}

template <typename T>
int Engine<T>::attach_device(int local, const T* dX, size_t rows, size_t cols, size_t ntot) {
  if (local < 0 || local >= (int)shards.size() || !dX || rows == 0 || cols == 0 || cols > (1u << 20))
    KM_FAIL(KM_EINVAL, "kmeans_attach_device: bad argument");
  if (d != 0 && d != (int)cols && local != 0) KM_FAIL(KM_EINVAL, "kmeans_attach_device: shards disagree on cols");
  Shard<T>& s = shards[local];
  DevGuard g(s.dev);
  if (s.X_owned && s.X_owned != dX) { km_free(s.X_owned); s.X_owned = nullptr; }
  s.X = dX;
  s.rows = rows;
  s.x_checked = false;
  weighted = false;
  // what the tensor-core path keeps per matrix (row norms, split copy, tensor maps) belongs to the old one,
  // even when the new one has the same address and shape
  s.tcp.xnorm_of = nullptr;
  s.tcp.xsplit_of = nullptr;
  s.tcp.ready = false;
  s.tcbp.ready = false;
  s.tcwp.ready = false;
  s.tcsp.ready = false;
  s.xpad_of = nullptr;
  if ((int)cols != d) have_centroids = false;
  d = (int)cols;
  n_total = ntot;
  if (s.labels_cap < rows) {
    km_free(s.labels);
    s.labels = nullptr;
    KM_CUDA(km_malloc(&s.labels, rows * sizeof(int)));
    s.labels_cap = rows;
  }
  KM_CUDA(cudaMemsetAsync(s.labels, 0xff, rows * sizeof(int), s.stream));
  return KM_OK;
}

// ---- element types a host matrix may arrive in -----------------------------------
inline size_t dtype_size(int dt) {
  switch (dt) {
    case KM_DTYPE_F32: case KM_DTYPE_I32: case KM_DTYPE_U32: return 4;
    case KM_DTYPE_F64: case KM_DTYPE_I64: case KM_DTYPE_U64: return 8;
    case KM_DTYPE_F16: case KM_DTYPE_I16: case KM_DTYPE_U16: return 2;
    case KM_DTYPE_I8: case KM_DTYPE_U8: return 1;
    default: return 0;
  }
}
// value conversion as numpy's astype does it (round to nearest even where the target is narrower)
template <typename T, typename S> __device__ __forceinline__ T convert_value(S v) { return (T)v; }
template <> __device__ __forceinline__ float convert_value<float, __half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ double convert_value<double, __half>(__half v) { return (double)__half2float(v); }

// src: column-major rows x cols (leading dimension rows) of S -> dst row-major of T
template <typename S, typename T>
__global__ void transpose_cm_kernel(const S* __restrict__ src, T* __restrict__ dst, size_t rows, int cols) {
  __shared__ T tile[32][33];
  size_t r0 = (size_t)blockIdx.x * 32;
  int c0 = blockIdx.y * 32;
  for (int j = threadIdx.y; j < 32; j += 8) {
    size_t r = r0 + threadIdx.x;
    int c = c0 + j;
    if (r < rows && c < cols) tile[j][threadIdx.x] = convert_value<T, S>(src[(size_t)c * rows + r]);
  }
  __syncthreads();
  for (int j = threadIdx.y; j < 32; j += 8) {
    size_t r = r0 + j;
    int c = c0 + threadIdx.x;
    if (r < rows && c < cols) dst[r * (size_t)cols + c] = tile[threadIdx.x][j];
  }
}

// Row-major matrix of S -> T, element by element: replaces the host-side astype copy of the
// wrapper (src/interface_py/h2o4gpu/solvers/utils.py:46-96), which for 8-bit data quadruples the
// bytes that cross the bus.  A thread converts E consecutive elements with one vector load and one
// vector store, so a warp reads and writes contiguous runs (bound by HBM: sizeof(S) + sizeof(T) bytes
// per element); four such groups are in flight per thread.
template <typename X, int E>
struct alignas(E * sizeof(X) > 16 ? 16 : E * sizeof(X)) ElemPack { X e[E]; };

template <typename S, typename T>
__global__ void __launch_bounds__(256)
convert_rm_kernel(const S* __restrict__ src, T* __restrict__ dst, size_t count) {
  constexpr int E = (sizeof(S) >= 8 || sizeof(T) >= 8) ? 2 : 4;
  constexpr int U = 4;
  using PS = ElemPack<S, E>;
  using PT = ElemPack<T, E>;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const bool aligned = (reinterpret_cast<uintptr_t>(src) % sizeof(PS)) == 0 &&
                       (reinterpret_cast<uintptr_t>(dst) % sizeof(PT)) == 0;
  const size_t nvec = aligned ? count / E : 0;
  const PS* vs = reinterpret_cast<const PS*>(src);
  PT* vd = reinterpret_cast<PT*>(dst);
  for (size_t i0 = tid; i0 < nvec; i0 += stride * U) {
    PS in[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const size_t i = i0 + (size_t)u * stride;
      if (i < nvec) in[u] = vs[i];
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const size_t i = i0 + (size_t)u * stride;
      if (i < nvec) {
        PT out;
#pragma unroll
        for (int e = 0; e < E; ++e) out.e[e] = convert_value<T, S>(in[u].e[e]);
        vd[i] = out;
      }
    }
  }
  for (size_t i = nvec * E + tid; i < count; i += stride) dst[i] = convert_value<T, S>(src[i]);
}

template <typename T, typename F>
inline bool dispatch_dtype(int dt, F&& f) {
  switch (dt) {
    case KM_DTYPE_F32: f((const float*)nullptr); return true;
    case KM_DTYPE_F64: f((const double*)nullptr); return true;
    case KM_DTYPE_F16: f((const __half*)nullptr); return true;
    case KM_DTYPE_I8: f((const signed char*)nullptr); return true;
    case KM_DTYPE_U8: f((const unsigned char*)nullptr); return true;
    case KM_DTYPE_I16: f((const short*)nullptr); return true;
    case KM_DTYPE_U16: f((const unsigned short*)nullptr); return true;
    case KM_DTYPE_I32: f((const int*)nullptr); return true;
    case KM_DTYPE_U32: f((const unsigned int*)nullptr); return true;
    case KM_DTYPE_I64: f((const long long*)nullptr); return true;
    case KM_DTYPE_U64: f((const unsigned long long*)nullptr); return true;
    default: return false;
  }
}

// ---- host -> device ingest -----------------------------------------------------
// A pinned (or registered) host matrix goes down in one asynchronous copy per shard.  A pageable
// one - what numpy hands over - would be staged by the driver through a single thread; instead
// worker threads copy 4 MB pieces into pinned buffers (two per worker, so a worker refills
// one while the other is on the bus) and queue them on their own streams.  The buffers live in
// a process-wide pool, created on first use and kept: pinning memory costs more than the copy.
// Replaces the pageable thrust::host_vector staging of copy_data (src/gpu/kmeans/kmeans_h2o4gpu.h:24-42).
struct StagePool {
  static constexpr size_t kPiece = (size_t)4 << 20;
  std::mutex busy;                 // one staged upload at a time
  std::vector<void*> bufs;
  static StagePool& get() {
    static StagePool* p = new StagePool();   // never destroyed: the CUDA runtime may be gone at exit
    return *p;
  }
  int ensure(size_t count) {
    while (bufs.size() < count) {
      void* b = nullptr;
      if (cudaHostAlloc(&b, kPiece, cudaHostAllocPortable) != cudaSuccess) {
        cudaGetLastError();
        return KM_ENOMEM;
      }
      bufs.push_back(b);
    }
    return KM_OK;
  }
};

inline bool host_pointer_is_pageable(const void* p) {
  cudaPointerAttributes a;
  if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
    cudaGetLastError();
    return true;
  }
  return a.type == cudaMemoryTypeUnregistered;
}

// one worker: pieces first, first + stride, ... of the byte range [src, src + bytes) of one shard
inline void stage_worker(int dev, const unsigned char* src, unsigned char* dst, size_t bytes, size_t first,
                         size_t stride, void* buf0, void* buf1, std::atomic<int>* err) {
  cudaStream_t st = nullptr;
  cudaEvent_t ev[2] = {nullptr, nullptr};
  void* buf[2] = {buf0, buf1};
  bool ok = cudaSetDevice(dev) == cudaSuccess && cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking) == cudaSuccess &&
            cudaEventCreateWithFlags(&ev[0], cudaEventDisableTiming) == cudaSuccess &&
            cudaEventCreateWithFlags(&ev[1], cudaEventDisableTiming) == cudaSuccess;
  const size_t piece = StagePool::kPiece;
  const size_t n_pieces = (bytes + piece - 1) / piece;
  size_t q = 0;
  for (size_t j = first; ok && j < n_pieces && err->load() == 0; j += stride, ++q) {
    const size_t off = j * piece, len = std::min(piece, bytes - off);
    const int b = (int)(q & 1);
    if (q >= 2) ok = cudaEventSynchronize(ev[b]) == cudaSuccess;   // the copy that used this buffer is done
    if (!ok) break;
    std::memcpy(buf[b], src + off, len);
    ok = cudaMemcpyAsync(dst + off, buf[b], len, cudaMemcpyHostToDevice, st) == cudaSuccess &&
         cudaEventRecord(ev[b], st) == cudaSuccess;
  }
  if (st && cudaStreamSynchronize(st) != cudaSuccess) ok = false;
  if (ev[0]) cudaEventDestroy(ev[0]);
  if (ev[1]) cudaEventDestroy(ev[1]);
  if (st) cudaStreamDestroy(st);
  if (!ok) err->store(1);
}

template <typename T>
int Engine<T>::upload_host_typed(const void* Xv, int src_dtype, size_t rows, size_t cols, char order, bool wait) {
  TraceRange trace_range("kmeans.upload");
  const size_t esz = dtype_size(src_dtype);
  if (!Xv || rows == 0 || cols == 0 || cols > (1u << 20)) KM_FAIL(KM_EINVAL, "kmeans_upload_host: bad argument");
  if (esz == 0) KM_FAIL(KM_EINVAL, "kmeans_upload_host_typed: unknown element type");
  if (order != 'r' && order != 'c') KM_FAIL(KM_EINVAL, "kmeans_upload_host: order must be 'r' or 'c'");
  if (world_size != (int)shards.size())
    KM_FAIL(KM_ESTATE, "kmeans_upload_host: one process must own all ranks; use kmeans_attach_device");
  KM_TRY(upload_wait());
  const bool native = src_dtype == (sizeof(T) == 8 ? KM_DTYPE_F64 : KM_DTYPE_F32);
  const unsigned char* X = static_cast<const unsigned char*>(Xv);
  upload_t0 = now_s();
  const size_t g = shards.size();
  // balanced contiguous split: shard i holds rows / g rows, the first rows % g shards one more, so no
  // shard is empty whenever rows >= g (a ceil split leaves the last ones empty, e.g. 9 rows on 8 devices)
  const size_t per = rows / g, extra = rows % g;
  static const bool stage_enabled = [] {
    const char* e = std::getenv("H2O4GPU_KM_STAGED_UPLOAD");
    return !(e && e[0] == '0');
  }();
  const bool staged = stage_enabled && order == 'r' && rows * cols * esz >= ((size_t)64 << 20) &&
                      host_pointer_is_pageable(X);
  int workers_per_shard = 0;
  if (staged) {
    // a single core copies far less than the bus carries (about 4 GB/s against 55 GB/s on the
    // hosts measured), so nearly all of them are put to work
    const unsigned hw = std::max(3u, std::thread::hardware_concurrency());
    workers_per_shard = (int)std::max<size_t>(1, std::min<size_t>(14, hw - 2) / g);
    StagePool& pool = StagePool::get();
    pool.busy.lock();
    upload_pool_locked = true;
    if (pool.ensure(2 * workers_per_shard * g) != KM_OK) {
      pool.busy.unlock();
      upload_pool_locked = false;
      workers_per_shard = 0;          // no pinned memory to be had: let the driver stage the copy
    }
  }
  upload_error.store(0);
  size_t off = 0;
  for (size_t i = 0; i < g; ++i) {
    Shard<T>& s = shards[i];
    const size_t r = per + (i < extra ? 1 : 0);
    if (r == 0) { upload_wait(); KM_FAIL(KM_EINVAL, "kmeans_upload_host: fewer rows than devices"); }
    DevGuard gd(s.dev);
    km_free(s.X_owned);
    s.X_owned = nullptr;
    km_free(s.raw);
    s.raw = nullptr;
    // bytes land in the matrix itself when they are T already and row-major, else in a raw
    // buffer that a kernel converts (and transposes) from
    const bool direct = native && order == 'r';
    if (km_malloc(&s.X_owned, r * cols * sizeof(T)) != cudaSuccess ||
        (!direct && km_malloc(&s.raw, r * cols * esz) != cudaSuccess)) {
      cudaGetLastError();
      upload_wait();
      KM_FAIL(KM_ENOMEM, "kmeans_upload_host: device allocation failed");
    }
    s.raw_dtype = src_dtype;
    unsigned char* dst = direct ? reinterpret_cast<unsigned char*>(s.X_owned) : static_cast<unsigned char*>(s.raw);
    if (order == 'r' && workers_per_shard > 0) {
      StagePool& pool = StagePool::get();
      for (int w = 0; w < workers_per_shard; ++w) {
        const size_t b = 2 * (i * workers_per_shard + w);
        upload_threads.emplace_back(stage_worker, s.dev, X + off * cols * esz, dst, r * cols * esz, (size_t)w,
                                    (size_t)workers_per_shard, pool.bufs[b], pool.bufs[b + 1], &upload_error);
      }
    } else if (order == 'r') {
      KM_CUDA(cudaMemcpyAsync(dst, X + off * cols * esz, r * cols * esz, cudaMemcpyHostToDevice, s.stream));
    } else {
      // column-major host matrix (leading dimension = total rows): strided copy of the
      // shard's rows of every column, then a converting transpose on the device
      KM_CUDA(cudaMemcpy2DAsync(dst, r * esz, X + off * esz, rows * esz, r * esz, cols, cudaMemcpyHostToDevice,
                                s.stream));
      dim3 grid((unsigned)((r + 31) / 32), (unsigned)((cols + 31) / 32));
      T* out = s.X_owned;
      cudaStream_t st = s.stream;
      dispatch_dtype<T>(src_dtype, [&](auto* tag) {
        using S = std::remove_cv_t<std::remove_pointer_t<decltype(tag)>>;
        transpose_cm_kernel<S, T><<<grid, dim3(32, 8), 0, st>>>(reinterpret_cast<const S*>(dst), out, r, (int)cols);
      });
      KM_CUDA(cudaGetLastError());
      KM_CUDA(cudaStreamSynchronize(s.stream));
      km_free(s.raw);
      s.raw = nullptr;
    }
    KM_TRY(attach_device((int)i, s.X_owned, r, cols, rows));
    s.row0 = off;
    off += r;
  }
  // a raw row-major buffer is converted once its bytes are down: upload_wait() does that
  bool pending_raw = false;
  for (auto& s : shards) pending_raw = pending_raw || s.raw != nullptr;
  if (wait || pending_raw) return upload_wait();
  return KM_OK;
}

template <typename T>
int Engine<T>::upload_wait() {
  for (auto& t : upload_threads)
    if (t.joinable()) t.join();
  upload_threads.clear();
  if (upload_pool_locked) {
    StagePool::get().busy.unlock();
    upload_pool_locked = false;
  }
  const bool copy_failed = upload_error.load() != 0;
  for (auto& s : shards) {
    if (!s.stream) continue;
    DevGuard gd(s.dev);
    if (s.raw && !copy_failed && s.X_owned) {
      const size_t count = s.rows * (size_t)d;
      T* out = s.X_owned;
      const void* raw = s.raw;
      cudaStream_t st = s.stream;
      const int grid = s.num_sms * 8;
      dispatch_dtype<T>(s.raw_dtype, [&](auto* tag) {
        using S = std::remove_cv_t<std::remove_pointer_t<decltype(tag)>>;
        convert_rm_kernel<S, T><<<grid, 256, 0, st>>>(static_cast<const S*>(raw), out, count);
      });
      KM_CUDA(cudaGetLastError());
    }
    KM_CUDA(cudaStreamSynchronize(s.stream));
    if (s.raw) { km_free(s.raw); s.raw = nullptr; }
  }
  if (upload_t0 > 0) { stats.seconds_upload = now_s() - upload_t0; upload_t0 = 0; }
  if (upload_error.exchange(0) != 0) KM_FAIL(KM_ECUDA, "kmeans_upload_host: a staged copy failed");
  return KM_OK;
}

// Buffers a fit of k clusters will ask for, allocated ahead of time (e.g. while an upload is
// still on the bus); fit() finds them in place.
template <typename T>
int Engine<T>::preallocate(int k_, int max_iter) {
  if (k_ < 1 || d == 0) return KM_OK;
  KM_TRY(ensure_buffers(k_));
  for (auto& s : shards) {
    DevGuard g(s.dev);
    if (s.dist_cap < s.rows && world_size == 1) {
      km_free(s.dist);
      s.dist = nullptr;
      KM_CUDA(km_malloc(&s.dist, s.rows * sizeof(double)));
      s.dist_cap = s.rows;
    }
    if (s.labels_prev_cap < s.rows) {
      km_free(s.labels_prev);
      km_free(s.moved_bits);
      s.labels_prev = nullptr;
      s.moved_bits = nullptr;
      KM_CUDA(km_malloc(&s.labels_prev, s.rows * sizeof(int)));
      KM_CUDA(km_malloc(&s.moved_bits, (s.rows / 32 + 8) * sizeof(unsigned int)));
      s.labels_prev_cap = s.rows;
    }
    if (std::is_same<T, float>::value && s.amb_cap < s.rows) {
      km_free(s.amb_rows);
      s.amb_rows = nullptr;
      KM_CUDA(km_malloc(&s.amb_rows, s.rows * sizeof(unsigned int)));
      s.amb_cap = s.rows;
    }
    if (std::is_same<T, float>::value && tc::shape_ok(k_, d) && s.amb_near_cap < s.rows) {
      km_free(s.amb_near);
      s.amb_near = nullptr;
      KM_CUDA(km_malloc(&s.amb_near, s.rows * sizeof(uint4)));
      s.amb_near_cap = s.rows;
    }
  }
  (void)max_iter;
  return KM_OK;
}

template <typename T>
int Engine<T>::ensure_buffers(int k_) {
  constexpr int NP = Fixed<T>::NP;
  for (auto& s : shards) {
    if (!s.X) KM_FAIL(KM_ESTATE, "no data attached to the handle");
    DevGuard g(s.dev);
    if (s.k_cap != k_ || s.d_cap != d) {
      km_free(s.gacc); km_free(s.pacc); s.pacc = nullptr; km_free(s.pflush); s.pflush = nullptr; km_free(s.C[0]); km_free(s.C[1]); km_free(s.cnorm);
      km_free(s.Cd[0]); km_free(s.Cd[1]); s.Cd[0] = s.Cd[1] = nullptr;
      km_free(s.shift_k); km_free(s.empties);
      s.gacc = nullptr; s.C[0] = s.C[1] = nullptr; s.cnorm = nullptr; s.shift_k = nullptr; s.empties = nullptr;
      size_t kd = (size_t)k_ * d;
      KM_CUDA(km_malloc(&s.gacc, ((size_t)(NP / 2) * kd + k_) * sizeof(long long)));
      KM_CUDA(km_malloc(&s.pacc, ((size_t)(NP / 2) * kd + k_) * sizeof(long long)));
      if (delta_smem_bytes<T>(k_, d) <= 200 * 1024) {
        const size_t fb = ((size_t)(NP / 2) * kd + k_) * kFlushPad * sizeof(long long);
        KM_CUDA(km_malloc(&s.pflush, fb));
        KM_CUDA(cudaMemsetAsync(s.pflush, 0, fb, s.stream));
      }
      KM_CUDA(km_malloc(&s.C[0], kd * sizeof(T)));
      KM_CUDA(km_malloc(&s.C[1], kd * sizeof(T)));
      if (!std::is_same<T, double>::value) {
        KM_CUDA(km_malloc(&s.Cd[0], kd * sizeof(double)));
        KM_CUDA(km_malloc(&s.Cd[1], kd * sizeof(double)));
      }
      KM_CUDA(km_malloc(&s.cnorm, k_ * sizeof(T)));
      KM_CUDA(km_malloc(&s.shift_k, k_ * sizeof(double)));
      KM_CUDA(km_malloc(&s.empties, k_ * sizeof(int)));
      if (s.far_out_cap < k_) {
        km_free(s.far.oval); km_free(s.far.orow);
        s.far.oval = nullptr; s.far.orow = nullptr;
        KM_CUDA(km_malloc(&s.far.oval, (size_t)k_ * sizeof(double)));
        KM_CUDA(km_malloc(&s.far.orow, (size_t)k_ * sizeof(unsigned long long)));
        s.far_out_cap = k_;
      }
      s.k_cap = k_;
      s.d_cap = d;
    }
  }
  return KM_OK;
}

// max of the weights and a flag for a negative or non-finite one
template <typename T>
__global__ void __launch_bounds__(256)
weight_stat_kernel(const T* __restrict__ w, size_t n, double* __restrict__ out_max, int* __restrict__ out_bad) {
  double m = 0;
  int bad = 0;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const double a = (double)w[i];
    bad |= !(a >= 0.0 && a <= 1.7976931348623157e308);
    m = fmax(m, a);
  }
  m = warp_max(m);
  bad = __any_sync(0xffffffffu, bad);
  if ((threadIdx.x & 31) == 0) {
    if (m > 0) atomicMax(reinterpret_cast<unsigned long long*>(out_max), (unsigned long long)__double_as_longlong(m));
    if (bad) atomicOr(out_bad, 1);
  }
}

template <typename T>
int Engine<T>::set_sample_weight(const T* host_w, size_t count) {
  if (!host_w) { weighted = false; return KM_OK; }
  size_t local = 0;
  for (auto& s : shards) {
    if (!s.X) KM_FAIL(KM_ESTATE, "kmeans_set_sample_weight: attach the data first");
    local += s.rows;
  }
  if (count != local) KM_FAIL(KM_EINVAL, "kmeans_set_sample_weight: one weight per local row expected");
  weighted = false;   // a refused set of weights leaves unit weights behind
  KM_TRY(upload_wait());
  size_t off = 0;
  for (auto& s : shards) {
    DevGuard g(s.dev);
    if (s.w_cap < s.rows) {
      km_free(s.w);
      s.w = nullptr;
      KM_CUDA(km_malloc(&s.w, s.rows * sizeof(T)));
      s.w_cap = s.rows;
    }
    KM_CUDA(cudaMemcpyAsync(s.w, host_w + off, s.rows * sizeof(T), cudaMemcpyHostToDevice, s.stream));
    KM_CUDA(cudaMemsetAsync(s.xstat, 0, 2 * sizeof(double), s.stream));
    weight_stat_kernel<T><<<s.num_sms * 4, 256, 0, s.stream>>>(s.w, s.rows, s.xstat, reinterpret_cast<int*>(s.xstat + 1));
    KM_CUDA(cudaGetLastError());
    off += s.rows;
  }
  if (world_size > 1) {
    NcclApi* api = NcclApi::get();
    KM_NCCL(api, api->GroupStart());
    for (auto& s : shards) KM_NCCL(api, api->AllReduce(s.xstat, s.xstat, 2, ncclDouble, ncclMax, s.comm, s.stream));
    KM_NCCL(api, api->GroupEnd());
  }
  double m = 0;
  for (auto& s : shards) {
    DevGuard g(s.dev);
    double h[2];
    KM_CUDA(cudaMemcpyAsync(h, s.xstat, sizeof(h), cudaMemcpyDeviceToHost, s.stream));
    KM_CUDA(cudaStreamSynchronize(s.stream));
    long long flag;
    std::memcpy(&flag, &h[1], sizeof(flag));
    if (flag != 0) KM_FAIL(KM_EINVAL, "sample weights must be finite and non-negative");
    m = std::max(m, h[0]);
  }
  if (!(m > 0)) KM_FAIL(KM_EINVAL, "sample weights are all zero");
  int e = 0;
  std::frexp(m, &e);
  if (sizeof(T) == 4 && (e > 100 || e < -100)) KM_FAIL(KM_EINVAL, "sample weights outside the supported range");
  wmax = m;
  w_scale = std::ldexp(1.0, kPieceBits - e);
  count_unit = std::ldexp(1.0, -(2 * kPieceBits - e));
  weighted = true;
  return KM_OK;
}

// max |x| over all ranks (sets the fixed-point scale) and the finiteness check
// the wrapper's do_checks performs on the host
// (src/interface_py/h2o4gpu/solvers/utils.py:144-158).
template <typename T>
int Engine<T>::check_data() {
  TraceRange trace_range("kmeans.check_data");
  bool all = true;
  for (auto& s : shards) all = all && s.x_checked;
  if (all) return KM_OK;
  constexpr int V = VecOf<T>::N;
  for (auto& s : shards) {
    DevGuard g(s.dev);
    KM_CUDA(cudaMemsetAsync(s.xstat, 0, 2 * sizeof(double), s.stream));
    size_t count = s.rows * (size_t)d;
    int grid = s.num_sms * 8;
    if ((reinterpret_cast<uintptr_t>(s.X) & 15) == 0)
      absmax_kernel<T, V><<<grid, 256, 0, s.stream>>>(s.X, count, s.xstat, reinterpret_cast<int*>(s.xstat + 1));
    else
      absmax_kernel<T, 1><<<grid, 256, 0, s.stream>>>(s.X, count, s.xstat, reinterpret_cast<int*>(s.xstat + 1));
    KM_CUDA(cudaGetLastError());
    ++launches;
  }
  if (world_size > 1) {
    NcclApi* api = NcclApi::get();
    KM_NCCL(api, api->GroupStart());
    for (auto& s : shards) {
      // both words are non-negative: max as doubles is right for the max and for the flag
      KM_NCCL(api, api->AllReduce(s.xstat, s.xstat, 2, ncclDouble, ncclMax, s.comm, s.stream));
    }
    KM_NCCL(api, api->GroupEnd());
  }
  for (auto& s : shards) {
    DevGuard g(s.dev);
    double h[2];
    KM_CUDA(cudaMemcpyAsync(h, s.xstat, sizeof(h), cudaMemcpyDeviceToHost, s.stream));
    KM_CUDA(cudaStreamSynchronize(s.stream));
    long long flag;
    std::memcpy(&flag, &h[1], sizeof(flag));
    if (flag != 0 || !(h[0] <= 1.7e308)) KM_FAIL(KM_ENONFINITE, "input data contains NaN or Inf");
    s.xmax = h[0];
    s.x_checked = true;
  }
  return KM_OK;
}

template <typename T>
int Engine<T>::set_centroids(int k_, const T* host_c) {
  if (k_ < 1 || !host_c) KM_FAIL(KM_EINVAL, "kmeans_set_centroids: bad argument");
  if (d == 0) KM_FAIL(KM_ESTATE, "kmeans_set_centroids: attach data first (defines cols)");
  double cmax = 0;
  for (size_t i = 0; i < (size_t)k_ * d; ++i) {
    if (!std::isfinite((double)host_c[i])) KM_FAIL(KM_ENONFINITE, "centroids contain NaN or Inf");
    cmax = std::max(cmax, std::fabs((double)host_c[i]));
  }
  cbound = cmax;
  KM_TRY(ensure_buffers(k_));
  k = k_;
  cur = 0;
  for (auto& s : shards) {
    DevGuard g(s.dev);
    KM_CUDA(cudaMemcpyAsync(s.C[0], host_c, (size_t)k * d * sizeof(T), cudaMemcpyHostToDevice, s.stream));
    cnorm_kernel<T><<<k, 128, 0, s.stream>>>(s.C[0], k, d, s.cnorm, s.Cd[0]);
    KM_CUDA(cudaGetLastError());
    ++launches;
    // host_c may be freed by the caller right after this returns
    KM_CUDA(cudaStreamSynchronize(s.stream));
  }
  have_centroids = true;
  return KM_OK;
}

// ---- kernel dispatch -----------------------------------------------------------
template <typename T, int BM, int BN, int BK, int TM, int TN>
static int launch_tile_cfg(const T* X, size_t n, int d, const T* C, int k, const T* cnorm, int* labels,
                           IterState* st, T* out, size_t ld_out, int mode, bool vec, cudaStream_t stream) {
  constexpr int V = VecOf<T>::N;
  constexpr int NT = (BM / TM) * (BN / TN);
  size_t grid = (n + BM - 1) / BM;
  if (grid > 0x7fffffffULL) KM_FAIL(KM_EINVAL, "shard too large for one launch");
  if (mode == MODE_ASSIGN) {
    if (vec) tile_kernel<T, BM, BN, BK, TM, TN, V, MODE_ASSIGN><<<(unsigned)grid, NT, 0, stream>>>(X, n, d, C, k, cnorm, labels, st, out, ld_out);
    else tile_kernel<T, BM, BN, BK, TM, TN, 1, MODE_ASSIGN><<<(unsigned)grid, NT, 0, stream>>>(X, n, d, C, k, cnorm, labels, st, out, ld_out);
  } else {
    if (vec) tile_kernel<T, BM, BN, BK, TM, TN, V, MODE_TRANSFORM><<<(unsigned)grid, NT, 0, stream>>>(X, n, d, C, k, cnorm, labels, st, out, ld_out);
    else tile_kernel<T, BM, BN, BK, TM, TN, 1, MODE_TRANSFORM><<<(unsigned)grid, NT, 0, stream>>>(X, n, d, C, k, cnorm, labels, st, out, ld_out);
  }
  KM_CUDA(cudaGetLastError());
  return KM_OK;
}

template <typename T> struct TileCfg;
template <> struct TileCfg<float> {
  static int go(const float* X, size_t n, int d, const float* C, int k, const float* cn, int* lab, IterState* st,
                float* out, size_t ld, int mode, bool vec, cudaStream_t s) {
    if (k <= 64) return launch_tile_cfg<float, 128, 64, 16, 8, 4>(X, n, d, C, k, cn, lab, st, out, ld, mode, vec, s);
    return launch_tile_cfg<float, 128, 128, 16, 8, 8>(X, n, d, C, k, cn, lab, st, out, ld, mode, vec, s);
  }
};
template <> struct TileCfg<double> {
  static int go(const double* X, size_t n, int d, const double* C, int k, const double* cn, int* lab, IterState* st,
                double* out, size_t ld, int mode, bool vec, cudaStream_t s) {
    // labels for more than a few centroids: the float64 matrix unit (km_assign_dmma.cuh)
    static const bool dmma_env = [] {
      const char* e = std::getenv("H2O4GPU_KM_DMMA");
      return !(e && e[0] == '0');
    }();
    if (dmma_env && mode == MODE_ASSIGN && vec && dmma::shape_ok(k, d) && (reinterpret_cast<uintptr_t>(C) & 15) == 0)
      return dmma::launch(X, n, d, C, k, cn, lab, st, s);
    return launch_tile_cfg<double, 64, 64, 16, 4, 4>(X, n, d, C, k, cn, lab, st, out, ld, mode, vec, s);
  }
};

template <typename T>
int Engine<T>::launch_tiles(Shard<T>& s, const T* Xp, size_t nrows, int* labels, int mode, T* out,
                            size_t ld_out, bool count_changes) {
  bool vec = (d % VecOf<T>::N == 0) && ((reinterpret_cast<uintptr_t>(Xp) & 15) == 0);
  ++launches;
  return TileCfg<T>::go(Xp, nrows, d, s.C[cur], k, s.cnorm, labels, count_changes ? s.st : nullptr, out, ld_out,
                        mode, vec, s.stream);
}

template <typename T, int V>
using SmallKFn = void (*)(const T*, size_t, int, const T*, int, const T*, int*, IterState*, long long*,
                          unsigned long long*, T, int, unsigned int);

template <typename T, int V, int RPW>
static SmallKFn<T, V> smallk_pick(int k, int* K) {
  // more rows per group only while the K x RPW dot products fit the register budget
#define KM_PICK(KK) if (k <= KK) { *K = KK; return smallk_kernel<T, KK, V, (KK <= 10 ? RPW : kSmallKRpw)>; }
  KM_PICK(1) KM_PICK(2) KM_PICK(3) KM_PICK(4) KM_PICK(5) KM_PICK(6) KM_PICK(8) KM_PICK(10) KM_PICK(12)
#undef KM_PICK
  *K = 16;
  return smallk_kernel<T, 16, V, kSmallKRpw>;
}
inline int smallk_bound(int k) {
  const int ks[] = {1, 2, 3, 4, 5, 6, 8, 10, 12, 16};
  for (int v : ks) if (k <= v) return v;
  return 16;
}

template <typename T>
bool Engine<T>::smallk_ok(bool update) const {
  if (k > 16) return false;
  const size_t smem = smallk_smem_bytes<T>(smallk_bound(k), d, update);
  // The fused step keeps fixed-point accumulators of the whole table in shared memory: good
  // while they are small (several CTAs per SM stay resident); for wide rows the E-step runs
  // alone and the sums come from the run-length / incremental kernels.
  if (update) return smem <= 48 * 1024;
  return smem <= kMaxDynSmem;
}

template <typename T>
int Engine<T>::launch_smallk(Shard<T>& s, bool update, T scale) {
  constexpr int V = VecOf<T>::N;
  int K = 0;
  bool vec = vec_ok(s);
  size_t smem;
  // rows per CTA: enough CTAs to fill the GPU twice over, never more rows than
  // the int32 accumulators can hold
  size_t target = (size_t)s.num_sms * 4;
  size_t rpc = (s.rows + target - 1) / target;
  rpc = std::max<size_t>(rpc, 512);
  rpc = std::min<size_t>(rpc, kFlushRows);
  size_t grid = (s.rows + rpc - 1) / rpc;
  cudaError_t e;
  if (vec) {
    auto fn = update ? smallk_pick<T, V, kSmallKRpw>(k, &K) : smallk_pick<T, V, kSmallKRpwAssign>(k, &K);
    smem = smallk_smem_bytes<T>(K, d, update);
    e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) KM_CUDA(e);
    // without this the driver sizes the shared-memory carve-out for one CTA and only one is resident
    cudaFuncSetAttribute(fn, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    fn<<<(unsigned)grid, kSmallKThreads, smem, s.stream>>>(s.X, s.rows, d, s.C[cur], k, s.cnorm, s.labels, s.st,
                                                          s.sums(), s.counts(k, d), scale, update ? 1 : 0,
                                                          (unsigned)rpc);
  } else {
    auto fn = update ? smallk_pick<T, 1, kSmallKRpw>(k, &K) : smallk_pick<T, 1, kSmallKRpwAssign>(k, &K);
    smem = smallk_smem_bytes<T>(K, d, update);
    e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) KM_CUDA(e);
    cudaFuncSetAttribute(fn, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    fn<<<(unsigned)grid, kSmallKThreads, smem, s.stream>>>(s.X, s.rows, d, s.C[cur], k, s.cnorm, s.labels, s.st,
                                                          s.sums(), s.counts(k, d), scale, update ? 1 : 0,
                                                          (unsigned)rpc);
  }
  KM_CUDA(cudaGetLastError());
  ++launches;
  return KM_OK;
}

template <int GS, int VPT>
static int launch_sorted_gs(const float* X, size_t rows, int d, const int* labels, int k, long long* gs,
                            unsigned long long* gc, float scale30, const SortPlan& p, cudaStream_t stream,
                            const unsigned long long* gate, unsigned long long limit) {
  KM_CUDA(cudaFuncSetAttribute(sorted_accumulate_kernel<GS, VPT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               (int)p.smem_bytes));
  sorted_accumulate_kernel<GS, VPT><<<p.grid, kSortThreads, p.smem_bytes, stream>>>(
      X, rows, d, labels, k, gs, gc, scale30, p.tile_rows, p.smem_acc, gate, limit);
  KM_CUDA(cudaGetLastError());
  return KM_OK;
}

// float shards with 16-byte rows: run-length kernel.  `scale` is 2^(15-e); the
// run-length kernel quantises with 2^(30-e) in one step, which gives the same integers.
template <typename T>
static int try_sorted_accumulate(Shard<T>& s, int d, int k, T scale, bool vec, bool* done, long long* gs,
                                 unsigned long long* gc, const unsigned long long* gate, unsigned long long limit) {
  *done = false;
  if constexpr (std::is_same<T, float>::value) {
    static const bool enabled = [] {
      const char* e = std::getenv("H2O4GPU_KM_ACC_SORTED");
      return !(e && e[0] == '0');
    }();
    SortPlan p;
    if (!enabled || !vec || !sorted_accumulate_plan(s.rows, d, k, s.num_sms, kMaxDynSmem, &p)) return KM_OK;
    const float scale30 = scale * 32768.0f;
    const int dv = d / 4;
    int rc;
    // two float4 per thread and row for rows wider than 256 columns (measured: 210 -> 175 us on 250,000 x 784;
    // on 64 and 128 columns the same change doubled the time - twice as many groups walk shorter pieces
    // of the sorted list)
    if (dv <= 8) rc = launch_sorted_gs<8, 1>(s.X, s.rows, d, s.labels, k, gs, gc, scale30, p, s.stream, gate, limit);
    else if (dv <= 16) rc = launch_sorted_gs<16, 1>(s.X, s.rows, d, s.labels, k, gs, gc, scale30, p, s.stream, gate, limit);
    else if (dv <= 32) rc = launch_sorted_gs<32, 1>(s.X, s.rows, d, s.labels, k, gs, gc, scale30, p, s.stream, gate, limit);
    else if (dv <= 64) rc = launch_sorted_gs<64, 1>(s.X, s.rows, d, s.labels, k, gs, gc, scale30, p, s.stream, gate, limit);
    else if (dv <= 128) rc = launch_sorted_gs<64, 2>(s.X, s.rows, d, s.labels, k, gs, gc, scale30, p, s.stream, gate, limit);
    else if (dv <= 256) rc = launch_sorted_gs<128, 2>(s.X, s.rows, d, s.labels, k, gs, gc, scale30, p, s.stream, gate, limit);
    else rc = launch_sorted_gs<256, 2>(s.X, s.rows, d, s.labels, k, gs, gc, scale30, p, s.stream, gate, limit);   // d <= 2048 (the plan's bound)
    KM_TRY(rc);
    *done = true;
  }
  return KM_OK;
}

template <typename T>
int Engine<T>::launch_accumulate(Shard<T>& s, T scale, long long* dst, const unsigned long long* gate,
                                 unsigned long long limit) {
  constexpr int V = VecOf<T>::N;
  constexpr int NP = Fixed<T>::NP;
  long long* gs = dst ? dst : s.sums();
  unsigned long long* gc = reinterpret_cast<unsigned long long*>(gs + (size_t)(NP / 2) * k * d);
  const T* W = weighted ? s.w : nullptr;
  if (!W) {
    bool done = false;
    KM_TRY(try_sorted_accumulate<T>(s, d, k, scale, vec_ok(s), &done, gs, gc, gate, limit));
    if (done) { ++launches; return KM_OK; }
  }
  const size_t per_cluster = (size_t)NP * d * sizeof(int) + 2 * sizeof(int);
  const size_t budget = 200 * 1024;
  if (per_cluster + 16 > budget) KM_FAIL(KM_EINVAL, "cols too large for the centroid-sum kernel");
  int kc_max = (int)((budget - 16) / per_cluster);
  int n_slices = (k + kc_max - 1) / kc_max;
  int kc = (k + n_slices - 1) / n_slices;
  size_t smem = accumulate_smem_bytes<T>(kc, d);
  int per_sm = (int)std::max<size_t>(1, std::min<size_t>(4, kMaxDynSmem / (smem + 1024)));
  size_t target = (size_t)s.num_sms * per_sm;
  size_t rpp = (s.rows + target - 1) / target;
  rpp = std::max<size_t>(rpp, 1024);
  rpp = std::min<size_t>(rpp, kFlushRows);
  size_t parts = (s.rows + rpp - 1) / rpp;
  size_t grid = parts * n_slices;
  if (grid > 0x7fffffffULL) KM_FAIL(KM_EINVAL, "shard too large for one launch");
  bool vec = vec_ok(s);
  int dv = vec ? d / V : d;
  if ((unsigned long long)rpp * dv * dv >= (1ULL << 40)) KM_FAIL(KM_EINVAL, "cols too large for the centroid-sum kernel");
  unsigned long long magic = fastdiv_magic((unsigned)dv);
  if (vec) {
    KM_CUDA(cudaFuncSetAttribute(accumulate_kernel<T, V>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    accumulate_kernel<T, V><<<(unsigned)grid, kAccThreads, smem, s.stream>>>(
        s.X, s.rows, d, s.labels, k, kc, n_slices, gs, gc, scale, (unsigned)rpp, magic, gate, limit, W, (T)w_scale);
  } else {
    KM_CUDA(cudaFuncSetAttribute(accumulate_kernel<T, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    accumulate_kernel<T, 1><<<(unsigned)grid, kAccThreads, smem, s.stream>>>(
        s.X, s.rows, d, s.labels, k, kc, n_slices, gs, gc, scale, (unsigned)rpp, magic, gate, limit, W, (T)w_scale);
  }
  KM_CUDA(cudaGetLastError());
  ++launches;
  return KM_OK;
}

// The tcgen05 kernel serves float32 shards with d in {32, 64} and 16 < k <= 128 on
// compute capability 10.x; everything else runs on the SIMT kernels.
template <typename T>
bool Engine<T>::tc_ok(int flags) const {
  if (!std::is_same<T, float>::value || (flags & KM_FIT_FORCE_SIMT)) return false;
  if (tc_kind() == 0) return false;
  for (const auto& s : shards) {
    if (s.cc_major != 10 || !s.x_checked) return false;
    if (d % 4 == 0) {
      if ((reinterpret_cast<uintptr_t>(s.X) & 15) != 0) return false;
    } else if (!(s.xpad && s.xpad_cap >= s.rows * (size_t)dtc())) {
      // the padded copy must fit beside the shard (with room to spare for the fit's own buffers)
      size_t free_b = 0, total_b = 0;
      DevGuard g(s.dev);
      if (cudaMemGetInfo(&free_b, &total_b) != cudaSuccess) return false;
      if (free_b < s.rows * (size_t)dtc() * sizeof(T) + ((size_t)1 << 30)) return false;
    }
  }
  double xmax = 0;
  for (const auto& s : shards) xmax = std::max(xmax, s.xmax);
  float sx, sb;
  return tc::pick_scales(xmax, std::max(xmax, cbound), &sx, &sb);
}

template <typename T>
int Engine<T>::tc_refresh(Shard<T>& s) {
  if constexpr (std::is_same<T, float>::value) {
    double xmax = 0;
    for (const auto& sh : shards) xmax = std::max(xmax, sh.xmax);
    if (!tc::pick_scales(xmax, std::max(xmax, cbound), &tc_sx, &tc_sb))
      KM_FAIL(KM_EINVAL, "data magnitude outside the range of the tensor-core kernel");
    if (s.rows > 0xffffffffULL) KM_FAIL(KM_EINVAL, "shard too large for the tensor-core kernel");
    if (s.amb_cap < s.rows) {
      km_free(s.amb_rows);
      s.amb_rows = nullptr;
      KM_CUDA(km_malloc(&s.amb_rows, s.rows * sizeof(unsigned int)));
      s.amb_cap = s.rows;
    }
    if (tc_kind() == 1 && s.amb_near_cap < s.rows) {
      km_free(s.amb_near);
      s.amb_near = nullptr;
      KM_CUDA(km_malloc(&s.amb_near, s.rows * sizeof(uint4)));
      s.amb_near_cap = s.rows;
    }
    const int kind = tc_kind();
    if (d % 4 != 0) KM_TRY(ensure_xpad(s));
    if (kind == 3) {
      KM_TRY(tc::ensure_xnorm(s.tcp, xtc(s), s.rows, dtc(), s.num_sms, s.stream));   // float4 loads: the aligned rows
      KM_TRY(tcw::wide_setup(s.tcwp, xtc(s), s.rows, k, d, dtc()));
      s.tcwp.sx = tc_sx;
      s.tcwp.sb = tc_sb;
      KM_TRY(tcw::wide_prep(s.tcwp, s.C[cur], s.cnorm, s.stream));
    } else if (kind == 4) {
      KM_TRY(stream_refresh(s));
    } else if (kind == 1) {
      KM_TRY(tc::setup(s.tcp, s.X, s.rows, k, d, s.num_sms, s.stream));
      s.tcp.sx = tc_sx;
      s.tcp.sb = tc_sb;
      KM_TRY(tc::prep(s.tcp, s.C[cur], s.cnorm, s.stream));
    } else {
      KM_TRY(tc::ensure_xnorm(s.tcp, xtc(s), s.rows, dtc(), s.num_sms, s.stream));   // float4 loads: the aligned rows
      KM_TRY(tcb::big_setup(s.tcbp, xtc(s), s.rows, k, d, dtc()));
      s.tcbp.sx = tc_sx;
      s.tcbp.sb = tc_sb;
      KM_TRY(tcb::big_prep(s.tcbp, s.C[cur], s.cnorm, s.stream));
    }
    ++launches;
  }
  return KM_OK;
}

template <typename T>
__global__ void __launch_bounds__(256)
pad_rows_kernel(const T* __restrict__ X, size_t rows, int d, int dp, T* __restrict__ out) {
  const size_t total = rows * (size_t)dp;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / dp;
    const int t = (int)(i - r * dp);
    out[i] = t < d ? X[r * (size_t)d + t] : (T)0;
  }
}

template <typename T>
int Engine<T>::ensure_xpad(Shard<T>& s) {
  if (s.xpad_of == s.X && s.xpad_rows == s.rows && s.xpad) return KM_OK;
  const size_t need = s.rows * (size_t)dtc();
  if (s.xpad_cap < need) {
    km_free(s.xpad);
    s.xpad = nullptr;
    s.xpad_cap = 0;
    KM_CUDA(km_malloc(&s.xpad, need * sizeof(T)));
    s.xpad_cap = need;
  }
  pad_rows_kernel<T><<<s.num_sms * 16, 256, 0, s.stream>>>(s.X, s.rows, d, dtc(), s.xpad);
  KM_CUDA(cudaGetLastError());
  ++launches;
  s.xpad_of = s.X;
  s.xpad_rows = s.rows;
  return KM_OK;
}

template <typename T>
int Engine<T>::stream_refresh(Shard<T>& s) {
  if constexpr (std::is_same<T, float>::value) {
    if (d % 4 != 0) KM_TRY(ensure_xpad(s));
    KM_TRY(tc::ensure_xnorm(s.tcp, xtc(s), s.rows, dtc(), s.num_sms, s.stream));   // float4 loads: the aligned rows
    KM_TRY(tcs::stream_setup(s.tcsp, xtc(s), s.rows, k, d, dtc()));
    s.tcsp.sx = tc_sx;
    s.tcsp.sb = tc_sb;
    KM_TRY(tcs::stream_prep(s.tcsp, s.C[cur], s.cnorm, s.stream));
  }
  return KM_OK;
}

template <typename T>
int Engine<T>::launch_assign(Shard<T>& s, bool use_tc, bool count_changes) {
  if constexpr (std::is_same<T, float>::value) {
    if (use_tc && tc_kind() == 4) {
      launches += 2;
      KM_TRY(tcs::stream_launch(s.tcsp, s.tcp.xnorm, s.labels, s.st, count_changes, s.amb_rows, tc::tol_rel_of(d), s.num_sms,
                                s.stream));
      KM_TRY(launch_refine_big(s, count_changes));
      KM_CUDA(cudaGetLastError());
      return KM_OK;
    }
    if (use_tc && tc_kind() == 3) {
      launches += 2;
      KM_TRY(tcw::wide_launch(s.tcwp, s.tcp.xnorm, s.labels, s.st, count_changes, s.amb_rows, tc::tol_rel_of(d), s.num_sms,
                              s.stream));
      KM_TRY(launch_refine_big(s, count_changes));
      KM_CUDA(cudaGetLastError());
      return KM_OK;
    }
    if (use_tc && tc_kind() == 2) {
      launches += 2;
      KM_TRY(tcb::big_launch(s.tcbp, s.tcp.xnorm, s.labels, s.st, count_changes, s.amb_rows, tc::tol_rel_of(d), s.num_sms,
                             s.stream));
      KM_TRY(launch_refine_big(s, count_changes));
      KM_CUDA(cudaGetLastError());
      return KM_OK;
    }
    if (use_tc) {
      launches += 2;
      unsigned int* bits = (count_changes && s.labels_prev_cap >= s.rows) ? s.moved_bits : nullptr;
      KM_TRY(tc::launch(s.tcp, s.labels, s.st, count_changes, s.amb_rows, tc::tol_rel_of(d), s.num_sms,
                        s.stream, bits, s.amb_near, tc_split_build));
      s.moved_bits_valid = bits != nullptr;
      refine_near_kernel<float><<<s.num_sms * 4, kRefineThreads, 0, s.stream>>>(
          s.X, d, s.C[cur], k, s.amb_rows, s.amb_near, s.st, s.labels, count_changes ? 1 : 0, bits);
      KM_CUDA(cudaGetLastError());
      return KM_OK;
    }
  }
  if constexpr (std::is_same<T, float>::value) {
    // few centroids, wide rows: the streaming small-k kernel
    const int K = (k + 3) / 4 * 4;
    if (k <= 16 && d >= 128 && vec_ok(s) && sks::smem_bytes(K, d) <= kMaxDynSmem) {
      const size_t smem = sks::smem_bytes(K, d);
      const size_t tiles = (s.rows + sks::kRows - 1) / sks::kRows;
      const int grid = (int)std::min<size_t>(tiles, (size_t)s.num_sms);
      IterState* stp = count_changes ? s.st : nullptr;
      auto go = [&](auto fn) -> int {
        KM_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        fn<<<grid, sks::kThreads, smem, s.stream>>>(s.X, s.rows, d, s.C[cur], k, s.cnorm, s.labels, stp);
        KM_CUDA(cudaGetLastError());
        ++launches;
        return KM_OK;
      };
      if (K == 4) return go(sks::assign_stream_kernel<4>);
      if (K == 8) return go(sks::assign_stream_kernel<8>);
      if (K == 12) return go(sks::assign_stream_kernel<12>);
      return go(sks::assign_stream_kernel<16>);
    }
  }
  if (smallk_ok(false)) {
    IterState* keep = s.st;
    if (!count_changes) s.st = nullptr;
    const int rc = launch_smallk(s, false, (T)1);
    s.st = keep;
    return rc;
  }
  return launch_tiles(s, s.X, s.rows, s.labels, MODE_ASSIGN, nullptr, 0, count_changes);
}

template <typename T>
int Engine<T>::allreduce_acc() { return allreduce_from(false); }

// Sums and counts of all ranks into the working array, read from the working array itself
// or from the label-only sums of the incremental M-step.
template <typename T>
int Engine<T>::allreduce_from(bool from_pure) {
  if (world_size <= 1) return KM_OK;
  {
    const size_t count = shards[0].gacc_count(k, d);
    static const bool push_env = [] {
      const char* e = std::getenv("H2O4GPU_KM_PUSH_ALLREDUCE");
      return !(e && e[0] == '0');
    }();
    if (push_env && !push_failed && count * sizeof(long long) <= kPushMaxBytes) {
      const size_t gslot = (((size_t)k * 32 + (size_t)k * d * sizeof(T)) + 15) / 16 * 16;
      if (!shards[0].push.ready || shards[0].push.count != count || shards[0].push.gslot != gslot) {
        if (push_setup(count) != KM_OK) { push_release(); push_failed = true; }
      }
      if (!push_failed) {
        const unsigned int seq = (unsigned int)poll_seq;   // one value per iteration, the same on every rank
        for (size_t i = 0; i < shards.size(); ++i) {
          Shard<T>& s = shards[i];
          DevGuard g(s.dev);
          push_allreduce_kernel<<<kPushCtas, kPushThreads, 0, s.stream>>>(
              from_pure ? s.pacc : s.gacc, s.gacc, count, world_rank0 + (int)i, world_size, s.push.d_peer_mailbox,
              s.push.d_peer_flags, s.push.mailbox, s.push.flags, s.push.done, seq, s.st, wait_limits().push_spins);
          KM_CUDA(cudaGetLastError());
          ++launches;
        }
        stats.allreduce_path = 1;
        return KM_OK;
      }
    }
  }
  NcclApi* api = NcclApi::get();
  KM_NCCL(api, api->GroupStart());
  for (auto& s : shards)
    KM_NCCL(api, api->AllReduce(from_pure ? s.pacc : s.gacc, s.gacc, s.gacc_count(k, d), ncclInt64, ncclSum, s.comm,
                                s.stream));
  KM_NCCL(api, api->GroupEnd());
  stats.allreduce_path = 2;
  return KM_OK;
}

template <typename T>
int Engine<T>::launch_delta(Shard<T>& s, T scale, const unsigned long long* gate, unsigned long long limit) {
  constexpr int V = VecOf<T>::N;
  constexpr int NP = Fixed<T>::NP;
  long long* ps = s.pacc;
  unsigned long long* pc = reinterpret_cast<unsigned long long*>(ps + (size_t)(NP / 2) * k * d);
  // the shared-memory netting kernels drain into the padded array (counts behind the sums)
  long long* fs = s.pflush;
  unsigned long long* fc = reinterpret_cast<unsigned long long*>(fs + (size_t)(NP / 2) * k * d * kFlushPad);
  const size_t smem = delta_smem_bytes<T>(k, d);
  static const bool bitmap_env = [] {
    const char* e = std::getenv("H2O4GPU_KM_DELTA_BITMAP");
    return e && e[0] == '1';
  }();
  const T* W = weighted ? s.w : nullptr;
  const T wsc = (T)w_scale;
  if (bitmap_env && !W && s.pflush && smem <= 100 * 1024 && s.moved_bits_valid && vec_ok(s)) {
    // the E-step left a map of the rows that moved: no label scan
    KM_CUDA(cudaFuncSetAttribute(delta_accumulate_bitmap_kernel<T, V>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem));
    delta_accumulate_bitmap_kernel<T, V><<<s.num_sms * 2, kDeltaThreads, smem, s.stream>>>(
        s.X, s.rows, d, s.labels, s.labels_prev, s.moved_bits, k, fs, fc, scale, gate, limit);
    KM_CUDA(cudaGetLastError());
    ++launches;
    return KM_OK;
  }
  if (smem <= 200 * 1024 && s.pflush) {
    // centroid table small enough for shared accumulators: one or two CTAs per SM net their rows' moves
    if (vec_ok(s)) {
      KM_CUDA(cudaFuncSetAttribute(delta_accumulate_smem_kernel<T, V>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   (int)smem));
      delta_accumulate_smem_kernel<T, V><<<s.num_sms * (smem <= 100 * 1024 ? 2 : 1), kDeltaThreads, smem, s.stream>>>(
          s.X, s.rows, d, s.labels, s.labels_prev, k, fs, fc, scale, gate, limit, W, wsc);
    } else {
      KM_CUDA(cudaFuncSetAttribute(delta_accumulate_smem_kernel<T, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   (int)smem));
      delta_accumulate_smem_kernel<T, 1><<<s.num_sms * (smem <= 100 * 1024 ? 2 : 1), kDeltaThreads, smem, s.stream>>>(
          s.X, s.rows, d, s.labels, s.labels_prev, k, fs, fc, scale, gate, limit, W, wsc);
    }
    KM_CUDA(cudaGetLastError());
    ++launches;
    return KM_OK;
  }
  const int grid = s.num_sms * 8;
  if (vec_ok(s))
    delta_accumulate_kernel<T, V><<<grid, 256, 0, s.stream>>>(s.X, s.rows, d, s.labels, s.labels_prev, k, ps, pc,
                                                              scale, gate, limit, W, wsc);
  else
    delta_accumulate_kernel<T, 1><<<grid, 256, 0, s.stream>>>(s.X, s.rows, d, s.labels, s.labels_prev, k, ps, pc,
                                                              scale, gate, limit, W, wsc);
  KM_CUDA(cudaGetLastError());
  ++launches;
  return KM_OK;
}

// Mailboxes of all ranks mapped into every local device.  Ranks of this process are reached
// through peer access, ranks of other processes through CUDA IPC handles gathered with NCCL.
// The mailboxes come from cudaMalloc, not from the pool: pool memory cannot be exported.
// Every rank walks through the same collectives whatever fails locally: a local failure only clears
// `ok`, the exchange then carries dummy handles, and the closing all-reduce of the failure words
// tells everybody - either all ranks push or all stay with NCCL.  Nothing returns between the
// first collective and the last (a rank that left early would leave its peers' NCCL kernels
// spinning without a bound).
template <typename T>
int Engine<T>::push_setup(size_t count) {
  push_release();
  NcclApi* api = NcclApi::get();
  if (!api || !api->AllGather) return KM_ENCCL;   // the same on every rank: nobody starts a collective
  const int W = world_size;
  const size_t g = shards.size();
  struct Handles { cudaIpcMemHandle_t mailbox, flags, gmail; };
  std::vector<Handles> all((size_t)W);
  std::memset(all.data(), 0, all.size() * sizeof(Handles));
  bool ok = true;
  // one candidate record per empty cluster, at most k of them: [val][id][label][weight] + the row
  const size_t gslot = (((size_t)k * 32 + (size_t)k * d * sizeof(T)) + 15) / 16 * 16;
  // 1. allocate, clear, export
  for (size_t i = 0; i < g; ++i) {
    Shard<T>& s = shards[i];
    DevGuard gd(s.dev);
    PushState& ps = s.push;
    ps.count = count;
    ps.world = W;
    ps.gslot = gslot;
    ps.peers.assign((size_t)W, PushPeer());
    const size_t mb = (size_t)2 * W * count * sizeof(long long), fb = (size_t)3 * W * sizeof(unsigned int);
    if (cudaMalloc(&ps.done, sizeof(unsigned int)) != cudaSuccess || cudaMalloc(&ps.mailbox, mb) != cudaSuccess ||
        cudaMalloc(&ps.flags, fb) != cudaSuccess || cudaMalloc(&ps.gmail, gslot * W) != cudaSuccess ||
        cudaMalloc(&ps.grec, gslot) != cudaSuccess ||
        cudaMalloc(&ps.d_peer_mailbox, W * sizeof(long long*)) != cudaSuccess ||
        cudaMalloc(&ps.d_peer_flags, W * sizeof(unsigned int*)) != cudaSuccess ||
        cudaMalloc(&ps.d_peer_gmail, W * sizeof(unsigned char*)) != cudaSuccess ||
        cudaMalloc(&ps.d_peer_gflags, W * sizeof(unsigned int*)) != cudaSuccess) {
      cudaGetLastError();
      ok = false;
      continue;
    }
    cudaMemsetAsync(ps.done, 0, sizeof(unsigned int), s.stream);
    cudaMemsetAsync(ps.mailbox, 0, mb, s.stream);
    cudaMemsetAsync(ps.flags, 0, fb, s.stream);
    cudaMemsetAsync(ps.gmail, 0, gslot * W, s.stream);
    Handles& h = all[(size_t)world_rank0 + i];
    if (cudaIpcGetMemHandle(&h.mailbox, ps.mailbox) != cudaSuccess ||
        cudaIpcGetMemHandle(&h.flags, ps.flags) != cudaSuccess ||
        cudaIpcGetMemHandle(&h.gmail, ps.gmail) != cudaSuccess) {
      cudaGetLastError();
      ok = false;
    }
  }
  // 2. every rank's handles to every process (device buffers, one all-gather per local shard).  The
  // exchange buffers are the engine's own candidate buffers (allocated when the engine was
  // created), so no allocation can fail between here and the agreement below.
  bool nccl_ok = true;
  if ((int)g != W) {
    static_assert(sizeof(Handles) * 64 <= 2048 * sizeof(unsigned long long), "exchange buffer too small for 64 ranks");
    for (size_t i = 0; i < g; ++i) {
      DevGuard gd(shards[i].dev);
      if (cudaMemcpyAsync(shards[i].cand_val, &all[(size_t)world_rank0 + i], sizeof(Handles), cudaMemcpyHostToDevice,
                          shards[i].stream) != cudaSuccess) { cudaGetLastError(); ok = false; }
    }
    ncclResult_t nr = api->GroupStart();
    for (size_t i = 0; i < g && nr == ncclSuccess; ++i)
      nr = api->AllGather(shards[i].cand_val, shards[i].cand_row, sizeof(Handles), ncclChar, shards[i].comm,
                          shards[i].stream);
    if (nr == ncclSuccess) nr = api->GroupEnd();
    if (nr != ncclSuccess) nccl_ok = false;
    if (nccl_ok) {
      DevGuard gd(shards[0].dev);
      if (cudaMemcpyAsync(all.data(), shards[0].cand_row, sizeof(Handles) * W, cudaMemcpyDeviceToHost,
                          shards[0].stream) != cudaSuccess ||
          cudaStreamSynchronize(shards[0].stream) != cudaSuccess) { cudaGetLastError(); ok = false; }
    }
    for (size_t i = 0; i < g; ++i) {
      DevGuard gd(shards[i].dev);
      cudaStreamSynchronize(shards[i].stream);
    }
  }
  // 3. map every rank's mailbox into every local device
  for (size_t i = 0; i < g && ok && nccl_ok; ++i) {
    Shard<T>& s = shards[i];
    DevGuard gd(s.dev);
    PushState& ps = s.push;
    std::vector<long long*> pm((size_t)W);
    std::vector<unsigned int*> pf((size_t)W), pgf((size_t)W);
    std::vector<unsigned char*> pg((size_t)W);
    for (int r = 0; r < W && ok; ++r) {
      const int local = r - world_rank0;
      PushPeer& pp = ps.peers[(size_t)r];
      if (local >= 0 && local < (int)g) {
        Shard<T>& o = shards[(size_t)local];
        if (o.dev != s.dev) {
          int can = 0;
          if (cudaDeviceCanAccessPeer(&can, s.dev, o.dev) != cudaSuccess || !can) { cudaGetLastError(); ok = false; break; }
          cudaError_t pe = cudaDeviceEnablePeerAccess(o.dev, 0);
          cudaGetLastError();
          if (pe != cudaSuccess && pe != cudaErrorPeerAccessAlreadyEnabled) { ok = false; break; }
        }
        pp.mailbox = o.push.mailbox;
        pp.flags = o.push.flags;
        pp.gmail = o.push.gmail;
      } else {
        void* a = nullptr;
        if (cudaIpcOpenMemHandle(&a, all[(size_t)r].mailbox, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
          cudaGetLastError();
          ok = false;
          break;
        }
        pp.mailbox = static_cast<long long*>(a);
        pp.ipc_mailbox = true;
        if (cudaIpcOpenMemHandle(&a, all[(size_t)r].flags, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
          cudaGetLastError();
          ok = false;
          break;
        }
        pp.flags = static_cast<unsigned int*>(a);
        pp.ipc_flags = true;
        if (cudaIpcOpenMemHandle(&a, all[(size_t)r].gmail, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
          cudaGetLastError();
          ok = false;
          break;
        }
        pp.gmail = static_cast<unsigned char*>(a);
        pp.ipc_gmail = true;
      }
      pm[(size_t)r] = pp.mailbox;
      pf[(size_t)r] = pp.flags;
      pg[(size_t)r] = pp.gmail;
      pgf[(size_t)r] = pp.flags + (size_t)2 * W;   // the gather flags lie behind the all-reduce flags
    }
    if (!ok) break;
    if (cudaMemcpyAsync(ps.d_peer_mailbox, pm.data(), W * sizeof(long long*), cudaMemcpyHostToDevice, s.stream) !=
            cudaSuccess ||
        cudaMemcpyAsync(ps.d_peer_flags, pf.data(), W * sizeof(unsigned int*), cudaMemcpyHostToDevice, s.stream) !=
            cudaSuccess ||
        cudaMemcpyAsync(ps.d_peer_gmail, pg.data(), W * sizeof(unsigned char*), cudaMemcpyHostToDevice, s.stream) !=
            cudaSuccess ||
        cudaMemcpyAsync(ps.d_peer_gflags, pgf.data(), W * sizeof(unsigned int*), cudaMemcpyHostToDevice, s.stream) !=
            cudaSuccess ||
        cudaStreamSynchronize(s.stream) != cudaSuccess) {
      cudaGetLastError();
      ok = false;
    }
  }
  // 4. agreement and barrier in one collective: the sum of the ranks' failure words (in the
  // engine's own small state buffer).  Nobody pushes before every mailbox is cleared and mapped,
  // and nobody pushes unless everybody can.  A rank whose NCCL call itself failed cannot take part
  // in a collective at all and reports the error; its peers run into NCCL's own error handling.
  if (!nccl_ok) return KM_ENCCL;
  unsigned int failures = 0;
  {
    for (size_t i = 0; i < g; ++i) {
      DevGuard gd(shards[i].dev);
      const unsigned int mine = ok ? 0u : 1u;
      unsigned int* word = reinterpret_cast<unsigned int*>(shards[i].sum_partials);
      if (cudaMemcpyAsync(word, &mine, sizeof(mine), cudaMemcpyHostToDevice, shards[i].stream) != cudaSuccess ||
          cudaStreamSynchronize(shards[i].stream) != cudaSuccess) {
        // the word keeps whatever it held: poison it so that the sum cannot come out as zero
        cudaGetLastError();
        cudaMemsetAsync(word, 0x01, sizeof(unsigned int), shards[i].stream);
        ok = false;
      }
    }
    ncclResult_t nr = api->GroupStart();
    for (size_t i = 0; i < g && nr == ncclSuccess; ++i) {
      unsigned int* word = reinterpret_cast<unsigned int*>(shards[i].sum_partials);
      nr = api->AllReduce(word, word, 1, ncclUint32, ncclSum, shards[i].comm, shards[i].stream);
    }
    if (nr == ncclSuccess) nr = api->GroupEnd();
    if (nr != ncclSuccess) return KM_ENCCL;
    for (size_t i = 0; i < g; ++i) {
      DevGuard gd(shards[i].dev);
      unsigned int f = 1;
      unsigned int* word = reinterpret_cast<unsigned int*>(shards[i].sum_partials);
      if (cudaMemcpyAsync(&f, word, sizeof(f), cudaMemcpyDeviceToHost, shards[i].stream) != cudaSuccess ||
          cudaStreamSynchronize(shards[i].stream) != cudaSuccess) { cudaGetLastError(); f = 1; }
      failures += f;
    }
  }
  if (failures != 0 || !ok) {
    log_msg(verbose, 300, "push all-reduce not available on %u rank(s): staying with NCCL", failures);
    return KM_ESTATE;
  }
  for (auto& s : shards) s.push.ready = true;
  return KM_OK;
}

template <typename T>
void Engine<T>::push_release() {
  for (auto& s : shards) {
    if (s.dev < 0) continue;
    DevGuard gd(s.dev);
    PushState& ps = s.push;
    if (s.stream) cudaStreamSynchronize(s.stream);
    for (auto& pp : ps.peers) {
      if (pp.ipc_mailbox && pp.mailbox) cudaIpcCloseMemHandle(pp.mailbox);
      if (pp.ipc_flags && pp.flags) cudaIpcCloseMemHandle(pp.flags);
      if (pp.ipc_gmail && pp.gmail) cudaIpcCloseMemHandle(pp.gmail);
    }
    ps.peers.clear();
    cudaFree(ps.mailbox); cudaFree(ps.flags); cudaFree(ps.done); cudaFree(ps.d_peer_mailbox); cudaFree(ps.d_peer_flags);
    cudaFree(ps.gmail); cudaFree(ps.grec); cudaFree(ps.d_peer_gmail); cudaFree(ps.d_peer_gflags);
    cudaGetLastError();
    ps = PushState();
  }
}

}  // namespace km

