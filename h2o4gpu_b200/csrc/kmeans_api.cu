// C ABI of the k-means engine: the reference's exported functions
// (src/include/solver/kmeans.h:56-76) plus the resident-handle extension.
// See include/h2o4gpu_kmeans.h for the contract of every entry point.
#include <cstdarg>
#include <cstdlib>
#include <ctime>
#include <numeric>
#include <random>

#include "km_fit.cuh"
#include "km_init.cuh"
#include "km_synth.cuh"

namespace km {

static thread_local std::string g_err;
// iterations and inertia of this thread's last fit through the host-pointer entry points
static thread_local int g_last_iterations = 0;
static thread_local double g_last_inertia = -1.0;
void set_error(const std::string& msg) { g_err = msg; }

// Levelled stderr logger with the reference's convention: a message of level L
// prints when 0 < L <= verbose (src/common/logger.h:10-25, logger.cpp:16-34).
void log_msg(int verbose, int level, const char* fmt, ...) {
  if (!(level > 0 && level <= verbose)) return;
  va_list ap;
  va_start(ap, fmt);
  fprintf(stderr, "[kmeans %d] ", level);
  vfprintf(stderr, fmt, ap);
  fprintf(stderr, "\n");
  va_end(ap);
  fflush(stderr);
}

}  // namespace km

struct km_engine {
  int dtype;
  km::Engine<float>* f32;
  km::Engine<double>* f64;
};

using km::set_error;
using km::km_malloc;
using km::km_free;

namespace {

// devices = (gpu_id + i) % visible, i < n_gpu, n_gpu clamped to the visible
// devices and to the row count (src/gpu/kmeans/kmeans_h2o4gpu.cu:585-603)
int device_list(int gpu_id, int n_gpu, size_t rows, std::vector<int>* out) {
  int visible = 0;
  if (cudaGetDeviceCount(&visible) != cudaSuccess || visible < 1) KM_FAIL(KM_ENODEV, "no CUDA device visible");
  if (n_gpu < 0 || n_gpu > visible) n_gpu = visible;
  if (n_gpu == 0) KM_FAIL(KM_ENODEV, "n_gpu == 0: this library has no CPU path");
  if ((size_t)n_gpu > rows) n_gpu = (int)rows;
  if (gpu_id < 0) gpu_id = 0;
  out->clear();
  for (int i = 0; i < n_gpu; ++i) out->push_back((gpu_id + i) % visible);
  return KM_OK;
}

template <typename T>
int out_buffer(T** slot, size_t count, bool* allocated) {
  *allocated = false;
  if (!slot) KM_FAIL(KM_EINVAL, "output pointer is NULL");
  if (*slot == nullptr) {
    *slot = static_cast<T*>(std::malloc(std::max<size_t>(count, 1) * sizeof(T)));
    if (!*slot) KM_FAIL(KM_ENOMEM, "host allocation failed");
    *allocated = true;
  }
  return KM_OK;
}

template <typename T>
int make_engine(const std::vector<int>& devs, std::unique_ptr<km::Engine<T>>* out) {
  std::unique_ptr<km::Engine<T>> e(new km::Engine<T>());
  KM_TRY(e->init((int)devs.size(), devs.data(), 0, (int)devs.size(), nullptr));
  *out = std::move(e);
  return KM_OK;
}

// seeded row choice of the reference: first k entries of a shuffle of 0..rows-1
// with std::default_random_engine(seed) (src/gpu/kmeans/kmeans_h2o4gpu.cu:662-669,
// 687-693); seed < 0 draws the engine's seed from the clock.
template <typename T>
void shuffled_rows_init(const T* X, size_t rows, size_t cols, int k, int seed, std::vector<T>* init) {
  std::vector<int> v(rows);
  std::iota(v.begin(), v.end(), 0);
  unsigned s = (seed >= 0) ? (unsigned)seed : (unsigned)std::time(nullptr);
  std::shuffle(v.begin(), v.end(), std::default_random_engine(s));
  init->resize((size_t)k * cols);
  for (int i = 0; i < k; ++i) std::memcpy(init->data() + (size_t)i * cols, X + (size_t)v[i] * cols, cols * sizeof(T));
}

template <typename T>
int fit_impl(int verbose, int seed, int gpu_id, int n_gpu, size_t rows, size_t cols, int k, int max_iter,
             int init_from_data, T threshold, const T* X, const T* centroids, T** pred_centroids, int** pred_labels) {
  if (!X || rows == 0 || cols == 0 || k < 1 || max_iter < 0) KM_FAIL(KM_EINVAL, "kmeans fit: bad argument");
  if (rows > 0x7fffffffULL) KM_FAIL(KM_EINVAL, "kmeans fit: more than INT_MAX rows through the host-pointer ABI");
  if ((size_t)k > rows) {
    km::log_msg(verbose, 300, "number of clusters adjusted to the number of rows");
    k = (int)rows;  // src/gpu/kmeans/kmeans_h2o4gpu.cu:629-635
  }
  if (init_from_data == 2 && !centroids) KM_FAIL(KM_EINVAL, "init_from_data == 2 needs initial centroids");
  static const bool trace = std::getenv("H2O4GPU_KM_TRACE") != nullptr;
  const double t_begin = km::now_s();
  std::vector<int> devs;
  KM_TRY(device_list(gpu_id, n_gpu, rows, &devs));
  std::unique_ptr<km::Engine<T>> e;
  KM_TRY(make_engine<T>(devs, &e));
  e->verbose = verbose;
  km::log_msg(verbose, 500, "rows %zu cols %zu k %d max_iter %d devices %zu", rows, cols, k, max_iter, devs.size());
  const double t_engine = km::now_s();
  // the copy goes down while the host allocates what the fit needs
  KM_TRY(e->upload_host(X, rows, cols, 'r', false));
  int prc = e->preallocate(k, max_iter);
  KM_TRY(e->upload_wait());
  KM_TRY(prc);
  const double t_upload = km::now_s();
  std::vector<T> init;
  const T* init_ptr = centroids;
  if (init_from_data == 1) {
    // k-means|| on the device (src/gpu/kmeans/kmeans_h2o4gpu.cu:331-563)
    KM_TRY(km::init_centroids<T>(*e, k, seed, 1, &init));
    init_ptr = init.data();
  } else if (init_from_data != 2) {
    shuffled_rows_init(X, rows, cols, k, seed, &init);   // 0 = seeded random rows
    init_ptr = init.data();
  }
  int flags = (threshold > 0) ? KM_FIT_CHECK_EVERY_ITER : 0;
  KM_TRY(e->fit(k, max_iter, (double)threshold, init_ptr, flags));
  const double e_fit_s = e->stats.seconds_fit;
  const float e_loop_ms = e->stats.ms_loop;
  bool a1 = false, a2 = false;
  KM_TRY(out_buffer(pred_centroids, (size_t)k * cols, &a1));
  int rc = out_buffer(pred_labels, rows, &a2);
  if (rc != KM_OK) { if (a1) { std::free(*pred_centroids); *pred_centroids = nullptr; } return rc; }
  // what sklearn reports as n_iter_ and inertia_ (the reference leaves inertia_ unset,
  // src/interface_py/h2o4gpu/solvers/kmeans.py:187) takes one more pass over X: its kernels are queued
  // first, and the labels (final: the fit has synchronised its streams) go back to the host on a
  // stream of their own meanwhile - a copy into pageable memory keeps the calling thread busy
  rc = e->inertia_launch();
  std::vector<cudaStream_t> side(e->shards.size(), nullptr);
  if (rc == KM_OK) {
    size_t off = 0;
    for (size_t i = 0; i < e->shards.size(); ++i) {
      km::Shard<T>& s = e->shards[i];
      km::DevGuard g(s.dev);
      if (cudaStreamCreateWithFlags(&side[i], cudaStreamNonBlocking) != cudaSuccess) { cudaGetLastError(); side[i] = nullptr; }
      cudaError_t ce = cudaMemcpyAsync(*pred_labels + off, s.labels, s.rows * sizeof(int), cudaMemcpyDeviceToHost,
                                       side[i] ? side[i] : s.stream);
      if (ce != cudaSuccess) rc = KM_ECUDA;
      off += s.rows;
    }
  }
  double inertia = -1.0;
  if (rc == KM_OK) {
    rc = e->inertia_collect(&inertia);
    km::g_last_iterations = e->stats.n_iter_converged > 0 ? e->stats.n_iter_converged : e->stats.iterations;
    km::g_last_inertia = inertia;
  }
  for (size_t i = 0; i < e->shards.size(); ++i) {
    km::Shard<T>& s = e->shards[i];
    km::DevGuard g(s.dev);
    cudaError_t ce = cudaStreamSynchronize(side[i] ? side[i] : s.stream);
    if (side[i]) cudaStreamDestroy(side[i]);
    if (ce != cudaSuccess && rc == KM_OK) { set_error(std::string("labels to host: ") + cudaGetErrorString(ce)); rc = KM_ECUDA; }
  }
  if (rc != KM_OK) {
    if (a1) { std::free(*pred_centroids); *pred_centroids = nullptr; }
    if (a2) { std::free(*pred_labels); *pred_labels = nullptr; }
    return rc;
  }
  {
    km::Shard<T>& s0 = e->shards[0];
    km::DevGuard g(s0.dev);
    KM_CUDA(cudaMemcpy(*pred_centroids, s0.C[e->cur], (size_t)k * cols * sizeof(T), cudaMemcpyDeviceToHost));
  }
  km::log_msg(verbose, 300, "fit: %d iterations, %.3f s upload, %.3f s fit", e->stats.iterations,
              e->stats.seconds_upload, e->stats.seconds_fit);
  if (trace) {
    const double t_out = km::now_s();
    e.reset();
    std::fprintf(stderr, "[kmeans] call: set-up %.2f ms, upload %.2f ms, fit %.2f ms (device loop %.2f ms), "
                 "results to host %.2f ms, release %.2f ms\n", 1e3 * (t_engine - t_begin), 1e3 * (t_upload - t_engine),
                 1e3 * e_fit_s, e_loop_ms, 1e3 * (t_out - t_upload - e_fit_s), 1e3 * (km::now_s() - t_out));
  }
  return KM_OK;
}

template <typename T>
int predict_impl(int verbose, int gpu_id, int n_gpu, size_t rows, size_t cols, int k, const T* X,
                 const T* centroids, int** pred_labels) {
  if (!X || !centroids || rows == 0 || cols == 0 || k < 1) KM_FAIL(KM_EINVAL, "kmeans predict: bad argument");
  std::vector<int> devs;
  KM_TRY(device_list(gpu_id, n_gpu, rows, &devs));
  std::unique_ptr<km::Engine<T>> e;
  KM_TRY(make_engine<T>(devs, &e));
  e->verbose = verbose;
  KM_TRY(e->upload_host(X, rows, cols, 'r'));
  KM_TRY(e->check_data());
  KM_TRY(e->set_centroids(k, centroids));
  KM_TRY(e->assign_all(0));
  bool a = false;
  KM_TRY(out_buffer(pred_labels, rows, &a));
  size_t off = 0;
  for (auto& s : e->shards) {
    km::DevGuard g(s.dev);
    KM_CUDA(cudaStreamSynchronize(s.stream));
    KM_CUDA(cudaMemcpy(*pred_labels + off, s.labels, s.rows * sizeof(int), cudaMemcpyDeviceToHost));
    off += s.rows;
  }
  return KM_OK;
}

template <typename T>
int transform_impl(int verbose, int gpu_id, int n_gpu, size_t rows, size_t cols, int k, const T* X,
                   const T* centroids, T** preds) {
  if (!X || !centroids || rows == 0 || cols == 0 || k < 1) KM_FAIL(KM_EINVAL, "kmeans transform: bad argument");
  std::vector<int> devs;
  KM_TRY(device_list(gpu_id, n_gpu, rows, &devs));
  std::unique_ptr<km::Engine<T>> e;
  KM_TRY(make_engine<T>(devs, &e));
  e->verbose = verbose;
  KM_TRY(e->upload_host(X, rows, cols, 'r'));
  KM_TRY(e->check_data());
  KM_TRY(e->set_centroids(k, centroids));
  bool a = false;
  KM_TRY(out_buffer(preds, rows * (size_t)k, &a));
  size_t off = 0;
  for (size_t i = 0; i < e->shards.size(); ++i) {
    KM_TRY(e->transform_shard((int)i, *preds + off, rows));
    off += e->shards[i].rows;
  }
  return KM_OK;
}

template <typename T>
int centroid_sums_impl(int gpu_id, const T* X, const int32_t* labels, size_t rows, size_t cols, int k, double* sums,
                       int64_t* counts) {
  if (!X || !labels || !sums || !counts || rows == 0 || cols == 0 || k < 1) KM_FAIL(KM_EINVAL, "centroid sums: bad argument");
  for (size_t i = 0; i < rows; ++i)
    if (labels[i] < 0 || labels[i] >= k) KM_FAIL(KM_EINVAL, "centroid sums: label out of range");
  std::vector<int> devs;
  KM_TRY(device_list(gpu_id, 1, rows, &devs));
  std::unique_ptr<km::Engine<T>> e;
  KM_TRY(make_engine<T>(devs, &e));
  KM_TRY(e->upload_host(X, rows, cols, 'r'));
  KM_TRY(e->check_data());
  e->k = k;
  KM_TRY(e->ensure_buffers(k));
  km::Shard<T>& s = e->shards[0];
  km::DevGuard g(s.dev);
  int ex = 0;
  if (s.xmax > 0) std::frexp(s.xmax, &ex);
  const int sa = km::kPieceBits - ex;
  KM_CUDA(cudaMemcpyAsync(s.labels, labels, rows * sizeof(int), cudaMemcpyHostToDevice, s.stream));
  KM_CUDA(cudaMemsetAsync(s.gacc, 0, s.gacc_count(k, (int)cols) * sizeof(long long), s.stream));
  KM_TRY(e->launch_accumulate(s, (T)std::ldexp(1.0, sa)));
  std::vector<long long> h(s.gacc_count(k, (int)cols));
  KM_CUDA(cudaMemcpyAsync(h.data(), s.gacc, h.size() * sizeof(long long), cudaMemcpyDeviceToHost, s.stream));
  KM_CUDA(cudaStreamSynchronize(s.stream));
  constexpr int NP = km::Fixed<T>::NP;
  const double inv = std::ldexp(1.0, -(sa + km::kPieceBits));
  const size_t kd = (size_t)k * cols;
  for (size_t i = 0; i < kd; ++i) {
    long long gp[NP / 2];
    for (int q = 0; q < NP / 2; ++q) gp[q] = h[(size_t)q * kd + i];
    sums[i] = km::fixed_to_double<NP>(gp, inv);
  }
  for (int j = 0; j < k; ++j) counts[j] = (int64_t)h[(size_t)(NP / 2) * kd + j];
  return KM_OK;
}

template <typename T>
int synth_impl(int gpu_id, T* dX, size_t rows, size_t cols, size_t row0, int kind, const T* centers_host, int n_comp,
               const T* weights_host, T sigma, uint64_t seed) {
  if (!dX || rows == 0 || cols == 0) KM_FAIL(KM_EINVAL, "synth: bad argument");
  if (kind != 1 && (!centers_host || n_comp < 1)) KM_FAIL(KM_EINVAL, "synth: mixture needs centers");
  km::DevGuard g(gpu_id);
  T* dc = nullptr;
  float* dcdf = nullptr;
  if (kind != 1) {
    std::vector<float> cdf(n_comp);
    double tot = 0, run = 0;
    for (int i = 0; i < n_comp; ++i) tot += weights_host ? (double)weights_host[i] : 1.0;
    for (int i = 0; i < n_comp; ++i) {
      run += (weights_host ? (double)weights_host[i] : 1.0) / tot;
      cdf[i] = (float)run;
    }
    cdf[n_comp - 1] = 1.0f;
    KM_CUDA(km_malloc(&dc, (size_t)n_comp * cols * sizeof(T)));
    KM_CUDA(km_malloc(&dcdf, n_comp * sizeof(float)));
    KM_CUDA(cudaMemcpy(dc, centers_host, (size_t)n_comp * cols * sizeof(T), cudaMemcpyHostToDevice));
    KM_CUDA(cudaMemcpy(dcdf, cdf.data(), n_comp * sizeof(float), cudaMemcpyHostToDevice));
  }
  km::synth_kernel<T><<<148 * 16, 256>>>(dX, rows, (int)cols, row0, kind, dc, n_comp, dcdf, sigma, seed);
  cudaError_t ce = cudaGetLastError();
  if (ce == cudaSuccess) ce = cudaDeviceSynchronize();
  km_free(dc);
  km_free(dcdf);
  if (ce != cudaSuccess) KM_FAIL(KM_ECUDA, std::string("synth: ") + cudaGetErrorString(ce));
  return KM_OK;
}

}  // namespace

template <typename T>
static int assign_sync(km::Engine<T>* e) {
  KM_TRY(e->check_data());
  if (e->shards.empty()) KM_FAIL(KM_ESTATE, "no data attached to the handle");
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  {
    km::DevGuard g(e->shards[0].dev);
    KM_CUDA(cudaEventCreate(&e0));
    KM_CUDA(cudaEventCreate(&e1));
    cudaEventRecord(e0, e->shards[0].stream);
  }
  int rc = e->assign_all(0);
  {
    km::DevGuard g(e->shards[0].dev);
    cudaEventRecord(e1, e->shards[0].stream);
  }
  for (auto& s : e->shards) {
    km::DevGuard g(s.dev);
    cudaError_t ce = cudaStreamSynchronize(s.stream);
    if (ce != cudaSuccess && rc == KM_OK) { set_error(std::string("assign sync: ") + cudaGetErrorString(ce)); rc = KM_ECUDA; }
  }
  float ms = 0;
  if (rc == KM_OK && cudaEventElapsedTime(&ms, e0, e1) == cudaSuccess) e->stats.ms_assign = ms;
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  return rc;
}

template <typename T>
static int get_centroids(km::Engine<T>* e, void* out) {
  if (!out) KM_FAIL(KM_EINVAL, "NULL output");
  if (!e->have_centroids) KM_FAIL(KM_ESTATE, "no centroids set");
  km::Shard<T>& s = e->shards[0];
  km::DevGuard g(s.dev);
  KM_CUDA(cudaStreamSynchronize(s.stream));
  KM_CUDA(cudaMemcpy(out, s.C[e->cur], (size_t)e->k * e->d * sizeof(T), cudaMemcpyDeviceToHost));
  return KM_OK;
}

template <typename T>
static int init_resident(km::Engine<T>* e, int k, int seed, int method, void* out, long long* rows_out) {
  if (!out) KM_FAIL(KM_EINVAL, "kmeans_init_resident: out is NULL");
  std::vector<T> c;
  std::vector<size_t> rows;
  KM_TRY(km::init_centroids<T>(*e, k, seed, method, &c, &rows));
  std::memcpy(out, c.data(), c.size() * sizeof(T));
  if (rows_out)
    for (size_t i = 0; i < rows.size(); ++i) rows_out[i] = (long long)rows[i];
  return KM_OK;
}
template <typename T>
static int get_labels(km::Engine<T>* e, int local, int32_t* out) {
  if (!out || local < 0 || local >= (int)e->shards.size()) KM_FAIL(KM_EINVAL, "kmeans_get_labels: bad argument");
  km::Shard<T>& s = e->shards[local];
  if (!s.labels) KM_FAIL(KM_ESTATE, "no labels yet");
  km::DevGuard g(s.dev);
  KM_CUDA(cudaStreamSynchronize(s.stream));
  KM_CUDA(cudaMemcpy(out, s.labels, s.rows * sizeof(int), cudaMemcpyDeviceToHost));
  return KM_OK;
}

template <typename T>
static int labels_dev(km::Engine<T>* e, int local, const int32_t** out) {
  if (!out || local < 0 || local >= (int)e->shards.size()) KM_FAIL(KM_EINVAL, "kmeans_labels_device: bad argument");
  *out = e->shards[local].labels;
  return KM_OK;
}

template <typename T>
static int get_stats(km::Engine<T>* e, kmeans_stats* out, int want_inertia) {
  if (!out) KM_FAIL(KM_EINVAL, "NULL output");
  if (want_inertia && e->have_centroids) {
    double v;
    KM_TRY(e->inertia(&v));
  }
  *out = e->stats;
  return KM_OK;
}

// ---- extern "C" surface ---------------------------------------------------------
extern "C" {

const char* kmeans_last_error(void) { return km::g_err.c_str(); }
int kmeans_trim_memory(void) {
  km::km_trim_pools();
  return KM_OK;
}
int kmeans_last_fit_info(int* iterations, double* inertia) {
  if (iterations) *iterations = km::g_last_iterations;
  if (inertia) *inertia = km::g_last_inertia;
  return KM_OK;
}

int kmeans_set_wait_limits(double peer_wait_ms, double mbarrier_wait_ms) {
  km::WaitLimits def;
  km::WaitLimits& w = km::wait_limits();
  // a peer-flag poll sleeps 40 ns and reads one word (about 0.1 us per poll in all); an mbarrier
  // poll parks the warp for at most 20 us
  w.push_spins = peer_wait_ms > 0 ? (unsigned int)std::min(4.0e9, std::max(1.0, peer_wait_ms * 1e4)) : def.push_spins;
  w.mbar_iters = mbarrier_wait_ms > 0 ? (unsigned int)std::min(2.0e9, std::max(1.0, mbarrier_wait_ms * 50.0)) : def.mbar_iters;
  return KM_OK;
}

int kmeans_selftest_wait_timeout(int gpu_id, int which, int* device_code) {
  int visible = 0;
  if (cudaGetDeviceCount(&visible) != cudaSuccess || gpu_id < 0 || gpu_id >= visible)
    KM_FAIL(KM_ENODEV, "kmeans_selftest_wait_timeout: bad device");
  if (which != 0 && which != 1) KM_FAIL(KM_EINVAL, "kmeans_selftest_wait_timeout: which must be 0 or 1");
  km::DevGuard g(gpu_id);
  km::IterState* st = nullptr;
  KM_CUDA(km_malloc(&st, sizeof(km::IterState)));
  cudaError_t ce = cudaMemset(st, 0, sizeof(km::IterState));
  long long* mailbox = nullptr;
  unsigned int* flags = nullptr;
  unsigned int* done = nullptr;
  long long** pm = nullptr;
  unsigned int** pf = nullptr;
  long long* vec = nullptr;
  if (which == 0) {
    // a world of two ranks on one device: both "peers" are this rank's own mailbox, and the second rank never
    // delivers, so the wait for its flag must give up
    const size_t count = 8;
    if (ce == cudaSuccess) ce = km_malloc(&mailbox, 2 * 2 * count * sizeof(long long));
    if (ce == cudaSuccess) ce = km_malloc(&flags, 2 * 2 * sizeof(unsigned int));
    if (ce == cudaSuccess) ce = km_malloc(&done, sizeof(unsigned int));
    if (ce == cudaSuccess) ce = km_malloc(&pm, 2 * sizeof(long long*));
    if (ce == cudaSuccess) ce = km_malloc(&pf, 2 * sizeof(unsigned int*));
    if (ce == cudaSuccess) ce = km_malloc(&vec, 2 * count * sizeof(long long));
    if (ce == cudaSuccess) ce = cudaMemset(mailbox, 0, 2 * 2 * count * sizeof(long long));
    if (ce == cudaSuccess) ce = cudaMemset(flags, 0, 2 * 2 * sizeof(unsigned int));
    if (ce == cudaSuccess) ce = cudaMemset(done, 0, sizeof(unsigned int));
    if (ce == cudaSuccess) ce = cudaMemset(vec, 0, 2 * count * sizeof(long long));
    long long* hm[2] = {mailbox, mailbox};
    unsigned int* hf[2] = {flags, flags};
    if (ce == cudaSuccess) ce = cudaMemcpy(pm, hm, sizeof(hm), cudaMemcpyHostToDevice);
    if (ce == cudaSuccess) ce = cudaMemcpy(pf, hf, sizeof(hf), cudaMemcpyHostToDevice);
    if (ce == cudaSuccess) {
      km::push_allreduce_kernel<<<km::kPushCtas, km::kPushThreads>>>(vec, vec + count, count, 0, 2, pm, pf, mailbox, flags,
                                                                     done, 1u, st, km::wait_limits().push_spins);
      ce = cudaGetLastError();
    }
  } else if (ce == cudaSuccess) {
    km::tc::mbar_timeout_probe_kernel<<<1, 32>>>(&st->error, km::wait_limits().mbar_iters);
    ce = cudaGetLastError();
  }
  if (ce == cudaSuccess) ce = cudaDeviceSynchronize();
  km::IterState hs{};
  if (ce == cudaSuccess) ce = cudaMemcpy(&hs, st, sizeof(hs), cudaMemcpyDeviceToHost);
  km_free(st); km_free(mailbox); km_free(flags); km_free(done); km_free(pm); km_free(pf); km_free(vec);
  if (ce != cudaSuccess) KM_FAIL(KM_ECUDA, std::string("kmeans_selftest_wait_timeout: ") + cudaGetErrorString(ce));
  if (device_code) *device_code = hs.error;
  if (hs.error != 0)
    KM_FAIL(KM_ETIMEOUT, "a bounded device-side wait gave up (code " + std::to_string(hs.error) + ")");
  return KM_OK;
}

int kmeans_device_count(void) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) return 0;
  return n;
}

void kmeans_free(void* p) { std::free(p); }

int kmeans_fit_f32(int verbose, int seed, int gpu_id, int n_gpu, size_t rows, size_t cols, int k, int max_iterations,
                   int init_from_data, float threshold, const float* srcdata, const float* centroids,
                   float** pred_centroids, int** pred_labels) {
  return fit_impl<float>(verbose, seed, gpu_id, n_gpu, rows, cols, k, max_iterations, init_from_data, threshold,
                         srcdata, centroids, pred_centroids, pred_labels);
}
int kmeans_fit_f64(int verbose, int seed, int gpu_id, int n_gpu, size_t rows, size_t cols, int k, int max_iterations,
                   int init_from_data, double threshold, const double* srcdata, const double* centroids,
                   double** pred_centroids, int** pred_labels) {
  return fit_impl<double>(verbose, seed, gpu_id, n_gpu, rows, cols, k, max_iterations, init_from_data, threshold,
                          srcdata, centroids, pred_centroids, pred_labels);
}
int kmeans_predict_f32(int verbose, int gpu_id, int n_gpu, size_t rows, size_t cols, int k, const float* srcdata,
                       const float* centroids, int** pred_labels) {
  return predict_impl<float>(verbose, gpu_id, n_gpu, rows, cols, k, srcdata, centroids, pred_labels);
}
int kmeans_predict_f64(int verbose, int gpu_id, int n_gpu, size_t rows, size_t cols, int k, const double* srcdata,
                       const double* centroids, int** pred_labels) {
  return predict_impl<double>(verbose, gpu_id, n_gpu, rows, cols, k, srcdata, centroids, pred_labels);
}
int kmeans_transform_f32(int verbose, int gpu_id, int n_gpu, size_t rows, size_t cols, int k, const float* srcdata,
                         const float* centroids, float** preds) {
  return transform_impl<float>(verbose, gpu_id, n_gpu, rows, cols, k, srcdata, centroids, preds);
}
int kmeans_transform_f64(int verbose, int gpu_id, int n_gpu, size_t rows, size_t cols, int k, const double* srcdata,
                         const double* centroids, double** preds) {
  return transform_impl<double>(verbose, gpu_id, n_gpu, rows, cols, k, srcdata, centroids, preds);
}

int kmeans_create(kmeans_handle_t* out, int dtype, int n_local, const int* device_ids, int world_rank0,
                  int world_size, const void* nccl_id) {
  if (!out || !device_ids || (dtype != 0 && dtype != 1)) KM_FAIL(KM_EINVAL, "kmeans_create: bad argument");
  std::unique_ptr<km_engine> h(new km_engine{dtype, nullptr, nullptr});
  int rc;
  if (dtype == 0) {
    h->f32 = new km::Engine<float>();
    rc = h->f32->init(n_local, device_ids, world_rank0, world_size, nccl_id);
  } else {
    h->f64 = new km::Engine<double>();
    rc = h->f64->init(n_local, device_ids, world_rank0, world_size, nccl_id);
  }
  if (rc != KM_OK) { delete h->f32; delete h->f64; return rc; }
  *out = h.release();
  return KM_OK;
}

int kmeans_destroy(kmeans_handle_t h) {
  if (!h) return KM_OK;
  delete h->f32;
  delete h->f64;
  delete h;
  return KM_OK;
}

int kmeans_nccl_unique_id(void* out128) {
  if (!out128) KM_FAIL(KM_EINVAL, "kmeans_nccl_unique_id: NULL");
  km::NcclApi* api = km::NcclApi::get();
  if (!api) KM_FAIL(KM_ENCCL, "libnccl.so.2 could not be loaded");
  ncclUniqueId id;
  KM_NCCL(api, api->GetUniqueId(&id));
  static_assert(sizeof(id) == 128, "ncclUniqueId size");
  std::memcpy(out128, &id, 128);
  return KM_OK;
}

#define KM_DISPATCH(h, call_f32, call_f64)                      \
  if (!(h)) KM_FAIL(KM_EINVAL, "NULL handle");                  \
  return (h)->dtype == 0 ? (call_f32) : (call_f64)

int kmeans_attach_device(kmeans_handle_t h, int local, const void* dX, size_t rows, size_t cols, size_t n_total) {
  KM_DISPATCH(h, h->f32->attach_device(local, static_cast<const float*>(dX), rows, cols, n_total),
              h->f64->attach_device(local, static_cast<const double*>(dX), rows, cols, n_total));
}
int kmeans_upload_host(kmeans_handle_t h, const void* X, size_t rows, size_t cols, char order) {
  KM_DISPATCH(h, h->f32->upload_host(static_cast<const float*>(X), rows, cols, order),
              h->f64->upload_host(static_cast<const double*>(X), rows, cols, order));
}
int kmeans_upload_host_typed(kmeans_handle_t h, const void* X, int src_dtype, size_t rows, size_t cols, char order) {
  KM_DISPATCH(h, h->f32->upload_host_typed(X, src_dtype, rows, cols, order),
              h->f64->upload_host_typed(X, src_dtype, rows, cols, order));
}
int kmeans_set_sample_weight(kmeans_handle_t h, const void* weights, size_t count) {
  KM_DISPATCH(h, h->f32->set_sample_weight(static_cast<const float*>(weights), count),
              h->f64->set_sample_weight(static_cast<const double*>(weights), count));
}
int kmeans_fit_resident(kmeans_handle_t h, int k, int max_iter, double threshold, const void* init, int flags) {
  KM_DISPATCH(h, h->f32->fit(k, max_iter, threshold, static_cast<const float*>(init), flags),
              h->f64->fit(k, max_iter, threshold, static_cast<const double*>(init), flags));
}
int kmeans_init_resident(kmeans_handle_t h, int k, int seed, int method, void* out, long long* rows_out) {
  KM_DISPATCH(h, init_resident(h->f32, k, seed, method, out, rows_out),
              init_resident(h->f64, k, seed, method, out, rows_out));
}

int kmeans_set_centroids(kmeans_handle_t h, int k, const void* c) {
  KM_DISPATCH(h, h->f32->set_centroids(k, static_cast<const float*>(c)),
              h->f64->set_centroids(k, static_cast<const double*>(c)));
}

int kmeans_assign_resident(kmeans_handle_t h) { KM_DISPATCH(h, assign_sync(h->f32), assign_sync(h->f64)); }

int kmeans_get_centroids(kmeans_handle_t h, void* out) { KM_DISPATCH(h, get_centroids(h->f32, out), get_centroids(h->f64, out)); }

int kmeans_get_labels(kmeans_handle_t h, int local, int32_t* out) {
  KM_DISPATCH(h, get_labels(h->f32, local, out), get_labels(h->f64, local, out));
}

int kmeans_labels_device(kmeans_handle_t h, int local, const int32_t** out) {
  KM_DISPATCH(h, labels_dev(h->f32, local, out), labels_dev(h->f64, local, out));
}
int kmeans_transform_resident(kmeans_handle_t h, int local, void* out, size_t ld) {
  KM_DISPATCH(h, h->f32->transform_shard(local, static_cast<float*>(out), ld),
              h->f64->transform_shard(local, static_cast<double*>(out), ld));
}

int kmeans_get_stats(kmeans_handle_t h, kmeans_stats* out) {
  KM_DISPATCH(h, get_stats(h->f32, out, 0), get_stats(h->f64, out, 0));
}
int kmeans_inertia(kmeans_handle_t h, double* out) {
  if (!out) KM_FAIL(KM_EINVAL, "NULL output");
  KM_DISPATCH(h, h->f32->inertia(out), h->f64->inertia(out));
}

int kmeans_centroid_sums_f32(int gpu_id, const float* X, const int32_t* labels, size_t rows, size_t cols, int k,
                             double* sums, int64_t* counts) {
  return centroid_sums_impl<float>(gpu_id, X, labels, rows, cols, k, sums, counts);
}
int kmeans_centroid_sums_f64(int gpu_id, const double* X, const int32_t* labels, size_t rows, size_t cols, int k,
                             double* sums, int64_t* counts) {
  return centroid_sums_impl<double>(gpu_id, X, labels, rows, cols, k, sums, counts);
}

int kmeans_synth_f32(int gpu_id, float* dX, size_t rows, size_t cols, size_t row0, int kind, const float* centers_host,
                     int n_comp, const float* weights_host, float sigma, uint64_t seed) {
  return synth_impl<float>(gpu_id, dX, rows, cols, row0, kind, centers_host, n_comp, weights_host, sigma, seed);
}
int kmeans_synth_f64(int gpu_id, double* dX, size_t rows, size_t cols, size_t row0, int kind,
                     const double* centers_host, int n_comp, const double* weights_host, double sigma, uint64_t seed) {
  return synth_impl<double>(gpu_id, dX, rows, cols, row0, kind, centers_host, n_comp, weights_host, sigma, seed);
}


}  // extern "C"

// ---- the reference header's C++-linkage names -------------------------------------
int make_ptr_float_kmeans(int dopredict, int verbose, int seed, int gpu_id, int n_gpu, size_t mTrain, size_t n, int k,
                          int max_iterations, int init_from_data, float threshold, const float* srcdata,
                          const float* centroids, float** pred_centroids, int** pred_labels) {
  if (dopredict == 0)
    return kmeans_fit_f32(verbose, seed, gpu_id, n_gpu, mTrain, n, k, max_iterations, init_from_data, threshold,
                          srcdata, centroids, pred_centroids, pred_labels);
  return kmeans_predict_f32(verbose, gpu_id, n_gpu, mTrain, n, k, srcdata, centroids, pred_labels);
}
int make_ptr_double_kmeans(int dopredict, int verbose, int seed, int gpu_id, int n_gpu, size_t mTrain, size_t n, int k,
                           int max_iterations, int init_from_data, double threshold, const double* srcdata,
                           const double* centroids, double** pred_centroids, int** pred_labels) {
  if (dopredict == 0)
    return kmeans_fit_f64(verbose, seed, gpu_id, n_gpu, mTrain, n, k, max_iterations, init_from_data, threshold,
                          srcdata, centroids, pred_centroids, pred_labels);
  return kmeans_predict_f64(verbose, gpu_id, n_gpu, mTrain, n, k, srcdata, centroids, pred_labels);
}
int kmeans_transform_float(int verbose, int gpu_id, int n_gpu, size_t m, size_t n, int k, const float* srcdata,
                           const float* centroids, float** preds) {
  return kmeans_transform_f32(verbose, gpu_id, n_gpu, m, n, k, srcdata, centroids, preds);
}
int kmeans_transform_double(int verbose, int gpu_id, int n_gpu, size_t m, size_t n, int k, const double* srcdata,
                            const double* centroids, double** preds) {
  return kmeans_transform_f64(verbose, gpu_id, n_gpu, m, n, k, srcdata, centroids, preds);
}
