// Initial centroids on the GPU: k-means|| (scalable k-means++) followed by a weighted
// k-means++ over the candidates, and seeded random rows.
//
// Replaces kmeans_parallel / kmeans_plus_plus / count_pts_per_centroid of the reference
// (src/gpu/kmeans/kmeans_h2o4gpu.cu:154-279, 331-563; src/gpu/kmeans/kmeans_h2o4gpu.h:44-126)
// and its seeded row shuffle (kmeans_h2o4gpu.cu:662-669, 687-693).  Same scheme as the
// reference:
//   1. one uniformly drawn row is the first candidate;
//   2. R = min(8, 2 + ln k) rounds: every row keeps the squared distance to its nearest
//      candidate so far (cost); with phi the summed cost, a row becomes a candidate
//      independently with probability min(1, 2 k cost / phi);
//   3. more than k candidates: each is weighted by the number of rows nearest to it and
//      k of them are drawn by D^2-weighted k-means++ (the reference does this step on the
//      host); at most k candidates: they are kept and seeded random rows fill the rest
//      (the reference leaves zeros there).
// What is new: the nearest-candidate search of every round runs through the same distance
// kernels as the Lloyd iteration (tensor cores where the shape allows), costs are exact
// squared distances in double, random numbers come from Philox4x32-10 keyed by the seed with
// the GLOBAL row index as counter (so the draw of a row does not depend on which GPU holds
// it), and the k-means++ stage runs on the device without a host round trip per centre.
#pragma once

#include <algorithm>
#include <cmath>
#include <numeric>
#include <random>
#include <vector>

#include "km_fit.cuh"
#include "km_synth.cuh"

namespace km {

constexpr unsigned int kStreamFirst = 8u, kStreamSample = 7u, kStreamPlusPlus = 9u, kStreamFill = 10u;

// uniform in the open interval (0, 1) from two 32-bit words: 52 random bits plus one half,
// so that every value (the largest included) is exact in double
__host__ __device__ inline double u01_53(unsigned int a, unsigned int b) {
  const unsigned long long v = ((unsigned long long)(a >> 6) << 26) | (unsigned long long)(b >> 6);
  return ((double)v + 0.5) * (1.0 / 4503599627370496.0);
}

// Philox4x32-10 on the host (same rounds as Philox::run on the device)
inline void philox_host(unsigned int c[4], unsigned int k0, unsigned int k1) {
  const unsigned long long M0 = 0xD2511F53ull, M1 = 0xCD9E8D57ull;
  for (int r = 0; r < 10; ++r) {
    const unsigned long long p0 = M0 * c[0], p1 = M1 * c[2];
    const unsigned int n0 = (unsigned int)(p1 >> 32) ^ c[1] ^ k0, n1 = (unsigned int)p1;
    const unsigned int n2 = (unsigned int)(p0 >> 32) ^ c[3] ^ k1, n3 = (unsigned int)p0;
    c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
}

__global__ void __launch_bounds__(256) fill_double_kernel(double* __restrict__ v, size_t n, double value) {
  for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (size_t)gridDim.x * 256) v[i] = value;
}

// cost[row] = min(cost[row], |x_row - C[label[row]]|^2), direct differences in double
template <typename T>
__global__ void __launch_bounds__(256)
mincost_update_kernel(const T* __restrict__ X, size_t n, int d, const int* __restrict__ labels,
                      const T* __restrict__ C, double* __restrict__ cost) {
  const int lane = threadIdx.x & 31;
  const size_t warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const size_t nwarp = ((size_t)gridDim.x * blockDim.x) >> 5;
  for (size_t row = warp; row < n; row += nwarp) {
    const T* x = X + row * (size_t)d;
    const T* c = C + (size_t)labels[row] * d;
    double s = 0;
    for (int t = lane; t < d; t += 32) {
      const double q = (double)x[t] - (double)c[t];
      s += q * q;
    }
    s = warp_sum(s);
    if (lane == 0) cost[row] = fmin(cost[row], s);
  }
}

// Bernoulli draw per row: selected when 2 k cost / phi exceeds the row's uniform number
// (cost = weight * squared distance when sample weights are set).
template <typename T>
__global__ void __launch_bounds__(256)
sample_rows_kernel(const double* __restrict__ cost, size_t n, size_t row0, double phi, double two_k,
                   unsigned long long seed, unsigned int round, unsigned int* __restrict__ list,
                   unsigned int cap, unsigned int* __restrict__ count, const T* __restrict__ W) {
  const uint2 key = make_uint2((unsigned int)seed, (unsigned int)(seed >> 32));
  for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (size_t)gridDim.x * 256) {
    const size_t gr = row0 + i;
    const uint4 r = Philox::run(make_uint4((unsigned int)gr, (unsigned int)(gr >> 32), round, kStreamSample), key);
    const double u = u01_53(r.x, r.y);
    const double cw = W ? cost[i] * (double)W[i] : cost[i];
    const double p = (two_k * cw) / phi;
    if (p > u) {
      const unsigned int pos = atomicAdd(count, 1u);
      if (pos < cap) list[pos] = (unsigned int)i;
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
gather_rows_kernel(const T* __restrict__ X, int d, const unsigned int* __restrict__ list, unsigned int m,
                   T* __restrict__ out) {
  const size_t total = (size_t)m * d;
  for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < total; i += (size_t)gridDim.x * 256) {
    const size_t j = i / d;
    out[i] = X[(size_t)list[j] * d + (i - j * d)];
  }
}

// rows (or, with sample weights, fixed-point weight units: integers, so the totals do not depend on
// the order of the additions) nearest to each candidate
template <typename T>
__global__ void __launch_bounds__(256)
label_histogram_kernel(const int* __restrict__ labels, size_t n, int m, unsigned long long* __restrict__ counts,
                       const T* __restrict__ W, T wscale) {
  for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (size_t)gridDim.x * 256) {
    const int l = labels[i];
    unsigned long long units = 1;
    if (W) {
      int pw[2];
      split_pieces<2>(W[i], wscale, pw);
      units = (unsigned long long)((long long)pw[0] * (1LL << kPieceBits) + (long long)pw[1]);
    }
    if ((unsigned)l < (unsigned)m && units) atomicAdd(counts + l, units);
  }
}

// ---- weighted k-means++ over m candidates, all on the device -------------------
// state[0] = index chosen by the last step.  mind[i] = squared distance of candidate i to
// the nearest chosen one (starts at +inf); wm[i] = weight * mind (weight alone before the
// first choice).
template <typename T>
__global__ void __launch_bounds__(256)
kpp_update_kernel(const T* __restrict__ Cd, int m, int d, const int* __restrict__ state,
                  const double* __restrict__ w, double* __restrict__ mind, double* __restrict__ wm) {
  const int c = state[0];
  for (int i = blockIdx.x * 256 + threadIdx.x; i < m; i += gridDim.x * 256) {
    const T* a = Cd + (size_t)i * d;
    const T* b = Cd + (size_t)c * d;
    double s = 0;
    for (int t = 0; t < d; ++t) {
      const double q = (double)a[t] - (double)b[t];
      s += q * q;
    }
    const double v = fmin(mind[i], s);
    mind[i] = v;
    wm[i] = w[i] * v;
  }
}

// One CTA: draws index i with probability wm[i] / sum(wm) (first index whose running sum
// exceeds u * total), records it in chosen[step] and state[0].  Running sums are formed
// in a fixed order (per-thread chunks, then the chunks in sequence) so the draw is
// reproducible; when everything left has weight zero the lowest unchosen index is taken.
__global__ void __launch_bounds__(1024)
kpp_select_kernel(const double* __restrict__ wm, int m, unsigned long long seed, int step, int* __restrict__ state,
                  int* __restrict__ chosen, unsigned char* __restrict__ taken) {
  __shared__ double local[1024];
  __shared__ double prefix[1025];
  __shared__ int s_pick;
  const int t = threadIdx.x;
  const int chunk = (m + 1023) / 1024;
  const int b = t * chunk, e = min(m, b + chunk);
  double s = 0;
  for (int i = b; i < e; ++i) s += wm[i];
  local[t] = s;
  if (t == 0) s_pick = -1;
  __syncthreads();
  if (t == 0) {
    double acc = 0;
    for (int j = 0; j < 1024; ++j) { prefix[j] = acc; acc += local[j]; }
    prefix[1024] = acc;
  }
  __syncthreads();
  const double total = prefix[1024];
  if (total > 0) {
    unsigned int c[4] = {(unsigned int)step, 0u, 0u, kStreamPlusPlus};
    const uint4 r = Philox::run(make_uint4(c[0], c[1], c[2], c[3]), make_uint2((unsigned int)seed, (unsigned int)(seed >> 32)));
    const double target = u01_53(r.x, r.y) * total;
    // the owner is the first chunk whose end sum exceeds the target
    if (prefix[t + 1] > target && !(prefix[t] > target) && b < e) {
      double acc = prefix[t];
      int pick = -1, last_pos = -1;
      for (int i = b; i < e; ++i) {
        if (wm[i] > 0) last_pos = i;
        acc += wm[i];
        if (acc > target) { pick = i; break; }
      }
      if (pick < 0) pick = last_pos;
      if (pick >= 0) s_pick = pick;
    }
  }
  __syncthreads();
  if (t == 0) {
    int pick = s_pick;
    if (pick < 0) {
      // zero total weight, or rounding pushed the target past the last sum
      if (total > 0) {
        for (int i = m - 1; i >= 0; --i)
          if (wm[i] > 0) { pick = i; break; }
      }
      if (pick < 0)
        for (int i = 0; i < m; ++i)
          if (!taken[i]) { pick = i; break; }
      if (pick < 0) pick = 0;
    }
    taken[pick] = 1;
    chosen[step] = pick;
    state[0] = pick;
  }
}

// seeded distinct rows: the first k entries of a shuffle of 0..n-1 with
// std::default_random_engine(seed), as copy_centroids_shuffled does
inline void shuffled_row_ids(size_t n, int k, int seed, std::vector<size_t>* out) {
  std::vector<int> v(n);
  std::iota(v.begin(), v.end(), 0);
  const unsigned s = (seed >= 0) ? (unsigned)seed : (unsigned)std::random_device{}();
  std::shuffle(v.begin(), v.end(), std::default_random_engine(s));
  out->assign(v.begin(), v.begin() + k);
}

// Rows (global indices, any order) of a one-process engine to the host, row-major k x d.
template <typename T>
int fetch_rows(Engine<T>& e, const std::vector<size_t>& rows, std::vector<T>* out) {
  out->assign(rows.size() * (size_t)e.d, (T)0);
  for (size_t j = 0; j < rows.size(); ++j) {
    bool found = false;
    for (auto& s : e.shards) {
      if (rows[j] >= s.row0 && rows[j] < s.row0 + s.rows) {
        DevGuard g(s.dev);
        KM_CUDA(cudaMemcpyAsync(out->data() + j * (size_t)e.d, s.X + (rows[j] - s.row0) * (size_t)e.d,
                                (size_t)e.d * sizeof(T), cudaMemcpyDeviceToHost, s.stream));
        found = true;
        break;
      }
    }
    if (!found) KM_FAIL(KM_EINVAL, "initialisation: row index outside the attached data");
  }
  for (auto& s : e.shards) {
    DevGuard g(s.dev);
    KM_CUDA(cudaStreamSynchronize(s.stream));
  }
  return KM_OK;
}

// method 0: seeded random rows; 1: k-means|| + weighted k-means++.  out: k x d row-major.
// `picked_rows` (optional) receives the global row index of every centre.
template <typename T>
int init_centroids(Engine<T>& e, int k, int seed, int method, std::vector<T>* out,
                   std::vector<size_t>* picked_rows = nullptr) {
  TraceRange trace_range("kmeans.init_centroids");
  if (e.shards.empty() || !e.shards[0].X) KM_FAIL(KM_ESTATE, "initialisation: no data attached");
  if (e.world_size != (int)e.shards.size())
    KM_FAIL(KM_ESTATE, "initialisation on the device needs one process owning all shards; pass explicit centroids");
  const size_t n = e.n_total;
  if (k < 1 || (size_t)k > n) KM_FAIL(KM_EINVAL, "initialisation: k must be in 1..rows");
  if (method != 0 && method != 1) KM_FAIL(KM_EINVAL, "initialisation: unknown method");
  const int d = e.d;
  std::vector<size_t> picked;
  if (method == 0) {
    if (n > 0x7fffffffULL) KM_FAIL(KM_EINVAL, "seeded row shuffle: more than INT_MAX rows");
    shuffled_row_ids(n, k, seed, &picked);
    KM_TRY(fetch_rows(e, picked, out));
    if (picked_rows) *picked_rows = picked;
    return KM_OK;
  }
  if (seed < 0) seed = (int)(std::random_device{}() & 0x7fffffff);
  const unsigned long long useed = (unsigned long long)(unsigned int)seed;
  KM_TRY(e.check_data());

  // 1. first candidate
  unsigned int c4[4] = {0u, 0u, 0u, kStreamFirst};
  philox_host(c4, (unsigned int)useed, (unsigned int)(useed >> 32));
  const size_t first = (size_t)((((unsigned long long)c4[0] << 32) | c4[1]) % (unsigned long long)n);
  picked.push_back(first);
  std::vector<T> all, fresh;
  KM_TRY(fetch_rows(e, picked, &fresh));
  all = fresh;

  // per-shard scratch
  const unsigned int cap = (unsigned int)std::min<size_t>((size_t)16 * k + 4096, n);
  std::vector<unsigned int*> d_list(e.shards.size(), nullptr), d_count(e.shards.size(), nullptr);
  std::vector<T*> d_rows(e.shards.size(), nullptr);
  auto release = [&]() {
    for (size_t i = 0; i < e.shards.size(); ++i) {
      DevGuard g(e.shards[i].dev);
      km_free(d_list[i]); km_free(d_count[i]); km_free(d_rows[i]);
    }
  };
  int rc = KM_OK;
  for (size_t i = 0; i < e.shards.size() && rc == KM_OK; ++i) {
    Shard<T>& s = e.shards[i];
    DevGuard g(s.dev);
    rc = ensure_dist(s);
    if (rc != KM_OK) break;
    if (km_malloc(&d_list[i], (size_t)cap * sizeof(unsigned int)) != cudaSuccess ||
        km_malloc(&d_count[i], sizeof(unsigned int)) != cudaSuccess ||
        km_malloc(&d_rows[i], (size_t)cap * d * sizeof(T)) != cudaSuccess) {
      set_error("initialisation: device allocation failed");
      rc = KM_ENOMEM;
      break;
    }
    fill_double_kernel<<<s.num_sms * 4, 256, 0, s.stream>>>(s.dist, s.rows, 1.7976931348623157e308);
  }
  if (rc != KM_OK) { release(); return rc; }

  // 2. sampling rounds
  const int rounds = std::min(8, (int)(2 + std::log((double)k)));
  for (int round = 0; round < rounds && rc == KM_OK; ++round) {
    const int m_new = (int)(fresh.size() / d);
    if (m_new > 0) {
      rc = e.set_centroids(m_new, fresh.data());
      if (rc == KM_OK) rc = e.assign_all(0);
      if (rc != KM_OK) break;
      for (auto& s : e.shards) {
        DevGuard g(s.dev);
        mincost_update_kernel<T><<<s.num_sms * 8, 256, 0, s.stream>>>(s.X, s.rows, d, s.labels, s.C[e.cur], s.dist);
      }
    }
    double phi = 0;
    for (auto& s : e.shards) {
      DevGuard g(s.dev);
      sum_partials_kernel<T><<<1024, 256, 0, s.stream>>>(s.dist, s.rows, s.sum_partials, e.weighted ? s.w : nullptr);
      sum_final_kernel<<<1, 32, 0, s.stream>>>(s.sum_partials, 1024, &s.st->inertia);
      double part = 0;
      if (cudaMemcpyAsync(&part, &s.st->inertia, sizeof(double), cudaMemcpyDeviceToHost, s.stream) != cudaSuccess ||
          cudaStreamSynchronize(s.stream) != cudaSuccess) {
        set_error("initialisation: cost reduction failed");
        rc = KM_ECUDA;
        break;
      }
      phi += part;
    }
    if (rc != KM_OK) break;
    log_msg(e.verbose, 400, "k-means|| round %d: %d new candidates, total cost %.6g", round, m_new, phi);
    fresh.clear();
    if (!(phi > 0)) continue;   // every row coincides with a candidate
    std::vector<size_t> round_rows;
    for (size_t i = 0; i < e.shards.size() && rc == KM_OK; ++i) {
      Shard<T>& s = e.shards[i];
      DevGuard g(s.dev);
      cudaMemsetAsync(d_count[i], 0, sizeof(unsigned int), s.stream);
      sample_rows_kernel<T><<<s.num_sms * 8, 256, 0, s.stream>>>(s.dist, s.rows, s.row0, phi, 2.0 * k, useed,
                                                                (unsigned int)round, d_list[i], cap, d_count[i],
                                                                e.weighted ? s.w : nullptr);
      unsigned int cnt = 0;
      if (cudaMemcpyAsync(&cnt, d_count[i], sizeof(cnt), cudaMemcpyDeviceToHost, s.stream) != cudaSuccess ||
          cudaStreamSynchronize(s.stream) != cudaSuccess) {
        set_error("initialisation: sampling failed");
        rc = KM_ECUDA;
        break;
      }
      if (cnt > cap) {
        log_msg(e.verbose, 300, "k-means||: %u rows drawn in one round, keeping %u", cnt, cap);
        cnt = cap;
      }
      if (cnt == 0) continue;
      std::vector<unsigned int> idx(cnt);
      if (cudaMemcpy(idx.data(), d_list[i], (size_t)cnt * sizeof(unsigned int), cudaMemcpyDeviceToHost) != cudaSuccess) {
        set_error("initialisation: sampling failed");
        rc = KM_ECUDA;
        break;
      }
      std::sort(idx.begin(), idx.end());   // the order of the atomic appends is not reproducible
      if (cudaMemcpy(d_list[i], idx.data(), (size_t)cnt * sizeof(unsigned int), cudaMemcpyHostToDevice) != cudaSuccess) {
        set_error("initialisation: sampling failed");
        rc = KM_ECUDA;
        break;
      }
      gather_rows_kernel<T><<<s.num_sms * 2, 256, 0, s.stream>>>(s.X, d, d_list[i], cnt, d_rows[i]);
      const size_t off = fresh.size();
      fresh.resize(off + (size_t)cnt * d);
      if (cudaMemcpyAsync(fresh.data() + off, d_rows[i], (size_t)cnt * d * sizeof(T), cudaMemcpyDeviceToHost,
                          s.stream) != cudaSuccess ||
          cudaStreamSynchronize(s.stream) != cudaSuccess) {
        set_error("initialisation: gather failed");
        rc = KM_ECUDA;
        break;
      }
      for (unsigned int j = 0; j < cnt; ++j) round_rows.push_back(s.row0 + idx[j]);
    }
    if (rc != KM_OK) break;
    all.insert(all.end(), fresh.begin(), fresh.end());
    picked.insert(picked.end(), round_rows.begin(), round_rows.end());
  }
  release();
  if (rc != KM_OK) return rc;

  const int m = (int)picked.size();
  log_msg(e.verbose, 400, "k-means||: %d candidates for k = %d", m, k);
  if (m <= k) {
    // keep them all; seeded distinct random rows fill the rest
    std::vector<size_t> rows = picked;
    std::vector<char> used_dummy;
    unsigned int ctr = 0;
    while ((int)rows.size() < k) {
      unsigned int c[4] = {ctr++, 0u, 0u, kStreamFill};
      philox_host(c, (unsigned int)useed, (unsigned int)(useed >> 32));
      const size_t r = (size_t)((((unsigned long long)c[0] << 32) | c[1]) % (unsigned long long)n);
      if (std::find(rows.begin(), rows.end(), r) == rows.end()) rows.push_back(r);
    }
    KM_TRY(fetch_rows(e, rows, out));
    if (picked_rows) *picked_rows = rows;
    return KM_OK;
  }

  // 3. weights = rows (sample weight) nearest to each candidate, then weighted k-means++ on the device
  KM_TRY(e.set_centroids(m, all.data()));
  KM_TRY(e.assign_all(0));
  std::vector<double> w(m, 0.0);
  {
    std::vector<unsigned long long> cnt(m);
    for (auto& s : e.shards) {
      DevGuard g(s.dev);
      unsigned long long* dc = nullptr;
      KM_CUDA(km_malloc(&dc, (size_t)m * sizeof(unsigned long long)));
      cudaMemsetAsync(dc, 0, (size_t)m * sizeof(unsigned long long), s.stream);
      label_histogram_kernel<T><<<s.num_sms * 8, 256, 0, s.stream>>>(s.labels, s.rows, m, dc,
                                                                    e.weighted ? s.w : nullptr, (T)e.w_scale);
      cudaError_t ce = cudaMemcpyAsync(cnt.data(), dc, (size_t)m * sizeof(unsigned long long), cudaMemcpyDeviceToHost,
                                       s.stream);
      if (ce == cudaSuccess) ce = cudaStreamSynchronize(s.stream);
      km_free(dc);
      if (ce != cudaSuccess) KM_FAIL(KM_ECUDA, "initialisation: candidate weights failed");
      for (int j = 0; j < m; ++j) w[j] += (double)cnt[j] * (e.weighted ? e.count_unit : 1.0);
    }
  }
  Shard<T>& s0 = e.shards[0];
  DevGuard g0(s0.dev);
  double *d_w = nullptr, *d_mind = nullptr, *d_wm = nullptr;
  int *d_state = nullptr, *d_chosen = nullptr;
  unsigned char* d_taken = nullptr;
  std::vector<int> chosen(k);
  cudaError_t ce = km_malloc(&d_w, (size_t)m * sizeof(double));
  if (ce == cudaSuccess) ce = km_malloc(&d_mind, (size_t)m * sizeof(double));
  if (ce == cudaSuccess) ce = km_malloc(&d_wm, (size_t)m * sizeof(double));
  if (ce == cudaSuccess) ce = km_malloc(&d_state, sizeof(int));
  if (ce == cudaSuccess) ce = km_malloc(&d_chosen, (size_t)k * sizeof(int));
  if (ce == cudaSuccess) ce = km_malloc(&d_taken, (size_t)m);
  if (ce == cudaSuccess) {
    cudaMemcpyAsync(d_w, w.data(), (size_t)m * sizeof(double), cudaMemcpyHostToDevice, s0.stream);
    cudaMemcpyAsync(d_wm, w.data(), (size_t)m * sizeof(double), cudaMemcpyHostToDevice, s0.stream);
    cudaMemsetAsync(d_taken, 0, (size_t)m, s0.stream);
    fill_double_kernel<<<64, 256, 0, s0.stream>>>(d_mind, (size_t)m, 1.7976931348623157e308);
    const int ugrid = std::max(1, std::min(s0.num_sms * 4, (m + 255) / 256));
    for (int step = 0; step < k; ++step) {
      kpp_select_kernel<<<1, 1024, 0, s0.stream>>>(d_wm, m, useed, step, d_state, d_chosen, d_taken);
      // candidates are the current centroid table of the engine (set above)
      kpp_update_kernel<T><<<ugrid, 256, 0, s0.stream>>>(s0.C[e.cur], m, d, d_state, d_w, d_mind, d_wm);
    }
    ce = cudaGetLastError();
    if (ce == cudaSuccess)
      ce = cudaMemcpyAsync(chosen.data(), d_chosen, (size_t)k * sizeof(int), cudaMemcpyDeviceToHost, s0.stream);
    if (ce == cudaSuccess) ce = cudaStreamSynchronize(s0.stream);
  }
  km_free(d_w); km_free(d_mind); km_free(d_wm); km_free(d_state); km_free(d_chosen); km_free(d_taken);
  if (ce != cudaSuccess) KM_FAIL(KM_ECUDA, std::string("initialisation: k-means++ stage: ") + cudaGetErrorString(ce));
  e.launches += 2 * k;
  out->resize((size_t)k * d);
  std::vector<size_t> rows(k);
  for (int j = 0; j < k; ++j) {
    const int c = chosen[j];
    if (c < 0 || c >= m) KM_FAIL(KM_ESTATE, "initialisation: k-means++ stage returned a bad index");
    std::copy(all.begin() + (size_t)c * d, all.begin() + (size_t)(c + 1) * d, out->begin() + (size_t)j * d);
    rows[j] = picked[c];
  }
  if (picked_rows) *picked_rows = rows;
  return KM_OK;
}

}  // namespace km
