// The Lloyd loop and the resident predict / transform / inertia passes.
#pragma once

#include "km_engine.cuh"

namespace km {

// The incremental M-step takes an iteration when at most 1 / kDeltaFraction of the shard's labels moved.
// Moving a row costs about three times its share of a full pass (two clusters touched, scattered
// reads), so the break-even lies near a third of the rows on wide rows and near a sixth on narrow
// ones (measured: 784 columns, 5.8 % moved: 0.35 ms against 2.39 ms for the full pass; 64 columns,
// 5.8 % moved: 0.24 ms against 0.63 ms).
constexpr unsigned long long kDeltaFraction = 8;

template <typename T>
static int ensure_dist(Shard<T>& s) {
  if (s.dist_cap < s.rows) {
    km_free(s.dist);
    s.dist = nullptr;
    KM_CUDA(km_malloc(&s.dist, s.rows * sizeof(double)));
    s.dist_cap = s.rows;
  }
  return KM_OK;
}

template <typename T>
static int ensure_logs(Shard<T>& s, int n) {
  if (s.log_cap < n) {
    km_free(s.shift_log); km_free(s.changed_log); km_free(s.reloc_log); km_free(s.amb_log);
    s.shift_log = nullptr; s.changed_log = nullptr; s.reloc_log = nullptr; s.amb_log = nullptr;
    KM_CUDA(km_malloc(&s.amb_log, n * sizeof(unsigned int)));
    KM_CUDA(km_malloc(&s.shift_log, n * sizeof(double)));
    KM_CUDA(km_malloc(&s.changed_log, n * sizeof(unsigned long long)));
    KM_CUDA(km_malloc(&s.reloc_log, n * sizeof(int)));
    s.log_cap = n;
  }
  return KM_OK;
}

// E-step on every local shard with the current centroids (final pass of fit,
// predict).  Labels change counters are not touched.
template <typename T>
int Engine<T>::assign_all(int flags) {
  TraceRange trace_range("kmeans.assign");
  if (!have_centroids) KM_FAIL(KM_ESTATE, "no centroids set");
  for (auto& s : shards) {
    if (!s.X) KM_FAIL(KM_ESTATE, "no data attached to the handle");
    DevGuard g(s.dev);
    // the same dispatch as the E-step of a fit (launch_assign picks the streaming kernel for few
    // centroids and wide rows, the small-k kernel for narrow ones)
    const bool use_tc = tc_ok(flags) && (!smallk_ok(false) || tc_kind() == 3);
    if (use_tc) {
      KM_TRY(tc_refresh(s));
      KM_CUDA(cudaMemsetAsync(&s.st->amb_count, 0, sizeof(unsigned int), s.stream));
    }
    KM_TRY(launch_assign(s, use_tc, false));
  }
  return KM_OK;
}

template <typename T>
int Engine<T>::relocate_multi(double scale, int seq, int* n_empty) {
  NcclApi* api = NcclApi::get();
  const size_t g = shards.size();
  std::vector<int> E(g, 0);
  for (size_t i = 0; i < g; ++i) {
    Shard<T>& s = shards[i];
    DevGuard gd(s.dev);
    // wait for this iteration's prepare kernel by polling the word it writes to pinned memory:
    // cheaper than a stream synchronisation, and the kernels queued behind it keep the GPU busy
    volatile int* seqp = reinterpret_cast<volatile int*>(&s.host_pin[3]);
    const double t0 = now_s();
    unsigned int spins = 0;
    while (*seqp != seq) {
      if ((++spins & 0xfff) == 0) {
        cudaError_t q = cudaStreamQuery(s.stream);
        if (q != cudaSuccess && q != cudaErrorNotReady) KM_CUDA(q);
        if (q == cudaSuccess && *seqp != seq) KM_FAIL(KM_ESTATE, "finalize kernel did not publish its sequence number");
        if (now_s() - t0 > 30.0) KM_FAIL(KM_ETIMEOUT, "timed out waiting for the iteration's cluster counts");
      }
    }
    E[i] = *reinterpret_cast<volatile int*>(&s.host_pin[2]);
  }
  for (size_t i = 1; i < g; ++i)
    if (E[i] != E[0]) KM_FAIL(KM_ESTATE, "shards disagree on the number of empty clusters");
  const int ne = E[0];
  *n_empty = ne;
  if (ne == 0) return KM_OK;
  const size_t rec_bytes = (size_t)ne * 32 + (size_t)ne * d * sizeof(T);
  // the buffers were sized for k records when the fit began: no rank can fail to allocate between
  // here and the all-gather and leave its peers waiting in it
  for (size_t i = 0; i < g; ++i) {
    Shard<T>& s = shards[i];
    DevGuard gd(s.dev);
    launch_rowdist(s, 1);
    KM_CUDA(cudaGetLastError());
    const T* Xp = s.X;
    size_t n = s.rows;
    int dd = d;
    const int* lab = s.labels;
    double* dist = s.dist;
    int ee = ne;
    unsigned long long id_base = (unsigned long long)(world_rank0 + (int)i) << 40;
    double* cv = s.cand_val;
    unsigned long long* cr = s.cand_row;
    unsigned char* rp = s.reloc_rec;
    const T* Wp = weighted ? s.w : nullptr;
    const IterState* gate = nullptr;
    FarScratch fs = s.far;
    void* args[] = {&Xp, &n, &dd, &lab, &dist, &ee, &id_base, &cv, &cr, &rp, &Wp, &gate, &fs};
    KM_CUDA(cudaLaunchCooperativeKernel((void*)select_far_kernel<T>, dim3(s.num_sms), dim3(256), args, 0, s.stream));
    launches += 2;
  }
  KM_NCCL(api, api->GroupStart());
  for (size_t i = 0; i < g; ++i)
    KM_NCCL(api, api->AllGather(shards[i].reloc_rec, shards[i].reloc_all, rec_bytes, ncclChar, shards[i].comm,
                                shards[i].stream));
  KM_NCCL(api, api->GroupEnd());
  for (size_t i = 0; i < g; ++i) {
    Shard<T>& s = shards[i];
    DevGuard gd(s.dev);
    apply_far_kernel<T><<<1, 256, 0, s.stream>>>(s.reloc_all, world_size, ne, rec_bytes, k, d, s.sums(),
                                                 s.counts(k, d), s.empties, s.st, (T)scale, weighted ? 1 : 0,
                                                 (T)w_scale);
    KM_CUDA(cudaGetLastError());
    ++launches;
  }
  return KM_OK;
}

template <typename T>
SplitTable Engine<T>::split_table(Shard<T>& s, bool use_tc) {
  SplitTable tp{nullptr, nullptr, nullptr, 0, 0, 0.f, 0.f};
  if constexpr (std::is_same<T, float>::value) {
    if (use_tc && tc_kind() == 4)
      tp = SplitTable{s.tcsp.bhi, s.tcsp.blo, s.tcsp.cn, s.tcsp.kpad, s.tcsp.dp, s.tcsp.sb, s.tcsp.sx * s.tcsp.sb};
    else if (use_tc && tc_kind() == 3)
      tp = SplitTable{s.tcwp.bhi, s.tcwp.blo, s.tcwp.cn, tcw::kNPad, s.tcwp.dp, s.tcwp.sb, s.tcwp.sx * s.tcwp.sb};
    else if (use_tc && tc_kind() == 1)
      tp = SplitTable{s.tcp.bhi, s.tcp.blo, s.tcp.cn, s.tcp.npad, 64, s.tcp.sb, s.tcp.sx * s.tcp.sb};
    else if (use_tc)
      tp = SplitTable{s.tcbp.bhi, s.tcbp.blo, s.tcbp.cn, s.tcbp.kpad, s.tcbp.dp, s.tcbp.sb, s.tcbp.sx * s.tcbp.sb};
  }
  return tp;
}

// Closes iteration `it` on a shard: new centroids into C[cur ^ 1] (and the tensor-core operand table)
template <typename T>
int Engine<T>::launch_close(Shard<T>& s, int run_if, int it, double inv, bool use_tc) {
  close_kernel<T><<<k, 128, 0, s.stream>>>(s.sums(), s.counts(k, d), k, d, inv, s.C[cur], s.C[cur ^ 1], s.cnorm,
                                           s.shift_k, s.st, s.Cd[cur ^ 1], run_if, weighted ? count_unit : 1.0,
                                           s.shift_log, s.changed_log, s.reloc_log, s.amb_log, it, &s.host_pin[0],
                                           reinterpret_cast<unsigned long long*>(&s.host_pin[1]), s.ticket,
                                           split_table(s, use_tc));
  KM_CUDA(cudaGetLastError());
  ++launches;
  return KM_OK;
}

template <typename T>
int Engine<T>::fit(int k_, int max_iter, double threshold, const T* init, int flags) {
  TraceRange trace_range("kmeans.fit");
  if (k_ < 1 || max_iter < 0 || !init) KM_FAIL(KM_EINVAL, "kmeans_fit_resident: bad argument");
  if (shards.empty() || !shards[0].X) KM_FAIL(KM_ESTATE, "kmeans_fit_resident: no data attached");
  if (world_size > 64) KM_FAIL(KM_EINVAL, "at most 64 ranks");
  const double t_start = now_s();
  launches = 0;
  KM_TRY(check_data());
  KM_TRY(set_centroids(k_, init));

  // fixed-point scale from the global max |x|: xmax < 2^e, first piece <= 2^15 (with sample
  // weights the sums hold w * x, bounded by the product of the two maxima)
  double xmax = 0;
  for (auto& s : shards) xmax = std::max(xmax, s.xmax);
  if (weighted) xmax *= wmax;
  int e = 0;
  if (xmax > 0) std::frexp(xmax, &e);
  const int sa = kPieceBits - e;
  const T scale = (T)std::ldexp(1.0, sa);
  const double inv = std::ldexp(1.0, -(sa + kPieceBits));
  if (!std::isfinite((double)scale) || scale == (T)0) KM_FAIL(KM_EINVAL, "data magnitude outside the supported range");

  // weighted fits take the general M-step kernel for full passes (the fused small-k update and
  // the sorted pass do not carry weights); the incremental sums do
  const bool fused = smallk_ok(true) && !(flags & KM_FIT_FORCE_SPLIT) && !weighted;
  const bool use_tc = !fused && tc_ok(flags);
  // the split copy of X (d = 64 tensor-core kernel without converter warps) costs about as much as
  // sixteen iterations save
  tc_split_build = max_iter >= 16 || (flags & KM_FIT_PRESPLIT);
  struct SplitBuildGuard { bool& f; ~SplitBuildGuard() { f = false; } } split_build_guard{tc_split_build};
  // incremental M-step (km_accumulate_delta.cuh): on unless the caller or the environment asks
  // for a full recomputation every iteration; a shard switches to it, on the device, in the
  // iterations where at most 1/8 of its labels moved (kDeltaFraction)
  static const bool delta_env = [] {
    const char* e = std::getenv("H2O4GPU_KM_DELTA_SUMS");
    return !(e && e[0] == '0');
  }();
  const bool delta = !fused && delta_env && !(flags & KM_FIT_FULL_SUMS);
  const bool multi = world_size > 1;
  const bool check = (threshold > 0) || (flags & KM_FIT_CHECK_EVERY_ITER);
  stats = kmeans_stats{};
  stats.path = fused ? 1 : (use_tc ? 3 : 2);
  stats.inertia = -1;

  for (auto& s : shards) {
    DevGuard g(s.dev);
    KM_TRY(ensure_logs(s, std::max(max_iter, 1)));
    KM_TRY(ensure_dist(s));
    if (multi) {
      // candidate records of the host-driven repair (several ranks over NCCL only), sized for k
      // records now so that no rank can fail to allocate once the ranks depend on one another
      const size_t need = ((size_t)k_ * 32 + (size_t)k_ * d * sizeof(T) + 15) / 16 * 16;
      if (s.reloc_cap < need) {
        km_free(s.reloc_rec); km_free(s.reloc_all);
        s.reloc_rec = s.reloc_all = nullptr;
        s.reloc_cap = 0;
        KM_CUDA(km_malloc(&s.reloc_rec, need));
        KM_CUDA(km_malloc(&s.reloc_all, need * (size_t)world_size));
        s.reloc_cap = need;
      }
    }
    KM_CUDA(cudaMemsetAsync(s.st, 0, sizeof(IterState), s.stream));
    KM_CUDA(cudaMemsetAsync(s.labels, 0xff, s.rows * sizeof(int), s.stream));
    if (delta && s.labels_prev_cap < s.rows) {
      km_free(s.labels_prev);
      km_free(s.moved_bits);
      s.labels_prev = nullptr;
      s.moved_bits = nullptr;
      KM_CUDA(km_malloc(&s.labels_prev, s.rows * sizeof(int)));
      KM_CUDA(km_malloc(&s.moved_bits, (s.rows / 32 + 8) * sizeof(unsigned int)));
      s.labels_prev_cap = s.rows;
    }
    s.moved_bits_valid = false;
    if (s.pflush)   // all zero between iterations; cleared here in case an earlier fit stopped half-way
      KM_CUDA(cudaMemsetAsync(s.pflush, 0, s.gacc_count(k, d) * kFlushPad * sizeof(long long), s.stream));
    if (use_tc) KM_TRY(tc_refresh(s));
  }

  // events on shard 0: [4*it + 0..3] = start, after E-step, after sums, after close
  Shard<T>& s0 = shards[0];
  std::vector<cudaEvent_t> ev((size_t)4 * std::max(max_iter, 1) + 2, nullptr);
  {
    DevGuard g(s0.dev);
    for (auto& x : ev) KM_CUDA(cudaEventCreate(&x));
  }
  auto free_events = [&]() {
    DevGuard g(s0.dev);
    for (auto& x : ev) if (x) cudaEventDestroy(x);
  };

  int it = 0;
  int rc = KM_OK;
  for (; it < max_iter; ++it) {
    TraceRange iteration_range("kmeans.iteration");   // host side: the launches of one iteration are queued here
    for (size_t i = 0; i < shards.size() && rc == KM_OK; ++i) {
      Shard<T>& s = shards[i];
      DevGuard g(s.dev);
      if (i == 0) cudaEventRecord(ev[4 * it + 0], s.stream);
      if (!delta) cudaMemsetAsync(s.gacc, 0, s.gacc_count(k, d) * sizeof(long long), s.stream);
      if (fused) {
        rc = launch_smallk(s, true, scale);
        if (i == 0) { cudaEventRecord(ev[4 * it + 1], s.stream); cudaEventRecord(ev[4 * it + 2], s.stream); }
      } else if (delta) {
        rc = launch_assign(s, use_tc, true);
        if (i == 0) cudaEventRecord(ev[4 * it + 1], s.stream);
        // both branches are launched; the label-change counter decides on the device which one works
        const unsigned long long* gate = (it == 0) ? nullptr : &s.st->changed;
        const unsigned long long limit = s.rows / kDeltaFraction;
        if (rc == KM_OK) {
          full_prologue_kernel<<<s.num_sms * 4, 256, 0, s.stream>>>(s.pacc, s.gacc_count(k, d), s.labels,
                                                                     s.labels_prev, s.rows, gate, limit);
          ++launches;
          rc = launch_accumulate(s, scale, s.pacc, gate, limit);
        }
        if (rc == KM_OK && it > 0) rc = launch_delta(s, scale, gate, limit);
        if (rc == KM_OK) {
          // fold the padded drain array into the label-only sums; one shard: also the working copy
          const size_t cnt = s.gacc_count(k, d);
          if (!multi || s.pflush) {
            fold_flush_kernel<<<(unsigned)std::min<size_t>((cnt + 255) / 256, (size_t)s.num_sms * 4), 256, 0, s.stream>>>(
                s.pflush, s.pacc, multi ? nullptr : s.gacc, cnt);
            ++launches;
          }
        }
        if (i == 0) cudaEventRecord(ev[4 * it + 2], s.stream);
      } else {
        rc = launch_assign(s, use_tc, true);
        if (i == 0) cudaEventRecord(ev[4 * it + 1], s.stream);
        if (rc == KM_OK) rc = launch_accumulate(s, scale);
        if (i == 0) cudaEventRecord(ev[4 * it + 2], s.stream);
      }
    }
    if (rc != KM_OK) break;
    const int seq = ++poll_seq;
    if (multi && (rc = allreduce_from(delta)) != KM_OK) break;
    // Empty clusters are repaired on the device whenever the ranks can reach one another's memory
    // (one rank, or the push path): the repair kernels are queued every iteration and return at
    // once unless the M-step left a cluster empty, and the closing kernel is queued twice, before
    // them for the usual case and behind them for the repaired one.  The host never waits.
    // Several ranks over NCCL only: the host reads the count of empty clusters (a pinned word) and
    // drives the repair, with the closing kernel queued ahead for the usual case.
    const bool host_repair = multi && stats.allreduce_path != 1;
    for (size_t i = 0; i < shards.size() && rc == KM_OK; ++i) {
      Shard<T>& s = shards[i];
      DevGuard g(s.dev);
      prepare_kernel<<<1, 256, 0, s.stream>>>(s.counts(k, d), k, s.st, s.empties,
                                             host_repair ? reinterpret_cast<int*>(&s.host_pin[2]) : nullptr,
                                             host_repair ? reinterpret_cast<int*>(&s.host_pin[3]) : nullptr, seq);
      ++launches;
      rc = launch_close(s, 0, it, inv, use_tc);
      if (rc != KM_OK || host_repair) continue;
      launch_rowdist(s, 0);
      ++launches;
      const T* Xp = s.X;
      size_t n = s.rows;
      int dd = d, kk = k;
      const int* lab = s.labels;
      double* dist = s.dist;
      double* cv = s.cand_val;
      unsigned long long* cr = s.cand_row;
      const T* Wp = weighted ? s.w : nullptr;
      cudaError_t ce;
      if (!multi) {
        long long* gs = s.sums();
        unsigned long long* gc = s.counts(k, d);
        const int* em = s.empties;
        IterState* st = s.st;
        T sc = scale;
        T wsc = (T)w_scale;
        FarScratch fs = s.far;
        void* args[] = {&Xp, &n, &dd, &lab, &kk, &dist, &gs, &gc, &em, &st, &cv, &cr, &sc, &Wp, &wsc, &fs};
        ce = cudaLaunchCooperativeKernel((void*)relocate_kernel<T>, dim3(s.num_sms), dim3(256), args, 0, s.stream);
        ++launches;
      } else {
        int ee = 0;
        unsigned long long id_base = (unsigned long long)(world_rank0 + (int)i) << 40;
        unsigned char* rp = s.push.grec;
        const IterState* gate = s.st;
        FarScratch fs = s.far;
        void* args[] = {&Xp, &n, &dd, &lab, &dist, &ee, &id_base, &cv, &cr, &rp, &Wp, &gate, &fs};
        ce = cudaLaunchCooperativeKernel((void*)select_far_kernel<T>, dim3(s.num_sms), dim3(256), args, 0, s.stream);
        if (ce == cudaSuccess) {
          gather_apply_kernel<T><<<1, 256, 0, s.stream>>>(
              s.push.grec, s.push.gslot, world_rank0 + (int)i, world_size, s.push.d_peer_gmail, s.push.d_peer_gflags,
              s.push.gmail, s.push.flags + (size_t)2 * world_size, (unsigned int)seq, wait_limits().push_spins, k, d,
              s.sums(), s.counts(k, d), s.empties, s.st, scale, weighted ? 1 : 0, (T)w_scale);
          ce = cudaGetLastError();
        }
        launches += 2;
      }
      if (ce != cudaSuccess) { set_error(std::string("repair launch: ") + cudaGetErrorString(ce)); rc = KM_ECUDA; }
      if (rc == KM_OK) rc = launch_close(s, 1, it, inv, use_tc);
    }
    if (rc != KM_OK) break;
    if (host_repair) {
      int ne = 0;
      if ((rc = relocate_multi((double)scale, seq, &ne)) != KM_OK) break;
      if (ne > 0)
        for (size_t i = 0; i < shards.size() && rc == KM_OK; ++i) {
          DevGuard g(shards[i].dev);
          rc = launch_close(shards[i], 1, it, inv, use_tc);
        }
      if (rc != KM_OK) break;
    }
    {
      DevGuard g(s0.dev);
      cudaEventRecord(ev[4 * it + 3], s0.stream);
    }
    cur ^= 1;   // (the closing kernel also wrote the tensor-core kernels' operand table for these centroids)
    if (check) {
      DevGuard g(s0.dev);
      cudaError_t ce = cudaStreamSynchronize(s0.stream);
      if (ce != cudaSuccess) { set_error(std::string("iteration sync: ") + cudaGetErrorString(ce)); rc = KM_ECUDA; break; }
      double shift = *reinterpret_cast<volatile double*>(&s0.host_pin[0]);
      unsigned long long changed = *reinterpret_cast<volatile unsigned long long*>(&s0.host_pin[1]);
      log_msg(verbose, 400, "iteration %d: shift^2 %.6g, %llu labels changed", it, shift, changed);
      // the reference's test, src/gpu/kmeans/kmeans_impl.h:202
      if (threshold > 0 && shift < threshold) { ++it; break; }
      if ((flags & KM_FIT_CHECK_EVERY_ITER) && changed == 0 && !multi) { ++it; break; }
    }
  }
  if (rc != KM_OK) { free_events(); return rc; }
  const int done = it;
  {
    DevGuard g(s0.dev);
    cudaEventRecord(ev[ev.size() - 2], s0.stream);
  }
  if (!(flags & KM_FIT_NO_FINAL_ASSIGN)) {
    rc = assign_all(flags);
    if (rc != KM_OK) { free_events(); return rc; }
  }
  {
    DevGuard g(s0.dev);
    cudaEventRecord(ev[ev.size() - 1], s0.stream);
  }
  for (auto& s : shards) {
    DevGuard g(s.dev);
    cudaError_t ce = cudaStreamSynchronize(s.stream);
    if (ce != cudaSuccess) { set_error(std::string("fit sync: ") + cudaGetErrorString(ce)); free_events(); return KM_ECUDA; }
  }
  for (auto& s : shards) {
    DevGuard g(s.dev);
    IterState hs;
    cudaError_t ce = cudaMemcpy(&hs, s.st, sizeof(hs), cudaMemcpyDeviceToHost);
    if (ce != cudaSuccess) { set_error(std::string("fit state: ") + cudaGetErrorString(ce)); free_events(); return KM_ECUDA; }
    if (hs.error != 0) {
      std::string msg = "a bounded device-side wait gave up (code " + std::to_string(hs.error) + ")";
      int diag[16][4];
      if (cudaMemcpyFromSymbol(diag, tc::g_wait_diag, sizeof(diag)) == cudaSuccess) {
        msg += "; waits [site: cta, tile counter, parity, 1 gave up / 2 saw abort]:";
        for (int c = 1; c < 16; ++c)
          if (diag[c][3] != 0)
            msg += " [" + std::to_string(c) + ": " + std::to_string(diag[c][0]) + ", " + std::to_string(diag[c][1]) +
                   ", " + std::to_string(diag[c][2]) + ", " + std::to_string(diag[c][3]) + "]";
      }
      set_error(msg);
      free_events();
      return KM_ETIMEOUT;
    }
  }
  // logs -> stats
  {
    DevGuard g(s0.dev);
    stats.iterations = done;
    if (done > 0) {
      std::vector<double> sh(done);
      std::vector<unsigned long long> ch(done);
      std::vector<int> rl(done);
      std::vector<unsigned int> am(done);
      KM_CUDA(cudaMemcpy(am.data(), s0.amb_log, done * sizeof(unsigned int), cudaMemcpyDeviceToHost));
      for (int i = 0; i < done; ++i) stats.refined_rows += (long long)am[i];
      KM_CUDA(cudaMemcpy(sh.data(), s0.shift_log, done * sizeof(double), cudaMemcpyDeviceToHost));
      KM_CUDA(cudaMemcpy(ch.data(), s0.changed_log, done * sizeof(unsigned long long), cudaMemcpyDeviceToHost));
      KM_CUDA(cudaMemcpy(rl.data(), s0.reloc_log, done * sizeof(int), cudaMemcpyDeviceToHost));
      stats.last_shift_sq = sh[done - 1];
      if (!multi) {
        for (int i = 0; i < done; ++i)
          if (ch[i] == 0) { stats.n_iter_converged = i + 1; break; }
      }
      for (int i = 0; i < done; ++i) stats.relocations += rl[i];
      if (delta)
        for (int i = 1; i < done; ++i) stats.incremental_iterations += (ch[i] <= s0.rows / kDeltaFraction);
      float a = 0, u = 0, ms = 0;
      static const bool trace = std::getenv("H2O4GPU_KM_TRACE") != nullptr;
      for (int i = 0; i < done; ++i) {
        float ma = 0, mu = 0;
        cudaEventElapsedTime(&ma, ev[4 * i + 0], ev[4 * i + 1]);
        a += ma;
        cudaEventElapsedTime(&mu, ev[4 * i + 1], ev[4 * i + 3]);
        u += mu;
        if (trace)
          std::fprintf(stderr, "[kmeans] iteration %d: %llu labels changed, %u rows re-evaluated, %d relocated, "
                       "E-step %.3f ms, M-step %.3f ms\n", i, ch[i], am[i], rl[i], ma, mu);
      }
      stats.ms_assign = a;
      stats.ms_update = u;
      cudaEventElapsedTime(&ms, ev[0], ev[ev.size() - 2]);
      stats.ms_loop = ms;
    }
    if (!(flags & KM_FIT_NO_FINAL_ASSIGN)) {
      float mf = 0;
      cudaEventElapsedTime(&mf, ev[ev.size() - 2], ev[ev.size() - 1]);
      stats.ms_final_assign = mf;
    }
  }
  free_events();
  stats.gpu_launches = launches;
  stats.seconds_fit = now_s() - t_start;
  return KM_OK;
}

// Sum of squared distances of every row to its assigned centre (direct
// differences, double), all local shards; all-reduced over ranks.
template <typename T>
int Engine<T>::inertia(double* out) {
  TraceRange trace_range("kmeans.inertia");
  KM_TRY(inertia_launch());
  return inertia_collect(out);
}

// the kernels of the inertia pass, queued; inertia_collect() waits for them and reads the sum
template <typename T>
int Engine<T>::inertia_launch() {
  if (!have_centroids) KM_FAIL(KM_ESTATE, "no centroids set");
  for (auto& s : shards) {
    DevGuard g(s.dev);
    KM_TRY(ensure_dist(s));
    launch_rowdist(s, 1);
    sum_partials_kernel<T><<<1024, 256, 0, s.stream>>>(s.dist, s.rows, s.sum_partials, weighted ? s.w : nullptr);
    sum_final_kernel<<<1, 32, 0, s.stream>>>(s.sum_partials, 1024, &s.st->inertia);
    KM_CUDA(cudaGetLastError());
    launches += 3;
  }
  if (world_size > 1) {
    NcclApi* api = NcclApi::get();
    KM_NCCL(api, api->GroupStart());
    for (auto& s : shards)
      KM_NCCL(api, api->AllReduce(&s.st->inertia, &s.st->inertia, 1, ncclDouble, ncclSum, s.comm, s.stream));
    KM_NCCL(api, api->GroupEnd());
  }
  return KM_OK;
}

template <typename T>
int Engine<T>::inertia_collect(double* out) {
  double total = 0;
  if (world_size > 1) {
    Shard<T>& s = shards[0];
    DevGuard g(s.dev);
    KM_CUDA(cudaMemcpyAsync(&total, &s.st->inertia, sizeof(double), cudaMemcpyDeviceToHost, s.stream));
    KM_CUDA(cudaStreamSynchronize(s.stream));
  } else {
    Shard<T>& s = shards[0];
    DevGuard g(s.dev);
    KM_CUDA(cudaMemcpyAsync(&total, &s.st->inertia, sizeof(double), cudaMemcpyDeviceToHost, s.stream));
    KM_CUDA(cudaStreamSynchronize(s.stream));
  }
  *out = total;
  stats.inertia = total;
  return KM_OK;
}

// Squared distances of one shard, column-major with leading dimension ld, to the host.
template <typename T>
int Engine<T>::transform_shard(int local, T* out_host, size_t ld) {
  TraceRange trace_range("kmeans.transform");
  if (local < 0 || local >= (int)shards.size() || !out_host) KM_FAIL(KM_EINVAL, "kmeans_transform_resident: bad argument");
  if (!have_centroids) KM_FAIL(KM_ESTATE, "no centroids set");
  Shard<T>& s = shards[local];
  if (ld < s.rows) KM_FAIL(KM_EINVAL, "kmeans_transform_resident: ld smaller than the shard");
  // max|x| (the tensor-core kernel's operand scale) is known after the data check; with several
  // processes that check is a collective and is left to the fit
  if (world_size == (int)shards.size()) KM_TRY(check_data());
  DevGuard g(s.dev);
  // row batches bound the device block to about 256 MB
  size_t batch = std::max<size_t>(128, ((size_t)1 << 28) / ((size_t)k * sizeof(T)));
  if (const char* e = std::getenv("H2O4GPU_KM_TRANSFORM_BATCH_ROWS")) {   // smaller blocks (tests of the batching)
    const long long v = std::atoll(e);
    if (v > 0) batch = (size_t)v;
  }
  batch = (batch + 127) / 128 * 128;
  batch = std::min(batch, (s.rows + 127) / 128 * 128);
  T* buf = nullptr;
  KM_CUDA(km_malloc(&buf, batch * (size_t)k * sizeof(T)));
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  cudaEventCreate(&e0);
  cudaEventCreate(&e1);
  float ms_kernels = 0;
  int rc = KM_OK;
  bool wide = false, streamed = false;
  if constexpr (std::is_same<T, float>::value) {
    // tensor-core kernels with a store epilogue (they need max|x| for the operand scales, i.e. a checked
    // matrix): the wide-row kernel for few centroids, the kernel that streams both operands for the rest
    if (tc_kind() == 3 && tc_ok(0)) {
      rc = tc_refresh(s);
      wide = rc == KM_OK;
    } else if (tcs::stream_shape_ok(k, dtc()) && tc_ok(0)) {
      if (tc_kind() == 4) {
        rc = tc_refresh(s);
      } else {
        // the shape's own labelling kernel keeps its plan; the streaming kernel gets one beside it
        double xmax = 0;
        for (const auto& sh : shards) xmax = std::max(xmax, sh.xmax);
        if (!tc::pick_scales(xmax, std::max(xmax, cbound), &tc_sx, &tc_sb)) rc = KM_EINVAL;
        if (rc == KM_OK) rc = stream_refresh(s);
        if (rc == KM_OK) ++launches;
      }
      streamed = rc == KM_OK;
      if (!streamed) rc = KM_OK;   // fall back to the FMA tile kernel
    }
  }
  for (size_t r = 0; r < s.rows && rc == KM_OK; r += batch) {
    size_t nr = std::min(batch, s.rows - r);
    cudaEventRecord(e0, s.stream);
    if constexpr (std::is_same<T, float>::value) {
      if (wide) {
        rc = tcw::wide_launch(s.tcwp, s.tcp.xnorm, nullptr, s.st, false, nullptr, tc::tol_rel_of(d), s.num_sms, s.stream, r, nr,
                              buf, batch);
        ++launches;
      } else if (streamed) {
        rc = tcs::stream_launch(s.tcsp, s.tcp.xnorm, nullptr, s.st, false, nullptr, tc::tol_rel_of(d), s.num_sms, s.stream, r,
                                nr, buf, batch);
        ++launches;
      }
    }
    if (!wide && !streamed) rc = launch_tiles(s, s.X + r * (size_t)d, nr, nullptr, MODE_TRANSFORM, buf, batch, false);
    if (rc != KM_OK) break;
    cudaEventRecord(e1, s.stream);
    cudaError_t ce = cudaMemcpy2DAsync(out_host + r, ld * sizeof(T), buf, batch * sizeof(T), nr * sizeof(T), k,
                                       cudaMemcpyDeviceToHost, s.stream);
    if (ce == cudaSuccess) ce = cudaStreamSynchronize(s.stream);
    if (ce != cudaSuccess) { set_error(std::string("transform copy: ") + cudaGetErrorString(ce)); rc = KM_ECUDA; }
    float ms = 0;
    if (cudaEventElapsedTime(&ms, e0, e1) == cudaSuccess) ms_kernels += ms;
  }
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  if (local == 0) {
    stats.ms_transform = ms_kernels;
    stats.path = (wide || streamed) ? 3 : 2;
  }
  km_free(buf);
  return rc;
}

}  // namespace km
