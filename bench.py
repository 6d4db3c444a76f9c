#!/usr/bin/env python
"""k-means throughput: points*iterations per second of the resident Lloyd loop.

A step is one Lloyd iteration (E-step + M-step) over the resident shard(s).
Workload at every N: the single-GPU bandwidth-regime configuration per GPU
(n = 10,000,000 rows, d = 64, k = 100, float32, 100-component Gaussian mixture
with Dirichlet(1) weights, sigma 1, centres U(-10,10)^64, init = 100 seeded
rows), i.e. weak scaling: rows are sharded over ranks, one NCCL all-reduce of the
k x d sums and k counts per iteration, X stays resident.  Inputs are synthetic
(seeded generator on the device); 2.56 GB per GPU, larger than L2, so no flush
is needed between iterations.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Under torchrun (N > 1) each rank drives its LOCAL_RANK GPU.  Rank 0 prints one
JSON line.  --impl reference times the reference's CPU path (scikit-learn's
Lloyd solver, which h2o4gpu.KMeans(n_gpus=0) runs) on the host cores.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (rows per GPU, d, k, mixture components, sigma, centre half-range, Dirichlet weights?)
    "c2": dict(n=10_000_000, d=64, k=100, comp=100, sigma=1.0, half=10.0, dirichlet=True, T=50),
    "c3": dict(n=25_000_000, d=128, k=1000, comp=1000, sigma=2.0, half=20.0, dirichlet=False, T=30),
    "c1": dict(n=100_000, d=32, k=8, comp=8, sigma=1.0, half=10.0, dirichlet=False, T=20),
    # contraction-bound shape (rows per GPU of the 8-GPU split of n = 4e7); offset centres N(0, 4I)
    # are approximated by U(-3.5, 3.5) centres of the same variance
    "c5": dict(n=5_000_000, d=256, k=4096, comp=4096, sigma=1.0, half=3.5, dirichlet=False, T=10),
    # image-like rows (0 with probability 0.8, else an integer in 1..255): bandwidth-bound, fused small-k kernel
    "c4": dict(n=2_000_000, d=784, k=10, comp=0, sigma=0.0, half=0.0, dirichlet=False, T=100, kind=1),
}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            j = json.load(f)
        return float(j["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def tensor_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return float(json.load(f)["bf16_tflops"])
    return 1590.0


class ClockSampler(object):
    """nvidia-smi clocks and throttle reasons during the timed region."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "--query-gpu=" + self.Q, "--format=csv,noheader,nounits",
                                          "-i", str(self.index), "-lms", "100"], stdout=subprocess.PIPE, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def mixture_params(w, seed=0):
    if w.get("kind", 0) == 1:
        return None, None
    rng = np.random.default_rng(seed)
    centers = rng.uniform(-w["half"], w["half"], (w["comp"], w["d"])).astype(np.float32)
    weights = rng.dirichlet(np.ones(w["comp"])).astype(np.float32) if w["dirichlet"] else None
    return centers, weights


def host_sample(w, n, seed=0):
    """The same distribution on the host (numpy), for the CPU arm."""
    rng = np.random.default_rng(seed)
    if w.get("kind", 0) == 1:
        X = np.where(rng.random((n, w["d"])) < 0.8, 0, rng.integers(1, 256, (n, w["d"]))).astype(np.float32)
        return X, X[:w["k"]].copy()
    centers = rng.uniform(-w["half"], w["half"], (w["comp"], w["d"]))
    weights = rng.dirichlet(np.ones(w["comp"])) if w["dirichlet"] else None
    comp = rng.choice(w["comp"], n, p=weights) if weights is not None else rng.integers(0, w["comp"], n)
    X = np.empty((n, w["d"]), np.float32)
    for s in range(0, n, 1 << 19):
        e = min(n, s + (1 << 19))
        X[s:e] = centers[comp[s:e]] + w["sigma"] * rng.standard_normal((e - s, w["d"]))
    init = X[np.sort(rng.choice(n, w["k"], replace=False))].copy()
    return X, init


def cpu_arm(w, n_sample, iters, warm):
    """scikit-learn Lloyd (the reference's CPU path) on a bounded sample, all host threads."""
    from oracle import sklearn_oracle as sk
    X, init = host_sample(w, n_sample)
    if warm > 0:
        sk.fit(X[: max(w["k"] * 4, n_sample // 8)], init, warm)
    r = sk.timed_fit(X, init, iters)
    info = sk.thread_info()
    threads = max([p["threads"] or 1 for p in info["pools"]] + [1])
    return {"value": r["points_iters_per_s"], "unit": "points*iters/s", "cores": threads, "kind": "port",
            "sample": "scikit-learn %s KMeans(algorithm='lloyd', n_init=1, tol=0) = the solver "
                      "h2o4gpu.KMeans(n_gpus=0) delegates to; n=%d of the workload's rows, same d/k/distribution, "
                      "%d iterations in %.2f s; host has %d logical cores" %
                      (__import__("sklearn").__version__, n_sample, r["n_iter"], r["seconds"], info["cpu_count"]),
            "_seconds": r["seconds"], "_iters": r["n_iter"]}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--workload", default=os.environ.get("KM_BENCH_WORKLOAD", "c2"))
    ap.add_argument("--rows", type=int, default=0, help="rows per GPU (default: the workload's)")
    ap.add_argument("--cpu-rows", type=int, default=2_000_000)
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--flags", type=int, default=0)
    args = ap.parse_args()
    w = dict(WORKLOADS[args.workload])
    if args.rows:
        w["n"] = args.rows
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    K, W = args.steps, max(args.warmup, 0)
    dist_name = ("image-like rows (0 w.p. 0.8, else 1..255)" if w.get("kind", 0) == 1
                 else "%d-component Gaussian mixture" % w["comp"])
    config = {"workload": "%s: n=%d rows/GPU x d=%d fp32, k=%d, %s, seeded init rows"
                          % (args.workload, w["n"], w["d"], w["k"], dist_name),
              "rows_per_gpu": w["n"], "d": w["d"], "k": w["k"], "sharding": "rows, dp%d" % world,
              "l2": "inputs (%.2f GB/GPU) exceed L2; no flush needed" % (w["n"] * w["d"] * 4 / 1e9)}

    if args.impl == "reference":
        if rank != 0:
            return
        n_s = min(args.cpu_rows, w["n"])
        c = cpu_arm(w, n_s, K, W)
        line = {"impl": "reference", "metric": "kmeans_points_iters_per_sec", "value": c["value"],
                "unit": "points*iters/s", "n_gpus": args.gpus, "steps": c["_iters"], "warmup": W,
                "ms_per_step": 1e3 * c["_seconds"] / max(c["_iters"], 1), "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config,
                "cpu_baseline": {k: v for k, v in c.items() if not k.startswith("_")},
                "e2e": {"value": c["value"], "unit": "points*iters/s", "h2d_bytes_per_step": 0,
                        "d2h_bytes_per_step": 0},
                "gpu_launches": 0}
        print(json.dumps(line))
        return

    import torch
    from h2o4gpu_b200 import engine
    from h2o4gpu_b200.libs import lib_kmeans
    lib_kmeans.get()  # no CUDA library / device -> raise, never a CPU path
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    nccl_id = None
    if world > 1:
        import torch.distributed as dist
        from h2o4gpu_b200 import dist as kd
        dist.init_process_group("nccl", device_id=dev)
        nccl_id = kd.broadcast_bytes(engine.ResidentKMeans.nccl_unique_id() if rank == 0 else bytes(128), 0, dev)

    n, d, k = w["n"], w["d"], w["k"]
    centers, weights = mixture_params(w)
    X = torch.empty((n, d), dtype=torch.float32, device=dev)
    engine.synth_device(X.data_ptr(), n, d, np.float32, row0=rank * n, kind=w.get("kind", 0), centers=centers, weights=weights,
                        sigma=w["sigma"], seed=1234, gpu_id=local_rank)
    # seeded initial rows, taken from rank 0's shard and shared
    rows0 = np.sort(np.random.default_rng(7).choice(n, k, replace=False))
    init = X[torch.from_numpy(rows0).to(dev)].cpu().numpy()
    if world > 1:
        init = kd.broadcast_array(init, 0, dev)

    h = engine.ResidentKMeans(np.float32, devices=(local_rank,), rank0=rank, world_size=world, nccl_id=nccl_id)
    h.attach_device(0, X.data_ptr(), n, d, n_total=n * world)
    # per-upload preparation (row norms, fp16-split copy of the rows for the d = 64 kernel) happens in the warm-up
    flags = engine.FIT_NO_FINAL_ASSIGN | engine.FIT_PRESPLIT | args.flags

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    if W > 0:
        h.fit(init, W, flags=flags)
    sampler = ClockSampler(local_rank)
    barrier()
    if rank == 0:
        sampler.start()
    t0 = time.perf_counter()
    h.fit(init, K, flags=flags)
    barrier()
    wall = time.perf_counter() - t0
    clocks = sampler.stop() if rank == 0 else None
    st = h.stats()
    dev_ms = st["ms_loop"]
    if world > 1:
        dev_ms = kd.max_over_ranks(dev_ms, dev)
        wall = kd.max_over_ranks(wall, dev)
    steps_done = st["iterations"]
    value = world * n * steps_done / (dev_ms * 1e-3)

    line = None
    if rank == 0:
        hbm_peak, peak_kind = peaks()
        alg_bytes = n * (d * 4 + 4)
        a_ms = st["ms_assign"] / max(steps_done, 1)
        u_ms = st["ms_update"] / max(steps_done, 1)
        top = max(a_ms, u_ms) if st["path"] != 1 else a_ms
        achieved = alg_bytes / (top * 1e-3) / 1e9
        flops = 2.0 * n * k * d
        line = {"metric": "kmeans_points_iters_per_sec", "value": value, "unit": "points*iters/s", "n_gpus": world,
                "steps": steps_done, "warmup": W, "ms_per_step": dev_ms / max(steps_done, 1),
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
                "data": "synthetic", "config": config, "clocks": clocks, "gpu_launches": st["gpu_launches"],
                "wall_ms_per_step": 1e3 * wall / max(steps_done, 1),
                "kernels_ms_per_step": {"assign": a_ms, "update": u_ms, "path": st["path"]},
                "roofline": None, "tensor": None,
                "refined_rows_per_step": st.get("refined_rows", 0) / max(steps_done, 1),
                "incremental_sum_steps": st.get("incremental_iterations", 0)}
        # DRAM bytes per row of the dominant kernel from the committed ncu captures (profiles/), taken on
        # a smaller case of the same shape and scaled by the rows of a launch (traffic grows in proportion)
        ncu_bytes_per_row = {("c2", 3): 269.2, ("c3", 3): 527.0}.get((args.workload, st["path"]))
        traffic = ncu_bytes_per_row * n if ncu_bytes_per_row else None
        tens = {"fp32_equiv_tflops": flops / (a_ms * 1e-3) / 1e12, "issued_tflops": 3 * flops / (a_ms * 1e-3) / 1e12,
                "peak_tflops": tensor_peak(), "frac": 3 * flops / (a_ms * 1e-3) / 1e12 / tensor_peak()}
        hbm = {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
               "traffic": traffic, "peak_kind": "of " + peak_kind,
               "kernel": "distance+argmin" if a_ms >= u_ms else "centroid sums",
               "algorithmic_bytes_per_launch": alg_bytes,
               "whole_step_frac": alg_bytes / (dev_ms / max(steps_done, 1) * 1e-3) / 1e9 / hbm_peak}
        if st["path"] == 3 and tens["frac"] > hbm["frac"]:
            # large centroid tables: the distance kernel is bound by the tensor pipe (2kd flops per row, three
            # half-precision products per flop pair); peak = measured bf16 GEMM burst
            line["roofline"] = {"bound": "tensor", "achieved": tens["issued_tflops"], "peak": tens["peak_tflops"],
                                "unit": "TFLOP/s", "frac": tens["frac"], "traffic": traffic,
                                "peak_kind": "of " + peak_kind, "kernel": "distance+argmin",
                                "algorithmic_flops_per_launch": 3 * flops, "hbm_frac": hbm["frac"]}
        else:
            line["roofline"] = hbm
        if st["path"] == 3:
            line["tensor"] = tens
    h.close()

    # end to end through the reference's entry point: pinned host X -> fit -> host labels
    if not args.no_e2e:
        e2e = None
        if world == 1:
            Xh = torch.empty((n, d), dtype=torch.float32, pin_memory=True)
            Xh.copy_(X)
            del X
            torch.cuda.empty_cache()
            lib = lib_kmeans.get()
            cen = np.zeros(k * d, np.float32)
            lab = np.zeros(n, np.int32)
            Xn = Xh.numpy().reshape(-1)
            best = None
            for rep in range(2):
                t0 = time.perf_counter()
                lib.make_ptr_float_kmeans(0, 0, 0, local_rank, 1, n, d, k, K, 2, 0.0, Xn, init.reshape(-1), cen, lab)
                dt = time.perf_counter() - t0
                best = dt if best is None else min(best, dt)
            # the same call on a pageable copy of the matrix (what numpy hands over): the library
            # stages it through its pinned pool
            Xp = np.array(Xn)
            pageable = None
            for rep in range(2):   # best of two, as above: the first pass over a fresh array pays page faults
                t0 = time.perf_counter()
                lib.make_ptr_float_kmeans(0, 0, 0, local_rank, 1, n, d, k, K, 2, 0.0, Xp, init.reshape(-1), cen, lab)
                dt = time.perf_counter() - t0
                pageable = dt if pageable is None else min(pageable, dt)
            del Xp
            e2e = {"value": n * K / best, "unit": "points*iters/s", "pageable_seconds_per_call": pageable,
                   "h2d_bytes_per_step": (n * d * 4 + k * d * 4) / K, "d2h_bytes_per_step": (n * 4 + k * d * 4) / K,
                   "seconds_per_call": best, "call": "make_ptr_float_kmeans(host X, init_from_data=2, max_iterations=%d), "
                   "one upload and one label download per call, bytes amortised over its %d steps" % (K, K)}
        else:
            # N > 1: the reference's entry point is one process driving n_gpu devices, so rank 0
            # runs it over all N GPUs with the whole pinned host matrix while the others wait on CPU
            gloo = dist.new_group(backend="gloo")
            if rank == 0:
                lib = lib_kmeans.get()
                Xh = torch.empty((world * n, d), dtype=torch.float32, pin_memory=True)
                for r in range(world):
                    engine.synth_device(X.data_ptr(), n, d, np.float32, row0=r * n, kind=w.get("kind", 0), centers=centers,
                                        weights=weights, sigma=w["sigma"], seed=1234, gpu_id=local_rank)
                    Xh[r * n:(r + 1) * n].copy_(X)
                torch.cuda.synchronize()
                cen = np.zeros(k * d, np.float32)
                lab = np.zeros(world * n, np.int32)
                Xn = Xh.numpy().reshape(-1)
                best = None
                for rep in range(2):   # the first call also creates contexts and communicators
                    t0 = time.perf_counter()
                    lib.make_ptr_float_kmeans(0, 0, 0, 0, world, world * n, d, k, K, 2, 0.0, Xn, init.reshape(-1),
                                              cen, lab)
                    dt = time.perf_counter() - t0
                    best = dt if best is None else min(best, dt)
                e2e = {"value": world * n * K / best, "unit": "points*iters/s",
                       "h2d_bytes_per_step": (world * n * d * 4 + k * d * 4) / K,
                       "d2h_bytes_per_step": (world * n * 4 + k * d * 4) / K, "seconds_per_call": best,
                       "call": "make_ptr_float_kmeans(host X, n_gpu=%d, init_from_data=2, max_iterations=%d) from one "
                               "process, one upload and one label download per call" % (world, K)}
            dist.barrier(group=gloo)
        if rank == 0 and line is not None:
            line["e2e"] = e2e

    if rank == 0 and world == 1 and not args.no_cpu:
        c = cpu_arm(w, min(args.cpu_rows, n), min(K, 20), 1)
        line["cpu_baseline"] = {kk: v for kk, v in c.items() if not kk.startswith("_")}
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
