#!/usr/bin/env python
"""k-means throughput: points*iterations per second of the resident Lloyd loop.

A step is one Lloyd iteration (E-step + M-step) over the resident shard(s); the closing
E-step that makes the labels match the returned centroids is inside the timed region.
Headline workload at every N: the single-GPU bandwidth-regime configuration per GPU
(n = 10,000,000 rows, d = 64, k = 100, float32, 100-component Gaussian mixture with
Dirichlet(1) weights, sigma 1, centres U(-10,10)^64, init = 100 seeded rows), i.e. weak
scaling: rows are sharded over ranks, one all-reduce of the k x d sums and k counts per
iteration, X stays resident.  Inputs are synthetic (seeded generator on the device);
2.56 GB per GPU, larger than L2, so no flush is needed between iterations.

The K-step fit is repeated until at least one second of device time has been measured
(five repeats or more); `value` comes from the median repeat.  Beside the headline the
line carries `extra`: the 2e8 x 128, k = 1000 configuration split over the N GPUs
(strong scaling), the 4e7 x 256, k = 4096 configuration at its 8-GPU shard size, and the
image-like 2e6 x 784, k = 10 configuration with its predict and transform passes.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Under torchrun (N > 1) each rank drives its LOCAL_RANK GPU.  Rank 0 prints one JSON
line.  --impl reference times the reference's CPU path (scikit-learn's Lloyd solver,
which h2o4gpu.KMeans(n_gpus=0) runs) on all host cores.
"""
import os
import sys

# torch.distributed.run exports OMP_NUM_THREADS=1 to its children; the CPU legs (the reference arm and
# the cpu_baseline beside the GPU number) must see every host core, so the limit goes before numpy,
# scikit-learn or a BLAS is loaded
for _v in ("OMP_NUM_THREADS", "OPENBLAS_NUM_THREADS", "MKL_NUM_THREADS"):
    if os.environ.get(_v) == "1":
        del os.environ[_v]

import argparse  # noqa: E402
import json  # noqa: E402
import subprocess  # noqa: E402
import threading  # noqa: E402
import time  # noqa: E402

import numpy as np  # noqa: E402

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: rows per GPU, d, k, mixture components, sigma, centre half-range, Dirichlet weights?
    "c2": dict(n=10_000_000, d=64, k=100, comp=100, sigma=1.0, half=10.0, dirichlet=True, T=50),
    "c3": dict(n=25_000_000, d=128, k=1000, comp=1000, sigma=2.0, half=20.0, dirichlet=False, T=30),
    "c1": dict(n=100_000, d=32, k=8, comp=8, sigma=1.0, half=10.0, dirichlet=False, T=20),
    # contraction-bound shape (rows per GPU of the 8-GPU split of n = 4e7); offset centres N(0, 4I)
    # are approximated by U(-3.5, 3.5) centres of the same variance
    "c5": dict(n=5_000_000, d=256, k=4096, comp=4096, sigma=1.0, half=3.5, dirichlet=False, T=10),
    # image-like rows (0 with probability 0.8, else an integer in 1..255): bandwidth-bound, few centroids
    "c4": dict(n=2_000_000, d=784, k=10, comp=0, sigma=0.0, half=0.0, dirichlet=False, T=100, kind=1),
}
C3_TOTAL_ROWS = 200_000_000


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            j = json.load(f)
        return float(j["hbm_gbs"]), float(j["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


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


def mixture_params(w, seed=0, dtype=np.float32):
    if w.get("kind", 0) == 1:
        return None, None
    rng = np.random.default_rng(seed)
    centers = rng.uniform(-w["half"], w["half"], (w["comp"], w["d"])).astype(dtype)
    weights = rng.dirichlet(np.ones(w["comp"])).astype(dtype) if w["dirichlet"] else None
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
        X[s:e] = centers[comp[s:e]] + w["sigma"] * rng.standard_normal((e - s, w["d"]), dtype=np.float32)
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
                      "%d iterations in %.2f s; host has %d logical cores, %d threads used" %
                      (__import__("sklearn").__version__, n_sample, r["n_iter"], r["seconds"], info["cpu_count"],
                       threads),
            "_seconds": r["seconds"], "_iters": r["n_iter"]}


class Ctx(object):
    """Rank layout and the torch.distributed plumbing of one bench process."""

    def __init__(self):
        import torch
        self.torch = torch
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        torch.cuda.set_device(self.local_rank)
        self.dev = torch.device("cuda", self.local_rank)
        self.dist = None
        self.kd = None
        if self.world > 1:
            import torch.distributed as dist
            from h2o4gpu_b200 import dist as kd
            dist.init_process_group("nccl", device_id=self.dev)
            self.dist, self.kd = dist, kd

    def barrier(self):
        self.torch.cuda.synchronize()
        if self.world > 1:
            self.dist.barrier()
            self.torch.cuda.synchronize()

    def max_over_ranks(self, v):
        return self.kd.max_over_ranks(v, self.dev) if self.world > 1 else v

    def gather(self, v):
        """One float per rank, in rank order, on every rank."""
        if self.world == 1:
            return [float(v)]
        t = self.torch.tensor([float(v)], dtype=self.torch.float64, device=self.dev)
        out = [self.torch.zeros_like(t) for _ in range(self.world)]
        self.dist.all_gather(out, t)
        return [float(o.item()) for o in out]


def run_case(ctx, w, K, W, flags, dtype=np.float32, weighted=False, min_seconds=1.0, min_repeats=5,
             max_repeats=100, sample_clocks=False, after_fit=None):
    """Generates the shard of this rank on the device, fits K steps `repeats` times and returns the
    timings (device time of loop + closing E-step, max over ranks per repeat)."""
    from h2o4gpu_b200 import engine
    torch = ctx.torch
    n, d, k = w["n"], w["d"], w["k"]
    tdt = torch.float64 if dtype == np.float64 else torch.float32
    centers, weights = mixture_params(w, dtype=dtype)
    X = torch.empty((n, d), dtype=tdt, device=ctx.dev)
    engine.synth_device(X.data_ptr(), n, d, dtype, row0=ctx.rank * n, kind=w.get("kind", 0), centers=centers,
                        weights=weights, sigma=w["sigma"], seed=1234, gpu_id=ctx.local_rank)
    # seeded initial rows, taken from rank 0's shard and shared
    if w.get("kind", 0) == 1:
        rows0 = np.arange(k)
    else:
        rows0 = np.sort(np.random.default_rng(7).choice(n, k, replace=False))
    init = X[torch.from_numpy(rows0).to(ctx.dev)].cpu().numpy()
    nccl_id = None
    if ctx.world > 1:
        init = ctx.kd.broadcast_array(init, 0, ctx.dev)
        nccl_id = ctx.kd.broadcast_bytes(engine.ResidentKMeans.nccl_unique_id() if ctx.rank == 0 else bytes(128), 0,
                                         ctx.dev)
    h = engine.ResidentKMeans(dtype, devices=(ctx.local_rank,), rank0=ctx.rank, world_size=ctx.world, nccl_id=nccl_id)
    h.attach_device(0, X.data_ptr(), n, d, n_total=n * ctx.world)
    if weighted:
        h.set_sample_weight(np.random.default_rng(11 + ctx.rank).gamma(2.0, 1.5, n).astype(dtype))
    # per-upload preparation (row norms, fp16-split copy of the rows for the d = 64 kernel) happens in the warm-up
    if W > 0:
        h.fit(init, W, flags=flags)
    sampler = ClockSampler(ctx.local_rank) if (sample_clocks and ctx.rank == 0) else None
    ctx.barrier()
    if sampler:
        sampler.start()
    reps = []
    total_ms = 0.0
    t_wall0 = time.perf_counter()
    while len(reps) < max_repeats and (len(reps) < min_repeats or total_ms < 1e3 * min_seconds):
        ctx.barrier()
        t0 = time.perf_counter()
        h.fit(init, K, flags=flags)
        ctx.barrier()
        wall = time.perf_counter() - t0
        st = h.stats()
        dev_ms = ctx.max_over_ranks(st["ms_loop"] + st["ms_final_assign"])
        st["_dev_ms"] = dev_ms
        st["_wall"] = ctx.max_over_ranks(wall)
        reps.append(st)
        total_ms += dev_ms
    wall_all = time.perf_counter() - t_wall0
    clocks = sampler.stop() if sampler else None
    order = np.argsort([r["_dev_ms"] for r in reps])
    med = reps[int(order[len(order) // 2])]
    steps = max(med["iterations"], 1)
    out = {"n": n, "d": d, "k": k, "steps": med["iterations"], "repeats": len(reps),
           "ms_per_step": med["_dev_ms"] / steps,
           "ms_per_step_min": reps[int(order[0])]["_dev_ms"] / steps,
           "ms_per_step_max": reps[int(order[-1])]["_dev_ms"] / steps,
           "ms_per_step_loop_only": med["ms_loop"] / steps,
           "ms_final_assign": med["ms_final_assign"],
           "assign_ms": med["ms_assign"] / steps, "update_ms": med["ms_update"] / steps,
           "wall_ms_per_step": 1e3 * med["_wall"] / steps,
           "value": ctx.world * n * steps / (med["_dev_ms"] * 1e-3),
           "ms_loop_per_rank": ctx.gather(med["ms_loop"] + med["ms_final_assign"]),
           "stats": med, "clocks": clocks, "timed_seconds": wall_all, "init": init}
    out["idle_ms_per_step"] = out["ms_per_step"] - out["assign_ms"] - out["update_ms"] - med["ms_final_assign"] / steps
    if after_fit is not None:
        out["after"] = after_fit(h, X)
    h.close()
    return out, X


def roofline_of(args_workload, r, hbm_peak, tensor_peak, peak_kind):
    """Roofline object of the dominant kernel of a finished case."""
    n, d, k = r["n"], r["d"], r["k"]
    st = r["stats"]
    alg_bytes = n * (d * 4 + 4)
    a_ms, u_ms = r["assign_ms"], r["update_ms"]
    # the dominant kernel is the one that streams X every iteration: distance + argmin (with the fused
    # small-k kernel it also forms the sums); the M-step moves only the rows whose label changed
    top = a_ms
    achieved = alg_bytes / (top * 1e-3) / 1e9
    flops = 2.0 * n * k * d
    # DRAM bytes per row of the dominant kernel from the committed ncu captures (profiles/), taken on
    # a smaller case of the same shape and scaled by the rows of a launch (traffic grows in proportion)
    ncu_bytes_per_row = {("c2", 3): 269.2, ("c3", 3): 527.7, ("c4", 3): 3163.3, ("c5", 3): 1063.4,
                         ("c4_k100", 3): 3162.5}.get((args_workload, st["path"]))
    traffic = ncu_bytes_per_row * n if ncu_bytes_per_row else None
    tens = {"fp32_equiv_tflops": flops / (a_ms * 1e-3) / 1e12, "issued_tflops": 3 * flops / (a_ms * 1e-3) / 1e12,
            "peak_tflops": tensor_peak, "frac": 3 * flops / (a_ms * 1e-3) / 1e12 / tensor_peak}
    hbm = {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
           "traffic": traffic, "peak_kind": "of " + peak_kind,
           "kernel": "distance+argmin" if st["path"] != 1 else "distance+argmin+sums (fused)",
           "algorithmic_bytes_per_launch": alg_bytes,
           "whole_step_frac": alg_bytes / (r["ms_per_step"] * 1e-3) / 1e9 / hbm_peak}
    if st["path"] == 3 and tens["frac"] > hbm["frac"]:
        # large centroid tables: the distance kernel is bound by the tensor pipe (2kd flops per row, three
        # half-precision products per flop pair); peak = measured bf16 GEMM burst
        roof = {"bound": "tensor", "achieved": tens["issued_tflops"], "peak": tens["peak_tflops"],
                "unit": "TFLOP/s", "frac": tens["frac"], "traffic": traffic, "peak_kind": "of " + peak_kind,
                "kernel": "distance+argmin", "algorithmic_flops_per_launch": 3 * flops, "hbm_frac": hbm["frac"]}
    else:
        roof = hbm
    return roof, (tens if st["path"] == 3 else None)


def brief(r, roof):
    return {"rows_per_gpu": r["n"], "d": r["d"], "k": r["k"], "steps": r["steps"], "repeats": r["repeats"],
            "ms_per_step": r["ms_per_step"], "ms_per_step_min": r["ms_per_step_min"],
            "ms_per_step_max": r["ms_per_step_max"], "value": r["value"], "unit": "points*iters/s",
            "kernels_ms_per_step": {"assign": r["assign_ms"], "update": r["update_ms"], "path": r["stats"]["path"]},
            "idle_ms_per_step": r["idle_ms_per_step"], "final_assign": "included",
            "allreduce": r["stats"].get("allreduce_path_name"), "roofline": roof}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--workload", default=os.environ.get("KM_BENCH_WORKLOAD", "c2"))
    ap.add_argument("--rows", type=int, default=0, help="rows per GPU (default: the workload's)")
    ap.add_argument("--d", type=int, default=0)
    ap.add_argument("--k", type=int, default=0)
    ap.add_argument("--cpu-rows", type=int, default=10_000_000)
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-extras", action="store_true")
    ap.add_argument("--single", action="store_true", help="one timed fit only (profiler captures)")
    ap.add_argument("--dtype", default="f32", choices=["f32", "f64"])
    ap.add_argument("--weighted", action="store_true", help="fit with gamma-distributed sample weights")
    ap.add_argument("--ingest", default="", choices=["", "u8"],
                    help="u8: upload an 8-bit host matrix in its own dtype (converted on the device), fit, exit")
    ap.add_argument("--flags", type=int, default=0)
    args = ap.parse_args()
    w = dict(WORKLOADS[args.workload])
    if args.rows:
        w["n"] = args.rows
    if args.d:
        w["d"] = args.d
    if args.k:
        w["k"] = args.k
        if w["comp"]:
            w["comp"] = args.k
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    K, W = args.steps, max(args.warmup, 0)
    dist_name = ("image-like rows (0 w.p. 0.8, else 1..255)" if w.get("kind", 0) == 1
                 else "%d-component Gaussian mixture" % w["comp"])
    config = {"workload": "%s: n=%d rows/GPU x d=%d %s, k=%d, %s, seeded init rows"
                          % (args.workload, w["n"], w["d"], args.dtype, w["k"], dist_name),
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

    from h2o4gpu_b200 import engine
    from h2o4gpu_b200.libs import lib_kmeans
    lib_kmeans.get()  # no CUDA library / device -> raise, never a CPU path
    ctx = Ctx()
    torch = ctx.torch
    local_rank = ctx.local_rank
    npdt = np.float64 if args.dtype == "f64" else np.float32

    if args.ingest == "u8":
        # 8-bit pixel matrix uploaded in its own dtype and converted on the device, then fitted
        rng = np.random.default_rng(0)
        n, d, k = w["n"], w["d"], w["k"]
        P = (rng.integers(1, 256, (n, d), dtype=np.uint8) * (rng.random((n, d), dtype=np.float32) < 0.2)).astype(np.uint8)
        h = engine.ResidentKMeans()
        h.upload(P)
        h.fit(P[:k].astype(np.float32), K)
        print(json.dumps({"ingest": "u8", "stats": h.stats()}))
        h.close()
        return

    flags = engine.FIT_PRESPLIT | args.flags
    kw = dict(min_seconds=0.0, min_repeats=1, max_repeats=1) if args.single else {}
    r, X = run_case(ctx, w, K, W, flags, dtype=npdt, weighted=args.weighted, sample_clocks=True, **kw)
    n, d, k = w["n"], w["d"], w["k"]
    init = r["init"]
    st = r["stats"]
    steps_done = r["steps"]

    line = None
    hbm_peak, tensor_peak, peak_kind = peaks()
    if rank == 0:
        roof, tens = roofline_of(args.workload, r, hbm_peak, tensor_peak, peak_kind)
        line = {"metric": "kmeans_points_iters_per_sec", "value": r["value"], "unit": "points*iters/s", "n_gpus": world,
                "steps": steps_done, "warmup": W, "ms_per_step": r["ms_per_step"],
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": args.dtype,
                "data": "synthetic", "config": config, "clocks": r["clocks"],
                "gpu_launches": st["gpu_launches"] * r["repeats"],
                "gpu_launches_per_fit": st["gpu_launches"],
                "repeats": r["repeats"], "ms_per_step_min": r["ms_per_step_min"],
                "ms_per_step_max": r["ms_per_step_max"], "ms_per_step_loop_only": r["ms_per_step_loop_only"],
                "final_assign": "included: the closing E-step (%.3f ms) is inside the timed region of every "
                                "%d-step fit" % (r["ms_final_assign"], steps_done),
                "ms_loop_per_rank": r["ms_loop_per_rank"], "idle_ms_per_step": r["idle_ms_per_step"],
                "allreduce": st.get("allreduce_path_name"),
                "wall_ms_per_step": r["wall_ms_per_step"],
                "kernels_ms_per_step": {"assign": r["assign_ms"], "update": r["update_ms"], "path": st["path"]},
                "roofline": roof, "tensor": tens,
                "refined_rows_per_step": st.get("refined_rows", 0) / max(steps_done, 1),
                "incremental_sum_steps": st.get("incremental_iterations", 0)}

    # end to end through the reference's entry point: pinned host X -> fit -> host labels
    if not args.no_e2e and args.dtype == "f32" and not args.weighted:
        e2e = None
        if world == 1:
            Xh = torch.empty((n, d), dtype=torch.float32, pin_memory=True)
            Xh.copy_(X)
            del X
            X = None
            torch.cuda.empty_cache()
            lib = lib_kmeans.get()
            cen = np.zeros(k * d, np.float32)
            lab = np.zeros(n, np.int32)
            Xn = Xh.numpy().reshape(-1)
            times = []
            for rep in range(5):
                t0 = time.perf_counter()
                lib.make_ptr_float_kmeans(0, 0, 0, local_rank, 1, n, d, k, K, 2, 0.0, Xn, init.reshape(-1), cen, lab)
                times.append(time.perf_counter() - t0)
            best = float(np.median(times[1:]))
            # the same call on a pageable copy of the matrix (what numpy hands over): the library
            # stages it through its pinned pool
            Xp = np.array(Xn)
            ptimes = []
            for rep in range(3):   # the first pass over a fresh array pays page faults
                t0 = time.perf_counter()
                lib.make_ptr_float_kmeans(0, 0, 0, local_rank, 1, n, d, k, K, 2, 0.0, Xp, init.reshape(-1), cen, lab)
                ptimes.append(time.perf_counter() - t0)
            del Xp
            e2e = {"value": n * K / best, "unit": "points*iters/s",
                   "pageable_seconds_per_call": float(np.median(ptimes[1:])),
                   "h2d_bytes_per_step": (n * d * 4 + k * d * 4) / K, "d2h_bytes_per_step": (n * 4 + k * d * 4) / K,
                   "seconds_per_call": best, "seconds_per_call_all": times,
                   "call": "make_ptr_float_kmeans(host X, init_from_data=2, max_iterations=%d), "
                   "one upload and one label download per call, bytes amortised over its %d steps; median of the "
                   "calls after the first" % (K, K)}
            del Xh
        else:
            # N > 1: the reference's entry point is one process driving n_gpu devices, so rank 0
            # runs it over all N GPUs with the whole pinned host matrix while the others wait on CPU
            gloo = ctx.dist.new_group(backend="gloo")
            if rank == 0:
                lib = lib_kmeans.get()
                centers, weights = mixture_params(w)
                Xh = torch.empty((world * n, d), dtype=torch.float32, pin_memory=True)
                for rr in range(world):
                    engine.synth_device(X.data_ptr(), n, d, np.float32, row0=rr * n, kind=w.get("kind", 0),
                                        centers=centers, weights=weights, sigma=w["sigma"], seed=1234,
                                        gpu_id=local_rank)
                    Xh[rr * n:(rr + 1) * n].copy_(X)
                torch.cuda.synchronize()
                cen = np.zeros(k * d, np.float32)
                lab = np.zeros(world * n, np.int32)
                Xn = Xh.numpy().reshape(-1)
                times = []
                for rep in range(4):   # the first call also creates contexts and communicators
                    t0 = time.perf_counter()
                    lib.make_ptr_float_kmeans(0, 0, 0, 0, world, world * n, d, k, K, 2, 0.0, Xn, init.reshape(-1),
                                              cen, lab)
                    times.append(time.perf_counter() - t0)
                best = float(np.median(times[1:]))
                e2e = {"value": world * n * K / best, "unit": "points*iters/s",
                       "h2d_bytes_per_step": (world * n * d * 4 + k * d * 4) / K,
                       "d2h_bytes_per_step": (world * n * 4 + k * d * 4) / K, "seconds_per_call": best,
                       "seconds_per_call_all": times,
                       "call": "make_ptr_float_kmeans(host X, n_gpu=%d, init_from_data=2, max_iterations=%d) from one "
                               "process, one upload and one label download per call; median of the calls after the "
                               "first" % (world, K)}
                del Xh
            ctx.dist.barrier(group=gloo)
        if rank == 0 and line is not None:
            line["e2e"] = e2e
    del X
    torch.cuda.empty_cache()
    lib_kmeans.cdll().kmeans_trim_memory()

    # ---- the other configurations, beside the headline --------------------------------------------------
    if not args.no_extras and args.workload == "c2" and not args.single:
        extra = {}
        # C3 split over the N GPUs (strong scaling: 2e8 / N rows each), generated on the device
        w3 = dict(WORKLOADS["c3"])
        w3["n"] = C3_TOTAL_ROWS // world
        r3, X3 = run_case(ctx, w3, 5, 2, engine.FIT_PRESPLIT, min_seconds=1.0, min_repeats=2, max_repeats=3)
        del X3
        torch.cuda.empty_cache()
        lib_kmeans.cdll().kmeans_trim_memory()
        if rank == 0:
            roof3, _ = roofline_of("c3", r3, hbm_peak, tensor_peak, peak_kind)
            extra["c3_strong"] = brief(r3, roof3)
            extra["c3_strong"]["total_rows"] = w3["n"] * world
            extra["c3_strong"]["scaling"] = "strong: 2e8 rows / N GPUs"
        # C5 at its 8-GPU shard size (weak: 5e6 rows per GPU)
        r5, X5 = run_case(ctx, WORKLOADS["c5"], 5, 2, engine.FIT_PRESPLIT, min_seconds=0.5, min_repeats=2, max_repeats=3)
        del X5
        torch.cuda.empty_cache()
        lib_kmeans.cdll().kmeans_trim_memory()
        if rank == 0:
            roof5, _ = roofline_of("c5", r5, hbm_peak, tensor_peak, peak_kind)
            extra["c5"] = brief(r5, roof5)
            extra["c5"]["scaling"] = "weak: 4e7 / 8 rows per GPU"

        # C4 split over the N GPUs, with predict and transform on the fitted centroids
        def c4_after(h, X4):
            n4, d4, k4 = X4.shape[0], X4.shape[1], h.k
            out = {}
            ts = []
            for _ in range(5):
                h.assign()
                ts.append(h.stats()["ms_assign"])
            ms = float(np.median(ts[1:]))
            out["predict"] = {"ms": ms, "rows_per_s": n4 / (ms * 1e-3), "bytes": n4 * (d4 * 4 + 4),
                              "hbm_frac": n4 * (d4 * 4 + 4) / (ms * 1e-3) / 1e9 / hbm_peak}
            ts, wl = [], []
            for _ in range(4):
                t0 = time.perf_counter()
                h.transform()
                wl.append(time.perf_counter() - t0)
                ts.append(h.stats()["ms_transform"])
            ms = float(np.median(ts[1:]))
            out["transform"] = {"ms_kernels": ms, "rows_per_s": n4 / (ms * 1e-3),
                                "bytes": n4 * (d4 * 4 + k4 * 4),
                                "hbm_frac": n4 * (d4 * 4 + k4 * 4) / (ms * 1e-3) / 1e9 / hbm_peak,
                                "seconds_with_copy_to_host": float(np.median(wl[1:])),
                                "note": "n x k squared distances, column-major; kernels timed with CUDA events, "
                                        "the host copy of the block (%d bytes) separately" % (n4 * k4 * 4)}
            return out
        w4 = dict(WORKLOADS["c4"])
        w4["n"] = w4["n"] // world
        r4, X4 = run_case(ctx, w4, 10, 2, 0, min_seconds=0.3, min_repeats=2, max_repeats=5, after_fit=c4_after)
        del X4
        torch.cuda.empty_cache()
        if rank == 0:
            roof4, _ = roofline_of("c4", r4, hbm_peak, tensor_peak, peak_kind)
            extra["c4"] = brief(r4, roof4)
            extra["c4"]["scaling"] = "strong: 2e6 rows / N GPUs"
            extra["c4_predict"] = r4["after"]["predict"]
            extra["c4_transform"] = r4["after"]["transform"]
        # wide rows with many centroids (d = 784, k = 100: the kernel that streams both operands), 5e5 rows per
        # GPU, and transform of the C2 shape (2e6 rows per GPU) through the same kernel's store epilogue
        w6 = dict(WORKLOADS["c4"])
        w6["k"], w6["n"] = 100, 500_000
        r6, X6 = run_case(ctx, w6, 10, 2, 0, min_seconds=0.3, min_repeats=2, max_repeats=5, after_fit=c4_after)
        del X6
        torch.cuda.empty_cache()
        w7 = dict(WORKLOADS["c2"])
        w7["n"] = 2_000_000
        r7, X7 = run_case(ctx, w7, 5, 2, 0, min_seconds=0.2, min_repeats=2, max_repeats=3, after_fit=c4_after)
        del X7
        torch.cuda.empty_cache()
        if rank == 0:
            roof6, _ = roofline_of("c4_k100", r6, hbm_peak, tensor_peak, peak_kind)
            extra["c4_k100"] = brief(r6, roof6)
            extra["c4_k100"]["scaling"] = "weak: 5e5 rows per GPU"
            extra["c4_k100_transform"] = r6["after"]["transform"]
            extra["c2_transform"] = r7["after"]["transform"]
            extra["c2_transform"]["rows_per_gpu"] = w7["n"]
            line["extra"] = extra

    if rank == 0 and world == 1 and not args.no_cpu:
        c = cpu_arm(w, min(args.cpu_rows, n), min(K, 20), 1)
        line["cpu_baseline"] = {kk: v for kk, v in c.items() if not kk.startswith("_")}
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        ctx.dist.barrier()
        ctx.dist.destroy_process_group()


if __name__ == "__main__":
    main()
