"""Small resident fit of a bench-shaped workload for profiler captures (Gaussian mixture with
as many components as clusters, seeded init rows; defaults: the C2 shape d=64, k=100):
    python h2o4gpu_b200/ncu_case.py [rows] [iterations] [d] [k] [mode]
mode "weighted": the same fit with gamma-distributed sample weights; mode "u8": an 8-bit pixel matrix
(80 % zeros) uploaded from the host in its own dtype and converted on the device, then fitted; mode "f64":
the mixture in float64 (the E-step then runs on the double-precision matrix unit)."""
import sys
import numpy as np
sys.path.insert(0, __import__('os').path.dirname(__import__('os').path.dirname(__import__('os').path.abspath(__file__))))
import torch
from h2o4gpu_b200 import engine
n = int(sys.argv[1]) if len(sys.argv) > 1 else 2_000_000
iters = int(sys.argv[2]) if len(sys.argv) > 2 else 3
d = int(sys.argv[3]) if len(sys.argv) > 3 else 64
k = int(sys.argv[4]) if len(sys.argv) > 4 else 100
mode = sys.argv[5] if len(sys.argv) > 5 else ""
dev = torch.device("cuda", 0)
rng = np.random.default_rng(0)
if mode == "u8":
    P = (rng.integers(1, 256, (n, d), dtype=np.uint8) * (rng.random((n, d), dtype=np.float32) < 0.2)).astype(np.uint8)
    h = engine.ResidentKMeans()
    h.upload(P)
    h.fit(P[:k].astype(np.float32), iters, flags=engine.FIT_NO_FINAL_ASSIGN)
    print(h.stats())
    h.close()
    sys.exit(0)
npdt, tdt = (np.float64, torch.float64) if mode == "f64" else (np.float32, torch.float32)
centers = rng.uniform(-10, 10, (k, d)).astype(npdt)
w = rng.dirichlet(np.ones(k)).astype(npdt)
X = torch.empty((n, d), dtype=tdt, device=dev)
engine.synth_device(X.data_ptr(), n, d, npdt, centers=centers, weights=w, sigma=1.0, seed=1)
init = X[torch.from_numpy(np.sort(rng.choice(n, k, replace=False))).to(dev)].cpu().numpy()
h = engine.ResidentKMeans(dtype=npdt)
h.attach_device(0, X.data_ptr(), n, d)
if mode == "weighted":
    h.set_sample_weight(rng.gamma(2.0, 1.5, n).astype(np.float32))
h.fit(init, iters, flags=engine.FIT_NO_FINAL_ASSIGN | engine.FIT_PRESPLIT)
print(h.stats())
h.close()
