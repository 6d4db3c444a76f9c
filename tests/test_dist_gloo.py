"""Host-side logic of the multi-rank path on CPU: two gloo ranks."""
import os
import socket
import sys

import numpy as np
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    from h2o4gpu_b200 import dist as kd
    from oracle import lloyd
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        assert kd.env_world() == (rank, rank, world)
        ident = kd.broadcast_bytes(bytes(range(128)) if rank == 0 else bytes(128))
        assert ident == bytes(range(128))
        rng = np.random.default_rng(5)
        X = rng.standard_normal((1001, 6)).astype(np.float32)
        C = kd.broadcast_array(X[:7].copy() if rank == 0 else np.zeros((7, 6), np.float32))
        start, rows = kd.shard_rows(1001, rank, world)
        labels = lloyd.assign(X[start:start + rows], C)
        sums, counts = lloyd.sums_counts(X[start:start + rows], labels, 7)
        import torch
        t = torch.from_numpy(np.concatenate([sums.ravel(), counts.astype(np.float64)]))
        dist.all_reduce(t)
        tot = t.numpy()
        full_s, full_c = lloyd.sums_counts(X, lloyd.assign(X, C), 7)
        assert np.allclose(tot[:42].reshape(7, 6), full_s, atol=1e-9)
        assert np.array_equal(tot[42:].astype(np.int64), full_c)
        assert kd.max_over_ranks(rank + 1.5) == world + 0.5
        assert kd.sum_over_ranks(rows) == 1001
        out[rank] = 1
    finally:
        dist.destroy_process_group()


def test_two_rank_sharded_step_equals_whole():
    world = 2
    port = _free_port()
    with mp.Manager() as m:
        out = m.dict()
        mp.spawn(_worker, args=(world, port, out), nprocs=world, join=True)
        assert dict(out) == {0: 1, 1: 1}


def test_shard_rows_cover_everything():
    from h2o4gpu_b200.dist import shard_rows
    for n in (1, 5, 7, 8, 9, 41, 1001, 10_000_000):
        for w in (1, 2, 3, 4, 8):
            parts = [shard_rows(n, r, w) for r in range(w)]
            assert sum(p[1] for p in parts) == n
            pos = 0
            for s, c in parts:
                assert s == pos
                pos += c
            counts = [p[1] for p in parts]
            assert max(counts) - min(counts) <= 1          # balanced: 9 rows on 8 ranks leave nobody empty
            if n >= w:
                assert min(counts) >= 1
