"""Host-side helpers for the one-process-per-GPU layout (torch.distributed is the
plumbing: rendezvous, barriers, max-over-ranks; the per-iteration all-reduce of
the centroid sums runs inside the native library on its own NCCL communicator)."""
import os

import numpy as np


def env_world():
    """(rank, local_rank, world_size) from the launcher's environment."""
    return (int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")),
            int(os.environ.get("WORLD_SIZE", "1")))


def shard_rows(n_total, rank, world):
    """Balanced contiguous split that covers every row: (first row, row count) of `rank`; the first
    n_total % world ranks hold one row more, so no rank is empty while n_total >= world (the split the
    library itself applies to a host matrix).  The reference uses floor(n / g) rows per GPU and drops
    the remainder (src/gpu/kmeans/kmeans_h2o4gpu.cu:649, 679)."""
    per, extra = divmod(n_total, world)
    start = rank * per + min(rank, extra)
    return start, per + (1 if rank < extra else 0)


def broadcast_bytes(payload, src=0, device=None):
    """Broadcast a bytes object of known length from `src` to every rank."""
    import torch
    import torch.distributed as dist
    n = len(payload)
    t = torch.tensor(list(payload), dtype=torch.uint8)
    if device is not None:
        t = t.to(device)
    dist.broadcast(t, src=src)
    out = bytes(t.cpu().tolist())
    assert len(out) == n
    return out


def broadcast_array(a, src=0, device=None):
    """Broadcast a numpy array (same shape and dtype on every rank)."""
    import torch
    import torch.distributed as dist
    t = torch.from_numpy(np.ascontiguousarray(a).copy())
    if device is not None:
        t = t.to(device)
    dist.broadcast(t, src=src)
    return t.cpu().numpy()


def max_over_ranks(value, device=None):
    import torch
    import torch.distributed as dist
    t = torch.tensor([float(value)], dtype=torch.float64)
    if device is not None:
        t = t.to(device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sum_over_ranks(value, device=None):
    import torch
    import torch.distributed as dist
    t = torch.tensor([float(value)], dtype=torch.float64)
    if device is not None:
        t = t.to(device)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())
