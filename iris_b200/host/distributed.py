"""Control plane: thin helpers over an existing ``torch.distributed`` process group.

The data plane never goes through these; they move a few bytes at set-up time (heap bases, socket
paths, IPC handles) and implement the host barrier. The process group must already exist, as in
the reference (iris/host/distributed/helpers.py:420-433); both ``nccl`` (GPU ranks) and ``gloo``
(CPU ranks) work.
"""
from __future__ import annotations

import numpy as np
import torch
import torch.distributed as dist


def init_distributed():
    """Return ``(comm, rank, world_size)`` of the default group; raise if none was initialised."""
    if not dist.is_available() or not dist.is_initialized():
        raise RuntimeError(
            "torch.distributed is not initialised: call dist.init_process_group(backend='nccl' or 'gloo') "
            "before creating an Iris context"
        )
    return None, dist.get_rank(), dist.get_world_size()


def _backend_device(group=None) -> torch.device:
    backend = dist.get_backend(group)
    if "nccl" in str(backend) and torch.cuda.is_available():
        return torch.device("cuda", torch.cuda.current_device())
    return torch.device("cpu")


def distributed_allgather(data: np.ndarray, group=None) -> np.ndarray:
    """All-gather a small numpy array; returns an array of shape ``(world, *data.shape)``."""
    data = np.ascontiguousarray(data)
    world = dist.get_world_size(group)
    dev = _backend_device(group)
    if data.dtype == np.uint64:  # neither gloo nor nccl reduce/gather uint64 reliably
        t = torch.from_numpy(data.view(np.int64).copy()).to(dev)
        out = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(out, t, group=group)
        return np.stack([o.cpu().numpy().view(np.uint64) for o in out])
    try:
        t = torch.from_numpy(data.copy()).to(dev)
    except TypeError:
        objs = [None] * world
        dist.all_gather_object(objs, data, group=group)
        return np.stack(objs)
    out = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(out, t, group=group)
    return np.stack([o.cpu().numpy() for o in out])


def distributed_allgather_multidim(data: np.ndarray, group=None) -> np.ndarray:
    return distributed_allgather(np.asarray(data), group)


def distributed_allgather_object(obj, group=None) -> list:
    world = dist.get_world_size(group)
    objs = [None] * world
    dist.all_gather_object(objs, obj, group=group)
    return objs


def distributed_broadcast_scalar(value, src: int = 0, group=None):
    """Broadcast a Python / numpy scalar (or any picklable object) from ``src``."""
    box = [value if dist.get_rank() == src else None]
    dist.broadcast_object_list(box, src=src, group=group)
    return box[0]


def distributed_broadcast_tensor(value, src: int = 0, group=None):
    """Broadcast a tensor or numpy array from ``src``; every rank gets one of the same type."""
    rank = dist.get_rank()
    is_np = isinstance(value, np.ndarray)
    meta = [None]
    if rank == src:
        t = torch.from_numpy(value) if is_np else value
        meta[0] = (tuple(t.shape), str(t.dtype).replace("torch.", ""), is_np)
    dist.broadcast_object_list(meta, src=src, group=group)
    shape, dtype_name, src_np = meta[0]
    dtype = getattr(torch, dtype_name)
    dev = _backend_device(group)
    if rank == src:
        buf = (torch.from_numpy(value) if is_np else value).detach().to(dev).contiguous()
    else:
        buf = torch.empty(shape, dtype=dtype, device=dev)
    dist.broadcast(buf, src=src, group=group)
    if src_np:
        return buf.cpu().numpy()
    if rank == src:
        return value
    return buf if isinstance(value, torch.Tensor) and value.device == buf.device else buf


def distributed_barrier(group=None) -> None:
    dist.barrier(group=group)


def extract_group_info(group, rank_global: int, world_global: int):
    """Describe ``group`` as ``(rank_in_group, rank_global, world_size, rank_start, rank_stride)``.

    Kernels address peers as ``rank_start + i * rank_stride``; groups whose global ranks are not
    an arithmetic progression are rejected (reference: iris/host/distributed/helpers.py:234-301).
    """
    if group is None:
        return rank_global, rank_global, world_global, 0, 1
    ranks = dist.get_process_group_ranks(group)
    if rank_global not in ranks:
        raise RuntimeError(f"rank {rank_global} is not a member of the process group {ranks}")
    n = len(ranks)
    if n == 1:
        return 0, rank_global, 1, ranks[0], 1
    stride = ranks[1] - ranks[0]
    if stride <= 0 or any(ranks[i + 1] - ranks[i] != stride for i in range(n - 1)):
        raise RuntimeError(f"process group ranks {ranks} must be evenly strided")
    return ranks.index(rank_global), rank_global, n, ranks[0], stride
