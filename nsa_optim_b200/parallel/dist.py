"""Process-group bootstrap and thin collective helpers.

Reference behaviour (nngabe/nsa_optim): ``setup_distributed`` train.py:65-80 reads
``RANK`` / ``WORLD_SIZE`` / ``LOCAL_RANK``, creates an NCCL group when the world is larger
than one and binds the process to a GPU; ``cleanup_distributed`` train.py:83-86.

Additions: the backend is selectable (``nccl`` on GPUs, ``gloo`` for CPU ranks), the device
index is ``LOCAL_RANK`` (so multi-node launches bind correctly), collectives that gloo lacks
are emulated (reduce-scatter as all-reduce + slice), and every rank can learn of a peer's
failure through a short process-group timeout rather than by hanging.
"""
from __future__ import annotations

import datetime
import os
from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist


@dataclass
class DistInfo:
    rank: int = 0
    world_size: int = 1
    local_rank: int = 0
    backend: Optional[str] = None
    device: torch.device = torch.device("cpu")

    @property
    def is_main(self) -> bool:
        return self.rank == 0


def setup_distributed(backend: Optional[str] = None, timeout_s: float = 1800.0,
                      device: Optional[str] = None) -> DistInfo:
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", rank))
    use_cuda = torch.cuda.is_available() and device != "cpu"
    if backend is None:
        backend = "nccl" if use_cuda else "gloo"
    if use_cuda and backend == "nccl":
        torch.cuda.set_device(local % torch.cuda.device_count())
        dev = torch.device("cuda", local % torch.cuda.device_count())
    elif use_cuda:
        dev = torch.device("cuda", local % torch.cuda.device_count())
        torch.cuda.set_device(dev)
    else:
        dev = torch.device("cpu")
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        kwargs = dict(backend=backend, rank=rank, world_size=world,
                      timeout=datetime.timedelta(seconds=timeout_s))
        if backend == "nccl":
            kwargs["device_id"] = dev
        dist.init_process_group(**kwargs)
    return DistInfo(rank, world, local, backend if world > 1 else None, dev)


def cleanup_distributed() -> None:
    if dist.is_available() and dist.is_initialized():
        dist.destroy_process_group()


def is_dist() -> bool:
    return dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1


def barrier() -> None:
    if is_dist():
        dist.barrier()


def all_gather_flat(out: torch.Tensor, shard: torch.Tensor, group=None, async_op: bool = False):
    """out (W*S) <- concatenation of every rank's ``shard`` (S)."""
    return dist.all_gather_into_tensor(out, shard, group=group, async_op=async_op)


def reduce_scatter_flat(out: torch.Tensor, inp: torch.Tensor, group=None) -> None:
    """out (S) <- this rank's slice of the elementwise sum of every rank's ``inp`` (W*S)."""
    backend = dist.get_backend(group)
    if backend == "nccl":
        dist.reduce_scatter_tensor(out, inp, op=dist.ReduceOp.SUM, group=group)
        return
    try:
        dist.reduce_scatter_tensor(out, inp, op=dist.ReduceOp.SUM, group=group)
    except (RuntimeError, NotImplementedError):
        tmp = inp.clone()
        dist.all_reduce(tmp, op=dist.ReduceOp.SUM, group=group)
        r, s = dist.get_rank(group), out.numel()
        out.copy_(tmp[r * s:(r + 1) * s])


def all_reduce_sum(t: torch.Tensor, group=None) -> torch.Tensor:
    if is_dist():
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
    return t


def all_reduce_min(t: torch.Tensor, group=None) -> torch.Tensor:
    if is_dist():
        dist.all_reduce(t, op=dist.ReduceOp.MIN, group=group)
    return t


def all_reduce_max(t: torch.Tensor, group=None) -> torch.Tensor:
    if is_dist():
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return t
