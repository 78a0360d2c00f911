"""Symmetric memory over CUDA IPC and the peer-memory collectives built on it.

Each rank allocates one arena (a plain CUDA tensor), exports it with PyTorch's CUDA IPC
machinery, and maps every peer's arena; all ranks carve the arena with the same offsets, so
"offset X in rank p's arena" is addressable from every rank.  Kernels get device arrays of W
base pointers.  The process group is used only to exchange the IPC handles (bootstrap).

Flag words (uint32 epochs) live at the start of the arena: ``channels`` rows of 32 slots; a rank
signals a channel by writing the epoch into slot [its rank] of that row in every peer's arena.
All waits inside the kernels are bounded (``max_wait_cycles``); a timeout is reported through
the native status block and surfaces as an exception from ``native.check_status()``.

The reference project has no counterpart: its only collectives are the ones FSDP issues
through NCCL (train.py:171-208).
"""
from __future__ import annotations

from ctypes import c_int, c_long, c_longlong, c_uint, c_void_p, c_float
from typing import List, Optional

import torch
import torch.distributed as dist

from ..ops import native, quant

FLAG_SLOTS = 32
DEFAULT_MAX_WAIT_CYCLES = 20_000_000_000      # about ten seconds at 2 GHz


def _round_up(x: int, m: int) -> int:
    return -(-x // m) * m


class SymmetricArena:
    """One IPC-shared allocation per rank, mapped by all ranks of the node."""

    def __init__(self, nbytes: int, channels: int, rank: int, world: int, device: torch.device, group=None,
                 local_peers: Optional[List[torch.Tensor]] = None):
        self.rank, self.world, self.device = rank, world, device
        self.flag_bytes = _round_up(channels * FLAG_SLOTS * 4, 4096)
        self.nbytes = self.flag_bytes + _round_up(nbytes, 4096)
        self.cursor = self.flag_bytes
        self.channels = channels
        self._raw_local = None
        self._raw_peers: List[int] = []
        if local_peers is not None:
            # single-process emulation: the "peers" are other tensors on this GPU
            self.peers = local_peers
            self.local = local_peers[rank]
        else:
            self._exchange(group)
        self._ptr_cache = {}

    @staticmethod
    def _wrap(ptr: int, nbytes: int, device: torch.device) -> torch.Tensor:
        """A uint8 tensor aliasing raw device memory (no ownership)."""
        class _Raw:
            pass
        raw = _Raw()
        raw.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}
        return torch.as_tensor(raw, device=device)

    def _exchange(self, group) -> None:
        """cudaMalloc the arena, export its IPC handle, and open every peer's handle with this
        rank's device current, so the mappings belong to the context whose kernels use them."""
        import ctypes
        lib = native.load()
        ptr = c_void_p()
        handle = (ctypes.c_ubyte * 64)()
        native._check(lib.nsa_ipc_alloc(c_long(self.nbytes), ctypes.byref(ptr), handle))
        self._raw_local = ptr.value
        self.local = self._wrap(ptr.value, self.nbytes, self.device)
        gathered: List = [None] * self.world
        dist.all_gather_object(gathered, bytes(handle), group=group)
        self.peers = []
        for r in range(self.world):
            if r == self.rank:
                self.peers.append(self.local)
                continue
            h = (ctypes.c_ubyte * 64).from_buffer_copy(gathered[r])
            pp = c_void_p()
            native._check(lib.nsa_ipc_open(h, ctypes.byref(pp)))
            self._raw_peers.append(pp.value)
            self.peers.append(self._wrap(pp.value, self.nbytes, self.device))
        dist.barrier(group=group)

    def close(self) -> None:
        """Unmap the peers and free the arena (call after a barrier, with no kernel in flight)."""
        lib = native.load()
        for p in self._raw_peers:
            lib.nsa_ipc_close(c_void_p(p))
        self._raw_peers = []
        if self._raw_local is not None:
            lib.nsa_ipc_free(c_void_p(self._raw_local))
            self._raw_local = None

    def alloc(self, nbytes: int, align: int = 1024) -> int:
        """Reserve ``nbytes`` at the same offset on every rank; returns the offset."""
        off = _round_up(self.cursor, align)
        if off + nbytes > self.nbytes:
            raise MemoryError(f"symmetric arena exhausted ({off + nbytes} > {self.nbytes})")
        self.cursor = off + nbytes
        return off

    def view(self, offset: int, numel: int, dtype: torch.dtype, peer: Optional[int] = None) -> torch.Tensor:
        t = self.local if peer is None else self.peers[peer]
        nb = numel * torch.empty((), dtype=dtype).element_size()
        return t[offset:offset + nb].view(dtype)

    def ptr_array(self, offset: int) -> torch.Tensor:
        """Device int64 tensor of W pointers: ``peer_base[p] + offset``."""
        key = offset
        arr = self._ptr_cache.get(key)
        if arr is None:
            arr = torch.tensor([self.peers[p].data_ptr() + offset for p in range(self.world)], dtype=torch.int64,
                               device=self.device)
            self._ptr_cache[key] = arr
        return arr

    def flag_row(self, channel: int) -> torch.Tensor:
        return self.view(channel * FLAG_SLOTS * 4, FLAG_SLOTS, torch.int32)

    def flag_row_ptrs(self, channel: int) -> torch.Tensor:
        return self.ptr_array(channel * FLAG_SLOTS * 4)


def _s():
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def signal(arena: SymmetricArena, channel: int, epoch: int) -> None:
    """After all work queued so far on the current stream, publish ``epoch`` on ``channel``."""
    rows = arena.flag_row_ptrs(channel)
    native._check(native.load().nsa_comm_signal(c_void_p(rows.data_ptr()), c_int(arena.world), c_int(arena.rank),
                                               c_uint(epoch), _s()))


def wait(arena: SymmetricArena, channel: int, epoch: int, max_cycles: int = DEFAULT_MAX_WAIT_CYCLES,
         n: Optional[int] = None) -> None:
    row = arena.flag_row(channel)
    native._check(native.load().nsa_comm_wait(c_void_p(row.data_ptr()), c_int(arena.world if n is None else n),
                                             c_uint(epoch), c_longlong(max_cycles), _s()))


def all_gather(arena: SymmetricArena, shard_offset: int, shard_bytes: int, out: torch.Tensor, channel: Optional[int],
               epoch: int, max_cycles: int = DEFAULT_MAX_WAIT_CYCLES, ctas_per_peer: int = 16) -> None:
    """out <- concatenation of every rank's shard; waits (bounded) for ``channel`` to reach ``epoch``."""
    ptrs = arena.ptr_array(shard_offset)
    flags = c_void_p(0) if channel is None else c_void_p(arena.flag_row(channel).data_ptr())
    native._check(native.load().nsa_comm_allgather(c_void_p(ptrs.data_ptr()), c_void_p(out.data_ptr()), c_long(shard_bytes),
                                                  c_int(arena.world), c_int(arena.rank), flags, c_uint(epoch),
                                                  c_longlong(max_cycles), c_int(ctas_per_peer), _s()))


def reduce_scatter(arena: SymmetricArena, grad_offset: int, grad_shard: torch.Tensor, scale: float, accumulate: bool,
                   channel: Optional[int], epoch: int, sumsq_partial: Optional[torch.Tensor] = None,
                   max_cycles: int = DEFAULT_MAX_WAIT_CYCLES) -> None:
    """grad_shard (+)= scale * sum over ranks of their fp32 gradient buffer slice [rank]."""
    ptrs = arena.ptr_array(grad_offset)
    flags = c_void_p(0) if channel is None else c_void_p(arena.flag_row(channel).data_ptr())
    native._check(native.load().nsa_comm_reduce_scatter(
        c_void_p(ptrs.data_ptr()), c_void_p(grad_shard.data_ptr()), c_long(grad_shard.numel()), c_int(arena.world),
        c_int(arena.rank), c_float(scale), c_int(int(accumulate)),
        c_void_p(0 if sumsq_partial is None else sumsq_partial.data_ptr()), flags, c_uint(epoch), c_longlong(max_cycles), _s()))


def reduce_scatter_parts() -> int:
    return int(native.load().nsa_comm_reduce_scatter_parts())


def rs_adamw8bit(arena: SymmetricArena, grad_offset: int, p_shard: torch.Tensor, mq, mabs, vq, vabs, wd_mask,
                 scale: float, step: int, lr: float, betas, eps: float, wd: float, channel: Optional[int], epoch: int,
                 max_cycles: int = DEFAULT_MAX_WAIT_CYCLES) -> None:
    """Reduce-scatter of the W gradient buffers fused with the blockwise 8-bit AdamW update of
    the owned shard."""
    ptrs = arena.ptr_array(grad_offset)
    flags = c_void_p(0) if channel is None else c_void_p(arena.flag_row(channel).data_ptr())
    cs, cu = quant.codebook(8, True, p_shard.device), quant.codebook(8, False, p_shard.device)
    native._check(native.load().nsa_comm_rs_adamw8bit(
        c_void_p(ptrs.data_ptr()), c_void_p(p_shard.data_ptr()), c_int(int(p_shard.dtype == torch.float32)),
        c_void_p(mq.data_ptr()), c_void_p(mabs.data_ptr()), c_void_p(vq.data_ptr()), c_void_p(vabs.data_ptr()),
        c_void_p(cs.data_ptr()), c_void_p(cu.data_ptr()), c_void_p(0 if wd_mask is None else wd_mask.data_ptr()),
        c_long(p_shard.numel()), c_int(arena.world), c_int(arena.rank), c_float(scale), c_int(step), c_float(lr),
        c_float(betas[0]), c_float(betas[1]), c_float(eps), c_float(wd), flags, c_uint(epoch), c_longlong(max_cycles), _s()))


def gemm_all_gather(arena: SymmetricArena, x: torch.Tensor, full: torch.Tensor, shard_offset: int, shard_elems: int,
                    b_elem_offset: int, N: int, chunk_flags: torch.Tensor, chunks_per_shard: int,
                    channel: Optional[int], epoch: int, max_cycles: int = DEFAULT_MAX_WAIT_CYCLES,
                    copy_ctas: int = 16) -> torch.Tensor:
    """y = x @ W^T with W (N, K) at ``b_elem_offset`` of the unit's gathered buffer ``full``, which
    the same kernel assembles from the ranks' shards.  Afterwards ``full`` holds the whole unit."""
    x2 = native._as_2d(x)
    M, K = x2.shape
    y = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
    ptrs = arena.ptr_array(shard_offset)
    flags = c_void_p(0) if channel is None else c_void_p(arena.flag_row(channel).data_ptr())
    native._check(native.load().nsa_gemm_bf16_ag(
        c_void_p(x2.data_ptr()), c_void_p(y.data_ptr()), c_int(M), c_int(N), c_int(K), c_int(x2.stride(0)), c_int(N),
        c_void_p(ptrs.data_ptr()), c_void_p(full.data_ptr()), c_long(shard_elems), c_long(b_elem_offset),
        c_int(arena.world), c_int(arena.rank), c_void_p(chunk_flags.data_ptr()), c_int(chunks_per_shard), flags,
        c_uint(epoch), c_longlong(max_cycles), c_int(copy_ctas), _s()))
    return y.view(*x.shape[:-1], N)
