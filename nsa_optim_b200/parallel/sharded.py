"""Sharded-parameter data-parallel runtime (the framework's replacement for PyTorch FSDP).

What the reference does with FSDP1 (nngabe/nsa_optim train.py:171-208): one flat parameter
per block class instance plus a root unit for embedding / final norm / head, bf16
all-gather before use, fp32 reduce-scatter of gradients, ``FULL_SHARD`` for Adam-family
optimizers and ``SHARD_GRAD_OP`` for SOAP / Shampoo.

Design here
-----------
* **Unit** = one block (or the root).  Its parameters live in one flat buffer in the compute
  dtype; every parameter starts on a 256-element boundary (so 8-bit optimizer blocks and
  16-byte TMA alignment never straddle parameters) and the buffer is padded to
  ``world * 256`` elements.  Rank r owns elements ``[r*S, (r+1)*S)``.
* **Execution** goes through one ``autograd.Function`` per block call.  With activation
  checkpointing the function saves only the block input and recomputes in backward;
  without it the block's local graph is kept and replayed.  Either way the function is the
  single place where gathers, reshards and gradient reduction are ordered, on explicit
  streams, with no module hooks.
* **Strategies**: ``FULL_SHARD`` frees the gathered buffer after forward and re-gathers in
  backward; ``SHARD_GRAD_OP`` keeps it between forward and backward; ``NO_SHARD`` (world 1)
  touches nothing.  On 180 GB parts ``SHARD_GRAD_OP`` is the default whenever the gathered
  model fits comfortably: one all-gather and one reduce-scatter per unit per optimizer step.
* **Gradients**: after a unit's backward its parameter gradients are packed into an fp32
  flat buffer, reduce-scattered (sum, then 1/world), and accumulated into the rank's fp32
  gradient shard.  Optimizers see per-parameter *pieces*: 1-D views of the owned shard with
  ``.grad`` views of the gradient shard, named like the original parameters.
* **Clipping** uses the true global norm (sum of squares over disjoint shards, one
  all-reduce) and hands the coefficient to the optimizer as a device scalar: no host sync.
* **Communication back ends**: ``nccl``/``gloo`` collectives through ``torch.distributed``
  (the measured baseline and the oracle) or ``fused`` peer-memory kernels from
  ``parallel/symm.py`` when available.
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass, field
from enum import Enum
from typing import Any, Callable, Dict, Iterable, List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn
from torch import Tensor

from .. import ops
from . import dist as pdist

ALIGN = 256


class ShardingStrategy(str, Enum):
    FULL_SHARD = "full_shard"
    SHARD_GRAD_OP = "shard_grad_op"
    NO_SHARD = "no_shard"


@dataclass
class ParamSlot:
    name: str
    shape: Tuple[int, ...]
    offset: int
    numel: int
    param: nn.Parameter


def _round_up(x: int, m: int) -> int:
    return -(-x // m) * m


@dataclass
class OwnedParam:
    """A 2-D parameter whose flat range is cut by shard boundaries, given as a whole to one rank
    (the owner) for optimizers that need whole matrices.  ``holders``: (rank, start, end) of every
    rank's piece in the parameter's own element coordinates."""
    unit: "FlatUnit"
    slot: ParamSlot
    owner: int
    holders: List[Tuple[int, int, int]]
    param: Optional[nn.Parameter] = None      # on the owner: the whole weight, compute dtype
    grad: Optional[Tensor] = None             # on the owner: the whole reduced gradient, fp32


class FlatUnit:
    """One communication unit: layout, owned shard, gathered buffer, gradient shard."""

    def __init__(self, name: str, module: Optional[nn.Module], named_params: List[Tuple[str, nn.Parameter]],
                 world: int, rank: int, device: torch.device, dtype: torch.dtype,
                 reduce_dtype: torch.dtype = torch.float32):
        self.name, self.module = name, module
        self.world, self.rank, self.device, self.dtype, self.reduce_dtype = world, rank, device, dtype, reduce_dtype
        self.slots: List[ParamSlot] = []
        off = 0
        # 1-D tensors (norm weights, per-head scalars, biases) first: they are needed before the
        # first matmul of the block, so a fused gather can fetch this small head region eagerly
        named_params = sorted(named_params, key=lambda np_: 0 if np_[1].ndim <= 1 else 1)
        self.head_elems = 0
        for n, p in named_params:
            self.slots.append(ParamSlot(n, tuple(p.shape), off, p.numel(), p))
            off = _round_up(off + p.numel(), ALIGN)
            if p.ndim <= 1:
                self.head_elems = off
        self.total = _round_up(max(off, ALIGN), world * ALIGN)
        self.shard_size = self.total // world
        # gathered buffer; parameters become views of an alias with its own version counter
        self.full = torch.zeros(self.total, dtype=dtype, device=device)
        for s in self.slots:
            self.full[s.offset:s.offset + s.numel].copy_(s.param.detach().reshape(-1).to(dtype))
        self._point_params()
        lo = rank * self.shard_size
        self.shard = self.full[lo:lo + self.shard_size].clone() if world > 1 else self.full
        self.grad_shard = torch.zeros(self.shard_size, dtype=torch.float32, device=device)
        self.gathered = True
        self.ready_event = None          # CUDA event: gathered buffer is valid
        self.reduce_event = None         # CUDA event: gradient shard holds this step's reduction
        self.pieces: List[Tuple[str, nn.Parameter]] = []
        self._build_pieces()

    # ---- parameter views
    def _point_params(self) -> None:
        alias = self.full.data
        for s in self.slots:
            s.param.data = alias[s.offset:s.offset + s.numel].view(s.shape)

    def _build_pieces(self) -> None:
        """Per-parameter views of the owned shard, exposed to optimizers."""
        lo, hi = self.rank * self.shard_size, (self.rank + 1) * self.shard_size
        self.pieces = []
        for s in self.slots:
            a, b = max(lo, s.offset), min(hi, _round_up(s.offset + s.numel, ALIGN))
            if b <= a or a >= s.offset + s.numel:
                continue
            whole = (a == s.offset and b >= s.offset + s.numel)
            if whole and self.world == 1:
                piece = s.param                       # NO_SHARD: the parameter itself
                piece._logical_numel = s.numel
                self.pieces.append((s.name, piece))
                continue
            # padded end: pieces of quantised states must cover whole 256-blocks
            b_eff = min(b, hi)
            view = self.shard[a - lo:b_eff - lo]
            piece = nn.Parameter(view, requires_grad=True)
            gview = self.grad_shard[a - lo:b_eff - lo]
            if view.dtype == gview.dtype:
                piece.grad = gview
            else:
                piece._fp32_grad = gview
            piece._logical_numel = s.numel
            piece._is_matrix = len(s.shape) >= 2
            piece._no_weight_decay = getattr(s.param, "_no_weight_decay", False) or len(s.shape) == 1
            if whole and len(s.shape) == 2 and (b_eff - a) == s.numel:
                piece._orig_2d_shape = s.shape
            self.pieces.append((s.name, piece))

    # ---- memory
    def free_full(self) -> None:
        if self.world > 1 and self.gathered:
            self.full.untyped_storage().resize_(0)
            self.gathered = False

    def alloc_full(self) -> None:
        if not self.gathered:
            self.full.untyped_storage().resize_(self.total * self.full.element_size())

    def nbytes_full(self) -> int:
        return self.total * self.full.element_size()


class _UnitFunction(torch.autograd.Function):
    """Runs one block as one autograd node; owns gather / recompute / gradient reduction."""

    @staticmethod
    def forward(ctx, runtime: "ShardedModel", unit: FlatUnit, hidden: Tensor, *args):
        ctx.runtime, ctx.unit, ctx.args = runtime, unit, args
        runtime._pre_forward(unit)
        if runtime._checkpointed(unit):
            with torch.no_grad():
                out = unit.module(hidden, *args)
            ctx.save_for_backward(hidden)
            ctx.local = None
        else:
            with torch.enable_grad():
                h = hidden.detach().requires_grad_(True)
                out_g = unit.module(h, *args)
            ctx.local = (h, out_g)
            out = out_g.detach()
        runtime._post_forward(unit)
        return out

    @staticmethod
    def backward(ctx, grad_out: Tensor):
        runtime, unit = ctx.runtime, ctx.unit
        recompute = ctx.local is None
        runtime._pre_backward(unit, recompute)
        if recompute:
            (hidden,) = ctx.saved_tensors
            with torch.enable_grad():
                h = hidden.detach().requires_grad_(True)
                out_g = unit.module(h, *ctx.args)
            runtime._after_recompute(unit)
        else:
            h, out_g = ctx.local
            ctx.local = None
        torch.autograd.backward(out_g, grad_out)
        runtime._post_backward(unit)
        return (None, None, h.grad) + (None,) * len(ctx.args)


class ShardedModel(nn.Module):
    """Wraps a model from ``nsa_optim_b200.models`` for sharded data-parallel training."""

    def __init__(self, model: nn.Module, info: Optional[pdist.DistInfo] = None,
                 strategy: "ShardingStrategy | str | None" = None,
                 param_dtype: Optional[torch.dtype] = None, reduce_dtype: torch.dtype = torch.float32,
                 activation_checkpointing: Optional[bool] = None, comm: str = "auto",
                 process_group=None, checkpoint_blocks: Optional[str] = None):
        super().__init__()
        self.module = model
        self.info = info or pdist.DistInfo(device=next(model.parameters()).device)
        self.world, self.rank = self.info.world_size, self.info.rank
        self.group = process_group
        device = self.info.device
        dtype = param_dtype or next(model.parameters()).dtype
        model.to(device=device)
        if self.world == 1:
            strategy = ShardingStrategy.NO_SHARD
        elif strategy is None:
            strategy = ShardingStrategy.SHARD_GRAD_OP
        self.strategy = ShardingStrategy(strategy)
        if activation_checkpointing is None:
            activation_checkpointing = bool(getattr(model, "gradient_checkpointing", False))
        self.activation_checkpointing = activation_checkpointing
        # With checkpointing on, ``checkpoint_blocks`` narrows it to the block kinds named (letters of
        # the hybrid pattern: M, D, A); the other blocks keep their activations.  Recomputing only the
        # cheap-to-recompute, activation-heavy kinds trades spare HBM for step time.
        self.checkpoint_kinds = set(checkpoint_blocks.upper()) if checkpoint_blocks else None
        self.comm_mode = self._resolve_comm(comm)
        # ---- units: root first (gathered for the whole step), then one per block
        blocks = model.block_modules()
        root_named = model.root_parameters()
        self.root = FlatUnit("root", None, root_named, self.world, self.rank, device, dtype, reduce_dtype)
        self.units: List[FlatUnit] = []
        prefix = "layers."
        for i, blk in enumerate(blocks):
            named = [(f"{prefix}{i}.{n}", p) for n, p in blk.named_parameters()]
            self.units.append(FlatUnit(f"{prefix}{i}", blk, named, self.world, self.rank, device, dtype, reduce_dtype))
        self._unit_of = {id(u.module): u for u in self.units}
        # buffers (rotary caches etc.) just move with the module
        for b in model.buffers():
            if b.is_floating_point() and b.dtype != torch.float32 and b.dtype != dtype:
                b.data = b.data.to(dtype)
        model.set_layer_runner(self._run_layer)
        self._cuda = device.type == "cuda"
        self.comm_stream = torch.cuda.Stream(device=device) if (self._cuda and self.world > 1) else None
        self._order: List[FlatUnit] = []
        self._exposed: list = []
        self.measure_exposed = False
        self.nvtx = False
        self._micro_steps = 0
        self.launch_counter = 0
        self.arena = None
        if self.comm_mode == "fused":
            try:
                self._setup_arena()
            except Exception as exc:  # noqa: BLE001 - fall back to the collective library, loudly
                if self.rank == 0:
                    print(f"[nsa_optim_b200] peer-memory setup failed ({type(exc).__name__}: {exc}); using NCCL collectives")
                self.comm_mode, self.arena = "torch", None
            ok = torch.tensor([1.0 if self.arena is not None else 0.0], device=device)
            pdist.all_reduce_min(ok, self.group)
            if float(ok) == 0.0:                      # every rank takes the same path
                self.comm_mode, self.arena = "torch", None
        if self.world > 1 and self.strategy == ShardingStrategy.FULL_SHARD:
            for u in self.units:
                u.free_full()

    # ------------------------------------------------------------------ peer-memory mode
    def _setup_arena(self) -> None:
        """Move every unit's shard and an fp32 gradient staging buffer into one IPC-shared arena
        and open three epoch channels per unit: shard-ready, grads-ready, grads-consumed."""
        from . import symm
        W = self.world
        units = self.all_units()
        es = units[0].shard.element_size()
        need = sum(_round_up(u.shard_size * es, 1024) + _round_up(W * u.shard_size * 4, 1024) for u in units) + 4096
        arena = symm.SymmetricArena(need, 3 * len(units), self.rank, W, self.info.device, self.group)
        for i, u in enumerate(units):
            u.off_shard = arena.alloc(u.shard_size * es)
            u.off_grad = arena.alloc(W * u.shard_size * 4)
            new_shard = arena.view(u.off_shard, u.shard_size, u.dtype)
            new_shard.copy_(u.shard)
            u.shard = new_shard
            u.grad_stage = arena.view(u.off_grad, W * u.shard_size, torch.float32)
            u.ch_shard, u.ch_grad, u.ch_done = 3 * i, 3 * i + 1, 3 * i + 2
            u.chunks_per_shard = max(1, min(1024, (u.shard_size * es) // (256 << 10)))
            u.chunk_flags = torch.zeros(W * u.chunks_per_shard, dtype=torch.int32, device=u.device)
            u.rs_partial = torch.zeros(symm.reduce_scatter_parts(), dtype=torch.float32, device=u.device)
            u._build_pieces()
        self.arena = arena
        self.shard_epoch = 1
        self.grad_epoch = 0
        self.fuse_first_gemm = True
        for u in units:
            symm.signal(arena, u.ch_shard, self.shard_epoch)
        torch.cuda.synchronize()
        pdist.barrier()

    def _fused_gather(self, unit: FlatUnit, lazy: bool) -> None:
        """P2P all-gather of a unit.  ``lazy`` (forward of a block): fetch only the small head
        region now and leave the rest to the first matmul of the block, whose kernel pulls the
        shards itself while it computes."""
        from . import symm
        from ..ops import native
        es = unit.shard.element_size()
        if lazy and self.fuse_first_gemm and unit.module is not None and unit.head_elems < unit.total:
            cur = torch.cuda.current_stream()
            symm.wait(self.arena, unit.ch_shard, self.shard_epoch)
            hi = unit.head_elems
            for p in range(self.world):
                a, b = p * unit.shard_size, min((p + 1) * unit.shard_size, hi)
                if a >= b:
                    break
                src = self.arena.view(unit.off_shard, unit.shard_size, unit.dtype, peer=p)[: b - a]
                unit.full[a:b].copy_(src, non_blocking=True)
            lo_ptr = unit.full.data_ptr()
            hi_ptr = lo_ptr + unit.total * es
            epoch = self.shard_epoch

            def run(x, weight, _u=unit):
                native.clear_pending_gather()
                # The per-chunk flags hold the epoch of the last gather.  Within one optimizer step the
                # epoch does not change, so a second gather of the same unit (next micro-batch under
                # gradient accumulation, after the buffer was freed and re-allocated) would find them
                # already set and let the GEMM read rows the copy CTAs have not written yet.
                _u.chunk_flags.zero_()
                y = symm.gemm_all_gather(self.arena, x, _u.full, _u.off_shard, _u.shard_size,
                                         (weight.data_ptr() - lo_ptr) // es, weight.shape[0], _u.chunk_flags,
                                         _u.chunks_per_shard, _u.ch_shard, epoch)
                _u.chunk_flags_epoch = epoch
                return y

            # chunk flags count epochs too: they are below `epoch` until this step's kernel sets them
            native.set_pending_gather(lo_ptr, hi_ptr, run, lambda _u=unit: self._fused_gather_now(_u))
            return
        self._fused_gather_now(unit)

    def _fused_gather_now(self, unit: FlatUnit) -> None:
        from . import symm
        es = unit.shard.element_size()
        symm.all_gather(self.arena, unit.off_shard, unit.shard_size * es, unit.full, unit.ch_shard, self.shard_epoch,
                        ctas_per_peer=max(4, 64 // self.world))

    def _fused_reduce(self, unit: FlatUnit) -> None:
        from . import symm
        epoch = self.grad_epoch
        if epoch > 1:
            symm.wait(self.arena, unit.ch_done, epoch - 1)         # peers have consumed the previous buffer
        stage = unit.grad_stage
        for s in unit.slots:
            g = s.param.grad
            dst = stage[s.offset:s.offset + s.numel]
            if g is not None:
                dst.copy_(g.reshape(-1))
                s.param.grad = None
            else:
                dst.zero_()
        symm.signal(self.arena, unit.ch_grad, epoch)
        self.comm_stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.comm_stream):
            symm.reduce_scatter(self.arena, unit.off_grad, unit.grad_shard, 1.0 / self.world, True, unit.ch_grad, epoch,
                                unit.rs_partial)
            symm.signal(self.arena, unit.ch_done, epoch)

    # ------------------------------------------------------------------ comm selection
    def _resolve_comm(self, comm: str) -> str:
        if self.world == 1:
            return "none"
        if comm in ("nccl", "gloo", "torch"):
            return "torch"
        if comm == "fused":
            return "fused"
        # auto: the peer-memory kernels wherever they can run (CUDA ranks of one node), else the library
        dev = self.info.device
        if dev.type == "cuda" and torch.cuda.device_count() >= self.world and os.environ.get("NSA_B200_COMM", "") != "nccl":
            return "fused"
        return "torch"

    # ------------------------------------------------------------------ gather / reduce
    def all_units(self) -> List[FlatUnit]:
        return [self.root] + self.units

    def _gather(self, unit: FlatUnit, async_: bool = True, lazy: bool = False) -> None:
        if self.world == 1 or unit.gathered:
            return
        unit.alloc_full()
        if self.arena is not None:
            if lazy:
                self._fused_gather(unit, True)          # on the compute stream, inside the first matmul
            else:
                self.comm_stream.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(self.comm_stream):
                    self._fused_gather_now(unit)
                    unit.ready_event = torch.cuda.Event()
                    unit.ready_event.record(self.comm_stream)
                unit.full.record_stream(self.comm_stream)
            unit.gathered = True
            return
        if self.comm_stream is not None:
            self.comm_stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.comm_stream):
                pdist.all_gather_flat(unit.full, unit.shard, self.group)
                unit.ready_event = torch.cuda.Event()
                unit.ready_event.record(self.comm_stream)
            unit.full.record_stream(self.comm_stream)
        else:
            pdist.all_gather_flat(unit.full, unit.shard, self.group)
        unit.gathered = True

    def _wait_ready(self, unit: FlatUnit) -> None:
        if unit.ready_event is not None:
            with self._exposed_wait():
                torch.cuda.current_stream().wait_event(unit.ready_event)
            unit.ready_event = None

    # ---- exposed communication: how long the compute stream stood still waiting for the
    # communication stream.  Each wait is bracketed by two events on the compute stream; the time
    # between them is the part of the collective that compute did not hide.  (A gather that runs
    # inside the consuming GEMM has no such wait; its stall, if any, is inside that kernel's time.)
    class _ExposedWait:
        def __init__(self, owner):
            self.owner = owner

        def __enter__(self):
            o = self.owner
            self.e0 = None
            if o.measure_exposed and o._cuda:
                self.e0 = torch.cuda.Event(enable_timing=True)
                self.e0.record()

        def __exit__(self, *exc):
            if self.e0 is not None:
                e1 = torch.cuda.Event(enable_timing=True)
                e1.record()
                self.owner._exposed.append((self.e0, e1))
            return False

    def _exposed_wait(self):
        return ShardedModel._ExposedWait(self)

    def pop_exposed_comm_ms(self) -> float:
        """Sum of the exposed waits recorded since the last call (call after a synchronize)."""
        total = sum(a.elapsed_time(b) for a, b in self._exposed)
        self._exposed = []
        return float(total)

    def _reduce_grads(self, unit: FlatUnit) -> None:
        """Pack parameter gradients, reduce-scatter, accumulate 1/world of the sum."""
        if self.world == 1:
            return
        if self.arena is not None:
            self._fused_reduce(unit)
            return
        flat = torch.zeros(unit.total, dtype=unit.reduce_dtype, device=unit.device)
        for s in unit.slots:
            g = s.param.grad
            if g is not None:
                flat[s.offset:s.offset + s.numel].copy_(g.reshape(-1))
                s.param.grad = None
        out = torch.empty(unit.shard_size, dtype=unit.reduce_dtype, device=unit.device)
        if self.comm_stream is not None:
            self.comm_stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.comm_stream):
                pdist.reduce_scatter_flat(out, flat, self.group)
                unit.grad_shard.add_(out, alpha=1.0 / self.world)
                unit.reduce_event = torch.cuda.Event()
                unit.reduce_event.record(self.comm_stream)
            flat.record_stream(self.comm_stream)
            out.record_stream(self.comm_stream)
        else:
            pdist.reduce_scatter_flat(out, flat, self.group)
            unit.grad_shard.add_(out.float(), alpha=1.0 / self.world)

    # ------------------------------------------------------------------ unit lifecycle
    def _neighbour(self, unit: FlatUnit, step: int) -> Optional[FlatUnit]:
        i = self.units.index(unit) + step
        return self.units[i] if 0 <= i < len(self.units) else None

    def _lazy(self) -> bool:
        return self.arena is not None and self.fuse_first_gemm

    def _pre_forward(self, unit: FlatUnit) -> None:
        if self._lazy():
            self._gather(unit, lazy=True)        # the block's first matmul pulls the shards itself
        else:
            self._gather(unit)
            nxt = self._neighbour(unit, +1)
            if nxt is not None:
                self._gather(nxt)
        self._wait_ready(unit)

    def _post_forward(self, unit: FlatUnit) -> None:
        if self.arena is not None:
            from ..ops import native
            native.flush_pending_gather()        # nothing consumed the deferred gather: do it now
        if self.strategy == ShardingStrategy.FULL_SHARD:
            unit.free_full()

    def _pre_backward(self, unit: FlatUnit, recompute: bool = False) -> None:
        """Re-gather for the backward pass.  A block that recomputes its forward first lets the
        recompute's first matmul gather the unit (the same fused kernel as in the forward pass); a
        block that kept its activations needs the weights for dX = dY W, where a shard covers a slice
        of the reduction dimension and no tile can start on local data alone, so its gather runs as
        the stand-alone kernel on the communication stream, issued one block ahead."""
        if recompute and self._lazy():
            self._gather(unit, lazy=True)
        else:
            self._gather(unit)
        prv = self._neighbour(unit, -1)
        if prv is not None and self.strategy == ShardingStrategy.FULL_SHARD and not (self._lazy() and self._checkpointed(prv)):
            self._gather(prv)
        self._wait_ready(unit)

    def _after_recompute(self, unit: FlatUnit) -> None:
        if self.arena is not None:
            from ..ops import native
            native.flush_pending_gather()        # nothing in the recompute consumed the deferred gather

    def _post_backward(self, unit: FlatUnit) -> None:
        self._reduce_grads(unit)
        if self.strategy == ShardingStrategy.FULL_SHARD:
            unit.free_full()

    def _checkpointed(self, unit: FlatUnit) -> bool:
        if not self.activation_checkpointing:
            return False
        if self.checkpoint_kinds is None:
            return True
        return getattr(unit.module, "block_kind", "A") in self.checkpoint_kinds

    def _run_layer(self, layer: nn.Module, hidden: Tensor, *args) -> Tensor:
        if self.nvtx:
            with torch.cuda.nvtx.range(f"{self._unit_of[id(layer)].name} {getattr(layer, 'block_kind', '')}"):
                return self._run_layer_impl(layer, hidden, *args)
        return self._run_layer_impl(layer, hidden, *args)

    def _run_layer_impl(self, layer: nn.Module, hidden: Tensor, *args) -> Tensor:
        unit = self._unit_of[id(layer)]
        if not (torch.is_grad_enabled() and self.module.training):
            self._pre_forward(unit)
            out = layer(hidden, *args)
            if self.strategy == ShardingStrategy.FULL_SHARD:
                unit.free_full()
            return out
        if self.world == 1 and not self._checkpointed(unit):
            return layer(hidden, *args)
        return _UnitFunction.apply(self, unit, hidden, *args)

    # ------------------------------------------------------------------ public step API
    def forward(self, *args, **kwargs):
        self._gather(self.root)
        self._wait_ready(self.root)
        if self.units and not self._lazy():
            self._gather(self.units[0])
        return self.module(*args, **kwargs)

    def backward(self, loss: Tensor) -> None:
        """``loss.backward()`` followed by the root unit's gradient reduction."""
        if self.arena is not None:
            self.grad_epoch += 1
        loss.backward()
        self._reduce_grads(self.root)
        self._micro_steps += 1

    def regather_all(self) -> None:
        """After an optimizer step the gathered copies are stale: mark and (for the keeping
        strategies) re-issue every all-gather on the communication stream."""
        if self.world == 1:
            return
        if self.arena is not None:
            from . import symm
            self.shard_epoch += 1
            for u in self.all_units():
                symm.signal(self.arena, u.ch_shard, self.shard_epoch)
        for u in self.all_units():
            u.gathered = False
            if u is self.root or (self.strategy != ShardingStrategy.FULL_SHARD and not self._lazy()):
                self._gather(u)
            elif self.strategy == ShardingStrategy.FULL_SHARD:
                u.full.untyped_storage().resize_(0)

    def wait_reductions(self) -> None:
        if self.comm_stream is not None:
            with self._exposed_wait():
                torch.cuda.current_stream().wait_stream(self.comm_stream)

    def zero_grad(self, set_to_none: bool = True) -> None:
        if self.world == 1:
            for p in self.module.parameters():
                p.grad = None
            return
        for u in self.all_units():
            u.grad_shard.zero_()
            for s in u.slots:
                s.param.grad = None

    # ------------------------------------------------------------------ whole-matrix ownership
    def enable_owner_preconditioning(self) -> int:
        """For optimizers that precondition whole matrices (SOAP, Shampoo).  Shards are contiguous
        ranges of a unit's flat buffer, so most large matrices are cut by a shard boundary and no rank
        sees their whole gradient.  Every such matrix gets one owner among the ranks that hold a piece
        (round robin, so the owners' work is spread): before the optimizer step the holders send
        their reduced gradient pieces to the owner, the owner updates the whole matrix with its whole
        state, and afterwards sends every holder its piece of the new weight.  The pieces leave the
        holders' optimizer lists, so nothing is updated twice and no matrix falls back to an
        elementwise rule.  (The reference keeps SOAP under FSDP by all-reducing Kronecker factors of
        flat shards, optimizers.py:873-905, and degrades to Adam where shapes are lost.)
        A matrix that lies whole inside one shard stays with that rank and is handed to the optimizer
        as a 2-D view of the shard.  Returns the number of matrices handled.  Call before building the
        optimizer, and again (rebuilding the optimizer's parameter list) if the shard storage moves."""
        self.owned: List[OwnedParam] = []
        if self.world == 1:
            return 0
        k = 0
        for u in self.all_units():
            full = None
            for s in u.slots:
                if len(s.shape) != 2:
                    continue
                holders = []
                for r in range(self.world):
                    lo, hi = r * u.shard_size, (r + 1) * u.shard_size
                    a, b = max(lo, s.offset), min(hi, s.offset + s.numel)
                    if b > a:
                        holders.append((r, a - s.offset, b - s.offset))
                if len(holders) == 1:
                    # whole inside one shard: that rank updates it in place, as a matrix, through 2-D
                    # views of its shard and gradient shard (no copy, nothing to exchange)
                    op = OwnedParam(u, s, holders[0][0], [])
                    if op.owner == self.rank:
                        base = s.offset - self.rank * u.shard_size
                        op.param = nn.Parameter(u.shard[base:base + s.numel].view(s.shape), requires_grad=True)
                        op.grad = u.grad_shard[base:base + s.numel].view(s.shape)
                        if op.param.dtype == torch.float32:
                            op.param.grad = op.grad
                        else:
                            op.param._fp32_grad = op.grad
                        op.param._logical_numel = s.numel
                        op.param._no_weight_decay = getattr(s.param, "_no_weight_decay", False)
                    self.owned.append(op)
                    continue
                owner = holders[k % len(holders)][0]
                k += 1
                op = OwnedParam(u, s, owner, holders)
                if owner == self.rank:
                    if full is None:
                        full = u.full if u.gathered else self._full_unit_tensor(u)
                    w = full[s.offset:s.offset + s.numel].view(s.shape).detach().clone()
                    op.param = nn.Parameter(w, requires_grad=True)
                    op.grad = torch.zeros(s.shape, dtype=torch.float32, device=u.device)
                    if w.dtype == torch.float32:
                        op.param.grad = op.grad
                    else:
                        op.param._fp32_grad = op.grad
                    op.param._logical_numel = s.numel
                    op.param._no_weight_decay = getattr(s.param, "_no_weight_decay", False)
                self.owned.append(op)
            if full is not None and full is not u.full:
                del full
        moved = {op.slot.name for op in self.owned}
        for u in self.all_units():
            u.pieces = [(n, p) for n, p in u.pieces if n not in moved]
        return len(self.owned)

    def _exchange_owned(self, to_owner: bool) -> None:
        """Moves every owned matrix's pieces between holders and owner: reduced gradients to the owner
        (``to_owner``) or updated weights back to the holders."""
        if not getattr(self, "owned", None):
            return
        p2p = []
        for op in self.owned:
            u, s = op.unit, op.slot
            base = s.offset - self.rank * u.shard_size          # slot coordinate -> index into this rank's shard
            for r, a, b in op.holders:
                mine = r == self.rank
                own = op.owner == self.rank
                if to_owner:
                    if mine and own:
                        op.grad.view(-1)[a:b].copy_(u.grad_shard[base + a:base + b])
                    elif mine:
                        p2p.append(dist.P2POp(dist.isend, u.grad_shard[base + a:base + b], op.owner, self.group))
                    elif own:
                        p2p.append(dist.P2POp(dist.irecv, op.grad.view(-1)[a:b], r, self.group))
                else:
                    if mine and own:
                        u.shard[base + a:base + b].copy_(op.param.data.view(-1)[a:b])
                    elif own:
                        p2p.append(dist.P2POp(dist.isend, op.param.data.view(-1)[a:b], r, self.group))
                    elif mine:
                        p2p.append(dist.P2POp(dist.irecv, u.shard[base + a:base + b], op.owner, self.group))
        if p2p:
            for req in dist.batch_isend_irecv(p2p):
                req.wait()

    def collect_owned_grads(self) -> None:
        self.wait_reductions()
        self._exchange_owned(True)

    def publish_owned_weights(self) -> None:
        self._exchange_owned(False)

    # ------------------------------------------------------------------ optimizer view
    def named_optimizer_parameters(self) -> List[Tuple[str, nn.Parameter]]:
        out = []
        for u in self.all_units():
            out.extend(u.pieces)
        for op in getattr(self, "owned", []):
            if op.param is not None:
                out.append((op.slot.name, op.param))
        return out

    def local_grads(self) -> List[Tensor]:
        if self.world == 1:
            return [p.grad for p in self.module.parameters() if p.grad is not None]
        return [u.grad_shard for u in self.all_units()]

    def clip_grad_norm(self, max_norm: float, local_only: bool = False) -> Tuple[Tensor, Optional[Tensor]]:
        """-> (global gradient norm, clip coefficient or None).  Both stay on the device; the
        coefficient is meant for ``optimizer.step(grad_scale=coef)``.  ``local_only`` reproduces
        the reference's behaviour of clipping by the local shard's norm (train.py:268-277)."""
        self.wait_reductions()
        grads = self.local_grads()
        if not grads:
            z = torch.zeros((), device=self.info.device)
            return z, None
        if self._cuda and ops.get_backend() != "torch":
            sq = ops.native_module().sumsq(grads)            # one small kernel pair per tensor, fp32 accumulation
        else:
            sq = torch.stack([g.float().pow(2).sum() for g in grads]).sum()
        if self.world > 1 and not local_only:
            pdist.all_reduce_sum(sq, self.group)
        norm = sq.sqrt()
        if max_norm is None or max_norm <= 0:
            return norm, None
        coef = (max_norm / (norm + 1e-6)).clamp(max=1.0)
        return norm, coef

    # ------------------------------------------------------------------ state dicts
    def _full_unit_tensor(self, u: FlatUnit) -> Tensor:
        if self.world == 1:
            return u.full
        out = torch.empty(u.total, dtype=u.dtype, device=u.device)
        self.wait_reductions()
        pdist.all_gather_flat(out, u.shard, self.group)
        return out

    def state_dict(self, rank0_only: bool = True, *args, **kwargs) -> Dict[str, Tensor]:
        """Full (unsharded) CPU state dict with the wrapped model's key names."""
        sd: Dict[str, Tensor] = {}
        keep = (not rank0_only) or self.rank == 0
        for u in self.all_units():
            full = self._full_unit_tensor(u)
            if keep:
                for s in u.slots:
                    sd[s.name] = full[s.offset:s.offset + s.numel].view(s.shape).detach().cpu().clone()
        if keep:
            params = {n for n, _ in self.module.named_parameters()}
            for k, v in self.module.state_dict().items():
                if k not in params:
                    sd[k] = v.detach().cpu().clone()
            order = list(self.module.state_dict().keys())
            sd = {k: sd[k] for k in order if k in sd}
        return sd

    def load_state_dict(self, state_dict: Dict[str, Tensor], strict: bool = True):
        missing = []
        for u in self.all_units():
            u.alloc_full()
            for s in u.slots:
                if s.name in state_dict:
                    u.full[s.offset:s.offset + s.numel].copy_(state_dict[s.name].reshape(-1).to(u.dtype))
                else:
                    missing.append(s.name)
            u.gathered = True
            if self.world > 1:
                lo = self.rank * u.shard_size
                u.shard.copy_(u.full[lo:lo + u.shard_size])
        bufs = {n for n, _ in self.module.named_buffers()}
        for k, v in state_dict.items():
            if k in bufs:
                self.module.get_buffer(k).copy_(v)
        if strict and missing:
            raise KeyError(f"missing keys in state_dict: {missing[:5]}{'...' if len(missing) > 5 else ''}")
        if self.world > 1 and self.strategy == ShardingStrategy.FULL_SHARD:
            for u in self.units:
                u.free_full()
        return missing

    def piece_map(self) -> Dict[int, Tuple[FlatUnit, ParamSlot, int, int]]:
        """id(piece) -> (unit, slot, start offset of the piece inside the parameter, length)."""
        out = {}
        for op in getattr(self, "owned", []):
            if op.param is not None:
                out[id(op.param)] = (op.unit, op.slot, 0, op.slot.numel)
        for u in self.all_units():
            lo = u.rank * u.shard_size
            by_name = {s.name: s for s in u.slots}
            for name, piece in u.pieces:
                s = by_name[name]
                if piece is s.param:
                    out[id(piece)] = (u, s, 0, s.numel)
                else:
                    a = max(lo, s.offset)
                    out[id(piece)] = (u, s, a - s.offset, piece.numel())
        return out


def wrap_model(model: nn.Module, info: Optional[pdist.DistInfo] = None, **kwargs) -> ShardedModel:
    return ShardedModel(model, info, **kwargs)
