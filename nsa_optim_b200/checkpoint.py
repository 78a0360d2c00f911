"""Checkpoint save / load in the reference's directory layout.

Reference behaviour (nngabe/nsa_optim train.py:342-517): directory
``{output_dir}/{run_name}/checkpoint-{step}/`` holding ``model.pt`` (full, unsharded CPU
state dict), ``optimizer.pt``, ``scheduler.pt`` and ``config.json`` with the keys
``step, model_type, model_size, attention_type, optimizer_type, max_seq_length, fsdp,
custom_optim``; rank 0 writes, then a barrier.  The reference does not restore SOAP/Shampoo
state, the data position or RNG state.

Kept: the layout, file names, key names, ``config.json`` fields, and the optimizer file as
``{"state": {parameter_name: {...}}, "param_groups": [...]}``.
Added: ``trainer_state.pt`` (RNG states, data position, token count) and, for sharded
runs, ``optimizer.rank{r}.pt`` with each rank's shard-local state so every optimizer type
(including the SOAP family) resumes exactly at the same world size.
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, Optional

import torch
import torch.nn as nn

from .models.kernels import remap_legacy_keys
from .parallel import dist as pdist
from .parallel.sharded import ShardedModel

CUSTOM_OPTIMIZERS = ("soap", "soap4bit", "soap8bit", "shampoo")


def checkpoint_dir(output_dir: str, run_name: str, step: int) -> str:
    return os.path.join(output_dir, run_name, f"checkpoint-{step}")


def _named_state(optimizer: torch.optim.Optimizer, names: Dict[int, str]) -> Dict[str, Any]:
    """Optimizer state keyed by parameter name instead of by tensor."""
    state = {}
    for p, st in optimizer.state.items():
        key = names.get(id(p))
        if key is None:
            continue
        state[key] = {k: (v.detach().cpu() if torch.is_tensor(v) else _to_cpu(v)) for k, v in st.items()}
    groups = []
    for g in optimizer.param_groups:
        gg = {k: v for k, v in g.items() if k != "params"}
        gg["params"] = [names.get(id(p), "?") for p in g["params"]]
        groups.append(gg)
    return {"state": state, "param_groups": groups}


def _to_cpu(v):
    if torch.is_tensor(v):
        return v.detach().cpu()
    if isinstance(v, (list, tuple)):
        return type(v)(_to_cpu(x) for x in v)
    if isinstance(v, dict):
        return {k: _to_cpu(x) for k, x in v.items()}
    return v


def _to_device(v, device):
    if torch.is_tensor(v):
        return v.to(device)
    if isinstance(v, (list, tuple)):
        return type(v)(_to_device(x, device) for x in v)
    if isinstance(v, dict):
        return {k: _to_device(x, device) for k, x in v.items()}
    return v


def _param_names(model) -> Dict[int, str]:
    if isinstance(model, ShardedModel):
        return {id(p): n for n, p in model.named_optimizer_parameters()}
    return {id(p): n for n, p in model.named_parameters()}


def _piece_layout(model) -> Dict[str, Any]:
    """name -> (offset of the piece inside its parameter, logical length, parameter shape)."""
    out = {}
    if isinstance(model, ShardedModel):
        names = _param_names(model)
        for pid, (unit, slot, start, length) in model.piece_map().items():
            name = names.get(pid)
            if name is not None:
                out[name] = (int(start), int(min(length, slot.numel - start)), tuple(slot.shape))
    return out


def _consolidate(path: str, world_size: int, optimizer) -> Optional[Dict[str, Any]]:
    """Builds the sharding-independent optimizer file from the per-rank files: per parameter name,
    ``step`` and full-shape fp32 ``exp_avg`` / ``exp_avg_sq`` assembled from every rank's piece
    (dequantised where the moments are stored as codes).  A state that is not elementwise
    (Kronecker factors and eigenbases of a matrix one rank owns whole) is carried over as saved."""
    from .optimizers import _moment_codec, state_moments
    bits, block = _moment_codec(optimizer)
    full: Dict[str, Dict[str, Any]] = {}
    shapes: Dict[str, tuple] = {}
    groups = None
    for r in range(world_size):
        f = os.path.join(path, f"optimizer.rank{r}.pt")
        if not os.path.exists(f):
            return None
        osd = torch.load(f, map_location="cpu", weights_only=False)
        groups = groups or osd.get("param_groups")
        layout = osd.get("piece_layout", {})
        for name, st in osd.get("state", {}).items():
            if name not in layout:
                continue
            start, length, shape = layout[name]
            numel = 1
            for d in shape:
                numel *= d
            mv = state_moments(st, bits, block)
            if mv is None:
                if start == 0 and length == numel:
                    full[name] = st
                continue
            shapes[name] = tuple(shape)
            step, m, v = mv
            ent = full.setdefault(name, {"step": step, "exp_avg": torch.zeros(numel)})
            if "exp_avg" not in ent or not torch.is_tensor(ent["exp_avg"]) or ent["exp_avg"].numel() != numel:
                continue
            ent["step"] = max(int(ent["step"]), step)
            ent["exp_avg"][start:start + length] = m[:length]
            if v is not None:
                ent.setdefault("exp_avg_sq", torch.zeros(numel))[start:start + length] = v[:length]
    for name, ent in full.items():
        for k in ("exp_avg", "exp_avg_sq"):
            t = ent.get(k)
            if torch.is_tensor(t) and t.dtype == torch.float32 and t.ndim == 1 and name in shapes:
                ent[k] = t.view(shapes[name])
    return {"state": full, "param_groups": groups or [], "consolidated": True, "sharded": False,
            "world_size": world_size}


def save_checkpoint(model, optimizer, scheduler, step: int, output_dir: str, run_name: str,
                    meta: Optional[Dict[str, Any]] = None, trainer_state: Optional[Dict[str, Any]] = None,
                    rank: int = 0, world_size: int = 1) -> str:
    """Writes ``model.pt`` (full state dict), ``optimizer.pt``, ``scheduler.pt``, ``config.json`` and
    ``trainer_state.pt``.  At world size 1 ``optimizer.pt`` is the optimizer's own state keyed by
    parameter name.  In a sharded run every rank writes ``optimizer.rank{r}.pt`` (exact resume at the
    same world size) and rank 0 assembles ``optimizer.pt`` from them as full tensors per parameter
    name, which any world size can load (the counterpart of the reference's gathered
    ``FSDP.optim_state_dict``, train.py:382-385).  The per-rank files must be visible to rank 0
    (one node, or a shared file system)."""
    path = checkpoint_dir(output_dir, run_name, step)
    sharded = isinstance(model, ShardedModel) and model.world > 1
    model_sd = model.state_dict() if isinstance(model, ShardedModel) else \
        {k: v.detach().cpu() for k, v in model.state_dict().items()}
    names = _param_names(model)
    opt_sd = _named_state(optimizer, names) if optimizer is not None else None
    if opt_sd is not None:
        opt_sd["sharded"] = sharded
        opt_sd["world_size"] = world_size
        opt_sd["piece_layout"] = _piece_layout(model)
    if rank == 0:
        os.makedirs(path, exist_ok=True)
    pdist.barrier()
    if sharded and opt_sd is not None:
        torch.save(opt_sd, os.path.join(path, f"optimizer.rank{rank}.pt"))
        pdist.barrier()
    if rank == 0:
        torch.save(model_sd, os.path.join(path, "model.pt"))
        if opt_sd is not None:
            full = _consolidate(path, world_size, optimizer) if sharded else opt_sd
            if full is not None:
                torch.save(full, os.path.join(path, "optimizer.pt"))
        if scheduler is not None:
            torch.save(scheduler.state_dict(), os.path.join(path, "scheduler.pt"))
        cfg = {"step": step, "fsdp": sharded}
        cfg.update(meta or {})
        cfg.setdefault("custom_optim", str(cfg.get("optimizer_type", "")) in CUSTOM_OPTIMIZERS)
        with open(os.path.join(path, "config.json"), "w") as f:
            json.dump(cfg, f, indent=2)
        ts = dict(trainer_state or {})
        ts["torch_rng"] = torch.get_rng_state()
        if torch.cuda.is_available():
            ts["cuda_rng"] = torch.cuda.get_rng_state_all()
        torch.save(ts, os.path.join(path, "trainer_state.pt"))
    pdist.barrier()
    return path


def _load_optimizer(path: str, model, optimizer, rank: int) -> Dict[str, Any]:
    """Restores optimizer state.  Order of preference: this rank's own file when it was written at
    the current world size; else the sharding-independent ``optimizer.pt`` (full tensors per
    parameter name, or a world-size-1 state), re-cut to this run's pieces; a file whose layout
    cannot be matched is skipped with a warning and the optimizer starts fresh.  Every restored
    tensor is checked against the size the update kernels will index."""
    from .optimizers import _moment_codec, install_moments, state_fits, state_moments
    names = _param_names(model)
    by_name = {n: p for p in (q for g in optimizer.param_groups for q in g["params"])
               for n in [names.get(id(p))] if n is not None}
    world = model.world if isinstance(model, ShardedModel) else 1
    report = {"optimizer_state_loaded": 0, "optimizer_state_skipped": 0, "optimizer_state_source": None}
    osd = None
    shard_file = os.path.join(path, f"optimizer.rank{rank}.pt")
    if world > 1 and os.path.exists(shard_file):
        cand = torch.load(shard_file, map_location="cpu", weights_only=False)
        if int(cand.get("world_size", -1)) == world and bool(cand.get("sharded", False)):
            osd, report["optimizer_state_source"] = cand, "rank file"
    exact = osd is not None
    if osd is None:
        opt_file = os.path.join(path, "optimizer.pt")
        if not os.path.exists(opt_file):
            return report
        osd = torch.load(opt_file, map_location="cpu", weights_only=False)
        saved_world = int(osd.get("world_size", 1))
        if osd.get("sharded", False) and not osd.get("consolidated", False):
            # a shard-local state written under the name of the full file: cannot be re-cut
            print(f"[checkpoint] {opt_file} holds the shard-local state of one rank of {saved_world}; "
                  f"optimizer state not restored")
            return report
        exact = (not osd.get("consolidated", False)) and world == 1 and saved_world == 1
        report["optimizer_state_source"] = "optimizer.pt" + ("" if exact else " (re-cut)")
    if exact:
        for name, st in osd.get("state", {}).items():
            p = by_name.get(name)
            if p is None:
                continue
            if not state_fits(optimizer, p, st):
                report["optimizer_state_skipped"] += 1
                continue
            optimizer.state[p] = {k: _to_device(v, p.device) for k, v in st.items()}
            report["optimizer_state_loaded"] += 1
    else:
        bits, block = _moment_codec(optimizer)
        layout = _piece_layout(model)
        for name, p in by_name.items():
            st = osd.get("state", {}).get(name)
            if st is None:
                continue
            start, length, shape = layout.get(name, (0, p.numel(), tuple(p.shape)))
            mv = state_moments(st, bits, block)
            if mv is None:
                # whole-matrix state: usable only by a piece that is the whole parameter
                if start == 0 and length == p.numel() and state_fits(optimizer, p, st):
                    optimizer.state[p] = {k: _to_device(v, p.device) for k, v in st.items()}
                    report["optimizer_state_loaded"] += 1
                else:
                    report["optimizer_state_skipped"] += 1
                continue
            step, m, v = mv
            if m.numel() < start + length:
                report["optimizer_state_skipped"] += 1
                continue

            def cut(t):
                if t is None:
                    return None
                out = torch.zeros(p.numel(), dtype=torch.float32)
                out[:length] = t.reshape(-1)[start:start + length]
                return out

            if install_moments(optimizer, p, step, cut(m), cut(v)):
                report["optimizer_state_loaded"] += 1
            else:
                report["optimizer_state_skipped"] += 1
    if report["optimizer_state_skipped"]:
        print(f"[checkpoint] {report['optimizer_state_skipped']} optimizer state entries did not match this "
              f"run's layout and start fresh")
    for g, gs in zip(optimizer.param_groups, osd.get("param_groups", [])):
        for k, v in gs.items():
            if k not in ("params", "param_names"):
                g[k] = v
    return report


def load_checkpoint(path: str, model, optimizer=None, scheduler=None, rank: int = 0,
                    strict: bool = True) -> Dict[str, Any]:
    """Restores model, optimizer (see :func:`_load_optimizer`) and scheduler.
    Returns ``config.json`` merged with ``trainer_state.pt`` (key ``step`` is the resume step)."""
    with open(os.path.join(path, "config.json")) as f:
        cfg = json.load(f)
    sd = remap_legacy_keys(torch.load(os.path.join(path, "model.pt"), map_location="cpu", weights_only=False))
    if isinstance(model, ShardedModel):
        model.load_state_dict(sd, strict=strict)
        if model.world > 1:
            model.regather_all()
    else:
        model.load_state_dict(sd, strict=strict)
    if optimizer is not None:
        cfg.update(_load_optimizer(path, model, optimizer, rank))
    sched_file = os.path.join(path, "scheduler.pt")
    if scheduler is not None and os.path.exists(sched_file):
        scheduler.load_state_dict(torch.load(sched_file, map_location="cpu", weights_only=False))
    ts_file = os.path.join(path, "trainer_state.pt")
    if os.path.exists(ts_file):
        ts = torch.load(ts_file, map_location="cpu", weights_only=False)
        if "torch_rng" in ts:
            torch.set_rng_state(ts.pop("torch_rng"))
        if "cuda_rng" in ts and torch.cuda.is_available():
            try:
                torch.cuda.set_rng_state_all(ts.pop("cuda_rng"))
            except Exception:  # noqa: BLE001 - device count changed between save and load
                ts.pop("cuda_rng", None)
        cfg.update(ts)
    return cfg
