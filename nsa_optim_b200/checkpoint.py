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


def save_checkpoint(model, optimizer, scheduler, step: int, output_dir: str, run_name: str,
                    meta: Optional[Dict[str, Any]] = None, trainer_state: Optional[Dict[str, Any]] = None,
                    rank: int = 0, world_size: int = 1) -> str:
    path = checkpoint_dir(output_dir, run_name, step)
    sharded = isinstance(model, ShardedModel) and model.world > 1
    model_sd = model.state_dict() if isinstance(model, ShardedModel) else \
        {k: v.detach().cpu() for k, v in model.state_dict().items()}
    names = _param_names(model)
    opt_sd = _named_state(optimizer, names) if optimizer is not None else None
    if rank == 0:
        os.makedirs(path, exist_ok=True)
    pdist.barrier()
    if sharded and opt_sd is not None:
        opt_sd["sharded"] = True
        opt_sd["world_size"] = world_size
        torch.save(opt_sd, os.path.join(path, f"optimizer.rank{rank}.pt"))
    if rank == 0:
        torch.save(model_sd, os.path.join(path, "model.pt"))
        if opt_sd is not None:
            torch.save(opt_sd, os.path.join(path, "optimizer.pt"))
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


def load_checkpoint(path: str, model, optimizer=None, scheduler=None, rank: int = 0,
                    strict: bool = True) -> Dict[str, Any]:
    """Restores model, optimizer (when its saved layout matches this run) and scheduler.
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
        names = _param_names(model)
        by_name = {n: p for p in (q for g in optimizer.param_groups for q in g["params"])
                   for n in [names.get(id(p))] if n is not None}
        shard_file = os.path.join(path, f"optimizer.rank{rank}.pt")
        opt_file = shard_file if os.path.exists(shard_file) else os.path.join(path, "optimizer.pt")
        if os.path.exists(opt_file):
            osd = torch.load(opt_file, map_location="cpu", weights_only=False)
            loaded = 0
            for name, st in osd.get("state", {}).items():
                p = by_name.get(name)
                if p is None:
                    continue
                ok = all((not torch.is_tensor(v)) or v.numel() in (p.numel(), v.numel()) for v in st.values())
                if not ok:
                    continue
                optimizer.state[p] = {k: _to_device(v, p.device) for k, v in st.items()}
                loaded += 1
            for g, gs in zip(optimizer.param_groups, osd.get("param_groups", [])):
                for k, v in gs.items():
                    if k not in ("params", "param_names"):
                        g[k] = v
            cfg["optimizer_state_loaded"] = loaded
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
