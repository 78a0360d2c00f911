"""Stage-by-stage device-memory profile of one training step.

Reference counterpart (nngabe/nsa_optim): profiling/profile_memory.py:14-247 prints allocated /
reserved / peak memory after model creation, after the first layer, after the forward pass and
at the loss, analyses an out-of-memory error when one occurs, and can export a chrome trace.
Here the same stages are reported for any model the trainer can build (same flags as
``train.py``), per block type, and the peak is set against the 180 GB of a B200.

    python -m nsa_optim_b200.profiling.profile_memory --block_pattern MDMA --attn_type nsa \
        --model_size 1B --context_length 65536 --gradient_checkpointing --synthetic_data [--detailed]
"""
from __future__ import annotations

import sys
from typing import Dict, List

import torch


def _gb(x: int) -> float:
    return x / 1e9


def snapshot(label: str, rows: List[Dict]) -> None:
    if torch.cuda.is_available():
        rec = {"stage": label, "allocated_gb": _gb(torch.cuda.memory_allocated()), "reserved_gb": _gb(torch.cuda.memory_reserved()),
               "peak_gb": _gb(torch.cuda.max_memory_allocated())}
    else:
        rec = {"stage": label, "allocated_gb": 0.0, "reserved_gb": 0.0, "peak_gb": 0.0}
    rows.append(rec)
    print(f"{label:<28s} allocated {rec['allocated_gb']:8.2f} GB  reserved {rec['reserved_gb']:8.2f} GB  peak {rec['peak_gb']:8.2f} GB")


def profile(argv=None, detailed: bool = False) -> List[Dict]:
    from ..train import Trainer, parse_args
    argv = list(sys.argv[1:] if argv is None else argv)
    if "--detailed" in argv:
        argv.remove("--detailed")
        detailed = True
    args = parse_args(argv)
    rows: List[Dict] = []
    snapshot("start", rows)
    tr = Trainer(args, verbose=False)
    snapshot("model + optimizer built", rows)
    batch = tr.next_batch()
    model = tr.model.module
    ids = batch["input_ids"].to(tr.device)
    try:
        with torch.no_grad():
            h = model.embed_tokens(ids)
            snapshot("after embedding", rows)
            pos = torch.arange(ids.shape[1], device=tr.device)
            seen = set()
            for layer in model.layers:
                h = layer(h, None, pos) if type(layer).__name__ != "TransformerBlock" else layer(h, None, pos)
                kind = type(layer).__name__
                if kind not in seen:
                    seen.add(kind)
                    snapshot(f"after first {kind}", rows)
            del h
        if torch.cuda.is_available():
            torch.cuda.reset_peak_memory_stats()
        if detailed and torch.cuda.is_available():
            from torch.profiler import ProfilerActivity, profile as tprofile
            with tprofile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA], profile_memory=True, record_shapes=True) as prof:
                tr.step([batch])
            prof.export_chrome_trace("memory_profile_trace.json")
            print("wrote memory_profile_trace.json")
        else:
            tr.step([batch])
        snapshot("after one training step", rows)
    except torch.cuda.OutOfMemoryError as exc:  # type: ignore[attr-defined]
        snapshot("out of memory", rows)
        print(f"OOM: {exc}")
        print("Largest tensors at this scale: logits (tokens x vocab) unless the chunked loss is on; per-block "
              "activations without --gradient_checkpointing; fp32 gradient staging of the sharded runtime.")
    total = torch.cuda.get_device_properties(0).total_memory if torch.cuda.is_available() else 0
    if total:
        print(f"peak {rows[-1]['peak_gb']:.2f} GB of {_gb(total):.0f} GB ({100 * rows[-1]['peak_gb'] / _gb(total):.1f} %)")
    return rows


if __name__ == "__main__":
    profile()
