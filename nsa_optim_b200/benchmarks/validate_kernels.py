"""End-to-end kernel validation: the same short training run on the native kernels and on the
PyTorch backend must end at the same loss.

Reference counterpart (nngabe/nsa_optim): benchmarks/validate_kernels.py:21-240 launches three
50-step trainings (baseline / triton / liger) as subprocesses, parses stdout and requires a
final-loss spread below 0.01.  Here both arms run in-process through ``Trainer`` with identical
seeds and data; the check is on the whole loss curve.

    python -m nsa_optim_b200.benchmarks.validate_kernels --steps 50
"""
from __future__ import annotations

import argparse
import json
import statistics
from typing import Dict, List


def run_arm(backend: str, steps: int, extra: List[str]) -> List[float]:
    import torch
    from .. import ops
    from ..train import Trainer, parse_args
    argv = ["--block_pattern", "MDA", "--block_repeats", "1", "--attn_type", "nsa", "--model_size", "100M",
            "--hidden_size", "512", "--vocab_size", "4096", "--intermediate_size", "1536", "--num_heads", "8",
            "--num_kv_heads", "2", "--head_dim", "64", "--mamba_d_state", "128", "--deltanet_head_dim", "128",
            "--deltanet_num_heads", "4", "--nsa_window_size", "128", "--nsa_num_selected_blocks", "4",
            "--context_length", "2048", "--batch_size", "2", "--gradient_accumulation_steps", "1",
            "--optimizer_type", "adamw8bit", "--synthetic_data", "--num_train_steps", str(steps), "--warmup_steps", "5",
            "-lr", "1e-3"] + extra
    losses = []
    with ops.backend(backend):
        torch.manual_seed(0)
        tr = Trainer(parse_args(argv), verbose=False)
        fixed = [tr.make_data().batch_at(i % 4) for i in range(steps)]      # four batches, repeated: the loss falls
        for i in range(steps):
            losses.append(float(tr.step([fixed[i]])["loss"]))
    return losses


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--tolerance", type=float, default=0.05)
    a = ap.parse_args()
    curves: Dict[str, List[float]] = {b: run_arm(b, a.steps, []) for b in ("native", "torch")}
    finals = [c[-1] for c in curves.values()]
    gap = max(abs(x - y) for x, y in zip(curves["native"], curves["torch"]))
    out = {"steps": a.steps, "final_loss": {k: v[-1] for k, v in curves.items()}, "final_loss_std": statistics.pstdev(finals),
           "max_curve_gap": gap, "first_loss": curves["native"][0], "passed": gap < a.tolerance}
    print(json.dumps(out, indent=2))
    raise SystemExit(0 if out["passed"] else 1)


if __name__ == "__main__":
    main()
