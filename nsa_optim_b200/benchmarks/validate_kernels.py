"""End-to-end kernel validation: the same short training run on the native kernels and on the
PyTorch backend must end at the same loss.

Reference counterpart (nngabe/nsa_optim): benchmarks/validate_kernels.py:21-240 launches three
50-step trainings (baseline / triton / liger) as subprocesses, parses stdout and requires a
final-loss spread below 0.01.  Here both arms run in-process through ``Trainer`` with identical
seeds and data; the check is on the whole loss curve.

    python -m nsa_optim_b200.benchmarks.validate_kernels --steps 50 [--out curves.json]

Under ``torch.distributed.run`` with more than one rank the two arms are instead the two
collective paths of the sharded runtime on the native kernels: NCCL (``--comm nccl``) and the
peer-memory kernels (``--comm fused``), same seeds, same data:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        --master-port 29500 -m nsa_optim_b200.benchmarks.validate_kernels --steps 200 --out curves.json
"""
from __future__ import annotations

import argparse
import json
import statistics
from typing import Dict, List


def run_arm(backend: str, steps: int, extra: List[str], info=None) -> List[float]:
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
        tr = Trainer(parse_args(argv), verbose=False, info=info)
        fixed = [tr.make_data().batch_at(i % 4) for i in range(steps)]      # four batches, repeated: the loss falls
        for i in range(steps):
            loss = tr.step([fixed[i]])["loss"].detach().float().clone()
            if tr.info.world_size > 1:
                torch.distributed.all_reduce(loss)
                loss /= tr.info.world_size
            losses.append(float(loss))
        if tr.device.type == "cuda" and backend != "torch":
            ops.native_module().check_status()
    return losses


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--tolerance", type=float, default=0.05)
    ap.add_argument("--out", default=None, help="write the summary and both loss curves to this JSON file")
    a = ap.parse_args()
    import os
    world = int(os.environ.get("WORLD_SIZE", 1))
    if world > 1:
        from ..parallel import dist as pdist
        info = pdist.setup_distributed()
        arms = {"nccl": ("native", ["--comm", "nccl"]), "fused": ("native", ["--comm", "fused"])}
        curves: Dict[str, List[float]] = {k: run_arm(b, a.steps, extra, info) for k, (b, extra) in arms.items()}
        main_rank = info.is_main
    else:
        curves = {b: run_arm(b, a.steps, []) for b in ("native", "torch")}
        main_rank = True
    (ka, ca), (kb, cb) = list(curves.items())
    finals = [c[-1] for c in curves.values()]
    gap = max(abs(x - y) for x, y in zip(ca, cb))
    out = {"arms": [ka, kb], "world_size": world, "steps": a.steps, "final_loss": {k: v[-1] for k, v in curves.items()},
           "final_loss_std": statistics.pstdev(finals), "max_curve_gap": gap, "first_loss": ca[0],
           "loss_fell_by": ca[0] - ca[-1], "passed": gap < a.tolerance}
    if main_rank:
        print(json.dumps(out, indent=2))
        if a.out:
            with open(a.out, "w") as f:
                json.dump(dict(out, curves={k: [round(x, 5) for x in v] for k, v in curves.items()}), f)
    if world > 1:
        pdist.cleanup_distributed()
    raise SystemExit(0 if out["passed"] else 1)


if __name__ == "__main__":
    main()
