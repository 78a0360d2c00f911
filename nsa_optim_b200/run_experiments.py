"""Experiment orchestration: manifest, per-experiment launch scripts, SLURM scripts, local runs,
resource estimates.

Reference counterpart (nngabe/nsa_optim): run_experiments.py:30-433 (modes generate | run |
slurm).  The reference file still uses enum fields that its config module dropped
(``config.model_size.value``, ``--attention_type``); this version is written against the
current configuration API and the flags ``train.py`` really accepts, and estimates memory
against a 180 GB B200 instead of an 80 GB A100.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
from typing import Dict, List, Optional

from .config import (AttentionType, OptimizerType, TrainingConfig, compute_model_dimensions, compute_transformer_params,
                     get_filtered_experiments, parse_model_size)

GPU_MEMORY_GB = 180.0


def experiment_command(cfg: TrainingConfig, n_gpus: int = 8, output_dir: str = "./outputs", synthetic: bool = False,
                       extra: Optional[List[str]] = None) -> List[str]:
    attn = {AttentionType.DENSE: "dense", AttentionType.NSA: "nsa", AttentionType.FSA: "fsa"}[cfg.attention_type]
    cmd = ["torchrun", "--standalone", "--local-addr", "127.0.0.1", f"--nproc_per_node={n_gpus}", "train.py",
           "--mamba_type", cfg.mamba_type.value if cfg.mamba_type.value != "mamba3" else "deltanet",
           "--attn_type", attn, "--model_size", cfg.model_size, "--optimizer_type", cfg.optimizer_type.value,
           "--context_length", str(cfg.max_seq_length), "--batch_size", str(cfg.batch_size),
           "--gradient_accumulation_steps", str(cfg.gradient_accumulation_steps),
           "--num_train_steps", str(cfg.num_train_steps), "--warmup_steps", str(cfg.warmup_steps),
           "--learning_rate", str(cfg.optimizer_config.learning_rate), "--weight_decay", str(cfg.optimizer_config.weight_decay),
           "--max_grad_norm", str(cfg.max_grad_norm), "--dtype", cfg.dtype, "--output_dir", output_dir,
           "--run_name", cfg.run_name, "--log_interval", str(cfg.log_interval), "--save_interval", str(cfg.save_interval)]
    if cfg.gradient_checkpointing:
        cmd.append("--gradient_checkpointing")
    if synthetic:
        cmd.append("--synthetic_data")
    return cmd + list(extra or [])


def estimate_resources(cfg: TrainingConfig, n_gpus: int = 8) -> Dict[str, float]:
    """Rough per-GPU memory (GB) under full sharding with per-block checkpointing, and GPU hours."""
    n = parse_model_size(cfg.model_size)
    width, depth, _, kv, _ = compute_model_dimensions(n)
    n_actual = compute_transformer_params(width, depth, kv)
    state_bytes = {"adamw": 8, "adamw8bit": 2, "adamw4bit": 1, "soap": 12, "soap4bit": 3, "soap8bit": 4, "shampoo": 10}
    per_param = 2 + 4 + state_bytes.get(cfg.optimizer_type.value, 8)          # bf16 weight + fp32 grad + state
    sharded = n_actual * per_param / n_gpus / 1e9
    gathered = n_actual * 2 / 1e9                                             # gathered bf16 copy kept per rank
    tokens = cfg.batch_size * cfg.max_seq_length
    acts = tokens * width * 2 * (depth + 12) / 1e9                            # block inputs + one live block
    total = sharded + gathered + acts
    tok_s_per_gpu = 3.0e4 * (1.1e9 / max(n_actual, 1))                        # measured 1B hybrid rate, scaled by size
    hours = cfg.num_train_steps * tokens * cfg.gradient_accumulation_steps / tok_s_per_gpu / 3600
    return {"params_b": n_actual / 1e9, "memory_gb_per_gpu": total, "fits": total < 0.9 * GPU_MEMORY_GB,
            "gpu_hours_total": hours * n_gpus, "wall_hours": hours}


def generate_experiment_manifest(experiments: List[TrainingConfig], path: str, n_gpus: int = 8) -> Dict:
    manifest = {"num_experiments": len(experiments), "n_gpus": n_gpus, "experiments": []}
    for i, cfg in enumerate(experiments):
        manifest["experiments"].append({
            "id": i, "run_name": cfg.run_name, "model_size": cfg.model_size, "attention_type": cfg.attention_type.value,
            "optimizer_type": cfg.optimizer_type.value, "context_length": cfg.max_seq_length, "batch_size": cfg.batch_size,
            "gradient_accumulation_steps": cfg.gradient_accumulation_steps, "num_train_steps": cfg.num_train_steps,
            "command": " ".join(experiment_command(cfg, n_gpus)), "resources": estimate_resources(cfg, n_gpus)})
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    with open(path, "w") as f:
        json.dump(manifest, f, indent=2)
    return manifest


def write_bash_script(cfg: TrainingConfig, script_dir: str, n_gpus: int = 8, synthetic: bool = False) -> str:
    os.makedirs(script_dir, exist_ok=True)
    path = os.path.join(script_dir, f"{cfg.run_name}.sh")
    with open(path, "w") as f:
        f.write("#!/bin/bash\nset -euo pipefail\nexport WANDB_MODE=${WANDB_MODE:-offline}\n")
        f.write(" ".join(experiment_command(cfg, n_gpus, synthetic=synthetic)) + "\n")
    os.chmod(path, 0o755)
    return path


def write_slurm_script(cfg: TrainingConfig, script_dir: str, n_gpus: int = 8, partition: str = "gpu", hours: int = 48) -> str:
    os.makedirs(script_dir, exist_ok=True)
    path = os.path.join(script_dir, f"{cfg.run_name}.slurm")
    with open(path, "w") as f:
        f.write(f"#!/bin/bash\n#SBATCH --job-name={cfg.run_name}\n#SBATCH --partition={partition}\n#SBATCH --nodes=1\n"
                f"#SBATCH --gres=gpu:{n_gpus}\n#SBATCH --time={hours}:00:00\n#SBATCH --output=logs/{cfg.run_name}_%j.out\n\n")
        f.write(" ".join(experiment_command(cfg, n_gpus)) + "\n")
    return path


def run_experiments_locally(experiments: List[TrainingConfig], script_dir: str, n_gpus: int = 8, dry_run: bool = False,
                            synthetic: bool = False) -> List[Dict]:
    results = []
    for cfg in experiments:
        script = write_bash_script(cfg, script_dir, n_gpus, synthetic)
        if dry_run:
            results.append({"run_name": cfg.run_name, "script": script, "returncode": None})
            continue
        r = subprocess.run(["bash", script])
        results.append({"run_name": cfg.run_name, "script": script, "returncode": r.returncode})
    return results


def main(argv: Optional[List[str]] = None) -> None:
    ap = argparse.ArgumentParser(description="Generate or run the ablation experiment grid")
    ap.add_argument("--mode", choices=["generate", "run", "slurm"], default="generate")
    ap.add_argument("--model_sizes", nargs="*", default=None)
    ap.add_argument("--attention_types", nargs="*", default=None, choices=[a.value for a in AttentionType] + ["nsa", "fsa"])
    ap.add_argument("--optimizer_types", nargs="*", default=None, choices=[o.value for o in OptimizerType])
    ap.add_argument("--context_lengths", nargs="*", type=int, default=None)
    ap.add_argument("--n_gpus", type=int, default=8)
    ap.add_argument("--output", default="./experiments")
    ap.add_argument("--dry_run", action="store_true")
    ap.add_argument("--synthetic_data", action="store_true")
    a = ap.parse_args(argv)
    from .config import resolve_attention_type
    exps = get_filtered_experiments(
        a.model_sizes, [resolve_attention_type(x) for x in a.attention_types] if a.attention_types else None,
        [OptimizerType(o) for o in a.optimizer_types] if a.optimizer_types else None, a.context_lengths)
    print(f"{len(exps)} experiments selected")
    manifest = generate_experiment_manifest(exps, os.path.join(a.output, "manifest.json"), a.n_gpus)
    if a.mode == "generate":
        for cfg in exps:
            write_bash_script(cfg, os.path.join(a.output, "scripts"), a.n_gpus, a.synthetic_data)
    elif a.mode == "slurm":
        for cfg in exps:
            write_slurm_script(cfg, os.path.join(a.output, "slurm"), a.n_gpus)
    else:
        res = run_experiments_locally(exps, os.path.join(a.output, "scripts"), a.n_gpus, a.dry_run, a.synthetic_data)
        print(json.dumps(res, indent=2))
    gpu_h = sum(e["resources"]["gpu_hours_total"] for e in manifest["experiments"])
    print(f"manifest: {os.path.join(a.output, 'manifest.json')}  (estimated {gpu_h:.0f} GPU-hours)")


if __name__ == "__main__":
    main()
