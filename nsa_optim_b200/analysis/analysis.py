"""Analysis of finished runs.

Reference counterpart (nngabe/nsa_optim): analysis/analysis.py:23-456 scans
``checkpoint-*/config.json`` plus optional ``metrics.json`` / ``training_log.jsonl`` (files the
reference trainer never writes), groups results, writes a JSON report, plots curves and evaluates
checkpoints.  This trainer does write ``training_log.jsonl`` and ``metrics.json`` in the run
directory, so every function here works on real output.

    python -m nsa_optim_b200.analysis.analysis --output_dir ./outputs [--plot]
"""
from __future__ import annotations

import argparse
import glob
import json
import os
import statistics
from dataclasses import asdict, dataclass, field
from typing import Any, Callable, Dict, List, Optional


@dataclass
class ExperimentResult:
    run_name: str
    path: str
    model_type: str = ""
    model_size: str = ""
    attention_type: str = ""
    optimizer_type: str = ""
    context_length: int = 0
    step: int = 0
    final_loss: Optional[float] = None
    tokens_per_sec: Optional[float] = None
    total_tokens: Optional[int] = None
    history: List[Dict[str, Any]] = field(default_factory=list)


def _latest_checkpoint(run_dir: str) -> Optional[str]:
    cks = glob.glob(os.path.join(run_dir, "checkpoint-*"))
    cks = [c for c in cks if os.path.exists(os.path.join(c, "config.json"))]
    return max(cks, key=lambda c: int(c.rsplit("-", 1)[1])) if cks else None


def load_experiment_results(output_dir: str) -> List[ExperimentResult]:
    results = []
    for run_dir in sorted(glob.glob(os.path.join(output_dir, "*"))):
        if not os.path.isdir(run_dir):
            continue
        ck = _latest_checkpoint(run_dir)
        if ck is None:
            continue
        with open(os.path.join(ck, "config.json")) as f:
            cfg = json.load(f)
        res = ExperimentResult(run_name=os.path.basename(run_dir), path=run_dir, model_type=cfg.get("model_type", ""),
                               model_size=str(cfg.get("model_size", "")), attention_type=cfg.get("attention_type", ""),
                               optimizer_type=cfg.get("optimizer_type", ""), context_length=int(cfg.get("max_seq_length", 0)),
                               step=int(cfg.get("step", 0)))
        log = os.path.join(run_dir, "training_log.jsonl")
        if os.path.exists(log):
            with open(log) as f:
                res.history = [json.loads(line) for line in f if line.strip()]
        metrics = os.path.join(run_dir, "metrics.json")
        if os.path.exists(metrics):
            with open(metrics) as f:
                m = json.load(f)
            res.final_loss, res.tokens_per_sec, res.total_tokens = m.get("final_loss"), m.get("tokens_per_sec"), m.get("total_tokens")
        elif res.history:
            res.final_loss, res.tokens_per_sec = res.history[-1].get("loss"), res.history[-1].get("tokens_per_sec")
        results.append(res)
    return results


def _group(results: List[ExperimentResult], key: Callable[[ExperimentResult], Any]) -> Dict[Any, Dict[str, Any]]:
    groups: Dict[Any, List[ExperimentResult]] = {}
    for r in results:
        groups.setdefault(key(r), []).append(r)
    out = {}
    for k, rs in groups.items():
        losses = [r.final_loss for r in rs if r.final_loss is not None]
        tps = [r.tokens_per_sec for r in rs if r.tokens_per_sec]
        out[k] = {"runs": len(rs), "mean_final_loss": statistics.mean(losses) if losses else None,
                  "best_final_loss": min(losses) if losses else None,
                  "std_final_loss": statistics.pstdev(losses) if len(losses) > 1 else 0.0,
                  "mean_tokens_per_sec": statistics.mean(tps) if tps else None, "run_names": [r.run_name for r in rs]}
    return out


def compare_optimizers(results):
    return _group(results, lambda r: r.optimizer_type)


def compare_attention_types(results):
    return _group(results, lambda r: r.attention_type)


def compare_context_lengths(results):
    return _group(results, lambda r: r.context_length)


def generate_report(results: List[ExperimentResult], path: Optional[str] = None) -> Dict[str, Any]:
    report = {"num_runs": len(results), "by_optimizer": compare_optimizers(results),
              "by_attention": compare_attention_types(results),
              "by_context_length": {str(k): v for k, v in compare_context_lengths(results).items()},
              "runs": [{k: v for k, v in asdict(r).items() if k != "history"} for r in results]}
    if path:
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        with open(path, "w") as f:
            json.dump(report, f, indent=2)
    return report


def plot_training_curves(results: List[ExperimentResult], path: str, key: str = "loss") -> Optional[str]:
    """Loss (or any logged key) against tokens, one line per run.  Needs matplotlib."""
    try:
        import matplotlib
        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
    except ImportError:
        return None
    fig, ax = plt.subplots(figsize=(9, 5))
    for r in results:
        if r.history:
            ax.plot([h.get("tokens", h["step"]) for h in r.history], [h.get(key) for h in r.history], label=r.run_name)
    ax.set_xlabel("tokens")
    ax.set_ylabel(key)
    ax.legend(fontsize=6)
    fig.savefig(path, dpi=150, bbox_inches="tight")
    plt.close(fig)
    return path


def evaluate_model(checkpoint_dir: str, argv: List[str], batches: int = 8) -> Dict[str, float]:
    """Rebuild the model from training flags ``argv``, load ``checkpoint_dir`` and report loss and
    perplexity on seeded synthetic batches (an offline stand-in for a held-out text set)."""
    import torch
    from ..checkpoint import load_checkpoint
    from ..data import create_synthetic_loader
    from ..train import Trainer, evaluate, parse_args
    args = parse_args(argv)
    tr = Trainer(args, verbose=False)
    load_checkpoint(checkpoint_dir, tr.model, None, None, tr.info.rank)
    data = create_synthetic_loader(tr.vocab_size(), tr.cfg.max_seq_length, tr.cfg.batch_size, seed=12345, rank=tr.info.rank)
    with torch.no_grad():
        return evaluate(tr.model, data, tr.device, batches)


def main(argv: Optional[List[str]] = None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--output_dir", default="./outputs")
    ap.add_argument("--report", default=None)
    ap.add_argument("--plot", action="store_true")
    a = ap.parse_args(argv)
    results = load_experiment_results(a.output_dir)
    report = generate_report(results, a.report or os.path.join(a.output_dir, "analysis_report.json"))
    print(json.dumps({k: v for k, v in report.items() if k != "runs"}, indent=2))
    if a.plot:
        print(plot_training_curves(results, os.path.join(a.output_dir, "training_curves.png")))


if __name__ == "__main__":
    main()
