"""Device time of one training step by kernel (torch.profiler, CUDA activities only).

    python -m nsa_optim_b200.profiling.profile_step [--top 40] [training flags ...]

Builds a ``Trainer`` from the usual training flags (default: the 1B MDMA-NSA hybrid at 64K context
with 8-bit AdamW), runs warm-up steps, profiles one step and prints the kernels sorted by total
device time together with the split forward+backward / clipping / optimizer.  The times are
device durations of the individual kernels; their sum can differ from the step's wall time by
the gaps between launches.
"""
from __future__ import annotations

import argparse
import sys
from typing import List


def default_flags() -> List[str]:
    return ["--block_pattern", "MDMA", "--block_repeats", "4", "--attn_type", "nsa", "--model_size", "1B",
            "--hidden_size", "2048", "--vocab_size", "32000", "--intermediate_size", "5632", "--num_heads", "32",
            "--num_kv_heads", "2", "--head_dim", "128", "--nsa_block_size", "64", "--nsa_num_selected_blocks", "16",
            "--nsa_window_size", "512", "--deltanet_head_dim", "128", "--deltanet_num_heads", "16",
            "--context_length", "65536", "--batch_size", "1", "--gradient_accumulation_steps", "1",
            "--optimizer_type", "adamw8bit", "--dtype", "bfloat16", "--synthetic_data", "-clip", "1.0"]


def main() -> None:
    ap = argparse.ArgumentParser(add_help=False)
    ap.add_argument("--top", type=int, default=40)
    ap.add_argument("--warmup", type=int, default=2)
    a, rest = ap.parse_known_args()
    import torch
    from torch.profiler import ProfilerActivity, profile

    from ..train import Trainer, parse_args
    tr = Trainer(parse_args(rest or default_flags()), verbose=False)
    data = tr.make_data()
    batch = {k: v.to(tr.device) for k, v in data.batch_at(0).items()}
    for _ in range(a.warmup):
        tr.step([batch])
    torch.cuda.synchronize()

    def mark():
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        return e

    e0 = mark()
    tr.micro_step(batch)
    e1 = mark()
    _, coef = tr.model.clip_grad_norm(tr.cfg.max_grad_norm)
    e2 = mark()
    tr.optimizer.step(grad_scale=coef)
    e3 = mark()
    tr.model.zero_grad(set_to_none=True)
    torch.cuda.synchronize()
    print(f"forward+backward {e0.elapsed_time(e1):.1f} ms | clip {e1.elapsed_time(e2):.1f} ms | "
          f"optimizer {e2.elapsed_time(e3):.1f} ms")
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        tr.step([batch])
        torch.cuda.synchronize()
    rows = sorted(((e.self_device_time_total / 1e3, e.count, e.key) for e in prof.key_averages()
                   if e.self_device_time_total > 0), reverse=True)
    total = sum(r[0] for r in rows)
    print(f"kernels: {sum(r[1] for r in rows)} launches, {total:.1f} ms device time")
    for ms, n, name in rows[:a.top]:
        print(f"{ms:9.2f} ms {100 * ms / total:5.1f}% x{n:5d}  {name[:100]}")


if __name__ == "__main__":
    main()
