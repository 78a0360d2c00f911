"""Mamba-2 block against the experimental Mamba-3 block: forward / backward time, tokens per
second and peak memory at several sequence lengths.

Reference counterpart (nngabe/nsa_optim): benchmarks/profile_mamba.py:23-214 (8K / 32K / 128K,
wall-clock).  Timed here with CUDA events after warm-up; Mamba-3 is forward only, as its kernel is.

    python -m nsa_optim_b200.benchmarks.profile_mamba --seq_lens 8192 32768
"""
from __future__ import annotations

import argparse
import json

import torch

from .kernel_benchmark import time_ms as time_cuda


def profile_block(kind: str, d_model: int, seq_len: int, batch: int = 1) -> dict:
    from ..models.mamba import Mamba2Mixer, Mamba3Block
    torch.cuda.reset_peak_memory_stats()
    if kind == "mamba2":
        blk = Mamba2Mixer(d_model, d_state=128, d_conv=4, expand=2, headdim=64).cuda().bfloat16()
    else:
        blk = Mamba3Block(d_model, d_state=128, expand=2, headdim=64).cuda().bfloat16()
    x = torch.randn(batch, seq_len, d_model, device="cuda", dtype=torch.bfloat16, requires_grad=(kind == "mamba2"))
    out = {"block": kind, "seq_len": seq_len, "d_model": d_model}
    with torch.no_grad():
        out["fwd_ms"] = time_cuda(lambda: blk(x), iters=5, warmup=2)
    if kind == "mamba2":
        def fb():
            blk(x).float().sum().backward()
        out["fwd_bwd_ms"] = time_cuda(fb, iters=5, warmup=2)
        out["tokens_per_s"] = batch * seq_len / out["fwd_bwd_ms"] * 1e3
    else:
        out["tokens_per_s_fwd"] = batch * seq_len / out["fwd_ms"] * 1e3
    out["peak_gb"] = torch.cuda.max_memory_allocated() / 2**30
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--seq_lens", type=int, nargs="*", default=[8192, 32768, 131072])
    ap.add_argument("--d_model", type=int, default=2048)
    ap.add_argument("--skip_mamba3", action="store_true")
    a = ap.parse_args()
    for L in a.seq_lens:
        print(json.dumps(profile_block("mamba2", a.d_model, L)))
        if not a.skip_mamba3:
            print(json.dumps(profile_block("mamba3", a.d_model, L)))


if __name__ == "__main__":
    main()
