"""Two real GPUs, one process each: the peer-memory (`--comm fused`) path against the NCCL
path of the same runtime on a tiny hybrid, and both against each other's loss curves."""
import json
import os
import subprocess
import sys
import textwrap

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent("""
    import json, os, sys, torch
    sys.path.insert(0, {root!r})
    from nsa_optim_b200 import ops
    from nsa_optim_b200.train import Trainer, parse_args
    from nsa_optim_b200.parallel import dist as pdist
    out, comm = sys.argv[1], sys.argv[2]
    args = parse_args(["--block_pattern", "MDA", "--block_repeats", "1", "--attn_type", "nsa", "--model_size", "100M",
                       "--hidden_size", "256", "--vocab_size", "1024", "--intermediate_size", "512", "--num_heads", "4",
                       "--num_kv_heads", "2", "--head_dim", "64", "--mamba_d_state", "64", "--deltanet_head_dim", "128",
                       "--deltanet_num_heads", "2", "--nsa_window_size", "64", "--nsa_num_selected_blocks", "4",
                       "--context_length", "512", "--batch_size", "1", "--gradient_accumulation_steps", "2",
                       "--optimizer_type", "adamw8bit", "--synthetic_data", "--num_train_steps", "4", "--warmup_steps", "0",
                       "-lr", "1e-3", "--comm", comm] + sys.argv[3:])
    tr = Trainer(args, verbose=False)
    losses = []
    for i in range(4):
        o = tr.step()
        l = o["loss"].detach().float().clone()
        torch.distributed.all_reduce(l); l /= tr.info.world_size
        losses.append(float(l))
    ops.native_module().check_status()
    if tr.info.rank == 0:
        json.dump({{"losses": losses, "norm": float(o["grad_norm"]), "comm": tr.model.comm_mode}},
                  open(os.path.join(out, f"res_{{comm}}.json"), "w"))
    pdist.cleanup_distributed()
""")


def _run(tmp_path, comm, port, extra=("--gradient_checkpointing",)):
    script = tmp_path / "worker.py"
    script.write_text(WORKER.format(root=ROOT))
    env = dict(os.environ, WANDB_MODE="disabled", NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", str(port), str(script), str(tmp_path), comm, *extra]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    return json.load(open(tmp_path / f"res_{comm}.json"))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_fused_comm_matches_nccl(tmp_path):
    a = _run(tmp_path, "nccl", 29811)
    b = _run(tmp_path, "fused", 29813)
    assert a["comm"] == "torch" and b["comm"] == "fused"
    for x, y in zip(a["losses"], b["losses"]):
        assert abs(x - y) < 3e-2, (a, b)
    assert abs(a["norm"] - b["norm"]) < 5e-2 * max(1.0, a["norm"])


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_fused_comm_under_gradient_accumulation_without_recompute(tmp_path):
    """Two micro-batches per step, fully sharded, nothing recomputed: every block is gathered by its
    first GEMM twice within one epoch, so the per-chunk flags of the first gather must not satisfy
    the second one (which reads a freshly allocated buffer)."""
    import math
    a = _run(tmp_path, "nccl", 29815, extra=("--block_pattern", "DADA"))
    b = _run(tmp_path, "fused", 29817, extra=("--block_pattern", "DADA"))
    assert b["comm"] == "fused" and all(math.isfinite(x) for x in b["losses"])
    for x, y in zip(a["losses"], b["losses"]):
        assert abs(x - y) < 3e-2, (a, b)
