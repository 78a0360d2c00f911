"""Sharded runtime: layout arithmetic, 1-vs-2-rank equality on gloo, checkpoint round trip,
rank-failure detection.  All on CPU; multi-rank cases run as child processes."""
import json
import os
import subprocess
import sys
import textwrap

import pytest
import torch

from nsa_optim_b200.models import HybridConfig, create_hybrid_model
from nsa_optim_b200.parallel.dist import DistInfo
from nsa_optim_b200.parallel.sharded import ALIGN, FlatUnit, ShardedModel, ShardingStrategy

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def tiny(ckpt=False):
    torch.manual_seed(0)
    return create_hybrid_model(HybridConfig(d_model=64, vocab_size=128, block_pattern="MDA", block_repeats=1,
                                            mamba_d_state=16, mamba_headdim=16, mamba_chunk=16, deltanet_head_dim=16,
                                            num_attention_heads=4, num_key_value_heads=2, rope_theta=1e4,
                                            intermediate_size=128, gradient_checkpointing=ckpt))


def test_flat_layout_alignment_and_coverage():
    ps = [("a", torch.nn.Parameter(torch.randn(10, 30))), ("b", torch.nn.Parameter(torch.randn(7))),
          ("c", torch.nn.Parameter(torch.randn(300, 3)))]
    world = 4
    units = [FlatUnit("u", None, [(n, torch.nn.Parameter(p.detach().clone())) for n, p in ps], world, r,
                      torch.device("cpu"), torch.float32) for r in range(world)]
    u0 = units[0]
    assert all(s.offset % ALIGN == 0 for s in u0.slots) and u0.total % (world * ALIGN) == 0
    # every logical element is owned by exactly one rank's piece
    owned = {n: 0 for n, _ in ps}
    for u in units:
        for name, piece in u.pieces:
            s = next(s for s in u.slots if s.name == name)
            lo = u.rank * u.shard_size
            a = max(lo, s.offset)
            owned[name] += min(piece.numel(), s.offset + s.numel - a)
    assert owned == {"a": 300, "b": 7, "c": 900}
    # gather(scatter(x)) == x
    full = torch.cat([u.shard for u in units])
    for s in u0.slots:
        assert torch.equal(full[s.offset:s.offset + s.numel].view(s.shape), dict(ps)[s.name].detach())


def test_world1_matches_plain_model():
    ids = torch.randint(0, 128, (2, 32))
    plain = tiny()
    plain(ids, labels=ids)[1].backward()
    ref = {n: p.grad.clone() for n, p in plain.named_parameters()}
    for ckpt in (False, True):
        sm = ShardedModel(tiny(ckpt), DistInfo())
        assert sm.strategy == ShardingStrategy.NO_SHARD
        _, loss, _ = sm(input_ids=ids, labels=ids)
        sm.backward(loss)
        for n, p in sm.module.named_parameters():
            assert torch.allclose(p.grad, ref[n], atol=1e-5), n
        norm, coef = sm.clip_grad_norm(1.0)
        expect = torch.sqrt(sum(g.pow(2).sum() for g in ref.values()))
        assert torch.allclose(norm, expect, atol=1e-4) and coef <= 1.0
        sm.zero_grad()


WORKER = textwrap.dedent("""
    import json, os, sys, torch
    sys.path.insert(0, {root!r})
    from nsa_optim_b200.train import Trainer, parse_args
    from nsa_optim_b200.parallel import dist as pdist
    mode = sys.argv[1]
    out = sys.argv[2]
    base = ["--block_pattern", "MDMA", "--block_repeats", "1", "--model_size", "100M", "--hidden_size", "64",
            "--vocab_size", "256", "--num_heads", "4", "--num_kv_heads", "2", "--mamba_d_state", "16", "--mamba_headdim", "16",
            "--deltanet_head_dim", "16", "--intermediate_size", "128", "--tie_embeddings", "--rope_theta", "1e4",
            "--context_length", "64", "--batch_size", "2", "--gradient_accumulation_steps", "1", "--num_train_steps", "4",
            "--warmup_steps", "0", "-lr", "3e-3", "--dtype", "float32", "--synthetic_data", "--device", "cpu",
            "--output_dir", out] + sys.argv[3:]
    args = parse_args(base)
    tr = Trainer(args, verbose=False)
    world, rank = tr.info.world_size, tr.info.rank
    data = tr.make_data()
    # both world sizes see the same global batch: rank r takes rows of the 4-sequence batch
    full = [type(data)(256, 64, 4, 0, 0).batch_at(i) for i in range(8)]
    def mine(b):
        per = 4 // world
        return {{k: v[rank * per:(rank + 1) * per] for k, v in b.items()}}
    losses = []
    if mode == "train":
        tr.cfg.batch_size = 4 // world
        for i in range(4):
            o = tr.step([mine(full[i])])
            l = o["loss"].detach().clone()
            if world > 1:
                torch.distributed.all_reduce(l); l /= world
            losses.append(float(l))
        wsq = sum(float(v.double().pow(2).sum()) for v in tr.model.state_dict(rank0_only=False).values())
        if rank == 0:
            json.dump({{"losses": losses, "norm": float(o["grad_norm"]), "wsq": wsq}},
                      open(os.path.join(out, f"res_w{{world}}.json"), "w"))
    elif mode == "save2":
        tr.cfg.batch_size = 4 // world
        for i in range(2):
            tr.step([mine(full[i])])
        tr.save()
    elif mode == "continue":
        tr.cfg.batch_size = 4 // world
        ckpt = os.path.join(out, tr.cfg.run_name, "checkpoint-2")
        assert tr.resume(ckpt) == 2
        n_state = sum(1 for p in tr.optimizer.state.values() if p)
        for i in range(2, 4):
            o = tr.step([mine(full[i])])
            l = o["loss"].detach().clone()
            if world > 1:
                torch.distributed.all_reduce(l); l /= world
            losses.append(float(l))
        if rank == 0:
            json.dump({{"losses": losses, "n_state": n_state}}, open(os.path.join(out, f"cont_w{{world}}.json"), "w"))
    elif mode == "resume":
        for i in range(2):
            tr.step([mine(full[i])])
        path = tr.save()
        for i in range(2, 4):
            o = tr.step([mine(full[i])])
        a = float(o["loss"])
        tr2 = Trainer(args, verbose=False, info=tr.info)
        step = tr2.resume(path)
        assert step == 2, step
        for i in range(2, 4):
            o = tr2.step([mine(full[i])])
        b = float(o["loss"])
        if rank == 0:
            json.dump({{"a": a, "b": b}}, open(os.path.join(out, f"resume_w{{world}}.json"), "w"))
    pdist.cleanup_distributed()
""")


def run_ranks(tmp_path, world, mode, extra=(), port=29731):
    script = tmp_path / "worker.py"
    script.write_text(WORKER.format(root=ROOT))
    env = dict(os.environ, WANDB_MODE="disabled", OMP_NUM_THREADS="2")
    if world == 1:
        cmd = [sys.executable, str(script), mode, str(tmp_path), *extra]
    else:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
               "--master-addr", "127.0.0.1", "--master-port", str(port), str(script), mode, str(tmp_path), *extra]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]


@pytest.mark.parametrize("opt,extra", [("adamw", ()), ("adamw8bit", ("--gradient_checkpointing",)),
                                       ("adamw", ("--sharding", "full_shard")),
                                       ("adamw", ("--sharding", "full_shard", "--gradient_checkpointing",
                                                  "--checkpoint_blocks", "M")),
                                       # whole-matrix optimizers: matrices cut by a shard boundary go to one
                                       # owner rank, so two ranks precondition exactly what one rank does
                                       ("soap", ("--precondition_frequency", "2")),
                                       ("shampoo", ("--precondition_frequency", "2"))])
def test_two_ranks_match_one_rank(tmp_path, opt, extra):
    args = ("--optimizer_type", opt) + tuple(extra)
    run_ranks(tmp_path, 1, "train", args)
    run_ranks(tmp_path, 2, "train", args, port=29733)
    r1 = json.load(open(tmp_path / "res_w1.json"))
    r2 = json.load(open(tmp_path / "res_w2.json"))
    tol = 2e-3 if opt in ("adamw8bit", "soap", "shampoo") else 2e-4
    for a, b in zip(r1["losses"], r2["losses"]):
        assert abs(a - b) < tol, (r1, r2)
    assert abs(r1["norm"] - r2["norm"]) < 1e-2 * max(1.0, r1["norm"])


def test_weight_decay_reaches_matrices_under_sharding(tmp_path):
    """Shard pieces are 1-D views; the decay / no-decay split must follow the original parameter."""
    from nsa_optim_b200.optimizers import get_param_groups
    ps = [("w", torch.nn.Parameter(torch.randn(512, 512))), ("norm.weight", torch.nn.Parameter(torch.ones(512)))]
    for world in (1, 2):
        u = FlatUnit("u", None, [(n, torch.nn.Parameter(p.detach().clone())) for n, p in ps], world, 0,
                     torch.device("cpu"), torch.float32)
        decay, no_decay = get_param_groups(u.pieces, 0.1)
        assert decay["param_names"] == ["w"] and no_decay["param_names"] == ["norm.weight"], world
    # and end to end: with a large decay the weights of a 2-rank run shrink as in the 1-rank run
    args = ("--optimizer_type", "adamw", "-wd", "3.0")
    run_ranks(tmp_path, 1, "train", args)
    run_ranks(tmp_path, 2, "train", args, port=29747)
    r1 = json.load(open(tmp_path / "res_w1.json"))
    r2 = json.load(open(tmp_path / "res_w2.json"))
    assert abs(r1["wsq"] - r2["wsq"]) < 1e-3 * r1["wsq"], (r1["wsq"], r2["wsq"])


@pytest.mark.parametrize("opt,save_world,load_world", [("adamw", 2, 1), ("adamw8bit", 2, 1), ("adamw8bit", 1, 2)])
def test_resume_at_another_world_size(tmp_path, opt, save_world, load_world):
    """optimizer.pt is sharding-independent: a run saved at one world size continues at another
    with the moments it had (compared against an uninterrupted run)."""
    args = ("--optimizer_type", opt)
    run_ranks(tmp_path, 1, "train", args)
    run_ranks(tmp_path, save_world, "save2", args, port=29751)
    run_ranks(tmp_path, load_world, "continue", args, port=29753)
    ref = json.load(open(tmp_path / "res_w1.json"))["losses"]
    got = json.load(open(tmp_path / f"cont_w{load_world}.json"))
    assert got["n_state"] > 0
    tol = 3e-3 if opt == "adamw8bit" else 3e-4
    for a, b in zip(ref[2:], got["losses"]):
        assert abs(a - b) < tol, (ref, got)


def test_checkpoint_of_another_layout_is_not_attached(tmp_path):
    """A state whose tensors do not have the size the kernels will index is refused."""
    from nsa_optim_b200.optimizers import AdamWLowBit, state_fits
    p = torch.nn.Parameter(torch.zeros(8192))
    opt = AdamWLowBit([p])
    good = {}
    opt._init(p, good)
    assert state_fits(opt, p, good)
    half = {k: (v[: v.numel() // 2] if torch.is_tensor(v) else v) for k, v in good.items()}
    assert not state_fits(opt, p, half)


@pytest.mark.parametrize("world", [1, 2])
def test_checkpoint_resume_reproduces_loss(tmp_path, world):
    run_ranks(tmp_path, world, "resume", ("--optimizer_type", "adamw8bit"), port=29735 + world)
    r = json.load(open(tmp_path / f"resume_w{world}.json"))
    assert abs(r["a"] - r["b"]) < 1e-5, r


FAIL_WORKER = textwrap.dedent("""
    import os, sys, time, datetime, torch, torch.distributed as dist
    rank = int(os.environ["RANK"])
    dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=5))
    t = torch.ones(4)
    dist.all_reduce(t)                      # step 0: everyone is alive
    if rank == 1:
        os._exit(17)                        # leaves between steps, nothing in flight
    try:
        dist.all_reduce(t)                  # step 1: the peer is gone
        print("NO_ERROR")
    except Exception as e:
        print("DETECTED", type(e).__name__)
        sys.exit(3)
""")


def test_rank_failure_is_detected_by_survivor(tmp_path):
    script = tmp_path / "fail.py"
    script.write_text(FAIL_WORKER)
    procs = []
    for r in range(2):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT="29741")
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE, text=True))
    out0, _ = procs[0].communicate(timeout=120)
    procs[1].wait(timeout=120)
    assert procs[1].returncode == 17
    assert "DETECTED" in out0 and procs[0].returncode == 3, out0
