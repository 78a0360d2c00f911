"""Host-side tools: data packer, CLI, checkpoint layout, experiment runner, analysis, FLOP model."""
import json
import os

import pytest
import torch

from nsa_optim_b200.config import AttentionType, ModelConfig, OptimizerType, TrainingConfig, get_filtered_experiments
from nsa_optim_b200.data import DataConfig, PackedDataset, SyntheticTokens, TokenizedDataset, collate_fn, create_dataloader


class FakeTok:
    bos_token_id, eos_token_id, pad_token_id = 1, 2, 0

    def encode(self, text, add_special_tokens=False):
        ids = [10 + (ord(c) % 50) for c in text]
        return ([self.bos_token_id] + ids + [self.eos_token_id]) if add_special_tokens else ids


def test_packed_dataset_packs_and_pads():
    docs = [{"text": "a" * 5}, {"text": "b" * 6}, {"text": "c" * 30}, {"text": "d" * 3}]
    ds = PackedDataset(DataConfig(max_seq_length=16), FakeTok(), dataset=docs)
    out = list(ds)
    assert len(out) == 3
    first = out[0]
    assert first["input_ids"].shape == (16,) and first["doc_boundaries"].tolist() == [0, 7]
    assert first["input_ids"][0] == 1 and first["input_ids"][6] == 2 and first["input_ids"][7] == 1
    assert (first["labels"][15:] == -100).all() and first["attention_mask"].sum() == 15
    assert out[1]["attention_mask"].sum() == 16          # the long document is truncated to the window
    batch = collate_fn(out[:2])
    assert set(batch) == {"input_ids", "attention_mask", "labels"} and batch["input_ids"].shape == (2, 16)
    dl = create_dataloader(DataConfig(max_seq_length=16), FakeTok(), batch_size=2, dataset=docs)
    assert next(iter(dl))["input_ids"].shape == (2, 16)
    single = list(TokenizedDataset(DataConfig(max_seq_length=8), FakeTok(), dataset=docs[:1]))[0]
    assert single["labels"][7] == -100 and single["input_ids"][0] == 1


def test_synthetic_tokens_are_seeded_and_resumable():
    a, b = SyntheticTokens(100, 8, 2, seed=3, rank=0), SyntheticTokens(100, 8, 2, seed=3, rank=0)
    ia, ib = iter(a), iter(b)
    x0, x1 = next(ia), next(ia)
    assert torch.equal(x0["input_ids"], next(ib)["input_ids"]) and not torch.equal(x0["input_ids"], x1["input_ids"])
    assert not torch.equal(SyntheticTokens(100, 8, 2, seed=3, rank=1).batch_at(0)["input_ids"], x0["input_ids"])
    c = SyntheticTokens(100, 8, 2, seed=3, rank=0)
    c.load_state_dict(a.state_dict())
    assert torch.equal(next(iter(c))["input_ids"], next(ia)["input_ids"])


def test_cli_flags_and_defaults():
    from nsa_optim_b200.train import build_parser, build_training_config, parse_args
    flags = {a.option_strings[-1] for a in build_parser()._actions}
    for f in ["--mamba_type", "--attn_type", "--block_pattern", "--block_repeats", "--mamba_d_state", "--mamba_d_conv",
              "--mamba_expand", "--mamba_headdim", "--nsa_block_size", "--nsa_window_size", "--nsa_num_selected_blocks",
              "--rope_theta", "--kernel_type", "--ce_kernel_type", "--model_size", "--optimizer_type", "--context_length",
              "--batch_size", "--gradient_accumulation_steps", "--num_train_steps", "--warmup_steps", "--learning_rate",
              "--weight_decay", "--max_grad_norm", "--precondition_frequency", "--shampoo_beta", "--max_precond_dim",
              "--dtype", "--gradient_checkpointing", "--dataset_name", "--dataset_subset", "--output_dir", "--run_name",
              "--resume_from", "--log_interval", "--save_interval"]:
        assert f in flags, f
    a = parse_args([])
    assert (a.mamba_type, a.attn_type, a.model_size, a.optimizer_type, a.context_length) == ("mamba2", "dense", "0.44B", "adamw", 8192)
    assert (a.gradient_accumulation_steps, a.num_train_steps, a.warmup_steps, a.learning_rate) == (4, 20000, 2000, 1e-4)
    assert (a.nsa_num_selected_blocks, a.rope_theta, a.max_precond_dim, a.precondition_frequency) == (32, 500000.0, 8192, 5)
    a = parse_args(["-attn", "nsa", "--block_pattern", "MDMA", "-lr", "1e-3", "-wd", "0.05", "-clip", "2.0"])
    cfg = build_training_config(a)
    assert cfg.attention_type == AttentionType.NSA and cfg.run_name == "0.44B_hybrid_MDMAx-1_adamw_ctx8192"
    assert cfg.optimizer_config.learning_rate == 1e-3 and cfg.max_grad_norm == 2.0
    with pytest.raises(SystemExit):
        parse_args(["--context_length", "1234"])


def test_log_line_format():
    from nsa_optim_b200.train import format_log_line
    line = format_log_line(10, 100, 1_310_720, 11.9412, 5e-5, 11589.4, 0.7321)
    assert line == "Step 10/100 | Tokens: 0.001B | Loss: 11.9412 | LR: 5.00e-05 | Tok/s: 11589 | Grad: 0.7321"


def test_checkpoint_layout_and_roundtrip(tmp_path):
    from nsa_optim_b200.train import Trainer, parse_args
    argv = ["--mamba_type", "none", "--model_size", "100M", "--hidden_size", "64", "--num_layers", "2", "--num_heads", "4",
            "--num_kv_heads", "2", "--intermediate_size", "128", "--vocab_size", "256", "--context_length", "32",
            "--synthetic_data", "--dtype", "float32", "--device", "cpu", "--num_train_steps", "2", "--warmup_steps", "0",
            "--gradient_accumulation_steps", "1", "--optimizer_type", "soap4bit", "--max_precond_dim", "64",
            "--output_dir", str(tmp_path)]
    tr = Trainer(parse_args(argv), verbose=False)
    tr.step(); tr.step()
    path = tr.save()
    assert path.endswith("checkpoint-2") and sorted(os.listdir(path)) == ["config.json", "model.pt", "optimizer.pt",
                                                                         "scheduler.pt", "trainer_state.pt"]
    cfg = json.load(open(os.path.join(path, "config.json")))
    for k in ("step", "model_type", "model_size", "attention_type", "optimizer_type", "max_seq_length", "fsdp", "custom_optim"):
        assert k in cfg
    assert cfg["custom_optim"] is True and cfg["model_type"] == "transformer"
    sd = torch.load(os.path.join(path, "model.pt"), weights_only=False)
    assert "layers.1.self_attn.o_proj.weight" in sd and "embed_tokens.weight" in sd
    osd = torch.load(os.path.join(path, "optimizer.pt"), weights_only=False)
    assert "layers.0.mlp.up_proj.weight" in osd["state"] and "QL_q_blocks" in osd["state"]["layers.0.mlp.up_proj.weight"]
    tr2 = Trainer(parse_args(argv), verbose=False)
    assert tr2.resume(path) == 2
    for (n, a), (_, b) in zip(tr.model.module.named_parameters(), tr2.model.module.named_parameters()):
        assert torch.equal(a, b), n
    l1, l2 = float(tr.step()["loss"]), float(tr2.step()["loss"])
    assert abs(l1 - l2) < 1e-5


def test_experiment_runner_dry_run(tmp_path):
    from nsa_optim_b200 import run_experiments as rx
    exps = get_filtered_experiments(model_sizes=["0.6B"], optimizer_types=[OptimizerType.ADAMW_8BIT], context_lengths=[32768])
    man = rx.generate_experiment_manifest(exps, str(tmp_path / "manifest.json"))
    assert man["num_experiments"] == 3 and "train.py" in man["experiments"][0]["command"]
    assert man["experiments"][0]["resources"]["fits"]
    res = rx.run_experiments_locally(exps, str(tmp_path / "scripts"), dry_run=True)
    assert all(os.path.exists(r["script"]) for r in res)
    assert "#SBATCH" in open(rx.write_slurm_script(exps[0], str(tmp_path / "slurm"))).read()
    rx.main(["--mode", "generate", "--model_sizes", "4B", "--optimizer_types", "soap4bit", "--output", str(tmp_path / "g")])
    assert os.path.exists(tmp_path / "g" / "manifest.json")


def test_analysis_on_run_directories(tmp_path):
    from nsa_optim_b200.analysis import generate_report, load_experiment_results, plot_training_curves
    for name, opt, loss in (("r1", "adamw", 3.0), ("r2", "soap4bit", 2.5)):
        ck = tmp_path / name / "checkpoint-10"
        ck.mkdir(parents=True)
        json.dump({"step": 10, "model_type": "hybrid", "model_size": "1B", "attention_type": "dense", "optimizer_type": opt,
                   "max_seq_length": 8192}, open(ck / "config.json", "w"))
        with open(tmp_path / name / "training_log.jsonl", "w") as f:
            for s in (5, 10):
                f.write(json.dumps({"step": s, "tokens": s * 100, "loss": loss + 1.0 / s, "tokens_per_sec": 1000.0}) + "\n")
        json.dump({"final_loss": loss, "tokens_per_sec": 1000.0, "total_tokens": 1000}, open(tmp_path / name / "metrics.json", "w"))
    res = load_experiment_results(str(tmp_path))
    assert [r.run_name for r in res] == ["r1", "r2"] and len(res[0].history) == 2
    rep = generate_report(res, str(tmp_path / "report.json"))
    assert rep["by_optimizer"]["soap4bit"]["best_final_loss"] == 2.5 and os.path.exists(tmp_path / "report.json")
    plot_training_curves(res, str(tmp_path / "c.png"))


def test_flop_model():
    from nsa_optim_b200.models import HybridConfig
    from nsa_optim_b200.profiling import calculate_arithmetic_intensity, calculate_flops_per_token, hybrid_flops_per_token
    cfg = ModelConfig("t", 1024, 28, 16, 8, 3072)
    dense = calculate_flops_per_token(cfg, 32768)
    assert dense["total"] == pytest.approx(3 * dense["forward"]) and dense["attention"] > dense["mlp"]
    sparse = calculate_flops_per_token(ModelConfig("t", 1024, 28, 16, 8, 3072, attention_type=AttentionType.NSA), 32768)
    assert sparse["attention"] < dense["attention"]
    assert calculate_arithmetic_intensity(cfg, 32768)["intensity"] > 100
    h = HybridConfig(d_model=2048, vocab_size=32000, block_pattern="MDMA", block_repeats=4, num_attention_heads=32,
                     num_key_value_heads=2, head_dim=128, intermediate_size=5632, deltanet_head_dim=128, deltanet_num_heads=16,
                     attention_type="nsa")
    f = hybrid_flops_per_token(h, 65536, training=True, recompute=True)
    assert 5.5e9 < f["model_flops"] < 9e9 and f["total"] > f["model_flops"]


def _tiny_trainer(tmp_path, *extra):
    from nsa_optim_b200.parallel.dist import DistInfo
    from nsa_optim_b200.train import Trainer, parse_args
    args = parse_args(["--block_pattern", "MDA", "--block_repeats", "1", "--model_size", "100M", "--hidden_size", "64",
                       "--vocab_size", "128", "--num_heads", "4", "--num_kv_heads", "2", "--mamba_d_state", "16",
                       "--mamba_headdim", "16", "--deltanet_head_dim", "16", "--intermediate_size", "128",
                       "--rope_theta", "1e4", "--context_length", "32", "--batch_size", "2", "--num_train_steps", "4",
                       "--warmup_steps", "0", "--dtype", "float32", "--synthetic_data", "--device", "cpu",
                       "--output_dir", str(tmp_path), *extra])
    return Trainer(args, info=DistInfo(), verbose=False)


def test_skip_nonfinite_leaves_parameters_and_optimizer_untouched(tmp_path):
    tr = _tiny_trainer(tmp_path, "--skip_nonfinite")
    tr.step()
    assert tr.skipped_steps == 0
    before = {n: p.detach().clone() for n, p in tr.model.module.named_parameters()}
    steps_before = [int(st["step"]) for st in tr.optimizer.state.values() if st]
    head = next(p for n, p in tr.model.module.named_parameters() if "norm" in n)
    poisoned = head.detach().clone()
    with torch.no_grad():
        head.fill_(float("inf"))
    out = tr.step()
    assert tr.skipped_steps == 1 and not torch.isfinite(out["loss"])
    with torch.no_grad():
        head.copy_(poisoned)
    for n, p in tr.model.module.named_parameters():
        assert torch.equal(p, before[n]), n
    assert [int(st["step"]) for st in tr.optimizer.state.values() if st] == steps_before
    tr.step()                                   # training goes on afterwards
    assert tr.skipped_steps == 1 and tr.step_count == 3


def test_loss_scaler_backs_off_on_overflow_and_grows_back():
    from nsa_optim_b200.train import LossScaler
    s = LossScaler(init_scale=1024.0, growth_interval=3)
    s.update(True)
    assert s.scale == 512.0 and s.overflows == 1
    for _ in range(3):
        s.update(False)
    assert s.scale == 1024.0 and s.good_steps == 0
    s.update(False)
    s.update(True)
    assert s.scale == 512.0 and s.good_steps == 0
    t = LossScaler()
    t.load_state_dict(s.state_dict())
    assert t.scale == 512.0 and t.overflows == 2


def test_overflow_under_loss_scaling_skips_the_step(tmp_path):
    from nsa_optim_b200.train import LossScaler
    tr = _tiny_trainer(tmp_path)
    tr.scaler = LossScaler(init_scale=float(2 ** 126))       # fp32 gradients overflow at this scale
    before = {n: p.detach().clone() for n, p in tr.model.module.named_parameters()}
    tr.step()
    assert tr.skipped_steps == 1 and tr.scaler.scale == float(2 ** 125)
    assert all(torch.equal(p, before[n]) for n, p in tr.model.module.named_parameters())
    tr.scaler = LossScaler(init_scale=64.0)
    out = tr.step()
    assert tr.skipped_steps == 1 and torch.isfinite(out["grad_norm"])
    assert any(not torch.equal(p, before[n]) for n, p in tr.model.module.named_parameters())


def test_a_recorded_kernel_status_aborts_the_step(tmp_path, monkeypatch):
    """The trainer reads the kernels' status block before the optimizer consumes a step's
    gradients; a recorded time-out (faked here: no GPU involved) must stop it."""
    import functools
    from nsa_optim_b200.ops import native
    tr = _tiny_trainer(tmp_path)
    monkeypatch.setattr(native, "read_status", lambda reset=True: (201, 3, 7, 1))
    monkeypatch.setattr(native, "_CANARY", False)
    tr._kernel_check = functools.partial(native.check_status)
    before = {n: p.detach().clone() for n, p in tr.model.module.named_parameters()}
    with pytest.raises(RuntimeError, match="status 201"):
        tr.step()
    assert all(torch.equal(p, before[n]) for n, p in tr.model.module.named_parameters())
    with pytest.raises(RuntimeError, match="status 201"):
        tr.save()
