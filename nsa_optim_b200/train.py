"""Command line and training loop.

Reference behaviour (nngabe/nsa_optim train.py): flags :757-848, alias folding and enum
mapping :855-872, auto run name :908-920, distributed setup :65-86, model setup :89-210,
train step :213-290, evaluation :293-339, checkpoints :342-517, loop and logging :520-754.

Same flag names, choices and defaults.  Added flags cover what a size string cannot express
(``--vocab_size --num_layers --hidden_size --intermediate_size --num_heads --num_kv_heads
--head_dim --tie_embeddings --deltanet_head_dim --deltanet_num_heads --nsa_compress_block
--nsa_compress_stride``), the workload (``--synthetic_data --seed``), and the runtime
(``--dist_backend --comm --sharding --master_weights --eval_interval --skip_nonfinite``).

Differences by design: the sharded runtime replaces FSDP; clipping uses the global gradient
norm unless ``--local_clip``; the clip coefficient and the loss stay on the device between
log lines (no per-micro-batch host sync); throughput is timed with CUDA events and reduced
with max over ranks; ``training_log.jsonl`` and ``metrics.json`` are written for the
analysis tools; ``evaluate`` is actually called every ``--eval_interval`` steps.
"""
from __future__ import annotations

import argparse
import contextlib
import json
import math
import os
import sys
import time
from typing import Any, Dict, Iterator, List, Optional

import torch
import torch.nn as nn

from . import checkpoint as ckpt
from . import ops
from .config import (AttentionType, MambaType, ModelConfig, OptimizerConfig, OptimizerType, TrainingConfig,
                     resolve_attention_type)
from .data import DataConfig, create_dataloader, create_synthetic_loader, get_tokenizer
from .models import (create_gated_deltanet, create_hybrid_model, create_mamba2, create_model,
                     get_deltanet_config, get_hybrid_config, get_mamba2_config, get_model_config,
                     get_model_type, print_hybrid_model_modules)
from .optimizers import create_optimizer, get_lr_scheduler, print_preconditioning_stats
from .parallel import dist as pdist
from .parallel.sharded import ShardedModel, ShardingStrategy

CONTEXT_CHOICES = [8192, 32768, 65536, 131072, 524288, 1048576]
DTYPES = {"float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16}


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(description="Train models for ablation study")
    # architecture
    p.add_argument("--mamba_type", type=str, default="mamba2", choices=["none", "mamba2", "deltanet"])
    p.add_argument("-attn", "--attn_type", type=str, default="dense",
                   choices=["dense", "native_sparse_attention", "nsa", "flash_sparse_attention", "fsa"])
    p.add_argument("--block_pattern", type=str, default=None,
                   help="hybrid pattern over M (Mamba-2), D (Gated DeltaNet), A (attention), e.g. MDMA")
    p.add_argument("--block_repeats", type=int, default=-1, help="-1 = derive from the model size")
    p.add_argument("--mamba_d_state", type=int, default=128)
    p.add_argument("--mamba_d_conv", type=int, default=4)
    p.add_argument("--mamba_expand", type=int, default=2)
    p.add_argument("--mamba_headdim", type=int, default=64)
    p.add_argument("--nsa_block_size", type=int, default=64)
    p.add_argument("--nsa_window_size", type=int, default=64)
    p.add_argument("--nsa_num_selected_blocks", type=int, default=32)
    p.add_argument("--rope_theta", type=float, default=500000.0)
    p.add_argument("--kernel_type", type=str, default="liger", choices=["baseline", "triton", "liger"])
    p.add_argument("--ce_kernel_type", type=str, default=None, choices=["baseline", "liger"])
    # experiment
    p.add_argument("--model_size", type=str, default="0.44B")
    p.add_argument("--optimizer_type", type=str, default="adamw",
                   choices=["adamw", "adamw4bit", "adamw8bit", "soap", "soap4bit", "soap8bit", "shampoo"])
    p.add_argument("--context_length", type=int, default=8192)
    # training
    p.add_argument("--batch_size", type=int, default=1)
    p.add_argument("--gradient_accumulation_steps", type=int, default=4)
    p.add_argument("--num_train_steps", type=int, default=20000)
    p.add_argument("--warmup_steps", type=int, default=2000)
    p.add_argument("-lr", "--learning_rate", type=float, default=1e-4)
    p.add_argument("-wd", "--weight_decay", type=float, default=0.1)
    p.add_argument("-clip", "--max_grad_norm", type=float, default=1.0)
    p.add_argument("--precondition_frequency", type=int, default=5)
    p.add_argument("--shampoo_beta", type=float, default=0.95)
    p.add_argument("--max_precond_dim", type=int, default=8192)
    p.add_argument("--dtype", type=str, default="bfloat16", choices=list(DTYPES))
    p.add_argument("--gradient_checkpointing", action="store_true")
    p.add_argument("--checkpoint_blocks", type=str, default=None,
                   help="with --gradient_checkpointing: recompute only these block kinds (letters M, D, A)")
    p.add_argument("--dataset_name", type=str, default="HuggingFaceFW/fineweb-edu")
    p.add_argument("--dataset_subset", type=str, default="sample-10BT")
    p.add_argument("--output_dir", type=str, default="./outputs")
    p.add_argument("--run_name", type=str, default="")
    p.add_argument("--resume_from", type=str, default=None)
    p.add_argument("--log_interval", type=int, default=10)
    p.add_argument("--save_interval", type=int, default=5000)
    # ---- additions
    g = p.add_argument_group("shape overrides")
    g.add_argument("--vocab_size", type=int, default=None)
    g.add_argument("--num_layers", type=int, default=None)
    g.add_argument("--hidden_size", type=int, default=None)
    g.add_argument("--intermediate_size", type=int, default=None)
    g.add_argument("--num_heads", type=int, default=None)
    g.add_argument("--num_kv_heads", type=int, default=None)
    g.add_argument("--head_dim", type=int, default=None)
    g.add_argument("--tie_embeddings", action="store_true")
    g.add_argument("--deltanet_head_dim", type=int, default=None)
    g.add_argument("--deltanet_num_heads", type=int, default=None)
    g.add_argument("--nsa_compress_block", type=int, default=32)
    g.add_argument("--nsa_compress_stride", type=int, default=16)
    g.add_argument("--nsa_block_scorer", type=str, default="compressed", choices=["compressed", "learned"],
                   help="block selection of sparse attention: from the compressed branch (default) or the "
                        "reference module's learned k_compress scorer (selected + window branches only)")
    g = p.add_argument_group("runtime")
    g.add_argument("--synthetic_data", action="store_true", help="uniform random token ids (seeded)")
    g.add_argument("--nvtx", action="store_true",
                   help="NVTX ranges around the phases of a step (forward+backward per micro-batch, clip, optimizer) "
                        "and around every block, for timeline profilers")
    g.add_argument("--seed", type=int, default=0)
    g.add_argument("--dist_backend", type=str, default=None, choices=["nccl", "gloo"])
    g.add_argument("--comm", type=str, default="auto", choices=["auto", "fused", "nccl", "gloo"])
    g.add_argument("--sharding", type=str, default=None, choices=[s.value for s in ShardingStrategy])
    g.add_argument("--master_weights", action="store_true")
    g.add_argument("--local_clip", action="store_true", help="clip by the local shard norm")
    g.add_argument("--eval_interval", type=int, default=0)
    g.add_argument("--eval_batches", type=int, default=50)
    g.add_argument("--skip_nonfinite", action="store_true", help="skip optimizer steps with NaN/Inf loss")
    g.add_argument("--device", type=str, default=None, choices=[None, "cpu", "cuda"])
    g.add_argument("--lr_scheduler_type", type=str, default="cosine",
                   choices=["cosine", "linear", "constant_with_warmup"])
    return p


def parse_args(argv: Optional[List[str]] = None) -> argparse.Namespace:
    args = build_parser().parse_args(argv)
    if args.context_length not in CONTEXT_CHOICES and not args.synthetic_data:
        raise SystemExit(f"--context_length must be one of {CONTEXT_CHOICES} (any value with --synthetic_data)")
    return args


def build_training_config(args: argparse.Namespace) -> TrainingConfig:
    attn = resolve_attention_type(args.attn_type)
    mamba = {"mamba2": MambaType.MAMBA2, "deltanet": MambaType.MAMBA3}.get(args.mamba_type, MambaType.NONE)
    opt_type = OptimizerType(args.optimizer_type)
    opt_cfg = OptimizerConfig(optimizer_type=opt_type, learning_rate=args.learning_rate,
                              weight_decay=args.weight_decay,
                              precondition_frequency=args.precondition_frequency,
                              shampoo_beta=args.shampoo_beta, max_precond_dim=args.max_precond_dim,
                              master_weights=args.master_weights)
    cfg = TrainingConfig(
        model_size=args.model_size, attention_type=attn, mamba_type=mamba, optimizer_type=opt_type,
        optimizer_config=opt_cfg, max_seq_length=args.context_length, batch_size=args.batch_size,
        gradient_accumulation_steps=args.gradient_accumulation_steps,
        num_train_steps=args.num_train_steps, warmup_steps=args.warmup_steps,
        max_grad_norm=args.max_grad_norm, dtype=args.dtype,
        gradient_checkpointing=args.gradient_checkpointing, dataset_name=args.dataset_name,
        dataset_subset=args.dataset_subset, output_dir=args.output_dir, run_name=args.run_name,
        log_interval=args.log_interval, save_interval=args.save_interval,
        eval_interval=args.eval_interval, seed=args.seed, synthetic_data=args.synthetic_data,
        lr_scheduler_type=args.lr_scheduler_type,
    )
    if not args.run_name:
        if args.block_pattern:
            arch = f"hybrid_{args.block_pattern}x{args.block_repeats}"
        elif args.mamba_type != "none":
            arch = args.mamba_type
        elif attn == AttentionType.NSA:
            arch = "nsa"
        elif attn == AttentionType.FSA:
            arch = "fsa"
        else:
            arch = "dense"
        cfg.run_name = f"{args.model_size}_{arch}_{opt_type.value}_ctx{args.context_length}"
    return cfg


def build_model(cfg: TrainingConfig, args: argparse.Namespace, verbose: bool = True):
    """-> (model, model_type, model_config).  CPU construction; the caller moves / wraps it."""
    model_type = get_model_type(cfg, args.block_pattern)
    kernel_type = args.kernel_type
    if model_type == "hybrid":
        mc = get_hybrid_config(
            cfg, args.block_pattern, args.block_repeats, args.mamba_d_state, args.mamba_d_conv,
            args.mamba_expand, args.mamba_headdim, args.rope_theta, vocab_size=args.vocab_size,
            verbose=verbose, d_model=args.hidden_size, intermediate_size=args.intermediate_size,
            num_attention_heads=args.num_heads, num_key_value_heads=args.num_kv_heads,
            head_dim=args.head_dim, tie_word_embeddings=args.tie_embeddings or None,
            deltanet_head_dim=args.deltanet_head_dim, deltanet_num_heads=args.deltanet_num_heads,
            nsa_block_size=args.nsa_block_size, nsa_window_size=args.nsa_window_size,
            nsa_num_selected_blocks=args.nsa_num_selected_blocks,
            nsa_compress_block=args.nsa_compress_block, nsa_compress_stride=args.nsa_compress_stride)
        if args.num_layers:
            mc.block_repeats = max(1, args.num_layers // len(mc.block_pattern))
        model = create_hybrid_model(mc)
    elif model_type == "mamba2":
        mc = get_mamba2_config(cfg, vocab_size=args.vocab_size, d_model=args.hidden_size,
                               n_layers=args.num_layers, d_state=args.mamba_d_state,
                               d_conv=args.mamba_d_conv, expand=args.mamba_expand, headdim=args.mamba_headdim)
        model = create_mamba2(mc)
    elif model_type == "deltanet":
        mc = get_deltanet_config(cfg, vocab_size=args.vocab_size, d_model=args.hidden_size,
                                 n_layers=args.num_layers, head_dim=args.deltanet_head_dim,
                                 num_heads=args.deltanet_num_heads)
        model = create_gated_deltanet(mc)
    else:
        mc = get_model_config(cfg, args.nsa_block_size, args.nsa_window_size,
                              args.nsa_num_selected_blocks, args.rope_theta, vocab_size=args.vocab_size,
                              hidden_size=args.hidden_size, num_hidden_layers=args.num_layers,
                              intermediate_size=args.intermediate_size,
                              num_attention_heads=args.num_heads, num_key_value_heads=args.num_kv_heads,
                              head_dim=args.head_dim, tie_word_embeddings=args.tie_embeddings or None,
                              nsa_compress_block=args.nsa_compress_block,
                              nsa_compress_stride=args.nsa_compress_stride,
                              nsa_block_scorer=args.nsa_block_scorer)
        model = create_model(mc, kernel_type)
    if args.ce_kernel_type is not None:
        from .models.kernels import create_cross_entropy_loss
        model.loss_fn = create_cross_entropy_loss(None, args.ce_kernel_type)
    if cfg.gradient_checkpointing:
        model.gradient_checkpointing_enable()
    return model, model_type, mc


@torch.no_grad()
def evaluate(model, dataloader, device, max_batches: int = 50) -> Dict[str, float]:
    """Mean token loss and perplexity over at most ``max_batches`` batches."""
    was_training = model.training
    model.eval()
    total, count = 0.0, 0
    for i, batch in enumerate(dataloader):
        if i >= max_batches:
            break
        ids = batch["input_ids"].to(device, non_blocking=True)
        labels = batch["labels"].to(device, non_blocking=True)
        _, loss, _ = model(input_ids=ids, labels=labels)
        n = int((labels[:, 1:] != -100).sum())
        total += float(loss) * n
        count += n
    model.train(was_training)
    mean = total / max(1, count)
    return {"loss": mean, "perplexity": math.exp(min(mean, 50.0)), "tokens": count}


class LossScaler:
    """Dynamic loss scaling for float16 training (the reference wraps its step in
    ``torch.cuda.amp.GradScaler``: train.py:255-283, 645-647).  The loss is multiplied by
    ``scale`` before backward; gradients are unscaled inside the optimizer update through its
    ``grad_scale`` argument.  A step whose gradient norm is not finite is skipped and the scale is
    halved; after ``growth_interval`` good steps in a row it is doubled."""

    def __init__(self, init_scale: float = 65536.0, growth_factor: float = 2.0, backoff_factor: float = 0.5,
                 growth_interval: int = 2000, min_scale: float = 1.0):
        self.scale = float(init_scale)
        self.growth_factor, self.backoff_factor = growth_factor, backoff_factor
        self.growth_interval, self.min_scale = growth_interval, min_scale
        self.good_steps = 0
        self.overflows = 0

    def update(self, found_inf: bool) -> None:
        if found_inf:
            self.scale = max(self.min_scale, self.scale * self.backoff_factor)
            self.good_steps = 0
            self.overflows += 1
        else:
            self.good_steps += 1
            if self.good_steps >= self.growth_interval:
                self.scale *= self.growth_factor
                self.good_steps = 0

    def state_dict(self) -> Dict[str, Any]:
        return {"scale": self.scale, "good_steps": self.good_steps, "overflows": self.overflows}

    def load_state_dict(self, sd: Dict[str, Any]) -> None:
        self.scale = float(sd.get("scale", self.scale))
        self.good_steps = int(sd.get("good_steps", 0))
        self.overflows = int(sd.get("overflows", 0))


class Trainer:
    """Builds model, runtime, optimizer, schedule and data from parsed flags; :meth:`step` is
    one optimizer step (all accumulation micro-batches)."""

    def __init__(self, args: argparse.Namespace, info: Optional[pdist.DistInfo] = None, verbose: bool = True):
        self.args = args
        self.cfg = build_training_config(args)
        self.info = info or pdist.setup_distributed(args.dist_backend, device=args.device)
        self.verbose = verbose and self.info.is_main
        self.device = self.info.device
        self.dtype = DTYPES[self.cfg.dtype]
        torch.manual_seed(self.cfg.seed)
        model, self.model_type, self.model_config = build_model(self.cfg, args, self.verbose)
        model.to(self.dtype)
        comm = args.comm
        sharding = args.sharding
        if sharding is None and self.info.world_size > 1:
            # the reference's rule (train.py:188-196): whole-matrix preconditioners keep parameters
            # gathered (SHARD_GRAD_OP), every other optimizer runs fully sharded
            keep = self.cfg.optimizer_type in (OptimizerType.SOAP, OptimizerType.SOAP_4BIT, OptimizerType.SOAP_8BIT,
                                               OptimizerType.SHAMPOO)
            sharding = (ShardingStrategy.SHARD_GRAD_OP if keep else ShardingStrategy.FULL_SHARD).value
        self.model = ShardedModel(model, self.info, strategy=sharding, param_dtype=self.dtype,
                                  activation_checkpointing=self.cfg.gradient_checkpointing, comm=comm,
                                  checkpoint_blocks=getattr(args, "checkpoint_blocks", None))
        self.model.nvtx = bool(getattr(args, "nvtx", False)) and self.device.type == "cuda"
        self.n_params = sum(p.numel() for p in model.parameters())
        if self.verbose:
            print(f"Model dtype: {self.cfg.dtype}")
            print(f"Model parameters: {self.n_params / 1e9:.2f}B")
            if self.model_type == "hybrid":
                print_hybrid_model_modules(model, self.model_config.block_pattern, self.model_config.block_repeats)
            if self.cfg.optimizer_type in (OptimizerType.SOAP, OptimizerType.SOAP_4BIT,
                                           OptimizerType.SOAP_8BIT, OptimizerType.SHAMPOO):
                print_preconditioning_stats(model, self.cfg.optimizer_config.max_precond_dim)
        self.whole_matrix_optimizer = self.cfg.optimizer_type in (OptimizerType.SOAP, OptimizerType.SOAP_4BIT,
                                                                  OptimizerType.SOAP_8BIT, OptimizerType.SHAMPOO)
        if self.whole_matrix_optimizer and self.info.world_size > 1:
            n = self.model.enable_owner_preconditioning()
            if self.verbose:
                print(f"Whole-matrix optimizer under sharding: {n} matrices cut by shard boundaries are each updated by one owner rank")
        self.optimizer = create_optimizer(self.model.named_optimizer_parameters(), self.cfg.optimizer_config,
                                          self.info.world_size)
        self.scheduler = get_lr_scheduler(self.optimizer, self.cfg.lr_scheduler_type,
                                          self.cfg.num_train_steps, self.cfg.warmup_steps, self.cfg.min_lr_ratio)
        self.scaler = LossScaler() if self.dtype == torch.float16 else None
        # Kernels never trap: a wait that ran out (a peer that stopped, a flag never set) leaves a
        # record in a host-mapped status block and the kernel returns without touching its output.
        # The step reads that block before it lets the optimizer consume the data.
        self._kernel_check = None
        if self.device.type == "cuda" and ops.get_backend() != "torch":
            self._kernel_check = ops.native_module().check_status
        self.step_count = 0
        self.total_tokens = 0
        self.skipped_steps = 0
        self.data = None
        self._iter: Optional[Iterator] = None

    # ---- data
    def vocab_size(self) -> int:
        mc = self.model_config
        return getattr(mc, "vocab_size")

    def make_data(self):
        if self.cfg.synthetic_data:
            self.data = create_synthetic_loader(self.vocab_size(), self.cfg.max_seq_length,
                                                self.cfg.batch_size, self.cfg.seed, self.info.rank,
                                                pin_memory=self.device.type == "cuda")
        else:
            tok = get_tokenizer("Qwen/Qwen3-0.6B")
            dc = DataConfig(dataset_name=self.cfg.dataset_name, dataset_subset=self.cfg.dataset_subset,
                            max_seq_length=self.cfg.max_seq_length)
            self.data = create_dataloader(dc, tok, self.cfg.batch_size, "train", self.info.rank,
                                          self.info.world_size)
        self._iter = iter(self.data)
        return self.data

    def next_batch(self) -> Dict[str, torch.Tensor]:
        if self._iter is None:
            self.make_data()
        try:
            return next(self._iter)
        except StopIteration:
            self._iter = iter(self.data)
            return next(self._iter)

    # ---- one optimizer step
    def micro_step(self, batch: Dict[str, torch.Tensor]) -> torch.Tensor:
        ids = batch["input_ids"].to(self.device, non_blocking=True)
        labels = batch["labels"].to(self.device, non_blocking=True)
        ctx = torch.autocast(self.device.type, dtype=torch.float16) if self.scaler else contextlib.nullcontext()
        with ctx:
            _, loss, _ = self.model(input_ids=ids, labels=labels)
        scaled = loss / self.cfg.gradient_accumulation_steps
        if self.scaler:
            scaled = scaled * self.scaler.scale
        self.model.backward(scaled)
        return loss.detach()

    def _range(self, name: str):
        """NVTX range when ``--nvtx`` is on (a no-op context otherwise)."""
        if getattr(self.args, "nvtx", False) and self.device.type == "cuda":
            return torch.cuda.nvtx.range(name)
        return contextlib.nullcontext()

    def step(self, batches: Optional[List[Dict[str, torch.Tensor]]] = None) -> Dict[str, Any]:
        """Runs ``gradient_accumulation_steps`` micro-batches and one optimizer update.
        Returned tensors (``loss``, ``grad_norm``) stay on the device."""
        accum = self.cfg.gradient_accumulation_steps
        losses = []
        for i in range(accum):
            batch = batches[i] if batches is not None else self.next_batch()
            with self._range(f"micro_step {i}"):
                losses.append(self.micro_step(batch))
        loss = torch.stack(losses).mean()
        with self._range("clip"):
            norm, coef = self.model.clip_grad_norm(self.cfg.max_grad_norm, local_only=self.args.local_clip)
        self.check_kernels(sync=False)
        do_step = True
        if self.scaler:
            # gradients carry the loss scale: unscale the norm, fold 1/scale into the update, and let
            # an overflow (non-finite norm, agreed by every rank because the norm is global) skip it
            inv = torch.tensor(1.0 / self.scaler.scale, device=self.device)
            norm = norm * inv
            coef = inv if coef is None else (self.cfg.max_grad_norm / (norm + 1e-6)).clamp(max=1.0) * inv
            do_step = bool(torch.isfinite(norm))
            self.scaler.update(not do_step)
        if self.args.skip_nonfinite and do_step:
            # one host read per step: the price of the flag (off by default)
            do_step = bool(torch.isfinite(loss) & torch.isfinite(norm))
        if do_step:
            with self._range("optimizer"):
                self.model.collect_owned_grads()         # whole-matrix optimizers: gradient pieces to their owners
                self.optimizer.step(grad_scale=coef)
                self.scheduler.step()
                self.model.publish_owned_weights()       # and the updated pieces back to their holders
                self.model.regather_all()
        else:
            self.skipped_steps += 1
        self.model.zero_grad(set_to_none=True)
        self.step_count += 1
        self.total_tokens += accum * self.cfg.batch_size * self.cfg.max_seq_length * self.info.world_size
        return {"loss": loss, "grad_norm": norm, "lr": self.scheduler.get_last_lr()[0]}

    def check_kernels(self, sync: bool = False) -> None:
        """Raises if a native kernel has reported a failure (see ``ops/native.py::check_status``).
        Without ``sync`` this is one read of host memory and sees reports of kernels that have
        finished so far; the training loop calls it with ``sync`` at every log point and before a
        checkpoint is written, so a failed collective never reaches a saved state."""
        if self._kernel_check is not None:
            self._kernel_check(sync)

    # ---- checkpointing
    def meta(self) -> Dict[str, Any]:
        return {"model_type": self.model_type, "model_size": self.cfg.model_size,
                "attention_type": self.cfg.attention_type.value,
                "optimizer_type": self.cfg.optimizer_type.value,
                "max_seq_length": self.cfg.max_seq_length}

    def save(self, step: Optional[int] = None) -> str:
        step = self.step_count if step is None else step
        self.check_kernels(sync=True)
        ts = {"total_tokens": self.total_tokens, "skipped_steps": self.skipped_steps}
        if self.scaler:
            ts["loss_scaler"] = self.scaler.state_dict()
        if hasattr(self.data, "state_dict"):
            ts["data"] = self.data.state_dict()
        return ckpt.save_checkpoint(self.model, self.optimizer, self.scheduler, step, self.cfg.output_dir,
                                    self.cfg.run_name, self.meta(), ts, self.info.rank, self.info.world_size)

    def resume(self, path: str) -> int:
        st = ckpt.load_checkpoint(path, self.model, self.optimizer, self.scheduler, self.info.rank)
        self.step_count = int(st.get("step", 0))
        self.total_tokens = int(st.get("total_tokens", self.step_count * self.cfg.gradient_accumulation_steps
                                       * self.cfg.batch_size * self.cfg.max_seq_length * self.info.world_size))
        if self.scaler and "loss_scaler" in st:
            self.scaler.load_state_dict(st["loss_scaler"])
        if self.data is None:
            self.make_data()
        if "data" in st and hasattr(self.data, "load_state_dict"):
            self.data.load_state_dict(st["data"])
            self._iter = iter(self.data)
        return self.step_count


def format_log_line(step: int, total_steps: int, tokens: int, loss: float, lr: float,
                    tok_s: float, grad: float) -> str:
    return (f"Step {step}/{total_steps} | Tokens: {tokens / 1e9:.3f}B | Loss: {loss:.4f} | "
            f"LR: {lr:.2e} | Tok/s: {tok_s:.0f} | Grad: {grad:.4f}")


def _model_flops_per_token(trainer: "Trainer") -> float:
    """Model FLOPs (forward + backward, no recompute) per trained token, 0 when the model family
    has no FLOP model."""
    from .models import HybridConfig
    from .profiling import calculate_flops_per_token, hybrid_flops_per_token
    mc = getattr(trainer.model.module if hasattr(trainer.model, "module") else trainer.model, "config", None)
    try:
        if isinstance(mc, HybridConfig):
            return float(hybrid_flops_per_token(mc, trainer.cfg.max_seq_length, training=True, recompute=False)["model_flops"])
        if isinstance(mc, ModelConfig):
            return float(calculate_flops_per_token(mc, trainer.cfg.max_seq_length)["total"])
    except Exception:  # noqa: BLE001 - the figure is informational
        pass
    return 0.0


def train(args: argparse.Namespace) -> Dict[str, Any]:
    trainer = Trainer(args)
    cfg, info = trainer.cfg, trainer.info
    wandb = None
    if info.is_main and os.environ.get("WANDB_MODE", "") != "disabled":
        try:
            import wandb as _w
            _w.init(project="nsa-optimizer-ablation", name=cfg.run_name, config=vars(args))
            wandb = _w
        except Exception:  # noqa: BLE001 - logging backend is optional
            wandb = None
    trainer.make_data()
    if args.resume_from:
        step = trainer.resume(args.resume_from)
        if info.is_main:
            print(f"Resumed from {args.resume_from} at step {step}")
    run_dir = os.path.join(cfg.output_dir, cfg.run_name)
    log_f = None
    if info.is_main:
        os.makedirs(run_dir, exist_ok=True)
        log_f = open(os.path.join(run_dir, "training_log.jsonl"), "a")
        eff = cfg.batch_size * cfg.gradient_accumulation_steps * info.world_size
        print(f"Effective batch: {eff} sequences x {cfg.max_seq_length} tokens "
              f"({cfg.batch_size} per GPU x {cfg.gradient_accumulation_steps} accumulation x {info.world_size} ranks)")
    use_events = trainer.device.type == "cuda"
    trainer.model.measure_exposed = use_events and info.world_size > 1
    flops_per_token = _model_flops_per_token(trainer)
    window_losses: List[torch.Tensor] = []
    window_tokens = 0
    last = {"loss": float("nan"), "tok_s": 0.0}

    def mark():
        if use_events:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            return e
        return time.perf_counter()

    t_start = mark()
    history = []
    while trainer.step_count < cfg.num_train_steps:
        out = trainer.step()
        window_losses.append(out["loss"])
        window_tokens += cfg.gradient_accumulation_steps * cfg.batch_size * cfg.max_seq_length * info.world_size
        s = trainer.step_count
        if s % cfg.log_interval == 0 or s == cfg.num_train_steps:
            t_end = mark()
            if use_events:
                torch.cuda.synchronize()
                trainer.check_kernels(sync=False)
                dt = t_start.elapsed_time(t_end) / 1e3
            else:
                dt = t_end - t_start
            dt_t = torch.tensor([dt], dtype=torch.float64, device=trainer.device)
            pdist.all_reduce_max(dt_t)
            dt = float(dt_t)
            loss = float(torch.stack(window_losses).mean())
            grad = float(out["grad_norm"])
            tok_s = window_tokens / max(dt, 1e-9)
            last = {"loss": loss, "tok_s": tok_s}
            if info.is_main:
                print(format_log_line(s, cfg.num_train_steps, trainer.total_tokens, loss, out["lr"], tok_s, grad),
                      flush=True)
                rec = {"step": s, "tokens": trainer.total_tokens, "loss": loss, "lr": out["lr"],
                       "tokens_per_sec": tok_s, "grad_norm": grad}
                if flops_per_token:
                    from .profiling import model_flops_utilisation
                    rec["mfu"] = model_flops_utilisation(flops_per_token, tok_s, info.world_size)
                if trainer.model.measure_exposed:
                    # time the compute stream waited for the communication stream in this window
                    ms = trainer.model.pop_exposed_comm_ms()
                    rec["exposed_comm_ms_per_step"] = ms / max(1, cfg.log_interval)
                    rec["exposed_comm_frac"] = ms / max(dt * 1e3, 1e-9)
                history.append(rec)
                log_f.write(json.dumps(rec) + "\n")
                log_f.flush()
                if wandb is not None:
                    wandb.log({"train/loss": loss, "train/lr": out["lr"], "train/tokens": trainer.total_tokens,
                               "train/tokens_per_sec": tok_s, "train/grad_norm": grad}, step=s)
            if not math.isfinite(loss) and not args.skip_nonfinite:
                raise FloatingPointError(f"non-finite loss {loss} at step {s}")
            window_losses, window_tokens = [], 0
            t_start = mark()
        if cfg.eval_interval and s % cfg.eval_interval == 0:
            ev_data = create_synthetic_loader(trainer.vocab_size(), cfg.max_seq_length, cfg.batch_size,
                                              cfg.seed + 7919, info.rank) if cfg.synthetic_data else trainer.data
            ev = evaluate(trainer.model, ev_data, trainer.device, args.eval_batches)
            if info.is_main:
                print(f"Eval step {s} | Loss: {ev['loss']:.4f} | Perplexity: {ev['perplexity']:.2f}", flush=True)
                if wandb is not None:
                    wandb.log({"eval/loss": ev["loss"], "eval/perplexity": ev["perplexity"]}, step=s)
        if cfg.save_interval and s % cfg.save_interval == 0 and s < cfg.num_train_steps:
            trainer.save(s)
    path = trainer.save(trainer.step_count)
    if info.is_main:
        with open(os.path.join(run_dir, "metrics.json"), "w") as f:
            json.dump({"final_loss": last["loss"], "tokens_per_sec": last["tok_s"],
                       "total_tokens": trainer.total_tokens, "steps": trainer.step_count,
                       "skipped_steps": trainer.skipped_steps, "n_params": trainer.n_params,
                       "history": history[-100:]}, f, indent=2)
        log_f.close()
        print(f"Saved final checkpoint to {path}")
    if wandb is not None:
        wandb.finish()
    return {"final_loss": last["loss"], "tokens_per_sec": last["tok_s"], "checkpoint": path}


def main(argv: Optional[List[str]] = None) -> None:
    args = parse_args(argv)
    try:
        train(args)
    finally:
        pdist.cleanup_distributed()


if __name__ == "__main__":
    main()
