"""Headline benchmark: training tokens/sec of the 1B MDMA hybrid with native sparse attention
at 64K context, AdamW8bit, bf16, sharded data parallel (one rank per GPU).

    python bench.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

Prints ONE JSON line on rank 0.  Timed regions of exactly K steps each, run alternately
(device, end to end, device, end to end); each kind reports the mean of its two repeats and both:
  * ``value``: device-timed (CUDA events), inputs already resident, max over ranks;
  * ``e2e``: the same steps through ``Trainer.step`` including, every step, the host->device
    copy of that step's token batch from pinned memory and a device->host read of the loss.
``gpu_launches`` is the number of this library's kernel launches in one region of K steps.
Model: 16 layers (MDMA x 4), d_model 2048, FFN 5632, vocab 32000; A blocks: 32 q / 2 kv heads of
128, compression 32/16, selection 64 x top-16, window 512; M blocks: d_state 128, headdim 64,
expand 2, chunk 256; D blocks: 16 heads of 128.  Random-init weights, uniform random tokens.
Weak scaling: one 65536-token sequence per GPU per step.

``--impl reference`` would run the unmodified reference from ``baseline/_ref``; it prints an
``unavailable`` line when that package cannot be imported.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "train tokens/sec/box (max over ranks) 1B MDMA-NSA 64K FSDP"
PUBLISHED_TOK_S = 11589.0   # the reference's only published throughput (0.5B MDMA, 8K ctx, unnamed 32 GB GPU)


def flagship_args(seq_len: int, extra=()):
    return [
        "--block_pattern", "MDMA", "--block_repeats", "4", "--attn_type", "nsa", "--model_size", "1B",
        "--hidden_size", "2048", "--vocab_size", "32000", "--intermediate_size", "5632",
        "--num_heads", "32", "--num_kv_heads", "2", "--head_dim", "128",
        "--nsa_compress_block", "32", "--nsa_compress_stride", "16", "--nsa_block_size", "64",
        "--nsa_num_selected_blocks", "16", "--nsa_window_size", "512",
        "--mamba_d_state", "128", "--mamba_headdim", "64", "--mamba_expand", "2",
        "--deltanet_head_dim", "128", "--deltanet_num_heads", "16",
        "--context_length", str(seq_len), "--batch_size", "1", "--gradient_accumulation_steps", "1",
        "--optimizer_type", "adamw8bit", "--dtype", "bfloat16", "--gradient_checkpointing",
        "--synthetic_data", "--num_train_steps", "1000000", "--warmup_steps", "10",
        "-lr", "1e-4", "-wd", "0.1", "-clip", "1.0",
    ] + list(extra)


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 8:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
                power.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


def reference_arm(a) -> None:
    """Runs the reference's own training step when it can be imported; otherwise prints why not.

    ``baseline/_ref`` holds the offline install of the reference (pip ``--no-deps --target``) plus
    its top-level modules ``config.py``, ``train.py``, ``optimizers.py``, ``data.py``, which its
    ``pyproject.toml`` does not package.  The import is attempted for real and the deepest frame
    inside the reference that failed is reported with file and line."""
    import traceback
    ref = os.path.join(ROOT, "baseline", "_ref")
    why = None
    if not os.path.isdir(ref):
        why = "baseline/_ref is absent (the offline install of the reference was not made)"
    else:
        sys.path.insert(0, ref)
        try:
            import models  # noqa: F401  (the reference's package)
            import train  # noqa: F401   (the reference's entry point)
        except Exception as exc:  # noqa: BLE001
            where = ""
            for fr in reversed(traceback.extract_tb(exc.__traceback__)):
                if ref in fr.filename:
                    where = f" at {os.path.relpath(fr.filename, ref)}:{fr.lineno} ({fr.line})"
                    break
            why = f"the reference cannot be imported offline: {type(exc).__name__}: {exc}{where}"
            if "mamba_ssm" in str(exc):
                # The only importable Mamba-2 layer here is fla.layers.mamba2.Mamba2, and without the
                # mamba_ssm / causal_conv1d kernels it runs its PyTorch path, whose intermediate
                # C[:, :, :, None] * B[:, :, None] has shape (batch, chunks, 256, 256, heads, d_state).
                chunks, heads, d_state = a.seq_len // 256, 64, 128
                gb = chunks * 256 * 256 * heads * d_state * 4 / 1e9
                why += (f"; mamba_ssm has no wheel here (torchao, causal_conv1d, native_sparse_attention are "
                        f"missing too), and fla's Mamba2 as a stand-in has only its PyTorch path, which needs a "
                        f"{gb:.0f} GB intermediate per layer at {a.seq_len} tokens")
    if why is None:
        why = ("the reference imports, but its --attn_type nsa hybrid trains dense attention blocks at 12 layers and "
               "vocabulary 151936 (models/hybrid.py:292-394): not the named config; not run")
    if int(os.environ.get("RANK", 0)) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why.replace("\n", " ")[:700]}))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", type=str, default="native", choices=["native", "reference", "torch", "library"],
                    help="native: this framework's kernels (the product); reference: the unmodified reference from "
                         "baseline/_ref; library: a diagnostic arm, this framework with third-party library kernels "
                         "(cuBLAS, flash_attn, fla, Liger) and NCCL collectives in place of its own; torch: the eager "
                         "PyTorch oracle")
    ap.add_argument("--seq_len", type=int, default=65536)
    ap.add_argument("--comm", type=str, default="auto")
    ap.add_argument("--skip_e2e", action="store_true")
    ap.add_argument("--checkpoint_blocks", type=str, default="auto",
                    help="block kinds whose activations are recomputed in backward ('MDA' = all, '' = none, "
                         "'auto' = none on a GPU with at least 170 GB, else the Mamba blocks)")
    a = ap.parse_args()
    if a.impl == "reference":
        reference_arm(a)
        return

    import torch
    import torch.distributed as dist
    from nsa_optim_b200 import ops
    from nsa_optim_b200.parallel import dist as pdist
    from nsa_optim_b200.train import Trainer, parse_args

    if a.impl == "torch":
        ops.set_backend("torch")
    if a.impl == "library":
        ops.set_backend("library")
        a.comm = "nccl"
    world = int(os.environ.get("WORLD_SIZE", 1))
    if world != a.gpus:
        raise SystemExit(f"--gpus {a.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    if a.checkpoint_blocks == "auto":
        # the 64K step keeps about 136 GB of activations alive when nothing is recomputed
        big = torch.cuda.is_available() and torch.cuda.get_device_properties(0).total_memory >= 170e9
        a.checkpoint_blocks = "" if (big and a.seq_len <= 65536) else "M"
    extra = ["--comm", a.comm]
    if a.checkpoint_blocks:
        extra += ["--checkpoint_blocks", a.checkpoint_blocks]
    args = parse_args(flagship_args(a.seq_len, extra))
    if not a.checkpoint_blocks:
        args.gradient_checkpointing = False
    tr = Trainer(args, verbose=False)
    info, dev = tr.info, tr.device
    native = ops.native_module() if a.impl in ("native", "library") else None
    K, W = a.steps, max(a.warmup, 3)
    tokens_per_step = args.batch_size * args.context_length * world

    # host batches in pinned memory (synthetic uniform tokens, seeded per rank and step)
    data = tr.make_data()
    host = [data.batch_at(i) for i in range(W + 2 * K)]
    h2d = sum(t.numel() * t.element_size() for k, t in host[0].items() if k in ("input_ids", "labels"))

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(W):
        out = tr.step([host[i]])
    sync_all()
    if native is not None:
        native.check_status()

    # ---- two kinds of timed region, run alternately (device, end to end, device, end to end) so that
    # a slow drift of the clocks shows up as a difference between the repeats instead of between the
    # kinds.  "value" and "e2e.value" are the means of their two repeats; both repeats are printed.
    #   device: CUDA events around K steps, inputs already resident on the device;
    #   e2e:    the same K steps through Trainer.step from pinned host batches, with the host->device
    #           copy of each batch and a device->host read of each step's loss inside the region.
    def device_region(batches):
        resident = [{k: v.to(dev) for k, v in b.items()} for b in batches]
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for b in resident:
            o = tr.step([b])
        e1.record()
        sync_all()
        t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
        pdist.all_reduce_max(t)
        return float(t), o

    def e2e_region(batches):
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        w0 = time.perf_counter()
        e0.record()
        nbytes = 0
        for b in batches:
            o = tr.step([b])                          # pinned host tensors; Trainer copies them in
            loss_host = o["loss"].float().cpu()       # device -> host read of the step's result
            nbytes = loss_host.numel() * loss_host.element_size()
        e1.record()
        sync_all()
        wall_ms = (time.perf_counter() - w0) * 1e3
        t = torch.tensor([max(e0.elapsed_time(e1), wall_ms)], dtype=torch.float64, device=dev)
        pdist.all_reduce_max(t)
        return float(t), nbytes

    repeats = 1 if a.skip_e2e else 2
    half = [host[W:W + K], host[W + K:W + 2 * K]]
    sampler = ClockSampler(info.local_rank)
    sync_all()
    sampler.start()
    l0 = native.launch_count() if native is not None else 0
    dev_ms, e2e_ms, d2h = [], [], 0
    steps_run = 0
    for r in range(repeats):
        ms_r, out = device_region(half[r % 2])
        dev_ms.append(ms_r)
        steps_run += K
        if not a.skip_e2e:
            ms_e, d2h = e2e_region(half[(r + 1) % 2])
            e2e_ms.append(ms_e)
            steps_run += K
    launches = ((native.launch_count() - l0) * K // steps_run) if native is not None else 0
    clocks = sampler.stop()
    ms = sum(dev_ms) / len(dev_ms)
    value = tokens_per_step * K / (ms / 1e3)
    final_loss = float(out["loss"])
    e2e = None
    if e2e_ms:
        em = sum(e2e_ms) / len(e2e_ms)
        e2e = {"value": tokens_per_step * K / (em / 1e3), "unit": "tokens/s", "ms_per_step": em / K,
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
               "repeats_ms_per_step": [round(x / K, 3) for x in e2e_ms]}
    if native is not None:
        native.check_status()
    fallbacks = native.fallback_counts() if native is not None else {}

    if info.is_main:
        line = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": value / PUBLISHED_TOK_S, "dtype": "bf16", "data": "synthetic uniform random tokens, random-init weights",
            "impl": a.impl,
            "config": {"model": "1B hybrid MDMAx4 (16 layers, d2048, FFN 5632, V32000; NSA 32q/2kv hd128 cmp32/16 sel64 top16 win512; "
                                "Mamba-2 N128 hd64 expand 2 (SSD kernels tile the scan in chunks of 128); GatedDeltaNet 16x128)",
                       "params": tr.n_params, "global_batch": args.batch_size * world, "seq_len": args.context_length,
                       "optimizer": "adamw8bit (block 256, dynamic-tree code book)", "grad_clip": 1.0,
                       "activation_checkpointing": (f"block kinds {a.checkpoint_blocks} recomputed, others keep activations"
                                                    if a.checkpoint_blocks else "off"),
                       "peak_memory_gb": round(torch.cuda.max_memory_allocated(dev) / 2**30, 2),
                       "peak_reserved_gb": round(torch.cuda.max_memory_reserved(dev) / 2**30, 2), "parallelism": f"dp{world} sharded ({tr.model.strategy.value})",
                       "comm": tr.model.comm_mode,
                       "l2": "no explicit flush: per-step working set (2.4 GB weights + >4 GB activations) exceeds the 126 MB L2",
                       "baseline_note": "vs_baseline divides by the reference's only published number (11589 tok/s, 0.5B MDMA, "
                                        "8K context, unnamed 32 GB GPU); it is not the same config"},
            "clocks": clocks, "gpu_launches": launches, "final_loss": final_loss,
            "loss_finite": bool(final_loss == final_loss and abs(final_loss) != float("inf")),
            "repeats_ms_per_step": [round(x / K, 3) for x in dev_ms], "region_order": "device, e2e, device, e2e",
            "torch_fallback_calls": fallbacks,
            "native_ops": sorted(native.SUPPORTED) if native is not None else [],
        }
        if e2e is not None:
            line["e2e"] = e2e
        if a.impl == "library":
            from nsa_optim_b200.ops import library_impl
            line["impl"] = "library (diagnostic: third-party kernels inside this framework; not the reference)"
            line["library_ops"] = library_impl.report()
        print(json.dumps(line), flush=True)
    pdist.cleanup_distributed()


if __name__ == "__main__":
    main()
