"""Peer-memory collectives and the fused all-gather GEMM on real peers, against NCCL.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port 29500 -m nsa_optim_b200.benchmarks.comm_benchmark [--unit_mb 121] [--iters 10]

One rank per GPU.  Every rank owns one shard of a sharded unit (default: the 121 MB Mamba block of
the 1B flagship) inside a CUDA-IPC arena that all ranks map.  Timed, each with CUDA events on the
launching stream after warm-up, a barrier before every iteration and the MAX over ranks taken:

  * all-gather of the unit: the peer-load kernel (``comm.cu``) and NCCL ``all_gather_into_tensor``;
  * reduce-scatter of the unit's fp32 gradients (+ scale + sum of squares): the peer-load kernel
    and NCCL ``reduce_scatter_tensor``;
  * y = x W^T with W inside the unit: the GEMM that gathers the unit itself (``gemm.cu``, copy CTAs
    pulling the peers' shards while the tcgen05 tiles run, swept over the number of copy CTAs),
    the peer-load all-gather followed by the plain GEMM, and NCCL's all-gather followed by it.

Rooflines: a gather must bring (W-1)/W of the unit over NVLink into every GPU; the measured peer
copy rate on this pool is 770 GB/s per direction per GPU (nominal 900).  The fused GEMM's target is
the slower of its FLOPs at the measured GEMM rate and those bytes at that link rate.
Rank 0 prints one JSON line per row.  The reference has no counterpart (it only calls NCCL through
FSDP: train.py:171-208).
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

LINK_GBS = 770.0          # measured peer copy, per direction per GPU, on this pool


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--unit_mb", type=float, default=121.0)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--m", type=int, default=65536)
    ap.add_argument("--n", type=int, default=8512)
    ap.add_argument("--k", type=int, default=2048)
    a = ap.parse_args()
    from .. import ops
    from ..parallel import dist as pdist
    from ..parallel import symm
    from .kernel_benchmark import peaks

    info = pdist.setup_distributed("nccl")
    W, rank, dev = info.world_size, info.rank, info.device
    native = ops.native_module()
    S = int(a.unit_mb * (1 << 20) / 2 / W) // 4096 * 4096          # bf16 elements per shard
    if a.n * a.k + 4096 > W * S:
        raise SystemExit("the weight does not fit into the unit")
    arena = symm.SymmetricArena(S * 2 + W * S * 4 + 65536, 4, rank, W, dev, None)
    off_sh, off_g = arena.alloc(S * 2), arena.alloc(W * S * 4)
    arena.view(off_sh, S, torch.bfloat16).normal_(0, 0.02)
    arena.view(off_g, W * S, torch.float32).normal_()
    full = torch.empty(W * S, dtype=torch.bfloat16, device=dev)
    shard = arena.view(off_sh, S, torch.bfloat16)
    gshard = torch.zeros(S, device=dev)
    gfull = arena.view(off_g, W * S, torch.float32)
    parts = torch.zeros(symm.reduce_scatter_parts(), device=dev)
    x = (torch.randn(a.m, a.k, device=dev) * 0.1).bfloat16()
    cps = max(1, min(1024, (S * 2) // (256 << 10)))
    flags = torch.zeros(W * cps, dtype=torch.int32, device=dev)
    epoch = [0]
    torch.cuda.synchronize()
    dist.barrier()

    def timed(fn, pre=None):
        ms = []
        for it in range(3 + a.iters):
            if pre is not None:
                pre()
            torch.cuda.synchronize()
            dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            if it >= 3:
                ms.append(e0.elapsed_time(e1))
        t = torch.tensor([sum(ms) / len(ms)], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    def publish():
        # every rank announces "my shard / my gradients are ready" under a fresh epoch
        epoch[0] += 1
        symm.signal(arena, 0, epoch[0])

    rows = []
    in_bytes = (W - 1) * S * 2

    def row(name, ms, nbytes=None, flops=None, **kw):
        r = {"op": name, "world": W, "ms": round(ms, 4)}
        if nbytes is not None:
            r["gbs_in_per_gpu"] = round(nbytes / ms / 1e6, 1)
            r["frac_of_link"] = round(nbytes / ms / 1e6 / LINK_GBS, 3)
        if flops is not None:
            r["tflops"] = round(flops / ms / 1e9, 1)
        r.update(kw)
        rows.append(r)

    # ---- all-gather
    ms = timed(lambda: symm.all_gather(arena, off_sh, S * 2, full, 0, epoch[0], ctas_per_peer=max(4, 64 // W)), publish)
    row(f"all_gather peer-load kernel, unit {W * S * 2 / 2**20:.0f} MB", ms, in_bytes)
    ref = full.clone()
    ms = timed(lambda: dist.all_gather_into_tensor(full, shard))
    row("all_gather NCCL", ms, in_bytes)
    ok_gather = bool(torch.equal(ref, full))

    # ---- reduce-scatter (fp32 gradients)
    rs_bytes = (W - 1) * S * 4
    ms = timed(lambda: symm.reduce_scatter(arena, off_g, gshard, 1.0 / W, False, 0, epoch[0], parts), publish)
    row("reduce_scatter peer-load kernel (+scale, +sum of squares), fp32", ms, rs_bytes)
    out = torch.empty(S, device=dev)
    ms = timed(lambda: dist.reduce_scatter_tensor(out, gfull))
    row("reduce_scatter NCCL, fp32", ms, rs_bytes)
    ok_rs = bool(torch.allclose(gshard, out / W, rtol=1e-4, atol=1e-5))

    # ---- GEMM that consumes the gathered unit
    flops = 2.0 * a.m * a.n * a.k
    w_view = full[4096:4096 + a.n * a.k].view(a.n, a.k)
    pk = peaks()
    t_flops = flops / (pk["bf16_tflops_sustained"] * 1e9)
    t_link = in_bytes / (LINK_GBS * 1e6)
    target = max(t_flops, t_link)
    ms_gemm = timed(lambda: native.gemm(x, w_view, False, False))
    row(f"plain GEMM {a.m}x{a.n}x{a.k} (unit already gathered)", ms_gemm, None, flops)
    ms = timed(lambda: (symm.all_gather(arena, off_sh, S * 2, full, 0, epoch[0], ctas_per_peer=max(4, 64 // W)),
                        native.gemm(x, w_view, False, False)), publish)
    row("peer-load all_gather, then GEMM", ms, None, flops, roofline_ms=round(target, 4), frac_of_roofline=round(target / ms, 3))
    y_ref = native.gemm(x, w_view, False, False).clone()
    ms = timed(lambda: (dist.all_gather_into_tensor(full, shard), native.gemm(x, w_view, False, False)))
    row("NCCL all_gather, then GEMM", ms, None, flops, roofline_ms=round(target, 4), frac_of_roofline=round(target / ms, 3))
    ok_fused = True
    for cc, which in ((0, "pair"), (16, "single"), (32, "single")):
        native.gemm_select(which)

        def pre():
            publish()
            flags.zero_()
        def fused(cc=cc):
            return symm.gemm_all_gather(arena, x, full, off_sh, S, 4096, a.n, flags, cps, 0, epoch[0], copy_ctas=cc)
        ms = timed(fused, pre)
        pre()
        y = fused()
        torch.cuda.synchronize()
        ok_fused = ok_fused and bool(torch.equal(y, y_ref)) and bool(torch.equal(full, ref))
        name = ("CTA-pair kernel, copy role in the idle MMA warps" if which == "pair"
                else f"single-CTA kernel, {cc} copy CTAs")
        row(f"GEMM with the all-gather inside: {name}", ms, None, flops, roofline_ms=round(target, 4),
            frac_of_roofline=round(target / ms, 3))
    native.gemm_select("default")
    native.check_status()
    dist.barrier()
    if rank == 0:
        for r in rows:
            print(json.dumps(r))
        print(json.dumps({"checks": {"gather_equals_nccl": ok_gather, "reduce_scatter_close_to_nccl": ok_rs,
                                     "fused_gemm_bitwise_equals_plain": ok_fused},
                          "roofline": {"flops_ms_at_sustained_peak": round(t_flops, 4), "link_ms_at_770GBs": round(t_link, 4)}}))
    arena.close()
    pdist.cleanup_distributed()


if __name__ == "__main__":
    main()
