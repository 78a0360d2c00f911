"""Kernel micro-benchmarks, timed on the device.

Reference counterpart (nngabe/nsa_optim): benchmarks/kernel_benchmark.py:41-559 and
benchmarks/profile_kernels.py:33-393 time RMSNorm / SwiGLU / RoPE / fused CE with a host
clock around ``cuda.synchronize``.  Here every number is CUDA-event time on the launching
stream after warm-up, with an L2 flush (a write larger than the 126 MB L2) between timed
iterations, and is reported next to the roofline it should be compared with
(``MEASURED_PEAKS.json`` when present, else 6650 GB/s and 1590 TFLOP/s).

    python -m nsa_optim_b200.benchmarks.kernel_benchmark --op gemm --m 8192 --n 8192 --k 8192
    python -m nsa_optim_b200.benchmarks.kernel_benchmark --op all --backend native|torch
"""
from __future__ import annotations

import argparse
import json
import os
from typing import Callable, Dict, List

import torch

from .. import ops


def peaks() -> Dict[str, float]:
    here = os.path.dirname(os.path.abspath(__file__))
    path = os.path.join(here, "..", "..", "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


_flush_buf = None


def flush_l2() -> None:
    global _flush_buf
    if _flush_buf is None:
        _flush_buf = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    _flush_buf.zero_()


def time_ms(fn: Callable[[], None], iters: int = 10, warmup: int = 3, flush: bool = True) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        if flush:
            flush_l2()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    return total / iters


def bench_gemm(m: int, n: int, k: int, a_mn: bool, b_mn: bool, backend: str, iters: int) -> Dict:
    a = torch.randn((k, m) if a_mn else (m, k), device="cuda").bfloat16()
    b = torch.randn((k, n) if b_mn else (n, k), device="cuda").bfloat16()
    if backend == "native":
        nat = ops.native_module()
        out = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
        fn = lambda: nat.gemm(a, b, a_mn, b_mn, out=out)
    else:
        A = a.t() if a_mn else a
        B = b if b_mn else b.t()
        fn = lambda: torch.matmul(A, B)
    ms = time_ms(fn, iters)
    tf = 2.0 * m * n * k / (ms * 1e-3) / 1e12
    pk = peaks()
    return {"op": f"gemm[{'mn' if a_mn else 'k'}{'mn' if b_mn else 'k'}] {m}x{n}x{k}", "backend": backend, "ms": ms,
            "tflops": tf, "frac_of_peak": tf / pk["bf16_tflops"], "peak": f"{pk['bf16_tflops']} TFLOP/s of {pk['source']}"}


MODEL_GEMMS = [(8192, 8192, 8192, False, False), (65536, 8512, 2048, False, False),
               (65536, 2048, 5632, False, False), (65536, 2048, 8512, False, True),
               (8512, 2048, 65536, True, True), (4096, 32000, 2048, False, False)]


def bench_gemm_compare(iters: int) -> List[Dict]:
    """The flagship model's GEMM shapes on the CTA-pair kernel, the single-CTA kernel and the
    library (cuBLAS through torch.matmul), in one process on the same tensors."""
    nat = ops.native_module()
    out = []
    for (m, n, k, a_mn, b_mn) in MODEL_GEMMS:
        a = torch.randn((k, m) if a_mn else (m, k), device="cuda").bfloat16()
        b = torch.randn((k, n) if b_mn else (n, k), device="cuda").bfloat16()
        c = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
        A, B = (a.t() if a_mn else a), (b if b_mn else b.t())
        row = {"op": f"gemm[{'mn' if a_mn else 'k'}{'mn' if b_mn else 'k'}] {m}x{n}x{k}"}
        flops = 2.0 * m * n * k
        for name in ("pair", "single"):
            nat.gemm_select(name)
            try:
                ms = time_ms(lambda: nat.gemm(a, b, a_mn, b_mn, out=c), iters)
            finally:
                nat.gemm_select("default")
            row[f"{name}_ms"], row[f"{name}_tflops"] = ms, flops / (ms * 1e-3) / 1e12
        ms = time_ms(lambda: torch.matmul(A, B, out=c), iters)
        row["library_ms"], row["library_tflops"] = ms, flops / (ms * 1e-3) / 1e12
        row["pair_over_library"] = row["pair_tflops"] / row["library_tflops"]
        out.append(row)
        del a, b, c
    return out


def _bw_row(name: str, backend: str, ms: float, nbytes: float) -> Dict:
    pk = peaks()
    gbs = nbytes / (ms * 1e-3) / 1e9
    return {"op": name, "backend": backend, "ms": ms, "gbs": gbs, "frac_of_peak": gbs / pk["hbm_gbs"],
            "peak": f"{pk['hbm_gbs']} GB/s of {pk['source']}"}


def bench_elementwise(backend: str, rows: int, d: int, ffn: int, iters: int) -> List[Dict]:
    out = []
    x = torch.randn(rows, d, device="cuda").bfloat16().requires_grad_()
    w = torch.ones(d, device="cuda").bfloat16().requires_grad_()
    g = torch.randn(rows, d, device="cuda").bfloat16()
    with ops.backend(backend):
        out.append(_bw_row(f"rmsnorm fwd {rows}x{d}", backend, time_ms(lambda: ops.rms_norm(x, w), iters), 2 * rows * d * 2))
        y = ops.rms_norm(x, w)
        out.append(_bw_row(f"rmsnorm bwd {rows}x{d}", backend,
                           time_ms(lambda: torch.autograd.grad(y, (x, w), g, retain_graph=True), iters), 3 * rows * d * 2))
        a = torch.randn(rows, ffn, device="cuda").bfloat16().requires_grad_()
        b = torch.randn(rows, ffn, device="cuda").bfloat16().requires_grad_()
        gg = torch.randn(rows, ffn, device="cuda").bfloat16()
        out.append(_bw_row(f"swiglu fwd {rows}x{ffn}", backend, time_ms(lambda: ops.swiglu(a, b), iters), 3 * rows * ffn * 2))
        z = ops.swiglu(a, b)
        out.append(_bw_row(f"swiglu bwd {rows}x{ffn}", backend,
                           time_ms(lambda: torch.autograd.grad(z, (a, b), gg, retain_graph=True), iters), 5 * rows * ffn * 2))
        q = torch.randn(1, rows, 32, 128, device="cuda").bfloat16()
        cos, sin = ops.oracle.rope_tables(128, rows, 1e4, device="cuda")
        out.append(_bw_row(f"rope fwd {rows}x32x128", backend, time_ms(lambda: ops.rope(q, cos, sin), iters), 2 * q.numel() * 2))
    return out


def bench_attention(backend: str, T: int, iters: int, window: int = 0) -> List[Dict]:
    """Causal GQA attention 32 q / 2 kv heads of 128, forward and forward+backward."""
    q = torch.randn(1, T, 32, 128, device="cuda").bfloat16().requires_grad_()
    k = torch.randn(1, T, 2, 128, device="cuda").bfloat16().requires_grad_()
    v = torch.randn(1, T, 2, 128, device="cuda").bfloat16().requires_grad_()
    keys = min(window, T) if window else T / 2
    flops_fwd = 4.0 * T * keys * 128 * 32
    pk = peaks()
    rows = []
    with ops.backend(backend):
        def fwd():
            with torch.no_grad():
                ops.attention(q, k, v, True, window)
        def fb():
            o = ops.attention(q, k, v, True, window)
            o.backward(torch.ones_like(o))
        for name, fn, mult in (("fwd", fwd, 1.0), ("fwd+bwd", fb, 3.5)):
            ms = time_ms(fn, iters)
            tf = flops_fwd * mult / (ms * 1e-3) / 1e12
            rows.append({"op": f"attention {name} T={T} window={window} 32q/2kv hd128", "backend": backend, "ms": ms,
                         "tflops": tf, "frac_of_peak": tf / pk["bf16_tflops"], "peak": f"{pk['bf16_tflops']} TFLOP/s of {pk['source']}"})
    if backend == "native" and window == 0:
        rows += _attention_library_rows(q, k, v, flops_fwd, iters)
    return rows


def _attention_library_rows(q, k, v, flops_fwd: float, iters: int) -> List[Dict]:
    """The same problem on the installed library kernels (flash_attn, PyTorch SDPA), local tensors
    only: the bar the native rows are read against, not a path of the framework."""
    rows = []
    T = q.shape[1]

    def add(label, fwd, fb):
        for name, fn, mult in (("fwd", fwd, 1.0), ("fwd+bwd", fb, 3.5)):
            try:
                ms = time_ms(fn, iters)
            except Exception as e:                       # a library that cannot run this shape here
                rows.append({"op": f"attention {name} T={T} ({label})", "backend": "library", "unavailable": str(e)[:120]})
                return
            rows.append({"op": f"attention {name} T={T} ({label})", "backend": "library", "ms": ms,
                         "tflops": flops_fwd * mult / (ms * 1e-3) / 1e12})

    try:
        from flash_attn import flash_attn_func

        def fa_fwd():
            with torch.no_grad():
                flash_attn_func(q, k, v, causal=True)

        def fa_fb():
            o = flash_attn_func(q, k, v, causal=True)
            o.backward(torch.ones_like(o))
        add("flash_attn", fa_fwd, fa_fb)
    except ImportError:
        pass
    qs, ks, vs = (t.transpose(1, 2) for t in (q, k, v))

    def sd_fwd():
        with torch.no_grad():
            torch.nn.functional.scaled_dot_product_attention(qs, ks, vs, is_causal=True, enable_gqa=True)

    def sd_fb():
        o = torch.nn.functional.scaled_dot_product_attention(qs, ks, vs, is_causal=True, enable_gqa=True)
        o.backward(torch.ones_like(o))
    add("torch SDPA", sd_fwd, sd_fb)
    return rows


def bench_mixers(backend: str, T: int, iters: int) -> List[Dict]:
    """Gated delta rule (16 heads, K128/V256) and Mamba-2 SSD (64 heads of 64, N128), fwd+bwd."""
    rows = []
    with ops.backend(backend):
        q = torch.nn.functional.normalize(torch.randn(1, T, 16, 128, device="cuda"), dim=-1).bfloat16().requires_grad_()
        k = torch.nn.functional.normalize(torch.randn(1, T, 16, 128, device="cuda"), dim=-1).bfloat16().requires_grad_()
        v = torch.randn(1, T, 16, 256, device="cuda").bfloat16().requires_grad_()
        g = (-torch.rand(1, T, 16, device="cuda") * 0.1).requires_grad_()
        beta = torch.rand(1, T, 16, device="cuda").requires_grad_()
        def gdn():
            o = ops.gated_delta_rule(q, k, v, g, beta)
            o.backward(torch.ones_like(o))
        rows.append({"op": f"gated_delta_rule fwd+bwd T={T}", "backend": backend, "ms": time_ms(gdn, iters)})
        x = torch.randn(1, T, 64, 64, device="cuda").bfloat16().requires_grad_()
        dt = (torch.rand(1, T, 64, device="cuda") * 0.1 + 0.001).requires_grad_()
        A = (-torch.rand(64, device="cuda") * 4 - 0.5).requires_grad_()
        Bm = torch.randn(1, T, 1, 128, device="cuda").bfloat16().requires_grad_()
        Cm = torch.randn(1, T, 1, 128, device="cuda").bfloat16().requires_grad_()
        def ssd():
            y = ops.ssd_scan(x, dt, A, Bm, Cm, None, 256)
            y.backward(torch.ones_like(y))
        rows.append({"op": f"ssd_scan fwd+bwd T={T}", "backend": backend, "ms": time_ms(ssd, iters)})
    return rows


def bench_nsa(backend: str, T: int, iters: int) -> List[Dict]:
    """Three-branch sparse attention (32 query / 2 KV heads, head_dim 128, compression 32/16,
    top-16 blocks of 64, window 512): forward and forward+backward."""
    torch.manual_seed(0)
    q = torch.randn(1, T, 32, 128, device="cuda").bfloat16().requires_grad_(True)
    k = torch.randn(1, T, 2, 128, device="cuda").bfloat16().requires_grad_(True)
    v = torch.randn(1, T, 2, 128, device="cuda").bfloat16().requires_grad_(True)
    g = torch.rand(1, T, 32, device="cuda").bfloat16()
    rows = []
    with ops.backend(backend):
        with torch.no_grad():
            ms = time_ms(lambda: ops.nsa_attention(q, k, v, g, g, g), iters)
        rows.append({"op": f"nsa_attention fwd T={T}", "backend": backend, "ms": ms})

        def fb():
            ops.nsa_attention(q, k, v, g, g, g).sum().backward()
        rows.append({"op": f"nsa_attention fwd+bwd T={T}", "backend": backend, "ms": time_ms(fb, iters)})
    return rows


def bench_comm(iters: int, world: int = 4, shard_mb: int = 32) -> List[Dict]:
    """Peer-memory kernels with the ranks emulated on ONE GPU (every "peer" buffer is local and
    every flag is set beforehand, so no kernel waits for another launch): the figures are the
    kernels' local memory throughput, an upper bound of what NVLink can feed them."""
    from ..parallel import symm
    from ..parallel.symm import SymmetricArena, _round_up
    W = world
    S = shard_mb * (1 << 20) // 2                      # bf16 elements per shard
    payload = S * 2 + W * S * 4 + 8192
    total = _round_up(8 * 32 * 4, 4096) + _round_up(payload, 4096)
    bufs = [torch.zeros(total, dtype=torch.uint8, device="cuda") for _ in range(W)]
    arenas = [SymmetricArena(payload, 8, r, W, torch.device("cuda"), local_peers=bufs) for r in range(W)]
    off_sh = [a.alloc(S * 2) for a in arenas][0]
    off_g = [a.alloc(W * S * 4) for a in arenas][0]
    for a in arenas:
        a.view(off_sh, S, torch.bfloat16).normal_()
        a.view(off_g, W * S, torch.float32).normal_()
        symm.signal(a, 0, 1)
    torch.cuda.synchronize()
    a0 = arenas[0]
    pk = peaks()
    rows = []
    full = torch.empty(W * S, dtype=torch.bfloat16, device="cuda")
    ms = time_ms(lambda: symm.all_gather(a0, off_sh, S * 2, full, 0, 1), iters)
    rows.append(_bw_row(f"p2p all_gather W={W} shard={shard_mb}MB (emulated)", "native", ms, 2.0 * W * S * 2))
    gs = torch.zeros(S, device="cuda")
    parts = torch.zeros(symm.reduce_scatter_parts(), device="cuda")
    ms = time_ms(lambda: symm.reduce_scatter(a0, off_g, gs, 1.0 / W, True, 0, 1, parts), iters)
    rows.append(_bw_row(f"p2p reduce_scatter+scale+sumsq W={W} (emulated)", "native", ms, (W + 2.0) * S * 4))
    M, K = 65536, 2048
    N = (W * S - 4096) // K // 8 * 8
    N = min(N, 8512)
    cps = max(1, min(1024, (S * 2) // (256 << 10)))
    x = torch.randn(M, K, device="cuda").bfloat16()
    nat = ops.native_module()
    symm.all_gather(a0, off_sh, S * 2, full, 0, 1)
    w_view = full[4096:4096 + N * K].view(N, K)
    flops = 2.0 * M * N * K
    ms = time_ms(lambda: nat.gemm(x, w_view, False, False), iters)
    rows.append({"op": f"plain gemm {M}x{N}x{K} (unit already gathered)", "backend": "native", "ms": ms, "tflops": flops / ms / 1e9})
    for which in ("pair", "single"):
        nat.gemm_select(which)

        def fused():
            flags = torch.zeros(W * cps, dtype=torch.int32, device="cuda")
            symm.gemm_all_gather(a0, x, full, off_sh, S, 4096, N, flags, cps, 0, 1)
        try:
            ms = time_ms(fused, iters)
        finally:
            nat.gemm_select("default")
        rows.append({"op": f"gemm + fused all_gather {M}x{N}x{K} W={W} (emulated, {which} kernel)", "backend": "native", "ms": ms,
                     "tflops": flops / ms / 1e9, "frac_of_peak": flops / ms / 1e9 / pk["bf16_tflops"],
                     "gathered_mb": W * S * 2 / 2**20})
    return rows


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", default="all", choices=["all", "gemm", "gemm_compare", "elementwise", "attention", "mixers", "nsa", "comm"])
    ap.add_argument("--backend", default="native", choices=["native", "torch"])
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--a_mn", action="store_true")
    ap.add_argument("--b_mn", action="store_true")
    ap.add_argument("--rows", type=int, default=65536)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--seq", type=int, default=16384)
    ap.add_argument("--window", type=int, default=0)
    a = ap.parse_args()
    rows: List[Dict] = []
    if a.op in ("all", "gemm"):
        if a.op == "gemm":
            rows.append(bench_gemm(a.m, a.n, a.k, a.a_mn, a.b_mn, a.backend, a.iters))
        else:
            for (m, n, k, am, bm) in MODEL_GEMMS:
                rows.append(bench_gemm(m, n, k, am, bm, a.backend, a.iters))
    if a.op == "gemm_compare":
        rows += bench_gemm_compare(a.iters)
    if a.op in ("all", "elementwise"):
        rows += bench_elementwise(a.backend, a.rows, 2048, 5632, a.iters)
    if a.op in ("all", "attention"):
        rows += bench_attention(a.backend, a.seq, a.iters, a.window)
    if a.op in ("all", "mixers"):
        rows += bench_mixers(a.backend, a.seq, a.iters)
    if a.op == "nsa":
        rows += bench_nsa(a.backend, a.seq, a.iters)
    if a.op == "comm":
        rows += bench_comm(a.iters)
    for r in rows:
        print(json.dumps(r))
    if a.backend == "native":
        ops.native_module().check_status()


if __name__ == "__main__":
    main()
