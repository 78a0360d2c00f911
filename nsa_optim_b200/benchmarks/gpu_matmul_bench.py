"""GEMM probe: the in-tree tcgen05 bf16 GEMM against the vendor library at LLM shapes.

Reference counterpart (nngabe/nsa_optim): benchmarks/gpu_matmul_bench.py:5-48 times fp16
``torch.matmul`` at three shapes with wall-clock timers.  Here both GEMMs are timed with CUDA
events after warm-up with an L2 flush between iterations, and reported as TFLOP/s and as a
fraction of the measured bf16 peak.

    python -m nsa_optim_b200.benchmarks.gpu_matmul_bench
"""
from __future__ import annotations

import json

import torch

from .kernel_benchmark import peaks, time_ms as time_cuda

SHAPES = [(8192, 8192, 8192), (65536, 8512, 2048), (65536, 2048, 5632), (65536, 11264, 2048), (32768, 32000, 2048)]


def main() -> None:
    from ..ops import native_module
    native = native_module()
    pk = peaks()
    rows = []
    for M, N, K in SHAPES:
        a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
        flops = 2.0 * M * N * K
        ms_own = time_cuda(lambda: native.gemm(a, w, False, False))
        ms_lib = time_cuda(lambda: torch.nn.functional.linear(a, w))
        rows.append({"M": M, "N": N, "K": K, "tcgen05_tflops": flops / ms_own / 1e9, "library_tflops": flops / ms_lib / 1e9,
                     "tcgen05_of_measured_peak": flops / ms_own / 1e9 / pk["bf16_tflops"]})
        print(json.dumps(rows[-1]))


if __name__ == "__main__":
    main()
