"""The "library" backend: the same ops computed by the third-party kernel libraries the reference
builds on, where they are installed.  It exists for one purpose: a same-box, same-model,
same-step comparison of this framework's own kernels against the library kernels (the reference
itself cannot be imported offline).  It is never the product path and never reported as the
reference.

What each op calls (reference call sites in parentheses):

  linear                  torch ``F.linear`` -> cuBLAS                         (models/kernels.py:123-125)
  rms_norm                Liger ``LigerRMSNormFunction``                       (models/kernels.py:319-324)
  swiglu                  Liger ``LigerSiLUMulFunction``                       (models/kernels.py:327-340)
  linear_cross_entropy    Liger ``LigerFusedLinearCrossEntropyFunction``       (models/transformer.py:33-36)
  attention               ``flash_attn_func`` (causal, optional window)        (models/hybrid.py:360-366)
  gated_delta_rule        (fla ``chunk_gated_delta_rule`` faulted on B200, see below: native)   (models/hybrid.py:252-263)
  nsa_attention           fla ``parallel_nsa`` (compression block = selection block = 64: fla's
                          definition, not the 32/16 of the named config)       (models/transformer.py:254-268)

Ops with no installed library counterpart (Mamba-2 SSD scan and causal conv1d: ``mamba_ssm`` and
``causal_conv1d`` are absent; RoPE, embedding, the gated norm, the optimizers) stay on this
framework's kernels, and :func:`report` says so.  Every library kernel receives local tensors
only.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch
import torch.nn.functional as F
from torch import Tensor

_used: Dict[str, str] = {}
_missing: Dict[str, str] = {}


def _note(op: str, what: str) -> None:
    _used.setdefault(op, what)


def _fail(op: str, exc: BaseException) -> None:
    _missing.setdefault(op, f"{type(exc).__name__}: {exc}"[:160])


def report() -> Dict[str, Dict[str, str]]:
    """Which library served which op so far, and which ops fell back to native kernels and why."""
    return {"library": dict(_used), "native_instead": dict(_missing)}


def linear(x: Tensor, weight: Tensor) -> Tensor:
    _note("linear", "torch F.linear (cuBLAS)")
    return F.linear(x, weight)


def rms_norm(x: Tensor, weight: Tensor, eps: float = 1e-6) -> Optional[Tensor]:
    try:
        from liger_kernel.ops.rms_norm import LigerRMSNormFunction
        y = LigerRMSNormFunction.apply(x, weight.to(x.dtype), eps, 0.0, "llama", False)
        _note("rms_norm", "liger_kernel LigerRMSNormFunction")
        return y
    except Exception as exc:  # noqa: BLE001 - diagnostic backend: any failure means "use native"
        _fail("rms_norm", exc)
        return None


def swiglu(gate: Tensor, up: Tensor) -> Optional[Tensor]:
    try:
        from liger_kernel.ops.swiglu import LigerSiLUMulFunction
        y = LigerSiLUMulFunction.apply(gate.contiguous(), up.contiguous())
        _note("swiglu", "liger_kernel LigerSiLUMulFunction")
        return y
    except Exception as exc:  # noqa: BLE001
        _fail("swiglu", exc)
        return None


def linear_cross_entropy(hidden: Tensor, weight: Tensor, labels: Tensor, ignore_index: int = -100) -> Optional[Tensor]:
    try:
        from liger_kernel.ops.fused_linear_cross_entropy import LigerFusedLinearCrossEntropyFunction
        out = LigerFusedLinearCrossEntropyFunction.apply(hidden.reshape(-1, hidden.shape[-1]), weight,
                                                         labels.reshape(-1), None, None, ignore_index)
        loss = out[0] if isinstance(out, (tuple, list)) else out
        _note("linear_cross_entropy", "liger_kernel LigerFusedLinearCrossEntropyFunction")
        return loss
    except Exception as exc:  # noqa: BLE001
        _fail("linear_cross_entropy", exc)
        return None


def attention(q: Tensor, k: Tensor, v: Tensor, causal: bool = True, window: int = 0,
              scale: Optional[float] = None) -> Optional[Tensor]:
    try:
        from flash_attn import flash_attn_func
        ws = (window - 1, 0) if window > 0 else (-1, -1)
        o = flash_attn_func(q, k, v, softmax_scale=scale, causal=causal, window_size=ws)
        _note("attention", "flash_attn flash_attn_func")
        return o
    except Exception as exc:  # noqa: BLE001
        _fail("attention", exc)
        return None


def gated_delta_rule(q, k, v, g, beta, scale=None) -> Optional[Tensor]:
    # fla 0.5.1's chunk_gated_delta_rule is not called: on a B200 its backward (prepare_wy_repr_bwd,
    # under Triton's autotuner) raised "CUDA error: misaligned address" at T = 65536, 16 heads, key
    # width 128, value width 256, which ended the process.  A kernel that has faulted is not run
    # again; the op stays on this framework's kernels in the library arm.
    _missing.setdefault("gated_delta_rule", "fla chunk_gated_delta_rule backward faulted on B200 (misaligned address); "
                                            "not run again")
    return None


def nsa_attention(q, k, v, g_cmp, g_slc, g_swa, sel_block=64, top_n=16, window=512, scale=None) -> Optional[Tensor]:
    try:
        from fla.ops.nsa import parallel_nsa
        o = parallel_nsa(q, k, v, g_cmp, g_slc, g_swa, block_counts=top_n, block_size=sel_block,
                         window_size=window, scale=scale)
        _note("nsa_attention", "fla parallel_nsa (compression block 64, its own definition)")
        return o
    except Exception as exc:  # noqa: BLE001
        _fail("nsa_attention", exc)
        return None
