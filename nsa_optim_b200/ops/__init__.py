"""Op dispatch: every model and optimizer calls the functions in this module.

CUDA tensors go to the hand-written sm_100a kernels (``ops/native.py`` over
``ops/csrc/*.cu``); CPU tensors, and CUDA tensors when the backend is forced to
``torch``, go to ``ops/torch_impl.py``.  The ``torch`` backend on a GPU is the
library-kernel comparison path (cuBLAS / SDPA), never the default.

Backend selection: environment variable ``NSA_B200_BACKEND`` = ``auto`` (default),
``native`` or ``torch``; or :func:`set_backend` / :func:`backend` at run time.
With ``auto`` on a CUDA tensor the native library must be loadable: a missing
library raises instead of silently falling back.
"""
from __future__ import annotations

import contextlib
import os
from typing import Optional

import torch
from torch import Tensor

from . import oracle, torch_impl

_BACKEND = os.environ.get("NSA_B200_BACKEND", "auto").lower()
_native = None
_native_err: Optional[BaseException] = None


def set_backend(name: str) -> None:
    global _BACKEND
    if name not in ("auto", "native", "torch", "library"):
        raise ValueError(name)
    _BACKEND = name


def get_backend() -> str:
    return _BACKEND


@contextlib.contextmanager
def backend(name: str):
    prev = get_backend()
    set_backend(name)
    try:
        yield
    finally:
        set_backend(prev)


def native_module():
    """The loaded native op module, or raise with the reason it cannot be loaded."""
    global _native, _native_err
    if _native is None and _native_err is None:
        try:
            from . import native as _n
            _n.load()
            _native = _n
        except BaseException as exc:  # noqa: BLE001 - reported verbatim to the caller
            _native_err = exc
    if _native is None:
        raise RuntimeError(
            "nsa_optim_b200 native library is not available on this CUDA machine "
            f"({_native_err!r}). Build it with `python -m nsa_optim_b200.ops.build` "
            "or set NSA_B200_BACKEND=torch to run the library-kernel comparison path."
        )
    return _native


def native_available() -> bool:
    try:
        native_module()
        return True
    except RuntimeError:
        return False


def _use_native(t: Tensor, op: str) -> bool:
    if not t.is_cuda or _BACKEND == "torch":
        return False
    n = native_module()
    return n.supports(op, t)


def native_op_names():
    """Names of the ops that run as native kernels for bf16 CUDA tensors."""
    return sorted(native_module().SUPPORTED)


def _library(t: Tensor):
    """The third-party-library implementations, when the diagnostic "library" backend is selected
    (see ``library_impl``); each returns None when its library cannot serve the call, and the op then
    runs on the native kernel."""
    if _BACKEND == "library" and t.is_cuda:
        from . import library_impl
        return library_impl
    return None


# ------------------------------------------------------------------ ops
def linear(x: Tensor, weight: Tensor) -> Tensor:
    """y = x @ weight^T (weight (out, in), no bias)."""
    if _library(x) is not None:
        return _library(x).linear(x, weight)
    if _use_native(x, "linear"):
        return native_module().linear(x, weight)
    return torch_impl.linear(x, weight)


def multi_linear(x: Tensor, weights) -> tuple:
    """Projections of one input by several weights, (x W_0^T, x W_1^T, ...).  On the native backend
    the input gradient is accumulated inside the GEMM epilogues instead of by separate additions."""
    weights = list(weights)
    if _library(x) is None and _use_native(x, "linear"):
        return native_module().multi_linear(x, weights)
    return tuple(linear(x, w) for w in weights)


def rms_norm(x: Tensor, weight: Tensor, eps: float = 1e-6) -> Tensor:
    if _library(x) is not None:
        y = _library(x).rms_norm(x, weight, eps)
        if y is not None:
            return y
    if _use_native(x, "rms_norm"):
        return native_module().rms_norm(x, weight, eps)
    return torch_impl.rms_norm(x, weight, eps)


def rms_norm_skip(x: Tensor, weight: Tensor, eps: float = 1e-6):
    """(rmsnorm(x) * weight, x).  Use the second value, not ``x``, for the residual branch: the
    native backward then adds the residual gradient inside the norm's backward kernel."""
    if _library(x) is not None:
        return rms_norm(x, weight, eps), x
    if _use_native(x, "rms_norm"):
        return native_module().rms_norm_skip(x, weight, eps)
    return torch_impl.rms_norm_skip(x, weight, eps)


def add_rms_norm(x: Tensor, r: Tensor, weight: Tensor, eps: float = 1e-6):
    """(h, rmsnorm(h) * weight) with h = x + r, one kernel each way on the native path."""
    if _library(x) is not None:
        h = x + r
        return h, rms_norm(h, weight, eps)
    if _use_native(x, "rms_norm"):
        return native_module().add_rms_norm(x, r, weight, eps)
    return torch_impl.add_rms_norm(x, r, weight, eps)


def gated_rms_norm(x: Tensor, gate: Tensor, weight: Tensor, eps: float = 1e-6,
                   norm_before_gate: bool = True) -> Tensor:
    if _use_native(x, "gated_rms_norm"):
        return native_module().gated_rms_norm(x, gate, weight, eps, norm_before_gate)
    return torch_impl.gated_rms_norm(x, gate, weight, eps, norm_before_gate)


def swiglu(gate: Tensor, up: Tensor) -> Tensor:
    if _library(gate) is not None:
        y = _library(gate).swiglu(gate, up)
        if y is not None:
            return y
    if _use_native(gate, "swiglu"):
        return native_module().swiglu(gate, up)
    return torch_impl.swiglu(gate, up)


def l2_norm(x: Tensor, eps: float = 1e-6) -> Tensor:
    if _use_native(x, "l2_norm"):
        return native_module().l2_norm(x, eps)
    return torch_impl.l2_norm(x, eps)


def rope(x: Tensor, cos: Tensor, sin: Tensor) -> Tensor:
    """x (B,T,H,D), cos/sin (T, D/2) fp32."""
    if _use_native(x, "rope"):
        return native_module().rope(x, cos, sin)
    return torch_impl.rope(x, cos, sin)


def embedding(ids: Tensor, weight: Tensor) -> Tensor:
    if _use_native(weight, "embedding"):
        return native_module().embedding(ids, weight)
    return torch_impl.embedding(ids, weight)


def attention(q: Tensor, k: Tensor, v: Tensor, causal: bool = True, window: int = 0,
              scale: Optional[float] = None) -> Tensor:
    if _library(q) is not None:
        o = _library(q).attention(q, k, v, causal, window, scale)
        if o is not None:
            return o
    if _use_native(q, "attention") and q.shape[1] == k.shape[1]:
        return native_module().attention(q, k, v, causal, window, scale)
    return torch_impl.attention(q, k, v, causal, window, scale)


def nsa_attention(q, k, v, g_cmp, g_slc, g_swa, cmp_block=32, cmp_stride=16, sel_block=64,
                  top_n=16, window=512, scale=None, gate_logits: Optional[Tensor] = None) -> Tensor:
    """Native sparse attention: compressed, selected and sliding-window branches combined with
    per-(token, head) gates.  The gates are either three tensors (B, T, Hq) already in (0, 1), or
    ``gate_logits`` (B, T, 3*Hq) in the order compressed, selected, window, whose sigmoid the native
    combine kernel takes itself."""
    if gate_logits is not None and not (_use_native(q, "nsa_attention") and _library(q) is None):
        Hq = q.shape[2]
        g_cmp, g_slc, g_swa = torch.sigmoid(gate_logits.float()).to(q.dtype)[..., :3 * Hq].split(Hq, dim=-1)
        gate_logits = None
    if _library(q) is not None:
        o = _library(q).nsa_attention(q, k, v, g_cmp, g_slc, g_swa, sel_block, top_n, window, scale)
        if o is not None:
            return o
    if _use_native(q, "nsa_attention"):
        return native_module().nsa_attention(q, k, v, g_cmp, g_slc, g_swa, cmp_block, cmp_stride,
                                             sel_block, top_n, window, scale, gate_logits)
    return torch_impl.nsa_attention(q, k, v, g_cmp, g_slc, g_swa, cmp_block, cmp_stride,
                                    sel_block, top_n, window, scale)


def nsa_attention_indexed(q, k, v, idx, g_slc, g_swa, sel_block=64, window=512, scale=None) -> Tensor:
    """Two-branch sparse attention (selected blocks ``idx`` (B, Hkv, T, n) + sliding window)."""
    if _use_native(q, "nsa_attention") and _library(q) is None:
        return native_module().nsa_attention_indexed(q, k, v, idx, g_slc, g_swa, sel_block, window, scale)
    return torch_impl.nsa_attention_indexed(q, k, v, idx, g_slc, g_swa, sel_block, window, scale)


def causal_conv1d(x: Tensor, weight: Tensor, bias: Optional[Tensor], activation: bool = True) -> Tensor:
    if _use_native(x, "causal_conv1d"):
        return native_module().causal_conv1d(x, weight, bias, activation)
    return torch_impl.causal_conv1d(x, weight, bias, activation)


def ssd_scan(x, dt, A, Bm, Cm, D=None, chunk: int = 256) -> Tensor:
    if _use_native(x, "ssd_scan"):
        return native_module().ssd_scan(x, dt, A, Bm, Cm, D, chunk)
    return torch_impl.ssd_scan(x, dt, A, Bm, Cm, D, chunk)


def gated_delta_rule(q, k, v, g, beta, scale=None, chunk: int = 64) -> Tensor:
    if _library(q) is not None:
        o = _library(q).gated_delta_rule(q, k, v, g, beta, scale)
        if o is not None:
            return o
    if _use_native(q, "gated_delta_rule"):
        return native_module().gated_delta_rule(q, k, v, g, beta, scale, chunk)
    return torch_impl.gated_delta_rule(q, k, v, g, beta, scale, chunk)


def linear_cross_entropy(hidden: Tensor, weight: Tensor, labels: Tensor, ignore_index: int = -100,
                         chunk: int = 4096) -> Tensor:
    if _library(hidden) is not None:
        loss = _library(hidden).linear_cross_entropy(hidden, weight, labels, ignore_index)
        if loss is not None:
            return loss
    if _use_native(hidden, "linear_cross_entropy"):
        return native_module().linear_cross_entropy(hidden, weight, labels, ignore_index, chunk)
    return torch_impl.linear_cross_entropy(hidden, weight, labels, ignore_index, chunk)
