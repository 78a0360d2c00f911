"""ctypes bindings and autograd wrappers for the sm_100a kernels in ``ops/csrc``.

The shared library ``libnsa_b200.so`` lives beside this file (built by ``ops/build.py``) and
exports plain C entry points that take device pointers, sizes and a stream; output tensors
are allocated here with PyTorch.  Each differentiable op is one ``autograd.Function`` whose
forward and backward both call native kernels.  ``SUPPORTED`` lists the ops that have a
native implementation; ``ops/__init__.py`` consults :func:`supports`.

Kernel failures do not raise from the device: kernels record a status block in pinned host
memory (bounded waits, argument checks); :func:`check_status` turns it into an exception.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_long, c_longlong, c_void_p
from typing import Optional, Tuple

import torch
from torch import Tensor

from . import quant, torch_impl

_LIB_PATH = os.environ.get("NSA_B200_LIB") or os.path.join(os.path.dirname(os.path.abspath(__file__)), "libnsa_b200.so")
_lib: Optional[ctypes.CDLL] = None

SUPPORTED = {
    "linear", "rms_norm", "gated_rms_norm", "swiglu", "l2_norm", "rope", "embedding",
    "causal_conv1d", "linear_cross_entropy", "adamw", "adamw_lowbit", "gated_delta_rule",
    "attention", "nsa_attention", "ssd_scan",
}

STATUS_NAMES = {
    101: "timeout waiting for a TMA stage (smem full barrier)",
    102: "timeout waiting for a free smem stage (smem empty barrier)",
    103: "timeout waiting for an accumulator (tmem full barrier)",
    104: "timeout waiting for a free accumulator (tmem empty barrier)",
    201: "timeout waiting for a flag written by a peer GPU",
    202: "timeout waiting for a flag written by another CTA",
    301: "bad argument",
    302: "an index read from a tensor was out of range (debug build)",
}


# Shapes a native kernel does not cover are computed by the PyTorch implementation of the same op.
# Every such call is counted per op, so that a benchmark or a test can show that none of its work
# took that route (``fallback_counts()``; ``NSA_B200_STRICT=1`` turns a fallback into an error).
_fallbacks: dict = {}
_STRICT = os.environ.get("NSA_B200_STRICT", "") not in ("", "0")


def _fallback(op: str, why: str = "") -> None:
    _fallbacks[op] = _fallbacks.get(op, 0) + 1
    if _STRICT:
        raise RuntimeError(f"native op '{op}' does not cover this call ({why}) and NSA_B200_STRICT is set")


def fallback_counts(reset: bool = False) -> dict:
    out = dict(_fallbacks)
    if reset:
        _fallbacks.clear()
    return out


def lib_path() -> str:
    return _LIB_PATH


def load() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            raise FileNotFoundError(f"{_LIB_PATH} is missing; run `python -m nsa_optim_b200.ops.build`")
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.nsa_last_error.restype = ctypes.c_char_p
        _lib.nsa_launch_count.restype = c_longlong
        _lib.nsa_conv1d_bwd_parts.restype = c_long
    return _lib


def supports(op: str, t: Tensor) -> bool:
    if op not in SUPPORTED or not t.is_cuda:
        return False
    if op in ("adamw", "adamw_lowbit"):
        return t.dtype in (torch.bfloat16, torch.float32)
    if op == "embedding":
        return t.dtype == torch.bfloat16
    return t.dtype == torch.bfloat16


def _check(rc: int) -> None:
    if rc != 0:
        raise RuntimeError(f"nsa_optim_b200 native call failed ({rc}): {load().nsa_last_error().decode()}")


def _stream() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _p(t: Optional[Tensor]) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


def launch_count() -> int:
    return int(load().nsa_launch_count())


def reset_launch_count() -> None:
    load().nsa_launch_count_reset()


def read_status(reset: bool = True) -> Tuple[int, int, int, int]:
    out = (c_int * 4)()
    _check(load().nsa_status_read(out, c_int(1 if reset else 0)))
    return tuple(int(v) for v in out)


# --------------------------------------------------------------------------------------
# Output allocation.  With NSA_B200_DEBUG_CANARY=1 every tensor a wrapper allocates for a kernel
# sits between two 4 KB guard zones filled with a pattern; ``check_canaries()`` (also run by
# ``check_status()``) verifies them, which catches a kernel writing past either end of its
# output: the stand-in for a memory sanitizer on machines where none may be run.
# --------------------------------------------------------------------------------------
_CANARY = os.environ.get("NSA_B200_DEBUG_CANARY", "") not in ("", "0")
_GUARD = 4096
_GUARD_BYTE = 0xA5
_guards: list = []


def _shape_of(size) -> tuple:
    if len(size) == 1 and isinstance(size[0], (tuple, list, torch.Size)):
        return tuple(int(x) for x in size[0])
    return tuple(int(x) for x in size)


def _guarded(shape, dtype, device, zero: bool) -> Tensor:
    dtype = dtype or torch.get_default_dtype()
    n = 1
    for d in shape:
        n *= d
    nbytes = n * torch.empty((), dtype=dtype).element_size()
    pad = (-nbytes) % 256
    buf = torch.empty(_GUARD + nbytes + pad + _GUARD, dtype=torch.uint8, device=device)
    buf[:_GUARD].fill_(_GUARD_BYTE)
    buf[_GUARD + nbytes:].fill_(_GUARD_BYTE)
    _guards.append((buf, nbytes))
    out = buf[_GUARD:_GUARD + nbytes].view(dtype).view(shape)
    return out.zero_() if zero else out


def _empty(*size, dtype=None, device=None) -> Tensor:
    if _CANARY and device is not None and torch.device(device).type == "cuda":
        return _guarded(_shape_of(size), dtype, device, False)
    return torch.empty(*size, dtype=dtype, device=device)


def _zeros(*size, dtype=None, device=None) -> Tensor:
    if _CANARY and device is not None and torch.device(device).type == "cuda":
        return _guarded(_shape_of(size), dtype, device, True)
    return torch.zeros(*size, dtype=dtype, device=device)


def _empty_like(t: Tensor, dtype=None) -> Tensor:
    if _CANARY and t.is_cuda:
        return _guarded(tuple(t.shape), dtype or t.dtype, t.device, False)
    return torch.empty_like(t, dtype=dtype, memory_format=torch.contiguous_format)


def _zeros_like(t: Tensor, dtype=None) -> Tensor:
    if _CANARY and t.is_cuda:
        return _guarded(tuple(t.shape), dtype or t.dtype, t.device, True)
    return torch.zeros_like(t, dtype=dtype, memory_format=torch.contiguous_format)


def check_canaries() -> int:
    """Verify and release the guard zones recorded so far; returns how many buffers were checked."""
    torch.cuda.synchronize()
    n = len(_guards)
    for k, (buf, nbytes) in enumerate(_guards):
        head_ok = bool((buf[:_GUARD] == _GUARD_BYTE).all())
        tail_ok = bool((buf[_GUARD + nbytes:] == _GUARD_BYTE).all())
        if not (head_ok and tail_ok):
            _guards.clear()
            side = "before" if not head_ok else "after"
            raise RuntimeError(f"guard zone {side} kernel output #{k} ({nbytes} bytes) was overwritten")
    _guards.clear()
    return n


def check_status(sync: bool = True) -> None:
    """Raise if any kernel since the last check reported a failure."""
    if sync and torch.cuda.is_available():
        torch.cuda.synchronize()
    if _CANARY:
        check_canaries()
    code, block, info, count = read_status(reset=True)
    if code != 0:
        raise RuntimeError(f"native kernel reported status {code} ({STATUS_NAMES.get(code, 'unknown')}); "
                           f"block {block}, detail {info}, {count} report(s)")


# --------------------------------------------------------------------------------------
# GEMM
# --------------------------------------------------------------------------------------
def _as_2d(x: Tensor) -> Tensor:
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(-1) != 1 or (x2.stride(0) % 8) or (x2.data_ptr() % 16):
        x2 = x2.contiguous()
    return x2


_SPLITK_MAX = int(os.environ.get("NSA_B200_SPLITK_MAX", "2"))
_gemm_which = "default"


def split_k_choice(M: int, N: int, K: int, clusters: int = 74) -> int:
    """Parts to cut the reduction of an M x N x K GEMM into.  The pair kernel gives each CTA pair
    256 x 256 tiles; with few tiles and a long reduction (weight gradients: K = tokens) the last wave
    is mostly empty, and splitting the reduction fills it.  Two parts added into a zeroed fp32 C
    give the same bits in either order, so the default limit of 2 keeps results reproducible;
    ``NSA_B200_SPLITK_MAX`` raises it."""
    tiles = -(-M // 256) * -(-N // 256)
    if K < 8192 or M <= 128 or tiles >= 6 * clusters:
        return 1

    def eff(S):
        w = tiles * S / clusters
        return w / -(-w // 1)

    best = max(range(1, _SPLITK_MAX + 1), key=lambda S: eff(S) - 0.01 * S)
    return best if eff(best) > eff(1) + 0.04 else 1


def gemm(a: Tensor, b: Tensor, a_mn: bool, b_mn: bool, out: Optional[Tensor] = None,
         out_dtype: torch.dtype = torch.bfloat16, accumulate: bool = False, max_ctas: int = 0,
         split_k: Optional[int] = None) -> Tensor:
    """C = op(A) op(B): a_mn False -> A is (M, K), True -> A is (K, M); b_mn False -> B is (N, K),
    True -> B is (K, N).  Row pitches may exceed the logical width (sliced views).  ``split_k``
    (default: chosen by :func:`split_k_choice`) cuts the reduction into parts that run on different
    CTA pairs and meet in fp32 through TMA reduce-add stores."""
    a, b = _as_2d(a), _as_2d(b)
    M, K = (a.shape[1], a.shape[0]) if a_mn else (a.shape[0], a.shape[1])
    N, Kb = (b.shape[1], b.shape[0]) if b_mn else (b.shape[0], b.shape[1])
    if K != Kb:
        raise ValueError(f"gemm: reduction sizes differ ({K} vs {Kb})")
    if out is None:
        out = _empty(M, N, dtype=out_dtype, device=a.device)
    if split_k is None:
        split_k = split_k_choice(M, N, K) if (max_ctas == 0 and _gemm_which != "single") else 1
    if split_k > 1 and M > 128:
        direct = out.dtype == torch.float32 and out.stride(1) == 1 and out.stride(0) % 4 == 0 and out.data_ptr() % 16 == 0
        if direct:
            ws = out
            if not accumulate:
                ws.zero_()
        else:
            ws = out.float() if accumulate else _zeros(M, N, dtype=torch.float32, device=a.device)
        _check(load().nsa_gemm_bf16_splitk(_p(a), _p(b), _p(ws), c_int(M), c_int(N), c_int(K), c_int(a.stride(0)),
                                           c_int(b.stride(0)), c_int(ws.stride(0)), c_int(int(a_mn)), c_int(int(b_mn)),
                                           c_int(split_k), _stream()))
        if not direct:
            out.copy_(ws)
        return out
    _check(load().nsa_gemm_bf16(_p(a), _p(b), _p(out), c_int(M), c_int(N), c_int(K), c_int(a.stride(0)),
                                c_int(b.stride(0)), c_int(out.stride(0)), c_int(int(a_mn)), c_int(int(b_mn)),
                                c_int(int(out.dtype == torch.float32)), c_int(int(accumulate)), c_int(max_ctas),
                                _stream()))
    return out


def gemm_select(which: str = "default") -> None:
    """Kernel used by plain GEMMs from now on: "pair" (two CTAs per 256 x 256 tile), "single"
    (one CTA per 128 x 256 tile) or "default" (pair unless NSA_B200_GEMM=single)."""
    global _gemm_which
    _gemm_which = which
    load().nsa_gemm_select(c_int({"default": 0, "single": 1, "pair": 2}[which]))


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: Tensor, w: Tensor):
        x2 = _as_2d(x)
        ctx.save_for_backward(x2, w)
        ctx.xshape = x.shape
        y = gemm(x2, w, False, False)
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy: Tensor):
        x2, w = ctx.saved_tensors
        dy2 = _as_2d(dy)
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, w, False, True).view(ctx.xshape)          # dy (M,N) @ w (N,K)
        if ctx.needs_input_grad[1]:
            dw = gemm(dy2, x2, True, True)                            # dy^T (N,M) @ x (M,K)
        return dx, dw


class _MultiLinear(torch.autograd.Function):
    """Several projections of one input, y_i = x W_i^T.  The forward is one GEMM per weight; the
    backward builds dx = sum_i dy_i W_i in place (the first GEMM stores, the others add through the
    epilogue's TMA reduce-add) instead of leaving len(ws) - 1 full-size additions to autograd."""

    @staticmethod
    def forward(ctx, x: Tensor, run_first, *ws: Tensor):
        x2 = _as_2d(x)
        ctx.save_for_backward(x2, *ws)
        ctx.xshape = x.shape
        ys = []
        for i, w in enumerate(ws):
            y = run_first(x2, w) if (i == 0 and run_first is not None) else gemm(x2, w, False, False)
            ys.append(y.view(*x.shape[:-1], w.shape[0]))
        return tuple(ys)

    @staticmethod
    def backward(ctx, *dys):
        x2, *ws = ctx.saved_tensors
        dx = None
        dws = []
        for i, (dy, w) in enumerate(zip(dys, ws)):
            if dy is None:
                dws.append(None)
                continue
            dy2 = _as_2d(dy)
            if ctx.needs_input_grad[0]:
                if dx is None:
                    dx = gemm(dy2, w, False, True)
                else:
                    gemm(dy2, w, False, True, out=dx, accumulate=True, split_k=1)
            dws.append(gemm(dy2, x2, True, True) if ctx.needs_input_grad[2 + i] else None)
        if dx is not None:
            dx = dx.view(ctx.xshape)
        return (dx, None) + tuple(dws)


def multi_linear(x: Tensor, ws) -> tuple:
    """(x W_0^T, x W_1^T, ...) for weights that share the input (see :class:`_MultiLinear`)."""
    ws = list(ws)
    if (x.shape[-1] % 8) or any(w.shape[0] % 8 for w in ws) or x.shape[0] == 0:
        return tuple(linear(x, w) for w in ws)
    rows = x.numel() // x.shape[-1]
    if rows <= 128:                        # the single-CTA kernel has no adding epilogue
        return tuple(linear(x, w) for w in ws)
    run = None
    pg = _pending_gather
    if pg is not None:
        if pg[0] <= ws[0].data_ptr() < pg[1] and ws[0].is_contiguous():
            run = pg[2]
        else:
            flush_pending_gather()
    return _MultiLinear.apply(x, run, *ws)


# A sharded unit may defer its all-gather to the first matmul that touches one of its weights:
# (lo, hi) is the address range of the unit's gathered buffer, ``run(x, w)`` launches the GEMM
# whose kernel also assembles that buffer, ``fallback()`` gathers it without a matmul.
_pending_gather = None


def set_pending_gather(lo: int, hi: int, run, fallback) -> None:
    global _pending_gather
    flush_pending_gather()
    _pending_gather = (lo, hi, run, fallback)


def clear_pending_gather() -> None:
    global _pending_gather
    _pending_gather = None


def flush_pending_gather() -> None:
    global _pending_gather
    if _pending_gather is not None:
        fb = _pending_gather[3]
        _pending_gather = None
        fb()


class _LinearGather(torch.autograd.Function):
    """y = x W^T where the kernel that computes y also gathers W's sharded unit (see
    ``parallel/symm.py``); the backward is the ordinary one."""

    @staticmethod
    def forward(ctx, x, w, run):
        x2 = _as_2d(x)
        y = run(x2, w)
        ctx.save_for_backward(x2, w)
        ctx.xshape = x.shape
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = _as_2d(dy)
        dx = gemm(dy2, w, False, True).view(ctx.xshape) if ctx.needs_input_grad[0] else None
        dw = gemm(dy2, x2, True, True) if ctx.needs_input_grad[1] else None
        return dx, dw, None


def linear(x: Tensor, w: Tensor) -> Tensor:
    if (x.shape[-1] % 8) or (w.shape[0] % 8):
        flush_pending_gather()
        _fallback("linear")
        return torch_impl.linear(x, w)
    pg = _pending_gather
    if pg is not None:
        if pg[0] <= w.data_ptr() < pg[1] and w.is_contiguous():
            return _LinearGather.apply(x, w, pg[2])
        flush_pending_gather()
    return _Linear.apply(x, w)


# --------------------------------------------------------------------------------------
# norms
# --------------------------------------------------------------------------------------
def _rms_fwd(x2, gate2, w, eps, mode):
    rows, d = x2.shape
    y = _empty_like(x2)
    rstd = _empty(rows, dtype=torch.float32, device=x2.device)
    _check(load().nsa_rmsnorm_fwd(_p(x2), _p(gate2), _p(w), _p(y), _p(rstd), c_long(rows), c_int(d),
                                  c_float(eps), c_int(mode), _stream()))
    return y, rstd


def _rms_bwd(x2, gate2, w, dy2, rstd, mode):
    rows, d = x2.shape
    dx = _empty_like(x2)
    dg = _empty_like(x2) if mode != 0 else None
    dw = _empty(d, dtype=torch.bfloat16, device=x2.device)
    parts = int(load().nsa_rmsnorm_bwd_parts(c_long(rows), c_int(d)))
    partial = _empty(parts * d, dtype=torch.float32, device=x2.device)
    _check(load().nsa_rmsnorm_bwd(_p(x2), _p(gate2), _p(w), _p(dy2), _p(rstd), _p(dx), _p(dg), _p(dw), c_void_p(0),
                                  _p(partial), c_long(rows), c_int(d), c_int(mode), _stream()))
    return dx, dg, dw


class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps):
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        wb = w.to(torch.bfloat16)
        y, rstd = _rms_fwd(x2, None, wb, eps, 0)
        ctx.save_for_backward(x2, wb, rstd)
        ctx.wdtype = w.dtype
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, wb, rstd = ctx.saved_tensors
        dx, _, dw = _rms_bwd(x2, None, wb, dy.reshape(x2.shape).contiguous(), rstd, 0)
        return dx.view(dy.shape), dw.to(ctx.wdtype), None


def _rms_bwd_res(x2, w, dy2, rstd, dres2):
    rows, d = x2.shape
    dx = _empty_like(x2)
    dw = _empty(d, dtype=torch.bfloat16, device=x2.device)
    parts = int(load().nsa_rmsnorm_bwd_parts(c_long(rows), c_int(d)))
    partial = _empty(parts * d, dtype=torch.float32, device=x2.device)
    _check(load().nsa_rmsnorm_bwd_res(_p(x2), _p(w), _p(dy2), _p(rstd), _p(dres2), _p(dx), _p(dw), c_void_p(0),
                                      _p(partial), c_long(rows), c_int(d), _stream()))
    return dx, dw


def _norm_grads(ctx, h2, wb, rstd, dres, dy):
    """Gradient at the input of a plain norm that also receives `dres` by the residual route."""
    if dy is None:
        return (dres, None)
    dy2 = dy.reshape(h2.shape).contiguous()
    if dres is None:
        dx, _, dw = _rms_bwd(h2, None, wb, dy2, rstd, 0)
    else:
        dx, dw = _rms_bwd_res(h2, wb, dy2, rstd, dres.reshape(h2.shape).contiguous())
    return dx.view(dy.shape), dw.to(ctx.wdtype)


class _RMSNormSkip(torch.autograd.Function):
    """(y, x) with y = rmsnorm(x) * w.  The second output is the input itself, handed on to the
    residual stream; in backward its gradient and the norm's gradient meet in one kernel instead
    of two kernels and an add."""

    @staticmethod
    def forward(ctx, x, w, eps):
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        wb = w.to(torch.bfloat16)
        y, rstd = _rms_fwd(x2, None, wb, eps, 0)
        ctx.save_for_backward(x2, wb, rstd)
        ctx.wdtype = w.dtype
        return y.view(x.shape), x.view_as(x)

    @staticmethod
    def backward(ctx, dy, dskip):
        x2, wb, rstd = ctx.saved_tensors
        dx, dw = _norm_grads(ctx, x2, wb, rstd, dskip, dy)
        return dx, dw, None


class _AddRMSNorm(torch.autograd.Function):
    """(h, y) with h = x + r and y = rmsnorm(h) * w in one pass; backward adds the gradient that
    reaches h directly to the norm's gradient in the same kernel, and x and r share the result."""

    @staticmethod
    def forward(ctx, x, r, w, eps):
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        r2 = r.reshape(-1, r.shape[-1]).contiguous()
        wb = w.to(torch.bfloat16)
        rows, d = x2.shape
        h = _empty_like(x2)
        y = _empty_like(x2)
        rstd = _empty(rows, dtype=torch.float32, device=x2.device)
        _check(load().nsa_rmsnorm_add_fwd(_p(x2), _p(r2), _p(wb), _p(h), _p(y), _p(rstd), c_long(rows), c_int(d),
                                          c_float(eps), _stream()))
        ctx.save_for_backward(h, wb, rstd)
        ctx.wdtype = w.dtype
        return h.view(x.shape), y.view(x.shape)

    @staticmethod
    def backward(ctx, dh, dy):
        h2, wb, rstd = ctx.saved_tensors
        dx, dw = _norm_grads(ctx, h2, wb, rstd, dh, dy)
        return dx, dx, dw, None


def rms_norm_skip(x, w, eps=1e-6):
    if x.shape[-1] % 8 or x.shape[-1] > 8192:
        _fallback("rms_norm_skip")
        return torch_impl.rms_norm_skip(x, w, eps)
    return _RMSNormSkip.apply(x, w, eps)


def add_rms_norm(x, r, w, eps=1e-6):
    if x.shape[-1] % 8 or x.shape[-1] > 8192 or x.shape != r.shape:
        _fallback("add_rms_norm")
        return torch_impl.add_rms_norm(x, r, w, eps)
    return _AddRMSNorm.apply(x, r, w, eps)


def _gate_rows(gate: Tensor):
    """(2-D gate, row pitch): a column slice of a wider row-major matrix is used in place when its
    rows are 16-byte aligned; anything else is made contiguous."""
    d = gate.shape[-1]
    if gate.dim() >= 2 and gate.stride(-1) == 1 and gate.data_ptr() % 16 == 0:
        pitch = gate.stride(-2)
        exp, ok = pitch, pitch % 8 == 0 and pitch >= d
        for k in range(gate.dim() - 2, -1, -1):
            if gate.shape[k] != 1 and gate.stride(k) != exp:
                ok = False
            exp *= gate.shape[k]
        if ok:
            rows = gate.numel() // d
            return torch.as_strided(gate, (rows, d), (pitch, 1)), pitch
    g2 = gate.reshape(-1, d).contiguous()
    return g2, d


class _GatedRMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gate, w, eps, norm_before_gate):
        mode = 1 if norm_before_gate else 2
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        g2, ldg = _gate_rows(gate)
        wb = w.to(torch.bfloat16)
        rows, d = x2.shape
        y = _empty_like(x2)
        rstd = _empty(rows, dtype=torch.float32, device=x2.device)
        _check(load().nsa_rmsnorm_fwd_ldg(_p(x2), _p(g2), c_long(ldg), _p(wb), _p(y), _p(rstd), c_long(rows), c_int(d),
                                          c_float(eps), c_int(mode), _stream()))
        ctx.save_for_backward(x2, g2, wb, rstd)
        ctx.mode, ctx.wdtype, ctx.gshape, ctx.ldg = mode, w.dtype, gate.shape, ldg
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, g2, wb, rstd = ctx.saved_tensors
        rows, d = x2.shape
        dy2 = dy.reshape(x2.shape).contiguous()
        dx, dg = _empty_like(x2), _empty_like(x2)
        dw = _empty(d, dtype=torch.bfloat16, device=x2.device)
        parts = int(load().nsa_rmsnorm_bwd_parts(c_long(rows), c_int(d)))
        partial = _empty(parts * d, dtype=torch.float32, device=x2.device)
        _check(load().nsa_rmsnorm_bwd_ldg(_p(x2), _p(g2), c_long(ctx.ldg), _p(wb), _p(dy2), _p(rstd), _p(dx), _p(dg), _p(dw),
                                          c_void_p(0), _p(partial), c_long(rows), c_int(d), c_int(ctx.mode), _stream()))
        return dx.view(dy.shape), dg.view(ctx.gshape), dw.to(ctx.wdtype), None, None


def rms_norm(x, w, eps=1e-6):
    d = x.shape[-1]
    if d % 8 or d > 8192:
        _fallback("rms_norm")
        return torch_impl.rms_norm(x, w, eps)
    return _RMSNorm.apply(x, w, eps)


def gated_rms_norm(x, gate, w, eps=1e-6, norm_before_gate=True):
    d = x.shape[-1]
    if d % 8 or d > 8192:
        _fallback("gated_rms_norm")
        return torch_impl.gated_rms_norm(x, gate, w, eps, norm_before_gate)
    return _GatedRMSNorm.apply(x, gate, w, eps, norm_before_gate)


class _L2Norm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, eps):
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        rows, d = x2.shape
        y = _empty_like(x2)
        rinv = _empty(rows, dtype=torch.float32, device=x.device)
        _check(load().nsa_l2norm_fwd(_p(x2), _p(y), _p(rinv), c_long(rows), c_int(d), c_float(eps), _stream()))
        ctx.save_for_backward(y, rinv)
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        y, rinv = ctx.saved_tensors
        dy2 = dy.reshape(y.shape).contiguous()
        dx = _empty_like(y)
        _check(load().nsa_l2norm_bwd(_p(y), _p(dy2), _p(rinv), _p(dx), c_long(y.shape[0]), c_int(y.shape[1]), _stream()))
        return dx.view(dy.shape), None


def l2_norm(x, eps=1e-6):
    d = x.shape[-1]
    if d % 8 or d > 512:
        _fallback("l2_norm")
        return torch_impl.l2_norm(x, eps)
    return _L2Norm.apply(x, eps)


# --------------------------------------------------------------------------------------
# SwiGLU, RoPE
# --------------------------------------------------------------------------------------
def _rows_view(t: Tensor) -> Tensor:
    t2 = t.reshape(-1, t.shape[-1])
    if t2.stride(-1) != 1 or t2.stride(0) % 8 or t2.data_ptr() % 16:
        t2 = t2.contiguous()
    return t2


class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate, up):
        g2, u2 = _rows_view(gate), _rows_view(up)
        rows, cols = g2.shape
        y = _empty(rows, cols, dtype=gate.dtype, device=gate.device)
        _check(load().nsa_swiglu_fwd(_p(g2), _p(u2), _p(y), c_long(rows), c_int(cols), c_long(g2.stride(0)),
                                     c_long(u2.stride(0)), _stream()))
        ctx.save_for_backward(g2, u2)
        return y.view(gate.shape)

    @staticmethod
    def backward(ctx, dy):
        g2, u2 = ctx.saved_tensors
        rows, cols = g2.shape
        dy2 = dy.reshape(rows, cols).contiguous()
        dg = _empty(rows, cols, dtype=dy.dtype, device=dy.device)
        du = _empty(rows, cols, dtype=dy.dtype, device=dy.device)
        _check(load().nsa_swiglu_bwd(_p(g2), _p(u2), _p(dy2), _p(dg), _p(du), c_long(rows), c_int(cols),
                                     c_long(g2.stride(0)), c_long(u2.stride(0)), c_long(cols), _stream()))
        return dg.view(dy.shape), du.view(dy.shape)


def swiglu(gate, up):
    if gate.shape[-1] % 8:
        _fallback("swiglu")
        return torch_impl.swiglu(gate, up)
    return _SwiGLU.apply(gate, up)


def _rope_call(x: Tensor, cos: Tensor, sin: Tensor, backward: bool) -> Tensor:
    B, T, H, D = x.shape
    xc = x.contiguous()
    y = _empty_like(xc)
    _check(load().nsa_rope(_p(xc), _p(cos), _p(sin), _p(y), c_long(B), c_int(T), c_int(H), c_int(D),
                           c_int(int(backward)), _stream()))
    return y


class _RoPE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos, sin):
        cos = cos.float().contiguous()
        sin = sin.float().contiguous()
        ctx.save_for_backward(cos, sin)
        return _rope_call(x, cos, sin, False)

    @staticmethod
    def backward(ctx, dy):
        cos, sin = ctx.saved_tensors
        return _rope_call(dy, cos, sin, True), None, None


def rope(x, cos, sin):
    if x.shape[-1] % 16 or cos.shape[0] != x.shape[1]:
        _fallback("rope")
        return torch_impl.rope(x, cos, sin)
    return _RoPE.apply(x, cos, sin)


# --------------------------------------------------------------------------------------
# causal conv1d
# --------------------------------------------------------------------------------------
class _Conv1d(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, activation):
        B, T, C = x.shape
        xv = x if (x.stride(2) == 1 and x.stride(1) % 8 == 0 and x.stride(0) == T * x.stride(1)
                   and x.data_ptr() % 16 == 0) else x.contiguous()
        wb = weight.to(torch.bfloat16).contiguous()
        bb = None if bias is None else bias.to(torch.bfloat16).contiguous()
        y = _empty(B, T, C, dtype=x.dtype, device=x.device)
        _check(load().nsa_conv1d_fwd(_p(xv), _p(wb), _p(bb), _p(y), c_int(B), c_int(T), c_int(C),
                                     c_long(xv.stride(1)), c_int(weight.shape[-1]), c_int(int(activation)), _stream()))
        ctx.save_for_backward(xv, wb, bb)
        ctx.activation, ctx.wdtype = activation, weight.dtype
        ctx.has_bias = bias is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        xv, wb, bb = ctx.saved_tensors
        B, T, C = xv.shape
        W = wb.shape[-1]
        dyc = dy.contiguous()
        dx = _empty(B, T, C, dtype=dy.dtype, device=dy.device)
        parts = int(load().nsa_conv1d_bwd_parts(c_int(B), c_int(T)))
        partial = _empty(parts * (W + 1) * C, dtype=torch.float32, device=dy.device)
        dwdb = _empty((W + 1) * C, dtype=torch.float32, device=dy.device)
        _check(load().nsa_conv1d_bwd(_p(xv), _p(wb), _p(bb), _p(dyc), _p(dx), _p(partial), _p(dwdb), c_int(B), c_int(T),
                                     c_int(C), c_long(xv.stride(1)), c_int(W), c_int(int(ctx.activation)), _stream()))
        dw = dwdb[: W * C].view(W, C).t().contiguous().to(ctx.wdtype)
        db = dwdb[W * C:].to(ctx.wdtype) if ctx.has_bias else None
        return dx, dw, db, None


def causal_conv1d(x, weight, bias, activation=True):
    if x.shape[-1] % 8 or weight.shape[-1] != 4:
        _fallback("causal_conv1d")
        return torch_impl.causal_conv1d(x, weight, bias, activation)
    return _Conv1d.apply(x, weight, bias, activation)


# --------------------------------------------------------------------------------------
# embedding
# --------------------------------------------------------------------------------------
class _Embedding(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, weight):
        flat = ids.reshape(-1).contiguous()
        n, d = flat.numel(), weight.shape[1]
        y = _empty(n, d, dtype=weight.dtype, device=weight.device)
        _check(load().nsa_embedding_fwd(_p(flat), _p(weight), _p(y), c_long(n), c_int(d), c_long(weight.shape[0]), _stream()))
        ctx.save_for_backward(flat)
        ctx.wshape, ctx.wdtype = weight.shape, weight.dtype
        return y.view(*ids.shape, d)

    @staticmethod
    def backward(ctx, dy):
        (flat,) = ctx.saved_tensors
        n, d = flat.numel(), ctx.wshape[1]
        sorted_ids, perm = torch.sort(flat, stable=True)
        dw = _zeros(ctx.wshape, dtype=torch.float32, device=dy.device)
        dy2 = dy.reshape(n, d).contiguous()
        _check(load().nsa_embedding_bwd(_p(sorted_ids), _p(perm), _p(dy2), _p(dw), c_long(n), c_int(d), _stream()))
        return None, dw.to(ctx.wdtype)


def embedding(ids, weight):
    if weight.shape[1] % 8 or ids.dtype != torch.long:
        _fallback("embedding")
        return torch_impl.embedding(ids, weight)
    return _Embedding.apply(ids, weight)


# --------------------------------------------------------------------------------------
# fused linear + cross entropy
# --------------------------------------------------------------------------------------
class _LinearCE(torch.autograd.Function):
    """Per token chunk: logits GEMM (tcgen05) -> softmax-CE kernel that overwrites the logits
    with their gradient -> two gradient GEMMs.  The (chunk, V) block is the largest temporary."""

    @staticmethod
    def forward(ctx, hidden, weight, labels, ignore_index, chunk):
        N, d = hidden.shape
        V = weight.shape[0]
        h = _as_2d(hidden)
        labels = labels.contiguous()
        need_h, need_w = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        n_valid = (labels != ignore_index).sum().clamp_min(1).float()
        inv = (1.0 / n_valid).reshape(1)
        loss_rows = _empty(N, dtype=torch.float32, device=hidden.device)
        dh = _empty_like(h) if need_h else None
        dw = _zeros(V, d, dtype=torch.float32, device=hidden.device) if need_w else None
        logits = _empty(min(chunk, N), V, dtype=torch.bfloat16, device=hidden.device)
        for s0 in range(0, N, chunk):
            s1 = min(N, s0 + chunk)
            lg = logits[: s1 - s0]
            gemm(h[s0:s1], weight, False, False, out=lg)
            _check(load().nsa_cross_entropy(_p(lg), _p(labels[s0:s1]), _p(loss_rows[s0:s1]), _p(inv), c_long(s1 - s0),
                                            c_int(V), c_long(lg.stride(0)), c_long(ignore_index),
                                            c_int(int(need_h or need_w)), _stream()))
            if need_h:
                gemm(lg, weight, False, True, out=dh[s0:s1])                   # dlogits (n,V) @ W (V,d)
            if need_w:
                gemm(lg, h[s0:s1], True, True, out=dw, accumulate=(s0 > 0))    # dlogits^T (V,n) @ h (n,d)
        ctx.save_for_backward(dh, dw)
        ctx.wdtype = weight.dtype
        return loss_rows.sum() * inv[0]

    @staticmethod
    def backward(ctx, gout):
        dh, dw = ctx.saved_tensors
        return (None if dh is None else dh * gout.to(dh.dtype),
                None if dw is None else (dw * gout).to(ctx.wdtype), None, None, None)


def linear_cross_entropy(hidden, weight, labels, ignore_index=-100, chunk=4096):
    if hidden.shape[-1] % 8 or weight.shape[0] % 8:
        _fallback("linear_cross_entropy")
        return torch_impl.linear_cross_entropy(hidden, weight, labels, ignore_index, chunk)
    return _LinearCE.apply(hidden, weight, labels, ignore_index, chunk)


# --------------------------------------------------------------------------------------
# optimizer steps
# --------------------------------------------------------------------------------------
def _require_numel(what: str, t: Optional[Tensor], n: int) -> None:
    """The update kernels index every state tensor with the parameter's element count; a state
    restored from a checkpoint of another sharding would make them run past its end."""
    if t is not None and t.numel() != n:
        raise ValueError(f"optimizer state '{what}' has {t.numel()} elements, the kernel needs {n}")


def adamw_step(p, g, m, v, master, step, lr, b1, b2, eps, wd, grad_scale):
    n = p.numel()
    _require_numel("grad", g, n)
    _require_numel("exp_avg", m, n)
    _require_numel("exp_avg_sq", v, n)
    _require_numel("master", master, n)
    gs = None if grad_scale is None else grad_scale.reshape(1).float()
    _check(load().nsa_adamw_step(_p(p), _p(g), _p(m), _p(v), _p(master), _p(gs), c_long(p.numel()),
                                 c_int(int(p.dtype == torch.float32)), c_int(int(g.dtype == torch.float32)),
                                 c_int(step), c_float(lr), c_float(b1), c_float(b2), c_float(eps), c_float(wd), _stream()))


def adamw8bit_step(p, g, mq, mabs, vq, vabs, step, lr, b1, b2, eps, wd, grad_scale, block):
    if block != 256:
        raise ValueError("the native 8-bit AdamW kernel uses 256-element blocks")
    n = p.numel()
    if n % block:
        raise ValueError(f"8-bit AdamW needs a multiple of {block} elements, got {n}")
    _require_numel("grad", g, n)
    _require_numel("exp_avg", mq, n)
    _require_numel("exp_avg_sq", vq, n)
    _require_numel("exp_avg_absmax", mabs, n // block)
    _require_numel("exp_avg_sq_absmax", vabs, n // block)
    gs = None if grad_scale is None else grad_scale.reshape(1).float()
    cs = quant.codebook(8, True, p.device)
    cu = quant.codebook(8, False, p.device)
    _check(load().nsa_adamw8bit_step(_p(p), _p(g), _p(mq), _p(mabs), _p(vq), _p(vabs), _p(cs), _p(cu), _p(gs),
                                     c_long(p.numel()), c_int(int(p.dtype == torch.float32)),
                                     c_int(int(g.dtype == torch.float32)), c_int(step), c_float(lr), c_float(b1),
                                     c_float(b2), c_float(eps), c_float(wd), _stream()))


# --------------------------------------------------------------------------------------
# gated delta rule (chunk 64, key width 128)
# --------------------------------------------------------------------------------------
class _GDNSeq(torch.autograd.Function):
    """Inter-chunk state recurrence of the gated delta rule on tcgen05 (``csrc/gdn.cu``).
    Inputs are the per-chunk operands of the WY form, (BH, NC, 64, .) contiguous bf16."""

    @staticmethod
    def forward(ctx, w, qd, kt, u, gamma):
        BH, NC, C, K = w.shape
        V = u.shape[-1]
        v_new = _empty_like(u)
        o_inter = _empty(BH, NC, C, V, dtype=torch.bfloat16, device=u.device)
        S_all = _empty(BH, NC, K, V, dtype=torch.bfloat16, device=u.device)
        _check(load().nsa_gdn_seq_fwd(_p(w), _p(qd), _p(kt), _p(u), _p(gamma), _p(v_new), _p(o_inter), _p(S_all),
                                      c_int(BH), c_int(NC), c_int(K), c_int(V), _stream()))
        ctx.save_for_backward(w, qd, kt, gamma, S_all, v_new)
        # o_inter leaves the kernel as bf16 (it is added to a bf16 matmul result next), so its gradient
        # also arrives as bf16 instead of making an fp32 round trip
        return v_new, o_inter

    @staticmethod
    def backward(ctx, dv_new, do_inter):
        w, qd, kt, gamma, S_all, v_new = ctx.saved_tensors
        BH, NC, C, K = w.shape
        V = v_new.shape[-1]
        nvt = V // 64
        dv = _zeros_like(v_new) if dv_new is None else dv_new.to(torch.bfloat16).contiguous()
        do = _zeros_like(v_new) if do_inter is None else do_inter.to(torch.bfloat16).contiguous()
        du = _empty_like(v_new)
        parts = _empty(3, nvt, BH, NC, C, K, dtype=torch.bfloat16, device=w.device)
        dgp = _empty(nvt, BH, NC, dtype=torch.float32, device=w.device)
        _check(load().nsa_gdn_seq_bwd(_p(w), _p(qd), _p(kt), _p(S_all), _p(v_new), _p(dv), _p(do), _p(gamma), _p(du),
                                      _p(parts[0]), _p(parts[1]), _p(parts[2]), _p(dgp), c_int(BH), c_int(NC),
                                      c_int(K), c_int(V), _stream()))
        red = _empty(3, BH, NC, C, K, dtype=torch.bfloat16, device=w.device)
        _check(load().nsa_sum_parts_bf16(_p(parts), _p(red), c_long(3), c_int(nvt), c_long(BH * NC * C * K), _stream()))
        return red[0], red[1], red[2], du, dgp.sum(0)


class _GDNPack(torch.autograd.Function):
    """Token-major q, k, v -> head-major chunk rows (B*H, Tp, .): copies qh, kh, vh and the
    decay-scaled operands qd = q * sq, kt = k * sk in one pass each way (``csrc/elementwise.cu``)."""

    @staticmethod
    def forward(ctx, q, k, v, sq, sk):
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        sq, sk = sq.float().contiguous(), sk.float().contiguous()
        B, T, H, K = q.shape
        V = v.shape[-1]
        Tp = sq.shape[-1]
        mk = lambda w: _empty(B * H, Tp, w, dtype=torch.bfloat16, device=q.device)
        qh, kh, vh, qd, kt = mk(K), mk(K), mk(V), mk(K), mk(K)
        _check(load().nsa_gdn_pack_fwd(_p(q), _p(k), _p(v), _p(sq), _p(sk), _p(qh), _p(kh), _p(vh), _p(qd), _p(kt),
                                       c_int(B), c_int(T), c_int(Tp), c_int(H), c_int(K), c_int(V), _stream()))
        ctx.save_for_backward(q, k, sq, sk)
        ctx.V = V
        return qh, kh, vh, qd, kt

    @staticmethod
    def backward(ctx, dqh, dkh, dvh, dqd, dkt):
        q, k, sq, sk = ctx.saved_tensors
        B, T, H, K = q.shape
        V, Tp = ctx.V, sq.shape[-1]
        c = lambda t: None if t is None else t.to(torch.bfloat16).contiguous()
        dqh, dkh, dvh, dqd, dkt = c(dqh), c(dkh), c(dvh), c(dqd), c(dkt)
        dq, dk = _empty_like(q), _empty_like(k)
        dv = _empty(B, T, H, V, dtype=torch.bfloat16, device=q.device)
        dsq, dsk = _empty_like(sq), _empty_like(sk)
        _check(load().nsa_gdn_pack_bwd(_p(q), _p(k), _p(sq), _p(sk), _p(dqh), _p(dkh), _p(dvh), _p(dqd), _p(dkt), _p(dq), _p(dk),
                                       _p(dv), _p(dsq), _p(dsk), c_int(B), c_int(T), c_int(Tp), c_int(H), c_int(K), c_int(V),
                                       _stream()))
        return dq, dk, dv, dsq, dsk


class _GDNTmat(torch.autograd.Function):
    """Per-chunk 64 x 64 matrices of the gated delta rule (``gdn_tmat_*`` in ``csrc/elementwise.cu``):
    from kk = K K^T, qkr = Q K^T (bf16), the cumulative gate gc and beta build
    Tu = X diag(beta), Tw = X diag(beta e^gc) with X = (I + A)^-1 and the decayed, scaled, causal qk.
    The backward needs dA = -(X^T dX X^T): two batched fp32 matmuls between two small kernels."""

    @staticmethod
    def forward(ctx, kk, qkr, gc, bh, scale):
        kk, qkr = kk.contiguous(), qkr.contiguous()
        gc, bh = gc.float().contiguous(), bh.float().contiguous()
        n = gc.numel() // 64
        Tu, Tw, qk = _empty_like(kk), _empty_like(kk), _empty_like(kk)
        X = _empty(kk.shape, dtype=torch.float32, device=kk.device)
        _check(load().nsa_gdn_tmat_fwd(_p(kk), _p(qkr), _p(gc), _p(bh), _p(Tu), _p(Tw), _p(qk), _p(X), c_long(n), c_float(scale),
                                       _stream()))
        ctx.save_for_backward(kk, qkr, gc, bh, X)
        ctx.scale = scale
        return Tu, Tw, qk

    @staticmethod
    def backward(ctx, dTu, dTw, dqk):
        kk, qkr, gc, bh, X = ctx.saved_tensors
        n = gc.numel() // 64
        z = lambda t: _zeros_like(kk) if t is None else t.to(torch.bfloat16).contiguous()
        dTu, dTw, dqk = z(dTu), z(dTw), z(dqk)
        dX = _empty_like(X)
        lib = load()
        _check(lib.nsa_gdn_tmat_dx(_p(dTu), _p(dTw), _p(gc), _p(bh), _p(dX), c_long(n), _stream()))
        Xt = X.transpose(-1, -2)
        dA = -torch.matmul(torch.matmul(Xt, dX), Xt)
        del dX
        dkk, dqkr = _empty_like(kk), _empty_like(kk)
        dgc, dbh = _empty_like(gc), _empty_like(bh)
        _check(lib.nsa_gdn_tmat_bwd(_p(dA.contiguous()), _p(kk), _p(qkr), _p(dqk), _p(dTu), _p(dTw), _p(X), _p(gc), _p(bh), _p(dkk),
                                    _p(dqkr), _p(dgc), _p(dbh), c_long(n), c_float(ctx.scale), _stream()))
        return dkk, dqkr, dgc, dbh, None


class _HeadToToken(torch.autograd.Function):
    """(B*H, Tp, D) head-major rows -> (B, T, H, D) token-major (T <= Tp), one coalesced copy each way
    (``permute_rows_kernel``) instead of a generic strided copy."""

    @staticmethod
    def forward(ctx, x, B, H, T):
        Tp, D = x.shape[-2], x.shape[-1]
        ctx.dims = (B, H, Tp, T, D)
        x = x.contiguous()
        y = _empty(B, T, H, D, dtype=x.dtype, device=x.device)
        _check(load().nsa_permute_rows(_p(x), _p(y), c_int(B), c_int(H), c_int(Tp), c_int(T), c_int(D), c_int(1), _stream()))
        return y

    @staticmethod
    def backward(ctx, dy):
        B, H, Tp, T, D = ctx.dims
        dy = dy.to(torch.bfloat16).contiguous()
        dx = _empty(B * H, Tp, D, dtype=dy.dtype, device=dy.device)
        _check(load().nsa_permute_rows(_p(dy), _p(dx), c_int(B), c_int(H), c_int(Tp), c_int(T), c_int(D), c_int(0), _stream()))
        return dx, None, None, None


def gated_delta_rule(q, k, v, g, beta, scale=None, chunk=64):
    """Chunkwise gated delta rule.  One layout pass brings q, k, v to head-major chunk rows together
    with the decay-scaled operands; K K^T, Q K^T and the applications of the per-chunk matrices are
    batched bf16 matmuls; the 64 x 64 matrices themselves (decay masks, the unit-triangular inverse
    by substitution, their gradients) come from one small kernel each way; the sequential state
    pass is the tcgen05 kernel of ``csrc/gdn.cu``."""
    B, T, H, K = q.shape
    V = v.shape[-1]
    if K != 128 or V % 64 or chunk != 64 or q.dtype != torch.bfloat16:
        _fallback("gated_delta_rule")
        return torch_impl.gated_delta_rule(q, k, v, g, beta, scale, chunk)
    scale = K ** -0.5 if scale is None else scale
    C = 64
    pad = (-T) % C
    Tp = T + pad
    nc = Tp // C
    f32, bf = torch.float32, torch.bfloat16
    gh = g.to(f32).permute(0, 2, 1)
    bh = beta.to(f32).permute(0, 2, 1)
    if pad:
        gh, bh = torch.nn.functional.pad(gh, (0, pad)), torch.nn.functional.pad(bh, (0, pad))
    gh, bh = gh.reshape(B * H, nc, C), bh.reshape(B * H, nc, C)
    gc = torch.cumsum(gh, -1)
    eg = torch.exp(gc)
    sq = (scale * eg).reshape(B * H, Tp)
    sk = torch.exp(gc[..., -1:] - gc).reshape(B * H, Tp)
    qh, kh, vh, qd, kt = (t.view(B * H, nc, C, -1) for t in _GDNPack.apply(q, k, v.to(bf), sq, sk))
    kT = kh.transpose(-1, -2)
    Tu, Tw, qk = _GDNTmat.apply(torch.matmul(kh, kT), torch.matmul(qh, kT), gc, bh, float(scale))
    u = torch.matmul(Tu, vh)
    w = torch.matmul(Tw, kh)
    gamma = eg[..., -1].contiguous()
    v_new, o_inter = _GDNSeq.apply(w, qd, kt, u, gamma)
    # o = o_inter + qk v_new in one batched GEMM with fp32 accumulation
    o = torch.baddbmm(o_inter.view(-1, C, V), qk.view(-1, C, C), v_new.view(-1, C, V))
    if o.dtype == torch.bfloat16 and V % 8 == 0:
        return _HeadToToken.apply(o.view(B * H, Tp, V), B, H, T).to(v.dtype)
    o = o.view(B, H, Tp, V).permute(0, 2, 1, 3)[:, :T]
    return o.to(v.dtype)


# --------------------------------------------------------------------------------------
# attention family (csrc/attention.cu)
# --------------------------------------------------------------------------------------
class _Attn(torch.autograd.Function):
    """Softmax attention on (B, T, H, D) tensors through the tcgen05 kernels.  ``tiles`` is
    ``None`` (contiguous key range bounded by causality / window) or the per-query-tile block
    lists from :func:`union_blocks` (selected-block attention).  Key positions are
    ``index * kp_stride + kp_off``.  Returns (output, L) with L the log2-sum-exp per row."""

    @staticmethod
    def forward(ctx, q, k, v, causal, window, scale, kp_stride, kp_off, tiles):
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        B, T, Hq, D = q.shape
        S, Hkv = k.shape[1], k.shape[2]
        o = _empty_like(q)
        L = _empty(B, T, Hq, dtype=torch.float32, device=q.device)
        tb, tm, tc, mu = tiles[:4] if tiles is not None else (None, None, None, 0)
        _check(load().nsa_attn_fwd(_p(q), _p(k), _p(v), _p(o), _p(L), c_int(B), c_int(T), c_int(S), c_int(Hq),
                                   c_int(Hkv), c_int(D), c_float(scale), c_int(int(causal)), c_int(window),
                                   c_int(kp_stride), c_int(kp_off), _p(tb), _p(tm), _p(tc), c_int(mu), _stream()))
        ctx.save_for_backward(q, k, v, o, L)
        ctx.cfg = (causal, window, scale, kp_stride, kp_off)
        ctx.tiles = tiles
        ctx.mark_non_differentiable(L)
        return o, L

    @staticmethod
    def backward(ctx, do, _dL):
        q, k, v, o, L = ctx.saved_tensors
        causal, window, scale, kp_stride, kp_off = ctx.cfg
        B, T, Hq, D = q.shape
        S, Hkv = k.shape[1], k.shape[2]
        do = do.contiguous()
        dq = _empty_like(q)
        dk = _zeros(k.shape, dtype=torch.float32, device=q.device)
        dv = _zeros(v.shape, dtype=torch.float32, device=q.device)
        delta = _empty(B, T, Hq, dtype=torch.float32, device=q.device)
        tb, tm, tc, mu = ctx.tiles[:4] if ctx.tiles is not None else (None, None, None, 0)
        G = Hq // Hkv
        split = D == 128 and os.environ.get("NSA_B200_ATTN_BWD", "split") == "split" and (ctx.tiles is None or G >= 8)
        if split:
            # dQ from the query-tile-outer kernel, dK / dV from the key-block-stationary kernel
            R = 128 // G
            inv = (None, None, None, 0, 0)
            visits = int(os.environ.get('NSA_B200_KV_VISITS', '128'))
            if ctx.tiles is not None:
                idx, nS = ctx.tiles[4], ctx.tiles[5]
                visits = int(os.environ.get('NSA_B200_KV_VISITS_SEL', '64'))
                inv = inverse_blocks(idx, nS, R, visits)
            _check(load().nsa_attn_bwd_split(_p(q), _p(k), _p(v), _p(o), _p(do), _p(L), _p(delta), _p(dq), _p(dk), _p(dv),
                                             c_int(B), c_int(T), c_int(S), c_int(Hq), c_int(Hkv), c_int(D), c_float(scale),
                                             c_int(int(causal)), c_int(window), c_int(kp_stride), c_int(kp_off),
                                             _p(tb), _p(tm), _p(tc), c_int(mu), _p(inv[0]), _p(inv[1]), _p(inv[2]),
                                             c_int(inv[3]), c_int(inv[4]), c_int(visits), _stream()))
        else:
            _check(load().nsa_attn_bwd(_p(q), _p(k), _p(v), _p(o), _p(do), _p(L), _p(delta), _p(dq), _p(dk), _p(dv),
                                       c_int(B), c_int(T), c_int(S), c_int(Hq), c_int(Hkv), c_int(D), c_float(scale),
                                       c_int(int(causal)), c_int(window), c_int(kp_stride), c_int(kp_off),
                                       _p(tb), _p(tm), _p(tc), c_int(mu), _stream()))
        return dq, dk.to(k.dtype), dv.to(v.dtype), None, None, None, None, None, None


def _attn_ok(q, k) -> bool:
    Hq, Hkv, D = q.shape[2], k.shape[2], q.shape[3]
    G = Hq // max(Hkv, 1)
    return D in (64, 128) and Hkv > 0 and Hq % Hkv == 0 and G <= 128 and (G & (G - 1)) == 0


def attention(q, k, v, causal=True, window=0, scale=None):
    if not _attn_ok(q, k) or q.shape[1] != k.shape[1]:
        _fallback("attention")
        return torch_impl.attention(q, k, v, causal, window, scale)
    scale = q.shape[-1] ** -0.5 if scale is None else scale
    return _Attn.apply(q, k, v, causal, int(window), float(scale), 1, 0, None)[0]


def union_blocks(idx: Tensor, G: int, nS: int):
    """idx (B, Hkv, T, top_n) int32 selection-block ids (-1 = none) -> per query tile
    (128 // G tokens) ascending union list, token bit masks and counts."""
    B, Hkv, T, top_n = idx.shape
    R = 128 // G
    nqt = -(-T // R)
    max_u = min(R * top_n, nS)
    max_u += max_u & 1
    tb = _empty(B, Hkv, nqt, max_u, dtype=torch.int32, device=idx.device)
    tm = _empty(B, Hkv, nqt, max_u, dtype=torch.int64, device=idx.device)
    tc = _empty(B, Hkv, nqt, dtype=torch.int32, device=idx.device)
    _check(load().nsa_union_blocks(_p(idx), _p(tb), _p(tm), _p(tc), c_int(B), c_int(T), c_int(Hkv), c_int(G),
                                   c_int(top_n), c_int(nS), c_int(max_u), _stream()))
    return tb, tm, tc, max_u


def inverse_blocks(idx: Tensor, nS: int, R: int, visits_per_cta: int):
    """Inverse of the selection map (count, scan, fill kernels of ``csrc/attention.cu``; no sort, the
    same lists on every run).  Same results as :func:`_inverse_blocks_torch`."""
    B, Hkv, T, n = idx.shape
    if not idx.is_cuda or nS > 12288 or n > 32:
        return _inverse_blocks_torch(idx, nS, R, visits_per_cta)
    dev = idx.device
    idx = idx.to(torch.int32).contiguous()
    lists = B * Hkv * nS
    chunks = -(-T // 256)
    tok = _empty(B * Hkv * T * n, dtype=torch.int32, device=dev)
    list_start = _empty(lists + 1, dtype=torch.int32, device=dev)
    item_start = _empty(lists + 1, dtype=torch.int32, device=dev)
    hist = _empty(B * Hkv * chunks * nS, dtype=torch.int32, device=dev)
    count = _empty(lists, dtype=torch.int32, device=dev)
    _check(load().nsa_inverse_blocks(_p(idx), _p(tok), _p(list_start), _p(item_start), _p(hist), _p(count), c_int(B * Hkv),
                                     c_int(T), c_int(n), c_int(nS), c_int(R), c_int(visits_per_cta), _stream()))
    bound = (B * Hkv * T * n) // (R * visits_per_cta) + lists
    return tok, list_start, item_start, nS, bound


def _inverse_blocks_torch(idx: Tensor, nS: int, R: int, visits_per_cta: int):
    """Inverse of the selection map.  idx (B, Hkv, T, top_n) -> (tok_list, list_start, item_start,
    nS, item_bound): for every (b, h, block) the ascending tokens that selected the block, laid out
    back to back; ``list_start`` / ``item_start`` are the exclusive prefixes of the list lengths and
    of the CTAs per list (a CTA covers ``visits_per_cta`` groups of R tokens); ``item_bound`` is a
    host-side upper bound of the CTA count, so nothing here waits for the device.  Entries that are
    negative, out of range or repeated inside a token's list are dropped."""
    B, Hkv, T, n = idx.shape
    dev = idx.device
    lists = B * Hkv * nS
    s, _ = idx.sort(dim=-1)
    ok = (s >= 0) & (s < nS)
    ok[..., 1:] &= s[..., 1:] != s[..., :-1]
    bh = torch.arange(B * Hkv, device=dev, dtype=torch.int64).view(B, Hkv, 1, 1)
    key = torch.where(ok, bh * nS + s.to(torch.int64), torch.full((), lists, device=dev, dtype=torch.int64)).reshape(-1)
    skey, order = key.sort(stable=True)                       # (b, h, t) order survives inside a list
    tok = ((order // n) % T).to(torch.int32)
    list_start = torch.searchsorted(skey, torch.arange(lists + 1, device=dev, dtype=torch.int64)).to(torch.int32)
    cnt = list_start[1:] - list_start[:-1]
    items = (-(-cnt // R) + visits_per_cta - 1) // visits_per_cta
    item_start = _zeros(lists + 1, dtype=torch.int32, device=dev)
    item_start[1:] = items.cumsum(0)
    bound = (B * Hkv * T * n) // (R * visits_per_cta) + lists
    return tok, list_start, item_start, nS, bound


def selected_attention(q, k, v, idx, scale=None):
    """Causal attention of each query token over its own list of 64-key blocks ``idx``
    (B, Hkv, T, top_n)."""
    scale = q.shape[-1] ** -0.5 if scale is None else scale
    G = q.shape[2] // k.shape[2]
    nS = -(-k.shape[1] // 64)
    idx = idx.to(torch.int32).contiguous()
    tiles = union_blocks(idx, G, nS) + (idx, nS)
    return _Attn.apply(q, k, v, True, 0, float(scale), 1, 0, tiles)[0]


def nsa_attention_indexed(q, k, v, idx, g_slc, g_swa, sel_block=64, window=512, scale=None):
    """Selected-block attention over caller-given block lists ``idx`` (B, Hkv, T, n) plus the sliding
    window, gated: both branches on the tcgen05 attention kernels."""
    B, T, Hq, D = q.shape
    G = Hq // k.shape[2]
    if not _attn_ok(q, k) or sel_block != 64 or G < 2 or G > 32:
        _fallback("nsa_attention_indexed")
        return torch_impl.nsa_attention_indexed(q, k, v, idx, g_slc, g_swa, sel_block, window, scale)
    scale = D ** -0.5 if scale is None else scale
    o_slc = selected_attention(q, k, v, idx, scale)
    o_swa = _Attn.apply(q, k, v, True, int(window), float(scale), 1, 0, None)[0]
    return g_slc.unsqueeze(-1) * o_slc + g_swa.unsqueeze(-1) * o_swa


def nsa_importance(q, k_cmp, L_cmp, nS, stride, block, scale):
    B, T, Hq, D = q.shape
    Hkv = k_cmp.shape[2]
    imp = _zeros(B, Hkv, T, nS, dtype=torch.float32, device=q.device)
    _check(load().nsa_attn_importance(_p(q.contiguous()), _p(k_cmp.contiguous()), _p(L_cmp), _p(imp), c_int(B), c_int(T),
                                      c_int(k_cmp.shape[1]), c_int(Hq), c_int(Hkv), c_int(D), c_float(scale),
                                      c_int(stride), c_int(block - 1), c_int(nS), _stream()))
    return imp


def nsa_select(imp: Tensor, sel_block: int, top_n: int) -> Tensor:
    """imp (B, Hkv, T, nS) -> int32 (B, Hkv, T, top_n): block 0, the query's own block and the one
    before it always, then the most important causal blocks (ties: lower index); -1 where fewer
    are visible.  One warp per row (``nsa_select_kernel``); more than 2048 blocks use torch.topk."""
    B, H, T, nS = imp.shape
    if imp.is_cuda and nS <= 2048 and imp.dtype == torch.float32:
        imp = imp.contiguous()
        idx = _empty(B, H, T, top_n, dtype=torch.int32, device=imp.device)
        _check(load().nsa_select_blocks(_p(imp), _p(idx), c_long(B * H * T), c_int(T), c_int(nS), c_int(sel_block),
                                        c_int(top_n), _stream()))
        return idx
    return _nsa_select_torch(imp, sel_block, top_n)


def _nsa_select_torch(imp: Tensor, sel_block: int, top_n: int) -> Tensor:
    B, H, T, nS = imp.shape
    own = (torch.arange(T, device=imp.device) // sel_block)[:, None]
    j = torch.arange(nS, device=imp.device)[None, :]
    forced = (j == 0) | (j == own) | (j == own - 1)
    score = imp.masked_fill(forced, float("inf")).masked_fill_(j > own, float("-inf"))
    n = min(top_n, nS)
    val, idx = torch.topk(score, n, dim=-1)
    idx = idx.masked_fill(val == float("-inf"), -1).to(torch.int32)
    if n < top_n:
        idx = torch.nn.functional.pad(idx, (0, top_n - n), value=-1)
    return idx.contiguous()


class _GateCombine(torch.autograd.Function):
    """o = g1 o1 + g2 o2 + g3 o3 with one gate per (token, head): the sigmoid-gated combine of the
    three sparse-attention branches in one pass each way (``csrc/elementwise.cu``)."""

    @staticmethod
    def forward(ctx, o1, o2, o3, g1, g2, g3):
        o1, o2, o3 = o1.contiguous(), o2.contiguous(), o3.contiguous()
        g1, g2, g3 = (g.to(torch.bfloat16).contiguous() for g in (g1, g2, g3))
        D = o1.shape[-1]
        rows = o1.numel() // D
        o = _empty_like(o1)
        _check(load().nsa_gate_combine_fwd(_p(o1), _p(o2), _p(o3), _p(g1), _p(g2), _p(g3), _p(o), c_long(rows), c_int(D),
                                           _stream()))
        ctx.save_for_backward(o1, o2, o3, g1, g2, g3)
        return o

    @staticmethod
    def backward(ctx, do):
        o1, o2, o3, g1, g2, g3 = ctx.saved_tensors
        do = do.contiguous()
        D = o1.shape[-1]
        rows = o1.numel() // D
        d1, d2, d3 = _empty_like(o1), _empty_like(o1), _empty_like(o1)
        e1, e2, e3 = _empty_like(g1), _empty_like(g1), _empty_like(g1)
        _check(load().nsa_gate_combine_bwd(_p(o1), _p(o2), _p(o3), _p(g1), _p(g2), _p(g3), _p(do), _p(d1), _p(d2), _p(d3),
                                           _p(e1), _p(e2), _p(e3), c_long(rows), c_int(D), _stream()))
        return d1, d2, d3, e1, e2, e3


class _GateCombineLogits(torch.autograd.Function):
    """The same combine with the three gates taken as logits straight from the gate projection:
    ``gates`` is (B, T, 3*Hq) (or wider; columns [0, Hq) compressed, [Hq, 2Hq) selected, [2Hq, 3Hq)
    window).  The sigmoid runs inside the combine kernel and its derivative inside the backward
    kernel, which writes d(logits) in the projection's own layout."""

    @staticmethod
    def forward(ctx, o1, o2, o3, gates):
        o1, o2, o3 = o1.contiguous(), o2.contiguous(), o3.contiguous()
        Hq, D = o1.shape[-2], o1.shape[-1]
        gl = gates.to(torch.bfloat16)
        if gl.stride(-1) != 1 or not gl.is_contiguous():
            gl = gl.contiguous()
        ldg = gl.shape[-1]
        rows = o1.numel() // D
        o = _empty_like(o1)
        es = gl.element_size()
        _check(load().nsa_gate_combine_fwd_ex(_p(o1), _p(o2), _p(o3), c_void_p(gl.data_ptr()), c_void_p(gl.data_ptr() + Hq * es),
                                              c_void_p(gl.data_ptr() + 2 * Hq * es), c_long(ldg), c_int(Hq), c_int(1), _p(o),
                                              c_long(rows), c_int(D), _stream()))
        ctx.save_for_backward(o1, o2, o3, gl)
        ctx.gdtype = gates.dtype
        return o

    @staticmethod
    def backward(ctx, do):
        o1, o2, o3, gl = ctx.saved_tensors
        do = do.contiguous()
        Hq, D = o1.shape[-2], o1.shape[-1]
        ldg = gl.shape[-1]
        rows = o1.numel() // D
        es = gl.element_size()
        d1, d2, d3 = _empty_like(o1), _empty_like(o1), _empty_like(o1)
        dgl = _zeros_like(gl) if ldg > 3 * Hq else _empty_like(gl)
        g0, dg0 = gl.data_ptr(), dgl.data_ptr()
        _check(load().nsa_gate_combine_bwd_ex(_p(o1), _p(o2), _p(o3), c_void_p(g0), c_void_p(g0 + Hq * es),
                                              c_void_p(g0 + 2 * Hq * es), c_long(ldg), c_int(Hq), c_int(1), _p(do), _p(d1), _p(d2),
                                              _p(d3), c_void_p(dg0), c_void_p(dg0 + Hq * es), c_void_p(dg0 + 2 * Hq * es),
                                              c_long(rows), c_int(D), _stream()))
        return d1, d2, d3, dgl.to(ctx.gdtype)


class _Pool(torch.autograd.Function):
    """Mean pooling of (B, T, H, D) keys / values over windows [i*stride, i*stride + block) ->
    (B, nC, H, D), forward and backward in ``csrc/elementwise.cu`` (fla's ``mean_pooling`` in the
    reference's NSA stack)."""

    @staticmethod
    def forward(ctx, x, block, stride):
        B, T, H, D = x.shape
        width = H * D
        ok = (x.stride(3) == 1 and x.stride(2) == D and x.stride(1) % 8 == 0 and x.stride(0) == T * x.stride(1)
              and x.data_ptr() % 16 == 0)
        xv = x if ok else x.contiguous()
        nC = (T - block) // stride + 1
        y = _empty(B, nC, H, D, dtype=x.dtype, device=x.device)
        _check(load().nsa_pool_fwd(_p(xv), _p(y), c_int(B), c_int(T), c_int(width), c_long(xv.stride(1)), c_int(block),
                                   c_int(stride), _stream()))
        ctx.shape, ctx.block, ctx.stride = (B, T, H, D), block, stride
        return y

    @staticmethod
    def backward(ctx, dy):
        B, T, H, D = ctx.shape
        dy = dy.contiguous()
        dx = _empty(B, T, H, D, dtype=dy.dtype, device=dy.device)
        _check(load().nsa_pool_bwd(_p(dy), _p(dx), c_int(B), c_int(T), c_int(H * D), c_int(ctx.block), c_int(ctx.stride),
                                   _stream()))
        return dx, None, None


def nsa_compress(x, block, stride):
    if x.dtype != torch.bfloat16 or (x.shape[2] * x.shape[3]) % 8 or x.shape[1] < block:
        _fallback("nsa_compress")
        return torch_impl.nsa_compress(x, block, stride)
    return _Pool.apply(x, int(block), int(stride))


def nsa_attention(q, k, v, g_cmp, g_slc, g_swa, cmp_block=32, cmp_stride=16, sel_block=64, top_n=16,
                  window=512, scale=None, gate_logits=None):
    """``gate_logits`` (B, T, 3*Hq), when given, replaces the three gate tensors: the sigmoid is taken
    inside the combine kernel."""
    B, T, Hq, D = q.shape
    Hkv = k.shape[2]
    G = Hq // Hkv
    if (not _attn_ok(q, k) or sel_block != 64 or sel_block != 4 * cmp_stride or cmp_block != 2 * cmp_stride
            or G < 2 or G > 32 or T < cmp_block):
        _fallback("nsa_attention")
        if gate_logits is not None:
            g_cmp, g_slc, g_swa = torch.sigmoid(gate_logits.float()).to(q.dtype)[..., :3 * Hq].split(Hq, dim=-1)
        return torch_impl.nsa_attention(q, k, v, g_cmp, g_slc, g_swa, cmp_block, cmp_stride, sel_block, top_n,
                                        window, scale)
    scale = D ** -0.5 if scale is None else scale
    kc = nsa_compress(k, cmp_block, cmp_stride)
    vc = nsa_compress(v, cmp_block, cmp_stride)
    o_cmp, L_cmp = _Attn.apply(q, kc, vc, True, 0, float(scale), cmp_stride, cmp_block - 1, None)
    nS = -(-T // sel_block)
    with torch.no_grad():
        imp = nsa_importance(q, kc, L_cmp, nS, cmp_stride, cmp_block, float(scale))
        idx = nsa_select(imp, sel_block, top_n)
        del imp
        tiles = union_blocks(idx, G, nS) + (idx, nS)
    o_slc = _Attn.apply(q, k, v, True, 0, float(scale), 1, 0, tiles)[0]
    o_swa = _Attn.apply(q, k, v, True, int(window), float(scale), 1, 0, None)[0]
    if gate_logits is not None:
        if q.dtype == torch.bfloat16 and D in (64, 128, 256):
            return _GateCombineLogits.apply(o_cmp, o_slc, o_swa, gate_logits)
        g_cmp, g_slc, g_swa = torch.sigmoid(gate_logits.float()).to(q.dtype)[..., :3 * Hq].split(Hq, dim=-1)
    if q.dtype == torch.bfloat16 and D in (64, 128, 256):
        return _GateCombine.apply(o_cmp, o_slc, o_swa, g_cmp, g_slc, g_swa)
    return g_cmp.unsqueeze(-1) * o_cmp + g_slc.unsqueeze(-1) * o_slc + g_swa.unsqueeze(-1) * o_swa


# --------------------------------------------------------------------------------------
# Mamba-2 SSD
# --------------------------------------------------------------------------------------
class _SSDStatePass(torch.autograd.Function):
    """Hprev[c+1] = gamma[c] * Hprev[c] + S[c] over chunks (``csrc/ssd.cu``).
    S (B, nc, H, P, N) fp32, gamma (B, nc, H) fp32 -> Hprev, same shape as S."""

    @staticmethod
    def forward(ctx, S, gamma):
        S, gamma = S.contiguous(), gamma.contiguous()
        B, nc, H = gamma.shape
        E = S[0, 0, 0].numel()
        Hprev = _empty_like(S)
        _check(load().nsa_ssd_state_fwd(_p(S), _p(gamma), _p(Hprev), c_void_p(0), c_void_p(0), c_int(B), c_int(nc),
                                        c_int(H), c_long(E), _stream()))
        ctx.save_for_backward(gamma, Hprev)
        return Hprev

    @staticmethod
    def backward(ctx, dHprev):
        gamma, Hprev = ctx.saved_tensors
        B, nc, H = gamma.shape
        E = Hprev[0, 0, 0].numel()
        dHprev = dHprev.contiguous().float()
        dS = _empty_like(Hprev)
        _check(load().nsa_ssd_state_bwd(_p(dHprev), _p(gamma), _p(dS), c_void_p(0), c_int(B), c_int(nc), c_int(H), c_long(E),
                                        _stream()))
        dgamma = (Hprev * dS).sum((-1, -2))
        return dS, dgamma


def _token_view(t: Tensor, inner: int):
    """(B, T, ..., inner-contiguous) view -> (tensor, token stride in elements) usable by a TMA
    map with rows = tokens; copies when the view is not row-strided."""
    B, T = t.shape[0], t.shape[1]
    width = t[0, 0].numel()
    ok = (t.stride(-1) == 1 and t.stride(0) == T * t.stride(1) and t.stride(1) % 8 == 0 and t.data_ptr() % 16 == 0
          and t[0, 0].is_contiguous())
    if not ok:
        t = t.contiguous()
    return t, t.stride(1) if ok else width


class _SSD(torch.autograd.Function):
    """Mamba-2 SSD through the tcgen05 chunk kernels of ``csrc/ssd.cu`` (chunk 128, d_state 128,
    headdim 64, one B/C group)."""

    @staticmethod
    def forward(ctx, x, dt, A, Bm, Cm, D):
        Bsz, T, H, P = x.shape
        N = Bm.shape[-1]
        nc = -(-T // 128)
        x, ldx = _token_view(x, P)
        Bm, ldb = _token_view(Bm, N)
        Cm, ldc = _token_view(Cm, N)
        dt = dt.float().contiguous()
        A = A.float().contiguous()
        Df = None if D is None else D.float().contiguous()
        dev = x.device
        S_loc = _empty(Bsz, nc, H, N, P, dtype=torch.float32, device=dev)
        gamma = _empty(Bsz, nc, H, dtype=torch.float32, device=dev)
        lib = load()
        _check(lib.nsa_ssd_chunk_state(c_int(0), _p(Bm), c_long(ldb), _p(x), c_long(ldx), _p(dt), _p(A), _p(S_loc), _p(gamma),
                                       c_int(Bsz), c_int(T), c_int(H), c_int(N), c_int(P), _stream()))
        Hb = _empty(Bsz, nc, H, N, P, dtype=torch.bfloat16, device=dev)
        _check(lib.nsa_ssd_state_fwd(_p(S_loc), _p(gamma), c_void_p(0), _p(Hb), c_void_p(0), c_int(Bsz), c_int(nc), c_int(H),
                                     c_long(N * P), _stream()))
        del S_loc
        y = _empty(Bsz, T, H, P, dtype=torch.bfloat16, device=dev)
        _check(lib.nsa_ssd_chunk_out(_p(Cm), c_long(ldc), _p(Bm), c_long(ldb), _p(x), c_long(ldx), _p(Hb), _p(dt), _p(A),
                                     _p(Df), _p(y), c_int(Bsz), c_int(T), c_int(H), c_int(N), c_int(P), _stream()))
        ctx.save_for_backward(x, dt, A, Bm, Cm, Df if Df is not None else _empty(0, device=dev), y, gamma, Hb)
        ctx.lds = (ldx, ldb, ldc)
        ctx.has_D = D is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        x, dt, A, Bm, Cm, Df, y, gamma, Hb = ctx.saved_tensors
        ldx, ldb, ldc = ctx.lds
        Df = Df if ctx.has_D else None
        Bsz, T, H, P = y.shape
        N = Bm.shape[-1]
        nc = gamma.shape[1]
        dev = y.device
        dy = dy.contiguous()
        lib = load()
        G = _empty(Bsz, nc, H, N, P, dtype=torch.float32, device=dev)
        _check(lib.nsa_ssd_chunk_state(c_int(1), _p(Cm), c_long(ldc), _p(dy), c_long(H * P), _p(dt), _p(A), _p(G), c_void_p(0),
                                       c_int(Bsz), c_int(T), c_int(H), c_int(N), c_int(P), _stream()))
        dHn = _empty(Bsz, nc, H, N, P, dtype=torch.bfloat16, device=dev)
        _check(lib.nsa_ssd_state_bwd(_p(G), _p(gamma), c_void_p(0), _p(dHn), c_int(Bsz), c_int(nc), c_int(H), c_long(N * P),
                                     _stream()))
        del G
        dx = _empty(Bsz, T, H, P, dtype=torch.bfloat16, device=dev)
        # dB / dC: every head writes its own bf16 rows, summed afterwards (64 heads reducing into the
        # same fp32 rows with vector atomics was the slowest part of the kernel)
        dBh = _empty(Bsz, T, H, N, dtype=torch.bfloat16, device=dev)
        dCh = _empty(Bsz, T, H, N, dtype=torch.bfloat16, device=dev)
        q = _empty(Bsz, T, H, dtype=torch.float32, device=dev)
        k = _empty(Bsz, T, H, dtype=torch.float32, device=dev)
        rdx = _empty(Bsz, T, H, dtype=torch.float32, device=dev) if ctx.has_D else None
        _check(lib.nsa_ssd_chunk_grad_heads(_p(Cm), c_long(ldc), _p(Bm), c_long(ldb), _p(x), c_long(ldx), _p(dy), _p(y), _p(Hb),
                                            _p(dHn), _p(dt), _p(A), _p(Df), _p(dx), _p(dBh), _p(dCh), _p(q), _p(k), _p(rdx),
                                            c_int(Bsz), c_int(T), c_int(H), c_int(N), c_int(P), _stream()))
        dB = dBh.sum(2, dtype=torch.float32)
        dC = dCh.sum(2, dtype=torch.float32)
        del dBh, dCh
        # d(cum_t) = dy_t.(y_t - D x_t) - x_t.dx_t ;  a_k = dt_k A enters every cum_t with t >= k
        # (suffix sum over time, taken with time innermost: a scan along an outer dimension is slow)
        dcum = (q - k).transpose(1, 2).contiguous()
        pre = torch.cumsum(dcum, -1)
        da = (pre[..., -1:] - pre + dcum).transpose(1, 2)
        ddt = da * A[None, None, :] + k / dt.clamp_min(1e-20)
        dA = (da * dt).sum((0, 1))
        dD = rdx.sum((0, 1)) if ctx.has_D else None
        return (dx, ddt, dA, dB.view(Bsz, T, 1, N).to(torch.bfloat16), dC.view(Bsz, T, 1, N).to(torch.bfloat16), dD)


def copy_columns(dst: Tensor, src: Tensor) -> bool:
    """dst[...] = src for two tensors that are column slices of row-major matrices (last dimension
    contiguous, one uniform row pitch): a pitched device copy instead of a generic strided kernel.
    Returns False (nothing done) when the layouts do not qualify."""
    if dst.shape != src.shape or dst.dtype != src.dtype or not (dst.is_cuda and src.is_cuda) or dst.dim() < 2:
        return False
    def pitch(t):
        if t.stride(-1) != 1:
            return None
        p = t.stride(-2)
        if p < t.shape[-1]:
            return None
        exp = p
        for d in range(t.dim() - 2, -1, -1):           # leading dims must fold into rows of pitch p
            if t.shape[d] != 1 and t.stride(d) != exp:
                return None
            exp *= t.shape[d]
        return p
    dp, sp = pitch(dst), pitch(src)
    if dp is None or sp is None:
        return False
    es = dst.element_size()
    rows = dst.numel() // dst.shape[-1]
    _check(load().nsa_copy2d(_p(dst), c_long(dp * es), _p(src), c_long(sp * es), c_long(dst.shape[-1] * es), c_long(rows),
                             _stream()))
    return True


def sumsq(tensors) -> Tensor:
    """Sum of squares over a list of bf16 / fp32 CUDA tensors -> fp32 device scalar (no host sync)."""
    lib = load()
    dev = tensors[0].device
    out = _zeros((), dtype=torch.float32, device=dev)
    partial = _empty(int(lib.nsa_sumsq_parts()), dtype=torch.float32, device=dev)
    for g in tensors:
        if g.dtype not in (torch.bfloat16, torch.float32) or not g.is_contiguous():
            g = g.float().contiguous()
        _check(lib.nsa_sumsq(_p(g), c_long(g.numel()), c_int(int(g.dtype == torch.float32)), _p(partial), _p(out), c_int(1),
                             _stream()))
    return out


def affine_quantize(t: Tensor, bits: int, q_block: int):
    """CUDA form of :func:`nsa_optim_b200.ops.quant.affine_quantize` for fp32 matrices."""
    rows, cols = t.shape
    nblk = -(-cols // q_block)
    t = t.float().contiguous()
    q = _empty(rows, nblk * q_block, dtype=torch.uint8, device=t.device)
    scale = _empty(rows, nblk, dtype=torch.float32, device=t.device)
    zero = _empty(rows, nblk, dtype=torch.float32, device=t.device)
    _check(load().nsa_affine_quant(_p(t), _p(q), _p(scale), _p(zero), c_long(rows), c_int(cols), c_int(q_block), c_int(bits),
                                   _stream()))
    return q, scale, zero, cols


def affine_dequantize(q: Tensor, scale: Tensor, zero: Tensor, orig_cols: int) -> Tensor:
    rows = q.shape[0]
    q_block = q.shape[1] // scale.shape[1]
    out = _empty(rows, orig_cols, dtype=torch.float32, device=q.device)
    _check(load().nsa_affine_dequant(_p(q.contiguous()), _p(scale.contiguous()), _p(zero.contiguous()), _p(out), c_long(rows),
                                     c_int(orig_cols), c_int(q_block), _stream()))
    return out


def mamba3_gate(u: Tensor, dt: Tensor, A: Tensor, Bc: Tensor, Cc: Tensor, D: Tensor) -> Tensor:
    """Forward-only sequential scan of the complex-state SSM (``csrc/mamba3.cu``).
    u, dt (B, L, H) ; A (H, N, 2) ; Bc, Cc (B, L, H, N, 2) ; D (H)  ->  gate (B, L, H) fp32 with
    gate_t = Re<C_t, h_t> + D; the block output is x_t * gate_t."""
    B, L, H = u.shape
    N = A.shape[1]
    f = lambda t: t.detach().float().contiguous()
    u, dt, A, Bc, Cc, D = f(u), f(dt), f(A), f(Bc), f(Cc), f(D)
    gate = _empty(B, L, H, dtype=torch.float32, device=u.device)
    _check(load().nsa_mamba3_scan(_p(u), _p(dt), _p(A), _p(Bc), _p(Cc), _p(D), _p(gate), c_int(B), c_int(L), c_int(H),
                                  c_int(N), _stream()))
    return gate


def ssd_scan(x, dt, A, Bm, Cm, D=None, chunk=256):
    """Mamba-2 SSD.  The shapes of the hybrid models (d_state 128, headdim 64, one group) run on
    the fused tcgen05 chunk kernels; other shapes use batched matmuls plus the native
    inter-chunk state pass."""
    if (x.shape[-1] == 64 and Bm.shape[-1] == 128 and Bm.shape[2] == 1 and x.dtype == torch.bfloat16
            and Bm.dtype == torch.bfloat16 and Cm.dtype == torch.bfloat16):
        return _SSD.apply(x, dt, A, Bm, Cm, D)
    return _ssd_scan_batched(x, dt, A, Bm, Cm, D, chunk)


def _ssd_scan_batched(x, dt, A, Bm, Cm, D=None, chunk=256):
    """Chunked SSD: the per-chunk terms are batched tensor-core matmuls over all chunks at once,
    the inter-chunk recurrence is one native kernel (forward) and one (backward)."""
    F = torch.nn.functional
    Bsz, T, H, P = x.shape
    G, N = Bm.shape[2], Bm.shape[3]
    L = min(chunk, 128, T)
    pad = (-T) % L
    if pad:
        x = F.pad(x, (0, 0, 0, 0, 0, pad))
        dt = F.pad(dt, (0, 0, 0, pad))
        Bm = F.pad(Bm, (0, 0, 0, 0, 0, pad))
        Cm = F.pad(Cm, (0, 0, 0, 0, 0, pad))
    Tp = T + pad
    nc = Tp // L
    rep = H // G
    cdt = x.dtype
    xr = x.reshape(Bsz, nc, L, H, P)
    dtr = dt.float().reshape(Bsz, nc, L, H)
    Br = Bm.reshape(Bsz, nc, L, G, N)
    Cr = Cm.reshape(Bsz, nc, L, G, N)
    a = dtr * A.float()[None, None, None, :]
    cum = torch.cumsum(a, dim=2)
    total = cum[:, :, -1]
    xdt = (xr.float() * dtr[..., None]).to(cdt)
    CB = torch.einsum("bclgn,bcsgn->bcgls", Cr, Br)                      # (B,nc,G,L,L) in the compute dtype
    seg = cum.permute(0, 1, 3, 2)                                        # (B,nc,H,L)
    tri = torch.ones(L, L, dtype=torch.bool, device=x.device).tril()
    dec = torch.exp((seg[..., :, None] - seg[..., None, :]).masked_fill(~tri, float("-inf"))).to(cdt)
    M = CB.repeat_interleave(rep, dim=2) * dec if rep > 1 else CB * dec  # (B,nc,H,L,L)
    y = torch.einsum("bchls,bcshp->bclhp", M, xdt)
    w_end = torch.exp(total[:, :, None, :] - cum)
    Bh = Br.repeat_interleave(rep, dim=3) if rep > 1 else Br
    S_loc = torch.einsum("bclhp,bclhn->bchpn", (xdt.float() * w_end[..., None]).to(cdt), Bh).float()
    Hprev = _SSDStatePass.apply(S_loc, torch.exp(total))                 # (B,nc,H,P,N) fp32
    Ch = Cr.repeat_interleave(rep, dim=3) if rep > 1 else Cr
    y_inter = torch.einsum("bclhn,bchpn->bclhp", (Ch.float() * torch.exp(cum)[..., None]).to(cdt), Hprev.to(cdt))
    y = (y + y_inter).reshape(Bsz, Tp, H, P)[:, :T]
    if D is not None:
        y = y + (x[:, :T].float() * D.float()[None, None, :, None]).to(cdt)
    return y.to(cdt)
