"""Optimizers, parameter grouping, learning-rate schedules and preconditioning reports.

Reference behaviour (nngabe/nsa_optim, optimizers.py): factory :22-62, param groups :65-83,
AdamW :86-94, low-bit AdamW :97-145, SOAP :152-179, Shampoo :182-244, SOAP low-bit factory
:247-284, SOAPReference :287-426, ShampooReference :429-538, SOAPLowBit :562-1007,
schedulers :1010-1046, coverage report :1049-1198.

The reference delegates AdamW8bit/4bit and SOAP to external packages (falling back to plain
AdamW when they are missing).  Here every optimizer type is implemented in-tree:

* :class:`AdamW` - decoupled weight decay Adam with fp32 maths on bf16 or fp32 parameters,
  optional fp32 master copy.
* :class:`AdamWLowBit` - the same update with blockwise dynamically quantised moments
  (8-bit: block 256, dynamic-tree code book, signed first / unsigned second moment; tensors
  below 4096 elements or not a multiple of the block keep fp32 moments).
* :class:`SOAPReference`, :class:`ShampooReference` - full precision references.
* :class:`SOAPLowBit` - block-diagonal SOAP: Kronecker factors ``L += G G^T``, ``R += G^T G``
  as EMAs, eigenbases refreshed every ``precondition_frequency`` steps by one
  power-iteration + QR step, Adam in the eigenbasis, eigenbases stored affine-quantised in
  sub-row blocks and Adam moments stored blockwise 4- or 8-bit.

On CUDA tensors the elementwise update kernels come from the native library
(``ops.native``); on CPU the PyTorch statements below run.  Every ``step`` accepts
``grad_scale`` (a 0-d tensor multiplied into each gradient inside the update), which lets a
clip coefficient stay on the device.
"""
from __future__ import annotations

import math
from typing import Any, Callable, Dict, Iterable, List, Optional, Tuple

import torch
import torch.nn as nn
from torch import Tensor
from torch.optim import Optimizer

from .config import OptimizerConfig, OptimizerType
from .ops import quant


# --------------------------------------------------------------------------------------
# parameter groups
# --------------------------------------------------------------------------------------
def is_no_decay(name: str, param: Tensor) -> bool:
    """1-D tensors, biases, and anything whose name mentions layernorm or embed skip decay.

    A shard piece handed out by the sharded runtime is always 1-D, whatever the parameter it was
    cut from; it carries ``_is_matrix`` / ``_no_weight_decay`` describing the original parameter,
    and those decide instead of ``ndim`` (otherwise every weight matrix would lose its decay as
    soon as the world size exceeds one)."""
    lname = name.lower()
    by_name = name.endswith(".bias") or "layernorm" in lname or "embed" in lname
    if hasattr(param, "_is_matrix"):
        return by_name or bool(getattr(param, "_no_weight_decay", False)) or not param._is_matrix
    return param.ndim == 1 or by_name or bool(getattr(param, "_no_weight_decay", False))


def get_param_groups(model_or_named, weight_decay: float) -> List[Dict[str, Any]]:
    named = model_or_named.named_parameters() if isinstance(model_or_named, nn.Module) else model_or_named
    decay, no_decay, dn, nn_ = [], [], [], []
    for name, p in named:
        if not p.requires_grad:
            continue
        if is_no_decay(name, p):
            no_decay.append(p)
            nn_.append(name)
        else:
            decay.append(p)
            dn.append(name)
    return [
        {"params": decay, "weight_decay": weight_decay, "param_names": dn},
        {"params": no_decay, "weight_decay": 0.0, "param_names": nn_},
    ]


def _native_for(t: Tensor):
    if not t.is_cuda:
        return None
    from . import ops
    if ops.get_backend() == "torch":
        return None
    return ops.native_module()


def _grad_of(p: Tensor) -> Optional[Tensor]:
    """Gradient of a parameter or of a shard piece (whose fp32 gradient view may differ in
    dtype from the piece and therefore cannot live in ``.grad``)."""
    g = getattr(p, "_fp32_grad", None)
    return g if g is not None else p.grad


def _scaled(grad: Tensor, grad_scale: Optional[Tensor]) -> Tensor:
    g = grad.float()
    return g if grad_scale is None else g * grad_scale.to(g.device, torch.float32)


# --------------------------------------------------------------------------------------
# AdamW
# --------------------------------------------------------------------------------------
class AdamW(Optimizer):
    def __init__(self, params, lr=1e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1,
                 master_weights: bool = False):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))
        self.master_weights = master_weights

    def _init(self, p: Tensor, state: dict):
        state["step"] = 0
        state["exp_avg"] = torch.zeros_like(p, dtype=torch.float32)
        state["exp_avg_sq"] = torch.zeros_like(p, dtype=torch.float32)
        if self.master_weights and p.dtype != torch.float32:
            state["master"] = p.detach().float().clone()

    @torch.no_grad()
    def step(self, closure: Optional[Callable] = None, grad_scale: Optional[Tensor] = None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            b1, b2 = group["betas"]
            lr, eps, wd = group["lr"], group["eps"], group["weight_decay"]
            for p in group["params"]:
                g_ = _grad_of(p)
                if g_ is None:
                    continue
                st = self.state[p]
                if not st:
                    self._init(p, st)
                st["step"] += 1
                t = st["step"]
                nat = _native_for(p)
                if nat is not None and nat.supports("adamw", p):
                    nat.adamw_step(p, g_, st["exp_avg"], st["exp_avg_sq"], st.get("master"),
                                   t, lr, b1, b2, eps, wd, grad_scale)
                    continue
                g = _scaled(g_, grad_scale)
                w = st.get("master")
                w = p.float() if w is None else w
                w.mul_(1 - lr * wd)
                st["exp_avg"].mul_(b1).add_(g, alpha=1 - b1)
                st["exp_avg_sq"].mul_(b2).addcmul_(g, g, value=1 - b2)
                denom = (st["exp_avg_sq"].sqrt() / math.sqrt(1 - b2 ** t)).add_(eps)
                w.addcdiv_(st["exp_avg"], denom, value=-lr / (1 - b1 ** t))
                p.copy_(w)
        return loss


# --------------------------------------------------------------------------------------
# low-bit AdamW
# --------------------------------------------------------------------------------------
class AdamWLowBit(Optimizer):
    """AdamW with blockwise dynamically quantised moments.

    State per parameter: ``step``, ``exp_avg`` / ``exp_avg_sq`` (uint8 codes, or fp32 for
    tensors that are too small or not a multiple of the block) and, for quantised tensors,
    ``exp_avg_absmax`` / ``exp_avg_sq_absmax`` (one fp32 scale per block).
    """

    MIN_QUANT_NUMEL = 4096

    def __init__(self, params, lr=1e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1,
                 bits: int = 8, block_size: Optional[int] = None):
        if bits not in (4, 8):
            raise ValueError("bits must be 4 or 8")
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))
        self.bits = bits
        self.block_size = block_size or (256 if bits == 8 else 128)

    def quantisable(self, p: Tensor) -> bool:
        n = getattr(p, "_logical_numel", p.numel())
        return n >= self.MIN_QUANT_NUMEL and p.numel() % self.block_size == 0

    def _init(self, p: Tensor, st: dict):
        st["step"] = 0
        if self.quantisable(p):
            n, nb = p.numel(), p.numel() // self.block_size
            nbytes = n if self.bits == 8 else n // 2
            zero_m = quant.quantize_blockwise(torch.zeros(self.block_size), self.bits, True, self.block_size)[0]
            zero_v = quant.quantize_blockwise(torch.zeros(self.block_size), self.bits, False, self.block_size)[0]
            st["exp_avg"] = torch.full((nbytes,), int(zero_m[0]), dtype=torch.uint8, device=p.device)
            st["exp_avg_sq"] = torch.full((nbytes,), int(zero_v[0]), dtype=torch.uint8, device=p.device)
            st["exp_avg_absmax"] = torch.zeros(nb, dtype=torch.float32, device=p.device)
            st["exp_avg_sq_absmax"] = torch.zeros(nb, dtype=torch.float32, device=p.device)
        else:
            st["exp_avg"] = torch.zeros_like(p, dtype=torch.float32)
            st["exp_avg_sq"] = torch.zeros_like(p, dtype=torch.float32)

    @torch.no_grad()
    def step(self, closure: Optional[Callable] = None, grad_scale: Optional[Tensor] = None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        B = self.block_size
        for group in self.param_groups:
            b1, b2 = group["betas"]
            lr, eps, wd = group["lr"], group["eps"], group["weight_decay"]
            for p in group["params"]:
                g_ = _grad_of(p)
                if g_ is None:
                    continue
                st = self.state[p]
                if not st:
                    self._init(p, st)
                st["step"] += 1
                t = st["step"]
                quantised = st["exp_avg"].dtype == torch.uint8
                nat = _native_for(p)
                if nat is not None and nat.supports("adamw_lowbit", p) and (self.bits == 8 or not quantised):
                    if quantised:
                        nat.adamw8bit_step(p, g_, st["exp_avg"], st["exp_avg_absmax"],
                                           st["exp_avg_sq"], st["exp_avg_sq_absmax"],
                                           t, lr, b1, b2, eps, wd, grad_scale, B)
                    else:
                        nat.adamw_step(p, g_, st["exp_avg"], st["exp_avg_sq"], None,
                                       t, lr, b1, b2, eps, wd, grad_scale)
                    continue
                g = _scaled(g_, grad_scale).reshape(-1)
                if quantised:
                    m = quant.dequantize_blockwise(st["exp_avg"], st["exp_avg_absmax"], self.bits, True, B)
                    v = quant.dequantize_blockwise(st["exp_avg_sq"], st["exp_avg_sq_absmax"], self.bits, False, B)
                else:
                    m, v = st["exp_avg"].reshape(-1), st["exp_avg_sq"].reshape(-1)
                m = m.mul_(b1).add_(g, alpha=1 - b1)
                v = v.mul_(b2).addcmul_(g, g, value=1 - b2)
                w = p.float().reshape(-1)
                w.mul_(1 - lr * wd)
                denom = (v.sqrt() / math.sqrt(1 - b2 ** t)).add_(eps)
                w.addcdiv_(m, denom, value=-lr / (1 - b1 ** t))
                p.copy_(w.view_as(p))
                if quantised:
                    st["exp_avg"], st["exp_avg_absmax"] = quant.quantize_blockwise(m, self.bits, True, B)
                    st["exp_avg_sq"], st["exp_avg_sq_absmax"] = quant.quantize_blockwise(v, self.bits, False, B)
        return loss


# --------------------------------------------------------------------------------------
# full-precision SOAP and Shampoo references
# --------------------------------------------------------------------------------------
def _power_qr(factor: Tensor, basis: Tensor) -> Tensor:
    """One orthogonal-iteration step: orthonormal basis of ``factor @ basis``."""
    return torch.linalg.qr(factor @ basis)[0]


class SOAPReference(Optimizer):
    """Full-precision SOAP: Adam run in the eigenbasis of the Shampoo Kronecker factors."""

    def __init__(self, params: Iterable, lr: float = 3e-3, betas: Tuple[float, float] = (0.9, 0.95),
                 shampoo_beta: float = 0.95, eps: float = 1e-8, weight_decay: float = 0.01,
                 precondition_frequency: int = 10, max_precond_dim: int = 8192):
        super().__init__(params, dict(lr=lr, betas=betas, shampoo_beta=shampoo_beta, eps=eps,
                                      weight_decay=weight_decay,
                                      precondition_frequency=precondition_frequency,
                                      max_precond_dim=max_precond_dim))
        self._step = 0

    @torch.no_grad()
    def step(self, closure: Optional[Callable] = None, grad_scale: Optional[Tensor] = None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        self._step += 1
        for group in self.param_groups:
            b1, b2 = group["betas"]
            sb, lr, eps, wd = group["shampoo_beta"], group["lr"], group["eps"], group["weight_decay"]
            freq, max_dim = group["precondition_frequency"], group["max_precond_dim"]
            for p in group["params"]:
                g_ = _grad_of(p)
                if g_ is None:
                    continue
                g = _scaled(g_, grad_scale)
                st = self.state[p]
                if not st:
                    st["step"] = 0
                    st["exp_avg"] = torch.zeros_like(p, dtype=torch.float32)
                    st["exp_avg_sq"] = torch.zeros_like(p, dtype=torch.float32)
                    if g.ndim == 2 and max(g.shape) <= max_dim:
                        r, c = g.shape
                        st["L"] = torch.zeros(r, r, device=g.device)
                        st["R"] = torch.zeros(c, c, device=g.device)
                        st["QL"] = torch.eye(r, device=g.device)
                        st["QR"] = torch.eye(c, device=g.device)
                st["step"] += 1
                t = st["step"]
                if wd > 0:
                    p.mul_(1 - lr * wd)
                m, v = st["exp_avg"], st["exp_avg_sq"]
                precond = "L" in st
                if precond:
                    st["L"].mul_(sb).add_(g @ g.T, alpha=1 - sb)
                    st["R"].mul_(sb).add_(g.T @ g, alpha=1 - sb)
                    if t % freq == 0:
                        ql, qr = st["QL"], st["QR"]
                        ql_new, qr_new = _power_qr(st["L"], ql), _power_qr(st["R"], qr)
                        # rotate the first moment into the new basis; the second moment is kept
                        m.copy_(ql_new.T @ (ql @ m @ qr.T) @ qr_new)
                        st["QL"], st["QR"] = ql_new, qr_new
                    g = st["QL"].T @ g @ st["QR"]
                m.mul_(b1).add_(g, alpha=1 - b1)
                v.mul_(b2).addcmul_(g, g, value=1 - b2)
                upd = m / ((v.sqrt() / math.sqrt(1 - b2 ** t)).add_(eps))
                if precond:
                    upd = st["QL"] @ upd @ st["QR"].T
                p.add_(upd.to(p.dtype), alpha=-lr / (1 - b1 ** t))
        return loss


class ShampooReference(Optimizer):
    """Full-precision Shampoo: inverse fourth roots of EMA'd Kronecker factors, refreshed every
    ``precondition_frequency`` steps, with momentum on the preconditioned gradient."""

    def __init__(self, params: Iterable, lr: float = 1e-3, betas: Tuple[float, float] = (0.9, 0.999),
                 eps: float = 1e-12, weight_decay: float = 0.01, precondition_frequency: int = 10,
                 max_precond_dim: int = 8192):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay,
                                      precondition_frequency=precondition_frequency,
                                      max_precond_dim=max_precond_dim))
        self._step = 0

    @staticmethod
    def _matrix_power(matrix: Tensor, power: float) -> Tensor:
        try:
            vals, vecs = torch.linalg.eigh(matrix.double())
            vals = vals.clamp_min(1e-10)
            return ((vecs * vals.pow(power)) @ vecs.T).float()
        except Exception:  # noqa: BLE001 - a failed decomposition leaves the step unpreconditioned
            return torch.eye(matrix.shape[0], device=matrix.device)

    @torch.no_grad()
    def step(self, closure: Optional[Callable] = None, grad_scale: Optional[Tensor] = None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        self._step += 1
        for group in self.param_groups:
            b1, b2 = group["betas"]
            lr, eps, wd = group["lr"], group["eps"], group["weight_decay"]
            freq, max_dim = group["precondition_frequency"], group["max_precond_dim"]
            for p in group["params"]:
                g_ = _grad_of(p)
                if g_ is None:
                    continue
                g = _scaled(g_, grad_scale)
                st = self.state[p]
                if not st:
                    st["step"] = 0
                    st["exp_avg"] = torch.zeros_like(p, dtype=torch.float32)
                    if g.ndim == 2 and max(g.shape) <= max_dim:
                        r, c = g.shape
                        st["L"] = torch.zeros(r, r, device=g.device)
                        st["R"] = torch.zeros(c, c, device=g.device)
                        st["L_inv"] = torch.eye(r, device=g.device)
                        st["R_inv"] = torch.eye(c, device=g.device)
                st["step"] += 1
                t = st["step"]
                if wd > 0:
                    p.mul_(1 - lr * wd)
                if "L" in st:
                    st["L"].mul_(b2).add_(g @ g.T, alpha=1 - b2)
                    st["R"].mul_(b2).add_(g.T @ g, alpha=1 - b2)
                    if t % freq == 0:
                        eye_l = torch.eye(st["L"].shape[0], device=g.device)
                        eye_r = torch.eye(st["R"].shape[0], device=g.device)
                        st["L_inv"] = self._matrix_power(st["L"] + eps * eye_l, -0.25)
                        st["R_inv"] = self._matrix_power(st["R"] + eps * eye_r, -0.25)
                    g = st["L_inv"] @ g @ st["R_inv"]
                st["exp_avg"].mul_(b1).add_(g, alpha=1 - b1)
                p.add_(st["exp_avg"].to(p.dtype), alpha=-lr / (1 - b1 ** t))
        return loss


# --------------------------------------------------------------------------------------
# low-bit SOAP
# --------------------------------------------------------------------------------------
class SOAPLowBit(Optimizer):
    """Block-diagonal SOAP with quantised state.

    A 2-D parameter (or a flat shard that carries ``_orig_2d_shape``) is tiled into blocks of
    at most ``max_precond_dim`` rows and columns.  Per block: EMA Kronecker factors ``L``,
    ``R`` (fp32), eigenbases ``QL``, ``QR`` stored affine-quantised (``bits``, sub-row blocks of
    ``q_block_size``), Adam moments in the eigenbasis stored blockwise ``bits``-bit
    (block ``moment_block``, default 64) when ``quantize_moments``.

    State keys per parameter follow the reference's layout (optimizers.py:828-871):
    ``step, exp_avg, exp_avg_sq, orig_2d_shape, num_blocks_row, num_blocks_col, block_size,
    QL_q_blocks, QR_q_blocks, block_shapes`` with ``Q*_q_blocks[i] = (codes, scale, zero_point,
    orig_cols)``; additions: ``L_blocks``, ``R_blocks`` and, for quantised moments,
    ``exp_avg_absmax`` / ``exp_avg_sq_absmax``.
    """

    def __init__(self, params: Iterable, lr: float = 3e-3, betas: Tuple[float, float] = (0.9, 0.95),
                 shampoo_beta: float = 0.95, eps: float = 1e-8, weight_decay: float = 0.01,
                 precondition_frequency: int = 10, max_precond_dim: int = 8192, bits: int = 4,
                 q_block_size: int = 32, use_optimized: bool = True, distributed: Optional[bool] = None,
                 orig_param_shapes: Optional[Dict[int, Tuple[str, Tuple[int, ...]]]] = None,
                 quantize_moments: bool = True, moment_block: int = 64, verbose: bool = False):
        super().__init__(params, dict(lr=lr, betas=betas, shampoo_beta=shampoo_beta, eps=eps,
                                      weight_decay=weight_decay,
                                      precondition_frequency=precondition_frequency,
                                      max_precond_dim=max_precond_dim, bits=bits))
        self._step = 0
        self.bits, self.q_block_size = bits, q_block_size
        self.quantize_moments, self.moment_block = quantize_moments, moment_block
        self.orig_param_shapes = orig_param_shapes or {}
        if distributed is None:
            import torch.distributed as dist
            distributed = dist.is_available() and dist.is_initialized()
        self.distributed = distributed
        if verbose:
            print(f"SOAPLowBit: {bits}-bit, block_size={q_block_size}"
                  f"{' (distributed)' if distributed else ''}")

    # ---- shape helpers
    def _get_orig_shape(self, p: Tensor) -> Optional[Tuple[int, ...]]:
        shape = getattr(p, "_orig_2d_shape", None)
        if shape is not None:
            return tuple(shape)
        rec = self.orig_param_shapes.get(p.data_ptr())
        return None if rec is None else tuple(rec[1])

    def _is_preconditionable(self, p: Tensor) -> Tuple[bool, Optional[Tuple[int, int]]]:
        if p.ndim == 2:
            return True, tuple(p.shape)
        shape = self._get_orig_shape(p)
        if shape is not None and len(shape) == 2 and p.numel() == shape[0] * shape[1]:
            return True, shape
        return False, None

    # ---- codecs
    def _quantize_block(self, t: Tensor):
        return quant.affine_quantize(t, self.bits, self.q_block_size)

    def _dequantize_block(self, q: Tensor, scale: Tensor, zp: Tensor, orig_cols: int) -> Tensor:
        return quant.affine_dequantize(q, scale, zp, orig_cols)

    def _quantize_per_tensor(self, t: Tensor):
        return quant.affine_quantize_tensor(t, self.bits)

    def _dequantize_per_tensor(self, q: Tensor, scale: Tensor, zp: Tensor) -> Tensor:
        return quant.affine_dequantize_tensor(q, scale, zp)

    def _moments_quantised(self, numel: int) -> bool:
        return self.quantize_moments and numel % self.moment_block == 0 and numel >= 4096

    def _load_moment(self, st: dict, key: str, signed: bool, shape) -> Tensor:
        if st[key].dtype == torch.uint8:
            return quant.dequantize_blockwise(st[key], st[key + "_absmax"], self.bits, signed,
                                              self.moment_block).view(shape)
        return st[key].view(shape)

    def _store_moment(self, st: dict, key: str, signed: bool, val: Tensor) -> None:
        if st[key].dtype == torch.uint8:
            st[key], st[key + "_absmax"] = quant.quantize_blockwise(
                val.reshape(-1), self.bits, signed, self.moment_block)
        else:
            st[key].copy_(val.view_as(st[key]))

    def _init_state(self, p: Tensor, st: dict, max_dim: int):
        st["step"] = 0
        ok, shape = self._is_preconditionable(p)
        n = p.numel()
        if ok and self._moments_quantised(n):
            zm = quant.quantize_blockwise(torch.zeros(self.moment_block), self.bits, True, self.moment_block)[0]
            zv = quant.quantize_blockwise(torch.zeros(self.moment_block), self.bits, False, self.moment_block)[0]
            nbytes = n if self.bits == 8 else n // 2
            st["exp_avg"] = torch.full((nbytes,), int(zm[0]), dtype=torch.uint8, device=p.device)
            st["exp_avg_sq"] = torch.full((nbytes,), int(zv[0]), dtype=torch.uint8, device=p.device)
            st["exp_avg_absmax"] = torch.zeros(n // self.moment_block, device=p.device)
            st["exp_avg_sq_absmax"] = torch.zeros(n // self.moment_block, device=p.device)
        else:
            st["exp_avg"] = torch.zeros(n, dtype=torch.float32, device=p.device)
            st["exp_avg_sq"] = torch.zeros(n, dtype=torch.float32, device=p.device)
        if not ok:
            return
        rows, cols = shape
        bs = max_dim
        nbr, nbc = -(-rows // bs), -(-cols // bs)
        st.update(orig_2d_shape=shape, num_blocks_row=nbr, num_blocks_col=nbc, block_size=bs,
                  QL_q_blocks=[], QR_q_blocks=[], block_shapes=[], L_blocks=[], R_blocks=[])
        for i in range(nbr):
            for j in range(nbc):
                r = min(bs, rows - i * bs)
                c = min(bs, cols - j * bs)
                st["block_shapes"].append((r, c))
                st["L_blocks"].append(torch.zeros(r, r, device=p.device))
                st["R_blocks"].append(torch.zeros(c, c, device=p.device))
                st["QL_q_blocks"].append(self._quantize_block(torch.eye(r, device=p.device)))
                st["QR_q_blocks"].append(self._quantize_block(torch.eye(c, device=p.device)))

    @torch.no_grad()
    def step(self, closure: Optional[Callable] = None, grad_scale: Optional[Tensor] = None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        self._step += 1
        for group in self.param_groups:
            b1, b2 = group["betas"]
            sb, lr, eps, wd = group["shampoo_beta"], group["lr"], group["eps"], group["weight_decay"]
            freq, max_dim = group["precondition_frequency"], group["max_precond_dim"]
            for p in group["params"]:
                g_ = _grad_of(p)
                if g_ is None:
                    continue
                st = self.state[p]
                if not st:
                    self._init_state(p, st, max_dim)
                st["step"] += 1
                t = st["step"]
                g_full = _scaled(g_, grad_scale)
                w = p.float()
                if wd > 0:
                    w.mul_(1 - lr * wd)
                bc1, bc2 = 1 - b1 ** t, 1 - b2 ** t
                if "orig_2d_shape" not in st:
                    m, v = st["exp_avg"].view_as(w), st["exp_avg_sq"].view_as(w)
                    m.mul_(b1).add_(g_full, alpha=1 - b1)
                    v.mul_(b2).addcmul_(g_full, g_full, value=1 - b2)
                    w.addcdiv_(m, (v.sqrt() / math.sqrt(bc2)).add_(eps), value=-lr / bc1)
                    p.copy_(w)
                    continue
                rows, cols = st["orig_2d_shape"]
                G = g_full.view(rows, cols)
                W = w.view(rows, cols)
                M = self._load_moment(st, "exp_avg", True, (rows, cols)).clone()
                V = self._load_moment(st, "exp_avg_sq", False, (rows, cols)).clone()
                bs, nbc = st["block_size"], st["num_blocks_col"]
                refresh = t % freq == 0
                nat = _native_for(p) if (cols % 8 == 0 and rows % 8 == 0 and bs % 8 == 0) else None
                # native path: every product below is a tcgen05 GEMM on bf16 operands with fp32
                # accumulation (the gradient is scaled once so that G G^T and G^T G accumulate straight
                # into the EMA factors); PyTorch fp32 matmuls otherwise
                Gs = (G * math.sqrt(1 - sb)).to(torch.bfloat16) if nat is not None else None
                Gh = G.to(torch.bfloat16) if nat is not None else None
                for bi in range(len(st["block_shapes"])):
                    i, j = divmod(bi, nbc)
                    r, c = st["block_shapes"][bi]
                    rs, cs = slice(i * bs, i * bs + r), slice(j * bs, j * bs + c)
                    Gb = G[rs, cs]
                    L, R = st["L_blocks"][bi], st["R_blocks"][bi]
                    if nat is not None:
                        gsb = Gs[rs, cs]
                        L.mul_(sb)
                        R.mul_(sb)
                        nat.gemm(gsb, gsb, False, False, out=L, accumulate=True)       # L += (1-sb) G G^T
                        nat.gemm(gsb, gsb, True, True, out=R, accumulate=True)         # R += (1-sb) G^T G
                    else:
                        L.mul_(sb).add_(Gb @ Gb.T, alpha=1 - sb)
                        R.mul_(sb).add_(Gb.T @ Gb, alpha=1 - sb)
                    QL = self._dequantize_block(*st["QL_q_blocks"][bi])
                    QR = self._dequantize_block(*st["QR_q_blocks"][bi])
                    if refresh:
                        QLn, QRn = _power_qr(L, QL), _power_qr(R, QR)
                        M[rs, cs] = QLn.T @ (QL @ M[rs, cs] @ QR.T) @ QRn
                        st["QL_q_blocks"][bi] = self._quantize_block(QLn)
                        st["QR_q_blocks"][bi] = self._quantize_block(QRn)
                        # use what will be read back next step, so projection and storage agree
                        QL = self._dequantize_block(*st["QL_q_blocks"][bi])
                        QR = self._dequantize_block(*st["QR_q_blocks"][bi])
                    if nat is not None:
                        QLh, QRh = QL.to(torch.bfloat16), QR.to(torch.bfloat16)
                        T1 = nat.gemm(QLh, Gh[rs, cs], True, True)                                 # QL^T G
                        Gp = nat.gemm(T1, QRh, False, True, out_dtype=torch.float32)               # (QL^T G) QR
                    else:
                        Gp = QL.T @ Gb @ QR
                    Mb = M[rs, cs].mul_(b1).add_(Gp, alpha=1 - b1)
                    Vb = V[rs, cs].mul_(b2).addcmul_(Gp, Gp, value=1 - b2)
                    upd = Mb / ((Vb.sqrt() / math.sqrt(bc2)).add_(eps))
                    if nat is not None:
                        U1 = nat.gemm(QLh, upd.to(torch.bfloat16), False, True)                    # QL upd
                        U = nat.gemm(U1, QRh, False, False, out_dtype=torch.float32)               # (QL upd) QR^T
                        W[rs, cs].add_(U, alpha=-lr / bc1)
                    else:
                        W[rs, cs].add_(QL @ upd @ QR.T, alpha=-lr / bc1)
                self._store_moment(st, "exp_avg", True, M)
                self._store_moment(st, "exp_avg_sq", False, V)
                p.copy_(W.view_as(p))
        return loss


# --------------------------------------------------------------------------------------
# sharding-independent view of elementwise state (used by checkpoints)
# --------------------------------------------------------------------------------------
_NOT_ELEMENTWISE = ("L", "R", "L_inv", "QL", "L_blocks", "orig_2d_shape")


def _moment_codec(optimizer: Optimizer) -> Tuple[int, int]:
    """(bits, block) of the blockwise moment codec of ``optimizer`` (0, 0 when moments are fp32)."""
    if isinstance(optimizer, AdamWLowBit):
        return optimizer.bits, optimizer.block_size
    if isinstance(optimizer, SOAPLowBit):
        return optimizer.bits, optimizer.moment_block
    return 0, 0


def state_moments(state: Dict[str, Any], bits: int, block: int) -> Optional[Tuple[int, Tensor, Optional[Tensor]]]:
    """``(step, exp_avg, exp_avg_sq)`` of one state entry as flat fp32 tensors, dequantised when
    they are stored as codes; ``None`` for an entry that is not purely elementwise (Kronecker
    factors, eigenbases) or has no first moment."""
    if "exp_avg" not in state or any(k in state for k in _NOT_ELEMENTWISE):
        return None

    def load(key: str, signed: bool) -> Optional[Tensor]:
        t = state.get(key)
        if t is None:
            return None
        if t.dtype == torch.uint8:
            return quant.dequantize_blockwise(t, state[key + "_absmax"], bits, signed, block).float().reshape(-1)
        return t.float().reshape(-1)

    return int(state.get("step", 0)), load("exp_avg", True), load("exp_avg_sq", False)


def fresh_state(optimizer: Optimizer, p: Tensor) -> Optional[Dict[str, Any]]:
    """The state ``optimizer`` would create for ``p`` on its first step (``None`` for the
    optimizers that build it inline)."""
    st: Dict[str, Any] = {}
    if isinstance(optimizer, (AdamW, AdamWLowBit)):
        optimizer._init(p, st)
    elif isinstance(optimizer, SOAPLowBit):
        group = next(g for g in optimizer.param_groups if any(q is p for q in g["params"]))
        optimizer._init_state(p, st, group["max_precond_dim"])
    else:
        return None
    return st


def install_moments(optimizer: Optimizer, p: Tensor, step: int, m: Tensor, v: Optional[Tensor]) -> bool:
    """Gives ``p`` a state whose moments are ``m`` / ``v`` (flat fp32, ``p.numel()`` long), in the
    storage format this optimizer uses for ``p``.  False when ``p`` does not take elementwise
    state here (a preconditioned matrix) and was left untouched."""
    st = fresh_state(optimizer, p)
    if st is None or any(k in st for k in _NOT_ELEMENTWISE) or m.numel() != p.numel():
        return False
    bits, block = _moment_codec(optimizer)
    for key, val, signed in (("exp_avg", m, True), ("exp_avg_sq", v, False)):
        if key not in st or val is None:
            continue
        val = val.to(p.device, torch.float32)
        if st[key].dtype == torch.uint8:
            st[key], st[key + "_absmax"] = quant.quantize_blockwise(val, bits, signed, block)
        else:
            st[key].copy_(val.view_as(st[key]))
    st["step"] = int(step)
    optimizer.state[p] = st
    return True


def state_fits(optimizer: Optimizer, p: Tensor, state: Dict[str, Any]) -> bool:
    """Whether a saved state entry has the tensor sizes this optimizer's kernels will index for
    ``p``.  Guards a resume against a checkpoint written under another sharding."""
    bits, block = _moment_codec(optimizer)
    n = p.numel()
    for key in ("exp_avg", "exp_avg_sq", "master"):
        t = state.get(key)
        if not torch.is_tensor(t):
            continue
        want = n // 2 if (t.dtype == torch.uint8 and bits == 4) else n
        if t.numel() != want:
            return False
        am = state.get(key + "_absmax")
        if t.dtype == torch.uint8 and (not torch.is_tensor(am) or block == 0 or am.numel() != n // block):
            return False
    shape = state.get("orig_2d_shape")
    if shape is not None and int(shape[0]) * int(shape[1]) != n:
        return False
    for key in ("L", "R", "QL", "QR", "L_inv", "R_inv"):
        t = state.get(key)
        if torch.is_tensor(t) and p.ndim == 2 and t.shape[0] not in p.shape:
            return False
    return True


# --------------------------------------------------------------------------------------
# factory
# --------------------------------------------------------------------------------------
def create_adamw(param_groups: List[Dict], config: OptimizerConfig) -> Optimizer:
    return AdamW(param_groups, lr=config.learning_rate, betas=(config.beta1, config.beta2),
                 eps=config.eps, weight_decay=config.weight_decay,
                 master_weights=getattr(config, "master_weights", False))


def create_adamw_lowbit(param_groups: List[Dict], config: OptimizerConfig, bits: int = 8) -> Optimizer:
    return AdamWLowBit(param_groups, lr=config.learning_rate, betas=(config.beta1, config.beta2),
                       eps=config.eps, weight_decay=config.weight_decay, bits=bits)


def create_soap(param_groups: List[Dict], config: OptimizerConfig) -> Optimizer:
    return SOAPReference(param_groups, lr=config.learning_rate, betas=(config.beta1, config.beta2),
                         shampoo_beta=config.shampoo_beta, eps=config.eps,
                         weight_decay=config.weight_decay,
                         precondition_frequency=config.precondition_frequency,
                         max_precond_dim=config.max_precond_dim)


def create_shampoo(param_groups: List[Dict], config: OptimizerConfig, tensor_parallel_size: int = 1) -> Optimizer:
    return ShampooReference(param_groups, lr=config.learning_rate, betas=(config.beta1, config.beta2),
                            eps=max(config.eps, 1e-12), weight_decay=config.weight_decay,
                            precondition_frequency=config.precondition_frequency,
                            max_precond_dim=config.max_precond_dim)


def create_soap_lowbit(param_groups: List[Dict], config: OptimizerConfig, bits: int = 4,
                       use_optimized: bool = True,
                       orig_param_shapes: Optional[Dict[int, Tuple[str, Tuple[int, ...]]]] = None) -> Optimizer:
    return SOAPLowBit(param_groups, lr=config.learning_rate, betas=(config.beta1, config.beta2),
                      shampoo_beta=config.shampoo_beta, eps=config.eps,
                      weight_decay=config.weight_decay,
                      precondition_frequency=config.precondition_frequency,
                      max_precond_dim=config.max_precond_dim, bits=bits,
                      use_optimized=use_optimized, orig_param_shapes=orig_param_shapes)


def create_optimizer(model, config: OptimizerConfig, tensor_parallel_size: int = 1,
                     orig_param_shapes: Optional[Dict[int, Tuple[str, Tuple[int, ...]]]] = None) -> Optimizer:
    """``model`` is an ``nn.Module`` or an iterable of ``(name, parameter)`` pairs (the sharded
    runtime passes its per-rank shard views)."""
    groups = get_param_groups(model, config.weight_decay)
    groups = [{k: v for k, v in g.items() if k != "param_names"} for g in groups]
    groups = [g for g in groups if g["params"]]
    t = config.optimizer_type
    if t == OptimizerType.ADAMW:
        return create_adamw(groups, config)
    if t == OptimizerType.ADAMW_4BIT:
        return create_adamw_lowbit(groups, config, bits=4)
    if t == OptimizerType.ADAMW_8BIT:
        return create_adamw_lowbit(groups, config, bits=8)
    if t == OptimizerType.SOAP:
        return create_soap(groups, config)
    if t == OptimizerType.SOAP_4BIT:
        return create_soap_lowbit(groups, config, bits=4, orig_param_shapes=orig_param_shapes)
    if t == OptimizerType.SOAP_8BIT:
        return create_soap_lowbit(groups, config, bits=8, orig_param_shapes=orig_param_shapes)
    if t == OptimizerType.SHAMPOO:
        return create_shampoo(groups, config, tensor_parallel_size)
    raise ValueError(f"Unknown optimizer type: {t}")


# --------------------------------------------------------------------------------------
# schedules
# --------------------------------------------------------------------------------------
def lr_multiplier(kind: str, step: int, total: int, warmup: int, min_ratio: float = 0.1) -> float:
    if step < warmup:
        return step / max(1, warmup)
    if kind == "constant_with_warmup":
        return 1.0
    progress = (step - warmup) / max(1, total - warmup)
    if kind == "cosine":
        return min_ratio + 0.5 * (1 - min_ratio) * (1 + math.cos(math.pi * progress))
    if kind == "linear":
        return max(min_ratio, 1 - progress * (1 - min_ratio))
    raise ValueError(f"Unknown scheduler type: {kind}")


def get_lr_scheduler(optimizer: Optimizer, scheduler_type: str, num_training_steps: int,
                     warmup_steps: int, min_lr_ratio: float = 0.1):
    if scheduler_type not in ("cosine", "linear", "constant_with_warmup"):
        raise ValueError(f"Unknown scheduler type: {scheduler_type}")
    return torch.optim.lr_scheduler.LambdaLR(
        optimizer, lambda s: lr_multiplier(scheduler_type, s, num_training_steps, warmup_steps, min_lr_ratio))


# --------------------------------------------------------------------------------------
# preconditioning coverage
# --------------------------------------------------------------------------------------
def analyze_preconditioning_coverage(model: nn.Module, max_precond_dim: int = 8192) -> Dict[str, Any]:
    """How much of the model a block-diagonal Kronecker preconditioner covers, and with how
    many blocks."""
    total = precond = 0
    layers = []
    for name, p in model.named_parameters():
        if not p.requires_grad:
            continue
        total += p.numel()
        if p.ndim != 2:
            continue
        r, c = p.shape
        nbr, nbc = -(-r // max_precond_dim), -(-c // max_precond_dim)
        precond += p.numel()
        layers.append(dict(name=name, shape=(r, c), blocks=nbr * nbc, rows=nbr, cols=nbc,
                           factor_elems=sum(min(max_precond_dim, r - i * max_precond_dim) ** 2 for i in range(nbr)) * nbc
                           + sum(min(max_precond_dim, c - j * max_precond_dim) ** 2 for j in range(nbc)) * nbr))
    return dict(total_params=total, preconditioned_params=precond,
                coverage=precond / max(1, total), num_2d=len(layers),
                num_blocks=sum(l["blocks"] for l in layers),
                multi_block=sorted((l for l in layers if l["blocks"] > 1), key=lambda l: -l["blocks"]),
                layers=layers)


def print_preconditioning_stats(model: nn.Module, max_precond_dim: int = 8192, top: int = 5) -> Dict[str, Any]:
    rep = analyze_preconditioning_coverage(model, max_precond_dim)
    print(f"Preconditioning coverage (max_precond_dim={max_precond_dim}):")
    print(f"  2-D parameters: {rep['num_2d']}  blocks: {rep['num_blocks']}")
    print(f"  preconditioned: {rep['preconditioned_params'] / 1e6:.1f}M of "
          f"{rep['total_params'] / 1e6:.1f}M params ({100 * rep['coverage']:.1f}%)")
    for l in rep["multi_block"][:top]:
        print(f"  multi-block: {l['name']} {l['shape']} -> {l['rows']}x{l['cols']} blocks")
    return rep
