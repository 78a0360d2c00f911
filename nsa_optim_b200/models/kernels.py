"""Shared building blocks: norm, rotary tables, SwiGLU MLP, loss helper, kernel factories.

Public surface mirrors the reference's ``models/kernels.py`` (RMSNorm :47-59,
RotaryEmbedding :62-96, rotate_half / apply_rotary_pos_emb :99-113, MLP :116-128,
factories and loss helper :304-423).  The reference chooses between PyTorch, Triton and
Liger kernels with ``kernel_type``; here the same strings are accepted and mean:

  ``baseline`` -> the PyTorch implementation (``ops.torch_impl``), on any device;
  ``triton`` / ``liger`` -> the framework's own kernels (sm_100a CUDA on a GPU,
  the PyTorch implementation on CPU).

Parameter names are the canonical ``mlp.{gate,up,down}_proj.weight``; checkpoints written
with the Liger wrapper's extra ``.mlp.`` level are remapped on load.
"""
from __future__ import annotations

import contextlib
from typing import Callable, Literal, Optional, Tuple

import torch
import torch.nn as nn
from torch import Tensor

from .. import ops

KernelType = Literal["baseline", "triton", "liger"]

# Import-compat flags: the reference exports these to say whether optional kernel
# libraries were importable.  Neither library is used here.
LIGER_AVAILABLE = False
TRITON_AVAILABLE = False


def _ctx(kernel_type: str):
    return ops.backend("torch") if kernel_type == "baseline" else contextlib.nullcontext()


class Linear(nn.Module):
    """Bias-free linear layer whose matmul goes through ``ops.linear`` (tcgen05 GEMM on GPU)."""

    def __init__(self, in_features: int, out_features: int, bias: bool = False):
        super().__init__()
        if bias:
            raise ValueError("bias-free projections only")
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features))
        nn.init.normal_(self.weight, mean=0.0, std=0.02)

    def forward(self, x: Tensor) -> Tensor:
        return ops.linear(x, self.weight)

    def extra_repr(self) -> str:
        return f"in_features={self.in_features}, out_features={self.out_features}, bias=False"


class Embedding(nn.Embedding):
    """Token embedding whose gather (and deterministic scatter-add backward) goes through
    ``ops.embedding``."""

    def forward(self, input_ids: Tensor) -> Tensor:
        return ops.embedding(input_ids, self.weight)


class RMSNorm(nn.Module):
    def __init__(self, hidden_size: int, eps: float = 1e-6, kernel_type: KernelType = "liger"):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden_size))
        self.variance_epsilon = eps
        self.kernel_type = kernel_type

    def forward(self, x: Tensor) -> Tensor:
        with _ctx(self.kernel_type):
            return ops.rms_norm(x, self.weight, self.variance_epsilon)

    def forward_skip(self, x: Tensor) -> Tuple[Tensor, Tensor]:
        """(norm(x), x): take the residual branch from the second value."""
        with _ctx(self.kernel_type):
            return ops.rms_norm_skip(x, self.weight, self.variance_epsilon)

    def forward_add(self, x: Tensor, r: Tensor) -> Tuple[Tensor, Tensor]:
        """(x + r, norm(x + r)) in one pass."""
        with _ctx(self.kernel_type):
            return ops.add_rms_norm(x, r, self.weight, self.variance_epsilon)


def residual_block(hidden: Tensor, norm1: nn.Module, mixer, norm2: nn.Module, mlp) -> Tensor:
    """``h = hidden + mixer(norm1(hidden)); return h + mlp(norm2(h))`` with the residual adds
    folded into the norm kernels where the norms support it (reference block structure:
    models/hybrid.py:221-236)."""
    if hasattr(norm1, "forward_skip") and hasattr(norm2, "forward_add"):
        x1, skip = norm1.forward_skip(hidden)
        h, x2 = norm2.forward_add(skip, mixer(x1))
        return h + mlp(x2)
    h = hidden + mixer(norm1(hidden))
    return h + mlp(norm2(h))


class RotaryEmbedding(nn.Module):
    """cos/sin cache of shape (T, D/2) in fp32; grows on demand.  ``forward`` returns the
    rows for ``position_ids`` (or the first ``seq_len`` rows)."""

    def __init__(self, dim: int, max_position_embeddings: int = 2048, base: float = 10000.0):
        super().__init__()
        self.dim, self.base = dim, base
        self.max_seq_len_cached = 0
        self.register_buffer("inv_freq", torch.empty(0), persistent=False)
        self.register_buffer("cos_cached", torch.empty(0), persistent=False)
        self.register_buffer("sin_cached", torch.empty(0), persistent=False)
        self._initial = max_position_embeddings

    def _set_cos_sin_cache(self, seq_len: int, device=None):
        cos, sin = ops.oracle.rope_tables(self.dim, seq_len, self.base, device=device)
        self.cos_cached, self.sin_cached = cos, sin
        self.max_seq_len_cached = seq_len

    def forward(self, x: Tensor, position_ids: Optional[Tensor] = None, seq_len: Optional[int] = None
                ) -> Tuple[Tensor, Tensor]:
        need = int(position_ids.max()) + 1 if position_ids is not None else (seq_len or x.shape[1])
        if need > self.max_seq_len_cached or self.cos_cached.device != x.device:
            self._set_cos_sin_cache(max(need, self._initial if self.max_seq_len_cached == 0 else need),
                                    device=x.device)
        if position_ids is None:
            return self.cos_cached[:need], self.sin_cached[:need]
        pid = position_ids.reshape(-1)[: x.shape[1]] if position_ids.dim() > 1 else position_ids
        return self.cos_cached[pid], self.sin_cached[pid]


def rotate_half(x: Tensor) -> Tensor:
    x1, x2 = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2:]
    return torch.cat((-x2, x1), dim=-1)


def apply_rotary_pos_emb(q: Tensor, k: Tensor, cos: Tensor, sin: Tensor) -> Tuple[Tensor, Tensor]:
    """q, k (B, T, H, D); cos/sin (T, D/2) (or (T, D) with duplicated halves)."""
    d2 = q.shape[-1] // 2
    if cos.shape[-1] == q.shape[-1]:
        cos, sin = cos[..., :d2], sin[..., :d2]
    return ops.rope(q, cos, sin), ops.rope(k, cos, sin)


class MLP(nn.Module):
    """SwiGLU feed-forward: down(silu(gate(x)) * up(x))."""

    def __init__(self, hidden_size: int, intermediate_size: int, kernel_type: KernelType = "liger"):
        super().__init__()
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.gate_proj = Linear(hidden_size, intermediate_size)
        self.up_proj = Linear(hidden_size, intermediate_size)
        self.down_proj = Linear(intermediate_size, hidden_size)
        self.kernel_type = kernel_type

    def forward(self, x: Tensor) -> Tensor:
        with _ctx(self.kernel_type):
            g, u = ops.multi_linear(x, (self.gate_proj.weight, self.up_proj.weight))
            return self.down_proj(ops.swiglu(g, u))


def create_rms_norm(hidden_size: int, eps: float = 1e-6, kernel_type: KernelType = "liger") -> nn.Module:
    return RMSNorm(hidden_size, eps, kernel_type)


def create_mlp(hidden_size: int, intermediate_size: int, kernel_type: KernelType = "liger") -> nn.Module:
    return MLP(hidden_size, intermediate_size, kernel_type)


def get_rotary_pos_emb_fn(kernel_type: KernelType = "liger") -> Callable:
    if kernel_type == "baseline":
        def fn(q, k, cos, sin):
            with ops.backend("torch"):
                return apply_rotary_pos_emb(q, k, cos, sin)
        return fn
    return apply_rotary_pos_emb


class FusedLinearCrossEntropy(nn.Module):
    """Chunked linear + cross-entropy that never materialises (tokens, vocab) logits."""

    def __init__(self, ignore_index: int = -100, chunk: int = 4096):
        super().__init__()
        self.ignore_index, self.chunk = ignore_index, chunk

    def forward(self, lin_weight: Tensor, hidden: Tensor, target: Tensor) -> Tensor:
        return ops.linear_cross_entropy(hidden, lin_weight, target, self.ignore_index, self.chunk)


def create_cross_entropy_loss(lm_head: Optional[nn.Module] = None, kernel_type: KernelType = "liger"):
    """``None`` selects the materialised-logits path in :func:`compute_cross_entropy_loss`."""
    return None if kernel_type == "baseline" else FusedLinearCrossEntropy()


def compute_cross_entropy_loss(hidden_states: Tensor, lm_head: nn.Module, labels: Tensor,
                               loss_fn=None) -> Tuple[Optional[Tensor], Tensor]:
    """Next-token loss.  Returns ``(logits or None, loss)``; with a fused ``loss_fn`` logits
    are not formed."""
    h = hidden_states[:, :-1, :].reshape(-1, hidden_states.shape[-1])
    y = labels[:, 1:].reshape(-1)
    if loss_fn is not None:
        return None, loss_fn(lm_head.weight, h, y)
    logits = ops.linear(hidden_states, lm_head.weight)
    loss = torch.nn.functional.cross_entropy(
        logits[:, :-1, :].reshape(-1, logits.shape[-1]).float(), y, ignore_index=-100)
    return logits, loss


def remap_legacy_keys(state_dict: dict) -> dict:
    """Accept checkpoints whose MLP weights carry the Liger wrapper's ``mlp.mlp.`` prefix."""
    return {k.replace(".mlp.mlp.", ".mlp."): v for k, v in state_dict.items()}


class _SplitLast(torch.autograd.Function):
    """``torch.split`` along the last dimension whose backward writes the incoming gradients into
    one preallocated tensor with plain strided copies.  (The stock backward is a concatenation
    kernel that runs at a small fraction of memory bandwidth for wide, uneven column groups:
    2.4 ms for a 65536 x 8512 bf16 tensor against 0.5 ms for the copies.)"""

    @staticmethod
    def forward(ctx, x, *sizes):
        ctx.sizes = sizes
        ctx.shape, ctx.dtype = x.shape, x.dtype
        return torch.split(x, list(sizes), dim=-1)

    @staticmethod
    def backward(ctx, *grads):
        ref = next(g for g in grads if g is not None)
        out = torch.empty(ctx.shape, dtype=ctx.dtype, device=ref.device)
        o = 0
        for g, n in zip(grads, ctx.sizes):
            if g is None:
                out[..., o:o + n].zero_()
            else:
                dst = out[..., o:o + n]
                done = False
                if dst.is_cuda and ops.get_backend() != "torch":
                    done = ops.native_module().copy_columns(dst, g)
                if not done:
                    dst.copy_(g)
            o += n
        return (out,) + (None,) * len(ctx.sizes)


def split_last(x: Tensor, sizes) -> tuple:
    """Column split of ``x`` (last dimension) into views of the given widths."""
    if not (x.requires_grad and torch.is_grad_enabled()):
        return torch.split(x, list(sizes), dim=-1)
    return _SplitLast.apply(x, *sizes)


def resolve_kv_heads(num_heads: int, num_kv_heads: int) -> int:
    """KV head count usable for grouped-query attention: the largest divisor of ``num_heads`` not
    above ``num_kv_heads``.  The size table gives the smallest models more KV heads than query
    heads (100M: 4 query / 8 KV heads, config.py:145), which no attention path can run; those
    shapes get one KV head per query head."""
    kv = max(1, min(num_kv_heads, num_heads))
    while num_heads % kv:
        kv -= 1
    return kv
