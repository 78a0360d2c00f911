"""Behaviour shared by the four model families.

All models are ``embed_tokens -> layers -> norm -> lm_head`` stacks whose forward returns
``(logits, loss, cache)`` (reference: models/hybrid.py:478-524, models/transformer.py:568-661).
This base class owns:

  * per-block activation checkpointing (non-reentrant, one checkpoint per block);
  * the hook through which the sharded-parameter runtime runs a block
    (``set_layer_runner``), so a block is one communication unit;
  * the loss dispatch: fused chunked linear+CE by default, materialised logits on request.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Tuple

import torch
import torch.nn as nn
from torch import Tensor
from torch.utils.checkpoint import checkpoint

from .kernels import FusedLinearCrossEntropy, compute_cross_entropy_loss


class CausalLMBase(nn.Module):
    gradient_checkpointing: bool = False
    _layer_runner: Optional[Callable] = None

    # ---- checkpointing switches (names used by the reference's trainer, train.py:160-163)
    def gradient_checkpointing_enable(self):
        self.gradient_checkpointing = True

    def gradient_checkpointing_disable(self):
        self.gradient_checkpointing = False

    # ---- sharded runtime integration
    def set_layer_runner(self, runner: Optional[Callable]) -> None:
        """``runner(layer, hidden, *args) -> hidden`` replaces the default block call."""
        object.__setattr__(self, "_layer_runner", runner)

    def block_modules(self) -> List[nn.Module]:
        return list(self.layers)

    def root_parameters(self) -> List[Tuple[str, nn.Parameter]]:
        """Parameters that do not belong to any block (embedding, final norm, head)."""
        block_ids = {id(p) for layer in self.layers for p in layer.parameters()}
        return [(n, p) for n, p in self.named_parameters() if id(p) not in block_ids]

    def run_layer(self, layer: nn.Module, hidden: Tensor, *args) -> Tensor:
        if self._layer_runner is not None:
            return self._layer_runner(layer, hidden, *args)
        if self.gradient_checkpointing and self.training and torch.is_grad_enabled():
            return checkpoint(layer, hidden, *args, use_reentrant=False)
        return layer(hidden, *args)

    # ---- loss
    def compute_loss(self, hidden: Tensor, labels: Optional[Tensor], want_logits: bool = False):
        head_w = self.output_weight()
        if labels is None:
            from .. import ops
            return ops.linear(hidden, head_w), None
        if want_logits or getattr(self, "loss_fn", None) is None:
            return compute_cross_entropy_loss(hidden, _WeightHolder(head_w), labels, None)
        return compute_cross_entropy_loss(hidden, _WeightHolder(head_w), labels, self.loss_fn)

    def output_weight(self) -> Tensor:
        head = getattr(self, "lm_head", None)
        return self.embed_tokens.weight if head is None else head.weight

    def num_parameters(self) -> int:
        return sum(p.numel() for p in self.parameters())


class _WeightHolder:
    __slots__ = ("weight",)

    def __init__(self, w: Tensor):
        self.weight = w


def default_loss_fn() -> FusedLinearCrossEntropy:
    return FusedLinearCrossEntropy()


def init_linear_embedding_(module: nn.Module, std: float = 0.02) -> None:
    """N(0, std) for every projection and embedding weight; biases to zero."""
    from .kernels import Linear
    if isinstance(module, (nn.Linear, Linear)):
        nn.init.normal_(module.weight, mean=0.0, std=std)
        if getattr(module, "bias", None) is not None:
            nn.init.zeros_(module.bias)
    elif isinstance(module, nn.Embedding):
        nn.init.normal_(module.weight, mean=0.0, std=std)
