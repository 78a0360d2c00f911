"""Gated DeltaNet model family.

Reference behaviour (nngabe/nsa_optim): GatedDeltaNetConfig/Block/Model
models/deltanet.py:67-267; the mixer there is the external ``fla.layers.GatedDeltaNet``
(mode 'chunk', gate on, short convolutions of width 4, expand_v 2).

The mixer here is self-contained and keeps that layer's parameter names and shapes:
  {q,k}_proj.weight [H*K, d], v_proj.weight [H*V, d] (V = expand_v*K),
  {a,b}_proj.weight [H, d], A_log [H], dt_bias [H], {q,k,v}_conv1d.weight [C,1,4] (no bias),
  g_proj.weight [H*V, d], o_norm.weight [V], o_proj.weight [d, H*V].
Data flow: projections -> causal depthwise conv + SiLU on q,k,v -> L2-normalise q,k ->
beta = sigmoid(b), g = -exp(A_log) * softplus(a + dt_bias) -> chunkwise gated delta rule
(chunk 64) -> rmsnorm(o) * w * silu(gate) -> o_proj.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

from .. import ops
from .kernels import Linear, create_mlp, create_rms_norm, residual_block
from .mamba import _SSMModel, _inv_softplus_dt, _mlp_width


class GatedDeltaNetMixer(nn.Module):
    def __init__(self, hidden_size: int, head_dim: int = 64, num_heads: Optional[int] = None,
                 expand_v: float = 2.0, use_gate: bool = True, use_short_conv: bool = True,
                 conv_size: int = 4, norm_eps: float = 1e-5, chunk_size: int = 64, layer_idx: int = 0):
        super().__init__()
        self.hidden_size = hidden_size
        self.head_k_dim = head_dim
        self.num_heads = num_heads if num_heads is not None else hidden_size // head_dim
        self.head_v_dim = int(head_dim * expand_v)
        self.key_dim = self.num_heads * self.head_k_dim
        self.value_dim = self.num_heads * self.head_v_dim
        self.use_gate, self.use_short_conv, self.conv_size = use_gate, use_short_conv, conv_size
        self.chunk_size, self.norm_eps = chunk_size, norm_eps
        self.q_proj = Linear(hidden_size, self.key_dim)
        self.k_proj = Linear(hidden_size, self.key_dim)
        self.v_proj = Linear(hidden_size, self.value_dim)
        self.a_proj = Linear(hidden_size, self.num_heads)
        self.b_proj = Linear(hidden_size, self.num_heads)
        self.A_log = nn.Parameter(torch.log(torch.empty(self.num_heads).uniform_(1e-3, 16)))
        self.dt_bias = nn.Parameter(_inv_softplus_dt(self.num_heads))
        self.A_log._no_weight_decay = True
        self.dt_bias._no_weight_decay = True
        if use_short_conv:
            self.q_conv1d = nn.Conv1d(self.key_dim, self.key_dim, conv_size, groups=self.key_dim,
                                      padding=conv_size - 1, bias=False)
            self.k_conv1d = nn.Conv1d(self.key_dim, self.key_dim, conv_size, groups=self.key_dim,
                                      padding=conv_size - 1, bias=False)
            self.v_conv1d = nn.Conv1d(self.value_dim, self.value_dim, conv_size, groups=self.value_dim,
                                      padding=conv_size - 1, bias=False)
        if use_gate:
            self.g_proj = Linear(hidden_size, self.value_dim)
        self.o_norm = create_rms_norm(self.head_v_dim, norm_eps)
        self.o_proj = Linear(self.value_dim, hidden_size)

    def forward(self, x: Tensor) -> Tensor:
        B, T, _ = x.shape
        H, K, V = self.num_heads, self.head_k_dim, self.head_v_dim
        ws = [self.q_proj.weight, self.k_proj.weight, self.v_proj.weight, self.b_proj.weight, self.a_proj.weight]
        if self.use_gate:
            ws.append(self.g_proj.weight)
        outs = ops.multi_linear(x, ws)           # one input, its gradient summed inside the GEMM epilogues
        q, k, v = outs[0], outs[1], outs[2]
        if self.use_short_conv:
            q = ops.causal_conv1d(q, self.q_conv1d.weight.squeeze(1), None, activation=True)
            k = ops.causal_conv1d(k, self.k_conv1d.weight.squeeze(1), None, activation=True)
            v = ops.causal_conv1d(v, self.v_conv1d.weight.squeeze(1), None, activation=True)
        else:
            q, k, v = F.silu(q), F.silu(k), F.silu(v)
        q = ops.l2_norm(q.view(B, T, H, K))
        k = ops.l2_norm(k.view(B, T, H, K))
        v = v.view(B, T, H, V)
        beta = torch.sigmoid(outs[3].float())
        g = -torch.exp(self.A_log.float()) * F.softplus(outs[4].float() + self.dt_bias.float())
        o = ops.gated_delta_rule(q, k, v, g, beta, scale=K ** -0.5, chunk=self.chunk_size)
        if self.use_gate:
            gate = outs[5].view(B, T, H, V)
            o = ops.gated_rms_norm(o, gate, self.o_norm.weight, self.norm_eps, norm_before_gate=True)
        else:
            o = self.o_norm(o)
        return self.o_proj(o.reshape(B, T, H * V))


@dataclass
class GatedDeltaNetConfig:
    d_model: int = 1024
    n_layers: int = 24
    d_state: int = 128
    head_dim: int = 64
    expand_v: float = 2.0
    vocab_size: int = 151936
    use_gate: bool = True
    use_short_conv: bool = True
    conv_size: int = 4
    norm_eps: float = 1e-6
    gradient_checkpointing: bool = False
    num_heads: Optional[int] = None


class GatedDeltaNetBlock(nn.Module):
    block_kind = "D"
    def __init__(self, config: GatedDeltaNetConfig, layer_idx: int):
        super().__init__()
        self.layer_idx = layer_idx
        self.input_layernorm = create_rms_norm(config.d_model, config.norm_eps)
        self.mixer = GatedDeltaNetMixer(config.d_model, config.head_dim, config.num_heads,
                                        config.expand_v, config.use_gate, config.use_short_conv,
                                        config.conv_size, layer_idx=layer_idx)
        self.post_attention_layernorm = create_rms_norm(config.d_model, config.norm_eps)
        self.mlp = create_mlp(config.d_model, _mlp_width(config.d_model))

    def forward(self, hidden_states: Tensor, attention_mask=None, position_ids=None) -> Tensor:
        return residual_block(hidden_states, self.input_layernorm, self.mixer, self.post_attention_layernorm, self.mlp)


class GatedDeltaNetModel(_SSMModel):
    def __init__(self, config: GatedDeltaNetConfig):
        super().__init__()
        self.config = config
        self._build(config.vocab_size, config.d_model,
                    [GatedDeltaNetBlock(config, i) for i in range(config.n_layers)],
                    config.norm_eps, config.gradient_checkpointing)


def create_gated_deltanet(config: GatedDeltaNetConfig) -> GatedDeltaNetModel:
    return GatedDeltaNetModel(config)
