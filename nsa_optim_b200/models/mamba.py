"""Mamba-2 model family and the experimental complex-state "Mamba-3" block.

Reference behaviour (nngabe/nsa_optim): Mamba2Config/Block/Model models/mamba.py:32-201
(the mixer itself is the external ``mamba_ssm.Mamba2``), Mamba-3 experiment :204-618.

The mixer here is self-contained.  Parameter names and shapes follow the Mamba-2 layer
convention so its checkpoints interchange:
  in_proj.weight [2*d_in + 2*G*N + H, d]  (row order z, x, B, C, dt)
  conv1d.weight [d_in + 2*G*N, 1, W], conv1d.bias, dt_bias [H], A_log [H], D [H],
  norm.weight [d_in], out_proj.weight [d, d_in];  d_in = expand*d, H = d_in/headdim, G = 1.
Data flow: in_proj -> split -> causal depthwise conv (+bias, SiLU) over [x, B, C]
-> dt = softplus(dt + dt_bias), A = -exp(A_log) -> SSD chunked scan (chunk 256)
-> rmsnorm(y * silu(z)) * w -> out_proj.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

from .. import ops
from .base import CausalLMBase, default_loss_fn, init_linear_embedding_
from .kernels import Embedding, Linear, create_mlp, create_rms_norm, residual_block, split_last


def _inv_softplus_dt(n: int, dt_min: float = 1e-3, dt_max: float = 1e-1, floor: float = 1e-4) -> Tensor:
    """Bias b such that softplus(b) is log-uniform in [dt_min, dt_max]."""
    dt = torch.exp(torch.rand(n) * (math.log(dt_max) - math.log(dt_min)) + math.log(dt_min)).clamp_min(floor)
    return dt + torch.log(-torch.expm1(-dt))


class Mamba2Mixer(nn.Module):
    def __init__(self, d_model: int, d_state: int = 128, d_conv: int = 4, expand: int = 2,
                 headdim: int = 64, ngroups: int = 1, chunk_size: int = 256, layer_idx: int = 0):
        super().__init__()
        self.d_model, self.d_state, self.d_conv = d_model, d_state, d_conv
        self.expand, self.headdim, self.ngroups, self.chunk_size = expand, headdim, ngroups, chunk_size
        self.d_inner = expand * d_model
        assert self.d_inner % headdim == 0
        self.nheads = self.d_inner // headdim
        self.conv_dim = self.d_inner + 2 * ngroups * d_state
        self.in_proj = Linear(d_model, 2 * self.d_inner + 2 * ngroups * d_state + self.nheads)
        self.conv1d = nn.Conv1d(self.conv_dim, self.conv_dim, d_conv, groups=self.conv_dim,
                                padding=d_conv - 1, bias=True)
        self.dt_bias = nn.Parameter(_inv_softplus_dt(self.nheads))
        self.A_log = nn.Parameter(torch.log(torch.empty(self.nheads).uniform_(1, 16)))
        self.D = nn.Parameter(torch.ones(self.nheads))
        self.norm = nn.Module()
        self.norm.weight = nn.Parameter(torch.ones(self.d_inner))
        self.norm_eps = 1e-5
        self.out_proj = Linear(self.d_inner, d_model)
        for p in (self.dt_bias, self.A_log, self.D):
            p._no_weight_decay = True

    def forward(self, u: Tensor) -> Tensor:
        B, T, _ = u.shape
        zxbcdt = self.in_proj(u)
        d_in, gn, H = self.d_inner, self.ngroups * self.d_state, self.nheads
        z, xBC, dt = split_last(zxbcdt, [d_in, d_in + 2 * gn, H])
        xBC = ops.causal_conv1d(xBC, self.conv1d.weight.squeeze(1), self.conv1d.bias, activation=True)
        x, Bm, Cm = split_last(xBC, [d_in, gn, gn])
        dt = F.softplus(dt.float() + self.dt_bias.float())
        A = -torch.exp(self.A_log.float())
        y = ops.ssd_scan(x.reshape(B, T, H, self.headdim), dt, A,
                         Bm.reshape(B, T, self.ngroups, self.d_state),
                         Cm.reshape(B, T, self.ngroups, self.d_state), self.D, self.chunk_size)
        y = ops.gated_rms_norm(y.reshape(B, T, d_in), z, self.norm.weight, self.norm_eps,
                               norm_before_gate=False)
        return self.out_proj(y)


@dataclass
class Mamba2Config:
    d_model: int = 1024
    n_layers: int = 24
    d_state: int = 128
    d_conv: int = 4
    expand: int = 2
    headdim: int = 64
    vocab_size: int = 151936
    use_triton: bool = True          # accepted for compatibility; kernels are always native
    gradient_checkpointing: bool = False
    rms_norm: bool = True
    residual_in_fp32: bool = True
    fused_add_norm: bool = True
    chunk_size: int = 256
    norm_eps: float = 1e-6


def _mlp_width(d_model: int) -> int:
    return -(-int(d_model * 8 / 3) // 64) * 64


class Mamba2Block(nn.Module):
    """norm -> mixer -> +residual -> norm -> SwiGLU MLP -> +residual."""
    block_kind = "M"

    def __init__(self, config: Mamba2Config, layer_idx: int):
        super().__init__()
        self.layer_idx = layer_idx
        self.norm = create_rms_norm(config.d_model, config.norm_eps)
        self.mixer = Mamba2Mixer(config.d_model, config.d_state, config.d_conv, config.expand,
                                 config.headdim, chunk_size=config.chunk_size, layer_idx=layer_idx)
        self.post_mixer_norm = create_rms_norm(config.d_model, config.norm_eps)
        self.mlp = create_mlp(config.d_model, _mlp_width(config.d_model))

    def forward(self, hidden_states: Tensor, attention_mask=None, position_ids=None) -> Tensor:
        return residual_block(hidden_states, self.norm, self.mixer, self.post_mixer_norm, self.mlp)


class _SSMModel(CausalLMBase):
    """embed -> blocks -> norm -> untied head, shared by the Mamba-2, Mamba-3 and
    Gated DeltaNet pure models."""

    def _build(self, vocab_size: int, d_model: int, blocks, norm_eps: float, ckpt: bool):
        self.embed_tokens = Embedding(vocab_size, d_model)
        self.layers = nn.ModuleList(blocks)
        self.norm = create_rms_norm(d_model, norm_eps)
        self.lm_head = Linear(d_model, vocab_size)
        self.gradient_checkpointing = ckpt
        self.loss_fn = default_loss_fn()
        for name in ("embed_tokens", "lm_head"):
            init_linear_embedding_(getattr(self, name))
        for blk in self.layers:
            blk.apply(init_linear_embedding_)

    def forward(self, input_ids: Tensor, attention_mask: Optional[Tensor] = None,
                labels: Optional[Tensor] = None, **_):
        h = self.embed_tokens(input_ids)
        for layer in self.layers:
            h = self.run_layer(layer, h)
        h = self.norm(h)
        logits, loss = self.compute_loss(h, labels)
        return logits, loss, None


class Mamba2Model(_SSMModel):
    def __init__(self, config: Mamba2Config):
        super().__init__()
        self.config = config
        self._build(config.vocab_size, config.d_model,
                    [Mamba2Block(config, i) for i in range(config.n_layers)],
                    config.norm_eps, config.gradient_checkpointing)


def create_mamba2(config: Mamba2Config) -> Mamba2Model:
    return Mamba2Model(config)


# --------------------------------------------------------------------------------------
# Experimental complex-state block ("Mamba-3"), forward-only kernel in the reference.
# --------------------------------------------------------------------------------------
def mamba3_scan(x: Tensor, dt: Tensor, A: Tensor, Bc: Tensor, Cc: Tensor, D: Tensor) -> Tensor:
    """Sequential complex diagonal SSM with bilinear discretisation.
    x (B,L,H*P); dt (B,L,H); A (H,N,2); Bc, Cc (B,L,H,N,2); D (H).
        z = A dt / 2;  Abar = (1+z)/(1-z);  Bbar = B dt/(1-z)
        h <- Abar h + Bbar * sum_p x_p ;  y = x * (Re<C,h> + D)"""
    Bsz, L, DI = x.shape
    H = dt.shape[2]
    P = DI // H
    needs_grad = torch.is_grad_enabled() and any(t.requires_grad for t in (x, dt, A, Bc, Cc, D))
    if x.is_cuda and not needs_grad and ops.get_backend() != "torch" and A.shape[1] <= 256:
        # forward-only CUDA scan, like the reference's kernel; training goes through the loop below
        xs = x.view(Bsz, L, H, P)
        gate = ops.native_module().mamba3_gate(xs.float().sum(-1), dt, A, Bc, Cc, D)
        return (xs.float() * gate[..., None]).reshape(Bsz, L, DI).to(x.dtype)
    Ac = torch.view_as_complex(A.float().contiguous())
    Bz = torch.view_as_complex(Bc.float().contiguous())
    Cz = torch.view_as_complex(Cc.float().contiguous())
    xs = x.float().view(Bsz, L, H, P)
    h = torch.zeros(Bsz, H, Ac.shape[1], dtype=torch.complex64, device=x.device)
    ys = []
    for t in range(L):
        z = Ac[None] * dt[:, t].float()[..., None] * 0.5
        abar = (1 + z) / (1 - z)
        bbar = Bz[:, t] * (dt[:, t].float()[..., None] / (1 - z))
        h = abar * h + bbar * xs[:, t].sum(-1, keepdim=True)
        yr = (Cz[:, t] * h).real.sum(-1)                               # (B,H)
        ys.append(xs[:, t] * (yr + D.float()[None])[..., None])
    return torch.stack(ys, 1).reshape(Bsz, L, DI).to(x.dtype)


@dataclass
class Mamba3Config:
    d_model: int = 1024
    n_layers: int = 24
    d_state: int = 128
    expand: int = 2
    headdim: int = 64
    vocab_size: int = 151936
    use_conv: bool = False
    use_complex: bool = True
    dt_min: float = 0.001
    dt_max: float = 0.1
    gradient_checkpointing: bool = False
    rms_norm: bool = True
    residual_in_fp32: bool = True


class Mamba3Block(nn.Module):
    block_kind = "M"
    def __init__(self, d_model: int, d_state: int = 128, expand: int = 2, headdim: int = 64,
                 use_conv: bool = False, use_complex: bool = True, dt_min: float = 0.001,
                 dt_max: float = 0.1):
        super().__init__()
        self.d_inner = int(expand * d_model)
        self.d_state, self.headdim = d_state, headdim
        self.nheads = self.d_inner // headdim
        self.use_conv, self.use_complex = use_conv, use_complex
        pf = 2 if use_complex else 1
        self.in_proj = Linear(d_model, self.d_inner * 2)
        if use_conv:
            self.conv1d = nn.Conv1d(self.d_inner, self.d_inner, 4, groups=self.d_inner, padding=3, bias=True)
        self.x_proj = Linear(self.d_inner, self.nheads * (1 + 2 * d_state * pf))
        dt = torch.exp(torch.rand(self.nheads) * (math.log(dt_max) - math.log(dt_min)) + math.log(dt_min))
        self.dt_projs_bias = nn.Parameter(torch.log(dt))
        self.dt_projs_weight = nn.Parameter(torch.randn(self.nheads, self.d_inner))
        a_re = -torch.rand(self.nheads, d_state)
        a_im = torch.randn(self.nheads, d_state) * 0.1 if use_complex else torch.zeros(self.nheads, d_state)
        self.A = nn.Parameter(torch.stack([a_re, a_im], -1) if use_complex else a_re)
        self.D = nn.Parameter(torch.ones(self.nheads))
        self.norm_B = create_rms_norm(d_state * pf, 1e-6)
        self.norm_C = create_rms_norm(d_state * pf, 1e-6)
        self.out_proj = Linear(self.d_inner, d_model)

    def forward(self, u: Tensor, inference_params=None) -> Tensor:
        B, L, _ = u.shape
        x, z = self.in_proj(u).chunk(2, dim=-1)
        if self.use_conv:
            x = ops.causal_conv1d(x, self.conv1d.weight.squeeze(1), self.conv1d.bias, activation=False)
        x = F.silu(x)
        dt = F.softplus(F.linear(x.float(), self.dt_projs_weight.float(), self.dt_projs_bias.float()))
        pf = 2 if self.use_complex else 1
        bc = self.x_proj(x).view(B, L, self.nheads, -1)[..., : 2 * self.d_state * pf]
        bc = bc.reshape(B, L, self.nheads, 2, self.d_state * pf)
        Bn = self.norm_B(bc[..., 0, :]).view(B, L, self.nheads, self.d_state, pf)
        Cn = self.norm_C(bc[..., 1, :]).view(B, L, self.nheads, self.d_state, pf)
        A = self.A
        if not self.use_complex:
            zero = torch.zeros_like(Bn)
            Bn, Cn = torch.cat([Bn, zero], -1), torch.cat([Cn, zero], -1)
            A = torch.stack([A, torch.zeros_like(A)], -1)
        y = mamba3_scan(x, dt, A, Bn, Cn, self.D)
        return self.out_proj(y * F.silu(z))


class _Mamba3Layer(nn.Module):
    def __init__(self, config: Mamba3Config):
        super().__init__()
        self.norm = create_rms_norm(config.d_model, 1e-6)
        self.mixer = Mamba3Block(config.d_model, config.d_state, config.expand, config.headdim,
                                 config.use_conv, config.use_complex, config.dt_min, config.dt_max)
        self.post_mixer_norm = create_rms_norm(config.d_model, 1e-6)
        self.mlp = create_mlp(config.d_model, _mlp_width(config.d_model))

    def forward(self, x: Tensor, inference_params=None) -> Tensor:
        return residual_block(x, self.norm, self.mixer, self.post_mixer_norm, self.mlp)


class Mamba3Model(_SSMModel):
    def __init__(self, config: Mamba3Config):
        super().__init__()
        self.config = config
        self._build(config.vocab_size, config.d_model,
                    [_Mamba3Layer(config) for _ in range(config.n_layers)], 1e-6,
                    config.gradient_checkpointing)


def create_mamba3(config: Mamba3Config) -> Mamba3Model:
    return Mamba3Model(config)
