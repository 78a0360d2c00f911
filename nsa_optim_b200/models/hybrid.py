"""Hybrid models: any string over {M, D, A} repeated ``block_repeats`` times.

M = Mamba-2 block, D = Gated DeltaNet block, A = attention block (dense or native sparse).
Reference behaviour (nngabe/nsa_optim): HybridConfig models/hybrid.py:95-136, rotary cache
:139-177, MambaBlock :200-238, DeltaNetBlock :241-289, AttentionBlock :292-394,
HybridModel :409-524 (scaled init :443-468), helpers :527-567.

State-dict names are kept: ``layers.{i}.norm``, ``layers.{i}.mixer.*``,
``layers.{i}.post_mixer_norm``, ``layers.{i}.mlp.*`` for M and D; for A the projections sit
on the block itself (``layers.{i}.{q,k,v,o}_proj``, ``post_attn_norm``).

Addition: the reference's A blocks are always dense; here ``attention_type`` reaches the
hybrid, so ``--block_pattern MDMA --attn_type nsa`` trains sparse A blocks
(extra parameters ``layers.{i}.gate_{cmp,slc,swa}.weight``).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Set

import torch
import torch.nn as nn
from torch import Tensor

from .. import ops
from ..config import AttentionType, resolve_attention_type
from .base import CausalLMBase, default_loss_fn, init_linear_embedding_
from .deltanet import GatedDeltaNetMixer
from .kernels import (Embedding, Linear, RotaryEmbedding, apply_rotary_pos_emb, create_mlp, create_rms_norm,
                      residual_block, resolve_kv_heads)
from .mamba import Mamba2Mixer


@dataclass
class HybridConfig:
    d_model: int = 1024
    vocab_size: int = 151936
    block_pattern: str = "MMDMMA"
    block_repeats: int = 5
    # Mamba-2
    mamba_d_state: int = 128
    mamba_d_conv: int = 4
    mamba_expand: int = 2
    mamba_headdim: int = 64
    mamba_chunk: int = 256
    # Gated DeltaNet
    deltanet_head_dim: int = 64
    deltanet_expand_v: int = 2
    deltanet_use_gate: bool = True
    deltanet_use_short_conv: bool = True
    deltanet_conv_size: int = 4
    deltanet_num_heads: Optional[int] = None      # default d_model // deltanet_head_dim
    # attention
    num_attention_heads: int = 16
    num_key_value_heads: int = 8
    head_dim: Optional[int] = None                # default d_model // num_attention_heads
    max_position_embeddings: int = 131072
    rope_theta: float = 100000.0
    attention_type: AttentionType = AttentionType.DENSE
    nsa_block_size: int = 64
    nsa_window_size: int = 512
    nsa_num_selected_blocks: int = 16
    nsa_compress_block: int = 32
    nsa_compress_stride: int = 16
    # common
    intermediate_size: Optional[int] = None
    norm_eps: float = 1e-6
    gradient_checkpointing: bool = False
    tie_word_embeddings: bool = False

    def __post_init__(self):
        if self.intermediate_size is None:
            self.intermediate_size = -(-int(self.d_model * 8 / 3) // 64) * 64
        if self.head_dim is None:
            self.head_dim = self.d_model // self.num_attention_heads
        self.attention_type = resolve_attention_type(self.attention_type)
        bad = set(self.block_pattern.upper()) - set("MDA")
        if bad:
            raise ValueError(f"Unknown block type(s) {sorted(bad)} in pattern {self.block_pattern!r}")
        self.block_pattern = self.block_pattern.upper()

    @property
    def n_layers(self) -> int:
        return len(self.block_pattern) * self.block_repeats


class HybridRotaryEmbedding(RotaryEmbedding):
    """(T, D/2) cos/sin cache; same object as :class:`RotaryEmbedding`, kept as a name."""


def apply_rotary_pos_emb_hybrid(q: Tensor, k: Tensor, cos: Tensor, sin: Tensor):
    return apply_rotary_pos_emb(q, k, cos, sin)


class MambaBlock(nn.Module):
    block_kind = "M"
    def __init__(self, config: HybridConfig, layer_idx: int):
        super().__init__()
        self.layer_idx = layer_idx
        self.norm = create_rms_norm(config.d_model, config.norm_eps)
        self.mixer = Mamba2Mixer(config.d_model, config.mamba_d_state, config.mamba_d_conv,
                                 config.mamba_expand, config.mamba_headdim,
                                 chunk_size=config.mamba_chunk, layer_idx=layer_idx)
        self.post_mixer_norm = create_rms_norm(config.d_model, config.norm_eps)
        self.mlp = create_mlp(config.d_model, config.intermediate_size)

    def forward(self, hidden_states: Tensor, attention_mask=None, position_ids=None) -> Tensor:
        return residual_block(hidden_states, self.norm, self.mixer, self.post_mixer_norm, self.mlp)


class DeltaNetBlock(nn.Module):
    block_kind = "D"
    def __init__(self, config: HybridConfig, layer_idx: int):
        super().__init__()
        self.layer_idx = layer_idx
        self.norm = create_rms_norm(config.d_model, config.norm_eps)
        heads = config.deltanet_num_heads or config.d_model // config.deltanet_head_dim
        self.mixer = GatedDeltaNetMixer(config.d_model, config.deltanet_head_dim, heads,
                                        config.deltanet_expand_v, config.deltanet_use_gate,
                                        config.deltanet_use_short_conv, config.deltanet_conv_size,
                                        layer_idx=layer_idx)
        self.post_mixer_norm = create_rms_norm(config.d_model, config.norm_eps)
        self.mlp = create_mlp(config.d_model, config.intermediate_size)

    def forward(self, hidden_states: Tensor, attention_mask=None, position_ids=None) -> Tensor:
        return residual_block(hidden_states, self.norm, self.mixer, self.post_mixer_norm, self.mlp)


class AttentionBlock(nn.Module):
    block_kind = "A"
    def __init__(self, config: HybridConfig, layer_idx: int):
        super().__init__()
        self.layer_idx = layer_idx
        self.num_heads = config.num_attention_heads
        self.num_kv_heads = resolve_kv_heads(self.num_heads, config.num_key_value_heads)
        self.head_dim = config.head_dim
        self.sparse = config.attention_type != AttentionType.DENSE
        d = config.d_model
        self.norm = create_rms_norm(d, config.norm_eps)
        self.q_proj = Linear(d, self.num_heads * self.head_dim)
        self.k_proj = Linear(d, self.num_kv_heads * self.head_dim)
        self.v_proj = Linear(d, self.num_kv_heads * self.head_dim)
        self.o_proj = Linear(self.num_heads * self.head_dim, d)
        if self.sparse:
            self.gate_cmp = Linear(d, self.num_heads)
            self.gate_slc = Linear(d, self.num_heads)
            self.gate_swa = Linear(d, self.num_heads)
            self.nsa = dict(cmp_block=config.nsa_compress_block, cmp_stride=config.nsa_compress_stride,
                            sel_block=config.nsa_block_size, top_n=config.nsa_num_selected_blocks,
                            window=config.nsa_window_size)
        self.rotary_emb = HybridRotaryEmbedding(self.head_dim, config.max_position_embeddings, config.rope_theta)
        self.post_attn_norm = create_rms_norm(d, config.norm_eps)
        self.mlp = create_mlp(d, config.intermediate_size)

    def forward(self, hidden_states: Tensor, attention_mask=None, position_ids=None) -> Tensor:
        return residual_block(hidden_states, self.norm, lambda x: self.attend(x, position_ids),
                              self.post_attn_norm, self.mlp)

    def attend(self, x: Tensor, position_ids=None) -> Tensor:
        """The attention mixer on the normed input: projections, RoPE, attention, output projection."""
        B, T, _ = x.shape
        ws = [self.q_proj.weight, self.k_proj.weight, self.v_proj.weight]
        if self.sparse:
            ws.append(torch.cat([self.gate_cmp.weight, self.gate_slc.weight, self.gate_swa.weight], 0))
        outs = ops.multi_linear(x, ws)           # one input, its gradient summed inside the GEMM epilogues
        q = outs[0].view(B, T, self.num_heads, self.head_dim)
        k = outs[1].view(B, T, self.num_kv_heads, self.head_dim)
        v = outs[2].view(B, T, self.num_kv_heads, self.head_dim)
        cos, sin = self.rotary_emb(x, position_ids, seq_len=T)
        q, k = apply_rotary_pos_emb(q, k, cos, sin)
        if self.sparse:
            o = ops.nsa_attention(q, k, v, None, None, None, gate_logits=outs[3], **self.nsa)
        else:
            o = ops.attention(q, k, v, causal=True)
        return self.o_proj(o.reshape(B, T, self.num_heads * self.head_dim))


_BLOCKS = {"M": MambaBlock, "D": DeltaNetBlock, "A": AttentionBlock}


def create_block(config: HybridConfig, block_type: str, layer_idx: int) -> nn.Module:
    try:
        return _BLOCKS[block_type](config, layer_idx)
    except KeyError:
        raise ValueError(f"Unknown block type: {block_type}") from None


class HybridModel(CausalLMBase):
    def __init__(self, config: HybridConfig):
        super().__init__()
        self.config = config
        self.embed_tokens = Embedding(config.vocab_size, config.d_model)
        kinds = config.block_pattern * config.block_repeats
        self.layers = nn.ModuleList([create_block(config, t, i) for i, t in enumerate(kinds)])
        self.norm = create_rms_norm(config.d_model, config.norm_eps)
        self.lm_head = None if config.tie_word_embeddings else Linear(config.d_model, config.vocab_size)
        self.gradient_checkpointing = config.gradient_checkpointing
        self.loss_fn = default_loss_fn()
        self._init_weights()

    def _init_weights(self):
        """N(0, 0.02) for projections and embeddings; residual-output projections (names
        containing ``o_proj`` or ``down_proj``) use 0.02/sqrt(2L); the head uses 0.02/sqrt(L)."""
        L = max(1, self.config.n_layers)
        for name, mod in self.named_modules():
            if isinstance(mod, (Linear, nn.Linear, nn.Embedding)):
                std = 0.02
                if "o_proj" in name or "down_proj" in name:
                    std = 0.02 / math.sqrt(2 * L)
                elif name == "lm_head":
                    std = 0.02 / math.sqrt(L)
                nn.init.normal_(mod.weight, mean=0.0, std=std)

    def forward(self, input_ids: Tensor, attention_mask: Optional[Tensor] = None,
                labels: Optional[Tensor] = None, position_ids: Optional[Tensor] = None, **_):
        T = input_ids.shape[1]
        if position_ids is None:
            position_ids = torch.arange(T, device=input_ids.device)
        h = self.embed_tokens(input_ids)
        for layer in self.layers:
            h = self.run_layer(layer, h, attention_mask, position_ids)
        h = self.norm(h)
        logits, loss = self.compute_loss(h, labels)
        return logits, loss, None


def create_hybrid_model(config: HybridConfig) -> HybridModel:
    return HybridModel(config)


def print_hybrid_model_modules(model: HybridModel, block_pattern: str, block_repeats: int) -> None:
    names = {"M": "Mamba2", "D": "GatedDeltaNet", "A": "Attention"}
    print(f"Hybrid model: pattern '{block_pattern}' x {block_repeats} = {len(model.layers)} layers")
    for i, layer in enumerate(model.layers):
        kind = block_pattern[i % len(block_pattern)]
        n = sum(p.numel() for p in layer.parameters())
        print(f"  [{i:3d}] {kind} {names[kind]:<14s} {type(layer).__name__:<15s} {n / 1e6:8.2f}M params")
    total = sum(p.numel() for p in model.parameters())
    print(f"  total {total / 1e9:.3f}B parameters")


def get_block_classes_from_pattern(pattern: str) -> Set[type]:
    """Block classes that appear in a pattern: the sharding units of the runtime."""
    return {_BLOCKS[c] for c in pattern.upper() if c in _BLOCKS}
