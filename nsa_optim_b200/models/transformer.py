"""Pure transformer family: dense GQA attention, native sparse attention (NSA), and the
``flash_sparse_attention`` choice, which runs on the same sparse kernels.

Reference behaviour (nngabe/nsa_optim): DenseAttention models/transformer.py:50-124,
NativeSparseAttention :127-311, FlashSparseAttention :314-426, TransformerBlock :433-478,
TransformerModel :481-661, create_model :664-666.  State-dict names are kept:
``layers.{i}.{input_layernorm,post_attention_layernorm}.weight``,
``layers.{i}.self_attn.{q,k,v,o}_proj.weight``, and for NSA
``self_attn.{k_compress,gate_slc,gate_swa}.weight`` (+ ``gate_cmp`` for the compressed
branch, which the reference does not have).

Differences by design: the reference's NSA scores blocks through a dense (T x T/block)
tensor and calls an external kernel without a compressed branch; here the three-branch
algorithm (compressed attention -> streaming top-n block selection -> selected-block
attention, plus sliding window, combined by per-head sigmoid gates) runs end to end.
"""
from __future__ import annotations

import math

from typing import Optional, Tuple

import torch
import torch.nn as nn
from torch import Tensor

from .. import ops
from ..config import AttentionType, ModelConfig
from .base import CausalLMBase, default_loss_fn, init_linear_embedding_
from .kernels import (Embedding, KernelType, Linear, RotaryEmbedding, apply_rotary_pos_emb, resolve_kv_heads,
                      create_mlp, create_rms_norm, residual_block)

FSA_AVAILABLE = True  # the sparse kernels are built in; kept for import compatibility


class _FrozenWeight(nn.Module):
    """A persistent, non-trainable ``weight`` buffer (keeps a state-dict key alive)."""

    def __init__(self, rows: int, cols: int):
        super().__init__()
        self.register_buffer("weight", torch.zeros(rows, cols))


class DenseAttention(nn.Module):
    """Causal grouped-query attention with rotary embeddings and an optional KV cache."""

    def __init__(self, config: ModelConfig, layer_idx: int, kernel_type: KernelType = "liger"):
        super().__init__()
        self.layer_idx = layer_idx
        self.hidden_size = config.hidden_size
        self.num_heads = config.num_attention_heads
        self.num_kv_heads = resolve_kv_heads(config.num_attention_heads, config.num_key_value_heads)
        self.head_dim = config.head_dim
        self.num_kv_groups = self.num_heads // self.num_kv_heads
        self.q_proj = Linear(self.hidden_size, self.num_heads * self.head_dim)
        self.k_proj = Linear(self.hidden_size, self.num_kv_heads * self.head_dim)
        self.v_proj = Linear(self.hidden_size, self.num_kv_heads * self.head_dim)
        self.o_proj = Linear(self.num_heads * self.head_dim, self.hidden_size)
        self.rotary_emb = RotaryEmbedding(self.head_dim, config.max_position_embeddings, config.rope_theta)

    def _qkv(self, x: Tensor, position_ids: Optional[Tensor]):
        B, T, _ = x.shape
        q, k, v = ops.multi_linear(x, (self.q_proj.weight, self.k_proj.weight, self.v_proj.weight))
        q = q.view(B, T, self.num_heads, self.head_dim)
        k = k.view(B, T, self.num_kv_heads, self.head_dim)
        v = v.view(B, T, self.num_kv_heads, self.head_dim)
        cos, sin = self.rotary_emb(x, position_ids, seq_len=T)
        q, k = apply_rotary_pos_emb(q, k, cos, sin)
        return q, k, v

    def forward(self, hidden_states: Tensor, attention_mask: Optional[Tensor] = None,
                position_ids: Optional[Tensor] = None,
                past_key_value: Optional[Tuple[Tensor, Tensor]] = None, use_cache: bool = False):
        B, T, _ = hidden_states.shape
        q, k, v = self._qkv(hidden_states, position_ids)
        if past_key_value is not None:
            k = torch.cat([past_key_value[0], k], dim=1)
            v = torch.cat([past_key_value[1], v], dim=1)
        cache = (k, v) if use_cache else None
        o = ops.attention(q, k, v, causal=True)
        return self.o_proj(o.reshape(B, T, self.num_heads * self.head_dim)), cache


class NativeSparseAttention(DenseAttention):
    """Three-branch sparse attention.  ``nsa_block_size`` is the selection block,
    ``nsa_num_selected_blocks`` the top-n, ``nsa_window_size`` the sliding window,
    ``nsa_compress_block`` / ``nsa_compress_stride`` the compressed-branch pooling."""

    def __init__(self, config: ModelConfig, layer_idx: int, kernel_type: KernelType = "liger"):
        super().__init__(config, layer_idx, kernel_type)
        self.block_size = config.nsa_block_size
        self.window_size = config.nsa_window_size
        self.num_selected_blocks = config.nsa_num_selected_blocks
        self.compress_block = config.nsa_compress_block
        self.compress_stride = config.nsa_compress_stride
        # The reference module's block scorer (models/transformer.py:172-214): a head_dim -> head_dim/4
        # projection applied to queries and to block-mean keys.  Its output only feeds a top-k, so it
        # receives no gradient there either: a persistent buffer, loaded from reference checkpoints.
        # With ``nsa_block_scorer="learned"`` it chooses the blocks (two branches, as the reference
        # module); by default the compressed branch's probabilities choose them (three branches).
        self.k_compress = _FrozenWeight(max(1, self.head_dim // 4), self.head_dim)
        self.block_scorer = getattr(config, "nsa_block_scorer", "compressed")
        if self.block_scorer == "learned":
            nn.init.normal_(self.k_compress.weight, std=self.head_dim ** -0.5)
        self.gate_cmp = Linear(self.hidden_size, self.num_heads)
        self.gate_slc = Linear(self.hidden_size, self.num_heads)
        self.gate_swa = Linear(self.hidden_size, self.num_heads)

    def gates(self, x: Tensor) -> Tuple[Tensor, Tensor, Tensor]:
        w = torch.cat([self.gate_cmp.weight, self.gate_slc.weight, self.gate_swa.weight], 0)
        g = torch.sigmoid(ops.linear(x, w).float()).to(x.dtype)
        return g.split(self.num_heads, dim=-1)

    @torch.no_grad()
    def learned_block_indices(self, q: Tensor, k: Tensor) -> Tensor:
        """(B, Hkv, T, n) int32 block lists from the learned scorer: score(t, block) = sum over the
        GQA group's heads of k_compress(q_t) . mean over the block of k_compress(k), divided by
        sqrt(head_dim / 4); blocks after the query's own are masked; top-n, ascending, -1 where a
        query sees fewer blocks.  (The reference scores per query head after repeating K; its kernel
        shares one list per KV head, so the group's scores are summed here.)"""
        B, T, Hq, D = q.shape
        Hkv, G, bs = self.num_kv_heads, self.num_kv_groups, self.block_size
        w = self.k_compress.weight.to(q.dtype)
        qc = torch.matmul(q, w.t()).view(B, T, Hkv, G, -1).sum(3).float()                 # B,T,Hkv,d4
        kc = torch.matmul(k, w.t()).float()
        nS = -(-T // bs)
        pad = nS * bs - T
        if pad:
            kc = torch.nn.functional.pad(kc, (0, 0, 0, 0, 0, pad))
        kbm = kc.view(B, nS, bs, Hkv, -1).mean(2)                                         # B,nS,Hkv,d4
        n = min(self.num_selected_blocks, nS)
        own = torch.arange(T, device=q.device) // bs
        out = torch.empty(B, Hkv, T, self.num_selected_blocks, dtype=torch.int32, device=q.device)
        for s0 in range(0, T, 8192):                                                      # bound the score matrix
            s1 = min(T, s0 + 8192)
            sc = torch.einsum("bthd,bnhd->bhtn", qc[:, s0:s1], kbm) / math.sqrt(kbm.shape[-1])
            vis = torch.arange(nS, device=q.device)[None, :] <= own[s0:s1, None]
            sc = sc.masked_fill(~vis, float("-inf"))
            top, ind = torch.topk(sc, n, dim=-1)
            ind = ind.masked_fill(top == float("-inf"), nS + 1).sort(-1).values
            ind = ind.masked_fill(ind > nS, -1)
            out[:, :, s0:s1, :n] = ind.to(torch.int32)
            out[:, :, s0:s1, n:] = -1
        return out

    def forward(self, hidden_states, attention_mask=None, position_ids=None,
                past_key_value=None, use_cache: bool = False):
        B, T, _ = hidden_states.shape
        q, k, v = self._qkv(hidden_states, position_ids)
        if past_key_value is not None:
            # incremental decoding attends densely over the cache
            k = torch.cat([past_key_value[0], k], dim=1)
            v = torch.cat([past_key_value[1], v], dim=1)
            o = ops.attention(q, k, v, causal=True)
        elif self.block_scorer == "learned":
            _, g_slc, g_swa = self.gates(hidden_states)
            idx = self.learned_block_indices(q, k)
            o = ops.nsa_attention_indexed(q, k, v, idx, g_slc, g_swa, sel_block=self.block_size,
                                          window=self.window_size)
        else:
            g_cmp, g_slc, g_swa = self.gates(hidden_states)
            o = ops.nsa_attention(q, k, v, g_cmp, g_slc, g_swa,
                                  cmp_block=self.compress_block, cmp_stride=self.compress_stride,
                                  sel_block=self.block_size, top_n=self.num_selected_blocks,
                                  window=self.window_size)
        cache = (k, v) if use_cache else None
        return self.o_proj(o.reshape(B, T, self.num_heads * self.head_dim)), cache


class FlashSparseAttention(NativeSparseAttention):
    """The ``flash_sparse_attention`` / ``fsa`` choice.  The reference wraps an external
    package that implements the same selected-block algorithm with a different kernel
    schedule; here it shares the NSA kernels."""


_ATTENTION = {
    AttentionType.DENSE: DenseAttention,
    AttentionType.NSA: NativeSparseAttention,
    AttentionType.FSA: FlashSparseAttention,
}


class TransformerBlock(nn.Module):
    block_kind = "A"
    def __init__(self, config: ModelConfig, layer_idx: int, kernel_type: KernelType = "liger"):
        super().__init__()
        self.layer_idx = layer_idx
        self.self_attn = _ATTENTION[config.attention_type](config, layer_idx, kernel_type)
        self.mlp = create_mlp(config.hidden_size, config.intermediate_size, kernel_type)
        self.input_layernorm = create_rms_norm(config.hidden_size, config.rms_norm_eps, kernel_type)
        self.post_attention_layernorm = create_rms_norm(config.hidden_size, config.rms_norm_eps, kernel_type)

    def forward(self, hidden_states: Tensor, attention_mask: Optional[Tensor] = None,
                position_ids: Optional[Tensor] = None, past_key_value=None, use_cache: bool = False):
        cache = [None]

        def attend(x: Tensor) -> Tensor:
            a, cache[0] = self.self_attn(x, attention_mask, position_ids, past_key_value, use_cache)
            return a

        h = residual_block(hidden_states, self.input_layernorm, attend, self.post_attention_layernorm, self.mlp)
        return (h, cache[0]) if use_cache else h


class TransformerModel(CausalLMBase):
    def __init__(self, config: ModelConfig, kernel_type: KernelType = "liger"):
        super().__init__()
        self.config = config
        self.kernel_type = kernel_type
        self.embed_tokens = Embedding(config.vocab_size, config.hidden_size)
        self.layers = nn.ModuleList(
            [TransformerBlock(config, i, kernel_type) for i in range(config.num_hidden_layers)])
        self.norm = create_rms_norm(config.hidden_size, config.rms_norm_eps, kernel_type)
        self.lm_head = None if config.tie_word_embeddings else Linear(config.hidden_size, config.vocab_size)
        self.gradient_checkpointing = bool(getattr(config, "gradient_checkpointing", False))
        self.loss_fn = None if kernel_type == "baseline" else default_loss_fn()
        self.apply(init_linear_embedding_)

    def forward(self, input_ids: Tensor, attention_mask: Optional[Tensor] = None,
                position_ids: Optional[Tensor] = None, past_key_values=None,
                labels: Optional[Tensor] = None, use_cache: bool = False):
        B, T = input_ids.shape
        past_len = 0 if past_key_values is None else past_key_values[0][0].shape[1]
        if position_ids is None:
            position_ids = torch.arange(past_len, past_len + T, device=input_ids.device)
        h = self.embed_tokens(input_ids)
        caches = [] if use_cache else None
        for i, layer in enumerate(self.layers):
            if use_cache or past_key_values is not None:
                out = layer(h, attention_mask, position_ids,
                            None if past_key_values is None else past_key_values[i], use_cache)
                h, c = out if use_cache else (out, None)
                if use_cache:
                    caches.append(c)
            else:
                h = self.run_layer(layer, h, attention_mask, position_ids)
        h = self.norm(h)
        logits, loss = self.compute_loss(h, labels)
        return logits, loss, caches


def create_model(config: ModelConfig, kernel_type: KernelType = "liger") -> TransformerModel:
    return TransformerModel(config, kernel_type)
