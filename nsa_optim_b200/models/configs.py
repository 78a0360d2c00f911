"""Model-config factories: from a :class:`TrainingConfig` (size string, context, flags) to
the per-family config objects.

Reference behaviour (nngabe/nsa_optim): get_model_config models/configs.py:28-44,
get_mamba2_config :47-71, get_deltanet_config :74-94, compute_block_repeats :97-118,
get_hybrid_config :121-165, get_model_type :168-182.  Width/depth always come from the
transformer size search; the hybrid keeps the searched width, heads and FFN and derives the
repeat count from the searched depth.

Additions: every factory takes keyword overrides for the shapes a size string cannot
express (vocab, depth, FFN, heads, head_dim, tying, DeltaNet head geometry, NSA pooling),
and the hybrid factory receives the attention type.
"""
from __future__ import annotations

from dataclasses import replace
from typing import Any, Optional

from ..config import (AttentionType, MambaType, ModelConfig, TrainingConfig,
                      compute_model_dimensions, get_model_config_for_size, parse_model_size)
from .deltanet import GatedDeltaNetConfig
from .hybrid import HybridConfig
from .mamba import Mamba2Config

DEFAULT_VOCAB = 151936


def _clean(d: dict) -> dict:
    return {k: v for k, v in d.items() if v is not None}


def get_model_config(training_config: TrainingConfig, nsa_block_size: int = 64,
                     nsa_window_size: int = 64, nsa_num_selected_blocks: int = 16,
                     rope_theta: float = 100000.0, vocab_size: Optional[int] = None,
                     **overrides: Any) -> ModelConfig:
    cfg = get_model_config_for_size(
        training_config.model_size,
        attention_type=training_config.attention_type,
        max_position_embeddings=training_config.max_seq_length,
        vocab_size=vocab_size or DEFAULT_VOCAB,
        nsa_block_size=nsa_block_size,
        nsa_window_size=nsa_window_size,
        nsa_num_selected_blocks=nsa_num_selected_blocks,
        rope_theta=rope_theta,
        **overrides,
    )
    cfg.gradient_checkpointing = training_config.gradient_checkpointing
    return cfg


def get_mamba2_config(training_config: TrainingConfig, vocab_size: Optional[int] = None,
                      **overrides: Any) -> Mamba2Config:
    vocab = vocab_size or DEFAULT_VOCAB
    width, depth, _, _, _ = compute_model_dimensions(parse_model_size(training_config.model_size),
                                                     vocab_size=DEFAULT_VOCAB)
    cfg = Mamba2Config(d_model=width, n_layers=depth, d_state=128, headdim=64, vocab_size=vocab,
                       expand=2, use_triton=True,
                       gradient_checkpointing=training_config.gradient_checkpointing)
    return replace(cfg, **_clean(overrides))


def get_deltanet_config(training_config: TrainingConfig, vocab_size: Optional[int] = None,
                        **overrides: Any) -> GatedDeltaNetConfig:
    vocab = vocab_size or DEFAULT_VOCAB
    width, depth, _, _, _ = compute_model_dimensions(parse_model_size(training_config.model_size),
                                                     vocab_size=DEFAULT_VOCAB)
    cfg = GatedDeltaNetConfig(d_model=width, n_layers=depth, d_state=128, head_dim=64,
                              vocab_size=vocab,
                              gradient_checkpointing=training_config.gradient_checkpointing)
    return replace(cfg, **_clean(overrides))


def compute_block_repeats(block_pattern: str, model_size: str) -> int:
    """Searched transformer depth for the size, divided by the pattern length (at least 1)."""
    _, depth, _, _, _ = compute_model_dimensions(parse_model_size(model_size))
    return max(1, depth // len(block_pattern))


def get_hybrid_config(training_config: TrainingConfig, block_pattern: str, block_repeats: int,
                      mamba_d_state: int = 128, mamba_d_conv: int = 4, mamba_expand: int = 2,
                      mamba_headdim: int = 64, rope_theta: float = 100000.0,
                      vocab_size: Optional[int] = None, verbose: bool = True,
                      **overrides: Any) -> HybridConfig:
    if block_repeats == -1:
        block_repeats = compute_block_repeats(block_pattern, training_config.model_size)
        if verbose:
            print(f"Auto-computed block_repeats={block_repeats} for pattern '{block_pattern}' "
                  f"at size {training_config.model_size}")
    width, _, heads, kv, ffn = compute_model_dimensions(parse_model_size(training_config.model_size),
                                                        vocab_size=DEFAULT_VOCAB)
    cfg = HybridConfig(
        d_model=width, vocab_size=vocab_size or DEFAULT_VOCAB, block_pattern=block_pattern,
        block_repeats=block_repeats, mamba_d_state=mamba_d_state, mamba_d_conv=mamba_d_conv,
        mamba_expand=mamba_expand, mamba_headdim=mamba_headdim, deltanet_head_dim=64,
        num_attention_heads=heads, num_key_value_heads=kv,
        max_position_embeddings=training_config.max_seq_length, rope_theta=rope_theta,
        intermediate_size=ffn, norm_eps=1e-6,
        gradient_checkpointing=training_config.gradient_checkpointing,
        attention_type=training_config.attention_type,
    )
    ov = _clean(overrides)
    if ov:
        if "head_dim" not in ov and ("d_model" in ov or "num_attention_heads" in ov):
            ov["head_dim"] = None
        cfg = replace(cfg, **ov)
    return cfg


def get_model_type(training_config: TrainingConfig, block_pattern: Optional[str] = None) -> str:
    if block_pattern:
        return "hybrid"
    if training_config.mamba_type == MambaType.MAMBA2:
        return "mamba2"
    if training_config.mamba_type == MambaType.MAMBA3:   # member re-used for pure DeltaNet
        return "deltanet"
    return "transformer"
