"""Closed-form FLOP counts per token and arithmetic intensity.

Reference counterpart (nngabe/nsa_optim): profiling/flops.py:12-246 counts a transformer's
forward FLOPs per token (training = 3 x forward), with sparse attention counted as
``block x selected`` keys.  This module keeps those two entry points and extends the model to
the hybrid's Mamba-2 and Gated DeltaNet blocks and to the three-branch sparse attention, so the
trainer and the benchmark can report model FLOP utilisation (MFU) against a measured peak.
All counts are multiply-accumulate x 2.
"""
from __future__ import annotations

from typing import Dict, Optional

from ..config import AttentionType, ModelConfig


def _mlp(d: int, ffn: int) -> float:
    return 2.0 * 3 * d * ffn


def attention_flops_per_token(cfg_heads: int, kv_heads: int, head_dim: int, d: int, seq_len: int,
                              attention_type: AttentionType = AttentionType.DENSE, block: int = 64, selected: int = 16,
                              window: int = 512, cmp_stride: int = 16) -> Dict[str, float]:
    proj = 2.0 * d * head_dim * (2 * cfg_heads + 2 * kv_heads)          # q, o, k, v projections
    if attention_type == AttentionType.DENSE:
        keys = seq_len / 2.0                                            # causal average
        core = 4.0 * cfg_heads * head_dim * keys
        extra = 0.0
    else:
        k_sel = min(seq_len / 2.0, block * selected)
        k_win = min(seq_len / 2.0, window)
        k_cmp = seq_len / (2.0 * cmp_stride)
        core = 4.0 * cfg_heads * head_dim * (k_sel + k_win + k_cmp) + 2.0 * cfg_heads * head_dim * k_cmp  # + importance pass
        extra = 2.0 * d * 3 * cfg_heads                                 # gate projections
    return {"proj": proj, "core": core, "extra": extra, "total": proj + core + extra}


def mamba2_flops_per_token(d: int, d_state: int = 128, expand: int = 2, headdim: int = 64, chunk: int = 128,
                           d_conv: int = 4) -> Dict[str, float]:
    d_in = expand * d
    heads = d_in // headdim
    proj = 2.0 * d * (2 * d_in + 2 * d_state + heads) + 2.0 * d_in * d
    conv = 2.0 * (d_in + 2 * d_state) * d_conv
    # per token: C.B against the chunk (chunk/2 causal average), P x, chunk state and state read
    ssd = 2.0 * d_state * chunk / 2 * heads + 2.0 * headdim * chunk / 2 * heads + 2 * 2.0 * d_state * headdim * heads
    return {"proj": proj, "conv": conv, "core": ssd, "total": proj + conv + ssd}


def deltanet_flops_per_token(d: int, heads: int, head_dim: int, expand_v: int = 2, chunk: int = 64, d_conv: int = 4) -> Dict[str, float]:
    K, V = head_dim, head_dim * expand_v
    proj = 2.0 * d * heads * (2 * K + 2 * V + 2) + 2.0 * heads * V * d
    conv = 2.0 * heads * (2 * K + V) * d_conv
    # per token and head: k k^T and q k^T rows (chunk), triangular solve (chunk/2 x (K+V)), state ops (4 K V)
    core = heads * (2 * 2.0 * K * chunk + 2.0 * chunk / 2 * (K + V) + 2.0 * chunk * V + 4 * 2.0 * K * V)
    return {"proj": proj, "conv": conv, "core": core, "total": proj + conv + core}


def calculate_flops_per_token(config: ModelConfig, seq_len: int, training: bool = True) -> Dict[str, float]:
    """Transformer FLOPs per token (forward, or forward + backward = 3x when ``training``)."""
    d, L = config.hidden_size, config.num_hidden_layers
    att = attention_flops_per_token(config.num_attention_heads, config.num_key_value_heads, config.head_dim, d, seq_len,
                                    config.attention_type, config.nsa_block_size, config.nsa_num_selected_blocks,
                                    config.nsa_window_size, config.nsa_compress_stride)
    mlp = _mlp(d, config.intermediate_size)
    head = 2.0 * d * config.vocab_size
    fwd = L * (att["total"] + mlp) + head
    mult = 3.0 if training else 1.0
    return {"attention": L * att["total"] * mult, "mlp": L * mlp * mult, "lm_head": head * mult, "total": fwd * mult,
            "forward": fwd}


def hybrid_flops_per_token(cfg, seq_len: int, training: bool = True, recompute: bool = False) -> Dict[str, float]:
    """FLOPs per token of a :class:`~nsa_optim_b200.models.hybrid.HybridConfig` model.  With
    per-block activation checkpointing (``recompute``) the blocks run forward twice: 4x instead of 3x."""
    d = cfg.d_model
    mlp = _mlp(d, cfg.intermediate_size)
    per = {"M": mamba2_flops_per_token(d, cfg.mamba_d_state, cfg.mamba_expand, cfg.mamba_headdim)["total"] + mlp,
           "D": deltanet_flops_per_token(d, cfg.deltanet_num_heads or d // cfg.deltanet_head_dim, cfg.deltanet_head_dim,
                                         cfg.deltanet_expand_v)["total"] + mlp,
           "A": attention_flops_per_token(cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, d, seq_len,
                                          cfg.attention_type, cfg.nsa_block_size, cfg.nsa_num_selected_blocks,
                                          cfg.nsa_window_size, cfg.nsa_compress_stride)["total"] + mlp}
    blocks = sum(per[c] for c in cfg.block_pattern) * cfg.block_repeats
    head = 2.0 * d * cfg.vocab_size
    mult_blocks = (4.0 if recompute else 3.0) if training else 1.0
    mult_head = 3.0 if training else 1.0
    return {"blocks_forward": blocks, "lm_head_forward": head, "per_block_forward": per,
            "total": blocks * mult_blocks + head * mult_head,
            "model_flops": (blocks + head) * (3.0 if training else 1.0)}


def calculate_arithmetic_intensity(config: ModelConfig, seq_len: int, batch_size: int = 1, bytes_per_param: int = 2) -> Dict[str, float]:
    """FLOPs per byte of parameter traffic for one forward pass over ``batch_size * seq_len`` tokens."""
    from ..config import compute_transformer_params
    flops = calculate_flops_per_token(config, seq_len, training=False)["total"] * batch_size * seq_len
    params = compute_transformer_params(config.hidden_size, config.num_hidden_layers, config.num_key_value_heads, config.vocab_size)
    act_bytes = 2.0 * batch_size * seq_len * config.hidden_size * config.num_hidden_layers * 8
    nbytes = params * bytes_per_param + act_bytes
    return {"flops": flops, "bytes": nbytes, "intensity": flops / nbytes}


def model_flops_utilisation(model_flops_per_token: float, tokens_per_second: float, n_gpus: int = 1,
                            peak_tflops: Optional[float] = None) -> float:
    """MFU against ``peak_tflops`` per GPU (default: the measured sustained bf16 GEMM rate)."""
    if peak_tflops is None:
        from ..benchmarks.kernel_benchmark import peaks
        peak_tflops = peaks()["bf16_tflops_sustained"]
    return model_flops_per_token * tokens_per_second / (n_gpus * peak_tflops * 1e12)
