"""Configuration layer: enums, dataclasses, size-string resolution and the experiment grid.

Behavioural parity targets in the reference project (paths inside nngabe/nsa_optim):
  * enums and dataclasses ............ config.py:14-65, config.py:324-413
  * size-string parser ............... config.py:68-101
  * parameter count + dimension search config.py:129-225
  * named config for a size .......... config.py:228-284
  * legacy fixed configs ............. config.py:288-321
  * experiment grid and filters ...... config.py:416-498

The resolution rule is a grid search (power-of-two widths x an even layer range that
depends on the size band) for the closed-form parameter count nearest the target; the
feed-forward width is the power of two nearest 8/3 of the width.  This module restates the
rule with a vectorised search and adds the override fields the B200 benchmark
configurations need (head_dim, vocab, FFN width, NSA compression block/stride, tying).
"""
from __future__ import annotations

import re
from dataclasses import dataclass, field, replace
from enum import Enum
from typing import Any, Dict, Iterable, List, Optional, Sequence, Tuple


# --------------------------------------------------------------------------------------
# Enums (str-valued so CLI strings map straight onto members)
# --------------------------------------------------------------------------------------
class AttentionType(str, Enum):
    DENSE = "dense"
    NSA = "native_sparse_attention"
    FSA = "flash_sparse_attention"


class MambaType(str, Enum):
    NONE = "none"
    MAMBA2 = "mamba2"
    MAMBA3 = "mamba3"  # the reference re-uses this member to mean "pure Gated DeltaNet"


class OptimizerType(str, Enum):
    ADAMW = "adamw"
    ADAMW_4BIT = "adamw4bit"
    ADAMW_8BIT = "adamw8bit"
    SOAP = "soap"
    SOAP_4BIT = "soap4bit"
    SOAP_8BIT = "soap8bit"
    SHAMPOO = "shampoo"


class ModelSize(str, Enum):
    """Legacy fixed sizes; free-form strings such as ``"1B"`` are preferred."""
    SMALL = "0.6B"
    MEDIUM = "4B"
    LARGE = "8B"
    XLARGE = "32B"


ATTENTION_ALIASES = {"nsa": AttentionType.NSA.value, "fsa": AttentionType.FSA.value}


def resolve_attention_type(name: "str | AttentionType") -> AttentionType:
    if isinstance(name, AttentionType):
        return name
    return AttentionType(ATTENTION_ALIASES.get(name, name))


# --------------------------------------------------------------------------------------
# Dataclasses
# --------------------------------------------------------------------------------------
@dataclass
class ModelConfig:
    """Transformer architecture description (reference: config.py:46-65)."""
    name: str
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    intermediate_size: int
    vocab_size: int = 151936
    max_position_embeddings: int = 32768
    rope_theta: float = 100000.0
    rms_norm_eps: float = 1e-6
    tie_word_embeddings: bool = False
    attention_type: AttentionType = AttentionType.DENSE
    # sparse-attention knobs shared with the reference
    nsa_block_size: int = 64
    nsa_window_size: int = 64
    nsa_num_selected_blocks: int = 16
    # additions: compressed branch geometry and an explicit head width
    nsa_compress_block: int = 32
    nsa_compress_stride: int = 16
    # how the selected branch picks its blocks: "compressed" = from the compressed branch's
    # attention probabilities (three branches); "learned" = the reference module's scorer, a
    # projection k_compress of queries and block-mean keys (two branches: selected + window)
    nsa_block_scorer: str = "compressed"
    head_dim: Optional[int] = None
    gradient_checkpointing: bool = False

    def __post_init__(self):
        if self.head_dim is None:
            self.head_dim = self.hidden_size // self.num_attention_heads
        self.attention_type = resolve_attention_type(self.attention_type)


@dataclass
class OptimizerConfig:
    """Optimizer hyper-parameters (reference: config.py:324-343)."""
    optimizer_type: OptimizerType
    learning_rate: float = 1e-4
    weight_decay: float = 0.1
    beta1: float = 0.9
    beta2: float = 0.95
    eps: float = 1e-8
    precondition_frequency: int = 5
    shampoo_beta: float = 0.95
    max_precond_dim: int = 1024
    use_4bit: bool = True
    use_8bit: bool = False
    shampoo_state_dtype: str = "bfloat16"
    # additions
    master_weights: bool = False  # keep an fp32 copy of each owned parameter shard

    def __post_init__(self):
        if not isinstance(self.optimizer_type, OptimizerType):
            self.optimizer_type = OptimizerType(self.optimizer_type)


@dataclass
class TrainingConfig:
    """Run description (reference: config.py:346-413)."""
    model_size: str = "0.6B"
    attention_type: AttentionType = AttentionType.DENSE
    mamba_type: MambaType = MambaType.NONE
    jamba_ratio: int = 7
    optimizer_type: OptimizerType = OptimizerType.ADAMW
    optimizer_config: Optional[OptimizerConfig] = None
    max_seq_length: int = 32768
    batch_size: int = 1
    gradient_accumulation_steps: int = 8
    num_train_steps: int = 100000
    warmup_steps: int = 2000
    max_grad_norm: float = 1.0
    lr_scheduler_type: str = "cosine"
    min_lr_ratio: float = 0.1
    dtype: str = "bfloat16"
    use_flash_attention: bool = True
    gradient_checkpointing: bool = True
    tensor_parallel_size: int = 1
    pipeline_parallel_size: int = 1
    data_parallel_size: int = 1
    log_interval: int = 10
    eval_interval: int = 1000
    save_interval: int = 5000
    dataset_name: str = "HuggingFaceFW/fineweb-edu"
    dataset_subset: str = "sample-10BT"
    output_dir: str = "./outputs"
    run_name: str = ""
    # additions
    seed: int = 0
    synthetic_data: bool = False

    def __post_init__(self):
        if isinstance(self.model_size, ModelSize):
            self.model_size = self.model_size.value
        self.attention_type = resolve_attention_type(self.attention_type)
        if not isinstance(self.mamba_type, MambaType):
            self.mamba_type = MambaType(self.mamba_type)
        if not isinstance(self.optimizer_type, OptimizerType):
            self.optimizer_type = OptimizerType(self.optimizer_type)
        if self.optimizer_config is None:
            self.optimizer_config = OptimizerConfig(optimizer_type=self.optimizer_type)
        if not self.run_name:
            self.run_name = default_run_name(self)


def default_run_name(cfg: TrainingConfig) -> str:
    """``{size}_{arch}_{optimizer}_ctx{N}``; arch naming follows config.py:402-413."""
    sparse = cfg.attention_type != AttentionType.DENSE
    if cfg.mamba_type != MambaType.NONE and sparse:
        arch = f"jamba_{cfg.mamba_type.value}_{cfg.attention_type.value}"
    elif cfg.mamba_type != MambaType.NONE:
        arch = cfg.mamba_type.value
    else:
        arch = cfg.attention_type.value
    return f"{cfg.model_size}_{arch}_{cfg.optimizer_type.value}_ctx{cfg.max_seq_length}"


# --------------------------------------------------------------------------------------
# Size strings
# --------------------------------------------------------------------------------------
_SIZE_RE = re.compile(r"^([\d.]+)\s*([BMK]?)$")
_SUFFIX = {"B": 1e9, "M": 1e6, "K": 1e3, "": 1.0}


def parse_model_size(size_str: str) -> int:
    """``"1B"``/``"1.5B"``/``"500M"``/``"42K"``/raw digits -> parameter count."""
    text = str(size_str).strip().upper()
    m = _SIZE_RE.match(text)
    if m:
        return int(float(m.group(1)) * _SUFFIX[m.group(2)])
    try:
        return int(float(text))
    except ValueError as exc:
        raise ValueError(
            f"Cannot parse model size: {size_str}. Use formats like '1B', '500M', '1.5B'"
        ) from exc


def _round_to_multiple(x: int, multiple: int) -> int:
    return ((x + multiple // 2) // multiple) * multiple


def _round_up_to_multiple(x: int, multiple: int) -> int:
    return -(-x // multiple) * multiple


def _nearest_power_of_2(x: int) -> int:
    if x <= 0:
        return 1
    lo = 1 << (x.bit_length() - 1)
    hi = lo * 2
    return lo if (x - lo) < (hi - x) else hi


VALID_HIDDEN_SIZES = [256, 512, 1024, 2048, 4096, 8192, 16384]


def compute_transformer_params(
    hidden_size: int,
    num_layers: int,
    num_kv_heads: int = 8,
    vocab_size: int = 151936,
    intermediate_multiplier: float = 8 / 3,
) -> int:
    """Closed-form count: untied embeddings, GQA with 64-wide heads, SwiGLU FFN whose width
    is 8/3 of the model width rounded up to 64, two norms per layer and a final norm."""
    head_dim = 64
    ffn = _round_up_to_multiple(int(hidden_size * intermediate_multiplier), 64)
    kv = num_kv_heads * head_dim
    per_layer = (
        2 * hidden_size * hidden_size      # q and o projections
        + 2 * hidden_size * kv             # k and v projections
        + 3 * hidden_size * ffn            # gate, up, down
        + 2 * hidden_size                  # two norms
    )
    return 2 * vocab_size * hidden_size + num_layers * per_layer + hidden_size


def _layer_candidates(target_params: int, min_layers: int, max_layers: int) -> range:
    if target_params < 500_000_000:
        return range(min_layers, min(32, max_layers + 1), 2)
    if target_params < 5_000_000_000:
        return range(12, min(48, max_layers + 1), 2)
    return range(24, max_layers + 1, 4)


def compute_model_dimensions(
    target_params: int,
    vocab_size: int = 151936,
    num_kv_heads: int = 8,
    head_dim: int = 64,
    intermediate_multiplier: float = 8 / 3,
    min_layers: int = 4,
    max_layers: int = 128,
) -> Tuple[int, int, int, int, int]:
    """-> (hidden, layers, heads, kv_heads, ffn) whose closed-form count is nearest the target.

    Ties keep the first candidate in (width ascending, depth ascending) order, which is what
    a strict ``<`` comparison in a nested loop yields.
    """
    layers = _layer_candidates(target_params, min_layers, max_layers)
    best: Optional[Tuple[int, int]] = None
    best_gap = None
    for width in VALID_HIDDEN_SIZES:
        for depth in layers:
            gap = abs(
                compute_transformer_params(width, depth, num_kv_heads, vocab_size, intermediate_multiplier)
                - target_params
            )
            if best_gap is None or gap < best_gap:
                best_gap, best = gap, (width, depth)
    if best is None:
        raise ValueError(f"Could not find valid configuration for {target_params} parameters")
    width, depth = best
    ffn = _nearest_power_of_2(int(width * intermediate_multiplier))
    return width, depth, width // head_dim, num_kv_heads, ffn


def format_param_count(n: int) -> str:
    return f"{n / 1e9:.2f}B" if n >= 1e9 else f"{n / 1e6:.0f}M"


def get_model_config_for_size(
    size_str: str,
    attention_type: AttentionType = AttentionType.DENSE,
    max_position_embeddings: int = 32768,
    vocab_size: int = 151936,
    nsa_block_size: int = 64,
    nsa_window_size: int = 64,
    nsa_num_selected_blocks: int = 16,
    rope_theta: float = 100000.0,
    **overrides: Any,
) -> ModelConfig:
    """Named transformer config for a size string; ``overrides`` replace resolved fields
    (``hidden_size``, ``num_hidden_layers``, ``num_attention_heads``, ``num_key_value_heads``,
    ``intermediate_size``, ``head_dim``, ``tie_word_embeddings``, NSA compression geometry)."""
    target = parse_model_size(size_str)
    width, depth, heads, kv, ffn = compute_model_dimensions(target, vocab_size=vocab_size)
    actual = compute_transformer_params(width, depth, kv, vocab_size)
    cfg = ModelConfig(
        name=f"transformer-{format_param_count(actual)}",
        hidden_size=width,
        num_hidden_layers=depth,
        num_attention_heads=heads,
        num_key_value_heads=kv,
        intermediate_size=ffn,
        vocab_size=vocab_size,
        max_position_embeddings=max_position_embeddings,
        rope_theta=rope_theta,
        attention_type=attention_type,
        nsa_block_size=nsa_block_size,
        nsa_window_size=nsa_window_size,
        nsa_num_selected_blocks=nsa_num_selected_blocks,
    )
    clean = {k: v for k, v in overrides.items() if v is not None}
    if clean:
        if "head_dim" not in clean and ("hidden_size" in clean or "num_attention_heads" in clean):
            clean["head_dim"] = None
        cfg = replace(cfg, **clean)
    return cfg


MODEL_CONFIGS: Dict[ModelSize, ModelConfig] = {
    ModelSize.SMALL: ModelConfig("transformer-0.6B", 1024, 28, 16, 8, 3072),
    ModelSize.MEDIUM: ModelConfig("transformer-4B", 2560, 36, 32, 8, 9216),
    ModelSize.LARGE: ModelConfig("transformer-8B", 4096, 36, 32, 8, 12288),
    ModelSize.XLARGE: ModelConfig("transformer-32B", 5120, 64, 40, 8, 25600),
}


# --------------------------------------------------------------------------------------
# Experiment grid
# --------------------------------------------------------------------------------------
CONTEXT_LENGTHS = {
    "standard": [32768, 131072],
    "extended_nsa": [524288, 1048576],
}

_BATCH_TABLE = (
    # (upper parameter bound, {context: (batch, accumulation)})
    (1e9, {32768: (4, 4), 131072: (1, 16), 524288: (1, 32), 1048576: (1, 64)}),
    (5e9, {32768: (2, 8), 131072: (1, 16), 524288: (1, 32), 1048576: (1, 64)}),
    (15e9, {32768: (1, 16), 131072: (1, 32), 524288: (1, 64), 1048576: (1, 128)}),
    (float("inf"), {32768: (1, 32), 131072: (1, 64), 524288: (1, 128), 1048576: (1, 256)}),
)


def _get_batch_config(model_size: str, ctx_len: int) -> Tuple[int, int]:
    n = parse_model_size(model_size)
    for bound, table in _BATCH_TABLE:
        if n < bound:
            return table.get(ctx_len, (1, 16))
    return (1, 16)


def _get_training_steps(model_size: str, ctx_len: int) -> int:
    """Keep the token budget roughly constant across context lengths (floor 10 000 steps)."""
    return max(10000, int(100000 * 32768 / ctx_len))


def get_experiment_grid() -> List[TrainingConfig]:
    """4 sizes x 3 attention types x 7 optimizers x contexts (extended ones for NSA only)."""
    grid: List[TrainingConfig] = []
    for size in ("0.6B", "4B", "8B", "32B"):
        for attn in AttentionType:
            contexts = list(CONTEXT_LENGTHS["standard"])
            if attn == AttentionType.NSA:
                contexts += CONTEXT_LENGTHS["extended_nsa"]
            for opt in OptimizerType:
                for ctx in contexts:
                    batch, accum = _get_batch_config(size, ctx)
                    grid.append(
                        TrainingConfig(
                            model_size=size,
                            attention_type=attn,
                            optimizer_type=opt,
                            max_seq_length=ctx,
                            batch_size=batch,
                            gradient_accumulation_steps=accum,
                            num_train_steps=_get_training_steps(size, ctx),
                        )
                    )
    return grid


def get_filtered_experiments(
    model_sizes: Optional[Sequence[str]] = None,
    attention_types: Optional[Sequence[AttentionType]] = None,
    optimizer_types: Optional[Sequence[OptimizerType]] = None,
    context_lengths: Optional[Sequence[int]] = None,
) -> List[TrainingConfig]:
    def keep(exp: TrainingConfig) -> bool:
        return (
            (not model_sizes or exp.model_size in model_sizes)
            and (not attention_types or exp.attention_type in attention_types)
            and (not optimizer_types or exp.optimizer_type in optimizer_types)
            and (not context_lengths or exp.max_seq_length in context_lengths)
        )

    return [e for e in get_experiment_grid() if keep(e)]


def print_model_config(size_str: str) -> None:
    cfg = get_model_config_for_size(size_str)
    n = compute_transformer_params(
        cfg.hidden_size, cfg.num_hidden_layers, cfg.num_key_value_heads, cfg.vocab_size
    )
    print(f"Model Configuration for '{size_str}':")
    for label, value in (
        ("Name", cfg.name),
        ("Hidden size", cfg.hidden_size),
        ("Num layers", cfg.num_hidden_layers),
        ("Num attention heads", cfg.num_attention_heads),
        ("Num KV heads", cfg.num_key_value_heads),
        ("Head dim", cfg.head_dim),
        ("Intermediate size", cfg.intermediate_size),
        ("Vocab size", cfg.vocab_size),
    ):
        print(f"  {label}: {value}")
    print(f"  Actual parameters: {n:,} ({n / 1e9:.3f}B)")


if __name__ == "__main__":
    for s in ("100M", "500M", "1B", "4B", "8B", "32B"):
        print_model_config(s)
        print()
