"""Config layer: size resolution table, enums, run names, experiment grid and filters."""
import pytest

from nsa_optim_b200.config import (AttentionType, MambaType, MODEL_CONFIGS, ModelSize, OptimizerConfig,
                                   OptimizerType, TrainingConfig, compute_model_dimensions,
                                   compute_transformer_params, get_experiment_grid, get_filtered_experiments,
                                   get_model_config_for_size, parse_model_size, resolve_attention_type,
                                   _get_batch_config, _get_training_steps, CONTEXT_LENGTHS)

RESOLVED = {
    "100M": (256, 24, 4, 8, 512), "0.44B": (1024, 12, 16, 8, 2048), "0.5B": (1024, 16, 16, 8, 2048),
    "0.6B": (1024, 24, 16, 8, 2048), "1B": (2048, 12, 32, 8, 4096), "4B": (4096, 16, 64, 8, 8192),
    "8B": (4096, 40, 64, 8, 8192), "32B": (8192, 44, 128, 8, 16384),
}


@pytest.mark.parametrize("size,dims", RESOLVED.items())
def test_size_resolution_table(size, dims):
    assert compute_model_dimensions(parse_model_size(size)) == dims


def test_parse_model_size():
    assert parse_model_size("1B") == 10 ** 9
    assert parse_model_size("1.5b") == 1_500_000_000
    assert parse_model_size("500M") == 500_000_000
    assert parse_model_size("42K") == 42_000
    assert parse_model_size("123456") == 123456
    with pytest.raises(ValueError):
        parse_model_size("big")


def test_legacy_configs_consistent():
    for size, cfg in MODEL_CONFIGS.items():
        assert cfg.hidden_size % cfg.num_attention_heads == 0
        assert cfg.num_attention_heads % cfg.num_key_value_heads == 0
        assert cfg.intermediate_size > cfg.hidden_size
    assert MODEL_CONFIGS[ModelSize.SMALL].num_hidden_layers == 28


def test_named_config_and_overrides():
    cfg = get_model_config_for_size("0.6B")
    assert cfg.name.startswith("transformer-") and cfg.hidden_size == 1024 and cfg.head_dim == 64
    cfg = get_model_config_for_size("0.6B", num_hidden_layers=28, intermediate_size=3072, num_attention_heads=16,
                                    head_dim=128, vocab_size=151936)
    assert (cfg.num_hidden_layers, cfg.intermediate_size, cfg.head_dim) == (28, 3072, 128)


def test_optimizer_config_defaults():
    c = OptimizerConfig(OptimizerType.SOAP_4BIT)
    assert (c.learning_rate, c.weight_decay, c.beta1, c.beta2, c.eps) == (1e-4, 0.1, 0.9, 0.95, 1e-8)
    assert (c.precondition_frequency, c.shampoo_beta, c.max_precond_dim) == (5, 0.95, 1024)


def test_run_names():
    assert TrainingConfig(model_size="1B").run_name == "1B_dense_adamw_ctx32768"
    c = TrainingConfig(model_size="1B", mamba_type=MambaType.MAMBA2, attention_type=AttentionType.NSA)
    assert c.run_name == "1B_jamba_mamba2_native_sparse_attention_adamw_ctx32768"
    assert TrainingConfig(model_size=ModelSize.SMALL).model_size == "0.6B"
    assert resolve_attention_type("nsa") is AttentionType.NSA and resolve_attention_type("fsa") is AttentionType.FSA


def test_grid_and_filters():
    grid = get_experiment_grid()
    assert len(grid) == 224
    ext = set(CONTEXT_LENGTHS["extended_nsa"])
    assert all(e.attention_type == AttentionType.NSA for e in grid if e.max_seq_length in ext)
    assert {e.optimizer_type for e in grid} == set(OptimizerType)
    f = get_filtered_experiments(model_sizes=["4B"], optimizer_types=[OptimizerType.SOAP_4BIT], context_lengths=[32768])
    assert len(f) == 3 and all(e.model_size == "4B" for e in f)
    assert _get_batch_config("0.6B", 32768) == (4, 4) and _get_batch_config("32B", 1048576) == (1, 256)
    assert _get_training_steps("4B", 131072) == 25000 and _get_training_steps("4B", 1048576) == 10000


def test_param_count_formula():
    n = compute_transformer_params(1024, 12)
    per_layer = 2 * 1024 * 1024 + 2 * 1024 * 512 + 3 * 1024 * 2752 + 2048
    assert n == 2 * 151936 * 1024 + 12 * per_layer + 1024
