"""Model families on CPU: shapes, state-dict key layout, init rules, gradients, KV cache."""
import math

import pytest
import torch

from nsa_optim_b200.config import AttentionType, ModelConfig, TrainingConfig
from nsa_optim_b200.models import (AttentionBlock, DeltaNetBlock, GatedDeltaNetConfig, HybridConfig, Mamba2Config,
                                   Mamba3Config, MambaBlock, MLP, RMSNorm, RotaryEmbedding, apply_rotary_pos_emb,
                                   compute_cross_entropy_loss, create_cross_entropy_loss, create_gated_deltanet,
                                   create_hybrid_model, create_mamba2, create_mamba3, create_mlp, create_model,
                                   create_rms_norm, get_block_classes_from_pattern, get_hybrid_config,
                                   get_mamba2_config, get_model_config, get_model_type, remap_legacy_keys)
from nsa_optim_b200.config import MambaType


def small_cfg(attn=AttentionType.DENSE, **kw):
    return ModelConfig("t", 64, 2, 4, 2, 128, vocab_size=100, max_position_embeddings=64, attention_type=attn,
                       nsa_block_size=8, nsa_window_size=8, nsa_num_selected_blocks=2, nsa_compress_block=4,
                       nsa_compress_stride=2, **kw)


def test_rmsnorm_rope_mlp_shapes():
    assert RMSNorm(32)(torch.randn(2, 5, 32)).shape == (2, 5, 32)
    rot = RotaryEmbedding(16, 8)
    cos, sin = rot(torch.randn(1, 20, 16), seq_len=20)
    assert cos.shape == (20, 8) and rot.max_seq_len_cached >= 20
    q, k = apply_rotary_pos_emb(torch.randn(1, 20, 2, 16), torch.randn(1, 20, 1, 16), cos, sin)
    assert q.shape == (1, 20, 2, 16) and k.shape == (1, 20, 1, 16)
    assert MLP(32, 64)(torch.randn(3, 32)).shape == (3, 32)
    assert isinstance(create_rms_norm(8, kernel_type="baseline"), RMSNorm) and isinstance(create_mlp(8, 16), MLP)


@pytest.mark.parametrize("attn", [AttentionType.DENSE, AttentionType.NSA, AttentionType.FSA])
def test_transformer_forward_backward(attn):
    m = create_model(small_cfg(attn))
    ids = torch.randint(0, 100, (2, 32))
    logits, loss, _ = m(ids, labels=ids)
    assert loss.item() > 0
    loss.backward()
    assert all(p.grad is not None for p in m.parameters())
    logits, loss, _ = m(ids)
    assert logits.shape == (2, 32, 100) and loss is None


def test_transformer_state_dict_keys():
    keys = set(create_model(small_cfg(AttentionType.NSA)).state_dict())
    for k in ("embed_tokens.weight", "norm.weight", "lm_head.weight", "layers.0.input_layernorm.weight",
              "layers.0.post_attention_layernorm.weight", "layers.1.self_attn.q_proj.weight",
              "layers.0.self_attn.k_compress.weight", "layers.0.self_attn.gate_slc.weight",
              "layers.0.self_attn.gate_swa.weight", "layers.0.mlp.gate_proj.weight", "layers.0.mlp.down_proj.weight"):
        assert k in keys, k
    assert not any("inv_freq" in k or "cos_cached" in k for k in keys)
    tied = create_model(small_cfg(tie_word_embeddings=True))
    assert "lm_head.weight" not in tied.state_dict()
    assert remap_legacy_keys({"layers.0.mlp.mlp.up_proj.weight": 1}) == {"layers.0.mlp.up_proj.weight": 1}


def test_kv_cache_matches_full_forward():
    m = create_model(small_cfg()).eval()
    ids = torch.randint(0, 100, (1, 12))
    full, _, _ = m(ids)
    _, _, cache = m(ids[:, :8], use_cache=True)
    assert cache[0][0].shape[1] == 8
    step, _, cache2 = m(ids[:, 8:], past_key_values=cache, use_cache=True)
    assert cache2[0][0].shape[1] == 12
    assert torch.allclose(step, full[:, 8:], atol=1e-4)


def test_gradient_checkpointing_same_grads():
    torch.manual_seed(0)
    m = create_model(small_cfg())
    ids = torch.randint(0, 100, (2, 16))
    m(ids, labels=ids)[1].backward()
    ref = [p.grad.clone() for p in m.parameters()]
    m.zero_grad()
    m.gradient_checkpointing_enable()
    m.train()
    m(ids, labels=ids)[1].backward()
    for a, p in zip(ref, m.parameters()):
        assert torch.allclose(a, p.grad, atol=1e-6)


def hybrid_cfg(**kw):
    base = dict(d_model=64, vocab_size=128, block_pattern="MDA", block_repeats=2, mamba_d_state=16, mamba_headdim=16,
                mamba_chunk=16, deltanet_head_dim=16, num_attention_heads=4, num_key_value_heads=2, rope_theta=1e4,
                intermediate_size=128, max_position_embeddings=64)
    base.update(kw)
    return HybridConfig(**base)


def test_hybrid_layout_and_init():
    m = create_hybrid_model(hybrid_cfg())
    assert [type(l) for l in m.layers] == [MambaBlock, DeltaNetBlock, AttentionBlock] * 2
    sd = m.state_dict()
    for k, shape in {
        "layers.0.norm.weight": (64,), "layers.0.post_mixer_norm.weight": (64,),
        "layers.0.mixer.in_proj.weight": (2 * 128 + 2 * 16 + 8, 64), "layers.0.mixer.conv1d.weight": (128 + 32, 1, 4),
        "layers.0.mixer.conv1d.bias": (160,), "layers.0.mixer.dt_bias": (8,), "layers.0.mixer.A_log": (8,),
        "layers.0.mixer.D": (8,), "layers.0.mixer.norm.weight": (128,), "layers.0.mixer.out_proj.weight": (64, 128),
        "layers.1.mixer.q_proj.weight": (64, 64), "layers.1.mixer.v_proj.weight": (128, 64),
        "layers.1.mixer.a_proj.weight": (4, 64), "layers.1.mixer.b_proj.weight": (4, 64),
        "layers.1.mixer.A_log": (4,), "layers.1.mixer.dt_bias": (4,), "layers.1.mixer.q_conv1d.weight": (64, 1, 4),
        "layers.1.mixer.v_conv1d.weight": (128, 1, 4), "layers.1.mixer.g_proj.weight": (128, 64),
        "layers.1.mixer.o_norm.weight": (32,), "layers.1.mixer.o_proj.weight": (64, 128),
        "layers.2.q_proj.weight": (64, 64), "layers.2.k_proj.weight": (32, 64), "layers.2.o_proj.weight": (64, 64),
        "layers.2.post_attn_norm.weight": (64,), "layers.2.mlp.up_proj.weight": (128, 64),
    }.items():
        assert tuple(sd[k].shape) == shape, (k, tuple(sd[k].shape))
    big = create_hybrid_model(hybrid_cfg(d_model=256, num_attention_heads=4, intermediate_size=1024, vocab_size=2000))
    L = big.config.n_layers
    assert abs(big.layers[2].o_proj.weight.std().item() - 0.02 / math.sqrt(2 * L)) < 2e-3
    assert abs(big.layers[0].mixer.out_proj.weight.std().item() - 0.02) < 2e-3      # 'out_proj' is not 'o_proj'
    assert abs(big.lm_head.weight.std().item() - 0.02 / math.sqrt(L)) < 2e-3
    assert get_block_classes_from_pattern("MDMA") == {MambaBlock, DeltaNetBlock, AttentionBlock}
    with pytest.raises(ValueError):
        hybrid_cfg(block_pattern="MXA")


@pytest.mark.parametrize("attn", ["dense", "nsa"])
def test_hybrid_forward_backward(attn):
    m = create_hybrid_model(hybrid_cfg(attention_type=attn, nsa_block_size=8, nsa_window_size=8,
                                       nsa_num_selected_blocks=2, nsa_compress_block=4, nsa_compress_stride=2))
    ids = torch.randint(0, 128, (2, 40))
    logits, loss, cache = m(ids, labels=ids)
    assert logits is None and cache is None and loss.item() > 0
    loss.backward()
    missing = [n for n, p in m.named_parameters() if p.grad is None]
    assert not missing, missing
    assert ("layers.2.gate_cmp.weight" in m.state_dict()) == (attn == "nsa")


def test_pure_ssm_models():
    m = create_mamba2(Mamba2Config(d_model=64, n_layers=2, d_state=16, headdim=16, vocab_size=50, chunk_size=16))
    ids = torch.randint(0, 50, (2, 20))
    _, loss, _ = m(ids, labels=ids)
    loss.backward()
    assert "layers.0.mixer.in_proj.weight" in m.state_dict() and "layers.0.post_mixer_norm.weight" in m.state_dict()
    g = create_gated_deltanet(GatedDeltaNetConfig(d_model=64, n_layers=2, head_dim=16, vocab_size=50))
    _, loss, _ = g(ids, labels=ids)
    loss.backward()
    assert "layers.0.input_layernorm.weight" in g.state_dict() and "layers.0.mixer.o_norm.weight" in g.state_dict()
    m3 = create_mamba3(Mamba3Config(d_model=32, n_layers=1, d_state=8, headdim=16, vocab_size=50))
    logits, _, _ = m3(ids[:, :6])
    assert logits.shape == (2, 6, 50)


def test_factories_and_model_type():
    tc = TrainingConfig(model_size="100M", max_seq_length=512)
    assert get_model_type(tc, "MDMA") == "hybrid" and get_model_type(tc) == "transformer"
    assert get_model_type(TrainingConfig(model_size="100M", mamba_type=MambaType.MAMBA2)) == "mamba2"
    assert get_model_type(TrainingConfig(model_size="100M", mamba_type=MambaType.MAMBA3)) == "deltanet"
    hc = get_hybrid_config(tc, "MDMA", -1, verbose=False)
    assert hc.block_repeats == 6 and hc.d_model == 256 and hc.deltanet_head_dim == 64
    assert hc.max_position_embeddings == 512 and hc.vocab_size == 151936
    mc = get_mamba2_config(tc)
    assert (mc.d_model, mc.n_layers, mc.d_state, mc.headdim) == (256, 24, 128, 64)
    tcfg = get_model_config(TrainingConfig(model_size="100M", attention_type=AttentionType.NSA), 64, 64, 4, 5e5)
    assert tcfg.attention_type == AttentionType.NSA and tcfg.rope_theta == 5e5 and tcfg.nsa_num_selected_blocks == 4


def test_loss_helpers():
    h = torch.randn(2, 6, 8)
    head = torch.nn.Linear(8, 11, bias=False)
    y = torch.randint(0, 11, (2, 6))
    logits, l1 = compute_cross_entropy_loss(h, head, y, None)
    none, l2 = compute_cross_entropy_loss(h, head, y, create_cross_entropy_loss(head, "liger"))
    assert logits.shape == (2, 6, 11) and none is None and torch.allclose(l1, l2, atol=1e-5)
    assert create_cross_entropy_loss(head, "baseline") is None


def test_split_last_backward_equals_torch_split():
    """The column split used by the Mamba mixer: same values and the same gradient as torch.split,
    including a group that receives no gradient."""
    from nsa_optim_b200.models.kernels import split_last
    torch.manual_seed(0)
    x = torch.randn(3, 5, 12, requires_grad=True)
    a, b, c = split_last(x, [4, 6, 2])
    ra, rb, rc = torch.split(x.detach().clone().requires_grad_(True), [4, 6, 2], dim=-1)
    assert torch.equal(a, ra) and torch.equal(b, rb) and torch.equal(c, rc)
    w = torch.randn(3, 5, 4)
    (g,) = torch.autograd.grad((a * w).sum() + (c ** 2).sum(), x)
    want = torch.zeros_like(x)
    want[..., :4] = w
    want[..., 10:] = 2 * x.detach()[..., 10:]
    assert torch.allclose(g, want)


def test_kv_heads_resolve_to_a_divisor_of_the_query_heads():
    """The size table gives 100M models 4 query and 8 KV heads; attention modules fall back to a
    usable grouping, and the 100M hybrid (the smoke-test size) runs a step."""
    from nsa_optim_b200.models.kernels import resolve_kv_heads
    assert resolve_kv_heads(4, 8) == 4 and resolve_kv_heads(32, 8) == 8 and resolve_kv_heads(6, 4) == 3
    cfg = HybridConfig(d_model=64, vocab_size=64, block_pattern="A", block_repeats=1, num_attention_heads=4,
                       num_key_value_heads=8, head_dim=16, intermediate_size=64)
    m = create_hybrid_model(cfg)
    ids = torch.randint(0, 64, (1, 16))
    _, loss, _ = m(input_ids=ids, labels=ids)
    loss.backward()
    assert m.layers[0].k_proj.weight.shape[0] == 4 * 16


def test_learned_block_scorer_mode_selects_causal_blocks_and_trains():
    """``nsa_block_scorer="learned"``: the reference module's k_compress scorer picks the blocks and
    the selected + window branches run on them (reference: models/transformer.py:172-268)."""
    from nsa_optim_b200.ops import torch_impl
    cfg = small_cfg(AttentionType.NSA, nsa_block_scorer="learned")
    m = create_model(cfg)
    attn = m.layers[0].self_attn
    assert attn.block_scorer == "learned" and float(attn.k_compress.weight.abs().sum()) > 0
    assert "layers.0.self_attn.k_compress.weight" in m.state_dict()
    B, T = 2, 40
    q = torch.randn(B, T, attn.num_heads, attn.head_dim)
    k = torch.randn(B, T, attn.num_kv_heads, attn.head_dim)
    idx = attn.learned_block_indices(q, k)
    assert idx.shape == (B, attn.num_kv_heads, T, cfg.nsa_num_selected_blocks) and idx.dtype == torch.int32
    own = (torch.arange(T) // cfg.nsa_block_size)[None, None, :, None]
    assert bool(((idx <= own) & (idx >= -1)).all())                         # never a block after the query's own
    first = idx[:, :, : cfg.nsa_block_size]                                 # queries of block 0 see exactly one block
    assert bool((first[..., 0] == 0).all()) and bool((first[..., 1:] == -1).all())
    srt = idx.masked_fill(idx < 0, 10 ** 6).sort(-1).values
    assert bool((srt[..., 1:] > srt[..., :-1]).logical_or(srt[..., 1:] == 10 ** 6).all())   # ascending, no repeats
    # with every visible block selected the selected branch is plain causal attention
    nS = -(-T // cfg.nsa_block_size)
    every = torch.arange(nS, dtype=torch.int32).expand(B, attn.num_kv_heads, T, nS)
    v = torch.randn(B, T, attn.num_kv_heads, attn.head_dim)
    full = torch_impl.selected_attention(q, k, v, every, cfg.nsa_block_size)
    assert torch.allclose(full, torch_impl.attention(q, k, v, True, 0, None), atol=1e-5)
    ids = torch.randint(0, 100, (2, 32))
    _, loss, _ = m(ids, labels=ids)
    loss.backward()
    assert all(p.grad is not None for n, p in m.named_parameters() if "gate_cmp" not in n)
