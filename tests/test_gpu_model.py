"""End-to-end on a GPU: the native backend against the PyTorch backend on a tiny hybrid, the
driver entry point, and a short training run whose loss must fall."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _tiny(attn="nsa"):
    from nsa_optim_b200.models import HybridConfig, create_hybrid_model
    cfg = HybridConfig(d_model=256, vocab_size=1024, block_pattern="MDA", block_repeats=1, mamba_d_state=64,
                       mamba_chunk=64, deltanet_head_dim=64, num_attention_heads=4, num_key_value_heads=2,
                       head_dim=64, rope_theta=1e4, intermediate_size=512, attention_type=attn,
                       nsa_window_size=64, nsa_num_selected_blocks=4)
    torch.manual_seed(1)
    return create_hybrid_model(cfg).cuda().bfloat16()


@pytest.mark.parametrize("attn", ["dense", "nsa"])
def test_native_matches_torch_backend(native, attn):
    from nsa_optim_b200 import ops
    m = _tiny(attn)
    ids = torch.randint(0, 1024, (2, 256), device="cuda")
    res = {}
    for be in ("native", "torch"):
        m.zero_grad()
        with ops.backend(be):
            _, loss, _ = m(ids, labels=ids)
            loss.backward()
        res[be] = (loss.item(), torch.cat([p.grad.float().reshape(-1) for p in m.parameters() if p.grad is not None]))
    assert abs(res["native"][0] - res["torch"][0]) < 5e-2
    gn, gt = res["native"][1], res["torch"][1]
    cos = torch.dot(gn, gt) / (gn.norm() * gt.norm() + 1e-12)
    assert cos > 0.98, cos.item()


def test_smoke_entry(native):
    import __graft_entry__ as g
    g.smoke()


def test_short_training_run_reduces_loss(native, tmp_path):
    from nsa_optim_b200.train import Trainer, parse_args
    args = parse_args(["--block_pattern", "MDA", "--block_repeats", "1", "--attn_type", "nsa", "--model_size", "100M",
                       "--hidden_size", "256", "--vocab_size", "512", "--intermediate_size", "512", "--num_heads", "4",
                       "--num_kv_heads", "2", "--head_dim", "64", "--mamba_d_state", "64", "--nsa_window_size", "64",
                       "--nsa_num_selected_blocks", "4", "--context_length", "256", "--batch_size", "4",
                       "--gradient_accumulation_steps", "1", "--optimizer_type", "adamw8bit", "--synthetic_data",
                       "--num_train_steps", "30", "--warmup_steps", "2", "-lr", "3e-3", "--output_dir", str(tmp_path)])
    tr = Trainer(args, verbose=False)
    data = tr.make_data()
    fixed = data.batch_at(0)
    first = last = None
    for i in range(30):
        out = tr.step([fixed])
        if i == 0:
            first = float(out["loss"])
        last = float(out["loss"])
    assert last < first - 0.5, (first, last)
