"""Optimizers on CPU: grouping, factory, update maths, low-bit states, schedules, coverage."""
import math

import pytest
import torch
import torch.nn as nn

from nsa_optim_b200.config import OptimizerConfig, OptimizerType
from nsa_optim_b200.optimizers import (AdamW, AdamWLowBit, SOAPLowBit, SOAPReference, ShampooReference,
                                       analyze_preconditioning_coverage, create_optimizer, get_lr_scheduler,
                                       get_param_groups, lr_multiplier, print_preconditioning_stats)


class Net(nn.Module):
    def __init__(self, d=64):
        super().__init__()
        self.embed_tokens = nn.Embedding(50, d)
        self.fc1 = nn.Linear(d, 2 * d)
        self.input_layernorm = nn.LayerNorm(2 * d)
        self.fc2 = nn.Linear(2 * d, d, bias=False)

    def forward(self, x):
        return self.fc2(self.input_layernorm(torch.relu(self.fc1(self.embed_tokens(x))))).pow(2).mean()


def test_param_groups():
    decay, no_decay = get_param_groups(Net(), 0.1)
    assert decay["weight_decay"] == 0.1 and no_decay["weight_decay"] == 0.0
    assert set(decay["param_names"]) == {"fc1.weight", "fc2.weight"}
    assert "embed_tokens.weight" in no_decay["param_names"] and "fc1.bias" in no_decay["param_names"]
    assert "input_layernorm.weight" in no_decay["param_names"]


@pytest.mark.parametrize("ot,cls", [(OptimizerType.ADAMW, AdamW), (OptimizerType.ADAMW_8BIT, AdamWLowBit),
                                    (OptimizerType.ADAMW_4BIT, AdamWLowBit), (OptimizerType.SOAP, SOAPReference),
                                    (OptimizerType.SOAP_4BIT, SOAPLowBit), (OptimizerType.SOAP_8BIT, SOAPLowBit),
                                    (OptimizerType.SHAMPOO, ShampooReference)])
def test_factory_and_one_step(ot, cls):
    net = Net()
    opt = create_optimizer(net, OptimizerConfig(ot, learning_rate=1e-2, precondition_frequency=2, max_precond_dim=64))
    assert isinstance(opt, cls)
    before = [p.detach().clone() for p in net.parameters()]
    for _ in range(3):
        opt.zero_grad()
        net(torch.randint(0, 50, (4, 7))).backward()
        opt.step()
    assert all(not torch.equal(a, p) for a, p in zip(before, net.parameters()))
    assert all(torch.isfinite(p).all() for p in net.parameters())


def test_adamw_matches_torch():
    torch.manual_seed(0)
    a, b = nn.Linear(8, 8), nn.Linear(8, 8)
    b.load_state_dict(a.state_dict())
    o1 = AdamW(a.parameters(), lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    o2 = torch.optim.AdamW(b.parameters(), lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    for _ in range(5):
        x = torch.randn(4, 8)
        for m, o in ((a, o1), (b, o2)):
            o.zero_grad()
            m(x).pow(2).sum().backward()
            o.step()
    assert torch.allclose(a.weight, b.weight, atol=1e-6)


def test_grad_scale_equals_scaled_gradient():
    p1, p2 = nn.Parameter(torch.randn(300)), None
    p2 = nn.Parameter(p1.detach().clone())
    g = torch.randn(300)
    o1, o2 = AdamW([p1], lr=1e-2), AdamW([p2], lr=1e-2)
    p1.grad, p2.grad = g.clone(), g * 0.25
    o1.step(grad_scale=torch.tensor(0.25))
    o2.step()
    assert torch.allclose(p1, p2, atol=1e-7)


def test_lowbit_state_layout_and_tracking():
    big, small = nn.Parameter(torch.randn(64, 128)), nn.Parameter(torch.randn(100))
    ref_p = nn.Parameter(big.detach().clone())
    opt = AdamWLowBit([big, small], lr=1e-2, weight_decay=0.0, bits=8)
    ref = AdamW([ref_p], lr=1e-2, weight_decay=0.0)
    for _ in range(10):
        g = torch.randn(64, 128)
        big.grad, ref_p.grad, small.grad = g.clone(), g.clone(), torch.randn(100)
        opt.step(); ref.step()
    st = opt.state[big]
    assert st["exp_avg"].dtype == torch.uint8 and st["exp_avg_absmax"].numel() == 64 * 128 // 256
    assert opt.state[small]["exp_avg"].dtype == torch.float32           # below 4096 elements: float state
    assert (big - ref_p).abs().max() < 2e-2


def test_soap_reference_keeps_orthonormal_bases_and_converges():
    torch.manual_seed(0)
    w = nn.Parameter(torch.randn(12, 8))
    target = torch.randn(12, 8)
    opt = SOAPReference([w], lr=5e-2, precondition_frequency=3, weight_decay=0.0)
    first = None
    for i in range(200):
        opt.zero_grad()
        loss = (w - target).pow(2).sum()
        first = first or loss.item()
        loss.backward()
        opt.step()
    st = opt.state[w]
    assert torch.allclose(st["QL"].T @ st["QL"], torch.eye(12), atol=1e-4)
    assert loss.item() < 1e-2 * first


def test_shampoo_inverse_root():
    m = torch.randn(6, 6)
    spd = m @ m.T + torch.eye(6)
    r = ShampooReference._matrix_power(spd, -0.25)
    assert torch.allclose(torch.linalg.matrix_power(r, 4) @ spd, torch.eye(6), atol=1e-3)


@pytest.mark.parametrize("bits", [4, 8])
def test_soap_lowbit_state_fields_and_blocks(bits):
    w = nn.Parameter(torch.randn(96, 80))
    v = nn.Parameter(torch.randn(40))
    opt = SOAPLowBit([w, v], lr=1e-2, precondition_frequency=2, max_precond_dim=64, bits=bits, distributed=False)
    for _ in range(4):
        w.grad, v.grad = torch.randn(96, 80), torch.randn(40)
        opt.step()
    st = opt.state[w]
    for key in ("step", "exp_avg", "exp_avg_sq", "orig_2d_shape", "num_blocks_row", "num_blocks_col", "block_size",
                "QL_q_blocks", "QR_q_blocks", "block_shapes", "L_blocks", "R_blocks"):
        assert key in st, key
    assert (st["num_blocks_row"], st["num_blocks_col"]) == (2, 2) and len(st["QL_q_blocks"]) == 4
    codes, scale, zp, cols = st["QL_q_blocks"][0]
    assert codes.dtype == torch.uint8 and cols == 64 and len(st["QL_q_blocks"][0]) == 4
    assert st["exp_avg"].dtype == torch.uint8 and "exp_avg_absmax" in st      # 7680 elements, block 64
    assert "orig_2d_shape" not in opt.state[v]
    ql = opt._dequantize_block(*st["QL_q_blocks"][0])
    assert (ql.T @ ql - torch.eye(64)).abs().max() < (0.6 if bits == 4 else 0.05)


def test_soap_lowbit_flat_shard_with_orig_shape():
    flat = nn.Parameter(torch.randn(32 * 16))
    flat._orig_2d_shape = (32, 16)
    opt = SOAPLowBit([flat], lr=1e-2, bits=8, distributed=False, max_precond_dim=64)
    flat.grad = torch.randn(32 * 16)
    opt.step()
    assert opt.state[flat]["orig_2d_shape"] == (32, 16)


def test_soap_lowbit_converges():
    torch.manual_seed(0)
    w = nn.Parameter(torch.zeros(128, 64))
    target = torch.randn(128, 64)
    opt = SOAPLowBit([w], lr=3e-2, precondition_frequency=5, bits=8, weight_decay=0.0, distributed=False)
    l0 = (w - target).pow(2).mean().item()
    for _ in range(150):
        opt.zero_grad()
        loss = (w - target).pow(2).mean()
        loss.backward()
        opt.step()
    assert loss.item() < 0.05 * l0


def test_lr_schedules():
    assert lr_multiplier("cosine", 0, 100, 10) == 0 and lr_multiplier("cosine", 5, 100, 10) == 0.5
    assert abs(lr_multiplier("cosine", 10, 100, 10) - 1.0) < 1e-9 and abs(lr_multiplier("cosine", 100, 100, 10) - 0.1) < 1e-9
    assert abs(lr_multiplier("cosine", 55, 100, 10) - 0.55) < 1e-9
    assert abs(lr_multiplier("linear", 55, 100, 10) - 0.55) < 1e-9 and lr_multiplier("linear", 100, 100, 10) == 0.1
    assert lr_multiplier("constant_with_warmup", 50, 100, 10) == 1.0
    opt = AdamW([nn.Parameter(torch.zeros(1))], lr=1.0)
    sch = get_lr_scheduler(opt, "cosine", 100, 10)
    lrs = []
    for _ in range(12):
        opt.step(); sch.step(); lrs.append(sch.get_last_lr()[0])
    assert abs(lrs[4] - 0.5) < 1e-9 and abs(lrs[9] - 1.0) < 1e-9
    with pytest.raises(ValueError):
        get_lr_scheduler(opt, "bogus", 10, 1)


def test_coverage_report(capsys):
    net = Net(64)
    rep = analyze_preconditioning_coverage(net, 64)
    assert rep["num_2d"] == 3 and rep["num_blocks"] == 1 + 2 + 2
    print_preconditioning_stats(net, 64)
    assert "multi-block" in capsys.readouterr().out


def test_quadratic_convergence_all_types():
    for ot in OptimizerType:
        torch.manual_seed(1)
        x = nn.Parameter(torch.randn(64, 64) * 3.0)
        opt = create_optimizer([("w", x)], OptimizerConfig(ot, learning_rate=0.1, weight_decay=0.0, max_precond_dim=64))
        for _ in range(100):
            opt.zero_grad()
            (x ** 2).mean().backward()
            opt.step()
        assert x.abs().mean().item() < 2.0, ot   # starts near 2.4
