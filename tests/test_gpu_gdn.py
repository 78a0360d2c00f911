"""Gated delta rule: native sequential state kernels (tcgen05) against the fp32 recurrence."""
import pytest
import torch

from nsa_optim_b200.ops import oracle, torch_impl

pytestmark = pytest.mark.gpu


def _inputs(B, T, H, K, V):
    q = oracle.l2_norm(torch.randn(B, T, H, K, device="cuda")).bfloat16()
    k = oracle.l2_norm(torch.randn(B, T, H, K, device="cuda")).bfloat16()
    v = torch.randn(B, T, H, V, device="cuda").bfloat16()
    g = (-torch.rand(B, T, H, device="cuda") * 0.3)
    beta = torch.rand(B, T, H, device="cuda")
    return q, k, v, g, beta


@pytest.mark.parametrize("T", [64, 200, 512, 4096])
def test_gdn_forward_backward(native, T):
    B, H, K, V = (2 if T <= 512 else 1), 2, 128, 256
    q, k, v, g, beta = _inputs(B, T, H, K, V)
    leaves = [t.clone().requires_grad_() for t in (q, k, v, g, beta)]
    o = native.gated_delta_rule(*leaves)
    do = torch.randn_like(o)
    o.backward(do)
    ref_leaves = [t.float().clone().requires_grad_() for t in (q, k, v, g, beta)]
    o_ref = torch_impl.gated_delta_rule(*ref_leaves, chunk=64)
    o_ref.backward(do.float())
    o_rec = oracle.gated_delta_rule(q, k, v, g, beta)
    assert (o_ref - o_rec.float()).abs().max() < 5e-2 * o_rec.float().abs().max() + 1e-2
    def close(a, b, name):
        err, scale = (a.float() - b.float()).abs().max().item(), b.float().abs().max().item()
        assert err <= 4e-2 * scale + 2e-2, (name, err, scale)
    close(o, o_ref, "o")
    for name, a, b in zip("qkvgb", leaves, ref_leaves):
        close(a.grad, b.grad, "d" + name)
