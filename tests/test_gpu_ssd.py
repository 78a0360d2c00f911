"""Mamba-2 SSD on the GPU: native state passing + batched per-chunk terms vs the fp32 recurrence."""
import pytest
import torch

from nsa_optim_b200.ops import oracle, torch_impl

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("T,chunk,P,N", [(300, 256, 64, 128), (512, 64, 64, 128), (129, 128, 64, 128),
                                          (300, 256, 32, 64)])
def test_ssd_forward_backward(native, T, chunk, P, N):
    B, H = 2, 4
    x = torch.randn(B, T, H, P, device="cuda").bfloat16()
    dt = torch.rand(B, T, H, device="cuda") * 0.1 + 0.001
    A = -torch.rand(H, device="cuda") * 4 - 0.5
    Bm = torch.randn(B, T, 1, N, device="cuda").bfloat16() * 0.3
    Cm = torch.randn(B, T, 1, N, device="cuda").bfloat16() * 0.3
    Dp = torch.randn(H, device="cuda")
    if P == 64:      # the mixer hands the kernels strided slices of one projection: exercise that
        packed = torch.cat([x.reshape(B, T, H * P), Bm.reshape(B, T, N), Cm.reshape(B, T, N)], -1).contiguous()
        x = packed[..., :H * P].view(B, T, H, P)
        Bm = packed[..., H * P:H * P + N].view(B, T, 1, N)
        Cm = packed[..., H * P + N:].view(B, T, 1, N)
    leaves = [t.clone().requires_grad_() for t in (x, dt, A, Bm, Cm, Dp)]
    y = native.ssd_scan(*leaves, chunk=chunk)
    dy = torch.randn_like(y)
    y.backward(dy)
    refs = [t.float().clone().requires_grad_() for t in (x, dt, A, Bm, Cm, Dp)]
    y_ref = torch_impl.ssd_scan(*refs, chunk=64)
    y_ref.backward(dy.float())
    y_rec = oracle.ssd_scan(*[t.float() for t in (x, dt, A, Bm, Cm, Dp)])
    def close(a, b, name, rtol=4e-2, atol=3e-2):
        err, scale = (a.float() - b.float()).abs().max().item(), b.float().abs().max().item()
        assert err <= rtol * scale + atol, (name, err, scale)
    close(y_ref, y_rec, "ref-vs-recurrence", 1e-3, 1e-3)
    close(y, y_ref, "y")
    for name, a, b in zip(("dx", "ddt", "dA", "dB", "dC", "dD"), leaves, refs):
        close(a.grad, b.grad, name)


def test_mamba3_forward_scan_matches_loop(native):
    """The forward-only CUDA scan of the complex-state block against the sequential torch loop."""
    from nsa_optim_b200 import ops
    from nsa_optim_b200.models.mamba import mamba3_scan
    torch.manual_seed(0)
    B, L, H, P, N = 2, 300, 3, 16, 40
    x = torch.randn(B, L, H * P, device="cuda")
    dt = torch.rand(B, L, H, device="cuda") * 0.1 + 0.001
    A = torch.stack([-torch.rand(H, N, device="cuda"), torch.randn(H, N, device="cuda") * 0.1], -1)
    Bc, Cc = torch.randn(B, L, H, N, 2, device="cuda"), torch.randn(B, L, H, N, 2, device="cuda")
    D = torch.randn(H, device="cuda")
    with torch.no_grad():
        got = mamba3_scan(x, dt, A, Bc, Cc, D)
        with ops.backend("torch"):
            want = mamba3_scan(x, dt, A, Bc, Cc, D)
    assert torch.allclose(got, want, rtol=1e-3, atol=1e-3 * want.abs().max().item())
