"""SOAP on the GPU: the tcgen05 path of ``SOAPLowBit`` (every per-step product a native bf16 GEMM with
fp32 accumulation) against the same optimizer on PyTorch fp32 matmuls and against the
full-precision ``SOAPReference``."""
import pytest
import torch
import torch.nn as nn

from nsa_optim_b200 import ops
from nsa_optim_b200.optimizers import SOAPLowBit, SOAPReference

pytestmark = pytest.mark.gpu


def _problem(rows, cols, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    w0 = torch.randn(rows, cols, device="cuda", generator=g) * 0.02
    # gradients with a decaying spectrum, so that the Kronecker factors have distinct leading directions
    u = torch.linalg.qr(torch.randn(rows, rows, device="cuda", generator=g))[0]
    v = torch.linalg.qr(torch.randn(cols, cols, device="cuda", generator=g))[0]
    sv = torch.logspace(0, -2, min(rows, cols), device="cuda")
    base = (u[:, : sv.numel()] * sv) @ v[:, : sv.numel()].T
    grads = [base + 0.05 * torch.randn(rows, cols, device="cuda", generator=g) for _ in range(8)]
    return w0, grads


def _run(opt_cls, w0, grads, backend, dtype, **kw):
    with ops.backend(backend):
        w = nn.Parameter(w0.clone().to(dtype))
        opt = opt_cls([w], lr=1e-2, weight_decay=0.0, precondition_frequency=3, **kw)
        deltas = []
        for g in grads:
            before = w.detach().float().clone()
            w.grad = g.to(dtype)
            opt.step()
            deltas.append(w.detach().float() - before)
    return w, opt, deltas


def _cos(a, b):
    return float((a * b).sum() / (a.norm() * b.norm() + 1e-30))


@pytest.mark.parametrize("rows,cols,max_dim", [(256, 384, 8192), (512, 320, 256)])
def test_soap_native_gemm_path_matches_the_torch_path(native, rows, cols, max_dim):
    w0, grads = _problem(rows, cols)
    kw = dict(bits=8, max_precond_dim=max_dim, distributed=False, quantize_moments=False)
    _, opt_n, d_n = _run(SOAPLowBit, w0, grads, "auto", torch.bfloat16, **kw)
    _, opt_t, d_t = _run(SOAPLowBit, w0, grads, "torch", torch.bfloat16, **kw)
    for step, (a, b) in enumerate(zip(d_n, d_t)):
        assert _cos(a, b) > 0.98, (step, _cos(a, b))
    st_n, st_t = list(opt_n.state.values())[0], list(opt_t.state.values())[0]
    for Ln, Lt in zip(st_n["L_blocks"], st_t["L_blocks"]):
        assert (Ln - Lt).norm() <= 2e-2 * Lt.norm()                 # bf16 operands, fp32 accumulation
    for Rn, Rt in zip(st_n["R_blocks"], st_t["R_blocks"]):
        assert (Rn - Rt).norm() <= 2e-2 * Rt.norm()


def test_soap_native_step_against_full_precision_reference(native):
    """Update direction and leading eigen-subspaces against ``SOAPReference`` (fp32, unquantised)."""
    rows, cols = 256, 256
    w0, grads = _problem(rows, cols, seed=1)
    _, opt_n, d_n = _run(SOAPLowBit, w0, grads, "auto", torch.bfloat16, bits=8, distributed=False, quantize_moments=False)
    _, opt_r, d_r = _run(SOAPReference, w0, grads, "torch", torch.float32)
    for step, (a, b) in enumerate(zip(d_n, d_r)):
        assert _cos(a, b) > 0.9, (step, _cos(a, b))
    st_n, st_r = list(opt_n.state.values())[0], list(opt_r.state.values())[0]
    QLn = opt_n._dequantize_block(*st_n["QL_q_blocks"][0])
    k = 8
    # largest principal angle between the spans of the k leading basis vectors: cos = sigma_min(Qa^T Qb)
    smin = torch.linalg.svdvals(QLn[:, :k].T @ st_r["QL"][:, :k]).min()
    assert float(smin) > 0.9, float(smin)
