"""Bandwidth-bound kernels, loss and optimizer kernels against the fp32 PyTorch oracles."""
import math

import pytest
import torch
import torch.nn.functional as F

from nsa_optim_b200.ops import oracle, quant, torch_impl

pytestmark = pytest.mark.gpu


def close(got, ref, rtol=2e-2, atol=2e-2):
    err = (got.float() - ref.float()).abs().max().item()
    scale = ref.float().abs().max().item()
    assert err <= rtol * scale + atol, (err, scale)


def bf(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).bfloat16()


@pytest.mark.parametrize("rows,d", [(37, 256), (9, 512), (5, 2048), (3, 4096), (2, 5632)])
def test_rmsnorm(native, rows, d):
    x, w = bf(rows, d).requires_grad_(), (1 + 0.1 * torch.randn(d, device="cuda")).bfloat16().requires_grad_()
    y = native.rms_norm(x, w, 1e-6)
    g = bf(rows, d)
    y.backward(g)
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yr = oracle.rms_norm(xr, wr, 1e-6)
    yr.backward(g.float())
    close(y, yr); close(x.grad, xr.grad); close(w.grad, wr.grad, atol=5e-2)


@pytest.mark.parametrize("rows,d", [(37, 256), (9, 512), (300, 2048), (3, 4096)])
def test_residual_fused_norms_match_the_unfused_block(native, rows, d):
    """norm -> branch -> (add + norm) -> branch -> add, with the adds folded into the norm kernels,
    against the same chain written with plain adds in fp32."""
    x = bf(rows, d).requires_grad_()
    w1 = (1 + 0.1 * torch.randn(d, device="cuda")).bfloat16().requires_grad_()
    w2 = (1 + 0.1 * torch.randn(d, device="cuda")).bfloat16().requires_grad_()
    a, b = bf(d, scale=0.5), bf(d, scale=0.5)             # stand-ins for the mixer and the MLP
    y1, skip = native.rms_norm_skip(x, w1, 1e-6)
    h, y2 = native.add_rms_norm(skip, y1 * a, w2, 1e-6)
    out = h + y2 * b
    g = bf(rows, d)
    out.backward(g)
    xr, w1r, w2r = (t.detach().float().requires_grad_() for t in (x, w1, w2))
    y1r = oracle.rms_norm(xr, w1r, 1e-6)
    hr = xr + y1r * a.float()
    outr = hr + oracle.rms_norm(hr, w2r, 1e-6) * b.float()
    outr.backward(g.float())
    close(out, outr); close(x.grad, xr.grad, rtol=3e-2); close(w1.grad, w1r.grad, atol=5e-2, rtol=3e-2)
    close(w2.grad, w2r.grad, atol=5e-2, rtol=3e-2)
    # the fused forward equals add-then-norm to the bit
    h2 = (x.detach() + (y1 * a).detach())
    assert torch.equal(h.detach(), h2) and torch.equal(y2.detach(), native.rms_norm(h2, w2.detach(), 1e-6))


@pytest.mark.parametrize("nbg", [True, False])
@pytest.mark.parametrize("rows,d", [(40, 256), (6, 4096)])
def test_gated_rmsnorm(native, rows, d, nbg):
    x, gt = bf(rows, d).requires_grad_(), bf(rows, d).requires_grad_()
    w = (1 + 0.1 * torch.randn(d, device="cuda")).bfloat16().requires_grad_()
    y = native.gated_rms_norm(x, gt, w, 1e-5, nbg)
    g = bf(rows, d)
    y.backward(g)
    xr, gr, wr = (t.detach().float().requires_grad_() for t in (x, gt, w))
    yr = oracle.gated_rms_norm(xr, gr, wr, 1e-5, nbg)
    yr.backward(g.float())
    close(y, yr); close(x.grad, xr.grad); close(gt.grad, gr.grad); close(w.grad, wr.grad, atol=5e-2)


@pytest.mark.parametrize("nbg", [True, False])
def test_gated_rmsnorm_with_gate_as_column_slice(native, nbg):
    """The gate is read in place from a slice of a wider matrix (as the Mamba-2 mixer hands it over)."""
    rows, d = 70, 512
    wide = bf(2, rows // 2, 3 * d + 64)
    gate = wide[..., d:2 * d].detach().requires_grad_()
    x = bf(2, rows // 2, d).requires_grad_()
    w = (1 + 0.1 * torch.randn(d, device="cuda")).bfloat16().requires_grad_()
    y = native.gated_rms_norm(x, gate, w, 1e-5, nbg)
    g = bf(2, rows // 2, d)
    y.backward(g)
    xr, gr, wr = (t.detach().float().requires_grad_() for t in (x, gate, w))
    yr = oracle.gated_rms_norm(xr, gr, wr, 1e-5, nbg)
    yr.backward(g.float())
    close(y, yr); close(x.grad, xr.grad); close(gate.grad, gr.grad); close(w.grad, wr.grad, atol=5e-2)


def test_l2norm(native):
    x = bf(2, 33, 4, 128).requires_grad_()
    y = native.l2_norm(x)
    g = bf(2, 33, 4, 128)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    yr = oracle.l2_norm(xr)
    yr.backward(g.float())
    close(y, yr); close(x.grad, xr.grad)


def test_swiglu(native):
    a, b = bf(70, 1536).requires_grad_(), bf(70, 1536).requires_grad_()
    y = native.swiglu(a, b)
    g = bf(70, 1536)
    y.backward(g)
    ar, br = a.detach().float().requires_grad_(), b.detach().float().requires_grad_()
    yr = oracle.swiglu(ar, br)
    yr.backward(g.float())
    close(y, yr); close(a.grad, ar.grad); close(b.grad, br.grad)


@pytest.mark.parametrize("D", [64, 128])
def test_rope(native, D):
    x = bf(2, 50, 3, D).requires_grad_()
    cos, sin = oracle.rope_tables(D, 50, 1e4, device="cuda")
    y = native.rope(x, cos, sin)
    g = bf(2, 50, 3, D)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    yr = oracle.rope(xr, cos, sin)
    yr.backward(g.float())
    close(y, yr); close(x.grad, xr.grad)


@pytest.mark.parametrize("bias", [True, False])
def test_causal_conv1d(native, bias):
    B, T, C = 2, 75, 136
    x = bf(B, T, C).requires_grad_()
    w = bf(C, 4, scale=0.5).requires_grad_()
    b = bf(C, scale=0.5).requires_grad_() if bias else None
    y = native.causal_conv1d(x, w, b, True)
    g = bf(B, T, C)
    y.backward(g)
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    brr = b.detach().float().requires_grad_() if bias else None
    yr = oracle.causal_conv1d(xr, wr, brr, True)
    yr.backward(g.float())
    close(y, yr); close(x.grad, xr.grad); close(w.grad, wr.grad, atol=8e-2)
    if bias:
        close(b.grad, brr.grad, atol=8e-2)


def test_causal_conv1d_many_tiles_and_pitched_input(native):
    """Several time tiles per CTA (double-buffered loads), two time segments, a partial channel tile
    and an input that is a column slice of a wider matrix."""
    B, T, C = 1, 700, 200
    wide = bf(B, T, C + 56)
    x = wide[..., 24:24 + C].detach().requires_grad_()
    w = bf(C, 4, scale=0.5).requires_grad_()
    b = bf(C, scale=0.5).requires_grad_()
    y = native.causal_conv1d(x, w, b, True)
    g = bf(B, T, C)
    y.backward(g)
    xr, wr, brr = (t.detach().float().requires_grad_() for t in (x, w, b))
    yr = oracle.causal_conv1d(xr, wr, brr, True)
    yr.backward(g.float())
    close(y, yr); close(x.grad, xr.grad); close(w.grad, wr.grad, atol=2e-1); close(b.grad, brr.grad, atol=2e-1)


def test_embedding(native):
    w = bf(500, 64).requires_grad_()
    ids = torch.randint(0, 500, (3, 40), device="cuda")
    y = native.embedding(ids, w)
    g = bf(3, 40, 64)
    y.backward(g)
    wr = w.detach().float().requires_grad_()
    yr = F.embedding(ids, wr)
    yr.backward(g.float())
    assert torch.equal(y.float(), yr)
    close(w.grad, wr.grad)


def test_linear_cross_entropy(native):
    N, d, V = 300, 128, 1000
    h = bf(N, d, scale=0.5).requires_grad_()
    w = bf(V, d, scale=0.1).requires_grad_()
    y = torch.randint(0, V, (N,), device="cuda")
    y[::7] = -100
    loss = native.linear_cross_entropy(h, w, y, -100, 128)
    loss.backward()
    hr, wr = h.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    lr = oracle.linear_cross_entropy(hr, wr, y)
    lr.backward()
    assert abs(loss.item() - lr.item()) < 2e-2
    close(h.grad, hr.grad, atol=1e-4, rtol=5e-2); close(w.grad, wr.grad, atol=1e-4, rtol=5e-2)


@pytest.mark.parametrize("pdt", [torch.bfloat16, torch.float32])
def test_adamw_kernel(native, pdt):
    n = 5000
    p = torch.randn(n, device="cuda").to(pdt)
    g = torch.randn(n, device="cuda")
    m, v = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    pr, mr, vr = p.float().clone(), m.clone(), v.clone()
    scale = torch.tensor(0.5, device="cuda")
    for t in (1, 2, 3):
        native.adamw_step(p, g, m, v, None, t, 1e-2, 0.9, 0.95, 1e-8, 0.1, scale)
        oracle.adamw_step(pr, g * 0.5, mr, vr, t, 1e-2, 0.9, 0.95, 1e-8, 0.1)
        if pdt == torch.bfloat16:
            pr = pr.bfloat16().float()
    close(m, mr, 1e-5, 1e-6); close(v, vr, 1e-5, 1e-6); close(p, pr, 1e-2 if pdt == torch.bfloat16 else 1e-5, 1e-5)


def test_adamw8bit_kernel_matches_torch_codec(native):
    n = 256 * 40
    p = torch.randn(n, device="cuda").bfloat16()
    pr = p.clone()
    mq = torch.full((n,), 127, dtype=torch.uint8, device="cuda"); vq = torch.zeros(n, dtype=torch.uint8, device="cuda")
    zero_m = quant.quantize_blockwise(torch.zeros(256), 8, True, 256)[0][0].item()
    mq.fill_(zero_m)
    mabs, vabs = torch.zeros(n // 256, device="cuda"), torch.zeros(n // 256, device="cuda")
    mr, vr = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    for t in (1, 2, 3, 4):
        g = torch.randn(n, device="cuda")
        native.adamw8bit_step(p, g, mq, mabs, vq, vabs, t, 1e-2, 0.9, 0.95, 1e-8, 0.1, None, 256)
        # reference: dequantise the previous reference state through the same codec
        mr = mr * 0.9 + 0.1 * g
        vr = vr * 0.95 + 0.05 * g * g
        w = pr.float() * (1 - 1e-2 * 0.1)
        w = w - (1e-2 / (1 - 0.9 ** t)) * mr / (vr.sqrt() / math.sqrt(1 - 0.95 ** t) + 1e-8)
        pr = w.bfloat16()
        cm, am = quant.quantize_blockwise(mr, 8, True, 256)
        cv, av = quant.quantize_blockwise(vr, 8, False, 256)
        mr = quant.dequantize_blockwise(cm, am, 8, True, 256)
        vr = quant.dequantize_blockwise(cv, av, 8, False, 256)
    md = quant.dequantize_blockwise(mq, mabs, 8, True, 256)
    vd = quant.dequantize_blockwise(vq, vabs, 8, False, 256)
    close(md, mr, 2e-2, 1e-3); close(vd, vr, 2e-2, 1e-3); close(p, pr, 2e-2, 2e-2)


@pytest.mark.parametrize("cols,q_block,bits", [(256, 64, 4), (100, 32, 8), (70, 64, 4)])
def test_affine_block_quant_matches_torch_form(native, cols, q_block, bits):
    """The CUDA affine codec of SOAP's eigenbases against the PyTorch form (same codes, scales, zeros)."""
    from nsa_optim_b200 import ops
    from nsa_optim_b200.ops import quant
    torch.manual_seed(0)
    t = torch.randn(37, cols, device="cuda")
    q, sc, zp, oc = quant.affine_quantize(t, bits, q_block)
    with ops.backend("torch"):
        q2, sc2, zp2, oc2 = quant.affine_quantize(t, bits, q_block)
        back2 = quant.affine_dequantize(q2, sc2, zp2, oc2)
    assert oc == oc2 and torch.allclose(sc, sc2, rtol=1e-6) and torch.equal(zp, zp2)
    assert (q[:, :cols].int() - q2[:, :cols].int()).abs().max() <= 1          # a tie may round either way
    assert (q[:, :cols] != q2[:, :cols]).float().mean() < 1e-3
    back = quant.affine_dequantize(q, sc, zp, oc)
    assert back.shape == (37, cols) and torch.allclose(back, back2, atol=float(sc.max()) * 1.01)
    assert (back - t).abs().max() <= float(sc.max()) * 1.01 + 1e-6


def test_canary_mode_catches_a_write_past_the_output(native, monkeypatch):
    """Debug allocation mode: outputs sit between guard zones; an intact run verifies clean, a byte
    written just past an output is reported."""
    monkeypatch.setattr(native, "_CANARY", True)
    native._guards.clear()
    x = torch.randn(64, 256, device="cuda").bfloat16()
    w = torch.ones(256, device="cuda").bfloat16()
    from nsa_optim_b200 import ops
    y = ops.rms_norm(x, w, 1e-6)
    assert torch.allclose(y.float(), oracle.rms_norm(x.float(), w.float(), 1e-6), atol=3e-2, rtol=3e-2)
    assert native.check_canaries() >= 1
    out = native._empty(16, dtype=torch.float32, device=x.device)
    buf, nbytes = native._guards[-1]
    buf[native._GUARD + nbytes] = 0                 # what a kernel writing one element too far would do
    with pytest.raises(RuntimeError, match="guard zone after"):
        native.check_canaries()
    assert out.numel() == 16


def test_pitched_column_copy(native):
    out = torch.zeros(3, 50, 40, device="cuda").bfloat16()
    g = torch.randn(3, 50, 16, device="cuda").bfloat16()
    assert native.copy_columns(out[..., 8:24], g)
    ref = torch.zeros_like(out)
    ref[..., 8:24] = g
    assert torch.equal(out, ref)
    assert not native.copy_columns(out[..., 8:24], g[:, :, :1].expand(3, 50, 16))     # broadcast source: not a pitched layout


def test_debug_build_reports_out_of_range_indices(tmp_path):
    """-DNSA_DEBUG_BOUNDS: a token id outside the vocabulary is recorded (status 302, the id as detail)
    and the gather continues with the clamped row; nothing faults.  Builds a small debug library
    (two translation units) beside the test and talks to it through ctypes."""
    import ctypes
    from ctypes import c_int, c_long, c_void_p
    from nsa_optim_b200.ops import build
    lib_file = build.build(debug=True, out=str(tmp_path / "libdebug.so"), only=["elementwise.cu"])
    lib = ctypes.CDLL(lib_file)
    vocab, d = 50, 64
    w = bf(vocab, d)
    ids = torch.tensor([3, 49, 77, 0], device="cuda", dtype=torch.long)       # 77 is out of range
    y = torch.empty(4, d, device="cuda", dtype=torch.bfloat16)
    st = c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.nsa_embedding_fwd(c_void_p(ids.data_ptr()), c_void_p(w.data_ptr()), c_void_p(y.data_ptr()), c_long(4), c_int(d),
                                 c_long(vocab), st) == 0
    torch.cuda.synchronize()
    out = (c_int * 4)()
    assert lib.nsa_status_read(out, c_int(1)) == 0
    assert out[0] == 302 and out[2] == 77 and out[3] == 1
    assert torch.equal(y[2], w[49]) and torch.equal(y[0], w[3])               # clamped, and the rest untouched by it
    ids[2] = 5
    lib.nsa_embedding_fwd(c_void_p(ids.data_ptr()), c_void_p(w.data_ptr()), c_void_p(y.data_ptr()), c_long(4), c_int(d),
                          c_long(vocab), st)
    torch.cuda.synchronize()
    lib.nsa_status_read(out, c_int(1))
    assert out[0] == 0
