"""tcgen05 GEMM against an fp32 PyTorch matmul of the same bf16 inputs."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, b, a_mn, b_mn):
    A = a.float().t() if a_mn else a.float()
    B = b.float() if b_mn else b.float().t()
    return A @ B


def _mk(M, N, K, a_mn, b_mn):
    a = torch.randn((K, M) if a_mn else (M, K), device="cuda").bfloat16()
    b = torch.randn((K, N) if b_mn else (N, K), device="cuda").bfloat16()
    return a, b


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("shape", [(128, 256, 64), (256, 512, 256), (1000, 264, 72), (4096, 2048, 1024),
                                   (136, 320, 200), (2048, 8512, 2048), (8512, 2048, 4096)])
def test_gemm_matches_fp32(native, shape, a_mn, b_mn):
    M, N, K = shape
    if (a_mn and M % 8) or (b_mn and N % 8):
        pytest.skip("MN-major operands need a leading dimension that is a multiple of 8")
    a, b = _mk(M, N, K, a_mn, b_mn)
    c = native.gemm(a, b, a_mn, b_mn)
    ref = _ref(a, b, a_mn, b_mn)
    err = (c.float() - ref).abs().max().item()
    scale = ref.abs().max().item()
    assert err <= 1e-2 * scale + 1e-2, (err, scale)


@pytest.mark.parametrize("which", ["single", "pair"])
def test_both_gemm_kernels_agree_with_fp32(native, which):
    """The CTA-pair kernel is the default; the single-CTA kernel stays selectable (and is the one the
    fused all-gather GEMM is built on).  Ragged M, N and K on both."""
    try:
        native.gemm_select(which)
        for (M, N, K) in [(777, 1096, 328), (4096, 5632, 2048)]:
            for a_mn, b_mn in [(False, False), (False, True), (True, True)]:
                if (a_mn and M % 8) or (b_mn and N % 8):
                    continue
                a, b = _mk(M, N, K, a_mn, b_mn)
                c = native.gemm(a, b, a_mn, b_mn)
                ref = _ref(a, b, a_mn, b_mn)
                assert (c.float() - ref).abs().max().item() <= 1e-2 * ref.abs().max().item() + 1e-2, (which, M, N, K)
    finally:
        native.gemm_select("default")


@pytest.mark.parametrize("split_k", [2, 3, 4])
@pytest.mark.parametrize("a_mn,b_mn", [(True, True), (False, False)])
def test_gemm_split_k_through_tma_reduce(native, split_k, a_mn, b_mn):
    """The reduction cut into parts that meet in fp32 through TMA reduce-add stores (weight-gradient
    shapes: few tiles, long K): bf16 and fp32 outputs, with and without accumulation, ragged edges."""
    M, N, K = 520, 776, 4104
    a, b = _mk(M, N, K, a_mn, b_mn)
    ref = _ref(a, b, a_mn, b_mn)
    tol = 1e-2 * ref.abs().max().item() + 1e-2
    c = native.gemm(a, b, a_mn, b_mn, split_k=split_k)
    assert (c.float() - ref).abs().max().item() <= tol
    c32 = torch.ones(M, N, device="cuda")
    native.gemm(a, b, a_mn, b_mn, out=c32, accumulate=True, split_k=split_k)
    assert (c32 - (ref + 1)).abs().max().item() <= tol
    c32 = torch.full((M, N), 7.0, device="cuda")
    native.gemm(a, b, a_mn, b_mn, out=c32, split_k=split_k)
    assert (c32 - ref).abs().max().item() <= tol
    if split_k == 2:                       # two parts into a zeroed C: the same bits whichever lands first
        assert torch.equal(c, native.gemm(a, b, a_mn, b_mn, split_k=2))


def test_split_k_is_chosen_for_the_mlp_weight_gradients(native):
    assert native.split_k_choice(5632, 2048, 65536) == 2 and native.split_k_choice(65536, 8512, 2048) == 1
    a, b = _mk(5632, 2048, 16384, True, True)
    c = native.gemm(a, b, True, True)                  # picks split_k = 2 by itself
    ref = _ref(a, b, True, True)
    assert (c.float() - ref).abs().max().item() <= 1e-2 * ref.abs().max().item() + 1e-2


def test_gemm_is_deterministic(native):
    a, b = _mk(3000, 2048, 1536, False, False)
    c1 = native.gemm(a, b, False, False)
    c2 = native.gemm(a, b, False, False)
    assert torch.equal(c1, c2)


def test_gemm_output_with_odd_pitch_and_bf16_accumulate(native):
    """Outputs a TMA store cannot address (row pitch not a multiple of 16 bytes) or that accumulate
    take the direct-store epilogue."""
    M, N, K = 520, 264, 192
    a, b = _mk(M, N, K, False, False)
    ref = _ref(a, b, False, False)
    base = torch.zeros(M, N + 3, device="cuda", dtype=torch.bfloat16)
    out = base[:, :N]
    native.gemm(a, b, False, False, out=out)
    assert (out.float() - ref).abs().max().item() <= 1e-2 * ref.abs().max().item() + 1e-2
    assert float(base[:, N:].abs().max()) == 0.0
    acc = torch.ones(M, N, device="cuda", dtype=torch.bfloat16)
    native.gemm(a, b, False, False, out=acc, accumulate=True)
    assert (acc.float() - (ref + 1)).abs().max().item() <= 2e-2 * ref.abs().max().item() + 2e-2


def test_gemm_fp32_accumulate(native):
    M, N, K = 512, 384, 320
    a, b = _mk(M, N, K, False, False)
    out = torch.ones(M, N, device="cuda", dtype=torch.float32)
    native.gemm(a, b, False, False, out=out, accumulate=True)
    ref = _ref(a, b, False, False) + 1.0
    assert torch.allclose(out, ref, rtol=1e-3, atol=1e-2)


def test_gemm_many_tiles_persistent(native):
    # more tiles than SMs: exercises the accumulator double-buffering and the stage ring wrap
    M, N, K = 8192, 4096, 512
    a, b = _mk(M, N, K, False, False)
    c = native.gemm(a, b, False, False)
    ref = _ref(a, b, False, False)
    assert (c.float() - ref).abs().max().item() <= 1e-2 * ref.abs().max().item() + 1e-2


def test_gemm_strided_views(native):
    base = torch.randn(300, 1024, device="cuda").bfloat16()
    a = base[:, 256:768]                      # row pitch 1024, width 512
    w = torch.randn(136, 512, device="cuda").bfloat16()
    c = native.gemm(a, w, False, False)
    ref = a.float() @ w.float().t()
    assert (c.float() - ref).abs().max().item() <= 1e-2 * ref.abs().max().item() + 1e-2


def test_linear_autograd(native):
    x = torch.randn(3, 200, 256, device="cuda").bfloat16().requires_grad_()
    w = (torch.randn(384, 256, device="cuda") * 0.05).bfloat16().requires_grad_()
    y = native.linear(x, w)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    wr = w.detach().float().requires_grad_()
    yr = torch.nn.functional.linear(xr, wr)
    yr.backward(g.float())
    for got, ref in ((y, yr), (x.grad, xr.grad), (w.grad, wr.grad)):
        assert (got.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item() + 1e-2


def test_gemm_bf16_accumulate_through_tma_reduce(native):
    """C += A B^T with bf16 C: the pair kernel's epilogue adds its tiles through TMA reduce stores."""
    torch.manual_seed(3)
    M, N, K = 1000, 520, 256
    a = torch.randn(M, K, device="cuda").bfloat16()
    b = torch.randn(N, K, device="cuda").bfloat16()
    c0 = torch.randn(M, N, device="cuda").bfloat16()
    c = c0.clone()
    native.gemm(a, b, False, False, out=c, accumulate=True, split_k=1)
    ref = c0.float() + a.float() @ b.float().t()
    assert (c.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item()
    c2 = c0.clone()
    native.gemm(a, b, False, False, out=c2, accumulate=True, split_k=1)
    assert torch.equal(c, c2)


def test_multi_linear_matches_separate_linears(native):
    torch.manual_seed(4)
    T, d = 700, 256
    x = torch.randn(1, T, d, device="cuda").bfloat16().requires_grad_()
    ws = [torch.randn(n, d, device="cuda").bfloat16().mul(0.05).requires_grad_() for n in (512, 64, 64, 24)]
    gs = [torch.randn(1, T, w.shape[0], device="cuda").bfloat16() for w in ws]
    ys = native.multi_linear(x, ws)
    torch.autograd.backward(ys, gs)
    dx, dws = x.grad.clone(), [w.grad.clone() for w in ws]
    x.grad = None
    for w in ws:
        w.grad = None
    ys2 = [native.linear(x, w) for w in ws]
    torch.autograd.backward(ys2, gs)
    for y, y2 in zip(ys, ys2):
        assert torch.equal(y, y2)
    for dw, w in zip(dws, ws):
        assert torch.equal(dw, w.grad)
    ref = sum(g.float().view(T, -1) @ w.float() for g, w in zip(gs, ws)).view(1, T, d)
    assert (dx.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item() + 1e-2
    assert (x.grad.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item() + 1e-2
