"""Chunked / streaming PyTorch implementations against the naive oracles (CPU, fp32)."""
import pytest
import torch

from nsa_optim_b200.ops import oracle, quant, torch_impl


def test_ssd_chunked_matches_recurrence():
    B, T, H, P, N = 2, 70, 4, 8, 16
    x, dt = torch.randn(B, T, H, P), torch.rand(B, T, H) * 0.5 + 0.01
    A = -torch.rand(H) - 0.1
    Bm, Cm, D = torch.randn(B, T, 1, N), torch.randn(B, T, 1, N), torch.randn(H)
    ref, sref = oracle.ssd_scan(x, dt, A, Bm, Cm, D, return_state=True)
    got, sgot = torch_impl.ssd_scan(x, dt, A, Bm, Cm, D, chunk=16, return_state=True)
    assert torch.allclose(got, ref, atol=1e-4, rtol=1e-4)
    assert torch.allclose(sgot, sref, atol=1e-4, rtol=1e-4)


def test_gated_delta_rule_chunked_matches_recurrence():
    B, T, H, K, V = 2, 50, 3, 16, 24
    q, k = oracle.l2_norm(torch.randn(B, T, H, K)), oracle.l2_norm(torch.randn(B, T, H, K))
    v = torch.randn(B, T, H, V)
    g = -torch.rand(B, T, H) * 0.5
    beta = torch.rand(B, T, H)
    ref, sref = oracle.gated_delta_rule(q, k, v, g, beta, return_state=True)
    got, sgot = torch_impl.gated_delta_rule(q, k, v, g, beta, chunk=16, return_state=True)
    assert torch.allclose(got, ref, atol=1e-4, rtol=1e-3)
    assert torch.allclose(sgot, sref, atol=1e-4, rtol=1e-3)


@pytest.mark.parametrize("T", [1, 63, 64, 65, 257])
def test_nsa_streaming_matches_oracle(T):
    B, Hq, Hkv, D = 1, 4, 2, 16
    q, k, v = torch.randn(B, T, Hq, D), torch.randn(B, T, Hkv, D), torch.randn(B, T, Hkv, D)
    g = torch.rand(3, B, T, Hq)
    kw = dict(cmp_block=8, cmp_stride=4, sel_block=16, top_n=3, window=24)
    ref = oracle.nsa_attention(q, k, v, g[0], g[1], g[2], **kw)
    got = torch_impl.nsa_attention(q, k, v, g[0], g[1], g[2], q_chunk=48, **kw)
    assert torch.allclose(got, ref, atol=1e-4, rtol=1e-4)


def test_nsa_selection_rules():
    T, sel = 128, 16
    p = torch.rand(1, 1, T, (T - 8) // 4 + 1)
    idx = oracle.nsa_select(p, T, 8, 4, sel, 4)
    for t in (0, 15, 16, 100, 127):
        own = t // sel
        chosen = set(idx[0, 0, t].tolist()) - {-1}
        assert 0 in chosen and own in chosen and (own - 1 in chosen or own == 0)
        assert all(j <= own for j in chosen)
    assert (idx[0, 0, 5] == -1).sum() == 3       # only block 0 is visible


def test_importance_band_is_1_2_2_2_1():
    w = oracle.nsa_importance_weights(40, 8, 32, 16, 64)
    assert w[3:8, 1].tolist() == [1, 2, 2, 2, 1] and w[:, 1].sum() == 8


def test_windowed_attention_matches_oracle():
    q, k, v = torch.randn(2, 90, 4, 16), torch.randn(2, 90, 2, 16), torch.randn(2, 90, 2, 16)
    assert torch.allclose(torch_impl.attention(q, k, v, True, 20), oracle.attention(q, k, v, True, 20), atol=1e-5)
    assert torch.allclose(torch_impl.attention(q, k, v, True, 0), oracle.attention(q, k, v, True, 0), atol=1e-5)


def test_linear_cross_entropy_chunked():
    h, w = torch.randn(50, 16, requires_grad=True), torch.randn(40, 16, requires_grad=True)
    y = torch.randint(0, 40, (50,))
    y[::5] = -100
    loss = torch_impl.linear_cross_entropy(h, w, y, -100, 16)
    loss.backward()
    h2, w2 = h.detach().clone().requires_grad_(), w.detach().clone().requires_grad_()
    ref = oracle.linear_cross_entropy(h2, w2, y)
    ref.backward()
    assert torch.allclose(loss, ref, atol=1e-5)
    assert torch.allclose(h.grad, h2.grad, atol=1e-5) and torch.allclose(w.grad, w2.grad, atol=1e-5)


def test_causal_conv1d_is_causal():
    x = torch.randn(1, 20, 8)
    w, b = torch.randn(8, 4), torch.randn(8)
    y = oracle.causal_conv1d(x, w, b)
    x2 = x.clone()
    x2[:, 10:] += 1.0
    y2 = oracle.causal_conv1d(x2, w, b)
    assert torch.equal(y[:, :10], y2[:, :10]) and not torch.equal(y[:, 10:], y2[:, 10:])


def test_rope_preserves_norm_and_relative_phase():
    cos, sin = oracle.rope_tables(16, 32, 1e4)
    x = torch.randn(1, 32, 2, 16)
    y = oracle.rope(x, cos, sin)
    assert torch.allclose(x.norm(dim=-1), y.norm(dim=-1), atol=1e-5)
    q = torch.randn(16).expand(1, 32, 1, 16)
    k = torch.randn(16).expand(1, 32, 1, 16)
    s = (oracle.rope(q, cos, sin)[0, 5:, 0] * oracle.rope(k, cos, sin)[0, :-5, 0]).sum(-1)
    assert torch.allclose(s, s[0].expand_as(s), atol=1e-4)


def test_dynamic_codebooks():
    for signed in (True, False):
        cb = quant.codebook(8, signed, "cpu")
        assert cb.numel() == 256 and torch.all(cb[1:] >= cb[:-1]) and cb.max() == 1.0
        assert (cb.min() < 0) == signed
    x = torch.randn(1024)
    codes, absmax = quant.quantize_blockwise(x, 8, True, 256)
    back = quant.dequantize_blockwise(codes, absmax, 8, True, 256)
    assert (back - x).abs().max() < 0.05 * x.abs().max()
    codes4, am4 = quant.quantize_blockwise(x, 4, True, 64)
    assert codes4.numel() == 512
    assert (quant.dequantize_blockwise(codes4, am4, 4, True, 64) - x).abs().mean() < 0.2


@pytest.mark.parametrize("bits,tol", [(8, 0.01), (4, 0.1)])
def test_affine_roundtrip(bits, tol):
    q_in = torch.linalg.qr(torch.randn(70, 70))[0]
    q, s, z, cols = quant.affine_quantize(q_in, bits, 32)
    assert q.dtype == torch.uint8 and cols == 70 and q.shape == (70, 96)
    back = quant.affine_dequantize(q, s, z, cols)
    assert (back - q_in).abs().max() < tol


def test_inverse_selection_map_lists_tokens_per_block():
    """inverse_blocks: for every (batch, head, block) the ascending tokens that selected it,
    duplicates and invalid entries dropped, plus a CTA bound that covers the work items."""
    from nsa_optim_b200.ops import native
    torch.manual_seed(0)
    B, Hkv, T, n, nS, R, C = 2, 2, 300, 4, 5, 8, 3
    idx = torch.randint(-1, nS, (B, Hkv, T, n), dtype=torch.int32)
    tok, ls, its, ns_out, bound = native.inverse_blocks(idx, nS, R, C)
    assert ns_out == nS and int(its[-1]) <= bound
    for b in range(B):
        for h in range(Hkv):
            for blk in range(nS):
                l = (b * Hkv + h) * nS + blk
                want = [t for t in range(T) if blk in idx[b, h, t].tolist()]
                assert tok[ls[l]:ls[l + 1]].tolist() == want
                assert int(its[l + 1] - its[l]) == -(-(-(-len(want) // R)) // C)


def test_bracket_table_lookup_equals_binary_search():
    """The 8-bit optimizer kernels find the nearest code through a bracket table indexed by the
    value's sign, exponent and top mantissa bits (csrc/codebook.cuh).  This restates that
    arithmetic with numpy integers and checks it against the plain binary search on both code
    books, on random values, every code, every midpoint and the edge cases."""
    import numpy as np
    from nsa_optim_b200.ops import quant
    K_BINS = 386

    def bin_index(x):
        b = x.astype(np.float32).view(np.uint32).astype(np.int64)
        k = ((b & 0x7FFFFFFF) >> 19) - (103 << 4)
        k = np.clip(k, -1, 384)
        return (b >> 31) * K_BINS + k + 1

    def bin_floor(e):
        sign, kk = (e >= K_BINS), (e - K_BINS if e >= K_BINS else e)
        if kk == 0:
            return -2.0 ** -24 if sign else 0.0
        k = kk - 1
        if k == 384:
            return -np.inf if sign else 1.0
        lower = np.array([(k + (103 << 4)) << 19], dtype=np.uint32).view(np.float32)[0]
        upper = np.array([(k + 1 + (103 << 4)) << 19], dtype=np.uint32).view(np.float32)[0]
        return -float(upper) if sign else float(lower)

    def binary(cb, x):
        lo, hi = 0, 255
        while hi - lo > 1:
            mid = (lo + hi) >> 1
            if cb[mid] <= x:
                lo = mid
            else:
                hi = mid
        return lo, hi

    rng = np.random.default_rng(0)
    for signed in (True, False):
        cb = quant.codebook(8, signed, "cpu").numpy().astype(np.float32)
        table = np.array([binary(cb, np.float32(bin_floor(e)))[0] if cb[0] <= bin_floor(e) else 0
                          for e in range(2 * K_BINS)])
        mids = ((cb[:-1].astype(np.float64) + cb[1:]) / 2).astype(np.float32)
        xs = np.concatenate([rng.uniform(-1, 1, 20000), 10.0 ** rng.uniform(-9, 0, 20000) * rng.choice([-1, 1], 20000),
                             cb, mids, np.nextafter(mids, 2), np.nextafter(mids, -2),
                             [0.0, -0.0, 1.0, -1.0, 1e-30, -1e-30, 2.0 ** -24, -2.0 ** -24]]).astype(np.float32)
        if not signed:
            xs = np.abs(xs)
        worst = 0
        for x, e in zip(xs, bin_index(xs)):
            lo, steps = int(table[e]), 0
            assert cb[lo] <= x or lo == 0
            while lo < 254 and cb[lo + 1] <= x:
                lo, steps = lo + 1, steps + 1
            worst = max(worst, steps)
            got = lo if (x - cb[lo] <= cb[lo + 1] - x) else lo + 1
            blo, bhi = binary(cb, x)
            want = blo if (x - cb[blo] <= cb[bhi] - x) else bhi
            assert got == want, (signed, float(x), got, want)
        assert worst <= 8, worst            # the scan stays short where the code book is densest


def test_multi_linear_equals_separate_linears_on_the_torch_backend():
    """``ops.multi_linear`` on CPU tensors is the per-weight ``ops.linear`` (values and gradients)."""
    from nsa_optim_b200 import ops
    torch.manual_seed(0)
    x = torch.randn(2, 5, 16, requires_grad=True)
    ws = [torch.randn(n, 16, requires_grad=True) for n in (8, 24, 3)]
    ys = ops.multi_linear(x, ws)
    assert [tuple(y.shape) for y in ys] == [(2, 5, 8), (2, 5, 24), (2, 5, 3)]
    sum(y.pow(2).sum() for y in ys).backward()
    gx, gws = x.grad.clone(), [w.grad.clone() for w in ws]
    x.grad = None
    for w in ws:
        w.grad = None
    sum(ops.linear(x, w).pow(2).sum() for w in ws).backward()
    assert torch.allclose(gx, x.grad, atol=1e-5)
    for a, w in zip(gws, ws):
        assert torch.allclose(a, w.grad, atol=1e-5)
