"""tcgen05 attention kernels against fp32 oracles: dense causal, sliding window, compressed
keys (affine key positions), selected blocks, importance pass, full three-branch NSA."""
import pytest
import torch

from nsa_optim_b200.ops import oracle, torch_impl

pytestmark = pytest.mark.gpu


def close(a, b, name, rtol=3e-2, atol=2e-2):
    err, scale = (a.float() - b.float()).abs().max().item(), b.float().abs().max().item()
    assert err <= rtol * scale + atol, (name, err, scale)


def mk(B, T, Hq, Hkv, D, S=None):
    S = S or T
    q = torch.randn(B, T, Hq, D, device="cuda").bfloat16()
    k = torch.randn(B, S, Hkv, D, device="cuda").bfloat16()
    v = torch.randn(B, S, Hkv, D, device="cuda").bfloat16()
    return q, k, v


def run_pair(fn_native, fn_ref, tensors):
    leaves = [t.clone().requires_grad_() for t in tensors]
    o = fn_native(*leaves)
    do = torch.randn_like(o)
    o.backward(do)
    refs = [t.float().clone().requires_grad_() for t in tensors]
    o_ref = fn_ref(*refs)
    o_ref.backward(do.float())
    close(o, o_ref, "out")
    for i, (a, b) in enumerate(zip(leaves, refs)):
        close(a.grad, b.grad, f"grad{i}")


@pytest.mark.parametrize("B,T,Hq,Hkv,D", [(2, 300, 4, 2, 64), (1, 1000, 8, 1, 128), (1, 257, 32, 2, 128), (2, 128, 2, 2, 64)])
def test_dense_causal(native, B, T, Hq, Hkv, D):
    run_pair(lambda q, k, v: native.attention(q, k, v, True, 0),
             lambda q, k, v: oracle.attention(q, k, v, True, 0), mk(B, T, Hq, Hkv, D))


@pytest.mark.parametrize("T,W", [(700, 100), (1500, 512), (65, 64)])
def test_sliding_window(native, T, W):
    run_pair(lambda q, k, v: native.attention(q, k, v, True, W),
             lambda q, k, v: oracle.attention(q, k, v, True, W), mk(1, T, 8, 2, 128))


def _cmp_ref(q, kc, vc, stride, block):
    B, T, Hq, D = q.shape
    G = Hq // kc.shape[2]
    s = torch.einsum("bthd,bchd->bhtc", q, kc.repeat_interleave(G, 2)) * D ** -0.5
    end = torch.arange(kc.shape[1], device=q.device) * stride + block - 1
    vis = end[None, :] <= torch.arange(T, device=q.device)[:, None]
    p = torch.nan_to_num(torch.softmax(s.masked_fill(~vis, float("-inf")), -1), nan=0.0)
    return torch.einsum("bhtc,bchd->bthd", p, vc.repeat_interleave(G, 2)), p


def test_compressed_branch_and_importance(native):
    B, T, Hq, Hkv, D, stride, block = 1, 900, 8, 2, 128, 16, 32
    q, k, v = mk(B, T, Hq, Hkv, D)
    kc, vc = torch_impl.nsa_compress(k, block, stride), torch_impl.nsa_compress(v, block, stride)
    run_pair(lambda q, kc, vc: native._Attn.apply(q, kc, vc, True, 0, D ** -0.5, stride, block - 1, None)[0],
             lambda q, kc, vc: _cmp_ref(q, kc, vc, stride, block)[0], (q, kc, vc))
    o, L = native._Attn.apply(q, kc, vc, True, 0, D ** -0.5, stride, block - 1, None)
    nS = -(-T // 64)
    imp = native.nsa_importance(q, kc, L, nS, stride, block, D ** -0.5)
    _, p = _cmp_ref(q.float(), kc.float(), vc.float(), stride, block)
    G = Hq // Hkv
    pg = p.view(B, Hkv, G, T, -1).sum(2)
    w = oracle.nsa_importance_weights(kc.shape[1], nS, block, stride, 64, device="cuda")
    close(imp, pg @ w, "importance", rtol=3e-2, atol=3e-2)


def _sel_ref(q, k, v, idx):
    B, T, Hq, D = q.shape
    Hkv = k.shape[2]
    G = Hq // Hkv
    nS = -(-T // 64)
    m = torch.zeros(B, Hkv, T, nS + 1, dtype=torch.bool, device=q.device)
    m.scatter_(-1, torch.where(idx < 0, torch.full_like(idx, nS), idx).long(), True)
    tok = m[..., :nS].repeat_interleave(64, -1)[..., :T]
    t = torch.arange(T, device=q.device)
    tok = tok & (t[None, :] <= t[:, None])
    s = torch.einsum("bthd,bshd->bhts", q, k.repeat_interleave(G, 2)) * D ** -0.5
    s = s.masked_fill(~tok.repeat_interleave(G, 1), float("-inf"))
    return torch.einsum("bhts,bshd->bthd", torch.softmax(s, -1), v.repeat_interleave(G, 2))


@pytest.mark.parametrize("Hq,Hkv,D", [(32, 2, 128), (4, 2, 64)])
def test_selected_blocks(native, Hq, Hkv, D):
    B, T, top_n = 1, 600, 5
    q, k, v = mk(B, T, Hq, Hkv, D)
    nS = -(-T // 64)
    t = torch.arange(T, device="cuda")
    own = (t // 64)[None, None, :, None]
    rnd = torch.randint(0, nS, (B, Hkv, T, top_n - 1), device="cuda")
    rnd = torch.where(rnd <= own, rnd, -torch.ones_like(rnd))
    idx = torch.cat([own.expand(B, Hkv, T, 1), rnd], -1).to(torch.int32)
    run_pair(lambda q, k, v: native.selected_attention(q, k, v, idx),
             lambda q, k, v: _sel_ref(q, k, v, idx), (q, k, v))


def test_full_nsa_close_to_streaming_reference(native):
    B, T, Hq, Hkv, D = 1, 1024, 16, 2, 128
    q, k, v = mk(B, T, Hq, Hkv, D)
    g = torch.rand(3, B, T, Hq, device="cuda").bfloat16()
    kw = dict(cmp_block=32, cmp_stride=16, sel_block=64, top_n=4, window=128)
    o = native.nsa_attention(q, k, v, g[0], g[1], g[2], **kw)
    ref = torch_impl.nsa_attention(q.float(), k.float(), v.float(), g[0].float(), g[1].float(), g[2].float(), **kw)
    # selection may differ on near-ties; require agreement on the bulk of the rows
    err = (o.float() - ref).abs().amax(dim=(-1, -2))
    assert (err < 0.05).float().mean() > 0.9, err.mean().item()


def test_backward_atomic_path_still_matches(native, monkeypatch):
    """head_dim 128 normally takes the split backward (dQ kernel + key-stationary dK/dV kernel);
    the single-kernel backward with per-tile reductions stays as the fallback for other shapes."""
    monkeypatch.setenv("NSA_B200_ATTN_BWD", "atomic")
    run_pair(lambda q, k, v: native.attention(q, k, v, True, 0),
             lambda q, k, v: oracle.attention(q, k, v, True, 0), mk(1, 500, 8, 1, 128))


@pytest.mark.parametrize("D", [64, 128])
def test_gate_combine_matches_torch(native, D):
    torch.manual_seed(1)
    rows_shape = (2, 37, 5)
    o = [torch.randn(*rows_shape, D, device="cuda").bfloat16().requires_grad_(True) for _ in range(3)]
    g = [torch.rand(*rows_shape, device="cuda").bfloat16().requires_grad_(True) for _ in range(3)]
    out = native._GateCombine.apply(*o, *g)
    ref = sum(gi.float().unsqueeze(-1) * oi.float() for gi, oi in zip(g, o))
    assert torch.allclose(out.float(), ref, atol=2e-2, rtol=2e-2)
    w = torch.randn_like(out)
    grads = torch.autograd.grad(out, o + g, w)
    refs = torch.autograd.grad(ref, o + g, w.float())
    for a, b in zip(grads, refs):
        assert torch.allclose(a.float(), b.float(), atol=3e-2 * max(1.0, b.abs().max().item()), rtol=3e-2)


@pytest.mark.parametrize("T,top_n", [(700, 5), (64 * 40, 16), (100, 16)])
def test_block_selection_kernel_matches_topk(native, T, top_n):
    """The warp-per-row selection against the torch.topk form: same set of blocks per row
    (random importances have no ties)."""
    torch.manual_seed(2)
    nS = -(-T // 64)
    imp = torch.rand(2, 2, T, nS, device="cuda")
    got = native.nsa_select(imp, 64, top_n)
    want = native._nsa_select_torch(imp, 64, top_n)
    assert got.shape == want.shape and got.dtype == torch.int32
    assert torch.equal(got.sort(-1).values, want.sort(-1).values)
    # forced blocks first, never a future block
    t = torch.arange(T, device="cuda")
    assert (got[..., 0] == 0).all() and (got.max(-1).values <= (t // 64)).all()


def _chunked_fp32_attention(q, k, v, causal=True, q_chunk=2048):
    """fp32 softmax attention evaluated per query chunk (no T x T matrix at once)."""
    B, T, Hq, D = q.shape
    G = Hq // k.shape[2]
    kh = k.float().permute(0, 2, 1, 3)[:, :, None]            # B,Hkv,1,T,D
    vh = v.float().permute(0, 2, 1, 3)[:, :, None]
    outs = []
    for s0 in range(0, T, q_chunk):
        s1 = min(T, s0 + q_chunk)
        qc = q[:, s0:s1].float().reshape(B, s1 - s0, -1, G, D).permute(0, 2, 3, 1, 4)
        sc = torch.matmul(qc, kh[:, :, :, :s1].transpose(-1, -2)) * D ** -0.5
        vis = torch.arange(s1, device=q.device)[None, :] <= torch.arange(s0, s1, device=q.device)[:, None]
        sc = sc.masked_fill(~vis, float("-inf"))
        outs.append(torch.matmul(torch.softmax(sc, -1), vh[:, :, :, :s1]).permute(0, 3, 1, 2, 4).reshape(B, s1 - s0, Hq, D))
    return torch.cat(outs, 1)


def test_dense_causal_at_16k_against_chunked_fp32(native):
    """Long rows: the online-softmax rescale chain is 256 visits long at T = 16384."""
    B, T, Hq, Hkv, D = 1, 16384, 32, 2, 128
    q, k, v = mk(B, T, Hq, Hkv, D)
    ql, kl, vl = (t.clone().requires_grad_() for t in (q, k, v))
    o = native.attention(ql, kl, vl, True, 0)
    do = torch.randn_like(o)
    o.backward(do)
    qr, kr, vr = (t.float().clone().requires_grad_() for t in (q, k, v))
    o_ref = _chunked_fp32_attention(qr, kr, vr)
    o_ref.backward(do.float())
    close(o, o_ref, "out", rtol=2e-2, atol=1e-2)
    # late rows average over thousands of keys: compare them on their own scale as well
    close(o[:, -2048:], o_ref[:, -2048:], "late rows", rtol=3e-2, atol=2e-3)
    for name, a, b in (("dq", ql, qr), ("dk", kl, kr), ("dv", vl, vr)):
        close(a.grad, b.grad, name)


def test_attention_forward_and_backward_repeat_bit_for_bit(native):
    """Same inputs twice -> the same bits, forward and the split (dQ pass + key-stationary dK/dV pass)
    backward: no reduction in these kernels depends on scheduling order."""
    q, k, v = mk(1, 2048, 32, 2, 128)
    do = torch.randn(1, 2048, 32, 128, device="cuda").bfloat16()
    results = []
    for _ in range(2):
        ql, kl, vl = (t.clone().requires_grad_() for t in (q, k, v))
        o = native.attention(ql, kl, vl, True, 0)
        o.backward(do)
        results.append((o.detach(), ql.grad, kl.grad, vl.grad))
    for a, b in zip(*results):
        assert torch.equal(a, b)
    nS = 2048 // 64
    t = torch.arange(2048, device="cuda")
    own = (t // 64)[None, None, :, None]
    rnd = torch.randint(0, nS, (1, 2, 2048, 7), device="cuda")
    idx = torch.cat([own.expand(1, 2, 2048, 1), torch.where(rnd <= own, rnd, -torch.ones_like(rnd))], -1).to(torch.int32)
    results = []
    for _ in range(2):
        ql, kl, vl = (t_.clone().requires_grad_() for t_ in (q, k, v))
        o = native.selected_attention(ql, kl, vl, idx)
        o.backward(do)
        results.append((o.detach(), ql.grad, kl.grad, vl.grad))
    for a, b in zip(*results):
        assert torch.equal(a, b)


def test_two_branch_nsa_over_given_block_lists(native):
    """The reference module's form: selected blocks chosen outside the attention op + sliding window."""
    B, T, Hq, Hkv, D, top_n = 1, 700, 32, 2, 128, 6
    q, k, v = mk(B, T, Hq, Hkv, D)
    nS = -(-T // 64)
    own = (torch.arange(T, device="cuda") // 64)[None, None, :, None]
    rnd = torch.randint(0, nS, (B, Hkv, T, top_n - 1), device="cuda")
    idx = torch.cat([own.expand(B, Hkv, T, 1), torch.where(rnd <= own, rnd, -torch.ones_like(rnd))], -1).to(torch.int32)
    g1 = torch.rand(B, T, Hq, device="cuda").bfloat16()
    g2 = torch.rand(B, T, Hq, device="cuda").bfloat16()
    run_pair(lambda q, k, v: native.nsa_attention_indexed(q, k, v, idx, g1, g2, 64, 128),
             lambda q, k, v: torch_impl.nsa_attention_indexed(q, k, v, idx, g1.float(), g2.float(), 64, 128), (q, k, v))


@pytest.mark.parametrize("T,nS,n", [(3000, 47, 16), (64, 1, 4), (5000, 2100, 8)])
def test_inverse_selection_map_kernels_match_the_sort_based_form(native, T, nS, n):
    """count -> scan -> fill against the stable-sort construction, with unused (-1), out-of-range and
    repeated entries in the lists."""
    B, Hkv, R, vpc = 2, 2, 8, 4
    idx = torch.randint(-1, nS + 1, (B, Hkv, T, n), device="cuda", dtype=torch.int32)      # nS itself is out of range
    idx[..., 1] = idx[..., 0]                                                              # a repeat in every list
    tok, ls, its, _, bound = native.inverse_blocks(idx, nS, R, vpc)
    tok_r, ls_r, its_r, _, bound_r = native._inverse_blocks_torch(idx, nS, R, vpc)
    assert torch.equal(ls, ls_r) and torch.equal(its, its_r) and bound == bound_r
    total = int(ls_r[-1])
    assert torch.equal(tok[:total], tok_r[:total])
    tok2, ls2, _, _, _ = native.inverse_blocks(idx, nS, R, vpc)                            # and the same bits again
    assert torch.equal(tok2[:total], tok[:total]) and torch.equal(ls2, ls)
