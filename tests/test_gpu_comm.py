"""Peer-memory kernels on ONE GPU: the W "ranks" are W arenas in the same process and the
kernels of each rank run one after another with flags set beforehand, so no kernel ever waits
for another launch.  Also the bounded-wait path: a flag nobody sets must produce a status code,
not a hang."""
import pytest
import torch

pytestmark = pytest.mark.gpu
W = 4


def make_arenas(payload_bytes, channels=4):
    from nsa_optim_b200.parallel.symm import SymmetricArena, _round_up
    total = _round_up(channels * 32 * 4, 4096) + _round_up(payload_bytes, 4096)
    bufs = [torch.zeros(total, dtype=torch.uint8, device="cuda") for _ in range(W)]
    return [SymmetricArena(payload_bytes, channels, r, W, torch.device("cuda"), local_peers=bufs) for r in range(W)]


def test_signal_allgather_reduce_scatter(native):
    from nsa_optim_b200.parallel import symm
    S = 256 * 40
    arenas = make_arenas(S * 2 + W * S * 4 + 4096)
    off_sh = arenas[0].alloc(S * 2)
    off_g = arenas[0].alloc(W * S * 4)
    for a in arenas[1:]:
        assert a.alloc(S * 2) == off_sh and a.alloc(W * S * 4) == off_g
    shards = [torch.randn(S, device="cuda").bfloat16() for _ in range(W)]
    grads = [torch.randn(W * S, device="cuda") for _ in range(W)]
    for r, a in enumerate(arenas):
        a.view(off_sh, S, torch.bfloat16).copy_(shards[r])
        a.view(off_g, W * S, torch.float32).copy_(grads[r])
        symm.signal(a, 0, 7)
    torch.cuda.synchronize()
    assert all(int(a.flag_row(0)[p]) == 7 for a in arenas for p in range(W))
    ref_full = torch.cat(shards)
    gsum = torch.stack(grads).sum(0)
    for r, a in enumerate(arenas):
        out = torch.empty(W * S, dtype=torch.bfloat16, device="cuda")
        symm.all_gather(a, off_sh, S * 2, out, 0, 7)
        assert torch.equal(out, ref_full)
        gs = torch.ones(S, device="cuda")
        parts = torch.zeros(symm.reduce_scatter_parts(), device="cuda")
        symm.reduce_scatter(a, off_g, gs, 0.25, True, 0, 7, parts)
        want = 1.0 + 0.25 * gsum[r * S:(r + 1) * S]
        assert torch.allclose(gs, want, atol=1e-5)
        assert torch.allclose(parts.sum(), want.pow(2).sum(), rtol=1e-4)
        # fixed rank order inside the kernel: a repeat gives the same bits, shard and partial sums alike
        gs2 = torch.ones(S, device="cuda")
        parts2 = torch.zeros(symm.reduce_scatter_parts(), device="cuda")
        symm.reduce_scatter(a, off_g, gs2, 0.25, True, 0, 7, parts2)
        assert torch.equal(gs, gs2) and torch.equal(parts, parts2)


def test_rs_adamw8bit_matches_unfused(native):
    from nsa_optim_b200.ops import quant
    from nsa_optim_b200.parallel import symm
    S = 256 * 24
    arenas = make_arenas(W * S * 4 + 4096)
    off_g = arenas[0].alloc(W * S * 4)
    for a in arenas[1:]:
        a.alloc(W * S * 4)
    grads = [torch.randn(W * S, device="cuda") for _ in range(W)]
    for r, a in enumerate(arenas):
        a.view(off_g, W * S, torch.float32).copy_(grads[r])
    r = 2
    p0 = torch.randn(S, device="cuda").bfloat16()
    zero_m = int(quant.quantize_blockwise(torch.zeros(256), 8, True, 256)[0][0])
    def state():
        return (torch.full((S,), zero_m, dtype=torch.uint8, device="cuda"), torch.zeros(S // 256, device="cuda"),
                torch.zeros(S, dtype=torch.uint8, device="cuda"), torch.zeros(S // 256, device="cuda"))
    pa, sa = p0.clone(), state()
    pb, sb = p0.clone(), state()
    mask = torch.ones(S // 256, dtype=torch.uint8, device="cuda")
    mask[::3] = 0
    for step in (1, 2):
        symm.rs_adamw8bit(arenas[r], off_g, pa, *sa, mask, 1.0 / W, step, 1e-2, (0.9, 0.95), 1e-8, 0.1, None, 0)
        g = torch.stack(grads).sum(0)[r * S:(r + 1) * S] / W
        for blk_wd, sel in ((0.1, mask.bool()), (0.0, ~mask.bool())):
            idx = sel.repeat_interleave(256)
            pp = pb[idx].clone()
            st = [sb[0][idx].clone(), sb[1][sel].clone(), sb[2][idx].clone(), sb[3][sel].clone()]
            native.adamw8bit_step(pp, g[idx].contiguous(), st[0], st[1], st[2], st[3], step, 1e-2, 0.9, 0.95, 1e-8, blk_wd, None, 256)
            pb[idx] = pp
            sb[0][idx], sb[1][sel], sb[2][idx], sb[3][sel] = st
    # the fused kernel sums the ranks in order before scaling; torch's sum may round differently
    assert (pa.float() - pb.float()).abs().max() < 2e-2
    assert (sa[0] == sb[0]).float().mean() > 0.99 and (sa[2] == sb[2]).float().mean() > 0.99


@pytest.mark.parametrize("which,M", [("pair", 700), ("pair", 4096), ("single", 700)])
def test_gemm_fused_allgather(native, which, M):
    """Both GEMM kernels can gather their own B operand: the CTA-pair kernel copies with the idle
    MMA warp of every odd CTA and sweeps the tiles shard by shard, the single-CTA kernel sets copy
    CTAs aside.  Ranks are emulated inside ONE launch here (copy role and consumers are parts of the
    same resident grid), so nothing waits on another launch."""
    from nsa_optim_b200.parallel import symm
    K, N = 256, 1000 - 1000 % 8
    w_off = 4096                                  # weight starts inside shard 0, spans several shards
    total = 4096 + N * K + 8192
    S = -(-total // (W * 256)) * 256
    arenas = make_arenas(S * 2 + 4096)
    off_sh = arenas[0].alloc(S * 2)
    for a in arenas[1:]:
        a.alloc(S * 2)
    unit = torch.randn(W * S, device="cuda").bfloat16()
    for r, a in enumerate(arenas):
        a.view(off_sh, S, torch.bfloat16).copy_(unit[r * S:(r + 1) * S])
    x = torch.randn(M, K, device="cuda").bfloat16()
    ref = x.float() @ unit[w_off:w_off + N * K].view(N, K).float().t()
    cps = 3
    native.gemm_select(which)
    try:
        for r, a in enumerate(arenas):
            full = torch.zeros(W * S, dtype=torch.bfloat16, device="cuda")
            flags = torch.zeros(W * cps, dtype=torch.int32, device="cuda")
            y = symm.gemm_all_gather(a, x, full, off_sh, S, w_off, N, flags, cps, None, 1, copy_ctas=8)
            assert torch.equal(full, unit)
            assert (y.float() - ref).abs().max().item() <= 1e-2 * ref.abs().max().item() + 1e-2
    finally:
        native.gemm_select("default")


def test_wait_times_out_with_status_not_hang(native):
    from nsa_optim_b200.parallel import symm
    a = make_arenas(4096)[0]
    symm.wait(a, 1, 5, max_cycles=2_000_000)       # nobody signals channel 1: ~1 ms budget
    torch.cuda.synchronize()
    code, block, info, count = native.read_status(reset=True)
    assert code == 201 and info == 5 and count == W
    out = torch.empty(W * 256, dtype=torch.bfloat16, device="cuda")
    symm.all_gather(a, a.alloc(512), 512, out, 2, 9, max_cycles=2_000_000)
    torch.cuda.synchronize()
    code, _, info, _ = native.read_status(reset=True)
    assert code == 201 and info == 9
    # the context is still usable
    assert float(torch.ones(4, device="cuda").sum()) == 4.0
