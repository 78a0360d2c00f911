"""Device-agnostic PyTorch implementations of the framework's ops.

This is the ``torch`` backend: chunked / streaming formulations that run on CPU (gloo
plumbing, unit tests) and on a GPU as the library-kernel comparison path.  Every function
is differentiable by autograd except where a custom ``autograd.Function`` is spelled out
(fused linear + cross-entropy).  The native sm_100a kernels in ``ops/csrc`` implement the
same signatures; ``ops/__init__.py`` picks between them.

Chunked algorithms implemented here:
  * Mamba-2 SSD: intra-chunk masked (C B^T o decay) x + inter-chunk state passing.
  * gated delta rule: per 64-token chunk, WY representation through a unit-lower
    triangular solve, then a sequential pass over chunks that carries the K x V state.
  * native sparse attention: query-chunked compressed attention that never builds a
    (T x T/stride) score tensor for the whole sequence, streaming top-n selection,
    gathered selected-block attention and banded sliding-window attention.
  * linear + cross-entropy over token chunks without materialising (T, V) logits.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F
from torch import Tensor

from . import oracle

# ------------------------------------------------------------------ simple ops
rms_norm = oracle.rms_norm
gated_rms_norm = oracle.gated_rms_norm


def rms_norm_skip(x: Tensor, weight: Tensor, eps: float = 1e-6):
    """(rmsnorm(x) * weight, x): the second value continues the residual stream."""
    return rms_norm(x, weight, eps), x


def add_rms_norm(x: Tensor, r: Tensor, weight: Tensor, eps: float = 1e-6):
    """(h, rmsnorm(h) * weight) with h = x + r."""
    h = x + r
    return h, rms_norm(h, weight, eps)
swiglu = oracle.swiglu
l2_norm = oracle.l2_norm
rope = oracle.rope
causal_conv1d = oracle.causal_conv1d


def linear(x: Tensor, weight: Tensor) -> Tensor:
    return F.linear(x, weight)


def embedding(ids: Tensor, weight: Tensor) -> Tensor:
    return F.embedding(ids, weight)


# ------------------------------------------------------------------ dense / windowed attention
def attention(q: Tensor, k: Tensor, v: Tensor, causal: bool = True, window: int = 0,
              scale: Optional[float] = None) -> Tensor:
    """(B, T, H, D) softmax attention.  Dense causal goes through SDPA; the windowed form is
    evaluated per query chunk against the band of keys it can see."""
    B, T, Hq, D = q.shape
    Hkv = k.shape[2]
    scale = D ** -0.5 if scale is None else scale
    S = k.shape[1]
    if S != T:
        # queries are the last T positions of an S-long key sequence (KV-cache decoding)
        return oracle.attention(q, k, v, causal, window, scale)
    if window <= 0 or window >= T:
        qh, kh, vh = (t.permute(0, 2, 1, 3) for t in (q, k, v))
        if Hq != Hkv:
            kh = kh.repeat_interleave(Hq // Hkv, dim=1)
            vh = vh.repeat_interleave(Hq // Hkv, dim=1)
        o = F.scaled_dot_product_attention(qh, kh, vh, is_causal=causal and T > 1, scale=scale)
        return o.permute(0, 2, 1, 3)
    G = Hq // Hkv
    chunk = max(window, 256)
    outs = []
    for s0 in range(0, T, chunk):
        s1 = min(T, s0 + chunk)
        k0 = max(0, s0 - window + 1)
        qc = q[:, s0:s1].reshape(B, s1 - s0, Hkv, G, D).permute(0, 2, 3, 1, 4)     # B,Hkv,G,tq,D
        kc = k[:, k0:s1].permute(0, 2, 1, 3)[:, :, None]                           # B,Hkv,1,tk,D
        vc = v[:, k0:s1].permute(0, 2, 1, 3)[:, :, None]
        sc = torch.matmul(qc, kc.transpose(-1, -2)).float() * scale
        ti = torch.arange(s0, s1, device=q.device)[:, None]
        si = torch.arange(k0, s1, device=q.device)[None, :]
        m = (si <= ti) & (si > ti - window) if causal else (si > ti - window)
        sc = sc.masked_fill(~m, float("-inf"))
        p = torch.softmax(sc, -1).to(q.dtype)
        oc = torch.matmul(p, vc)                                                   # B,Hkv,G,tq,D
        outs.append(oc.permute(0, 3, 1, 2, 4).reshape(B, s1 - s0, Hq, D))
    return torch.cat(outs, 1)


# ------------------------------------------------------------------ native sparse attention
def nsa_compress(x: Tensor, block: int, stride: int) -> Tensor:
    """(B, T, H, D) -> (B, nC, H, D) mean pooling over windows [i*stride, i*stride+block)."""
    B, T, H, D = x.shape
    if T < block:
        return x.new_zeros(B, 0, H, D)
    xt = x.permute(0, 2, 3, 1).reshape(B, H * D, T)
    y = F.avg_pool1d(xt.float(), kernel_size=block, stride=stride)
    return y.to(x.dtype).reshape(B, H, D, -1).permute(0, 3, 1, 2)


def selected_attention(q: Tensor, k: Tensor, v: Tensor, idx: Tensor, sel_block: int = 64,
                       scale: Optional[float] = None, q_chunk: int = 1024) -> Tensor:
    """Causal attention of every query over its own list of key blocks.  q (B,T,Hq,D), k/v (B,T,Hkv,D),
    idx (B,Hkv,T,n) block numbers (-1 = unused); the heads of a GQA group share a list."""
    B, T, Hq, D = q.shape
    Hkv = k.shape[2]
    G = Hq // Hkv
    scale = D ** -0.5 if scale is None else scale
    kh, vh = k.permute(0, 2, 1, 3).float(), v.permute(0, 2, 1, 3).float()
    blk = torch.arange(T, device=q.device) // sel_block
    outs = []
    for s0 in range(0, T, q_chunk):
        s1 = min(T, s0 + q_chunk)
        qc = q[:, s0:s1].reshape(B, s1 - s0, Hkv, G, D).permute(0, 2, 3, 1, 4).float()      # B,Hkv,G,tq,D
        sc = torch.matmul(qc, kh[:, :, None].transpose(-1, -2)) * scale                     # B,Hkv,G,tq,T
        chosen = (idx[:, :, s0:s1, :, None] == blk[None, None, None, None, :]).any(3)       # B,Hkv,tq,T
        causal = torch.arange(T, device=q.device)[None, :] <= torch.arange(s0, s1, device=q.device)[:, None]
        sc = sc.masked_fill(~(chosen & causal)[:, :, None], float("-inf"))
        p = torch.nan_to_num(torch.softmax(sc, -1), nan=0.0)
        outs.append(torch.matmul(p, vh[:, :, None]).permute(0, 3, 1, 2, 4).reshape(B, s1 - s0, Hq, D))
    return torch.cat(outs, 1).to(q.dtype)


def nsa_attention_indexed(q: Tensor, k: Tensor, v: Tensor, idx: Tensor, g_slc: Tensor, g_swa: Tensor,
                          sel_block: int = 64, window: int = 512, scale: Optional[float] = None) -> Tensor:
    """Selected-block attention over given block lists plus sliding-window attention, combined by
    per-(token, head) gates: the two-branch form of the reference's NativeSparseAttention module."""
    o_slc = selected_attention(q, k, v, idx, sel_block, scale)
    o_swa = attention(q, k, v, True, window, scale)
    return g_slc.unsqueeze(-1) * o_slc + g_swa.unsqueeze(-1) * o_swa


def _importance_band(cmp_block: int, cmp_stride: int, sel_block: int):
    """Offsets and weights of the compressed blocks that overlap selection block j, relative
    to ``j * sel_block / cmp_stride``."""
    r = sel_block // cmp_stride
    span = cmp_block // cmp_stride
    offs, wts = [], []
    for o in range(-(span - 1), r):
        lo, hi = o * cmp_stride, o * cmp_stride + cmp_block
        a, b = max(lo, 0), min(hi, sel_block)
        if b > a:
            offs.append(o)
            wts.append((b - a) / cmp_stride)
    return r, offs, wts


def nsa_importance(p_group: Tensor, n_sel: int, cmp_block: int, cmp_stride: int, sel_block: int) -> Tensor:
    """(…, nC) group-summed compressed probabilities -> (…, n_sel) block importance."""
    r, offs, wts = _importance_band(cmp_block, cmp_stride, sel_block)
    nC = p_group.shape[-1]
    lo_pad = -min(offs)
    need = n_sel * r + max(offs) + 1
    pp = F.pad(p_group, (lo_pad, max(0, need - nC)))
    imp = None
    for o, w in zip(offs, wts):
        sl = pp[..., lo_pad + o: lo_pad + o + n_sel * r: r][..., :n_sel]
        imp = sl * w if imp is None else imp + sl * w
    return imp


def nsa_topk(imp: Tensor, t_idx: Tensor, sel_block: int, top_n: int) -> Tensor:
    """imp (…, tq, nS), t_idx (tq) absolute query positions -> int64 (…, tq, top_n) block ids
    sorted by descending priority; -1 pads rows with fewer visible blocks."""
    nS = imp.shape[-1]
    own = (t_idx // sel_block)[:, None]
    j = torch.arange(nS, device=imp.device)[None, :]
    forced = (j == 0) | (j == own) | (j == own - 1)
    score = torch.where(forced, torch.full_like(imp, float("inf")), imp)
    score = torch.where(j <= own, score, torch.full_like(imp, float("-inf")))
    n = min(top_n, nS)
    order = torch.sort(score, dim=-1, descending=True, stable=True)
    idx, val = order.indices[..., :n], order.values[..., :n]
    idx = torch.where(torch.isinf(val) & (val < 0), torch.full_like(idx, -1), idx)
    if n < top_n:
        idx = F.pad(idx, (0, top_n - n), value=-1)
    return idx


def nsa_attention(q: Tensor, k: Tensor, v: Tensor, g_cmp: Tensor, g_slc: Tensor, g_swa: Tensor,
                  cmp_block: int = 32, cmp_stride: int = 16, sel_block: int = 64, top_n: int = 16,
                  window: int = 512, scale: Optional[float] = None, q_chunk: int = 1024) -> Tensor:
    """Three-branch sparse attention evaluated per query chunk (see ``oracle.nsa_attention``)."""
    B, T, Hq, D = q.shape
    Hkv = k.shape[2]
    G = Hq // Hkv
    scale = D ** -0.5 if scale is None else scale
    kc = nsa_compress(k, cmp_block, cmp_stride)
    vc = nsa_compress(v, cmp_block, cmp_stride)
    nC = kc.shape[1]
    nS = -(-T // sel_block)
    kh = k.permute(0, 2, 1, 3)            # B,Hkv,T,D
    vh = v.permute(0, 2, 1, 3)
    kch = kc.permute(0, 2, 1, 3)          # B,Hkv,nC,D
    vch = vc.permute(0, 2, 1, 3)
    cmp_end = torch.arange(nC, device=q.device) * cmp_stride + cmp_block - 1
    outs = []
    for s0 in range(0, T, q_chunk):
        s1 = min(T, s0 + q_chunk)
        tq = s1 - s0
        t_idx = torch.arange(s0, s1, device=q.device)
        qc = q[:, s0:s1].reshape(B, tq, Hkv, G, D).permute(0, 2, 3, 1, 4)          # B,Hkv,G,tq,D
        # compressed branch (only blocks that end before the chunk's last query can matter)
        n_vis = int((cmp_end <= s1 - 1).sum())
        if n_vis > 0:
            sc = torch.matmul(qc, kch[:, :, None, :n_vis].transpose(-1, -2)).float() * scale
            vis = cmp_end[None, :n_vis] <= t_idx[:, None]
            sc = sc.masked_fill(~vis, float("-inf"))
            p = torch.nan_to_num(torch.softmax(sc, -1), nan=0.0)                   # B,Hkv,G,tq,n_vis
            o_cmp = torch.matmul(p.to(q.dtype), vch[:, :, None, :n_vis])
            with torch.no_grad():
                imp = nsa_importance(p.sum(2), nS, cmp_block, cmp_stride, sel_block)
        else:
            o_cmp = torch.zeros_like(qc)
            imp = torch.zeros(B, Hkv, tq, nS, device=q.device)
        with torch.no_grad():
            idx = nsa_topk(imp, t_idx, sel_block, top_n)                           # B,Hkv,tq,n
            tok = idx.clamp_min(0)[..., None] * sel_block + torch.arange(sel_block, device=q.device)
            ok = (idx >= 0)[..., None] & (tok <= t_idx[None, None, :, None, None]) & (tok < T)
            tok = tok.clamp_max(T - 1).reshape(B, Hkv, tq * top_n * sel_block)
            ok = ok.reshape(B, Hkv, 1, tq, top_n * sel_block)
        # selected branch: gather the chosen key/value rows for each query
        gi = tok[..., None].expand(-1, -1, -1, D)
        ks = torch.gather(kh, 2, gi).reshape(B, Hkv, tq, top_n * sel_block, D)
        vs = torch.gather(vh, 2, gi).reshape(B, Hkv, tq, top_n * sel_block, D)
        ss = torch.einsum("bhgtd,bhtsd->bhgts", qc, ks).float() * scale
        ss = ss.masked_fill(~ok, float("-inf"))
        ps = torch.softmax(ss, -1).to(q.dtype)
        o_slc = torch.einsum("bhgts,bhtsd->bhgtd", ps, vs)
        # sliding-window branch
        k0 = max(0, s0 - window + 1)
        sw = torch.matmul(qc, kh[:, :, None, k0:s1].transpose(-1, -2)).float() * scale
        si = torch.arange(k0, s1, device=q.device)[None, :]
        mw = (si <= t_idx[:, None]) & (si > t_idx[:, None] - window)
        sw = sw.masked_fill(~mw, float("-inf"))
        o_swa = torch.matmul(torch.softmax(sw, -1).to(q.dtype), vh[:, :, None, k0:s1])

        def gate(g):
            return g[:, s0:s1].reshape(B, tq, Hkv, G).permute(0, 2, 3, 1)[..., None].to(o_slc.dtype)

        oc = gate(g_cmp) * o_cmp.to(o_slc.dtype) + gate(g_slc) * o_slc + gate(g_swa) * o_swa
        outs.append(oc.permute(0, 3, 1, 2, 4).reshape(B, tq, Hq, D))
    return torch.cat(outs, 1)


# ------------------------------------------------------------------ Mamba-2 SSD (chunked)
def ssd_scan(x: Tensor, dt: Tensor, A: Tensor, Bm: Tensor, Cm: Tensor, D: Optional[Tensor] = None,
             chunk: int = 256, initial_state: Optional[Tensor] = None, return_state: bool = False):
    """Chunked evaluation of ``oracle.ssd_scan``.  fp32 decays and states, matmuls in the
    input dtype."""
    Bsz, T, H, P = x.shape
    G, N = Bm.shape[2], Bm.shape[3]
    L = min(chunk, T)
    pad = (-T) % L
    if pad:
        x = F.pad(x, (0, 0, 0, 0, 0, pad))
        dt = F.pad(dt, (0, 0, 0, pad))
        Bm = F.pad(Bm, (0, 0, 0, 0, 0, pad))
        Cm = F.pad(Cm, (0, 0, 0, 0, 0, pad))
    Tp = T + pad
    nc = Tp // L
    rep = H // G
    cdt = x.dtype
    xr = x.reshape(Bsz, nc, L, H, P)
    dtr = dt.float().reshape(Bsz, nc, L, H)
    Br = Bm.reshape(Bsz, nc, L, G, N)
    Cr = Cm.reshape(Bsz, nc, L, G, N)
    a = dtr * A.float()[None, None, None, :]                   # (B,nc,L,H) <= 0
    cum = torch.cumsum(a, dim=2)
    total = cum[:, :, -1]                                      # (B,nc,H)
    xdt = (xr.float() * dtr[..., None]).to(cdt)                # (B,nc,L,H,P)
    # intra-chunk: Y[i] = sum_{j<=i} (C_i . B_j) exp(cum_i - cum_j) dt_j x_j
    CB = torch.einsum("bclgn,bcsgn->bcgls", Cr, Br).float()    # (B,nc,G,L,L)
    seg = cum.permute(0, 1, 3, 2)                              # (B,nc,H,L)
    dec = seg[..., :, None] - seg[..., None, :]                # (B,nc,H,L,L)
    tri = torch.ones(L, L, dtype=torch.bool, device=x.device).tril()
    dec = torch.exp(dec.masked_fill(~tri, float("-inf")))
    M = (CB.repeat_interleave(rep, dim=2) * dec).to(cdt)       # (B,nc,H,L,L)
    y = torch.einsum("bchls,bcshp->bclhp", M, xdt)
    # chunk-local end states: S_c = sum_j exp(total - cum_j) dt_j x_j (outer) B_j
    w_end = torch.exp(total[:, :, None, :] - cum)              # (B,nc,L,H)
    Bh = Br.repeat_interleave(rep, dim=3) if rep > 1 else Br   # (B,nc,L,H,N)
    S_loc = torch.einsum("bclhp,bclhn->bchpn", (xdt.float() * w_end[..., None]).to(cdt), Bh).float()
    # inter-chunk pass (sequential over chunks, fp32)
    h = x.new_zeros(Bsz, H, P, N, dtype=torch.float32) if initial_state is None else initial_state.float()
    prev = []
    chunk_decay = torch.exp(total)                             # (B,nc,H)
    for c in range(nc):
        prev.append(h)
        h = h * chunk_decay[:, c][..., None, None] + S_loc[:, c]
    Hprev = torch.stack(prev, 1)                               # (B,nc,H,P,N) state entering chunk c
    Ch = Cr.repeat_interleave(rep, dim=3) if rep > 1 else Cr
    y_inter = torch.einsum("bclhn,bchpn->bclhp", (Ch.float() * torch.exp(cum)[..., None]).to(cdt),
                           Hprev.to(cdt))
    y = (y + y_inter).reshape(Bsz, Tp, H, P)[:, :T]
    if D is not None:
        y = y + (x[:, :T].float() * D.float()[None, None, :, None]).to(cdt)
    y = y.to(cdt)
    return (y, h) if return_state else y


# ------------------------------------------------------------------ gated delta rule (chunked)
def gated_delta_rule(q: Tensor, k: Tensor, v: Tensor, g: Tensor, beta: Tensor,
                     scale: Optional[float] = None, chunk: int = 64,
                     initial_state: Optional[Tensor] = None, return_state: bool = False):
    """Chunkwise evaluation of ``oracle.gated_delta_rule`` (WY representation)."""
    B, T, H, K = q.shape
    V = v.shape[-1]
    scale = K ** -0.5 if scale is None else scale
    C = min(chunk, T)
    pad = (-T) % C
    if pad:
        q, k, v = (F.pad(t, (0, 0, 0, 0, 0, pad)) for t in (q, k, v))
        g, beta = F.pad(g, (0, 0, 0, pad)), F.pad(beta, (0, 0, 0, pad))
    Tp = T + pad
    nc = Tp // C
    f32 = torch.float32
    # (B,H,nc,C,·) layouts, fp32 maths
    qf = q.to(f32).permute(0, 2, 1, 3).reshape(B, H, nc, C, K) * scale
    kf = k.to(f32).permute(0, 2, 1, 3).reshape(B, H, nc, C, K)
    vf = v.to(f32).permute(0, 2, 1, 3).reshape(B, H, nc, C, V)
    gf = g.to(f32).permute(0, 2, 1).reshape(B, H, nc, C)
    bf = beta.to(f32).permute(0, 2, 1).reshape(B, H, nc, C)
    gc = torch.cumsum(gf, -1)                                  # within-chunk cumulative log decay
    diff = gc[..., :, None] - gc[..., None, :]
    lower = torch.ones(C, C, dtype=torch.bool, device=q.device).tril(-1)
    incl = torch.ones(C, C, dtype=torch.bool, device=q.device).tril(0)
    kk = torch.matmul(kf, kf.transpose(-1, -2))
    Amat = (bf[..., None] * kk * torch.exp(diff.masked_fill(~lower, float("-inf"))))
    eye = torch.eye(C, device=q.device, dtype=f32)
    # T = (I + A)^-1 applied to [beta v, beta k exp(gc)]
    rhs = torch.cat([vf * bf[..., None], kf * (bf * torch.exp(gc))[..., None]], -1)
    sol = torch.linalg.solve_triangular(eye + Amat, rhs, upper=False, unitriangular=True)
    u, w = sol[..., :V], sol[..., V:]
    qk = torch.matmul(qf, kf.transpose(-1, -2)) * torch.exp(diff.masked_fill(~incl, float("-inf")))
    q_dec = qf * torch.exp(gc)[..., None]
    k_tail = kf * torch.exp(gc[..., -1:] - gc)[..., None]
    chunk_decay = torch.exp(gc[..., -1])                       # (B,H,nc)
    S = qf.new_zeros(B, H, K, V) if initial_state is None else initial_state.to(f32)
    outs = []
    for c in range(nc):
        v_new = u[:, :, c] - torch.matmul(w[:, :, c], S)
        outs.append(torch.matmul(q_dec[:, :, c], S) + torch.matmul(qk[:, :, c], v_new))
        S = S * chunk_decay[:, :, c][..., None, None] + torch.matmul(k_tail[:, :, c].transpose(-1, -2), v_new)
    o = torch.stack(outs, 2).reshape(B, H, Tp, V).permute(0, 2, 1, 3)[:, :T].to(v.dtype)
    return (o, S) if return_state else o


# ------------------------------------------------------------------ fused linear + CE
class _LinearCrossEntropy(torch.autograd.Function):
    """Token-chunked ``mean CE(h W^T, y)``; gradients are produced during the forward pass so
    that the (chunk, V) logits block is the largest temporary."""

    @staticmethod
    def forward(ctx, hidden: Tensor, weight: Tensor, labels: Tensor, ignore_index: int, chunk: int):
        N, d = hidden.shape
        n_valid = (labels != ignore_index).sum().clamp_min(1)
        need_h, need_w = hidden.requires_grad, weight.requires_grad
        dh = torch.empty_like(hidden) if need_h else None
        dw = torch.zeros(weight.shape, dtype=torch.float32, device=weight.device) if need_w else None
        loss = torch.zeros((), dtype=torch.float32, device=hidden.device)
        inv = 1.0 / n_valid.float()
        for s0 in range(0, N, chunk):
            s1 = min(N, s0 + chunk)
            hc, yc = hidden[s0:s1], labels[s0:s1]
            logits = F.linear(hc, weight).float()
            lse = torch.logsumexp(logits, -1)
            valid = yc != ignore_index
            tgt = logits.gather(1, yc.clamp_min(0)[:, None])[:, 0]
            loss += ((lse - tgt) * valid).sum()
            if need_h or need_w:
                p = torch.exp(logits - lse[:, None])
                p.scatter_add_(1, yc.clamp_min(0)[:, None], -torch.ones_like(p[:, :1]))
                p *= (valid.float() * inv)[:, None]
                pc = p.to(hidden.dtype)
                if need_h:
                    dh[s0:s1] = pc @ weight
                if need_w:
                    dw += (pc.t() @ hc).float()
        ctx.save_for_backward(dh, dw)
        ctx.wdtype = weight.dtype
        return loss * inv

    @staticmethod
    def backward(ctx, gout):
        dh, dw = ctx.saved_tensors
        return (None if dh is None else dh * gout.to(dh.dtype),
                None if dw is None else (dw * gout).to(ctx.wdtype), None, None, None)


def linear_cross_entropy(hidden: Tensor, weight: Tensor, labels: Tensor, ignore_index: int = -100,
                         chunk: int = 4096) -> Tensor:
    return _LinearCrossEntropy.apply(hidden, weight, labels, ignore_index, chunk)
