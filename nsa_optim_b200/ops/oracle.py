"""Plain fp32 PyTorch statements of every op, written for obviousness rather than speed.

These are the numerical oracles: each CUDA kernel and each chunked/streaming torch
implementation is tested against the function of the same name here.  Nothing in this
file is used on a training hot path.

Semantics they pin down (reference project paths):
  * RMSNorm, RoPE (non-interleaved halves), SwiGLU ....... models/kernels.py:47-128
  * causal GQA attention on (B, T, H, D) .................. models/hybrid.py:360-382
  * native sparse attention: compressed / selected / sliding branches and the sigmoid
    gated combine ......................................... models/transformer.py:127-311
    (the reference delegates the kernel; the three-branch algorithm is defined here)
  * Mamba-2 SSD recurrence, causal conv1d + SiLU, gated RMSNorm ... models/mamba.py:65-72
  * gated delta rule recurrence ........................... models/deltanet.py:104-115
  * token-mean cross entropy with ignore_index -100 ....... models/kernels.py:380-423
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F
from torch import Tensor


# ------------------------------------------------------------------ elementwise / norms
def rms_norm(x: Tensor, weight: Tensor, eps: float = 1e-6) -> Tensor:
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (y * weight.float()).to(x.dtype)


def gated_rms_norm(x: Tensor, gate: Tensor, weight: Tensor, eps: float = 1e-6,
                   norm_before_gate: bool = True) -> Tensor:
    """``norm_before_gate=True``: rmsnorm(x)*w*silu(gate)  (Gated DeltaNet output norm).
    ``False``: rmsnorm(x*silu(gate))*w  (Mamba-2 mixer norm)."""
    xf, gf = x.float(), gate.float()
    if norm_before_gate:
        y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * weight.float()
        y = y * F.silu(gf)
    else:
        xf = xf * F.silu(gf)
        y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * weight.float()
    return y.to(x.dtype)


def swiglu(gate: Tensor, up: Tensor) -> Tensor:
    return (F.silu(gate.float()) * up.float()).to(gate.dtype)


def l2_norm(x: Tensor, eps: float = 1e-6) -> Tensor:
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).sum(-1, keepdim=True) + eps)).to(x.dtype)


def rope_tables(head_dim: int, seq_len: int, theta: float, device=None) -> Tuple[Tensor, Tensor]:
    """cos/sin of shape (T, D/2), fp32."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=device) / head_dim))
    ang = torch.outer(torch.arange(seq_len, dtype=torch.float32, device=device), inv)
    return ang.cos(), ang.sin()


def rope(x: Tensor, cos: Tensor, sin: Tensor) -> Tensor:
    """x (B, T, H, D); cos/sin (T, D/2); halves layout: pairs are (x[i], x[i + D/2])."""
    d2 = x.shape[-1] // 2
    xf = x.float()
    x1, x2 = xf[..., :d2], xf[..., d2:]
    c, s = cos[None, :, None, :].float(), sin[None, :, None, :].float()
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).to(x.dtype)


# ------------------------------------------------------------------ attention
def _expand_kv(x: Tensor, groups: int) -> Tensor:
    return x.repeat_interleave(groups, dim=2) if groups > 1 else x


def attention(q: Tensor, k: Tensor, v: Tensor, causal: bool = True, window: int = 0,
              scale: Optional[float] = None) -> Tensor:
    """Softmax attention on (B, T, H, D) tensors, GQA by head grouping.
    ``window`` > 0 keeps keys with ``t - window < s <= t``."""
    B, T, Hq, D = q.shape
    S = k.shape[1]
    g = Hq // k.shape[2]
    scale = D ** -0.5 if scale is None else scale
    qf = q.float().permute(0, 2, 1, 3)
    kf = _expand_kv(k, g).float().permute(0, 2, 1, 3)
    vf = _expand_kv(v, g).float().permute(0, 2, 1, 3)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    ti = torch.arange(T, device=q.device)[:, None] + (S - T)
    si = torch.arange(S, device=q.device)[None, :]
    mask = torch.ones(T, S, dtype=torch.bool, device=q.device)
    if causal:
        mask &= si <= ti
    if window > 0:
        mask &= si > ti - window
    s = s.masked_fill(~mask, float("-inf"))
    p = torch.softmax(s, dim=-1)
    p = torch.nan_to_num(p, nan=0.0)
    return torch.matmul(p, vf).permute(0, 2, 1, 3).to(q.dtype)


# ------------------------------------------------------------------ native sparse attention
def nsa_compress(x: Tensor, block: int, stride: int) -> Tensor:
    """(B, T, H, D) -> (B, nC, H, D): mean of tokens [i*stride, i*stride + block)."""
    B, T, H, D = x.shape
    n = (T - block) // stride + 1 if T >= block else 0
    if n <= 0:
        return x.new_zeros(B, 0, H, D)
    out = [x[:, i * stride:i * stride + block].float().mean(1) for i in range(n)]
    return torch.stack(out, 1).to(x.dtype)


def nsa_importance_weights(n_cmp: int, n_sel: int, cmp_block: int, cmp_stride: int, sel_block: int,
                           device=None) -> Tensor:
    """(n_cmp, n_sel) map from compressed-block probability to selection-block importance:
    entry (i, j) is the number of ``cmp_stride``-sized cells that compressed block i
    shares with selection block j.  For 32/16/64 this is the band (1, 2, 2, 2, 1)."""
    w = torch.zeros(n_cmp, n_sel, device=device)
    for i in range(n_cmp):
        lo, hi = i * cmp_stride, i * cmp_stride + cmp_block
        for j in range(n_sel):
            a, b = max(lo, j * sel_block), min(hi, (j + 1) * sel_block)
            if b > a:
                w[i, j] = (b - a) / cmp_stride
    return w


def nsa_select(p_cmp: Tensor, T: int, cmp_block: int, cmp_stride: int, sel_block: int, top_n: int) -> Tensor:
    """p_cmp (B, Hkv, T, nC): compressed-branch probabilities summed over each GQA group.
    Returns int64 (B, Hkv, T, top_n) selection-block ids, -1 where fewer blocks are visible.
    Block 0, the query's own block and the one before it are always kept; the rest are the
    highest-importance causal blocks; ties resolve to the lower block id."""
    B, H, _, nC = p_cmp.shape
    nS = -(-T // sel_block)
    w = nsa_importance_weights(nC, nS, cmp_block, cmp_stride, sel_block, device=p_cmp.device)
    imp = torch.matmul(p_cmp.float(), w)                       # (B, H, T, nS)
    t = torch.arange(T, device=p_cmp.device)
    own = (t // sel_block)[:, None]
    j = torch.arange(nS, device=p_cmp.device)[None, :]
    visible = j <= own
    forced = (j == 0) | (j == own) | (j == own - 1)
    score = torch.where(forced, torch.full_like(imp, float("inf")), imp)
    score = torch.where(visible, score, torch.full_like(imp, float("-inf")))
    n = min(top_n, nS)
    # stable descending sort => ties keep the lower block id first
    order = torch.sort(score, dim=-1, descending=True, stable=True)
    idx = order.indices[..., :n]
    val = order.values[..., :n]
    idx = torch.where(torch.isinf(val) & (val < 0), torch.full_like(idx, -1), idx)
    if n < top_n:
        idx = F.pad(idx, (0, top_n - n), value=-1)
    return idx


def nsa_attention(q: Tensor, k: Tensor, v: Tensor, g_cmp: Tensor, g_slc: Tensor, g_swa: Tensor,
                  cmp_block: int = 32, cmp_stride: int = 16, sel_block: int = 64, top_n: int = 16,
                  window: int = 512, scale: Optional[float] = None,
                  return_parts: bool = False):
    """Three-branch native sparse attention.  q (B,T,Hq,D), k/v (B,T,Hkv,D), gates (B,T,Hq)
    already passed through a sigmoid.  Output (B,T,Hq,D)."""
    B, T, Hq, D = q.shape
    Hkv = k.shape[2]
    G = Hq // Hkv
    scale = D ** -0.5 if scale is None else scale
    qf = q.float()
    # ---- compressed branch
    kc, vc = nsa_compress(k, cmp_block, cmp_stride).float(), nsa_compress(v, cmp_block, cmp_stride).float()
    nC = kc.shape[1]
    t = torch.arange(T, device=q.device)
    if nC > 0:
        s = torch.einsum("bthd,bchd->bhtc", qf, _expand_kv(kc, G)) * scale
        end = torch.arange(nC, device=q.device) * cmp_stride + cmp_block - 1
        vis = end[None, :] <= t[:, None]
        s = s.masked_fill(~vis, float("-inf"))
        p = torch.nan_to_num(torch.softmax(s, -1), nan=0.0)          # (B,Hq,T,nC)
        o_cmp = torch.einsum("bhtc,bchd->bthd", p, _expand_kv(vc, G))
        p_group = p.view(B, Hkv, G, T, nC).sum(2)
    else:
        o_cmp = torch.zeros_like(qf)
        p_group = qf.new_zeros(B, Hkv, T, 0)
    # ---- selection
    idx = nsa_select(p_group, T, cmp_block, cmp_stride, sel_block, top_n)   # (B,Hkv,T,n)
    nS = -(-T // sel_block)
    blk_mask = torch.zeros(B, Hkv, T, nS + 1, dtype=torch.bool, device=q.device)
    blk_mask.scatter_(-1, torch.where(idx < 0, torch.full_like(idx, nS), idx), True)
    blk_mask = blk_mask[..., :nS]
    tok_mask = blk_mask.repeat_interleave(sel_block, dim=-1)[..., :T]           # (B,Hkv,T,T)
    tok_mask &= (t[None, :] <= t[:, None])
    s = torch.einsum("bthd,bshd->bhts", qf, _expand_kv(k, G).float()) * scale
    s_slc = s.masked_fill(~tok_mask.repeat_interleave(G, dim=1), float("-inf"))
    o_slc = torch.einsum("bhts,bshd->bthd", torch.softmax(s_slc, -1), _expand_kv(v, G).float())
    # ---- sliding window
    o_swa = attention(q, k, v, causal=True, window=window, scale=scale).float()
    out = (g_cmp.float()[..., None] * o_cmp + g_slc.float()[..., None] * o_slc
           + g_swa.float()[..., None] * o_swa)
    if return_parts:
        return out.to(q.dtype), (o_cmp, o_slc, o_swa, idx)
    return out.to(q.dtype)


# ------------------------------------------------------------------ Mamba-2
def causal_conv1d(x: Tensor, weight: Tensor, bias: Optional[Tensor], activation: bool = True) -> Tensor:
    """Depthwise causal convolution over time.  x (B, T, C), weight (C, W), bias (C)."""
    B, T, C = x.shape
    W = weight.shape[-1]
    xf = F.pad(x.float().transpose(1, 2), (W - 1, 0))
    y = F.conv1d(xf, weight.float().view(C, 1, W), None if bias is None else bias.float(), groups=C)
    y = y.transpose(1, 2)
    if activation:
        y = F.silu(y)
    return y.to(x.dtype)


def ssd_scan(x: Tensor, dt: Tensor, A: Tensor, Bm: Tensor, Cm: Tensor, D: Optional[Tensor] = None,
             initial_state: Optional[Tensor] = None, return_state: bool = False):
    """Selective state-space recurrence, one step at a time.
    x (B,T,H,P); dt (B,T,H) positive step sizes; A (H) negative; Bm, Cm (B,T,G,N); D (H).
        h_t = exp(dt_t A) h_{t-1} + dt_t * x_t (outer) B_t ;  y_t = h_t C_t + D x_t"""
    Bsz, T, H, P = x.shape
    G, N = Bm.shape[2], Bm.shape[3]
    rep = H // G
    xf, dtf = x.float(), dt.float()
    Bf = Bm.float().repeat_interleave(rep, dim=2)
    Cf = Cm.float().repeat_interleave(rep, dim=2)
    h = xf.new_zeros(Bsz, H, P, N) if initial_state is None else initial_state.float().clone()
    ys = []
    for t in range(T):
        decay = torch.exp(dtf[:, t] * A.float()[None, :])                      # (B,H)
        h = h * decay[..., None, None] + (dtf[:, t, :, None] * xf[:, t])[..., None] * Bf[:, t, :, None, :]
        ys.append(torch.einsum("bhpn,bhn->bhp", h, Cf[:, t]))
    y = torch.stack(ys, 1)
    if D is not None:
        y = y + xf * D.float()[None, None, :, None]
    y = y.to(x.dtype)
    return (y, h) if return_state else y


# ------------------------------------------------------------------ gated delta rule
def gated_delta_rule(q: Tensor, k: Tensor, v: Tensor, g: Tensor, beta: Tensor,
                     scale: Optional[float] = None, initial_state: Optional[Tensor] = None,
                     return_state: bool = False):
    """q, k (B,T,H,K) (already L2-normalised by the caller); v (B,T,H,V); g (B,T,H) log-decay
    (<= 0); beta (B,T,H) in (0,1).  State S (K x V) per head:
        S <- exp(g_t) S ;  S <- S + k_t (outer) beta_t (v_t - S^T k_t) ;  o_t = scale * S^T q_t"""
    B, T, H, K = q.shape
    V = v.shape[-1]
    scale = K ** -0.5 if scale is None else scale
    qf, kf, vf, gf, bf = (t.float() for t in (q, k, v, g, beta))
    S = qf.new_zeros(B, H, K, V) if initial_state is None else initial_state.float().clone()
    outs = []
    for t in range(T):
        S = S * torch.exp(gf[:, t])[..., None, None]
        pred = torch.einsum("bhkv,bhk->bhv", S, kf[:, t])
        delta = (vf[:, t] - pred) * bf[:, t][..., None]
        S = S + kf[:, t][..., None] * delta[..., None, :]
        outs.append(torch.einsum("bhkv,bhk->bhv", S, qf[:, t]) * scale)
    o = torch.stack(outs, 1).to(v.dtype)
    return (o, S) if return_state else o


# ------------------------------------------------------------------ loss
def linear_cross_entropy(hidden: Tensor, weight: Tensor, labels: Tensor, ignore_index: int = -100) -> Tensor:
    """mean over valid tokens of CE(hidden @ weight^T, labels); hidden (N, d), labels (N)."""
    logits = hidden.float() @ weight.float().t()
    return F.cross_entropy(logits, labels, ignore_index=ignore_index, reduction="mean")


# ------------------------------------------------------------------ optimizer maths
def adamw_step(p: Tensor, g: Tensor, m: Tensor, v: Tensor, step: int, lr: float, beta1: float,
               beta2: float, eps: float, weight_decay: float) -> None:
    """Decoupled-weight-decay Adam on fp32 tensors, in place (torch.optim.AdamW semantics)."""
    p.mul_(1 - lr * weight_decay)
    m.mul_(beta1).add_(g, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    bc1, bc2 = 1 - beta1 ** step, 1 - beta2 ** step
    denom = (v.sqrt() / math.sqrt(bc2)).add_(eps)
    p.addcdiv_(m, denom, value=-lr / bc1)
