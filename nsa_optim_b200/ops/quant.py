"""Low-bit optimizer-state codecs (PyTorch statements; the CUDA kernels use the same tables).

Two families:

* **Blockwise dynamic quantisation** for Adam moments.  A block of ``block`` consecutive
  values is scaled by its absolute maximum and every value is replaced by the index of the
  nearest entry of a fixed non-uniform code book.  The 8-bit code book is the *dynamic tree*
  map: for each decade ``10^(i-6)``, i = 0..6, it holds ``2^i`` (signed map; ``2^(i+1)`` for
  the unsigned one) midpoints of a uniform grid over [0.1, 1], mirrored for the signed map,
  plus 0 and 1 -> 256 entries.  Signed for the first moment, unsigned for the second.  This is
  the scheme of the 8-bit AdamW the reference selects (optimizers.py:124-141).
  The 4-bit code books have 16 entries; two codes are packed per byte.

* **Affine (asymmetric min/max) quantisation** in sub-row blocks for SOAP eigenbases
  (reference: optimizers.py:652-801): ``code = round((x - min)/scale)``, one
  ``(scale, zero_point)`` pair per ``q_block`` consecutive values of a row, codes stored
  one per byte for both 4- and 8-bit.
"""
from __future__ import annotations

import functools
from typing import Tuple

import torch
import torch.nn.functional as F
from torch import Tensor


# ------------------------------------------------------------------ code books
def _dynamic_tree(signed: bool, total_bits: int = 8, max_exponent_bits: int = 7) -> Tensor:
    non_sign_bits = total_bits - 1
    vals = []
    for i in range(max_exponent_bits):
        n = 2 ** (i + non_sign_bits - max_exponent_bits) + 1 if signed else \
            2 ** (i + non_sign_bits - max_exponent_bits + 1) + 1
        edges = torch.linspace(0.1, 1, n, dtype=torch.float64)
        mids = (edges[:-1] + edges[1:]) / 2
        scale = 10.0 ** (-(max_exponent_bits - 1) + i)
        vals += (scale * mids).tolist()
        if signed:
            vals += (-scale * mids).tolist()
    vals += [0.0, 1.0]
    vals += [0.0] * (2 ** total_bits - len(vals))
    return torch.tensor(sorted(vals), dtype=torch.float32)


@functools.lru_cache(maxsize=None)
def _codebook_cpu(bits: int, signed: bool) -> Tensor:
    if bits == 8:
        return _dynamic_tree(signed)
    if bits == 4:
        if signed:
            # 7 negative, 0, 8 positive levels, denser near zero (cubic spacing)
            pos = (torch.linspace(0, 1, 9)[1:]) ** 2
            neg = -(torch.linspace(0, 1, 8)[1:]) ** 2
            return torch.cat([neg.flip(0), torch.zeros(1), pos]).float()
        # no zero entry: a second moment that rounds to 0 would turn the update into m/eps
        return (torch.linspace(0, 1, 17)[1:] ** 2).float()
    raise ValueError(bits)


_DEV_CACHE = {}


def codebook(bits: int, signed: bool, device) -> Tensor:
    key = (bits, signed, str(device))
    cb = _DEV_CACHE.get(key)
    if cb is None:
        cb = _codebook_cpu(bits, signed).to(device)
        _DEV_CACHE[key] = cb
    return cb


# ------------------------------------------------------------------ blockwise dynamic codec
def quantize_blockwise(x: Tensor, bits: int, signed: bool, block: int) -> Tuple[Tensor, Tensor]:
    """x: any shape, numel divisible by ``block`` -> (codes uint8 [numel or numel/2], absmax fp32
    [numel/block])."""
    cb = codebook(bits, signed, x.device)
    xb = x.float().reshape(-1, block)
    absmax = xb.abs().amax(dim=1)
    scaled = xb / absmax.clamp_min(1e-30)[:, None]
    mids = (cb[:-1] + cb[1:]) / 2
    codes = torch.bucketize(scaled, mids).to(torch.uint8).reshape(-1)
    if bits == 4:
        codes = codes[0::2] | (codes[1::2] << 4)
    return codes, absmax


def dequantize_blockwise(codes: Tensor, absmax: Tensor, bits: int, signed: bool, block: int) -> Tensor:
    cb = codebook(bits, signed, codes.device)
    if bits == 4:
        lo, hi = codes & 0xF, codes >> 4
        codes = torch.stack([lo, hi], dim=1).reshape(-1)
    vals = cb[codes.long()].reshape(-1, block)
    return (vals * absmax[:, None]).reshape(-1)


def _native_ok() -> bool:
    from . import get_backend
    return get_backend() != "torch"


# ------------------------------------------------------------------ affine sub-row codec
def affine_quantize(t: Tensor, bits: int, q_block: int) -> Tuple[Tensor, Tensor, Tensor, int]:
    """2-D ``t`` -> (uint8 codes [rows, cols_padded], scale [rows, nblk], zero_point [rows, nblk],
    original column count)."""
    rows, cols = t.shape
    if t.is_cuda and _native_ok():
        from . import native
        return native.affine_quantize(t, bits, q_block)
    pad = (-cols) % q_block
    tp = F.pad(t.float(), (0, pad)) if pad else t.float()
    if pad:
        # padding repeats the last column so it does not widen the block's range
        tp[:, cols:] = tp[:, cols - 1:cols]
    blk = tp.reshape(rows, -1, q_block)
    lo, hi = blk.amin(-1), blk.amax(-1)
    qmax = float(2 ** bits - 1)
    scale = ((hi - lo) / qmax).clamp_min(1e-12)
    # The zero point is kept as a float and NOT clamped to the code range: a block whose values are
    # all of one sign has its zero outside [0, qmax], and clamping it (as integer-zero-point codecs
    # do) would saturate the whole block.
    zp = torch.round(-lo / scale)
    q = torch.round(blk / scale[..., None] + zp[..., None]).clamp_(0, qmax).to(torch.uint8)
    return q.reshape(rows, -1), scale, zp, cols


def affine_dequantize(q: Tensor, scale: Tensor, zero_point: Tensor, orig_cols: int) -> Tensor:
    if q.is_cuda and q.dim() == 2 and scale.dim() == 2 and _native_ok():
        from . import native
        return native.affine_dequantize(q, scale, zero_point, orig_cols)
    rows = q.shape[0]
    nblk = scale.shape[1]
    blk = q.reshape(rows, nblk, -1).float()
    out = (blk - zero_point[..., None]) * scale[..., None]
    return out.reshape(rows, -1)[:, :orig_cols]


def affine_quantize_tensor(t: Tensor, bits: int) -> Tuple[Tensor, Tensor, Tensor, None]:
    """Per-tensor variant for 1-D states."""
    lo, hi = t.float().min(), t.float().max()
    qmax = float(2 ** bits - 1)
    scale = ((hi - lo) / qmax).clamp_min(1e-12)
    zp = torch.round(-lo / scale)
    q = torch.round(t.float() / scale + zp).clamp_(0, qmax).to(torch.uint8)
    return q, scale, zp, None


def affine_dequantize_tensor(q: Tensor, scale: Tensor, zero_point: Tensor) -> Tensor:
    return (q.float() - zero_point) * scale
