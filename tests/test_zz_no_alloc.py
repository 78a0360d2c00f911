"""The allocation-free RMSNorm backward, called through its exported C symbol.

Some users of the library run the backward pass from places where they may not allocate
device memory (a fixed memory budget, a thread that must not enter the allocator, a loop
that cannot tolerate an allocation's synchronisation).  ``nsa_rmsnorm_bwd_noalloc`` serves
them: same inputs and outputs as ``nsa_rmsnorm_bwd`` but the partial-sum scratch is a static
array inside the library.  This test checks it against ``nsa_rmsnorm_bwd`` on two calls in
a row (the second with different data, so leftovers of the first in the shared scratch would
show), and checks that an over-size problem is refused.  It is collected last on purpose.
"""
import ctypes
from ctypes import c_float, c_int, c_long, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ptr(t):
    return c_void_p(0 if t is None else t.data_ptr())


def _run(lib, entry, x, gate, w, dy, mode, scratch=None):
    rows, d = x.shape
    y = torch.empty_like(x)
    rstd = torch.empty(rows, dtype=torch.float32, device="cuda")
    st = c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.nsa_rmsnorm_fwd(_ptr(x), _ptr(gate), _ptr(w), _ptr(y), _ptr(rstd), c_long(rows), c_int(d),
                               c_float(1e-6), c_int(mode), st) == 0
    dx, dw = torch.empty_like(x), torch.empty(d, dtype=torch.float32, device="cuda")
    dg = torch.empty_like(x) if mode else None
    if entry == "noalloc":
        rc = lib.nsa_rmsnorm_bwd_noalloc(_ptr(x), _ptr(gate), _ptr(w), _ptr(dy), _ptr(rstd), _ptr(dx), _ptr(dg),
                                         c_void_p(0), _ptr(dw), c_long(rows), c_int(d), c_int(mode), st)
    else:
        rc = lib.nsa_rmsnorm_bwd(_ptr(x), _ptr(gate), _ptr(w), _ptr(dy), _ptr(rstd), _ptr(dx), _ptr(dg),
                                 c_void_p(0), _ptr(dw), _ptr(scratch), c_long(rows), c_int(d), c_int(mode), st)
    torch.cuda.synchronize()
    return rc, dx, dg, dw


@pytest.mark.parametrize("rows,d,mode,rows2", [(3000, 2048, 0, 3000), (777, 256, 1, 777), (64, 4096, 2, 64),
                                                (60000, 1024, 0, 40)])
def test_noalloc_matches_allocating_entry_twice(rows, d, mode, rows2):
    """Two calls in a row; in the last case the second call is much smaller than the first, so it
    uses fewer partial-sum rows and anything it wrongly read from the first call's leftovers in
    the shared scratch would change dw."""
    from nsa_optim_b200.ops import native
    lib = native.load()
    assert hasattr(lib, "nsa_rmsnorm_bwd_noalloc")
    for call in range(2):
        if call == 1:
            rows = rows2
        parts = lib.nsa_rmsnorm_bwd_parts(c_long(rows), c_int(d))
        torch.manual_seed(100 + call)
        x = torch.randn(rows, d, device="cuda").bfloat16() * (1 + call)
        gate = torch.randn(rows, d, device="cuda").bfloat16() if mode else None
        w = (1 + 0.1 * torch.randn(d, device="cuda")).bfloat16()
        dy = torch.randn(rows, d, device="cuda").bfloat16()
        scratch = torch.empty(parts * d, dtype=torch.float32, device="cuda")
        rc_a, dx_a, dg_a, dw_a = _run(lib, "alloc", x, gate, w, dy, mode, scratch)
        rc_n, dx_n, dg_n, dw_n = _run(lib, "noalloc", x, gate, w, dy, mode)
        assert rc_a == 0 and rc_n == 0, native.load().nsa_last_error()
        assert torch.equal(dx_n, dx_a)
        if mode:
            assert torch.equal(dg_n, dg_a)
        # same grid, same fixed-order reduction: the two entry points agree to the bit
        assert torch.equal(dw_n, dw_a)
    native.check_status()


def test_noalloc_rejects_oversize():
    from nsa_optim_b200.ops import native
    lib = native.load()
    rows, d = 100000, 8192                                   # 592 parts * 8192 columns > built-in scratch
    z = torch.zeros(8, device="cuda")
    rc = lib.nsa_rmsnorm_bwd_noalloc(_ptr(z), c_void_p(0), _ptr(z), _ptr(z), _ptr(z), _ptr(z), c_void_p(0),
                                     c_void_p(0), _ptr(z), c_long(rows), c_int(d), c_int(0), c_void_p(0))
    assert rc == 5
    assert b"built-in scratch" in lib.nsa_last_error()
