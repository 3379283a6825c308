"""The allocation-free RMSNorm backward entry point, called through its exported C symbol.

Some users of this library run where device memory cannot be requested at call time (a serving process with a fixed
memory plan, a real-time loop, a plugin inside a host application that owns the GPU's memory).  For them the library
exports ``dewb_rmsnorm_bwd_noalloc``, whose scratch is a fixed array inside the library.  This test drives that symbol
with ctypes exactly as such a caller would, twice in a row on different inputs (the array keeps the first call's
contents, which must not leak into the second), and compares against the ordinary entry point, which takes its
scratch from the caller.  It is collected last so that a run that stops at the first failure has already run every
other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_D, ERR_TOO_LARGE = 4096, -20


def _lib():
    from dew_b200.ops import library as L
    lib = L.load()
    assert hasattr(lib, "dewb_rmsnorm_bwd_noalloc"), "the library was built without the allocation-free entry point"
    return lib


def _p(t):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _inputs(rows, d, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    mk = lambda *s: torch.randn(*s, device="cuda", generator=g)
    x = mk(rows, d).to(torch.bfloat16)
    dy = mk(rows, d).to(torch.bfloat16)
    dres = mk(rows, d).to(torch.bfloat16)
    w = (1 + 0.1 * mk(d)).to(torch.bfloat16)
    rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-6).contiguous()
    return x, dy, dres, w, rstd


def _ordinary(lib, x, dy, dres, w, rstd):
    rows, d = x.shape
    blocks = lib.dewb_rmsnorm_bwd_blocks(ctypes.c_longlong(rows))
    scratch = torch.empty(blocks, d, dtype=torch.float32, device="cuda")
    dx = torch.empty_like(x)
    dw = torch.empty(d, dtype=torch.float32, device="cuda")
    rc = lib.dewb_rmsnorm_bwd(_p(dy), _p(x), _p(w), _p(rstd), _p(dres), _p(None), _p(dx), _p(None), _p(scratch), _p(dw),
                              _p(None), ctypes.c_int(0), ctypes.c_longlong(rows), ctypes.c_int(d),
                              ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    return dx, dw


def _noalloc(lib, x, dy, dres, w, rstd, dx, dw):
    rows, d = x.shape
    return lib.dewb_rmsnorm_bwd_noalloc(_p(dy), _p(x), _p(w), _p(rstd), _p(dres), _p(dx), _p(dw), _p(None), ctypes.c_int(0),
                                        ctypes.c_longlong(rows), ctypes.c_int(d), ctypes.c_int(torch.cuda.current_device()),
                                        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


def test_noalloc_entry_matches_ordinary_entry_twice_in_a_row():
    lib = _lib()
    torch.cuda.set_device(0)
    # outputs are allocated up front: the calls under test allocate nothing themselves
    cases = [_inputs(1000, 2560, seed=1), _inputs(333, 4096, seed=2)]
    outs = [(torch.empty_like(c[0]), torch.empty(c[0].shape[1], dtype=torch.float32, device="cuda")) for c in cases]
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    for (x, dy, dres, w, rstd), (dx, dw) in zip(cases, outs):          # two calls in a row, sharing the array
        assert _noalloc(lib, x, dy, dres, w, rstd, dx, dw) == 0
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before     # sees torch's allocator only; that the library allocates nothing rests on its source
    assert torch.cuda.current_device() == 0            # the call leaves the caller's current device as it found it
    for (x, dy, dres, w, rstd), (dx, dw) in zip(cases, outs):
        ref_dx, ref_dw = _ordinary(lib, x, dy, dres, w, rstd)
        torch.cuda.synchronize()
        assert torch.equal(dx, ref_dx)                                     # same kernels, same arithmetic
        err = float((dw - ref_dw).norm() / ref_dw.norm())
        assert err < 1e-5, err                                             # a different split count reorders fp32 sums
        # and both agree with the plain PyTorch fp32 formula
        xf, wf = x.float(), w.float()
        xhat = xf * rstd[:, None]
        gw = dy.float() * wf
        want_dx = rstd[:, None] * (gw - xhat * (gw * xhat).mean(-1, keepdim=True)) + dres.float()
        assert float((dx.float() - want_dx).norm() / want_dx.norm()) < 1e-2
        want_dw = (dy.float() * xhat).sum(0)
        assert float((dw - want_dw).norm() / want_dw.norm()) < 1e-4


def test_noalloc_entry_rejects_rows_wider_than_its_array():
    lib = _lib()
    x, dy, dres, w, rstd = _inputs(8, MAX_D + 8, seed=3)
    dx, dw = torch.empty_like(x), torch.empty(MAX_D + 8, dtype=torch.float32, device="cuda")
    assert _noalloc(lib, x, dy, dres, w, rstd, dx, dw) == ERR_TOO_LARGE
