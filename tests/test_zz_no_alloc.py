"""The allocation-free RMSNorm backward, called through its exported C symbol.

Some callers of this library cannot allocate device memory when they need a weight gradient:
they run inside a frozen memory plan, own no allocator, or sit at the memory limit.  For them
``olb_rmsnorm_bwd_noalloc`` keeps its scratch in a device array inside the library.  This test
calls that symbol with ctypes (no torch allocation happens inside the call), twice in a row -
the array is shared and keeps the previous call's contents - and checks both results against
the regular entry point, within the tolerance of the other kernel tests.

The file name sorts last on purpose: a run that stops at the first failure has then already run
every other test.  The test also passes alone in a fresh process.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from optimus_lm_b200.ops import extension
    mod = extension()
    mod = getattr(mod, "_mod", mod)  # unwrap the launch-counting proxy if it is active
    lib = ctypes.CDLL(mod.__file__)
    fn = lib.olb_rmsnorm_bwd_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                   ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    lib.olb_noalloc_strerror.restype = ctypes.c_char_p
    lib.olb_noalloc_strerror.argtypes = [ctypes.c_int]
    return lib, fn


def _rel_err(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


def _case(rows, cols, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(rows, cols, device="cuda", generator=g).to(torch.bfloat16)
    dy = torch.randn(rows, cols, device="cuda", generator=g).to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(cols, device="cuda", generator=g)).to(torch.bfloat16)
    return x, dy, w


def _regular(x, dy, w):
    """dx, dw from the existing entry point (caller-allocated scratch)."""
    from optimus_lm_b200.ops import extension
    C = extension()
    rows, cols = x.shape
    y = torch.empty_like(x)
    rstd = torch.empty(rows, dtype=torch.float32, device="cuda")
    C.rmsnorm_fwd(x, w, y, rstd, 1e-5)
    nb = C.rmsnorm_bwd_blocks(rows)
    partial = torch.empty((nb, cols), dtype=torch.float32, device="cuda")
    dx = torch.empty_like(x)
    dw = torch.empty_like(w)
    C.rmsnorm_bwd(dy, x, w, rstd, dx, partial)
    C.colsum_finalize(partial, nb, dw, False)
    return rstd, dx, dw


def test_noalloc_matches_regular_entry_point_twice():
    lib, fn = _lib()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    # two different problems back to back: the second must not see leftovers of the first
    # (2048 and 512 take the register-resident kernel, 7168 and 8192 the shared-memory one with its opt-in limit)
    for rows, cols, seed in ((1000, 2048, 1), (333, 512, 2), (64, 7168, 3), (64, 8192, 4)):
        x, dy, w = _case(rows, cols, seed)
        rstd, dx_ref, dw_ref = _regular(x, dy, w)
        dx = torch.empty_like(x)
        dw = torch.empty_like(w)
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        rc = fn(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx.data_ptr(), dw.data_ptr(), 0, rows,
                cols, stream)
        assert rc == 0, lib.olb_noalloc_strerror(rc).decode()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert _rel_err(dx, dx_ref) < 1e-2
        assert _rel_err(dw, dw_ref) < 1e-2
        # fp32 weight-gradient output
        dw32 = torch.empty(cols, dtype=torch.float32, device="cuda")
        rc = fn(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx.data_ptr(), dw32.data_ptr(), 1, rows,
                cols, stream)
        assert rc == 0, lib.olb_noalloc_strerror(rc).decode()
        torch.cuda.synchronize()
        assert _rel_err(dw32, dw_ref) < 1e-2


def test_noalloc_rejects_oversize_and_bad_cols():
    lib, fn = _lib()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    t = torch.zeros(8, dtype=torch.bfloat16, device="cuda")
    r = torch.zeros(8, dtype=torch.float32, device="cuda")
    rc = fn(t.data_ptr(), t.data_ptr(), t.data_ptr(), r.data_ptr(), t.data_ptr(), t.data_ptr(), 0, 1, 8192 + 8, stream)
    assert rc == -20 and b"8192" in lib.olb_noalloc_strerror(rc)
    rc = fn(t.data_ptr(), t.data_ptr(), t.data_ptr(), r.data_ptr(), t.data_ptr(), t.data_ptr(), 0, 1, 12, stream)
    assert rc == -1
    # a null output with work to do is refused before any launch
    rc = fn(t.data_ptr(), t.data_ptr(), t.data_ptr(), r.data_ptr(), None, t.data_ptr(), 0, 1, 8, stream)
    assert rc == -23 and b"null" in lib.olb_noalloc_strerror(rc)
    rc = fn(t.data_ptr(), t.data_ptr(), t.data_ptr(), r.data_ptr(), t.data_ptr(), None, 0, 1, 8, stream)
    assert rc == -23
    torch.cuda.synchronize()
