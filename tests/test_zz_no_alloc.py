"""The allocation-free RMSNorm backward, called through its exported C symbol.

Some users of the kernel library hold raw device pointers and may not allocate device memory at
call time (a plugin inside another runtime's memory pool, a host with a fixed device memory map).
``mmt_rmsnorm_bwd_noalloc`` serves them: its scratch lives inside the library.  This test loads the
shared library with ctypes, calls the symbol directly, and checks its outputs against the regular
entry point (``mmt_rmsnorm_bwd``, caller-provided scratch) on two calls in a row, the second with
different data and shape so that stale scratch contents would show.  The file sorts last on purpose,
so a run that stops at the first failure has already run every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from multimodal_training_b200.ops import native as nv
    assert nv.available(), "libmmt_b200.so must be built"
    lib = ctypes.CDLL(str(nv.LIB_PATH))
    P, L, I = ctypes.c_void_p, ctypes.c_long, ctypes.c_int
    lib.mmt_rmsnorm_bwd_noalloc.restype = I
    lib.mmt_rmsnorm_bwd_noalloc.argtypes = [P, P, P, P, P, P, L, I, I, P]
    lib.mmt_rmsnorm_bwd.restype = I
    lib.mmt_rmsnorm_bwd.argtypes = [P, P, P, P, P, P, P, L, I, I, P]
    lib.mmt_rmsnorm_bwd_parts.restype = I
    lib.mmt_rmsnorm_bwd_parts.argtypes = [L]
    lib.mmt_rmsnorm_fwd.restype = I
    lib.mmt_rmsnorm_fwd.argtypes = [P, P, P, P, L, I, ctypes.c_float, P]
    return lib


def _case(lib, rows, cols, seed, accumulate):
    dev = "cuda"
    torch.manual_seed(seed)
    x = torch.randn(rows, cols, device=dev, dtype=torch.bfloat16)
    dy = torch.randn(rows, cols, device=dev, dtype=torch.bfloat16)
    w = (1 + 0.1 * torch.randn(cols, device=dev)).to(torch.bfloat16)
    y = torch.empty_like(x)
    rstd = torch.empty(rows, device=dev, dtype=torch.float32)
    st = torch.cuda.current_stream().cuda_stream
    assert lib.mmt_rmsnorm_fwd(x.data_ptr(), w.data_ptr(), y.data_ptr(), rstd.data_ptr(), rows, cols, 1e-6, st) == 0
    dw0 = torch.randn(cols, device=dev, dtype=torch.bfloat16) if accumulate else torch.zeros(cols, device=dev,
                                                                                            dtype=torch.bfloat16)
    # regular entry point: the caller allocates the scratch
    parts = lib.mmt_rmsnorm_bwd_parts(rows)
    scratch = torch.empty(parts * cols, device=dev, dtype=torch.float32)
    dx_ref, dw_ref = torch.empty_like(x), dw0.clone()
    assert lib.mmt_rmsnorm_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx_ref.data_ptr(),
                               dw_ref.data_ptr(), scratch.data_ptr(), rows, cols, int(accumulate), st) == 0
    # allocation-free entry point: inputs and outputs only
    dx, dw = torch.empty_like(x), dw0.clone()
    rc = lib.mmt_rmsnorm_bwd_noalloc(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx.data_ptr(),
                                     dw.data_ptr(), rows, cols, int(accumulate), st)
    assert rc == 0
    torch.cuda.synchronize()

    def rel(a, b):
        return ((a.float() - b.float()).abs().max() / (b.float().abs().max() + 1e-9)).item()

    assert rel(dx, dx_ref) < 1e-2, rel(dx, dx_ref)
    assert rel(dw, dw_ref) < 1e-2, rel(dw, dw_ref)
    # and both agree with an fp32 PyTorch evaluation of the same formula
    xf, wf, dyf = x.float(), w.float(), dy.float()
    g = dyf * wf
    r = rstd[:, None]
    dx_t = r * (g - xf * r * r * (g * xf).mean(-1, keepdim=True))
    dw_t = (dyf * xf * r).sum(0) + (dw0.float() if accumulate else 0)
    assert rel(dx, dx_t) < 1e-2 and rel(dw, dw_t) < 1e-2


def test_noalloc_matches_regular_entry_point_twice():
    lib = _lib()
    _case(lib, rows=1000, cols=3584, seed=0, accumulate=False)
    _case(lib, rows=333, cols=1280, seed=1, accumulate=True)   # second call: other shape, stale scratch in place


def test_noalloc_with_capped_partial_rows_and_on_a_side_stream():
    """cols = 8192 with thousands of rows: the number of per-CTA partial rows is capped by the size of the built-in
    scratch (2^21 / 8192 = 256 rows of partial sums, fewer than the regular entry point would use), with and without
    accumulation into dw, and launched on a stream that is not the default one."""
    lib = _lib()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        _case(lib, rows=2000, cols=8192, seed=2, accumulate=False)
        _case(lib, rows=2176, cols=8192, seed=3, accumulate=True)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()


def test_noalloc_rejects_sizes_beyond_the_maximum():
    lib = _lib()
    t = torch.zeros(8, device="cuda", dtype=torch.bfloat16)
    f = torch.zeros(8, device="cuda", dtype=torch.float32)
    p = t.data_ptr()
    assert lib.mmt_rmsnorm_bwd_noalloc(p, p, p, f.data_ptr(), p, p, 1, 8192 + 8, 0, None) == -5
    assert lib.mmt_rmsnorm_bwd_noalloc(p, p, p, f.data_ptr(), p, p, 1, 12, 0, None) == -2
    assert lib.mmt_rmsnorm_bwd_noalloc(p, p, p, f.data_ptr(), p, p, 1, 0, 0, None) == -5
    assert lib.mmt_rmsnorm_bwd_noalloc(p, p, p, f.data_ptr(), p, p, -1, 8, 0, None) == -5
