"""The allocation-free layer-norm backward (``cw_layer_norm_bwd_noalloc`` in libcubework_noalloc.so).

Some users of these kernels are not allowed to allocate device memory while they run — code embedded in
another runtime's fixed memory plan, a latency-critical loop that forbids allocator calls after start-up, a
section that is being recorded for replay.  For them the library exports one C function whose only
temporary storage is a fixed array inside the library image.  This test calls that function the way such a
user would — through the exported C symbol, passing raw device pointers — and checks dx, dgamma and dbeta
against the package's regular layer-norm backward, twice in a row (the second call reuses the array that
the first one left dirty), plus the rejection of an oversized hidden dimension.

Collected last on purpose: a run that stops at the first failure has then already run every other test.
"""
import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_HIDDEN = 8192


def _lib():
    from cubework_b200.ops import build
    path = build.build_noalloc()       # rebuilds only when the source or the header is newer than the library
    lib = ctypes.CDLL(path)
    fn = lib.cw_layer_norm_bwd_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 8 + [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    return fn


def _rel(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


def _case(fn, rows, hidden, dtype, seed):
    from cubework_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = (torch.randn(rows, hidden, device="cuda", generator=g) * 1.5 + 0.3).to(dtype)
    dy = torch.randn(rows, hidden, device="cuda", generator=g).to(dtype)
    gamma = torch.randn(hidden, device="cuda", generator=g)
    beta = torch.randn(hidden, device="cuda", generator=g)
    _, mean, rstd = ops.layer_norm_fwd(x, gamma, beta, 1e-5)
    dx_ref, dg_ref, db_ref = ops.layer_norm_bwd(dy, x, mean, rstd, gamma)
    # the caller owns every output; the entry point allocates nothing
    dx = torch.empty_like(x)
    dg = torch.empty(hidden, device="cuda")
    db = torch.empty(hidden, device="cuda")
    torch.cuda.synchronize()
    rc = fn(dy.data_ptr(), x.data_ptr(), mean.data_ptr(), rstd.data_ptr(), gamma.data_ptr(), dx.data_ptr(),
            dg.data_ptr(), db.data_ptr(), rows, hidden, 1 if dtype == torch.bfloat16 else 0,
            torch.cuda.current_stream().cuda_stream)
    assert rc == 0, f"entry point returned {rc}"
    torch.cuda.synchronize()
    assert _rel(dx, dx_ref) < 6e-3, _rel(dx, dx_ref)
    assert _rel(dg, dg_ref) < 1e-3 and _rel(db, db_ref) < 1e-3, (_rel(dg, dg_ref), _rel(db, db_ref))


def test_noalloc_layer_norm_backward_matches_regular_entry_point_twice():
    fn = _lib()
    # two calls in a row share (and overwrite) the same built-in array; shapes differ so stale partials from the
    # first call would show up in the second if any word were read before being written
    _case(fn, 777, 1600, torch.bfloat16, 1)
    _case(fn, 300, 640, torch.bfloat16, 2)
    _case(fn, 64, MAX_HIDDEN, torch.float16, 3)


def test_noalloc_rejects_sizes_beyond_the_built_in_array():
    fn = _lib()
    t = torch.zeros(16, device="cuda")
    p = t.data_ptr()
    assert fn(p, p, p, p, p, p, p, p, 4, MAX_HIDDEN + 8, 1, 0) == 1      # too large: nothing launched
    assert fn(p, p, p, p, p, p, p, p, 4, 12, 1, 0) == 2                  # not a multiple of 8
    assert fn(None, p, p, p, p, p, p, p, 4, 64, 1, 0) == 2               # null pointer
    torch.cuda.synchronize()
