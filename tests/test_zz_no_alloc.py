"""The allocation-free projection entry point against the ordinary one.

Some callers hold device buffers but may not allocate: they run inside a region
that is being captured or replayed, or in a loop that must not touch the
allocator, or under a host that owns the device heap.  `rg_linear_row_noalloc`
serves them with scratch that lives inside the library image.  This test feeds
it device buffers it did not allocate (torch tensors stand in for the caller's
memory) and compares with `rg_matmul` + `rg_add`, the entry points every other
caller uses, on two calls in a row - the second call reuses the shared scratch
with different sizes, which is where stale contents would show.

Collected last on purpose: a run that stops at the first failure has then
already run every other test."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _reference(be, x, w, b):
    y = be.add(be.matmul(be.from_slice(x, [1, x.size]), be.from_slice(w, list(w.shape))), be.from_slice(b, [1, b.size]))
    return be.to_vec(y)


def test_noalloc_projection_matches_matmul_twice(backend):
    import torch
    from rustygradients_b200 import _lib
    import rustygradients_b200 as rg

    lib = _lib.load()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    stream = torch.cuda.current_stream(dev)
    rng = np.random.default_rng(123)
    for K, N in ((768, 3072), (3072, 768)):     # two calls in a row, different shapes, same scratch
        x = rng.standard_normal(K).astype(np.float32)
        w = (rng.standard_normal((K, N)) * 0.05).astype(np.float32)
        b = rng.standard_normal(N).astype(np.float32)
        tx, tw, tb = (torch.from_numpy(a).to(dev) for a in (x, w, b))
        ty = torch.full((N,), float("nan"), device=dev)
        torch.cuda.synchronize(dev)
        st = lib.rg_linear_row_noalloc(C.c_void_p(tx.data_ptr()), C.c_void_p(tw.data_ptr()), C.c_void_p(tb.data_ptr()),
                                       C.c_void_p(ty.data_ptr()), K, N, C.c_void_p(stream.cuda_stream))
        _lib.check(st)
        torch.cuda.synchronize(dev)
        got = ty.cpu().numpy()
        want = _reference(backend, x, w, b)
        assert np.isfinite(got).all()
        assert np.abs(got - want).max() <= 1e-3          # the f32 tolerance of the parity tests
        assert np.abs(got - (x.astype(np.float64) @ w + b)).max() <= 1e-3
    # odd sizes and no bias: K neither a multiple of 8 nor of the k-split, N not a multiple of the column tile
    K, N = 773, 132
    x = rng.standard_normal(K).astype(np.float32)
    w = (rng.standard_normal((K, N)) * 0.05).astype(np.float32)
    tx, tw = torch.from_numpy(x).to(dev), torch.from_numpy(w).to(dev)
    ty = torch.full((N,), float("nan"), device=dev)
    torch.cuda.synchronize(dev)
    _lib.check(lib.rg_linear_row_noalloc(C.c_void_p(tx.data_ptr()), C.c_void_p(tw.data_ptr()), None, C.c_void_p(ty.data_ptr()),
                                         K, N, C.c_void_p(stream.cuda_stream)))
    torch.cuda.synchronize(dev)
    assert np.abs(ty.cpu().numpy() - x.astype(np.float64) @ w).max() <= 1e-3
    # sizes beyond the built-in scratch are refused with a clear message, not truncated
    st = lib.rg_linear_row_noalloc(C.c_void_p(tx.data_ptr()), C.c_void_p(tw.data_ptr()), None, C.c_void_p(ty.data_ptr()),
                                   16, 16388, C.c_void_p(stream.cuda_stream))
    assert st == _lib.RG_ERR_INVALID_INPUT and b"16384" in lib.rg_last_error()
    with pytest.raises(rg.InvalidInput):
        _lib.check(lib.rg_linear_row_noalloc(C.c_void_p(tx.data_ptr()), C.c_void_p(tw.data_ptr()), None,
                                             C.c_void_p(ty.data_ptr()), 40000, 16, C.c_void_p(stream.cuda_stream)))
