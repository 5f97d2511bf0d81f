"""The library's ops against the reference's OWN CUDA kernels (src/backend/cuda_kernels.cu), compiled in place for this
GPU by oracle/build_ref.py into oracle/_ref/libref_kernels.so (a built file that travels with the tree; the test is
skipped where it was not built).  This pins the op level to outputs of reference code executed here, with the
tolerances of the reference's own kernel test (examples/cuda_kernels_test.rs: 1e-5 elementwise, 1e-6 on softmax row
sums), and prints the device time of both sides for the shapes of the GPT-2-small prompt pass."""
import ctypes as C
import os
import time

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

LIB = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref", "libref_kernels.so")
KINDS = dict(add=0, mul=1, sub=2, relu=3, sigmoid=4, gelu=5, exp=6, log=7, softmax=8, layernorm=9)


@pytest.fixture(scope="module")
def ref():
    if not os.path.exists(LIB):
        pytest.skip("oracle/_ref/libref_kernels.so was not built (no reference tree on the build machine)")
    lib = C.CDLL(LIB)
    fp = C.POINTER(C.c_float)
    lib.ref_run.argtypes = [C.c_int, fp, fp, fp, fp, C.c_int, C.c_int, C.c_float]
    lib.ref_time.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, fp]

    def run(kind, a, b=None, c=None, eps=1e-5):
        a = np.ascontiguousarray(a, np.float32)
        batch, n = a.reshape(-1, a.shape[-1]).shape
        out = np.empty_like(a)
        bb = None if b is None else np.ascontiguousarray(b, np.float32)
        cc = None if c is None else np.ascontiguousarray(c, np.float32)
        rc = lib.ref_run(KINDS[kind], a.ctypes.data_as(fp), None if bb is None else bb.ctypes.data_as(fp),
                         None if cc is None else cc.ctypes.data_as(fp), out.ctypes.data_as(fp), batch, n, eps)
        assert rc == 0, f"reference kernel {kind}: cudaError {rc}"
        return out

    def device_ms(kind, batch, n, iters=20):
        ms = C.c_float(0)
        assert lib.ref_time(KINDS[kind], batch, n, iters, C.byref(ms)) == 0
        return ms.value

    run.device_ms = device_ms
    return run


def test_ops_match_the_reference_kernels(backend, ref):
    rng = np.random.default_rng(12)
    be = backend
    x = (rng.standard_normal((37, 300)) * 2).astype(np.float32)
    y = (rng.standard_normal((37, 300)) * 2).astype(np.float32)
    sx, sy = be.from_slice(x.reshape(-1), x.shape), be.from_slice(y.reshape(-1), y.shape)
    for name, fn in (("add", be.add), ("mul", be.mul), ("sub", be.sub)):
        assert np.array_equal(be.to_array(fn(sx, sy)), ref(name, x, y)), name          # one rounding each: bit-exact
    assert np.array_equal(be.to_array(be.relu(sx)), ref("relu", x))
    for name, fn, inp in (("sigmoid", be.sigmoid, x), ("gelu", be.gelu, x), ("exp", be.exp, x), ("log", be.log, np.abs(x) + 0.1)):
        got = be.to_array(fn(be.from_slice(inp.reshape(-1), inp.shape)))
        want = ref(name, inp)
        assert np.abs(got - want).max() <= 1e-5 * max(1.0, np.abs(want).max()), name
    got, want = be.to_array(be.softmax(sx)), ref("softmax", x)
    assert np.abs(got - want).max() <= 1e-6 and np.abs(got.sum(-1) - 1).max() <= 1e-6
    g, b = (1 + 0.1 * rng.standard_normal(300)).astype(np.float32), (0.1 * rng.standard_normal(300)).astype(np.float32)
    got = be.to_array(be.layer_norm(sx, be.from_slice(g, g.shape), be.from_slice(b, b.shape), 1e-5))
    want = ref("layernorm", x, g, b, eps=1e-5)
    assert np.abs(got - want).max() <= 1e-5
    # the reference's own known answers (examples/cuda_kernels_test.rs): LayerNorm of a ramp row has mean 0, variance 1
    ramp = np.arange(1, 9, dtype=np.float32)[None, :]
    r = ref("layernorm", ramp, np.ones(8, np.float32), np.zeros(8, np.float32))
    assert abs(r.mean()) < 1e-5 and abs(r.var() - 1) < 1e-3


def test_device_time_beside_the_reference_kernels(backend, ref):
    """Shapes of the GPT-2-small prompt pass on 8,192 rows.  Reference side: CUDA events around 20 launches on resident
    data.  Library side: wall clock around 20 calls of the public op + synchronise (each call also allocates its
    output, like the reference's wrapper does), so the printed ratio is a lower bound on the kernels' own ratio."""
    be = backend
    rng = np.random.default_rng(0)
    for name, batch, n in (("layernorm", 8192, 768), ("softmax", 24576, 256), ("gelu", 8192, 3072), ("add", 8192, 768)):
        ref_ms = ref.device_ms(name, batch, n)
        x = rng.standard_normal((batch, n)).astype(np.float32)
        sx = be.from_slice(x.reshape(-1), x.shape)
        if name == "layernorm":
            g, b = be.ones([n]), be.zeros([n])
            op = lambda: be.layer_norm(sx, g, b, 1e-5)
        else:
            op = {"softmax": lambda: be.softmax(sx), "gelu": lambda: be.gelu(sx), "add": lambda: be.add(sx, sx)}[name]
        for _ in range(3):
            op()
        be.synchronize()
        t = time.perf_counter()
        for _ in range(20):
            op()
        be.synchronize()
        lib_ms = (time.perf_counter() - t) / 20 * 1e3
        gb = batch * n * 4 * (3 if name == "add" else 2) / 1e9
        print(f"{name} [{batch} x {n}]: reference kernel {ref_ms * 1e3:.1f} us ({gb / ref_ms * 1e3:.0f} GB/s), "
              f"library op incl. allocation {lib_ms * 1e3:.1f} us ({gb / lib_ms * 1e3:.0f} GB/s)")
        assert ref_ms > 0 and lib_ms > 0
