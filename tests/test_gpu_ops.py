"""GPU parity of the Backend-trait ops (C ABI, through the host mirror) against
the oracle: the reference's own known answers and ramp inputs at its tolerances
(examples/cuda_kernels_test.rs:146-256), then seeded random and edge shapes."""
import numpy as np
import pytest

import rustygradients_b200 as rg
from oracle import gpt_oracle as O

pytestmark = pytest.mark.gpu


def arr(be, st):
    return be.to_array(st)


def test_reference_kats(backend):
    be, k = backend, O.reference_kats()
    m = k["matmul_2x2"]   # src/backend/cuda.rs:545-571
    c = arr(be, be.matmul(be.from_slice(m["a"], [2, 2]), be.from_slice(m["b"], [2, 2])))
    assert np.abs(c - m["out"]).max() <= m["tol"]
    for key in ("relu_4", "relu_5"):
        x = k[key]
        assert np.array_equal(arr(be, be.relu(be.from_slice(x["x"], [x["x"].size]))), x["out"])
    assert abs(arr(be, be.sigmoid(be.from_slice([0.0], [1])))[0] - 0.5) <= 1e-6
    ln = k["layernorm_1234"]
    y = arr(be, be.layer_norm(be.from_slice(ln["x"], [1, 4]), be.from_slice(ln["gamma"], [1, 4]),
                              be.from_slice(ln["beta"], [1, 4]), ln["eps"]))
    assert abs(float(y.mean())) < 1e-3 and abs(float(y.var()) - 1.0) < 0.1
    assert np.abs(y - O.layernorm_two_pass(ln["x"], ln["gamma"], ln["beta"], ln["eps"])).max() < 1e-6
    g = arr(be, be.gelu(be.from_slice([0.0, 1.0], [2])))
    assert abs(g[0]) < 1e-6 and 0.8 < g[1] < 0.9


def test_reference_ramps(backend):
    be, k = backend, O.reference_kats()
    r = k["ramp_add"]
    a, b = be.from_slice(r["a"], [1024]), be.from_slice(r["b"], [1024])
    assert np.abs(arr(be, be.add(a, b)) - (r["a"] + r["b"])).max() <= r["tol"]
    assert np.abs(arr(be, be.mul(a, b)) - (r["a"] * r["b"])).max() <= k["ramp_mul"]["tol"]
    r = k["ramp_relu"]
    assert np.abs(arr(be, be.relu(be.from_slice(r["x"], [1024]))) - O.relu(r["x"])).max() <= r["tol"]
    r = k["ramp_sigmoid"]
    assert np.abs(arr(be, be.sigmoid(be.from_slice(r["x"], [1024]))) - O.sigmoid(r["x"])).max() <= r["tol"]
    r = k["ramp_exp"]
    assert np.abs(arr(be, be.exp(be.from_slice(r["x"], [1024]))) - np.exp(r["x"])).max() <= r["tol"]
    r = k["ramp_softmax"]
    y = arr(be, be.softmax(be.from_slice(r["x"], [8, 128])))
    assert np.abs(y - O.softmax_lastaxis(r["x"])).max() <= r["tol"]
    assert np.abs(y.sum(-1) - 1).max() < 1e-5


def test_memory_ops(backend):
    be = backend
    z = be.zeros([10, 20])   # src/backend/cuda.rs:526-543
    assert z.shape == [10, 20] and len(z) == 200 and not arr(be, z).any()
    assert np.all(arr(be, be.ones([3, 1, 5])) == 1)
    x = np.arange(24, dtype=np.float32)
    s = be.from_slice(x, [2, 3, 4])
    assert np.array_equal(be.to_vec(s), x) and be.shape(s) == [2, 3, 4]
    assert len(be.zeros([0, 4])) == 0 and arr(be, be.zeros([0, 4])).shape == (0, 4)
    with pytest.raises(rg.ShapeError):
        be.from_slice(x, [5, 5])
    be.synchronize()
    assert be.device_type() == ("cuda", 0) and rg.B200Backend.is_available()


def test_broadcast_arithmetic(backend):
    be = backend
    rng = np.random.default_rng(0)
    cases = [((2, 5, 16), (1, 16)), ((2, 5, 16), (2, 5, 16)), ((4, 3, 7, 7), ()), ((3, 1, 5), (1, 4, 1)),
             ((1, 6, 128), (2, 6, 128)), ((1023,), (1023,)), ((5,), (1,))]
    for sa, sb in cases:
        a = rng.standard_normal(sa).astype(np.float32)
        b = rng.standard_normal(sb).astype(np.float32)
        A, Bs = be.from_slice(a, list(sa)), be.from_slice(b, list(sb))
        for name, f in (("add", np.add), ("sub", np.subtract), ("mul", np.multiply)):
            got = arr(be, getattr(be, name)(A, Bs))
            want = f(a, b)
            assert got.shape == want.shape and np.array_equal(got, want), (name, sa, sb)
    with pytest.raises(rg.ShapeError):
        be.add(be.zeros([2, 3]), be.zeros([3, 2]))


def test_matmul_ranks(backend):
    be = backend
    rng = np.random.default_rng(1)
    for sa, sb in [((33, 70), (70, 45)), ((2, 5, 16), (16, 10)), ((3, 17, 40), (3, 40, 9)),
                   ((2, 4, 13, 32), (2, 4, 32, 13)), ((1, 1), (1, 1)), ((128, 768), (768, 130))]:
        a = rng.standard_normal(sa).astype(np.float32)
        b = rng.standard_normal(sb).astype(np.float32)
        got = arr(be, be.matmul(be.from_slice(a, list(sa)), be.from_slice(b, list(sb))))
        want = np.matmul(a.astype(np.float64), b.astype(np.float64))
        assert got.shape == want.shape
        assert np.abs(got - want).max() <= 1e-5 * max(1.0, np.abs(want).max()) * np.sqrt(sa[-1])
    with pytest.raises(rg.ShapeError):
        be.matmul(be.zeros([2, 3]), be.zeros([4, 5]))
    with pytest.raises(rg.ShapeError):
        be.matmul(be.zeros([2, 3, 4]), be.zeros([3, 4, 5]))
    with pytest.raises(rg.ShapeError):
        be.matmul(be.zeros([3]), be.zeros([3]))


def test_unary_and_rows(backend):
    be = backend
    rng = np.random.default_rng(2)
    x = (rng.standard_normal((7, 333)) * 2).astype(np.float32)
    X = be.from_slice(x, [7, 333])
    assert np.abs(arr(be, be.gelu(X)) - O.gelu_tanh(x)).max() < 1e-6
    assert np.abs(arr(be, be.exp(X)) - np.exp(x)).max() <= 1e-5 * np.exp(x).max()
    assert np.abs(arr(be, be.log(be.from_slice(np.abs(x) + 1, [7, 333]))) - np.log(np.abs(x) + 1)).max() < 1e-6
    assert np.abs(arr(be, be.powf(be.from_slice(np.abs(x), [7, 333]), 2.5)) - np.abs(x) ** 2.5).max() < 1e-3
    assert np.abs(arr(be, be.softmax(X)) - O.softmax_lastaxis(x)).max() < 1e-6
    big = (rng.standard_normal((3, 5000)) * 4).astype(np.float32)
    assert np.abs(arr(be, be.softmax(be.from_slice(big, [3, 5000]))) - O.softmax_lastaxis(big)).max() < 1e-6
    for D in (4, 128, 768, 1600):
        h = (rng.standard_normal((2, 5, D)) * 3 + 0.5).astype(np.float32)
        g = (1 + 0.1 * rng.standard_normal((1, D))).astype(np.float32)
        b = (0.1 * rng.standard_normal((1, D))).astype(np.float32)
        got = arr(be, be.layer_norm(be.from_slice(h, [2, 5, D]), be.from_slice(g, [1, D]), be.from_slice(b, [1, D]), 1e-5))
        assert np.abs(got - O.layernorm_two_pass(h, g, b)).max() < 5e-6
    with pytest.raises(rg.ShapeError):
        be.layer_norm(X, be.ones([1, 5]), be.zeros([1, 333]), 1e-5)
    assert abs(arr(be, be.sum(X))[0] - x.astype(np.float64).sum()) < 1e-2
    for ax in (0, 1):
        assert np.abs(arr(be, be.sum_axis(X, ax)) - x.sum(ax)).max() < 1e-3
    with pytest.raises(rg.ShapeError):
        be.sum_axis(X, 2)
    lg = rng.standard_normal((6, 11)).astype(np.float32)
    tg = np.array([0, 10, 3, 3, 7, 1], np.float32)
    p = O.softmax_lastaxis(lg)
    want = float(np.mean(-np.log(p[np.arange(6), tg.astype(int)])))
    assert abs(arr(be, be.sparse_cross_entropy(be.from_slice(lg, [6, 11]), be.from_slice(tg, [6])))[0] - want) < 1e-5
    with pytest.raises(rg.ShapeError):
        be.sparse_cross_entropy(be.from_slice(lg, [6, 11]), be.from_slice(tg + 20, [6]))


def test_transform_and_embedding(backend):
    be = backend
    x = np.arange(2 * 3 * 4 * 5, dtype=np.float32).reshape(2, 3, 4, 5)
    X = be.from_slice(x, [2, 3, 4, 5])
    for a1, a2 in ((1, 2), (2, 3), (0, 3), (1, 1)):
        assert np.array_equal(arr(be, be.transpose(X, a1, a2)), np.swapaxes(x, a1, a2))
    assert np.array_equal(arr(be, be.reshape(X, [6, 20])), x.reshape(6, 20))
    with pytest.raises(rg.ShapeError):
        be.reshape(X, [7, 7])
    with pytest.raises(rg.ShapeError):
        be.transpose(X, 0, 4)
    table = np.random.default_rng(3).standard_normal((52, 128)).astype(np.float32)
    ids = np.array([[0, 51, 7], [7, 7, 3]], np.float32)
    T = be.from_slice(table, [52, 128])
    got = arr(be, be.embedding(be.from_slice(ids, [2, 3]), T))
    assert np.array_equal(got, O.embedding(ids, table))
    assert arr(be, be.embedding(be.from_slice(ids[0], [3]), T)).shape == (3, 128)
    with pytest.raises(rg.InvalidInput):     # src/ops/embedding.rs:51-56
        be.embedding(be.from_slice([[52.0]], [1, 1]), T)
    with pytest.raises(rg.ShapeError):       # src/backend/cpu.rs:319-324
        be.embedding(be.from_slice(ids, [2, 3]), be.zeros([4]))
    # the context survives the error
    assert np.array_equal(arr(be, be.embedding(be.from_slice(ids, [2, 3]), T)), O.embedding(ids, table))


def test_attention_from_ops_matches_oracle(backend):
    """MultiHeadAttention::forward written with Backend ops only (src/nn/attention.rs:57-105),
    on the reference's own test shape [2,5,16] with 4 heads (tests/nn_test.rs:60-75)."""
    be = backend
    cfg = O.GptConfig(8, 10, 1, 4, 16)
    p = O.make_params(cfg, 11)[2:10]
    x = np.random.default_rng(4).standard_normal((2, 5, 16)).astype(np.float32)
    want = O.attention(x, p, 4, causal=False)
    X = be.from_slice(x, [2, 5, 16])
    P = [be.from_slice(t, list(t.shape)) for t in p]

    def lin(inp, w, b):
        return be.add(be.matmul(inp, w), b)

    def heads(t):
        return be.transpose(be.reshape(t, [2, 5, 4, 4]), 1, 2)

    q, k, v = heads(lin(X, P[0], P[1])), heads(lin(X, P[2], P[3])), heads(lin(X, P[4], P[5]))
    s = be.matmul(q, be.transpose(k, 2, 3))
    s = be.mul(s, be.from_slice([0.5], []))
    a = be.matmul(be.softmax(s), v)
    a = be.reshape(be.transpose(a, 1, 2), [2, 5, 16])
    got = arr(be, lin(a, P[6], P[7]))
    assert np.abs(got - want).max() < 1e-6


def test_tensor_core_projection_with_a_ragged_last_k_block(backend):
    """K need not be a multiple of the kernel's 64-wide k-blocks (a tensor-parallel shard of the hidden layer can be
    800 wide): the last block is zero-filled by the tensor maps.  The check runs inside the library (rg_debug_hook 8)."""
    import ctypes as C
    from rustygradients_b200 import _lib
    lib = _lib.load()
    for K in (64, 72, 192, 800, 1600, 3208):
        _lib.check(lib.rg_debug_hook(backend._ctx, None, 8, K))
    with pytest.raises(rg.InvalidInput):
        _lib.check(lib.rg_debug_hook(backend._ctx, None, 8, 100))
