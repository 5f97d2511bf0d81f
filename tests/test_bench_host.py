"""Host-side pieces of bench.py that need no GPU."""
import importlib.util
import os

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_pooled_params_are_deterministic_windows():
    b = _bench()
    V = 301
    shapes = [(V, 64), (16, 64), (1, 64), (64, 192), (1, 192), (64, V), (1, V)]
    p1, p2 = b._pooled_params(shapes, V, 7), b._pooled_params(shapes, V, 7)
    assert [p.shape for p in p1] == shapes
    assert all(np.array_equal(a, c) for a, c in zip(p1, p2))               # every rank builds the same list
    assert all(p.dtype == np.float32 and p.flags["C_CONTIGUOUS"] for p in p1)
    assert np.array_equal(p1[2], np.ones((1, 64), np.float32)) and np.array_equal(p1[4], np.ones((1, 192), np.float32))
    assert p1[6].std() > 0 and abs(float(p1[0].std()) - 0.02) < 2e-3        # LM-head bias and matrices are draws
    assert not np.array_equal(p1[3].reshape(-1)[:64], p1[5].reshape(-1)[:64])   # different windows
    assert not np.array_equal(b._pooled_params(shapes, V, 8)[0], p1[0])


def test_bench_entry_points_exist():
    b = _bench()
    assert b.EXTRAS_BUDGET_S >= 120
    for name in ("run_ours", "run_batched", "run_tp", "run_tp_trace", "cpu_reference_tokens_per_s"):
        assert callable(getattr(b, name))
