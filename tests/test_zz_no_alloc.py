"""GPU check of add_sum_by_axis_noalloc, the row/column-sum entry point for callers that
may not allocate device memory (a host whose own pool owns the GPU, or one that cannot
afford the device-wide synchronisation of an allocation): it must give what add_sum_by_axis
gives, on two calls in a row that share its fixed scratch array, and refuse matrices whose
partial sums do not fit.  Collected last on purpose, so a run that stops at the first failure
has already run every other test; it also passes alone in a fresh process."""
import ctypes as ct

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def get(m):
    return np.array(m.asarray(), copy=True)


def test_noalloc_sums_match_the_allocating_entry_point_twice_in_a_row(cm):
    rng = np.random.default_rng(2024)
    # (rows, cols): split row sums (scratch in use), a single-split case, column sums
    cases = [((8192, 1024), 1, -1.0), ((500, 4097), 1, 0.5), ((96, 64), 1, 2.0), ((1000, 300), 0, 1.5)]
    for (shape, axis, mult) in cases:
        a = (1.1 + rng.standard_normal(shape)).astype(np.float32)
        g = cm.CUDAMatrix(a)
        n = shape[0] if axis == 1 else shape[1]
        init = rng.standard_normal((n, 1) if axis == 1 else (1, n)).astype(np.float32)
        want = cm.CUDAMatrix(init)
        want.add_sums(g, axis=axis, mult=mult)
        for _ in range(2):                       # the second call reuses whatever the first left behind
            got = cm.CUDAMatrix(init)
            got.add_sums_noalloc(g, axis=axis, mult=mult)
            np.testing.assert_allclose(get(got), get(want), rtol=1e-5, atol=1e-3)   # the bound of the axis-sum tests
        ref = init + mult * a.astype(np.float64).sum(axis=1 if axis == 1 else 0).reshape(init.shape)
        np.testing.assert_allclose(get(want), ref, rtol=1e-5, atol=2e-3)


def test_noalloc_back_to_back_calls_on_different_matrices(cm):
    rng = np.random.default_rng(7)
    a = rng.standard_normal((4096, 2048)).astype(np.float32)
    b = rng.standard_normal((2048, 512)).astype(np.float32)
    ga, gb = cm.CUDAMatrix(a), cm.CUDAMatrix(b)
    ta, tb = cm.empty((4096, 1)), cm.empty((2048, 1))
    ta.add_sums_noalloc(ga, axis=1)               # both enqueued before either result is read
    tb.add_sums_noalloc(gb, axis=1)
    wa, wb = cm.empty((4096, 1)), cm.empty((2048, 1))
    wa.add_sums(ga, axis=1)
    wb.add_sums(gb, axis=1)
    np.testing.assert_allclose(get(ta), get(wa), rtol=1e-5, atol=1e-3)
    np.testing.assert_allclose(get(tb), get(wb), rtol=1e-5, atol=1e-3)


def test_noalloc_refuses_what_does_not_fit_and_bad_shapes(cm):
    # 17000 rows need 2 column splits on a 148-SM device: 34000 partial sums > 32768
    g = cm.empty((17000, 256))
    t = cm.empty((17000, 1))
    with pytest.raises(cm.CUDAMatException):
        t.add_sums_noalloc(g, axis=1)
    t.add_sums(g, axis=1)                         # the allocating entry point still takes it
    assert cm._lib.add_sum_by_axis_noalloc(g.p_mat, cm.empty((5, 1)).p_mat, ct.c_int(1), ct.c_float(1.0)) == -1
    assert cm.read_status() == 0
