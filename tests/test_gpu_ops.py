"""GPU parity of the per-operation C ABI against the CPU oracle, through the ctypes
boundary.  Integer/0-1 work (random words, Bernoulli thresholds, arg-max one-hots) is
bit-exact; floating point within the tolerances of cudamat/test_cudamat.py (1e-4
elementwise, 1e-3 sums) or tighter."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

SHAPES = [(256, 128), (1, 1), (7, 5), (100, 3), (1000, 37), (4, 1024)]


def both(cm, oracle, a):
    return cm.CUDAMatrix(a), oracle.EigenMatrix(a)


def get(m):
    return np.array(m.asarray(), copy=True)


@pytest.mark.parametrize("shape", SHAPES)
def test_unary_and_scalar_ops(cm, oracle, shape):
    rng = np.random.default_rng(10)
    a = rng.standard_normal(shape).astype(np.float32) * 3
    g, o = both(cm, oracle, a)
    np.testing.assert_allclose(get(cm.sigmoid(g, target=cm.empty(shape))),
                               get(oracle.sigmoid(o, target=oracle.empty(shape))), rtol=1e-6, atol=1e-7)
    # the whole finite range of exp(-x): saturation at both ends, no NaN
    w = np.linspace(-100, 100, int(np.prod(shape)), dtype=np.float32).reshape(shape)
    gw, ow = both(cm, oracle, w)
    np.testing.assert_allclose(get(cm.sigmoid(gw, target=cm.empty(shape))),
                               get(oracle.sigmoid(ow, target=oracle.empty(shape))), rtol=1e-6, atol=1.2e-38)  # results below the smallest normal are flushed
    np.testing.assert_allclose(get(cm.exp(g, target=cm.empty(shape))), np.exp(a), rtol=1e-6)
    np.testing.assert_allclose(get(cm.log_1_plus_exp(g, target=cm.empty(shape))),
                               get(oracle.log_1_plus_exp(o, target=oracle.empty(shape))), rtol=1e-5, atol=1e-6)
    for name, val in (("mult", 0.37), ("add", -1.5), ("divide", 3.0), ("subtract", 0.25)):
        r1 = getattr(g, name)(val, target=cm.empty(shape))
        r2 = getattr(o, name)(val, target=oracle.empty(shape))
        np.testing.assert_array_equal(get(r1), get(r2))
    np.testing.assert_array_equal(get(g.greater_than(0.1, target=cm.empty(shape))), (a > np.float32(0.1)).astype(np.float32))
    np.testing.assert_array_equal(get(g.sign(target=cm.empty(shape))), np.sign(a))
    t = cm.empty(shape)
    t.assign(2.5)
    assert (get(t) == 2.5).all()
    t.assign(g)
    np.testing.assert_array_equal(get(t), a)


@pytest.mark.parametrize("shape", SHAPES)
def test_binary_ops(cm, oracle, shape):
    rng = np.random.default_rng(11)
    a = rng.standard_normal(shape).astype(np.float32)
    b = rng.standard_normal(shape).astype(np.float32) + 3
    ga, oa = both(cm, oracle, a)
    gb, ob = both(cm, oracle, b)
    for name in ("add", "subtract", "mult", "divide", "less_than", "greater_than"):
        r1 = getattr(ga, name)(gb, target=cm.empty(shape))
        r2 = getattr(oa, name)(ob, target=oracle.empty(shape))
        np.testing.assert_array_equal(get(r1), get(r2), err_msg=name)
    # axpy: the oracle rounds product and sum separately, the GPU may fuse them
    ga.add_mult(gb, 1.5)
    oa.add_mult(ob, 1.5)
    np.testing.assert_allclose(get(ga), get(oa), rtol=1e-6, atol=1e-6)
    ga.add_mult_sign(gb, 0.01)
    oa.add_mult_sign(ob, 0.01)
    np.testing.assert_allclose(get(ga), get(oa), rtol=1e-6, atol=1e-6)


@pytest.mark.parametrize("shape", SHAPES)
def test_broadcasts(cm, oracle, shape):
    rng = np.random.default_rng(12)
    h, w = shape
    a = rng.standard_normal(shape).astype(np.float32)
    col = rng.standard_normal((h, 1)).astype(np.float32) + 2
    row = rng.standard_normal((1, w)).astype(np.float32) + 2
    g, o = both(cm, oracle, a)
    gc, oc = both(cm, oracle, col)
    gr, orow = both(cm, oracle, row)
    for name, gv, ov, extra in (("add_col_vec", gc, oc, ()), ("add_col_mult", gc, oc, (0.5,)),
                                ("add_row_vec", gr, orow, ()), ("add_row_mult", gr, orow, (-1.0,)),
                                ("mult_by_col", gc, oc, ()), ("mult_by_row", gr, orow, ()),
                                ("div_by_col", gc, oc, ()), ("div_by_row", gr, orow, ())):
        r1 = getattr(g, name)(gv, *extra, target=cm.empty(shape))
        r2 = getattr(o, name)(ov, *extra, target=oracle.empty(shape))
        np.testing.assert_allclose(get(r1), get(r2), rtol=1e-6, atol=1e-6, err_msg=name)


@pytest.mark.parametrize("shape", SHAPES + [(500, 100), (8192, 64), (33, 4097)])
def test_reductions(cm, oracle, shape):
    rng = np.random.default_rng(13)
    h, w = shape
    a = (1.1 + rng.standard_normal(shape)).astype(np.float32)
    g, o = both(cm, oracle, a)
    a64 = a.astype(np.float64)
    tol = 1e-3  # cudamat/test_cudamat.py:293
    np.testing.assert_allclose(get(g.sum(axis=0)), a64.sum(axis=0).reshape(1, -1), rtol=1e-5, atol=tol)
    np.testing.assert_allclose(get(g.sum(axis=1)), a64.sum(axis=1).reshape(-1, 1), rtol=1e-5, atol=tol)
    t = cm.CUDAMatrix(np.ones((h, 1), np.float32))
    t.add_sums(g, axis=1, mult=-2.0)
    np.testing.assert_allclose(get(t), 1 - 2 * a64.sum(axis=1).reshape(-1, 1), rtol=1e-5, atol=2 * tol)
    t0 = cm.CUDAMatrix(np.ones((1, w), np.float32))
    t0.add_sums(g, axis=0, mult=0.5)
    np.testing.assert_allclose(get(t0), 1 + 0.5 * a64.sum(axis=0).reshape(1, -1), rtol=1e-5, atol=tol)
    # sums through a transposed handle (cudamat/test_cudamat.py:298-327)
    np.testing.assert_allclose(get(cm.sum(g.T, axis=0)), a64.sum(axis=1).reshape(1, -1), rtol=1e-5, atol=tol)
    np.testing.assert_array_equal(get(g.max(axis=0)), get(o.max(axis=0)))
    np.testing.assert_array_equal(get(g.max(axis=1)), get(o.max(axis=1)))
    assert abs(g.euclid_norm() - o.euclid_norm()) <= 1e-5 * o.euclid_norm() + 1e-6
    assert abs(g.sum() - a64.sum()) <= 1e-5 * np.abs(a64).sum() + 1e-5
    b = rng.standard_normal(shape).astype(np.float32)
    gb = cm.CUDAMatrix(b)
    assert abs(cm.vdot(g, gb) - (a64 * b).sum()) <= 1e-5 * np.abs(a64 * b).sum() + 1e-5
    acc = cm.CUDAMatrix(np.array([[2.0]], np.float32))
    cm._check(cm._lib.add_sq_diff(g.p_mat, gb.p_mat, acc.p_mat))
    want = 2.0 + ((a64 - b) ** 2).sum()
    assert abs(get(acc)[0, 0] - want) <= 1e-5 * want


@pytest.mark.parametrize("shape", [(100, 10), (10000, 7), (5, 300), (1, 4)])
def test_softmax_and_argmax_family(cm, oracle, shape):
    rng = np.random.default_rng(14)
    a = rng.standard_normal(shape).astype(np.float32)
    a[0, 0] = a.max() + 1
    if shape[0] > 2:
        a[2, -1] = a[1, -1] = a[:, -1].max() + 1   # a tie: the first maximum wins
    g, o = both(cm, oracle, a)
    np.testing.assert_allclose(get(g.apply_softmax(target=cm.empty(shape))),
                               get(o.apply_softmax(target=oracle.empty(shape))), rtol=2e-6, atol=1e-9)
    np.testing.assert_array_equal(get(g.choose_max(axis=0, target=cm.empty(shape))),
                                  get(o.choose_max(axis=0, target=oracle.empty(shape))))
    np.testing.assert_array_equal(get(g.argmax(axis=0)), get(o.argmax(axis=0)))
    acc_g, acc_o = both(cm, oracle, np.ones(shape, np.float32))
    g.choose_max_and_accumulate(acc_g)
    o.choose_max_and_accumulate(acc_o)
    np.testing.assert_array_equal(get(acc_g), get(acc_o))
    # in place, as replicated_softmax_layer.py:55 calls it
    g2 = cm.CUDAMatrix(a)
    g2.choose_max(axis=0)
    np.testing.assert_array_equal(get(g2), get(o.choose_max(axis=0, target=oracle.empty(shape))))


@pytest.mark.parametrize("shape,col0", [((37, 10), 0), ((128, 256), 0), ((5, 6), 8), ((1000, 3), 4), ((3, 1), 0)])
def test_random_stream_is_bit_identical_to_the_oracle(cm, oracle, shape, col0):
    seed = 4242
    cm.CUDAMatrix.init_random(seed)
    cm.set_rng_column_offset(col0)
    oracle.EigenMatrix.init_random(seed, col0=col0)
    try:
        u_g = get(cm.empty(shape).fill_with_rand())
        u_o = get(oracle.empty(shape).fill_with_rand())
        np.testing.assert_array_equal(u_g, u_o)
        assert u_g.min() > 0 and u_g.max() <= 1
        n_g = get(cm.empty(shape).fill_with_randn())
        n_o = get(oracle.empty(shape).fill_with_randn())
        np.testing.assert_allclose(n_g, n_o, rtol=0, atol=2e-5)
        # Bernoulli: same probabilities, same uniforms (call 2 of the stream) -> identical bits
        rng = np.random.default_rng(15)
        p = rng.random(shape).astype(np.float32)
        s_g = get(cm.CUDAMatrix(p).sample_bernoulli(target=cm.empty(shape)))
        s_o = get(oracle.EigenMatrix(p).sample_bernoulli(target=oracle.empty(shape)))
        np.testing.assert_array_equal(s_g, s_o)
        assert set(np.unique(s_g)) <= {0.0, 1.0}
        # exponential-race perturbation: log differs in the last ulp between libm and the GPU
        q_g = get(cm.CUDAMatrix(p).perturb_prob_for_softmax_sampling(target=cm.empty(shape)))
        q_o = get(oracle.EigenMatrix(p).perturb_prob_for_softmax_sampling(target=oracle.empty(shape)))
        np.testing.assert_allclose(q_g, q_o, rtol=1e-5)
    finally:
        cm.set_rng_column_offset(0)
        oracle.EigenMatrix.init_random(0, col0=0)


def test_random_moments_like_reference_test(cm):
    # cudamat/test_cudamat.py:882-893
    cm.CUDAMatrix.init_random(1)
    u = get(cm.empty((128, 256)).fill_with_rand())
    n = get(cm.empty((128, 256)).fill_with_randn())
    assert abs(u.mean() - 0.5) < 1e-2 and abs(n.mean()) < 1e-2 and abs(n.var() - 1) < 3e-2


def test_views_slices_reshape_and_errors(cm):
    rng = np.random.default_rng(16)
    a = rng.standard_normal((12, 20)).astype(np.float32)
    g = cm.CUDAMatrix(a)
    s = g.slice(3, 9)                                   # cudamat/test_cudamat.py:148-160
    np.testing.assert_array_equal(get(s), a[:, 3:9])
    s.mult(2.0)                                         # a view writes through to its parent
    a[:, 3:9] *= 2
    np.testing.assert_array_equal(get(g), a)
    assert g.T.shape == (20, 12)
    v = cm.CUDAMatrix(np.arange(10, dtype=np.float32).reshape(10, 1))
    np.testing.assert_array_equal(get(v.slice(2, 5)).ravel(), [2, 3, 4])
    g.reshape((20, 12))                                 # cudamat/test_cudamat.py:12-28
    np.testing.assert_array_equal(get(g), a.reshape((20, 12), order="F"))
    with pytest.raises(cm.CUDAMatException):
        g.reshape((7, 7))
    with pytest.raises(cm.CUDAMatException):
        g.add(cm.empty((3, 3)))
    with pytest.raises(cm.CUDAMatException):
        g.add_col_vec(cm.empty((3, 1)))
    with pytest.raises(cm.CUDAMatException):
        cm.dot(cm.empty((3, 4)), cm.empty((5, 6)))
    with pytest.raises(cm.CUDAMatException):
        g.slice(5, 50)
    g.overwrite(np.ones((20, 12)))
    assert (get(g) == 1).all()
    assert cm.read_status() == 0


@pytest.mark.parametrize("shape", [(33, 17), (500, 784), (1024, 4096), (1, 5)])
def test_transpose_copy_and_norm_limit(cm, oracle, shape):
    # cudamat/cudamat.py:422-433 (copy_transpose) and :1000-1016 (normlimit_by_axis, axis 0)
    rng = np.random.default_rng(31)
    x = rng.standard_normal(shape).astype(np.float32)
    g = cm.CUDAMatrix(x)
    np.testing.assert_array_equal(get(g.transpose()), x.T)
    limit = float(np.median(np.sqrt((x.astype(np.float64) ** 2).sum(axis=0))))
    got = get(g.norm_limit(limit, axis=0, target=cm.empty(shape)))
    want = oracle.EigenMatrix(x).norm_limit(limit, axis=0, target=oracle.empty(shape)).asarray()
    np.testing.assert_allclose(got, want, rtol=2e-6, atol=1e-7)
    lengths = np.sqrt((got.astype(np.float64) ** 2).sum(axis=0))
    assert lengths.max() <= limit * (1 + 1e-5)
    with pytest.raises(cm.CUDAMatException):
        g.norm_limit(limit, axis=1)


def test_ones_vector_is_filled_at_start_up(cm):
    # cudamat/cudamat.py:1879-1885: callers take sums as products with CUDAMatrix.ones
    assert cm.CUDAMatrix.ones is not None and cm.CUDAMatrix.ones.shape == (1024 * 256, 1)
    x = np.arange(12, dtype=np.float32).reshape(3, 4)
    s = cm.dot(cm.CUDAMatrix(x), cm.CUDAMatrix(np.ones((4, 1), np.float32)))
    np.testing.assert_allclose(get(s).ravel(), x.sum(axis=1))
    assert float(np.array(cm.CUDAMatrix.ones.asarray()).min()) == 1.0


@pytest.mark.parametrize("shape", [(8192, 4096), (500, 100), (33, 7), (784, 1), (4, 5000)])
def test_single_launch_statistics(cm, oracle, shape):
    # row_sum_diff = sum(axis=1) then add_sums(axis=1, mult=-1) (deepnet/layer.py:202-213); add_sq_diff twice in a row
    rng = np.random.default_rng(shape[0])
    a = rng.random(shape).astype(np.float32)
    b = rng.random(shape).astype(np.float32)
    ga, gb = cm.CUDAMatrix(a), cm.CUDAMatrix(b)
    want = oracle.EigenMatrix(a).sum(axis=1)
    want.add_sums(oracle.EigenMatrix(b), axis=1, mult=-1.0)
    for _ in range(2):                     # the ticket counters are back at zero after every call
        t = cm.empty((shape[0], 1))
        cm._check(cm._lib.row_sum_diff(ga.p_mat, gb.p_mat, t.p_mat))
        np.testing.assert_allclose(get(t), get(want), rtol=1e-5, atol=1e-5 * shape[1])
    ref = a.astype(np.float64).sum(axis=1) - b.astype(np.float64).sum(axis=1)
    np.testing.assert_allclose(get(t).ravel(), ref, rtol=1e-5, atol=2e-6 * shape[1])
    acc = cm.empty((1, 1))
    for _ in range(2):
        cm._check(cm._lib.add_sq_diff(ga.p_mat, gb.p_mat, acc.p_mat))
    sq = ((a.astype(np.float64) - b) ** 2).sum()
    assert abs(float(get(acc)[0, 0]) - 2 * sq) < 1e-5 * 2 * sq


def test_single_launch_statistics_after_a_shutdown(cm):
    """cublas_shutdown frees the library's scratch, the ticket counters of the single-launch
    reductions with it; the next call gets new, zeroed ones (no pointer kept from before)."""
    rng = np.random.default_rng(9)
    a = rng.random((512, 300)).astype(np.float32)
    b = rng.random((512, 300)).astype(np.float32)
    ga, gb = cm.CUDAMatrix(a), cm.CUDAMatrix(b)
    ref = a.astype(np.float64).sum(axis=1) - b.astype(np.float64).sum(axis=1)
    for cycle in range(2):
        t, acc = cm.empty((512, 1)), cm.empty((1, 1))
        acc.assign(0)
        cm._check(cm._lib.row_sum_diff(ga.p_mat, gb.p_mat, t.p_mat))
        cm._check(cm._lib.add_sq_diff(ga.p_mat, gb.p_mat, acc.p_mat))
        np.testing.assert_allclose(get(t).ravel(), ref, rtol=1e-5, atol=1e-3)
        sq = ((a.astype(np.float64) - b) ** 2).sum()
        assert abs(float(get(acc)[0, 0]) - sq) < 1e-5 * sq
        cm.cublas_shutdown()
        cm.cublas_init()
