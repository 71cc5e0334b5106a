"""CPU checks of the oracle itself: it must agree with the numpy formulas the reference's
own tests use (eigenmat/test.py:10-76, cudamat/test_cudamat.py) before anything is
compared against it, and with the committed golden fixtures."""
import os

import numpy as np
import pytest

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_philox_known_answers(oracle):
    # Published known-answer vectors of Philox4x32-10 (Random123 distribution).
    kat = [
        ([0, 0, 0, 0], [0, 0], [0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8]),
        ([0xffffffff] * 4, [0xffffffff] * 2, [0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd]),
        ([0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344], [0xa4093822, 0x299f31d0],
         [0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1]),
    ]
    for ctr, key, want in kat:
        assert oracle.philox4x32_10(ctr, key) == want


def test_philox_stream_matches_golden_and_layout(oracle):
    g = np.load(os.path.join(GOLDEN, "philox.npz"))
    oracle.EigenMatrix.init_random(seed=12345)
    u = oracle.empty((37, 10)).fill_with_rand().asarray()
    n = oracle.empty((37, 10)).fill_with_randn().asarray()
    assert np.array_equal(u, g["u"])
    np.testing.assert_allclose(n, g["n"], rtol=0, atol=1e-6)
    # element (r, c) takes word c & 3 of philox(r, c >> 2, call, seed), mapped to (0, 1]
    w = oracle.philox4x32_10([5, 7 >> 2, 0, 0], [12345, 0])
    assert u[5, 7] == np.float32((np.float32(w[7 & 3]) + np.float32(1)) * np.float32(2.0 ** -32))
    assert u.min() > 0 and u.max() <= 1
    # a shard starting at global column 8 sees columns 8.. of the global stream
    oracle.EigenMatrix.init_random(seed=7, col0=0)
    full = oracle.empty((5, 14)).fill_with_rand().asarray().copy()
    oracle.EigenMatrix.init_random(seed=7, col0=8)
    shard = oracle.empty((5, 6)).fill_with_rand().asarray()
    assert np.array_equal(shard, full[:, 8:14])
    assert np.array_equal(shard, g["u_col0_8"])
    oracle.EigenMatrix.init_random(seed=0, col0=0)


def test_add_like_reference_test(oracle):
    # eigenmat/test.py:10-21
    rng = np.random.default_rng(1)
    x, y = rng.standard_normal((10, 10)), rng.standard_normal((10, 10))
    z = oracle.empty((10, 10))
    oracle.EigenMatrix(x).add(oracle.EigenMatrix(y), target=z)
    assert ((z.asarray() - (x + y)) ** 2).sum() < 1e-10


@pytest.mark.parametrize("shape", [(500, 1000, 600), (128, 256, 64), (7, 5, 3)])
def test_dot_like_reference_tests(oracle, shape):
    # eigenmat/test.py:23-47, cudamat/test_cudamat.py:796-846
    m, k, n = shape
    rng = np.random.default_rng(2)
    x, y = rng.standard_normal((m, k)), rng.standard_normal((k, n))
    ex, ey = oracle.EigenMatrix(x), oracle.EigenMatrix(y)
    z = oracle.dot(ex, ey)
    assert ((z.asarray() - x.dot(y)) ** 2).sum() < 1e-3
    yt = oracle.EigenMatrix(y.T)
    z2 = oracle.dot(ex, yt.T)
    assert ((z2.asarray() - x.dot(y)) ** 2).sum() < 1e-3
    xt = oracle.EigenMatrix(x.T)
    z3 = oracle.dot(xt.T, ey)
    assert ((z3.asarray() - x.dot(y)) ** 2).sum() < 1e-3
    # add_dot / subtract_dot (cudamat/test_cudamat.py:829-880)
    base = rng.standard_normal((m, n))
    acc = oracle.EigenMatrix(base)
    acc.add_dot(ex, ey)
    np.testing.assert_allclose(acc.asarray(), base + x.dot(y), rtol=1e-3, atol=1e-3)
    acc.subtract_dot(ex, ey)
    np.testing.assert_allclose(acc.asarray(), base, rtol=1e-3, atol=1e-3)


def test_sum_by_axis_like_reference_test(oracle):
    # eigenmat/test.py:49-63
    rng = np.random.default_rng(3)
    x = 1.1 + rng.standard_normal((10, 1000))
    ex = oracle.EigenMatrix(x)
    y, z = oracle.empty((1, 1000)), oracle.empty((10, 1))
    ex.sum(axis=0, target=y)
    ex.sum(axis=1, target=z)
    assert ((y.asarray() - x.sum(axis=0).reshape(1, -1)) ** 2).sum() < 1e-5
    assert ((z.asarray() - x.sum(axis=1).reshape(-1, 1)) ** 2).sum() < 1e-4
    # add_sums with a multiplier (cudamat/test_cudamat.py:329-354)
    t = oracle.EigenMatrix(np.ones((10, 1)))
    t.add_sums(ex, axis=1, mult=-2.0)
    np.testing.assert_allclose(t.asarray(), 1 - 2 * x.sum(axis=1).reshape(-1, 1), rtol=1e-4)
    assert abs(ex.sum() - x.sum()) < 1e-2


def test_softmax_like_reference_test(oracle):
    # eigenmat/test.py:65-76
    rng = np.random.default_rng(4)
    x = rng.standard_normal((100, 10))
    y = oracle.empty((100, 10))
    oracle.EigenMatrix(x).apply_softmax(target=y)
    want = np.exp(x - x.max(axis=0))
    want /= want.sum(axis=0)
    assert ((y.asarray() - want) ** 2).sum() < 1e-10


def test_elementwise_and_broadcast_like_reference_tests(oracle):
    # cudamat/test_cudamat.py:162-266, 476-493, 613-627 (tolerance 1e-4 as there)
    rng = np.random.default_rng(5)
    a = rng.standard_normal((256, 128)).astype(np.float32)
    col = rng.standard_normal((256, 1)).astype(np.float32)
    row = rng.standard_normal((1, 128)).astype(np.float32)
    A, C, R = oracle.EigenMatrix(a), oracle.EigenMatrix(col), oracle.EigenMatrix(row)
    t = oracle.empty(a.shape)
    A.add_col_vec(C, target=t); assert np.abs(t.asarray() - (a + col)).max() < 1e-4
    A.add_col_mult(C, 0.5, target=t); assert np.abs(t.asarray() - (a + 0.5 * col)).max() < 1e-4
    A.add_row_vec(R, target=t); assert np.abs(t.asarray() - (a + row)).max() < 1e-4
    A.add_row_mult(R, -2.0, target=t); assert np.abs(t.asarray() - (a - 2 * row)).max() < 1e-4
    A.mult_by_col(C, target=t); assert np.abs(t.asarray() - a * col).max() < 1e-4
    A.mult_by_row(R, target=t); assert np.abs(t.asarray() - a * row).max() < 1e-4
    A.div_by_row(R, target=t); assert np.abs(t.asarray() - a / row).max() < 1e-2
    oracle.sigmoid(A, target=t); assert np.abs(t.asarray() - 1 / (1 + np.exp(-a))).max() < 1e-6
    b = rng.standard_normal((256, 128)).astype(np.float32)
    A2 = oracle.EigenMatrix(a); A2.add_mult(oracle.EigenMatrix(b), 1.5)
    assert np.abs(A2.asarray() - (a + 1.5 * b)).max() < 1e-5
    m = oracle.EigenMatrix(a).max(axis=0); assert np.array_equal(m.asarray(), a.max(axis=0).reshape(1, -1))
    assert abs(oracle.EigenMatrix(a).euclid_norm() - np.sqrt((a.astype(np.float64) ** 2).sum())) < 1e-2
    assert abs(oracle.vdot(oracle.EigenMatrix(a), oracle.EigenMatrix(b)) - (a.astype(np.float64) * b).sum()) < 1e-2


def test_sampling_ops_semantics(oracle):
    # eigenmat/eigenmat.cc:195-204 (p > u), :238-247 (-p / log u), :641-685 (first maximum wins)
    p = np.array([[0.2, 0.5], [0.5, 1.0]], np.float32)
    u = np.array([[0.2, 0.4999], [0.5001, 1.0]], np.float32)
    s = oracle.EigenMatrix(p).sample_bernoulli(target=oracle.empty((2, 2)), uniforms=oracle.EigenMatrix(u))
    assert np.array_equal(s.asarray(), np.array([[0, 1], [0, 0]], np.float32))
    x = np.array([[1, 3], [3, 3], [2, 1]], np.float32)
    oh = oracle.EigenMatrix(x).choose_max(axis=0, target=oracle.empty((3, 2)))
    assert np.array_equal(oh.asarray(), np.array([[0, 1], [1, 0], [0, 0]], np.float32))
    acc = oracle.EigenMatrix(np.ones((3, 2)))
    oracle.EigenMatrix(x).choose_max_and_accumulate(acc)
    assert np.array_equal(acc.asarray(), np.array([[1, 2], [2, 1], [1, 1]], np.float32))
    pp = oracle.EigenMatrix(p).perturb_prob_for_softmax_sampling(target=oracle.empty((2, 2)),
                                                                 uniforms=oracle.EigenMatrix(u))
    with np.errstate(divide="ignore"):
        np.testing.assert_allclose(pp.asarray(), -p / np.log(u), rtol=1e-6)


def test_momentum_update_equals_call_sequence(oracle):
    # deepnet/dbm.py:254 + deepnet/parameter.py:89-106 issued call by call vs the one-pass form
    rng = np.random.default_rng(6)
    w0, d0, s0 = (rng.standard_normal((33, 17)).astype(np.float32) for _ in range(3))
    w, d, g, s = (oracle.EigenMatrix(x) for x in (w0, d0, np.zeros_like(w0), s0))
    g.add_mult(s, -1.0 / 100)
    d.mult(0.7)
    d.add_mult(w, 2e-4)
    d.add_mult_sign(w, 1e-3)
    d.add_mult(g)
    w.add_mult(d, -0.1)
    w2, d2, g2 = oracle.EigenMatrix(w0), oracle.EigenMatrix(d0), oracle.EigenMatrix(np.zeros_like(w0))
    w2.momentum_update(d2, g2, oracle.EigenMatrix(s0), 1.0 / 100, 0.7, 0.1, l2=2e-4, l1=1e-3)
    assert np.array_equal(w.asarray(), w2.asarray())
    assert np.array_equal(d.asarray(), d2.asarray())
    assert not g2.asarray().any()


def test_reference_uniform_generator_is_degenerate_on_lp64(oracle):
    # eigenmat/ziggurat.cc:344-358 compiled in place: documents why uniforms are injected.
    so = os.path.join(os.path.dirname(oracle.__file__), "_ref", "libziggurat_ref.so")
    if not os.path.exists(so):
        pytest.skip("reference generator not built (reference tree not mounted at build time)")
    u = oracle.reference_r4_uni(2, 1000)
    assert (u == np.float32(0.5)).mean() > 0.9


@pytest.mark.parametrize("name,config,scale,cases,steps", [
    ("cd1_c0.npz", 0, 0.25, 300, 3), ("cd1_c1.npz", 1, 0.0625, 768, 3), ("pcd_c3.npz", 3, 0.1, 200, 2)])
def test_training_trace_matches_golden(oracle, name, config, scale, cases, steps):
    from deepnet_b200 import configs, dbm
    g = np.load(os.path.join(GOLDEN, name))
    cfg = configs.build(config, cases=cases, dims_scale=scale)
    B = cfg["batchsize"]
    m = dbm.DBM(oracle, cfg["layers"], cfg["edges"], cfg["hyperparams"], B, cfg["optimizer"], seed=cfg["seed"])
    data = oracle.CUDAMatrix(cfg["data"])
    losses = []
    for step in range(steps):
        s = (step % (cases // B)) * B
        m.SetBatch([data.slice(s, s + B)])
        losses.append(m.TrainOneBatch(step)[0])
    np.testing.assert_allclose(losses, g["losses"], rtol=1e-4)
    for i, e in enumerate(m.edge):
        np.testing.assert_allclose(e.params["weight"].asarray(), g["W%d" % i], rtol=0, atol=2e-5)


def test_cd_learning_reduces_reconstruction_error(oracle):
    from deepnet_b200 import configs, dbm
    cfg = configs.build(0, cases=500, dims_scale=0.25)
    B = cfg["batchsize"]
    m = dbm.DBM(oracle, cfg["layers"], cfg["edges"], cfg["hyperparams"], B, cfg["optimizer"], seed=cfg["seed"])
    data = oracle.CUDAMatrix(cfg["data"])
    losses = []
    for step in range(20):
        s = (step % 5) * B
        m.SetBatch([data.slice(s, s + B)])
        losses.append(m.TrainOneBatch(step)[0])
    assert losses[-1] < 0.5 * losses[0]


def _numpy_twin_cd1(w_vh, w_v, w_h, v_true, uniforms, epsilon):
    """One minibatch of the reference's numpy RBM example (cudamat/examples/rbm_numpy.py:33-68)
    restated for Python 3 in float64, from zero update history (so its momentum factor does not
    enter) and with the uniforms passed in instead of drawn by np.random.rand (:52)."""
    batch_size = v_true.shape[1]
    v = v_true
    h = 1. / (1 + np.exp(-(np.dot(w_vh.T, v) + w_h)))                    # :44
    wu_vh = np.dot(v, h.T)                                               # :46-48
    wu_v = v.sum(1)[:, np.newaxis]
    wu_h = h.sum(1)[:, np.newaxis]
    h = 1. * (h > uniforms)                                              # :51
    v = 1. / (1 + np.exp(-(np.dot(w_vh, h) + w_v)))                      # :54-55
    h = 1. / (1 + np.exp(-(np.dot(w_vh.T, v) + w_h)))
    wu_vh = wu_vh - np.dot(v, h.T)                                       # :57-59
    wu_v = wu_v - v.sum(1)[:, np.newaxis]
    wu_h = wu_h - h.sum(1)[:, np.newaxis]
    new = (w_vh + epsilon / batch_size * wu_vh, w_v + epsilon / batch_size * wu_v,   # :62-64
           w_h + epsilon / batch_size * wu_h)
    return dict(wu_vh=wu_vh, wu_v=wu_v, wu_h=wu_h, v=v, h=h, new=new, err=np.mean((v - v_true) ** 2))   # :66


def test_cd1_step_matches_the_reference_numpy_twin(oracle):
    """The one numerical twin of a CD-1 step the reference holds is its numpy RBM example.  From zero
    update history, without weight decay and with momentum-free first step, the deepnet call
    sequence restated in deepnet_b200/dbm.py over the oracle must give the example's positive minus
    negative statistics, reconstruction and first parameter update."""
    from deepnet_b200 import dbm, synthetic
    V, H, B, seed, eps = 96, 80, 40, 77, 0.05
    rng = np.random.default_rng(9)
    w = (rng.standard_normal((V, H)) * 0.1).astype(np.float32)
    bv = (rng.standard_normal((V, 1)) * 0.1).astype(np.float32)
    bh = (rng.standard_normal((H, 1)) * 0.1).astype(np.float32)
    data, _ = synthetic.binary_data(V, B, 5)
    hyp = dbm.Hyperparams(base_epsilon=eps, initial_momentum=0.9, final_momentum=0.9, gibbs_steps=1)
    layers = [dict(name="v", activation=dbm.LOGISTIC, numdims=V, is_input=True, bias=bv),
              dict(name="h", activation=dbm.LOGISTIC, numdims=H, bias=bh)]
    m = dbm.DBM(oracle, layers, [dict(node1="v", node2="h", weight=w)], hyp, B, dbm.CD, seed=seed)
    m.SetBatch([oracle.CUDAMatrix(data)])
    loss = m.TrainOneBatch(0)[0]
    # the hidden draw is the first sampling call of the step: its uniforms are call 0 of the stream
    oracle.EigenMatrix.init_random(seed=seed)
    u = np.array(oracle.empty((H, B)).fill_with_rand().asarray(), np.float64)
    twin = _numpy_twin_cd1(w.astype(np.float64), bv.astype(np.float64), bh.astype(np.float64),
                           data.astype(np.float64), u, eps)
    e, lv, lh = m.edge[0], m.GetLayerByName("v"), m.GetLayerByName("h")
    scale = np.abs(twin["wu_vh"]).max()
    assert np.abs(e.suff_stats.asarray() - twin["wu_vh"]).max() < 1e-5 * max(scale, 1.0)
    assert np.abs(lv.suff_stats.asarray() - twin["wu_v"]).max() < 1e-5 * B
    assert np.abs(lh.suff_stats.asarray() - twin["wu_h"]).max() < 1e-5 * B
    assert np.abs(lv.state.asarray() - twin["v"]).max() < 1e-6        # reconstruction (mean-field)
    assert np.abs(lh.state.asarray() - twin["h"]).max() < 1e-6
    assert abs(loss / (V * B) - twin["err"]) < 1e-6                    # summed vs mean squared error
    assert np.abs(e.params["weight"].asarray() - twin["new"][0]).max() < 1e-6
    assert np.abs(lv.params["bias"].asarray() - twin["new"][1]).max() < 1e-6
    assert np.abs(lh.params["bias"].asarray() - twin["new"][2]).max() < 1e-6


def test_norm_limit_follows_the_cudamat_kernel(oracle):
    # cudamat/cudamat_kernels.cu:1068-1088: factor 1 below the limit, norm / length above it
    x = np.array([[3, 0.3], [4, 0.4]], np.float32)
    y = oracle.EigenMatrix(x).norm_limit(1.0, axis=0, target=oracle.empty((2, 2))).asarray()
    np.testing.assert_allclose(y, np.array([[0.6, 0.3], [0.8, 0.4]], np.float32), rtol=1e-6)
    np.testing.assert_array_equal(oracle.EigenMatrix(x).transpose().asarray(), x.T)


def test_softmax_label_layer_step_runs_on_the_oracle(oracle):
    """The DBM with a softmax label layer (deepnet/softmax_layer.py) through the call-by-call driver:
    one-hot clamping, softmax reconstruction summing to one, one categorical draw per case."""
    from deepnet_b200 import dbm, synthetic
    rng = np.random.default_rng(2)
    V, H, L, B = 24, 16, 5, 12
    hyp = dbm.Hyperparams(base_epsilon=0.05, mf_steps=2, gibbs_steps=2)
    # an input layer feeds its means upward unless sample_input is set (deepnet/dbm.py:217-222)
    layers = [dict(name="v", activation=dbm.LOGISTIC, numdims=V, is_input=True),
              dict(name="y", activation=dbm.SOFTMAX, numdims=L, is_input=True, hyperparams=hyp.copy(sample_input=True)),
              dict(name="h", activation=dbm.LOGISTIC, numdims=H)]
    edges = [dict(node1="v", node2="h", weight=(rng.standard_normal((V, H)) * 0.1).astype(np.float32)),
             dict(node1="y", node2="h", weight=(rng.standard_normal((L, H)) * 0.1).astype(np.float32))]
    m = dbm.DBM(oracle, layers, edges, hyp, B, dbm.PCD, seed=4)
    data, _ = synthetic.binary_data(V, B, 3)
    lab = rng.integers(0, L, (1, B)).astype(np.float32)
    m.SetBatch([oracle.CUDAMatrix(data), oracle.CUDAMatrix(lab)])
    losses = m.TrainOneBatch(0)
    assert len(losses) == 2 and all(np.isfinite(losses))
    y = m.GetLayerByName("y")
    onehot = np.zeros((L, B), np.float32)
    onehot[lab[0].astype(int), np.arange(B)] = 1
    # the positive state is the reconstruction at this point: columns of a softmax sum to one
    np.testing.assert_allclose(y.pos_state.asarray().sum(axis=0), np.ones(B), rtol=1e-5)
    assert abs(losses[1] - ((y.pos_state.asarray() - onehot) ** 2).sum()) < 1e-4
    s = y.neg_sample.asarray()
    assert set(np.unique(s)) <= {0.0, 1.0} and np.array_equal(s.sum(axis=0), np.ones(B))
