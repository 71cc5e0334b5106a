"""The device-resident data feed (what GPUCache of deepnet/datahandler.py:259-416 does for the
trainer): on the CPU twin here, and twin-vs-GPU (bit-exact: the feed only moves and scales data);
plus the reference's two index operations (select_columns, swap_columns)."""
import numpy as np
import pytest

from deepnet_b200.datahandler import DeviceFeed


def get(m):
    return np.array(m.asarray(), copy=True)


def _index_ops(backend):
    rng = np.random.default_rng(31)
    a = rng.standard_normal((12, 20)).astype(np.float32)
    g = backend.CUDAMatrix(a)
    idx = np.array([[3, 0, 19, 3, -1]], np.float32)
    t = backend.empty((12, 5))
    g.select_columns(backend.CUDAMatrix(idx), t)
    i1 = np.array([[0, 5, 7]], np.float32)
    i2 = np.array([[10, 2, 19]], np.float32)
    g.swap_columns(backend.CUDAMatrix(i1), backend.CUDAMatrix(i2), target=g)
    return a, get(t), get(g)


def test_index_ops_on_the_oracle(oracle):
    a, sel, swapped = _index_ops(oracle)
    np.testing.assert_array_equal(sel, a[:, [3, 0, 19, 3, 19]])       # cudamat/cudamat.py:1478-1493
    want = a.copy()
    want[:, [0, 5, 7, 10, 2, 19]] = a[:, [10, 2, 19, 0, 5, 7]]          # cudamat/cudamat.py:1496-1512
    np.testing.assert_array_equal(swapped, want)


@pytest.mark.parametrize("n", [1, 2, 3, 5, 64, 100, 1000, 4097, 60000])
def test_epoch_order_is_a_permutation(oracle, n):
    for key in ((0, 0), (9, 1), (9, 2), (123456789, 77)):
        p = oracle.feed_permutation(n, key)
        assert np.array_equal(np.sort(p), np.arange(n))
    if n >= 64:
        a, b = oracle.feed_permutation(n, (9, 1)), oracle.feed_permutation(n, (9, 2))
        assert (a != b).mean() > 0.9 and (a != np.arange(n)).mean() > 0.9        # epochs differ, nothing stays put
        # neighbours in the epoch are not neighbours in storage
        assert (np.abs(np.diff(a)) == 1).mean() < 0.05


def _epochs(backend, n_cases, batch, n_batches, normalize=False, binary=False, randomize=True, last=False):
    rng = np.random.default_rng(5)
    x = (rng.random((n_cases, 40)) < 0.3).astype(np.float32) if binary else rng.standard_normal((n_cases, 40)).astype(np.float32)
    y = rng.integers(0, 10, (n_cases, 1)).astype(np.float32)
    feed = DeviceFeed(backend, [x, y], randomize=randomize, seed=9)
    assert feed.packed[0] == binary
    if normalize:
        feed.SetDataStats(0, x.mean(axis=0), x.std(axis=0))
    out = []
    for _ in range(n_batches):
        b = feed.Get(batch, get_last_piece=last)
        out.append((get(b[0]), get(b[1])))
    return x, y, out, feed


@pytest.mark.parametrize("binary", [False, True])
def test_feed_epochs_visit_every_case_once_and_keep_modalities_aligned(oracle, binary):
    x, y, out, _ = _epochs(oracle, 64, 16, 8, binary=binary)
    orders = []
    for epoch in range(2):
        xs = np.concatenate([o[0] for o in out[4 * epoch:4 * epoch + 4]], axis=1).T
        ys = np.concatenate([o[1] for o in out[4 * epoch:4 * epoch + 4]], axis=1).T
        order = oracle.feed_permutation(64, (9, epoch))
        np.testing.assert_array_equal(xs, x[order])        # every case exactly once, in the epoch's order
        np.testing.assert_array_equal(ys, y[order])        # labels moved with their cases
        orders.append(order)
    assert not np.array_equal(orders[0], orders[1])        # and the next epoch has another order
    # without randomize the stored order is kept
    x2, _, out2, _ = _epochs(oracle, 64, 16, 4, randomize=False)
    np.testing.assert_array_equal(np.concatenate([o[0] for o in out2], axis=1).T, x2)
    # short tails are skipped (datahandler.py:403-409) unless asked for
    _, _, out3, _ = _epochs(oracle, 40, 16, 3)
    assert all(o[0].shape[1] == 16 for o in out3)
    _, _, out4, _ = _epochs(oracle, 40, 16, 4, last=True)
    assert [o[0].shape[1] for o in out4] == [16, 16, 8, 16]


def test_feed_normalises_while_gathering(oracle):
    x, _, out, feed = _epochs(oracle, 32, 32, 1, normalize=True)
    want = ((x - x.mean(axis=0)) / (np.float32(1e-10) + x.std(axis=0)))[feed.order()]
    np.testing.assert_allclose(out[0][0].T, want, rtol=1e-5, atol=1e-6)


@pytest.mark.gpu
def test_index_ops_match_the_oracle_on_gpu(cm, oracle):
    for a, b in zip(_index_ops(cm)[1:], _index_ops(oracle)[1:]):
        np.testing.assert_array_equal(a, b)
    # out-of-range indices: NaN columns on select, skipped on swap
    g = cm.CUDAMatrix(np.ones((8, 4), np.float32))
    t = cm.empty((8, 2))
    g.select_columns(cm.CUDAMatrix(np.array([[1, 9]], np.float32)), t)
    r = get(t)
    assert (r[:, 0] == 1).all() and np.isnan(r[:, 1]).all()
    # large, 128-bit path: 8192-row columns
    rng = np.random.default_rng(1)
    big = rng.standard_normal((8192, 300)).astype(np.float32)
    perm = rng.permutation(300)
    gb, ob = cm.CUDAMatrix(big), oracle.CUDAMatrix(big)
    for m, be in ((gb, cm), (ob, oracle)):
        m.swap_columns(be.CUDAMatrix(perm[:150].reshape(1, -1)), be.CUDAMatrix(perm[150:].reshape(1, -1)), target=m)
    np.testing.assert_array_equal(get(gb), get(ob))


@pytest.mark.gpu
@pytest.mark.parametrize("binary,normalize", [(False, False), (False, True), (True, False)])
def test_feed_matches_its_cpu_twin_on_gpu(cm, oracle, binary, normalize):
    _, _, go, gfeed = _epochs(cm, 100, 16, 14, normalize=normalize, binary=binary)
    _, _, oo, _ = _epochs(oracle, 100, 16, 14, normalize=normalize, binary=binary)
    for (gx, gy), (ox, oy) in zip(go, oo):
        np.testing.assert_array_equal(gx, ox)              # same arithmetic, same order: the same bits
        np.testing.assert_array_equal(gy, oy)
    for n in (1, 3, 100, 4097):
        np.testing.assert_array_equal(cm.feed_permutation(n, (9, 3)), oracle.feed_permutation(n, (9, 3)))
    assert cm.read_status() == 0


@pytest.mark.gpu
def test_bit_packed_feed_drives_the_half_precision_engine(cm, monkeypatch):
    """A 0/1 data set stored one bit per value: the gather expands a minibatch and writes its
    half-precision form in the same pass; the engine fed this way gives the bits it gives on
    the same minibatches uploaded as fp32."""
    from deepnet_b200 import configs
    from deepnet_b200.fused_rbm import FusedRBM
    monkeypatch.setenv("B200_RBM_STATE_AUX", "1")
    monkeypatch.setenv("B200_RBM_F16", "1")
    cfg = configs.build(0, cases=512, dims_scale=0.25)
    B = cfg["batchsize"]
    V, H = cfg["layers"][0]["numdims"], cfg["layers"][1]["numdims"]
    feed = DeviceFeed(cm, [cfg["data"].T], randomize=True, seed=4, aux_mode=2, aux_exp=14)
    assert feed.packed == [True] and feed.data[0].shape == ((V + 31) // 32, 512)
    mk = lambda: FusedRBM(cm, V, H, B, cfg["edges"][0]["weight"], cfg["hyperparams"],
                          edge_hyperparams=cfg["edges"][0].get("hyperparams"), binary_data=True, seed=cfg["seed"])
    eng = mk()
    order = feed.order()
    for step in range(4):
        (batch,) = feed.Get(B)
        np.testing.assert_array_equal(get(batch), cfg["data"][:, order[step * B:(step + 1) * B]])
        eng.TrainOneBatch(step, batch, data_aux=feed.last_aux)
    ref = mk()
    for step in range(4):
        ref.TrainOneBatch(step, cm.CUDAMatrix(cfg["data"][:, order[step * B:(step + 1) * B]]))
    np.testing.assert_array_equal(get(eng.W), get(ref.W))
    assert eng.read_loss() == ref.read_loss()
    assert cm.read_status() == 0
