"""The device-resident data feed (GPUCache semantics of deepnet/datahandler.py:259-416) and its
two index operations: on the oracle here, and oracle-vs-GPU (bit-exact, they only move data)."""
import numpy as np
import pytest

from deepnet_b200.datahandler import GPUCache, HostSource


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


def _epochs(backend, n_cases, capacity, batch, n_batches, normalize=False):
    rng = np.random.default_rng(5)
    x = rng.standard_normal((n_cases, 16)).astype(np.float32)
    y = rng.integers(0, 10, (n_cases, 1)).astype(np.float32)
    cache = GPUCache(backend, HostSource([x, y]), capacity, randomize=True, seed=9)
    if normalize:
        cache.SetDataStats(0, x.mean(axis=0), x.std(axis=0))
    out = []
    for _ in range(n_batches):
        b = cache.Get(batch)
        out.append((get(b[0]), get(b[1])))
    return x, y, out


def test_cache_epochs_shuffle_in_place_and_keep_modalities_aligned(oracle):
    x, y, out = _epochs(oracle, 64, 64, 16, 8)
    for epoch in range(2):
        xs = np.concatenate([o[0] for o in out[4 * epoch:4 * epoch + 4]], axis=1).T
        ys = np.concatenate([o[1] for o in out[4 * epoch:4 * epoch + 4]], axis=1).T
        order = [int(np.where((x == row).all(axis=1))[0][0]) for row in xs]
        assert sorted(order) == list(range(64))            # every case exactly once per epoch
        np.testing.assert_array_equal(ys, y[order])        # labels moved with their cases
        assert order != list(range(64))                    # and the order changed
    # a cache smaller than the data set walks the chunks of its parent without shuffling them
    x2, _, out2 = _epochs(oracle, 64, 32, 16, 4)
    np.testing.assert_array_equal(np.concatenate([o[0] for o in out2], axis=1).T, x2)
    # short tails are skipped (datahandler.py:403-409)
    _, _, out3 = _epochs(oracle, 40, 40, 16, 3)
    assert all(o[0].shape[1] == 16 for o in out3)


def test_cache_normalises_on_load(oracle):
    x, _, out = _epochs(oracle, 32, 32, 32, 1, normalize=True)
    got = out[0][0].T
    want = (x - x.mean(axis=0)) / (1e-10 + x.std(axis=0))
    assert sorted(map(tuple, np.round(got, 4))) == sorted(map(tuple, np.round(want, 4)))


@pytest.mark.gpu
def test_index_ops_and_cache_match_the_oracle_on_gpu(cm, oracle):
    for a, b in zip(_index_ops(cm)[1:], _index_ops(oracle)[1:]):
        np.testing.assert_array_equal(a, b)
    # out-of-range indices: NaN columns on select, skipped on swap
    g = cm.CUDAMatrix(np.ones((8, 4), np.float32))
    t = cm.empty((8, 2))
    g.select_columns(cm.CUDAMatrix(np.array([[1, 9]], np.float32)), t)
    r = get(t)
    assert (r[:, 0] == 1).all() and np.isnan(r[:, 1]).all()
    _, _, go = _epochs(cm, 64, 64, 16, 8, normalize=True)
    _, _, oo = _epochs(oracle, 64, 64, 16, 8, normalize=True)
    for (gx, gy), (ox, oy) in zip(go, oo):
        np.testing.assert_allclose(gx, ox, rtol=1e-6, atol=1e-6)
        np.testing.assert_array_equal(gy, oy)
    # large, 128-bit path: 8192-row columns
    rng = np.random.default_rng(1)
    big = rng.standard_normal((8192, 300)).astype(np.float32)
    perm = rng.permutation(300)
    gb, ob = cm.CUDAMatrix(big), oracle.CUDAMatrix(big)
    for m, be in ((gb, cm), (ob, oracle)):
        m.swap_columns(be.CUDAMatrix(perm[:150].reshape(1, -1)), be.CUDAMatrix(perm[150:].reshape(1, -1)), target=m)
    np.testing.assert_array_equal(get(gb), get(ob))
