"""DBN stacking (deepnet/dbn.py:202-209) and the representation writer (deepnet/dbm.py:365-398,
extract_rbm_representation.py, DataWriter of deepnet/datahandler.py:636-746): host logic on the CPU
restatement here, the fused forms on the device against it."""
import glob
import os

import numpy as np
import pytest

from deepnet_b200 import configs, dbm, dbn


def get(m):
    return np.array(m.asarray(), copy=True)


def test_get_bytes():
    assert dbn.get_bytes("2K") == 2048 and dbn.get_bytes("1.5M") == int(1.5 * 1024 ** 2) and dbn.get_bytes("123") == 123


def test_shard_writer_names_sizes_and_order(tmp_path):
    rng = np.random.default_rng(0)
    a, b = rng.standard_normal((250, 6)).astype(np.float32), rng.standard_normal((250, 2)).astype(np.float32)
    # 8 floats per case, 4 bytes each: 3200 bytes hold 100 cases -> three shards of 100, 100, 50
    w = dbn.ShardWriter(["h", "y"], str(tmp_path), "3200", [6, 2], 250)
    for s in range(0, 250, 30):                      # minibatches that straddle shard boundaries
        w.submit([a[s:s + 30], b[s:s + 30]])
    assert w.commit() == [250, 250]
    files = sorted(os.path.basename(f) for f in glob.glob(str(tmp_path / "h-*")))
    assert files == ["h-00001-of-00003.npy", "h-00002-of-00003.npy", "h-00003-of-00003.npy"]
    got = np.concatenate([np.load(str(tmp_path / f)) for f in files])
    np.testing.assert_array_equal(got, a)
    np.testing.assert_array_equal(np.concatenate([np.load(f) for f in sorted(glob.glob(str(tmp_path / "y-*")))]), b)
    assert [len(np.load(str(tmp_path / f))) for f in files] == [100, 100, 50]


def _stack(backend, fused_top, steps=3):
    """A 2-layer stack: a fixed lower RBM layer below a top RBM trained with CD-1 on its output."""
    cfg = configs.build(0, cases=300, dims_scale=0.25)
    B = cfg["batchsize"]
    V, H1 = cfg["layers"][0]["numdims"], cfg["layers"][1]["numdims"]
    H2 = 64
    rng = np.random.default_rng(12)
    w1 = cfg["edges"][0]["weight"]
    b1 = (rng.standard_normal(H1) * 0.1).astype(np.float32)
    w2 = (rng.standard_normal((H1, H2)) * 0.01).astype(np.float32)
    hyp = cfg["hyperparams"]
    data = backend.CUDAMatrix(cfg["data"])
    if fused_top:
        from deepnet_b200.fused_rbm import FusedRBM
        top = FusedRBM(backend, H1, H2, B, w2, hyp, seed=cfg["seed"])        # real-valued inputs: not binary
        net = dbn.DBN(backend, [(w1, b1, dbm.LOGISTIC)], top, B, binary_data=True)
        for step in range(steps):
            net.TrainOneBatch(step, data.slice(step * B, (step + 1) * B))
        rep = net.Represent(data)
        return get(top.W), top.read_loss(), rep
    # the reference's form: upward net call by call, the top RBM through the call-by-call driver
    layers = [dict(name="v", activation=dbm.LOGISTIC, numdims=H1, is_input=True),
              dict(name="h", activation=dbm.LOGISTIC, numdims=H2)]
    m = dbm.DBM(backend, layers, [dict(node1="v", node2="h", weight=w2)], hyp, B, dbm.CD, seed=cfg["seed"])
    up = dbn.UpwardNet(backend, [(w1, b1, dbm.LOGISTIC)], B, fused=False)
    loss = 0.0
    for step in range(steps):
        m.SetBatch([up.forward(data.slice(step * B, (step + 1) * B))])
        loss += m.TrainOneBatch(step)[0]
    reps = []
    for i in range(300 // B):
        m.SetBatch([up.forward(data.slice(i * B, (i + 1) * B))])
        m.PositivePhase(train=False)
        reps.append(get(m.GetLayerByName("h").state).T)
    return get(m.edge[0].params["weight"]), loss, np.concatenate(reps, axis=0)


def test_stacked_training_and_extraction_on_the_cpu_restatement(oracle, tmp_path):
    W, loss, rep = _stack(oracle, fused_top=False)
    assert np.isfinite(loss) and rep.shape == (300, 64) and 0 < rep.min() and rep.max() < 1
    # the representation of the whole set, sharded and described for the next stage
    B = 100
    batches = [rep[i:i + B] for i in range(0, 300, B)]
    entries = dbn.extract_representations(lambda b: [b], {"train": (batches, 300)}, ["hidden2"], [64], str(tmp_path),
                                          "rbm2", memory="1G")
    assert entries == [("hidden2_train", os.path.join("train", "hidden2-*-of-*.npy"), 300, 64)]
    got = np.load(str(tmp_path / "train" / "hidden2-00001-of-00001.npy"))
    np.testing.assert_array_equal(got, rep)
    text = open(str(tmp_path / "data.pbtxt")).read()
    assert 'name: "hidden2_train"' in text and "size: 300" in text and "dimensions: 64" in text


@pytest.mark.gpu
def test_stacked_training_on_the_device_matches_the_cpu_restatement(cm, oracle):
    Wg, lg, rg = _stack(cm, fused_top=True)
    Wo, lo, ro = _stack(oracle, fused_top=False)
    assert abs(lg - lo) < 1e-5 * lo
    assert np.abs(Wg - Wo).max() / np.abs(Wo).max() < 1e-5
    assert np.abs(rg - ro).max() < 1e-5
    # the call-by-call upward net on the device equals the fused one
    Wc, lc, rc = _stack(cm, fused_top=False)
    assert np.abs(rc - ro).max() < 1e-5 and abs(lc - lo) < 1e-5 * lo
    assert cm.read_status() == 0
