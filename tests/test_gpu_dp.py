"""Two-GPU data parallelism on the real path: two child processes (one per GPU) train the two
halves of every global minibatch with the fused engine and one NCCL all-reduce of the packed
statistics per update; the result must equal one GPU training the whole minibatch: identical
Bernoulli bits (the random stream is indexed by global column), weights within 1e-5, and
bit-identical replicas.  Skipped when fewer than two GPUs are visible."""
import os
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.parametrize("form,scale,peer", [("derived", 0.5, 0), ("f16", 0.5, 0), ("f16", 0.512, 0), ("derived", 0.512, 1),
                                             ("f16", 0.512, 1), ("derived", 1.02, 1), ("f16", 1.02, 1)])
def test_two_gpu_shards_match_one_gpu(cm, tmp_path, form, scale, peer, monkeypatch):
    if cm._lib.b200_device_count() < 2:
        pytest.skip("needs two GPUs")
    # "f16": the operand form of the big model (aux matrices in scaled half precision, W's exponent
    # kept on each replica by its update kernel), forced here at test size; at scale 0.512 the hidden
    # layer has 256 units, which the data-parallel step cuts into 4 column panels of W (statistics,
    # side-stream all-reduce and update per panel), as it does at full size
    monkeypatch.setenv("B200_RBM_STATE_AUX", "1" if form == "f16" else "0")
    monkeypatch.setenv("B200_RBM_F16", "1" if form == "f16" else "0")
    # peer = 1: the exchange and the update run as one pass over peer memory (plain loads and stores,
    # bounded flag waits) instead of an NCCL all-reduce followed by the update
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", B200_DP_PEER=str(peer))
    if scale == 0.512 and not peer:
        env.update(B200_DP_PANELS="4", B200_DP_PANEL_PRODUCTS="1")
    procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "dp_worker.py"), str(r), "2", str(tmp_path), str(scale)], env=env)
             for r in range(2)]
    try:
        codes = [p.wait(timeout=300) for p in procs]
    finally:
        # a rank that outlives a failed or timed-out peer would sit in its all-reduce on a shared
        # GPU: no child is left behind, whatever happened above
        for p in procs:
            if p.poll() is None:
                p.kill()
                p.wait()
    assert codes == [0, 0]
    r0, r1 = (np.load(os.path.join(tmp_path, "rank%d.npz" % r)) for r in range(2))
    assert int(r0["status"]) == 0 and int(r1["status"]) == 0
    assert int(r0["peer"]) == peer and int(r1["peer"]) == peer
    # 512 hidden units (scale 1.02) are one 256-column tile per rank: the statistics product delivers
    # the panels to their owners itself; 256 units (0.512) are half a tile each: the owners fetch them
    # (800 x 512, not 804 x 512: there one draw of the second update has its uniform within 1e-7 of its
    # probability and falls differently on one GPU and on two, whose sums differ in the last bit)
    want_mode = 0 if not peer else (2 if scale == 1.02 else 1)
    assert int(r0["peer_mode"]) == want_mode and int(r1["peer_mode"]) == want_mode
    assert np.array_equal(r0["W"], r1["W"])                 # replicas stay bit-identical

    from deepnet_b200 import configs
    from deepnet_b200.fused_rbm import FusedRBM
    cfg = configs.build(0, cases=400, dims_scale=scale)
    gb = cfg["batchsize"]
    V, H = cfg["layers"][0]["numdims"], cfg["layers"][1]["numdims"]
    eng = FusedRBM(cm, V, H, gb, cfg["edges"][0]["weight"], cfg["hyperparams"],
                   edge_hyperparams=cfg["edges"][0].get("hyperparams"), binary_data=True, seed=cfg["seed"])
    assert eng.f16 == (form == "f16")
    data = cm.CUDAMatrix(cfg["data"])
    for step in range(3):
        eng.TrainOneBatch(step, data.slice(step * gb, (step + 1) * gb))
    W1 = np.array(eng.W.asarray())
    hs = np.array(eng.h_samp.asarray())
    cm.set_rng_column_offset(0)
    assert np.abs(r0["W"] - W1).max() / np.abs(W1).max() < 1e-5
    assert np.array_equal(np.concatenate([r0["hs"], r1["hs"]], axis=1), hs)
    total = eng.read_loss()
    assert abs(float(r0["loss"]) + float(r1["loss"]) - total) < 1e-5 * total


def test_a_rank_that_does_not_join_makes_the_peer_wait_run_out(cm, tmp_path):
    """Failure detection without a fault: rank 1 stays alive but never enqueues its update; rank 0's
    update waits for rank 1's statistics under a short limit, its kernels return by themselves, the
    status word says which wait gave up (21: statistics never became ready) and the context still works."""
    if cm._lib.b200_device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", B200_DP_PEER="1")
    procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "dp_worker.py"), str(r), "2", str(tmp_path), "1.02", "absent"],
                              env=env) for r in range(2)]
    try:
        codes = [p.wait(timeout=300) for p in procs]
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
                p.wait()
    assert codes == [0, 0]
    r0 = np.load(os.path.join(tmp_path, "rank0.npz"))
    assert int(r0["peer"]) == 1
    assert int(r0["status"]) in (21, 22)
    assert bool(r0["usable"])
