"""Regenerates the fixtures in this folder:  python tests/golden/make_golden.py

The reference ships no golden vectors for the contrastive-divergence path (its tests
compare against numpy formulas on random inputs), and its Python is Python-2 only, so
it cannot be imported to produce any.  These fixtures are therefore regression pins
produced by the CPU oracle (oracle/eigenmat_port.c through oracle/eigenmat_oracle.py):
the CUDA library is checked against them on the GPU box, where neither the reference
tree nor this script's inputs are needed.

  philox.npz    uniforms / normals of the shared Philox4x32-10 stream for fixed (seed, call)
  cd1_c0.npz    a 3-step CD-1 trace of a small binary RBM (config 0 at 1/4 size)
  cd1_c1.npz    the same for a small Gaussian-visible RBM (config 1 at 1/16 size)
  pcd_c3.npz    a 2-step PCD trace of a small 3-layer DBM (config 3 at 1/10 size)
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import eigenmat_oracle as em  # noqa: E402
from deepnet_b200 import configs, dbm  # noqa: E402


def philox():
    em.EigenMatrix.init_random(seed=12345)
    u = em.empty((37, 10)).fill_with_rand().asarray().copy()
    n = em.empty((37, 10)).fill_with_randn().asarray().copy()
    em.EigenMatrix.init_random(seed=7, col0=8)
    u8 = em.empty((5, 6)).fill_with_rand().asarray().copy()
    np.savez(os.path.join(HERE, "philox.npz"), u=u, n=n, u_col0_8=u8)


def trace(config, scale, cases, steps, name):
    cfg = configs.build(config, cases=cases, dims_scale=scale)
    B = cfg["batchsize"]
    m = dbm.DBM(em, cfg["layers"], cfg["edges"], cfg["hyperparams"], B, cfg["optimizer"], seed=cfg["seed"])
    data = em.CUDAMatrix(cfg["data"])
    out = {"losses": []}
    for step in range(steps):
        s = (step % (cases // B)) * B
        m.SetBatch([data.slice(s, s + B)])
        out["losses"].append(m.TrainOneBatch(step)[0])
    for i, e in enumerate(m.edge):
        out["W%d" % i] = e.params["weight"].asarray().copy()
        out["dW%d" % i] = e.gradient_history.asarray().copy()
    for l in m.layer:
        out["b_" + l.name] = l.params["bias"].asarray().copy()
        out["state_" + l.name] = l.state.asarray().copy()
    out["losses"] = np.array(out["losses"], np.float64)
    np.savez_compressed(os.path.join(HERE, name), **out)


if __name__ == "__main__":
    philox()
    trace(0, 0.25, 300, 3, "cd1_c0.npz")
    trace(1, 0.0625, 768, 3, "cd1_c1.npz")
    trace(3, 0.1, 200, 2, "pcd_c3.npz")
    print("wrote", sorted(f for f in os.listdir(HERE) if f.endswith(".npz")))
