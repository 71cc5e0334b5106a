"""Annealed importance sampling (deepnet/ais.py:131-208) on the matrix API: the CPU restatement
against exact enumeration, and the device run against both."""
import numpy as np
import pytest

from deepnet_b200 import ais


def small_rbm(V=12, H=10, scale=0.5, seed=3):
    rng = np.random.default_rng(seed)
    return ((rng.standard_normal((V, H)) * scale).astype(np.float32),
            (rng.standard_normal(H) * 0.3).astype(np.float32), (rng.standard_normal(V) * 0.3).astype(np.float32))


def brute_force_log_z(w, a, b):
    V, H = w.shape
    x = ((np.arange(1 << V)[None, :] >> np.arange(V)[:, None]) & 1).astype(np.float64)
    act = w.astype(np.float64).T @ x + a.astype(np.float64)[:, None]
    lp = np.logaddexp(0, act).sum(axis=0) + b.astype(np.float64) @ x
    return lp.max() + np.log(np.exp(lp - lp.max()).sum())


def test_exact_enumeration_matches_numpy(oracle):
    w, a, b = small_rbm()
    assert abs(ais.exact_log_z(oracle, w, a, b) - brute_force_log_z(w, a, b)) < 1e-4


def test_ais_on_the_cpu_restatement_agrees_with_enumeration(oracle):
    w, a, b = small_rbm()
    schedule = np.linspace(0.0, 1.0, 400)
    log_z, logw = ais.ais_binary_rbm(oracle, w, a, b, 512, schedule, seed=5, fused=False)
    assert logw.shape == (512,)
    assert abs(log_z - brute_force_log_z(w, a, b)) < 0.15


def test_zero_rbm_has_log_z_of_the_uniform_model(oracle):
    V, H = 8, 6
    log_z, logw = ais.ais_binary_rbm(oracle, np.zeros((V, H)), np.zeros(H), np.zeros(V), 16, np.linspace(0, 1, 5),
                                     fused=False)
    assert np.allclose(logw, 0.0) and abs(log_z - (V + H) * np.log(2)) < 1e-6


@pytest.mark.gpu
@pytest.mark.parametrize("fused", [False, True])
def test_ais_on_the_device_matches_the_cpu_restatement(cm, oracle, fused):
    w, a, b = small_rbm(V=16, H=24)
    schedule = np.linspace(0.0, 1.0, 300)
    want, logw_o = ais.ais_binary_rbm(oracle, w, a, b, 256, schedule, seed=7, fused=False)
    got, logw_g = ais.ais_binary_rbm(cm, w, a, b, 256, schedule, seed=7, fused=fused)
    # same random stream: the chains coincide unless a probability lands within rounding of its uniform
    close = np.abs(logw_g - logw_o) < 1e-3 * np.maximum(1.0, np.abs(logw_o))
    assert close.mean() > 0.95
    assert abs(got - want) < 0.05
    assert abs(got - brute_force_log_z(w, a, b)) < 0.25
    assert abs(ais.exact_log_z(cm, w, a, b) - brute_force_log_z(w, a, b)) < 1e-3


@pytest.mark.gpu
def test_ais_at_layer_sizes_of_the_reference_models(cm):
    # 784 x 500 RBM, small weights: against the second-order cumulant expansion of
    # log E[exp(v'Wh)] under the uniform distribution (E[v_i h_j] = 1/4, Var = 3/16, covariance
    # 1/16 between entries that share a unit); the next cumulant is below 0.1 at this scale
    rng = np.random.default_rng(11)
    V, H = 784, 500
    w = (rng.standard_normal((V, H)) * 0.01).astype(np.float32)
    log_z, logw = ais.ais_binary_rbm(cm, w, np.zeros(H), np.zeros(V), 128, np.linspace(0, 1, 200), seed=1)
    assert np.isfinite(log_z) and logw.std() < 1.0
    w64 = w.astype(np.float64)
    sq = (w64 ** 2).sum()
    var = 3.0 / 16 * sq + 1.0 / 16 * ((w64.sum(axis=1) ** 2).sum() - sq + (w64.sum(axis=0) ** 2).sum() - sq)
    want = (V + H) * np.log(2) + w64.sum() / 4 + var / 2
    assert abs(log_z - want) < 0.5
