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


def small_rs_rbm(V=30, H=8, seed=4):
    rng = np.random.default_rng(seed)
    return ((rng.standard_normal((V, H)) * 0.3).astype(np.float32), (rng.standard_normal(H) * 0.1).astype(np.float32),
            (rng.standard_normal(V) * 0.5).astype(np.float32))


def test_replicated_softmax_enumeration_against_brute_force():
    # tiny model: every document of D words over V words, every hidden configuration
    import itertools
    rng = np.random.default_rng(0)
    V, H, D = 3, 2, 3
    w, a, b = rng.standard_normal((V, H)), rng.standard_normal(H), rng.standard_normal(V)
    total = []
    for h in itertools.product((0, 1), repeat=H):
        h = np.array(h, float)
        for doc in itertools.product(range(V), repeat=D):      # word sequences, as the base-rate term D logsumexp counts them
            v = np.bincount(doc, minlength=V).astype(float)
            total.append(v @ w @ h + b @ v + D * (a @ h))
    want = ais.log_sum_exp(np.array(total))
    assert abs(ais.exact_log_z_replicated_softmax(w, a, b, D) - want) < 1e-9


def test_replicated_softmax_ais_on_the_cpu_restatement_agrees_with_enumeration(oracle):
    w, a, b = small_rs_rbm()
    D = 6
    schedule = np.linspace(0.0, 1.0, 300)
    log_z, logw = ais.ais_replicated_softmax(oracle, w, a, b, D, 256, schedule=schedule, seed=3, fused=False)
    assert logw.shape == (256,)
    assert abs(log_z - ais.exact_log_z_replicated_softmax(w, a, b, D)) < 0.15
    # a model without weights or hidden biases equals its base-rate model at f = 1
    z0, lw0 = ais.ais_replicated_softmax(oracle, np.zeros((5, 3)), np.zeros(3), b[:5], 4, 8, schedule=np.linspace(0, 1, 4),
                                         fused=False, base_rate_fraction=1.0)
    assert np.allclose(lw0, 0) and abs(z0 - (4 * ais.log_sum_exp(b[:5].astype(np.float64)) + 3 * np.log(2))) < 1e-6
    sched = ais.replicated_softmax_schedule()                   # deepnet/ais.py:62-68: 700 + 2000 + 5000 steps (+1 by rounding)
    assert len(sched) in (7700, 7701) and sched[0] == 0 and 0.9999 < sched[-1] < 1


@pytest.mark.gpu
@pytest.mark.parametrize("fused", [False, True])
def test_replicated_softmax_ais_on_the_device_matches_the_cpu_restatement(cm, oracle, fused):
    w, a, b = small_rs_rbm(V=60, H=10)
    D = 12
    schedule = np.linspace(0.0, 1.0, 200)
    want, logw_o = ais.ais_replicated_softmax(oracle, w, a, b, D, 128, schedule=schedule, seed=7, fused=False)
    got, logw_g = ais.ais_replicated_softmax(cm, w, a, b, D, 128, schedule=schedule, seed=7, fused=fused)
    assert cm.CUDAMatrix.rnd_state.calls == oracle._Rng.calls          # D calls per softmax draw, one per hidden draw
    # same random stream: chains coincide unless a value lands within rounding of a tie or a uniform
    close = np.abs(logw_g - logw_o) < 1e-3 * np.maximum(1.0, np.abs(logw_o))
    assert close.mean() > 0.9
    assert abs(got - want) < 0.1
    assert abs(got - ais.exact_log_z_replicated_softmax(w, a, b, D)) < 0.3
    assert cm.read_status() == 0


@pytest.mark.gpu
def test_fused_gumbel_draws_equal_the_call_by_call_loop(cm, oracle):
    rng = np.random.default_rng(8)
    V, B, D = 500, 37, 9
    e = (rng.standard_normal((V, B)) * 2).astype(np.float32)
    counts = {}
    for backend in (cm, oracle):
        backend.CUDAMatrix.init_random(6)
        en, smp, tmp = backend.CUDAMatrix(e), backend.empty((V, B)), backend.empty((V, B))
        ais.sample_energy_softmax(backend, en, smp, tmp, D, fused=False)
        counts[backend] = np.array(smp.asarray(), copy=True)
    cm.CUDAMatrix.init_random(6)
    fused = cm.empty((V, B))
    cm.CUDAMatrix(e).sample_energy_softmax(fused, D)
    got = np.array(fused.asarray())
    np.testing.assert_array_equal(got, counts[cm])                    # same GPU arithmetic: identical counts
    assert np.abs(got - counts[oracle]).sum() <= 4                    # libm vs GPU logf may move a rare near-tie
    np.testing.assert_array_equal(got.sum(axis=0), np.full(B, D))
    assert cm.CUDAMatrix.rnd_state.calls == D
