"""Annealed importance sampling estimates of the partition function of a binary RBM and of a
replicated-softmax RBM (`ais_replicated_softmax`, deepnet/ais.py:61-129), on the `cm`
matrix API (b200mat on the device; the CPU restatement of eigenmat offers the same calls).

The call sequence is that of deepnet/ais.py:131-171 (`AISBinaryRbm`): chains start from the uniform
base-rate model (all parameters zero), the intermediate distributions scale weights and both
biases by the inverse temperature schedule[i], and each step adds
    sum_j [log(1 + exp(s_i (W'v + a)_j)) - log(1 + exp(s_{i-1} (W'v + a)_j))] + (s_i - s_{i-1}) b'x
to the log importance weight of every chain, then runs one Gibbs sweep h|v, v|h at s_i.  As in the
reference, x in the bias term is the visible STATE left by the previous sweep (the activation
probabilities, deepnet/ais.py:158), not the sample.  `exact_log_z` is deepnet/ais.py:182-208
(`ExactZ_binary_binary`): the sum over all 2^V visible configurations with the hidden units
summed out analytically.

On b200mat the two products of a step go through `fused_gemm` (bias and the schedule factor in
the epilogue); `fused=False` keeps the reference's call-by-call form, which the CPU restatement
runs too.  Both forms consume the random stream identically (two sampling calls per step).
"""
import numpy as np


def log_mean_exp(x):
    """deepnet/ais.py:31-33."""
    x = np.asarray(x, np.float64)
    offset = x.max()
    return offset + np.log(np.exp(x - offset).mean())


def ais_binary_rbm(cm, weight, hidden_bias, visible_bias, num_chains, schedule, seed=0, fused=None):
    """log Z estimate of the RBM  E(v, h) = -v'Wh - b'v - a'h  (weight V x H, a = hidden bias,
    b = visible bias) from `num_chains` annealing runs along `schedule` (inverse temperatures
    from 0 to 1).  Returns (log_z, log_weights[num_chains])."""
    w = cm.CUDAMatrix(np.asarray(weight, np.float32))
    V, H = w.shape
    a = cm.CUDAMatrix(np.asarray(hidden_bias, np.float32).reshape(H, 1))
    b = cm.CUDAMatrix(np.asarray(visible_bias, np.float32).reshape(V, 1))
    if fused is None:
        fused = hasattr(cm, "fused_gemm")
    cm.CUDAMatrix.init_random(seed)
    B = num_chains
    v_state, v_sample = cm.empty((V, B)), cm.empty((V, B))
    h_state, h_temp, h_deriv, h_sample = cm.empty((H, B)), cm.empty((H, B)), cm.empty((H, B)), cm.empty((H, B))
    # chains start from the uniform model: state = sigmoid(0), one Bernoulli draw (deepnet/ais.py:146-148)
    v_state.assign(0)
    cm.sigmoid(v_state)
    v_state.sample_bernoulli(target=v_sample)
    w_ais = cm.CUDAMatrix(np.zeros((1, B), np.float32))
    w_aux = w.split_bf16(cm.empty_aux((V, H))) if fused else None
    for i in range(1, len(schedule)):
        s_prev, s = float(schedule[i - 1]), float(schedule[i])
        # hidden pre-activation W'v + a (deepnet/ais.py:153-154)
        if fused:
            cm.fused_gemm(cm.split_passes(w.T, v_sample, exact_b=True, a_aux=w_aux), out=h_state, bias=a)
        else:
            cm.dot(w.T, v_sample, target=h_state)
            h_state.add_col_vec(a)
        # importance weight (deepnet/ais.py:156-162)
        h_state.mult(s_prev, target=h_temp)
        h_state.mult(s)
        cm.log_1_plus_exp(h_state, target=h_deriv)
        cm.log_1_plus_exp(h_temp)
        h_deriv.subtract(h_temp)
        w_ais.add_sums(h_deriv, axis=0)
        w_ais.add_dot(b.T, v_state, mult=s - s_prev)
        # Gibbs sweep at inverse temperature s (deepnet/ais.py:164-170)
        cm.sigmoid(h_state)
        h_state.sample_bernoulli(target=h_sample)
        if fused:
            cm.fused_gemm(cm.split_passes(w, h_sample, exact_b=True, a_aux=w_aux), out=v_state, bias=b)
        else:
            cm.dot(w, h_sample, target=v_state)
            v_state.add_col_vec(b)
        v_state.mult(s)
        cm.sigmoid(v_state)
        v_state.sample_bernoulli(target=v_sample)
    logw = np.array(w_ais.asarray(), np.float64).reshape(-1)
    return log_mean_exp(logw) + (V + H) * np.log(2.0), logw


def log_sum_exp(x):
    """deepnet/ais.py:35-37."""
    x = np.asarray(x, np.float64)
    offset = x.max()
    return offset + np.log(np.exp(x - offset).sum())


def replicated_softmax_schedule():
    """The inverse temperatures of deepnet/ais.py:62-68: 700 + 2000 + 5000 steps, finer towards 1."""
    return np.concatenate((np.arange(0.0, 0.7, 0.001), np.arange(0.7, 0.9, 0.0001), np.arange(0.9, 1.0, 0.00002)))


def sample_energy_softmax(cm, energy, sample, temp, ndraws, fused):
    """deepnet/ais.py:16-30: `ndraws` Gumbel-max draws per column, counted per word."""
    if fused:
        energy.sample_energy_softmax(sample, ndraws)
        return
    sample.assign(0)
    for _ in range(ndraws):
        energy.perturb_energy_for_softmax_sampling(target=temp)
        temp.choose_max_and_accumulate(sample)


def ais_replicated_softmax(cm, weight, hidden_bias, visible_bias, D, num_chains, schedule=None, seed=0, fused=None,
                           base_rate_fraction=0.1):
    """log Z estimate of a replicated-softmax RBM for documents of D words (deepnet/ais.py:61-129):
    E(v, h) = -v'Wh - b'v - D a'h over word-count vectors v with D words.  Chains start from the
    base-rate model that keeps the fraction f = 0.1 of the visible biases; step i adds
        sum_j [log(1 + exp(s_{i+1} x_j)) - log(1 + exp(s_i x_j))] + (1 - f)(s_{i+1} - s_i) b'v,   x = W'v + D a
    to every chain's log weight and resamples h | v and v | h at s_{i+1}; the words are drawn D at
    a time by Gumbel-max on the energies.  log Z_base = D logsumexp(f b) + H log 2.
    On b200mat the D draws of a step are one kernel and the two products go through `fused_gemm`;
    `fused=False` keeps the reference's call-by-call form, which the CPU restatement runs too; both
    consume the random stream identically.  Returns (log_z, log_weights[num_chains])."""
    if schedule is None:
        schedule = replicated_softmax_schedule()
    w = cm.CUDAMatrix(np.asarray(weight, np.float32))
    V, H = w.shape
    a = cm.CUDAMatrix(np.asarray(hidden_bias, np.float32).reshape(H, 1))
    b = cm.CUDAMatrix(np.asarray(visible_bias, np.float32).reshape(V, 1))
    if fused is None:
        fused = hasattr(cm, "fused_gemm")
    f, B, D = float(base_rate_fraction), num_chains, int(D)
    cm.CUDAMatrix.init_random(seed)
    v_state, v_sample, v_temp = cm.empty((V, B)), cm.empty((V, B)), cm.empty((V, B))
    h_state, h_temp, h_deriv, h_sample = cm.empty((H, B)), cm.empty((H, B)), cm.empty((H, B)), cm.empty((H, B))
    # chains start from the base-rate model: energies f b (deepnet/ais.py:87-91)
    v_state.assign(0)
    v_state.add_col_mult(b, f)
    sample_energy_softmax(cm, v_state, v_sample, v_temp, D, fused)
    w_ais = cm.CUDAMatrix(np.zeros((1, B), np.float32))
    w_aux = w.split_bf16(cm.empty_aux((V, H))) if fused else None
    for i in range(len(schedule) - 1):
        s0, s1 = float(schedule[i]), float(schedule[i + 1])
        # hidden pre-activation W'v + D a: the counts are small integers, exact in TF32 (deepnet/ais.py:104-105)
        if fused:
            cm.fused_gemm(cm.split_passes(w.T, v_sample, exact_b=True, a_aux=w_aux), out=h_state)
        else:
            cm.dot(w.T, v_sample, target=h_state)
        h_state.add_col_mult(a, D)
        # importance weight (deepnet/ais.py:107-113)
        h_state.mult(s0, target=h_temp)
        h_state.mult(s1)
        cm.log_1_plus_exp(h_state, target=h_deriv)
        cm.log_1_plus_exp(h_temp)
        h_deriv.subtract(h_temp)
        w_ais.add_sums(h_deriv, axis=0)
        w_ais.add_dot(b.T, v_sample, mult=(1 - f) * (s1 - s0))
        # Gibbs sweep at s1 (deepnet/ais.py:115-122)
        cm.sigmoid(h_state)
        h_state.sample_bernoulli(target=h_sample)
        if fused:
            cm.fused_gemm(cm.split_passes(w, h_sample, exact_b=True, a_aux=w_aux), out=v_state, bias=b)
        else:
            cm.dot(w, h_sample, target=v_state)
            v_state.add_col_vec(b)
        v_state.mult(s1)
        v_state.add_col_mult(b, f * (1 - s1))
        sample_energy_softmax(cm, v_state, v_sample, v_temp, D, fused)
    logw = np.array(w_ais.asarray(), np.float64).reshape(-1)
    base = D * log_sum_exp(f * np.asarray(visible_bias, np.float64)) + H * np.log(2.0)
    return log_mean_exp(logw) + base, logw


def exact_log_z_replicated_softmax(weight, hidden_bias, visible_bias, D):
    """log Z of the replicated-softmax RBM by enumeration of the 2^H hidden configurations, the D
    words summed out analytically (they are independent given h): float64 on the host; H <= 20."""
    w = np.asarray(weight, np.float64)
    a, b = np.asarray(hidden_bias, np.float64).ravel(), np.asarray(visible_bias, np.float64).ravel()
    V, H = w.shape
    assert H <= 20, "enumeration over 2^H hidden states"
    h = ((np.arange(1 << H)[None, :] >> np.arange(H)[:, None]) & 1).astype(np.float64)       # H x 2^H
    act = w @ h + b[:, None]                                                                  # V x 2^H
    m = act.max(axis=0)
    lp = D * (a @ h) + D * (m + np.log(np.exp(act - m).sum(axis=0)))
    return log_sum_exp(lp)


def exact_log_z(cm, weight, hidden_bias, visible_bias):
    """log Z by enumeration of the 2^V visible configurations (deepnet/ais.py:173-208); V <= 20."""
    weight = np.asarray(weight, np.float32)
    V, H = weight.shape
    assert V <= 20, "enumeration over 2^V visible states"
    n = 1 << V
    x = ((np.arange(n)[None, :] >> np.arange(V)[:, None]) & 1).astype(np.float32)
    w = cm.CUDAMatrix(weight)
    a = cm.CUDAMatrix(np.asarray(hidden_bias, np.float32).reshape(H, 1))
    b = cm.CUDAMatrix(np.asarray(visible_bias, np.float32).reshape(V, 1))
    xs = cm.CUDAMatrix(x)
    h = cm.empty((H, n))
    cm.dot(w.T, xs, target=h)
    h.add_col_vec(a)
    cm.log_1_plus_exp(h)
    logp = cm.CUDAMatrix(np.zeros((1, n), np.float32))
    logp.add_sums(h, axis=0)
    logp.add_dot(b.T, xs)
    lp = np.array(logp.asarray(), np.float64).reshape(-1)
    offset = lp.max()
    return offset + np.log(np.exp(lp - offset).sum())
