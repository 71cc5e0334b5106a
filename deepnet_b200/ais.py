"""Annealed importance sampling estimate of the partition function of a binary RBM, on the `cm`
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
