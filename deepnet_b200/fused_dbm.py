"""PCD training of a deep Boltzmann machine (a chain of logistic layers) on fused kernels.

Same arithmetic, order and random stream as `dbm.DBM.TrainOneBatch` with the PCD optimizer
(deepnet/dbm.py:118-181 mean-field positive phase and particle initialisation, :183-238
Gibbs sweeps on persistent particles, :240-261 updates), but a layer update - the products
with BOTH neighbouring layers, bias, logistic, Bernoulli draw - is one `fused_gemm` call whose
pass list mixes the two inner dimensions, and positive-minus-negative edge statistics are one
call per edge.  Split-TF32 as in fused_rbm: a real-valued matrix x is multiplied as
x.y (TF32) + lo_x.y + x.lo_y (bfloat16 planes of the aux matrices); a binary one (data, samples)
needs no low-part term.
"""
import numpy as np

from .dbm import Parameter


class FusedDBM(object):
    def __init__(self, cm, sizes, batchsize, weights, hyperparams, seed=0):
        """sizes = [visible, hidden1, ...]; weights[i] is sizes[i] x sizes[i+1]."""
        self.cm, self.sizes, self.B, self.hyp = cm, list(sizes), batchsize, hyperparams
        self.L = len(sizes)
        cm.CUDAMatrix.init_random(seed)
        z = lambda r, c: cm.empty((r, c))
        za = lambda r, c: cm.empty_aux((r, c))
        B = batchsize
        self.W, self.W_aux, self.dW, self.suff_W = [], [], [], []
        for i, w in enumerate(weights):
            w = np.asarray(w, np.float32)
            assert w.shape == (sizes[i], sizes[i + 1])
            W = cm.CUDAMatrix(w)
            self.W.append(W)
            self.W_aux.append(W.split_bf16(za(*w.shape)))   # bfloat16 planes read by the correction products
            self.dW.append(z(*w.shape))
            self.suff_W.append(z(*w.shape))
        self.b = [z(n, 1) for n in sizes]
        self.db = [z(n, 1) for n in sizes]
        self.suff_b = [z(n, 1) for n in sizes]
        self.pos = [z(n, B) for n in sizes]
        self.pos_aux = [za(n, B) for n in sizes]
        self.neg = [z(n, B) for n in sizes]
        self.neg_aux = [za(n, B) for n in sizes]
        self.neg_sample = [z(n, B) for n in sizes]
        self.neg_sample_aux = [za(n, B) for n in sizes]
        self.data_aux = za(sizes[0], B)
        # fp32 low parts of the statistics operands (every term of that product is a TF32 product)
        self.pos_lo = [z(n, B) for n in sizes]
        self.neg_lo = [z(n, B) for n in sizes]
        self.loss_acc = z(1, 1)
        self._sched = Parameter(cm, hyperparams)
        self.kernel_launches = 0

    def _update_layer(self, j, below, above, out, out_aux, sample, sample_aux):
        """state_j = sigmoid(W[j-1]' below + W[j] above + b_j) (deepnet/dbm.py:82-105), optional draw.
        below / above = (state, its aux matrix, exact): exact states (0/1) need no low-part term."""
        P = self.cm.split_passes
        passes = []
        if below is not None:
            passes += P(self.W[j - 1].T, self.W_aux[j - 1].T, below[0], below[1], exact_x=below[2])
        if above is not None:
            passes += P(self.W[j], self.W_aux[j], above[0], above[1], exact_x=above[2])
        self.cm.fused_gemm(passes, out=out, out_aux=out_aux, sample=sample, sample_aux=sample_aux, bias=self.b[j],
                           activation=1)
        self.kernel_launches += 1

    def TrainOneBatch(self, step, data):
        cm, L, hyp = self.cm, self.L, self.hyp
        self.kernel_launches = 0
        pos, pos_aux, neg, neg_aux = self.pos, self.pos_aux, self.neg, self.neg_aux
        ns, ns_aux = self.neg_sample, self.neg_sample_aux
        data_aux = data.split_bf16(self.data_aux)
        # ---- positive phase: data clamped, hidden layers start at zero, mean-field sweeps
        for j in range(1, L):
            pos[j].assign(0)
            pos_aux[j].assign(0)
        for _ in range(hyp.mf_steps):
            for j in range(1, L):
                below = (data, data_aux, True) if j == 1 else (pos[j - 1], pos_aux[j - 1], False)
                above = (pos[j + 1], pos_aux[j + 1], False) if j < L - 1 else None
                self._update_layer(j, below, above, pos[j], pos_aux[j], None, None)
        # bias statistics of the positive phase (the visible state is the data here)
        data.sum(axis=1, target=self.suff_b[0])
        for j in range(1, L):
            pos[j].sum(axis=1, target=self.suff_b[j])
        # PCD reports the reconstruction of the input from the first hidden layer (deepnet/dbm.py:163-166)
        self._update_layer(0, None, (pos[1], pos_aux[1], False), pos[0], pos_aux[0], None, None)
        cm._check(cm._lib.add_sq_diff(pos[0].p_mat, data.p_mat, self.loss_acc.p_mat))
        # ---- particles start from the positive states at step 0 (deepnet/dbm.py:169-181, 270-271)
        if step == 0:
            for j in range(L):
                neg[j].assign(pos[j])
                neg_aux[j].assign(pos_aux[j])
                neg[j].sample_bernoulli(target=ns[j])
                ns[j].split_bf16(ns_aux[j])
        # ---- negative phase: Gibbs sweeps on the particles, neighbours' samples as input
        gibbs = hyp.gibbs_steps
        if hyp.start_step_up_cd_after > 0 and hyp.start_step_up_cd_after < step:
            gibbs = hyp.gibbs_steps + 1 + (step - hyp.start_step_up_cd_after) // hyp.step_up_cd_after
        for _ in range(gibbs):
            for j in range(L):
                # the visible "sample" is its mean (sample_input off), so it carries a low part
                below = None if j == 0 else ((neg[0], neg_aux[0], False) if j == 1 else (ns[j - 1], ns_aux[j - 1], True))
                above = (ns[j + 1], ns_aux[j + 1], True) if j < L - 1 else None
                self._update_layer(j, below, above, neg[j], neg_aux[j], ns[j] if j > 0 else None,
                                   ns_aux[j] if j > 0 else None)
        # ---- statistics pos - neg and updates
        for j in range(L):
            self.suff_b[j].add_sums(neg[j], axis=1, mult=-1.0)
        for i in range(L - 1):
            # the difference of two nearly equal products: all-TF32 terms on fp32 low parts
            T = cm.tf32_passes
            if i == 0:
                for j in range(L):
                    if j > 0:
                        pos[j].split_tf32(self.pos_lo[j])
                    neg[j].split_tf32(self.neg_lo[j])
            plo, nlo = self.pos_lo, self.neg_lo
            # the data are exact: only the hidden means carry a low part
            p = T(data if i == 0 else pos[i], None if i == 0 else plo[i], pos[i + 1].T, plo[i + 1].T)
            n = T(neg[i], nlo[i], neg[i + 1].T, nlo[i + 1].T, negate=1)
            cm.fused_gemm(p + n, out=self.suff_W[i])
        inv_b = 1.0 / self.B
        mom, eps = self._sched.GetMomentumAndEpsilon(step)
        h = hyp
        l2 = h.l2_decay if h.apply_l2_decay else 0.0
        l1 = h.l1_decay if (h.apply_l1_decay and step > h.apply_l1decay_after) else 0.0
        for j in range(L):
            self.b[j].momentum_update(self.db[j], None, self.suff_b[j], inv_b, mom, eps)
        for i in range(L - 1):
            self.W[i].momentum_update(self.dW[i], None, self.suff_W[i], inv_b, mom, eps, l2=l2, l1=l1,
                                      w_aux=self.W_aux[i])

    def read_loss(self, reset=True):
        v = float(np.array(self.loss_acc.asarray())[0, 0])
        if reset:
            self.loss_acc.assign(0)
        return v
