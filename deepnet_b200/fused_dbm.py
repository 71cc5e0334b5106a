"""PCD training of a deep Boltzmann machine (a chain of logistic layers) on fused kernels.

Same arithmetic, order and random stream as `dbm.DBM.TrainOneBatch` with the PCD optimizer
(deepnet/dbm.py:118-181 mean-field positive phase and particle initialisation, :183-238
Gibbs sweeps on persistent particles, :240-261 updates), but a layer update - the products
with BOTH neighbouring layers, bias, logistic, Bernoulli draw - is one `fused_gemm` call whose
pass list mixes the two inner dimensions, and positive-minus-negative edge statistics are one
call per edge.  Split-TF32 as in fused_rbm: a real-valued matrix x is multiplied as
x.y plus correction terms over its low part x - tf32(x), which the kernel derives from x itself;
a binary one (data, samples) has no low part.
"""
import ctypes as ct
import os

import numpy as np

from .dbm import Parameter
from .fused_rbm import LossReadback


class FusedDBM(LossReadback):
    def __init__(self, cm, sizes, batchsize, weights, hyperparams, seed=0):
        """sizes = [visible, hidden1, ...]; weights[i] is sizes[i] x sizes[i+1]."""
        self.cm, self.sizes, self.B, self.hyp = cm, list(sizes), batchsize, hyperparams
        self.L = len(sizes)
        cm.CUDAMatrix.init_random(seed)
        z = lambda r, c: cm.empty((r, c))
        B = batchsize
        self.W, self.W_aux, self.dW, self.suff_W = [], [], [], []
        for i, w in enumerate(weights):
            w = np.asarray(w, np.float32)
            assert w.shape == (sizes[i], sizes[i + 1])
            self.W.append(cm.CUDAMatrix(w))
            self.W_aux.append(self.W[-1].split_bf16(cm.empty_aux(w.shape)))   # bfloat16 parts, rewritten by the update
            self.dW.append(z(*w.shape))
            self.suff_W.append(z(*w.shape))
        self.b = [z(n, 1) for n in sizes]
        self.db = [z(n, 1) for n in sizes]
        self.suff_b = [z(n, 1) for n in sizes]
        self.pos = [z(n, B) for n in sizes]
        self.neg = [z(n, B) for n in sizes]
        self.neg_sample = [z(n, B) for n in sizes]
        self.loss_acc = z(1, 1)
        self._sched = Parameter(cm, hyperparams)
        self.kernel_launches = 0
        # the step is recorded once per (Gibbs sweeps, first step) and replayed with one library call;
        # B200_RBM_PROGRAM=0 issues every operation through its own call instead
        self.use_program = os.environ.get("B200_RBM_PROGRAM", "1") != "0"
        self._programs = {}
        self._batch = cm.CUDAMatrix._from_mat(cm.cudamat())

    def _update_layer(self, X, j, below, above, out, sample):
        """state_j = sigmoid(W[j-1]' below + W[j] above + b_j) (deepnet/dbm.py:82-105), optional draw.
        below / above = (state, exact): exact states (0/1) have no low part."""
        P = self.cm.split_passes
        passes = []
        if below is not None:
            passes += P(self.W[j - 1].T, below[0], exact_b=below[1], a_aux=self.W_aux[j - 1])
        if above is not None:
            passes += P(self.W[j], above[0], exact_b=above[1], a_aux=self.W_aux[j])
        X.fused_gemm(passes, out=out, sample=sample, bias=self.b[j], activation=1)
        self.kernel_launches += 1

    def TrainOneBatch(self, step, data):
        cm, hyp = self.cm, self.hyp
        gibbs = hyp.gibbs_steps
        if hyp.start_step_up_cd_after > 0 and hyp.start_step_up_cd_after < step:
            gibbs = hyp.gibbs_steps + 1 + (step - hyp.start_step_up_cd_after) // hyp.step_up_cd_after
        mom, eps = self._sched.GetMomentumAndEpsilon(step)
        l2 = hyp.l2_decay if hyp.apply_l2_decay else 0.0
        l1 = hyp.l1_decay if (hyp.apply_l1_decay and step > hyp.apply_l1decay_after) else 0.0
        if not self.use_program:
            self.kernel_launches = 0
            self._issue(cm.Immediate(), data, gibbs, step == 0, mom, eps, l2, l1)
            return
        key = (gibbs, step == 0)
        rec = self._programs.get(key)
        if rec is None:
            prog = cm.Program()
            self.kernel_launches = 0
            handles = self._issue(prog, self._batch, gibbs, step == 0, mom, eps, l2, l1)
            rec = self._programs[key] = (prog, handles, self.kernel_launches)
        prog, (bias_ops, weight_ops), self.kernel_launches = rec
        ct.memmove(ct.byref(self._batch.mat), ct.byref(data.mat), ct.sizeof(data.mat))
        self._batch.mat.owns_data = 0
        self._batch_owner = data
        for i in bias_ops:
            prog.set_floats(i, f1=mom, f2=eps)
        for i in weight_ops:
            prog.set_floats(i, f1=mom, f2=eps, f3=l2, f4=l1)
        prog.run()

    def _issue(self, X, data, gibbs, first_step, mom, eps, l2, l1):
        cm, L = self.cm, self.L
        pos, neg, ns = self.pos, self.neg, self.neg_sample
        # ---- positive phase: data clamped, hidden layers start at zero, mean-field sweeps
        for j in range(1, L):
            X.assign_scalar(pos[j], 0)
        for _ in range(self.hyp.mf_steps):
            for j in range(1, L):
                below = (data, True) if j == 1 else (pos[j - 1], False)
                above = (pos[j + 1], False) if j < L - 1 else None
                self._update_layer(X, j, below, above, pos[j], None)
        # PCD reports the reconstruction of the input from the first hidden layer (deepnet/dbm.py:163-166)
        self._update_layer(X, 0, None, (pos[1], False), pos[0], None)
        X.sq_diff(pos[0], data, self.loss_acc)
        # ---- particles start from the positive states at step 0 (deepnet/dbm.py:169-181, 270-271)
        if first_step:
            for j in range(L):
                X.copy(pos[j], neg[j])
                X.sample_bernoulli(neg[j], ns[j])
        # ---- negative phase: Gibbs sweeps on the particles, neighbours' samples as input
        for _ in range(gibbs):
            for j in range(L):
                # the visible "sample" is its mean (sample_input off), so it carries a low part
                below = None if j == 0 else ((neg[0], False) if j == 1 else (ns[j - 1], True))
                above = (ns[j + 1], True) if j < L - 1 else None
                self._update_layer(X, j, below, above, neg[j], ns[j] if j > 0 else None)
        # ---- statistics pos - neg and updates: bias statistics are row sums of pos - neg, one launch
        # a layer (the visible positive state is the data)
        for j in range(L):
            X.row_sum_diff(data if j == 0 else pos[j], neg[j], self.suff_b[j])
        for i in range(L - 1):
            # the difference of two nearly equal products: TF32 correction terms; the data are exact
            P = cm.split_passes
            p = P(data if i == 0 else pos[i], pos[i + 1].T, exact_a=(i == 0), terms="tf32")
            n = P(neg[i], neg[i + 1].T, negate=1, terms="tf32")
            X.fused_gemm(p + n, out=self.suff_W[i])
        self.kernel_launches += (L - 1) + L + 1 + (L - 1) + (2 * L if first_step else 0)
        inv_b = 1.0 / self.B
        bias_ops = [X.momentum_update(self.b[j], self.db[j], None, self.suff_b[j], inv_b, mom, eps) for j in range(L)]
        weight_ops = [X.momentum_update(self.W[i], self.dW[i], None, self.suff_W[i], inv_b, mom, eps, l2=l2, l1=l1,
                                        w_aux=self.W_aux[i]) for i in range(L - 1)]
        self.kernel_launches += 2 * L - 1
        return bias_ops, weight_ops

    def read_loss(self, reset=True):
        v = float(np.array(self.loss_acc.asarray())[0, 0])
        if reset:
            self.loss_acc.assign(0)
        return v
