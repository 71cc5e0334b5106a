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
import numpy as np

from .dbm import Parameter


class FusedDBM(object):
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

    def _update_layer(self, j, below, above, out, sample):
        """state_j = sigmoid(W[j-1]' below + W[j] above + b_j) (deepnet/dbm.py:82-105), optional draw.
        below / above = (state, exact): exact states (0/1) have no low part."""
        P = self.cm.split_passes
        passes = []
        if below is not None:
            passes += P(self.W[j - 1].T, below[0], exact_b=below[1], a_aux=self.W_aux[j - 1])
        if above is not None:
            passes += P(self.W[j], above[0], exact_b=above[1], a_aux=self.W_aux[j])
        self.cm.fused_gemm(passes, out=out, sample=sample, bias=self.b[j], activation=1)
        self.kernel_launches += 1

    def TrainOneBatch(self, step, data):
        cm, L, hyp = self.cm, self.L, self.hyp
        self.kernel_launches = 0
        pos, neg, ns = self.pos, self.neg, self.neg_sample
        # ---- positive phase: data clamped, hidden layers start at zero, mean-field sweeps
        for j in range(1, L):
            pos[j].assign(0)
        for _ in range(hyp.mf_steps):
            for j in range(1, L):
                below = (data, True) if j == 1 else (pos[j - 1], False)
                above = (pos[j + 1], False) if j < L - 1 else None
                self._update_layer(j, below, above, pos[j], None)
        # bias statistics of the positive phase (the visible state is the data here)
        data.sum(axis=1, target=self.suff_b[0])
        for j in range(1, L):
            pos[j].sum(axis=1, target=self.suff_b[j])
        # PCD reports the reconstruction of the input from the first hidden layer (deepnet/dbm.py:163-166)
        self._update_layer(0, None, (pos[1], False), pos[0], None)
        cm._check(cm._lib.add_sq_diff(pos[0].p_mat, data.p_mat, self.loss_acc.p_mat))
        # ---- particles start from the positive states at step 0 (deepnet/dbm.py:169-181, 270-271)
        if step == 0:
            for j in range(L):
                neg[j].assign(pos[j])
                neg[j].sample_bernoulli(target=ns[j])
        # ---- negative phase: Gibbs sweeps on the particles, neighbours' samples as input
        gibbs = hyp.gibbs_steps
        if hyp.start_step_up_cd_after > 0 and hyp.start_step_up_cd_after < step:
            gibbs = hyp.gibbs_steps + 1 + (step - hyp.start_step_up_cd_after) // hyp.step_up_cd_after
        for _ in range(gibbs):
            for j in range(L):
                # the visible "sample" is its mean (sample_input off), so it carries a low part
                below = None if j == 0 else ((neg[0], False) if j == 1 else (ns[j - 1], True))
                above = (ns[j + 1], True) if j < L - 1 else None
                self._update_layer(j, below, above, neg[j], ns[j] if j > 0 else None)
        # ---- statistics pos - neg and updates
        for j in range(L):
            self.suff_b[j].add_sums(neg[j], axis=1, mult=-1.0)
        for i in range(L - 1):
            # the difference of two nearly equal products: TF32 correction terms; the data are exact
            P = cm.split_passes
            p = P(data if i == 0 else pos[i], pos[i + 1].T, exact_a=(i == 0), terms="tf32")
            n = P(neg[i], neg[i + 1].T, negate=1, terms="tf32")
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
