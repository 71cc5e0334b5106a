"""The CD-k step of an RBM on the fused entry points of b200mat.

Same arithmetic and the same random stream as `dbm.DBM.TrainOneBatch` (one sampling
call for the positive hidden sample, one per Gibbs step), but every group of
reference calls is one kernel:

  dot + add_col_vec + sigmoid + sample_bernoulli   -> fused_gemm (bias, activation, Bernoulli in the
      (deepnet/dbm.py:88-105, logistic_layer.py:11-15)  epilogue)
  dot(v, h.T) and add_dot(..., mult=-1)            -> one fused_gemm with negated passes
      (deepnet/edge.py:236,242)
  add_mult / mult / add_mult / assign(0)           -> momentum_update (one pass over W)
      (deepnet/dbm.py:242,254, parameter.py:89-106)
  subtract + euclid_norm()**2                      -> add_sq_diff, accumulated on the device
      (deepnet/logistic_layer.py:48-52)

fp32-grade products: the tensor core reads an fp32 operand as TF32 (low 13 mantissa
bits ignored); the kernel derives lo = x - tf32(x) from the staged tile of x and adds the
correction terms lo_x.y + x.lo_y to x.y - as bfloat16 products (twice the TF32 rate) for
the activation products, as TF32 products for the statistics, whose positive and negative
halves nearly cancel.  Binary matrices (data, Bernoulli samples) have lo = 0 and need one
term fewer.  For the big products the bfloat16 parts come from aux matrices kept beside W
(rewritten by the update) and beside the states (written by the epilogue that produced
them): deriving them in the kernel costs shared-memory bandwidth next to the tensor core's
own operand reads.

With more than one rank the sufficient statistics of the ranks' minibatch shards are
summed by one NCCL all-reduce of a packed buffer before the update.
"""
import ctypes as ct
import os

import numpy as np

from .dbm import LINEAR, LOGISTIC, REPLICATED_SOFTMAX, Parameter


class LossReadback(object):
    """The accumulated loss of an engine (`self.loss_acc`) read back without stalling the thread that
    issues the updates: `loss_begin(slot)` after an update copies the accumulator aside, clears it and
    starts a device-to-host copy behind the enqueued work; `loss_end(slot)` - an update or more later -
    returns the value.  Two slots let the loss of update n travel while update n + 1 is issued."""

    def loss_begin(self, slot=0):
        cm = self.cm
        if getattr(self, "_loss_host", None) is None:
            self._loss_host = cm.host_alloc((8, 1))
            self._loss_dev = cm.empty((1, 8))
        keep = self._loss_dev.slice(slot, slot + 1)
        keep.assign(self.loss_acc)
        self.loss_acc.assign(0)
        cm.readback_begin(keep, self._loss_host[1] + 4 * slot, 4, slot)

    def loss_end(self, slot=0):
        self.cm.readback_wait(slot)
        return float(self._loss_host[0][slot, 0])


class FusedRBM(LossReadback):
    def __init__(self, cm, V, H, batchsize, weight, hyperparams, edge_hyperparams=None, visible=LOGISTIC,
                 binary_data=False, bias_v=None, bias_h=None, seed=0, world_size=1, rank=0, group=None):
        """binary_data: the caller states that every input is exactly 0 or 1 (or, for word counts, a
        small integer): such data have no low part, so the products over them run one term shorter
        and, for a big logistic model, on the scaled half-precision form.  Real-valued inputs
        (grey levels in [0, 1], standardised features) must leave it False: with it set their low
        parts would be dropped without notice.

        With world_size > 1 the replicated-softmax model draws its multinomial samples from the
        rank's own call numbers: its random stream then depends on the number of ranks (the Bernoulli
        paths do not: they are indexed by global column only).

        group: the `rendezvous.Group` of the ranks.  With it the exchange and the update of a data-parallel
        step run as one pass over peer memory (`dp_peer_update`: every rank reduces and updates its own
        columns of W and stores them into every replica) instead of an NCCL all-reduce followed by the
        update; B200_DP_PEER=0 keeps NCCL."""
        if visible == LINEAR and hyperparams.sample_input:
            # the reference's linear layer has no draw (deepnet/linear_layer.py:24-27 is a no-op without
            # learned precision), so its `sample` buffer would feed stale values upward
            raise ValueError("sample_input with a linear visible layer is not supported")
        self.cm = cm
        self.V, self.H, self.B = V, H, batchsize
        self.visible = visible
        self.binary_data = binary_data
        self.hyp = hyperparams
        self.ehyp = edge_hyperparams or hyperparams
        self.world_size = world_size
        cm.CUDAMatrix.init_random(seed)
        cm.set_rng_column_offset(rank * batchsize)
        z = lambda r, c: cm.empty((r, c))
        w = np.asarray(weight, np.float32)
        assert w.shape == (V, H)
        self.W = cm.CUDAMatrix(w)
        # bfloat16 parts of W kept in memory (rewritten by every update): the big products read
        # them instead of deriving them, as they do for the states that feed the next product
        self.W_aux = self.W.split_bf16(cm.empty_aux((V, H)))
        # ... and for the states only when the products are big: a small model is bound by launch
        # latency, where the extra split launch and the wider epilogue cost more than they save
        env = os.environ.get("B200_RBM_STATE_AUX")
        self.state_aux = (V * H * batchsize >= 1 << 32) if env is None else env != "0"
        # With 0/1 data and logistic units every operand's range is known, and the big products run
        # on the scaled half-precision form of W and of the states (three fp16 terms, no TF32 term,
        # no fp32 operand read): W * 2^e with e kept by the update kernel, states * 2^14.
        self.f16 = (self.state_aux and binary_data and visible == LOGISTIC
                    and os.environ.get("B200_RBM_F16", "1") != "0")
        if self.f16:
            self.W_scale = cm.f16_scale_state(float(np.abs(w).max()))
            self.W_exp = self.W_scale.slice(0, 1)
            self.W.split_f16(self.W_aux, exp_dev=self.W_exp)
        # both bias vectors, their update histories and their statistics are packed [b_v | b_h], so
        # one kernel updates them
        b0 = np.zeros((V + H, 1), np.float32)
        if bias_v is not None:
            b0[:V, 0] = np.asarray(bias_v, np.float32).ravel()
        if bias_h is not None:
            b0[V:, 0] = np.asarray(bias_h, np.float32).ravel()
        self.b, self.db = cm.CUDAMatrix(b0), z(V + H, 1)
        self.bv, self.bh = self.b.slice(0, V), self.b.slice(V, V + H)
        self.dbv, self.dbh = self.db.slice(0, V), self.db.slice(V, V + H)
        self.dW = z(V, H)
        # packed statistics [W | b_v | b_h]: one buffer, one all-reduce
        self.pack = z(V * H + V + H, 1)
        self.suff_W = self.pack.slice(0, V * H).reshape((V, H))
        self.suff_bv = self.pack.slice(V * H, V * H + V)
        self.suff_bh = self.pack.slice(V * H + V, V * H + V + H)
        self.suff_b = self.pack.slice(V * H, V * H + V + H)
        B = batchsize
        za = lambda r, c: cm.empty_aux((r, c))
        self.h_pos, self.h_samp, self.h_samp_aux = z(H, B), z(H, B), za(H, B)
        self.v_neg, self.v_neg_aux, self.h_neg = z(V, B), za(V, B), z(H, B)
        self.data_aux = za(V, B)
        self.h_pos_aux, self.h_neg_aux = (za(H, B), za(H, B)) if getattr(self, "f16", False) else (None, None)
        self.v_samp = self.v_samp_aux = None      # allocated when sample_input asks for visible draws
        self.loss_acc = z(1, 1)
        if visible == REPLICATED_SOFTMAX:
            # document lengths, length-normalised visible states (the statistics use state / NN,
            # deepnet/edge.py:225-228) and the multinomial sample fed upward
            self.NN = z(1, B)
            self.v0n, self.v_negn = z(V, B), z(V, B)
            self.v_samp = z(V, B)
            self.v_act = z(V, B)                  # W h + b_v before the softmax
            self.tiny = 1e-10
        self._sched = Parameter(cm, self.hyp)
        self._esched = Parameter(cm, self.ehyp)
        self.kernel_launches = 0
        self.timeline = None   # set to a list to record (name, flops, bytes, start, end) per launch
        # the step is recorded once per (Gibbs steps, visible draw) and replayed with one library call;
        # B200_RBM_PROGRAM=0 issues every operation through its own call instead
        self.use_program = os.environ.get("B200_RBM_PROGRAM", "1") != "0"
        self._programs = {}
        # data parallel, big model: the all-reduce and the update (and with B200_DP_PANEL_PRODUCTS the
        # statistics product, which then leaves the all-reduce some SMs) can run in column panels of W,
        # the all-reduce on a side stream.  Measured on two B200s neither form changed the time of an
        # update (the panel products run 40 % slower than the one product; the update is too short
        # to matter), so one all-reduce between product and update stays the default.
        self.dp_panels = int(os.environ.get("B200_DP_PANELS", "1"))
        self.dp_panel_products = os.environ.get("B200_DP_PANEL_PRODUCTS", "0") != "0"
        cols = os.environ.get("B200_DP_PANEL_COLS", "")          # e.g. "5888,2304": unequal panels
        self.dp_panel_cols = [int(c) for c in cols.split(",")] if cols else None
        self.dp_reserved_sms = int(os.environ.get("B200_DP_RESERVED_SMS", "12"))
        self.dp_peer = False
        if (world_size > 1 and group is not None and visible != REPLICATED_SOFTMAX and H % world_size == 0 and V % 4 == 0
                and os.environ.get("B200_DP_PEER", "1") != "0"):
            # (False on every rank when any of them could not map a peer: all keep the NCCL all-reduce)
            self.dp_peer = cm.dp_peer_setup(group, self.pack, self.W, self.W_aux)
            self._peer_group = group if self.dp_peer else None   # the first update starts with a host barrier: ranks may finish set-up seconds apart
        self._batch = cm.CUDAMatrix._from_mat(cm.cudamat())   # the recorded step's view of the current minibatch
        self._batch_aux = cm.CUDAMatrix._from_mat(cm.cudamat())   # ... and of its 16-bit parts, when the caller has them
        self._given_aux = None

    def _act(self, layer_activation):
        return 1 if layer_activation == LOGISTIC else 0

    def _gibbs_steps(self, step):
        """deepnet/dbm.py:202-208: the step-up schedule adds a Gibbs step every step_up_cd_after updates."""
        h = self.hyp
        if 0 < h.start_step_up_cd_after < step:
            return h.gibbs_steps + 1 + (step - h.start_step_up_cd_after) // h.step_up_cd_after
        return h.gibbs_steps

    def _sample_visible(self, step):
        """deepnet/dbm.py:217-222: the visible layer feeds a draw upward instead of its means."""
        return bool(self.hyp.sample_input) and self.hyp.sample_input_after <= step

    # launches behind one operation of the vocabulary (row and column sums: partial + finishing launch)
    _LAUNCHES = dict(sum=2, add_sums=2, sm_limit=0, allreduce_end=0)

    def _op(self, X, name, flops, nbytes, method, *args, **kw):
        """Names one operation of the step to the executor X (`Immediate` or a recording `Program`);
        with a timeline attached, brackets the immediate call with CUDA events."""
        self.kernel_launches += self._LAUNCHES.get(method, 1)
        fn = getattr(X, method)
        if self.timeline is None or isinstance(X, self.cm.Program):
            return fn(*args, **kw)
        e0 = self.cm.Event().record()
        r = fn(*args, **kw)
        e1 = self.cm.Event().record()
        self.timeline.append((name, flops, nbytes, e0, e1))
        return r

    def TrainOneBatch(self, step, data, data_aux=None):
        """One CD-k update on `data` (V x B device matrix).  Nothing returns to the host.
        data_aux: the 16-bit parts of `data` in the form this engine's products read (the data
        feed writes them while gathering the minibatch); without it the step begins by splitting."""
        cm = self.cm
        if self.dp_peer and self._peer_group is not None:
            self._peer_group.barrier()
            self._peer_group = None
        k, draw_v = self._gibbs_steps(step), self._sample_visible(step)
        if self.visible == LINEAR:
            draw_v = False
        mom, eps = self._sched.GetMomentumAndEpsilon(step)
        emom, eeps = self._esched.GetMomentumAndEpsilon(step)
        eh = self.ehyp
        l2 = eh.l2_decay if eh.apply_l2_decay else 0.0
        l1 = eh.l1_decay if (eh.apply_l1_decay and step > eh.apply_l1decay_after) else 0.0
        sc = dict(mom=mom, eps=eps, emom=emom, eeps=eeps, l2=l2, l1=l1, inv_b=1.0 / (self.B * self.world_size))
        if draw_v and self.v_samp is None:
            self.v_samp, self.v_samp_aux = cm.empty((self.V, self.B)), cm.empty_aux((self.V, self.B))
        body = (self._issue_replicated_softmax if self.visible == REPLICATED_SOFTMAX
                else (self._issue_f16 if self.f16 else self._issue))
        if data_aux is not None and not (self.state_aux and self.visible != REPLICATED_SOFTMAX):
            data_aux = None                      # this engine derives the parts of the data in its kernels
        self._given_aux = data_aux
        if not self.use_program or self.timeline is not None:
            self.kernel_launches = 0
            return body(cm.Immediate(), data, k, draw_v, sc)
        key = (k, draw_v, data_aux is not None)
        rec = self._programs.get(key)
        if rec is None:
            prog = cm.Program()
            self.kernel_launches = 0
            self._given_aux = self._batch_aux if data_aux is not None else None
            handles = body(prog, self._batch, k, draw_v, sc)
            rec = self._programs[key] = (prog, handles, self.kernel_launches)
        prog, (ub, uw), self.kernel_launches = rec
        # the recorded step reads the minibatch through one handle: point it at this batch
        for view, m in ((self._batch, data), (self._batch_aux, data_aux)):
            if m is not None:
                ct.memmove(ct.byref(view.mat), ct.byref(m.mat), ct.sizeof(m.mat))
                view.mat.owns_data = 0
        self._batch_owner = (data, data_aux)
        if isinstance(ub, tuple):       # the peer-memory update: one operation carries every scalar
            prog.set_floats(ub[1], f0=sc["inv_b"], f1=mom, f2=eps, f3=emom, f4=eeps, f5=l2, f6=l1)
        else:
            prog.set_floats(ub, f0=sc["inv_b"], f1=mom, f2=eps)
            for op in (uw if isinstance(uw, list) else [uw]):
                prog.set_floats(op, f0=sc["inv_b"], f1=emom, f2=eeps, f3=l2, f4=l1)
        prog.run()

    def _issue_updates(self, X, sc, wb, w_scale=None):
        """All-reduce of the packed statistics, then the two updates (biases are not regularised,
        deepnet/dbm.py:249).  Returns the operations whose scalars follow the schedules."""
        V, H = self.V, self.H
        if self.dp_peer:
            # exchange + update of every parameter in one pass over peer memory (no NCCL)
            u = self._op(X, "peer_update", 0, 6 * wb, "dp_peer_update", self.W, self.dW, self.W_aux, w_scale, self.pack,
                         self.b, self.db, sc["inv_b"], sc["mom"], sc["eps"], sc["emom"], sc["eeps"], l2=sc["l2"], l1=sc["l1"])
            return ("peer", u), None
        if self.world_size > 1:
            self._op(X, "allreduce", 0, 4.0 * (V * H + V + H), "allreduce", self.pack)
        ub = self._op(X, "update_bias", 0, 20.0 * (V + H), "momentum_update", self.b, self.db, None, self.suff_b,
                      sc["inv_b"], sc["mom"], sc["eps"])
        uw = self._op(X, "update_W", 0, 6 * wb, "momentum_update", self.W, self.dW, None, self.suff_W, sc["inv_b"],
                      sc["emom"], sc["eeps"], l2=sc["l2"], l1=sc["l1"], w_aux=self.W_aux, w_scale=w_scale)
        return ub, uw

    def _issue(self, X, data, k, draw_v, sc):
        """CD-k with split-TF32 products (parts derived in the kernel, or bfloat16 parts from aux matrices)."""
        cm = self.cm
        V, H, B = self.V, self.H, self.B
        W, Wa, P = self.W, self.W_aux, cm.split_passes
        v0 = data
        gf = 2.0 * V * H * B                      # algorithmic flops of one product
        vb, hb, wb = 4.0 * V * B, 4.0 * H * B, 4.0 * V * H
        exact = self.binary_data                  # 0/1 data have no low part
        sa = self.state_aux
        v0a = self._given_aux if self._given_aux is not None else self.data_aux
        if sa and self._given_aux is None:
            self._op(X, "split", 0, 2 * vb, "split_bf16", v0, v0a)
        h_samp_aux, v_neg_aux = (self.h_samp_aux, self.v_neg_aux) if sa else (None, None)
        # positive phase: h0 = sigmoid(W' v0 + b_h), and its Bernoulli sample
        self._op(X, "gemm_up", gf, 2.5 * hb, "fused_gemm",
                 P(W.T, v0, exact_b=exact, a_aux=Wa, b_aux=v0a if sa else None),
                 out=self.h_pos, sample=self.h_samp, sample_aux=h_samp_aux, bias=self.bh, activation=1)
        # negative phase: k Gibbs steps; the visible means feed upward, or with sample_input (logistic
        # visible units only) their Bernoulli draw, which costs one sampling call per step
        for i in range(k):
            self._op(X, "gemm_down", gf, 2 * vb, "fused_gemm",
                     P(W, self.h_samp, exact_b=True, a_aux=Wa, b_aux=h_samp_aux), out=self.v_neg,
                     out_aux=None if draw_v else v_neg_aux, sample=self.v_samp if draw_v else None,
                     sample_aux=self.v_samp_aux if (draw_v and sa) else None, bias=self.bv,
                     activation=self._act(self.visible))
            if i == 0:
                self._op(X, "sq_err", 0, 2 * vb, "sq_diff", self.v_neg, v0, self.loss_acc)
            # the hidden means are only read after the last step (statistics); before that the draw suffices
            up = (P(W.T, self.v_samp, exact_b=True, a_aux=Wa, b_aux=self.v_samp_aux if sa else None) if draw_v
                  else P(W.T, self.v_neg, a_aux=Wa, b_aux=v_neg_aux))
            self._op(X, "gemm_up", gf, 2.5 * hb, "fused_gemm", up,
                     out=self.h_neg if i == k - 1 else None, sample=self.h_samp, sample_aux=h_samp_aux,
                     bias=self.bh, activation=1)
        # statistics: pos - neg in one product: the difference of two nearly equal products, so its
        # correction terms are TF32 products too; bias statistics: row sums of pos - neg, one launch a layer
        pos = P(v0, self.h_pos.T, exact_a=exact, terms="tf32")
        neg = P(self.v_neg, self.h_neg.T, negate=1, terms="tf32")
        self._op(X, "gemm_stats", 2 * gf, wb, "fused_gemm", pos + neg, out=self.suff_W)
        self._op(X, "row_sum", 0, 2 * vb, "row_sum_diff", v0, self.v_neg, self.suff_bv)
        self._op(X, "row_sum", 0, 2 * hb, "row_sum_diff", self.h_pos, self.h_neg, self.suff_bh)
        return self._issue_updates(X, sc, wb)

    def _issue_f16(self, X, data, k, draw_v, sc):
        """The binary-data, logistic-units CD-k update with every big product on scaled
        half-precision operands: states and data as x * 2^14 = hi + lo in fp16 (written by the
        producing epilogue, `split_f16` for the data), W as W * 2^e (written by the update kernel,
        which also keeps e); a product is hi.lo + lo.hi + hi.hi, 0/1 operands need hi only."""
        cm = self.cm
        V, H, B = self.V, self.H, self.B
        W, Wa, We, F = self.W, self.W_aux, self.W_exp, cm.f16_passes
        E = 14                                     # exponent of every state: values in [0, 1]
        v0, v0a = data, (self._given_aux if self._given_aux is not None else self.data_aux)
        gf = 2.0 * V * H * B
        vb, hb, wb = 4.0 * V * B, 4.0 * H * B, 4.0 * V * H
        act = dict(scale_exp=We, scale_exp_const=E, aux_f16=True, aux_exp=E)
        if self._given_aux is None:
            self._op(X, "split", 0, 2 * vb, "split_f16", v0, v0a, None, E)
        # positive phase: h0 = sigmoid(W' v0 + b_h), its Bernoulli sample, and the parts of both
        self._op(X, "gemm_up", gf, 3.5 * hb, "fused_gemm", F(W.T, Wa, v0, v0a, exact_b=True), out=self.h_pos,
                 out_aux=self.h_pos_aux, sample=self.h_samp, sample_aux=self.h_samp_aux, bias=self.bh, activation=1,
                 **act)
        for i in range(k):
            last = i == k - 1
            # the fp32 visible means are read by the error of the first reconstruction and by the
            # statistics after the last step; in between only their half-precision form is (and not
            # even that when the draw feeds upward: sample_input, one more sampling call per step)
            self._op(X, "gemm_down", gf, 2 * vb, "fused_gemm", F(W, Wa, self.h_samp, self.h_samp_aux, exact_b=True),
                     out=self.v_neg if (i == 0 or last) else None,
                     out_aux=self.v_neg_aux if (last or not draw_v) else None,
                     sample_aux=self.v_samp_aux if draw_v else None, bias=self.bv, activation=1, **act)
            if i == 0:
                self._op(X, "sq_err", 0, 2 * vb, "sq_diff", self.v_neg, v0, self.loss_acc)
            # the hidden means (and their parts) are only read after the last step, by the statistics
            # (the next product reads the draw's half-precision plane; the fp32 draw is kept for the caller)
            up = (F(W.T, Wa, self.v_samp, self.v_samp_aux, exact_b=True) if draw_v
                  else F(W.T, Wa, self.v_neg, self.v_neg_aux))
            self._op(X, "gemm_up", gf, 2.5 * hb, "fused_gemm", up,
                     out=self.h_neg if last else None, out_aux=self.h_neg_aux if last else None,
                     sample=self.h_samp if last else None, sample_aux=self.h_samp_aux, bias=self.bh, activation=1,
                     **act)
        # column panels of W as (first column, columns): equal ones, or the widths asked for
        bounds = []
        if self.world_size > 1 and not self.dp_peer:
            widths = self.dp_panel_cols or ([H // self.dp_panels] * self.dp_panels if self.dp_panels > 1 else [])
            if 1 < len(widths) < 8 and sum(widths) == H and all(w > 0 and w % 8 == 0 for w in widths):
                first = 0
                for w in widths:
                    bounds.append((first, w))
                    first += w
        panels = len(bounds) if bounds else 1
        if panels == 1:
            pos = F(v0, v0a, self.h_pos.T, self.h_pos_aux, exact_a=True)
            neg = F(self.v_neg, self.v_neg_aux, self.h_neg.T, self.h_neg_aux, negate=1)
            self._op(X, "gemm_stats", 2 * gf, wb, "fused_gemm", pos + neg, out=self.suff_W, scale_exp_const=2 * E)
            self._op(X, "row_sum", 0, 2 * vb, "row_sum_diff", v0, self.v_neg, self.suff_bv)
            self._op(X, "row_sum", 0, 2 * hb, "row_sum_diff", self.h_pos, self.h_neg, self.suff_bh)
            self.kernel_launches += 2                  # the exponent launch and the pass that writes W's aux
            return self._issue_updates(X, sc, wb, w_scale=self.W_scale)
        # Data parallel: the statistics are multiplied, all-reduced and applied in column panels of W.
        # Panel p's all-reduce runs on a side stream while panel p + 1 multiplies (the persistent
        # product kernel leaves it a few SMs), and each panel is updated as its sum arrives, so
        # the exchange hides behind the product instead of standing between product and update.
        if self.dp_panel_products:
            for p, (c0, nc) in enumerate(bounds):
                if p == 1:   # from the second panel on an all-reduce runs beside the product
                    self._op(X, "sm_limit", 0, 0, "sm_limit", max(cm.sm_count() - self.dp_reserved_sms, 2))
                win = (c0, nc)
                pos = F(v0, v0a, self.h_pos.T, self.h_pos_aux, exact_a=True, b_rows=win)
                neg = F(self.v_neg, self.v_neg_aux, self.h_neg.T, self.h_neg_aux, negate=1, b_rows=win)
                panel = self.suff_W.slice(c0, c0 + nc)
                self._op(X, "gemm_stats", 2 * gf * nc / H, wb * nc / H, "fused_gemm", pos + neg, out=panel,
                         scale_exp_const=2 * E)
                self._op(X, "allreduce_begin", 0, 0, "allreduce_begin", panel, p)
            self._op(X, "sm_limit", 0, 0, "sm_limit", 0)
        else:
            # one product on every SM, then the all-reduce in panels beside the panels' updates
            pos = F(v0, v0a, self.h_pos.T, self.h_pos_aux, exact_a=True)
            neg = F(self.v_neg, self.v_neg_aux, self.h_neg.T, self.h_neg_aux, negate=1)
            self._op(X, "gemm_stats", 2 * gf, wb, "fused_gemm", pos + neg, out=self.suff_W, scale_exp_const=2 * E)
            for p, (c0, nc) in enumerate(bounds):
                self._op(X, "allreduce_begin", 0, 0, "allreduce_begin", self.suff_W.slice(c0, c0 + nc), p)
        self._op(X, "row_sum", 0, 2 * vb, "row_sum_diff", v0, self.v_neg, self.suff_bv)
        self._op(X, "row_sum", 0, 2 * hb, "row_sum_diff", self.h_pos, self.h_neg, self.suff_bh)
        self._op(X, "allreduce_begin", 0, 0, "allreduce_begin", self.suff_b, panels)
        uw = []
        for p, (c0, nc) in enumerate(bounds):
            self._op(X, "allreduce_end", 0, 0, "allreduce_end", p)
            uw.append(self._op(X, "update_W", 0, 6 * wb * nc / H, "momentum_update_columns", self.W, self.dW, None,
                               self.suff_W, c0, nc, sc["inv_b"], sc["emom"], sc["eeps"], l2=sc["l2"], l1=sc["l1"],
                               w_aux=self.W_aux, w_scale=self.W_scale))
        self._op(X, "allreduce_end", 0, 0, "allreduce_end", panels)
        ub = self._op(X, "update_bias", 0, 20.0 * (V + H), "momentum_update", self.b, self.db, None, self.suff_b,
                      sc["inv_b"], sc["mom"], sc["eps"])
        self.kernel_launches += 2
        return ub, uw

    def _issue_replicated_softmax(self, X, data, k, draw_v, sc):
        """CD-k with a replicated-softmax visible layer (word-count columns): the call sequence of
        deepnet/dbm.py:118-238 with replicated_softmax_layer.py:12-60,90-154 and edge.py:222-246, on
        fused kernels.  Same random stream as the call-by-call driver: one call for the positive
        hidden draw, then per Gibbs step one call per document for the multinomial draw (with
        sample_input) and one for the hidden draw."""
        cm = self.cm
        V, H, B = self.V, self.H, self.B
        W, Wa, P = self.W, self.W_aux, cm.split_passes   # the small state matrices' parts are derived in the kernel
        gf = 2.0 * V * H * B
        vb, hb, wb = 4.0 * V * B, 4.0 * H * B, 4.0 * V * H
        v0 = data                                              # integer counts: exact in TF32
        # GetData: NN = column sums + tiny; v0n = data / NN for the statistics
        self._op(X, "col_sum", 0, vb, "sum", v0, 0, self.NN)
        self._op(X, "add_scalar", 0, 8.0 * B, "add_scalar", self.NN, self.tiny)
        self._op(X, "div_by_row", 0, 2 * vb, "div_by_row", v0, self.NN, self.v0n)
        # positive phase: hidden bias is scaled by the document length (deepnet/dbm.py:101-104)
        self._op(X, "gemm_up", gf, 2 * hb, "fused_gemm", P(W.T, v0, exact_b=True, a_aux=Wa), out=self.h_pos,
                 sample=self.h_samp, bias=self.bh, col_scale=self.NN, activation=1)
        for i in range(k):
            # visible: NN * softmax(W h + b_v)
            self._op(X, "gemm_down", gf, vb, "fused_gemm", P(W, self.h_samp, exact_b=True, a_aux=Wa), out=self.v_act,
                     bias=self.bv, activation=0)
            self._op(X, "softmax", 0, 2 * vb, "softmax_scaled", self.v_act, self.NN, self.v_neg)
            self._op(X, "div_by_row", 0, 2 * vb, "div_by_row", self.v_neg, self.NN, self.v_negn)
            if i == 0:   # squared error between state / NN and the counts (replicated_softmax_layer.py:128-135)
                self._op(X, "sq_err", 0, 2 * vb, "sq_diff", self.v_negn, v0, self.loss_acc)
            if draw_v:   # word counts drawn from the softmax feed upward
                self._op(X, "multinomial", 0, 2 * vb, "sample_multinomial", self.v_neg, self.NN, self.v_samp)
                up = P(W.T, self.v_samp, exact_b=True, a_aux=Wa)
            else:        # sample_input off: the expected counts do (deepnet/dbm.py:222)
                up = P(W.T, self.v_neg, a_aux=Wa)
            self._op(X, "gemm_up", gf, 2 * hb, "fused_gemm", up,
                     out=self.h_neg, sample=self.h_samp, bias=self.bh, col_scale=self.NN, activation=1)
        pos = P(self.v0n, self.h_pos.T, terms="tf32")
        neg = P(self.v_negn, self.h_neg.T, negate=1, terms="tf32")
        self._op(X, "gemm_stats", 2 * gf, wb, "fused_gemm", pos + neg, out=self.suff_W)
        self._op(X, "row_sum", 0, 2 * vb, "row_sum_diff", self.v0n, self.v_negn, self.suff_bv)
        self._op(X, "row_sum", 0, 2 * hb, "row_sum_diff", self.h_pos, self.h_neg, self.suff_bh)
        return self._issue_updates(X, sc, wb)

    def refresh_weight_aux(self):
        """Rebuilds the 16-bit parts of W after W was written from outside (a loaded checkpoint)."""
        if self.f16:
            w = np.array(self.W.asarray())
            self.W_scale = self.cm.f16_scale_state(float(np.abs(w).max()))
            self.W_exp = self.W_scale.slice(0, 1)
            self.W.split_f16(self.W_aux, exp_dev=self.W_exp)
        else:
            self.W.split_bf16(self.W_aux)

    def Inference(self, data, input_recon=False):
        """Hidden representation of `data` (V x cases device matrix), minibatch by minibatch:
        the inference-only positive phase of deepnet/dbm.py:340-398 (extract_rbm_representation.py)
        as one fused product per minibatch.  Returns (cases x H) host array, and with input_recon
        also the summed squared error of the input reconstructed from the hidden means."""
        cm, B, W, P = self.cm, self.B, self.W, self.cm.split_passes
        Wa = None if self.f16 else self.W_aux     # the bfloat16 parts exist only in that form of the aux
        n = data.shape[1] // B
        rep = np.zeros((n * B, self.H), np.float32)
        err = 0.0
        soft = self.visible == REPLICATED_SOFTMAX
        for b in range(n):
            v0 = data.slice(b * B, (b + 1) * B)
            if soft:
                v0.sum(axis=0, target=self.NN)
                self.NN.add(self.tiny)
            cm.fused_gemm(P(W.T, v0, exact_b=soft or self.binary_data, a_aux=Wa), out=self.h_pos, bias=self.bh, activation=1,
                          col_scale=self.NN if soft else None)
            if input_recon:
                down = P(W, self.h_pos, a_aux=Wa)
                if soft:
                    cm.fused_gemm(down, out=self.v_act, bias=self.bv, activation=0)
                    self.v_act.softmax_scaled(self.NN, target=self.v_neg)
                    self.v_neg.div_by_row(self.NN, target=self.v_negn)
                    cm._check(cm._lib.add_sq_diff(self.v_negn.p_mat, v0.p_mat, self.loss_acc.p_mat))
                else:
                    cm.fused_gemm(down, out=self.v_neg, bias=self.bv, activation=self._act(self.visible))
                    cm._check(cm._lib.add_sq_diff(self.v_neg.p_mat, v0.p_mat, self.loss_acc.p_mat))
            rep[b * B:(b + 1) * B, :] = np.array(self.h_pos.asarray()).T
        if input_recon:
            err = self.read_loss()
            return rep, err
        return rep

    def read_loss(self, reset=True):
        """Sum of squared reconstruction errors accumulated since the last reset (blocks)."""
        v = float(np.array(self.loss_acc.asarray())[0, 0])
        if reset:
            self.loss_acc.assign(0)
        return v

    def close(self, group=None):
        """Ends the peer-memory exchange (if this engine set it up): waits for the enqueued work, meets
        the other ranks (nobody unmaps a replica while a peer may still store into it; pass the group
        for that), unmaps the peers and stops the delivery of the statistics panels.  Call it before
        the engine's matrices are freed; the all-reduce form needs no closing."""
        if not self.dp_peer:
            return
        self.cm.cuda_sync_threads()
        if group is not None:
            group.barrier()
        self.cm.dp_peer_close()
        self.dp_peer = False
