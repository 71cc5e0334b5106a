"""Contrastive-divergence / PCD training step of an RBM or DBM over a `cm` backend.

A Python-3 restatement of the call sequence of the reference's hot path, one `cm`
call per reference call, so that the same driver runs on b200mat (GPU) and, in the
tests, on the CPU oracle:

  deepnet/dbm.py:15-26    SetPhase             deepnet/dbm.py:64-115   ComputeUp
  deepnet/dbm.py:118-167  PositivePhase        deepnet/dbm.py:169-181  InitializeNegPhase
  deepnet/dbm.py:183-238  NegativePhase        deepnet/dbm.py:240-261  UpdateLayerParams / UpdateEdgeParams
  deepnet/dbm.py:268-274  TrainOneBatch        deepnet/parameter.py:80-125  Update / GetMomentumAndEpsilon
  deepnet/layer.py:128-213, logistic_layer.py, linear_layer.py, replicated_softmax_layer.py,
  deepnet/edge.py:222-246.

Configuration is plain Python (the reference reads protobuf text files; the
hyper-parameter names are the ones of deepnet/protos/deepnet.proto:89-179).
Dropout, sparsity, tied parameters and weight-norm limits are not on the path of the
benchmark configurations and are not restated.
"""
import numpy as np

LOGISTIC, LINEAR, REPLICATED_SOFTMAX, SOFTMAX = "LOGISTIC", "LINEAR", "REPLICATED_SOFTMAX", "SOFTMAX"
CD, PCD = "CD", "PCD"


class Hyperparams(object):
    """The fields of deepnet.proto Hyperparams that the path reads (defaults as in the proto)."""

    def __init__(self, **kw):
        self.base_epsilon = 0.01
        self.epsilon_decay = "NONE"           # NONE | INVERSE_T | EXPONENTIAL
        self.epsilon_decay_half_life = 1000
        self.initial_momentum = 0.0
        self.final_momentum = 0.0
        self.momentum_change_steps = 10
        self.apply_l2_decay = False
        self.l2_decay = 0.01
        self.apply_l1_decay = False
        self.l1_decay = 0.01
        self.apply_l1decay_after = 0
        self.start_learning_after = 0
        self.sample_input = False
        self.sample_input_after = 0
        self.mf_steps = 1
        self.gibbs_steps = 1
        self.start_step_up_cd_after = 0
        self.step_up_cd_after = 0
        self.adaptive_prior = 0
        for k, v in kw.items():
            if not hasattr(self, k):
                raise AttributeError("unknown hyperparameter %s" % k)
            setattr(self, k, v)

    def copy(self, **kw):
        h = Hyperparams(**self.__dict__)
        for k, v in kw.items():
            setattr(h, k, v)
        return h


class Parameter(object):
    """deepnet/parameter.py: holds params, gradient, gradient_history; momentum update."""

    def __init__(self, cm, hyperparams):
        self.cm = cm
        self.hyperparams = hyperparams
        self.params = {}
        self.gradient = None
        self.gradient_history = None
        self.num_grads_received = 0
        self.num_shares = 1

    def GetMomentumAndEpsilon(self, step):
        """deepnet/parameter.py:108-125."""
        h = self.hyperparams
        momentum = h.final_momentum - (h.final_momentum - h.initial_momentum) * \
            np.exp(-float(step) / h.momentum_change_steps)
        epsilon = h.base_epsilon
        if h.epsilon_decay == "INVERSE_T":
            epsilon = h.base_epsilon / (1 + float(step) / h.epsilon_decay_half_life)
        elif h.epsilon_decay == "EXPONENTIAL":
            epsilon = h.base_epsilon / np.power(2, float(step) / h.epsilon_decay_half_life)
        if step < h.start_learning_after:
            epsilon = 0.0
        return momentum, epsilon

    def Update(self, param_name, step, no_reg=False):
        """deepnet/parameter.py:80-106."""
        h = self.hyperparams
        momentum, epsilon = self.GetMomentumAndEpsilon(step)
        w = self.params[param_name]
        w_delta = self.gradient_history
        gradient = self.gradient
        w_delta.mult(momentum)
        if not no_reg and h.apply_l2_decay:
            w_delta.add_mult(w, h.l2_decay)
        if not no_reg and h.apply_l1_decay and step > h.apply_l1decay_after:
            w_delta.add_mult_sign(w, h.l1_decay)
        w_delta.add_mult(gradient)
        w.add_mult(w_delta, -epsilon)
        self.num_grads_received = 0
        gradient.assign(0)


class Layer(Parameter):
    """deepnet/layer.py: state / sample / data / statistics buffers of one layer."""

    activation = None

    def __init__(self, cm, name, numdims, hyperparams, is_input=False, optimizer=CD, bias=None):
        super(Layer, self).__init__(cm, hyperparams)
        self.name = name
        self.numdims = numdims
        self.is_input = is_input
        self.optimizer = optimizer
        self.sample_input = hyperparams.sample_input
        self.incoming_edge = []
        self.incoming_neighbour = []
        self.replicated_neighbour = None
        self.replicate_bias = True
        self.tiny = 1e-10
        self.data = None
        b = np.zeros((numdims, 1), np.float32) if bias is None else np.asarray(bias, np.float32).reshape(numdims, 1)
        self.params["bias"] = cm.CUDAMatrix(b)

    def AllocateMemory(self, batchsize):
        """deepnet/layer.py:157-200."""
        cm, n = self.cm, self.numdims
        self.batchsize = batchsize
        z = lambda r, c: cm.CUDAMatrix(np.zeros((r, c), np.float32))
        self.statesize = z(n, batchsize)
        self.batchsize_temp = z(1, batchsize)
        self.state = z(n, batchsize)
        self.gradient = z(n, 1)
        self.gradient_history = z(n, 1)
        self.suff_stats = cm.empty((n, 1))
        if self.optimizer == PCD:
            self.pos_state = self.state
            self.pos_sample = z(n, batchsize)
            self.neg_state = z(n, batchsize)
            self.neg_sample = z(n, batchsize)
            self.sample = self.pos_sample
        else:
            self.sample = z(n, batchsize)
        if self.is_input:
            self.data = z(n, batchsize)

    def AddIncomingEdge(self, edge):
        """deepnet/layer.py:103-112."""
        if edge not in self.incoming_edge:
            self.incoming_edge.append(edge)
            neighbour = edge.node2 if self is edge.node1 else edge.node1
            self.incoming_neighbour.append(neighbour)
            if neighbour.replicate_bias and neighbour.activation == REPLICATED_SOFTMAX:
                self.replicated_neighbour = neighbour

    def SetData(self, data):
        self.data = data

    def ResetState(self, rand=False):
        """deepnet/layer.py:128-133."""
        if rand:
            self.state.fill_with_randn()
            self.ApplyActivation()
        else:
            self.state.assign(0)

    def GetData(self):
        self.state.assign(self.data)

    def CollectSufficientStatistics(self, neg=False):
        """deepnet/layer.py:202-213 (without sparsity)."""
        if not neg:
            self.state.sum(axis=1, target=self.suff_stats)
        else:
            self.suff_stats.add_sums(self.state, axis=1, mult=-1.0)

    def _squared_loss(self):
        target = self.statesize
        self.state.subtract(self.data, target=target)
        return target.euclid_norm() ** 2


class LogisticLayer(Layer):
    """deepnet/logistic_layer.py:11-15,48-52."""
    activation = LOGISTIC

    def ApplyActivation(self):
        self.cm.sigmoid(self.state)

    def Sample(self):
        self.state.sample_bernoulli(target=self.sample)

    def GetLoss(self):
        return self._squared_loss()


class LinearLayer(Layer):
    """deepnet/linear_layer.py:11-32,47-58 (no learned precision)."""
    activation = LINEAR

    def ApplyActivation(self):
        pass

    def Sample(self):
        pass

    def GetLoss(self):
        return self._squared_loss()


class ReplicatedSoftmaxLayer(Layer):
    """deepnet/replicated_softmax_layer.py."""
    activation = REPLICATED_SOFTMAX

    def AllocateMemory(self, batchsize):
        super(ReplicatedSoftmaxLayer, self).AllocateMemory(batchsize)
        cm, n = self.cm, self.numdims
        self.expanded_batch = cm.CUDAMatrix(np.zeros((n, batchsize), np.float32))
        self.NN = cm.CUDAMatrix(np.ones((1, batchsize), np.float32))
        self.big_sample_matrix = cm.empty((n, 1000))

    def ApplyActivation(self):
        """:12-21: state = NN * softmax over the vocabulary of each column."""
        state, temp = self.state, self.batchsize_temp
        state.max(axis=0, target=temp)
        state.add_row_mult(temp, -1)
        self.cm.exp(state)
        state.sum(axis=0, target=temp)
        self.NN.divide(temp, target=temp)
        state.mult_by_row(temp)

    def Sample(self):
        """:23-60: NN[i] multinomial draws per document by the exponential-race trick."""
        sample, state = self.sample, self.state
        if self.hyperparams.adaptive_prior > 0:
            sample.assign(0)
            temp_sample = self.expanded_batch
            for _ in range(int(self.hyperparams.adaptive_prior)):
                state.perturb_prob_for_softmax_sampling(target=temp_sample)
                temp_sample.choose_max_and_accumulate(sample)
        else:
            NN = np.array(self.NN.asarray()).reshape(-1)
            max_samples = self.big_sample_matrix.shape[1]
            for i in range(self.batchsize):
                nn = int(NN[i])
                factor = 1
                if nn > max_samples:
                    nn = max_samples
                    factor = float(nn) / max_samples
                if nn <= 0:
                    sample.slice(i, i + 1).assign(0)
                    continue
                samples = self.big_sample_matrix.slice(0, nn)
                samples.assign(0)
                samples.add_col_vec(state.slice(i, i + 1))
                samples.perturb_prob_for_softmax_sampling()
                samples.choose_max(axis=0)
                samples.sum(axis=1, target=sample.slice(i, i + 1))
                if factor > 1:
                    sample.slice(i, i + 1).mult(factor)

    def ResetState(self, rand=False):
        self.NN.assign(1)
        super(ReplicatedSoftmaxLayer, self).ResetState(rand=rand)

    def GetData(self):
        """:90-105 (no priors)."""
        self.state.assign(self.data)
        self.state.sum(axis=0, target=self.NN)
        self.NN.add(self.tiny)
        h = self.hyperparams
        if h.adaptive_prior > 0:
            self.state.div_by_row(self.NN)
            self.state.mult(h.adaptive_prior)
            self.NN.assign(h.adaptive_prior)

    def GetLoss(self):
        """:107-141 with normalize_error off."""
        temp, target = self.batchsize_temp, self.statesize
        self.data.sum(axis=0, target=temp)
        temp.add(self.tiny)
        self.state.div_by_row(temp, target=target)
        target.subtract(self.data)
        return target.euclid_norm() ** 2

    def CollectSufficientStatistics(self, neg=False):
        """:146-154."""
        self.state.div_by_row(self.NN)
        if not neg:
            self.state.sum(axis=1, target=self.suff_stats)
        else:
            self.suff_stats.add_sums(self.state, axis=1, mult=-1.0)
        self.state.mult_by_row(self.NN)


class SoftmaxLayer(Layer):
    """deepnet/softmax_layer.py: one softmax over `numdims` labels per case (dimensions = 1, the
    label layer of deepnet/examples/dbm/model.pbtxt:57-81).  As an input its data is a 1 x batch
    row of label indices, expanded to one-hot columns (:35-36)."""
    activation = SOFTMAX

    def AllocateMemory(self, batchsize):
        super(SoftmaxLayer, self).AllocateMemory(batchsize)
        cm, n = self.cm, self.numdims
        self.expansion_matrix = cm.CUDAMatrix(np.eye(n, dtype=np.float32))
        self.deriv = cm.CUDAMatrix(np.zeros((n, batchsize), np.float32))
        if self.is_input:
            self.data = cm.CUDAMatrix(np.zeros((1, batchsize), np.float32))

    def ApplyActivation(self):
        """:11-12."""
        self.state.apply_softmax()

    def Sample(self):
        """:14-16: one categorical draw per column by the exponential race, as a one-hot."""
        self.state.perturb_prob_for_softmax_sampling(target=self.sample)
        self.sample.choose_max(axis=0)

    def GetData(self):
        """:35-36."""
        self.expansion_matrix.select_columns(self.data, target=self.state)

    def GetLoss(self):
        """:86-89 (SQUARED_LOSS): deriv = state - onehot(label) (apply_softmax_grad,
        cudamat/cudamat_kernels.cu:819-825), error = its squared norm."""
        self.expansion_matrix.select_columns(self.data, target=self.deriv)
        self.state.subtract(self.deriv, target=self.deriv)
        return self.deriv.euclid_norm() ** 2


_LAYER_TYPES = {LOGISTIC: LogisticLayer, LINEAR: LinearLayer, REPLICATED_SOFTMAX: ReplicatedSoftmaxLayer,
                SOFTMAX: SoftmaxLayer}


class Edge(Parameter):
    """deepnet/edge.py: weight (node1 units x node2 units) and its statistics."""

    def __init__(self, cm, node1, node2, hyperparams, weight, up_factor=1.0, down_factor=1.0):
        super(Edge, self).__init__(cm, hyperparams)
        self.node1, self.node2 = node1, node2
        self.name = "%s:%s" % (node1.name, node2.name)
        self.up_factor, self.down_factor = up_factor, down_factor
        w = np.asarray(weight, np.float32)
        assert w.shape == (node1.numdims, node2.numdims)
        self.params["weight"] = cm.CUDAMatrix(w)
        self.gradient = cm.CUDAMatrix(np.zeros(w.shape, np.float32))
        self.gradient_history = cm.CUDAMatrix(np.zeros(w.shape, np.float32))
        self.suff_stats = cm.empty(w.shape)
        node1.AddIncomingEdge(self)
        node2.AddIncomingEdge(self)

    def CollectSufficientStatistics(self, neg=False):
        """deepnet/edge.py:222-246 (without sparsity)."""
        n1, n2 = self.node1, self.node2
        if n1.activation == REPLICATED_SOFTMAX:
            n1.state.div_by_row(n1.NN)
        if n2.activation == REPLICATED_SOFTMAX:
            n2.state.div_by_row(n2.NN)
        if not neg:
            self.cm.dot(n1.state, n2.state.T, target=self.suff_stats)
        else:
            self.suff_stats.add_dot(n1.state, n2.state.T, mult=-1.0)
        if n1.activation == REPLICATED_SOFTMAX:
            n1.state.mult_by_row(n1.NN)
        if n2.activation == REPLICATED_SOFTMAX:
            n2.state.mult_by_row(n2.NN)


class DBM(object):
    """deepnet/dbm.py: an RBM is the one-edge case.

    layers: list of dicts {name, activation, numdims, is_input, hyperparams?, bias?}
    edges:  list of dicts {node1, node2, weight, hyperparams?, up_factor?, down_factor?}
    """

    def __init__(self, cm, layers, edges, hyperparams, batchsize, optimizer=CD, seed=0):
        self.cm = cm
        self.hyperparams = hyperparams
        self.batchsize = batchsize
        self.optimizer = optimizer
        self.cd = optimizer == CD
        cm.CUDAMatrix.init_random(seed)
        self.layer = []
        for spec in layers:
            cls = _LAYER_TYPES[spec["activation"]]
            l = cls(cm, spec["name"], spec["numdims"], spec.get("hyperparams", hyperparams),
                    is_input=spec.get("is_input", False), optimizer=optimizer, bias=spec.get("bias"))
            l.AllocateMemory(batchsize)
            self.layer.append(l)
        by_name = dict((l.name, l) for l in self.layer)
        self.edge = []
        for spec in edges:
            self.edge.append(Edge(cm, by_name[spec["node1"]], by_name[spec["node2"]],
                                  spec.get("hyperparams", hyperparams), spec["weight"],
                                  spec.get("up_factor", 1.0), spec.get("down_factor", 1.0)))
        self.input_datalayer = [l for l in self.layer if l.is_input]
        self.node_list = self.Sort()
        self.train_stop_steps = 0

    def GetLayerByName(self, name):
        for l in self.layer:
            if l.name == name:
                return l
        raise KeyError(name)

    def Sort(self):
        """deepnet/dbm.py:34-59: inputs first; both phase orders follow the layer list."""
        non_input = [n for n in self.layer if not n.is_input]
        node_list = list(self.input_datalayer) + non_input
        self.pos_phase_order = non_input
        self.neg_phase_order = node_list
        return node_list

    def SetPhase(self, layer, pos=True):
        if pos:
            layer.state, layer.sample = layer.pos_state, layer.pos_sample
        else:
            layer.state, layer.sample = layer.neg_state, layer.neg_sample

    def ComputeUp(self, layer, train=False, compute_input=False, step=0, maxsteps=0, use_samples=False,
                  neg_phase=False):
        """deepnet/dbm.py:64-105 (dropout branch not restated)."""
        cm = self.cm
        if layer.is_input and not compute_input:
            layer.GetData()
            return
        for i, edge in enumerate(layer.incoming_edge):
            neighbour = layer.incoming_neighbour[i]
            inputs = neighbour.sample if use_samples else neighbour.state
            if edge.node2 is layer:
                w = edge.params["weight"].T
                factor = edge.up_factor
            else:
                w = edge.params["weight"]
                factor = edge.down_factor
            if i == 0:
                cm.dot(w, inputs, target=layer.state)
                if factor != 1:
                    layer.state.mult(factor)
            else:
                layer.state.add_dot(w, inputs, mult=factor)
        b = layer.params["bias"]
        if layer.replicated_neighbour is None:
            layer.state.add_col_vec(b)
        else:
            layer.state.add_dot(b, layer.replicated_neighbour.NN)
        layer.ApplyActivation()

    def PositivePhase(self, train=False, evaluate=False, step=0):
        """deepnet/dbm.py:118-167."""
        for node in self.node_list:
            if node.is_input:
                self.ComputeUp(node, train=train)
            else:
                node.ResetState(rand=False)
        for _ in range(self.hyperparams.mf_steps):
            for node in self.pos_phase_order:
                self.ComputeUp(node, train=train, step=step, maxsteps=self.train_stop_steps)
        losses = []
        if train:
            for node in self.layer:
                node.CollectSufficientStatistics()
            for edge in self.edge:
                edge.CollectSufficientStatistics()
        if not self.cd or evaluate:
            for node in self.input_datalayer:
                self.ComputeUp(node, compute_input=True, step=step, maxsteps=self.train_stop_steps)
                losses.append(node.GetLoss())
        return losses

    def InitializeNegPhase(self, to_pos=False):
        """deepnet/dbm.py:169-181."""
        for layer in self.layer:
            self.SetPhase(layer, pos=False)
            if to_pos:
                layer.state.assign(layer.pos_state)
            else:
                layer.ResetState(rand=True)
            layer.Sample()
            self.SetPhase(layer, pos=True)

    def NegativePhase(self, step=0, train=True, gibbs_steps=-1):
        """deepnet/dbm.py:183-238."""
        losses = []
        if self.cd:
            for node in self.node_list:
                if not node.is_input:
                    node.Sample()
        else:
            for node in self.layer:
                self.SetPhase(node, pos=False)
        if gibbs_steps < 0:
            h = self.hyperparams
            start_after = h.start_step_up_cd_after
            if start_after > 0 and start_after < step:
                gibbs_steps = h.gibbs_steps + 1 + (step - start_after) // h.step_up_cd_after
            else:
                gibbs_steps = h.gibbs_steps
        for i in range(gibbs_steps):
            for node in self.neg_phase_order:
                self.ComputeUp(node, train=train, step=step, maxsteps=self.train_stop_steps, use_samples=True,
                               compute_input=True, neg_phase=True)
                if i == 0 and node.is_input and self.cd:
                    losses.append(node.GetLoss())
                if node.is_input:
                    if node.sample_input and node.hyperparams.sample_input_after <= step:
                        node.Sample()
                    else:
                        node.sample.assign(node.state)
                else:
                    node.Sample()
        if train:
            for node in self.layer:
                node.CollectSufficientStatistics(neg=True)
                self.UpdateLayerParams(node, step=step)
            for edge in self.edge:
                edge.CollectSufficientStatistics(neg=True)
                self.UpdateEdgeParams(edge, step=step)
        if not self.cd:
            for node in self.layer:
                self.SetPhase(node, pos=True)
        return losses

    def UpdateLayerParams(self, layer, step=0):
        """deepnet/dbm.py:240-249: biases are not regularised."""
        layer.gradient.add_mult(layer.suff_stats, -1.0 / layer.batchsize)
        layer.num_grads_received += 1
        if layer.num_grads_received == layer.num_shares:
            layer.Update("bias", step, no_reg=True)

    def UpdateEdgeParams(self, edge, step):
        """deepnet/dbm.py:251-261."""
        numcases = edge.node1.batchsize
        edge.gradient.add_mult(edge.suff_stats, -1.0 / numcases)
        edge.num_grads_received += 1
        if edge.num_grads_received == edge.num_shares:
            edge.Update("weight", step)

    def Inference(self, data, layernames, batchsize=None, input_recon=False):
        """Representations of `data` (dims x cases device matrix) at the named layers.

        deepnet/dbm.py:340-398 (Inference / WriteRepresentationToDisk) without the disk writer:
        per minibatch a positive phase with train=False, then each layer's state transposed to
        (cases x dims).  With input_recon the input is also reconstructed (evaluate=True) and
        the summed squared error returned under the key 'error'.
        """
        B = batchsize or self.batchsize
        n = data.shape[1] // B
        reps = dict((name, np.zeros((n * B, self.GetLayerByName(name).numdims), np.float32)) for name in layernames)
        err = 0.0
        for b in range(n):
            self.SetBatch([data.slice(b * B, (b + 1) * B)])
            losses = self.PositivePhase(train=False, evaluate=input_recon)
            err += float(np.sum(losses)) if losses else 0.0
            for name in layernames:
                reps[name][b * B:(b + 1) * B, :] = np.array(self.GetLayerByName(name).state.asarray()).T
        if input_recon:
            reps["error"] = err
        return reps

    def SetBatch(self, data_by_layer):
        """Stand-in for GetTrainBatch (deepnet/neuralnet.py:628-632): data is a device matrix per input."""
        for node, d in zip(self.input_datalayer, data_by_layer):
            node.SetData(d)

    def TrainOneBatch(self, step):
        """deepnet/dbm.py:268-274."""
        losses1 = self.PositivePhase(train=True, step=step)
        if step == 0 and self.optimizer == PCD:
            self.InitializeNegPhase(to_pos=True)
        losses2 = self.NegativePhase(step, train=True)
        losses1.extend(losses2)
        return losses1
