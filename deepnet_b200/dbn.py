"""Greedy stacking of RBMs into a deep belief network, and the representation writer that feeds it.

deepnet/dbn.py:6-16,202-209: a DBN is a stack of already trained RBMs turned into a fixed upward
(feed-forward) net, plus one RBM on top that is trained on what the upward net produces:
`TrainOneBatch` = forward pass through the lower layers, then a contrastive-divergence update of
the top RBM.  Here every lower layer is one fused product (bias and logistic in the epilogue) and
the top RBM is the fused engine.

deepnet/dbm.py:365-398 + extract_rbm_representation.py:4-53: the hidden representation of a whole
data set is written to disk as `<layer>-NNNNN-of-MMMMM.npy` shards (deepnet/datahandler.py:636-746)
with a `data.pbtxt` listing them, which is how a trained RBM's output becomes the next RBM's data.
"""
import os

import numpy as np

from .dbm import LINEAR, LOGISTIC


def get_bytes(mem_str):
    """deepnet/datahandler.py:418-435: '2.1M' -> bytes (K, M, G are powers of 1024)."""
    s = str(mem_str)
    units = {"K": 1024, "M": 1024 ** 2, "G": 1024 ** 3}
    if s[-1] in units:
        return int(float(s[:-1]) * units[s[-1]])
    return int(s)


class UpwardNet(object):
    """The lower layers of a DBN as a fixed feed-forward net (deepnet/dbn.py:9, 202-203): layer i
    computes act(W_i' x + b_i).  specs: list of (weight V_i x H_i, hidden bias, activation)."""

    def __init__(self, cm, specs, batchsize, fused=None):
        """fused: one product per layer with bias and activation in its epilogue (default where the
        backend has `fused_gemm`); False keeps the reference's three calls per layer."""
        self.cm, self.B = cm, batchsize
        self.layers = []
        for w, b, act in specs:
            w = np.asarray(w, np.float32)
            W = cm.CUDAMatrix(w)
            self.layers.append(dict(W=W, W_aux=W.split_bf16(cm.empty_aux(w.shape)) if hasattr(cm, "empty_aux") else None,
                                    b=cm.CUDAMatrix(np.asarray(b, np.float32).reshape(-1, 1)),
                                    act=1 if act == LOGISTIC else 0, state=cm.empty((w.shape[1], batchsize))))
        self.fused = hasattr(cm, "fused_gemm") if fused is None else bool(fused)

    def forward(self, data, exact_input=False):
        """States of the top lower layer for the minibatch `data` (dims x batch); exact_input: the
        data are 0/1 (no low part)."""
        cm, x, exact = self.cm, data, exact_input
        for l in self.layers:
            if self.fused:
                cm.fused_gemm(cm.split_passes(l["W"].T, x, exact_b=exact, a_aux=l["W_aux"]), out=l["state"], bias=l["b"],
                              activation=l["act"])
            else:   # the reference's calls (deepnet/neuralnet.py ForwardPropagate: dot, add_col_vec, activation)
                cm.dot(l["W"].T, x, target=l["state"])
                l["state"].add_col_vec(l["b"])
                if l["act"]:
                    cm.sigmoid(l["state"])
            x, exact = l["state"], False
        return x


class DBN(object):
    """deepnet/dbn.py: `lower` trained layers below an RBM that is being trained (`top`: an engine with
    TrainOneBatch(step, data) / Inference)."""

    def __init__(self, cm, lower_specs, top, batchsize, binary_data=False):
        self.cm, self.top = cm, top
        self.up = UpwardNet(cm, lower_specs, batchsize)
        self.binary_data = binary_data

    def TrainOneBatch(self, step, data):
        """deepnet/dbn.py:202-204."""
        return self.top.TrainOneBatch(step, self.up.forward(data, self.binary_data))

    def Represent(self, data):
        """deepnet/dbn.py:206-209 with train=False: the top RBM's hidden means for `data` (dims x cases)."""
        B = self.up.B
        n = data.shape[1] // B
        out = []
        for i in range(n):
            x = self.up.forward(data.slice(i * B, (i + 1) * B), self.binary_data)
            out.append(self.top.Inference(x))
        return np.concatenate(out, axis=0)


class ShardWriter(object):
    """Buffers rows of several named arrays and writes them as numbered .npy shards:
    `<name>-00001-of-0000N.npy`, N fixed up front from the total number of rows
    (deepnet/datahandler.py:636-746).  `memory` bounds the buffers of all names together, shared in
    proportion to their widths, so every name changes shard at the same row."""

    def __init__(self, names, output_dir, memory, numdims, datasize):
        os.makedirs(output_dir, exist_ok=True)
        self.names, self.output_dir, self.numdims = list(names), output_dir, list(numdims)
        total = min(get_bytes(memory), datasize * 4 * sum(numdims))
        self.rows_per_shard = max(1, total // (4 * sum(numdims)))
        self.num_shards = max(1, -(-datasize // self.rows_per_shard))
        self.buffers = [np.zeros((self.rows_per_shard, d), np.float32) for d in numdims]
        self.fill = [0] * len(names)
        self.shard = [0] * len(names)
        self.written = [0] * len(names)

    def _dump(self, i):
        if self.fill[i] == 0:
            return
        self.shard[i] += 1
        path = os.path.join(self.output_dir, "%s-%.5d-of-%.5d" % (self.names[i], self.shard[i], self.num_shards))
        np.save(path, self.buffers[i][:self.fill[i]])
        self.written[i] += self.fill[i]
        self.fill[i] = 0

    def submit(self, arrays):
        for i, rows in enumerate(arrays):
            rows = np.asarray(rows, np.float32)
            while len(rows):
                room = self.rows_per_shard - self.fill[i]
                take = rows[:room]
                self.buffers[i][self.fill[i]:self.fill[i] + len(take)] = take
                self.fill[i] += len(take)
                rows = rows[room:]
                if self.fill[i] == self.rows_per_shard:
                    self._dump(i)

    def commit(self):
        for i in range(len(self.names)):
            self._dump(i)
        return list(self.written)


def write_representations(represent, batches, names, numdims, datasize, output_dir, memory="1G", tag="train"):
    """deepnet/dbm.py:365-398: `represent(batch)` returns, per name, the (cases x dims) rows of one
    minibatch; they are sharded under output_dir.  Returns the rows written per name."""
    writer = ShardWriter(names, output_dir, memory, numdims, datasize)
    for batch in batches:
        writer.submit(represent(batch))
    return writer.commit()


def write_data_pbtxt(path, name, entries, prefix="", gpu_memory="2G", main_memory="30G"):
    """The text-format `Dataset` message that lists written representations
    (extract_rbm_representation.py:26-50; fields of deepnet/protos/deepnet.proto:278-296).
    entries: (data name, file pattern, size, dimensions)."""
    lines = ['name: "%s"' % name]
    for dname, pattern, size, dims in entries:
        lines += ["data {", '  name: "%s"' % dname, '  file_pattern: "%s"' % pattern, "  size: %d" % size,
                  "  dimensions: %d" % dims, "}"]
    lines += ['gpu_memory: "%s"' % gpu_memory, 'main_memory: "%s"' % main_memory, 'prefix: "%s"' % prefix]
    with open(path, "w") as f:
        f.write("\n".join(lines) + "\n")


def extract_representations(represent, datasets, names, numdims, base_output_dir, model_name, memory="10G"):
    """extract_rbm_representation.py:4-53: for every data set (tag -> (batches, size)) write the named
    layers' representations under base_output_dir/<tag>/ and describe them all in data.pbtxt."""
    os.makedirs(base_output_dir, exist_ok=True)
    entries = []
    for tag, (batches, size) in datasets.items():
        written = write_representations(represent, batches, names, numdims, size, os.path.join(base_output_dir, tag),
                                        memory=memory, tag=tag)
        for n, d, rows in zip(names, numdims, written):
            entries.append(("%s_%s" % (n, tag), os.path.join(tag, "%s-*-of-*.npy" % n), rows, d))
    write_data_pbtxt(os.path.join(base_output_dir, "data.pbtxt"), model_name, entries, prefix=base_output_dir)
    return entries
