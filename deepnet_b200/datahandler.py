"""Device-resident data feed: what the reference's GPU cache does for the training loop
(`GPUCache`, deepnet/datahandler.py:259-416: the data set in device memory, minibatches cut from
it, a shuffle per epoch, mean / standard-deviation normalisation and additive Gaussian noise on
the device), built for a GPU that holds the whole data set.

Differences in design, not in what the trainer sees:
  * 0/1 data are stored one bit per value (`cm.feed_pack`): configuration 4's million
    8192-dimensional cases take 1 GB, not 33, and a minibatch that has to cross PCIe is 4 MB, not 134.
  * nothing is shuffled in place.  An epoch has a key; position p of the epoch reads stored column
    perm_key(p), a bijection the gather kernel evaluates on the fly (`cm.feed_gather`).  The host
    draws no permutation and uploads no index vectors (the reference shuffles a host index array
    and swaps columns, datahandler.py:364-375).
  * normalisation is applied while gathering, to the minibatch only; the stored data stay raw.
  * the gather also writes the 16-bit parts of the minibatch that the tensor-core products read
    (otherwise a separate pass over the minibatch at the start of every update).
Every modality of a case (data, labels) shares the epoch's key, so they stay aligned.
Image translations (datahandler.py:340-362) are not on the contrastive-divergence path and are left out.
"""
import numpy as np


class DeviceFeed(object):
    def __init__(self, cm, arrays, randomize=False, binary=None, add_noise=None, sigma=0.01, seed=0, aux_mode=0, aux_exp=14):
        """arrays: host arrays (cases x dims), one per modality, as the reference's caches hold them.
        binary[i]: store modality i one bit per value (default: detect 0/1 data).  aux_mode: 16-bit
        parts written beside modality 0 (0 none, 1 bfloat16 parts, 2 scaled half precision)."""
        self.cm = cm
        self.num_data = len(arrays)
        self.datasize = int(np.asarray(arrays[0]).shape[0])
        self.randomize, self.seed, self.epoch = randomize, int(seed), 0
        self.add_noise = add_noise or [False] * self.num_data
        self.sigma = sigma
        self.aux_mode, self.aux_exp = aux_mode, aux_exp
        self.dims, self.packed, self.data = [], [], []
        for i, a in enumerate(arrays):
            a = np.asarray(a, np.float32)
            assert a.shape[0] == self.datasize
            is_bits = bool(np.isin(a, (0, 1)).all()) if binary is None else bool(binary[i])
            self.dims.append(a.shape[1])
            self.packed.append(is_bits)
            self.data.append(cm.feed_pack(a.T) if is_bits else cm.CUDAMatrix(a.T))
        self.means = [None] * self.num_data
        self.stds = [None] * self.num_data
        self._pos = 0
        self._out = {}          # (modality, batch size) -> output buffers, reused

    def SetDataStats(self, i, mean, std):
        """datahandler.py:377-383 (statistics passed in instead of read from a stats file)."""
        cm = self.cm
        self.means[i] = cm.CUDAMatrix(np.asarray(mean, np.float32).reshape(-1, 1))
        self.stds[i] = cm.CUDAMatrix((1e-10 + np.asarray(std, np.float32)).astype(np.float32).reshape(-1, 1))

    def key(self):
        return (self.seed, self.epoch)

    def order(self):
        """Stored case read at each position of the current epoch."""
        if not self.randomize:
            return np.arange(self.datasize)
        return self.cm.feed_permutation(self.datasize, self.key())

    def _buffers(self, i, count):
        buf = self._out.get((i, count))
        if buf is None:
            cm = self.cm
            aux = cm.empty_aux((self.dims[i], count)) if (i == 0 and self.aux_mode) else None
            buf = self._out[(i, count)] = (cm.empty((self.dims[i], count)), aux)
        return buf

    def Get(self, batchsize, get_last_piece=False):
        """The next `batchsize` cases of every modality as (dims x batch) device matrices; an epoch
        that ends with fewer is cut short (or, with get_last_piece, returns them), then the next
        epoch starts with a new key (datahandler.py:385-416).  The matrices are reused by the
        next call with the same batch size."""
        if self._pos == self.datasize:
            self._pos = 0
            self.epoch += 1
        start, end = self._pos, self._pos + batchsize
        if end > self.datasize:
            end = self.datasize
            if not get_last_piece or end == start:
                self._pos = self.datasize
                return self.Get(batchsize, get_last_piece=get_last_piece)
        self._pos = end
        batch = []
        for i in range(self.num_data):
            out, aux = self._buffers(i, end - start)
            self.cm.feed_gather(self.data[i], self.packed[i], self.dims[i], self.key(), self.randomize, start, out,
                                mean=self.means[i], std=self.stds[i], out_aux=aux, aux_mode=self.aux_mode if aux else 0,
                                aux_exp=self.aux_exp)
            if self.add_noise[i]:
                out.sample_gaussian(mult=self.sigma)          # datahandler.py:335-337
            batch.append(out)
        self.last_aux = self._buffers(0, end - start)[1]
        return batch
