"""Device-resident data feed: the GPU cache of the reference's data pipeline.

Restates `GPUCache` of deepnet/datahandler.py:259-416 over a `cm` backend: the data set
(or a chunk of it) lives in one (dims x cases) device matrix per modality, a minibatch
is a column slice (a view, no copy), an epoch ends with an in-place shuffle by
`swap_columns` on disjoint index halves, and mean / standard-deviation normalisation and
additive Gaussian noise run on the device.  The parent (disk and host caches of the
reference, datahandler.py:14-257) is reduced to a host array that is cut into chunks of
`capacity` cases; image translations (datahandler.py:340-362) are not restated.
"""
import numpy as np


class HostSource(object):
    """Parent of the device cache: hands out consecutive chunks of host arrays (cases x dims)."""

    def __init__(self, arrays, randomize=False, seed=0):
        self.arrays = [np.asarray(a, dtype=np.float32) for a in arrays]
        self.num_data = len(self.arrays)
        self.datasize = self.arrays[0].shape[0]
        self._maxpos = self.datasize
        self._pos = 0
        self.randomize = randomize
        self.rng = np.random.RandomState(seed)

    def Get(self, n):
        if self._pos >= self.datasize:
            self._pos = 0
            if self.randomize:
                perm = self.rng.permutation(self.datasize)
                self.arrays = [a[perm] for a in self.arrays]
        end = min(self._pos + n, self.datasize)
        out = [a[self._pos:end] for a in self.arrays]
        self._pos = end
        return out


class GPUCache(object):
    """deepnet/datahandler.py:259-416."""

    def __init__(self, cm, parent, capacity, randomize=False, add_noise=None, sigma=0.01, seed=0):
        self.cm = cm
        self.parent = parent
        self.num_data = parent.num_data
        self._maxpos = min(int(capacity), parent._maxpos)
        self._pos = 0
        self.datasize = 0
        self.randomize = randomize
        self.data = [None] * self.num_data
        self.empty = True
        self.allocated_memory_size = [0] * self.num_data
        self.normalize = [False] * self.num_data
        self.means = [None] * self.num_data
        self.stds = [None] * self.num_data
        self.add_noise = add_noise or [False] * self.num_data
        self.sigma = sigma
        self.rng = np.random.RandomState(seed)   # the reference shuffles with numpy's global generator

    def SetDataStats(self, i, mean, std):
        """:377-383 (statistics passed in instead of read from a stats file)."""
        self.normalize[i] = True
        self.means[i] = self.cm.CUDAMatrix(np.asarray(mean, np.float32).reshape(-1, 1))
        self.stds[i] = self.cm.CUDAMatrix(1e-10 + np.asarray(std, np.float32).reshape(-1, 1))

    def Normalize(self):
        """:299-306."""
        for i, batch in enumerate(self.data):
            if self.normalize[i]:
                batch.add_col_mult(self.means[i], mult=-1.0)
                batch.div_by_col(self.stds[i])

    def LoadData(self):
        """:308-333: pull the next chunk from the parent, reuse the device buffer when it fits."""
        data_cpu = self.parent.Get(self._maxpos)
        datasize = data_cpu[0].shape[0]
        assert datasize <= self._maxpos
        self.datasize = datasize
        for i, d in enumerate(data_cpu):
            mat = d.T
            size = mat.shape[0] * mat.shape[1]
            if size != self.allocated_memory_size[i]:
                if self.data[i] is not None:
                    self.data[i].free_device_memory()
                self.data[i] = self.cm.CUDAMatrix(mat)
                self.allocated_memory_size[i] = size
            else:
                self.data[i].overwrite(mat)
        self.Normalize()

    def ShuffleData(self):
        """:364-375: in-place shuffle, columns indices1[k] and indices2[k] change places."""
        indices = np.arange(self.datasize)
        self.rng.shuffle(indices)
        half = self.datasize // 2
        if half == 0:
            return
        indices1 = self.cm.CUDAMatrix(indices[:half].reshape(1, -1))
        indices2 = self.cm.CUDAMatrix(indices[half:2 * half].reshape(1, -1))
        for d in self.data:
            d.swap_columns(indices1, indices2, target=d)
        indices1.free_device_memory()
        indices2.free_device_memory()

    def Get(self, batchsize, get_last_piece=False):
        """:385-416: the next `batchsize` cases as column-slice views; short tails are skipped."""
        skip = False
        if self._pos == self.datasize:
            self._pos = 0
        if self._pos == 0:
            if self.empty or self._maxpos < self.parent._maxpos:
                self.LoadData()
                self.empty = False
            if self.randomize and self._maxpos == self.parent._maxpos:
                self.ShuffleData()
        start = self._pos
        end = self._pos + batchsize
        if end > self.datasize:
            end = self.datasize
            skip = not get_last_piece
        self._pos = end
        if skip:
            return self.Get(batchsize, get_last_piece=get_last_piece)
        batch = [d.slice(start, end) for d in self.data]
        for i in range(self.num_data):
            if self.add_noise[i]:
                batch[i].sample_gaussian(mult=self.sigma)
        return batch
