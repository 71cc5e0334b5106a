"""CPU oracle with the `cm` module surface of the reference's eigenmat backend.

TEST INFRASTRUCTURE ONLY.  This module is the checker for the CUDA library and the
timed CPU baseline; the product never imports it.  It mirrors
eigenmat/eigenmat.py (class EigenMatrix, alias CUDAMatrix at eigenmat.py:1338, module
functions dot/sigmoid/exp/sum/...), backed by oracle/eigenmat_port.c for the loops
whose order or arithmetic matters and by numpy float32 (OpenBLAS sgemm for `dot`,
like Eigen a float32 GEMM) for the rest.  Arrays are float32 in Fortran order, the
layout eigenmat wraps without copying (eigenmat/eigenmat.py:199-203).

Random numbers come from the Philox4x32-10 stream shared with the CUDA library
(`philox_uniform` in eigenmat_port.c): each sampling call consumes one call counter.
Parity unpinned for the sampling ops: the reference has no test for them and its own
generator (eigenmat/ziggurat.cc r4_uni) is degenerate on LP64.
"""
import ctypes as ct
import os
import subprocess

# libgomp's idle threads would otherwise spin and starve the BLAS threads between loops
os.environ.setdefault("OMP_WAIT_POLICY", "passive")

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))


def build(force=False):
    """Compile eigenmat_port.c (and the reference's ziggurat.cc when it is mounted)."""
    so = os.path.join(_HERE, "liboracle.so")
    src = os.path.join(_HERE, "eigenmat_port.c")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        # the reference project, when present, sits next to this repository (or where DEEPNET_REFERENCE says)
        ref = os.environ.get("DEEPNET_REFERENCE", os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference"))
        subprocess.check_call(["make", "-s", "-C", _HERE, "REF=" + (ref if os.path.isdir(ref) else "")])
    return so


_lib = ct.CDLL(build())


class _Mat(ct.Structure):
    _fields_ = [("data", ct.POINTER(ct.c_float)), ("size", ct.c_int * 2),
                ("is_trans", ct.c_int), ("owns_data", ct.c_int)]


_lib.euclid_norm.restype = ct.c_float
_lib.sum_all.restype = ct.c_float
_lib.vdot.restype = ct.c_float
_lib.philox_uniform.argtypes = [ct.c_uint64, ct.c_uint64, ct.c_int, ct.c_void_p]
_lib.philox_normal.argtypes = [ct.c_uint64, ct.c_uint64, ct.c_int, ct.c_void_p]


class EigenMatException(Exception):
    pass


def _check(err):
    if err:
        raise EigenMatException("oracle error code %d" % err)


class _Rng(object):
    seed = 0
    calls = 0
    col0 = 0      # first global column of this rank's minibatch shard

    @classmethod
    def next_call(cls):
        c = cls.calls
        cls.calls += 1
        return c


def philox4x32_10(ctr, key):
    c = (ct.c_uint32 * 4)(*ctr)
    k = (ct.c_uint32 * 2)(*key)
    o = (ct.c_uint32 * 4)()
    _lib.philox4x32_10(c, k, o)
    return [int(x) for x in o]


class EigenMatrix(object):
    """Column-major float32 matrix; same methods as cudamat.CUDAMatrix (cudamat/cudamat.py:126)."""

    def __init__(self, array, copy=True, _trans=False):
        a = np.asarray(array)
        if a.ndim == 1:
            a = a.reshape(-1, 1)
        if copy or a.dtype != np.float32 or not a.flags.f_contiguous:
            a = np.array(a, dtype=np.float32, order="F")
        self.numpy_array = a
        self.is_trans = _trans
        self._refresh()

    def _refresh(self):
        a = self.numpy_array
        self.mat = _Mat()
        self.mat.data = a.ctypes.data_as(ct.POINTER(ct.c_float))
        self.mat.size[0], self.mat.size[1] = a.shape
        self.mat.is_trans = int(self.is_trans)
        self.p_mat = ct.pointer(self.mat)

    # -- structure ---------------------------------------------------------
    @property
    def shape(self):
        s = self.numpy_array.shape
        return (s[1], s[0]) if self.is_trans else s

    @property
    def T(self):
        return EigenMatrix(self.numpy_array, copy=False, _trans=not self.is_trans)

    def asarray(self):
        return self.numpy_array.T if self.is_trans else self.numpy_array

    def copy_to_host(self):
        pass

    def free_device_memory(self):
        pass

    def slice(self, first_col, last_col):
        return EigenMatrix(self.numpy_array[:, int(first_col):int(last_col)], copy=False)

    def reshape(self, shape):
        self.numpy_array = self.numpy_array.reshape(shape, order="F")
        self._refresh()
        return self

    def overwrite(self, array):
        self.numpy_array[...] = np.asarray(array, dtype=np.float32).reshape(self.numpy_array.shape)

    def assign(self, val):
        if isinstance(val, EigenMatrix):
            if val.numpy_array.shape != self.numpy_array.shape:
                raise EigenMatException("incompatible dimensions")
            self.numpy_array[...] = val.numpy_array
        else:
            self.numpy_array[...] = np.float32(val)
        return self

    # -- random ------------------------------------------------------------
    @staticmethod
    def init_random(seed=0, col0=0):
        _Rng.seed, _Rng.calls, _Rng.col0 = int(seed), 0, int(col0)

    def _uniforms(self):
        u = EigenMatrix(np.empty(self.numpy_array.shape, np.float32, order="F"), copy=False)
        _check(_lib.philox_uniform(_Rng.seed, _Rng.next_call(), _Rng.col0, ct.cast(u.p_mat, ct.c_void_p)))
        return u

    def fill_with_rand(self):
        _check(_lib.philox_uniform(_Rng.seed, _Rng.next_call(), _Rng.col0, ct.cast(self.p_mat, ct.c_void_p)))
        return self

    def fill_with_randn(self):
        _check(_lib.philox_normal(_Rng.seed, _Rng.next_call(), _Rng.col0, ct.cast(self.p_mat, ct.c_void_p)))
        return self

    def sample_bernoulli(self, target=None, uniforms=None):
        target = target or self
        u = uniforms if uniforms is not None else self._uniforms()
        _check(_lib.sample_bernoulli_u(self.p_mat, u.p_mat, target.p_mat))
        return target

    def sample_gaussian(self, target=None, mult=1.0):
        target = target or self
        z = EigenMatrix(np.empty(self.numpy_array.shape, np.float32, order="F"), copy=False).fill_with_randn()
        _check(_lib.sample_gaussian_z(self.p_mat, z.p_mat, target.p_mat, ct.c_float(mult)))
        return target

    def perturb_prob_for_softmax_sampling(self, target=None, uniforms=None):
        target = target or self
        u = uniforms if uniforms is not None else self._uniforms()
        _check(_lib.perturb_prob_u(self.p_mat, u.p_mat, target.p_mat))
        return target

    def perturb_energy_for_softmax_sampling(self, target=None, uniforms=None):
        target = target or self
        u = uniforms if uniforms is not None else self._uniforms()
        _check(_lib.perturb_energy_u(self.p_mat, u.p_mat, target.p_mat))
        return target

    # -- broadcasts --------------------------------------------------------
    def add_col_vec(self, vec, target=None):
        target = target or self
        _check(_lib.add_col_vec(self.p_mat, vec.p_mat, target.p_mat))
        return target

    def add_col_mult(self, vec, mult, target=None):
        target = target or self
        _check(_lib.add_col_mult(self.p_mat, vec.p_mat, target.p_mat, ct.c_float(mult)))
        return target

    def add_row_vec(self, vec, target=None):
        target = target or self
        _check(_lib.add_row_vec(self.p_mat, vec.p_mat, target.p_mat))
        return target

    def add_row_mult(self, vec, mult, target=None):
        target = target or self
        _check(_lib.add_row_mult(self.p_mat, vec.p_mat, target.p_mat, ct.c_float(mult)))
        return target

    def mult_by_col(self, vec, target=None):
        target = target or self
        _check(_lib.mult_by_col_vec(self.p_mat, vec.p_mat, target.p_mat))
        return target

    def mult_by_row(self, vec, target=None):
        target = target or self
        _check(_lib.mult_by_row_vec(self.p_mat, vec.p_mat, target.p_mat))
        return target

    def div_by_col(self, vec, target=None):
        target = target or self
        _check(_lib.div_by_col_vec(self.p_mat, vec.p_mat, target.p_mat))
        return target

    def div_by_row(self, vec, target=None):
        target = target or self
        _check(_lib.div_by_row_vec(self.p_mat, vec.p_mat, target.p_mat))
        return target

    # -- reductions --------------------------------------------------------
    def sum(self, axis=None, target=None):
        if axis is None:
            return float(_lib.sum_all(self.p_mat))
        return sum(self, axis, target)

    def add_sums(self, mat, axis, mult=1.0):
        _check(_lib.add_sum_by_axis(mat.p_mat, self.p_mat, int(axis), ct.c_float(mult), ct.c_float(1.0)))
        return self

    def max(self, axis, target=None):
        h, w = self.numpy_array.shape
        if target is None:
            target = empty((1, w) if axis == 0 else (h, 1))
        _check(_lib.max_by_axis(self.p_mat, target.p_mat, int(axis)))
        return target

    def argmax(self, axis, target=None):
        h, w = self.numpy_array.shape
        if target is None:
            target = empty((1, w) if axis == 0 else (h, 1))
        _check(_lib.argmax_by_axis(self.p_mat, target.p_mat, int(axis)))
        return target

    def choose_max(self, axis, target=None):
        target = target or self
        _check(_lib.choose_max_by_axis(self.p_mat, target.p_mat, int(axis)))
        return target

    def choose_max_and_accumulate(self, acc):
        _check(_lib.choose_max_and_accumulate(self.p_mat, acc.p_mat))
        return acc

    def euclid_norm(self):
        return float(_lib.euclid_norm(self.p_mat))

    def norm_limit(self, norm, axis, target=None):
        """Columns whose Euclidean norm exceeds `norm` are scaled back to it.  eigenmat leaves this
        unimplemented (eigenmat/eigenmat.cc:761-767 returns an error), so the cudamat kernel's
        meaning is restated (cudamat/cudamat_kernels.cu:1068-1088): float32 sum of squares per
        column, factor 1 when the norm is below the limit, else norm / length."""
        if axis != 0:
            raise EigenMatException("norm_limit is defined along axis 0 only (cudamat/cudamat.cu:1310)")
        target = target or self
        a = self.numpy_array
        length = np.sqrt((a.astype(np.float32) ** 2).sum(axis=0, dtype=np.float32)).astype(np.float32)
        f = np.where(length < np.float32(norm), np.float32(1), np.float32(norm) / length).astype(np.float32)
        target.numpy_array[...] = a * f[None, :]
        return target

    def transpose(self, target=None):
        """eigenmat/eigenmat.py:307-318 (copy_transpose): target = self' as a new dense matrix."""
        h, w = self.numpy_array.shape
        if target is None:
            target = empty((w, h))
        target.numpy_array[...] = self.numpy_array.T
        return target

    def apply_softmax(self, target=None):
        target = target or self
        _check(_lib.apply_softmax(self.p_mat, target.p_mat))
        return target

    # -- elementwise -------------------------------------------------------
    def _binary(self, val, target, op):
        target = target or self
        if isinstance(val, EigenMatrix):
            if val.numpy_array.shape != self.numpy_array.shape:
                raise EigenMatException("incompatible dimensions")
            rhs = val.numpy_array
        else:
            rhs = np.float32(val)
        with np.errstate(all="ignore"):
            target.numpy_array[...] = op(self.numpy_array, rhs)
        return target

    def add(self, val, target=None):
        return self._binary(val, target, np.add)

    def subtract(self, val, target=None):
        return self._binary(val, target, np.subtract)

    def mult(self, val, target=None):
        return self._binary(val, target, np.multiply)

    def divide(self, val, target=None):
        return self._binary(val, target, np.divide)

    def greater_than(self, val, target=None):
        return self._binary(val, target, lambda a, b: (a > b).astype(np.float32))

    def less_than(self, val, target=None):
        return self._binary(val, target, lambda a, b: (a < b).astype(np.float32))

    def add_mult(self, mat2, mult=1.0, alpha=None):
        _check(_lib.add_mult(self.p_mat, mat2.p_mat, ct.c_float(mult if alpha is None else alpha)))
        return self

    def subtract_mult(self, mat2, mult=1.0):
        return self.add_mult(mat2, -mult)

    def add_mult_sign(self, mat2, mult=1.0):
        _check(_lib.add_mult_sign(self.p_mat, mat2.p_mat, ct.c_float(mult)))
        return self

    def dot(self, mat2, mult=1.0, target=None):
        return dot(self, mat2, mult, target)

    def add_dot(self, m1, m2, mult=1.0):
        _dot_into(m1, m2, self, 1.0, mult)
        return self

    def subtract_dot(self, m1, m2):
        return self.add_dot(m1, m2, -1.0)

    def select_columns(self, indices, target):
        _check(_lib.selectCols(self.p_mat, target.p_mat, indices.p_mat))
        return target

    def swap_columns(self, indices1, indices2, target):
        _check(_lib.swapCols(self.p_mat, target.p_mat, indices1.p_mat, indices2.p_mat))
        return target

    def momentum_update(self, delta, grad, suff, inv_batch, momentum, eps, l2=0.0, l1=0.0):
        """deepnet/dbm.py:242,254 + deepnet/parameter.py:80-106 in one pass (self is the parameter)."""
        _check(_lib.momentum_update(self.p_mat, delta.p_mat, grad.p_mat, suff.p_mat, ct.c_float(inv_batch),
                                    ct.c_float(momentum), ct.c_float(eps), ct.c_float(l2), ct.c_float(l1)))
        return self


CUDAMatrix = EigenMatrix


def empty(shape):
    return EigenMatrix(np.zeros(shape, dtype=np.float32, order="F"), copy=False)


def sum(mat, axis, target=None):
    h, w = mat.numpy_array.shape
    phys_axis = 1 - axis if mat.is_trans else axis
    if target is None:
        target = empty((1, w) if phys_axis == 0 else (h, 1))
    _check(_lib.add_sum_by_axis(mat.p_mat, target.p_mat, int(axis), ct.c_float(1.0), ct.c_float(0.0)))
    return target


# Products this small go through the plain-C triple loop (one running float sum per
# output); larger ones through OpenBLAS sgemm, like Eigen a blocked float32 GEMM.
_C_DOT_LIMIT = 1 << 18


def _dot_into(m1, m2, target, beta, alpha):
    a, b = m1.asarray(), m2.asarray()
    if a.shape[1] != b.shape[0] or target.numpy_array.shape != (a.shape[0], b.shape[1]):
        raise EigenMatException("incompatible dimensions")
    if a.shape[0] * a.shape[1] * b.shape[1] <= _C_DOT_LIMIT:
        _check(_lib.dot(m1.p_mat, m2.p_mat, target.p_mat, ct.c_float(beta), ct.c_float(alpha)))
        return
    # target is Fortran-ordered: form (a b)' = b' a' straight into its C-ordered transpose view
    tt = target.numpy_array.T
    if beta == 0:
        np.matmul(b.T, a.T, out=tt)
        if alpha != 1:
            tt *= np.float32(alpha)
    else:
        prod = np.matmul(b.T, a.T)
        if alpha != 1:
            prod *= np.float32(alpha)
        if beta != 1:
            tt *= np.float32(beta)
        tt += prod


def dot(m1, m2, mult=1.0, target=None):
    if target is None:
        target = empty((m1.shape[0], m2.shape[1]))
    _dot_into(m1, m2, target, 0.0, mult)
    return target


def vdot(m1, m2):
    err = ct.c_int(0)
    r = _lib.vdot(m1.p_mat, m2.p_mat, ct.byref(err))
    _check(err.value)
    return float(r)


def sigmoid(mat, target=None):
    target = target or mat
    _check(_lib.apply_sigmoid(mat.p_mat, target.p_mat))
    return target


def exp(mat, target=None):
    target = target or mat
    _check(_lib.apply_exp(mat.p_mat, target.p_mat))
    return target


def log_1_plus_exp(mat, target=None):
    target = target or mat
    _check(_lib.apply_log_1_plus_exp(mat.p_mat, target.p_mat))
    return target


def cuda_set_device(dev_id):
    pass


def cublas_init():
    pass


init = cublas_init


def cublas_shutdown():
    pass


shutdown = cublas_shutdown


def cuda_sync_threads():
    pass


# -- the reference's own CPU generator, compiled in place from eigenmat/ziggurat.cc ----
def reference_r4_uni(seed, n):
    """Draw n uniforms from the reference's r4_uni (eigenmat/ziggurat.cc:344-358).

    Exists to document that generator's behaviour on LP64 (its state is an
    `unsigned long`); it is not used to compare training curves.
    """
    so = os.path.join(_HERE, "_ref", "libziggurat_ref.so")
    lib = ct.CDLL(so)
    f = lib._Z6r4_uniPm
    f.restype = ct.c_float
    state = ct.c_ulong(seed)
    return np.array([f(ct.byref(state)) for _ in range(n)], dtype=np.float32)


# ---- device-resident data feed: CPU twin of feed_pack / feed_gather / feed_permutation ----------
# (the reference's GPUCache, deepnet/datahandler.py:259-416, shuffles with a host-drawn permutation;
# the feed evaluates a keyed Feistel bijection instead, restated here in numpy uint32 arithmetic)
def _feed_mix(r, k):
    h = (r * np.uint32(0x9E3779B1) + k).astype(np.uint32)
    h ^= h >> np.uint32(15)
    h = (h * np.uint32(0x85EBCA77)).astype(np.uint32)
    h ^= h >> np.uint32(13)
    h = (h * np.uint32(0xC2B2AE3D)).astype(np.uint32)
    h ^= h >> np.uint32(16)
    return h


def feed_permutation(n, key, rounds=6):
    bits = 2
    while bits < 32 and (1 << bits) < n:
        bits += 1
    a = bits >> 1
    b = bits - a
    mask_a, mask_b = np.uint32((1 << a) - 1), np.uint32((1 << b) - 1)
    klo, khi = np.uint32(key[0] & 0xffffffff), np.uint32(key[1] & 0xffffffff)
    x = np.arange(n, dtype=np.uint32)
    todo = np.ones(n, bool)
    with np.errstate(over="ignore"):
        while todo.any():
            L, R = x[todo] >> np.uint32(a), x[todo] & mask_a
            for rnd in range(rounds):
                k = np.uint32(klo * np.uint32(0x9E3779B9) + khi * np.uint32(0x85EBCA6B) + np.uint32(rnd) * np.uint32(0xC2B2AE35))
                if rnd % 2 == 0:
                    L = L ^ (_feed_mix(R, k) & mask_b)
                else:
                    R = R ^ (_feed_mix(L, k) & mask_a)
            x[todo] = (L << np.uint32(a)) | R
            todo = x >= n
    return x.astype(np.int64)


def feed_pack(array):
    """Keeps the 0/1 data as they are (the packing is a storage detail of the device library)."""
    a = np.asarray(array, np.float32)
    if not np.isin(a, (0, 1)).all():
        raise ValueError("only 0/1 data can be stored one bit per value")
    return EigenMatrix(a)


def feed_gather(src, packed, dims, key, shuffle, start, out, mean=None, std=None, out_aux=None, aux_mode=0, aux_exp=0):
    n, count = src.numpy_array.shape[1], out.numpy_array.shape[1]
    cols = np.arange(start, start + count)
    if shuffle:
        cols = feed_permutation(n, key)[cols]
    x = src.numpy_array[:, cols].astype(np.float32)
    if mean is not None:
        x = ((x + (-mean.numpy_array.reshape(-1, 1))) / std.numpy_array.reshape(-1, 1)).astype(np.float32)
    out.numpy_array[...] = x
    return out
