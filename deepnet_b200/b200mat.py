"""ctypes wrapper over libb200mat.so with the `cm` module surface of cudamat.

Mirrors cudamat/cudamat.py: class CUDAMatrix (:126-1531), empty (:1533), sum (:1546),
dot (:1579), vdot (:1596), sigmoid/exp/log_1_plus_exp (:1607-1700), cuda_set_device,
cublas_init/shutdown, cuda_sync_threads, so deepnet's dbm.py / layer.py / edge.py /
parameter.py run on it unchanged.  Matrices are float32, column-major; `.T` and
`slice` are non-owning views.  Extra entry points (fused_gemm, momentum_update,
split_tf32, dp_*) have no counterpart in the reference.

There is no CPU fallback: importing works without a GPU (so the symbols can be
inspected), but the first operation fails loudly if the library or a device is missing.
"""
import ctypes as ct
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libb200mat.so")

MAX_PASS = 8


def _load():
    alt = os.environ.get("B200MAT_LIBRARY")       # another build of the same library (instrumented, say)
    if alt:
        return ct.CDLL(alt)
    if not os.path.exists(_LIB_PATH):
        raise ImportError(
            "libb200mat.so is missing: build it with `python -m deepnet_b200.build` "
            "(nvcc, sm_100a); there is no CPU fallback")
    return ct.CDLL(_LIB_PATH)


_lib = _load()


class cudamat(ct.Structure):
    """struct cudamat of cudamat/cudamat.cuh:21-29."""
    _fields_ = [("data_host", ct.POINTER(ct.c_float)), ("data_device", ct.POINTER(ct.c_float)),
                ("on_device", ct.c_int), ("on_host", ct.c_int), ("size", ct.c_int * 2),
                ("is_trans", ct.c_int), ("owns_data", ct.c_int)]


class rnd_struct(ct.Structure):
    _fields_ = [("seed", ct.c_ulonglong), ("calls", ct.c_ulonglong)]


class _Pass(ct.Structure):
    _fields_ = [("a", ct.POINTER(cudamat)), ("b", ct.POINTER(cudamat)), ("negate", ct.c_int),
                ("a_part", ct.c_int), ("b_part", ct.c_int),
                ("a_aux", ct.POINTER(cudamat)), ("b_aux", ct.POINTER(cudamat)),
                ("a_row0", ct.c_int), ("a_rows", ct.c_int), ("b_row0", ct.c_int), ("b_rows", ct.c_int)]


class _FusedGemm(ct.Structure):
    _fields_ = [("npass", ct.c_int), ("passes", _Pass * MAX_PASS), ("alpha", ct.c_float), ("beta", ct.c_float),
                ("bias", ct.POINTER(cudamat)), ("col_scale", ct.POINTER(cudamat)), ("activation", ct.c_int),
                ("out", ct.POINTER(cudamat)), ("out_aux", ct.POINTER(cudamat)), ("sample", ct.POINTER(cudamat)),
                ("sample_aux", ct.POINTER(cudamat)), ("scale_exp", ct.POINTER(cudamat)),
                ("scale_exp_const", ct.c_int), ("aux_f16", ct.c_int), ("aux_exp", ct.c_int)]


_lib.get_last_cuda_error.restype = ct.c_char_p
_lib.euclid_norm.restype = ct.c_float
_lib.vdot.restype = ct.c_float
_lib.sum_all.restype = ct.c_float
_lib.b200_host_alloc.restype = ct.c_void_p
_lib.b200_host_alloc.argtypes = [ct.c_size_t]
_lib.b200_host_free.argtypes = [ct.c_void_p]
_lib.b200_get_stream.restype = ct.c_void_p
_lib.b200_set_stream.argtypes = [ct.c_void_p]
_lib.copy_from_host_ptr.argtypes = [ct.POINTER(cudamat), ct.c_void_p, ct.c_size_t]
_lib.b200_prefetch.argtypes = [ct.POINTER(cudamat), ct.c_void_p, ct.c_size_t]
_lib.b200_event_create.restype = ct.c_void_p
_lib.b200_event_record.argtypes = [ct.c_void_p]
_lib.b200_event_elapsed_ms.argtypes = [ct.c_void_p, ct.c_void_p]
_lib.b200_event_elapsed_ms.restype = ct.c_float
_lib.b200_event_destroy.argtypes = [ct.c_void_p]
_lib.b200_event_destroy.restype = None
_lib.init_from_array.restype = None
_lib.set_transpose.restype = None
_lib.cuda_sync_threads.restype = None


class CUDAMatException(Exception):
    pass


_ERRORS = {
    -1: "Incompatible matrix dimensions.",
    -2: "CUBLAS error.",
    -4: "Operation not supported on views.",
    -5: "Operation not supported on transposed matrices.",
    -6: "",
    -7: "Incompatible transposedness.",
    -8: "Matrix is not in device memory.",
    -9: "Operation not supported.",
    -11: "A device-side wait ran out of time.",
}


def generate_exception(err_code):
    """Error-code mapping of cudamat/cudamat.py:101-123 (plus -10 NCCL, -11 device timeout)."""
    text = _lib.get_last_cuda_error().decode("utf-8", "replace")     # reading it clears it
    if err_code in (-3, -10):
        return CUDAMatException(("CUDA error: " if err_code == -3 else "NCCL error: ") + text)
    msg = _ERRORS.get(err_code, "error code %d" % err_code)
    if err_code == -9 and text and text != "no error":
        msg += " " + text                                            # why the library refused
    return CUDAMatException(msg)


def _check(err_code):
    if err_code:
        raise generate_exception(err_code)


_device_checked = False


def _require_device():
    global _device_checked
    if not _device_checked:
        if _lib.b200_device_count() <= 0:
            raise CUDAMatException("no CUDA device is visible; b200mat has no CPU fallback")
        _check(_lib.cublas_init())
        _device_checked = True
        cublas_init()


class CUDAMatrix(object):
    """A float32 column-major matrix in GPU memory (cudamat/cudamat.py:126)."""

    rnd_state = rnd_struct()
    rnd_state_p = ct.pointer(rnd_state)
    ones = None

    def __init__(self, array, copy_to_device=True, copy_on_host=True):
        _require_device()
        array = np.asarray(array)
        if array.ndim == 1:
            array = array.reshape(-1, 1)
        # cudamat/cudamat.py:183-195 keeps a Fortran-order float32 host copy
        self.numpy_array = np.array(array, dtype=np.float32, order="F") if copy_on_host else reformat(array)
        self.mat = cudamat()
        self.p_mat = ct.pointer(self.mat)
        _lib.init_from_array(self.p_mat, self.numpy_array.ctypes.data_as(ct.POINTER(ct.c_float)),
                             ct.c_int(self.numpy_array.shape[0]), ct.c_int(self.numpy_array.shape[1]))
        if copy_to_device:
            _check(_lib.copy_to_device(self.p_mat))

    @classmethod
    def _from_mat(cls, mat):
        obj = cls.__new__(cls)
        obj.mat = mat
        obj.p_mat = ct.pointer(mat)
        obj.numpy_array = None
        return obj

    @property
    def T(self):
        """cudamat/cudamat.py:139-146: a view of the same storage with is_trans = 1."""
        t = TransposedCUDAMatrix(self.mat)
        t._parent = self  # keep the owner (and its device memory) alive
        return t

    def __del__(self):
        try:
            if self.mat.owns_data and self.mat.on_device:
                _lib.free_device_memory(self.p_mat)
        except Exception:
            pass

    # -- random ------------------------------------------------------------
    @staticmethod
    def init_random(seed=0):
        """cudamat/cudamat.py:209-224; here: Philox key = seed, call counter = 0."""
        _check(_lib.init_random(CUDAMatrix.rnd_state_p, ct.c_int(seed), None))

    # -- structure ---------------------------------------------------------
    @property
    def shape(self):
        return (self.mat.size[0], self.mat.size[1])

    def set_shape(self, shape):
        _check(_lib.set_shape(self.p_mat, ct.c_uint(shape[0]), ct.c_uint(shape[1])))
        return self

    def reshape(self, shape):
        _check(_lib.reshape(self.p_mat, ct.c_uint(shape[0]), ct.c_uint(shape[1])))
        if self.numpy_array is not None:
            self.numpy_array = self.numpy_array.reshape(shape, order="F")
            self.mat.data_host = self.numpy_array.ctypes.data_as(ct.POINTER(ct.c_float))
        return self

    def set_trans(self, is_trans):
        _lib.set_transpose(self.p_mat, ct.c_int(1 if is_trans else 0))

    def asarray(self):
        self.copy_to_host()
        return self.numpy_array

    def copy_to_device(self):
        _check(_lib.copy_to_device(self.p_mat))

    def copy_to_host(self):
        if not self.mat.on_host or self.numpy_array is None or tuple(self.numpy_array.shape) != tuple(self.shape):
            self.numpy_array = np.empty(self.shape, dtype=np.float32, order="F")
            self.mat.data_host = self.numpy_array.ctypes.data_as(ct.POINTER(ct.c_float))
            self.mat.on_host = 1
        _check(_lib.copy_to_host(self.p_mat))

    def overwrite(self, array):
        """cudamat/cudamat.py:152-168: replace the contents from a host array of the same shape."""
        array = np.asarray(array)
        if array.ndim == 1:
            array = array.reshape(-1, 1)
        if tuple(array.shape) != tuple(self.shape):
            raise CUDAMatException("Incompatible matrix dimensions.")
        self.numpy_array = np.array(array, dtype=np.float32, order="F")
        self.mat.data_host = self.numpy_array.ctypes.data_as(ct.POINTER(ct.c_float))
        self.mat.on_host = 1
        _check(_lib.copy_to_device(self.p_mat))

    def overwrite_from_pinned(self, ptr, nbytes):
        """Asynchronous host-to-device copy from a pinned buffer (see host_alloc)."""
        _check(_lib.copy_from_host_ptr(self.p_mat, ct.c_void_p(ptr), ct.c_size_t(nbytes)))

    def prefetch_from_pinned(self, ptr, nbytes):
        """Host-to-device copy on the copy stream; pair with prefetch_wait() / prefetch_fence()."""
        _check(_lib.b200_prefetch(self.p_mat, ct.c_void_p(ptr), ct.c_size_t(nbytes)))

    def assign(self, val):
        if isinstance(val, CUDAMatrix):
            _check(_lib.copy_on_device(val.p_mat, self.p_mat))
        elif isinstance(val, (int, float, np.floating, np.integer)):
            _check(_lib.assign_scalar(self.p_mat, ct.c_float(val)))
        else:
            raise ValueError("Assigned value must be of type CUDAMatrix, int, or float.")
        return self

    def free_device_memory(self):
        _check(_lib.free_device_memory(self.p_mat))

    def slice(self, first_col, last_col):
        mat = cudamat()
        if self.mat.size[0] == 1 or self.mat.size[1] == 1:
            _check(_lib.get_vector_slice(self.p_mat, ct.pointer(mat), ct.c_uint(int(first_col)), ct.c_uint(int(last_col))))
        else:
            _check(_lib.get_slice(self.p_mat, ct.pointer(mat), ct.c_uint(int(first_col)), ct.c_uint(int(last_col))))
        new = CUDAMatrix._from_mat(mat)
        new._parent = self  # keep the owner alive
        return new

    get_col_slice = slice

    # -- random ops --------------------------------------------------------
    def fill_with_rand(self):
        _check(_lib.fill_with_rand(CUDAMatrix.rnd_state_p, self.p_mat))
        return self

    def fill_with_randn(self):
        _check(_lib.fill_with_randn(CUDAMatrix.rnd_state_p, self.p_mat))
        return self

    def sample_bernoulli(self, target=None):
        target = target or self
        _check(_lib.sample_bernoulli(CUDAMatrix.rnd_state_p, self.p_mat, target.p_mat))
        return target

    def sample_bernoulli_tanh(self, target=None):
        target = target or self
        _check(_lib.sample_bernoulli_tanh(CUDAMatrix.rnd_state_p, self.p_mat, target.p_mat))
        return target

    def sample_gaussian(self, target=None, mult=1.0):
        target = target or self
        _check(_lib.sample_gaussian(CUDAMatrix.rnd_state_p, self.p_mat, target.p_mat, ct.c_float(mult)))
        return target

    def perturb_energy_for_softmax_sampling(self, target=None):
        target = target or self
        _check(_lib.perturb_energy(CUDAMatrix.rnd_state_p, self.p_mat, target.p_mat))
        return target

    def perturb_prob_for_softmax_sampling(self, target=None):
        target = target or self
        _check(_lib.perturb_prob(CUDAMatrix.rnd_state_p, self.p_mat, target.p_mat))
        return target

    def dropout(self, dropprob, val=0.0):
        _check(_lib.dropout(CUDAMatrix.rnd_state_p, self.p_mat, ct.c_float(dropprob), ct.c_float(val)))
        return self

    # -- broadcasts --------------------------------------------------------
    def _vec_op(self, fn, vec, target, *extra):
        target = target or self
        _check(fn(self.p_mat, vec.p_mat, target.p_mat, *extra))
        return target

    def add_col_vec(self, vec, target=None):
        return self._vec_op(_lib.add_col_vec, vec, target)

    def add_col_mult(self, vec, mult, target=None):
        return self._vec_op(_lib.add_col_mult, vec, target, ct.c_float(mult))

    def add_row_vec(self, vec, target=None):
        return self._vec_op(_lib.add_row_vec, vec, target)

    def add_row_mult(self, vec, mult, target=None):
        return self._vec_op(_lib.add_row_mult, vec, target, ct.c_float(mult))

    def mult_by_col(self, vec, target=None):
        return self._vec_op(_lib.mult_by_col_vec, vec, target)

    def mult_by_row(self, vec, target=None):
        return self._vec_op(_lib.mult_by_row_vec, vec, target)

    def div_by_col(self, vec, target=None):
        return self._vec_op(_lib.div_by_col_vec, vec, target)

    def div_by_row(self, vec, target=None):
        return self._vec_op(_lib.div_by_row_vec, vec, target)

    # -- reductions --------------------------------------------------------
    def sum(self, axis=None, target=None):
        if axis is None:
            err = ct.c_int(0)
            r = _lib.sum_all(self.p_mat, ct.byref(err))
            _check(err.value)
            return r
        return sum(self, axis, target)

    def add_sums(self, mat, axis, mult=1.0):
        _check(_lib.add_sum_by_axis(mat.p_mat, self.p_mat, ct.c_int(axis), ct.c_float(mult)))
        return self

    def add_sums_noalloc(self, mat, axis, mult=1.0):
        """add_sums for hosts that may not allocate device memory (their own pool owns the GPU, or
        they cannot afford an allocation's device-wide synchronisation): same result, but the
        partial sums go to a fixed 128 KiB array inside the library.  Raises for matrices whose
        partial sums do not fit; calls must not overlap on the GPU."""
        _check(_lib.add_sum_by_axis_noalloc(mat.p_mat, self.p_mat, ct.c_int(axis), ct.c_float(mult)))
        return self

    def max(self, axis, target=None):
        m, n = self.shape
        if target is None:
            target = empty((1, n)) if axis == 0 else empty((m, 1))
        _check(_lib.max_by_axis(self.p_mat, target.p_mat, ct.c_int(axis)))
        return target

    def argmax(self, axis, target=None):
        m, n = self.shape
        if target is None:
            target = empty((1, n)) if axis == 0 else empty((m, 1))
        _check(_lib.argmax_by_axis(self.p_mat, target.p_mat, ct.c_int(axis)))
        return target

    def choose_max(self, axis, target=None):
        target = target or self
        _check(_lib.choose_max_by_axis(self.p_mat, target.p_mat, ct.c_int(axis)))
        return target

    def choose_max_and_accumulate(self, acc):
        _check(_lib.choose_max_and_accumulate(self.p_mat, acc.p_mat))
        return acc

    def euclid_norm(self):
        err = ct.c_int(0)
        r = _lib.euclid_norm(self.p_mat, ct.byref(err))
        _check(err.value)
        return r

    def apply_softmax(self, target=None):
        target = target or self
        _check(_lib.softmax(self.p_mat, target.p_mat))
        return target

    def norm_limit(self, norm, axis, target=None):
        """cudamat/cudamat.py:1000-1016: columns longer than `norm` are scaled back to it (axis 0 only)."""
        target = target or self
        _check(_lib.normlimit_by_axis(self.p_mat, target.p_mat, ct.c_int(axis), ct.c_float(norm)))
        return target

    def transpose(self, target=None):
        """cudamat/cudamat.py:422-433: target = self' as a dense matrix (a copy, not a view)."""
        if target is None:
            target = empty((self.shape[1], self.shape[0]))
        _check(_lib.copy_transpose(self.p_mat, target.p_mat))
        return target

    # -- elementwise -------------------------------------------------------
    def _scalar_or_mat(self, val, target, fn_mat, fn_scalar):
        target = target or self
        if isinstance(val, CUDAMatrix):
            _check(fn_mat(self.p_mat, val.p_mat, target.p_mat))
        elif isinstance(val, (int, float, np.floating, np.integer)):
            _check(fn_scalar(self.p_mat, ct.c_float(val), target.p_mat))
        else:
            raise ValueError("Value must be of type CUDAMatrix, int, or float.")
        return target

    def add(self, val, target=None):
        return self._scalar_or_mat(val, target, _lib.add_elementwise, _lib.add_scalar)

    def subtract(self, val, target=None):
        if isinstance(val, CUDAMatrix):
            return self._scalar_or_mat(val, target, _lib.subtract_elementwise, None)
        return self._scalar_or_mat(-val, target, None, _lib.add_scalar)

    def mult(self, val, target=None):
        return self._scalar_or_mat(val, target, _lib.mult_elementwise, _lib.mult_by_scalar)

    def divide(self, val, target=None):
        return self._scalar_or_mat(val, target, _lib.divide_elementwise, _lib.divide_by_scalar)

    def less_than(self, val, target=None):
        return self._scalar_or_mat(val, target, _lib.less_than, _lib.less_than_scalar)

    def less_than_eq(self, val, target=None):
        return self._scalar_or_mat(val, target, _lib.less_than_eq, _lib.less_than_eq_scalar)

    def greater_than(self, val, target=None):
        return self._scalar_or_mat(val, target, _lib.greater_than, _lib.greater_than_scalar)

    def greater_than_eq(self, val, target=None):
        return self._scalar_or_mat(val, target, _lib.greater_than_eq, _lib.greater_than_eq_scalar)

    def upper_bound(self, val, target=None):
        return self._scalar_or_mat(val, target, _lib.upper_bound, _lib.upper_bound_scalar)

    def lower_bound(self, val, target=None):
        return self._scalar_or_mat(val, target, _lib.lower_bound, _lib.lower_bound_scalar)

    def sign(self, target=None):
        target = target or self
        _check(_lib.sign(self.p_mat, target.p_mat))
        return target

    def apply_sigmoid(self, target=None):
        return sigmoid(self, target)

    def reciprocal(self, target=None):
        target = target or self
        _check(_lib.reciprocal(self.p_mat, target.p_mat))
        return target

    def apply_logistic_deriv(self, val, target=None):
        target = target or self
        _check(_lib.apply_logistic_deriv(self.p_mat, val.p_mat, target.p_mat))
        return target

    def add_mult(self, mat2, mult=1.0, alpha=None):
        """self += mult * mat2 (cudamat names the scalar `mult`, eigenmat `alpha`)."""
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
        _check(_lib.dot(m1.p_mat, m2.p_mat, self.p_mat, ct.c_float(1.0), ct.c_float(mult)))
        return self

    def subtract_dot(self, m1, m2):
        return self.add_dot(m1, m2, -1.0)

    def softmax_scaled(self, scale, target=None):
        """target[:, j] = scale[j] * softmax(self[:, j]) (deepnet/replicated_softmax_layer.py:12-21 fused)."""
        target = target or self
        _check(_lib.softmax_scaled(self.p_mat, scale.p_mat, target.p_mat))
        return target

    def softmax_sample(self, state, sample=None, bias=None):
        """state = softmax over each column of self (+ bias); sample = one categorical draw per column
        as a one-hot (deepnet/softmax_layer.py:11-16 in one kernel, one sampling call)."""
        _check(_lib.softmax_sample(CUDAMatrix.rnd_state_p, self.p_mat, bias.p_mat if bias is not None else None,
                                   state.p_mat, sample.p_mat if sample is not None else None))
        return state

    def sample_energy_softmax(self, target, ndraws):
        """target = counts over ndraws Gumbel-max draws per column from the softmax with energies self
        (deepnet/ais.py:16-30 in one kernel; consumes ndraws sampling calls)."""
        _check(_lib.sample_energy_softmax(CUDAMatrix.rnd_state_p, self.p_mat, target.p_mat, ct.c_int(int(ndraws))))
        return target

    def sample_multinomial(self, nn, target, max_draws=1000):
        """target[:, i] = counts of int(nn[i]) draws from self[:, i] (replicated_softmax_layer.py:43-60 fused)."""
        _check(_lib.sample_multinomial(CUDAMatrix.rnd_state_p, self.p_mat, nn.p_mat, target.p_mat, ct.c_int(max_draws)))
        return target

    def select_columns(self, indices, target):
        """cudamat/cudamat.py:1478-1493: target[:, c] = self[:, indices[c]] (indices: float32 row vector)."""
        _check(_lib.selectRows(self.p_mat, target.p_mat, indices.p_mat))
        return target

    def swap_columns(self, indices1, indices2, target):
        """cudamat/cudamat.py:1496-1512: columns indices1 of self and indices2 of target change places."""
        assert indices1.shape == indices2.shape
        _check(_lib.swapColumns(self.p_mat, target.p_mat, indices1.p_mat, indices2.p_mat))
        return target

    # -- fused entry points (no counterpart in the reference API) -------------
    def momentum_update(self, delta, grad, suff, inv_batch, momentum, eps, l2=0.0, l1=0.0, w_aux=None, w_scale=None):
        """deepnet/dbm.py:242,254 + deepnet/parameter.py:80-106 in one kernel; self is the parameter.
        w_aux (optional, from `empty_aux`) receives the bfloat16 parts of the updated parameter, or,
        with w_scale (the 1 x 4 device matrix of `f16_scale_state`), its scaled half-precision form."""
        _check(_lib.momentum_update(self.p_mat, delta.p_mat, grad.p_mat if grad is not None else None, suff.p_mat,
                                    w_aux.p_mat if w_aux is not None else None,
                                    w_scale.p_mat if w_scale is not None else None,
                                    ct.c_float(inv_batch), ct.c_float(momentum), ct.c_float(eps), ct.c_float(l2),
                                    ct.c_float(l1)))
        return self

    def split_bf16(self, aux):
        """Fills `aux` (from `empty_aux(self.shape)`) with the bfloat16 parts of self that the
        correction terms of a product read: plane 0 = bf16(self - tf32(self)), plane 1 =
        bf16(self).  Returns aux."""
        _check(_lib.split_bf16(self.p_mat, aux.p_mat))
        return aux

    def split_f16(self, aux, exp_dev=None, exp_const=0):
        """Fills `aux` with self in scaled half-precision form: with xs = self * 2^(exp_dev + exp_const)
        (exp_dev: 1 x 1 device matrix or None), plane 1 = fp16(xs), plane 0 = fp16(xs - plane 1).
        Returns aux."""
        _check(_lib.split_f16(self.p_mat, aux.p_mat, exp_dev.p_mat if exp_dev is not None else None,
                              ct.c_int(int(exp_const))))
        return aux

    def split_tf32(self, lo, hi=None):
        """lo = self - tf32(self); hi (optional) = self with the low 13 mantissa bits cleared."""
        _check(_lib.split_tf32(self.p_mat, hi.p_mat if hi is not None else None, lo.p_mat))
        return lo


class TransposedCUDAMatrix(CUDAMatrix):
    """cudamat/cudamat.py:139-146: same storage, is_trans flipped, never owns the data."""

    def __init__(self, mat):
        self.mat = cudamat()
        ct.memmove(ct.pointer(self.mat), ct.pointer(mat), ct.sizeof(self.mat))
        self.mat.is_trans = 0 if mat.is_trans else 1
        self.mat.owns_data = 0
        self.p_mat = ct.pointer(self.mat)
        self.numpy_array = None

    @property
    def shape(self):
        return (self.mat.size[1], self.mat.size[0]) if self.mat.is_trans else (self.mat.size[0], self.mat.size[1])

    def __del__(self):
        pass


class AuxMatrix(CUDAMatrix):
    """The bfloat16 parts of a rows x cols matrix kept in device memory (see `split_bf16`):
    storage of lda x cols floats, lda = rows rounded up to 8; column c holds lda bfloat16 of
    plane 0 (bf16(x - tf32(x))) and lda of plane 1 (bf16(x)), the first `rows` of each in use.
    Passed as `a_aux` / `b_aux` of a term, written as `out_aux` / `sample_aux` / `w_aux`."""

    def __init__(self, shape):
        _require_device()
        self.rows, self.cols = int(shape[0]), int(shape[1])
        self.mat = cudamat()
        _check(_lib.init_empty(ct.pointer(self.mat), ct.c_int((self.rows + 7) // 8 * 8), ct.c_int(self.cols)))
        self.p_mat = ct.pointer(self.mat)
        self.numpy_array = None

    def planes(self):
        """Host copy of the two planes as float32 arrays (rows x cols each)."""
        raw = np.array(self.asarray(), copy=True)                       # lda x cols floats
        words = np.ascontiguousarray(raw.T).view(np.uint16)             # cols x (2 lda) bfloat16
        lda = raw.shape[0]
        f = lambda w: (np.ascontiguousarray(w).astype(np.uint32) << 16).view(np.float32).T[:self.rows]
        return f(words[:, :lda]), f(words[:, lda:])


def empty_aux(shape):
    """Zero-filled aux matrix for a matrix of this shape."""
    return AuxMatrix(shape)


# What of an fp32 matrix a term of `fused_gemm` multiplies: x read as TF32, x - tf32(x) read as
# TF32, bfloat16(x - tf32(x)), bfloat16(x).  The kernel derives the parts from the matrix itself,
# or reads the two bfloat16 ones from the matrix's aux when one is given.
PART_X, PART_LO32, PART_LO16, PART_B16, PART_F16LO, PART_F16HI = 0, 1, 2, 3, 4, 5


class Part(object):
    """A part of a matrix (or of its transpose) as a `fused_gemm` operand; aux: its AuxMatrix."""

    def __init__(self, mat, part, aux=None):
        self.mat, self.part, self.aux, self.p_mat = mat, part, aux, mat.p_mat

    @property
    def T(self):
        return Part(self.mat.T, self.part, self.aux)


def lo32(x):
    return Part(x, PART_LO32)


def lo16(x, aux=None):
    return Part(x, PART_LO16, aux)


def b16(x, aux=None):
    return Part(x, PART_B16, aux)


def f16_passes(a, a_aux, b, b_aux, negate=0, exact_a=False, exact_b=False, a_rows=None, b_rows=None):
    """The terms of a . b over aux matrices in scaled half-precision form (`split_f16`): with
    x * 2^e = hi + lo,  a . b * 2^(ea + eb) ~= hi(a).lo(b) + lo(a).hi(b) + hi(a).hi(b), three
    half-precision products (no TF32 term, no fp32 operand read), below 2^-21 per term.  The
    caller passes the exponent sum to `fused_gemm` (scale_exp / scale_exp_const).  exact_a /
    exact_b: that operand is exact in fp16 (0/1 data and samples), its lo plane is not read."""
    win = dict(a_rows=a_rows, b_rows=b_rows) if (a_rows or b_rows) else None   # (first stored row, count): see fused_gemm
    p = []
    if not exact_b:
        p.append((Part(a, PART_F16HI, a_aux), Part(b, PART_F16LO, b_aux), negate, win))
    if not exact_a:
        p.append((Part(a, PART_F16LO, a_aux), Part(b, PART_F16HI, b_aux), negate, win))
    p.append((Part(a, PART_F16HI, a_aux), Part(b, PART_F16HI, b_aux), negate, win))
    return p


def f16_scale_state(max_abs):
    """The 1 x 4 device matrix `momentum_update` keeps for a parameter in scaled half-precision
    form: {exponent, -, max |w| of the running update (bits), -}; the exponent puts the largest
    magnitude at or below 2^13.  `.slice(0, 1)` is the `scale_exp` of a product."""
    e = float(np.floor(np.log2(8192.0 / max(float(max_abs), 1e-30))))
    return CUDAMatrix(np.array([[e, e, 0.0, 0.0]], np.float32))


def split_passes(a, b, negate=0, exact_a=False, exact_b=False, terms="bf16", a_aux=None, b_aux=None, a_rows=None,
                 b_rows=None):
    """The terms of a . b at fp32 grade, small terms first.  terms="bf16": the corrections are
    bfloat16 products, lo16(a).b16(b) + b16(a).lo16(b) (twice the TF32 rate; 2^-18 per term);
    terms="tf32": TF32 products lo32(a).b + a.lo32(b) (2^-20 per term: for products whose
    difference is wanted, like positive minus negative statistics).  exact_a / exact_b: that
    operand is exact in TF32 (0/1 data and samples, small counts), its low part is skipped.
    a_aux / b_aux: AuxMatrix of a / b (of the untransposed matrix): the bfloat16 parts are read
    from it instead of being derived in the kernel, which the big products need to run at the
    tensor pipe's rate."""
    win = dict(a_rows=a_rows, b_rows=b_rows) if (a_rows or b_rows) else None
    p = []
    if terms == "bf16":
        if not exact_a:
            p.append((lo16(a, a_aux), b16(b, b_aux), negate, win))
        if not exact_b:
            p.append((b16(a, a_aux), lo16(b, b_aux), negate, win))
        p.append((Part(a, PART_X, a_aux), Part(b, PART_X, b_aux), negate, win))
    else:
        if not exact_a:
            p.append((lo32(a), b, negate, win))
        if not exact_b:
            p.append((a, lo32(b), negate, win))
        p.append((a, b, negate, win))
    return p


def empty(shape):
    """cudamat/cudamat.py:1533-1544; zero-filled like eigenmat's (eigenmat/eigenmat.py:1339-1343)."""
    _require_device()
    mat = cudamat()
    _check(_lib.init_empty(ct.pointer(mat), ct.c_int(shape[0]), ct.c_int(shape[1])))
    return CUDAMatrix._from_mat(mat)


def reformat(array):
    """cudamat/cudamat.py:1863-1868."""
    return np.array(array, dtype=np.float32, order="F")


def sum(mat, axis, target=None):
    m = _lib.get_leading_dimension(mat.p_mat)
    n = _lib.get_nonleading_dimension(mat.p_mat)
    if target is None:
        target = empty((1, n)) if axis == 0 else empty((m, 1))
    _check(_lib.sum_by_axis(mat.p_mat, target.p_mat, ct.c_int(axis)))
    return target


def dot(m1, m2, mult=1.0, target=None):
    if target is None:
        m = _lib.get_leading_dimension(m1.p_mat)
        n = _lib.get_nonleading_dimension(m2.p_mat)
        target = empty((m, n))
    _check(_lib.dot(m1.p_mat, m2.p_mat, target.p_mat, ct.c_float(0.0), ct.c_float(mult)))
    return target


def vdot(m1, m2):
    err = ct.c_int(0)
    r = _lib.vdot(m1.p_mat, m2.p_mat, ct.byref(err))
    _check(err.value)
    return r


def _unary(fn):
    def op(mat, target=None):
        target = target or mat
        _check(fn(mat.p_mat, target.p_mat))
        return target
    return op


sigmoid = _unary(_lib.apply_sigmoid)
tanh = _unary(_lib.apply_tanh)
abs = _unary(_lib.apply_abs)
log_1_plus_exp = _unary(_lib.apply_log_1_plus_exp)
exp = _unary(_lib.apply_exp)
sqrt = _unary(_lib.apply_sqrt)


def log(mat, target=None, tiny=0.0):
    target = target or mat
    _check(_lib.apply_log(mat.p_mat, target.p_mat, ct.c_float(tiny)))
    return target


def pow(mat, p, target=None):
    target = target or mat
    _check(_lib.apply_pow(mat.p_mat, ct.c_float(p), target.p_mat))
    return target


def cross_entropy_bernoulli(mat, p, target=None, tiny=1e-10):
    target = target or mat
    _check(_lib.compute_cross_entropy_bernoulli(mat.p_mat, p.p_mat, target.p_mat, ct.c_float(tiny)))
    return target


def correct_preds(mat, p, target=None, cutoff=0.5):
    target = target or mat
    _check(_lib.correct_preds(mat.p_mat, p.p_mat, target.p_mat, ct.c_float(cutoff)))
    return target


def fused_gemm(passes, out=None, sample=None, bias=None, col_scale=None, activation=0, alpha=1.0, beta=0.0,
               out_aux=None, sample_aux=None, scale_exp=None, scale_exp_const=0, aux_f16=False, aux_exp=0):
    """out = act(alpha * sum_p (+/-) a_p . b_p + beta * out + bias (x) col_scale) in one kernel.

    `passes` is a list of (a, b) or (a, b, negate); a and b are fp32 matrices, `.T` views, or
    parts of them (`lo32(x)`, `lo16(x)`, `b16(x)`, see `split_passes`); both operands of a
    term are fp32-wide (a TF32 product) or both bfloat16.  Optional outputs: a Bernoulli draw
    of the result (consumes one sampling call of the global random state) and the aux matrices
    (bfloat16 parts) of result and draw.  With operands in scaled half-precision form
    (`f16_passes`) the terms carry 2^(scale_exp + scale_exp_const) (scale_exp: 1 x 1 device matrix
    or None), which the kernel divides out; aux_f16: the aux outputs are written in that form
    with exponent aux_exp.  Replaces the dot / add_dot / add_col_vec / sigmoid /
    sample_bernoulli group of deepnet/dbm.py:88-105.
    """
    f = _build_fused_gemm(passes, out, sample, bias, col_scale, activation, alpha, beta, out_aux, sample_aux, scale_exp,
                          scale_exp_const, aux_f16, aux_exp)
    _check(_lib.fused_gemm(CUDAMatrix.rnd_state_p, ct.byref(f)))


def _build_fused_gemm(passes, out=None, sample=None, bias=None, col_scale=None, activation=0, alpha=1.0, beta=0.0,
                      out_aux=None, sample_aux=None, scale_exp=None, scale_exp_const=0, aux_f16=False, aux_exp=0):
    """The argument block of `fused_gemm` (it points into the matrices' handles: keep them alive)."""
    f = _FusedGemm()
    f.npass = len(passes)
    if not 0 < f.npass <= MAX_PASS:
        raise CUDAMatException("fused_gemm takes 1..%d passes" % MAX_PASS)
    for i, p in enumerate(passes):
        f.passes[i].a = p[0].p_mat
        f.passes[i].b = p[1].p_mat
        for side, op in (("a", p[0]), ("b", p[1])):
            is_part = isinstance(op, Part)
            setattr(f.passes[i], side + "_part", op.part if is_part else PART_X)
            if is_part and op.aux is not None:
                setattr(f.passes[i], side + "_aux", op.aux.p_mat)
        f.passes[i].negate = int(p[2]) if len(p) > 2 else 0
        if len(p) > 3 and p[3]:      # row windows: dict(a_rows=(first, count), b_rows=(first, count))
            for side in ("a", "b"):
                win = p[3].get(side + "_rows")
                if win:
                    setattr(f.passes[i], side + "_row0", int(win[0]))
                    setattr(f.passes[i], side + "_rows", int(win[1]))
    f.alpha, f.beta, f.activation = alpha, beta, activation
    f.scale_exp_const, f.aux_f16, f.aux_exp = int(scale_exp_const), int(bool(aux_f16)), int(aux_exp)
    for name, m in (("bias", bias), ("col_scale", col_scale), ("out", out), ("sample", sample),
                    ("out_aux", out_aux), ("sample_aux", sample_aux), ("scale_exp", scale_exp)):
        if m is not None:
            setattr(f, name, m.p_mat)
    return f


# -- one call per training step ---------------------------------------------------------
# The operations a training step is made of, under one vocabulary with two executors: `Immediate`
# issues each through its own library call as it is named; `Program` records them once and
# replays the whole list from C with a single call per step (b200_run_program), which is what
# the small configurations need: their kernels are shorter than a call from Python.
(OP_FUSED_GEMM, OP_SUM_AXIS, OP_ADD_SUM_AXIS, OP_ROW_SUM_DIFF, OP_ADD_SQ_DIFF, OP_MOMENTUM_UPDATE, OP_SPLIT_F16,
 OP_SPLIT_BF16, OP_ALLREDUCE, OP_SOFTMAX_SCALED, OP_SAMPLE_MULTINOMIAL, OP_DIV_BY_ROW, OP_ADD_SCALAR, OP_ASSIGN_SCALAR,
 OP_COPY, OP_SAMPLE_BERNOULLI, OP_SOFTMAX_SAMPLE, OP_MOMENTUM_UPDATE_COLUMNS, OP_ALLREDUCE_BEGIN, OP_ALLREDUCE_END,
 OP_SM_LIMIT, OP_DP_PEER_UPDATE) = range(22)


class _Op(ct.Structure):
    _fields_ = [("kind", ct.c_int), ("i0", ct.c_int), ("i1", ct.c_int), ("i2", ct.c_int),
                ("f0", ct.c_float), ("f1", ct.c_float), ("f2", ct.c_float), ("f3", ct.c_float), ("f4", ct.c_float),
                ("f5", ct.c_float), ("f6", ct.c_float), ("f7", ct.c_float),
                ("m", ct.POINTER(cudamat) * 8), ("gemm", ct.POINTER(_FusedGemm))]


_lib.b200_run_program.argtypes = [ct.POINTER(rnd_struct), ct.POINTER(_Op), ct.c_int, ct.POINTER(ct.c_int)]


class Immediate(object):
    """Issues every operation at once, one library call each."""

    launches = {OP_FUSED_GEMM: 1}

    def fused_gemm(self, passes, **kw):
        fused_gemm(passes, **kw)

    def sum(self, mat, axis, target):
        sum(mat, axis, target)

    def add_sums(self, target, mat, axis, mult=1.0):
        target.add_sums(mat, axis, mult)

    def row_sum_diff(self, a, b, target):
        _check(_lib.row_sum_diff(a.p_mat, b.p_mat, target.p_mat))

    def sq_diff(self, a, b, acc):
        _check(_lib.add_sq_diff(a.p_mat, b.p_mat, acc.p_mat))

    def momentum_update(self, w, delta, grad, suff, inv_batch, momentum, eps, l2=0.0, l1=0.0, w_aux=None, w_scale=None):
        w.momentum_update(delta, grad, suff, inv_batch, momentum, eps, l2=l2, l1=l1, w_aux=w_aux, w_scale=w_scale)

    def momentum_update_columns(self, w, delta, grad, suff, col0, ncols, inv_batch, momentum, eps, l2=0.0, l1=0.0,
                                w_aux=None, w_scale=None):
        p = lambda m: m.p_mat if m is not None else None
        _check(_lib.momentum_update_columns(w.p_mat, delta.p_mat, p(grad), suff.p_mat, p(w_aux), p(w_scale), ct.c_int(col0),
                                            ct.c_int(ncols), ct.c_float(inv_batch), ct.c_float(momentum), ct.c_float(eps),
                                            ct.c_float(l2), ct.c_float(l1)))

    def split_f16(self, x, aux, exp_dev=None, exp_const=0):
        x.split_f16(aux, exp_dev, exp_const)

    def split_bf16(self, x, aux):
        x.split_bf16(aux)

    def allreduce(self, mat):
        dp_allreduce(mat)

    def allreduce_begin(self, mat, slot):
        _check(_lib.dp_allreduce_begin(mat.p_mat, ct.c_int(slot)))

    def allreduce_end(self, slot):
        _check(_lib.dp_allreduce_end(ct.c_int(slot)))

    def sm_limit(self, sms):
        _check(_lib.b200_set_sm_limit(ct.c_int(sms)))

    def dp_peer_update(self, w, delta, w_aux, w_scale, pack, b, db, inv_batch, mom_b, eps_b, mom_w, eps_w, l2=0.0, l1=0.0):
        p = lambda m: m.p_mat if m is not None else None
        _check(_lib.dp_peer_update(w.p_mat, delta.p_mat, p(w_aux), p(w_scale), pack.p_mat, b.p_mat, db.p_mat,
                                   ct.c_float(inv_batch), ct.c_float(mom_b), ct.c_float(eps_b), ct.c_float(mom_w),
                                   ct.c_float(eps_w), ct.c_float(l2), ct.c_float(l1)))

    def softmax_scaled(self, mat, scale, target):
        mat.softmax_scaled(scale, target)

    def sample_multinomial(self, probs, nn, target, max_draws=1000):
        probs.sample_multinomial(nn, target, max_draws)

    def div_by_row(self, mat, vec, target):
        mat.div_by_row(vec, target)

    def add_scalar(self, mat, val, target=None):
        mat.add(val, target)

    def assign_scalar(self, mat, val):
        mat.assign(val)

    def copy(self, src, dst):
        dst.assign(src)

    def sample_bernoulli(self, mat, target):
        mat.sample_bernoulli(target)

    def softmax_sample(self, pre, state, sample=None, bias=None):
        pre.softmax_sample(state, sample, bias)


class Program(object):
    """Records the operations of a step (same methods as `Immediate`), then `run()` replays them
    with one call.  Every method returns the index of the recorded operation; `set_floats`
    changes the scalars of one (momentum and learning rate follow their schedules)."""

    def __init__(self):
        self._ops, self._keep, self._arr = [], [], None

    def _add(self, kind, mats=(), ints=(), floats=(), gemm=None):
        op = _Op()
        op.kind = kind
        for i, m in enumerate(mats):
            if m is not None:
                op.m[i] = m.p_mat
                self._keep.append(m)
        for name, v in zip(("i0", "i1", "i2"), ints):
            setattr(op, name, int(v))
        for name, v in zip(("f0", "f1", "f2", "f3", "f4", "f5", "f6", "f7"), floats):
            setattr(op, name, float(v))
        if gemm is not None:
            op.gemm = ct.pointer(gemm)
            self._keep.append(gemm)
        self._ops.append(op)
        self._arr = None
        return len(self._ops) - 1

    def fused_gemm(self, passes, **kw):
        for p in passes:
            self._keep.extend([p[0], p[1]])
        self._keep.extend(v for v in kw.values() if isinstance(v, CUDAMatrix))
        return self._add(OP_FUSED_GEMM, gemm=_build_fused_gemm(passes, **kw))

    def sum(self, mat, axis, target):
        return self._add(OP_SUM_AXIS, (mat, target), (axis,))

    def add_sums(self, target, mat, axis, mult=1.0):
        return self._add(OP_ADD_SUM_AXIS, (mat, target), (axis,), (mult,))

    def row_sum_diff(self, a, b, target):
        return self._add(OP_ROW_SUM_DIFF, (a, b, target))

    def sq_diff(self, a, b, acc):
        return self._add(OP_ADD_SQ_DIFF, (a, b, acc))

    def momentum_update(self, w, delta, grad, suff, inv_batch, momentum, eps, l2=0.0, l1=0.0, w_aux=None, w_scale=None):
        return self._add(OP_MOMENTUM_UPDATE, (w, delta, grad, suff, w_aux, w_scale), (), (inv_batch, momentum, eps, l2, l1))

    def momentum_update_columns(self, w, delta, grad, suff, col0, ncols, inv_batch, momentum, eps, l2=0.0, l1=0.0,
                                w_aux=None, w_scale=None):
        return self._add(OP_MOMENTUM_UPDATE_COLUMNS, (w, delta, grad, suff, w_aux, w_scale), (col0, ncols),
                         (inv_batch, momentum, eps, l2, l1))

    def allreduce_begin(self, mat, slot):
        return self._add(OP_ALLREDUCE_BEGIN, (mat,), (slot,))

    def allreduce_end(self, slot):
        return self._add(OP_ALLREDUCE_END, (), (slot,))

    def sm_limit(self, sms):
        return self._add(OP_SM_LIMIT, (), (sms,))

    def dp_peer_update(self, w, delta, w_aux, w_scale, pack, b, db, inv_batch, mom_b, eps_b, mom_w, eps_w, l2=0.0, l1=0.0):
        return self._add(OP_DP_PEER_UPDATE, (w, delta, w_aux, w_scale, pack, b, db), (),
                         (inv_batch, mom_b, eps_b, mom_w, eps_w, l2, l1))

    def split_f16(self, x, aux, exp_dev=None, exp_const=0):
        return self._add(OP_SPLIT_F16, (x, aux, exp_dev), (exp_const,))

    def split_bf16(self, x, aux):
        return self._add(OP_SPLIT_BF16, (x, aux))

    def allreduce(self, mat):
        return self._add(OP_ALLREDUCE, (mat,))

    def softmax_scaled(self, mat, scale, target):
        return self._add(OP_SOFTMAX_SCALED, (mat, scale, target))

    def sample_multinomial(self, probs, nn, target, max_draws=1000):
        return self._add(OP_SAMPLE_MULTINOMIAL, (probs, nn, target), (max_draws,))

    def div_by_row(self, mat, vec, target):
        return self._add(OP_DIV_BY_ROW, (mat, vec, target))

    def add_scalar(self, mat, val, target=None):
        return self._add(OP_ADD_SCALAR, (mat, target or mat), (), (val,))

    def assign_scalar(self, mat, val):
        return self._add(OP_ASSIGN_SCALAR, (mat,), (), (val,))

    def copy(self, src, dst):
        return self._add(OP_COPY, (src, dst))

    def sample_bernoulli(self, mat, target):
        return self._add(OP_SAMPLE_BERNOULLI, (mat, target))

    def softmax_sample(self, pre, state, sample=None, bias=None):
        return self._add(OP_SOFTMAX_SAMPLE, (pre, bias, state, sample))

    def __len__(self):
        return len(self._ops)

    def _array(self):
        if self._arr is None:
            self._arr = (_Op * len(self._ops))(*self._ops)
        return self._arr

    def set_floats(self, index, **kw):
        """kw: f0..f4 of operation `index` (momentum_update: f0 1/batch, f1 momentum, f2 epsilon, f3 l2, f4 l1)."""
        op = self._array()[index]
        for k, v in kw.items():
            setattr(op, k, float(v))

    def run(self):
        failed = ct.c_int(-1)
        err = _lib.b200_run_program(CUDAMatrix.rnd_state_p, self._array(), len(self._ops), ct.byref(failed))
        if err:
            e = generate_exception(err)
            raise CUDAMatException("operation %d of the recorded step failed: %s" % (failed.value, e))


# -- device-resident data feed -----------------------------------------------------------
_lib.feed_permutation_at.restype = ct.c_uint
_lib.feed_permutation_at.argtypes = [ct.c_uint, ct.c_uint, ct.c_uint, ct.c_uint]


def feed_pack(array):
    """A (dims x cases) 0/1 host array as a device matrix of one bit per value: ceil(dims / 32) x cases
    32-bit words, bit r % 32 of word r // 32 of a column = row r (see `feed_gather`)."""
    a = np.asarray(array)
    dims, n = a.shape
    if not np.isin(a, (0, 1)).all():
        raise ValueError("only 0/1 data can be stored one bit per value")
    words = (dims + 31) // 32
    bits = np.zeros((n, words * 32), np.uint8)
    bits[:, :dims] = a.T
    packed = np.packbits(bits, axis=1, bitorder="little").view("<u4")            # cases x words
    # the words travel as float32 storage (same-type copies keep every bit); they are never read as floats
    return CUDAMatrix(np.ascontiguousarray(packed.T).view(np.float32))


def feed_gather(src, packed, dims, key, shuffle, start, out, mean=None, std=None, out_aux=None, aux_mode=0, aux_exp=0):
    """out = stored columns perm(start ..) of the data set `src` (see include/b200mat.h); key = (lo, hi)."""
    _check(_lib.feed_gather(src.p_mat, ct.c_int(int(bool(packed))), ct.c_int(dims), ct.c_uint(key[0] & 0xffffffff),
                            ct.c_uint(key[1] & 0xffffffff), ct.c_int(int(bool(shuffle))), ct.c_int(int(start)),
                            mean.p_mat if mean is not None else None, std.p_mat if std is not None else None,
                            out.p_mat, out_aux.p_mat if out_aux is not None else None, ct.c_int(aux_mode),
                            ct.c_int(aux_exp)))
    return out


def feed_permutation(n, key):
    """The stored column read at every position of the epoch keyed `key`, as the device evaluates it."""
    return np.array([_lib.feed_permutation_at(i, n, key[0] & 0xffffffff, key[1] & 0xffffffff) for i in range(n)], np.int64)


# -- device / library control -----------------------------------------------------
def cuda_set_device(dev_id):
    _check(_lib.cuda_set_device(ct.c_int(dev_id)))


MAX_ONES = 1024 * 256


def cublas_init():
    """cudamat/cudamat.py:1879-1885: brings the library up and fills `CUDAMatrix.ones`, the column
    of ones the reference's callers multiply with for sums."""
    _require_device()
    if CUDAMatrix.ones is None:
        CUDAMatrix.ones = CUDAMatrix(np.ones((MAX_ONES, 1), dtype=np.float32, order="F"))


init = cublas_init


def cublas_shutdown():
    CUDAMatrix.ones = None
    _lib.cublas_shutdown()


shutdown = cublas_shutdown


def cuda_sync_threads():
    _lib.cuda_sync_threads()


def set_gemm_path(path):
    """0 auto, 1 tensor cores only, 2 CUDA cores only."""
    _lib.b200_set_gemm_path(ct.c_int(path))


def set_dot_precision(mode):
    """0: fp32-grade split-TF32 `dot` (default); 1: one TF32 pass."""
    _lib.b200_set_dot_precision(ct.c_int(mode))


def set_sm_limit(sms):
    """SMs the library's kernels size their grids for (0 = all of the device)."""
    _check(_lib.b200_set_sm_limit(ct.c_int(int(sms))))


def sm_count():
    return _lib.b200_sm_count()


def set_split_k(mode):
    """Split-K of the tensor-core product: 0 automatic (default), 1 never, n > 1 always n splits."""
    _lib.b200_set_split_k(ct.c_int(mode))


def set_rng_column_offset(col0):
    _check(_lib.set_rng_column_offset(ct.c_int(col0)))


def read_status():
    """Non-zero if a kernel's bounded wait gave up since the last call (blocks)."""
    return _lib.b200_read_status()


def set_wait_limit(iterations):
    """Iterations a device-side wait may spin before its kernel gives up and records a status
    (default 2^24, one to two seconds; 0 restores the default)."""
    _check(_lib.b200_set_wait_limit(ct.c_uint(int(iterations))))


def set_dependent_launch(on):
    """Programmatic dependent launch of the step's kernels (on by default): a kernel is scheduled
    while its predecessor drains and touches global memory only after that one has completed."""
    _check(_lib.b200_set_dependent_launch(1 if on else 0))


class Event(object):
    """A CUDA event on the library stream: e.record(); ...; start.elapsed_ms(end)."""

    def __init__(self):
        _require_device()
        self.ev = _lib.b200_event_create()
        if not self.ev:
            raise CUDAMatException("cudaEventCreate failed")

    def record(self):
        _check(_lib.b200_event_record(ct.c_void_p(self.ev)))
        return self

    def elapsed_ms(self, end):
        ms = _lib.b200_event_elapsed_ms(ct.c_void_p(self.ev), ct.c_void_p(end.ev))
        if ms < 0:
            raise CUDAMatException("event timing failed: " + _lib.get_last_cuda_error().decode("utf-8", "replace"))
        return ms

    def __del__(self):
        try:
            _lib.b200_event_destroy(ct.c_void_p(self.ev))
        except Exception:
            pass


def host_alloc(shape):
    """Returns (array, ptr): a pinned float32 Fortran-order host array; free with host_free(ptr)."""
    n = int(np.prod(shape))
    ptr = _lib.b200_host_alloc(ct.c_size_t(n * 4))
    if not ptr:
        raise CUDAMatException("pinned host allocation failed")
    buf = (ct.c_float * n).from_address(ptr)
    arr = np.frombuffer(buf, dtype=np.float32).reshape(shape, order="F")
    return arr, ptr


def readback_begin(src, host_ptr, nbytes, slot=0):
    """Starts a device-to-host copy of `src` into pinned host memory, ordered after the work enqueued so
    far, without blocking (slot 0..7); `readback_wait(slot)` blocks until it has landed."""
    _check(_lib.b200_readback_begin(src.p_mat, ct.c_void_p(host_ptr), ct.c_size_t(nbytes), ct.c_int(slot)))


def readback_wait(slot=0):
    _check(_lib.b200_readback_wait(ct.c_int(slot)))


def prefetch_wait():
    _check(_lib.b200_prefetch_wait())


def prefetch_fence():
    _check(_lib.b200_prefetch_fence())


def host_free(ptr):
    _lib.b200_host_free(ct.c_void_p(ptr))


# -- data parallelism ------------------------------------------------------------------
def dp_unique_id():
    buf = ct.create_string_buffer(128)
    _check(_lib.dp_unique_id(buf))
    return buf.raw


def dp_init(unique_id, nranks, rank):
    _check(_lib.dp_init(ct.c_char_p(unique_id), ct.c_int(nranks), ct.c_int(rank)))


def dp_allreduce(mat):
    _check(_lib.dp_allreduce(mat.p_mat))


def dp_check():
    _check(_lib.dp_check())


def dp_destroy():
    _lib.dp_destroy()


def dp_peer_setup(group, pack, w, w_aux):
    """Maps every rank's statistics, parameter, its 16-bit planes, flag array and receive buffer into
    this process (CUDA IPC) for `dp_peer_update`; from here on the product whose result is the
    statistics area of `pack` delivers its column panels to their owners' receive buffers.  group: a `rendezvous.Group` (the handles travel through it).
    Returns True when EVERY rank has mapped every peer; otherwise every rank has closed what it
    opened and gets False (the ranks agree, so that all of them fall back to the all-reduce)."""
    n = _lib.dp_peer_handle_bytes()
    mine = b""
    try:
        for m in (pack, w, w_aux):
            buf = ct.create_string_buffer(n)
            if m is not None:
                _check(_lib.dp_peer_export(m.p_mat, buf))
            mine += buf.raw
        buf = ct.create_string_buffer(n)
        _check(_lib.dp_peer_export_flags(buf))
        mine += buf.raw
        buf = ct.create_string_buffer(n)
        _check(_lib.dp_peer_export_recv(ct.c_long(w.shape[0] * w.shape[1]), buf))
        mine += buf.raw
    except CUDAMatException:
        mine = b""                              # told to the peers through the exchange itself
    payloads = group.exchange("peer_handles", mine)
    failed = 0.0
    if any(len(x) != 5 * n for x in payloads):
        failed = 1.0
    else:
        err = _lib.dp_peer_setup(ct.c_int(group.world), ct.c_int(group.rank), ct.c_char_p(b"".join(payloads)), pack.p_mat,
                                 w.p_mat, w_aux.p_mat if w_aux is not None else None)
        failed = 1.0 if err else 0.0
    if group.max(failed) > 0:
        _lib.dp_peer_close()
        return False
    return True


def dp_peer_close():
    _lib.dp_peer_close()


def dp_peer_mode():
    """0: not set up; 1: the owners fetch the statistics panels; 2: the statistics product delivers them."""
    return _lib.dp_peer_mode()


def dp_wait(timeout_ms=30000):
    """Blocks until the enqueued work (all-reduces included) is done; a collective that does not
    complete within timeout_ms (a peer never joined) is aborted and raises."""
    _check(_lib.dp_wait(ct.c_int(int(timeout_ms))))


def dp_abort():
    """Tears the communicator down without waiting for collectives in flight (a peer is gone)."""
    _lib.dp_abort()
