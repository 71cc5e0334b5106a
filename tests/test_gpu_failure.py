"""Failure detection on the device without faulting it: a wait of the tensor-core product that
cannot complete must run into its limit, leave a status word for the host and let the kernel
return by itself, and the next product must work.  The failure is injected on the host (the
product is told to expect more bytes per stage than its copies deliver); nothing traps,
reads a bad address or waits without bound."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def get(m):
    return np.array(m.asarray(), copy=True)


@pytest.mark.parametrize("m,n,k,form", [(512, 512, 512, "derived"), (256, 128, 256, "derived"), (512, 512, 512, "f16")])
def test_a_wait_that_cannot_complete_times_out_and_the_library_recovers(cm, m, n, k, form):
    rng = np.random.default_rng(3)
    A = (rng.standard_normal((m, k)) * 0.05).astype(np.float32)
    B = rng.random((k, n)).astype(np.float32)
    a, b, out = cm.CUDAMatrix(A), cm.CUDAMatrix(B), cm.empty((m, n))
    scale = cm.f16_scale_state(np.abs(A).max())
    xa = a.split_f16(cm.empty_aux(A.shape), exp_dev=scale.slice(0, 1))
    xb = b.split_f16(cm.empty_aux(B.shape), exp_const=14)

    def product():
        if form == "f16":     # every tile comes from memory: the copies report to the issuer's barrier
            cm.fused_gemm(cm.f16_passes(a, xa, b, xb), out=out, scale_exp=scale.slice(0, 1), scale_exp_const=14)
        else:                 # parts derived in the kernel: the converter warps wait for the copies
            cm.fused_gemm(cm.split_passes(a, b, terms="tf32"), out=out)

    cm.set_gemm_path(1)
    assert cm.read_status() == 0
    cm.set_wait_limit(20000)                      # a few milliseconds instead of seconds
    try:
        cm._lib.b200_test_inject_stage_bytes(64)
        product()
        status = cm.read_status()                 # blocks until the kernel has returned by itself
        assert status != 0
        assert cm.read_status() == 0              # reading clears it
    finally:
        cm.set_wait_limit(0)
        cm.set_gemm_path(0)
    cm.set_gemm_path(1)
    product()                                     # the injection applied to one product only
    cm.set_gemm_path(0)
    want = A.astype(np.float64) @ B.astype(np.float64)
    assert np.abs(get(out) - want).max() / np.abs(want).max() < 1e-5
    assert cm.read_status() == 0
