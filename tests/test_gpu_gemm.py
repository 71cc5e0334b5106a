"""GPU parity of the matrix product: the tcgen05 split-TF32 kernel and the CUDA-core
kernel against float64 numpy and the oracle, all four transpose layouts, ragged edges,
and the fused epilogue (bias, logistic, Bernoulli draw, TF32 split, negated passes).

Tolerance: 1e-5 of the largest magnitude of the exact result (the bound the path must
meet on activations and gradients); the single-pass TF32 mode is checked at 2e-3."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

TOL = 1e-5


def get(m):
    return np.array(m.asarray(), copy=True)


def relerr(got, want):
    return np.abs(got - want).max() / max(np.abs(want).max(), 1e-30)


@pytest.fixture(autouse=True)
def _auto_path(cm):
    yield
    cm.set_gemm_path(0)
    cm.set_dot_precision(0)


def make(cm, x, trans):
    """A handle whose op() equals x: stored transposed when trans."""
    if trans:
        return cm.CUDAMatrix(np.ascontiguousarray(x.T)).T
    return cm.CUDAMatrix(x)


@pytest.mark.parametrize("path", [1, 2])
@pytest.mark.parametrize("ta,tb", [(0, 0), (1, 0), (0, 1), (1, 1)])
@pytest.mark.parametrize("m,n,k", [(128, 64, 32), (500, 1000, 600), (128, 256, 64), (4, 4, 4), (132, 68, 36),
                                   (784, 100, 500), (1024, 256, 4096)])
def test_dot_all_layouts(cm, path, ta, tb, m, n, k):
    rng = np.random.default_rng(m * 7 + n * 3 + k)
    A = rng.standard_normal((m, k)).astype(np.float32)
    B = rng.standard_normal((k, n)).astype(np.float32)
    cm.set_gemm_path(path)
    out = cm.empty((m, n))
    cm.dot(make(cm, A, ta), make(cm, B, tb), target=out)
    want = A.astype(np.float64) @ B.astype(np.float64)
    assert relerr(get(out), want) < TOL
    assert cm.read_status() == 0


@pytest.mark.parametrize("m,n,k", [(7, 5, 3), (127, 33, 65), (1, 1, 1), (1, 257, 19)])
def test_dot_untileable_shapes_use_cuda_cores(cm, m, n, k):
    # leading dimensions that TMA cannot address: auto falls back, tensor-core-only refuses
    rng = np.random.default_rng(5)
    A = rng.standard_normal((m, k)).astype(np.float32)
    B = rng.standard_normal((k, n)).astype(np.float32)
    out = cm.dot(cm.CUDAMatrix(A), cm.CUDAMatrix(B))
    assert relerr(get(out), A.astype(np.float64) @ B) < TOL
    if m % 4 or k % 4:
        cm.set_gemm_path(1)
        with pytest.raises(cm.CUDAMatException):
            cm.dot(cm.CUDAMatrix(A), cm.CUDAMatrix(B))


def test_add_dot_subtract_dot_and_scaling(cm):
    # cudamat/test_cudamat.py:829-880
    rng = np.random.default_rng(6)
    A = rng.standard_normal((128, 64)).astype(np.float32)
    B = rng.standard_normal((64, 256)).astype(np.float32)
    C = rng.standard_normal((128, 256)).astype(np.float32)
    for path in (1, 2):
        cm.set_gemm_path(path)
        c = cm.CUDAMatrix(C)
        c.add_dot(cm.CUDAMatrix(A), cm.CUDAMatrix(B), mult=0.5)
        want = C + 0.5 * (A.astype(np.float64) @ B)
        assert relerr(get(c), want) < TOL
        c.subtract_dot(cm.CUDAMatrix(A), cm.CUDAMatrix(B))
        assert relerr(get(c), want - A.astype(np.float64) @ B) < TOL


def test_single_pass_tf32_mode_truncates_operands(cm):
    rng = np.random.default_rng(7)
    A = rng.standard_normal((256, 512)).astype(np.float32)
    B = rng.standard_normal((512, 128)).astype(np.float32)
    cm.set_gemm_path(1)
    cm.set_dot_precision(1)
    out = get(cm.dot(cm.CUDAMatrix(A), cm.CUDAMatrix(B)))
    tr = lambda x: (x.view(np.uint32) & np.uint32(0xffffe000)).view(np.float32).astype(np.float64)
    assert relerr(out, tr(A) @ tr(B)) < TOL          # the tensor core drops the low 13 mantissa bits
    assert relerr(out, A.astype(np.float64) @ B) < 2e-3


def test_split_tf32_is_exact(cm):
    rng = np.random.default_rng(8)
    x = (rng.standard_normal((100, 33)) * 10.0 ** rng.integers(-3, 4, (100, 33))).astype(np.float32)
    g = cm.CUDAMatrix(x)
    hi, lo = cm.empty(x.shape), cm.empty(x.shape)
    g.split_tf32(lo, hi=hi)
    h, l = get(hi), get(lo)
    np.testing.assert_array_equal(h, (x.view(np.uint32) & np.uint32(0xffffe000)).view(np.float32))
    np.testing.assert_array_equal(h + l, x)


def bf16_round(x):
    """float32 -> nearest bfloat16 (ties to even), as float32."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7fff + ((u >> 16) & 1)) >> 16).astype(np.uint32) << 16
    return r.view(np.float32).reshape(np.shape(x))


def tf32_trunc(x):
    return (np.ascontiguousarray(x, np.float32).view(np.uint32) & np.uint32(0xffffe000)).view(np.float32)


def part_values(x, part):
    """What the kernels multiply for each operand part (float32)."""
    if part == 0:
        return tf32_trunc(x)
    lo = (x - tf32_trunc(x)).astype(np.float32)
    if part == 1:
        return tf32_trunc(lo)
    return bf16_round(lo) if part == 2 else bf16_round(x)


@pytest.mark.parametrize("path", [1, 2])
@pytest.mark.parametrize("ta,tb", [(0, 0), (1, 0), (0, 1), (1, 1)])
@pytest.mark.parametrize("m,n,k", [(500, 300, 784), (128, 64, 96), (260, 36, 40), (1000, 520, 2100)])
def test_operand_parts_in_all_layouts(cm, path, ta, tb, m, n, k):
    """One term over parts of the operands = the exact product of the parts' values (fp32
    accumulation): the converter warps write what TMA would have delivered, in all four layouts."""
    rng = np.random.default_rng(13)
    A = rng.standard_normal((m, k)).astype(np.float32)
    B = rng.standard_normal((k, n)).astype(np.float32)
    cm.set_gemm_path(path)
    sa, sb = (A.T if ta else A), (B.T if tb else B)          # stored forms
    ga, gb = cm.CUDAMatrix(np.asfortranarray(sa)), cm.CUDAMatrix(np.asfortranarray(sb))
    oa, ob = (ga.T if ta else ga), (gb.T if tb else gb)
    for pa, pb in ((0, 0), (1, 0), (0, 1), (3, 3), (2, 3), (3, 2)):
        out = cm.empty((m, n))
        cm.fused_gemm([(cm.Part(oa, pa), cm.Part(ob, pb))], out=out)
        want = part_values(A, pa).astype(np.float64) @ part_values(B, pb).astype(np.float64)
        assert relerr(get(out), want) < 5e-6, (pa, pb)   # fp32 accumulation of k mixed-sign terms
    assert cm.read_status() == 0


@pytest.mark.parametrize("shape", [(100, 33), (500, 100), (128, 256), (7, 5)])
def test_split_bf16_planes(cm, shape):
    rng = np.random.default_rng(12)
    x = (rng.standard_normal(shape) * 10.0 ** rng.integers(-3, 4, shape)).astype(np.float32)
    aux = cm.CUDAMatrix(x).split_bf16(cm.empty_aux(shape))
    lo, b = aux.planes()
    np.testing.assert_array_equal(lo, bf16_round(x - tf32_trunc(x)))
    np.testing.assert_array_equal(b, bf16_round(x))


@pytest.mark.parametrize("path", [1, 2])
@pytest.mark.parametrize("ta,tb", [(0, 0), (1, 0), (0, 1), (1, 1)])
@pytest.mark.parametrize("m,n,k", [(500, 300, 784), (260, 36, 40), (1000, 520, 2100)])
def test_bfloat16_parts_read_from_aux_matrices(cm, path, ta, tb, m, n, k):
    """The bfloat16 parts loaded from aux matrices give the same products as the parts the
    kernel derives, in all four layouts, also with the aux of one operand only."""
    rng = np.random.default_rng(15)
    A = rng.standard_normal((m, k)).astype(np.float32)
    B = rng.standard_normal((k, n)).astype(np.float32)
    cm.set_gemm_path(path)
    sa, sb = (A.T if ta else A), (B.T if tb else B)          # stored forms
    ga, gb = cm.CUDAMatrix(np.asfortranarray(sa)), cm.CUDAMatrix(np.asfortranarray(sb))
    xa, xb = ga.split_bf16(cm.empty_aux(sa.shape)), gb.split_bf16(cm.empty_aux(sb.shape))
    oa, ob = (ga.T if ta else ga), (gb.T if tb else gb)
    for pa, pb in ((3, 3), (2, 3), (3, 2)):
        want = part_values(A, pa).astype(np.float64) @ part_values(B, pb).astype(np.float64)
        for aux_a, aux_b in ((xa, xb), (xa, None), (None, xb)):
            out = cm.empty((m, n))
            cm.fused_gemm([(cm.Part(oa, pa, aux_a), cm.Part(ob, pb, aux_b))], out=out)
            assert relerr(get(out), want) < 5e-6, (pa, pb)
    # the full term list of a split product, every bfloat16 part from memory
    out = cm.empty((m, n))
    cm.fused_gemm(cm.split_passes(oa, ob, a_aux=xa, b_aux=xb), out=out)
    assert relerr(get(out), A.astype(np.float64) @ B.astype(np.float64)) < (2e-6 if path == 1 else 1e-5)
    assert cm.read_status() == 0


def f16_planes(aux):
    """(lo, hi) planes of an aux matrix in scaled half-precision form, as float32."""
    raw = np.array(aux.asarray(), copy=True)
    words = np.ascontiguousarray(raw.T).view(np.uint16)
    lda = raw.shape[0]
    f = lambda w: np.ascontiguousarray(w).view(np.float16).astype(np.float32).T[:aux.rows]
    return f(words[:, :lda]), f(words[:, lda:])


@pytest.mark.parametrize("path", [1, 2])
@pytest.mark.parametrize("ta,tb", [(0, 0), (1, 0), (0, 1), (1, 1)])
@pytest.mark.parametrize("m,n,k", [(500, 300, 784), (260, 36, 40), (1024, 512, 4096)])
def test_scaled_half_precision_product_in_all_layouts(cm, path, ta, tb, m, n, k):
    """x * 2^e = hi + lo in fp16: hi.lo + lo.hi + hi.hi, divided by 2^(ea + eb), is the product to
    fp32 grade; the planes hold exactly the fp16 roundings."""
    rng = np.random.default_rng(16)
    A = (rng.standard_normal((m, k)) * 0.03).astype(np.float32)       # weights-like
    B = rng.random((k, n)).astype(np.float32)                          # probabilities-like
    cm.set_gemm_path(path)
    sa, sb = (A.T if ta else A), (B.T if tb else B)
    ga, gb = cm.CUDAMatrix(np.asfortranarray(sa)), cm.CUDAMatrix(np.asfortranarray(sb))
    scale = cm.f16_scale_state(np.abs(A).max())
    ea, eb = float(get(scale)[0, 0]), 14
    assert np.abs(A).max() * 2.0 ** ea <= 8192 < np.abs(A).max() * 2.0 ** (ea + 1)
    xa = ga.split_f16(cm.empty_aux(sa.shape), exp_dev=scale.slice(0, 1))
    xb = gb.split_f16(cm.empty_aux(sb.shape), exp_const=eb)
    lo, hi = f16_planes(xa)
    want_hi = (sa * np.float32(2.0 ** ea)).astype(np.float16)
    np.testing.assert_array_equal(hi, want_hi.astype(np.float32))
    np.testing.assert_array_equal(lo, (sa * np.float32(2.0 ** ea) - want_hi.astype(np.float32)).astype(np.float16).astype(np.float32))
    oa, ob = (ga.T if ta else ga), (gb.T if tb else gb)
    out = cm.empty((m, n))
    cm.fused_gemm(cm.f16_passes(oa, xa, ob, xb), out=out, scale_exp=scale.slice(0, 1), scale_exp_const=eb)
    want = A.astype(np.float64) @ B.astype(np.float64)
    assert relerr(get(out), want) < (1e-6 if path == 1 else 1e-5)
    # a 0/1 operand needs its hi plane only
    Bb = (rng.random((k, n)) < 0.3).astype(np.float32)
    sbb = Bb.T if tb else Bb
    gbb = cm.CUDAMatrix(np.asfortranarray(sbb))
    xbb = gbb.split_f16(cm.empty_aux(sbb.shape), exp_const=eb)
    cm.fused_gemm(cm.f16_passes(oa, xa, gbb.T if tb else gbb, xbb, exact_b=True), out=out,
                  scale_exp=scale.slice(0, 1), scale_exp_const=eb)
    assert relerr(get(out), A.astype(np.float64) @ Bb.astype(np.float64)) < (1e-6 if path == 1 else 1e-5)
    assert cm.read_status() == 0


@pytest.mark.parametrize("path", [1, 2])
def test_scaled_half_precision_difference_of_products(cm, path):
    """Positive minus negative statistics: two nearly equal products subtracted in one accumulator."""
    rng = np.random.default_rng(17)
    M, N, K = 512, 384, 1024
    sig = lambda x: 1 / (1 + np.exp(-x))
    Ap = sig(rng.standard_normal((M, K)) * 0.3).astype(np.float32)
    Bp = sig(rng.standard_normal((K, N)) * 0.3).astype(np.float32)
    An = (Ap + rng.standard_normal((M, K)).astype(np.float32) * 0.02).clip(0, 1).astype(np.float32)
    Bn = (Bp + rng.standard_normal((K, N)).astype(np.float32) * 0.02).clip(0, 1).astype(np.float32)
    cm.set_gemm_path(path)
    mats = [cm.CUDAMatrix(x) for x in (Ap, Bp, An, Bn)]
    auxs = [g.split_f16(cm.empty_aux(g.shape), exp_const=14) for g in mats]
    out = cm.empty((M, N))
    P = cm.f16_passes
    cm.fused_gemm(P(mats[0], auxs[0], mats[1], auxs[1]) + P(mats[2], auxs[2], mats[3], auxs[3], negate=1), out=out,
                  scale_exp_const=28)
    want = Ap.astype(np.float64) @ Bp.astype(np.float64) - An.astype(np.float64) @ Bn.astype(np.float64)
    # each product is ~256, their difference ~1: 5e-5 of the difference is 2e-7 of the products,
    # the grade of an fp32 product (numpy's float32 matmul is at 2e-4 here)
    f32 = Ap @ Bp - An @ Bn
    # (the CUDA-core kernel adds the 1024 same-sign terms of each product one by one in fp32)
    assert relerr(get(out), want) < (min(1e-4, relerr(f32, want)) if path == 1 else 3e-3)


@pytest.mark.parametrize("path", [1, 2])
@pytest.mark.parametrize("m,n,k", [(500, 100, 784), (1024, 512, 2048)])
def test_fused_epilogue_writes_scaled_half_precision_aux(cm, oracle, path, m, n, k):
    rng = np.random.default_rng(18)
    W = (rng.standard_normal((k, m)) * 0.1).astype(np.float32)
    X = (rng.random((k, n)) < 0.3).astype(np.float32)
    b = rng.standard_normal((m, 1)).astype(np.float32)
    cm.set_gemm_path(path)
    cm.CUDAMatrix.init_random(99)
    oracle.EigenMatrix.init_random(99)
    w, x, bias = cm.CUDAMatrix(W), cm.CUDAMatrix(X), cm.CUDAMatrix(b)
    scale = cm.f16_scale_state(np.abs(W).max())
    w_aux = w.split_f16(cm.empty_aux(W.shape), exp_dev=scale.slice(0, 1))
    x_aux = x.split_f16(cm.empty_aux(X.shape), exp_const=14)
    out, smp = cm.empty((m, n)), cm.empty((m, n))
    out_aux, smp_aux = cm.empty_aux((m, n)), cm.empty_aux((m, n))
    cm.fused_gemm(cm.f16_passes(w.T, w_aux, x, x_aux, exact_b=True), out=out, sample=smp, out_aux=out_aux,
                  sample_aux=smp_aux, bias=bias, activation=1, scale_exp=scale.slice(0, 1), scale_exp_const=14,
                  aux_f16=True, aux_exp=14)
    got = get(out)
    assert relerr(got, 1 / (1 + np.exp(-(W.astype(np.float64).T @ X + b)))) < TOL
    lo, hi = f16_planes(out_aux)
    want_hi = (got * np.float32(16384)).astype(np.float16)
    np.testing.assert_array_equal(hi, want_hi.astype(np.float32))
    np.testing.assert_array_equal(lo, (got * np.float32(16384) - want_hi.astype(np.float32)).astype(np.float16).astype(np.float32))
    want_s = get(oracle.EigenMatrix(got).sample_bernoulli(target=oracle.empty((m, n))))
    np.testing.assert_array_equal(get(smp), want_s)
    np.testing.assert_array_equal(f16_planes(smp_aux)[1], want_s * 16384)
    assert cm.read_status() == 0


def test_momentum_update_keeps_the_scaled_half_precision_form(cm):
    rng = np.random.default_rng(19)
    shape = (256, 96)
    w0 = (rng.standard_normal(shape) * 0.01).astype(np.float32)
    w, d = cm.CUDAMatrix(w0), cm.CUDAMatrix(np.zeros(shape, np.float32))
    scale = cm.f16_scale_state(np.abs(w0).max())
    aux = w.split_f16(cm.empty_aux(shape), exp_dev=scale.slice(0, 1))
    for step in range(3):
        # the middle update multiplies the weights' magnitude by hundreds: the exponent must follow at once
        s = cm.CUDAMatrix((rng.standard_normal(shape) * (500.0 if step == 1 else 0.1)).astype(np.float32))
        w.momentum_update(d, None, s, 1.0 / 10, 0.5, 0.1, w_aux=aux, w_scale=scale)
        now = get(w)
        e = float(get(scale)[0, 0])
        # the exponent is kept while the largest scaled magnitude stays in (2^11, 2^15] and follows at
        # once when the weights leave that range (the jump of the middle update)
        top = np.abs(now).max() * 2.0 ** e
        assert 2.0 ** 11 < top <= 2.0 ** 15
        if step == 1:
            assert e == np.floor(np.log2(8192.0 / np.abs(now).max()))
        lo, hi = f16_planes(aux)
        want_hi = (now * np.float32(2.0 ** e)).astype(np.float16)
        assert np.isfinite(hi).all()
        np.testing.assert_array_equal(hi, want_hi.astype(np.float32))
        np.testing.assert_array_equal(lo, (now * np.float32(2.0 ** e) - want_hi.astype(np.float32)).astype(np.float16).astype(np.float32))


@pytest.mark.parametrize("path", [1, 2])
@pytest.mark.parametrize("m,n,k", [(500, 100, 784), (128, 256, 64), (260, 36, 40), (1024, 512, 2048)])
def test_fused_epilogue_bias_logistic_sample(cm, oracle, path, m, n, k):
    rng = np.random.default_rng(9)
    W = (rng.standard_normal((k, m)) * 0.1).astype(np.float32)
    X = (rng.random((k, n)) < 0.3).astype(np.float32)
    b = rng.standard_normal((m, 1)).astype(np.float32)
    cm.set_gemm_path(path)
    seed = 99
    cm.CUDAMatrix.init_random(seed)
    oracle.EigenMatrix.init_random(seed)
    w, x, bias = cm.CUDAMatrix(W), cm.CUDAMatrix(X), cm.CUDAMatrix(b)
    out, smp = cm.empty((m, n)), cm.empty((m, n))
    out_aux, smp_aux = cm.empty_aux((m, n)), cm.empty_aux((m, n))
    w_aux, x_aux = w.split_bf16(cm.empty_aux(W.shape)), x.split_bf16(cm.empty_aux(X.shape))
    cm.fused_gemm(cm.split_passes(w.T, x, exact_b=True, a_aux=w_aux, b_aux=x_aux), out=out, sample=smp,
                  out_aux=out_aux, sample_aux=smp_aux, bias=bias, activation=1, alpha=1.0)
    pre = W.astype(np.float64).T @ X + b
    want = 1 / (1 + np.exp(-pre))
    got = get(out)
    assert relerr(got, want) < TOL
    lo, bb = out_aux.planes()                       # the bfloat16 parts of the result
    np.testing.assert_array_equal(lo, bf16_round(got - tf32_trunc(got)))
    np.testing.assert_array_equal(bb, bf16_round(got))
    # the draw thresholds the probabilities the kernel itself produced against the shared
    # uniforms of call 0: bit-exact with the oracle fed the same probabilities
    want_s = get(oracle.EigenMatrix(got).sample_bernoulli(target=oracle.empty((m, n))))
    np.testing.assert_array_equal(get(smp), want_s)
    np.testing.assert_array_equal(smp_aux.planes()[1], want_s)
    assert cm.CUDAMatrix.rnd_state.calls == 1
    assert cm.read_status() == 0


@pytest.mark.parametrize("path", [1, 2])
@pytest.mark.parametrize("terms", ["bf16", "tf32"])
@pytest.mark.parametrize("m,n,k", [(512, 256, 4096), (500, 100, 784)])
def test_split_product_is_fp32_grade(cm, path, terms, m, n, k):
    """x.y plus its two correction terms against the float64 product of same-sign operands
    (the worst case for a truncating or biased scheme)."""
    rng = np.random.default_rng(14)
    A = rng.random((m, k)).astype(np.float32)
    B = rng.random((k, n)).astype(np.float32)
    cm.set_gemm_path(path)
    out = cm.empty((m, n))
    cm.fused_gemm(cm.split_passes(cm.CUDAMatrix(A), cm.CUDAMatrix(B), terms=terms), out=out)
    # the CUDA-core kernel adds k same-sign terms one by one in fp32; the TF32 correction terms
    # truncate x - tf32(x) to 10 bits (a one-sided error on same-sign data), the bfloat16 ones round
    tol = 3e-5 if path == 2 else (3e-6 if terms == "tf32" else 2e-6)
    assert relerr(get(out), A.astype(np.float64) @ B.astype(np.float64)) < tol


@pytest.mark.parametrize("path", [1, 2])
def test_fused_negated_passes_with_unequal_depths_and_col_scale(cm, path):
    rng = np.random.default_rng(10)
    m, n = 132, 72
    A1 = rng.standard_normal((m, 48)).astype(np.float32)
    B1 = rng.standard_normal((48, n)).astype(np.float32)
    A2 = rng.standard_normal((m, 100)).astype(np.float32)
    B2 = rng.standard_normal((100, n)).astype(np.float32)
    b = rng.standard_normal((m, 1)).astype(np.float32)
    cs = rng.random((1, n)).astype(np.float32) * 50
    old = rng.standard_normal((m, n)).astype(np.float32)
    cm.set_gemm_path(path)
    cm.set_dot_precision(1)
    out = cm.CUDAMatrix(old)
    cm.fused_gemm([(cm.CUDAMatrix(A1), cm.CUDAMatrix(B1)), (cm.CUDAMatrix(A2), cm.CUDAMatrix(B2), 1)], out=out,
                  bias=cm.CUDAMatrix(b), col_scale=cm.CUDAMatrix(cs), alpha=0.5, beta=2.0)
    # a pass multiplies its operands as TF32 on either path
    tr = lambda x: (x.view(np.uint32) & np.uint32(0xffffe000)).view(np.float32).astype(np.float64)
    want = 0.5 * (tr(A1) @ tr(B1) - tr(A2) @ tr(B2)) + 2.0 * old + b * cs
    assert relerr(get(out), want) < TOL


@pytest.mark.parametrize("shape", [(33, 17), (784, 500), (8192, 1), (1, 4)])
@pytest.mark.parametrize("with_grad", [True, False])
def test_momentum_update_is_bit_exact(cm, oracle, shape, with_grad):
    rng = np.random.default_rng(11)
    w0, d0, s0 = (rng.standard_normal(shape).astype(np.float32) for _ in range(3))
    g0 = rng.standard_normal(shape).astype(np.float32) if with_grad else np.zeros(shape, np.float32)
    args = (1.0 / 100, 0.7, 0.1)
    wo, do, go = oracle.EigenMatrix(w0), oracle.EigenMatrix(d0), oracle.EigenMatrix(g0)
    wo.momentum_update(do, go, oracle.EigenMatrix(s0), *args, l2=2e-4, l1=1e-3)
    wg, dg = cm.CUDAMatrix(w0), cm.CUDAMatrix(d0)
    gg = cm.CUDAMatrix(g0) if with_grad else None
    aux = cm.empty_aux(shape)
    wg.momentum_update(dg, gg, cm.CUDAMatrix(s0), *args, l2=2e-4, l1=1e-3, w_aux=aux)
    np.testing.assert_array_equal(get(wg), get(wo))
    np.testing.assert_array_equal(get(dg), get(do))
    if with_grad:
        assert not get(gg).any()
    lo, b = aux.planes()
    np.testing.assert_array_equal(lo, bf16_round(get(wg) - tf32_trunc(get(wg))))
    np.testing.assert_array_equal(b, bf16_round(get(wg)))


@pytest.mark.parametrize("k,form", [(8192, "f16"), (8192, "tf32"), (10000, "tf32"), (10000, "bf16")])
def test_long_same_sign_products_keep_the_bound(cm, k, form):
    """The tensor core truncates its accumulator at every MMA, so a long same-sign sum drifts; the
    kernel folds chunks of the product into fp32 registers (128 products for linear outputs, 2048
    behind a logistic).  Worst case for that rule: all-positive operands at the longest inner
    dimensions of the path (8192 hidden units, a 10 000-word vocabulary), linear and logistic."""
    rng = np.random.default_rng(k)
    m, n = 256, 512
    # weights sized so that the same-sign sum stays a few units (a logistic unit's working range: at
    # |sum| = 40 the 1e-5 absolute bound would be 2.5e-7 relative, below fp32 itself)
    A = (rng.random((k, m)) * 0.002).astype(np.float32)           # stored k x m, used transposed (the up product)
    B = rng.random((k, n)).astype(np.float32)
    b = (-(A.astype(np.float64).T @ B).mean(axis=1, keepdims=True)).astype(np.float32)   # centres the logistic
    cm.set_gemm_path(1)
    a, x, bias = cm.CUDAMatrix(A), cm.CUDAMatrix(B), cm.CUDAMatrix(b)
    lin, sig = cm.empty((m, n)), cm.empty((m, n))
    if form == "f16":
        scale = cm.f16_scale_state(np.abs(A).max())
        xa = a.split_f16(cm.empty_aux(A.shape), exp_dev=scale.slice(0, 1))
        xb = x.split_f16(cm.empty_aux(B.shape), exp_const=14)
        kw = dict(scale_exp=scale.slice(0, 1), scale_exp_const=14)
        cm.fused_gemm(cm.f16_passes(a.T, xa, x, xb), out=lin, **kw)
        cm.fused_gemm(cm.f16_passes(a.T, xa, x, xb), out=sig, bias=bias, activation=1, **kw)
    else:
        cm.fused_gemm(cm.split_passes(a.T, x, terms=form), out=lin)
        cm.fused_gemm(cm.split_passes(a.T, x, terms=form), out=sig, bias=bias, activation=1)
    pre = A.astype(np.float64).T @ B.astype(np.float64)
    assert relerr(get(lin), pre) < (4e-6 if form != "bf16" else TOL)
    assert np.abs(get(sig) - 1 / (1 + np.exp(-(pre + b)))).max() < TOL
    assert cm.read_status() == 0


@pytest.mark.parametrize("splits", [2, 5, 16])
@pytest.mark.parametrize("ta,tb", [(0, 0), (1, 0), (0, 1), (1, 1)])
@pytest.mark.parametrize("m,n,k", [(500, 100, 784), (1024, 256, 4096), (132, 68, 1000)])
def test_split_k_dot_matches_float64(cm, splits, ta, tb, m, n, k):
    """The inner dimension cut into work items (tile, split) with a finishing kernel: what fills the
    SMs when a product has few output tiles (config 1's down product is 1024 x 256 with K = 4096)."""
    rng = np.random.default_rng(m + n + k + splits)
    A = rng.standard_normal((m, k)).astype(np.float32)
    B = rng.standard_normal((k, n)).astype(np.float32)
    cm.set_gemm_path(1)
    cm.set_split_k(splits)
    try:
        out = cm.CUDAMatrix(rng.standard_normal((m, n)).astype(np.float32))
        base = get(out)
        out.add_dot(make(cm, A, ta), make(cm, B, tb), mult=0.5)          # beta = 1, alpha = 0.5 in the finishing kernel
    finally:
        cm.set_split_k(0)
    want = base + 0.5 * (A.astype(np.float64) @ B.astype(np.float64))
    assert relerr(get(out), want) < TOL
    assert cm.read_status() == 0


@pytest.mark.parametrize("splits", [1, 3, 8])
@pytest.mark.parametrize("form", ["bf16", "f16"])
def test_split_k_epilogue_equals_the_unsplit_one(cm, oracle, splits, form):
    """Bias, logistic, Bernoulli draw and the 16-bit parts of result and draw behind a split product:
    probabilities within rounding of the unsplit kernel's, the draw bit-exact against the oracle fed
    the kernel's own probabilities, the parts exactly those of the stored result."""
    rng = np.random.default_rng(40 + splits)
    m, n, k = 500, 100, 2048
    W = (rng.standard_normal((k, m)) * 0.05).astype(np.float32)
    X = (rng.random((k, n)) < 0.3).astype(np.float32)
    b = rng.standard_normal((m, 1)).astype(np.float32)
    cm.set_gemm_path(1)
    w, x, bias = cm.CUDAMatrix(W), cm.CUDAMatrix(X), cm.CUDAMatrix(b)
    out, smp = cm.empty((m, n)), cm.empty((m, n))
    out_aux, smp_aux = cm.empty_aux((m, n)), cm.empty_aux((m, n))
    if form == "f16":
        scale = cm.f16_scale_state(np.abs(W).max())
        wa = w.split_f16(cm.empty_aux(W.shape), exp_dev=scale.slice(0, 1))
        xa = x.split_f16(cm.empty_aux(X.shape), exp_const=14)
        passes = cm.f16_passes(w.T, wa, x, xa, exact_b=True)
        kw = dict(scale_exp=scale.slice(0, 1), scale_exp_const=14, aux_f16=True, aux_exp=14)
    else:
        wa, xa = w.split_bf16(cm.empty_aux(W.shape)), x.split_bf16(cm.empty_aux(X.shape))
        passes = cm.split_passes(w.T, x, exact_b=True, a_aux=wa, b_aux=xa)
        kw = {}
    cm.CUDAMatrix.init_random(5)
    oracle.EigenMatrix.init_random(5)
    cm.set_split_k(splits)
    try:
        cm.fused_gemm(passes, out=out, sample=smp, out_aux=out_aux, sample_aux=smp_aux, bias=bias, activation=1, **kw)
    finally:
        cm.set_split_k(0)
    got = get(out)
    want = 1 / (1 + np.exp(-(W.astype(np.float64).T @ X + b)))
    assert relerr(got, want) < TOL
    want_s = get(oracle.EigenMatrix(got).sample_bernoulli(target=oracle.empty((m, n))))
    np.testing.assert_array_equal(get(smp), want_s)
    if form == "f16":
        lo, hi = f16_planes(out_aux)
        want_hi = (got * np.float32(2.0 ** 14)).astype(np.float16).astype(np.float32)
        np.testing.assert_array_equal(hi, want_hi)
        np.testing.assert_array_equal(lo, (got * np.float32(2.0 ** 14) - want_hi).astype(np.float16).astype(np.float32))
        np.testing.assert_array_equal(f16_planes(smp_aux)[1], want_s * 2.0 ** 14)
    else:
        lo, bb = out_aux.planes()
        np.testing.assert_array_equal(bb, bf16_round(got))
        np.testing.assert_array_equal(lo, bf16_round(got - tf32_trunc(got)))
        np.testing.assert_array_equal(smp_aux.planes()[1], want_s)
    assert cm.read_status() == 0


@pytest.mark.parametrize("path", [1, 2])
@pytest.mark.parametrize("form", ["f16", "tf32", "bf16 aux"])
def test_row_windows_give_the_panels_of_the_full_product(cm, path, form):
    """A term may read a window of the stored rows of a (a panel of the output's rows) or of a
    transposed b (a panel of its columns): how the data-parallel step cuts its statistics product
    v h' into column panels of W without copying h.  Every panel equals the full product's."""
    rng = np.random.default_rng(50)
    M, N, K = 384, 512, 640
    A = rng.random((M, K)).astype(np.float32)                  # stored M x K: op(a) = a
    Bt = rng.random((N, K)).astype(np.float32)                 # stored N x K, used transposed: op(b) = b'
    cm.set_gemm_path(path)
    a, bt = cm.CUDAMatrix(A), cm.CUDAMatrix(Bt)
    if form == "f16":
        xa, xb = a.split_f16(cm.empty_aux(A.shape), exp_const=14), bt.split_f16(cm.empty_aux(Bt.shape), exp_const=14)
        passes = lambda **w: cm.f16_passes(a, xa, bt.T, xb, **w)
        kw = dict(scale_exp_const=28)
    elif form == "bf16 aux":
        xa, xb = a.split_bf16(cm.empty_aux(A.shape)), bt.split_bf16(cm.empty_aux(Bt.shape))
        passes = lambda **w: cm.split_passes(a, bt.T, a_aux=xa, b_aux=xb, **w)
        kw = {}
    else:
        passes = lambda **w: cm.split_passes(a, bt.T, terms="tf32", **w)
        kw = {}
    full = cm.empty((M, N))
    cm.fused_gemm(passes(), out=full, **kw)
    want = get(full)
    assert relerr(want, A.astype(np.float64) @ Bt.astype(np.float64).T) < TOL
    cols = cm.empty((M, N))
    for n0 in range(0, N, 128):                                # column panels: windows of b's stored rows
        cm.fused_gemm(passes(b_rows=(n0, 128)), out=cols.slice(n0, n0 + 128), **kw)
    np.testing.assert_array_equal(get(cols), want)
    for m0, rows in ((0, 128), (128, 256)):                    # row panels: windows of a's stored rows
        part = cm.empty((rows, N))
        cm.fused_gemm(passes(a_rows=(m0, rows)), out=part, **kw)
        np.testing.assert_array_equal(get(part), want[m0:m0 + rows])
    with pytest.raises(cm.CUDAMatException):                   # a window must start on a multiple of 8 rows
        cm.fused_gemm(passes(b_rows=(4, 128)), out=cols.slice(0, 128), **kw)
    assert cm.read_status() == 0


@pytest.mark.parametrize("mode", ["plain", "bf16", "f16"])
def test_momentum_update_by_column_panels_equals_the_whole_update(cm, mode):
    rng = np.random.default_rng(51)
    shape = (256, 96)
    w0 = (rng.standard_normal(shape) * 0.01).astype(np.float32)
    d0 = (rng.standard_normal(shape) * 0.001).astype(np.float32)
    s0 = rng.standard_normal(shape).astype(np.float32)
    out = []
    for panels in (1, 3):
        w, d, s = cm.CUDAMatrix(w0), cm.CUDAMatrix(d0), cm.CUDAMatrix(s0)
        aux = cm.empty_aux(shape) if mode != "plain" else None
        scale = cm.f16_scale_state(np.abs(w0).max()) if mode == "f16" else None
        if mode == "f16":
            w.split_f16(aux, exp_dev=scale.slice(0, 1))
        X = cm.Immediate()
        step = shape[1] // panels
        for p in range(panels):
            X.momentum_update_columns(w, d, None, s, p * step, step, 1.0 / 10, 0.5, 0.1, l2=2e-4, w_aux=aux, w_scale=scale)
        out.append((get(w), get(d), get(aux) if aux is not None else None, get(scale) if scale is not None else None))
    for a, b in zip(out[0], out[1]):
        if a is not None:
            np.testing.assert_array_equal(a, b)
