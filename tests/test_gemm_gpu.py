"""Parity of the device GEMM (through the C ABI) with the CPU oracle and with the reference's
own known answers.  Tolerances are the ones the path is specified with:
f32  |delta| <= 1e-4 * ||a_row|| * ||b_col||,  f64  <= 1e-12 of the same norm,  integers bit-exact."""
import numpy as np
import pytest
import torch

from conftest import fval

pytestmark = pytest.mark.gpu

F32_TOL, F64_TOL = 1e-4, 1e-12
DT = {"float32": np.float32, "float64": np.float64, "int32": np.int32, "int64": np.int64}


def norm_scaled_error(c, ref, a2, b2):
    """max over outputs of |c - ref| / (||a_row|| * ||b_col||); a2 is [..,M,K], b2 is [..,K,N] (logical)."""
    na = np.linalg.norm(a2.astype(np.float64), axis=-1)[..., :, None]
    nb = np.linalg.norm(b2.astype(np.float64), axis=-2)[..., None, :]
    scale = na * nb
    scale[scale == 0] = 1.0
    return float((np.abs(c.astype(np.float64) - ref.astype(np.float64)) / scale).max()) if c.size else 0.0


def dev(be, a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(be.device)


def run_gemm(be, a, b, **kw):
    out = be.gemm(dev(be, a), dev(be, b), **kw)
    be.sync()
    return out.cpu().numpy()


# ------------------------------------------------------------------ reference known answers via the Tensor mirror
def test_reference_known_answers(be, golden):
    import minitensor_b200.tensor as mt
    for case in golden["matmul"]:
        dt = case["dtype"]
        a = mt.Tensor(np.array(case["a"], dtype=DT[dt]).reshape(case["a_shape"]))
        b = mt.Tensor(np.array(case["b"], dtype=DT[dt]).reshape(case["b_shape"]))
        out = a.matmul(b) if len(case["a_shape"]) != 3 else a.bmm(b)
        assert list(out.shape) == case["out_shape"], case["source"]
        np.testing.assert_array_equal(out.numpy().ravel(), np.array(case["out"], dtype=DT[dt]), err_msg=case["source"])


def test_reference_backward_known_answers(be, golden):
    import minitensor_b200.tensor as mt
    for case in golden["matmul_backward_ones"]:
        a = mt.Tensor(np.array(case["a"], dtype=np.float32).reshape(case["a_shape"]), requires_grad=True)
        b = mt.Tensor(np.array(case["b"], dtype=np.float32).reshape(case["b_shape"]), requires_grad=True)
        a.matmul(b).sum().backward()
        np.testing.assert_array_equal(a.grad.numpy().ravel(), np.array(case["da"], dtype=np.float32))
        np.testing.assert_array_equal(b.grad.numpy().ravel(), np.array(case["db"], dtype=np.float32))


def test_reference_error_cases(be):
    """tests/ops/test_logic_broadcast_linalg.py:618-708 and engine/src/operations/linalg/triangular.rs:208-336."""
    import minitensor_b200.tensor as mt
    with pytest.raises(ValueError):
        mt.Tensor([[1.0, 2.0]]).matmul(mt.Tensor([[3.0, 4.0, 5.0]]))
    with pytest.raises(TypeError):
        mt.Tensor([[1.0, 2.0]], dtype="float32").matmul(mt.Tensor([[3.0], [4.0]], dtype="float64"))
    with pytest.raises(ValueError):
        mt.Tensor([[True, False], [False, True]], dtype="bool").matmul(
            mt.Tensor([[True, True], [False, False]], dtype="bool"))
    with pytest.raises((ValueError, RuntimeError)):
        mt.Tensor(2.0).matmul(mt.Tensor(3.0))
    with pytest.raises(ValueError):
        mt.Tensor(np.ones((2, 3), np.float32)).bmm(mt.Tensor(np.ones((2, 3, 3), np.float32)))
    a = mt.Tensor(np.arange(12, dtype=np.float32).reshape(2, 2, 3))
    b = mt.Tensor(np.arange(18, dtype=np.float32).reshape(3, 3, 2))
    with pytest.raises(ValueError):
        a.bmm(b)
    with pytest.raises(ValueError):
        a.matmul(b)


def test_requires_grad_flags_and_self_matmul(be):
    """tests/ops/test_logic_broadcast_linalg.py:741-752; tests/tensor/test_tensor_core.py:636-642."""
    import minitensor_b200.tensor as mt
    a = mt.Tensor(np.arange(4, dtype=np.float32).reshape(2, 2), requires_grad=True)
    b = mt.Tensor(np.arange(4, dtype=np.float32).reshape(2, 2), requires_grad=False)
    a.matmul(b).sum().backward()
    assert a.grad is not None and b.grad is None
    x = mt.Tensor(np.array([[1.0, 2.0], [3.0, 4.0]], np.float32), requires_grad=True)
    (x @ x).sum().backward()
    xn = x.numpy()
    ones = np.ones((2, 2), np.float32)
    np.testing.assert_allclose(x.grad.numpy(), ones @ xn.T + xn.T @ ones)


def test_batch_broadcast_and_gradient_reduction(be, orc, rng):
    """[2,3,4] @ [4,5] and [1,3,4] @ [7,4,5] (matmul.rs:324-345); gradients reduce over the broadcast dims."""
    import minitensor_b200.tensor as mt
    for sa, sb in [((2, 3, 4), (4, 5)), ((1, 3, 4), (7, 4, 5))]:
        an, bn = rng.standard_normal(sa).astype(np.float32), rng.standard_normal(sb).astype(np.float32)
        a, b = mt.Tensor(an, requires_grad=True), mt.Tensor(bn, requires_grad=True)
        c = a.matmul(b)
        ref = np.matmul(an.astype(np.float64), bn.astype(np.float64))
        np.testing.assert_allclose(c.numpy(), ref, rtol=1e-5, atol=1e-5)
        c.sum().backward()
        g = np.ones(ref.shape)
        ga = np.matmul(g, np.swapaxes(np.broadcast_to(bn, ref.shape[:-2] + bn.shape[-2:]), -1, -2))
        gb = np.matmul(np.swapaxes(np.broadcast_to(an, ref.shape[:-2] + an.shape[-2:]), -1, -2), g)
        while ga.ndim > an.ndim:
            ga = ga.sum(0)
        if an.shape[0] == 1 and ga.shape[0] != 1:
            ga = ga.sum(0, keepdims=True)
        while gb.ndim > bn.ndim:
            gb = gb.sum(0)
        np.testing.assert_allclose(a.grad.numpy(), ga, rtol=1e-5, atol=1e-4)
        np.testing.assert_allclose(b.grad.numpy(), gb, rtol=1e-5, atol=1e-4)


def test_inf_nan_propagation(be):
    """tests/ops/test_logic_broadcast_linalg.py:718-722, plus: Inf times a finite value stays Inf."""
    a = np.array([[np.inf, np.nan], [1.0, 2.0]], np.float32)
    b = np.array([[1.0, 2.0], [3.0, 4.0]], np.float32)
    out = run_gemm(be, a, b)
    assert np.isnan(out[0]).all()
    np.testing.assert_array_equal(out[1], [7.0, 10.0])
    a = np.array([[np.inf, 1.0], [-np.inf, 2.0], [3.0, 4.0]], np.float32)
    b = np.array([[1.0, -1.0, 0.0], [1.0, 1.0, 1.0]], np.float32)
    out = run_gemm(be, a, b)
    with np.errstate(invalid="ignore"):
        ref = a @ b
    np.testing.assert_array_equal(np.isnan(out), np.isnan(ref))
    np.testing.assert_array_equal(out[~np.isnan(ref)], ref[~np.isnan(ref)])
    # a later clean call is not affected by the earlier non-finite one
    c = run_gemm(be, np.ones((4, 8), np.float32), np.ones((8, 4), np.float32))
    np.testing.assert_array_equal(c, np.full((4, 4), 8.0, np.float32))


# ------------------------------------------------------------------ f32 parity with the oracle
SHAPES = [(1, 1, 1), (2, 3, 2), (7, 5, 3), (17, 63, 65), (64, 64, 64), (127, 129, 31), (128, 256, 64),
          (130, 257, 100), (256, 256, 256), (300, 1000, 777), (32, 10, 128), (32, 128, 784), (1, 513, 1030),
          (513, 1, 9), (1024, 1024, 1024)]


@pytest.mark.parametrize("m,n,k", SHAPES)
def test_f32_matches_oracle(be, orc, rng, m, n, k):
    a = rng.standard_normal((m, k)).astype(np.float32)
    b = rng.standard_normal((k, n)).astype(np.float32)
    c = run_gemm(be, a, b)
    ref = orc.matmul(a, b)                       # reference-order f32
    wide = orc.matmul_acc_wide(a, b)             # f64-accumulated
    assert norm_scaled_error(c, ref, a, b) <= F32_TOL
    assert norm_scaled_error(c, wide, a, b) <= F32_TOL
    # the default mode is f32-accurate: no worse than a small multiple of the CPU f32 kernel's own error
    assert norm_scaled_error(c, wide, a, b) <= 4e-6


@pytest.mark.parametrize("variant", [1, 2, 3, 4, 5, 6])
@pytest.mark.parametrize("mode", [3, 6, 9])
def test_f32_tile_variants_and_modes(be, orc, rng, variant, mode):
    m, n, k = 257, 300, 193
    a = rng.standard_normal((m, k)).astype(np.float32)
    b = rng.standard_normal((k, n)).astype(np.float32)
    c = run_gemm(be, a, b, f32_mode=mode, variant=variant)
    assert norm_scaled_error(c, orc.matmul_acc_wide(a, b), a, b) <= (F32_TOL if mode == 3 else 4e-6)


@pytest.mark.parametrize("ta,tb", [(False, True), (True, False), (True, True)])
def test_f32_transposed_operands(be, orc, rng, ta, tb):
    """The two products of MatMulBackward and the DenseLayer forward use these forms."""
    m, n, k = 200, 300, 150
    a = rng.standard_normal((k, m) if ta else (m, k)).astype(np.float32)
    b = rng.standard_normal((n, k) if tb else (k, n)).astype(np.float32)
    c = run_gemm(be, a, b, trans_a=ta, trans_b=tb)
    al, bl = (a.T if ta else a), (b.T if tb else b)
    assert norm_scaled_error(c, orc.matmul(np.ascontiguousarray(al), np.ascontiguousarray(bl)), al, bl) <= F32_TOL


def test_f32_backward_config1(be, orc):
    """1024^3, N(0,1) entries from seed 7, forward plus backward with an all-ones upstream gradient."""
    import minitensor_b200.tensor as mt
    g = np.random.default_rng(7)
    an = g.standard_normal((1024, 1024)).astype(np.float32)
    bn = g.standard_normal((1024, 1024)).astype(np.float32)
    a, b = mt.Tensor(an, requires_grad=True), mt.Tensor(bn, requires_grad=True)
    c = a.matmul(b)
    c.sum().backward()
    dy = np.ones((1024, 1024), np.float32)
    da, db = orc.matmul_backward(an, bn, dy)
    assert norm_scaled_error(c.numpy(), orc.matmul(an, bn), an, bn) <= F32_TOL
    assert norm_scaled_error(a.grad.numpy(), da, dy, bn.T) <= F32_TOL
    assert norm_scaled_error(b.grad.numpy(), db, an.T, dy) <= F32_TOL


def test_bmm_f32(be, orc, rng):
    a = rng.standard_normal((5, 64, 96)).astype(np.float32)
    b = rng.standard_normal((5, 96, 80)).astype(np.float32)
    c = run_gemm(be, a, b)
    assert norm_scaled_error(c, orc.matmul(a, b), a, b) <= F32_TOL
    a = rng.standard_normal((64, 128, 128)).astype(np.float32)
    b = rng.standard_normal((64, 128, 128)).astype(np.float32)
    assert norm_scaled_error(run_gemm(be, a, b), orc.matmul(a, b), a, b) <= F32_TOL


def test_bmm_f32_config_size(be, orc):
    """bmm [64,512,512] x [64,512,512] at size: in EVERY batch entry, sampled rows against the oracle in the
    reference's order (1e-4) and against the f64-accumulated oracle (4e-6), through the Tensor mirror's bmm."""
    import minitensor_b200.tensor as mt
    g = np.random.default_rng(7)
    a = g.standard_normal((64, 512, 512)).astype(np.float32)
    b = g.standard_normal((64, 512, 512)).astype(np.float32)
    c = mt.Tensor(a).bmm(mt.Tensor(b)).numpy()
    assert c.shape == (64, 512, 512)
    pick = np.random.default_rng(8)
    for i in range(64):
        rows = np.sort(pick.choice(512, 6, replace=False))
        ar = np.ascontiguousarray(a[i][rows])
        assert norm_scaled_error(c[i][rows], orc.matmul(ar, b[i]), ar, b[i]) <= F32_TOL, i
        assert norm_scaled_error(c[i][rows], orc.matmul_acc_wide(ar, b[i]), ar, b[i]) <= 4e-6, i


def test_fused_epilogues_match_unfused_oracle(be, orc, rng):
    m, n, k = 100, 200, 300
    x = rng.standard_normal((m, k)).astype(np.float32)
    w = rng.standard_normal((n, k)).astype(np.float32)
    bias = rng.standard_normal(n).astype(np.float32)
    z = orc.dense_forward(x, w, bias)
    y = run_gemm(be, x, w, trans_b=True, bias=dev(be, bias))
    assert norm_scaled_error(y, z, x, w.T) <= F32_TOL
    relu_ref, mask = orc.relu(z)
    y = run_gemm(be, x, w, trans_b=True, bias=dev(be, bias), epilogue=1)
    assert norm_scaled_error(y, relu_ref, x, w.T) <= F32_TOL
    for epi, approx in ((2, False), (3, True)):
        y = run_gemm(be, x, w, trans_b=True, bias=dev(be, bias), epilogue=epi)
        assert norm_scaled_error(y, orc.gelu(z, approx), x, w.T) <= F32_TOL
    # ReluBackward fused: (dy @ w2) * (h > 0)
    h = relu_ref
    dy = rng.standard_normal((m, 50)).astype(np.float32)
    w2 = rng.standard_normal((50, n)).astype(np.float32)
    got = run_gemm(be, dy, w2, epilogue=4, aux=dev(be, h))
    exp = orc.relu_backward(mask, orc.matmul(dy, w2))
    assert norm_scaled_error(got, exp, dy, w2) <= F32_TOL


def test_zero_sized_and_degenerate(be):
    for (m, n, k) in [(0, 3, 4), (3, 0, 4), (2, 3, 0)]:
        c = run_gemm(be, np.zeros((m, k), np.float32), np.zeros((k, n), np.float32))
        assert c.shape == (m, n) and not c.any()
    # K == 0 with a fused bias + relu yields relu(bias) in every row
    bias = np.array([-1.0, 2.0, 0.5], np.float32)
    c = run_gemm(be, np.zeros((2, 0), np.float32), np.zeros((0, 3), np.float32), bias=dev(be, bias), epilogue=1)
    np.testing.assert_array_equal(c, np.tile(np.maximum(bias, 0), (2, 1)))


def test_deterministic(be, rng):
    a = dev(be, rng.standard_normal((300, 500)).astype(np.float32))
    b = dev(be, rng.standard_normal((500, 260)).astype(np.float32))
    c1 = be.gemm(a, b).clone()
    c2 = be.gemm(a, b)
    be.sync()
    assert torch.equal(c1, c2)


# ------------------------------------------------------------------ f64 / integers
@pytest.mark.parametrize("m,n,k", [(2, 2, 3), (17, 63, 65), (128, 128, 16), (130, 70, 33), (256, 256, 256),
                                   (300, 200, 1000), (1024, 1024, 1024)])
def test_f64_matches_oracle(be, orc, rng, m, n, k):
    a = rng.standard_normal((m, k))
    b = rng.standard_normal((k, n))
    c = run_gemm(be, a, b)
    assert norm_scaled_error(c, orc.matmul(a, b), a, b) <= F64_TOL
    assert norm_scaled_error(c, orc.matmul_acc_wide(a, b), a, b) <= F64_TOL


@pytest.mark.parametrize("ta,tb", [(False, True), (True, False), (True, True)])
def test_f64_transposed_and_batched(be, orc, rng, ta, tb):
    m, n, k = 100, 90, 80
    a = rng.standard_normal((3, k, m) if ta else (3, m, k))
    b = rng.standard_normal((3, n, k) if tb else (3, k, n))
    c = run_gemm(be, a, b, trans_a=ta, trans_b=tb)
    al = np.ascontiguousarray(np.swapaxes(a, -1, -2) if ta else a)
    bl = np.ascontiguousarray(np.swapaxes(b, -1, -2) if tb else b)
    assert norm_scaled_error(c, orc.matmul(al, bl), al, bl) <= F64_TOL


@pytest.mark.parametrize("dtype", [np.int32, np.int64])
@pytest.mark.parametrize("m,n,k", [(2, 2, 3), (17, 63, 65), (130, 70, 33), (256, 256, 256), (1024, 1024, 1024)])
def test_int_bit_exact(be, orc, rng, dtype, m, n, k):
    a = rng.integers(-8, 9, (m, k)).astype(dtype)
    b = rng.integers(-8, 9, (k, n)).astype(dtype)
    np.testing.assert_array_equal(run_gemm(be, a, b), orc.matmul(a, b))


@pytest.mark.parametrize("dtype", [np.int32, np.int64])
def test_int_wraps_like_release_build(be, orc, rng, dtype):
    info = np.iinfo(dtype)
    a = rng.integers(info.min, info.max, (65, 70), dtype=dtype)
    b = rng.integers(info.min, info.max, (70, 33), dtype=dtype)
    np.testing.assert_array_equal(run_gemm(be, a, b), orc.matmul(a, b))
    a3 = rng.integers(-8, 9, (3, 20, 30)).astype(dtype)
    b3 = rng.integers(-8, 9, (3, 30, 10)).astype(dtype)
    np.testing.assert_array_equal(run_gemm(be, a3, b3), orc.matmul(a3, b3))


# ------------------------------------------------------------------ full-size properties
def test_large_f32_sampled_rows_and_linearity(be, orc):
    """4096^3 (the headline size): sampled rows against the f64-accumulated oracle, plus linearity
    C(A, B1 + B2) = C(A, B1) + C(A, B2) within the same tolerance."""
    g = torch.Generator(device="cpu").manual_seed(11)
    n = 4096
    a = torch.randn(n, n, generator=g)
    b = torch.randn(n, n, generator=g)
    ad, bd = a.to(be.device), b.to(be.device)
    c = be.gemm(ad, bd)
    be.sync()
    rows = np.random.default_rng(5).choice(n, 24, replace=False)
    an, bn = a.numpy(), b.numpy()
    wide = orc.matmul_acc_wide(np.ascontiguousarray(an[rows]), bn)
    assert norm_scaled_error(c[rows].cpu().numpy(), wide, an[rows], bn) <= F32_TOL
    b2 = torch.randn(n, n, generator=g).to(be.device)
    lhs = be.gemm(ad, bd + b2)
    rhs = c + be.gemm(ad, b2)
    be.sync()
    scale = (ad.double().norm(dim=1)[:, None] * (bd + b2).double().norm(dim=0)[None, :])
    assert float(((lhs - rhs).double().abs() / scale).max()) <= F32_TOL


def test_large_int_modular_identity(be, orc):
    """i32 4096^3, entries in [-8,8]: sum_j C[i,j] r[j] == sum_l A[i,l] (B r)[l], exact in wrapping arithmetic."""
    n = 4096
    g = torch.Generator(device="cpu").manual_seed(3)
    a = torch.randint(-8, 9, (n, n), generator=g, dtype=torch.int32).to(be.device)
    b = torch.randint(-8, 9, (n, n), generator=g, dtype=torch.int32).to(be.device)
    r = torch.randint(-3, 4, (n, 1), generator=g, dtype=torch.int32).to(be.device)
    c = be.gemm(a, b)
    lhs = be.gemm(c, r)
    rhs = be.gemm(a, be.gemm(b, r))
    be.sync()
    assert torch.equal(lhs, rhs)
    assert int(c.abs().max()) <= 64 * n  # |sum| <= 8*8*K: no overflow at these magnitudes
    # sampled rows, every column, against the reference's triple loop
    rows = np.random.default_rng(4).choice(n, 12, replace=False)
    np.testing.assert_array_equal(c[rows].cpu().numpy(),
                                  orc.matmul(np.ascontiguousarray(a[rows].cpu().numpy()), b.cpu().numpy()))


# ------------------------------------------------------------------ fp16 two-plane mode (the default for large outputs)
@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("mode", [23, 6])
def test_f16x3_and_bf16x6_agree_with_oracle_all_orientations(be, orc, rng, ta, tb, mode):
    m, n, k = 300, 520, 777
    a = rng.standard_normal((k, m) if ta else (m, k)).astype(np.float32)
    b = rng.standard_normal((n, k) if tb else (k, n)).astype(np.float32)
    c = run_gemm(be, a, b, trans_a=ta, trans_b=tb, f32_mode=mode)
    al = np.ascontiguousarray(a.T if ta else a)
    bl = np.ascontiguousarray(b.T if tb else b)
    assert norm_scaled_error(c, orc.matmul_acc_wide(al, bl), al, bl) <= 4e-6
    assert norm_scaled_error(c, orc.matmul(al, bl), al, bl) <= F32_TOL


def test_f16x3_row_and_column_scaling_covers_the_f32_range(be, orc, rng):
    """Rows of A and columns of B spanning 2^-60 .. 2^60, and a row of subnormals: the per-row / per-column
    power-of-two scaling keeps every output within the norm-scaled tolerance."""
    m, n, k = 260, 300, 512
    a = rng.standard_normal((m, k)).astype(np.float32) * np.exp2(rng.integers(-60, 60, (m, 1))).astype(np.float32)
    b = rng.standard_normal((k, n)).astype(np.float32) * np.exp2(rng.integers(-60, 60, (1, n))).astype(np.float32)
    a[3] = np.float32(1e-41)            # subnormal row
    a[5] = 0.0                          # zero row
    b[:, 7] = 0.0
    wide = orc.matmul_acc_wide(a, b)
    keep = np.arange(m) != 3
    for mode in (0, 23):
        c = run_gemm(be, a, b, f32_mode=mode)
        assert np.isfinite(c).all()
        assert norm_scaled_error(c[keep], wide[keep], a[keep], b) <= 4e-6
        assert not c[5].any() and not c[:, 7].any()
        # the subnormal row: products with small columns fall below the smallest f32 subnormal, so allow
        # one subnormal step (2^-149) on top of the norm-scaled bound
        scale3 = np.linalg.norm(a[3].astype(np.float64)) * np.linalg.norm(b.astype(np.float64), axis=0)
        assert np.all(np.abs(c[3].astype(np.float64) - wide[3]) <= 4e-6 * scale3 + 2.0 ** -149)
    # wide range INSIDE a row: small elements lose at most 2^-39 of the row maximum
    a2 = rng.standard_normal((m, k)).astype(np.float32) * np.exp2(rng.integers(-20, 20, (m, k))).astype(np.float32)
    c = run_gemm(be, a2, b, f32_mode=23)
    assert norm_scaled_error(c, orc.matmul_acc_wide(a2, b), a2, b) <= 4e-6


def test_f16x3_batched_and_epilogue(be, orc, rng):
    a = rng.standard_normal((3, 200, 150)).astype(np.float32)
    b = rng.standard_normal((3, 150, 300)).astype(np.float32)
    c = run_gemm(be, a, b, f32_mode=23)
    assert norm_scaled_error(c, orc.matmul(a, b), a, b) <= F32_TOL
    w = rng.standard_normal((150, 300)).astype(np.float32)          # one B broadcast over the batch
    c = run_gemm(be, a, w, f32_mode=23)
    assert norm_scaled_error(c, orc.matmul(a, np.broadcast_to(w, (3, 150, 300)).copy()), a, w) <= F32_TOL
    x = rng.standard_normal((260, 300)).astype(np.float32)
    wt = rng.standard_normal((200, 300)).astype(np.float32)
    bias = rng.standard_normal(200).astype(np.float32)
    y = run_gemm(be, x, wt, trans_b=True, bias=dev(be, bias), epilogue=1, f32_mode=23)
    ref, _ = orc.relu(orc.dense_forward(x, wt, bias))
    assert norm_scaled_error(y, ref, x, wt.T) <= F32_TOL
    with pytest.raises(ValueError):                                  # the mode needs the pair-tile kernel
        run_gemm(be, x[:64], wt, trans_b=True, f32_mode=23)


# ------------------------------------------------------------------ int32 on the integer tensor cores (byte limbs)
@pytest.mark.parametrize("m,n,k", [(1, 1, 1), (130, 70, 33), (128, 128, 64), (300, 260, 1000), (64, 200, 9000)])
@pytest.mark.parametrize("full_range", [False, True])
def test_i32_limb_path_bit_exact(be, orc, rng, m, n, k, full_range):
    """The tensor-core limb kernel (forced with variant byte 0xfd) and the CUDA-core kernel (0xfe) both equal the
    reference's wrapping triple loop, for small entries (one signed-byte product) and for the full int32 range
    (ten unsigned limb products, reductions longer than 8192 chained)."""
    info = np.iinfo(np.int32)
    lo, hi = (info.min, info.max) if full_range else (-8, 9)
    a = rng.integers(lo, hi, (m, k), dtype=np.int64).astype(np.int32)
    b = rng.integers(lo, hi, (k, n), dtype=np.int64).astype(np.int32)
    ref = orc.matmul(a, b)
    np.testing.assert_array_equal(run_gemm(be, a, b, variant=0xFD), ref)
    np.testing.assert_array_equal(run_gemm(be, a, b, variant=0xFE), ref)


def test_i32_limb_path_transposed_batched_and_mixed_range(be, orc, rng):
    a = rng.integers(-2 ** 31, 2 ** 31, (3, 80, 65), dtype=np.int64).astype(np.int32)     # [b][K][M]
    b = rng.integers(-8, 9, (3, 90, 80), dtype=np.int64).astype(np.int32)                 # [b][N][K]: small, A is wide
    got = run_gemm(be, a, b, trans_a=True, trans_b=True, variant=0xFD)
    ref = orc.matmul(np.ascontiguousarray(np.swapaxes(a, -1, -2)), np.ascontiguousarray(np.swapaxes(b, -1, -2)))
    np.testing.assert_array_equal(got, ref)
    # a wide call followed by a narrow one: the per-call range flag does not leak
    s1 = rng.integers(-8, 9, (140, 70), dtype=np.int64).astype(np.int32)
    s2 = rng.integers(-8, 9, (70, 150), dtype=np.int64).astype(np.int32)
    np.testing.assert_array_equal(run_gemm(be, s1, s2, variant=0xFD), s1 @ s2)
    # boundary of the signed-byte range
    e1 = np.full((130, 64), -128, np.int32)
    e2 = np.full((64, 130), 127, np.int32)
    np.testing.assert_array_equal(run_gemm(be, e1, e2, variant=0xFD), e1 @ e2)
    e1[0, 0] = 128
    np.testing.assert_array_equal(run_gemm(be, e1, e2, variant=0xFD), e1 @ e2)


def test_largest_square_sizes_f32_f64_i32(be, orc):
    """8192^3, the largest square of the sweep: f32 sampled rows against the f64-accumulated oracle; i32 with the
    modular identity sum_j C[i,j] r[j] = sum_l A[i,l] (B r)[l]; f64 (at 4096^3) sampled rows against the oracle."""
    g = torch.Generator(device="cpu").manual_seed(23)
    n = 8192
    a = torch.randn(n, n, generator=g)
    b = torch.randn(n, n, generator=g)
    c = be.gemm(a.to(be.device), b.to(be.device))
    be.sync()
    rows = np.random.default_rng(6).choice(n, 8, replace=False)
    an, bn = a.numpy(), b.numpy()
    wide = orc.matmul_acc_wide(np.ascontiguousarray(an[rows]), bn)
    assert norm_scaled_error(c[rows].cpu().numpy(), wide, an[rows], bn) <= 4e-6
    del c
    ai = torch.randint(-8, 9, (n, n), generator=g, dtype=torch.int32).to(be.device)
    bi = torch.randint(-8, 9, (n, n), generator=g, dtype=torch.int32).to(be.device)
    r = torch.randint(-3, 4, (n, 1), generator=g, dtype=torch.int32).to(be.device)
    ci = be.gemm(ai, bi)
    assert torch.equal(be.gemm(ci, r), be.gemm(ai, be.gemm(bi, r)))
    rows_i = rows[:4]
    np.testing.assert_array_equal(ci[rows_i].cpu().numpy(),
                                  orc.matmul(np.ascontiguousarray(ai[rows_i].cpu().numpy()), bi.cpu().numpy()))
    del ai, bi, ci
    m = 4096
    a64 = torch.randn(m, m, generator=g, dtype=torch.float64)
    b64 = torch.randn(m, m, generator=g, dtype=torch.float64)
    c64 = be.gemm(a64.to(be.device), b64.to(be.device))
    be.sync()
    rows64 = rows[:6] % m
    ref = orc.matmul(np.ascontiguousarray(a64.numpy()[rows64]), b64.numpy())
    assert norm_scaled_error(c64[rows64].cpu().numpy(), ref, a64.numpy()[rows64], b64.numpy()) <= 1e-13


def test_f64_8192_sampled_rows(be, orc):
    """f64 8192^3, the largest f64 square of the sweep: sampled rows against the oracle in the reference's order
    and against the extended-precision (long double) accumulation, both at the f64 tolerance."""
    g = torch.Generator(device="cpu").manual_seed(29)
    n = 8192
    a = torch.randn(n, n, generator=g, dtype=torch.float64)
    b = torch.randn(n, n, generator=g, dtype=torch.float64)
    c = be.gemm(a.to(be.device), b.to(be.device))
    be.sync()
    rows = np.random.default_rng(9).choice(n, 6, replace=False)
    an, bn = a.numpy(), b.numpy()
    ar = np.ascontiguousarray(an[rows])
    got = c[rows].cpu().numpy()
    assert norm_scaled_error(got, orc.matmul(ar, bn), ar, bn) <= F64_TOL
    assert norm_scaled_error(got, orc.matmul_acc_wide(ar, bn), ar, bn) <= 1e-13


# ------------------------------------------------------------------ tail splitting (a short last round cut into K ranges)
@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)])
def test_tail_split_tiles_match_oracle(be, orc, rng, ta, tb):
    """77 pair tiles on 74 SM pairs: the last three tiles are computed as four K ranges each and finished by the
    fix-up kernel (sum in range order, scaling, bias, activation).  Sampled rows - the tail tiles' among them -
    against the f64-accumulated oracle, with every epilogue the fix-up implements."""
    m, n, k = 2816 - 5, 1792 - 3, 2100
    a = rng.standard_normal((k, m) if ta else (m, k)).astype(np.float32)
    b = rng.standard_normal((n, k) if tb else (k, n)).astype(np.float32)
    al = np.ascontiguousarray(a.T if ta else a)
    bl = np.ascontiguousarray(b.T if tb else b)
    rows = np.unique(np.concatenate([np.arange(0, m, 61), np.arange(2048, m, 23)]))
    wide = orc.matmul_acc_wide(np.ascontiguousarray(al[rows]), bl)
    ad, bd = dev(be, a), dev(be, b)
    c = be.gemm(ad, bd, trans_a=ta, trans_b=tb)
    be.sync()
    assert norm_scaled_error(c[rows].cpu().numpy(), wide, al[rows], bl) <= 4e-6
    if not (ta or tb):
        bias = rng.standard_normal(n).astype(np.float32)
        aux = rng.standard_normal((m, n)).astype(np.float32)
        y = be.gemm(ad, bd, bias=dev(be, bias), epilogue=1)
        z = be.gemm(ad, bd, epilogue=4, aux=dev(be, aux))
        w6 = be.gemm(ad, bd, f32_mode=6)                      # the bf16 six-product mode splits its tail too
        be.sync()
        assert norm_scaled_error(y[rows].cpu().numpy(), np.maximum(wide + bias, 0.0), al[rows], bl) <= 4e-6
        assert norm_scaled_error(z[rows].cpu().numpy(), wide * (aux[rows] > 0), al[rows], bl) <= 4e-6
        assert norm_scaled_error(w6[rows].cpu().numpy(), wide, al[rows], bl) <= 4e-6
        c2 = be.gemm(ad, bd)
        be.sync()
        assert torch.equal(c, c2)                             # fixed summation order: bit-identical repeats


def test_tail_split_batched(be, orc, rng):
    """5 x (1024 x 1024) = 80 pair tiles: six tail tiles, some of them in the last batch entry."""
    a = rng.standard_normal((5, 1024, 2048)).astype(np.float32)
    b = rng.standard_normal((5, 2048, 1024)).astype(np.float32)
    c = run_gemm(be, a, b)
    rows = np.arange(0, 1024, 37)
    for i in (0, 3, 4):
        wide = orc.matmul_acc_wide(np.ascontiguousarray(a[i][rows]), b[i])
        assert norm_scaled_error(c[i][rows], wide, a[i][rows], b[i]) <= 4e-6


def test_gemm_sm_limit_changes_nothing_but_the_grid(be, rng):
    """Fewer SMs for the persistent kernel (room for a collective beside it).  This shape has too few K blocks for
    any tile to be cut into K ranges, so the result does not depend on the grid at all: same bits for every limit."""
    a = dev(be, rng.standard_normal((1500, 700)).astype(np.float32))
    b = dev(be, rng.standard_normal((700, 2100)).astype(np.float32))
    ref = be.gemm(a, b)
    try:
        for sms in (140, 64, 3, 2):
            be.set_gemm_sm_limit(sms)
            assert torch.equal(be.gemm(a, b), ref)
    finally:
        be.set_gemm_sm_limit(0)
    be.sync()
    with pytest.raises(ValueError):
        be.set_gemm_sm_limit(-1)


def test_dependent_launch_changes_no_bit(be, rng, monkeypatch):
    """The kernels of a call are launched with programmatic stream serialization and wait for their predecessors
    inside the kernel; a handle created with MTB200_NO_PDL=1 launches them the plain way.  Same bits either way, for
    the one-launch preparation + one-CTA kernel (small), the pair-tile kernel with cut tail tiles and fix-up (mid)
    and an Inf operand that takes the gated redo."""
    from minitensor_b200.backend import Backend
    monkeypatch.setenv("MTB200_NO_PDL", "1")
    plain = Backend(be.device.index or 0)
    monkeypatch.delenv("MTB200_NO_PDL")
    try:
        for (m, k, n) in ((512, 512, 512), (768, 1024, 640), (1024, 1024, 1024), (2048, 512, 2304)):
            a = dev(be, rng.standard_normal((m, k)).astype(np.float32))
            b = dev(be, rng.standard_normal((k, n)).astype(np.float32))
            for _ in range(3):                       # back to back: every kernel's set-up overlaps a predecessor's tail
                got = be.gemm(a, b)
            ref = plain.gemm(a, b)
            be.sync(); plain.sync()
            assert torch.equal(got, ref), (m, k, n)
        a[3, 5] = float("inf")
        got, ref = be.gemm(a, b), plain.gemm(a, b)
        be.sync(); plain.sync()
        assert torch.equal(torch.nan_to_num(got, nan=7.0), torch.nan_to_num(ref, nan=7.0))
        assert bool(torch.isinf(got[3]).all())
    finally:
        plain.close()


def test_plain_gemm_replays_from_a_cuda_graph(be, rng):
    """A mid-size f32 product (operands prepared on two streams, tail tiles cut, fix-up kernel) recorded into a
    CUDA graph after one eager call and replayed on new operand contents: same bits as the eager call."""
    a = dev(be, rng.standard_normal((768, 1024)).astype(np.float32))
    b = dev(be, rng.standard_normal((1024, 640)).astype(np.float32))
    out = torch.empty(768, 640, device=be.device)
    be.gemm(a, b, out=out)                       # sizes the scratch memory: nothing may allocate while capturing
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        be.gemm(a, b, out=out)
    a2 = dev(be, rng.standard_normal((768, 1024)).astype(np.float32))
    b2 = dev(be, rng.standard_normal((1024, 640)).astype(np.float32))
    ref = be.gemm(a2, b2)
    a.copy_(a2)
    b.copy_(b2)
    out.zero_()
    graph.replay()
    torch.cuda.synchronize()
    be.sync()
    assert torch.equal(out, ref)


def test_nonfinite_redo_decides_afresh_on_every_graph_replay(be, rng):
    """The Inf / NaN redo is gated by a per-call flag that the call itself clears, sets and tests on the stream, so
    a captured product takes the decision on every replay: finite -> Inf in an operand -> finite again gives,
    each time, the bits of the eager call on the same contents (the reference's Inf where Inf meets finite values)."""
    m, n, k = 384, 512, 256
    a = dev(be, rng.standard_normal((m, k)).astype(np.float32))
    b = dev(be, rng.standard_normal((k, n)).astype(np.float32))
    out = torch.empty(m, n, device=be.device)
    be.gemm(a, b, out=out)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        be.gemm(a, b, out=out)
    for _ in range(70):                                    # more eager calls than there are flag slots
        be.gemm(a[:130], b)
    finite_a = a.clone()
    inf_a = a.clone()
    inf_a[5, 7] = float("inf")
    inf_a[9, 1] = float("-inf")
    for contents in (finite_a, inf_a, finite_a, inf_a):
        a.copy_(contents)
        out.zero_()
        graph.replay()
        torch.cuda.synchronize()
        ref = be.gemm(contents.clone(), b)
        be.sync()
        assert torch.equal(torch.isnan(out), torch.isnan(ref))
        assert torch.equal(out[~torch.isnan(ref)], ref[~torch.isnan(ref)])
        if contents is inf_a:
            assert torch.isinf(out[5]).all() and torch.isinf(out[9]).all() and not torch.isnan(out).any()
            assert torch.isfinite(out[6]).all()
