"""The CPU oracle against the known answers of the reference's own tests, and against
NumPy on small random inputs (how the reference's Python tests check the same ops)."""
import math

import numpy as np
import pytest

from conftest import fval

DT = {"float32": np.float32, "float64": np.float64, "int32": np.int32, "int64": np.int64}


def _mm_any_rank(orc, a, b):
    """The 1-D promotion of matmul (matmul.rs:282-308) around the oracle's core."""
    a1, b1 = a.ndim == 1, b.ndim == 1
    a2 = a.reshape(1, -1) if a1 else a
    b2 = b.reshape(-1, 1) if b1 else b
    out = orc.matmul(a2, b2)
    dims = list(out.shape)
    if b1:
        dims.pop(len(dims) - 1)
    if a1:
        dims.pop(len(dims) - 1 if b1 else len(dims) - 2)
    return out.reshape(dims)


def test_matmul_known_answers(orc, golden):
    for case in golden["matmul"]:
        dt = DT[case["dtype"]]
        a = np.array(case["a"], dtype=dt).reshape(case["a_shape"])
        b = np.array(case["b"], dtype=dt).reshape(case["b_shape"])
        out = _mm_any_rank(orc, a, b)
        assert list(out.shape) == case["out_shape"], case["source"]
        np.testing.assert_array_equal(out.ravel(), np.array(case["out"], dtype=dt), err_msg=case["source"])


def test_matmul_backward_known_answers(orc, golden):
    for case in golden["matmul_backward_ones"]:
        a = np.array(case["a"], dtype=np.float32).reshape(case["a_shape"])
        b = np.array(case["b"], dtype=np.float32).reshape(case["b_shape"])
        dy = np.ones(a.shape[:-1] + (b.shape[-1],), dtype=np.float32)
        da, db = orc.matmul_backward(a, b, dy)
        np.testing.assert_array_equal(da.ravel(), np.array(case["da"], dtype=np.float32), err_msg=case["source"])
        np.testing.assert_array_equal(db.ravel(), np.array(case["db"], dtype=np.float32), err_msg=case["source"])
        da_only, none = orc.matmul_backward(a, b, dy, need_b=False)  # requires_grad flags (tests.rs:456-495)
        assert none is None and da_only is not None


def test_conv2d_known_answers(orc, golden):
    for case in golden["conv2d"]:
        x = np.array(case["x"], dtype=np.float32).reshape(case["x_shape"])
        w = np.array(case["w"], dtype=np.float32).reshape(case["w_shape"])
        bias = None if case["bias"] is None else np.array(case["bias"], dtype=np.float32)
        y = orc.conv2d(x, w, bias, tuple(case["stride"]), tuple(case["padding"]))
        assert list(y.shape) == case["out_shape"], case["source"]
        np.testing.assert_array_equal(y.ravel(), np.array(case["out"], dtype=np.float32), err_msg=case["source"])
    for case in golden["conv2d_invalid"]:
        with pytest.raises(ValueError):
            orc.conv2d(np.zeros(case["x_shape"], np.float32), np.zeros(case["w_shape"], np.float32), None,
                       tuple(case["stride"]), tuple(case["padding"]))


def test_adam_known_answer(orc, golden):
    for case in golden["adam"]:
        p = np.array(case["param"], dtype=np.float32)
        g = np.array(case["grad"], dtype=np.float32)
        m, v = np.zeros_like(p), np.zeros_like(p)
        orc.adam_step(p, g, m, v, case["lr"], case["beta1"], case["beta2"], case["eps"], step=1)
        assert np.all(np.abs(p - case["expected"]) < case["atol"]), case["source"]


def test_relu_backward_nan(orc, golden):
    for case in golden["relu_backward"]:
        x = np.array([fval(v) for v in case["x"]], dtype=np.float32)
        go = np.array([fval(v) for v in case["grad_out"]], dtype=np.float32)
        y, mask = orc.relu(x)
        gi = orc.relu_backward(mask, go)
        exp = np.array([fval(v) for v in case["grad_in"]], dtype=np.float32)
        np.testing.assert_array_equal(np.isnan(gi), np.isnan(exp))
        np.testing.assert_array_equal(gi[~np.isnan(exp)], exp[~np.isnan(exp)])
        assert np.isnan(y[1]) and y[0] == 0.0 and y[2] == 1.0  # NaN passes through relu


def test_cross_entropy_limits(orc, golden):
    for case in golden["cross_entropy_limits"]:
        loss, _ = orc.cross_entropy(np.array(case["logits"], np.float32), np.array(case["label"]))
        assert math.isinf(loss) and loss > 0, case["source"]
    # a masked NON-target entry gives NaN (-inf * 0), the reference's quirk (regression.rs:205-210)
    loss, _ = orc.cross_entropy(np.array([[1000.0, -1000.0]], np.float32), np.array([0]))
    assert math.isnan(loss)
    with pytest.raises(IndexError):
        orc.cross_entropy(np.zeros((2, 3), np.float32), np.array([0, 3]))


def test_gelu_formulas(orc, golden):
    for case in golden["gelu"]:
        x = np.array(case["x"], dtype=np.float32)
        approx = case["approximate"] == "tanh"
        y = orc.gelu(x, approx)
        g = orc.gelu_backward(x, np.ones_like(x), approx)
        if approx:
            k = np.sqrt(np.array(2.0 / np.pi, dtype=x.dtype))
            inner = k * (x + 0.044715 * x ** 3)
            exp = 0.5 * x * (1.0 + np.tanh(inner))
            th = np.tanh(inner)
            expg = 0.5 * (1.0 + th) + 0.5 * x * (1.0 - th ** 2) * k * (1.0 + 3.0 * 0.044715 * x ** 2)
        else:
            erfv = np.array([math.erf(float(v)) for v in (x / np.sqrt(np.float32(2.0)))], dtype=x.dtype)
            exp = 0.5 * x * (1.0 + erfv)
            expg = 0.5 * (1.0 + erfv) + x * np.exp(-0.5 * x ** 2) / np.sqrt(np.float32(2.0 * np.pi))
        np.testing.assert_allclose(y, exp, rtol=case["rtol"], atol=max(case["atol"], 1e-7), err_msg=case["source"])
        np.testing.assert_allclose(g, expg, rtol=case["rtol"], atol=max(case["atol"], 1e-7), err_msg=case["source"])


@pytest.mark.parametrize("dtype", [np.float32, np.float64, np.int32, np.int64])
def test_matmul_vs_numpy_small(orc, rng, dtype):
    for (bsz, m, k, n) in [(1, 5, 4, 3), (3, 7, 9, 2), (1, 1, 1, 1), (2, 33, 300, 17)]:
        if np.issubdtype(dtype, np.integer):
            a = rng.integers(-8, 9, (bsz, m, k)).astype(dtype)
            b = rng.integers(-8, 9, (bsz, k, n)).astype(dtype)
            np.testing.assert_array_equal(orc.matmul(a, b), np.matmul(a, b))
        else:
            a = rng.standard_normal((bsz, m, k)).astype(dtype)
            b = rng.standard_normal((bsz, k, n)).astype(dtype)
            ref = np.matmul(a.astype(np.float64), b.astype(np.float64))
            np.testing.assert_allclose(orc.matmul(a, b), ref, rtol=1e-4 if dtype == np.float32 else 1e-12,
                                       atol=1e-4 if dtype == np.float32 else 1e-12)


def test_int_matmul_wraps(orc):
    a = np.full((1, 2), 2 ** 30, dtype=np.int32)
    b = np.full((2, 1), 4, dtype=np.int32)
    assert orc.matmul(a, b)[0, 0] == 0  # 2 * 2^32 mod 2^32
    a64 = np.full((1, 2), 2 ** 62, dtype=np.int64)
    b64 = np.full((2, 1), 4, dtype=np.int64)
    assert orc.matmul(a64, b64)[0, 0] == 0


def test_conv_backward_finite_difference(orc, rng):
    """The reference checks conv gradients by finite differences (tests/nn/test_layers.py:160-204)."""
    for stride, padding in [((1, 1), (0, 0)), ((2, 2), (1, 1)), ((1, 2), (2, 1))]:
        x = rng.standard_normal((2, 2, 5, 6)).astype(np.float32)
        w = rng.standard_normal((3, 2, 3, 2)).astype(np.float32)
        b = rng.standard_normal(3).astype(np.float32)
        y = orc.conv2d(x, w, b, stride, padding)
        go = rng.standard_normal(y.shape).astype(np.float32)
        gx, gw, gb = orc.conv2d_backward(x, w, go, stride, padding)
        f = lambda xx, ww, bb: float((orc.conv2d(xx, ww, bb, stride, padding).astype(np.float64) * go).sum())
        eps = 1e-2
        for arr, grad in ((x, gx), (w, gw), (b, gb)):
            for idx in [tuple(rng.integers(0, s) for s in arr.shape) for _ in range(4)]:
                old = arr[idx]
                arr[idx] = old + eps
                fp = f(x, w, b)
                arr[idx] = old - eps
                fm = f(x, w, b)
                arr[idx] = old
                num = (fp - fm) / (2 * eps)
                assert abs(num - grad[idx]) <= 1e-2 * max(1.0, abs(num))


def test_mlp_step_matches_composition(orc, rng):
    """orc.mlp_train_step equals the composition of the single-op oracles."""
    dims = [6, 5, 4]
    bsz = 7
    x = rng.standard_normal((bsz, dims[0])).astype(np.float32)
    lab = rng.integers(0, dims[-1], bsz)
    w1 = rng.standard_normal((5, 6)).astype(np.float32)
    b1 = rng.standard_normal(5).astype(np.float32)
    w2 = rng.standard_normal((4, 5)).astype(np.float32)
    b2 = rng.standard_normal(4).astype(np.float32)
    params = np.concatenate([w1.ravel(), b1, w2.ravel(), b2]).astype(np.float32)
    m, v = np.zeros_like(params), np.zeros_like(params)
    p0 = params.copy()
    loss, grads = orc.mlp_train_step(dims, x, lab, params, m, v, 1e-3, 0.9, 0.999, 1e-8, 1, want_grads=True)
    z1 = orc.dense_forward(x, w1, b1)
    h1, mask = orc.relu(z1)
    z2 = orc.dense_forward(h1, w2, b2)
    l2, g2 = orc.cross_entropy(z2, lab)
    assert loss == pytest.approx(float(l2), rel=0, abs=0)
    gb2 = orc.sum_dim0(g2)
    gh1, gw2t = orc.matmul_backward(h1, np.ascontiguousarray(w2.T), g2)
    gz1 = orc.relu_backward(mask, gh1)
    gb1 = orc.sum_dim0(gz1)
    _, gw1t = orc.matmul_backward(x, np.ascontiguousarray(w1.T), gz1, need_a=False)
    exp = np.concatenate([gw1t.T.ravel(), gb1, gw2t.T.ravel(), gb2])
    np.testing.assert_array_equal(grads, exp)
    pe, me, ve = p0.copy(), np.zeros_like(p0), np.zeros_like(p0)
    orc.adam_step(pe, exp, me, ve, 1e-3, 0.9, 0.999, 1e-8, step=1)
    np.testing.assert_array_equal(params, pe)


# ------------------------------------------------------------------ training-step ops beside the GEMMs
def test_cross_entropy_general_known_answers(orc, golden):
    for case in golden["cross_entropy_general"]:
        logits = np.array(case["logits"], dtype=np.float32)
        targets = np.array(case["labels"], dtype=np.int64) if "labels" in case else np.array(case["targets"], np.float32)
        loss, grad = orc.cross_entropy_ex(logits, targets, case["reduction"])
        if case["loss"] == "inf":
            assert np.isinf(loss) and loss > 0
        else:
            np.testing.assert_allclose(loss, np.array(case["loss"], dtype=np.float64), rtol=1e-5, atol=1e-8)
    # class indices and their one-hot matrix are the same computation (regression.rs:769-862)
    rng = np.random.default_rng(0)
    x = rng.standard_normal((6, 5)).astype(np.float32)
    lab = rng.integers(0, 5, 6)
    onehot = np.eye(5, dtype=np.float32)[lab]
    for red in ("sum", "mean", "none"):
        la, ga = orc.cross_entropy_ex(x, lab, red)
        lb, gb = orc.cross_entropy_ex(x, onehot, red)
        np.testing.assert_array_equal(la, lb)
        np.testing.assert_array_equal(ga, gb)
    l_old, g_old = orc.cross_entropy(x, lab, mean=True)
    l_new, g_new = orc.cross_entropy_ex(x, lab, "mean")
    assert l_old == l_new and np.array_equal(g_old, g_new)


def test_sgd_rmsprop_clipping_known_answers(orc, golden):
    for case in golden["sgd"]:
        dt = np.dtype(case["dtype"])
        p = np.array(case["param"], dtype=dt)
        v = np.zeros_like(p) if case["momentum"] > 0 else None
        orc.sgd_step(p, np.array(case["grad"], dtype=dt), v, case["lr"], case["momentum"], case["dampening"],
                     case["weight_decay"], case["nesterov"])
        np.testing.assert_allclose(p, case["expected"], rtol=0, atol=case["atol"])
    for case in golden["rmsprop"]:
        p = np.array(case["param"], dtype=np.float32)
        sq = np.zeros_like(p)
        mb = np.zeros_like(p) if case["momentum"] > 0 else None
        ga = np.zeros_like(p) if case["centered"] else None
        orc.rmsprop_step(p, np.array(case["grad"], dtype=np.float32), sq, mb, ga, case["lr"], case["alpha"], case["eps"],
                         case["weight_decay"], case["momentum"])
        assert np.all(p < case["upper_bound"])
    for case in golden["grad_clipping"]:
        g = np.array(case["grad"], dtype=np.float32)
        if case["kind"] == "norm":
            norm = orc.clip_grad_norm([g], case["max_norm"])
            assert abs(norm - case["norm"]) < 1e-10 * max(1.0, case["norm"]) + 1e-6
            if "expected" in case:
                np.testing.assert_allclose(g, case["expected"], rtol=0, atol=case["atol"])
            else:
                assert np.sqrt(orc.sumsq(g)) <= case["norm_after_at_most"]
        else:
            orc.clip_grad_value([g], case["min"], case["max"])
            np.testing.assert_allclose(g, case["expected"], rtol=0, atol=case["atol"])
    # NaN survives a clamp, as f32::clamp does
    g = np.array([np.nan, 5.0], dtype=np.float32)
    orc.clip_grad_value([g], -1.0, 1.0)
    assert np.isnan(g[0]) and g[1] == 1.0


def test_batch_norm_known_answers(orc, golden):
    for case in golden["batch_norm"]:
        if case.get("eval_only"):
            rm = np.array(case["running_mean"], np.float32)
            rv = np.array(case["running_var"], np.float32)
        else:
            x = np.array(case["train_x"], np.float32)
            c = x.shape[1]
            rm, rv = np.zeros(c, np.float32), np.ones(c, np.float32)
            w = np.array(case["weight"], np.float32) if "weight" in case else None
            b = np.array(case["bias"], np.float32) if "bias" in case else None
            y, _, _ = orc.batch_norm(x, w, b, rm, rv, True, case["momentum"], case["eps"])
            if "train_y" in case:
                np.testing.assert_allclose(y, case["train_y"], rtol=0, atol=case["atol"])
            if "running_mean_after" in case:
                np.testing.assert_allclose(rm, case["running_mean_after"], rtol=0, atol=case["atol"])
            if "running_var_after" in case:
                np.testing.assert_allclose(rv, case["running_var_after"], rtol=0, atol=case["atol"])
        if "eval_x" in case:
            before = rm.copy()
            y, _, _ = orc.batch_norm(np.array(case["eval_x"], np.float32), None, None, rm, rv, False, 0.1, case["eps"])
            np.testing.assert_allclose(y, case["eval_y"], rtol=0, atol=case["atol"])
            np.testing.assert_array_equal(rm, before)      # eval leaves the running estimates alone


def test_batch_norm_backward_finite_difference_and_dropout_mask(orc, rng):
    x = rng.standard_normal((5, 3, 4)).astype(np.float64)
    w = rng.standard_normal(3)
    b = rng.standard_normal(3)
    go = rng.standard_normal(x.shape)
    y, mean, invstd = orc.batch_norm(x, w, b, None, None, True, 0.1, 1e-5)
    dx, dw, db = orc.batch_norm_backward(x, go, w, mean, invstd, True)
    f = lambda xx, ww, bb: float((orc.batch_norm(xx, ww, bb, None, None, True, 0.1, 1e-5)[0] * go).sum())
    h = 1e-6
    for idx in [(0, 0, 0), (2, 1, 3), (4, 2, 1)]:
        xp, xm = x.copy(), x.copy()
        xp[idx] += h
        xm[idx] -= h
        assert abs((f(xp, w, b) - f(xm, w, b)) / (2 * h) - dx[idx]) < 1e-5
    for c in range(3):
        wp, wm = w.copy(), w.copy()
        wp[c] += h
        wm[c] -= h
        assert abs((f(x, wp, b) - f(x, wm, b)) / (2 * h) - dw[c]) < 1e-5
    np.testing.assert_allclose(db, go.sum(axis=(0, 2)), rtol=1e-12)
    # dropout mask: extreme probabilities (tests/nn/test_functional.py:498-506), scale, keep rate, determinism
    assert np.all(orc.dropout_mask(100, 0.0, 1) == 1.0) and not orc.dropout_mask(100, 1.0, 1).any()
    m = orc.dropout_mask(200_000, 0.3, seed=42)
    assert set(np.unique(m)) == {np.float32(0.0), np.float32(1.0) / np.float32(0.7)}
    assert abs((m != 0).mean() - 0.7) < 0.005
    np.testing.assert_array_equal(m, orc.dropout_mask(200_000, 0.3, seed=42))
    np.testing.assert_array_equal(m[1000:], orc.dropout_mask(199_000, 0.3, seed=42, offset=1000))
    assert (orc.dropout_mask(200_000, 0.3, seed=43) != m).mean() > 0.3
