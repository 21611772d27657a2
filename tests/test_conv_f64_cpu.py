"""The float64 conv statement used by the GPU parity tests agrees with the oracle (the restatement of the
reference's loops) and with itself: full tensors, per-output norms and the single-output samplers."""
import numpy as np
import pytest

from oracle import conv_f64

GEOMS = [  # n, c, h, w, co, kh, kw, stride, padding
    (2, 3, 8, 9, 5, 3, 3, (1, 1), (1, 1)),
    (2, 3, 8, 9, 5, 3, 2, (2, 1), (1, 2)),
    (2, 4, 9, 9, 6, 5, 5, (3, 3), (2, 2)),
    (3, 2, 20, 5, 4, 2, 4, (1, 1), (0, 3)),
]


@pytest.mark.parametrize("geom", GEOMS)
def test_f64_statement_matches_oracle(orc, rng, geom):
    n, c, h, w, co, kh, kw, stride, padding = geom
    x = rng.standard_normal((n, c, h, w)).astype(np.float32)
    wt = rng.standard_normal((co, c, kh, kw)).astype(np.float32)
    b = rng.standard_normal(co).astype(np.float32)
    y = conv_f64.forward(x, wt, b, stride, padding)
    ref = orc.conv2d(x, wt, b, stride, padding)
    assert y.shape == ref.shape
    assert np.abs(y - ref).max() <= 1e-6 * (conv_f64.forward_norms(x, wt, stride, padding).max() + np.abs(b).max())
    go = rng.standard_normal(ref.shape).astype(np.float32)
    gx, gw, _ = orc.conv2d_backward(x, wt, go, stride, padding, need_b=False)
    dx = conv_f64.grad_input(go, wt, x.shape, stride, padding)
    dw = conv_f64.grad_weight(go, x, wt.shape, stride, padding)
    assert np.abs(dx - gx).max() <= 1e-6 * conv_f64.grad_input_norms(go, wt, x.shape, stride, padding).max()
    assert np.abs(dw - gw).max() <= 1e-6 * conv_f64.grad_weight_norms(go, x, wt.shape, stride, padding).max()
    # Cauchy-Schwarz: every output is bounded by its own norm product
    assert (np.abs(y - b[None, :, None, None]) <= conv_f64.forward_norms(x, wt, stride, padding) * (1 + 1e-12)).all()
    assert (np.abs(dx) <= conv_f64.grad_input_norms(go, wt, x.shape, stride, padding) * (1 + 1e-12) + 1e-300).all()
    assert (np.abs(dw) <= conv_f64.grad_weight_norms(go, x, wt.shape, stride, padding) * (1 + 1e-12)).all()


def test_single_output_samplers(rng):
    n, c, h, w, co, k, pad = 3, 4, 7, 6, 5, 3, (1, 1)
    x = rng.standard_normal((n, c, h, w)).astype(np.float32)
    wt = rng.standard_normal((co, c, k, k)).astype(np.float32)
    b = rng.standard_normal(co).astype(np.float32)
    go = rng.standard_normal((n, co, h, w)).astype(np.float32)
    y = conv_f64.forward(x, wt, b, (1, 1), pad)
    yn = conv_f64.forward_norms(x, wt, (1, 1), pad)
    dx = conv_f64.grad_input(go, wt, x.shape, (1, 1), pad)
    dxn = conv_f64.grad_input_norms(go, wt, x.shape, (1, 1), pad)
    dw = conv_f64.grad_weight(go, x, wt.shape, (1, 1), pad)
    dwn = conv_f64.grad_weight_norms(go, x, wt.shape, (1, 1), pad)
    for _ in range(60):
        i, o, yy, xx = rng.integers(n), rng.integers(co), rng.integers(h), rng.integers(w)
        v, s = conv_f64.sample_forward(x, wt, b, pad, i, o, yy, xx)
        assert abs(v - y[i, o, yy, xx]) <= 1e-12 * s + 1e-12 and abs(s - yn[i, o, yy, xx]) <= 1e-12 * s
        ch = rng.integers(c)
        v, s = conv_f64.sample_grad_input(go, wt, pad, i, ch, yy, xx)
        assert abs(v - dx[i, ch, yy, xx]) <= 1e-12 * s and abs(s - dxn[i, ch, yy, xx]) <= 1e-12 * s
        ti, tj = rng.integers(k), rng.integers(k)
        v, s = conv_f64.sample_grad_weight(go, x, pad, o, ch, ti, tj)
        assert abs(v - dw[o, ch, ti, tj]) <= 1e-12 * s and abs(s - dwn[o, ch, ti, tj]) <= 1e-12 * s
