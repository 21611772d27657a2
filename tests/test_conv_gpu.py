"""conv2d forward / backward on the device against the reference's known answers and the oracle."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

F32_TOL = 1e-4


def test_known_answers_and_errors(be, golden):
    import minitensor_b200.nn as nn
    import minitensor_b200.tensor as mt
    for case in golden["conv2d"]:
        x = mt.Tensor(np.array(case["x"], np.float32).reshape(case["x_shape"]))
        w = mt.Tensor(np.array(case["w"], np.float32).reshape(case["w_shape"]))
        b = None if case["bias"] is None else mt.Tensor(np.array(case["bias"], np.float32))
        y = nn.conv2d(x, w, b, stride=tuple(case["stride"]), padding=tuple(case["padding"]))
        assert list(y.shape) == case["out_shape"], case["source"]
        np.testing.assert_array_equal(y.numpy().ravel(), np.array(case["out"], np.float32), err_msg=case["source"])
    for case in golden["conv2d_invalid"]:
        with pytest.raises(Exception):
            nn.conv2d(mt.Tensor(np.zeros(case["x_shape"], np.float32)), mt.Tensor(np.zeros(case["w_shape"], np.float32)))
    x = mt.Tensor(np.zeros((1, 2, 4, 4), np.float32))
    with pytest.raises(ValueError):
        nn.conv2d(x, mt.Tensor(np.zeros((3, 1, 2, 2), np.float32)))            # channel mismatch
    with pytest.raises(ValueError):
        nn.conv2d(x, mt.Tensor(np.zeros((3, 2, 2, 2), np.float32)), stride=0)  # zero stride
    with pytest.raises(ValueError):
        nn.conv2d(x, mt.Tensor(np.zeros((3, 2, 2, 2), np.float32)), mt.Tensor(np.zeros(2, np.float32)))  # bias length
    with pytest.raises(ValueError):
        nn.conv2d(mt.Tensor(np.zeros((2, 4, 4), np.float32)), mt.Tensor(np.zeros((3, 2, 2, 2), np.float32)))


GEOMS = [  # n, c, h, w, co, kh, kw, stride, padding
    (1, 1, 5, 5, 1, 3, 3, (1, 1), (0, 0)),
    (2, 3, 8, 9, 5, 3, 3, (1, 1), (1, 1)),
    (2, 3, 8, 9, 5, 3, 2, (2, 1), (1, 2)),
    (4, 16, 14, 14, 32, 3, 3, (2, 2), (1, 1)),
    (3, 7, 11, 13, 130, 1, 1, (1, 1), (0, 0)),
    (2, 4, 9, 9, 6, 5, 5, (3, 3), (2, 2)),
    (8, 64, 28, 28, 64, 3, 3, (1, 1), (1, 1)),   # the large config's layer at reduced batch / resolution
]


@pytest.mark.parametrize("geom", GEOMS)
def test_forward_backward_match_oracle(be, orc, rng, geom):
    import minitensor_b200.nn as nn
    import minitensor_b200.tensor as mt
    n, c, h, w, co, kh, kw, stride, padding = geom
    xn = rng.standard_normal((n, c, h, w)).astype(np.float32)
    wn = (rng.standard_normal((co, c, kh, kw)) * np.sqrt(2.0 / (c * kh * kw))).astype(np.float32)
    bn = rng.standard_normal(co).astype(np.float32)
    x, wt, b = mt.Tensor(xn, requires_grad=True), mt.Tensor(wn, requires_grad=True), mt.Tensor(bn, requires_grad=True)
    y = nn.conv2d(x, wt, b, stride=stride, padding=padding)
    ref = orc.conv2d(xn, wn, bn, stride, padding)
    assert y.shape == ref.shape
    # every output is a dot product of <= c*kh*kw terms: scale the tolerance by the operand norms
    xnorm = np.sqrt(c * kh * kw) * np.abs(xn).max()
    wnorm = np.linalg.norm(wn.reshape(co, -1), axis=1).max()
    assert np.abs(y.numpy() - ref).max() <= F32_TOL * xnorm * wnorm
    go = rng.standard_normal(ref.shape).astype(np.float32)
    y.backward(mt.Tensor(go))
    gx, gw, gb = orc.conv2d_backward(xn, wn, go, stride, padding)
    gnorm = np.abs(go).max()
    assert np.abs(x.grad.numpy() - gx).max() <= F32_TOL * np.sqrt(co * kh * kw) * gnorm * np.abs(wn).max() * np.sqrt(co * kh * kw)
    k_w = n * ref.shape[2] * ref.shape[3]
    assert np.abs(wt.grad.numpy() - gw).max() <= F32_TOL * k_w * gnorm * np.abs(xn).max()
    assert np.abs(b.grad.numpy() - gb).max() <= 1e-5 * k_w * gnorm


def test_conv2d_layer_defaults(be):
    import minitensor_b200.nn as nn
    import minitensor_b200.tensor as mt
    layer = nn.Conv2d(3, 8, 3, stride=1, padding=1, rng=np.random.default_rng(0))
    assert layer.weight.shape == (8, 3, 3, 3) and not layer.bias.numpy().any()
    assert np.abs(layer.weight.numpy()).max() <= np.sqrt(6.0 / 27)             # He-uniform bound
    y = layer(mt.Tensor(np.ones((2, 3, 6, 6), np.float32)))
    assert y.shape == (2, 8, 6, 6)


def test_full_size_layer_properties(be):
    """[128,64,56,56] * [64,64,3,3], stride 1, pad 1 (the large conv config): the convolution is linear in
    x and in w, and db equals the sum of dy; checked at full size where the oracle would take minutes."""
    g = torch.Generator(device="cpu").manual_seed(1)
    x = torch.randn(128, 64, 56, 56, generator=g).to(be.device)
    w = (torch.randn(64, 64, 3, 3, generator=g) * (2.0 / 576) ** 0.5).to(be.device)
    w2 = (torch.randn(64, 64, 3, 3, generator=g) * (2.0 / 576) ** 0.5).to(be.device)
    b = torch.randn(64, generator=g).to(be.device)
    y1 = be.conv2d_fwd(x, w, b, (1, 1), (1, 1))
    y2 = be.conv2d_fwd(x, w2, None, (1, 1), (1, 1))
    y12 = be.conv2d_fwd(x, w + w2, b, (1, 1), (1, 1))
    be.sync()
    assert float((y12 - (y1 + y2)).abs().max()) <= 1e-4 * 24 * 4   # ||patch|| ~ 24, ||w row|| ~ 1.4 (x2 for the sum)
    # adjoint identity: <conv(x, w), dy> == <x, conv_bwd_data(dy, w)> == <w, conv_bwd_weight(dy, x)>
    dy = torch.randn(128, 64, 56, 56, generator=g).to(be.device)
    dx = be.conv2d_bwd_data(dy, w, x.shape, (1, 1), (1, 1))
    dw = be.conv2d_bwd_weight(dy, x, w.shape, (1, 1), (1, 1))
    db = be.conv2d_bwd_bias(dy)
    be.sync()
    lhs = float((y1 - b.view(1, -1, 1, 1)).double().mul(dy.double()).sum())
    assert abs(lhs - float(x.double().mul(dx.double()).sum())) <= 1e-5 * abs(lhs) + 1.0
    assert abs(lhs - float(w.double().mul(dw.double()).sum())) <= 1e-5 * abs(lhs) + 1.0
    ref_db = dy.double().sum(dim=(0, 2, 3))
    assert float((db.double() - ref_db).abs().max()) <= 1e-5 * float(dy.abs().double().sum(dim=(0, 2, 3)).max())


@pytest.mark.parametrize("geom", [g for g in GEOMS if g[7] == (1, 1)] + [(2, 5, 9, 300, 3, 3, 3, (1, 1), (1, 1)),
                                                                         (1, 70, 6, 13, 9, 3, 3, (1, 1), (2, 2)),
                                                                         (3, 2, 20, 5, 4, 2, 4, (1, 1), (0, 3))])
@pytest.mark.parametrize("lowering", ["implicit", "explicit"])
def test_both_lowerings_match_oracle(be, orc, rng, geom, lowering):
    """Stride-1 forward and data gradient exist twice: as implicit GEMM over channels-last planes
    (default; falls back by itself when a row is wider than 256) and as the gathered-patch lowering
    (forced here with the variant byte 0xff)."""
    n, c, h, w, co, kh, kw, stride, padding = geom
    mode = 0 if lowering == "implicit" else 0xFF00
    xn = rng.standard_normal((n, c, h, w)).astype(np.float32)
    wn = (rng.standard_normal((co, c, kh, kw)) * np.sqrt(2.0 / (c * kh * kw))).astype(np.float32)
    bn = rng.standard_normal(co).astype(np.float32)
    dev = lambda a: torch.from_numpy(a).to(be.device)
    y = be.conv2d_fwd(dev(xn), dev(wn), dev(bn), stride, padding, f32_mode=mode)
    ref = orc.conv2d(xn, wn, bn, stride, padding)
    go = rng.standard_normal(ref.shape).astype(np.float32)
    dx = be.conv2d_bwd_data(dev(go), dev(wn), xn.shape, stride, padding, f32_mode=mode)
    dw = be.conv2d_bwd_weight(dev(go), dev(xn), wn.shape, stride, padding, f32_mode=mode)
    be.sync()
    gx, gw, _ = orc.conv2d_backward(xn, wn, go, stride, padding, need_b=False)
    k_w = n * ref.shape[2] * ref.shape[3]
    assert np.abs(dw.cpu().numpy() - gw).max() <= F32_TOL * k_w * np.abs(go).max() * np.abs(xn).max()
    xnorm = np.sqrt(c * kh * kw) * np.abs(xn).max()
    wnorm = np.linalg.norm(wn.reshape(co, -1), axis=1).max()
    assert np.abs(y.cpu().numpy() - ref).max() <= F32_TOL * xnorm * wnorm
    assert np.abs(dx.cpu().numpy() - gx).max() <= F32_TOL * (co * kh * kw) * np.abs(go).max() * np.abs(wn).max()


def test_implicit_conv_scales_every_image_on_its_own(be, orc, rng):
    """The default mode of the stride-1 kernels (two fp16 planes) scales each image by its own power of two:
    images 40 orders of magnitude apart, an all-zero image and an image holding an Inf keep, per image, the
    accuracy of the plain case, and the Inf stays inside the windows that touch it."""
    n, c, h, w, co = 5, 6, 9, 11, 7
    xn = rng.standard_normal((n, c, h, w)).astype(np.float32)
    xn[0] *= 1e-20
    xn[2] *= 1e20
    xn[3] = 0.0
    xn[4, 2, 4, 5] = np.inf
    wn = (rng.standard_normal((co, c, 3, 3)) * np.sqrt(2.0 / (c * 9))).astype(np.float32)
    dev = lambda a: torch.from_numpy(a).to(be.device)
    y = be.conv2d_fwd(dev(xn), dev(wn), None, (1, 1), (1, 1)).cpu().numpy()
    wnorm = np.linalg.norm(wn.reshape(co, -1), axis=1).max()
    for i in range(4):
        ref = orc.conv2d(xn[i:i + 1], wn, None, (1, 1), (1, 1))[0]
        assert np.abs(y[i] - ref).max() <= F32_TOL * np.sqrt(c * 9) * np.abs(xn[i]).max() * wnorm, i
    assert not y[3].any()
    finite_part = xn[4:5].copy()
    finite_part[0, 2, 4, 5] = 0.0
    ref = orc.conv2d(finite_part, wn, None, (1, 1), (1, 1))[0]
    touched = np.zeros((h, w), bool)
    touched[3:6, 4:7] = True                       # outputs whose 3x3 window covers (4, 5)
    assert not np.isfinite(y[4][:, touched]).any()
    assert np.abs(y[4][:, ~touched] - ref[:, ~touched]).max() <= F32_TOL * np.sqrt(c * 9) * np.abs(finite_part).max() * wnorm
    # the data gradient runs on the same kernel with dy as the image operand
    go = rng.standard_normal((n, co, h, w)).astype(np.float32)
    go[1] *= 1e-25
    go[2] *= 1e15
    dx = be.conv2d_bwd_data(dev(go), dev(wn), xn.shape, (1, 1), (1, 1)).cpu().numpy()
    for i in range(n):
        gx, _, _ = orc.conv2d_backward(np.zeros_like(xn[i:i + 1]), wn, go[i:i + 1], (1, 1), (1, 1), need_b=False)
        assert np.abs(dx[i] - gx[0]).max() <= F32_TOL * (co * 9) * np.abs(go[i]).max() * np.abs(wn).max(), i
