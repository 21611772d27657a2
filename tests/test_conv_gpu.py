"""conv2d forward / backward on the device against the reference's known answers and the oracle."""
import numpy as np
import pytest
import torch

from oracle import conv_f64

pytestmark = pytest.mark.gpu

# The path's tolerance: |device - reference loops (oracle)| <= F32_TOL * (norm product of the output's two operand
# vectors), per output.  TIGHT is what the default arithmetic (22 bits kept per operand, f32 accumulation) has to
# meet against float64 dot products: an order of magnitude below what a single 16-bit product would give.
F32_TOL = 1e-4
TIGHT = 8e-6


def check_outputs(name, got, ref32, ref64, norms, extra=0.0):
    """got vs the oracle at F32_TOL and vs float64 at TIGHT, both relative to each output's own norm product."""
    floor = np.finfo(np.float32).tiny
    e32 = np.abs(got.astype(np.float64) - ref32.astype(np.float64)) / (norms + extra + floor)
    e64 = np.abs(got.astype(np.float64) - ref64) / (norms + extra + floor)
    assert e32.max() <= F32_TOL, (name, "vs oracle", float(e32.max()))
    assert e64.max() <= TIGHT, (name, "vs float64", float(e64.max()))
    return float(e64.max())


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
    # the bias is one more term of every output's sum
    check_outputs("y", y.numpy(), ref, conv_f64.forward(xn, wn, bn, stride, padding),
                  conv_f64.forward_norms(xn, wn, stride, padding), extra=np.abs(bn)[None, :, None, None])
    go = rng.standard_normal(ref.shape).astype(np.float32)
    y.backward(mt.Tensor(go))
    gx, gw, gb = orc.conv2d_backward(xn, wn, go, stride, padding)
    check_outputs("dx", x.grad.numpy(), gx, conv_f64.grad_input(go, wn, xn.shape, stride, padding),
                  conv_f64.grad_input_norms(go, wn, xn.shape, stride, padding))
    check_outputs("dw", wt.grad.numpy(), gw, conv_f64.grad_weight(go, xn, wn.shape, stride, padding),
                  conv_f64.grad_weight_norms(go, xn, wn.shape, stride, padding))
    # db[o] = <dy[:,o], ones>
    k_w = n * ref.shape[2] * ref.shape[3]
    gbn = np.sqrt((go.astype(np.float64) ** 2).sum(axis=(0, 2, 3)) * k_w)
    assert (np.abs(b.grad.numpy() - gb) <= F32_TOL * gbn).all()
    assert (np.abs(b.grad.numpy() - go.astype(np.float64).sum(axis=(0, 2, 3))) <= TIGHT * gbn).all()


def test_tolerance_tells_a_single_product_from_the_default(be, orc, rng):
    """The bounds above are not vacuous: the same layer computed with ONE bf16 product per f32 product
    (mode BF16X1, 8 bits kept) fails the float64 bound for y, dx and dw, and by a wide margin."""
    n, c, h, w, co, k = 8, 64, 28, 28, 64, 3
    xn = rng.standard_normal((n, c, h, w)).astype(np.float32)
    wn = (rng.standard_normal((co, c, k, k)) * np.sqrt(2.0 / (c * k * k))).astype(np.float32)
    go = rng.standard_normal((n, co, h, w)).astype(np.float32)
    dev = lambda a: torch.from_numpy(a).to(be.device)
    s1, p1 = (1, 1), (1, 1)
    refs = (conv_f64.forward(xn, wn, None, s1, p1), conv_f64.grad_input(go, wn, xn.shape, s1, p1),
            conv_f64.grad_weight(go, xn, wn.shape, s1, p1))
    norms = (conv_f64.forward_norms(xn, wn, s1, p1), conv_f64.grad_input_norms(go, wn, xn.shape, s1, p1),
             conv_f64.grad_weight_norms(go, xn, wn.shape, s1, p1))
    for mode, passes in ((0, True), (1, False)):
        outs = (be.conv2d_fwd(dev(xn), dev(wn), None, s1, p1, f32_mode=mode),
                be.conv2d_bwd_data(dev(go), dev(wn), xn.shape, s1, p1, f32_mode=mode),
                be.conv2d_bwd_weight(dev(go), dev(xn), wn.shape, s1, p1, f32_mode=mode))
        be.sync()
        for name, out, ref, nrm in zip(("y", "dx", "dw"), outs, refs, norms):
            err = float((np.abs(out.cpu().numpy() - ref) / nrm).max())
            assert (err <= TIGHT) == passes, (name, mode, err)
            if not passes:
                assert err >= 3 * TIGHT, (name, mode, err)


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
    # element-wise at full size: 256 outputs each of y, dx and dw as float64 dot products on the host
    # (576 terms for y and dx, 128*56*56 = 401,408 terms for dw), each within TIGHT of its own norm product
    xh, wh, bh, dyh = x.cpu().numpy(), w.cpu().numpy(), b.cpu().numpy(), dy.cpu().numpy()
    yh, dxh, dwh = y1.cpu().numpy(), dx.cpu().numpy(), dw.cpu().numpy()
    pick = np.random.default_rng(11)
    worst = {"y": 0.0, "dx": 0.0, "dw": 0.0}
    for _ in range(256):
        n_, o_, c_ = pick.integers(128), pick.integers(64), pick.integers(64)
        # image borders are where the zero fill matters: half of the samples sit on one
        edge = pick.integers(2)
        h_ = int(pick.choice([0, 55])) if edge else int(pick.integers(56))
        w_ = int(pick.choice([0, 55])) if pick.integers(2) else int(pick.integers(56))
        v, s = conv_f64.sample_forward(xh, wh, bh, (1, 1), n_, o_, h_, w_)
        worst["y"] = max(worst["y"], abs(float(yh[n_, o_, h_, w_]) - v) / (s + abs(float(bh[o_]))))
        v, s = conv_f64.sample_grad_input(dyh, wh, (1, 1), n_, c_, h_, w_)
        worst["dx"] = max(worst["dx"], abs(float(dxh[n_, c_, h_, w_]) - v) / s)
        i_, j_ = pick.integers(3), pick.integers(3)
        v, s = conv_f64.sample_grad_weight(dyh, xh, (1, 1), o_, c_, i_, j_)
        worst["dw"] = max(worst["dw"], abs(float(dwh[o_, c_, i_, j_]) - v) / s)
    assert max(worst.values()) <= TIGHT, worst


@pytest.mark.parametrize("geom", [g for g in GEOMS if g[7] == (1, 1)] + [(2, 5, 9, 300, 3, 3, 3, (1, 1), (1, 1)),
                                                                         (1, 70, 6, 13, 9, 3, 3, (1, 1), (2, 2)),
                                                                         (3, 2, 20, 5, 4, 2, 4, (1, 1), (0, 3)),
                                                                         (2, 40, 23, 61, 140, 5, 5, (1, 1), (2, 2)),
                                                                         (2, 33, 9, 250, 20, 3, 3, (1, 1), (1, 1)),
                                                                         (1, 8, 40, 12, 8, 7, 7, (1, 1), (3, 3)),
                                                                         (2, 6, 5, 254, 4, 1, 3, (1, 1), (0, 2))])
@pytest.mark.parametrize("lowering", ["implicit", "implicit_bf16x6", "channels_on_m", "channels_on_m_bf16x6", "per_tap",
                                      "explicit"])
def test_both_lowerings_match_oracle(be, orc, rng, geom, lowering):
    """Stride-1 forward and data gradient exist four times.  Implicit GEMM over channels-last planes with the image
    block staged once per channel block as a halo tile: output pixels on the MMA's M side (default; two fp16 planes,
    or three bf16 planes when a bf16 mode is asked for) or output channels on the M side (variant byte 0xfb).
    Implicit GEMM that fetches the window of every tap (variant byte 0xfc; the last resort of the implicit path).
    And the gathered-patch lowering (variant byte 0xff; taken by itself when a row is wider than 256).
    The weight gradient exists three times: implicit GEMM over one staged halo block of x per step with two taps
    per MMA (default, fp16 planes), implicit GEMM with a window of x per tap (the bf16 modes, rows wider than 254,
    and variant byte 0xfc), and the gathered-patch lowering."""
    n, c, h, w, co, kh, kw, stride, padding = geom
    mode = {"implicit": 0, "implicit_bf16x6": 6, "channels_on_m": 0xFB00, "channels_on_m_bf16x6": 0xFB06,
            "per_tap": 0xFC00, "explicit": 0xFF00}[lowering]
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
    check_outputs("y", y.cpu().numpy(), ref, conv_f64.forward(xn, wn, bn, stride, padding),
                  conv_f64.forward_norms(xn, wn, stride, padding), extra=np.abs(bn)[None, :, None, None])
    check_outputs("dx", dx.cpu().numpy(), gx, conv_f64.grad_input(go, wn, xn.shape, stride, padding),
                  conv_f64.grad_input_norms(go, wn, xn.shape, stride, padding))
    check_outputs("dw", dw.cpu().numpy(), gw, conv_f64.grad_weight(go, xn, wn.shape, stride, padding),
                  conv_f64.grad_weight_norms(go, xn, wn.shape, stride, padding))


STRIDED = [  # n, c, h, w, co, kh, kw, stride, padding
    (2, 3, 8, 9, 5, 3, 2, (2, 1), (1, 2)),
    (4, 16, 14, 14, 32, 3, 3, (2, 2), (1, 1)),
    (2, 4, 9, 9, 6, 5, 5, (3, 3), (2, 2)),
    (3, 64, 56, 56, 64, 3, 3, (2, 2), (1, 1)),        # the large config's layer, strided, at reduced batch
    (2, 8, 15, 17, 12, 1, 1, (2, 2), (0, 0)),          # 1 x 1 filter: three of the four phase images are never read
    (1, 5, 7, 30, 9, 3, 3, (1, 2), (1, 1)),
    (2, 6, 33, 33, 10, 7, 7, (2, 2), (3, 3)),          # odd extent: phase images of different true size
    (1, 3, 20, 20, 4, 4, 4, (4, 4), (0, 0)),           # stride = filter size: every phase holds exactly one tap
    (2, 70, 12, 300, 130, 3, 3, (2, 2), (1, 1)),       # wide rows, two channel blocks of the image, > 128 output channels
]


@pytest.mark.parametrize("geom", STRIDED)
@pytest.mark.parametrize("lowering", ["implicit", "explicit"])
def test_strided_both_lowerings(be, orc, rng, geom, lowering):
    """Strided convolutions run the implicit kernels too.  Forward: the image planes are written as stride_h x
    stride_w phase images, which turns every filter tap into a stride-1 window of one of them.  Data gradient: one
    phase of dx at a time, each a stride-1 data gradient of dy under the sub-filter of taps with that phase's
    parity, scattered with the strides (phases no tap reaches stay zero).  Same bounds as the stride-1 path, against
    the oracle and float64, for both those kernels and the gathered-patch lowering."""
    n, c, h, w, co, kh, kw, stride, padding = geom
    mode = 0 if lowering == "implicit" else 0xFF00
    xn = rng.standard_normal((n, c, h, w)).astype(np.float32)
    wn = (rng.standard_normal((co, c, kh, kw)) * np.sqrt(2.0 / (c * kh * kw))).astype(np.float32)
    bn = rng.standard_normal(co).astype(np.float32)
    dev = lambda a: torch.from_numpy(a).to(be.device)
    y = be.conv2d_fwd(dev(xn), dev(wn), dev(bn), stride, padding, f32_mode=mode)
    be.sync()
    ref = orc.conv2d(xn, wn, bn, stride, padding)
    assert tuple(y.shape) == ref.shape
    check_outputs("y", y.cpu().numpy(), ref, conv_f64.forward(xn, wn, bn, stride, padding),
                  conv_f64.forward_norms(xn, wn, stride, padding), extra=np.abs(bn)[None, :, None, None])
    go = rng.standard_normal(ref.shape).astype(np.float32)
    dx = be.conv2d_bwd_data(dev(go), dev(wn), xn.shape, stride, padding, f32_mode=mode)
    dw = be.conv2d_bwd_weight(dev(go), dev(xn), wn.shape, stride, padding, f32_mode=mode)
    be.sync()
    gx, gw, _ = orc.conv2d_backward(xn, wn, go, stride, padding, need_b=False)
    check_outputs("dx", dx.cpu().numpy(), gx, conv_f64.grad_input(go, wn, xn.shape, stride, padding),
                  conv_f64.grad_input_norms(go, wn, xn.shape, stride, padding))
    check_outputs("dw", dw.cpu().numpy(), gw, conv_f64.grad_weight(go, xn, wn.shape, stride, padding),
                  conv_f64.grad_weight_norms(go, xn, wn.shape, stride, padding))


def test_implicit_conv_scales_every_image_on_its_own(be, orc, rng):
    """The default mode of the stride-1 kernels (two fp16 planes) scales each image by its own power of two:
    images 40 orders of magnitude apart and an all-zero image keep, per output, the accuracy of the plain case."""
    n, c, h, w, co = 4, 6, 9, 11, 7
    xn = rng.standard_normal((n, c, h, w)).astype(np.float32)
    xn[0] *= 1e-20
    xn[2] *= 1e20
    xn[3] = 0.0
    wn = (rng.standard_normal((co, c, 3, 3)) * np.sqrt(2.0 / (c * 9))).astype(np.float32)
    dev = lambda a: torch.from_numpy(a).to(be.device)
    s1, p1 = (1, 1), (1, 1)
    y = be.conv2d_fwd(dev(xn), dev(wn), None, s1, p1).cpu().numpy()
    check_outputs("y", y, orc.conv2d(xn, wn, None, s1, p1), conv_f64.forward(xn, wn, None, s1, p1),
                  conv_f64.forward_norms(xn, wn, s1, p1))
    assert not y[3].any()
    # the data gradient runs on the same kernel with dy as the image operand
    go = rng.standard_normal((n, co, h, w)).astype(np.float32)
    go[1] *= 1e-25
    go[2] *= 1e15
    dx = be.conv2d_bwd_data(dev(go), dev(wn), xn.shape, s1, p1).cpu().numpy()
    gx, _, _ = orc.conv2d_backward(np.zeros_like(xn), wn, go, s1, p1, need_b=False)
    check_outputs("dx", dx, gx, conv_f64.grad_input(go, wn, xn.shape, s1, p1),
                  conv_f64.grad_input_norms(go, wn, xn.shape, s1, p1))


@pytest.mark.parametrize("stride", [(1, 1), (2, 2)])
def test_nonfinite_operands_give_the_reference_results(be, orc, rng, stride):
    """Inf and NaN in x, w or dy: the reference's direct loops give +-Inf where an Inf meets finite values and NaN
    where it meets a zero, an Inf of the other sign or a NaN.  The split-plane kernels cannot (Inf times a zero
    low-order plane is NaN), so a call whose operands held a non-finite value is recomputed on the CUDA cores in
    the reference's own summation order: every output then equals the oracle's, non-finite ones included, and a
    later call on finite data is the tensor-core result again."""
    n, c, h, w, co = 3, 6, 10, 12, 7
    p1 = (1, 1)
    xn = rng.standard_normal((n, c, h, w)).astype(np.float32)
    wn = (rng.standard_normal((co, c, 3, 3)) * np.sqrt(2.0 / (c * 9))).astype(np.float32)
    xn[0, 2, 4, 5] = np.inf
    xn[1, 0, 0, 0] = -np.inf
    xn[1, 3, 7, 7] = np.nan
    wn[2, 1, 1, 1] = 0.0            # Inf * 0 = NaN in the outputs of channel 2 whose centre tap sees an Inf
    dev = lambda a: torch.from_numpy(a).to(be.device)
    y = be.conv2d_fwd(dev(xn), dev(wn), None, stride, p1).cpu().numpy()
    ref = orc.conv2d(xn, wn, None, stride, p1)
    assert np.isinf(ref).any() and np.isnan(ref).any() and np.isfinite(ref).any()
    np.testing.assert_array_equal(y, ref)          # NaN == NaN here; signs of the infinities included
    go = rng.standard_normal(ref.shape).astype(np.float32)
    go[2, 1, 1, 2] = np.inf
    go[0, 0, 0, 0] = np.nan
    xf = rng.standard_normal((n, c, h, w)).astype(np.float32)
    wf = np.abs(wn) + 0.01
    wf[3, 2, 0, 0] = -np.inf
    gx, _, _ = orc.conv2d_backward(xf, wf, go, stride, p1, need_w=False, need_b=False)
    dx = be.conv2d_bwd_data(dev(go), dev(wf), xn.shape, stride, p1).cpu().numpy()
    assert np.isinf(gx).any() and np.isnan(gx).any()
    np.testing.assert_array_equal(dx, gx)
    _, gw, _ = orc.conv2d_backward(xn, wn, go, stride, p1, need_x=False, need_b=False)
    dw = be.conv2d_bwd_weight(dev(go), dev(xn), wn.shape, stride, p1).cpu().numpy()
    assert (~np.isfinite(gw)).any()
    assert np.array_equal(np.isnan(dw), np.isnan(gw)) and np.array_equal(np.isposinf(dw), np.isposinf(gw))
    assert np.array_equal(np.isneginf(dw), np.isneginf(gw))
    fin = np.isfinite(gw)
    nrm = conv_f64.grad_weight_norms(np.where(np.isfinite(go), go, 0), np.where(np.isfinite(xn), xn, 0), wn.shape, stride, p1)
    assert (np.abs(dw[fin] - gw[fin]) <= F32_TOL * nrm[fin]).all()
    # the flag is per call: finite operands afterwards take the tensor-core path and meet its bounds
    xc = rng.standard_normal((n, c, h, w)).astype(np.float32)
    wc = (rng.standard_normal((co, c, 3, 3)) * np.sqrt(2.0 / (c * 9))).astype(np.float32)
    y2 = be.conv2d_fwd(dev(xc), dev(wc), None, stride, p1).cpu().numpy()
    check_outputs("y after a non-finite call", y2, orc.conv2d(xc, wc, None, stride, p1),
                  conv_f64.forward(xc, wc, None, stride, p1), conv_f64.forward_norms(xc, wc, stride, p1))


def test_dependent_launch_changes_no_bit_of_a_convolution(be, rng, monkeypatch):
    """The kernels of a conv2d call are chained by programmatic dependent launch (each waits for its predecessor
    inside the kernel); a handle created with MTB200_NO_PDL=1 launches them the plain way.  Forward, data gradient
    and weight gradient give the same bits either way, stride 1 and strided, calls issued back to back."""
    from minitensor_b200.backend import Backend
    monkeypatch.setenv("MTB200_NO_PDL", "1")
    plain = Backend(be.device.index or 0)
    monkeypatch.delenv("MTB200_NO_PDL")
    try:
        for (n, c, h, w, co, k, stride, pad) in ((8, 64, 28, 28, 64, 3, (1, 1), (1, 1)), (4, 16, 14, 14, 32, 3, (2, 2), (1, 1))):
            x = torch.from_numpy(rng.standard_normal((n, c, h, w)).astype(np.float32)).to(be.device)
            wt = torch.from_numpy((rng.standard_normal((co, c, k, k)) * 0.05).astype(np.float32)).to(be.device)
            bias = torch.from_numpy(rng.standard_normal(co).astype(np.float32)).to(be.device)
            for _ in range(2):
                y = be.conv2d_fwd(x, wt, bias, stride, pad)
                dy = torch.ones_like(y) * 0.5 + y * 0.01
                dx = be.conv2d_bwd_data(dy, wt, x.shape, stride, pad)
                dw = be.conv2d_bwd_weight(dy, x, wt.shape, stride, pad)
            y0 = plain.conv2d_fwd(x, wt, bias, stride, pad)
            dx0 = plain.conv2d_bwd_data(dy, wt, x.shape, stride, pad)
            dw0 = plain.conv2d_bwd_weight(dy, x, wt.shape, stride, pad)
            be.sync(); plain.sync()
            for name, got, ref in (("y", y, y0), ("dx", dx, dx0), ("dw", dw, dw0)):
                diff = (got - ref).abs()
                assert torch.equal(got, ref), (name, (n, c, h, w, stride), float(diff.max()), int((diff > 0).sum()),
                                               float(ref.abs().max()))
    finally:
        plain.close()


def test_a_second_handle_does_not_shrink_what_the_first_may_launch(be, rng):
    """The opt-in shared-memory size of a kernel belongs to the device, not to a handle: a second handle whose
    layer needs less must not lower it under the first handle's feet (the launch would fail with 'invalid
    argument').  First handle: a layer with a large step; second handle: a small layer; first handle again."""
    from minitensor_b200.backend import Backend
    other = Backend(be.device.index or 0)
    try:
        big = (4, 64, 30, 120, 64, 3)
        small = (2, 3, 8, 9, 5, 3)
        mk = lambda n, c, h, w, co, k: (torch.from_numpy(rng.standard_normal((n, c, h, w)).astype(np.float32)).to(be.device),
                                        torch.from_numpy(rng.standard_normal((n, co, h, w)).astype(np.float32)).to(be.device),
                                        (co, c, k, k))
        xb, dyb, wsb = mk(*big)
        xs, dys, wss = mk(*small)
        first = be.conv2d_bwd_weight(dyb, xb, wsb, (1, 1), (1, 1))
        y1 = be.conv2d_fwd(xb, torch.ones(wsb, device=be.device), None, (1, 1), (1, 1))
        other.conv2d_bwd_weight(dys, xs, wss, (1, 1), (1, 1))
        other.conv2d_fwd(xs, torch.ones(wss, device=be.device), None, (1, 1), (1, 1))
        again = be.conv2d_bwd_weight(dyb, xb, wsb, (1, 1), (1, 1))
        y2 = be.conv2d_fwd(xb, torch.ones(wsb, device=be.device), None, (1, 1), (1, 1))
        be.sync(); other.sync()
        assert torch.equal(first, again) and torch.equal(y1, y2)
    finally:
        other.close()
