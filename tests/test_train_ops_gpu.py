"""SGD, RMSprop, gradient clipping and the general cross entropy through the C ABI against the oracle
(bit-exact for the optimizers and the clipping arithmetic) and the reference's own known answers."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def dev(be, a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(be.device)


# ------------------------------------------------------------------ SGD
@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("momentum,dampening,nesterov,wd", [(0.0, 0.0, False, 0.0), (0.0, 0.0, False, 0.01),
                                                            (0.9, 0.0, False, 0.0), (0.9, 0.1, True, 1e-3)])
def test_sgd_bit_exact_three_steps(be, orc, rng, dtype, momentum, dampening, nesterov, wd):
    n = 100_003
    p = rng.standard_normal(n).astype(dtype)
    v = np.zeros(n, dtype) if momentum > 0 else None
    pd, vd = dev(be, p), (dev(be, v) if v is not None else None)
    for _ in range(3):
        g = rng.standard_normal(n).astype(dtype)
        orc.sgd_step(p, g, v, 0.05, momentum, dampening, wd, nesterov)
        be.sgd_step(pd, dev(be, g), vd, lr=0.05, momentum=momentum, dampening=dampening, weight_decay=wd,
                    nesterov=nesterov)
    be.sync()
    np.testing.assert_array_equal(pd.cpu().numpy(), p)
    if v is not None:
        np.testing.assert_array_equal(vd.cpu().numpy(), v)


def test_sgd_known_answers_and_mirror(be, golden):
    import minitensor_b200.optim as optim
    import minitensor_b200.tensor as mt
    for case in golden["sgd"]:
        p = mt.Tensor(np.array(case["param"], dtype=case["dtype"]), requires_grad=True)
        p.grad = mt.Tensor(np.array(case["grad"], dtype=case["dtype"]))
        opt = optim.SGD([p], lr=case["lr"], momentum=case["momentum"], weight_decay=case["weight_decay"],
                        dampening=case["dampening"], nesterov=case["nesterov"])
        opt.step()
        np.testing.assert_allclose(p.numpy(), case["expected"], rtol=0, atol=case["atol"])
        assert opt.step_count == 1
    with pytest.raises(ValueError):
        optim.SGD([mt.Tensor(np.zeros(3, np.int32))])


# ------------------------------------------------------------------ RMSprop
@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("momentum,centered,wd", [(0.0, False, 0.0), (0.9, False, 1e-3), (0.0, True, 0.0), (0.9, True, 1e-2)])
def test_rmsprop_bit_exact_three_steps(be, orc, rng, dtype, momentum, centered, wd):
    n = 65_537
    p = rng.standard_normal(n).astype(dtype)
    sq = np.zeros(n, dtype)
    mb = np.zeros(n, dtype) if momentum > 0 else None
    ga = np.zeros(n, dtype) if centered else None
    pd, sqd = dev(be, p), dev(be, sq)
    mbd = dev(be, mb) if mb is not None else None
    gad = dev(be, ga) if ga is not None else None
    for _ in range(3):
        g = rng.standard_normal(n).astype(dtype)
        orc.rmsprop_step(p, g, sq, mb, ga, 0.01, 0.99, 1e-8, wd, momentum)
        be.rmsprop_step(pd, dev(be, g), sqd, mbd, gad, lr=0.01, alpha=0.99, eps=1e-8, weight_decay=wd, momentum=momentum)
    be.sync()
    np.testing.assert_array_equal(pd.cpu().numpy(), p)
    np.testing.assert_array_equal(sqd.cpu().numpy(), sq)
    if mb is not None:
        np.testing.assert_array_equal(mbd.cpu().numpy(), mb)
    if ga is not None:
        np.testing.assert_array_equal(gad.cpu().numpy(), ga)


def test_rmsprop_known_answers_via_mirror(be, golden):
    import minitensor_b200.optim as optim
    import minitensor_b200.tensor as mt
    for case in golden["rmsprop"]:
        p = mt.Tensor(np.array(case["param"], dtype=np.float32), requires_grad=True)
        p.grad = mt.Tensor(np.array(case["grad"], dtype=np.float32))
        optim.RMSprop([p], lr=case["lr"], alpha=case["alpha"], epsilon=case["eps"], weight_decay=case["weight_decay"],
                      momentum=case["momentum"], centered=case["centered"]).step()
        assert np.all(p.numpy() < case["upper_bound"])


# ------------------------------------------------------------------ clipping
def test_grad_clipping_known_answers(be, golden):
    for case in golden["grad_clipping"]:
        g = dev(be, np.array(case["grad"], dtype=np.float32))
        if case["kind"] == "norm":
            norm = be.clip_grad_norm([g], case["max_norm"])
            assert abs(norm - case["norm"]) < 1e-6
            if "expected" in case:
                np.testing.assert_allclose(g.cpu().numpy(), case["expected"], rtol=0, atol=case["atol"])
            else:
                assert be.grad_norm([g]) <= case["norm_after_at_most"]
        else:
            be.clip_grad_value([g], case["min"], case["max"])
            np.testing.assert_allclose(g.cpu().numpy(), case["expected"], rtol=0, atol=case["atol"])


def test_grad_norm_and_clipping_against_oracle(be, orc, rng):
    grads = [rng.standard_normal(1_000_003).astype(np.float32) * 3, rng.standard_normal(4099).astype(np.float64),
             np.zeros(0, np.float32)]
    gd = [dev(be, g) for g in grads]
    ref_norm = float(np.sqrt(sum(orc.sumsq(g) for g in grads)))
    norm = be.grad_norm(gd)
    assert abs(norm - ref_norm) <= 1e-12 * ref_norm          # both accumulate in f64; only the order differs
    assert be.grad_norm(gd) == norm                           # deterministic
    ref = [g.copy() for g in grads]
    # scale with the SAME coefficient: the arithmetic itself is bit-exact
    coef = 10.0 / (norm + 1e-6)
    total = be.clip_grad_norm(gd, 10.0)
    assert total == norm
    np.testing.assert_array_equal(gd[0].cpu().numpy(), ref[0] * np.float32(coef))
    np.testing.assert_array_equal(gd[1].cpu().numpy(), ref[1] * coef)
    assert be.clip_grad_norm(gd, 1e9) <= 10.0 + 1e-3          # within the threshold: untouched
    vals = [g.copy() for g in (a.cpu().numpy() for a in gd[:2])]
    vals[0][5] = np.nan
    vd = [dev(be, v) for v in vals]
    orc.clip_grad_value(vals, -0.01, 0.02)
    be.clip_grad_value(vd, -0.01, 0.02)
    np.testing.assert_array_equal(vd[0].cpu().numpy(), vals[0])   # NaN stays NaN
    np.testing.assert_array_equal(vd[1].cpu().numpy(), vals[1])
    with pytest.raises(ValueError):
        be.clip_grad_value(vd, 1.0, -1.0)
    with pytest.raises(TypeError):
        be.grad_norm([torch.zeros(4, dtype=torch.int32, device=be.device)])


def test_optimizer_clipping_before_step(be):
    import minitensor_b200.optim as optim
    import minitensor_b200.tensor as mt
    p = mt.Tensor(np.ones(3, np.float32), requires_grad=True)
    p.grad = mt.Tensor(np.full(3, 3.0, np.float32))
    optim.SGD([p], lr=1.0).with_gradient_clipping(max_norm=1.0).step()
    # gradient scaled to norm ~1: each component 1/sqrt(3)
    np.testing.assert_allclose(p.numpy(), 1.0 - 1.0 / np.sqrt(3.0), atol=1e-5)
    q = mt.Tensor(np.zeros(3, np.float32), requires_grad=True)
    q.grad = mt.Tensor(np.array([-2.0, 0.5, 2.0], np.float32))
    optim.SGD([q], lr=1.0).with_gradient_clipping(min_value=-1.0, max_value=1.0).step()
    np.testing.assert_allclose(q.numpy(), [1.0, -0.5, -1.0], atol=1e-6)


# ------------------------------------------------------------------ cross entropy, general form
@pytest.mark.parametrize("reduction", ["mean", "sum", "none"])
@pytest.mark.parametrize("soft", [False, True])
def test_cross_entropy_general_against_oracle(be, orc, rng, reduction, soft):
    bsz, ncls = 257, 1000
    x = (rng.standard_normal((bsz, ncls)) * 3).astype(np.float32)
    if soft:
        t = rng.random((bsz, ncls)).astype(np.float32)
        t /= t.sum(axis=1, keepdims=True)
    else:
        t = rng.integers(0, ncls, bsz)
    rows = rng.standard_normal(bsz).astype(np.float32) if reduction == "none" else None
    ref_loss, ref_grad = orc.cross_entropy_ex(x, t, reduction, upstream=0.5, upstream_rows=rows)
    loss, grad = be.cross_entropy_ex(dev(be, x), dev(be, t), reduction=reduction, upstream=0.5,
                                     upstream_rows=dev(be, rows) if rows is not None else None)
    be.sync()
    np.testing.assert_allclose(loss.cpu().numpy().reshape(np.shape(ref_loss)), ref_loss, rtol=2e-5, atol=1e-6)
    np.testing.assert_allclose(grad.cpu().numpy(), ref_grad, rtol=1e-4, atol=2e-6)


def test_cross_entropy_general_known_answers_and_nn_mirror(be, golden):
    import minitensor_b200.nn as nn
    import minitensor_b200.tensor as mt
    for case in golden["cross_entropy_general"]:
        x = mt.Tensor(np.array(case["logits"], dtype=np.float32), requires_grad=True)
        t = mt.Tensor(np.array(case["labels"], dtype=np.int64)) if "labels" in case else \
            mt.Tensor(np.array(case["targets"], dtype=np.float32))
        loss = nn.cross_entropy(x, t, reduction=case["reduction"])
        if case["loss"] == "inf":
            assert np.isinf(loss.numpy()) and loss.numpy() > 0
        else:
            np.testing.assert_allclose(loss.numpy(), np.array(case["loss"]), rtol=1e-5, atol=1e-8)
    # the dim argument: classes along axis 1 of a [2, 3, 4] tensor, per-position losses (regression.rs:253-308)
    x_np = np.arange(24, dtype=np.float32).reshape(2, 3, 4) * 0.1
    t_np = np.array([[0, 1, 2, 1], [2, 0, 1, 2]], dtype=np.int64)
    x = mt.Tensor(x_np, requires_grad=True)
    loss = nn.cross_entropy(x, mt.Tensor(t_np), reduction="none", dim=1)
    sh = x_np - x_np.max(axis=1, keepdims=True)
    sm = np.exp(sh) / np.exp(sh).sum(axis=1, keepdims=True)
    expected = -np.log(np.take_along_axis(sm, t_np[:, None, :], axis=1).squeeze(1))
    assert loss.shape == expected.shape
    np.testing.assert_allclose(loss.numpy(), expected, rtol=1e-5, atol=1e-6)
    loss.sum().backward()
    onehot = np.moveaxis(np.eye(3, dtype=np.float32)[t_np], -1, 1)
    np.testing.assert_allclose(x.grad.numpy(), sm - onehot, rtol=1e-4, atol=1e-6)
    with pytest.raises(IndexError):
        nn.cross_entropy(x, mt.Tensor(t_np), dim=3)
    with pytest.raises(ValueError):
        nn.cross_entropy(x, mt.Tensor(t_np), reduction="avg")
    with pytest.raises(IndexError):                                   # class index out of range
        nn.cross_entropy(mt.Tensor(np.zeros((2, 3), np.float32)), mt.Tensor(np.array([0, 3], np.int64)))


# ------------------------------------------------------------------ batch norm
@pytest.mark.parametrize("shape", [(64, 128), (37, 5), (8, 6, 50), (4, 3, 17, 19), (300, 4096),
                                   (256, 300, 3, 2),      # N * C = 76,800 (n, c) planes: beyond a 16-bit grid dimension
                                   (2, 3, 1500, 3)])      # planes of 4500 elements: several spans, the last one ragged
@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_batch_norm_forward_backward_against_oracle(be, orc, rng, shape, dtype):
    x = (rng.standard_normal(shape) * 3 + 7).astype(dtype)      # a mean well away from zero
    c = shape[1]
    w, b = rng.standard_normal(c).astype(dtype), rng.standard_normal(c).astype(dtype)
    rm, rv = rng.standard_normal(c).astype(dtype), (rng.random(c) + 0.5).astype(dtype)
    go = rng.standard_normal(shape).astype(dtype)
    tol = 2e-5 if dtype == np.float32 else 1e-11
    for training in (True, False):
        rm_o, rv_o = rm.copy(), rv.copy()
        rm_d, rv_d = dev(be, rm), dev(be, rv)
        y_ref, mean_ref, inv_ref = orc.batch_norm(x, w, b, rm_o, rv_o, training, 0.1, 1e-5)
        y, mean, inv, batch_stats = be.batch_norm_fwd(dev(be, x), dev(be, w), dev(be, b), rm_d, rv_d, training=training,
                                                      momentum=0.1, eps=1e-5)
        assert batch_stats == training
        be.sync()
        np.testing.assert_allclose(y.cpu().numpy(), y_ref, rtol=tol, atol=tol * 10)
        np.testing.assert_allclose(rm_d.cpu().numpy(), rm_o, rtol=tol, atol=tol)
        np.testing.assert_allclose(rv_d.cpu().numpy(), rv_o, rtol=tol, atol=tol)
        dx_ref, dw_ref, db_ref = orc.batch_norm_backward(x, go, w, mean_ref, inv_ref, batch_stats)
        dx, dw, db = be.batch_norm_bwd(dev(be, x), dev(be, go), dev(be, w), mean, inv, batch_stats=batch_stats)
        be.sync()
        scale = max(1.0, float(np.abs(dw_ref).max()))
        np.testing.assert_allclose(dx.cpu().numpy(), dx_ref, rtol=tol * 5, atol=tol * 50)
        np.testing.assert_allclose(dw.cpu().numpy(), dw_ref, rtol=tol * 5, atol=tol * 5 * scale)
        np.testing.assert_allclose(db.cpu().numpy(), db_ref, rtol=tol * 5, atol=tol * 5 * scale)


def test_batch_norm_refused_geometry_leaves_running_estimates_alone(be):
    """A geometry the kernels cannot take is refused before anything is launched: the running estimates keep
    their values (the call's only side effect besides its outputs)."""
    import ctypes as C
    rm = torch.full((4,), 3.0, device=be.device)
    rv = torch.full((4,), 5.0, device=be.device)
    x = torch.zeros(16, device=be.device)
    rc = be.lib.mtb200_batch_norm_fwd(be._h, 0, 2 ** 31, 4, 2, C.c_void_p(x.data_ptr()), None, None,
                                      C.c_void_p(rm.data_ptr()), C.c_void_p(rv.data_ptr()), 1, 0.1, 1e-5,
                                      C.c_void_p(x.data_ptr()), None, None)
    assert rc == 1
    be.sync()
    assert float(rm.min()) == 3.0 == float(rm.max()) and float(rv.min()) == 5.0 == float(rv.max())


def test_batch_norm_known_answers_and_layers(be, golden):
    import minitensor_b200.nn as nn
    import minitensor_b200.tensor as mt
    for case in golden["batch_norm"]:
        if case.get("eval_only"):
            rm = mt.Tensor(np.array(case["running_mean"], np.float32))
            rv = mt.Tensor(np.array(case["running_var"], np.float32))
        else:
            x = mt.Tensor(np.array(case["train_x"], np.float32))
            c = x.shape[1]
            rm, rv = mt.Tensor(np.zeros(c, np.float32)), mt.Tensor(np.ones(c, np.float32))
            w = mt.Tensor(np.array(case["weight"], np.float32)) if "weight" in case else None
            b = mt.Tensor(np.array(case["bias"], np.float32)) if "bias" in case else None
            y = nn.batch_norm(x, rm, rv, w, b, training=True, momentum=case["momentum"], eps=case["eps"])
            if "train_y" in case:
                np.testing.assert_allclose(y.numpy(), case["train_y"], rtol=0, atol=case["atol"])
            if "running_mean_after" in case:
                np.testing.assert_allclose(rm.numpy(), case["running_mean_after"], rtol=0, atol=case["atol"])
            if "running_var_after" in case:
                np.testing.assert_allclose(rv.numpy(), case["running_var_after"], rtol=0, atol=case["atol"])
        if "eval_x" in case:
            y = nn.batch_norm(mt.Tensor(np.array(case["eval_x"], np.float32)), rm, rv, training=False, eps=case["eps"])
            np.testing.assert_allclose(y.numpy(), case["eval_y"], rtol=0, atol=case["atol"])
    # layers: tests/nn/test_layers.py:48-70
    layer = nn.BatchNorm1d(2)
    out = layer(mt.Tensor(np.array([[1.0, 2.0], [3.0, 4.0]], np.float32))).numpy()
    assert np.allclose(out.mean(axis=0), 0.0, atol=1e-5) and np.allclose(out.var(axis=0), 1.0, atol=1e-4)
    assert layer.running_mean.numpy()[0] != 0.0
    before = layer.running_mean.numpy().copy()
    layer.eval()
    layer(mt.Tensor(np.array([[5.0, 6.0], [7.0, 8.0]], np.float32)))
    np.testing.assert_array_equal(layer.running_mean.numpy(), before)
    l2 = nn.BatchNorm2d(3)
    x = mt.Tensor(np.random.default_rng(0).standard_normal((2, 3, 4, 4)).astype(np.float32), requires_grad=True)
    y = l2(x)
    assert np.all(y.numpy().var(axis=(0, 2, 3)) > 0)
    y.sum().backward()
    assert np.abs(x.grad.numpy()).max() < 1e-4        # the sum of a normalised batch does not depend on x
    np.testing.assert_allclose(l2.bias.grad.numpy(), [32.0, 32.0, 32.0])
    with pytest.raises(ValueError):
        layer(mt.Tensor(np.zeros((4, 3), np.float32)))
    with pytest.raises(ValueError):
        layer(mt.Tensor(np.zeros(2, np.float32)))


# ------------------------------------------------------------------ dropout
def test_dropout_mask_equals_oracle_and_layers(be, orc):
    import minitensor_b200.nn as nn
    import minitensor_b200.tensor as mt
    for p, seed, off in [(0.3, 42, 0), (0.5, 7, 12345), (0.9, 1, 0), (0.0, 3, 0), (1.0, 3, 0)]:
        m = be.dropout_mask(100_003, p, seed, off)
        be.sync()
        np.testing.assert_array_equal(m.cpu().numpy(), orc.dropout_mask(100_003, p, seed, off))
    m64 = be.dropout_mask(1000, 0.25, 5, 0, torch.float64).cpu().numpy()
    assert set(np.unique(m64)) <= {0.0, 1.0 / 0.75}
    x_np = np.array([[1.0, 2.0], [3.0, 4.0]], np.float32)
    x = mt.Tensor(x_np)
    assert np.array_equal(nn.dropout(x, 0.0, True).numpy(), x_np)            # tests/nn/test_functional.py:498-506
    assert not nn.dropout(x, 1.0, True).numpy().any()
    assert np.array_equal(nn.dropout(x, 0.5, False).numpy(), x_np)
    big = mt.Tensor(np.ones((512, 1024), np.float32), requires_grad=True)
    y = nn.dropout(big, 0.3, True, seed=11)
    kept = (y.numpy() != 0)
    assert abs(kept.mean() - 0.7) < 0.01
    np.testing.assert_allclose(y.numpy()[kept], 1.0 / 0.7, rtol=1e-6)
    y.sum().backward()
    np.testing.assert_array_equal(big.grad.numpy(), y.numpy())               # the same mask scales the gradient
    np.testing.assert_array_equal(nn.dropout(big, 0.3, True, seed=11).numpy(), y.numpy())
    nn.manual_seed(5)
    a = nn.Dropout(0.5)(big).numpy()
    b = nn.Dropout(0.5)(big).numpy()
    nn.manual_seed(5)
    assert np.array_equal(nn.Dropout(0.5)(big).numpy(), a) and not np.array_equal(a, b)
    img = mt.Tensor(np.ones((8, 16, 5, 7), np.float32))
    z = nn.Dropout2d(0.5)(img).numpy()
    per_channel = z.reshape(8, 16, -1)
    assert np.all((per_channel == per_channel[:, :, :1]).all(axis=2))        # whole channels kept or dropped
    assert 0 < (per_channel[:, :, 0] == 0).mean() < 1
    with pytest.raises(ValueError):
        nn.Dropout2d(0.5)(big)
    with pytest.raises(ValueError):
        nn.Dropout(1.5)


def test_dropout_apply_equals_mask_product(be, orc, rng):
    """The fused call (mask generated on the fly) equals x * oracle mask for both mask shapes and odd offsets."""
    x = rng.standard_normal(100_001).astype(np.float32)
    for p, seed, off in [(0.3, 42, 0), (0.5, 9, 7), (0.0, 1, 0), (1.0, 1, 0)]:
        y = be.dropout_apply(dev(be, x), p, seed, off)
        be.sync()
        np.testing.assert_array_equal(y.cpu().numpy(), x * orc.dropout_mask(x.size, p, seed, off))
    img = rng.standard_normal((4, 6, 5, 7)).astype(np.float32)
    y = be.dropout_apply(dev(be, img), 0.4, 3, 0, inner=35)
    be.sync()
    mask = orc.dropout_mask(24, 0.4, 3, 0).reshape(4, 6, 1, 1)
    np.testing.assert_array_equal(y.cpu().numpy(), img * mask)
    x64 = rng.standard_normal(1001)
    y64 = be.dropout_apply(dev(be, x64), 0.25, 5)
    be.sync()
    np.testing.assert_array_equal(y64.cpu().numpy() != 0, orc.dropout_mask(1001, 0.25, 5) != 0)
