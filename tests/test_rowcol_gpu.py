"""Column sum (bias gradient), activations, cross entropy and Adam on the device vs the oracle."""
import math

import numpy as np
import pytest
import torch

from conftest import fval

pytestmark = pytest.mark.gpu


def dev(be, a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(be.device)


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("m,n", [(1, 1), (33, 7), (32, 128), (32, 10), (1000, 130), (4096, 515), (65536, 64)])
def test_colsum_matches_oracle(be, orc, rng, dtype, m, n):
    x = rng.standard_normal((m, n)).astype(dtype)
    got = be.colsum(dev(be, x))
    again = be.colsum(dev(be, x))
    be.sync()
    assert torch.equal(got, again)  # deterministic
    ref = orc.sum_dim0(x)           # ascending-row f32 sum; the reference's own order is rayon-dependent
    exact = x.astype(np.float64).sum(0)
    tol = (1e-6 if dtype == np.float32 else 1e-14) * np.abs(x).astype(np.float64).sum(0) + 1e-30
    assert np.all(np.abs(got.cpu().numpy() - exact) <= tol)
    assert np.all(np.abs(ref - exact) <= 64 * tol)


def test_colsum_empty_rows(be):
    out = be.colsum(torch.empty((0, 5), dtype=torch.float32, device=be.device))
    be.sync()
    assert not out.cpu().numpy().any()


def test_relu_forward_backward_known_answer(be, golden):
    for case in golden["relu_backward"]:
        x = np.array([fval(v) for v in case["x"]], np.float32)
        go = np.array([fval(v) for v in case["grad_out"]], np.float32)
        y = be.act_fwd(dev(be, x), 1)
        gi = be.act_bwd(y, dev(be, go), 1).cpu().numpy()
        exp = np.array([fval(v) for v in case["grad_in"]], np.float32)
        np.testing.assert_array_equal(np.isnan(gi), np.isnan(exp))
        np.testing.assert_array_equal(gi[~np.isnan(exp)], exp[~np.isnan(exp)])
        yn = y.cpu().numpy()
        assert yn[0] == 0 and np.isnan(yn[1]) and yn[2] == 1


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_activations_match_oracle(be, orc, rng, dtype):
    x = (rng.standard_normal(10007) * 3).astype(dtype)
    go = rng.standard_normal(10007).astype(dtype)
    y, mask = orc.relu(x)
    yd = be.act_fwd(dev(be, x), 1)
    np.testing.assert_array_equal(yd.cpu().numpy(), y)
    np.testing.assert_array_equal(be.act_bwd(yd, dev(be, go), 1).cpu().numpy(), orc.relu_backward(mask, go))
    rtol = 2e-6 if dtype == np.float32 else 1e-13
    for act, approx in ((2, False), (3, True)):
        np.testing.assert_allclose(be.act_fwd(dev(be, x), act).cpu().numpy(), orc.gelu(x, approx), rtol=rtol,
                                   atol=rtol)
        np.testing.assert_allclose(be.act_bwd(dev(be, x), dev(be, go), act).cpu().numpy(),
                                   orc.gelu_backward(x, go, approx), rtol=rtol, atol=rtol)


def test_gelu_reference_points(be, golden):
    import minitensor_b200.tensor as mt
    for case in golden["gelu"]:
        data = np.array(case["x"], np.float32)
        t = mt.Tensor(data, requires_grad=True)
        out = t.gelu(approximate=case["approximate"])
        out.sum().backward()
        if case["approximate"] == "tanh":
            k = np.sqrt(np.array(2.0 / np.pi, dtype=data.dtype))
            inner = k * (data + 0.044715 * data ** 3)
            th = np.tanh(inner)
            exp = 0.5 * data * (1.0 + th)
            expg = 0.5 * (1.0 + th) + 0.5 * data * (1.0 - th ** 2) * k * (1.0 + 3.0 * 0.044715 * data ** 2)
        else:
            erfv = np.array([math.erf(float(v)) for v in (data / np.sqrt(np.float32(2.0)))], dtype=data.dtype)
            exp = 0.5 * data * (1.0 + erfv)
            expg = 0.5 * (1.0 + erfv) + data * np.exp(-0.5 * data ** 2) / np.sqrt(np.float32(2.0 * np.pi))
        np.testing.assert_allclose(out.numpy(), exp, rtol=case["rtol"], atol=max(case["atol"], 1e-7))
        np.testing.assert_allclose(t.grad.numpy(), expg, rtol=case["rtol"], atol=max(case["atol"], 1e-7))


@pytest.mark.parametrize("bsz,ncls", [(32, 10), (7, 33), (100, 1000), (1, 2), (513, 5)])
@pytest.mark.parametrize("label_dtype", [np.int64, np.int32])
def test_cross_entropy_matches_oracle(be, orc, rng, bsz, ncls, label_dtype):
    logits = (rng.standard_normal((bsz, ncls)) * 3).astype(np.float32)
    labels = rng.integers(0, ncls, bsz).astype(label_dtype)
    for mean in (True, False):
        loss, grad = be.cross_entropy(dev(be, logits), dev(be, labels), mean=mean)
        be.sync()
        ref_loss, ref_grad = orc.cross_entropy(logits, labels, mean=mean)
        assert abs(float(loss.item()) - float(ref_loss)) <= 2e-6 * max(1.0, abs(float(ref_loss)))
        np.testing.assert_allclose(grad.cpu().numpy(), ref_grad, rtol=1e-5, atol=2e-6)  # expf differs by ulps


def test_cross_entropy_limits_and_bad_label(be, orc, golden):
    for case in golden["cross_entropy_limits"]:
        loss, _ = be.cross_entropy(dev(be, np.array(case["logits"], np.float32)), dev(be, np.array(case["label"])))
        be.sync()
        assert math.isinf(loss.item()) and loss.item() > 0
    loss, _ = be.cross_entropy(dev(be, np.array([[1000.0, -1000.0]], np.float32)), dev(be, np.array([0])))
    be.sync()
    assert math.isnan(loss.item())  # the reference's -inf * 0 quirk, kept
    be.cross_entropy(dev(be, np.zeros((2, 3), np.float32)), dev(be, np.array([0, 3])))
    with pytest.raises(IndexError):
        be.sync()
    be.sync()  # the flag is cleared once reported


def test_adam_bit_exact_with_oracle(be, orc, rng, golden):
    for case in golden["adam"]:
        p = dev(be, np.array(case["param"], np.float32))
        g = dev(be, np.array(case["grad"], np.float32))
        m, v = torch.zeros_like(p), torch.zeros_like(p)
        be.adam_step(p, g, m, v, lr=case["lr"], beta1=case["beta1"], beta2=case["beta2"], eps=case["eps"], step=1)
        assert np.all(np.abs(p.cpu().numpy() - case["expected"]) < case["atol"])
    n = 100003
    p0 = rng.standard_normal(n).astype(np.float32)
    for wd, dec in ((0.0, False), (0.01, False), (0.01, True)):
        pn, mn, vn = p0.copy(), np.zeros(n, np.float32), np.zeros(n, np.float32)
        pd, md, vd = dev(be, p0), dev(be, mn), dev(be, vn)
        for step in (1, 2, 3):
            g = (rng.standard_normal(n) * 10.0 ** rng.integers(-6, 2, n)).astype(np.float32)
            orc.adam_step(pn, g, mn, vn, 1e-3, 0.9, 0.999, 1e-8, weight_decay=wd, decoupled=dec, step=step)
            be.adam_step(pd, dev(be, g), md, vd, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=wd,
                         decoupled=dec, step=step)
        be.sync()
        np.testing.assert_array_equal(pd.cpu().numpy(), pn)
        np.testing.assert_array_equal(md.cpu().numpy(), mn)
        np.testing.assert_array_equal(vd.cpu().numpy(), vn)


def test_wrappers_refuse_buffers_the_library_would_misread(be, rng):
    """The C ABI reads raw dense memory: a strided view, a host tensor or a buffer of another element type is
    refused by the Python layer instead of being read as something else."""
    x = torch.from_numpy(rng.standard_normal((64, 48)).astype(np.float32)).to(be.device)
    with pytest.raises(ValueError):
        be.colsum(x.t())                                   # transposed view
    with pytest.raises(ValueError):
        be.colsum(x.cpu())                                 # host memory
    with pytest.raises(ValueError):
        be.conv2d_fwd(torch.zeros(2, 4, 6, 6, device=be.device).to(memory_format=torch.channels_last),
                      torch.zeros(3, 4, 3, 3, device=be.device), None, (1, 1), (1, 1))
    p = torch.zeros(100, dtype=torch.float64, device=be.device)
    with pytest.raises(TypeError):
        be.adam_step(p, p, p, p, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8)          # Adam is f32 only
    with pytest.raises(TypeError):
        be.sgd_step(p, torch.zeros(100, device=be.device), lr=0.1)                   # f64 parameters, f32 gradient
    with pytest.raises(TypeError):
        be.cross_entropy(torch.zeros(4, 3, dtype=torch.float64, device=be.device),
                         torch.zeros(4, dtype=torch.int64, device=be.device))
    with pytest.raises(ValueError):
        be.sgd_step(torch.zeros(10, device=be.device), torch.zeros(9, device=be.device), lr=0.1)


def test_expired_wait_is_reported_and_the_context_survives(be, rng):
    """Every wait inside the tensor-core kernels is bounded.  The self-test launches a block that waits 2 ms on a
    barrier nothing signals: the next sync reports MTB200_ERR_DEVICE_WAIT exactly once, and the handle keeps
    working (a GEMM right after gives the usual result)."""
    from minitensor_b200._lib import ERR_DEVICE_WAIT, Mtb200Error, check
    be.sync()
    check(be.lib.mtb200_selftest_wait_expiry(be._h, 2000))
    with pytest.raises(Mtb200Error) as err:
        be.sync()
    assert err.value.status == ERR_DEVICE_WAIT and "bounded wait" in str(err.value)
    be.sync()                                              # reported once, then cleared
    a = rng.standard_normal((300, 200)).astype(np.float32)
    b = rng.standard_normal((200, 260)).astype(np.float32)
    c = be.gemm(torch.from_numpy(a).to(be.device), torch.from_numpy(b).to(be.device))
    be.sync()
    ref = a.astype(np.float64) @ b.astype(np.float64)
    scale = np.linalg.norm(a, axis=1)[:, None] * np.linalg.norm(b, axis=0)[None, :]
    assert (np.abs(c.cpu().numpy() - ref) / scale).max() <= 4e-6
    with pytest.raises(ValueError):
        check(be.lib.mtb200_selftest_wait_expiry(be._h, 0))


@pytest.mark.parametrize("dtype", [np.float32, np.float64, np.int32, np.int64])
def test_add_inplace_is_the_elementwise_sum(be, rng, dtype):
    """mtb200_add_inplace: y += x, bit-exact with the host sum for floats, wrapping for integers; shapes and dtypes
    must agree (arithmetic::add_inplace refuses both mismatches)."""
    n = 100_003
    if np.issubdtype(dtype, np.integer):
        info = np.iinfo(dtype)
        x = rng.integers(info.min, info.max, n, dtype=dtype, endpoint=True)
        y = rng.integers(info.min, info.max, n, dtype=dtype, endpoint=True)
        with np.errstate(over="ignore"):
            want = (x.astype(np.uint64) + y.astype(np.uint64)).astype(np.uint32 if dtype == np.int32 else np.uint64).view(dtype)
    else:
        x, y = rng.standard_normal(n).astype(dtype), rng.standard_normal(n).astype(dtype)
        want = y + x
    yd = dev(be, y)
    out = be.add_inplace(yd, dev(be, x))
    be.sync()
    assert out.data_ptr() == yd.data_ptr()
    assert np.array_equal(out.cpu().numpy(), want)
    with pytest.raises(ValueError):
        be.add_inplace(yd, dev(be, x[:-1]))
    with pytest.raises(TypeError):
        be.add_inplace(yd, dev(be, x.astype(np.float64 if dtype != np.float64 else np.float32)))


@pytest.mark.parametrize("shape,dims", [((5, 7), (0, 1)), ((300, 1000), (0, 1)), ((33, 65), (-1, -2)), ((4, 37, 129), (1, 2)),
                                        ((6, 5, 4, 3), (0, 2)), ((2, 3, 4, 5), (1, 3)), ((3, 1, 8), (0, 2)), ((7, 9), (1, 1)),
                                        ((2, 70000, 3), (0, 1))])
@pytest.mark.parametrize("dtype", [np.float32, np.float64, np.int32])
def test_swap_dims_is_the_materialised_transpose(be, rng, shape, dims, dtype):
    """mtb200_swap_dims against numpy's swapaxes for matrix transposes (tiled kernel), batched ones and swaps of
    dimensions with others between and after them (element kernel)."""
    x = (rng.standard_normal(shape) * 100).astype(dtype)
    got = be.swap_dims(dev(be, x), *dims)
    be.sync()
    want = np.ascontiguousarray(np.swapaxes(x, *dims))
    assert tuple(got.shape) == want.shape and got.is_contiguous()
    assert np.array_equal(got.cpu().numpy(), want)
    with pytest.raises(IndexError):
        be.swap_dims(dev(be, x), 0, len(shape))


def test_tape_arithmetic_runs_on_the_library(be, rng, monkeypatch):
    """Tensor.sum, transpose, equal-shape add, broadcast gradients and gradient accumulation of the tape go through
    the library's kernels: the results match numpy, and the launch counter moves where torch arithmetic would not
    move it."""
    import minitensor_b200.tensor as mt
    a = rng.standard_normal((6, 5)).astype(np.float32)
    b = rng.standard_normal((5, 4)).astype(np.float32)
    x, w = mt.Tensor(a, requires_grad=True), mt.Tensor(b, requires_grad=True)
    before = be.launches
    y = (x @ w).transpose(0, 1)                  # [4, 6]
    z = y + y                                    # equal shapes; the same tensor feeds both operands
    loss = z.sum()
    assert be.launches - before >= 5
    loss.backward()
    assert abs(float(loss.numpy()) - 2.0 * float((a.astype(np.float64) @ b).sum())) <= 1e-4 * np.abs(a).sum() * np.abs(b).max()
    # d loss / d x = 2 * ones[6,4] @ w^T, accumulated from the two uses of y
    gx = 2.0 * np.ones((6, 4)) @ b.T.astype(np.float64)
    gw = 2.0 * a.T.astype(np.float64) @ np.ones((6, 4))
    assert np.allclose(x.grad.numpy(), gx, rtol=1e-5, atol=1e-5)
    assert np.allclose(w.grad.numpy(), gw, rtol=1e-5, atol=1e-5)
    # a second backward pass accumulates into the leaves' gradients in place
    gptr = x.grad._buf.data_ptr()
    ((x @ w).sum()).backward()
    assert x.grad._buf.data_ptr() == gptr
    assert np.allclose(x.grad.numpy(), gx * 1.5, rtol=1e-5, atol=1e-5)
    # broadcast over a leading batch dimension: the gradient of the 2-D operand is the sum over the batch
    l3 = mt.Tensor(rng.standard_normal((3, 6, 5)).astype(np.float32), requires_grad=True)
    w2 = mt.Tensor(b, requires_grad=True)
    (l3 @ w2).sum().backward()
    assert np.allclose(w2.grad.numpy(), l3.numpy().astype(np.float64).sum(0).T @ np.ones((6, 4)), rtol=1e-5, atol=1e-4)
