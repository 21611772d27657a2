"""mtb200_dense_forward / mtb200_dense_backward (shared operand preparation) against the oracle's
DenseLayer forward and MatMulBackward + bias reduction, and against the one-product-per-call path."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

TIGHT = 4e-6      # against the f64-accumulated oracle: the fp16 two-plane mode keeps 22 bits per operand
F32_TOL = 1e-4    # the path's stated tolerance, norm-scaled


def dev(be, a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(be.device)


def nerr(c, ref, a2, b2):
    """max |c - ref| / (||row of a2|| * ||column of b2||) for c = a2 @ b2."""
    na = np.linalg.norm(a2.astype(np.float64), axis=1)[:, None]
    nb = np.linalg.norm(b2.astype(np.float64), axis=0)[None, :]
    scale = na * nb
    scale[scale == 0] = 1.0
    return float((np.abs(c.astype(np.float64) - ref) / scale).max())


def run_pair(be, x, w, bias, dy, *, relu=True, need_dx=True, need_db=True, use_saved=True):
    rows, fin = x.shape
    fout = w.shape[0]
    xd, wd, dyd = dev(be, x), dev(be, w), dev(be, dy)
    nbytes = be.dense_saved_bytes(rows, fin, fout)
    saved = torch.empty(nbytes, dtype=torch.uint8, device=be.device) if (use_saved and nbytes) else None
    y = be.dense_forward(xd, wd, dev(be, bias) if bias is not None else None, 1 if relu else 0, saved=saved)
    prev = dev(be, (np.abs(x) > 0.5).astype(np.float32))   # stands for the previous layer's ReLU output
    dx, dw, db = be.dense_backward(xd, wd, dyd, saved, need_dx=need_dx, dx_epilogue=4 if need_dx else 0,
                                   dx_aux=prev if need_dx else None, need_db=need_db)
    be.sync()
    return (y.cpu().numpy(), None if dx is None else dx.cpu().numpy(), dw.cpu().numpy(),
            None if db is None else db.cpu().numpy(), nbytes)


def check_against_oracle(orc, x, w, bias, dy, y, dx, dw, db, relu=True, tol=TIGHT):
    x64, w64, dy64 = x.astype(np.float64), w.astype(np.float64), dy.astype(np.float64)
    pre = x64 @ w64.T + (bias.astype(np.float64) if bias is not None else 0.0)
    ref_y = np.maximum(pre, 0.0) if relu else pre
    assert nerr(y, ref_y, x, w.T) <= tol
    assert nerr(dw, dy64.T @ x64, dy.T, x) <= tol
    if dx is not None:
        mask = (np.abs(x) > 0.5).astype(np.float64)
        assert nerr(dx, (dy64 @ w64) * mask, dy, w) <= tol
    if db is not None:
        ref_db = dy64.sum(axis=0)
        assert np.all(np.abs(db - ref_db) <= 1e-5 * np.abs(dy64).sum(axis=0) + 1e-30)


@pytest.mark.parametrize("rows,fin,fout", [(300, 200, 260), (512, 256, 384), (1000, 130, 129)])
def test_dense_pair_matches_oracle(be, orc, rng, rows, fin, fout):
    x = rng.standard_normal((rows, fin)).astype(np.float32)
    w = rng.standard_normal((fout, fin)).astype(np.float32) / np.float32(np.sqrt(fin))
    bias = rng.standard_normal(fout).astype(np.float32)
    dy = rng.standard_normal((rows, fout)).astype(np.float32)
    y, dx, dw, db, nbytes = run_pair(be, x, w, bias, dy)
    assert nbytes > 0
    check_against_oracle(orc, x, w, bias, dy, y, dx, dw, db)
    # the oracle's reference-ordered operators agree as well (f32 accumulation: the path's stated tolerance)
    gx, gwt = orc.matmul_backward(x, np.ascontiguousarray(w.T), dy)
    assert nerr(dw, gwt.T.astype(np.float64), dy.T, x) <= F32_TOL
    np.testing.assert_allclose(db, orc.sum_dim0(dy), rtol=1e-4, atol=1e-4)


def test_dense_pair_optional_outputs_and_plain_fallback(be, orc, rng):
    rows, fin, fout = 260, 192, 320
    x = rng.standard_normal((rows, fin)).astype(np.float32)
    w = rng.standard_normal((fout, fin)).astype(np.float32)
    dy = rng.standard_normal((rows, fout)).astype(np.float32)
    y, dx, dw, db, _ = run_pair(be, x, w, None, dy, relu=False, need_dx=False, need_db=False)
    assert dx is None and db is None
    check_against_oracle(orc, x, w, None, dy, y, dx, dw, db, relu=False)
    # without a saved block both calls are the plain products: same tolerance, same interface
    y2, dx2, dw2, db2, _ = run_pair(be, x, w, None, dy, relu=False, use_saved=False)
    check_against_oracle(orc, x, w, None, dy, y2, dx2, dw2, db2, relu=False)
    np.testing.assert_array_equal(y, y2)   # the forward product is the same kernel on the same planes
    # a dimension of 128 or less: no block is asked for, the pair still works
    xs, ws, dys = x[:100], w[:, :], dy[:100]
    assert be.dense_saved_bytes(100, fin, fout) == 0
    ys, dxs, dws, dbs, nb = run_pair(be, xs, ws, None, dys, relu=False)
    assert nb == 0
    check_against_oracle(orc, xs, ws, None, dys, ys, dxs, dws, dbs, relu=False, tol=F32_TOL)


def test_dense_pair_wide_ranges_zero_rows_and_columns(be, orc, rng):
    """Rows of x, W and dY and columns of dY spanning many binades, plus empty rows / columns of dY:
    the exponent bookkeeping (integer maxima, folded row scales) stays exact and finite."""
    rows, fin, fout = 384, 256, 300
    x = rng.standard_normal((rows, fin)).astype(np.float32) * np.exp2(rng.integers(-30, 30, (rows, 1))).astype(np.float32)
    w = rng.standard_normal((fout, fin)).astype(np.float32) * np.exp2(rng.integers(-20, 20, (fout, 1))).astype(np.float32)
    dy = rng.standard_normal((rows, fout)).astype(np.float32)
    dy *= np.exp2(rng.integers(-25, 25, (rows, 1))).astype(np.float32)
    dy *= np.exp2(rng.integers(-25, 25, (1, fout))).astype(np.float32)
    dy[5] = 0.0
    dy[:, 9] = 0.0
    dy[17, 3] = np.float32(1e-42)      # a subnormal entry
    y, dx, dw, db, _ = run_pair(be, x, w, None, dy, relu=False)
    assert np.isfinite(y).all() and np.isfinite(dx).all() and np.isfinite(dw).all()
    assert not dx[5].any() and not dw[9].any() and db[9] == 0.0
    x64, w64, dy64 = x.astype(np.float64), w.astype(np.float64), dy.astype(np.float64)
    assert nerr(y, x64 @ w64.T, x, w.T) <= TIGHT
    # the folded scales bound each term's error by 2^-22 of (|dY| x row maximum of x or W): compare against the
    # magnitude sums those bounds give
    mask = (np.abs(x) > 0.5).astype(np.float64)
    bound_dw = np.abs(dy64).T @ np.abs(x64).max(axis=1, keepdims=True).repeat(fin, axis=1)
    assert np.all(np.abs(dw - dy64.T @ x64) <= 2e-5 * bound_dw + 1e-300)
    bound_dx = np.abs(dy64) @ np.abs(w64).max(axis=1, keepdims=True).repeat(fin, axis=1)
    assert np.all(np.abs(dx - (dy64 @ w64) * mask) <= 2e-5 * bound_dx + 1e-300)


def test_dense_pair_nonfinite_inputs_follow_ieee(be, rng):
    """Inf / NaN anywhere in x, W or dY: the results are those of plain f32 multiply-add (the gated redo)."""
    rows, fin, fout = 260, 200, 270
    x = rng.standard_normal((rows, fin)).astype(np.float32)
    w = rng.standard_normal((fout, fin)).astype(np.float32)
    dy = rng.standard_normal((rows, fout)).astype(np.float32)
    for where in ("x", "w", "dy"):
        xs, ws, dys = x.copy(), w.copy(), dy.copy()
        {"x": xs, "w": ws, "dy": dys}[where][7, 11] = np.inf
        {"x": xs, "w": ws, "dy": dys}[where][8, 13] = np.nan
        y, dx, dw, db, _ = run_pair(be, xs, ws, None, dys, relu=False)
        with np.errstate(invalid="ignore", over="ignore"):
            ref_y = xs.astype(np.float64) @ ws.astype(np.float64).T
            ref_dw = dys.astype(np.float64).T @ xs.astype(np.float64)
            ref_dx = (dys.astype(np.float64) @ ws.astype(np.float64)) * (np.abs(xs) > 0.5)
        for got, ref in ((y, ref_y), (dw, ref_dw), (dx, ref_dx)):
            assert np.array_equal(np.isnan(got), np.isnan(ref))
            fin_mask = np.isfinite(ref)
            assert np.array_equal(np.isinf(got), np.isinf(ref))
            assert np.allclose(got[fin_mask], ref[fin_mask], rtol=1e-3, atol=1e-3)


def test_dense_pair_argument_errors(be):
    x = torch.zeros(300, 200, device=be.device)
    w = torch.zeros(260, 200, device=be.device)
    dy = torch.zeros(300, 260, device=be.device)
    with pytest.raises(ValueError):
        be.dense_forward(x, torch.zeros(260, 199, device=be.device))
    with pytest.raises(ValueError):
        be.dense_backward(x, w, torch.zeros(300, 259, device=be.device), None)
    with pytest.raises(ValueError):                      # ReLU backward without the activation
        be.dense_backward(x, w, dy, None, dx_epilogue=4)
    with pytest.raises(ValueError):                      # forward epilogue out of range
        be.dense_forward(x, w, epilogue=4)
    with pytest.raises(TypeError):
        be.dense_forward(x.to(torch.int32), w.to(torch.int32))


def test_mlp_trainer_fused_dense_matches_oracle(be, orc):
    """A three-layer MLP wide enough for the fused pair (all dims and the batch above 128), two steps,
    fused against the oracle's reference-ordered step and against the unfused trainer."""
    from minitensor_b200.mlp import MLPTrainer, mlp_layout
    dims, batch = [200, 260, 192, 150], 320
    g = np.random.default_rng(11)
    x = g.standard_normal((batch, dims[0])).astype(np.float32)
    labels = g.integers(0, dims[-1], batch)
    _, _, total = mlp_layout(dims)
    tr0 = MLPTrainer(dims, batch, seed=5, fused_dense=False)
    init = tr0.params.cpu().numpy().copy()
    tr1 = MLPTrainer(dims, batch, init_params=init, fused_dense=True)
    assert all(s is not None for s in tr1.saved)
    params, m, v = init.copy(), np.zeros_like(init), np.zeros_like(init)
    xd, yd = dev(be, x), torch.from_numpy(labels).to(be.device)
    for step in (1, 2):
        l0, l1 = tr0.step(xd, yd), tr1.step(xd, yd)
        be.sync()
        ref_loss, ref_grads = orc.mlp_train_step(dims, x, labels, params, m, v, 1e-3, 0.9, 0.999, 1e-8, step,
                                                 want_grads=True)
        assert abs(l1.item() - ref_loss) <= 2e-5 * max(1.0, abs(ref_loss))
        scale = np.linalg.norm(x, axis=0).max()
        assert float(np.abs(tr1.grads.cpu().numpy().astype(np.float64) - ref_grads).max()) <= F32_TOL * scale
        assert float((tr1.grads - tr0.grads).abs().max()) <= 1e-5 * scale


def test_nn_dense_layer_uses_the_pair_when_training(be, orc, rng):
    """The host mirror's DenseLayer at a shape the pair serves: forward and all three gradients against the
    oracle's reference-ordered operators."""
    import minitensor_b200.nn as nn
    import minitensor_b200.tensor as mt
    layer = nn.DenseLayer(200, 260, rng=np.random.default_rng(4))
    xn = rng.standard_normal((300, 200)).astype(np.float32)
    x = mt.Tensor(xn, requires_grad=True)
    y = layer(x)
    wn, bn = layer.weight.numpy(), layer.bias.numpy()
    assert nerr(y.numpy(), orc.dense_forward(xn, wn, bn).astype(np.float64), xn, wn.T) <= F32_TOL
    go = rng.standard_normal((300, 260)).astype(np.float32)
    y.backward(mt.Tensor(go))
    gx, gwt = orc.matmul_backward(xn, np.ascontiguousarray(wn.T), go)
    assert nerr(x.grad.numpy(), gx.astype(np.float64), go, wn) <= F32_TOL
    assert nerr(layer.weight.grad.numpy(), gwt.T.astype(np.float64), go.T, xn) <= F32_TOL
    np.testing.assert_allclose(layer.bias.grad.numpy(), orc.sum_dim0(go), rtol=1e-4, atol=1e-4)


def test_mlp_trainer_overlapped_schedule_gives_identical_parameters(be):
    """The multi-GPU backward order (input-gradient chain first, parameter gradients from the first layer on,
    per-layer Adam on a side stream) on one GPU: same bits as the default order."""
    from minitensor_b200.mlp import MLPTrainer
    dims, batch = [200, 260, 192, 150], 320
    g = np.random.default_rng(12)
    x = dev(be, g.standard_normal((batch, dims[0])).astype(np.float32))
    y = torch.from_numpy(g.integers(0, dims[-1], batch)).to(be.device)
    a = MLPTrainer(dims, batch, seed=3)
    b = MLPTrainer(dims, batch, seed=3, overlap_comm=True)
    assert not a.overlap_comm and b.overlap_comm
    for _ in range(3):
        la, lb = a.step(x, y), b.step(x, y)
    be.sync()
    torch.cuda.synchronize()
    assert la.item() == lb.item()
    assert torch.equal(a.grads, b.grads)
    assert torch.equal(a.params, b.params) and torch.equal(a.m, b.m) and torch.equal(a.v, b.v)


def test_large_mlp_step_full_size_properties(be, orc):
    """One training step of the large MLP at its full size (8192-4096-4096-4096-1000, batch 65536):
    sampled rows of the first activation and sampled rows of the last weight gradient against f64 arithmetic,
    the identity sum_j db_last[j] = 0 (every softmax row sums to one), the loss against the logits the step
    produced, and bit-identical repeats."""
    from minitensor_b200.mlp import MLPTrainer
    dims, batch = [8192, 4096, 4096, 4096, 1000], 65536
    g = torch.Generator(device="cpu").manual_seed(31)
    x = torch.randn(batch, dims[0], generator=g).to(be.device)
    y = torch.randint(0, dims[-1], (batch,), generator=g).to(be.device)
    tr = MLPTrainer(dims, batch, seed=0)
    w1 = tr.W[0].cpu().numpy().copy()
    b1 = tr.b[0].cpu().numpy().copy()
    loss = tr.step(x, y)
    be.sync()
    logits = tr.h[3].cpu().numpy().astype(np.float64)                  # the loss against the logits the step produced
    lse = np.log(np.exp(logits - logits.max(axis=1, keepdims=True)).sum(axis=1)) + logits.max(axis=1)
    ref_loss = float((lse - logits[np.arange(batch), y.cpu().numpy()]).mean())
    assert abs(loss.item() - ref_loss) <= 2e-5 * ref_loss
    assert np.log(1000.0) - 0.5 < ref_loss < np.log(1000.0) + 4.0      # random labels at initialisation
    del logits, lse
    rows = np.random.default_rng(2).choice(batch, 4, replace=False)
    xr = x[rows].cpu().numpy()
    ref_h1 = np.maximum(xr.astype(np.float64) @ w1.astype(np.float64).T + b1, 0.0)
    assert nerr(tr.h[0][rows].cpu().numpy(), ref_h1, xr, w1.T) <= TIGHT
    db_last = tr.db[3].cpu().numpy().astype(np.float64)
    assert abs(db_last.sum()) <= 1e-5 * np.abs(db_last).sum() + 1e-7
    # dW_last[o, :] = sum_b g[b, o] * h3[b, :] for three sampled outputs (g = dlogits is still in the trainer)
    outs = [0, 499, 999]
    gcols = tr.g[3][:, outs].cpu().numpy().astype(np.float64)          # [batch, 3]
    h3 = tr.h[2].cpu().numpy()
    ref_dw = gcols.T @ h3.astype(np.float64)
    got = tr.dW[3][outs].cpu().numpy()
    scale = np.linalg.norm(gcols, axis=0)[:, None] * np.linalg.norm(h3.astype(np.float64), axis=0)[None, :]
    assert float((np.abs(got - ref_dw) / scale).max()) <= F32_TOL
    grads_first = tr.grads.clone()
    tr2 = MLPTrainer(dims, batch, seed=0)
    tr2.step(x, y)
    be.sync()
    assert torch.equal(tr2.grads, grads_first) and torch.equal(tr2.params, tr.params)


def test_dense_backward_in_two_calls_with_a_carried_dy_block(be, rng):
    """dy_mode 1 (input and bias gradient now, dY's weight-gradient operand kept) followed by dy_mode 2 (weight
    gradient from the kept block, dY not read) gives the bits of the single call; misuse is refused."""
    rows, fin, fout = 384, 256, 300
    x = dev(be, rng.standard_normal((rows, fin)).astype(np.float32))
    w = dev(be, rng.standard_normal((fout, fin)).astype(np.float32))
    dy = dev(be, rng.standard_normal((rows, fout)).astype(np.float32))
    saved = torch.empty(be.dense_saved_bytes(rows, fin, fout), dtype=torch.uint8, device=be.device)
    block = torch.empty(be.dense_dy_bytes(rows, fin, fout), dtype=torch.uint8, device=be.device)
    assert block.numel() > 0 and be.dense_dy_bytes(100, fin, fout) == 0
    be.dense_forward(x, w, None, 0, saved=saved)
    dx0, dw0, db0 = be.dense_backward(x, w, dy, saved)
    dx1, none_dw, db1 = be.dense_backward(x, w, dy, saved, need_dw=False, dy_block=block, dy_mode=1)
    dy_scrambled = torch.full_like(dy, float("nan"))          # the second call must not look at dY
    none_dx, dw1, none_db = be.dense_backward(x, w, dy_scrambled, saved, need_dx=False, need_db=False,
                                              dy_block=block, dy_mode=2)
    be.sync()
    assert none_dw is None and none_dx is None and none_db is None
    assert torch.equal(dx0, dx1) and torch.equal(db0, db1) and torch.equal(dw0, dw1)
    with pytest.raises(ValueError):
        be.dense_backward(x, w, dy, saved, dy_block=block, dy_mode=1)                       # dW asked for in mode 1
    with pytest.raises(ValueError):
        be.dense_backward(x, w, dy, saved, need_dx=False, dy_block=block, dy_mode=2)        # db asked for in mode 2
    with pytest.raises(ValueError):
        be.dense_backward(x, w, dy, saved, dy_block=block, dy_mode=3)
