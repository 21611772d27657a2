"""DenseLayer / Sequential / CrossEntropy / Adam through the host mirror, against the oracle's
reference-ordered composition of the same operators."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

F32_TOL = 1e-4


def _close(got, ref, scale, tol=F32_TOL):
    return float(np.abs(got.astype(np.float64) - ref.astype(np.float64)).max()) <= tol * scale


def test_dense_layer_forward_backward(be, orc, rng):
    import minitensor_b200.nn as nn
    import minitensor_b200.tensor as mt
    layer = nn.DenseLayer(20, 13, rng=np.random.default_rng(1))
    assert layer.weight.shape == (13, 20) and not layer.bias.numpy().any()   # [out, in], zero bias
    xn = rng.standard_normal((9, 20)).astype(np.float32)
    bn = rng.standard_normal(13).astype(np.float32)
    layer.bias = mt.Tensor(bn, requires_grad=True)
    x = mt.Tensor(xn, requires_grad=True)
    y = layer(x)
    wn = layer.weight.numpy()
    ref = orc.dense_forward(xn, wn, bn)
    np.testing.assert_allclose(y.numpy(), ref, rtol=1e-5, atol=1e-5)
    go = rng.standard_normal((9, 13)).astype(np.float32)
    y.backward(mt.Tensor(go))
    gx, gwt = orc.matmul_backward(xn, np.ascontiguousarray(wn.T), go)
    np.testing.assert_allclose(x.grad.numpy(), gx, rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(layer.weight.grad.numpy(), gwt.T, rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(layer.bias.grad.numpy(), orc.sum_dim0(go), rtol=1e-5, atol=1e-5)
    # functional form, 3-D input, and the checks of dense_layer.rs:142-154
    x3 = mt.Tensor(rng.standard_normal((2, 4, 20)).astype(np.float32))
    assert nn.dense_layer(x3, layer.weight, layer.bias).shape == (2, 4, 13)
    with pytest.raises(ValueError):
        layer(mt.Tensor(np.zeros((3, 19), np.float32)))
    with pytest.raises(ValueError):
        layer(mt.Tensor(np.zeros(20, np.float32)))


def test_sequential_fused_equals_unfused(be, rng):
    import minitensor_b200.nn as nn
    import minitensor_b200.tensor as mt
    g = np.random.default_rng(2)
    layers = [nn.DenseLayer(30, 40, rng=g), nn.ReLU(), nn.DenseLayer(40, 7, rng=g)]
    xn = rng.standard_normal((11, 30)).astype(np.float32)
    outs, grads = [], []
    for fuse in (True, False):
        for p in layers[0].parameters() + layers[2].parameters():
            p.grad = None
        model = nn.Sequential(layers, fuse=fuse)
        x = mt.Tensor(xn, requires_grad=True)
        y = model(x)
        y.sum().backward()
        outs.append(y.numpy())
        grads.append([x.grad.numpy()] + [p.grad.numpy() for p in model.parameters()])
    np.testing.assert_array_equal(outs[0], outs[1])          # the fused epilogue changes nothing
    for a, b in zip(grads[0], grads[1]):
        np.testing.assert_array_equal(a, b)


def _config2(seed):
    """784 -> 128 -> ReLU -> 10, batch 32, N(0,1) inputs, labels in [0,10), Kaiming-uniform weights."""
    g = np.random.default_rng(seed)
    x = g.standard_normal((32, 784)).astype(np.float32)
    labels = g.integers(0, 10, 32)
    w1 = g.uniform(-1, 1, (128, 784)).astype(np.float32) * np.float32(np.sqrt(6.0 / 784))
    w2 = g.uniform(-1, 1, (10, 128)).astype(np.float32) * np.float32(np.sqrt(6.0 / 128))
    return x, labels, w1.astype(np.float32), np.zeros(128, np.float32), w2.astype(np.float32), np.zeros(10, np.float32)


def test_mlp_step_config2_via_nn_and_optim(be, orc):
    """One Adam step (lr 1e-3, betas 0.9/0.999, eps 1e-8) of the small MLP through nn/optim:
    loss, every gradient, updated parameters against the oracle's reference-ordered step."""
    import minitensor_b200.nn as nn
    import minitensor_b200.optim as optim
    import minitensor_b200.tensor as mt
    x, labels, w1, b1, w2, b2 = _config2(7)
    l1, l2 = nn.DenseLayer(784, 128), nn.DenseLayer(128, 10)
    l1.weight, l1.bias = mt.Tensor(w1, requires_grad=True), mt.Tensor(b1, requires_grad=True)
    l2.weight, l2.bias = mt.Tensor(w2, requires_grad=True), mt.Tensor(b2, requires_grad=True)
    model = nn.Sequential([l1, nn.ReLU(), l2])
    opt = optim.Adam(model.parameters(), lr=1e-3, betas=(0.9, 0.999), epsilon=1e-8)
    loss = nn.CrossEntropyLoss()(model(mt.Tensor(x)), mt.Tensor(labels))
    loss.backward()
    got_grads = np.concatenate([p.grad.numpy().ravel() for p in model.parameters()])
    opt.step()
    got_params = np.concatenate([p.numpy().ravel() for p in model.parameters()])

    params = np.concatenate([w1.ravel(), b1, w2.ravel(), b2]).astype(np.float32)
    m, v = np.zeros_like(params), np.zeros_like(params)
    ref_loss, ref_grads = orc.mlp_train_step([784, 128, 10], x, labels, params, m, v, 1e-3, 0.9, 0.999, 1e-8, 1,
                                             want_grads=True)
    assert abs(loss.item() - ref_loss) <= 1e-5
    # gradients are sums of <= 32 (batch) or 128 products of O(1) factors: scale by those norms
    assert _close(got_grads, ref_grads, scale=np.linalg.norm(x, axis=0).max() * 1.0)
    # Adam's first step moves every weight by ~lr * sign(g); where |g| is at rounding level the sign is noise
    big = np.abs(ref_grads) > 1e-6
    np.testing.assert_allclose(got_params[big], params[big], rtol=0, atol=2e-5)
    assert np.all(np.abs(got_params - params) <= 2.1e-3)
    opt.zero_grad()
    assert all(p.grad is None for p in model.parameters())


def test_mlp_trainer_matches_oracle_three_steps(be, orc):
    """The flat-buffer trainer (the multi-GPU building block) for three steps of the small MLP."""
    from minitensor_b200.mlp import MLPTrainer
    x, labels, w1, b1, w2, b2 = _config2(7)
    init = np.concatenate([w1.ravel(), b1, w2.ravel(), b2]).astype(np.float32)
    tr = MLPTrainer([784, 128, 10], 32, lr=1e-3, init_params=init)
    params, m, v = init.copy(), np.zeros_like(init), np.zeros_like(init)
    xd = torch.from_numpy(x).to(be.device)
    yd = torch.from_numpy(labels).to(be.device)
    for step in (1, 2, 3):
        loss = tr.step(xd, yd)
        be.sync()
        ref_loss, ref_grads = orc.mlp_train_step([784, 128, 10], x, labels, params, m, v, 1e-3, 0.9, 0.999, 1e-8,
                                                 step, want_grads=True)
        assert abs(loss.item() - ref_loss) <= 2e-5 * max(1.0, abs(ref_loss))
        assert _close(tr.grads.cpu().numpy(), ref_grads, scale=np.linalg.norm(x, axis=0).max())
    # the loss goes down, as in the reference's training smoke tests
    first = orc.mlp_train_step([784, 128, 10], x, labels, init.copy(), np.zeros_like(init), np.zeros_like(init),
                               0.0, 0.9, 0.999, 1e-8, 1)[0]
    assert ref_loss < first


def test_mlp_trainer_host_batches(be):
    """prefetch() + step_slot(): batches that arrive in pinned host memory give the same result."""
    from minitensor_b200.mlp import MLPTrainer
    x, labels, w1, b1, w2, b2 = _config2(3)
    init = np.concatenate([w1.ravel(), b1, w2.ravel(), b2]).astype(np.float32)
    a = MLPTrainer([784, 128, 10], 32, init_params=init)
    b = MLPTrainer([784, 128, 10], 32, init_params=init)
    xh, yh = torch.from_numpy(x).pin_memory(), torch.from_numpy(labels).pin_memory()
    la = a.step(xh.to(be.device), yh.to(be.device))
    lb = b.step_slot(b.prefetch(xh, yh))
    be.sync()
    assert la.item() == lb.item()
    assert torch.equal(a.params, b.params)


@pytest.mark.parametrize("dims,batch", [([784, 128, 10], 32), ([200, 260, 192, 150], 320)])
def test_mlp_trainer_graph_replay_equals_eager_steps(be, dims, batch):
    """capture(): the step recorded into a CUDA graph, replayed, gives the same bits as eager steps, with
    Adam's step count advancing on the device."""
    from minitensor_b200.mlp import MLPTrainer
    g = np.random.default_rng(21)
    xs = [torch.from_numpy(g.standard_normal((batch, dims[0])).astype(np.float32)).to(be.device) for _ in range(4)]
    ys = [torch.from_numpy(g.integers(0, dims[-1], batch)).to(be.device) for _ in range(4)]
    a = MLPTrainer(dims, batch, seed=9)
    b = MLPTrainer(dims, batch, seed=9)
    with pytest.raises(RuntimeError):
        b.capture(xs[0], ys[0])                       # needs one eager step first
    losses_a = [a.step(x, y).item() for x, y in zip(xs, ys)]
    xb, yb = xs[0].clone(), ys[0].clone()
    losses_b = [b.step(xb, yb).item()]
    replay = b.capture(xb, yb)
    for x, y in zip(xs[1:], ys[1:]):
        xb.copy_(x)
        yb.copy_(y)
        losses_b.append(replay().item())
    be.sync()
    torch.cuda.synchronize()
    assert b.step_count == 4
    assert losses_a == losses_b
    assert torch.equal(a.params, b.params) and torch.equal(a.m, b.m) and torch.equal(a.v, b.v)
    # eager steps still work after a capture
    la, lb = a.step(xs[0], ys[0]).item(), b.step(xs[0], ys[0]).item()
    assert la == lb and torch.equal(a.params, b.params)


def test_mlp_trainer_checkpoint_resume(be, tmp_path):
    """Save after two steps, restore into a fresh trainer, continue: same bits as the uninterrupted run."""
    from minitensor_b200.mlp import MLPTrainer
    from minitensor_b200.checkpoint import load_mlp_trainer, save_mlp_trainer
    x, labels, *_ = _config2(5)
    xd, yd = torch.from_numpy(x).to(be.device), torch.from_numpy(labels).to(be.device)
    a = MLPTrainer([784, 128, 10], 32, seed=2)
    for _ in range(2):
        a.step(xd, yd)
    path = str(tmp_path / "mlp.json")
    save_mlp_trainer(a, path)
    b = MLPTrainer([784, 128, 10], 32, seed=99)
    load_mlp_trainer(b, path)
    assert b.step_count == 2 and torch.equal(a.params, b.params) and torch.equal(a.m, b.m)
    la, lb = a.step(xd, yd).item(), b.step(xd, yd).item()
    be.sync()
    assert la == lb and torch.equal(a.params, b.params) and torch.equal(a.v, b.v)
