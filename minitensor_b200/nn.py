"""Mirror of the ``minitensor.nn`` pieces on the dense-contraction path.

``DenseLayer`` / ``dense_layer`` (``engine/src/nn/dense_layer.rs:24-188``,
``bindings/src/nn/module.rs:69-94``), ``ReLU`` / ``GELU``
(``engine/src/nn/activation.rs:88-91,378-390``), ``Sequential``
(``engine/src/nn/sequential.rs:74-83``), ``Conv2d`` / ``conv2d``
(``engine/src/nn/conv.rs:24-226``, ``engine/src/operations/conv.rs:24-206``),
``cross_entropy`` / ``CrossEntropyLoss`` (``engine/src/nn/loss.rs:434-436``,
``engine/src/operations/loss/regression.rs:178-251``).

What differs from the reference is only where the arithmetic happens: the
bias add (and a directly following ReLU / GELU inside ``Sequential``) is the
epilogue of the GEMM kernel, the weight transpose is a descriptor choice, and
the backward products are launched without materialised transposes.
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple, Union

import numpy as np
import torch

from ._lib import EPI_GELU_ERF, EPI_GELU_TANH, EPI_NONE, EPI_RELU, EPI_RELU_BWD
from .tensor import Tensor, _be

_Pair = Union[int, Tuple[int, int]]


def _pair(v: _Pair, name: str) -> Tuple[int, int]:
    """int-or-pair parsing of ``bindings/src/nn/module.rs:96-137``."""
    if isinstance(v, int):
        return (v, v)
    if isinstance(v, (tuple, list)) and len(v) == 2 and all(isinstance(i, int) for i in v):
        return (int(v[0]), int(v[1]))
    raise ValueError(f"{name} must be an int or a pair of ints")


# ---------------------------------------------------------------------- init
def _uniform(shape, bound: float, dtype: str, rng: Optional[np.random.Generator]) -> np.ndarray:
    rng = rng or np.random.default_rng()
    return rng.uniform(-bound, bound, size=shape).astype(dtype)


def xavier_uniform(shape, dtype="float32", rng=None) -> np.ndarray:
    """bound = sqrt(6 / (fan_in + fan_out)) (``engine/src/nn/init.rs:393-443``)."""
    fan_in, fan_out = _fans(shape)
    return _uniform(shape, math.sqrt(6.0 / (fan_in + fan_out)), dtype, rng)


def he_uniform(shape, dtype="float32", rng=None) -> np.ndarray:
    """bound = sqrt(6 / fan_in) (``engine/src/nn/init.rs:419-430``)."""
    fan_in, _ = _fans(shape)
    return _uniform(shape, math.sqrt(6.0 / fan_in), dtype, rng)


def _normal(shape, std: float, dtype: str, rng: Optional[np.random.Generator]) -> np.ndarray:
    rng = rng or np.random.default_rng()
    return (rng.standard_normal(size=shape) * std).astype(dtype)


def he_normal(shape, dtype="float32", rng=None) -> np.ndarray:
    """Kaiming-normal: mean 0, std = sqrt(2 / fan_in) (``engine/src/nn/init.rs:432-443``,
    ``InitMethod::HeNormal`` at ``:37,68``) - the distribution of the large conv config's weights."""
    fan_in, _ = _fans(shape)
    return _normal(shape, math.sqrt(2.0 / fan_in), dtype, rng)


def xavier_normal(shape, dtype="float32", rng=None) -> np.ndarray:
    """std = sqrt(2 / (fan_in + fan_out)) (``engine/src/nn/init.rs:406-417``)."""
    fan_in, fan_out = _fans(shape)
    return _normal(shape, math.sqrt(2.0 / (fan_in + fan_out)), dtype, rng)


def init_tensor(method, shape, dtype="float32", rng=None) -> np.ndarray:
    """``InitMethod::init_tensor`` (``engine/src/nn/init.rs:14-74``).  ``method`` is a name - "zeros", "ones",
    "xavier_uniform", "xavier_normal", "he_uniform", "he_normal", "lecun_uniform", "lecun_normal" - or a tuple
    ("constant", v), ("uniform", a, b), ("normal", mean, std)."""
    name, args = (method, ()) if isinstance(method, str) else (method[0], tuple(method[1:]))
    fan_in, _ = _fans(shape)
    if name == "zeros":
        return np.zeros(shape, dtype=dtype)
    if name == "ones":
        return np.ones(shape, dtype=dtype)
    if name == "constant":
        return np.full(shape, args[0], dtype=dtype)
    if name == "uniform":
        return (rng or np.random.default_rng()).uniform(args[0], args[1], size=shape).astype(dtype)
    if name == "normal":
        return (args[0] + _normal(shape, args[1], "float64", rng)).astype(dtype)
    if name == "xavier_uniform":
        return xavier_uniform(shape, dtype, rng)
    if name == "xavier_normal":
        return xavier_normal(shape, dtype, rng)
    if name == "he_uniform":
        return he_uniform(shape, dtype, rng)
    if name == "he_normal":
        return he_normal(shape, dtype, rng)
    if name == "lecun_uniform":
        return _uniform(shape, math.sqrt(3.0 / fan_in), dtype, rng)
    if name == "lecun_normal":
        return _normal(shape, math.sqrt(1.0 / fan_in), dtype, rng)
    raise ValueError(f"unknown initialisation method {method!r}")


def _fans(shape) -> Tuple[int, int]:
    """calculate_fan_in_fan_out (``engine/src/nn/init.rs:471-491``): scalar (1, 1); vector (d0, d0); matrix
    (d1, d0); beyond that dims[1] and dims[0] times the receptive field."""
    shape = tuple(int(d) for d in shape)
    if len(shape) == 0:
        return 1, 1
    if len(shape) == 1:
        return shape[0], shape[0]
    recept = int(np.prod(shape[2:])) if len(shape) > 2 else 1
    return shape[1] * recept, shape[0] * recept


# ---------------------------------------------------------------------- dense
def dense_layer(input: Tensor, weight: Tensor, bias: Optional[Tensor] = None, *, _epilogue: int = EPI_NONE) -> Tensor:
    """``input @ weight^T + bias`` with ``weight`` stored ``[out_features, in_features]``."""
    if input.ndim < 2:
        raise ValueError("DenseLayer expects input with at least 2 dimensions")
    out_f, in_f = weight.shape
    if input.shape[-1] != in_f:
        raise ValueError(f"shape mismatch: expected last dim {in_f}, got {input.shape[-1]}")
    if input.dtype != weight.dtype or (bias is not None and bias.dtype != weight.dtype):
        raise TypeError("type mismatch between input, weight and bias")
    be = _be()
    x2 = input._buf.reshape(-1, in_f)
    bbuf = bias._buf if bias is not None else None
    # training: keep the prepared operands for the backward products (mtb200_dense_forward / _backward)
    saved = None
    if weight.requires_grad and x2.is_contiguous():
        nbytes = be.dense_saved_bytes(x2.shape[0], in_f, out_f, x2.dtype)
        if nbytes:
            saved = torch.empty(nbytes, dtype=torch.uint8, device=x2.device)
    if saved is not None:
        y2 = be.dense_forward(x2, weight._buf, bbuf, _epilogue, saved=saved)
    else:
        y2 = be.gemm(x2, weight._buf, trans_b=True, bias=bbuf, epilogue=_epilogue)
    out_shape = input.shape[:-1] + (out_f,)
    parents = (input, weight) + ((bias,) if bias is not None else ())

    def bw(g):
        g2 = g.reshape(-1, out_f).contiguous()
        if _epilogue == EPI_RELU:
            g2 = be.act_bwd(y2, g2, EPI_RELU)
        elif _epilogue in (EPI_GELU_ERF, EPI_GELU_TANH):
            raise RuntimeError("fused GELU keeps no pre-activation; use the unfused layer for training")
        want_b = bias is not None and bias.requires_grad
        if saved is not None:
            gx, gw, gb = be.dense_backward(x2, weight._buf, g2, saved, need_dx=input.requires_grad, need_db=want_b)
            gx = gx.reshape(input.shape) if gx is not None else None
            return (gx, gw, gb)[: len(parents)]
        gx = be.gemm(g2, weight._buf).reshape(input.shape) if input.requires_grad else None   # dX = dY W
        gw = be.gemm(g2, x2, trans_a=True) if weight.requires_grad else None                  # dW = dY^T X
        gb = be.colsum(g2) if want_b else None
        return (gx, gw, gb)[: len(parents)]

    return input._result(y2.reshape(out_shape), parents, bw)


class Module:
    def parameters(self) -> List[Tensor]:
        return []

    def __call__(self, x: Tensor) -> Tensor:
        return self.forward(x)


class DenseLayer(Module):
    """Weight ``[out, in]`` Xavier-uniform, bias zeros (``dense_layer.rs:47-49``, ``init.rs:503-506``);
    ``weight_init`` / ``bias_init`` choose other methods as ``DenseLayer::new_with_init`` does
    (``dense_layer.rs:68-100``; see :func:`init_tensor` for the names)."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, dtype: str = "float32",
                 rng: Optional[np.random.Generator] = None, weight_init="xavier_uniform", bias_init="zeros"):
        if in_features <= 0 or out_features <= 0:
            raise ValueError("in_features and out_features must be positive")
        self.in_features, self.out_features = in_features, out_features
        self.weight = Tensor(init_tensor(weight_init, (out_features, in_features), dtype, rng), requires_grad=True)
        self.bias = Tensor(init_tensor(bias_init, (out_features,), dtype, rng), requires_grad=True) if bias else None

    def forward(self, x: Tensor, _epilogue: int = EPI_NONE) -> Tensor:
        return dense_layer(x, self.weight, self.bias, _epilogue=_epilogue)

    def parameters(self) -> List[Tensor]:
        return [self.weight] + ([self.bias] if self.bias is not None else [])


class ReLU(Module):
    def forward(self, x: Tensor) -> Tensor:
        return x.relu()


class GELU(Module):
    """The layer form uses the tanh approximation (``engine/src/nn/activation.rs:378-390``)."""

    def __init__(self, approximate: str = "tanh"):
        self.approximate = approximate

    def forward(self, x: Tensor) -> Tensor:
        return x.gelu(self.approximate)


class Sequential(Module):
    """Runs layers in order; a ``DenseLayer`` directly followed by ``ReLU`` runs as one GEMM
    with the activation in its epilogue (results equal the unfused pair)."""

    def __init__(self, layers: Sequence[Module], fuse: bool = True):
        self.layers = list(layers)
        self.fuse = fuse

    def forward(self, x: Tensor) -> Tensor:
        i = 0
        while i < len(self.layers):
            layer = self.layers[i]
            nxt = self.layers[i + 1] if i + 1 < len(self.layers) else None
            if self.fuse and isinstance(layer, DenseLayer) and isinstance(nxt, ReLU):
                x = layer.forward(x, _epilogue=EPI_RELU)
                i += 2
            else:
                x = layer(x)
                i += 1
        return x

    def parameters(self) -> List[Tensor]:
        return [p for l in self.layers for p in l.parameters()]


# ---------------------------------------------------------------------- batch norm, dropout
def batch_norm(input: Tensor, running_mean: Optional[Tensor] = None, running_var: Optional[Tensor] = None,
               weight: Optional[Tensor] = None, bias: Optional[Tensor] = None, training: bool = False,
               momentum: float = 0.1, eps: float = 1e-5) -> Tensor:
    """``batch_norm`` of the reference (``engine/src/operations/normalization.rs:64-187``): channel dimension 1,
    running estimates updated in place while training."""
    if input.ndim < 2:
        raise ValueError("batch_norm expects input with at least 2 dimensions")
    c = input.shape[1]
    for t in (weight, bias, running_mean, running_var):
        if t is not None and (t.ndim != 1 or t.shape[0] != c):
            raise ValueError(f"shape mismatch: expected [{c}], got {list(t.shape)}")
    if input.dtype not in ("float32", "float64"):
        raise TypeError("batch_norm supports float32/float64 tensors")
    be = _be()
    x = input._buf.contiguous()
    wb = weight._buf if weight is not None else None
    y, mean, invstd, batch_stats = be.batch_norm_fwd(
        x, wb, bias._buf if bias is not None else None, running_mean._buf if running_mean is not None else None,
        running_var._buf if running_var is not None else None, training=training, momentum=momentum, eps=eps)
    parents = (input,) + ((weight,) if weight is not None else ()) + ((bias,) if bias is not None else ())

    def bw(g):
        dx, dw, db = be.batch_norm_bwd(x, g.contiguous(), wb, mean, invstd, batch_stats=batch_stats,
                                       need_dx=input.requires_grad,
                                       need_dw=weight is not None and weight.requires_grad,
                                       need_db=bias is not None and bias.requires_grad)
        return (dx,) + ((dw,) if weight is not None else ()) + ((db,) if bias is not None else ())

    return input._result(y, parents, bw)


class _BatchNorm(Module):
    """Weight ones, bias zeros, running mean zeros, running variance ones (``engine/src/nn/normalization.rs``)."""
    _ndims: Tuple[int, ...] = ()

    def __init__(self, num_features: int, eps: float = 1e-5, momentum: float = 0.1, dtype: str = "float32"):
        if num_features <= 0:
            raise ValueError("num_features must be positive")
        self.num_features, self.eps, self.momentum = num_features, eps, momentum
        self.weight = Tensor(np.ones(num_features, dtype=dtype), requires_grad=True)
        self.bias = Tensor(np.zeros(num_features, dtype=dtype), requires_grad=True)
        self.running_mean = Tensor(np.zeros(num_features, dtype=dtype))
        self.running_var = Tensor(np.ones(num_features, dtype=dtype))
        self.training = True

    def train(self):
        self.training = True
        return self

    def eval(self):
        self.training = False
        return self

    def forward(self, x: Tensor) -> Tensor:
        if x.ndim not in self._ndims:
            raise ValueError(f"{type(self).__name__} expects input with {' or '.join(map(str, self._ndims))} dimensions")
        if x.shape[1] != self.num_features:
            raise ValueError(f"shape mismatch: expected {self.num_features} features, got {x.shape[1]}")
        return batch_norm(x, self.running_mean, self.running_var, self.weight, self.bias, self.training,
                          self.momentum, self.eps)

    def parameters(self) -> List[Tensor]:
        return [self.weight, self.bias]


class BatchNorm1d(_BatchNorm):
    _ndims = (2, 3)


class BatchNorm2d(_BatchNorm):
    _ndims = (4,)


_dropout_calls = [0]


def dropout(input: Tensor, p: float = 0.5, training: bool = True, seed: Optional[int] = None, *, _channels: bool = False) -> Tensor:
    """``Dropout::forward`` (``engine/src/nn/dropout.rs:164-187``): identity when not training or p = 0, zeros for
    p = 1, otherwise the input times a mask of 0 / 1/(1-p) entries.  ``seed`` fixes the mask; without it every call
    takes the next stream of the process-wide generator (``manual_seed``)."""
    if not (0.0 <= p <= 1.0):
        raise ValueError(f"dropout probability must be between 0 and 1, got {p}")
    if _channels and input.ndim != 4:
        raise ValueError("Dropout2d expects 4D input tensor with shape [batch_size, channels, height, width]")
    if not training or p == 0.0:
        return input
    be = _be()
    if seed is None:
        _dropout_calls[0] += 1
        seed = (_global_seed[0] * 0x9E3779B1 + _dropout_calls[0]) & 0xFFFFFFFFFFFFFFFF
    x = input._buf.contiguous()
    inner = x.shape[2] * x.shape[3] if _channels else 1
    y = be.dropout_apply(x, p, seed, 0, inner)       # the mask is never stored: the backward pass regenerates it
    return input._result(y, (input,), lambda g: (be.dropout_apply(g.contiguous(), p, seed, 0, inner),))


_global_seed = [0]


def manual_seed(seed: int) -> None:
    """Seeds the dropout generator of this process (the counterpart of ``mt.manual_seed``)."""
    _global_seed[0] = int(seed)
    _dropout_calls[0] = 0


class Dropout(Module):
    def __init__(self, p: float = 0.5):
        if not (0.0 <= p <= 1.0):
            raise ValueError(f"dropout probability must be between 0 and 1, got {p}")
        self.p, self.training = p, True

    def train(self):
        self.training = True
        return self

    def eval(self):
        self.training = False
        return self

    def forward(self, x: Tensor) -> Tensor:
        return dropout(x, self.p, self.training)


class Dropout2d(Dropout):
    def forward(self, x: Tensor) -> Tensor:
        return dropout(x, self.p, self.training, _channels=True)


# ---------------------------------------------------------------------- conv
def conv2d(input: Tensor, weight: Tensor, bias: Optional[Tensor] = None, stride: _Pair = 1,
           padding: _Pair = 0) -> Tensor:
    """NCHW x OIHW convolution, f32 only, with the reference's checks (``conv.rs:32-93``)."""
    stride, padding = _pair(stride, "stride"), _pair(padding, "padding")
    if input.ndim != 4:
        raise ValueError("conv2d expects 4D input tensor [N, C_in, H, W]")
    if weight.ndim != 4:
        raise ValueError("conv2d expects 4D weight tensor [C_out, C_in, kH, kW]")
    n, c, h, w = input.shape
    co, ci, kh, kw = weight.shape
    if c != ci:
        raise ValueError(f"shape mismatch: [{ci}] vs [{c}]")
    if bias is not None and (bias.ndim != 1 or bias.shape[0] != co):
        raise ValueError(f"shape mismatch: [{co}] vs {list(bias.shape)}")
    if stride[0] <= 0 or stride[1] <= 0:
        raise ValueError("stride values must be greater than zero")
    if padding[0] < 0 or padding[1] < 0:
        raise ValueError("padding must be non-negative")
    if kh > h + 2 * padding[0] or kw > w + 2 * padding[1]:
        raise ValueError("kernel size cannot be larger than padded input")
    if input.dtype != "float32" or weight.dtype != "float32" or (bias is not None and bias.dtype != "float32"):
        raise ValueError("conv2d is implemented only for Float32 tensors")
    be = _be()
    y = be.conv2d_fwd(input._buf, weight._buf, bias._buf if bias is not None else None, stride, padding)
    parents = (input, weight) + ((bias,) if bias is not None else ())

    def bw(g):  # Conv2dBackward (engine/src/autograd/mod/shape.rs:57-197)
        g = g.contiguous()
        gx = be.conv2d_bwd_data(g, weight._buf, input.shape, stride, padding) if input.requires_grad else None
        gw = be.conv2d_bwd_weight(g, input._buf, weight.shape, stride, padding) if weight.requires_grad else None
        gb = be.conv2d_bwd_bias(g) if (bias is not None and bias.requires_grad) else None
        return (gx, gw, gb)[: len(parents)]

    return input._result(y, parents, bw)


class Conv2d(Module):
    """He-uniform weight, zero bias (``engine/src/nn/conv.rs:60-74``); ``weight_init`` picks another method of
    :func:`init_tensor`, e.g. "he_normal" for the Kaiming-normal weights of the large conv config."""

    def __init__(self, in_channels: int, out_channels: int, kernel_size: _Pair, stride: _Pair = 1,
                 padding: _Pair = 0, bias: bool = True, rng: Optional[np.random.Generator] = None,
                 weight_init="he_uniform"):
        kh, kw = _pair(kernel_size, "kernel_size")
        if in_channels <= 0 or out_channels <= 0 or kh <= 0 or kw <= 0:
            raise ValueError("channels and kernel size must be positive")
        self.stride, self.padding = _pair(stride, "stride"), _pair(padding, "padding")
        self.weight = Tensor(init_tensor(weight_init, (out_channels, in_channels, kh, kw), "float32", rng),
                             requires_grad=True)
        self.bias = Tensor(np.zeros(out_channels, dtype=np.float32), requires_grad=True) if bias else None

    def forward(self, x: Tensor) -> Tensor:
        return conv2d(x, self.weight, self.bias, self.stride, self.padding)

    def parameters(self) -> List[Tensor]:
        return [self.weight] + ([self.bias] if self.bias is not None else [])


# ---------------------------------------------------------------------- loss
def cross_entropy(input: Tensor, target: Tensor, reduction: str = "mean", dim: int = -1) -> Tensor:
    """``cross_entropy`` of the reference (``engine/src/operations/loss/regression.rs:253-308``): f32 logits with the
    classes along ``dim``; ``target`` holds class indices (int32 / int64, the logits' shape without ``dim``) or
    probabilities (float32, the logits' shape); ``reduction`` is "mean", "sum" or "none"."""
    if reduction not in ("mean", "sum", "none"):
        raise ValueError(f"Invalid reduction mode: {reduction}. Must be 'mean', 'sum', or 'none'")
    nd = input.ndim
    if nd < 1:
        raise ValueError("cross entropy expects at least 1-D logits")
    d = dim + nd if dim < 0 else dim
    if d < 0 or d >= nd:
        raise IndexError("dim out of range in cross_entropy")
    if input.dtype != "float32":
        raise TypeError("cross entropy on this path takes float32 logits")
    if target.dtype not in ("int32", "int64", "float32"):
        raise TypeError("Unsupported target dtype for classification loss")
    soft = target.dtype == "float32"
    rest = tuple(s_ for i_, s_ in enumerate(input.shape) if i_ != d)
    if (soft and target.shape != input.shape) or (not soft and target.shape != rest):
        raise ValueError(f"shape mismatch: {input.shape} vs {target.shape}")
    ncls = input.shape[d]
    # class dimension last, everything else flattened (regression.rs:264-291)
    x2 = input._buf.movedim(d, -1).reshape(-1, ncls).contiguous()
    t2 = (target._buf.movedim(d, -1).reshape(-1, ncls) if soft else target._buf.reshape(-1)).contiguous()
    be = _be()
    loss, dl = be.cross_entropy_ex(x2, t2, reduction=reduction, want_grad=input.requires_grad)
    be.sync()  # surfaces an out-of-range class index as IndexError, as the reference does eagerly
    moved_shape = tuple(rest) + (ncls,)

    def bw(g):
        gg = g.reshape(-1, 1) if reduction == "none" else g.reshape(())
        return ((dl * gg).reshape(moved_shape).movedim(-1, d).contiguous(),)

    out = loss.reshape(rest) if reduction == "none" else loss.reshape(())
    return input._result(out, (input,), bw)


class CrossEntropyLoss(Module):
    def __init__(self, reduction: str = "mean"):
        if reduction not in ("mean", "sum", "none"):
            raise ValueError(f"Invalid reduction mode: {reduction}. Must be 'mean', 'sum', or 'none'")
        self.reduction = reduction

    def __call__(self, input: Tensor, target: Tensor) -> Tensor:
        return cross_entropy(input, target, self.reduction)
