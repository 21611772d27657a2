"""Host-side mirror of minitensor's ``Tensor`` for the dense-contraction path.

Same names, argument meaning and error behaviour as the reference's Python
surface (``bindings/src/tensor/pytensor/*.rs``) for the operators on the path:
``matmul`` / ``@`` / ``bmm`` (``engine/src/operations/linalg/matmul.rs:261-416,
738-763``), ``transpose``, broadcast ``+`` of a bias, ``relu`` / ``gelu``,
``sum`` and ``backward``.  Data lives in device memory (a torch CUDA tensor is
the buffer); every product, activation and reduction listed above runs in
``libmtb200.so``.  Shape bookkeeping (reshape, batch broadcast, gradient
accumulation) stays on the host side as in the reference.

Autograd is a small tape: each result remembers a closure that maps its
upstream gradient to gradients of its inputs, and ``backward`` walks the graph
in reverse topological order accumulating by tensor identity, like
``ComputationGraph::backward`` (``engine/src/autograd/graph.rs:222-282``).
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from . import backend as _bk
from ._lib import EPI_GELU_ERF, EPI_GELU_TANH, EPI_RELU

_NAMES = {"float32": torch.float32, "float64": torch.float64, "int32": torch.int32,
          "int64": torch.int64, "bool": torch.bool}
_REV = {v: k for k, v in _NAMES.items()}


def _be() -> _bk.Backend:
    return _bk.get_backend(torch.cuda.current_device())


def _sum_leading(g: torch.Tensor, extra: int) -> torch.Tensor:
    """Sum of ``g`` over its first ``extra`` dimensions."""
    kept = g.shape[extra:]
    rows = 1
    for d in g.shape[:extra]:
        rows *= d
    cols = g.numel() // max(rows, 1)
    if g.dtype not in (torch.float32, torch.float64):
        raise TypeError("broadcast gradients are provided for float32/float64 tensors")
    return _be().colsum(g.reshape(rows, cols)).reshape(kept)


def _sum_dim_keep(g: torch.Tensor, dim: int) -> torch.Tensor:
    """Sum of ``g`` over dimension ``dim``, kept with extent 1."""
    outer = 1
    for d in g.shape[:dim]:
        outer *= d
    n = g.shape[dim]
    inner = g.numel() // max(outer * n, 1)
    view = g.reshape(outer, n, inner)
    out = torch.empty(outer, inner, dtype=g.dtype, device=g.device)
    for o in range(outer):
        _be().colsum(view[o], out=out[o])
    return out.reshape(g.shape[:dim] + (1,) + g.shape[dim + 1:])


class Tensor:
    """Device tensor with the reference's matmul-path methods."""

    def __init__(self, data, dtype: Optional[str] = None, requires_grad: bool = False, device=None,
                 _buf: Optional[torch.Tensor] = None):
        if _buf is not None:
            buf = _buf
        else:
            if isinstance(data, Tensor):
                arr = data.numpy()
            else:
                arr = np.asarray(data)
            if dtype is None:
                # numpy arrays keep their dtype; Python lists of floats take the
                # reference's default dtype (float32), lists of ints int64
                if arr.dtype == np.bool_:
                    dtype = "bool"
                elif isinstance(data, np.ndarray) and arr.dtype.name in _NAMES:
                    dtype = arr.dtype.name
                elif np.issubdtype(arr.dtype, np.integer):
                    dtype = "int64"
                else:
                    dtype = "float32"
            if dtype not in _NAMES:
                raise TypeError(f"unsupported dtype {dtype!r}")
            buf = torch.from_numpy(arr.astype(_np_dtype(dtype), order="C", copy=True)).to(_be().device)
        self._buf = buf.contiguous()
        self.requires_grad = bool(requires_grad)
        self.grad: Optional["Tensor"] = None
        self._parents: Tuple["Tensor", ...] = ()
        self._backward_fn: Optional[Callable[["torch.Tensor"], Sequence[Optional[torch.Tensor]]]] = None

    # ------------------------------------------------------------------ basics
    @property
    def shape(self) -> Tuple[int, ...]:
        return tuple(self._buf.shape)

    @property
    def ndim(self) -> int:
        return self._buf.dim()

    @property
    def dtype(self) -> str:
        return _REV[self._buf.dtype]

    def numpy(self) -> np.ndarray:
        return self._buf.detach().cpu().numpy()

    def detach(self) -> "Tensor":
        return Tensor(None, _buf=self._buf)

    def item(self):
        return self.numpy().item()

    def zero_grad(self) -> None:
        self.grad = None

    def _result(self, buf: torch.Tensor, parents: Tuple["Tensor", ...], fn) -> "Tensor":
        out = Tensor(None, _buf=buf)
        if any(p.requires_grad for p in parents):
            out.requires_grad = True
            out._parents = parents
            out._backward_fn = fn
        return out

    # ------------------------------------------------------------------ shape helpers (host side)
    def reshape(self, *shape) -> "Tensor":
        if len(shape) == 1 and isinstance(shape[0], (tuple, list)):
            shape = tuple(shape[0])
        old = self.shape
        return self._result(self._buf.reshape(shape), (self,), lambda g: (g.reshape(old),))

    def transpose(self, dim0: int, dim1: int) -> "Tensor":
        """Materialised transpose (``engine/src/operations/linalg/diagonal.rs:8-108``)."""
        be = _be()
        buf = be.swap_dims(self._buf, dim0, dim1)
        return self._result(buf, (self,), lambda g: (be.swap_dims(g.contiguous(), dim0, dim1),))

    def _expand_to(self, shape: Tuple[int, ...]) -> "Tensor":
        old = self.shape
        buf = self._buf.expand(shape).contiguous()

        def bw(g):
            # the gradient of a broadcast is the sum over the broadcast dimensions: the library's column sum over
            # the rows of a [rows, kept] view, slice by slice where the summed dimension is not the leading one
            extra = len(shape) - len(old)
            if extra:
                g = _sum_leading(g.contiguous(), extra)
            for i, d in enumerate(old):
                if d == 1 and g.shape[i] != 1:
                    g = _sum_dim_keep(g.contiguous(), i)
            return (g.contiguous(),)

        return self._result(buf, (self,), bw)

    # ------------------------------------------------------------------ matmul / bmm
    def matmul(self, other: "Tensor") -> "Tensor":
        return matmul(self, other)

    __matmul__ = matmul

    def bmm(self, other: "Tensor") -> "Tensor":
        return bmm(self, other)

    # ------------------------------------------------------------------ elementwise on the path
    def __add__(self, other: "Tensor") -> "Tensor":
        return add(self, other)

    def relu(self) -> "Tensor":
        return _activation(self, EPI_RELU)

    def gelu(self, approximate: str = "none") -> "Tensor":
        if approximate not in ("none", "tanh"):
            raise ValueError("approximate must be 'none' or 'tanh'")
        return _activation(self, EPI_GELU_ERF if approximate == "none" else EPI_GELU_TANH)

    def sum(self) -> "Tensor":
        shape = self.shape
        if self._buf.dtype not in (torch.float32, torch.float64):
            raise TypeError("sum over all elements is provided for float32/float64 tensors")
        buf = _be().colsum(self._buf.contiguous().reshape(-1, 1)).reshape(())     # one column: the sum of all rows
        return self._result(buf, (self,), lambda g: (g.reshape(()).expand(shape).contiguous(),))

    # ------------------------------------------------------------------ autograd
    def backward(self, gradient: Optional["Tensor"] = None) -> None:
        if not self.requires_grad:
            raise RuntimeError("Tensor does not require gradients")
        if gradient is None:
            if self._buf.numel() != 1:
                raise RuntimeError("backward without a gradient needs a scalar tensor")
            g0 = torch.ones_like(self._buf)
        else:
            g0 = gradient._buf
        order: List[Tensor] = []
        seen = set()
        stack = [(self, False)]
        while stack:  # iterative DFS, as the reference's ensure_topological_order
            node, done = stack.pop()
            if done:
                order.append(node)
                continue
            if id(node) in seen:
                continue
            seen.add(id(node))
            stack.append((node, True))
            for p in node._parents:
                if p.requires_grad and id(p) not in seen:
                    stack.append((p, False))
        grads = {id(self): g0}
        for node in reversed(order):
            g = grads.pop(id(node), None)
            if g is None:
                continue
            if node._backward_fn is None:  # leaf
                if node.grad is None:
                    node.grad = Tensor(None, _buf=g.clone())    # its own buffer: later contributions add in place
                else:   # accumulate into the existing gradient (add_inplace, engine/src/autograd/mod/core.rs:168)
                    _be().add_inplace(node.grad._buf, g.contiguous())
                continue
            for p, pg in zip(node._parents, node._backward_fn(g)):
                if pg is None or not p.requires_grad:
                    continue
                if id(p) not in grads:
                    grads[id(p)] = pg
                else:   # accumulate_grad: a fresh buffer, the first contribution may alias a saved tensor
                    acc = grads[id(p)].clone()
                    grads[id(p)] = _be().add_inplace(acc, pg.contiguous())


def _np_dtype(name: str):
    return {"float32": np.float32, "float64": np.float64, "int32": np.int32, "int64": np.int64,
            "bool": np.bool_}[name]


# ---------------------------------------------------------------------- operators
def matmul(lhs: Tensor, rhs: Tensor) -> Tensor:
    """``lhs @ rhs`` with the reference's checks, 1-D promotion and batch broadcast
    (``engine/src/operations/linalg/matmul.rs:261-416``)."""
    if lhs._buf.device != rhs._buf.device:
        raise ValueError(f"device mismatch: {lhs._buf.device} vs {rhs._buf.device}")
    if lhs.dtype != rhs.dtype:
        raise TypeError(f"type mismatch: {lhs.dtype} vs {rhs.dtype}")
    lhs_1d, rhs_1d = lhs.ndim == 1, rhs.ndim == 1
    if lhs_1d or rhs_1d:
        l2 = lhs.reshape(1, lhs.shape[0]) if lhs_1d else lhs
        r2 = rhs.reshape(rhs.shape[0], 1) if rhs_1d else rhs
        prom = matmul(l2, r2)
        dims = list(prom.shape)
        n = len(dims)
        if rhs_1d:
            dims.pop(n - 1)
        if lhs_1d:
            dims.pop(n - 2)
        return prom.reshape(tuple(dims))
    if lhs.ndim < 2 or rhs.ndim < 2:
        raise ValueError("Matrix multiplication requires tensors with at least 1 dimension "
                         "(scalars are not valid operands)")
    lb, rb = lhs.shape[:-2], rhs.shape[:-2]
    if lb != rb:
        try:
            batch = tuple(np.broadcast_shapes(lb, rb))
        except ValueError:
            raise ValueError(f"shape mismatch: {lhs.shape} vs {rhs.shape}") from None
        return matmul(lhs._expand_to(batch + lhs.shape[-2:]), rhs._expand_to(batch + rhs.shape[-2:]))
    m, k = lhs.shape[-2:]
    k2, n = rhs.shape[-2:]
    if k != k2:
        raise ValueError(f"shape mismatch: [{m}, {k}] vs [{k2}, {n}]")
    if lhs.dtype == "bool":
        raise ValueError("Matrix multiplication not supported for boolean tensors")
    be = _be()
    a3 = lhs._buf.reshape((-1, m, k)) if lhs.ndim != 2 else lhs._buf
    b3 = rhs._buf.reshape((-1, k, n)) if rhs.ndim != 2 else rhs._buf
    out_shape = lb + (m, n)
    out = be.gemm(a3, b3).reshape(out_shape)

    def bw(g):  # MatMulBackward (engine/src/autograd/mod/core.rs:752-789), transposes folded into the GEMM
        g3 = g.reshape((-1, m, n)).contiguous() if lhs.ndim != 2 else g.contiguous()
        ga = be.gemm(g3, b3, trans_b=True).reshape(lhs.shape) if lhs.requires_grad else None
        gb = be.gemm(a3, g3, trans_a=True).reshape(rhs.shape) if rhs.requires_grad else None
        return ga, gb

    return lhs._result(out, (lhs, rhs), bw)


def bmm(lhs: Tensor, rhs: Tensor) -> Tensor:
    """``engine/src/operations/linalg/matmul.rs:738-763``."""
    if lhs.ndim != 3 or rhs.ndim != 3:
        raise ValueError("bmm expects both inputs to be 3D tensors")
    if lhs.shape[0] != rhs.shape[0]:
        raise ValueError(f"shape mismatch: {lhs.shape} vs {rhs.shape}")
    if lhs.shape[2] != rhs.shape[1]:
        raise ValueError(f"shape mismatch: [{lhs.shape[2]}] vs [{rhs.shape[1]}]")
    return matmul(lhs, rhs)


def add(x: Tensor, y: Tensor) -> Tensor:
    """``x + y`` for the two cases on the path: equal shapes, or ``[..., N] + [N]``
    (bias broadcast, ``engine/src/operations/arithmetic/kernels.rs:191-334``); the gradient of the
    broadcast operand is the dim-0 sum (``engine/src/autograd/mod/core.rs:195-223``)."""
    if x.dtype != y.dtype:
        raise TypeError(f"type mismatch: {x.dtype} vs {y.dtype}")
    be = _be()
    if x.shape == y.shape:
        return x._result(be.add_inplace(x._buf.clone(), y._buf.contiguous()), (x, y), lambda g: (g, g))
    if y.ndim == 1 and x.ndim >= 2 and x.shape[-1] == y.shape[0]:
        out = be.bias_act(x._buf, y._buf, 0)
        n = y.shape[0]
        return x._result(out, (x, y), lambda g: (g, be.colsum(g.reshape(-1, n).contiguous())))
    raise ValueError(f"shape mismatch: {x.shape} vs {y.shape}")


def _activation(x: Tensor, act: int) -> Tensor:
    if x.dtype not in ("float32", "float64"):
        raise TypeError("activation needs a floating tensor")
    be = _be()
    y = be.act_fwd(x._buf, act)
    ref = y if act == EPI_RELU else x._buf  # relu keeps its output sign, gelu its input
    return x._result(y, (x,), lambda g: (be.act_bwd(ref, g.contiguous(), act),))


def device(name: str = "cuda"):
    """Accepts the reference's device strings (``engine/src/device.rs:119-141``); only CUDA exists here."""
    if not name.startswith("cuda"):
        raise ValueError("mtb200 tensors live on a CUDA device")
    return name
