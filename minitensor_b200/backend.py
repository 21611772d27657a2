"""Device backend: a thin object over one ``mtb200`` handle.

It plays the role of minitensor's ``CudaBackend`` + ``CudaOps`` pair
(``engine/src/backends/cuda/mod.rs:164-317,396-655``): it owns the device
context for one GPU and exposes the operators of the dense-contraction path on
raw device buffers.  Buffers are ``torch`` CUDA tensors (torch is used for
device memory and streams only); every computation goes through the C ABI.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import numpy as np
import torch

from . import _lib
from ._lib import (EPI_GELU_ERF, EPI_GELU_TANH, EPI_NONE, EPI_RELU, EPI_RELU_BWD, F32, F64, I32,
                   I64, check)

# the current stream's handle without building a torch.cuda.Stream object per call (a few microseconds on a path
# whose whole host cost is about twenty); absent from a torch build, the public call serves
_RAW_STREAM = getattr(torch._C, "_cuda_getCurrentRawStream", None)

_DTYPES = {torch.float32: F32, torch.float64: F64, torch.int32: I32, torch.int64: I64}


def dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.bool:
        raise TypeError("Matrix multiplication not supported for boolean tensors")
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise TypeError(f"unsupported dtype {t.dtype}") from None


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    """Device address of a buffer handed to the C ABI.  The library reads raw dense row-major memory, so a strided
    view (a transpose, a channels_last tensor) or a host tensor would be read as something else: refuse it here
    rather than copy, so that training buffers keep their aliasing."""
    if t is None or t.numel() == 0:
        return None
    if not t.is_cuda:
        raise ValueError("mtb200 operators take CUDA tensors")
    if not t.is_contiguous():
        raise ValueError("mtb200 operators take contiguous (dense row-major) tensors")
    return t.data_ptr()


def _same_dtype(what: str, first: torch.Tensor, *rest: Optional[torch.Tensor], want=None) -> None:
    """Every buffer of one call must have the element type the kernel is about to read it as."""
    if want is not None and first.dtype != want:
        raise TypeError(f"{what}: expected dtype {want}, got {first.dtype}")
    for t in rest:
        if t is not None and t.dtype != first.dtype:
            raise TypeError(f"{what}: dtype mismatch ({first.dtype} vs {t.dtype})")


class Backend:
    """One handle on one CUDA device; work is enqueued on torch's current stream."""

    def __init__(self, device: int = 0):
        self.lib = _lib.load()
        if not torch.cuda.is_available():
            raise RuntimeError("mtb200 needs a CUDA device (B200, sm_100a); none is visible")
        self.device = torch.device("cuda", device)
        h = C.c_void_p()
        check(self.lib.mtb200_create(device, C.byref(h)))
        self._h = h
        self.launches = 0  # kernels this backend enqueued (operand splits count)
        self._dev_index = device
        self._bound_stream = None
        self._bind_stream()

    def _bind_stream(self) -> None:
        """Point the handle at torch's current stream; the C call is made only when that stream changed."""
        s = _RAW_STREAM(self._dev_index) if _RAW_STREAM else torch.cuda.current_stream(self.device).cuda_stream
        if s != self._bound_stream:
            check(self.lib.mtb200_set_stream(self._h, C.c_void_p(s)))
            self._bound_stream = s

    def close(self) -> None:
        if getattr(self, "_h", None):
            self.lib.mtb200_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def set_gemm_sm_limit(self, sms: int) -> None:
        """SMs the persistent GEMM kernels may occupy (0 = all): leaves room for kernels that run beside them."""
        check(self.lib.mtb200_set_gemm_sm_limit(self._h, int(sms)))

    def sync(self) -> None:
        """Wait for the stream and raise if a kernel reported an expired wait or a bad label."""
        check(self.lib.mtb200_sync(self._h))

    def profile(self, on: bool) -> None:
        """Start (clearing earlier records) or stop per-launch event timing inside the library."""
        check(self.lib.mtb200_profile_enable(self._h, int(on)))

    def profile_read(self, kernel_class: int = 0):
        """(launches, total device ms, total algorithmic work) of one kernel class since profile(True)."""
        n, ms, work = C.c_int64(), C.c_double(), C.c_double()
        check(self.lib.mtb200_profile_read(self._h, kernel_class, C.byref(n), C.byref(ms), C.byref(work)))
        return n.value, ms.value, work.value

    def workspace_bytes(self) -> int:
        n = C.c_size_t()
        check(self.lib.mtb200_workspace_bytes(self._h, C.byref(n)))
        return n.value

    # ------------------------------------------------------------------ GEMM
    def gemm(self, a: torch.Tensor, b: torch.Tensor, *, trans_a: bool = False, trans_b: bool = False,
             bias: Optional[torch.Tensor] = None, epilogue: int = EPI_NONE,
             aux: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
             f32_mode: int = 0, variant: int = 0) -> torch.Tensor:
        """``out[b] = epilogue(op(a[b]) @ op(b[b]) + bias)`` for 2-D or 3-D contiguous operands.

        A 2-D operand next to a 3-D one is broadcast over the batch.
        """
        if a.dtype != b.dtype:
            raise TypeError(f"dtype mismatch: {a.dtype} vs {b.dtype}")
        dt = dtype_code(a)
        if not (a.is_contiguous() and b.is_contiguous()):
            raise ValueError("operands must be contiguous")
        if a.dim() not in (2, 3) or b.dim() not in (2, 3):
            raise ValueError("operands must be 2-D or 3-D")
        batch = 1
        if a.dim() == 3:
            batch = a.shape[0]
        if b.dim() == 3:
            if a.dim() == 3 and b.shape[0] != batch:
                raise ValueError(f"batch mismatch: {tuple(a.shape)} vs {tuple(b.shape)}")
            batch = b.shape[0]
        am, ak = (a.shape[-1], a.shape[-2]) if trans_a else (a.shape[-2], a.shape[-1])
        bk, bn = (b.shape[-1], b.shape[-2]) if trans_b else (b.shape[-2], b.shape[-1])
        if ak != bk:
            raise ValueError(f"shape mismatch: [{am}, {ak}] x [{bk}, {bn}]")
        m, n, k = am, bn, ak
        stride_a = a.shape[-1] * a.shape[-2] if a.dim() == 3 else 0
        stride_b = b.shape[-1] * b.shape[-2] if b.dim() == 3 else 0
        batched = a.dim() == 3 or b.dim() == 3
        shape = (batch, m, n) if batched else (m, n)
        if out is None:
            out = torch.empty(shape, dtype=a.dtype, device=a.device)
        elif tuple(out.shape) != shape or out.dtype != a.dtype or not out.is_contiguous():
            raise ValueError("bad output tensor")
        self._bind_stream()
        check(self.lib.mtb200_gemm(self._h, dt, int(trans_a), int(trans_b), batch, m, n, k,
                                   _ptr(a), stride_a, _ptr(b), stride_b, _ptr(out), m * n,
                                   _ptr(bias), epilogue, _ptr(aux), (variant << 8) | f32_mode))
        self.launches += 4 if dt == F32 else 1  # two operand splits, GEMM, gated f32 redo
        return out

    # ------------------------------------------------------------------ dense layer (shared operand preparation)
    def dense_saved_bytes(self, rows: int, in_features: int, out_features: int, dtype=torch.float32) -> int:
        """Bytes of the block ``dense_forward`` leaves for ``dense_backward`` (0: the pair runs as plain products)."""
        n = C.c_size_t(0)
        code = dtype_code(torch.empty(0, dtype=dtype))
        check(self.lib.mtb200_dense_saved_bytes(code, rows, in_features, out_features, C.byref(n)))
        return int(n.value)

    def dense_dy_bytes(self, rows: int, in_features: int, out_features: int, dtype=torch.float32) -> int:
        """Bytes of the block that carries dY's prepared operand between two ``dense_backward`` calls (0: unused)."""
        n = C.c_size_t(0)
        code = dtype_code(torch.empty(0, dtype=dtype))
        check(self.lib.mtb200_dense_dy_bytes(code, rows, in_features, out_features, C.byref(n)))
        return int(n.value)

    def dense_forward(self, x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
                      epilogue: int = EPI_NONE, out: Optional[torch.Tensor] = None,
                      saved: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``epilogue(x @ w.T + bias)`` for ``x [rows, in]``, ``w [out, in]``; ``saved`` (uint8, device) receives
        the prepared operands for ``dense_backward``."""
        rows, fin = x.shape
        fout = w.shape[0]
        if w.shape[1] != fin or x.dtype != w.dtype:
            raise ValueError(f"shape/dtype mismatch: x {tuple(x.shape)} {x.dtype}, w {tuple(w.shape)} {w.dtype}")
        _same_dtype("dense_forward", x, w, bias, out)
        if out is None:
            out = torch.empty(rows, fout, dtype=x.dtype, device=x.device)
        self._bind_stream()
        check(self.lib.mtb200_dense_forward(self._h, dtype_code(x), rows, fin, fout, _ptr(x), _ptr(w), _ptr(bias),
                                            epilogue, _ptr(out), _ptr(saved)))
        self.launches += 5 if saved is not None else 4
        return out

    def dense_backward(self, x: torch.Tensor, w: torch.Tensor, dy: torch.Tensor, saved: Optional[torch.Tensor], *,
                       dx: Optional[torch.Tensor] = None, need_dx: bool = True, dx_epilogue: int = EPI_NONE,
                       dx_aux: Optional[torch.Tensor] = None, dw: Optional[torch.Tensor] = None, need_dw: bool = True,
                       db: Optional[torch.Tensor] = None, need_db: bool = True,
                       dy_block: Optional[torch.Tensor] = None, dy_mode: int = 0):
        """Gradients of ``dense_forward``: returns ``(dx or None, dw or None, db or None)``.

        ``dy_block`` / ``dy_mode``: a call with ``dy_mode=1`` (no ``dw``) also leaves dY's prepared weight-gradient
        operand in ``dy_block`` (``dense_dy_bytes`` bytes); a later call with ``dy_mode=2`` (no ``dx``, no ``db``)
        computes ``dw`` from it without reading ``dy`` again."""
        rows, fin = x.shape
        fout = w.shape[0]
        _same_dtype("dense_backward", x, w, dy, dx, dx_aux, dw, db)
        if tuple(dy.shape) != (rows, fout):
            raise ValueError(f"dy must be [{rows}, {fout}], got {tuple(dy.shape)}")
        if need_dx and dx is None:
            dx = torch.empty(rows, fin, dtype=x.dtype, device=x.device)
        if need_dw and dw is None:
            dw = torch.empty(fout, fin, dtype=x.dtype, device=x.device)
        if need_db and db is None:
            db = torch.empty(fout, dtype=x.dtype, device=x.device)
        self._bind_stream()
        check(self.lib.mtb200_dense_backward(self._h, dtype_code(x), rows, fin, fout, _ptr(x), _ptr(w), _ptr(dy),
                                             _ptr(saved), _ptr(dx) if need_dx else None, dx_epilogue, _ptr(dx_aux),
                                             _ptr(dw) if need_dw else None, _ptr(db) if need_db else None,
                                             _ptr(dy_block), dy_mode if dy_block is not None else 0))
        products = int(need_dx) + int(need_dw)
        prep = 1 if (dy_mode == 2 and dy_block is not None) else 5
        self.launches += (prep + 2 * products) if saved is not None else (4 * products + 2 * int(need_db))
        return (dx if need_dx else None), (dw if need_dw else None), (db if need_db else None)

    # ------------------------------------------------------------------ reductions / elementwise
    def colsum(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        m, n = x.shape
        _same_dtype("colsum", x, out)
        if out is None:
            out = torch.empty(n, dtype=x.dtype, device=x.device)
        self._bind_stream()
        check(self.lib.mtb200_colsum(self._h, dtype_code(x), m, n, _ptr(x), _ptr(out)))
        self.launches += 2
        return out

    def add_inplace(self, y: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
        """``y += x`` on the device (gradient accumulation); shapes and dtypes must agree, as the reference demands."""
        if tuple(y.shape) != tuple(x.shape):
            raise ValueError(f"shape mismatch: {tuple(y.shape)} vs {tuple(x.shape)}")
        _same_dtype("add_inplace", y, x)
        self._bind_stream()
        check(self.lib.mtb200_add_inplace(self._h, dtype_code(y), y.numel(), _ptr(y), _ptr(x)))
        self.launches += 1
        return y

    def swap_dims(self, x: torch.Tensor, dim0: int, dim1: int) -> torch.Tensor:
        """Materialised ``x.transpose(dim0, dim1)`` of a dense tensor, written by the library's kernel."""
        nd = x.dim()
        d0, d1 = (dim0 + nd if dim0 < 0 else dim0), (dim1 + nd if dim1 < 0 else dim1)
        if not (0 <= d0 < nd and 0 <= d1 < nd):
            raise IndexError(f"dimension out of range for a tensor of {nd} dimensions")
        if d0 == d1:
            return x.clone()
        if d0 > d1:
            d0, d1 = d1, d0
        if x.element_size() not in (4, 8):
            raise TypeError(f"unsupported dtype {x.dtype}")
        shape = list(x.shape)
        prod = lambda xs: int(np.prod(xs, dtype=np.int64)) if len(xs) else 1
        outer, mid, inner = prod(shape[:d0]), prod(shape[d0 + 1:d1]), prod(shape[d1 + 1:])
        shape[d0], shape[d1] = shape[d1], shape[d0]
        y = torch.empty(shape, dtype=x.dtype, device=x.device)
        self._bind_stream()
        check(self.lib.mtb200_swap_dims(self._h, x.element_size(), outer, x.shape[d0], mid, x.shape[d1], inner, _ptr(x),
                                        _ptr(y)))
        self.launches += 1
        return y

    def bias_act(self, x: torch.Tensor, bias: Optional[torch.Tensor], act: int = 0) -> torch.Tensor:
        """``act(x + bias)`` with ``bias`` broadcast over the rows of the 2-D view of ``x``."""
        n = x.shape[-1]
        _same_dtype("bias_act", x, bias)
        y = torch.empty_like(x)
        self._bind_stream()
        check(self.lib.mtb200_bias_act(self._h, dtype_code(x), x.numel() // max(n, 1), n, _ptr(x), _ptr(bias),
                                       act, _ptr(y)))
        self.launches += 1
        return y

    def act_fwd(self, x: torch.Tensor, act: int) -> torch.Tensor:
        y = torch.empty_like(x)
        self._bind_stream()
        check(self.lib.mtb200_act_fwd(self._h, dtype_code(x), act, x.numel(), _ptr(x), _ptr(y)))
        self.launches += 1
        return y

    def act_bwd(self, ref: torch.Tensor, dy: torch.Tensor, act: int) -> torch.Tensor:
        _same_dtype("act_bwd", dy, ref)
        dx = torch.empty_like(dy)
        self._bind_stream()
        check(self.lib.mtb200_act_bwd(self._h, dtype_code(dy), act, dy.numel(), _ptr(ref), _ptr(dy), _ptr(dx)))
        self.launches += 1
        return dx

    def cross_entropy(self, logits: torch.Tensor, labels: torch.Tensor, *, mean: bool = True,
                      upstream: float = 1.0, want_grad: bool = True):
        """Returns ``(loss[1], dlogits or None)``; labels int32/int64 class indices."""
        bsz, ncls = logits.shape
        _same_dtype("cross_entropy", logits, want=torch.float32)
        if labels.dtype not in (torch.int32, torch.int64):
            raise TypeError("Unsupported target dtype for classification loss")
        if tuple(labels.shape) != (bsz,):
            raise ValueError(f"shape mismatch: labels {tuple(labels.shape)} for logits {tuple(logits.shape)}")
        loss = torch.empty(1, dtype=torch.float32, device=logits.device)
        dl = torch.empty_like(logits) if want_grad else None
        self._bind_stream()
        check(self.lib.mtb200_cross_entropy(self._h, bsz, ncls, _ptr(logits), _ptr(labels),
                                            _DTYPES[labels.dtype], int(mean), float(upstream),
                                            _ptr(loss), _ptr(dl)))
        self.launches += 2
        return loss, dl

    def cross_entropy_into(self, logits: torch.Tensor, labels: torch.Tensor, dlogits: torch.Tensor, *,
                           mean: bool = True, upstream: float = 1.0):
        """Same as :meth:`cross_entropy` with the gradient written into ``dlogits``."""
        bsz, ncls = logits.shape
        _same_dtype("cross_entropy", logits, want=torch.float32)
        if labels.dtype not in (torch.int32, torch.int64):
            raise TypeError("Unsupported target dtype for classification loss")
        if tuple(dlogits.shape) != (bsz, ncls) or dlogits.dtype != torch.float32 or tuple(labels.shape) != (bsz,):
            raise ValueError("bad gradient buffer or label shape")
        loss = torch.empty(1, dtype=torch.float32, device=logits.device)
        self._bind_stream()
        check(self.lib.mtb200_cross_entropy(self._h, bsz, ncls, _ptr(logits), _ptr(labels),
                                            _DTYPES[labels.dtype], int(mean), float(upstream),
                                            _ptr(loss), _ptr(dlogits)))
        self.launches += 2
        return loss, dlogits

    def adam_step(self, p: torch.Tensor, g: torch.Tensor, m: torch.Tensor, v: torch.Tensor, *,
                  lr: float, beta1: float, beta2: float, eps: float, weight_decay: float = 0.0,
                  decoupled: bool = False, step: int = 1, grad_scale: float = 1.0) -> None:
        _same_dtype("adam_step", p, g, m, v, want=torch.float32)
        if not (p.numel() == g.numel() == m.numel() == v.numel()):
            raise ValueError("adam_step: parameter, gradient and moment buffers differ in length")
        self._bind_stream()
        check(self.lib.mtb200_adam_step(self._h, p.numel(), _ptr(p), _ptr(g), _ptr(m), _ptr(v), lr, beta1,
                                        beta2, eps, weight_decay, int(decoupled), step, grad_scale))
        self.launches += 1

    def cross_entropy_ex(self, logits: torch.Tensor, targets: torch.Tensor, *, reduction: str = "mean",
                         upstream: float = 1.0, upstream_rows: Optional[torch.Tensor] = None,
                         want_grad: bool = True):
        """General cross entropy: ``targets`` are class indices ``[B]`` (int32/int64) or probabilities
        ``[B, C]`` (float32); ``reduction`` is "sum", "mean" or "none".  Returns ``(loss, dlogits or None)``,
        the loss a 1-element tensor or ``[B]`` for "none"."""
        bsz, ncls = logits.shape
        _same_dtype("cross_entropy", logits, upstream_rows, want=torch.float32)
        red = {"sum": 0, "mean": 1, "none": 2}.get(reduction)
        if red is None:
            raise ValueError(f"Invalid reduction mode: {reduction}. Must be 'mean', 'sum', or 'none'")
        if targets.dtype in (torch.int32, torch.int64):
            if tuple(targets.shape) != (bsz,):
                raise ValueError(f"shape mismatch: targets {tuple(targets.shape)} for logits {tuple(logits.shape)}")
        elif targets.dtype == torch.float32:
            if tuple(targets.shape) != (bsz, ncls):
                raise ValueError(f"shape mismatch: targets {tuple(targets.shape)} for logits {tuple(logits.shape)}")
        else:
            raise TypeError("Unsupported target dtype for classification loss")
        loss = torch.empty(bsz if red == 2 else 1, dtype=torch.float32, device=logits.device)
        dl = torch.empty_like(logits) if want_grad else None
        self._bind_stream()
        check(self.lib.mtb200_cross_entropy_ex(self._h, bsz, ncls, _ptr(logits), _ptr(targets), _DTYPES[targets.dtype],
                                               red, float(upstream), _ptr(upstream_rows), _ptr(loss), _ptr(dl)))
        self.launches += 1 if red == 2 else 2
        return loss, dl

    def sgd_step(self, p: torch.Tensor, g: torch.Tensor, v: Optional[torch.Tensor] = None, *, lr: float,
                 momentum: float = 0.0, dampening: float = 0.0, weight_decay: float = 0.0,
                 nesterov: bool = False) -> None:
        _same_dtype("sgd_step", p, g, v)
        if p.numel() != g.numel() or (v is not None and v.numel() != p.numel()):
            raise ValueError("sgd_step: buffers differ in length")
        self._bind_stream()
        check(self.lib.mtb200_sgd_step(self._h, dtype_code(p), p.numel(), _ptr(p), _ptr(g), _ptr(v), lr, momentum,
                                       dampening, weight_decay, int(nesterov)))
        self.launches += 1

    def rmsprop_step(self, p: torch.Tensor, g: torch.Tensor, sq: torch.Tensor, mb: Optional[torch.Tensor] = None,
                     ga: Optional[torch.Tensor] = None, *, lr: float, alpha: float = 0.99, eps: float = 1e-8,
                     weight_decay: float = 0.0, momentum: float = 0.0) -> None:
        _same_dtype("rmsprop_step", p, g, sq, mb, ga)
        if any(t is not None and t.numel() != p.numel() for t in (g, sq, mb, ga)):
            raise ValueError("rmsprop_step: buffers differ in length")
        self._bind_stream()
        check(self.lib.mtb200_rmsprop_step(self._h, dtype_code(p), p.numel(), _ptr(p), _ptr(g), _ptr(sq), _ptr(mb),
                                           _ptr(ga), lr, alpha, eps, weight_decay, momentum))
        self.launches += 1

    def grad_norm(self, grads) -> float:
        """L2 norm over a list of f32/f64 tensors, squares accumulated in f64 on the device (one read-back)."""
        acc = torch.zeros(1, dtype=torch.float64, device=self.device)
        self._bind_stream()
        for i, g in enumerate(grads):
            check(self.lib.mtb200_sumsq(self._h, dtype_code(g), g.numel(), _ptr(g), _ptr(acc), int(i > 0)))
            self.launches += 2
        return float(acc.item()) ** 0.5

    def clip_grad_norm(self, grads, max_norm: float) -> float:
        """``GradientUtils::clip_grad_norm``: scales every gradient by max_norm / (norm + 1e-6) when the
        norm exceeds max_norm; returns the norm before clipping."""
        total = self.grad_norm(grads)
        if total > max_norm:
            coef = max_norm / (total + 1e-6)
            for g in grads:
                check(self.lib.mtb200_scale(self._h, dtype_code(g), g.numel(), _ptr(g), coef))
                self.launches += 1
        return total

    def clip_grad_value(self, grads, lo: float, hi: float) -> None:
        self._bind_stream()
        for g in grads:
            check(self.lib.mtb200_clamp(self._h, dtype_code(g), g.numel(), _ptr(g), lo, hi))
            self.launches += 1

    def adam_step_counted(self, p: torch.Tensor, g: torch.Tensor, m: torch.Tensor, v: torch.Tensor, *, lr: float,
                          beta1: float, beta2: float, eps: float, counter: torch.Tensor, advance: bool = True,
                          weight_decay: float = 0.0, decoupled: bool = False, grad_scale: float = 1.0) -> None:
        """Adam with the step count in the one-element int64 device tensor ``counter`` (graph-replayable)."""
        if counter.dtype != torch.int64 or counter.numel() != 1:
            raise ValueError("counter must be a one-element int64 device tensor")
        _same_dtype("adam_step_counted", p, g, m, v, want=torch.float32)
        self._bind_stream()
        check(self.lib.mtb200_adam_step_counted(self._h, p.numel(), _ptr(p), _ptr(g), _ptr(m), _ptr(v), lr, beta1,
                                                beta2, eps, weight_decay, int(decoupled), _ptr(counter), int(advance),
                                                grad_scale))
        self.launches += 2 if advance else 1

    # ------------------------------------------------------------------ batch norm / dropout
    @staticmethod
    def _ncs(x: torch.Tensor):
        if x.dim() < 2:
            raise ValueError("batch_norm expects input with at least 2 dimensions")
        sp = 1
        for d in x.shape[2:]:
            sp *= d
        return x.shape[0], x.shape[1], sp

    def batch_norm_fwd(self, x: torch.Tensor, weight=None, bias=None, running_mean=None, running_var=None, *,
                       training: bool = True, momentum: float = 0.1, eps: float = 1e-5):
        """Returns ``(y, save_mean, save_invstd, used_batch_stats)``; running estimates are updated in place."""
        n, c, sp = self._ncs(x)
        _same_dtype("batch_norm", x, weight, bias, running_mean, running_var)
        y = torch.empty_like(x)
        mean = torch.empty(c, dtype=x.dtype, device=x.device)
        invstd = torch.empty(c, dtype=x.dtype, device=x.device)
        self._bind_stream()
        check(self.lib.mtb200_batch_norm_fwd(self._h, dtype_code(x), n, c, sp, _ptr(x), _ptr(weight), _ptr(bias),
                                             _ptr(running_mean), _ptr(running_var), int(training), momentum, eps,
                                             _ptr(y), _ptr(mean), _ptr(invstd)))
        batch_stats = training or running_mean is None or running_var is None
        self.launches += 3 if batch_stats else 2
        return y, mean, invstd, batch_stats

    def batch_norm_bwd(self, x, dy, weight, mean, invstd, *, batch_stats: bool = True, need_dx: bool = True,
                       need_dw: bool = True, need_db: bool = True):
        n, c, sp = self._ncs(x)
        _same_dtype("batch_norm_backward", x, dy, weight, mean, invstd)
        if dy.shape != x.shape:
            raise ValueError("batch_norm_backward: dy and x differ in shape")
        dx = torch.empty_like(x) if need_dx else None
        dw = torch.empty(c, dtype=x.dtype, device=x.device) if need_dw else None
        db = torch.empty(c, dtype=x.dtype, device=x.device) if need_db else None
        self._bind_stream()
        check(self.lib.mtb200_batch_norm_bwd(self._h, dtype_code(x), n, c, sp, _ptr(x), _ptr(dy), _ptr(weight),
                                             _ptr(mean), _ptr(invstd), int(batch_stats), _ptr(dx), _ptr(dw), _ptr(db)))
        self.launches += 3 if need_dx else 2
        return dx, dw, db

    def dropout_mask(self, n: int, p: float, seed: int, offset: int = 0, dtype=torch.float32) -> torch.Tensor:
        mask = torch.empty(n, dtype=dtype, device=self.device)
        self._bind_stream()
        check(self.lib.mtb200_dropout_mask(self._h, _DTYPES[dtype], n, p, seed, offset, _ptr(mask)))
        self.launches += 1
        return mask

    def dropout_apply(self, x: torch.Tensor, p: float, seed: int, offset: int = 0, inner: int = 1) -> torch.Tensor:
        """``x * mask`` with the mask generated on the fly from ``(seed, offset)``; call it again on the upstream
        gradient for the backward pass."""
        y = torch.empty_like(x)
        self._bind_stream()
        check(self.lib.mtb200_dropout_apply(self._h, dtype_code(x), x.numel(), inner, _ptr(x), p, seed, offset, _ptr(y)))
        self.launches += 1
        return y

    def mask_mul(self, x: torch.Tensor, mask: torch.Tensor, inner: int = 1) -> torch.Tensor:
        _same_dtype("mask_mul", x, mask)
        y = torch.empty_like(x)
        self._bind_stream()
        check(self.lib.mtb200_mask_mul(self._h, dtype_code(x), x.numel(), inner, _ptr(x), _ptr(mask), _ptr(y)))
        self.launches += 1
        return y

    # ------------------------------------------------------------------ conv2d
    @staticmethod
    def _geom(xshape, wshape, stride, padding):
        n, c, h, w = xshape
        co, ci, kh, kw = wshape
        return [n, c, h, w, co, kh, kw, stride[0], stride[1], padding[0], padding[1]]

    def conv2d_fwd(self, x, w, bias, stride, padding, f32_mode: int = 0):
        n, c, h, wd = x.shape
        co, ci, kh, kw = w.shape
        _same_dtype("conv2d", x, w, bias, want=torch.float32)
        oh = (h + 2 * padding[0] - kh) // stride[0] + 1 if stride[0] > 0 else 0
        ow = (wd + 2 * padding[1] - kw) // stride[1] + 1 if stride[1] > 0 else 0
        y = torch.empty((n, co, max(oh, 0), max(ow, 0)), dtype=torch.float32, device=x.device)
        self._bind_stream()
        check(self.lib.mtb200_conv2d_fwd(self._h, *self._geom(x.shape, w.shape, stride, padding),
                                         _ptr(x), _ptr(w), _ptr(bias), _ptr(y), f32_mode))
        self.launches += 3
        return y

    def conv2d_bwd_data(self, dy, w, xshape, stride, padding, f32_mode: int = 0):
        _same_dtype("conv2d_bwd_data", dy, w, want=torch.float32)
        dx = torch.empty(tuple(xshape), dtype=torch.float32, device=dy.device)
        self._bind_stream()
        check(self.lib.mtb200_conv2d_bwd_data(self._h, *self._geom(xshape, w.shape, stride, padding),
                                              _ptr(dy), _ptr(w), _ptr(dx), f32_mode))
        self.launches += 4
        return dx

    def conv2d_bwd_weight(self, dy, x, wshape, stride, padding, f32_mode: int = 0):
        _same_dtype("conv2d_bwd_weight", dy, x, want=torch.float32)
        dw = torch.empty(tuple(wshape), dtype=torch.float32, device=dy.device)
        self._bind_stream()
        check(self.lib.mtb200_conv2d_bwd_weight(self._h, *self._geom(x.shape, wshape, stride, padding),
                                                _ptr(dy), _ptr(x), _ptr(dw), f32_mode))
        self.launches += 4
        return dw

    def conv2d_bwd_bias(self, dy):
        n, co, oh, ow = dy.shape
        _same_dtype("conv2d_bwd_bias", dy, want=torch.float32)
        db = torch.empty(co, dtype=torch.float32, device=dy.device)
        self._bind_stream()
        check(self.lib.mtb200_conv2d_bwd_bias(self._h, n, co, oh, ow, _ptr(dy), _ptr(db)))
        self.launches += 2
        return db


_default: dict[int, Backend] = {}


def get_backend(device: int = 0) -> Backend:
    """Per-device singleton, like ``get_backend(Device)`` (engine/src/backends/mod.rs:50-64)."""
    if device not in _default:
        _default[device] = Backend(device)
    return _default[device]


__all__ = ["Backend", "get_backend", "EPI_NONE", "EPI_RELU", "EPI_GELU_ERF", "EPI_GELU_TANH",
           "EPI_RELU_BWD"]
