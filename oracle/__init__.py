"""NumPy-facing binding of the CPU oracle (``oracle/oracle.cpp``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by ``__graft_entry__.smoke``
and by the CPU-baseline / reference legs of ``bench.py``.  Nothing under
``minitensor_b200/`` may import it.  Each function documents the minitensor
source it restates in ``oracle.cpp``.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "liboracle.so")
_lib = None

_i64, _f32, _f64, _int = C.c_int64, C.c_float, C.c_double, C.c_int
_p = C.c_void_p


def build(force: bool = False) -> str:
    """Compile ``liboracle.so`` with the Makefile beside this file."""
    src = os.path.join(_HERE, "oracle.cpp")
    if force or not os.path.exists(LIB_PATH) or os.path.getmtime(src) > os.path.getmtime(LIB_PATH):
        subprocess.run(["make", "-C", _HERE, "-B", "liboracle.so"], check=True,
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    return LIB_PATH


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            build()
        _lib = C.CDLL(LIB_PATH)
        _lib.orc_mlp_train_step_f32.restype = _f32
        _lib.orc_num_threads.restype = _int
        _lib.orc_conv2d_f32.restype = _int
        _lib.orc_cross_entropy_f32.restype = _int
        _lib.orc_cross_entropy_ex_f32.restype = _int
        _lib.orc_sumsq_f32.restype = _f64
        _lib.orc_sumsq_f64.restype = _f64
    return _lib


def num_threads() -> int:
    return int(lib().orc_num_threads())


def _c(a: np.ndarray, dtype) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=dtype)


def _ptr(a):
    return None if a is None else a.ctypes.data_as(_p)


_MM = {np.dtype(np.float32): "orc_matmul_f32", np.dtype(np.float64): "orc_matmul_f64",
       np.dtype(np.int32): "orc_matmul_i32", np.dtype(np.int64): "orc_matmul_i64"}


def matmul(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """Row-major ``[..., M, K] @ [..., K, N]`` with identical batch dims, in the operand dtype."""
    if a.dtype != b.dtype:
        raise TypeError("dtype mismatch")
    fn = getattr(lib(), _MM[a.dtype])
    a = np.ascontiguousarray(a)
    b = np.ascontiguousarray(b)
    m, k = a.shape[-2:]
    k2, n = b.shape[-2:]
    assert k == k2 and a.shape[:-2] == b.shape[:-2]
    batch = int(np.prod(a.shape[:-2], dtype=np.int64)) if a.ndim > 2 else 1
    out = np.zeros(a.shape[:-2] + (m, n), dtype=a.dtype)
    if out.size and k:
        fn(_i64(batch), _i64(m), _i64(k), _i64(n), _ptr(a), _ptr(b), _ptr(out))
    return out


def matmul_acc_wide(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """f32 operands accumulated in f64 (or f64 operands in long double); result is f64."""
    a = np.ascontiguousarray(a)
    b = np.ascontiguousarray(b)
    m, k = a.shape[-2:]
    n = b.shape[-1]
    batch = int(np.prod(a.shape[:-2], dtype=np.int64)) if a.ndim > 2 else 1
    out = np.zeros(a.shape[:-2] + (m, n), dtype=np.float64)
    fn = lib().orc_matmul_f32_acc64 if a.dtype == np.float32 else lib().orc_matmul_f64_acc80
    if out.size and k:
        fn(_i64(batch), _i64(m), _i64(k), _i64(n), _ptr(a), _ptr(b), _ptr(out))
    return out


def matmul_backward(a: np.ndarray, b: np.ndarray, dy: np.ndarray, need_a=True, need_b=True):
    """(dA, dB) of ``a @ b`` for upstream ``dy`` (f32 / f64), transposes materialised."""
    a = np.ascontiguousarray(a)
    b = np.ascontiguousarray(b)
    dy = np.ascontiguousarray(dy)
    m, k = a.shape[-2:]
    n = b.shape[-1]
    batch = int(np.prod(a.shape[:-2], dtype=np.int64)) if a.ndim > 2 else 1
    da = np.zeros_like(a) if need_a else None
    db = np.zeros_like(b) if need_b else None
    fn = lib().orc_matmul_backward_f32 if a.dtype == np.float32 else lib().orc_matmul_backward_f64
    fn(_i64(batch), _i64(m), _i64(k), _i64(n), _ptr(a), _ptr(b), _ptr(dy), _ptr(da), _ptr(db))
    return da, db


def dense_forward(x: np.ndarray, w: np.ndarray, bias) -> np.ndarray:
    x = _c(x, np.float32)
    w = _c(w, np.float32)
    bias = None if bias is None else _c(bias, np.float32)
    rows = int(np.prod(x.shape[:-1], dtype=np.int64))
    out_f, in_f = w.shape
    y = np.zeros(x.shape[:-1] + (out_f,), dtype=np.float32)
    lib().orc_dense_forward_f32(_i64(rows), _i64(in_f), _i64(out_f), _ptr(x), _ptr(w), _ptr(bias), _ptr(y))
    return y


def sum_dim0(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x)
    out = np.zeros(x.shape[1], dtype=x.dtype)
    fn = lib().orc_sum_dim0_f32 if x.dtype == np.float32 else lib().orc_sum_dim0_f64
    fn(_i64(x.shape[0]), _i64(x.shape[1]), _ptr(x), _ptr(out))
    return out


def relu(x: np.ndarray):
    """Returns (y, mask) as the reference's relu does (mask = x > 0, false for NaN)."""
    x = np.ascontiguousarray(x)
    y = np.empty_like(x)
    mask = np.empty(x.shape, dtype=np.uint8)
    fn = lib().orc_relu_f32 if x.dtype == np.float32 else lib().orc_relu_f64
    fn(_i64(x.size), _ptr(x), _ptr(y), _ptr(mask))
    return y, mask


def relu_backward(mask: np.ndarray, go: np.ndarray) -> np.ndarray:
    go = np.ascontiguousarray(go)
    mask = _c(mask, np.uint8)
    gi = np.empty_like(go)
    fn = lib().orc_relu_backward_f32 if go.dtype == np.float32 else lib().orc_relu_backward_f64
    fn(_i64(go.size), _ptr(mask), _ptr(go), _ptr(gi))
    return gi


def gelu(x: np.ndarray, approximate: bool = False) -> np.ndarray:
    x = np.ascontiguousarray(x)
    y = np.empty_like(x)
    fn = lib().orc_gelu_f32 if x.dtype == np.float32 else lib().orc_gelu_f64
    fn(_i64(x.size), _ptr(x), _ptr(y), _int(int(approximate)))
    return y


def gelu_backward(x: np.ndarray, go: np.ndarray, approximate: bool = False) -> np.ndarray:
    x = np.ascontiguousarray(x)
    go = np.ascontiguousarray(go)
    gi = np.empty_like(x)
    fn = lib().orc_gelu_backward_f32 if x.dtype == np.float32 else lib().orc_gelu_backward_f64
    fn(_i64(x.size), _ptr(x), _ptr(go), _ptr(gi), _int(int(approximate)))
    return gi


def conv2d(x, w, bias, stride, padding) -> np.ndarray:
    x = _c(x, np.float32)
    w = _c(w, np.float32)
    bias = None if bias is None else _c(bias, np.float32)
    n, c, h, wd = x.shape
    o, _, kh, kw = w.shape
    if stride[0] == 0 or stride[1] == 0:
        raise ValueError("stride values must be greater than zero")
    if kh > h + 2 * padding[0] or kw > wd + 2 * padding[1]:
        raise ValueError("kernel size cannot be larger than padded input")
    oh = (h + 2 * padding[0] - kh) // stride[0] + 1
    ow = (wd + 2 * padding[1] - kw) // stride[1] + 1
    y = np.zeros((n, o, oh, ow), dtype=np.float32)
    rc = lib().orc_conv2d_f32(*[_i64(v) for v in (n, c, h, wd, o, kh, kw, stride[0], stride[1], padding[0],
                                                 padding[1])], _ptr(x), _ptr(w), _ptr(bias), _ptr(y))
    if rc:
        raise ValueError("conv2d: invalid geometry")
    return y


def conv2d_backward(x, w, go, stride, padding, need_x=True, need_w=True, need_b=True):
    x = _c(x, np.float32)
    w = _c(w, np.float32)
    go = _c(go, np.float32)
    n, c, h, wd = x.shape
    o, _, kh, kw = w.shape
    gx = np.zeros_like(x) if need_x else None
    gw = np.zeros_like(w) if need_w else None
    gb = np.zeros(o, dtype=np.float32) if need_b else None
    lib().orc_conv2d_backward_f32(*[_i64(v) for v in (n, c, h, wd, o, kh, kw, stride[0], stride[1], padding[0],
                                                      padding[1])], _ptr(x), _ptr(w), _ptr(go), _ptr(gx),
                                  _ptr(gw), _ptr(gb))
    return gx, gw, gb


def cross_entropy(logits, labels, mean: bool = True, upstream: float = 1.0, want_grad: bool = True):
    logits = _c(logits, np.float32)
    labels = _c(labels, np.int64)
    bsz, ncls = logits.shape
    loss = np.zeros(1, dtype=np.float32)
    grad = np.zeros_like(logits) if want_grad else None
    rc = lib().orc_cross_entropy_f32(_i64(bsz), _i64(ncls), _ptr(logits), _ptr(labels), _int(int(mean)),
                                     _f32(upstream), _ptr(loss), _ptr(grad))
    if rc:
        raise IndexError("class index out of range")
    return loss[0], grad


def cross_entropy_ex(logits, targets, reduction: str = "mean", upstream: float = 1.0, upstream_rows=None,
                     want_grad: bool = True):
    """General form: ``targets`` are class indices ``[B]`` (integer dtype) or probabilities ``[B, C]`` (float);
    ``reduction`` in ("sum", "mean", "none").  Returns (loss scalar or ``[B]`` array, grad or None)."""
    logits = _c(logits, np.float32)
    bsz, ncls = logits.shape
    targets = np.asarray(targets)
    labels = soft = None
    if targets.dtype.kind in "iu":
        labels = _c(targets, np.int64)
    else:
        soft = _c(targets, np.float32)
        assert soft.shape == logits.shape
    red = {"sum": 0, "mean": 1, "none": 2}[reduction]
    loss = np.zeros(bsz if red == 2 else 1, dtype=np.float32)
    grad = np.zeros_like(logits) if want_grad else None
    rows = _c(upstream_rows, np.float32) if upstream_rows is not None else None
    rc = lib().orc_cross_entropy_ex_f32(_i64(bsz), _i64(ncls), _ptr(logits), _ptr(labels), _ptr(soft), _int(red),
                                        _f32(upstream), _ptr(rows), _ptr(loss), _ptr(grad))
    if rc:
        raise IndexError("class index out of range")
    return (loss if red == 2 else loss[0]), grad


def _sfx(a: np.ndarray) -> str:
    assert a.dtype in (np.float32, np.float64) and a.flags.c_contiguous
    return "f32" if a.dtype == np.float32 else "f64"


def sgd_step(p, g, v=None, lr=0.01, momentum=0.0, dampening=0.0, weight_decay=0.0, nesterov=False) -> None:
    """In place on ``p`` (and ``v`` when ``momentum > 0``); float32 or float64 arrays."""
    g = _c(g, p.dtype)
    getattr(lib(), "orc_sgd_step_" + _sfx(p))(_i64(p.size), _ptr(p), _ptr(g), _ptr(v), _f64(lr), _f64(momentum),
                                              _f64(dampening), _f64(weight_decay), _int(int(nesterov)))


def rmsprop_step(p, g, sq, mb=None, ga=None, lr=0.01, alpha=0.99, eps=1e-8, weight_decay=0.0, momentum=0.0) -> None:
    """In place on ``p``, ``sq`` and the optional momentum / centered buffers."""
    g = _c(g, p.dtype)
    getattr(lib(), "orc_rmsprop_step_" + _sfx(p))(_i64(p.size), _ptr(p), _ptr(g), _ptr(sq), _ptr(mb), _ptr(ga),
                                                  _f64(lr), _f64(alpha), _f64(eps), _f64(weight_decay), _f64(momentum))


def sumsq(x) -> float:
    x = np.ascontiguousarray(x)
    return float(getattr(lib(), "orc_sumsq_" + _sfx(x))(_i64(x.size), _ptr(x)))


def clip_grad_norm(grads, max_norm: float) -> float:
    """GradientUtils::clip_grad_norm over a list of arrays (in place); returns the norm before clipping."""
    total = float(np.sqrt(sum(sumsq(g) for g in grads)))
    if total > max_norm:
        coef = max_norm / (total + 1e-6)
        for g in grads:
            getattr(lib(), "orc_scale_" + _sfx(g))(_i64(g.size), _ptr(g), _f64(coef))
    return total


def clip_grad_value(grads, lo: float, hi: float) -> None:
    for g in grads:
        getattr(lib(), "orc_clamp_" + _sfx(g))(_i64(g.size), _ptr(g), _f64(lo), _f64(hi))


def batch_norm(x, weight=None, bias=None, running_mean=None, running_var=None, training=True, momentum=0.1,
               eps=1e-5):
    """``x [N, C, *spatial]`` float32/float64; running estimates are updated in place while training.
    Returns ``(y, save_mean, save_invstd)``."""
    x = np.ascontiguousarray(x)
    sfx = _sfx(x)
    n, c = x.shape[0], x.shape[1]
    sp = int(np.prod(x.shape[2:])) if x.ndim > 2 else 1
    y = np.empty_like(x)
    mean = np.empty(c, x.dtype)
    invstd = np.empty(c, x.dtype)
    w = _c(weight, x.dtype) if weight is not None else None
    b = _c(bias, x.dtype) if bias is not None else None
    for r in (running_mean, running_var):
        assert r is None or (r.dtype == x.dtype and r.flags.c_contiguous)
    getattr(lib(), "orc_batch_norm_fwd_" + sfx)(_i64(n), _i64(c), _i64(sp), _ptr(x), _ptr(w), _ptr(b),
                                                _ptr(running_mean), _ptr(running_var), _int(int(training)),
                                                _f64(momentum), _f64(eps), _ptr(y), _ptr(mean), _ptr(invstd))
    return y, mean, invstd


def batch_norm_backward(x, dy, weight, mean, invstd, batch_stats=True):
    x = np.ascontiguousarray(x)
    sfx = _sfx(x)
    dy = _c(dy, x.dtype)
    n, c = x.shape[0], x.shape[1]
    sp = int(np.prod(x.shape[2:])) if x.ndim > 2 else 1
    dx = np.empty_like(x)
    dw = np.empty(c, x.dtype)
    db = np.empty(c, x.dtype)
    w = _c(weight, x.dtype) if weight is not None else None
    getattr(lib(), "orc_batch_norm_bwd_" + sfx)(_i64(n), _i64(c), _i64(sp), _ptr(x), _ptr(dy), _ptr(w),
                                                _ptr(_c(mean, x.dtype)), _ptr(_c(invstd, x.dtype)),
                                                _int(int(batch_stats)), _ptr(dx), _ptr(dw), _ptr(db))
    return dx, dw, db


def dropout_mask(n: int, p: float, seed: int, offset: int = 0) -> np.ndarray:
    mask = np.empty(n, np.float32)
    lib().orc_dropout_mask_f32(_i64(n), _f64(p), C.c_uint64(seed), C.c_uint64(offset), _ptr(mask))
    return mask


def adam_step(p, g, m, v, lr, beta1, beta2, eps, weight_decay=0.0, decoupled=False, step=1) -> None:
    """In place on ``p``, ``m``, ``v`` (contiguous float32 arrays)."""
    for a in (p, m, v):
        assert a.dtype == np.float32 and a.flags.c_contiguous
    g = _c(g, np.float32)
    lib().orc_adam_step_f32(_i64(p.size), _ptr(p), _ptr(g), _ptr(m), _ptr(v), _f64(lr), _f64(beta1), _f64(beta2),
                            _f64(eps), _f64(weight_decay), _int(int(decoupled)), _i64(step))


def mlp_train_step(dims, x, labels, params, m, v, lr, beta1, beta2, eps, step, want_grads=False):
    """One reference-ordered MLP training step; params/m/v are flat float32 arrays updated in place."""
    dims_a = np.asarray(dims, dtype=np.int64)
    x = _c(x, np.float32)
    labels = _c(labels, np.int64)
    grads = np.zeros_like(params) if want_grads else None
    loss = lib().orc_mlp_train_step_f32(_i64(len(dims) - 1), _ptr(dims_a), _i64(x.shape[0]), _ptr(x), _ptr(labels),
                                        _ptr(params), _ptr(m), _ptr(v), _ptr(grads), _f64(lr), _f64(beta1),
                                        _f64(beta2), _f64(eps), _i64(step))
    return float(loss), grads
