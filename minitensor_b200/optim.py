"""The reference's optimizers over the device kernels: ``Adam`` / ``AdamW`` (``bindings/src/optim.rs:355-455``,
``engine/src/optim/adam.rs:202-376,483-514``), ``SGD`` (``engine/src/optim/sgd.rs``), ``RMSprop``
(``engine/src/optim/rmsprop.rs``) and gradient clipping (``engine/src/optim/optimizer.rs:55-62,199-227``,
``engine/src/optim/utils.rs:16-112``)."""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch

from .tensor import Tensor, _be


class Adam:
    def __init__(self, parameters: Sequence[Tensor], lr: float = 1e-3,
                 betas: Optional[Tuple[float, float]] = None, beta1: Optional[float] = None,
                 beta2: Optional[float] = None, epsilon: float = 1e-8, weight_decay: float = 0.0,
                 decoupled_weight_decay: bool = False):
        if betas is not None and (beta1 is not None or beta2 is not None):
            raise ValueError("pass either betas or beta1/beta2, not both")
        b1, b2 = betas if betas is not None else (beta1 if beta1 is not None else 0.9,
                                                  beta2 if beta2 is not None else 0.999)
        if lr < 0 or not (0.0 <= b1 < 1.0) or not (0.0 <= b2 < 1.0) or epsilon < 0:
            raise ValueError("invalid Adam hyper-parameter")
        self.params: List[Tensor] = list(parameters)
        for p in self.params:
            if p.dtype != "float32":
                raise TypeError("Adam on this path updates float32 parameters")
        self.lr, self.beta1, self.beta2, self.epsilon = lr, b1, b2, epsilon
        self.weight_decay, self.decoupled = weight_decay, decoupled_weight_decay
        self.step_count = 0
        self._m = [torch.zeros_like(p._buf) for p in self.params]
        self._v = [torch.zeros_like(p._buf) for p in self.params]

    def step(self) -> None:
        """One update of every parameter that has a gradient (``adam.rs:483-514``)."""
        self.step_count += 1
        be = _be()
        for p, m, v in zip(self.params, self._m, self._v):
            if p.grad is None:
                continue
            if p.grad.shape != p.shape:
                raise ValueError(f"shape mismatch: {p.shape} vs {p.grad.shape}")
            be.adam_step(p._buf, p.grad._buf, m, v, lr=self.lr, beta1=self.beta1, beta2=self.beta2,
                         eps=self.epsilon, weight_decay=self.weight_decay, decoupled=self.decoupled,
                         step=self.step_count)

    def zero_grad(self) -> None:
        for p in self.params:
            p.grad = None


class AdamW(Adam):
    """Adam with decoupled weight decay (``adam.rs``: ``decoupled_weight_decay``), default decay 0.01."""

    def __init__(self, parameters: Sequence[Tensor], lr: float = 1e-3, betas: Optional[Tuple[float, float]] = None,
                 epsilon: float = 1e-8, weight_decay: float = 0.01):
        super().__init__(parameters, lr=lr, betas=betas, epsilon=epsilon, weight_decay=weight_decay,
                         decoupled_weight_decay=True)


class _Clipping:
    """``GradientClipping::{None, ByNorm, ByValue}`` applied before a step, as ``Optimizer::clip_gradients`` does."""

    def __init__(self):
        self._clip = None

    def with_gradient_clipping(self, *, max_norm: Optional[float] = None, min_value: Optional[float] = None,
                               max_value: Optional[float] = None):
        if max_norm is not None:
            self._clip = ("norm", float(max_norm))
        elif min_value is not None and max_value is not None:
            self._clip = ("value", float(min_value), float(max_value))
        else:
            self._clip = None
        return self

    def _apply_clipping(self, params: Sequence[Tensor]) -> None:
        if self._clip is None:
            return
        grads = [p.grad._buf for p in params if p.grad is not None and p.grad.dtype in ("float32", "float64")]
        if self._clip[0] == "norm":
            _be().clip_grad_norm(grads, self._clip[1])
        else:
            _be().clip_grad_value(grads, self._clip[1], self._clip[2])


def _check_float_params(params: Sequence[Tensor], who: str) -> None:
    for p in params:
        if p.dtype not in ("float32", "float64"):
            raise ValueError(f"{who} only supports float32/float64 tensors")


class SGD(_Clipping):
    def __init__(self, parameters: Sequence[Tensor], lr: float = 0.01, momentum: float = 0.0, weight_decay: float = 0.0,
                 dampening: float = 0.0, nesterov: bool = False):
        super().__init__()
        self.params: List[Tensor] = list(parameters)
        _check_float_params(self.params, "SGD")
        self.lr, self.momentum, self.weight_decay = lr, momentum, weight_decay
        self.dampening, self.nesterov = dampening, nesterov
        self.step_count = 0
        self._v = [None] * len(self.params)

    def step(self) -> None:
        self._apply_clipping(self.params)
        self.step_count += 1
        be = _be()
        for i, p in enumerate(self.params):
            if not p.requires_grad or p.grad is None:
                continue
            if p.grad.shape != p.shape:
                raise ValueError(f"shape mismatch: {p.shape} vs {p.grad.shape}")
            if self.momentum > 0.0 and self._v[i] is None:
                self._v[i] = torch.zeros_like(p._buf)
            be.sgd_step(p._buf, p.grad._buf, self._v[i], lr=self.lr, momentum=self.momentum, dampening=self.dampening,
                        weight_decay=self.weight_decay, nesterov=self.nesterov)

    def zero_grad(self) -> None:
        for p in self.params:
            p.grad = None


class RMSprop(_Clipping):
    def __init__(self, parameters: Sequence[Tensor], lr: float = 0.01, alpha: float = 0.99, epsilon: float = 1e-8,
                 weight_decay: float = 0.0, momentum: float = 0.0, centered: bool = False):
        super().__init__()
        self.params: List[Tensor] = list(parameters)
        _check_float_params(self.params, "RMSprop")
        self.lr, self.alpha, self.epsilon = lr, alpha, epsilon
        self.weight_decay, self.momentum, self.centered = weight_decay, momentum, centered
        self.step_count = 0
        self._sq = [None] * len(self.params)
        self._mb = [None] * len(self.params)
        self._ga = [None] * len(self.params)

    def step(self) -> None:
        self._apply_clipping(self.params)
        self.step_count += 1
        be = _be()
        for i, p in enumerate(self.params):
            if not p.requires_grad or p.grad is None:
                continue
            if p.grad.shape != p.shape:
                raise ValueError(f"shape mismatch: {p.shape} vs {p.grad.shape}")
            if self._sq[i] is None:
                self._sq[i] = torch.zeros_like(p._buf)
            if self.momentum > 0.0 and self._mb[i] is None:
                self._mb[i] = torch.zeros_like(p._buf)
            if self.centered and self._ga[i] is None:
                self._ga[i] = torch.zeros_like(p._buf)
            be.rmsprop_step(p._buf, p.grad._buf, self._sq[i], self._mb[i], self._ga[i], lr=self.lr, alpha=self.alpha,
                            eps=self.epsilon, weight_decay=self.weight_decay, momentum=self.momentum)

    def zero_grad(self) -> None:
        for p in self.params:
            p.grad = None
