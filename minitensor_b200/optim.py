"""``optim.Adam`` of the reference (``bindings/src/optim.rs:355-455``,
``engine/src/optim/adam.rs:202-376,483-514``) over the fused device kernel."""
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
