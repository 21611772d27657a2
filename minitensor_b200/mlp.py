"""Device-resident MLP training step: DenseLayer -> ReLU -> ... -> DenseLayer,
CrossEntropyLoss(mean), Adam.

This is the reference's training loop of ``nn.Sequential`` + ``nn.CrossEntropyLoss``
+ ``optim.Adam`` (``engine/src/nn/sequential.rs:74-83``, ``nn/dense_layer.rs:139-169``,
``operations/loss/regression.rs:178-251``, ``autograd/graph.rs:222-282``,
``optim/adam.rs:483-514``) laid out for one GPU per process:

* parameters, gradients and Adam moments are four flat f32 buffers in layer
  order (W [out,in] then b [out] per layer); one Adam launch updates everything;
* activations and gradient buffers are allocated once;
* forward   h_{l+1} = relu(h_l W_l^T + b_l)     one GEMM, bias + ReLU in the epilogue
* backward  db_l = colsum(g), dW_l = g^T h_l     GEMM writes straight into the flat gradient
            g   <- (g W_l) * (h_l > 0)           one GEMM, ReLU mask in the epilogue
  (no dX for the first layer: the input does not require grad, ``autograd/mod/core.rs:763``);
* with ``world_size`` > 1 the batch is sharded by rows, each layer's slice of the
  flat gradient is all-reduced (sum; NCCL through the library's ``mtb200_allreduce_sum_f32``)
  as soon as it is written, while the remaining backward GEMMs run, and Adam applies
  ``1/world_size`` so every rank takes the same step on the mean of the per-rank gradients.
  ``torch.distributed`` is used only to hand the NCCL id from rank 0 to the other ranks.
"""
from __future__ import annotations

import math
import os
from typing import List, Optional, Sequence

import numpy as np
import torch

from ._lib import EPI_NONE, EPI_RELU, EPI_RELU_BWD
from .backend import Backend, get_backend


def mlp_layout(dims: Sequence[int]):
    """Offsets of every layer's W and b in the flat parameter buffer: (w_off, b_off, total)."""
    w_off, b_off, total = [], [], 0
    for l in range(len(dims) - 1):
        w_off.append(total)
        total += int(dims[l]) * int(dims[l + 1])
        b_off.append(total)
        total += int(dims[l + 1])
    return w_off, b_off, total


def shard_rows(n_rows: int, world_size: int, rank: int):
    """Row range [lo, hi) of the global batch that ``rank`` trains on (equal shards)."""
    if n_rows % world_size:
        raise ValueError(f"global batch {n_rows} is not divisible by world size {world_size}")
    per = n_rows // world_size
    return rank * per, (rank + 1) * per


def mlp_flops_per_sample(dims: Sequence[int]) -> int:
    """2*in*out per layer forward, twice that backward, minus the first layer's dX."""
    fwd = sum(2 * int(dims[l]) * int(dims[l + 1]) for l in range(len(dims) - 1))
    return 3 * fwd - 2 * int(dims[0]) * int(dims[1])


class MLPTrainer:
    def __init__(self, dims: Sequence[int], batch: int, *, lr: float = 1e-3, beta1: float = 0.9,
                 beta2: float = 0.999, eps: float = 1e-8, device: int = 0, world_size: int = 1,
                 seed: int = 0, f32_mode: int = 0, init_params: Optional[np.ndarray] = None,
                 fused_dense: Optional[bool] = None, overlap_comm: Optional[bool] = None, comm=None):
        """``batch`` is the number of rows THIS process handles per step.

        ``fused_dense`` (default: on for the default f32 mode) runs every layer through the dense-layer
        entry points, whose backward re-uses the operands the forward prepared; off, each product is a
        separate GEMM call as the reference's autograd issues them.  ``overlap_comm`` (default: on when
        ``world_size > 1``) selects the backward order that hides the gradient all-reduces and the Adam
        update behind the products (see ``_backward_overlapped``); the results do not depend on it.
        ``comm``: the :class:`minitensor_b200.comm.Communicator` of this rank; by default one is formed over
        the initialised ``torch.distributed`` group when ``world_size > 1``."""
        if len(dims) < 2 or any(d <= 0 for d in dims) or batch <= 0:
            raise ValueError("dims needs at least two positive entries and batch must be positive")
        self.dims = [int(d) for d in dims]
        self.nl = len(dims) - 1
        self.batch = int(batch)
        self.lr, self.beta1, self.beta2, self.eps = lr, beta1, beta2, eps
        self.world_size = int(world_size)
        self.f32_mode = f32_mode
        self.fused_dense = (f32_mode == 0) if fused_dense is None else bool(fused_dense)
        if self.fused_dense and f32_mode != 0:
            raise ValueError("fused_dense uses the default f32 mode")
        self.overlap_comm = (self.world_size > 1) if overlap_comm is None else bool(overlap_comm)
        # MTB200_COMM_BUCKET=1: no overlap at all - the whole flat gradient is reduced once, after the backward pass,
        # with every SM free for it (a measurement aid: what the overlapped schedule has to beat)
        self.single_bucket = self.world_size > 1 and os.environ.get("MTB200_COMM_BUCKET", "0") == "1"
        if self.single_bucket:
            self.overlap_comm = False
        # SMs left to the collectives that overlap the backward products (MTB200_COMM_SMS, default 16 when world > 1:
        # the library's communicator asks NCCL for at most 16 CTAs, so the collectives fit beside the products)
        self.comm_sms = int(os.environ.get("MTB200_COMM_SMS", "16")) if self.world_size > 1 else 0
        self.be: Backend = get_backend(device)
        dev = self.be.device
        self.w_off, self.b_off, total = mlp_layout(self.dims)
        self.n_params = total
        if init_params is None:
            # He-uniform weights (bound sqrt(6/fan_in), engine/src/nn/init.rs:471-491), zero biases;
            # the same seed gives every rank the same replica
            rng = np.random.default_rng(seed)
            init_params = np.zeros(total, dtype=np.float32)
            for l in range(self.nl):
                fan_in, out_f = self.dims[l], self.dims[l + 1]
                bound = math.sqrt(6.0 / fan_in)
                init_params[self.w_off[l]:self.w_off[l] + fan_in * out_f] = rng.uniform(
                    -bound, bound, fan_in * out_f).astype(np.float32)
        if init_params.shape != (total,) or init_params.dtype != np.float32:
            raise ValueError("init_params must be a flat float32 array of all W, b in layer order")
        self.params = torch.from_numpy(init_params.copy()).to(dev)
        self.grads = torch.zeros(total, dtype=torch.float32, device=dev)
        self.m = torch.zeros_like(self.grads)
        self.v = torch.zeros_like(self.grads)
        self.step_count = 0
        self.W = [self.params[self.w_off[l]:self.w_off[l] + self.dims[l] * self.dims[l + 1]].view(
            self.dims[l + 1], self.dims[l]) for l in range(self.nl)]
        self.b = [self.params[self.b_off[l]:self.b_off[l] + self.dims[l + 1]] for l in range(self.nl)]
        self.dW = [self.grads[self.w_off[l]:self.w_off[l] + self.dims[l] * self.dims[l + 1]].view(
            self.dims[l + 1], self.dims[l]) for l in range(self.nl)]
        self.db = [self.grads[self.b_off[l]:self.b_off[l] + self.dims[l + 1]] for l in range(self.nl)]
        B = self.batch
        self.h = [torch.empty(B, self.dims[l + 1], dtype=torch.float32, device=dev) for l in range(self.nl)]
        self.g = [torch.empty(B, self.dims[l + 1], dtype=torch.float32, device=dev) for l in range(self.nl)]
        self.saved = [None] * self.nl
        if self.fused_dense:
            for l in range(self.nl):
                nbytes = self.be.dense_saved_bytes(B, self.dims[l], self.dims[l + 1])
                if nbytes:
                    self.saved[l] = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        # double-buffered staging for batches that arrive from host memory
        self._x_dev = [None, None]
        self._y_dev = [None, None]
        self._copy_stream = torch.cuda.Stream(device=dev)
        self._copy_done = [None, None]
        self._slot = 0
        self._side_stream = None
        self._comm_stream = None
        self.comm = comm
        if self.world_size > 1:
            if self.comm is None:
                from .comm import Communicator
                self.comm = Communicator.from_process_group(device)
            if self.comm.world_size != self.world_size:
                raise ValueError("communicator and trainer disagree on the world size")
            self._comm_stream = torch.cuda.Stream(device=dev)
        self._dy_blocks = None
        self._counted = False
        self._step_dev = None
        self._graph = None

    # ------------------------------------------------------------------ host batches
    def prefetch(self, x_host: torch.Tensor, labels_host: torch.Tensor) -> int:
        """Start the host->device copy of a batch (pinned memory) on the copy stream; returns its slot."""
        slot = self._slot
        self._slot ^= 1
        dev = self.be.device
        if self._x_dev[slot] is None:
            self._x_dev[slot] = torch.empty(self.batch, self.dims[0], dtype=torch.float32, device=dev)
            self._y_dev[slot] = torch.empty(self.batch, dtype=torch.int64, device=dev)
        # the slot may still be read by the step that used it last
        self._copy_stream.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(self._copy_stream):
            self._x_dev[slot].copy_(x_host, non_blocking=True)
            self._y_dev[slot].copy_(labels_host, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(self._copy_stream)
        self._copy_done[slot] = ev
        return slot

    def step_slot(self, slot: int) -> torch.Tensor:
        torch.cuda.current_stream(self.be.device).wait_event(self._copy_done[slot])
        return self.step(self._x_dev[slot], self._y_dev[slot])

    # ------------------------------------------------------------------ one step
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        be, a = self.be, x
        for l in range(self.nl):
            epi = EPI_RELU if l + 1 < self.nl else EPI_NONE
            if self.fused_dense:
                be.dense_forward(a, self.W[l], self.b[l], epi, out=self.h[l], saved=self.saved[l])
            else:
                be.gemm(a, self.W[l], trans_b=True, bias=self.b[l], epilogue=epi, out=self.h[l], f32_mode=self.f32_mode)
            a = self.h[l]
        return a

    def capture(self, x: torch.Tensor, labels: torch.Tensor):
        """Record one training step on the fixed device buffers ``x`` / ``labels`` into a CUDA graph and return
        ``replay() -> loss``: every later step is one graph launch instead of some forty kernel launches, which
        is what bounds small models.  New batches are copied INTO ``x`` / ``labels`` before a replay.  At least
        one eager ``step`` must have run (it sizes the library's scratch memory, which may not grow while a
        stream is being captured); Adam's step count moves to device memory so replays keep advancing it."""
        if self.world_size != 1:
            raise ValueError("capture() records single-GPU steps")
        if self.step_count < 1:
            raise RuntimeError("run one eager step() before capture()")
        if tuple(x.shape) != (self.batch, self.dims[0]):
            raise ValueError(f"expected input of shape {(self.batch, self.dims[0])}, got {tuple(x.shape)}")
        dev = self.be.device
        self._step_dev = torch.full((1,), self.step_count, dtype=torch.int64, device=dev)
        torch.cuda.synchronize(dev)
        graph = torch.cuda.CUDAGraph()
        self._counted = True
        try:
            with torch.cuda.graph(graph):
                loss = self.step(x, labels)
        finally:
            self._counted = False
        self.step_count -= 1   # recording ran no kernel

        def replay() -> torch.Tensor:
            graph.replay()
            self.step_count += 1
            return loss

        self._graph = graph    # keeps the recorded buffers alive
        return replay

    def step(self, x: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
        """One training step on device-resident ``x [batch, in]`` / ``labels [batch]``; returns the
        (local-shard mean) loss as a 1-element device tensor."""
        be = self.be
        if tuple(x.shape) != (self.batch, self.dims[0]):
            raise ValueError(f"expected input of shape {(self.batch, self.dims[0])}, got {tuple(x.shape)}")
        logits = self.forward(x)
        loss, _ = be.cross_entropy_into(logits, labels, self.g[self.nl - 1])
        self.step_count += 1
        if self.overlap_comm and self.fused_dense:
            self._backward_overlapped(x)
            return loss
        for l in range(self.nl - 1, -1, -1):
            g = self.g[l]
            a_in = x if l == 0 else self.h[l - 1]
            if self.fused_dense:
                # db, dW = g^T a and (g W) * relu' from two passes over g and the forward pass's planes
                be.dense_backward(a_in, self.W[l], g, self.saved[l], need_dx=l > 0, dx=self.g[l - 1] if l > 0 else None,
                                  dx_epilogue=EPI_RELU_BWD if l > 0 else EPI_NONE, dx_aux=self.h[l - 1] if l > 0 else None,
                                  dw=self.dW[l], db=self.db[l])
            else:
                be.colsum(g, out=self.db[l])
                be.gemm(g, a_in, trans_a=True, out=self.dW[l], f32_mode=self.f32_mode)      # dW = g^T a
            if self.world_size > 1 and not self.single_bucket:
                lo = self.w_off[l]
                hi = self.b_off[l] + self.dims[l + 1]
                self._all_reduce(lo, hi)
            if l > 0 and not self.fused_dense:
                be.gemm(g, self.W[l], epilogue=EPI_RELU_BWD, aux=self.h[l - 1], out=self.g[l - 1],
                        f32_mode=self.f32_mode)                                            # (g W) * relu'
        if self.single_bucket and not self._counted:
            # the backward pass is done: reduce layer by layer on the communication stream and update each layer on
            # the side stream as soon as its slice has landed, so the (HBM-bound) update of layer l hides behind the
            # reduction of layer l + 1 and nothing runs beside the products
            main = torch.cuda.current_stream(be.device)
            if self._side_stream is None:
                self._side_stream = torch.cuda.Stream(device=be.device)
            side = self._side_stream
            for l in range(self.nl):
                lo, hi = self.w_off[l], self.b_off[l] + self.dims[l + 1]
                self._all_reduce(lo, hi)
                side.wait_stream(self._comm_stream)
                with torch.cuda.stream(side):
                    be.adam_step(self.params[lo:hi], self.grads[lo:hi], self.m[lo:hi], self.v[lo:hi], lr=self.lr,
                                 beta1=self.beta1, beta2=self.beta2, eps=self.eps, step=self.step_count,
                                 grad_scale=1.0 / self.world_size)
            main.wait_stream(side)
            return loss
        if self.single_bucket:
            self._all_reduce(0, self.n_params)
        if self.world_size > 1:
            torch.cuda.current_stream(be.device).wait_stream(self._comm_stream)
        if self._counted:
            be.adam_step_counted(self.params, self.grads, self.m, self.v, lr=self.lr, beta1=self.beta1,
                                 beta2=self.beta2, eps=self.eps, counter=self._step_dev, advance=True)
        else:
            be.adam_step(self.params, self.grads, self.m, self.v, lr=self.lr, beta1=self.beta1, beta2=self.beta2,
                         eps=self.eps, step=self.step_count, grad_scale=1.0 / self.world_size)
        return loss

    def _backward_overlapped(self, x: torch.Tensor) -> None:
        """Backward + update for data-parallel runs, ordered so that communication hides behind the products:
        first the chain of input gradients (no parameter gradient yet), then the parameter gradients from the
        FIRST layer on - the first layer's is the largest, so its all-reduce starts earliest and the one
        left exposed at the end is the last layer's small one - and each layer's Adam update on a side
        stream as soon as its all-reduce has landed (HBM-bound, so it overlaps the tensor-bound products)."""
        be = self.be
        if self._dy_blocks is None:
            self._dy_blocks = [None] * self.nl
            for l in range(1, self.nl):
                nbytes = be.dense_dy_bytes(self.batch, self.dims[l], self.dims[l + 1]) if self.saved[l] is not None else 0
                if nbytes:
                    self._dy_blocks[l] = torch.empty(nbytes, dtype=torch.uint8, device=be.device)
        for l in range(self.nl - 1, 0, -1):
            # input gradient and bias gradient now; dY's operand for the weight gradient is kept for the second pass
            be.dense_backward(self.h[l - 1], self.W[l], self.g[l], self.saved[l], need_dx=True, dx=self.g[l - 1],
                              dx_epilogue=EPI_RELU_BWD, dx_aux=self.h[l - 1], need_dw=False,
                              need_db=self._dy_blocks[l] is not None, db=self.db[l],
                              dy_block=self._dy_blocks[l], dy_mode=1)
        if self.comm_sms > 0:   # from here on all-reduces run beside the products: leave them SMs of their own
            sm_total = torch.cuda.get_device_properties(be.device).multi_processor_count
            be.set_gemm_sm_limit(sm_total - self.comm_sms)
        main = torch.cuda.current_stream(be.device)
        if self._side_stream is None:
            self._side_stream = torch.cuda.Stream(device=be.device)
        side = self._side_stream
        for l in range(self.nl):
            a_in = x if l == 0 else self.h[l - 1]
            if self._dy_blocks[l] is not None:
                be.dense_backward(a_in, self.W[l], self.g[l], self.saved[l], need_dx=False, dw=self.dW[l], need_db=False,
                                  dy_block=self._dy_blocks[l], dy_mode=2)
            else:
                be.dense_backward(a_in, self.W[l], self.g[l], self.saved[l], need_dx=False, dw=self.dW[l], db=self.db[l])
            lo, hi = self.w_off[l], self.b_off[l] + self.dims[l + 1]
            if self.world_size > 1:
                self._all_reduce(lo, hi)
                side.wait_stream(self._comm_stream)   # the side stream waits for the collective, the main stream keeps issuing products
            else:
                side.wait_stream(main)
            with torch.cuda.stream(side):
                be.adam_step(self.params[lo:hi], self.grads[lo:hi], self.m[lo:hi], self.v[lo:hi], lr=self.lr,
                             beta1=self.beta1, beta2=self.beta2, eps=self.eps, step=self.step_count,
                             grad_scale=1.0 / self.world_size)
        main.wait_stream(side)
        if self.comm_sms > 0:
            be.set_gemm_sm_limit(0)   # the forward pass has nothing running beside it

    def _all_reduce(self, lo: int, hi: int) -> None:
        """Sum ``grads[lo:hi]`` over the ranks on the communication stream, ordered after the work enqueued so far
        on the current stream (the product that wrote the slice)."""
        self._comm_stream.wait_stream(torch.cuda.current_stream(self.be.device))
        self.comm.all_reduce_sum(self.grads[lo:hi], self._comm_stream)

    def params_checksum(self) -> torch.Tensor:
        """[sum, sum of squares] of the parameters in f64 on the device: equal on every rank while the replicas agree."""
        p = self.params.double()
        return torch.stack([p.sum(), (p * p).sum()])

    def flops_per_sample(self) -> int:
        return mlp_flops_per_sample(self.dims)
