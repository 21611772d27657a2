"""The gradient-exchange entry points (NCCL all-reduce behind the C ABI) on one GPU: a world of one rank
sums over itself, so the result is the input times `scale`; both ways of forming a communicator."""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_world_of_one_through_the_python_object(be, rng):
    from minitensor_b200.comm import Communicator
    uid = Communicator.unique_id()
    assert len(uid) == 128 and any(uid)
    comm = Communicator(1, 0, be.device.index, uid)
    x = rng.standard_normal(100_003).astype(np.float32)
    t = torch.from_numpy(x).to(be.device)
    stream = torch.cuda.Stream(device=be.device)
    stream.wait_stream(torch.cuda.current_stream(be.device))
    comm.all_reduce_sum(t, stream)
    comm.all_reduce_sum(t[1:], stream, scale=0.25)         # a slice that is not 16-byte aligned
    stream.synchronize()
    exp = x.copy()
    exp[1:] *= np.float32(0.25)
    np.testing.assert_array_equal(t.cpu().numpy(), exp)
    with pytest.raises(ValueError):
        comm.all_reduce_sum(t.double(), stream)
    with pytest.raises(ValueError):
        Communicator(2, 2, be.device.index, uid)            # rank outside the world
    comm.close()


def test_single_process_form_and_argument_checks(be):
    lib = be.lib
    h = C.c_void_p()
    devs = (C.c_int32 * 1)(be.device.index)
    assert lib.mtb200_comm_init(1, devs, C.byref(h)) == 0 and h.value
    t = torch.arange(1000, dtype=torch.float32, device=be.device)
    torch.cuda.synchronize()
    assert lib.mtb200_comm_group_begin(h) == 0
    assert lib.mtb200_allreduce_sum_f32(h, 0, C.c_void_p(t.data_ptr()), t.numel(), 2.0) == 0
    assert lib.mtb200_comm_group_end(h) == 0
    torch.cuda.synchronize()
    assert torch.equal(t.cpu(), torch.arange(1000, dtype=torch.float32) * 2)
    assert lib.mtb200_allreduce_sum_f32(h, 1, C.c_void_p(t.data_ptr()), 4, 1.0) == 1      # no such local rank
    assert lib.mtb200_allreduce_sum_f32(h, 0, None, 4, 1.0) == 1
    assert lib.mtb200_allreduce_sum_f32(h, 0, None, 0, 1.0) == 0                            # nothing to do
    assert lib.mtb200_comm_destroy(h) == 0
    bad = (C.c_int32 * 1)(99)
    assert lib.mtb200_comm_init(1, bad, C.byref(h)) == 1
    assert lib.mtb200_comm_init(0, devs, C.byref(h)) == 1
    assert lib.mtb200_allreduce_sum_f32(None, 0, None, 0, 1.0) == 1
