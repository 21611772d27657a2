"""The allocation-free column sum (mtb200_colsum_noalloc) against the regular one.

Some users of the library cannot let a call allocate device memory: their application's own pool
owns the whole GPU, or they cannot afford the device-wide stall of cudaMalloc.  For them the
library offers a column sum whose scratch is a fixed array inside the library.  This file checks, through the C ABI, that it returns what mtb200_colsum
returns, on two calls in a row that share that array, and that inputs wider than the fixed
scratch are refused.  It is named so that pytest collects it last.
"""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _scratch_bytes() -> int:
    """The limit as the header states it (MTB200_COLSUM_NOALLOC_SCRATCH_BYTES), so a changed macro is noticed."""
    import os
    import re
    from conftest import ROOT
    text = open(os.path.join(ROOT, "include", "mtb200.h")).read()
    m = re.search(r"#define\s+MTB200_COLSUM_NOALLOC_SCRATCH_BYTES\s+\((\d+)u?\s*<<\s*(\d+)\)", text)
    assert m, "the header no longer defines the scratch size in the expected form"
    return int(m.group(1)) << int(m.group(2))


SCRATCH_BYTES = _scratch_bytes()


def _call_noalloc(lib, x: torch.Tensor) -> torch.Tensor:
    from minitensor_b200 import _lib
    m, n = x.shape
    out = torch.empty(n, dtype=x.dtype, device=x.device)
    stream = torch.cuda.current_stream(x.device).cuda_stream
    code = _lib.F32 if x.dtype == torch.float32 else _lib.F64
    _lib.check(lib.mtb200_colsum_noalloc(C.c_void_p(stream), code, m, n, x.data_ptr(), out.data_ptr()))
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_two_calls_in_a_row_match_the_regular_entry_point(be, dtype):
    lib = be.lib
    g = torch.Generator(device="cpu").manual_seed(5)
    # the second input is narrower and shorter, so it reuses part of the scratch the first one filled
    for (m, n) in [(4096, 515), (1000, 130)]:
        x = torch.randn(m, n, generator=g, dtype=dtype).to(be.device)
        got = _call_noalloc(lib, x)
        ref = be.colsum(x)
        be.sync()
        torch.cuda.synchronize()
        # both are deterministic sums in a different band split: same tolerance as the colsum tests
        tol = (1e-6 if dtype == torch.float32 else 1e-14) * x.abs().double().sum(0) + 1e-30
        assert bool(((got.double() - ref.double()).abs() <= 2 * tol).all())
        exact = x.double().sum(0)
        assert bool(((got.double() - exact).abs() <= tol).all())


def test_wide_input_uses_few_bands_and_too_wide_is_refused(be):
    lib = be.lib
    n = SCRATCH_BYTES // 4            # exactly fills the scratch with one band of f32
    x = torch.ones(3, n, dtype=torch.float32, device=be.device)
    got = _call_noalloc(lib, x)
    torch.cuda.synchronize()
    assert bool((got == 3.0).all())
    x = torch.ones(2, n + 1, dtype=torch.float32, device=be.device)
    with pytest.raises(ValueError, match="fixed scratch"):
        _call_noalloc(lib, x)
    empty = torch.empty(0, 7, dtype=torch.float32, device=be.device)
    assert not _call_noalloc(lib, empty).cpu().numpy().any()
