"""The entry point that allocates nothing (tg_fp8_gemm_pertensor_smallm_static).

Some callers cannot call cudaMalloc: a serving process whose pool already owns
the GPU, or a decode loop that must not hit the allocator's device-wide
synchronisation.  For them the small-M GEMM keeps its split-K scratch in a
fixed __device__ array inside the library.  The test calls that entry point
through the C ABI twice in a row - the second call finds the first call's
leftovers in the shared array - and compares each result with the regular
entry point's on the same inputs, under the tolerance of the other GEMM tests.
The file name sorts last so that a run that stops at the first failure has
already run every other test.
"""

import ctypes

import pytest
import torch

from oracle import torch_ref as R

pytestmark = pytest.mark.gpu

import tilegym_b200 as tg  # noqa: E402
from tilegym_b200 import _lib  # noqa: E402


def _static_call(a, b, sa, sb, out, bias=None):
    rc = _lib.lib().tg_fp8_gemm_pertensor_smallm_static(
        _lib.ref(_lib.desc(out)), _lib.ref(_lib.desc(a)), _lib.ref(_lib.desc(b)), sa.data_ptr(), sb.data_ptr(),
        ctypes.c_float(1.0), _lib.ref(_lib.desc(bias)), ctypes.c_float(0.0), out.device.index,
        torch.cuda.current_stream(out.device).cuda_stream,
    )
    _lib.check_rc(rc)
    return out


def test_two_calls_in_a_row_match_the_regular_entry_point(dev):
    cases = [(64, 4096, 4096, 31), (16, 6144, 4096, 32)]  # the second call reuses scratch the first one dirtied
    for M, N, K, seed in cases:
        a8, b8, sa, sb = (t.to(dev) for t in R.gen_per_tensor_case(M, N, K, seed))
        bias = torch.randn(N, device=dev)
        expect = tg.fp8_scaled_mm(a8, b8, sa, sb, bias)
        out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev)
        _static_call(a8, b8, sa, sb, out, bias)
        res = R.check_tolerance(out, expect)
        assert res["ok"], (M, N, K, res)
    _lib.device_status(dev.index)


def test_same_call_twice_gives_identical_bits(dev):
    a8, b8, sa, sb = (t.to(dev) for t in R.gen_per_tensor_case(8, 4096, 14336, 33))
    out1 = torch.empty(8, 4096, dtype=torch.bfloat16, device=dev)
    out2 = torch.empty_like(out1)
    tg.fp8_scaled_mm_no_alloc(a8, b8, sa, sb, out1)
    tg.fp8_scaled_mm_no_alloc(a8, b8, sa, sb, out2)
    assert torch.equal(out1, out2)
    assert R.check_tolerance(out1, R.ref_fp8_scaled_mm(a8.cpu(), b8.cpu(), sa.cpu(), sb.cpu()))["ok"]


def test_sizes_beyond_the_static_scratch_are_rejected(dev):
    a = torch.zeros(65, 128, dtype=torch.float8_e4m3fn, device=dev)
    b = torch.zeros(256, 128, dtype=torch.float8_e4m3fn, device=dev)
    out = torch.empty(65, 256, dtype=torch.bfloat16, device=dev)
    with pytest.raises(RuntimeError, match="exceeds the 64 rows"):
        tg.fp8_scaled_mm_no_alloc(a, b, None, None, out)
