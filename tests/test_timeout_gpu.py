"""The bounded device-side wait really gives up, cleanly.

Every wait inside the kernels (for a TMA copy, the tensor core, a released buffer) carries a time limit; when
it runs out the kernel records a code, leaves its loops, frees its TMEM and returns, and the host reads
TG_ERR_TIMEOUT (-7) from tg_device_status.  Here that path runs once on purpose through
tg_selftest_wait_timeout: one thread block with the kernels' role layout waits - with the kernels' own wait
code and a limit of about a millisecond - for a barrier that nothing arrives on.  The block returns by
itself; nothing faults or spins without bound, and the CUDA context stays usable, which the test proves by
running a normal GEMM afterwards."""

import time

import pytest
import torch

from oracle import torch_ref as R

pytestmark = pytest.mark.gpu

import tilegym_b200 as tg  # noqa: E402
from tilegym_b200 import _lib  # noqa: E402


def test_expired_wait_reports_timeout_and_the_context_survives(dev):
    L = _lib.lib()
    _lib.device_status(dev.index)  # clean start
    t0 = time.perf_counter()
    _lib.check_rc(L.tg_selftest_wait_timeout(1000, dev.index, torch.cuda.current_stream(dev).cuda_stream))
    with pytest.raises(_lib.TileGymB200Error) as err:
        _lib.device_status(dev.index)
    elapsed = time.perf_counter() - t0
    assert err.value.rc == -7 and "site 99" in str(err.value)
    assert elapsed < 5.0, f"the wait took {elapsed:.2f} s to give up"
    # the status word was cleared by the read, and ordinary work runs on the same context
    _lib.device_status(dev.index)
    tg.reset_workspaces()
    a8, b8, sa, sb = R.gen_per_tensor_case(256, 512, 1024, seed=2)
    out = tg.fp8_scaled_mm(a8.to(dev), b8.to(dev), sa.to(dev), sb.to(dev))
    assert R.check_tolerance(out, R.ref_fp8_scaled_mm(a8, b8, sa, sb))["ok"]
    _lib.device_status(dev.index)


def test_wait_limit_is_a_runtime_setting_the_kernels_accept(dev):
    """A short but sufficient limit (50 ms against kernels of microseconds) changes nothing in the results."""
    L = _lib.lib()
    prev = L.tg_set_wait_limit_us(50_000)
    try:
        for M in (8, 300, 1024):
            a8, b8, sa, sb = R.gen_per_tensor_case(M, 768, 2048, seed=M)
            out = tg.fp8_scaled_mm(a8.to(dev), b8.to(dev), sa.to(dev), sb.to(dev))
            assert R.check_tolerance(out, R.ref_fp8_scaled_mm(a8, b8, sa, sb))["ok"]
        _lib.device_status(dev.index)
    finally:
        L.tg_set_wait_limit_us(prev)
