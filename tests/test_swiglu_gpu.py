"""Fused gate/up GEMM + SwiGLU epilogue against the oracle and against the two-step path."""
import pytest
import torch

from oracle import torch_ref as R

pytestmark = pytest.mark.gpu

import tilegym_b200 as tg  # noqa: E402
from tilegym_b200 import _lib  # noqa: E402
from tilegym_b200.linear import FP8SwiGLUMLP  # noqa: E402


def make(M, I, K, seed, bias=False):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g)
    wg = torch.randn(I, K, generator=g) * 0.05
    wu = torch.randn(I, K, generator=g) * 0.05
    a8, sa = R.ref_quant_per_tensor(x)
    w = tg.interleave_gate_up(wg, wu)
    b8, sb = R.ref_quant_per_tensor(w)
    bi = tg.interleave_gate_up(torch.randn(I, generator=g), torch.randn(I, generator=g)) if bias else None
    return a8, b8, sa, sb, bi


def test_interleave_layout():
    g = torch.arange(64).float().unsqueeze(1).expand(64, 3)
    u = g + 1000
    w = tg.interleave_gate_up(g, u)
    assert w.shape == (128, 3)
    assert torch.equal(w[:32], g[:32]) and torch.equal(w[32:64], u[:32]) and torch.equal(w[64:96], g[32:])


@pytest.mark.parametrize("M,I,K,bias", [(512, 1024, 1024, False), (300, 448, 528, True), (4096, 3584, 1024, False),
                                         (1, 64, 256, True), (70, 192, 2048, False)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_swiglu_epilogue_matches_oracle(dev, M, I, K, bias, dtype):
    a8, b8, sa, sb, bi = make(M, I, K, seed=M + I + K, bias=bias)
    ref = R.ref_fp8_scaled_mm_swiglu(a8, b8, sa, sb, bi, dtype)
    out = tg.fp8_scaled_mm_swiglu(a8.to(dev), b8.to(dev), sa.to(dev), sb.to(dev), bi.to(dev) if bias else None, dtype)
    assert out.shape == (M, I) and out.dtype == dtype
    res = R.check_tolerance(out.float(), ref.float())
    assert res["ok"], res
    _lib.device_status(dev.index)


def test_swiglu_equals_two_step_path_within_rounding(dev):
    """Against matmul -> silu_and_mul on the bf16 intermediate (what the reference MLP does): the fused result
    skips one bf16 rounding, so the two agree to a bf16 ulp or two."""
    a8, b8, sa, sb, _ = make(1024, 2048, 1024, seed=5)
    args = [t.to(dev) for t in (a8, b8, sa, sb)]
    fused = tg.fp8_scaled_mm_swiglu(*args)
    y = tg.fp8_scaled_mm(*args).float().reshape(1024, -1, 2, 32)
    two_step = (torch.nn.functional.silu(y[:, :, 0]) * y[:, :, 1]).reshape(1024, 2048)
    torch.testing.assert_close(fused.float(), two_step, rtol=2e-2, atol=2e-2 * float(two_step.abs().max()) / 16)


def test_swiglu_mlp_module(dev):
    torch.manual_seed(0)
    H, I = 512, 1024
    gate, up, down = (torch.nn.Linear(H, I, bias=False), torch.nn.Linear(H, I, bias=False),
                      torch.nn.Linear(I, H, bias=False))
    mods = [m.to(dev).to(torch.bfloat16) for m in (gate, up, down)]
    mlp = FP8SwiGLUMLP(*mods)
    x = torch.randn(4, 96, H, device=dev, dtype=torch.bfloat16)
    y = mlp(x)
    ref = mods[2](torch.nn.functional.silu(mods[0](x)) * mods[1](x))
    assert y.shape == ref.shape
    err = (y.float() - ref.float()).abs().max() / ref.float().abs().max()
    assert float(err) < 0.08  # e4m3 quantisation of activations and weights, three GEMMs deep


def test_swiglu_argument_errors(dev):
    a8, b8, sa, sb, _ = [t.to(dev) if t is not None else None for t in make(256, 128, 256, seed=1)]
    with pytest.raises(RuntimeError):
        tg.fp8_scaled_mm_swiglu(a8, b8, sa, sb, out_dtype=torch.float32)
    with pytest.raises(AssertionError):
        tg.fp8_scaled_mm_swiglu(a8, b8[:192], sa, sb)  # 2*I must be a multiple of 128
