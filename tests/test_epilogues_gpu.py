"""Parity of the epilogue and operand-format variants around the FP8 GEMM kernels, through the C ABI:
bias and beta * C on the block-scaled GEMM (dense and grouped), gemm_alpha_beta on 16-bit operands (the
reference test's f16 -> f16 and bf16 -> bf16 rows), e5m2 matmul, and bmm.  Tolerances are written at each test."""

import pytest
import torch

from conftest import load_golden16
from oracle import torch_ref as R

pytestmark = pytest.mark.gpu

import tilegym_b200 as tg  # noqa: E402
from tilegym_b200 import _lib  # noqa: E402

KNOBS = ("TILEGYM_B200_SPLITS", "TILEGYM_B200_BS_WIDE", "TILEGYM_B200_BS_SMALLM", "TILEGYM_B200_TMA_STORE")


@pytest.fixture(autouse=True)
def clean_knobs_and_status(dev):
    for k in KNOBS:
        _lib.set_knob(k, None)
    yield
    for k in KNOBS:
        _lib.set_knob(k, None)
    _lib.device_status(dev.index)


# ------------------------------------------------------------ block-scaled GEMM: bias and beta * C
@pytest.mark.parametrize("bias_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("M,N,K", [(128, 3072, 5120), (4096, 3072, 1536), (300, 520, 1040), (64, 256, 2048)])
def test_block_scaled_bias_joins_the_fp32_sum_before_the_rounding(dev, M, N, K, bias_dtype):
    """Every block-scaled kernel (128 x 128 with and without K split, wide tile, small M) adds the
    bias in fp32 before the single rounding to bf16: 2 bf16 ulps / 1e-2 relative against the oracle."""
    g = torch.Generator().manual_seed(M + N + K)
    A = (torch.randn(M, K, generator=g) * 0.5).to(torch.float8_e4m3fn)
    B = (torch.randn(N, K, generator=g) * 0.1).to(torch.float8_e4m3fn)
    As = torch.rand(M, -(-K // 128), generator=g) + 0.1
    Bs = torch.rand(-(-N // 128), -(-K // 128), generator=g) + 0.1
    bias = (torch.randn(N, generator=g) * 3.0).to(bias_dtype)
    ref = R.ref_fp8_block_scaled_mm(A, B, As, Bs, bias, torch.bfloat16)
    out = tg.fp8_block_scaled_mm(A.to(dev), B.to(dev), As.to(dev), Bs.to(dev), bias.to(dev), torch.bfloat16)
    res = R.check_tolerance(out, ref)
    assert res["ok"], res


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("M,N,K,splits", [(256, 512, 1024, None), (128, 384, 2048, "4"), (2500, 3900, 400, "1")])
def test_block_scaled_beta_accumulates_in_place(dev, M, N, K, splits, out_dtype):
    if splits is not None:
        _lib.set_knob("TILEGYM_B200_SPLITS", splits)
    g = torch.Generator().manual_seed(7 + M)
    A = (torch.randn(M, K, generator=g) * 0.5).to(torch.float8_e4m3fn)
    B = (torch.randn(N, K, generator=g) * 0.1).to(torch.float8_e4m3fn)
    As = torch.rand(M, -(-K // 128), generator=g) + 0.1
    Bs = torch.rand(-(-N // 128), -(-K // 128), generator=g) + 0.1
    bias = torch.randn(N, generator=g)
    c0 = torch.randn(M, N, generator=g).to(out_dtype)
    ref = R.ref_fp8_block_scaled_mm(A, B, As, Bs, bias, out_dtype, c0, 0.75)
    c = c0.to(dev)
    out = tg.fp8_block_scaled_mm(A.to(dev), B.to(dev), As.to(dev), Bs.to(dev), bias.to(dev), out=c, beta=0.75)
    assert out.data_ptr() == c.data_ptr()
    if out_dtype == torch.float32:
        torch.testing.assert_close(out.cpu(), ref, rtol=1e-4, atol=1e-4)
    else:
        assert R.check_tolerance(out, ref)["ok"]


def test_grouped_block_scaled_bias_per_group(dev):
    sizes = [200, 0, 333, 128]
    Q, N, K = len(sizes), 384, 512
    g = torch.Generator().manual_seed(5)
    total = sum(sizes)
    a = (torch.randn(total, K, generator=g) * 0.5).to(torch.float8_e4m3fn)
    b = (torch.randn(Q, N, K, generator=g) * 0.1).to(torch.float8_e4m3fn)
    As = torch.rand(total, K // 128, generator=g) + 0.1
    Bs = torch.rand(Q, N // 128, K // 128, generator=g) + 0.1
    bias = torch.randn(Q, N, generator=g) * 2.0
    ind = torch.tensor([0] + list(torch.tensor(sizes).cumsum(0)), dtype=torch.int32)
    out = tg.ragged_block_scaled_bmm(a.to(dev), b.to(dev), As.to(dev), Bs.to(dev), ind.to(dev), max(sizes),
                                     bias=bias.to(dev))
    lo = 0
    for q, sz in enumerate(sizes):
        if sz:
            ref = R.ref_fp8_block_scaled_mm(a[lo:lo + sz], b[q], As[lo:lo + sz], Bs[q], bias[q], torch.bfloat16)
            res = R.check_tolerance(out[lo:lo + sz], ref)
            assert res["ok"], (q, res)
        lo += sz


# ------------------------------------------------------------ gemm_alpha_beta on 16-bit operands
@pytest.mark.parametrize("tag,dt", [("f16", torch.float16), ("bf16", torch.bfloat16)])
def test_gemm_alpha_beta_16bit_against_reference_fixture(dev, tag, dt):
    """Same comparison and tolerance (rtol = atol = 1e-2) as the reference's own test,
    tests/suites/flashinfer/test_flashinfer_gemm_alpha_beta.py:44-75, on its (f16 -> f16), (bf16 -> bf16) rows."""
    a, b, c, ref_out, alpha, beta = load_golden16(f"gemm_alpha_beta_{tag}_256_1.5_2.0.npz", dt)
    cd = c.to(dev)
    out = tg.gemm_alpha_beta(a.to(dev), b.to(dev), cd, False, True, alpha, beta)
    assert out.data_ptr() == cd.data_ptr() and out.dtype == dt
    torch.testing.assert_close(out.float().cpu(), ref_out.float(), rtol=1e-2, atol=1e-2)
    tight = R.ref_gemm_alpha_beta(a, b, c, alpha, beta)  # fp32 accumulate, one rounding: within one ulp of ours
    torch.testing.assert_close(out.float().cpu(), tight.float(), rtol=2.0 ** -7 if dt == torch.bfloat16 else 2.0 ** -10,
                               atol=1e-3)


@pytest.mark.parametrize("dt", [torch.float16, torch.bfloat16])
def test_gemm_alpha_beta_16bit_reference_recipe_4096(dev, dt):
    torch.manual_seed(0)
    m = n = k = 4096
    a = torch.rand(m * k, dtype=torch.float16).to(dt).view(m, k)
    b = torch.rand(k * n, dtype=torch.float16).to(dt).view(n, k)
    c = torch.rand((m, n), dtype=dt)
    ref = R.ref_gemm_alpha_beta(a, b, c, 1.5, 2.0)
    out = tg.gemm_alpha_beta(a.to(dev), b.to(dev), c.to(dev), False, True, 1.5, 2.0)
    torch.testing.assert_close(out.float().cpu(), ref.float(), rtol=1e-2, atol=1e-2)


def test_gemm_alpha_beta_other_transposes(dev):
    torch.manual_seed(1)
    a = torch.rand(384, 256, dtype=torch.float16).to(torch.float8_e4m3fn)  # [K, M] with trans_a
    b = torch.rand(384, 512, dtype=torch.float16).to(torch.float8_e4m3fn)  # [K, N] without trans_b
    c = torch.zeros(256, 512, dtype=torch.bfloat16)
    ref = R.ref_gemm_alpha_beta(a.t(), b.t(), c, 0.5, 0.0)
    out = tg.gemm_alpha_beta(a.to(dev), b.to(dev), c.to(dev), True, False, 0.5, 0.0)
    assert R.check_tolerance(out, ref)["ok"]


# ------------------------------------------------------------ e5m2 operands
@pytest.mark.parametrize("M,N,K", [(512, 768, 1024), (16, 1024, 2048), (128, 640, 512)])
def test_e5m2_matmul_all_kernel_families(dev, M, N, K):
    """e5m2 operands run the same kernels with the other operand-format field of the instruction descriptor
    (CTA pair, small M, single CTA).  Checked in bf16 (2 ulps / 1e-2) and in the input dtype like the reference
    (src/tilegym/ops/cutile/matmul.py:446; its own fp8 tolerance is atol = rtol = 1, tests/ops/test_matmul.py:231-236)."""
    g = torch.Generator().manual_seed(M + K)
    a = (torch.randn(M, K, generator=g) * 0.5).to(torch.float8_e5m2)
    b = (torch.randn(K, N, generator=g) * 0.1).to(torch.float8_e5m2)
    exact = a.float() @ b.float()
    out_bf = tg.matmul(a.to(dev), b.to(dev), out_dtype=torch.bfloat16)
    assert R.check_tolerance(out_bf, exact.to(torch.bfloat16))["ok"]
    out = tg.matmul(a.to(dev), b.to(dev))
    assert out.dtype == torch.float8_e5m2
    ref = R.ref_matmul(a, b)
    # one e5m2 rounding step (2 mantissa bits) of slack for sums that land on a rounding boundary
    torch.testing.assert_close(out.float().cpu(), ref.float(), rtol=0.25, atol=0.05)


def test_e5m2_and_e4m3_cannot_be_mixed(dev):
    a = torch.zeros(64, 128, dtype=torch.float8_e5m2, device=dev)
    b = torch.zeros(128, 64, dtype=torch.float8_e4m3fn, device=dev)
    with pytest.raises(NotImplementedError):
        tg.matmul(a, b)


# ------------------------------------------------------------ bmm
@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("m,n,k", [(128, 256, 511), (1024, 512, 512), (128, 512, 1023)])
def test_bmm_f16_reference_test_shapes(dev, m, n, k, ta, tb):
    """Shapes, operand recipe and tolerance class of tests/ops/test_bmm.py:32-110 (batch 4, rand f16,
    K that is not a multiple of 8 included); compared with the fp32-accumulating oracle at rtol 1e-3."""
    torch.manual_seed(0)
    a = torch.rand((4, k, m) if ta else (4, m, k), dtype=torch.float16)
    b = torch.rand((4, n, k) if tb else (4, k, n), dtype=torch.float16)
    ref = R.ref_bmm(a, b, ta, tb)
    out = tg.bmm(a.to(dev), b.to(dev), ta, tb)
    assert out.shape == (4, m, n) and out.dtype == torch.float16
    torch.testing.assert_close(out.cpu(), ref, rtol=1e-3, atol=1e-3)


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float8_e4m3fn])
def test_bmm_other_dtypes(dev, dt):
    g = torch.Generator().manual_seed(3)
    a = (torch.randn(3, 200, 384, generator=g) * 0.5).to(dt)
    b = (torch.randn(3, 320, 384, generator=g) * 0.1).to(dt)
    out = tg.bmm(a.to(dev), b.to(dev), False, True)
    ref = R.ref_bmm(a, b, False, True)
    assert out.dtype == dt
    if dt == torch.bfloat16:
        assert R.check_tolerance(out.reshape(-1, 320), ref.reshape(-1, 320))["ok"]
    else:
        torch.testing.assert_close(out.float().cpu(), ref.float(), rtol=0.13, atol=0.05)
