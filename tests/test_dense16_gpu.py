"""The unquantised bf16 / f16 path of `matmul` (tcgen05 kind::f16) against the oracle."""
import pytest
import torch

from oracle import torch_ref as R

pytestmark = pytest.mark.gpu

import tilegym_b200 as tg  # noqa: E402
from tilegym_b200 import _lib  # noqa: E402


@pytest.mark.parametrize("M,N,K", [(256, 256, 256), (1024, 2048, 1024), (4096, 4096, 4096), (300, 520, 1048),
                                    (1, 64, 72), (130, 1000, 8), (2048, 6144, 4096)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_dense_matmul_matches_oracle(dev, M, N, K, dtype):
    """Shapes of the reference test (tests/ops/test_matmul.py: 1024 / 4096 cubes) plus ragged ones; fp32
    accumulation, output in the input dtype; tolerance of that test for 16-bit types: 1e-2 / 1e-2."""
    g = torch.Generator().manual_seed(M + N + K)
    a = torch.randn(M, K, generator=g).to(dtype)
    b = torch.randn(N, K, generator=g).to(dtype)
    ref = R.ref_matmul(a, b, trans_b=True)
    out = tg.matmul(a.to(dev), b.to(dev), trans_b=True)
    assert out.dtype == dtype and out.shape == (M, N)
    scale = float(ref.float().abs().max())
    torch.testing.assert_close(out.float().cpu(), ref.float(), rtol=1e-2, atol=1e-2 * scale / 8)
    _lib.device_status(dev.index)


def test_dense_matmul_kn_layout_and_fp32_out(dev):
    g = torch.Generator().manual_seed(7)
    a = torch.randn(512, 768, generator=g).to(torch.bfloat16)
    b = torch.randn(768, 640, generator=g).to(torch.bfloat16)  # [K, N], as torch.matmul takes it
    ref = a.float() @ b.float()
    out = tg.matmul(a.to(dev), b.to(dev), out_dtype=torch.float32)
    assert out.dtype == torch.float32
    torch.testing.assert_close(out.cpu(), ref, rtol=1e-4, atol=1e-3)


def test_dense_matmul_rejects_mixed_dtypes(dev):
    a = torch.zeros(64, 64, dtype=torch.bfloat16, device=dev)
    with pytest.raises(NotImplementedError):
        tg.matmul(a, a.half())
    with pytest.raises(NotImplementedError):
        tg.matmul(a.float(), a.float())
