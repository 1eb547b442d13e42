"""Seeded random shapes through every GEMM entry point, against the oracle."""
import random

import pytest
import torch

from oracle import torch_ref as R

pytestmark = pytest.mark.gpu

import tilegym_b200 as tg  # noqa: E402
from tilegym_b200 import _lib  # noqa: E402


def _shapes(seed, n, max_m, max_n, max_k):
    rng = random.Random(seed)
    out = []
    for _ in range(n):
        m = rng.choice([1, 2, 7, 16, 17, 63, 64, 65, 128, 129, 255, 256, 257]) if rng.random() < 0.5 else rng.randint(1, max_m)
        out.append((m, rng.randint(1, max_n), 16 * rng.randint(1, max_k // 16)))
    return out


@pytest.mark.parametrize("M,N,K", _shapes(1, 36, 900, 1400, 2304))
def test_per_tensor_random_shapes(dev, M, N, K):
    g = torch.Generator().manual_seed(M * 7919 + N * 104729 + K)
    a = (torch.randn(M, K, generator=g) * 2).to(torch.float8_e4m3fn)
    b = (torch.randn(N, K, generator=g) * 0.5).to(torch.float8_e4m3fn)
    sa, sb = torch.rand(1, generator=g) + 0.5, torch.rand(1, generator=g) * 0.01 + 0.001
    bias = torch.randn(N, generator=g) if (M + N) % 3 == 0 else None
    dtype = [torch.bfloat16, torch.float16, torch.float32][(M + K) % 3]
    ref = R.ref_fp8_scaled_mm(a, b, sa, sb, bias, dtype)
    out = tg.fp8_scaled_mm(a.to(dev), b.to(dev), sa.to(dev), sb.to(dev), bias.to(dev) if bias is not None else None,
                           dtype)
    if dtype == torch.float32:
        torch.testing.assert_close(out.cpu(), ref, rtol=2e-4, atol=2e-4 * float(ref.abs().max()))
    else:
        res = R.check_tolerance(out.float(), ref.float())
        assert res["ok"], (M, N, K, res)


@pytest.mark.parametrize("M,N,K", _shapes(2, 30, 700, 1200, 2304))
def test_block_scaled_random_shapes(dev, M, N, K):
    g = torch.Generator().manual_seed(M * 31 + N * 17 + K)
    a = (torch.randn(M, K, generator=g) * 0.3).to(torch.float8_e4m3fn)
    b = (torch.randn(N, K, generator=g) * 0.3).to(torch.float8_e4m3fn)
    As = torch.rand(M, -(-K // 128), generator=g) + 0.1
    Bs = torch.rand(-(-N // 128), -(-K // 128), generator=g) + 0.1
    dtype = [torch.bfloat16, torch.float32, torch.float16][(N + K) % 3]
    ref = R.ref_w8a8_block_fp8_matmul(a, b, As, Bs, [128, 128], dtype)
    out = tg.w8a8_block_fp8_matmul(a.to(dev), b.to(dev), As.to(dev), Bs.to(dev), [128, 128], dtype)
    if dtype == torch.float32:
        torch.testing.assert_close(out.cpu(), ref, rtol=2e-4, atol=2e-4 * float(ref.abs().max()))
    else:
        res = R.check_tolerance(out.float(), ref.float())
        assert res["ok"], (M, N, K, res)


@pytest.mark.parametrize("seed", range(8))
def test_grouped_random_routing(dev, seed):
    rng = random.Random(100 + seed)
    G = rng.randint(1, 40)
    sizes = [rng.choice([0, 1, 5, 127, 128, 129, 300]) if rng.random() < 0.6 else rng.randint(0, 400) for _ in range(G)]
    if sum(sizes) == 0:
        sizes[0] = 3
    N, K = rng.randint(1, 700), 16 * rng.randint(1, 64)
    g = torch.Generator().manual_seed(seed)
    total, kb, nb = sum(sizes), -(-K // 128), -(-N // 128)
    a = torch.randn(total, K, generator=g).to(torch.float8_e4m3fn)
    b = (torch.randn(G, N, K, generator=g) * 0.5).to(torch.float8_e4m3fn)
    As = torch.rand(total, kb, generator=g) * 0.02 + 0.001
    Bs = torch.rand(G, nb, kb, generator=g) * 0.01 + 0.001
    ind = torch.tensor([0] + [int(v) for v in torch.tensor(sizes).cumsum(0)], dtype=torch.int32)
    ref = R.ref_ragged_block_scaled_bmm(a, b, As, Bs, ind)
    out = tg.ragged_block_scaled_bmm(a.to(dev), b.to(dev), As.to(dev), Bs.to(dev), ind.to(dev), max(sizes))
    res = R.check_tolerance(out.float(), ref.float())
    assert res["ok"], (sizes, N, K, res)
    _lib.device_status(dev.index)
