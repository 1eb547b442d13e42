"""The quantisers and the block dequantiser against the oracle: bit-exact."""

import pytest
import torch

from conftest import load_golden
from oracle import torch_ref as R

pytestmark = pytest.mark.gpu

import tilegym_b200 as tg  # noqa: E402


def same_bits(a, b):
    return bool((a.cpu().view(torch.uint8) == b.view(torch.uint8)).all())


@pytest.mark.parametrize("name", ["act_quant_64x1024.npz", "act_quant_128x384.npz", "act_quant_4x128.npz"])
def test_act_quant_fixtures(dev, name):
    g = load_golden(name)
    y, s = tg.act_quant(g["x"].to(dev), 128)
    assert y.dtype == torch.float8_e4m3fn and y.shape == g["x"].shape
    assert same_bits(y, g["y"]) and torch.equal(s.cpu(), g["s"])


@pytest.mark.parametrize("shape", [(256, 256), (1024, 4096), (2048, 8192), (3, 5, 384)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_act_quant_reference_test_shapes(dev, shape, dtype):
    torch.manual_seed(42)
    x = torch.randn(*shape, dtype=dtype)
    y, s = tg.act_quant(x.to(dev))
    yr, sr = R.ref_act_quant(x)
    assert s.shape == (*shape[:-1], shape[-1] // 128)
    assert same_bits(y, yr) and torch.equal(s.cpu(), sr)


def test_act_quant_rejects_ragged_last_dim(dev):
    with pytest.raises(AssertionError):
        tg.act_quant(torch.zeros(4, 100, dtype=torch.bfloat16, device=dev))


@pytest.mark.parametrize("name", ["weight_dequant_256x256.npz", "weight_dequant_130x200.npz"])
def test_weight_dequant_fixtures(dev, name):
    g = load_golden(name)
    y = tg.weight_dequant(g["x"].to(dev), g["s"].to(dev), 128, torch.bfloat16)
    assert torch.equal(y.cpu().view(torch.int16), g["y"].view(torch.int16))


@pytest.mark.parametrize("shape", [(512, 1024), (384, 768), (2048, 4096), (130, 200)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_weight_dequant_reference_test_shapes(dev, shape, dtype):
    torch.manual_seed(42)
    x = torch.randn(*shape).to(torch.float8_e4m3fn)
    s = torch.rand(-(-shape[0] // 128), -(-shape[1] // 128)) + 0.1
    y = tg.weight_dequant(x.to(dev), s.to(dev), 128, dtype)
    assert torch.equal(y.cpu(), R.ref_weight_dequant(x, s, 128, dtype))


@pytest.mark.parametrize("shape", [(4096, 4096), (300, 515), (1, 7), (0, 16)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_quant_per_tensor(dev, shape, dtype):
    x = (R.gen_activations(max(shape[0], 1), shape[1], 5)[: shape[0]]).to(dtype)
    q, s = tg.quant_per_tensor(x.to(dev))
    if x.numel() == 0:
        assert q.shape == x.shape
        return
    qr, sr = R.ref_quant_per_tensor(x)
    assert torch.equal(s.cpu(), sr) and same_bits(q, qr)


def test_quant_per_tensor_all_zero(dev):
    q, s = tg.quant_per_tensor(torch.zeros(8, 64, device=dev))
    assert float(s) == 1.0 and float(q.float().abs().max()) == 0.0


@pytest.mark.parametrize("shape", [(256, 256), (300, 520), (129, 130), (4096, 1536)])
def test_weight_quant_block(dev, shape):
    w = R.gen_weights(*shape, seed=6)
    w[:128, :128] = 0  # an all-zero block -> scale 1.0
    q, s = tg.weight_quant_block(w.to(dev))
    qr, sr = R.ref_weight_quant_block(w)
    assert torch.equal(s.cpu(), sr) and same_bits(q, qr)
    assert float(s[0, 0]) == 1.0
    back = tg.weight_dequant(q, s, 128, torch.float32)
    assert float((back.cpu() - w).abs().max()) <= float(w.abs().max()) * 2.0 ** -4
