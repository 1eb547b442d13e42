"""The quantisers and the block dequantiser against the oracle: bit-exact."""

import pytest
import torch

from conftest import load_golden
from oracle import torch_ref as R

pytestmark = pytest.mark.gpu

import tilegym_b200 as tg  # noqa: E402
from tilegym_b200 import _lib  # noqa: E402


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


@pytest.mark.parametrize("shape", [(1, 8), (1, 4096), (16, 4096), (9, 14336), (64, 4096), (31, 8200), (64, 4104)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_quant_per_tensor_decode_sizes(dev, shape, dtype):
    """Up to 262144 16-bit elements the quantiser is one launch (a cluster of 1 .. 8 CTAs holding the tensor in
    registers); the last shape is just past it and takes the two-pass form.  Same bytes and scale as the oracle."""
    x = R.gen_activations(shape[0], shape[1], 7).to(dtype)
    q, s = tg.quant_per_tensor(x.to(dev))
    qr, sr = R.ref_quant_per_tensor(x)
    assert torch.equal(s.cpu(), sr) and same_bits(q, qr)
    z = torch.zeros(shape, dtype=dtype, device=dev)
    z[-1, -1] = -0.0
    q, s = tg.quant_per_tensor(z)
    assert float(s) == 1.0 and float(q.float().abs().max()) == 0.0


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


# ------------------------------------------------------------ per-token group quantiser
from test_oracle import GROUP_QUANT, group_quant_case  # noqa: E402


@pytest.mark.parametrize("name", GROUP_QUANT)
def test_per_token_group_quant_fixtures(dev, name):
    g = load_golden(name)
    gs, dst, ue = group_quant_case(name)
    q, s = tg.per_token_group_quant_8bit(g["x"].to(dev), gs, 1e-10, dst, column_major_scales=ue, scale_ue8m0=ue)
    assert q.dtype == dst and q.shape == g["x"].shape
    assert same_bits(q, g["q"]) and torch.equal(s.cpu(), g["s"])


@pytest.mark.parametrize("num_tokens", [512, 513])
@pytest.mark.parametrize("group_size", [16, 32, 64, 128])
@pytest.mark.parametrize("dst_dtype", [torch.float8_e4m3fn, torch.int8])
@pytest.mark.parametrize("layout", ["row", "col", "col_aligned", "col_ue8m0", "col_aligned_ue8m0"])
def test_per_token_group_quant_reference_test_grid(dev, num_tokens, group_size, dst_dtype, layout):
    """The parameter grid of the reference test (test_per_token_group_quant_8bit.py:72-84), its seed and
    input recipe; results must equal the oracle bit for bit in every scale layout."""
    torch.manual_seed(0)
    x = torch.randn(num_tokens, 2048, dtype=torch.bfloat16)
    col, aligned, ue = layout != "row", "aligned" in layout, "ue8m0" in layout
    qr, sr = R.ref_per_token_group_quant_8bit(x, group_size, 1e-10, dst_dtype, ue)
    q, s = tg.per_token_group_quant_8bit(x.to(dev), group_size, 1e-10, dst_dtype, col, aligned, ue)
    assert s.shape == sr.shape
    if col and not aligned:
        assert s.stride() == (1, num_tokens)  # column-major view, as the reference returns it
    assert same_bits(q, qr) and torch.equal(s.cpu(), sr)


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_per_token_group_quant_other_inputs_and_zero_groups(dev, dtype):
    torch.manual_seed(3)
    x = torch.randn(3, 7, 512, dtype=dtype) * 5
    if dtype == torch.float32:
        x[1, 2, 128:256] = 0  # eps clamp (in f16 eps = 1e-10 underflows and the torch reference divides 0 by 0)
    x[2, 0, 0] = 1e6 if dtype == torch.float32 else 6e4  # a large outlier
    for dst in (torch.float8_e4m3fn, torch.float8_e5m2, torch.int8):
        qr, sr = R.ref_per_token_group_quant_8bit(x, 128, 1e-10, dst)
        q, s = tg.per_token_group_quant_8bit(x.to(dev), 128, 1e-10, dst)
        assert q.shape == x.shape and s.shape == (3, 7, 4)
        assert same_bits(q, qr) and torch.equal(s.cpu(), sr)


@pytest.mark.parametrize("dst", [torch.float8_e4m3fn, torch.float8_e5m2, torch.int8])
def test_quantisers_equal_ieee_division_on_16m_elements(dev, dst):
    """The kernels divide through a shared reciprocal plus a guarded correction; over 16.8 M elements with row
    magnitudes spread over 12 decades the bytes must still equal the oracle's x / s."""
    g = torch.Generator().manual_seed(11)
    x = torch.randn(4096, 4096, generator=g) * torch.logspace(-6, 6, 4096).unsqueeze(1)
    x = x.to(torch.bfloat16)
    qr, sr = R.ref_per_token_group_quant_8bit(x, 64, 1e-10, dst)
    q, s = tg.per_token_group_quant_8bit(x.to(dev), 64, 1e-10, dst)
    assert torch.equal(s.cpu(), sr) and same_bits(q, qr)
    if dst == torch.float8_e4m3fn:
        yr, s2r = R.ref_act_quant(x)
        y, s2 = tg.act_quant(x.to(dev))
        assert torch.equal(s2.cpu(), s2r) and same_bits(y, yr)
        pr, psr = R.ref_quant_per_tensor(x)
        pq, ps = tg.quant_per_tensor(x.to(dev))
        assert torch.equal(ps.cpu(), psr) and same_bits(pq, pr)


@pytest.mark.parametrize("src", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("dst", [torch.float8_e4m3fn, torch.float8_e5m2, torch.int8])
def test_division_free_quotient_equals_ieee_division_for_every_16_bit_case(dev, src, dst):
    """For 16-bit inputs the kernels form x / s as a + (x - a s) r with a = x r, r = RN(1 / s), without a test.
    The library's self-test walks every (group maximum, element) pair of the input type - all finite positive
    maxima, every |x| <= maximum of both signs, zeros and NaN, the plain scale and the power-of-two one - and
    compares bytes with cast(div.rn(x, s)): none may differ, and the scale itself must equal div.rn(amax, qmax)."""
    counts = torch.full((4,), -1, dtype=torch.int64, device=dev)
    rc = _lib.lib().tg_selftest_quant16(_lib.DTYPE_CODES[src], _lib.DTYPE_CODES[dst], counts.data_ptr(), dev.index,
                                        torch.cuda.current_stream(dev).cuda_stream)
    _lib.check_rc(rc)
    bad, seen, bad_scales, skipped = (int(v) for v in counts.cpu())
    assert bad == 0 and bad_scales == 0, (bad, seen, bad_scales, skipped)
    # pairs hold two quotients (+x, -x); bf16 maxima below 4.5e-18 or above 4.5e22 have scales outside the
    # fast path's range (the kernels divide there) and are skipped, f16 has none
    assert seen > 5e8 and skipped < (16000 if src == torch.bfloat16 else 1), (seen, skipped)


def test_per_token_group_quant_f16_zero_group_keeps_fp32_eps(dev):
    """Where eps underflows in x's dtype the kernel keeps the fp32 eps (as the reference kernel does,
    per_token_group_quant_8bit.py:50-52) instead of dividing zero by zero."""
    x = torch.zeros(2, 128, dtype=torch.float16, device=dev)
    x[1] = 1.0
    q, s = tg.per_token_group_quant_8bit(x, 128)
    assert bool((q[0].float() == 0).all()) and float(s[0, 0]) == float(torch.tensor(1e-10) / 448.0)
    assert bool((q[1].float() == 448).all())


def test_per_token_group_quant_rejects_bad_arguments(dev):
    x = torch.randn(8, 256, dtype=torch.bfloat16, device=dev)
    with pytest.raises(AssertionError):
        tg.per_token_group_quant_8bit(x, 48)
    with pytest.raises(AssertionError):
        tg.per_token_group_quant_8bit(x, 64, scale_ue8m0=True)  # needs column-major scales
    with pytest.raises(RuntimeError):
        tg.per_token_group_quant_8bit(x, 4)  # divides 256 but is not a supported group size
    q, s = tg.per_token_group_quant_8bit(x, 8)  # the smallest supported group
    qr, sr = R.ref_per_token_group_quant_8bit(x.cpu(), 8)
    assert same_bits(q, qr) and torch.equal(s.cpu(), sr)
