"""The CPU oracle against the golden fixtures made from TileGym's own test
references (tests/golden/make_golden.py), plus self-checks of its helpers."""

import glob
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN, load_golden, load_golden16
from oracle import torch_ref as R


def test_e4m3_table_matches_torch_cast():
    tab = torch.from_numpy(R.e4m3_table())
    via_torch = torch.arange(256, dtype=torch.int32).to(torch.uint8).view(torch.float8_e4m3fn).float()
    nan = torch.isnan(tab)
    assert nan.sum() == 2 and bool((torch.isnan(via_torch) == nan).all())
    assert bool((tab[~nan] == via_torch[~nan]).all())
    assert float(tab[~nan].abs().max()) == R.E4M3_MAX


@pytest.mark.parametrize("name", sorted(os.path.basename(p) for p in glob.glob(os.path.join(GOLDEN, "w8a8_block_*.npz"))))
def test_block_scaled_gemm_matches_reference_fixture(name):
    g = load_golden(name)
    out = R.ref_w8a8_block_fp8_matmul(g["A"], g["B"], g["As"], g["Bs"], [128, 128], torch.float32)
    # same dequantised operands, same fp32 matmul: equal up to summation order inside torch.matmul
    torch.testing.assert_close(out, g["C_f32"], rtol=1e-5, atol=1e-5)
    out_bf16 = R.ref_w8a8_block_fp8_matmul(g["A"], g["B"], g["As"], g["Bs"], None, torch.bfloat16)
    res = R.check_tolerance(out_bf16, g["C_bf16"], ulps=1.0)
    assert res["ok"], res


@pytest.mark.parametrize("name", ["act_quant_64x1024.npz", "act_quant_128x384.npz", "act_quant_4x128.npz"])
def test_act_quant_matches_reference_fixture(name):
    g = load_golden(name)
    y, s = R.ref_act_quant(g["x"], 128)
    assert bool((y.view(torch.uint8) == g["y"].view(torch.uint8)).all())
    assert bool((s == g["s"]).all())
    if name == "act_quant_4x128.npz":
        assert float(s[1, 0]) == 1.0  # all-zero block


@pytest.mark.parametrize("name", ["ragged_bmm_q4_m128_256x256.npz", "ragged_bmm_q3_m256_384x512.npz"])
def test_ragged_block_scaled_bmm_matches_reference_fixture(name):
    g = load_golden(name)
    out = R.ref_ragged_block_scaled_bmm(g["a"], g["b"], g["a_scale"], g["b_scale"], g["m_indptr"])
    assert bool((out.view(torch.int16) == g["c"].view(torch.int16)).all())


def test_ragged_block_scaled_bmm_is_the_dense_gemm_per_group():
    a8, b8, As, Bs = R.gen_block_scaled_case(96, 256, 384, seed=5)
    ind = torch.tensor([0, 40, 40, 96], dtype=torch.int32)  # one empty group
    b3 = torch.stack([b8, b8.flip(0), b8])
    bs3 = torch.stack([Bs, Bs.flip(0), Bs])
    out = R.ref_ragged_block_scaled_bmm(a8, b3, As, bs3, ind)
    assert torch.equal(out[:40], R.ref_w8a8_block_fp8_matmul(a8[:40], b8, As[:40], Bs, None, torch.bfloat16))
    assert torch.equal(out[40:], R.ref_w8a8_block_fp8_matmul(a8[40:], b8, As[40:], Bs, None, torch.bfloat16))


GROUP_QUANT = sorted(os.path.basename(p) for p in glob.glob(os.path.join(GOLDEN, "group_quant_*.npz")))


def group_quant_case(name):
    """(group_size, dst_dtype, scale_ue8m0) from a fixture name group_quant_<T>x<H>_g<g>_<dtype>_ue<0|1>.npz."""
    parts = name[:-4].split("_")
    dst = {"e4m3": torch.float8_e4m3fn, "e5m2": torch.float8_e5m2, "int8": torch.int8}[parts[4]]
    return int(parts[3][1:]), dst, parts[5] == "ue1"


@pytest.mark.parametrize("name", GROUP_QUANT)
def test_per_token_group_quant_matches_reference_fixture(name):
    assert len(GROUP_QUANT) == 5
    g = load_golden(name)
    gs, dst, ue = group_quant_case(name)
    q, s = R.ref_per_token_group_quant_8bit(g["x"], gs, 1e-10, dst, ue)
    assert bool((q.view(torch.uint8) == g["q"].view(torch.uint8)).all())
    assert bool((s == g["s"]).all())
    if ue:  # powers of two
        m, _ = torch.frexp(s)
        assert bool((m == 0.5).all())


@pytest.mark.parametrize("name", ["weight_dequant_256x256.npz", "weight_dequant_130x200.npz"])
def test_weight_dequant_matches_reference_fixture(name):
    g = load_golden(name)
    y = R.ref_weight_dequant(g["x"], g["s"], 128, torch.bfloat16)
    assert bool((y.view(torch.int16) == g["y"].view(torch.int16)).all())


@pytest.mark.parametrize("name", ["gemm_alpha_beta_256_1.0_0.0.npz", "gemm_alpha_beta_256_1.5_2.0.npz"])
def test_gemm_alpha_beta_matches_reference_fixture(name):
    g = load_golden(name)
    # the reference test's own (bf16) form reproduces its stored output
    bf = R.ref_gemm_alpha_beta_bf16(g["a"], g["b"], g["c"], g["alpha"], g["beta"])
    torch.testing.assert_close(bf.float(), g["out"].float(), rtol=1e-2, atol=1e-2)
    # the fp32-accumulate form the kernels follow agrees within the reference test's tolerance
    f32 = R.ref_gemm_alpha_beta(g["a"], g["b"], g["c"], g["alpha"], g["beta"])
    torch.testing.assert_close(f32.float(), g["out"].float(), rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("tag,dt", [("f16", torch.float16), ("bf16", torch.bfloat16)])
def test_gemm_alpha_beta_16bit_matches_reference_fixture(tag, dt):
    """The (float16 -> float16) and (bfloat16 -> bfloat16) rows of the reference test, its tolerance."""
    a, b, c, out, alpha, beta = load_golden16(f"gemm_alpha_beta_{tag}_256_1.5_2.0.npz", dt)
    f32 = R.ref_gemm_alpha_beta(a, b, c, alpha, beta)
    assert f32.dtype == dt
    torch.testing.assert_close(f32.float(), out.float(), rtol=1e-2, atol=1e-2)


def test_block_scaled_bias_form_reduces_to_the_reference_form():
    a8, b8, As, Bs = R.gen_block_scaled_case(40, 256, 384, seed=2)
    plain = R.ref_w8a8_block_fp8_matmul(a8, b8, As, Bs, None, torch.float32)
    assert torch.equal(R.ref_fp8_block_scaled_mm(a8, b8, As, Bs, None, torch.float32), plain)
    bias = torch.randn(256)
    c = torch.randn(40, 256)
    full = R.ref_fp8_block_scaled_mm(a8, b8, As, Bs, bias, torch.float32, c, 0.5)
    torch.testing.assert_close(full, plain + bias + 0.5 * c, rtol=1e-6, atol=1e-6)


def test_moe_oracle_matches_the_reference_torch_moe():
    """The MoE oracle against outputs of the reference's own torch code on the dequantised operands of the
    fixture: its first GEMM stage equals tilegym.ops.moe_interface.fused_moe_torch to fp32 summation order, and
    the whole layer agrees with tests/ops/test_moe.py's Test_MOE.reference within that test's fp8 tolerance
    (and much closer: the only difference is the e4m3 rounding of the intermediate, which the reference's
    FP8 path performs and its torch test reference does not)."""
    g = load_golden("moe_16x256x128_e4_k2.npz")
    T, topk = g["ids"].shape
    fc1 = torch.stack([torch.stack([R.ref_w8a8_block_fp8_matmul(g["a8"][t:t + 1], g["w1"][int(g["ids"][t, j])],
                                                                 g["a_s"][t:t + 1], g["w1_s"][int(g["ids"][t, j])],
                                                                 [128, 128], torch.float32)[0] for j in range(topk)])
                       for t in range(T)])
    torch.testing.assert_close(fc1, g["stage1_f32"], rtol=1e-4, atol=1e-4)
    for mode in ("ones", "block"):
        out = R.ref_fused_experts_fp8(g["a8"], g["a_s"], g["w1"], g["w1_s"], g["w2"], g["w2_s"], g["wts"], g["ids"],
                                      torch.float16, mode)
        torch.testing.assert_close(out.float(), g["full_f32"], rtol=5e-1, atol=5e-1)  # the reference test's bound
        assert float((out.float() - g["full_f32"]).abs().max()) <= 0.05 * float(g["full_f32"].abs().max())
    torch.testing.assert_close(g["stage2_f32"].sum(1), g["full_f32"], rtol=1e-4, atol=1e-4)


def test_ref_bmm_follows_torch_bmm():
    torch.manual_seed(1)
    a, b = torch.rand(3, 20, 33, dtype=torch.float16), torch.rand(3, 40, 33, dtype=torch.float16)
    torch.testing.assert_close(R.ref_bmm(a, b, False, True), torch.bmm(a, b.transpose(1, 2)), rtol=1e-3, atol=1e-3)
    at = a.transpose(1, 2).contiguous()
    assert torch.equal(R.ref_bmm(at, b, True, True), R.ref_bmm(a, b, False, True))


def test_per_tensor_forms_agree():
    a8, b8, sa, sb = R.gen_per_tensor_case(64, 96, 256, seed=5)
    x = R.ref_fp8_scaled_mm(a8, b8, sa, sb)
    c = torch.zeros(64, 96, dtype=torch.bfloat16)
    y = R.ref_gemm_alpha_beta(a8, b8, c, alpha=float(sa) * float(sb), beta=0.0)
    assert R.check_tolerance(x, y, ulps=1.0)["ok"]


def test_quant_per_tensor_roundtrip_and_zero():
    x = R.gen_activations(32, 4096, seed=9)
    q, s = R.ref_quant_per_tensor(x)
    assert float(s) == pytest.approx(float(x.abs().max()) / 448.0)
    assert float(q.float().abs().max()) == 448.0
    q0, s0 = R.ref_quant_per_tensor(torch.zeros(4, 16))
    assert float(s0) == 1.0 and float(q0.float().abs().max()) == 0.0


def test_weight_quant_block_inverts_dequant():
    w = R.gen_weights(200, 300, seed=4)
    q, s = R.ref_weight_quant_block(w)
    assert s.shape == (2, 3)
    back = R.ref_weight_dequant(q, s, 128, torch.float32)
    # e4m3 has 3 mantissa bits: relative error <= 2^-4 of the block maximum
    assert float((back - w).abs().max()) <= float(w.abs().max()) * 2.0 ** -4


def test_generators_are_seeded_and_have_outliers():
    a = R.gen_activations(16, 4096, seed=1)
    b = R.gen_activations(16, 4096, seed=1)
    assert bool((a == b).all())
    col_rms = a.pow(2).mean(0).sqrt()
    assert int((col_rms > 8).sum()) == 4  # 0.1 % of 4096 channels scaled x20


def test_tolerance_checker_accepts_one_ulp_and_rejects_more():
    ref = torch.full((4, 4), 3.0)
    ok = ref.clone(); ok[0, 0] += R.ulp_bf16(3.0)
    bad = ref.clone(); bad[0, 0] += 4 * R.ulp_bf16(3.0)
    assert R.check_tolerance(ok, ref)["ok"]
    assert not R.check_tolerance(bad, ref)["ok"]
    assert not R.check_tolerance(torch.full((4, 4), float("nan")), ref)["ok"]
    assert R.ulp_bf16(1.0) == 2.0 ** -7
