"""Parity of the CUDA FP8 GEMM paths (through the C ABI) with the CPU oracle.

Tolerance (stated by the task): max relative error <= 1e-2 and max absolute
error <= 2 bf16 ulps of the reference output's magnitude; `check_tolerance`
implements it (relative error is taken over elements above 2^-10 of the
output's magnitude, the rest are held to 2 ulps of that floor).
"""

import os

import pytest
import torch

from conftest import load_golden
from oracle import torch_ref as R

pytestmark = pytest.mark.gpu

import tilegym_b200 as tg  # noqa: E402
from tilegym_b200 import _lib  # noqa: E402

KNOBS = ("TILEGYM_B200_BN", "TILEGYM_B200_SPLITS", "TILEGYM_B200_FORCE_PATH", "TILEGYM_B200_SMALLM_WS",
         "TILEGYM_B200_2CTA", "TILEGYM_B200_GROUP_M", "TILEGYM_B200_BS_WIDE", "TILEGYM_B200_TILE_ROWS", "TILEGYM_B200_TAIL_DIV", "TILEGYM_B200_PDL", "TILEGYM_B200_STATIC_WEIGHTS", "TILEGYM_B200_TMA_STORE", "TILEGYM_B200_BS_SMALLM")


@pytest.fixture(autouse=True)
def clean_env_and_status(dev):
    for k in KNOBS:
        _lib.set_knob(k, None)
    yield
    for k in KNOBS:
        _lib.set_knob(k, None)
    _lib.device_status(dev.index)  # raises if any bounded device-side wait expired


def run_pt(dev, M, N, K, seed, bias=False, out_dtype=torch.bfloat16, outliers=True):
    a8, b8, sa, sb = R.gen_per_tensor_case(M, N, K, seed, outliers)
    bvec = torch.randn(N, generator=torch.Generator().manual_seed(seed + 7)) if bias else None
    ref = R.ref_fp8_scaled_mm(a8, b8, sa, sb, bvec, out_dtype)
    out = tg.fp8_scaled_mm(a8.to(dev), b8.to(dev), sa.to(dev), sb.to(dev), bvec.to(dev) if bias else None, out_dtype)
    assert out.dtype == out_dtype and out.shape == (M, N)
    res = R.check_tolerance(out, ref)
    assert res["ok"], res
    return out


# ------------------------------------------------------------ per-tensor path
def test_config1_1024_cube(dev):
    """BASELINE config 1: M=N=K=1024, N(0,1) operands, per-tensor scales."""
    a8, sa = R.ref_quant_per_tensor(R.gen_activations(1024, 1024, 100, outliers=False))
    b8, sb = R.ref_quant_per_tensor(R.gen_weights(1024, 1024, 101, std=1.0))
    ref = R.ref_fp8_scaled_mm(a8, b8, sa, sb)
    out = tg.fp8_scaled_mm(a8.to(dev), b8.to(dev), sa.to(dev), sb.to(dev))
    assert R.check_tolerance(out, ref)["ok"]


@pytest.mark.parametrize("N,K", [(6144, 4096), (4096, 4096), (28672, 4096), (4096, 14336)])
def test_llama8b_prefill_shapes(dev, N, K):
    """BASELINE config 2 at full size: M=4096, outlier channels, N(0,0.02) weights."""
    run_pt(dev, 4096, N, K, seed=2000 + N + K)


@pytest.mark.parametrize("N", [7168, 28672])
def test_llama70b_gate_up_shard_shapes(dev, N):
    """BASELINE config 5, the GEMM one rank runs when the 57344 weight rows are sharded 8 or 2 ways
    (M = 8192, K = 8192): operands drawn and quantised on the GPU with the configuration's distributions,
    64 sampled rows of the result (all N columns) against the CPU oracle on the same bits."""
    M, K = 8192, 8192
    g = torch.Generator(device=dev).manual_seed(5000 + N)
    x = torch.randn(M, K, generator=g, device=dev, dtype=torch.bfloat16)
    cols = torch.randperm(K, generator=g, device=dev)[: max(1, round(0.001 * K))]
    x[:, cols] *= 20.0
    a8, sa = tg.quant_per_tensor(x)
    del x
    w = torch.randn(N, K, generator=g, device=dev, dtype=torch.bfloat16) * 0.02
    b8, sb = tg.quant_per_tensor(w)
    del w
    out = tg.fp8_scaled_mm(a8, b8, sa, sb)
    rows = torch.randperm(M, generator=torch.Generator().manual_seed(N))[:64].sort().values
    ref = R.ref_fp8_scaled_mm(a8[rows.to(dev)].cpu(), b8.cpu(), sa.cpu(), sb.cpu())
    res = R.check_tolerance(out[rows.to(dev)], ref)
    assert res["ok"], res


@pytest.mark.parametrize("M", [1, 8, 16, 64])
@pytest.mark.parametrize("N,K", [(6144, 4096), (4096, 4096), (28672, 4096), (4096, 14336)])
def test_llama8b_decode_shapes(dev, M, N, K):
    """BASELINE config 3 at full size (swap-AB split-K path)."""
    run_pt(dev, M, N, K, seed=3000 + M + N + K)


@pytest.mark.parametrize("bn", ["256", "128", "64"])
@pytest.mark.parametrize("M,N,K", [(128, 256, 128), (300, 520, 1040), (1, 16, 16), (129, 257 * 8, 144)])
def test_tile_widths_and_tails(dev, bn, M, N, K):
    _lib.set_knob("TILEGYM_B200_BN", bn)
    _lib.set_knob("TILEGYM_B200_FORCE_PATH", "gemm")
    run_pt(dev, M, N, K, seed=11, bias=True)


@pytest.mark.parametrize("M", [1, 2, 7, 16, 17, 31, 32, 33, 63, 64, 65, 127, 128, 129])
def test_m_sweep_across_both_paths(dev, M):
    run_pt(dev, M, 384, 2048, seed=40 + M, bias=(M % 2 == 0))


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("M", [5, 200])
def test_output_dtypes_and_unaligned_n(dev, out_dtype, M):
    # N = 100 is not a multiple of 8: rows of C are not 16-byte aligned, scalar stores
    run_pt(dev, M, 100, 512, seed=77, bias=True, out_dtype=out_dtype)


@pytest.mark.parametrize("splits", ["1", "2", "5"])
@pytest.mark.parametrize("M", [16, 256])
def test_split_k_matches_unsplit(dev, splits, M):
    _lib.set_knob("TILEGYM_B200_SPLITS", splits)
    run_pt(dev, M, 512, 4096, seed=5)


@pytest.mark.parametrize("M", [1, 16, 40, 64])
@pytest.mark.parametrize("ws", ["0", "1"])
def test_small_m_cluster_and_workspace_reductions_agree(dev, M, ws):
    """The K splits are reduced either through distributed shared memory (cluster, default) or through
    the global workspace; both add the partial sums in split order, so the bits are identical."""
    a8, b8, sa, sb = (t.to(dev) for t in R.gen_per_tensor_case(M, 1024, 8192, 60 + M))
    _lib.set_knob("TILEGYM_B200_SPLITS", "4")  # same split count on both paths
    _lib.set_knob("TILEGYM_B200_SMALLM_WS", ws)
    out = tg.fp8_scaled_mm(a8, b8, sa, sb)
    _lib.set_knob("TILEGYM_B200_SMALLM_WS", "1" if ws == "0" else "0")
    other = tg.fp8_scaled_mm(a8, b8, sa, sb)
    assert R.check_tolerance(out, R.ref_fp8_scaled_mm(a8.cpu(), b8.cpu(), sa.cpu(), sb.cpu()))["ok"]
    assert torch.equal(out, other)


@pytest.mark.parametrize("group_m", ["1", "3", "64"])
def test_cta_pair_kernel_raster_groups(dev, group_m):
    _lib.set_knob("TILEGYM_B200_GROUP_M", group_m)
    run_pt(dev, 1280, 1536, 512, seed=12, bias=True)


@pytest.mark.parametrize("tail_div", ["1", "2", "4"])
@pytest.mark.parametrize("M,N,K", [(512, 768, 1024), (1000, 1100, 400), (4096, 6144, 512)])
def test_cta_pair_kernel_tail_slices(dev, tail_div, M, N, K):
    """The tiles of the last wave are cut into 1, 2 or 4 column slices; the result does not change."""
    _lib.set_knob("TILEGYM_B200_TAIL_DIV", tail_div)
    out = run_pt(dev, M, N, K, seed=14, bias=True)
    _lib.set_knob("TILEGYM_B200_TAIL_DIV", "1")
    a8, b8, sa, sb = (t.to(dev) for t in R.gen_per_tensor_case(M, N, K, 14))
    bvec = torch.randn(N, generator=torch.Generator().manual_seed(21)).to(dev)
    assert torch.equal(out, tg.fp8_scaled_mm(a8, b8, sa, sb, bvec))


def test_cta_pair_and_single_cta_kernels_agree(dev):
    a8, b8, sa, sb = (t.to(dev) for t in R.gen_per_tensor_case(1024, 768, 2048, 13))
    pair = tg.fp8_scaled_mm(a8, b8, sa, sb)
    _lib.set_knob("TILEGYM_B200_2CTA", "0")
    single = tg.fp8_scaled_mm(a8, b8, sa, sb)
    assert torch.equal(pair, single)  # same fp32 accumulation order inside the tensor core, same epilogue


def test_static_weights_mode_back_to_back(dev):
    """With the static-weights promise, decode GEMMs launched back to back (programmatic dependent launch:
    weights stream in before the previous kernel has finished) still read the activations the previous
    kernel wrote: a chain y1 = x W1^T, y2 = quant(y1) W2^T equals the chain without the promise."""
    g = torch.Generator().manual_seed(3)
    w1 = (torch.randn(4096, 4096, generator=g) * 0.02).to(dev)
    w2 = (torch.randn(4096, 4096, generator=g) * 0.02).to(dev)
    q1, s1 = tg.quant_per_tensor(w1)
    q2, s2 = tg.quant_per_tensor(w2)
    x, sx = tg.quant_per_tensor(torch.randn(16, 4096, generator=g).to(dev))

    def chain():
        outs = []
        for _ in range(4):
            y1 = tg.fp8_scaled_mm(x, q1, sx, s1)
            yq, sy = tg.quant_per_tensor(y1)
            outs.append(tg.fp8_scaled_mm(yq, q2, sy, s2))
            outs.append(tg.fp8_scaled_mm(x, q2, sx, s2))  # two GEMMs directly behind each other
        return torch.stack(outs)

    base = chain()
    prev = tg.set_static_weights(True)
    try:
        fast = chain()
    finally:
        tg.set_static_weights(prev)
    assert torch.equal(base, fast)


def test_split_k_is_bit_stable(dev):
    """The split-K reduction adds partial sums in split order, so repeated
    runs give identical bits (the reference checks determinism over repeated
    runs the same way, tests/common.py:374-504)."""
    a8, b8, sa, sb = R.gen_per_tensor_case(16, 4096, 4096, 8)
    a, b, sa, sb = a8.to(dev), b8.to(dev), sa.to(dev), sb.to(dev)
    first = tg.fp8_scaled_mm(a, b, sa, sb).clone()
    for _ in range(20):
        again = tg.fp8_scaled_mm(a, b, sa, sb)
        assert torch.equal(first, again)


def test_workspace_counters_are_left_zero(dev):
    from tilegym_b200 import ops

    run_pt(dev, 16, 4096, 4096, seed=8)
    ws = ops._workspace(dev)
    assert int(ws[: 64 << 10].view(torch.int32).abs().max()) == 0


def test_leading_dims_are_flattened(dev):
    a8, b8, sa, sb = R.gen_per_tensor_case(6 * 50, 256, 512, 21)
    ref = R.ref_fp8_scaled_mm(a8, b8, sa, sb).view(6, 50, 256)
    out = tg.fp8_scaled_mm(a8.view(6, 50, 512).to(dev), b8.to(dev), sa.to(dev), sb.to(dev))
    assert out.shape == (6, 50, 256) and R.check_tolerance(out, ref)["ok"]


def test_empty_inputs(dev):
    b8 = torch.zeros(256, 128, dtype=torch.float8_e4m3fn, device=dev)
    out = tg.fp8_scaled_mm(torch.zeros(0, 128, dtype=torch.float8_e4m3fn, device=dev), b8)
    assert out.shape == (0, 256)


def test_linearity_in_the_scales_at_full_size(dev):
    """Size-independent property: doubling scale_a doubles every output
    exactly (a power-of-two factor commutes with all roundings)."""
    M, N, K = 4096, 4096, 4096
    a = torch.randn(M, K, device=dev).to(torch.float8_e4m3fn)
    b = (torch.randn(N, K, device=dev) * 0.02).to(torch.float8_e4m3fn)
    s1 = torch.tensor([0.031], device=dev)
    c1 = tg.fp8_scaled_mm(a, b, s1, s1)
    c2 = tg.fp8_scaled_mm(a, b, s1 * 2, s1)
    assert torch.equal(c1.float() * 2, c2.float())


# -------------------------------------------------------- gemm_alpha_beta API
@pytest.mark.parametrize("name", ["gemm_alpha_beta_256_1.0_0.0.npz", "gemm_alpha_beta_256_1.5_2.0.npz"])
def test_gemm_alpha_beta_against_reference_fixture(dev, name):
    """Same comparison and tolerance as the reference's own test
    (tests/suites/flashinfer/test_flashinfer_gemm_alpha_beta.py:68-75)."""
    g = load_golden(name)
    c = g["c"].to(dev)
    out = tg.gemm_alpha_beta(g["a"].to(dev), g["b"].to(dev), c, False, True, g["alpha"], g["beta"])
    assert out.data_ptr() == c.data_ptr()  # in place
    torch.testing.assert_close(out.float().cpu(), g["out"].float(), rtol=1e-2, atol=1e-2)
    tight = R.ref_gemm_alpha_beta(g["a"], g["b"], g["c"], g["alpha"], g["beta"])
    assert R.check_tolerance(out, tight)["ok"]


def test_gemm_alpha_beta_reference_recipe_4096(dev):
    """The reference test's recipe at one of its own sizes: rand() operands, seed 0."""
    torch.manual_seed(0)
    m = n = k = 4096
    a = torch.rand(m * k, dtype=torch.float16).to(torch.float8_e4m3fn).view(m, k)
    b = torch.rand(k * n, dtype=torch.float16).to(torch.float8_e4m3fn).view(n, k)
    c = torch.rand((m, n), dtype=torch.bfloat16)
    ref = R.ref_gemm_alpha_beta(a, b, c, 1.5, 2.0)
    out = tg.gemm_alpha_beta(a.to(dev), b.to(dev), c.to(dev), False, True, 1.5, 2.0)
    assert R.check_tolerance(out, ref)["ok"]


def test_gemm_alpha_beta_beta_zero_ignores_c_contents(dev):
    g = load_golden("gemm_alpha_beta_256_1.0_0.0.npz")
    c = torch.full((256, 256), float("nan"), dtype=torch.bfloat16, device=dev)
    out = tg.gemm_alpha_beta(g["a"].to(dev), g["b"].to(dev), c, alpha=1.0, beta=0.0)
    assert bool(torch.isfinite(out).all())


def test_matmul_keeps_input_dtype(dev):
    a = (torch.randn(64, 256) * 0.3).to(torch.float8_e4m3fn)
    b = (torch.randn(256, 128) * 0.3).to(torch.float8_e4m3fn)
    out = tg.matmul(a.to(dev), b.to(dev))
    assert out.dtype == torch.float8_e4m3fn and out.shape == (64, 128)
    ref = R.ref_matmul(a, b)
    # the reference's own tolerance for fp8 outputs is atol = rtol = 1 (tests/ops/test_matmul.py:231-236)
    torch.testing.assert_close(out.float().cpu(), ref.float(), rtol=0.13, atol=0.5)
    out2 = tg.matmul(a.to(dev), b.t().contiguous().to(dev), trans_b=True, out_dtype=torch.bfloat16)
    assert R.check_tolerance(out2, (a.float() @ b.float()).to(torch.bfloat16))["ok"]


# ---------------------------------------------------------- block-scaled path
@pytest.mark.parametrize(
    "name", ["w8a8_block_128x128x128.npz", "w8a8_block_256x256x256.npz", "w8a8_block_7x200x320.npz", "w8a8_block_1x128x256.npz"]
)
def test_block_scaled_against_reference_fixtures(dev, name):
    g = load_golden(name)
    args = [g[k].to(dev) for k in ("A", "B", "As", "Bs")]
    out = tg.w8a8_block_fp8_matmul(*args, [128, 128])  # default output dtype: float32, as in the reference
    assert out.dtype == torch.float32
    # the reference test's tolerance (tests/suites/unsloth/test_fp8.py:224-231) ...
    torch.testing.assert_close(out.cpu(), g["C_f32"], rtol=5e-2, atol=5e-2)
    # ... and fp32-accumulation-order tightness
    torch.testing.assert_close(out.cpu(), g["C_f32"], rtol=1e-4, atol=1e-4)
    out_bf = tg.w8a8_block_fp8_matmul(*args, None, torch.bfloat16)
    assert R.check_tolerance(out_bf, g["C_bf16"])["ok"]


@pytest.mark.parametrize("M", [128, 4096])
@pytest.mark.parametrize("N,K", [(24576, 1536), (5120, 12288), (3072, 5120)])
def test_deepseek_block_scaled_shapes(dev, M, N, K):
    """BASELINE config 4 at full size."""
    a8, b8, As, Bs = R.gen_block_scaled_case(M, N, K, seed=4000 + M + N)
    ref = R.ref_w8a8_block_fp8_matmul(a8, b8, As, Bs, [128, 128], torch.bfloat16)
    out = tg.w8a8_block_fp8_matmul(a8.to(dev), b8.to(dev), As.to(dev), Bs.to(dev), [128, 128], torch.bfloat16)
    res = R.check_tolerance(out, ref)
    assert res["ok"], res


@pytest.mark.parametrize("shape", [(512, 1024, 512), (1024, 2048, 1024)])
def test_block_scaled_reference_test_shapes(dev, shape):
    """The larger shapes of the reference test, its recipe and seed (test_fp8.py:193-222)."""
    M, N, K = shape
    torch.manual_seed(42)
    A = (torch.randn(M, K) * 0.1).to(torch.float8_e4m3fn)
    B = (torch.randn(N, K) * 0.1).to(torch.float8_e4m3fn)
    As = torch.rand(M, K // 128) + 0.1
    Bs = torch.rand(N // 128, K // 128) + 0.1
    ref = R.ref_w8a8_block_fp8_matmul(A, B, As, Bs, [128, 128])
    out = tg.w8a8_block_fp8_matmul(A.to(dev), B.to(dev), As.to(dev), Bs.to(dev), [128, 128])
    torch.testing.assert_close(out.cpu(), ref, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("M,N,K,dtype", [(2500, 3900, 400, torch.float32), (4096, 2304, 1152, torch.bfloat16),
                                         (1300, 7200, 2176, torch.float16)])
def test_block_scaled_wide_tile_kernel_tails_and_agreement(dev, M, N, K, dtype):
    """Problems whose 128 x 256 tiles fill the GPU take the wide-tile kernel: ragged M / N / K against the
    oracle, and bit-for-bit against the 128 x 128 kernel (same k-block order, same fused multiply-adds)."""
    g = torch.Generator().manual_seed(M + N + K)
    A = (torch.randn(M, K, generator=g) * 0.1).to(torch.float8_e4m3fn)
    B = (torch.randn(N, K, generator=g) * 0.1).to(torch.float8_e4m3fn)
    As = torch.rand(M, -(-K // 128), generator=g) + 0.1
    Bs = torch.rand(-(-N // 128), -(-K // 128), generator=g) + 0.1
    ref = R.ref_w8a8_block_fp8_matmul(A, B, As, Bs, [128, 128], dtype)
    args = [t.to(dev) for t in (A, B, As, Bs)]
    _lib.set_knob("TILEGYM_B200_SPLITS", "1")
    _lib.set_knob("TILEGYM_B200_BS_WIDE", "1")
    wide = tg.w8a8_block_fp8_matmul(*args, [128, 128], dtype)
    if dtype == torch.float32:
        torch.testing.assert_close(wide.cpu(), ref, rtol=1e-4, atol=1e-4)
    else:
        assert R.check_tolerance(wide, ref)["ok"]
    _lib.set_knob("TILEGYM_B200_BS_WIDE", "0")
    narrow = tg.w8a8_block_fp8_matmul(*args, [128, 128], dtype)
    assert torch.equal(wide, narrow)


@pytest.mark.parametrize("splits", [None, "1", "2", "3", "8"])
@pytest.mark.parametrize("M", [1, 7, 32, 33, 64, 100, 128])
def test_block_scaled_small_m_kernel_against_oracle_and_tile_kernel(dev, M, splits):
    """M <= 128 takes the swap-AB kernel (weights on the MMA M axis, K splits reduced inside a cluster): ragged
    N and K, every split count, against the oracle; without a K split also bit for bit against the 128 x 128
    tile kernel (same k-block order, same fused multiply-adds)."""
    N, K = 520, 2064  # 5 weight tiles (the last one 8 rows), 17 k-blocks (the last one 16 deep)
    g = torch.Generator().manual_seed(M)
    A = (torch.randn(M, K, generator=g) * 0.5).to(torch.float8_e4m3fn)
    B = (torch.randn(N, K, generator=g) * 0.1).to(torch.float8_e4m3fn)
    As = torch.rand(M, -(-K // 128), generator=g) + 0.1
    Bs = torch.rand(-(-N // 128), -(-K // 128), generator=g) + 0.1
    ref = R.ref_w8a8_block_fp8_matmul(A, B, As, Bs, [128, 128], torch.bfloat16)
    args = [t.to(dev) for t in (A, B, As, Bs)]
    if splits is not None:
        _lib.set_knob("TILEGYM_B200_SPLITS", splits)
    out = tg.w8a8_block_fp8_matmul(*args, [128, 128], torch.bfloat16)
    res = R.check_tolerance(out, ref)
    assert res["ok"], res
    if splits == "1":
        _lib.set_knob("TILEGYM_B200_BS_SMALLM", "0")
        tile = tg.w8a8_block_fp8_matmul(*args, [128, 128], torch.bfloat16)
        assert torch.equal(out, tile)


@pytest.mark.parametrize("out_dtype,N", [(torch.float32, 384), (torch.float16, 384), (torch.bfloat16, 100), (torch.float32, 130)])
@pytest.mark.parametrize("M", [5, 128])
def test_block_scaled_small_m_output_dtypes_and_unaligned_n(dev, M, out_dtype, N):
    K = 1024
    g = torch.Generator().manual_seed(M + N)
    A = (torch.randn(M, K, generator=g) * 0.5).to(torch.float8_e4m3fn)
    B = (torch.randn(N, K, generator=g) * 0.1).to(torch.float8_e4m3fn)
    As = torch.rand(M, K // 128, generator=g) + 0.1
    Bs = torch.rand(-(-N // 128), K // 128, generator=g) + 0.1
    ref = R.ref_w8a8_block_fp8_matmul(A, B, As, Bs, [128, 128], out_dtype)
    for splits in ("1", "4"):
        _lib.set_knob("TILEGYM_B200_SPLITS", splits)
        out = tg.w8a8_block_fp8_matmul(A.to(dev), B.to(dev), As.to(dev), Bs.to(dev), [128, 128], out_dtype)
        if out_dtype == torch.float32:
            torch.testing.assert_close(out.cpu(), ref, rtol=1e-4, atol=1e-4)
        else:
            assert R.check_tolerance(out, ref)["ok"]


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("M", [1, 16, 33, 64])
def test_block_scaled_small_m_with_many_weight_tiles(dev, M, out_dtype):
    """M <= 64, a short K and at least as many weight tiles as SMs (DeepSeek's N = 24576, K = 1536 in small): one
    short CTA per (row tile, weight tile), two per SM.  Against the oracle, with bias and a ragged N, and bit for bit
    against the 128 x 128 tile kernel."""
    N, K = 150 * 128 + 40, 640
    g = torch.Generator().manual_seed(M + 3)
    A = (torch.randn(M, K, generator=g) * 0.5).to(torch.float8_e4m3fn)
    B = (torch.randn(N, K, generator=g) * 0.1).to(torch.float8_e4m3fn)
    As = torch.rand(M, K // 128, generator=g) + 0.1
    Bs = torch.rand(-(-N // 128), K // 128, generator=g) + 0.1
    bias = torch.randn(N, generator=g).to(torch.bfloat16)
    ref = R.ref_fp8_block_scaled_mm(A, B, As, Bs, bias=bias, out_dtype=out_dtype)
    args = [t.to(dev) for t in (A, B, As, Bs)]
    out = tg.fp8_block_scaled_mm(*args, bias=bias.to(dev), out_dtype=out_dtype)
    if out_dtype == torch.float32:
        torch.testing.assert_close(out.cpu(), ref, rtol=1e-4, atol=1e-4 * float(ref.abs().max()))
    else:
        assert R.check_tolerance(out, ref)["ok"]
    _lib.set_knob("TILEGYM_B200_BS_SMALLM", "0")
    try:
        tile = tg.fp8_block_scaled_mm(*args, bias=bias.to(dev), out_dtype=out_dtype)
    finally:
        _lib.set_knob("TILEGYM_B200_BS_SMALLM", None)
    assert torch.equal(out, tile)
    _lib.device_status(dev.index)


def test_block_scaled_small_m_is_bit_stable_and_back_to_back(dev):
    a8, b8, As, Bs = (t.to(dev) for t in R.gen_block_scaled_case(128, 3072, 5120, seed=12))
    first = tg.w8a8_block_fp8_matmul(a8, b8, As, Bs, [128, 128], torch.bfloat16).clone()
    for _ in range(10):
        assert torch.equal(first, tg.w8a8_block_fp8_matmul(a8, b8, As, Bs, [128, 128], torch.bfloat16))


def test_block_scaled_split_k_and_leading_dims(dev):
    _lib.set_knob("TILEGYM_B200_SPLITS", "3")
    a8, b8, As, Bs = R.gen_block_scaled_case(2 * 70, 256, 2048, seed=9)
    ref = R.ref_w8a8_block_fp8_matmul(a8, b8, As, Bs, None, torch.bfloat16).view(2, 70, 256)
    out = tg.w8a8_block_fp8_matmul(a8.view(2, 70, 2048).to(dev), b8.to(dev), As.view(2, 70, 16).to(dev), Bs.to(dev),
                                   None, torch.bfloat16)
    assert out.shape == (2, 70, 256) and R.check_tolerance(out, ref)["ok"]


def test_block_scaled_forced_split_count_is_clamped_to_the_workspace(dev):
    """A split count whose partial tiles would not fit the workspace (here 192 tiles x 12 splits x 64 KiB) is
    reduced by the library instead of being taken literally."""
    _lib.set_knob("TILEGYM_B200_SPLITS", "12")
    _lib.set_knob("TILEGYM_B200_BS_WIDE", "0")
    a8, b8, As, Bs = R.gen_block_scaled_case(128, 24576, 1536, seed=77)
    ref = R.ref_w8a8_block_fp8_matmul(a8, b8, As, Bs, [128, 128], torch.bfloat16)
    out = tg.w8a8_block_fp8_matmul(a8.to(dev), b8.to(dev), As.to(dev), Bs.to(dev), [128, 128], torch.bfloat16)
    res = R.check_tolerance(out, ref)
    assert res["ok"], res
    _lib.device_status(dev.index)  # no fault, no expired wait


def test_block_scaled_rejects_other_blocks_and_dtypes(dev):
    a = torch.zeros(128, 128, dtype=torch.float8_e4m3fn, device=dev)
    with pytest.raises(RuntimeError, match="INVALID_ARGS"):
        tg.w8a8_block_fp8_matmul(a, a, torch.ones(128, 2, device=dev), torch.ones(2, 2, device=dev), [64, 64])
    with pytest.raises(RuntimeError, match="INVALID_ARGS"):
        tg.w8a8_block_fp8_matmul(a, a, torch.ones(128, 1, device=dev), torch.ones(1, 1, device=dev), None, torch.int32)


def test_act_quant_feeds_block_scaled_gemm(dev):
    """Quantise on the GPU, multiply on the GPU, compare with the oracle chain."""
    x = torch.randn(256, 1024, dtype=torch.bfloat16)
    w = R.gen_weights(384, 1024, 3)
    yq, ys = R.ref_act_quant(x)
    wq, ws = R.ref_weight_quant_block(w)
    ref = R.ref_w8a8_block_fp8_matmul(yq, wq, ys, ws, None, torch.bfloat16)
    gy, gs = tg.act_quant(x.to(dev))
    gw, gws = tg.weight_quant_block(w.to(dev))
    out = tg.w8a8_block_fp8_matmul(gy, gw, gs, gws, None, torch.bfloat16)
    assert R.check_tolerance(out, ref)["ok"]
