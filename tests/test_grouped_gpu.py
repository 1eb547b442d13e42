"""Grouped (ragged, MoE-style) block-scaled GEMM against the oracle."""
import pytest
import torch

from conftest import load_golden
from oracle import torch_ref as R

pytestmark = pytest.mark.gpu

import tilegym_b200 as tg  # noqa: E402
from tilegym_b200 import _lib  # noqa: E402


def make_case(sizes, N, K, seed):
    """Stacked rows of all groups and one weight per group; any N and K (K a multiple of 16)."""
    g = torch.Generator().manual_seed(seed)
    total, G, kb, nb = sum(sizes), len(sizes), -(-K // 128), -(-N // 128)
    a8 = torch.randn(total, K, generator=g).clamp(-448, 448).to(torch.float8_e4m3fn)
    b = (torch.randn(G, N, K, generator=g) * 0.5).to(torch.float8_e4m3fn)
    As = torch.rand(total, kb, generator=g) * 0.02 + 0.001
    bs = torch.rand(G, nb, kb, generator=g) * 0.01 + 0.001
    ind = torch.tensor([0] + [int(v) for v in torch.tensor(sizes).cumsum(0)], dtype=torch.int32)
    return a8, b, As, bs, ind


@pytest.mark.parametrize("name", ["ragged_bmm_q4_m128_256x256.npz", "ragged_bmm_q3_m256_384x512.npz"])
def test_fixtures_from_the_reference_test(dev, name):
    g = load_golden(name)
    out = tg.ragged_block_scaled_bmm(g["a"].to(dev), g["b"].to(dev), g["a_scale"].to(dev), g["b_scale"].to(dev),
                                     g["m_indptr"].to(dev), 0)
    assert out.dtype == torch.bfloat16 and out.shape == g["c"].shape
    res = R.check_tolerance(out, g["c"])
    assert res["ok"], res


@pytest.mark.parametrize("num_groups,m", [(4, 128), (16, 512)])
@pytest.mark.parametrize("n,k", [(2048, 2048), (4096, 4096)])
def test_reference_test_grid(dev, num_groups, m, n, k):
    """Corners of the reference test's grid (test_flashinfer_ragged_block_scaled_bmm.py:219-224), aligned
    segments, held to this repository's tolerance instead of the reference's atol = rtol = 1."""
    a8, b, As, bs, ind = make_case([m] * num_groups, n, k, seed=300 + num_groups + n)
    ref = R.ref_ragged_block_scaled_bmm(a8, b, As, bs, ind)
    out = tg.ragged_block_scaled_bmm(a8.to(dev), b.to(dev), As.to(dev), bs.to(dev), ind.to(dev), m)
    res = R.check_tolerance(out, ref)
    assert res["ok"], res


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32, torch.float16])
def test_ragged_unaligned_and_empty_groups(dev, out_dtype):
    """Segments of any length (1 row, 129 rows, empty), N not a multiple of 256, K not a multiple of 128."""
    sizes = [1, 129, 0, 300, 77, 0, 128, 31]
    a8, b, As, bs, ind = make_case(sizes, 328, 400, seed=41)
    ref = R.ref_ragged_block_scaled_bmm(a8, b, As, bs, ind, out_dtype=out_dtype)
    out = tg.ragged_block_scaled_bmm(a8.to(dev), b.to(dev), As.to(dev), bs.to(dev), ind.to(dev), 300,
                                     out_dtype=out_dtype)
    if out_dtype == torch.float32:
        torch.testing.assert_close(out.cpu(), ref, rtol=1e-4, atol=1e-4 * float(ref.abs().max()))
    else:
        res = R.check_tolerance(out.float(), ref.float())
        assert res["ok"], res
    _lib.device_status(dev.index)


@pytest.mark.parametrize("tile", ["32", "64", None])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32, torch.float16])
def test_small_groups_take_the_swap_ab_kernel(dev, tile, out_dtype):
    """Groups of a few rows (a mixture-of-experts layer at decode sizes) run on the grouped form of the small-M
    kernel: groups of 1 row, empty groups, groups longer than the 32- / 64-row tile (two or three tiles), N not a
    multiple of 128, K not a multiple of 128, bias per group and a factor per row."""
    sizes = [1, 0, 7, 33, 2, 0, 0, 70, 5, 1, 16, 3, 0, 9, 32, 4]
    N, K = 328, 400
    a8, b, As, bs, ind = make_case(sizes, N, K, seed=17)
    g = torch.Generator().manual_seed(5)
    bias = torch.randn(len(sizes), N, generator=g).to(torch.bfloat16)
    rs = torch.rand(sum(sizes), generator=g) + 0.25
    ref = R.ref_ragged_block_scaled_bmm(a8, b, As, bs, ind, out_dtype=torch.float32)
    lo = 0
    for q, sz in enumerate(sizes):
        ref[lo:lo + sz] = ref[lo:lo + sz] * rs[lo:lo + sz, None] + bias[q].float()
        lo += sz
    ref = ref.to(out_dtype)
    _lib.set_knob("TILEGYM_B200_GROUPED_SMALLM", tile)
    try:
        out = tg.ragged_block_scaled_bmm(a8.to(dev), b.to(dev), As.to(dev), bs.to(dev), ind.to(dev), max(sizes),
                                         out_dtype=out_dtype, bias=bias.to(dev), row_scale=rs.to(dev))
        torch.cuda.synchronize(dev)
    finally:
        _lib.set_knob("TILEGYM_B200_GROUPED_SMALLM", None)
    if out_dtype == torch.float32:
        torch.testing.assert_close(out.cpu(), ref, rtol=1e-4, atol=1e-4 * float(ref.abs().max()))
    else:
        res = R.check_tolerance(out.float(), ref.float())
        assert res["ok"], res
    _lib.device_status(dev.index)


def test_small_group_kernel_equals_the_tile_kernel_bit_for_bit(dev):
    """Same k-block order and the same fused multiply-adds per element: the two grouped kernels agree exactly."""
    sizes = [3, 20, 0, 31, 8, 1, 12, 5]
    a8, b, As, bs, ind = make_case(sizes, 512, 1024, seed=23)
    args = [t.to(dev) for t in (a8, b, As, bs, ind)]
    outs = {}
    for tile in ("0", "32", "64"):
        _lib.set_knob("TILEGYM_B200_GROUPED_SMALLM", tile)
        try:
            outs[tile] = tg.ragged_block_scaled_bmm(*args, max(sizes)).clone()
        finally:
            _lib.set_knob("TILEGYM_B200_GROUPED_SMALLM", None)
    assert torch.equal(outs["0"], outs["32"]) and torch.equal(outs["0"], outs["64"])
    _lib.device_status(dev.index)


@pytest.mark.parametrize("seed", list(range(8)))
def test_random_small_groups_agree_with_the_tile_kernel_and_the_oracle(dev, seed):
    """Seeded random problems: group count, group sizes (many empty), N and K vary; the small-group kernel (tile
    height chosen by the library), the forced other height and the 128-row tile kernel must agree bit for bit, and
    all must meet the oracle."""
    g = torch.Generator().manual_seed(1000 + seed)
    G = int(torch.randint(1, 40, (1,), generator=g))
    hi = int(torch.randint(2, 70, (1,), generator=g))
    sizes = [int(v) for v in torch.randint(0, hi, (G,), generator=g)]
    if sum(sizes) == 0:
        sizes[0] = 1
    N = int(torch.randint(1, 5, (1,), generator=g)) * 128 + int(torch.randint(0, 2, (1,), generator=g)) * 72
    K = int(torch.randint(1, 9, (1,), generator=g)) * 128 + int(torch.randint(0, 2, (1,), generator=g)) * 48
    a8, b, As, bs, ind = make_case(sizes, N, K, seed=2000 + seed)
    ref = R.ref_ragged_block_scaled_bmm(a8, b, As, bs, ind)
    args = [t.to(dev) for t in (a8, b, As, bs, ind)]
    outs = []
    for tile in (None, "0", "32", "64"):
        _lib.set_knob("TILEGYM_B200_GROUPED_SMALLM", tile)
        try:
            outs.append(tg.ragged_block_scaled_bmm(*args, max(sizes)).clone())
        finally:
            _lib.set_knob("TILEGYM_B200_GROUPED_SMALLM", None)
    torch.cuda.synchronize(dev)
    _lib.device_status(dev.index)
    for o in outs[1:]:
        assert torch.equal(outs[0], o), (G, sizes, N, K)
    res = R.check_tolerance(outs[0], ref)
    assert res["ok"], (res, G, N, K)


def test_each_group_equals_the_dense_kernel(dev):
    """Per group the grouped kernel runs the same k-block order and the same fused multiply-adds as the dense
    block-scaled kernel: identical bits."""
    import os

    sizes = [256, 384, 128]
    a8, b, As, bs, ind = make_case(sizes, 512, 1024, seed=9)
    args = [t.to(dev) for t in (a8, b, As, bs, ind)]
    out = tg.ragged_block_scaled_bmm(*args, 384)
    _lib.set_knob("TILEGYM_B200_SPLITS", "1")  # the dense kernel would split K on problems this small
    try:
        lo = 0
        for q, sz in enumerate(sizes):
            dense = tg.w8a8_block_fp8_matmul(args[0][lo:lo + sz], args[1][q], args[2][lo:lo + sz], args[3][q],
                                             [128, 128], torch.bfloat16)
            assert torch.equal(out[lo:lo + sz], dense)
            lo += sz
    finally:
        _lib.set_knob("TILEGYM_B200_SPLITS", None)


def test_rows_outside_every_group_are_left_alone_and_bad_offsets_are_clamped(dev):
    a8, b, As, bs, _ = make_case([200, 56], 256, 256, seed=3)
    ind = torch.tensor([64, 200, 100000], dtype=torch.int32)  # starts late, last offset far past the end
    ref = R.ref_ragged_block_scaled_bmm(a8, b, As, bs, torch.tensor([64, 200, 256], dtype=torch.int32))
    L = _lib.lib()
    c = torch.full((256, 256), 7.0, dtype=torch.bfloat16, device=dev)
    args = [t.to(dev) for t in (a8, b, As, bs, ind)]
    rc = L.tg_fp8_gemm_blockscaled_grouped(_lib.ref(_lib.desc(c)), *[_lib.ref(_lib.desc(t)) for t in args[:4]],
                                            args[4].data_ptr(), 128, 128, None, 0.0, 0, dev.index,
                                           torch.cuda.current_stream().cuda_stream)
    _lib.check_rc(rc)
    _lib.device_status(dev.index)
    assert bool((c[:64] == 7.0).all())
    res = R.check_tolerance(c[64:], ref[64:])
    assert res["ok"], res


def test_argument_errors(dev):
    a8, b, As, bs, ind = [t.to(dev) for t in make_case([128], 256, 256, seed=1)]
    with pytest.raises(AssertionError):
        tg.ragged_block_scaled_bmm(a8, b, As, bs, ind, 128, transpose_b=False)
    with pytest.raises(RuntimeError):
        tg.ragged_block_scaled_bmm(a8, b, As, bs, ind.long(), 128)
    with pytest.raises(AssertionError):
        tg.ragged_block_scaled_bmm(a8, b, As, bs, ind[:1], 128)
