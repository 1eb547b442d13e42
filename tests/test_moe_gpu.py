"""The FP8 mixture-of-experts path through the C ABI: routing tables, the row gather, silu * mul + quantise,
the two grouped GEMMs with the routing weight in the second one's epilogue, and the sum back in token order -
against the CPU oracle (which is pinned to the reference's torch MoE references by tests/test_oracle.py).

Tolerance of the end-to-end checks: |t - r| <= 2 bf16 ulps of max|r| + 1e-2 |r|.  The layer rounds twice on the
way (the first GEMM's output to 16 bits, silu * mul to e4m3): an fp32 summation-order difference can flip such a
rounding, which moves one of the I intermediate values by one e4m3 step, so small outputs carry an absolute,
not a relative, error.  The reference's own test allows atol = rtol = 0.5 for fp8 (tests/ops/test_moe.py:172-174).
"""

import pytest
import torch

from conftest import load_golden
from oracle import torch_ref as R

pytestmark = pytest.mark.gpu

import tilegym_b200 as tg  # noqa: E402
from tilegym_b200 import _lib, moe  # noqa: E402


def close_enough(out, ref):
    o, r = out.float().cpu(), ref.float()
    bound = 2.0 * R.ulp_bf16(float(r.abs().max())) + 1e-2 * r.abs()
    bad = (o - r).abs() > bound
    assert not bool(bad.any()), (int(bad.sum()), float((o - r).abs().max()), float(r.abs().max()))


def make_case(T, H, I, E, topk, seed, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    x = torch.empty(T, H).normal_(0, 0.5, generator=g)
    w1 = torch.empty(E, 2 * I, H).normal_(0, 0.1, generator=g)
    w2 = torch.empty(E, H, I).normal_(0, 0.1, generator=g)
    ids = torch.randint(0, E, (T, topk), generator=g, dtype=torch.long)
    wts = torch.softmax(torch.randn(T, topk, generator=g), dim=-1)
    q1 = [R.ref_weight_quant_block(w1[e]) for e in range(E)]
    q2 = [R.ref_weight_quant_block(w2[e]) for e in range(E)]
    return (x.to(dtype), torch.stack([q for q, _ in q1]), torch.stack([s for _, s in q1]),
            torch.stack([q for q, _ in q2]), torch.stack([s for _, s in q2]), wts, ids)


@pytest.mark.parametrize("T,topk,E", [(300, 6, 40), (70000, 4, 100), (64, 2, 5000)])
def test_routing_tables(dev, T, topk, E):
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, E, (T, topk), generator=g, dtype=torch.int32)
    ids[5, topk - 1] = -3   # invalid ids take part in nothing
    ids[9, 0] = E
    wts = torch.rand(T, topk, generator=g)
    m_indptr, sorted_ids, pos, w_sorted = (t.cpu() for t in moe.moe_route(ids.to(dev), wts.to(dev), E))
    flat = ids.reshape(-1).long()
    valid = (flat >= 0) & (flat < E)
    counts = torch.bincount(flat[valid], minlength=E)
    assert torch.equal(m_indptr.long(), torch.cat([torch.zeros(1, dtype=torch.long), counts.cumsum(0)]))
    n_valid = int(valid.sum())
    srt = sorted_ids[:n_valid].long()
    assert torch.equal(srt.sort().values, torch.nonzero(valid).flatten())  # a permutation of the valid pairs
    for e in range(E):  # every segment holds exactly the pairs of its expert
        seg = srt[int(m_indptr[e]):int(m_indptr[e + 1])]
        assert bool((flat[seg] == e).all())
    assert torch.equal(pos[srt].long(), torch.arange(n_valid))  # pos inverts sorted_ids
    assert bool((pos[~valid] == -1).all())
    assert torch.equal(w_sorted[:n_valid], wts.reshape(-1)[srt])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("T,H,topk,E", [(37, 512, 4, 9), (1, 128, 1, 3), (300, 2048, 6, 64)])
def test_quantise_and_scatter_equals_act_quant_then_gather(dev, T, H, topk, E, dtype):
    """16-bit activations go into expert order in one pass: the bytes and scales of act_quant followed by the row
    gather, including tokens with an invalid expert id (skipped) and an all-zero block (scale 1)."""
    g = torch.Generator().manual_seed(T + H)
    x = (torch.randn(T, H, generator=g) * 3).to(dtype)
    x[0, :128] = 0
    ids = torch.randint(0, E, (T, topk), generator=g, dtype=torch.int32)
    ids[T // 2, 0] = -1
    xd, idd = x.to(dev), ids.to(dev)
    m_indptr, sorted_ids, pos, _ = moe.moe_route(idd, None, E)
    n_rows = T * topk
    a8, a_s = tg.act_quant(xd, 128)
    L = _lib.lib()
    stream = torch.cuda.current_stream(dev).cuda_stream
    ref_a = torch.zeros((n_rows, H), dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)
    ref_s = torch.zeros((n_rows, H // 128), dtype=torch.float32, device=dev)
    _lib.check_rc(L.tg_moe_permute_rows(_lib.desc(ref_a), _lib.desc(ref_s), _lib.desc(a8), _lib.desc(a_s),
                                        sorted_ids.data_ptr(), m_indptr.data_ptr(), E, topk, dev.index, stream))
    out_a = torch.zeros((n_rows, H), dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)
    out_s = torch.zeros((n_rows, H // 128), dtype=torch.float32, device=dev)
    _lib.check_rc(L.tg_moe_quant_permute_rows(_lib.desc(out_a), _lib.desc(out_s), _lib.desc(xd), pos.data_ptr(), topk,
                                              dev.index, stream))
    torch.cuda.synchronize(dev)
    assert torch.equal(out_a.view(torch.uint8), ref_a.view(torch.uint8)) and torch.equal(out_s, ref_s)
    yr, sr = R.ref_act_quant(x, 128)
    rows = int(m_indptr[-1])
    src = (sorted_ids[:rows].cpu().long() // topk)
    assert torch.equal(out_a[:rows].cpu().view(torch.uint8), yr.view(torch.uint8)[src]) and torch.equal(out_s[:rows].cpu(), sr[src])


def test_moe_align_block_size_tables(dev):
    """Semantics of src/tilegym/ops/moe_interface.py:30-81: each expert's pairs padded to a multiple of the block
    with the value tokens * top_k, one expert id per block."""
    T, topk, E, block = 70, 4, 9, 16
    ids = torch.randint(0, E, (T, topk), generator=torch.Generator().manual_seed(2), dtype=torch.int64)
    ids[ids == 3] = 4  # an expert without tokens
    stid, eids, npad, cumsum, max_cnt = (t.cpu() for t in moe.moe_align_block_size(ids.to(dev), block, E))
    n = T * topk
    counts = torch.bincount(ids.reshape(-1), minlength=E)
    blocks = (counts + block - 1) // block
    assert int(npad) == int(blocks.sum()) * block and int(max_cnt) == int(counts.max())
    assert torch.equal(cumsum.long(), torch.cat([torch.zeros(1, dtype=torch.long), (blocks * block).cumsum(0)]))
    lo = 0
    for e in range(E):
        seg = stid[lo:lo + int(blocks[e]) * block].long()
        real = seg[seg < n]
        assert real.numel() == int(counts[e]) and bool((ids.reshape(-1)[real] == e).all())
        assert bool((seg[int(counts[e]):] == n).all())
        assert bool((eids[lo // block: lo // block + int(blocks[e])] == e).all())
        lo += int(blocks[e]) * block
    assert bool((stid[lo:] == n).all()) and bool((eids[lo // block:] == -1).all())


@pytest.mark.parametrize("a2_quant", ["ones", "block"])
def test_fused_experts_against_reference_fixture(dev, a2_quant):
    g = load_golden("moe_16x256x128_e4_k2.npz")
    ids = g["ids"]
    ref = R.ref_fused_experts_fp8(g["a8"], g["a_s"], g["w1"], g["w1_s"], g["w2"], g["w2_s"], g["wts"], ids,
                                  torch.float16, a2_quant)
    out = moe.fused_experts_impl(g["a8"].to(dev), g["w1"].to(dev), g["w2"].to(dev), g["wts"].to(dev), ids.to(dev),
                                 use_fp8_w8a8=True, w1_scale=g["w1_s"].to(dev), w2_scale=g["w2_s"].to(dev),
                                 a1_scale=g["a_s"].to(dev), a2_quant=a2_quant)
    assert out.dtype == torch.float16 and out.shape == (16, 256)
    close_enough(out, ref)
    # the reference test's own comparison: its torch MoE on the dequantised operands, atol = rtol = 0.5
    torch.testing.assert_close(out.float().cpu(), g["full_f32"], rtol=5e-1, atol=5e-1)


@pytest.mark.parametrize("T,H,I,E,topk", [(16, 512, 256, 8, 2), (32, 1024, 512, 16, 4), (64, 1024, 512, 20, 8),
                                          (700, 512, 384, 6, 3)])
def test_fused_experts_reference_test_shapes(dev, T, H, I, E, topk):
    """Shapes of tests/ops/test_moe.py:70-76 (plus one with long, uneven segments); e4m3 activations in."""
    x, w1, w1s, w2, w2s, wts, ids = make_case(T, H, I, E, topk, seed=T + E)
    a8, a_s = R.ref_act_quant(x, 128)
    ref = R.ref_fused_experts_fp8(a8, a_s, w1, w1s, w2, w2s, wts, ids, torch.float16)
    out = moe.fused_experts_impl(a8.to(dev), w1.to(dev), w2.to(dev), wts.to(dev), ids.to(dev), use_fp8_w8a8=True,
                                 w1_scale=w1s.to(dev), w2_scale=w2s.to(dev), a1_scale=a_s.to(dev))
    close_enough(out, ref)
    _lib.device_status(dev.index)


@pytest.mark.parametrize("fuse", [True, False])
@pytest.mark.parametrize("a2_quant", ["ones", "block"])
@pytest.mark.parametrize("dtype", [torch.float8_e4m3fn, torch.bfloat16])
@pytest.mark.parametrize("T,H,I,E,topk", [(64, 1024, 512, 20, 8), (700, 512, 384, 6, 3), (300, 256, 256, 2, 2),
                                          (5, 256, 128, 3, 1)])
def test_interleaved_gate_up_weights(dev, T, H, I, E, topk, dtype, a2_quant, fuse):
    """With the gate / up rows of w1 interleaved in blocks of 128 the first GEMM can apply silu * mul and the e4m3
    quantisation itself (fuse, taken where an expert has more than 64 rows on average: the second and third shape);
    without it, and for small groups, the separate pass reads the interleaved columns.  Same oracle, same tolerance."""
    x, w1, w1s, w2, w2s, wts, ids = make_case(T, H, I, E, topk, seed=3 * T + E)
    a8, a_s = R.ref_act_quant(x.to(torch.bfloat16) if dtype == torch.bfloat16 else x, 128)
    out_dtype = torch.bfloat16 if dtype == torch.bfloat16 else torch.float16
    ref = R.ref_fused_experts_fp8(a8, a_s, w1, w1s, w2, w2s, wts, ids, out_dtype, a2_quant)
    w1i, w1si = moe.interleave_gate_up_blocks(w1.to(dev), w1s.to(dev))
    hidden = x.to(torch.bfloat16).to(dev) if dtype == torch.bfloat16 else a8.to(dev)
    out = moe.fused_experts_impl(hidden, w1i, w2.to(dev), wts.to(dev), ids.to(dev), use_fp8_w8a8=True, w1_scale=w1si,
                                 w2_scale=w2s.to(dev), a1_scale=None if dtype == torch.bfloat16 else a_s.to(dev),
                                 a2_quant=a2_quant, w1_interleaved=True, fuse_silu_epilogue=fuse)
    assert out.dtype == out_dtype
    close_enough(out, ref)
    _lib.device_status(dev.index)


def test_fused_moe_bf16_activations_are_quantised_on_the_way(dev):
    x, w1, w1s, w2, w2s, wts, ids = make_case(48, 512, 256, 8, 2, seed=11, dtype=torch.bfloat16)
    a8, a_s = R.ref_act_quant(x, 128)
    ref = R.ref_fused_experts_fp8(a8, a_s, w1, w1s, w2, w2s, wts, ids, torch.bfloat16, "block")
    out = moe.fused_moe(x.to(dev), w1.to(dev), w2.to(dev), wts.to(dev), ids.to(torch.int32).to(dev),
                        w1_scale=w1s.to(dev), w2_scale=w2s.to(dev), a2_quant="block")
    assert out.dtype == torch.bfloat16
    close_enough(out, ref)


def test_fp8moe_module_from_16bit_weights(dev):
    g = torch.Generator().manual_seed(4)
    w1 = torch.empty(4, 512, 256).normal_(0, 0.1, generator=g)
    w2 = torch.empty(4, 256, 256).normal_(0, 0.1, generator=g)
    x = torch.empty(2, 9, 256).normal_(0, 0.5, generator=g).to(torch.bfloat16)
    ids = torch.randint(0, 4, (2, 9, 2), generator=g)
    wts = torch.softmax(torch.randn(2, 9, 2, generator=g), dim=-1)
    mod = moe.FP8MoE.from_weights(w1.to(dev).to(torch.bfloat16), w2.to(dev).to(torch.bfloat16))
    out = mod(x.to(dev), wts.to(dev), ids.to(dev))
    assert out.shape == x.shape and out.dtype == torch.bfloat16
    # against the unquantised layer: e4m3 weights and activations keep ~2 significant digits
    xf, w1f, w2f = x.float().reshape(-1, 256), w1.to(torch.bfloat16).float(), w2.to(torch.bfloat16).float()
    ref = torch.zeros(18, 256)
    for t in range(18):
        for j in range(2):
            e = int(ids.reshape(-1, 2)[t, j])
            h = xf[t] @ w1f[e].T
            ref[t] += float(wts.reshape(-1, 2)[t, j]) * ((torch.nn.functional.silu(h[:256]) * h[256:]) @ w2f[e].T)
    cos = torch.nn.functional.cosine_similarity(out.float().cpu().flatten(), ref.flatten(), dim=0)
    assert cos > 0.995, float(cos)


def test_silu_mul_quant_and_unpermute_sum_pieces(dev):
    R_, I = 50, 384
    g = torch.Generator().manual_seed(6)
    x = (torch.randn(R_, 2 * I, generator=g) * 2).to(torch.float16)
    ind = torch.tensor([0, 20, 50], dtype=torch.int32, device=dev)  # device operands stay referenced until the
    xd = x.to(dev)                                                  # kernels that read them have been enqueued
    for mode, name in ((0, "ones"), (1, "block")):
        y = torch.zeros(R_, I, dtype=torch.float8_e4m3fn, device=dev)
        s = torch.zeros(R_, I // 128, device=dev)
        rc = _lib.lib().tg_moe_silu_mul_quant(_lib.desc(y), _lib.desc(s), _lib.desc(xd), ind.data_ptr(), 2,
                                              mode, dev.index, torch.cuda.current_stream(dev).cuda_stream)
        _lib.check_rc(rc)
        yr, sr = R.ref_moe_silu_mul_quant(x, name)
        torch.testing.assert_close(s.cpu(), sr.reshape(R_, -1), rtol=1e-6, atol=0)
        # exp() differs in the last fp32 bit between the two: a 16-bit rounding may flip, then at most one e4m3 step
        got, want = y.cpu().float() * s.cpu().repeat_interleave(128, 1), yr.float() * sr.reshape(R_, -1).repeat_interleave(128, 1)
        assert float(((got - want).abs() / want.abs().clamp_min(1e-3)).max()) <= 0.13
        assert float((y.cpu().view(torch.uint8) != yr.view(torch.uint8)).float().mean()) < 1e-3
    # sum over top-k rows in token order, pairs with pos = -1 skipped
    T, topk, H = 30, 3, 256
    c = torch.randn(T * topk, H, generator=g).to(torch.bfloat16)
    pos = torch.randperm(T * topk, generator=g).to(torch.int32)
    pos[7] = -1
    out = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
    cd, posd = c.to(dev), pos.to(dev)
    _lib.check_rc(_lib.lib().tg_moe_unpermute_sum(_lib.desc(out), _lib.desc(cd), posd.data_ptr(), topk,
                                                   dev.index, torch.cuda.current_stream(dev).cuda_stream))
    rows = c.float()[pos.long().clamp_min(0)] * (pos >= 0).float()[:, None]
    assert torch.equal(out.cpu(), rows.view(T, topk, H).sum(1).to(torch.bfloat16))


def test_bf16_weight_path_is_refused(dev):
    x = torch.zeros(4, 256, dtype=torch.bfloat16, device=dev)
    w1 = torch.zeros(2, 256, 256, dtype=torch.bfloat16, device=dev)
    w2 = torch.zeros(2, 256, 128, dtype=torch.bfloat16, device=dev)
    with pytest.raises(NotImplementedError, match="FP8 W8A8 path only"):
        moe.fused_moe(x, w1, w2, torch.ones(4, 1, device=dev), torch.zeros(4, 1, dtype=torch.int64, device=dev))
