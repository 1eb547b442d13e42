"""FP8 mixture-of-experts layer on the grouped block-scaled GEMM.

Entry points with the reference's names and signatures (src/tilegym/ops/moe_interface.py):
`fused_experts_impl` (:116-322), `fused_moe` (:325-372), `moe_align_block_size` (:22-81).  Only the FP8 W8A8
path with 128 x 128 weight scales and 1 x 128 activation scales is implemented (use_fp8_w8a8=True, the
`fused_moe_kernel<..., USE_FP8_SCALES>` arithmetic of src/tilegym/ops/tilecpp/moe.cuh:175-191); the bf16 and
int8 paths of the reference raise NotImplementedError.

How it differs inside (same results): the reference pads each expert's token list to the tile height and
gathers rows in every GEMM tile through sorted_token_ids.  Here

    route          counting sort of the (token, slot) pairs by expert, on the device      (tg_moe_route)
    permute        e4m3 rows + their scales gathered into expert order, once              (tg_moe_permute_rows)
    fc1            grouped GEMM on contiguous segments -> [rows, 2 I] in 16 bits           (tg_fp8_gemm_blockscaled_grouped)
    silu * mul     rounded to 16 bits like the reference's intermediate, then to e4m3     (tg_moe_silu_mul_quant)
    fc2            grouped GEMM, routing weight applied per row in fp32 before rounding   (row_scale)
    sum            out[t] = sum of the token's top-k rows, un-permutation folded in       (tg_moe_unpermute_sum)

Nothing is read back to the host, so the whole layer can be captured in a CUDA graph whose routing changes
between replays.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib, ops

_FP8 = torch.float8_e4m3fn


def moe_route(topk_ids: torch.Tensor, topk_weights: Optional[torch.Tensor], num_experts: int):
    """(m_indptr [E+1] int32, sorted_ids [T*k] int32, pos [T*k] int32, w_sorted [T*k] f32): the rows of expert e
    are sorted positions m_indptr[e] .. m_indptr[e+1]; sorted row r is pair sorted_ids[r] = token * k + slot;
    pos is the inverse (-1 for ids outside [0, E)); w_sorted the routing weights in sorted order."""
    dev = ops._need_cuda(topk_ids, topk_weights)
    assert topk_ids.dim() == 2
    if topk_ids.dtype not in (torch.int32, torch.int64):
        raise _lib.TileGymB200Error(-2, f"topk_ids must be int32 or int64, got {topk_ids.dtype}")
    if not topk_ids.is_contiguous():
        topk_ids = topk_ids.contiguous()
    if topk_weights is not None and not topk_weights.is_contiguous():
        topk_weights = topk_weights.contiguous()
    n = topk_ids.numel()
    m_indptr = torch.empty(num_experts + 1, dtype=torch.int32, device=dev)
    sorted_ids = torch.empty(max(n, 1), dtype=torch.int32, device=dev)
    pos = torch.empty(max(n, 1), dtype=torch.int32, device=dev)
    w_sorted = torch.empty(max(n, 1), dtype=torch.float32, device=dev)
    scratch = torch.empty(num_experts, dtype=torch.int32, device=dev)
    rc = _lib.lib().tg_moe_route(
        _lib.desc(topk_ids), _lib.desc(topk_weights), int(num_experts), m_indptr.data_ptr(), sorted_ids.data_ptr(),
        pos.data_ptr(), w_sorted.data_ptr(), scratch.data_ptr(), dev.index, ops._stream(dev),
    )
    _lib.check_rc(rc)
    return m_indptr, sorted_ids[:n], pos[:n], w_sorted[:n]


def moe_align_block_size(
    topk_ids: torch.Tensor, block_size: int, num_experts: int
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """The reference's padded routing tables (src/tilegym/ops/moe_interface.py:30-81), for callers that want
    them: (sorted_token_ids, expert_ids, num_tokens_post_padded, expert_cumsum, max_expert_cnt).  Every expert's
    pair list is padded to a multiple of `block_size` with the value tokens * top_k.  Built from `moe_route`
    with a few tensor operations on the device; the table is sized for the worst case (every expert one partly
    filled block), so nothing is read back: entries past num_tokens_post_padded hold the padding value and
    expert id -1.  `fused_experts_impl` itself does not use these tables."""
    dev = topk_ids.device
    n = topk_ids.numel()
    m_indptr, sorted_ids, _, _ = moe_route(topk_ids, None, num_experts)
    counts = (m_indptr[1:] - m_indptr[:-1]).to(torch.int64)
    blocks = (counts + block_size - 1) // block_size
    padded_start = torch.zeros(num_experts + 1, dtype=torch.int64, device=dev)
    padded_start[1:] = torch.cumsum(blocks * block_size, 0)
    max_blocks = (n + block_size - 1) // block_size + num_experts
    sorted_token_ids = torch.full((max_blocks * block_size,), n, dtype=torch.int32, device=dev)
    # sorted row r of expert e goes to padded_start[e] + (r - m_indptr[e])
    r = torch.arange(n, device=dev, dtype=torch.int64)
    e_of_r = torch.searchsorted(m_indptr[1:].to(torch.int64), r, right=True).clamp_(max=num_experts - 1)
    valid = r < m_indptr[-1].to(torch.int64)
    dest = padded_start[e_of_r] + (r - m_indptr[:-1].to(torch.int64)[e_of_r])
    dest = torch.where(valid, dest, torch.full_like(dest, max_blocks * block_size - 1))
    vals = torch.where(valid, sorted_ids.to(torch.int32), torch.full_like(sorted_ids, n))
    sorted_token_ids.scatter_(0, dest, vals)
    block_idx = torch.arange(max_blocks, device=dev, dtype=torch.int64) * block_size
    expert_ids = torch.searchsorted(padded_start[1:], block_idx, right=True)
    expert_ids = torch.where(block_idx < padded_start[-1], expert_ids, torch.full_like(expert_ids, -1)).to(torch.int32)
    num_tokens_post_padded = padded_start[-1:].to(torch.int32)
    return sorted_token_ids, expert_ids, num_tokens_post_padded, padded_start.to(torch.int32), counts.max()


def fused_experts_impl(
    hidden_states: torch.Tensor,
    w1: torch.Tensor,
    w2: torch.Tensor,
    topk_weights: torch.Tensor,
    topk_ids: torch.Tensor,
    inplace: bool = False,
    use_fp8_w8a8: bool = False,
    use_int8_w8a16: bool = False,
    w1_scale: Optional[torch.Tensor] = None,
    w2_scale: Optional[torch.Tensor] = None,
    a1_scale: Optional[torch.Tensor] = None,
    a2_quant: str = "ones",
    w1_interleaved: bool = False,
    fuse_silu_epilogue: bool = False,
) -> torch.Tensor:
    """out[t] = sum_j topk_weights[t, j] * w2[e] . (silu(gate) * up),  [gate | up] = w1[e] . x[t],  e = topk_ids[t, j].

    Signature of src/tilegym/ops/moe_interface.py:116-128 (plus `a2_quant`).  FP8 path only:
    hidden_states (T, H) e4m3 with a1_scale (T, H / 128) f32 - or 16-bit hidden_states, which are quantised
    here with act_quant (an addition) - w1 (E, 2 I, H) e4m3 with w1_scale (E, 2 I / 128, H / 128), w2 (E, H, I)
    e4m3 with w2_scale (E, H / 128, I / 128).  Like the reference the result is float16 for e4m3 (or f16)
    hidden_states and bfloat16 for bf16 ones, the first GEMM's output and silu * mul are rounded to that
    type, and the intermediate is cast to e4m3 with scale 1 (`a2_quant="ones"`, moe_interface.py:269-279);
    `a2_quant="block"` quantises it per 1 x 128 with amax / 448 instead, which keeps more of its range.
    `w1_interleaved=True` says that w1 / w1_scale were rearranged by `interleave_gate_up_blocks` (128 gate rows,
    128 up rows, alternating).  With `fuse_silu_epilogue=True` (which needs that layout) the first GEMM applies
    silu * mul and the quantisation in its epilogue and the [rows, 2 I] intermediate is never written: it saves
    that tensor (151 MB at 4096 tokens of the DeepSeek-V2-Lite shape) and costs about 7 % of the layer's time,
    because the epilogue's exponentials cannot overlap the next tile; the default runs the separate pass."""
    if use_int8_w8a16:
        raise NotImplementedError("tilegym_b200.fused_experts_impl implements the FP8 W8A8 path only (no int8 weights)")
    if not use_fp8_w8a8 or w1_scale is None or w2_scale is None:
        raise NotImplementedError(
            "tilegym_b200.fused_experts_impl implements the FP8 W8A8 path only: pass use_fp8_w8a8=True with e4m3 "
            "weights and their 128 x 128 scales (FP8MoE.from_weights quantises bf16 expert weights once)"
        )
    assert a2_quant in ("ones", "block")
    dev = ops._need_cuda(hidden_states, w1, w2, topk_weights, topk_ids, w1_scale, w2_scale)
    assert hidden_states.shape[1] == w1.shape[2], "Hidden size mismatch"
    assert topk_weights.shape == topk_ids.shape, "topk shape mismatch"
    assert hidden_states.is_contiguous(), "Hidden_states must be contiguous"
    assert w1.is_contiguous(), "Expert weights1 must be contiguous"
    assert w2.is_contiguous(), "Expert weights2 must be contiguous"
    assert hidden_states.dtype in [torch.float8_e4m3fn, torch.float32, torch.float16, torch.bfloat16]
    assert w1.dtype == _FP8 and w2.dtype == _FP8, "use_fp8_w8a8 needs float8_e4m3fn expert weights"
    T, H = hidden_states.shape
    E, N1, _ = w1.shape
    inter = N1 // 2
    assert w2.shape == (E, H, inter), "w2 must be [experts, hidden, intermediate]"
    assert N1 % 256 == 0 and H % 128 == 0, "hidden and intermediate sizes must be multiples of 128"
    assert tuple(w1_scale.shape) == (E, N1 // 128, H // 128), "w1_scale must hold one scale per 128 x 128 block"
    assert tuple(w2_scale.shape) == (E, H // 128, inter // 128), "w2_scale must hold one scale per 128 x 128 block"
    topk = topk_ids.shape[1]
    out_dtype = torch.bfloat16 if hidden_states.dtype == torch.bfloat16 else torch.float16
    L, stream = _lib.lib(), ops._stream(dev)
    m_indptr, sorted_ids, pos, w_sorted = moe_route(topk_ids, topk_weights, E)
    R = T * topk
    a_sorted = torch.empty((R, H), dtype=_FP8, device=dev)
    as_sorted = torch.empty((R, H // 128), dtype=torch.float32, device=dev)
    if hidden_states.dtype == _FP8:
        assert a1_scale is not None and tuple(a1_scale.shape) == (T, H // 128), "a1_scale must be [tokens, hidden / 128]"
        a8, a_s = hidden_states, a1_scale.to(torch.float32)
        _lib.check_rc(L.tg_moe_permute_rows(_lib.desc(a_sorted), _lib.desc(as_sorted), _lib.desc(a8), _lib.desc(a_s),
                                            sorted_ids.data_ptr(), m_indptr.data_ptr(), E, topk, dev.index, stream))
    elif hidden_states.dtype in (torch.bfloat16, torch.float16):
        # 16-bit activations: quantised (the arithmetic of act_quant) and scattered into expert order in one pass
        _lib.check_rc(L.tg_moe_quant_permute_rows(_lib.desc(a_sorted), _lib.desc(as_sorted), _lib.desc(hidden_states),
                                                  pos.data_ptr(), topk, dev.index, stream))
    else:
        a8, a_s = ops.act_quant(hidden_states, 128)
        _lib.check_rc(L.tg_moe_permute_rows(_lib.desc(a_sorted), _lib.desc(as_sorted), _lib.desc(a8), _lib.desc(a_s),
                                            sorted_ids.data_ptr(), m_indptr.data_ptr(), E, topk, dev.index, stream))
    y8 = torch.empty((R, inter), dtype=_FP8, device=dev)
    y_s = torch.empty((R, inter // 128), dtype=torch.float32, device=dev)
    mode = 1 if a2_quant == "block" else 0
    # With few rows per expert (decode sizes) the first GEMM runs on the small-group kernel, which has no fused
    # epilogue: the separate silu * mul pass reads whichever column order the weights produce.
    small_groups = R <= 64 * E and H <= 4096
    assert not fuse_silu_epilogue or w1_interleaved, "the fused epilogue needs interleave_gate_up_blocks weights"
    if fuse_silu_epilogue and not small_groups:
        # fc1 with silu * mul and the quantisation in its epilogue
        _lib.check_rc(L.tg_fp8_gemm_blockscaled_grouped_swiglu(
            _lib.desc(y8), _lib.desc(y_s), _lib.desc(a_sorted), _lib.desc(w1), _lib.desc(as_sorted), _lib.desc(w1_scale),
            m_indptr.data_ptr(), _lib.DTYPE_CODES[out_dtype], mode, dev.index, stream))
    else:
        # fc1 on contiguous expert segments: [rows, 2 I] in the 16-bit type, then silu * mul + quantise
        c1 = ops.ragged_block_scaled_bmm(a_sorted, w1, as_sorted, w1_scale, m_indptr, R, out_dtype=out_dtype)
        _lib.check_rc(L.tg_moe_silu_mul_quant(_lib.desc(y8), _lib.desc(y_s), _lib.desc(c1), m_indptr.data_ptr(), E,
                                              mode | (2 if w1_interleaved else 0), dev.index, stream))
    # fc2, routing weight applied to the fp32 sums before the rounding
    c3 = ops.ragged_block_scaled_bmm(y8, w2, y_s, w2_scale, m_indptr, R, out_dtype=out_dtype, row_scale=w_sorted)
    out = hidden_states if (inplace and hidden_states.dtype == out_dtype) else torch.empty((T, H), dtype=out_dtype, device=dev)
    _lib.check_rc(L.tg_moe_unpermute_sum(_lib.desc(out), _lib.desc(c3), pos.data_ptr(), topk, dev.index, stream))
    return out


def interleave_gate_up_blocks(w1: torch.Tensor, w1_scale: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Rearranges a fused gate / up weight (E, 2 I, H) = [gate rows | up rows] and its 128 x 128 scales
    (E, 2 I / 128, H / 128) into the order the fused first GEMM reads: 128 gate rows, the 128 up rows of the same
    outputs, the next 128 gate rows, ...  Done once, at load time."""
    E, n2, H = w1.shape
    inter = n2 // 2
    assert inter % 128 == 0
    w = w1.view(torch.uint8) if w1.dtype == _FP8 else w1
    w = w.reshape(E, 2, inter // 128, 128, H).transpose(1, 2).reshape(E, n2, H).contiguous()
    sc = w1_scale.reshape(E, 2, inter // 128, -1).transpose(1, 2).reshape(E, n2 // 128, -1).contiguous()
    return (w.view(_FP8) if w1.dtype == _FP8 else w), sc


def fused_moe(
    hidden_states: torch.Tensor,
    w1: torch.Tensor,
    w2: torch.Tensor,
    topk_weights: torch.Tensor,
    topk_ids: torch.Tensor,
    **fp8_kwargs,
) -> torch.Tensor:
    """Signature of src/tilegym/ops/moe_interface.py:325-372.  The reference's form runs the unquantised
    (16-bit weights) path, which this package does not implement; with `w1_scale=` / `w2_scale=` (and
    `a1_scale=` for e4m3 activations) it forwards to the FP8 path of `fused_experts_impl`."""
    if "w1_scale" not in fp8_kwargs:
        raise NotImplementedError(
            "tilegym_b200.fused_moe runs the FP8 W8A8 path only: pass w1_scale= / w2_scale= (see FP8MoE.from_weights)"
        )
    return fused_experts_impl(hidden_states, w1, w2, topk_weights, topk_ids, use_fp8_w8a8=True, **fp8_kwargs)


class FP8MoE(torch.nn.Module):
    """Expert weights quantised once (128 x 128 blocks, amax / 448) and kept in e4m3; forward takes 16-bit
    hidden states and the router's top-k weights and ids."""

    def __init__(self, w1_fp8, w1_scale, w2_fp8, w2_scale, a2_quant: str = "block", fuse_silu_epilogue: bool = False):
        super().__init__()
        # gate / up rows in alternating blocks of 128: the order the fused epilogue needs; the separate pass reads it too
        w1_fp8, w1_scale = interleave_gate_up_blocks(w1_fp8, w1_scale)
        self.fuse_silu_epilogue = fuse_silu_epilogue  # True: no [rows, 2 I] intermediate, about 7 % slower
        self.register_buffer("w1", w1_fp8)
        self.register_buffer("w1_scale", w1_scale)
        self.register_buffer("w2", w2_fp8)
        self.register_buffer("w2_scale", w2_scale)
        self.a2_quant = a2_quant

    @classmethod
    def from_weights(cls, w1: torch.Tensor, w2: torch.Tensor, a2_quant: str = "block") -> "FP8MoE":
        """w1 (E, 2 I, H), w2 (E, H, I) in bf16 / f16 / f32 on a CUDA device."""
        q1 = [ops.weight_quant_block(w1[e]) for e in range(w1.shape[0])]
        q2 = [ops.weight_quant_block(w2[e]) for e in range(w2.shape[0])]
        return cls(torch.stack([q for q, _ in q1]), torch.stack([s for _, s in q1]), torch.stack([q for q, _ in q2]),
                   torch.stack([s for _, s in q2]), a2_quant)

    def forward(self, hidden_states: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor) -> torch.Tensor:
        shape = hidden_states.shape
        x = hidden_states.reshape(-1, shape[-1]).contiguous()
        out = fused_experts_impl(x, self.w1, self.w2, topk_weights.reshape(x.shape[0], -1),
                                 topk_ids.reshape(x.shape[0], -1), use_fp8_w8a8=True, w1_scale=self.w1_scale,
                                 w2_scale=self.w2_scale, a2_quant=self.a2_quant, w1_interleaved=True,
                                 fuse_silu_epilogue=self.fuse_silu_epilogue)
        return out.reshape(shape)
