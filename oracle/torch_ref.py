"""CPU oracle for the FP8 scaled-GEMM path.  TEST INFRASTRUCTURE ONLY.

Nothing in the product package imports this module: it is the checker that the
tests, the smoke entry and the CPU-baseline leg of the benchmark run beside the
CUDA kernels.  Every function restates, in plain PyTorch CPU arithmetic, the
torch reference that TileGym's own tests use for the same operator; the file
and line of the function it follows is given in each docstring (paths are
relative to the TileGym source tree).

Parity status: PINNED.  `tests/golden/make_golden.py` imports TileGym's test
classes, runs their `reference` functions on the seeds and shapes the tests use
and stores inputs and outputs under `tests/golden/`; `tests/test_oracle.py`
checks every function below against those files.
"""

from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

E4M3_MAX = 448.0


# --------------------------------------------------------------------------
# e4m3 decode table, built from the format definition (independent of torch's
# cast): 1 sign, 4 exponent (bias 7), 3 mantissa bits, no infinities, the
# all-ones pattern S.1111.111 is NaN.
# --------------------------------------------------------------------------
def e4m3_table() -> np.ndarray:
    out = np.empty(256, dtype=np.float32)
    for b in range(256):
        s = -1.0 if b & 0x80 else 1.0
        e = (b >> 3) & 0xF
        m = b & 0x7
        if e == 0xF and m == 0x7:
            v = float("nan")
        elif e == 0:
            v = s * (m / 8.0) * 2.0 ** (-6)
        else:
            v = s * (1.0 + m / 8.0) * 2.0 ** (e - 7)
        out[b] = v
    return out


def e4m3_decode(bytes_u8: np.ndarray) -> np.ndarray:
    """uint8 bit patterns -> float32 values, through the table above."""
    return e4m3_table()[bytes_u8]


# --------------------------------------------------------------------------
# Quantisers
# --------------------------------------------------------------------------
def ref_act_quant(x: torch.Tensor, block_size: int = 128) -> Tuple[torch.Tensor, torch.Tensor]:
    """1 x block_size activation quantisation to e4m3.

    Follows tests/suites/unsloth/test_fp8.py:81-97 (Test_Unsloth_ActQuant.reference):
    s = amax/448 per block of `block_size` contiguous elements, 1.0 for an
    all-zero block, y = (x / s) cast to e4m3 (true division, no clamp: x/s never
    exceeds 448 in magnitude by construction).
    """
    x_flat = x.contiguous().view(-1)
    n_blocks = x_flat.numel() // block_size
    x_f32 = x_flat.view(n_blocks, block_size).float()
    s = x_f32.abs().max(dim=-1).values / E4M3_MAX
    s = torch.where(s == 0, torch.ones_like(s), s)
    y = (x_f32 / s.unsqueeze(-1)).to(torch.float8_e4m3fn)
    return y.view(x.shape), s.view(*x.shape[:-1], x.shape[-1] // block_size)


def ref_weight_dequant(
    x: torch.Tensor, s: torch.Tensor, block_size: int = 128, dtype: torch.dtype = torch.bfloat16
) -> torch.Tensor:
    """block x block weight dequantisation: y[i, j] = x[i, j] * s[i // b, j // b].

    Follows tests/suites/unsloth/test_fp8.py:22-39 (Test_Unsloth_WeightDequant.reference),
    with the Python double loop replaced by an index expansion of the scale grid.
    """
    M, N = x.shape
    s_full = s.repeat_interleave(block_size, dim=0)[:M].repeat_interleave(block_size, dim=1)[:, :N]
    return (x.float() * s_full).to(dtype)


def ref_quant_per_tensor(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-tensor e4m3 quantisation: scale = amax/448 (fp32, 1.0 if the tensor
    is all zero), q = clamp(x/scale, +-448) cast to e4m3.

    This is the quantiser the benchmark configurations state in words ("each
    quantised to e4m3 with a per-tensor fp32 scale = amax/448"); the clamp
    before the cast follows tests/suites/flashinfer/test_per_token_group_quant_8bit.py:41-68
    (torch's cast to e4m3 produces NaN above 464, so the clamp is required).
    """
    xf = x.float()
    amax = xf.abs().max()
    scale = amax / E4M3_MAX
    scale = torch.where(scale == 0, torch.ones_like(scale), scale)
    q = (xf / scale).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    return q, scale.reshape(1)


def ref_weight_quant_block(w: torch.Tensor, block: int = 128) -> Tuple[torch.Tensor, torch.Tensor]:
    """block x block weight quantisation (one fp32 scale = amax/448 per block,
    1.0 for an all-zero block) - the producer of `Bs`, inverse of
    `ref_weight_dequant` (tests/suites/unsloth/test_fp8.py:22-39)."""
    N, K = w.shape
    nb, kb = math.ceil(N / block), math.ceil(K / block)
    wp = torch.zeros(nb * block, kb * block, dtype=torch.float32)
    wp[:N, :K] = w.float()
    blocks = wp.view(nb, block, kb, block)
    amax = blocks.abs().amax(dim=(1, 3))
    s = amax / E4M3_MAX
    s = torch.where(s == 0, torch.ones_like(s), s)
    q = (blocks / s[:, None, :, None]).clamp(-E4M3_MAX, E4M3_MAX)
    q = q.reshape(nb * block, kb * block)[:N, :K].contiguous().to(torch.float8_e4m3fn)
    return q, s


def ref_per_token_group_quant_8bit(
    x: torch.Tensor,
    group_size: int,
    eps: float = 1e-10,
    dst_dtype: torch.dtype = torch.float8_e4m3fn,
    scale_ue8m0: bool = False,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-token group quantisation to e4m3 / e5m2 / int8, the torch reference of
    tests/suites/flashinfer/test_per_token_group_quant_8bit.py:41-68: per group of `group_size` contiguous
    elements amax is clamped from below by eps (in x's dtype), scale = amax / dtype_max in fp32, optionally
    rounded up to a power of two, q = clamp(x / scale, min, max) cast to the target (int8 truncates).
    Scales come back row-major, shape x.shape[:-1] + (H / group_size,); the layouts the operator offers
    (column-major, padded) hold the same numbers."""
    assert x.shape[-1] % group_size == 0 and x.is_contiguous()
    if dst_dtype == torch.int8:
        lo, hi = float(torch.iinfo(dst_dtype).min), float(torch.iinfo(dst_dtype).max)
    else:
        lo, hi = torch.finfo(dst_dtype).min, torch.finfo(dst_dtype).max
    g = x.reshape(x.numel() // group_size, group_size)
    amax = g.abs().max(dim=-1, keepdim=True)[0].clamp(min=eps).to(torch.float32)
    s = amax / hi
    if scale_ue8m0:
        floor = torch.tensor(1e-10, dtype=s.dtype)
        s = torch.exp2(torch.ceil(torch.log2(torch.maximum(s.abs(), floor))))
    q = (g / s).clamp(min=lo, max=hi).to(dst_dtype).reshape(x.shape)
    return q, s.reshape(x.shape[:-1] + (x.shape[-1] // group_size,))


# --------------------------------------------------------------------------
# GEMMs
# --------------------------------------------------------------------------
def dequant_block_scaled(
    A: torch.Tensor, B: torch.Tensor, As: torch.Tensor, Bs: torch.Tensor, block_n: int, block_k: int
) -> Tuple[torch.Tensor, torch.Tensor]:
    """fp32 dequantisation of both operands (the first half of
    tests/suites/unsloth/test_fp8.py:158-188), vectorised with repeat_interleave
    the way tests/suites/flashinfer/test_flashinfer_ragged_block_scaled_bmm.py:121-131 does."""
    K = A.shape[-1]
    N = B.shape[0]
    A2 = A.reshape(-1, K).float()
    As2 = As.reshape(A2.shape[0], -1).float()
    A_deq = A2 * As2.repeat_interleave(block_k, dim=1)[:, :K]
    Bs_full = Bs.float().repeat_interleave(block_n, dim=0)[:N].repeat_interleave(block_k, dim=1)[:, :K]
    B_deq = B.float() * Bs_full
    return A_deq, B_deq


def ref_w8a8_block_fp8_matmul(
    A: torch.Tensor,
    B: torch.Tensor,
    As: torch.Tensor,
    Bs: torch.Tensor,
    block_size: Optional[Sequence[int]] = None,
    output_dtype: torch.dtype = torch.float32,
) -> torch.Tensor:
    """Block-scaled W8A8 GEMM: C = dequant(A) @ dequant(B).T, fp32, cast.

    Follows tests/suites/unsloth/test_fp8.py:158-191
    (Test_Unsloth_W8A8_FP8_Matmul.reference): A[m, k] * As[m, k // bk],
    B[n, k] * Bs[n // bn, k // bk], one fp32 matmul, `.to(output_dtype)`.
    Leading dimensions of A are flattened as the operator does
    (src/tilegym/suites/unsloth/cutile/fp8.py:412-414).
    """
    block_n, block_k = (128, 128) if block_size is None else block_size
    A_deq, B_deq = dequant_block_scaled(A, B, As, Bs, block_n, block_k)
    C = A_deq @ B_deq.T
    return C.to(output_dtype).reshape(*A.shape[:-1], B.shape[0])


def ref_fp8_block_scaled_mm(
    A: torch.Tensor,
    B: torch.Tensor,
    As: torch.Tensor,
    Bs: torch.Tensor,
    bias: Optional[torch.Tensor] = None,
    out_dtype: torch.dtype = torch.bfloat16,
    c: Optional[torch.Tensor] = None,
    beta: float = 0.0,
) -> torch.Tensor:
    """The block-scaled GEMM above with the epilogue of a Linear layer: the fp32 product of
    tests/suites/unsloth/test_fp8.py:158-191 plus bias[n] (and beta * c) in fp32, ONE cast at the end.
    The reference operator has no bias; this is the form the benchmark description states
    (fp32 accumulate, optional bias, one rounding to bf16)."""
    A_deq, B_deq = dequant_block_scaled(A, B, As, Bs, 128, 128)
    C = A_deq @ B_deq.T
    if bias is not None:
        C = C + bias.float()
    if beta != 0.0:
        C = C + beta * c.float().reshape(C.shape)
    return C.to(out_dtype).reshape(*A.shape[:-1], B.shape[0])


def ref_ragged_block_scaled_bmm(
    a: torch.Tensor,
    b: torch.Tensor,
    a_scale: torch.Tensor,
    b_scale: torch.Tensor,
    m_indptr: torch.Tensor,
    block_n: int = 128,
    block_k: int = 128,
    out_dtype: torch.dtype = torch.bfloat16,
) -> torch.Tensor:
    """Ragged block-scaled GEMM, the torch reference of
    tests/suites/flashinfer/test_flashinfer_ragged_block_scaled_bmm.py:77-136: for every group q the rows
    [m_indptr[q], m_indptr[q+1]) of `a` are dequantised per (row, 128-K block), weight b[q] per 128 x 128
    block, multiplied in fp32 and cast.  Rows outside every group stay zero; empty groups are skipped (the
    reference asserts they do not occur)."""
    total_m, K = a.shape
    Q, N, _ = b.shape
    af, bf = a.float(), b.float()
    c = torch.zeros((total_m, N), dtype=out_dtype)
    for q in range(Q):
        lo, hi = int(m_indptr[q]), int(m_indptr[q + 1])
        if hi <= lo:
            continue
        sa = torch.repeat_interleave(a_scale[lo:hi], block_k, dim=1)[:, :K]
        sb = torch.repeat_interleave(b_scale[q], block_n, dim=0)[:N]
        sb = torch.repeat_interleave(sb, block_k, dim=1)[:, :K]
        c[lo:hi] = torch.mm(af[lo:hi] * sa, (bf[q] * sb).t()).to(out_dtype)
    return c


def ref_fp8_scaled_mm(
    A: torch.Tensor,
    B: torch.Tensor,
    scale_a: torch.Tensor,
    scale_b: torch.Tensor,
    bias: Optional[torch.Tensor] = None,
    out_dtype: torch.dtype = torch.bfloat16,
) -> torch.Tensor:
    """Per-tensor scaled GEMM: ((A*sa) @ (B*sb).T + bias) in fp32, cast to bf16.

    The dequantise -> fp32 matmul -> cast form of tests/suites/unsloth/test_fp8.py:158-191
    with a single scale per operand (the wording of the first benchmark configuration).
    """
    K = A.shape[-1]
    A_deq = A.reshape(-1, K).float() * scale_a.float().reshape(())
    B_deq = B.float() * scale_b.float().reshape(())
    C = A_deq @ B_deq.T
    if bias is not None:
        C = C + bias.float()
    return C.to(out_dtype).reshape(*A.shape[:-1], B.shape[0])


def ref_fp8_scaled_mm_swiglu(
    A: torch.Tensor,
    B_interleaved: torch.Tensor,
    scale_a: torch.Tensor,
    scale_b: torch.Tensor,
    bias_interleaved: Optional[torch.Tensor] = None,
    out_dtype: torch.dtype = torch.bfloat16,
) -> torch.Tensor:
    """silu(gate) * up of a fused gate/up projection whose weight rows alternate 32 gate rows and 32 up rows:
    the fp32 per-tensor GEMM above, then silu_and_mul (src/tilegym/ops/fused_mlp.py:97-102, torch semantics
    x[..., :I] -> silu, times x[..., I:]) in fp32, one cast at the end."""
    y = ref_fp8_scaled_mm(A, B_interleaved, scale_a, scale_b, bias_interleaved, torch.float32)
    N = B_interleaved.shape[0]
    y = y.reshape(-1, N // 64, 2, 32)
    gate, up = y[:, :, 0, :], y[:, :, 1, :]
    out = torch.nn.functional.silu(gate) * up
    return out.reshape(*A.shape[:-1], N // 2).to(out_dtype)


def ref_gemm_alpha_beta(
    a: torch.Tensor, b: torch.Tensor, c: torch.Tensor, alpha: float = 1.0, beta: float = 0.0
) -> torch.Tensor:
    """C = alpha * a @ b.T + beta * c with fp32 accumulation and an fp32
    epilogue, cast to c's dtype - the arithmetic of the kernel at
    src/tilegym/suites/flashinfer/cutile/gemm/gemm_alpha_beta.py:161-173
    (trans_a=False, trans_b=True).  Does not modify `c`."""
    acc = a.float() @ b.float().T
    out = alpha * acc
    if beta != 0.0:
        out = out + beta * c.float()
    return out.to(c.dtype)


def ref_gemm_alpha_beta_bf16(
    a: torch.Tensor, b: torch.Tensor, c: torch.Tensor, alpha: float = 1.0, beta: float = 0.0
) -> torch.Tensor:
    """Secondary cross-check: the reference test's own form, computed in bf16
    (tests/suites/flashinfer/test_flashinfer_gemm_alpha_beta.py:16-21).  Does not modify `c`."""
    dt = c.dtype
    return torch.addmm(c.clone(), a.to(dt), b.to(dt).t(), beta=beta, alpha=alpha).to(dt)


def ref_matmul(a: torch.Tensor, b: torch.Tensor, trans_b: bool = False) -> torch.Tensor:
    """Unscaled fp8 matmul, output in the input dtype
    (tests/ops/test_matmul.py:46-51; the cast back to e4m3 is clamped)."""
    bb = b.float().T if trans_b else b.float()
    out = a.float() @ bb
    if a.dtype == torch.float8_e4m3fn:
        return out.clamp(-E4M3_MAX, E4M3_MAX).to(a.dtype)
    if a.dtype == torch.float8_e5m2:
        return out.clamp(-57344.0, 57344.0).to(a.dtype)
    return out.to(a.dtype)


def ref_moe_silu_mul_quant(x: torch.Tensor, mode: str = "ones") -> Tuple[torch.Tensor, torch.Tensor]:
    """The step between the two expert GEMMs of fused_experts_impl (src/tilegym/ops/moe_interface.py:262-279):
    silu_and_mul of [rows, 2 I] into [rows, I] (fp32 arithmetic, result in x's 16-bit dtype), then the cast to
    e4m3 with an a2_scale of ones ("ones", the reference; values beyond +-448 saturate here where torch's cast
    would give NaN) or a 1 x 128 amax / 448 quantisation ("block", ref_act_quant)."""
    inter = x.shape[-1] // 2
    act = (torch.nn.functional.silu(x[..., :inter].float()) * x[..., inter:].float()).to(x.dtype)
    if mode == "block":
        return ref_act_quant(act, 128)
    y = act.float().clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    return y, torch.ones(*act.shape[:-1], inter // 128, dtype=torch.float32)


def ref_fused_experts_fp8(
    a8: torch.Tensor,
    a1_scale: torch.Tensor,
    w1: torch.Tensor,
    w1_scale: torch.Tensor,
    w2: torch.Tensor,
    w2_scale: torch.Tensor,
    topk_weights: torch.Tensor,
    topk_ids: torch.Tensor,
    out_dtype: torch.dtype = torch.float16,
    a2_quant: str = "ones",
) -> torch.Tensor:
    """The FP8 W8A8 path of fused_experts_impl (src/tilegym/ops/moe_interface.py:116-322) with the block-scale
    arithmetic of its kernel (src/tilegym/ops/tilecpp/moe.cuh:175-200): per (token, slot) pair with expert e,
    fc1 = dequant(a8[t]) . dequant(w1[e])^T in fp32 -> out_dtype; silu_and_mul -> out_dtype -> e4m3 (scale 1);
    fc2 = dequant . dequant(w2[e])^T times the routing weight in fp32 -> out_dtype; out[t] = sum over the slots
    (fp32) -> out_dtype.  Pairs are processed expert by expert (row order inside an expert does not matter)."""
    T, H = a8.shape
    E = w1.shape[0]
    topk = topk_ids.shape[1]
    c3 = torch.zeros(T, topk, w2.shape[1], dtype=out_dtype)
    flat_ids = topk_ids.reshape(-1)
    for e in range(E):
        pairs = torch.nonzero(flat_ids == e).flatten()
        if pairs.numel() == 0:
            continue
        tok = pairs // topk
        fc1 = ref_w8a8_block_fp8_matmul(a8[tok], w1[e], a1_scale[tok], w1_scale[e], [128, 128], out_dtype)
        y8, y_s = ref_moe_silu_mul_quant(fc1, a2_quant)
        a_deq, b_deq = dequant_block_scaled(y8, w2[e], y_s, w2_scale[e], 128, 128)
        fc2 = (a_deq @ b_deq.T) * topk_weights.reshape(-1)[pairs].float()[:, None]
        c3.view(T * topk, -1)[pairs] = fc2.to(out_dtype)
    return c3.float().sum(dim=1).to(out_dtype)


def ref_bmm(a: torch.Tensor, b: torch.Tensor, transpose_a: bool = False, transpose_b: bool = False) -> torch.Tensor:
    """Batched matmul, output in the input dtype (tests/ops/test_bmm.py:17-23: transpose, torch.bmm).  Computed
    in fp32 with one cast at the end (torch.bmm on f16 CPU tensors accumulates in fp32 as well); 8-bit inputs
    are clamped to the format's range before the cast back, as ref_matmul does."""
    af = (a.transpose(1, 2) if transpose_a else a).float()
    bf = (b.transpose(1, 2) if transpose_b else b).float()
    out = torch.bmm(af, bf)
    if a.dtype == torch.float8_e4m3fn:
        return out.clamp(-E4M3_MAX, E4M3_MAX).to(a.dtype)
    if a.dtype == torch.float8_e5m2:
        return out.clamp(-57344.0, 57344.0).to(a.dtype)
    return out.to(a.dtype)


# --------------------------------------------------------------------------
# Seeded input generators for the benchmark configurations.  All tensors are
# drawn on the CPU so the oracle and the GPU kernels see the same bits.
# --------------------------------------------------------------------------
def gen_activations(M: int, K: int, seed: int, outliers: bool = True) -> torch.Tensor:
    """N(0,1) activations; with `outliers`, 0.1 % of the K channels
    (max(1, round(0.001*K)) columns) are scaled by 20."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g, dtype=torch.float32)
    if outliers:
        n_out = max(1, round(0.001 * K))
        cols = torch.randperm(K, generator=g)[:n_out]
        x[:, cols] *= 20.0
    return x


def gen_weights(N: int, K: int, seed: int, std: float = 0.02) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    return torch.randn(N, K, generator=g, dtype=torch.float32) * std


def gen_per_tensor_case(M: int, N: int, K: int, seed: int, outliers: bool = True, w_std: float = 0.02):
    """(A8, B8, scale_a, scale_b) of a per-tensor-scaled case."""
    a8, sa = ref_quant_per_tensor(gen_activations(M, K, seed, outliers))
    b8, sb = ref_quant_per_tensor(gen_weights(N, K, seed + 1, w_std))
    return a8, b8, sa, sb


def gen_block_scaled_case(M: int, N: int, K: int, seed: int):
    """(A8, B8, As, Bs) of a 1x128 / 128x128 block-scaled case."""
    a8, As = ref_act_quant(gen_activations(M, K, seed, outliers=False), 128)
    b8, Bs = ref_weight_quant_block(gen_weights(N, K, seed + 1), 128)
    return a8, b8, As, Bs


# --------------------------------------------------------------------------
# Tolerance check: max relative error <= 1e-2 and max absolute error <= 2 bf16
# ulps of the reference output's magnitude.
# --------------------------------------------------------------------------
def ulp_bf16(x: float) -> float:
    """Spacing of bf16 numbers at magnitude x (8 significand bits)."""
    if x == 0.0:
        return 0.0
    return 2.0 ** (math.floor(math.log2(abs(x))) - 7)


def check_tolerance(test: torch.Tensor, ref: torch.Tensor, rel: float = 1e-2, ulps: float = 2.0) -> dict:
    """Compare `test` with the oracle output `ref`.

    With R = max|ref| and floor = 2^-10 * R:
      (1) max|t - r| <= ulps * ulp_bf16(R);
      (2) max|t - r| / |r| <= rel over the elements with |r| >= floor;
      (3) max|t - r| <= ulps * ulp_bf16(floor) over the elements below the
          floor, where cancellation makes a relative error meaningless.
    Returns the figures and `ok`.
    """
    t = test.detach().float().cpu().reshape(-1)
    r = ref.detach().float().cpu().reshape(-1)
    if t.numel() == 0:
        return {"ok": True, "R": 0.0, "max_abs": 0.0, "max_rel": 0.0, "n_below_floor": 0, "max_abs_below": 0.0}
    finite = bool(torch.isfinite(t).all())
    R = float(r.abs().max())
    diff = (t - r).abs()
    max_abs = float(diff.max())
    floor = R * 2.0 ** -10
    big = r.abs() >= floor
    max_rel = float((diff[big] / r[big].abs()).max()) if bool(big.any()) else 0.0
    small = ~big
    max_abs_below = float(diff[small].max()) if bool(small.any()) else 0.0
    ok = (
        finite
        and max_abs <= ulps * ulp_bf16(R) + 0.0
        and max_rel <= rel
        and max_abs_below <= ulps * ulp_bf16(floor)
    ) or (R == 0.0 and max_abs == 0.0)
    return {
        "ok": bool(ok),
        "finite": finite,
        "R": R,
        "floor": floor,
        "max_abs": max_abs,
        "max_abs_ulps_of_R": max_abs / ulp_bf16(R) if R else 0.0,
        "max_rel": max_rel,
        "n_below_floor": int(small.sum()),
        "max_abs_below": max_abs_below,
    }
