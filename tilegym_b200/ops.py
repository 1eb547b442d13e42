"""Operator entry points: same names, arguments and error behaviour as the
reference's operator stubs, routed to the sm_100a kernels through the C ABI.

There is no dispatch table and no fallback: every function needs CUDA tensors
and the built shared library, and raises otherwise.  All work is enqueued on
`torch.cuda.current_stream()` without synchronising, like the reference
(src/tilegym/suites/unsloth/cutile/fp8.py:424).
"""

from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch

from . import _lib

_OUT_DTYPES = (torch.float32, torch.float16, torch.bfloat16)
_IN_DTYPES = (torch.float32, torch.float16, torch.bfloat16)
_FP8 = torch.float8_e4m3fn
_FP8_TYPES = (torch.float8_e4m3fn, torch.float8_e5m2)
_FP8_MAX = {torch.float8_e4m3fn: 448.0, torch.float8_e5m2: 57344.0}

# One zero-initialised scratch buffer per (device, stream): the split-K paths
# keep partial sums and arrival counters there and leave the counters zero.
_workspaces: Dict[Tuple[int, int], torch.Tensor] = {}
_amax_scratch: Dict[Tuple[int, int], torch.Tensor] = {}
_MAX_STREAM_WORKSPACES = 8  # 48 MiB each


def _need_cuda(*tensors: Optional[torch.Tensor]) -> torch.device:
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError(
                "tilegym_b200 operators run on CUDA tensors only (there is no CPU implementation in this package)"
            )
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise RuntimeError(f"tensors are on different devices: {dev} and {t.device}")
    assert dev is not None
    return dev


def _stream(dev: torch.device) -> int:
    return torch._C._cuda_getCurrentRawStream(dev.index)


def _workspace(dev: torch.device) -> torch.Tensor:
    """Scratch of the current stream.  While a CUDA graph is being captured a
    dedicated per-device buffer is used instead (allocated beforehand, outside
    any capture), so that no allocation or zero-fill is recorded into the graph;
    graphs replayed concurrently on one device would share it and race."""
    nbytes = None
    cap_key = (dev.index, -1)
    if cap_key not in _workspaces:
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError("call a tilegym_b200 GEMM once on this device before capturing it into a CUDA graph")
        nbytes = int(_lib.lib().tg_fp8_gemm_workspace_bytes(0, 0, 0))
        _workspaces[cap_key] = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
    if torch.cuda.is_current_stream_capturing():
        return _workspaces[cap_key]
    key = (dev.index, _stream(dev))
    ws = _workspaces.get(key)
    if ws is None:
        nbytes = nbytes or int(_lib.lib().tg_fp8_gemm_workspace_bytes(0, 0, 0))
        ws = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
        # keep at most _MAX_STREAM_WORKSPACES per-stream buffers: the oldest is dropped (the caching allocator
        # frees it in stream order, so launches still queued on its stream are safe; a stream that comes back
        # simply gets a fresh zeroed buffer)
        live = [k for k in _workspaces if k[1] != -1]
        if len(live) >= _MAX_STREAM_WORKSPACES:
            del _workspaces[live[0]]
        _workspaces[key] = ws
    return ws


def reset_workspaces() -> None:
    """Drops every cached scratch buffer (they are re-created, zeroed, on demand).  Call after
    `_lib.device_status` has reported an expired device-side wait: the launch that gave up may have left
    split-K arrival counters non-zero in the buffer it used."""
    _workspaces.clear()
    _amax_scratch.clear()


# ----------------------------------------------------------------------------
# Block-scaled GEMM and its quantisers (reference: tilegym.suites.unsloth.ops)
# ----------------------------------------------------------------------------
def w8a8_block_fp8_matmul(
    A: torch.Tensor,
    B: torch.Tensor,
    As: torch.Tensor,
    Bs: torch.Tensor,
    block_size: Optional[List[int]] = None,
    output_dtype: torch.dtype = torch.float32,
) -> torch.Tensor:
    """Block-wise FP8 matrix multiplication (W8A8): C = dequant(A) @ dequant(B).T.

    Signature and preconditions of src/tilegym/suites/unsloth/ops.py:240-265 and
    src/tilegym/suites/unsloth/cutile/fp8.py:388-414: A (..., K) e4m3 contiguous,
    B (N, K) e4m3 contiguous, As (..., ceil(K/block_k)) f32, Bs (ceil(N/block_n),
    ceil(K/block_k)) f32; returns a new (..., N) tensor of `output_dtype`.
    Differences: only block_size [128, 128] is implemented, and an output dtype
    outside {f32, f16, bf16} is rejected (the reference silently computes f32).
    """
    if block_size is None:
        block_n, block_k = 128, 128
    else:
        assert len(block_size) == 2
        block_n, block_k = int(block_size[0]), int(block_size[1])
    dev = _need_cuda(A, B, As, Bs)
    assert B.ndim == 2 and B.is_contiguous() and Bs.ndim == 2
    N, K = B.shape
    assert A.shape[-1] == B.shape[-1]
    assert A.shape[:-1] == As.shape[:-1] and A.is_contiguous()
    assert math.ceil(A.shape[-1] / block_k) == As.shape[-1]
    assert math.ceil(N / block_n) == Bs.shape[0]
    assert math.ceil(K / block_k) == Bs.shape[1]
    if output_dtype not in _OUT_DTYPES:
        raise _lib.TileGymB200Error(-6, f"output_dtype {output_dtype} is not one of f32, f16, bf16")
    if (block_n, block_k) != (128, 128):
        raise _lib.TileGymB200Error(-6, f"only block_size [128, 128] is implemented, got [{block_n}, {block_k}]")
    return fp8_block_scaled_mm(A, B, As, Bs, None, output_dtype)


def fp8_block_scaled_mm(
    A: torch.Tensor,
    B: torch.Tensor,
    As: torch.Tensor,
    Bs: torch.Tensor,
    bias: Optional[torch.Tensor] = None,
    out_dtype: torch.dtype = torch.bfloat16,
    out: Optional[torch.Tensor] = None,
    beta: float = 0.0,
) -> torch.Tensor:
    """`w8a8_block_fp8_matmul` (1 x 128 activation scales, 128 x 128 weight scales) with the epilogue a Linear
    needs: C = dequant(A) @ dequant(B).T + bias (+ beta * out), the bias added in fp32 before the one rounding
    to `out_dtype`.  The reference operator (src/tilegym/suites/unsloth/ops.py:240-265) has no bias; this is
    the block-scaled twin of `fp8_scaled_mm`.  With `out` the result is written (or, beta != 0, accumulated)
    in place."""
    dev = _need_cuda(A, B, As, Bs)
    N, K = B.shape
    M = A.numel() // K
    if out is None:
        assert beta == 0.0, "beta needs an `out` tensor to accumulate into"
        if out_dtype not in _OUT_DTYPES:
            raise _lib.TileGymB200Error(-6, f"out_dtype {out_dtype} is not one of f32, f16, bf16")
        out = A.new_empty(A.shape[:-1] + (N,), dtype=out_dtype)
    else:
        assert out.shape == A.shape[:-1] + (N,) and out.is_contiguous()
    if not A.is_contiguous():
        A = A.contiguous()
    if not B.is_contiguous():
        B = B.contiguous()
    if bias is not None and not bias.is_contiguous():
        bias = bias.contiguous()
    ws = _workspace(dev)
    a2, as2, c2 = A.view(M, K), As.contiguous().view(M, -1), out.view(M, N)
    bs2 = Bs.contiguous()
    rc = _lib.lib().tg_fp8_gemm_blockscaled(
        _lib.desc(c2), _lib.desc(a2), _lib.desc(B), _lib.desc(as2), _lib.desc(bs2), 128, 128, _lib.desc(bias),
        float(beta), ws.data_ptr(), ws.numel(), dev.index, _stream(dev),
    )
    _lib.check_rc(rc)
    return out


def ragged_block_scaled_bmm(
    a: torch.Tensor,
    b: torch.Tensor,
    a_scale: torch.Tensor,
    b_scale: torch.Tensor,
    m_indptr: torch.Tensor,
    max_m: int,
    max_m_device: Optional[torch.Tensor] = None,
    transpose_a: bool = False,
    transpose_b: bool = True,
    out_dtype: Optional[torch.dtype] = None,
    bias: Optional[torch.Tensor] = None,
    out: Optional[torch.Tensor] = None,
    beta: float = 0.0,
    row_scale: Optional[torch.Tensor] = None,
    **kwargs,
) -> torch.Tensor:
    """Ragged (grouped) block-scaled FP8 GEMM: rows [m_indptr[q], m_indptr[q+1]) of `a` times weight b[q].T.

    Signature and preconditions of src/tilegym/suites/flashinfer/ops.py:126-158 and
    src/tilegym/suites/flashinfer/cutile/gemm/ragged_block_scaled_bmm.py:497-545: a (total_m, K) e4m3,
    b (Q, N, K) e4m3, a_scale (total_m, ceil(K/128)) f32, b_scale (Q, ceil(N/128), ceil(K/128)) f32, m_indptr
    (Q+1,) int32 on the device; returns a new (total_m, N) tensor (bf16 unless out_dtype says otherwise).
    Differences: segments need no alignment to 128 rows and may be empty; `max_m` / `max_m_device` are accepted
    and not needed (the kernel reads m_indptr itself, nothing is read back to the host); only 128 x 128 scale
    blocks and e4m3 inputs are implemented.  Additions (keyword only in effect): `bias` (Q, N) adds row q to
    the rows of group q, `out` / `beta` write into (accumulate onto) a caller's tensor, `row_scale` (total_m,)
    f32 multiplies every row of the product (a mixture-of-experts routing weight).
    """
    assert transpose_a is False and transpose_b is True, "Only NT layout is supported"
    dev = _need_cuda(a, b, a_scale, b_scale, m_indptr)
    assert a.is_contiguous(), "A matrix must be contiguous"
    assert b.is_contiguous(), "B matrix must be contiguous"
    assert a_scale.is_contiguous(), "A scale matrix must be contiguous"
    assert b_scale.is_contiguous(), "B scale matrix must be contiguous"
    assert m_indptr.is_contiguous(), "m_indptr must be contiguous"
    total_m, K_A = a.shape
    Q, N, K_B = b.shape
    assert K_A == K_B, f"K dimensions must match: {K_A} != {K_B}"
    assert m_indptr.shape[0] == Q + 1, "m_indptr must have Q+1 elements"
    assert a_scale.shape[0] == total_m, "a_scale total_m dimension mismatch"
    assert b_scale.shape[0] == Q, "b_scale Q dimension mismatch"
    if m_indptr.dtype != torch.int32:
        raise _lib.TileGymB200Error(-2, f"m_indptr must be int32, got {m_indptr.dtype}")
    if out_dtype is None:
        out_dtype = torch.bfloat16
    if out_dtype not in _OUT_DTYPES:
        raise _lib.TileGymB200Error(-6, f"out_dtype {out_dtype} is not one of f32, f16, bf16")
    if out is not None:
        assert out.shape == (total_m, N) and out.is_contiguous()
        c = out
    else:
        assert beta == 0.0, "beta needs an `out` tensor to accumulate into"
        c = torch.empty((total_m, N), device=dev, dtype=out_dtype)
    if bias is not None and not bias.is_contiguous():
        bias = bias.contiguous()
    if row_scale is not None:
        assert row_scale.dtype == torch.float32 and row_scale.is_contiguous() and row_scale.numel() >= total_m
    rc = _lib.lib().tg_fp8_gemm_blockscaled_grouped(
        _lib.ref(_lib.desc(c)), _lib.ref(_lib.desc(a)), _lib.ref(_lib.desc(b)), _lib.ref(_lib.desc(a_scale)),
        _lib.ref(_lib.desc(b_scale)), m_indptr.data_ptr(), 128, 128, _lib.desc(bias), float(beta),
        row_scale.data_ptr() if row_scale is not None else 0, dev.index, _stream(dev),
    )
    _lib.check_rc(rc)
    return c


def act_quant(x: torch.Tensor, block_size: int = 128) -> Tuple[torch.Tensor, torch.Tensor]:
    """FP8 block-wise activation quantisation: (y e4m3, s f32 per block).

    Signature of src/tilegym/suites/unsloth/ops.py:223-237; host behaviour of
    src/tilegym/suites/unsloth/cutile/fp8.py:369-385 (x made contiguous, last
    dimension divisible by block_size).
    """
    dev = _need_cuda(x)
    if not x.is_contiguous():
        x = x.contiguous()
    assert x.shape[-1] % block_size == 0
    y = torch.empty_like(x, dtype=_FP8)
    s = x.new_empty(*x.size()[:-1], x.size(-1) // block_size, dtype=torch.float32)
    rc = _lib.lib().tg_act_quant(
        _lib.ref(_lib.desc(y.view(-1))), _lib.ref(_lib.desc(s.view(-1))), _lib.ref(_lib.desc(x.view(-1))),
        int(block_size), dev.index, _stream(dev),
    )
    _lib.check_rc(rc)
    return y, s


def per_token_group_quant_8bit(
    x: torch.Tensor,
    group_size: int,
    eps: float = 1e-10,
    dst_dtype: Optional[torch.dtype] = None,
    column_major_scales: bool = False,
    scale_tma_aligned: bool = False,
    scale_ue8m0: bool = False,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-token group 8-bit quantisation (e4m3 default, e5m2 or int8): (x_q, x_s).

    Signature, preconditions and scale layouts of src/tilegym/suites/flashinfer/ops.py:238-267 and
    src/tilegym/suites/flashinfer/cutile/per_token_group_quant_8bit.py:152-272: row-major scales have shape
    x.shape[:-1] + (H / group_size,); column-major scales are a (tokens, groups) view with strides
    (1, tokens); with scale_tma_aligned the kernel writes into a (groups, ceil4(tokens)) buffer and the
    (tokens, groups) result is returned contiguous, as the reference does.  One kernel serves all layouts
    (it writes the scale through the strides it is given).  eps is applied in x's dtype, like the torch
    reference of the operator's test.
    """
    dev = _need_cuda(x)
    if dst_dtype is None:
        dst_dtype = _FP8
    assert x.shape[-1] % group_size == 0, (
        f"the last dimension of `x` {x.shape[-1]} must be divisible by `group_size` {group_size}"
    )
    assert x.is_contiguous(), "`x` must be contiguous"
    if scale_tma_aligned or scale_ue8m0:
        assert column_major_scales, "scale_tma_aligned or scale_ue8m0 requires column_major_scales=True"
    H = x.shape[-1]
    G = H // group_size
    x2 = x.view(-1, H)
    T = x2.shape[0]
    x_q = torch.empty_like(x, dtype=dst_dtype)
    raw = None
    if column_major_scales:
        assert x.dim() == 2, "column-major scales need a 2-D input [num_tokens, hidden_dim]"
        if scale_tma_aligned:
            raw = torch.empty((G, (T + 3) // 4 * 4), device=dev, dtype=torch.float32)
            x_s = raw[:, :T].t()  # (T, G) view, strides (1, aligned T)
        else:
            x_s = torch.empty((G, T), device=dev, dtype=torch.float32).t()  # (T, G), strides (1, T)
        s2 = x_s
    else:
        x_s = torch.empty(x.shape[:-1] + (G,), device=dev, dtype=torch.float32)
        s2 = x_s.view(T, G)
    eps_in_dtype = float(torch.tensor(eps, dtype=x.dtype))
    if eps_in_dtype == 0.0 and eps > 0:
        eps_in_dtype = float(eps)  # f16: 1e-10 underflows; keep the fp32 value rather than divide 0 by 0
    rc = _lib.lib().tg_per_token_group_quant(
        _lib.ref(_lib.desc(x_q.view(-1, H))), _lib.ref(_lib.desc(s2)), _lib.ref(_lib.desc(x2)), int(group_size),
        eps_in_dtype, 1 if scale_ue8m0 else 0, dev.index, _stream(dev),
    )
    _lib.check_rc(rc)
    if raw is not None:
        x_s = x_s.contiguous()
    return x_q, x_s


def weight_dequant(
    x: torch.Tensor, s: torch.Tensor, block_size: int = 128, dtype: torch.dtype = torch.bfloat16
) -> torch.Tensor:
    """FP8 block-wise weight dequantisation, y = x * s[i//block, j//block].

    Signature of src/tilegym/suites/unsloth/ops.py:199-220; host behaviour of
    src/tilegym/suites/unsloth/cutile/fp8.py:348-367.
    """
    dev = _need_cuda(x, s)
    if not x.is_contiguous():
        x = x.contiguous()
    if not s.is_contiguous():
        s = s.contiguous()
    assert x.dim() == 2 and s.dim() == 2
    y = torch.empty_like(x, dtype=dtype)
    rc = _lib.lib().tg_weight_dequant(
        _lib.ref(_lib.desc(y)), _lib.ref(_lib.desc(x)), _lib.ref(_lib.desc(s)), int(block_size), dev.index,
        _stream(dev),
    )
    _lib.check_rc(rc)
    return y


def weight_quant_block(w: torch.Tensor, block_size: int = 128) -> Tuple[torch.Tensor, torch.Tensor]:
    """128 x 128 block quantisation of a weight (N, K): (q e4m3, s f32 [ceil(N/128), ceil(K/128)]).
    The producer of `Bs`; inverse of `weight_dequant`."""
    dev = _need_cuda(w)
    if not w.is_contiguous():
        w = w.contiguous()
    assert w.dim() == 2
    N, K = w.shape
    q = torch.empty_like(w, dtype=_FP8)
    s = w.new_empty(math.ceil(N / block_size), math.ceil(K / block_size), dtype=torch.float32)
    rc = _lib.lib().tg_weight_quant_block(
        _lib.ref(_lib.desc(q)), _lib.ref(_lib.desc(s)), _lib.ref(_lib.desc(w)), int(block_size), dev.index,
        _stream(dev),
    )
    _lib.check_rc(rc)
    return q, s


# ----------------------------------------------------------------------------
# Per-tensor-scaled GEMM (reference: tilegym.suites.flashinfer.ops.gemm_alpha_beta)
# ----------------------------------------------------------------------------
def _pertensor(
    c2: torch.Tensor,
    a2: torch.Tensor,
    b2: torch.Tensor,
    scale_a: Optional[torch.Tensor],
    scale_b: Optional[torch.Tensor],
    alpha: float,
    bias: Optional[torch.Tensor],
    beta: float,
    dev: torch.device,
    flags: int = 0,
) -> None:
    ws = _workspace(dev)
    rc = _lib.lib().tg_fp8_gemm_pertensor(
        c2 if isinstance(c2, bytes) else _lib.desc(c2), a2 if isinstance(a2, bytes) else _lib.desc(a2), _lib.desc(b2),
        scale_a.data_ptr() if scale_a is not None else 0, scale_b.data_ptr() if scale_b is not None else 0,
        float(alpha), _lib.ref(_lib.desc(bias)), float(beta), ws.data_ptr(), ws.numel(), flags, dev.index,
        _stream(dev),
    )
    _lib.check_rc(rc)


def _scalar_f32(s: Optional[torch.Tensor], dev: torch.device, name: str) -> Optional[torch.Tensor]:
    if s is None:
        return None
    if not torch.is_tensor(s):
        return torch.tensor([float(s)], dtype=torch.float32, device=dev)
    if s.numel() != 1:
        raise _lib.TileGymB200Error(-6, f"{name} must hold exactly one element (per-tensor scale)")
    if s.dtype != torch.float32 or s.device != dev:
        s = s.to(device=dev, dtype=torch.float32)
    return s  # one element: only its address is used


def fp8_scaled_mm(
    A: torch.Tensor,
    B: torch.Tensor,
    scale_a: Optional[torch.Tensor] = None,
    scale_b: Optional[torch.Tensor] = None,
    bias: Optional[torch.Tensor] = None,
    out_dtype: torch.dtype = torch.bfloat16,
    out: Optional[torch.Tensor] = None,
    static_weights: bool = False,
) -> torch.Tensor:
    """C = (scale_a * A) @ (scale_b * B).T + bias, fp32 accumulation, `out_dtype` result.

    A (..., K) e4m3, B (N, K) e4m3 (the layout of nn.Linear.weight), scales are
    one-element fp32 tensors kept on the device (no host synchronisation).
    The reference has no per-tensor-scaled GEMM with a bias vector; this is the
    operator its gemm_alpha_beta (alpha = scale_a * scale_b) approximates.
    `static_weights=True` promises that B is not written by the kernel that runs just before this call on the
    stream (the parameters of a Linear layer): decode-sized calls (at most 64 rows) then start streaming B
    while that kernel is still finishing.  FP8Linear passes it.
    """
    dev = _need_cuda(A, B)
    assert A.dtype == _FP8 and B.dtype == _FP8, "A and B must be float8_e4m3fn"
    assert B.ndim == 2 and A.shape[-1] == B.shape[-1]
    if not A.is_contiguous():
        A = A.contiguous()
    if not B.is_contiguous():
        B = B.contiguous()
    N, K = B.shape
    M = A.numel() // K
    if out is None:
        out = A.new_empty(A.shape[:-1] + (N,), dtype=out_dtype)
    else:
        assert out.shape == A.shape[:-1] + (N,) and out.is_contiguous()
    if bias is not None and not bias.is_contiguous():
        bias = bias.contiguous()
    # contiguous (..., N) / (..., K) tensors are (M, N) / (M, K) matrices: describe them without making views
    _pertensor(_lib.desc2d(out.data_ptr(), M, N, N, out.dtype), _lib.desc2d(A.data_ptr(), M, K, K, A.dtype), B,
               _scalar_f32(scale_a, dev, "scale_a"), _scalar_f32(scale_b, dev, "scale_b"), 1.0, bias, 0.0, dev,
               1 if static_weights else 0)
    return out


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """Stacks a gate and an up projection (weights [I, K] or biases [I], I a multiple of 32) in the row order
    `fp8_scaled_mm_swiglu` expects: 32 gate rows, 32 up rows, 32 gate rows, ...  Done once, at load time."""
    assert gate.shape == up.shape and gate.shape[0] % 32 == 0
    blocks = gate.shape[0] // 32
    g = gate.reshape(blocks, 32, *gate.shape[1:])
    u = up.reshape(blocks, 32, *up.shape[1:])
    return torch.stack((g, u), dim=1).reshape(2 * gate.shape[0], *gate.shape[1:]).contiguous()


def fp8_scaled_mm_swiglu(
    A: torch.Tensor,
    B: torch.Tensor,
    scale_a: Optional[torch.Tensor] = None,
    scale_b: Optional[torch.Tensor] = None,
    bias: Optional[torch.Tensor] = None,
    out_dtype: torch.dtype = torch.bfloat16,
    out: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """silu(gate) * up of a fused gate/up projection, computed in the GEMM epilogue.

    A (..., K) e4m3; B (2*I, K) e4m3 with rows ordered by `interleave_gate_up`; per-tensor scales as in
    `fp8_scaled_mm`; bias (2*I,) in the same row order or None.  Returns (..., I) in bf16 / f16: the
    [..., 2*I] intermediate of matmul + silu_and_mul (src/tilegym/ops/fused_mlp.py:85-107) is never written.
    """
    dev = _need_cuda(A, B)
    assert A.dtype == _FP8 and B.dtype == _FP8, "A and B must be float8_e4m3fn"
    assert B.ndim == 2 and A.shape[-1] == B.shape[-1] and B.shape[0] % 128 == 0
    if out_dtype not in (torch.bfloat16, torch.float16):
        raise _lib.TileGymB200Error(-6, f"out_dtype {out_dtype} is not bf16 or f16")
    if not A.is_contiguous():
        A = A.contiguous()
    if not B.is_contiguous():
        B = B.contiguous()
    N, K = B.shape
    M = A.numel() // K
    if out is None:
        out = A.new_empty(A.shape[:-1] + (N // 2,), dtype=out_dtype)
    else:
        assert out.shape == A.shape[:-1] + (N // 2,) and out.is_contiguous()
    if bias is not None and not bias.is_contiguous():
        bias = bias.contiguous()
    sa, sb = _scalar_f32(scale_a, dev, "scale_a"), _scalar_f32(scale_b, dev, "scale_b")
    rc = _lib.lib().tg_fp8_gemm_pertensor_swiglu(
        _lib.desc2d(out.data_ptr(), M, N // 2, N // 2, out.dtype), _lib.desc2d(A.data_ptr(), M, K, K, A.dtype),
        _lib.desc(B), sa.data_ptr() if sa is not None else 0, sb.data_ptr() if sb is not None else 0, 1.0,
        _lib.desc(bias), dev.index, _stream(dev),
    )
    _lib.check_rc(rc)
    return out


def fp8_scaled_mm_no_alloc(
    A: torch.Tensor,
    B: torch.Tensor,
    scale_a: Optional[torch.Tensor],
    scale_b: Optional[torch.Tensor],
    out: torch.Tensor,
    bias: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """`fp8_scaled_mm` for decode-sized inputs (at most 64 rows) without any
    device allocation, for callers whose memory pool owns the GPU or whose
    loop must not reach the allocator.  Everything is supplied by the caller
    (contiguous e4m3 operands, one-element fp32 device scales or None, the
    output tensor); the split-K scratch is a fixed array inside the library,
    shared by all calls on the device, so do not overlap calls on different
    streams.  Make the first call on a device before capturing any stream."""
    dev = _need_cuda(A, B, out)
    M, K = A.shape
    rc = _lib.lib().tg_fp8_gemm_pertensor_smallm_static(
        _lib.ref(_lib.desc(out)), _lib.ref(_lib.desc(A)), _lib.ref(_lib.desc(B)),
        scale_a.data_ptr() if scale_a is not None else 0, scale_b.data_ptr() if scale_b is not None else 0,
        1.0, _lib.ref(_lib.desc(bias)), 0.0, dev.index, _stream(dev),
    )
    _lib.check_rc(rc)
    return out


def gemm_alpha_beta(
    a: torch.Tensor,
    b: torch.Tensor,
    c: torch.Tensor,
    trans_a: bool = False,
    trans_b: bool = True,
    alpha: float = 1.0,
    beta: float = 0.0,
    num_sms: Optional[int] = None,
    **kwargs,
) -> torch.Tensor:
    """C = alpha * A @ B.T + beta * C, in place, returns `c`.

    Signature of src/tilegym/suites/flashinfer/ops.py:25-55 and
    src/tilegym/suites/flashinfer/cutile/gemm/gemm_alpha_beta.py:336-381 (the
    same contiguity asserts) for the dtype pairs of its test
    (tests/suites/flashinfer/test_flashinfer_gemm_alpha_beta.py:44-53): e4m3 (or e5m2) operands with a
    bf16 / f16 / f32 `c`, and f16 -> f16 / bf16 -> bf16 through the dense tcgen05 kind::f16 path.
    trans_a=False, trans_b=True (a [M, K], b [N, K]) is the native layout; the other settings are served by
    one transposed copy of the operand.  `num_sms` and tuning kwargs (`use_autotune`, `backend`, ...) are
    accepted and ignored: the kernel always uses every SM.  Unlike the reference kernel, `c` is not
    read when beta == 0, so an uninitialised `c` cannot inject NaNs.
    """
    dev = _need_cuda(a, b, c)
    dense16 = a.dtype in (torch.bfloat16, torch.float16) and b.dtype == a.dtype
    if not dense16 and (a.dtype not in _FP8_TYPES or b.dtype != a.dtype):
        raise NotImplementedError(
            "tilegym_b200.gemm_alpha_beta takes float8_e4m3fn, float8_e5m2, bfloat16 or float16 operands (a and b alike)"
        )
    # the kernels read both operands K-major: a as [M, K], b as [N, K]; other layouts cost one transposed copy
    a2 = a.t().contiguous() if trans_a else a
    b2 = b if trans_b else b.t().contiguous()
    M, K = a2.shape
    N, KB = b2.shape
    assert K == KB, "incompatible dimensions"
    assert c.shape == (M, N), "C must have shape [M, N]"
    assert a.is_contiguous(), "A matrix must be contiguous"
    assert b.is_contiguous(), "B matrix must be contiguous"
    assert c.is_contiguous(), "C matrix must be contiguous"
    if dense16:
        rc = _lib.lib().tg_gemm_dense16(_lib.desc(c), _lib.desc(a2), _lib.desc(b2), float(alpha), None, float(beta),
                                        dev.index, _stream(dev))
        _lib.check_rc(rc)
    else:
        _pertensor(c, a2, b2, None, None, alpha, None, beta, dev)
    return c


def matmul(
    a: torch.Tensor,
    b: torch.Tensor,
    trans_a: Optional[bool] = None,
    trans_b: Optional[bool] = None,
    static_persistent: bool = True,
    use_tma: Optional[bool] = None,
    **kwargs,
) -> torch.Tensor:
    """Unscaled FP8 matmul with the reference's signature (src/tilegym/ops/ops.py:715-741).

    e4m3 or e5m2 (a and b alike) and bf16 / f16 inputs.  With trans_b=True, b is [N, K] and is used as is; otherwise
    b is [K, N] and is transposed into the K-major layout the kernel reads (one
    copy).  The result keeps the input dtype like the reference
    (src/tilegym/ops/cutile/matmul.py:446): fp32 accumulation, clamp to the format's
    largest finite value (448 / 57344), cast back.  Pass out_dtype=torch.bfloat16 to skip the narrowing cast.
    Tuning kwargs and `backend=` are accepted and ignored.
    """
    dev = _need_cuda(a, b)
    dense16 = a.dtype in (torch.bfloat16, torch.float16) and b.dtype == a.dtype
    if not dense16 and (a.dtype not in _FP8_TYPES or b.dtype != a.dtype):
        raise NotImplementedError(
            "tilegym_b200.matmul implements float8_e4m3fn, float8_e5m2, bfloat16 and float16 inputs (a and b alike)"
        )
    if trans_a:
        a = a.t()
    if not a.is_contiguous():
        a = a.contiguous()
    bt = b if trans_b else b.t()
    if not bt.is_contiguous():
        bt = bt.contiguous()
    M, K = a.shape
    N = bt.shape[0]
    assert bt.shape[1] == K, "incompatible dimensions"
    out_dtype = kwargs.pop("out_dtype", None)
    if dense16:
        # unquantised path (what the reference's Linear patch calls today): tcgen05 kind::f16, fp32 accumulate,
        # output in the input dtype (src/tilegym/ops/cutile/matmul.py:446)
        c = torch.empty((M, N), dtype=a.dtype if out_dtype is None else out_dtype, device=dev)
        rc = _lib.lib().tg_gemm_dense16(_lib.desc(c), _lib.desc(a), _lib.desc(bt), 1.0, None, 0.0, dev.index,
                                        _stream(dev))
        _lib.check_rc(rc)
        return c
    c = torch.empty((M, N), dtype=torch.float32 if out_dtype is None else out_dtype, device=dev)
    _pertensor(c, a, bt, None, None, 1.0, None, 0.0, dev)
    if out_dtype is None:
        hi = _FP8_MAX[a.dtype]
        return c.clamp_(-hi, hi).to(a.dtype)
    return c


def bmm(
    a: torch.Tensor,
    b: torch.Tensor,
    transpose_a: Optional[bool] = None,
    transpose_b: Optional[bool] = None,
    static_persistent: Optional[bool] = True,
    **kwargs,
) -> torch.Tensor:
    """Batched matmul with the reference's signature (src/tilegym/ops/ops.py:873-896, implementation
    src/tilegym/ops/cutile/bmm.py:290-330): a (Q, M, K) (or (Q, K, M) with transpose_a), b (Q, K, N) (or
    (Q, N, K) with transpose_b), result (Q, M, N) in the input dtype.  bf16 / f16 run the dense tcgen05
    kind::f16 kernel, e4m3 / e5m2 the kind::f8f6f4 one (fp32 accumulation, result clamped and cast back),
    one launch per batch entry on the current stream.  The kernels read K-major operands with 16-byte row
    pitches: (Q, N, K) weights are used as they are, any other layout (and a K that is not a multiple of
    8 / 16 elements) costs one padded / transposed copy.  Tuning kwargs are accepted and ignored."""
    dev = _need_cuda(a, b)
    assert a.dim() == 3 and b.dim() == 3, "bmm takes 3-D tensors"
    dense16 = a.dtype in (torch.bfloat16, torch.float16) and b.dtype == a.dtype
    if not dense16 and (a.dtype not in _FP8_TYPES or b.dtype != a.dtype):
        raise NotImplementedError("tilegym_b200.bmm implements float8, bfloat16 and float16 inputs (a and b alike)")
    am = a.transpose(1, 2) if transpose_a else a      # (Q, M, K)
    bt = b if transpose_b else b.transpose(1, 2)      # (Q, N, K)
    Q, M, K = am.shape
    assert bt.shape[0] == Q and bt.shape[2] == K, "incompatible dimensions"
    N = bt.shape[1]
    kq = 8 if dense16 else 16  # elements per 16 bytes
    if K % kq != 0:
        pad = kq - K % kq  # zero columns add nothing to the products
        if dense16:
            am, bt = torch.nn.functional.pad(am, (0, pad)), torch.nn.functional.pad(bt, (0, pad))
        else:
            am = torch.nn.functional.pad(am.view(torch.uint8), (0, pad)).view(a.dtype)
            bt = torch.nn.functional.pad(bt.view(torch.uint8), (0, pad)).view(a.dtype)
    am, bt = am.contiguous(), bt.contiguous()
    out = torch.empty((Q, M, N), dtype=a.dtype if dense16 else torch.float32, device=dev)
    L, stream = _lib.lib(), _stream(dev)
    for q in range(Q):
        if dense16:
            rc = L.tg_gemm_dense16(_lib.desc(out[q]), _lib.desc(am[q]), _lib.desc(bt[q]), 1.0, None, 0.0, dev.index, stream)
            _lib.check_rc(rc)
        else:
            _pertensor(out[q], am[q], bt[q], None, None, 1.0, None, 0.0, dev)
    if dense16:
        return out
    hi = _FP8_MAX[a.dtype]
    return out.clamp_(-hi, hi).to(a.dtype)


def set_static_weights(on: bool = True) -> bool:
    """Promise (process-wide) that the weight operand of decode-sized GEMMs (at most 64 rows) is never
    written by the kernel that runs just before the GEMM on its stream - true for the parameters of a
    Linear layer.  The small-M kernel is launched with programmatic dependent launch and then starts
    streaming weights while the previous kernel's last thread blocks are still finishing; activations,
    scales, bias and the output are still only touched after the previous kernel has completed.
    Returns the previous setting."""
    return bool(_lib.lib().tg_set_static_weights(1 if on else 0))


def quant_per_tensor(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-tensor e4m3 quantisation: (q, scale) with scale = amax/448 as a
    one-element fp32 device tensor (1.0 for an all-zero input)."""
    dev = _need_cuda(x)
    if x.dtype not in _IN_DTYPES:
        raise _lib.TileGymB200Error(-2, f"quant_per_tensor takes f32, f16 or bf16, got {x.dtype}")
    if not x.is_contiguous():
        x = x.contiguous()
    q = torch.empty_like(x, dtype=_FP8)
    scale = torch.empty(1, dtype=torch.float32, device=dev)
    key = (dev.index, _stream(dev))
    scratch = _amax_scratch.get(key)
    if scratch is None:
        scratch = torch.zeros(1, dtype=torch.int32, device=dev)
        _amax_scratch[key] = scratch
    rc = _lib.lib().tg_quant_pertensor(
        _lib.ref(_lib.desc(q.view(-1))), scale.data_ptr(), _lib.ref(_lib.desc(x.view(-1))), scratch.data_ptr(),
        dev.index, _stream(dev),
    )
    _lib.check_rc(rc)
    return q, scale
