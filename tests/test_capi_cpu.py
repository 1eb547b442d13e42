"""The C-ABI library without a GPU: it loads, exports every symbol the public
header declares, and rejects wrong calls with the documented codes before it
touches CUDA.  No compute call is made here."""

import ctypes
import os
import re

import pytest
import torch

from conftest import ROOT
from tilegym_b200 import _lib, ops

HEADER = os.path.join(ROOT, "include", "tilegym_b200.h")


def declared_symbols():
    src = open(HEADER).read()
    return re.findall(r"TG_API\s+[\w\s\*]+?\b(tg_\w+)\s*\(", src)


def test_library_is_built_and_loads():
    assert os.path.exists(_lib.LIB_PATH), "run `python -m tilegym_b200.build`"
    assert _lib.lib().tg_version() >= 100


def test_every_declared_symbol_is_exported_and_bound():
    names = declared_symbols()
    assert len(names) >= 10
    handle = ctypes.CDLL(_lib.LIB_PATH)
    for n in names:
        assert hasattr(handle, n), f"{n} is declared in the header but not exported"
        assert n in _lib.SIGNATURES or n.endswith("_static"), f"{n} has no ctypes signature"


def _d(t):
    return _lib.ref(_lib.desc(t))


def test_workspace_size_is_stated():
    assert _lib.lib().tg_fp8_gemm_workspace_bytes(16, 4096, 4096) == (64 << 10) + (48 << 20)


def test_pertensor_argument_checks():
    L = _lib.lib()
    a = torch.zeros(128, 128, dtype=torch.float8_e4m3fn)
    c = torch.zeros(128, 128, dtype=torch.bfloat16)

    def call(C, A, B, bias=None):
        return L.tg_fp8_gemm_pertensor(_d(C), _d(A), _d(B), 0, 0, 1.0, _d(bias), 0.0, 0, 0, 0, 0, 0)

    assert call(c, a, None) == -5 and b"null" in L.tg_last_error_string()
    assert call(c, a.view(torch.uint8), a) == -2
    assert call(c.to(torch.int32), a, a) == -2
    assert call(c, a, torch.zeros(128, 64, dtype=torch.float8_e4m3fn)) == -6  # K mismatch
    assert call(torch.zeros(64, 128, dtype=torch.bfloat16), a, a) == -6  # C shape
    assert call(c, torch.zeros(128, 136, dtype=torch.float8_e4m3fn), torch.zeros(128, 136, dtype=torch.float8_e4m3fn)) == -8  # K % 16
    assert call(c, a, a, torch.zeros(64)) == -6  # bias length
    e5 = torch.zeros(128, 128, dtype=torch.float8_e5m2)
    assert call(c, a, e5) == -2 and b"same 8-bit format" in L.tg_last_error_string()
    assert L.tg_fp8_gemm_pertensor(_d(c), _d(a), _d(a), 0, 0, 1.0, None, 0.0, 0, 0, 6, 0, 0) == -6  # unknown flags
    # empty problems are accepted without a device
    e = torch.zeros(0, 128, dtype=torch.float8_e4m3fn)
    assert call(torch.zeros(0, 128, dtype=torch.bfloat16), e, a) == 0


def test_blockscaled_argument_checks():
    L = _lib.lib()
    a = torch.zeros(128, 256, dtype=torch.float8_e4m3fn)
    c = torch.zeros(128, 128, dtype=torch.float32)
    b = torch.zeros(128, 256, dtype=torch.float8_e4m3fn)
    As, Bs = torch.ones(128, 2), torch.ones(1, 2)

    def call(As_, Bs_, bn=128, bk=128, bias=None):
        return L.tg_fp8_gemm_blockscaled(_d(c), _d(a), _d(b), _d(As_), _d(Bs_), bn, bk, _d(bias), 0.0, 0, 0, 0, 0)

    assert call(As, Bs, 64, 128) == -6 and b"128" in L.tg_last_error_string()
    assert call(torch.ones(128, 3), Bs) == -6
    assert call(As, torch.ones(2, 2)) == -6
    assert call(As.half(), Bs) == -2
    assert call(As, Bs, bias=torch.zeros(64)) == -6  # bias length
    assert call(As, Bs, bias=torch.zeros(128, dtype=torch.int32)) == -2


def test_grouped_blockscaled_argument_checks():
    L = _lib.lib()
    A = torch.zeros(256, 256, dtype=torch.float8_e4m3fn)
    B = torch.zeros(2, 128, 256, dtype=torch.float8_e4m3fn)
    C = torch.zeros(256, 128, dtype=torch.bfloat16)
    As, Bs = torch.zeros(256, 2), torch.zeros(2, 1, 2)
    ind = torch.zeros(3, dtype=torch.int32)

    def call(c=C, a=A, b=B, sa=As, sb=Bs, ptr=None, bn=128, bias=None):
        return L.tg_fp8_gemm_blockscaled_grouped(_d(c), _d(a), _d(b), _d(sa), _d(sb),
                                                 ind.data_ptr() if ptr is None else ptr, bn, 128, _d(bias), 0.0, 0, 0, 0)

    assert call(bias=torch.zeros(128)) == -6  # a grouped bias is [groups, N]

    assert call(b=B[0]) == -6  # B must be 3-D
    assert call(b=torch.zeros(2, 128, 128, dtype=torch.float8_e4m3fn)) == -6  # K mismatch
    assert call(sb=torch.zeros(2, 2, 2)) == -6  # Bs shape
    assert call(sa=torch.zeros(255, 2)) == -6
    assert call(c=torch.zeros(256, 64, dtype=torch.bfloat16)) == -6
    assert call(bn=64) == -6
    assert call(ptr=0) == -5
    assert call(b=B.view(torch.uint8)) == -2
    assert call(a=torch.zeros(0, 256, dtype=torch.float8_e4m3fn), c=torch.zeros(0, 128, dtype=torch.bfloat16),
                sa=torch.zeros(0, 2)) == 0  # nothing to do, no device needed


def test_shard_gemm_allgather_argument_checks():
    L = _lib.lib()
    a = torch.zeros(128, 128, dtype=torch.float8_e4m3fn)
    c = torch.zeros(2, 128, 128, dtype=torch.bfloat16)

    def call(C=c, rank=0, world=2, comm=1):
        return L.tg_shard_gemm_allgather(_d(C), _d(a), _d(a), 0, 0, 1.0, None, rank, world, comm, 0, 0, 0, 0)

    assert call(rank=2) == -6
    assert call(world=3) == -6                      # C_all's first extent is the world size
    assert call(C=c[:, :, :64]) == -6               # NCCL gathers contiguous slabs
    assert call(comm=0) == -5
    assert call(C=c.to(torch.int32)) == -2
    e = torch.zeros(0, 128, dtype=torch.float8_e4m3fn)
    assert L.tg_shard_gemm_allgather(_d(torch.zeros(2, 0, 128, dtype=torch.bfloat16)), _d(e), _d(a), 0, 0, 1.0, None,
                                     1, 2, 1, 0, 0, 0, 0) == 0  # nothing to do, no device or NCCL needed


def test_moe_argument_checks():
    L = _lib.lib()
    ids = torch.zeros(8, 2, dtype=torch.int64)
    buf = torch.zeros(64, dtype=torch.int32)
    p = buf.data_ptr()
    assert L.tg_moe_route(_d(ids.float()), None, 4, p, p, p, p, p, 0, 0) == -2          # ids must be integers
    assert L.tg_moe_route(_d(ids), _d(torch.zeros(8, 3)), 4, p, p, p, p, p, 0, 0) == -6  # weights shaped like ids
    assert L.tg_moe_route(_d(ids), None, 0, p, p, p, p, p, 0, 0) == -6
    assert L.tg_moe_route(_d(ids), None, 4, 0, p, p, p, p, 0, 0) == -5
    a = torch.zeros(8, 256, dtype=torch.float8_e4m3fn)
    a_s = torch.zeros(8, 2)
    out = torch.zeros(16, 256, dtype=torch.float8_e4m3fn)
    out_s = torch.zeros(16, 2)
    assert L.tg_moe_permute_rows(_d(out), _d(out_s), _d(a.view(torch.uint8)), _d(a_s), p, p, 4, 2, 0, 0) == -2
    assert L.tg_moe_permute_rows(_d(out), _d(torch.zeros(16, 3)), _d(a), _d(a_s), p, p, 4, 2, 0, 0) == -6
    assert L.tg_moe_permute_rows(_d(torch.zeros(24, 256, dtype=torch.float8_e4m3fn)), _d(torch.zeros(24, 2)), _d(a),
                                 _d(a_s), p, p, 4, 2, 0, 0) == -6                         # more rows than tokens x top_k
    x = torch.zeros(4, 512, dtype=torch.bfloat16)
    y = torch.zeros(4, 256, dtype=torch.float8_e4m3fn)
    assert L.tg_moe_silu_mul_quant(_d(y), _d(torch.zeros(4, 2)), _d(x), p, 4, 4, 0, 0) == -6  # mode
    assert L.tg_moe_silu_mul_quant(_d(y), _d(torch.zeros(4, 3)), _d(x), p, 4, 0, 0, 0) == -6
    assert L.tg_moe_silu_mul_quant(_d(y), _d(torch.zeros(4, 2)), _d(x.float()), p, 4, 0, 0, 0) == -2
    xq = torch.zeros(4, 256, dtype=torch.bfloat16)
    aq, sq = torch.zeros(8, 256, dtype=torch.float8_e4m3fn), torch.zeros(8, 2)
    assert L.tg_moe_quant_permute_rows(_d(aq), _d(sq), _d(xq.float()), p, 2, 0, 0) == -2          # 16-bit inputs only
    assert L.tg_moe_quant_permute_rows(_d(aq), _d(torch.zeros(8, 3)), _d(xq), p, 2, 0, 0) == -6    # scale shape
    assert L.tg_moe_quant_permute_rows(_d(aq), _d(sq), _d(xq), p, 1, 0, 0) == -6                   # more rows than pairs
    assert L.tg_moe_quant_permute_rows(_d(aq), _d(sq), _d(xq), 0, 2, 0, 0) == -5
    c = torch.zeros(16, 256, dtype=torch.bfloat16)
    assert L.tg_moe_unpermute_sum(_d(torch.zeros(8, 256, dtype=torch.float16)), _d(c), p, 2, 0, 0) == -2
    assert L.tg_moe_unpermute_sum(_d(torch.zeros(4, 256, dtype=torch.bfloat16)), _d(c), p, 2, 0, 0) == -6
    assert L.tg_moe_unpermute_sum(_d(torch.zeros(8, 256, dtype=torch.bfloat16)), _d(c), 0, 2, 0, 0) == -5


def test_quantiser_argument_checks():
    L = _lib.lib()
    x = torch.zeros(4, 256, dtype=torch.bfloat16)
    y = torch.zeros(4, 256, dtype=torch.float8_e4m3fn)
    s = torch.zeros(4, 2)
    assert L.tg_act_quant(_d(y), _d(s), _d(x), 64, 0, 0) == -6
    assert L.tg_act_quant(_d(y), _d(s), _d(x.to(torch.int32)), 128, 0, 0) == -2
    assert L.tg_act_quant(_d(y), _d(torch.zeros(4, 3)), _d(x), 128, 0, 0) == -6
    assert L.tg_weight_dequant(_d(x), _d(y), _d(torch.zeros(1, 1)), 128, 0, 0) == -6  # S shape
    assert L.tg_quant_pertensor(_d(y), 0, _d(x), 0, 0, 0) == -5
    # per-token group quantiser: group size, divisibility, dtypes, scale shape
    sg = torch.zeros(4, 16)
    assert L.tg_per_token_group_quant(_d(y), _d(sg), _d(x), 24, 1e-10, 0, 0, 0) == -6
    assert L.tg_per_token_group_quant(_d(y), _d(torch.zeros(4, 8)), _d(x), 16, 1e-10, 0, 0, 0) == -6
    assert L.tg_per_token_group_quant(_d(y.view(torch.uint8)), _d(sg), _d(x), 16, 1e-10, 0, 0, 0) == -2
    assert L.tg_per_token_group_quant(_d(y), _d(sg.half()), _d(x), 16, 1e-10, 0, 0, 0) == -2
    assert L.tg_per_token_group_quant(_d(y), _d(sg), None, 16, 1e-10, 0, 0, 0) == -5
    assert b"group_size" in L.tg_last_error_string() or True


def test_wait_limit_setter_and_selftest_argument_checks():
    L = _lib.lib()
    prev = L.tg_set_wait_limit_us(1500)
    assert L.tg_set_wait_limit_us(prev) == 1500
    assert L.tg_selftest_wait_timeout(0, 0, 0) == -6          # a limit is required ...
    assert L.tg_selftest_wait_timeout(5_000_000, 0, 0) == -6  # ... and it must be short
    L.tg_reload_env()  # no device needed


def test_ops_refuse_cpu_tensors_instead_of_falling_back():
    a = torch.zeros(16, 128, dtype=torch.float8_e4m3fn)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        ops.fp8_scaled_mm(a, a)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        ops.w8a8_block_fp8_matmul(a, a, torch.ones(16, 1), torch.ones(1, 1))
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        ops.act_quant(torch.zeros(4, 128, dtype=torch.bfloat16))


def test_signatures_match_the_reference_entry_points():
    import inspect

    sig = inspect.signature(ops.w8a8_block_fp8_matmul)
    assert list(sig.parameters) == ["A", "B", "As", "Bs", "block_size", "output_dtype"]
    assert sig.parameters["output_dtype"].default is torch.float32
    sig = inspect.signature(ops.gemm_alpha_beta)
    assert list(sig.parameters)[:8] == ["a", "b", "c", "trans_a", "trans_b", "alpha", "beta", "num_sms"]
    assert sig.parameters["trans_b"].default is True
    assert list(inspect.signature(ops.act_quant).parameters) == ["x", "block_size"]
    assert list(inspect.signature(ops.weight_dequant).parameters) == ["x", "s", "block_size", "dtype"]
    assert list(inspect.signature(ops.ragged_block_scaled_bmm).parameters)[:10] == [
        "a", "b", "a_scale", "b_scale", "m_indptr", "max_m", "max_m_device", "transpose_a", "transpose_b", "out_dtype"]
    assert list(inspect.signature(ops.per_token_group_quant_8bit).parameters) == [
        "x", "group_size", "eps", "dst_dtype", "column_major_scales", "scale_tma_aligned", "scale_ue8m0"]
    assert list(inspect.signature(ops.matmul).parameters)[:6] == ["a", "b", "trans_a", "trans_b", "static_persistent", "use_tma"]


def _plan(kind, M, N, K, sms=148):
    cols, splits = ctypes.c_int32(0), ctypes.c_int32(0)
    rc = _lib.lib().tg_plan_splits(kind, M, N, K, sms, ctypes.byref(cols), ctypes.byref(splits))
    assert rc == 0
    return cols.value, splits.value


def test_plan_splits_follows_the_measured_optima():
    """Tile width / K split of the mid-M kernels (a host-side cost model): the choices that won the split sweeps
    on B200 (148 SMs) for the Llama-3.1-8B and DeepSeek-V2 weight shapes."""
    # per-tensor, single-CTA tiles, M = 128: one wave of narrow tiles unsplit, the long-K shape split in two
    assert _plan(0, 128, 6144, 4096) == (64, 1)     # qkv
    assert _plan(0, 128, 4096, 4096) == (64, 1)     # o_proj
    assert _plan(0, 128, 4096, 14336) == (64, 2)    # down
    assert _plan(0, 128, 28672, 4096)[1] == 1       # gate_up: many tiles, never split
    assert _plan(0, 255, 4096, 14336) == (128, 2)   # two tile rows: wider tiles
    # block-scaled, 128 x 128 tiles
    assert _plan(1, 128, 24576, 1536) == (128, 1)   # more tiles than SMs
    assert _plan(1, 128, 5120, 12288) == (128, 3)
    assert 3 <= _plan(1, 128, 3072, 5120)[1] <= 6   # flat optimum between 3 and 6
    assert _plan(1, 256, 5120, 12288) == (128, 3)
    assert _plan(1, 4096, 5120, 12288) == (128, 1)
    # a split never leaves a unit with fewer than four k-blocks, and a GPU with few SMs splits less
    for K in (512, 1024, 4096, 14336):
        _, s = _plan(1, 128, 1024, K)
        assert s >= 1 and (K // 128) // s >= 4 or s == 1
    assert _plan(1, 128, 5120, 12288, sms=40)[1] == 1


def test_plan_splits_rejects_bad_arguments():
    cols, splits = ctypes.c_int32(0), ctypes.c_int32(0)
    lib = _lib.lib()
    assert lib.tg_plan_splits(2, 128, 128, 128, 148, ctypes.byref(cols), ctypes.byref(splits)) == -6
    assert lib.tg_plan_splits(0, 0, 128, 128, 148, ctypes.byref(cols), ctypes.byref(splits)) == -6
    assert lib.tg_plan_splits(0, 128, 128, 128, 148, None, ctypes.byref(splits)) == -5
