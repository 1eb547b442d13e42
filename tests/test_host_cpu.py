"""Host-side logic that needs no GPU: shard arithmetic (incl. a world_size-2 gloo run that gathers oracle
slabs), the model-level entry points' signatures and kwargs filtering, FP8Linear construction rules."""

import inspect
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import torch_ref as R
from tilegym_b200 import monkey_patch, sharded
from tilegym_b200.linear import FP8Linear


def test_shard_bounds_and_errors():
    assert sharded.shard_bounds(57344, 8, 0) == (0, 7168)
    assert sharded.shard_bounds(57344, 8, 7) == (50176, 57344)
    assert [sharded.shard_bounds(1024, 4, r) for r in range(4)] == [(0, 256), (256, 512), (512, 768), (768, 1024)]
    with pytest.raises(ValueError):
        sharded.shard_bounds(1000, 8, 0)  # not a multiple of 8 * 128
    with pytest.raises(ValueError):
        sharded.shard_bounds(1024, 4, 4)


def test_shard_weight_and_assemble_roundtrip():
    B = torch.arange(512 * 32, dtype=torch.float32).view(512, 32)
    Bs = torch.arange(4 * 1, dtype=torch.float32).view(4, 1)
    parts = [sharded.shard_weight(B, 2, r, Bs) for r in range(2)]
    assert torch.equal(torch.cat([p[0] for p in parts]), B) and torch.equal(torch.cat([p[1] for p in parts]), Bs)
    A = torch.randn(8, 32)
    slabs = torch.stack([A @ p[0].T for p in parts])  # [G, M, N/G]
    assert torch.equal(sharded.assemble(slabs), A @ B.T)
    view = sharded.gathered_view(slabs)
    assert view.shape == (8, 2, 256) and torch.equal(view.reshape(8, 512), A @ B.T)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _gloo_worker(rank, world, port, M, N, K, result_path):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    a8, b8, sa, sb = R.gen_per_tensor_case(M, N, K, seed=77)  # same seed everywhere: replicated A, global scale
    b_shard = sharded.shard_weight(b8.view(torch.uint8), world, rank).view(torch.float8_e4m3fn)
    mine = R.ref_fp8_scaled_mm(a8, b_shard, sa, sb)  # the oracle stands in for the GPU GEMM on CPU ranks
    slabs = torch.empty(world, M, N // world, dtype=torch.bfloat16)
    dist.all_gather_into_tensor(slabs.view(torch.int32).view(-1), mine.contiguous().view(torch.int32).view(-1))
    if rank == 0:
        full = R.ref_fp8_scaled_mm(a8, b8, sa, sb)
        torch.save({"equal": bool(torch.equal(sharded.assemble(slabs), full))}, result_path)
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_gloo_gather_equals_unsharded(tmp_path):
    """Column-parallel shards + all-gather reproduce the 1-rank result bit for bit (the weight is
    quantised before sharding, so both ranks use the global scale)."""
    path = str(tmp_path / "res.pt")
    mp.spawn(_gloo_worker, args=(2, _free_port(), 16, 512, 256, path), nprocs=2, join=True)
    assert torch.load(path)["equal"]


def test_model_entry_points_keep_reference_signature():
    # keyword lists of src/tilegym/transformers/monkey_patch.py:24-31, 64-72, 118-125, 158-166, 240-246, 293-300,
    # 350-357, 393-400, 437-444, 495-502 and its registry at :555-566
    base = ["rope", "rms_norm", "swiglu", "attn", "model", "use_cutile"]
    ref_params = {
        "llama": base, "mistral": base, "qwen2": base, "phi3": base, "olmo3": base,
        "deepseek_v2": ["rope", "rms_norm", "swiglu", "attn", "moe", "model", "use_cutile"],
        "qwen3_5": ["rope", "rms_norm", "swiglu", "attn", "gated_delta_rule", "model", "use_cutile"],
        "gpt_oss": ["rope", "rms_norm", "swiglu", "attn", "use_cutile"],
        "gemma3": ["rope", "rms_norm", "mlp", "attn", "model", "use_cutile"],
        "olmoe": ["rope", "rms_norm", "attn", "moe", "model", "use_cutile"],
    }
    assert set(monkey_patch.MODEL_TYPE_TO_APPLY_TILEGYM_FN) == set(ref_params)
    for name, fn in monkey_patch.MODEL_TYPE_TO_APPLY_TILEGYM_FN.items():
        params = inspect.signature(fn).parameters
        assert list(params)[:len(ref_params[name])] == ref_params[name], name
        assert list(params)[len(ref_params[name]):] == ["fp8_linear", "fp8_mode"]
        assert params["use_cutile"].default is False and params["fp8_linear"].default is False
        fn()  # the defaults change nothing and need no GPU
    assert inspect.signature(monkey_patch.apply_tilegym_kernel_to_gpt_oss).parameters["swiglu"].default is False
    monkey_patch.apply_tilegym_kernel_to_deepseek_v2(True, True, True, True, False, None, False)  # positional use
    with pytest.raises(TypeError):
        monkey_patch.apply_tilegym_kernel_to_llama(no_such_flag=True)
    # defaults (fp8_linear=False) change nothing and need no GPU
    monkey_patch.apply_tilegym_kernel_to_llama()
    monkey_patch._apply_tilegym_kernel("llama", rope=True, not_a_kwarg=1)
    monkey_patch._apply_tilegym_kernel("no_such_model", rope=True)
    monkey_patch._apply_tilegym_kernel("")


def test_fp8linear_construction_rules():
    lin = FP8Linear(256, 384, bias=True, mode="block")
    assert lin.weight_fp8.shape == (384, 256) and lin.weight_scale.shape == (3, 2)
    assert FP8Linear(64, 10, bias=False).weight_scale.shape == (1,)
    with pytest.raises(ValueError):
        FP8Linear(100, 10)
    with pytest.raises(ValueError):
        FP8Linear(64, 10, mode="block")
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        FP8Linear(64, 10)(torch.zeros(2, 64))
