"""The fused GEMM + all-gather kernel on two GPUs (skipped on a single-GPU box): every rank's [M, N] buffer
must equal the 1-GPU oracle result after one call, and agree bit for bit with the NCCL all-gather path."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, path):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dev = torch.device(f"cuda:{rank}")
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from oracle import torch_ref as R
    from tilegym_b200 import _lib, sharded

    M, N, K = 512, 512 * world, 1024
    a8, b8, sa, sb = R.gen_per_tensor_case(M, N, K, 9)
    ref = R.ref_fp8_scaled_mm(a8, b8, sa, sb)
    shard = sharded.shard_weight(b8.view(torch.uint8), world, rank).view(torch.float8_e4m3fn).to(dev)
    fused = sharded.FusedColumnParallelFP8Gemm(shard, sb.to(dev), M)
    out = fused.forward(a8.to(dev), sa.to(dev))
    torch.cuda.synchronize(dev)
    ok_oracle = R.check_tolerance(out, ref)["ok"]
    nccl = sharded.ColumnParallelFP8Gemm(shard, sb.to(dev), M, chunks=2)
    slabs = nccl.forward(a8.to(dev), sa.to(dev))  # [chunks, G, M/chunks, n]
    via_nccl = slabs.permute(0, 2, 1, 3).reshape(M, N)
    same = bool(torch.equal(via_nccl, out))
    _lib.device_status(rank)
    flags = torch.tensor([int(ok_oracle), int(same)], device=dev)
    dist.all_reduce(flags, op=dist.ReduceOp.MIN)
    if rank == 0:
        torch.save({"oracle": int(flags[0]), "same_as_nccl": int(flags[1])}, path)
    dist.barrier()
    dist.destroy_process_group()


def test_fused_allgather_two_gpus(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    path = str(tmp_path / "res.pt")
    mp.spawn(_worker, args=(2, _free_port(), path), nprocs=2, join=True)
    res = torch.load(path)
    assert res["oracle"] == 1 and res["same_as_nccl"] == 1, res


def _worker_c_entry(rank, world, port, path):
    """tg_shard_gemm_allgather with an ncclComm_t made here through NCCL's own C API (ctypes), the way a
    host in another language would hand one over; torch.distributed (gloo) only carries the unique id."""
    import ctypes

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dev = torch.device(f"cuda:{rank}")
    torch.cuda.set_device(dev)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import torch_ref as R
    from tilegym_b200 import _lib, sharded

    nccl = ctypes.CDLL("libnccl.so.2")  # the copy torch has already loaded

    class UniqueId(ctypes.Structure):
        _fields_ = [("internal", ctypes.c_byte * 128)]

    uid = UniqueId()
    if rank == 0:
        assert nccl.ncclGetUniqueId(ctypes.byref(uid)) == 0
    raw = torch.frombuffer(bytearray(bytes(uid)), dtype=torch.uint8).clone()
    dist.broadcast(raw, src=0)
    ctypes.memmove(ctypes.byref(uid), bytes(raw.tolist()), 128)
    comm = ctypes.c_void_p()
    nccl.ncclCommInitRank.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, UniqueId, ctypes.c_int]
    assert nccl.ncclCommInitRank(ctypes.byref(comm), world, uid, rank) == 0

    M, n, K = 384, 256, 1024
    N = n * world
    a8, b8, sa, sb = R.gen_per_tensor_case(M, N, K, 21)
    bias = torch.randn(N, generator=torch.Generator().manual_seed(5)).to(torch.bfloat16)  # the same on every rank
    ref = R.ref_fp8_scaled_mm(a8, b8, sa, sb, bias=bias)
    shard = sharded.shard_weight(b8.view(torch.uint8), world, rank).view(torch.float8_e4m3fn).to(dev)
    bias_shard = bias[rank * n:(rank + 1) * n].contiguous().to(dev)
    a_d, sa_d, sb_d = a8.to(dev), sa.to(dev), sb.to(dev)
    c_all = torch.full((world, M, n), float("nan"), dtype=torch.bfloat16, device=dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    rc = _lib.lib().tg_shard_gemm_allgather(_lib.desc(c_all), _lib.desc(a_d), _lib.desc(shard), sa_d.data_ptr(),
                                            sb_d.data_ptr(), 1.0, _lib.desc(bias_shard), rank, world, comm.value,
                                            0, 0, rank, stream)
    torch.cuda.synchronize(dev)
    _lib.device_status(rank)
    full = c_all.permute(1, 0, 2).reshape(M, N)
    res = R.check_tolerance(full, ref)
    ok = rc == 0 and res["ok"]
    if not ok:
        print(f"rank {rank}: rc={rc} {_lib.lib().tg_last_error_string()} {res}", flush=True)
    nccl.ncclCommDestroy.argtypes = [ctypes.c_void_p]
    nccl.ncclCommDestroy(comm)
    flags = torch.tensor([int(ok)])
    dist.all_reduce(flags, op=dist.ReduceOp.MIN)
    if rank == 0:
        torch.save({"ok": int(flags[0])}, path)
    dist.barrier()
    dist.destroy_process_group()


def test_c_entry_gemm_then_nccl_allgather_two_gpus(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    path = str(tmp_path / "res.pt")
    mp.spawn(_worker_c_entry, args=(2, _free_port(), path), nprocs=2, join=True)
    assert torch.load(path)["ok"] == 1
