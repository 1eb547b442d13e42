"""Column-parallel (N-sharded) FP8 GEMM across the GPUs of one node.

The reference is single-GPU; this layer is new.  Rank g of G holds the weight
rows [g*N/G, (g+1)*N/G) (quantised BEFORE sharding, so the per-tensor scale is
the global one and results match the 1-GPU GEMM bit for bit), activations are
replicated, every rank computes C_g = A . B_g^T with the same kernels as the
1-GPU path, and one all-gather of the bf16 slabs over NCCL / NVLink completes
the output.  One process per GPU; `torch.distributed` carries the collective.
The index arithmetic is plain Python so it can be tested on CPU ranks (gloo).
"""

from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist


def shard_bounds(N: int, world: int, rank: int, align: int = 128) -> Tuple[int, int]:
    """Rows [lo, hi) of the weight that `rank` owns.  Shards are equal and a
    multiple of `align` rows (the weight-scale block), so block scales shard
    with the rows; N must divide accordingly."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError(f"bad rank {rank} of {world}")
    if N % (world * align) != 0:
        raise ValueError(f"N={N} does not split into {world} shards of a multiple of {align} rows")
    per = N // world
    return rank * per, (rank + 1) * per


def shard_weight(B: torch.Tensor, world: int, rank: int, Bs: Optional[torch.Tensor] = None, block: int = 128):
    """This rank's slab of an already-quantised weight (and of its 128x128 block scales)."""
    lo, hi = shard_bounds(B.shape[0], world, rank, block)
    b = B[lo:hi].contiguous()
    if Bs is None:
        return b
    return b, Bs[lo // block : hi // block].contiguous()


def gathered_view(slabs: torch.Tensor) -> torch.Tensor:
    """[G, M, N/G] gathered slabs -> [M, G, N/G] strided view (no copy):
    view[m, g, j] is C[m, g * N/G + j]."""
    return slabs.permute(1, 0, 2)


def assemble(slabs: torch.Tensor) -> torch.Tensor:
    """[G, M, N/G] -> contiguous [M, N] (one extra pass over the output)."""
    G, M, n = slabs.shape
    return slabs.permute(1, 0, 2).reshape(M, G * n)


class ColumnParallelFP8Gemm:
    """C = (sa*A) . (sb*B)^T with B row-sharded over the ranks of `group`.

    The M rows are processed in `chunks` slabs: the local GEMM of slab c writes straight into this
    rank's part of `out` ([chunks, G, M/chunks, N/G]), and the all-gather of slab c runs on a second
    stream while the GEMM of slab c+1 computes, so the NVLink transfer hides behind the tensor cores
    as far as the bandwidth allows.  Logical element C[m, g*N/G + j] is out[m // mc, g, m % mc, j].
    """

    def __init__(self, B_shard: torch.Tensor, scale_b: torch.Tensor, M: int, group=None,
                 bias_shard: Optional[torch.Tensor] = None, out_dtype: torch.dtype = torch.bfloat16,
                 chunks: int = 1):
        from . import ops  # the CUDA path; imported here so the index helpers above stay importable on CPU

        if M % chunks != 0:
            raise ValueError(f"M={M} is not divisible into {chunks} chunks")
        self._ops = ops
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.B, self.scale_b, self.bias = B_shard, scale_b, bias_shard
        self.chunks, self.mc = chunks, M // chunks
        n = B_shard.shape[0]
        self.out = torch.empty(chunks, self.world, self.mc, n, dtype=out_dtype, device=B_shard.device)
        self.out_slabs = self.out[0] if chunks == 1 else None  # [G, M, N/G] when not chunked
        self._comm_stream = torch.cuda.Stream(device=B_shard.device) if self.world > 1 else None
        self._events = [torch.cuda.Event() for _ in range(chunks)]

    def forward(self, A: torch.Tensor, scale_a: torch.Tensor, gather: bool = True) -> torch.Tensor:
        main = torch.cuda.current_stream(A.device)
        do_gather = gather and self.world > 1
        for c in range(self.chunks):
            mine = self.out[c, self.rank]
            a_c = A[c * self.mc:(c + 1) * self.mc]
            self._ops.fp8_scaled_mm(a_c, self.B, scale_a, self.scale_b, self.bias, mine.dtype, out=mine)
            if do_gather:
                self._events[c].record(main)
                with torch.cuda.stream(self._comm_stream):
                    self._comm_stream.wait_event(self._events[c])
                    dist.all_gather_into_tensor(self.out[c].view(-1), mine.view(-1), group=self.group)
        if do_gather:
            main.wait_stream(self._comm_stream)
        return self.out

    def logical(self) -> torch.Tensor:
        """[chunks, M/chunks, G, N/G] strided view of the gathered result (no copy):
        view[c, i, g, j] = C[c * M/chunks + i, g * N/G + j]."""
        return self.out.permute(0, 2, 1, 3)


class FusedColumnParallelFP8Gemm:
    """Column-parallel GEMM whose kernel also performs the all-gather.

    Every rank owns a full [M, N] output in symmetric (peer-mapped) memory.  The GEMM epilogue of rank g
    stores each finished tile of its slab C[:, g*n:(g+1)*n] into its own buffer and, through bulk tensor
    stores to peer memory over NVLink, into the same columns of every other rank's buffer; the transfer
    runs tile by tile behind the tensor cores, and the result lands directly in row-major [M, N] (the NCCL
    path produces slab-major [G, M, N/G]).  `forward` ends with a symmetric-memory barrier, after which
    every rank may read the whole output.
    """

    def __init__(self, B_shard: torch.Tensor, scale_b: torch.Tensor, M: int, group=None,
                 bias_shard: Optional[torch.Tensor] = None, out_dtype: torch.dtype = torch.bfloat16):
        import ctypes

        import torch.distributed._symmetric_memory as symm_mem

        from . import _lib, ops

        self._lib, self._ops, self._ctypes = _lib, ops, ctypes
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.B, self.scale_b, self.bias = B_shard, scale_b, bias_shard
        self.n = B_shard.shape[0]
        self.M, self.N = M, self.n * self.world
        dev = B_shard.device
        self.out = symm_mem.empty((M, self.N), dtype=out_dtype, device=dev)
        self.handle = symm_mem.rendezvous(self.out, group=self.group)
        esz = self.out.element_size()
        col_off = self.rank * self.n * esz
        # rank g sends to g+1, g+2, ... so that at any moment the ranks' stores fan out to different receivers
        ptrs = self.handle.buffer_ptrs
        peers = [int(ptrs[(self.rank + i) % self.world]) + col_off for i in range(1, self.world)]
        self._peer_arr = (ctypes.c_uint64 * max(1, len(peers)))(*peers)
        self._num_peers = len(peers)
        self.mine = self.out[:, self.rank * self.n:(self.rank + 1) * self.n]  # [M, n] view, row stride N

    def forward(self, A: torch.Tensor, scale_a: torch.Tensor, sync: bool = True) -> torch.Tensor:
        _lib = self._lib
        dev = A.device
        if sync:
            self.handle.barrier()  # nobody is still reading the previous result while peers overwrite it
        rc = _lib.lib().tg_fp8_gemm_pertensor_allgather(
            _lib.ref(_lib.desc(self.mine)), _lib.ref(_lib.desc(A)), _lib.ref(_lib.desc(self.B)),
            scale_a.data_ptr(), self.scale_b.data_ptr(), 1.0, _lib.ref(_lib.desc(self.bias)), self._peer_arr,
            self._num_peers, dev.index, torch.cuda.current_stream(dev).cuda_stream,
        )
        _lib.check_rc(rc)
        if sync:
            self.handle.barrier()  # every rank's stores into this buffer have completed
        return self.out


def reference_gather(shards: List[torch.Tensor]) -> torch.Tensor:
    """What the sharded path must equal: the column-wise concatenation."""
    return torch.cat(shards, dim=-1)
