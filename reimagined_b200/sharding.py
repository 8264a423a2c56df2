"""Multi-GPU partitioning of the ternary linear (one process per GPU, torch.distributed).

Rows of the activation matrix (tokens / sequences) are independent, so the default partition is
"rows": every rank holds all weights and a contiguous slice of the rows; no collective is needed.
The one shape that is also split by output columns is the largest one (K = N = 16384): rank r owns
the weight rows [r*N/g, (r+1)*N/g) -- in the canonical packing a contiguous run of words, i.e. a
self-contained packed matrix that keeps the GLOBAL weight_scale -- computes y[:, its columns] for all
rows, and one all-gather assembles y -- or, for prefill-sized batches, no collective at all: the GEMM's epilogue
stores every tile into all GPUs' copies of y over NVLink (PeerOutput + forward_fused below), so the exchange
runs under the tensor-core work.  The reference has no multi-GPU inference at all
(OXN/nsos/src/fabric_v2.cpp is an optional host-staged MPI layer for gradients); this module is the
B200 counterpart of "one GPU lane per model" (OXN/nsos/include/jamba.h:739-747) at g lanes.
"""
from __future__ import annotations

from typing import Tuple

import numpy as np


def row_range(total_rows: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous, balanced slice [lo, hi) of the rows owned by `rank` (earlier ranks take the remainder)."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError("bad world/rank")
    base, rem = divmod(total_rows, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def column_range(out_features: int, world: int, rank: int) -> Tuple[int, int]:
    """Output columns (weight rows) owned by `rank`; requires an even split so the all-gather is regular."""
    if out_features % world != 0:
        raise ValueError("column split needs out_features divisible by the number of ranks")
    per = out_features // world
    return rank * per, (rank + 1) * per


def column_shard_words(words: np.ndarray, out_features: int, in_features: int, world: int, rank: int) -> np.ndarray:
    """The canonical words of the rank's weight rows.  Needs in_features % 16 == 0 so rows start on word
    boundaries; the shard is itself a valid canonical packing of an [N/world, K] matrix."""
    if in_features % 16 != 0:
        raise ValueError("column split needs in_features % 16 == 0")
    lo, hi = column_range(out_features, world, rank)
    wpr = in_features // 16
    return np.ascontiguousarray(words.reshape(out_features, wpr)[lo:hi]).reshape(-1)


def gather_buffer(rows: int, n_local: int, world: int, device="cuda"):
    """The all-gather buffer [world, rows, n_local]: rank r's linear writes its block into slot r of it (no copy
    before the collective), the all-gather fills the other slots in place."""
    import torch
    return torch.empty((world, rows, n_local), dtype=torch.float32, device=device)


def gather_columns_inplace(stacked, rank: int, group=None):
    """In-place all-gather of a buffer whose slot `rank` already holds this rank's block.  NCCL sees
    sendbuff == recvbuff + rank * count and moves nothing locally; data from the other ranks lands in local
    memory (no peer loads afterwards)."""
    import torch.distributed as dist
    world = stacked.shape[0]
    if dist.get_backend(group) == "nccl":
        dist.all_gather_into_tensor(stacked.view(-1), stacked[rank].reshape(-1), group=group)
    else:   # gloo (CPU tests): list form, the views alias `stacked`
        dist.all_gather([stacked[r] for r in range(world)], stacked[rank].clone(), group=group)
    return stacked


def retile(stacked, out=None):
    """[world, rows, n_local] -> [rows, world*n_local].  On CUDA: the library's re-tile kernel (tbl_retile_columns);
    on the CPU (gloo tests) the same index map in torch."""
    import torch
    world, rows, n_local = stacked.shape
    if out is None:
        out = torch.empty((rows, world * n_local), dtype=stacked.dtype, device=stacked.device)
    if stacked.is_cuda:
        from . import capi
        capi.check(capi.lib().tbl_retile_columns(stacked.data_ptr(), world, rows, n_local, out.data_ptr(),
                                                 torch.cuda.current_stream().cuda_stream), "tbl_retile_columns")
    else:
        out.copy_(stacked.permute(1, 0, 2).reshape(rows, world * n_local))
    return out


def gather_columns(y_local, world: int, group=None, rank=None):
    """All-gathers per-rank [M, N/world] blocks into [M, N] (a copy into the gather buffer first: prefer
    ColumnParallelBitLinear.forward, whose linear writes into the buffer directly)."""
    import torch.distributed as dist
    rank = dist.get_rank(group) if rank is None else rank
    m, n_local = y_local.shape
    stacked = gather_buffer(m, n_local, world, y_local.device)
    stacked[rank].copy_(y_local)
    return retile(gather_columns_inplace(stacked, rank, group))


class PeerOutput:
    """An fp32 [rows, n_total] output that exists on every GPU of the group at once and is mapped into every
    process (torch symmetric memory): `pointers[r]` is rank r's copy as seen from this GPU.  Writers use plain
    stores; `barrier()` orders all ranks on the current stream (call it after the writing kernels and before the
    output is read, and again before the buffer is overwritten by a next step)."""

    def __init__(self, rows: int, n_total: int, group=None):
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm
        group = group if group is not None else dist.group.WORLD
        self.tensor = symm.empty((rows, n_total), dtype=torch.float32, device=torch.device("cuda", torch.cuda.current_device()))
        self.handle = symm.rendezvous(self.tensor, group)
        self.rank, self.world = int(self.handle.rank), int(self.handle.world_size)
        self.pointers = [int(p) for p in self.handle.buffer_ptrs]
        self.rows, self.n_total = rows, n_total

    def barrier(self):
        self.handle.barrier()


class ColumnParallelBitLinear:
    """Column-split ternary linear: each rank runs a BitLinear over its slice of the output columns with
    the global weight_scale, then the outputs are all-gathered."""

    def __init__(self, full_layer, world: int, rank: int):
        from .bitlinear import BitLinear
        lo, hi = column_range(full_layer.out_features, world, rank)
        shard = BitLinear(full_layer.in_features, hi - lo, full_layer.use_bias)
        shard.packed_weights = column_shard_words(full_layer.packed_weights, full_layer.out_features,
                                                  full_layer.in_features, world, rank)
        shard.weight_scale = full_layer.weight_scale          # absmean of the WHOLE matrix
        shard.magnitude = np.ascontiguousarray(full_layer.magnitude[lo:hi])
        shard.bias = np.ascontiguousarray(full_layer.bias[lo:hi]) if full_layer.use_bias else full_layer.bias
        shard.exact_linear_mode = full_layer.exact_linear_mode
        shard.precision_bits = full_layer.precision_bits
        shard.rms_mode = full_layer.rms_mode
        self.shard, self.world, self.rank = shard, world, rank

    def to(self, device: str = "cuda"):
        self.shard.to(device)
        return self

    def forward(self, x, group=None, stacked=None, out=None):
        """x [M, K] (replicated) -> y [M, N]: the shard's epilogue writes its [M, N/world] block into slot `rank`
        of the gather buffer, one in-place all-gather, one re-tile pass over local memory."""
        m = x.numel() // self.shard.in_features
        if stacked is None:
            stacked = gather_buffer(m, self.shard.out_features, self.world, x.device)
        self.shard.forward(x, out=stacked[self.rank])
        gather_columns_inplace(stacked, self.rank, group)
        return retile(stacked, out)

    def forward_fused(self, x, peer_out: PeerOutput):
        """x [M, K] (replicated), M > 64 -> y [M, N] in `peer_out.tensor` on every rank: the shard's tcgen05 GEMM
        stores each of its output tiles into all ranks' copies of y (its own last, the peers starting from the
        next rank so that the ranks do not all target the same GPU at once); one barrier across the ranks, no
        all-gather, no re-tile."""
        import ctypes
        import torch
        from . import capi
        sh = self.shard
        if sh._dev is None or sh._dev["w_i8"] is None:
            raise RuntimeError("forward_fused needs the int8 expansion: to('cuda', with_int8=True)")
        k, n = sh.in_features, sh.out_features
        m = x.numel() // k
        if (m, n * self.world) != (peer_out.rows, peer_out.n_total):
            raise ValueError("peer output has the wrong shape")
        order = [(self.rank + 1 + i) % self.world for i in range(self.world)]
        dests = (ctypes.c_void_p * self.world)(*[peer_out.pointers[r] for r in order])
        ws = sh._workspace(m)
        d = sh._dev
        exact = sh.exact_linear_mode
        rc = capi.lib().tbl_linear_forward_scatter(
            x.data_ptr(), d["w_i8"].data_ptr(), sh.weight_scale, m, k, n, sh.precision_bits, 0 if exact else sh.rms_mode,
            None if exact else d["magnitude"].data_ptr(), d["bias"].data_ptr() if sh.use_bias else None,
            dests, self.world, n * self.world, n * self.rank, ws.data_ptr(), ws.numel(),
            torch.cuda.current_stream().cuda_stream)
        capi.check(rc, "tbl_linear_forward_scatter")
        peer_out.barrier()
        return peer_out.tensor
