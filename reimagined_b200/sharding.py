"""Multi-GPU partitioning of the ternary linear (one process per GPU, torch.distributed).

Rows of the activation matrix (tokens / sequences) are independent, so the default partition is
"rows": every rank holds all weights and a contiguous slice of the rows; no collective is needed.
The one shape that is also split by output columns is the largest one (K = N = 16384): rank r owns
the weight rows [r*N/g, (r+1)*N/g) -- in the canonical packing a contiguous run of words, i.e. a
self-contained packed matrix that keeps the GLOBAL weight_scale -- computes y[:, its columns] for all
rows, and one all-gather assembles y.  The reference has no multi-GPU inference at all
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


def gather_columns(y_local, world: int, group=None):
    """All-gathers per-rank [M, N/world] blocks into [M, N] (torch tensors, any backend).  The gathered
    data lands in local memory first and is re-tiled there; no peer loads are involved."""
    import torch
    import torch.distributed as dist
    m, n_local = y_local.shape
    stacked = torch.empty((world, m, n_local), dtype=y_local.dtype, device=y_local.device)
    # list form of all_gather: supported by NCCL and gloo alike; the views alias `stacked`
    dist.all_gather([stacked[r] for r in range(world)], y_local.contiguous(), group=group)
    return stacked.permute(1, 0, 2).reshape(m, world * n_local).contiguous()


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

    def forward(self, x, group=None):
        return gather_columns(self.shard.forward(x), self.world, group)
