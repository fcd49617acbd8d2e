"""Multi-GPU plumbing: one process per GPU, torch.distributed for the exchange.

The path shards without a data-path collective: a column-parallel quantized dense /
DotGeneral gives every rank the columns [r*N/g, (r+1)*N/g) of the weights, scales and
bias (x is replicated); SDPA gives every rank a contiguous group of KV heads and their
query heads.  The only exchange is the all-gather of the per-rank output slices where a
consumer needs the full vector (NCCL on GPUs, gloo in the CPU tests).
"""
from __future__ import annotations

from typing import Optional, Tuple

import numpy as np


def column_shard(n: int, rank: int, world: int, multiple: int = 16) -> slice:
    """Columns of rank `rank`; shards must be equal and a multiple of `multiple`
    (16 keeps 16-byte alignment of int8 rows; scale blocks along N must not straddle shards)."""
    if n % world != 0 or (n // world) % multiple != 0:
        raise ValueError(f"N={n} cannot be split into {world} equal shards that are multiples of {multiple}")
    w = n // world
    return slice(rank * w, (rank + 1) * w)


def shard_quantized_dense(w: np.ndarray, scales: np.ndarray, bias: Optional[np.ndarray], scale_layout: str,
                          block_size: int, rank: int, world: int):
    """This rank's (weights, scales, bias).  scale_layout: "ref" [K, ceil(N/block)], "channel" [N], "kgroup" [K/g, N]."""
    n = w.shape[1]
    cols = column_shard(n, rank, world, block_size if scale_layout == "ref" else 16)
    if scale_layout == "ref":
        s = scales[:, cols.start // block_size: cols.stop // block_size]
    elif scale_layout == "channel":
        s = scales[cols]
    else:
        s = scales[:, cols]
    return (np.ascontiguousarray(w[:, cols]), np.ascontiguousarray(s),
            None if bias is None else np.ascontiguousarray(bias[cols]))


def kv_head_shard(hq: int, hkv: int, rank: int, world: int) -> Tuple[slice, slice]:
    """(query heads, kv heads) of this rank: whole KV-head groups."""
    if hkv % world != 0:
        raise ValueError(f"{hkv} KV heads cannot be split over {world} ranks")
    per = hkv // world
    group = hq // hkv
    return slice(rank * per * group, (rank + 1) * per * group), slice(rank * per, (rank + 1) * per)


def all_gather_columns(local, group=None):
    """[M, N/g] per rank -> [M, N] on every rank (torch tensors; NCCL or gloo)."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    local = local.contiguous()
    stacked = torch.empty((world,) + tuple(local.shape), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(stacked.view(-1), local.view(-1), group=group)
    # [g, M, N/g] -> [M, g, N/g] -> [M, N]
    return stacked.permute(1, 0, 2).reshape(local.shape[0], world * local.shape[1])
