"""Resharding of checkpoint tensors between parallel layouts
(cf. fairseq2 ``model_checkpoint/common.py:15-166``).

A tensor is stored as ``splits[tp][dp]``: data-parallel (FSDP) shards are
slices of dim 0, tensor-parallel shards are slices of the parameter's shard
dim. ``reshard_tensor`` rebuilds the slice needed by a target
``(tp_rank, dp_rank)`` of a different ``(tp_size, dp_size)`` while touching
only the source shards that overlap the request.
"""
from __future__ import annotations

from typing import Mapping, Sequence

import torch
from torch import Tensor


def _cat_dp(shards: Sequence[Tensor]) -> Tensor:
    parts = [s for s in shards if s.numel() > 0 or len(shards) == 1]
    if not parts:
        return shards[0]
    return parts[0] if len(parts) == 1 else torch.cat(parts, dim=0)


def reshard_tensor(key: str, splits: Sequence[Sequence[Tensor]], source_shard_sizes: tuple[int, int],
                   target_shard_sizes: tuple[int, int], target_shard_ranks: tuple[int, int],
                   shard_dims: Mapping[str, int]) -> Tensor:
    """``splits[tp][dp]`` -> the tensor of target ``(tp_rank, dp_rank)``.

    ``*_shard_sizes`` are ``(tp_size, dp_size)``. ``shard_dims`` maps parameter
    names to their tensor-parallel dimension; names that are absent are
    replicated over tp. dp (FSDP) sharding is always on dim 0 with
    ``ceil(n / dp)`` rows per rank.
    """
    src_tp, src_dp = source_shard_sizes
    tgt_tp, tgt_dp = target_shard_sizes
    tgt_tp_rank, tgt_dp_rank = target_shard_ranks
    if len(splits) != src_tp or any(len(s) != src_dp for s in splits):
        raise ValueError(f"`splits` of '{key}' must have shape [{src_tp}][{src_dp}].")
    dim = shard_dims.get(key)

    # 1. undo dp sharding per tp shard
    tp_shards = [_cat_dp(dp_splits) for dp_splits in splits]

    # 2. rebuild what the target tp rank owns
    if dim is None or (src_tp == 1 and tgt_tp == 1):
        full_tp = tp_shards[0]
    elif src_tp == tgt_tp:
        full_tp = tp_shards[tgt_tp_rank]
    else:
        if src_tp % tgt_tp == 0:
            # each target shard is the concatenation of consecutive source shards
            f = src_tp // tgt_tp
            full_tp = torch.cat(tp_shards[tgt_tp_rank * f:(tgt_tp_rank + 1) * f], dim=dim)
        elif tgt_tp % src_tp == 0:
            f = tgt_tp // src_tp
            src = tp_shards[tgt_tp_rank // f]
            n = src.shape[dim] // f
            full_tp = src.narrow(dim, (tgt_tp_rank % f) * n, n)
        else:
            whole = torch.cat(tp_shards, dim=dim)
            n = whole.shape[dim] // tgt_tp
            full_tp = whole.narrow(dim, tgt_tp_rank * n, n)

    # 3. apply target dp sharding on dim 0
    if tgt_dp == 1 or full_tp.ndim == 0:
        return full_tp
    d0 = full_tp.shape[0]
    chunk = (d0 + tgt_dp - 1) // tgt_dp
    lo = min(tgt_dp_rank * chunk, d0)
    hi = min(lo + chunk, d0)
    return full_tp[lo:hi]
