"""Sequence-split decode attention: one sequence's packed pages spread over ranks.

The reference has no multi-GPU path (utils_kv_per_layer.py:16).  Here rank r
reduces a contiguous range of the common packed pages; rank 0 also takes the
sink tokens, the last rank the tail (extra key pages, Q-buffers, value ring) —
the last rank is the one that receives appended tokens and performs flushes.
Every rank emits (acc[128], max, sum) per query head, the [B, H_Q, 130] fp32
partials are all-gathered (NCCL over NVLink on GPUs) and merged identically on
every rank.  The exchange is 520 bytes per query head per rank: latency-bound,
one collective per layer, no peer-memory kernels.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch


def split_pages(n_pages: int, world: int) -> list[tuple[int, int]]:
    """Contiguous, balanced page ranges [lo, hi) per rank (earlier ranks get the remainder)."""
    base, rem = divmod(max(n_pages, 0), world)
    out, lo = [], 0
    for r in range(world):
        hi = lo + base + (1 if r < rem else 0)
        out.append((lo, hi))
        lo = hi
    return out


def rank_flags(rank: int, world: int) -> int:
    """bit0: this rank reduces the sink tokens; bit1: this rank reduces the tail."""
    return (1 if rank == 0 else 0) | (2 if rank == world - 1 else 0)


def _cuda_partial(query, layer, num_kv_heads, scaling, lo, hi, flags):
    from .attention import decode_attention

    B, H_Q, _, D = query.shape
    part = torch.empty((B, H_Q, D + 2), dtype=torch.float32, device=query.device)
    decode_attention(query, layer, num_kv_heads, scaling, page_begin=lo, page_end=hi, flags=flags, partial_out=part)
    return part


def _cuda_merge(parts, dtype):
    from .attention import lse_merge

    return lse_merge(parts, dtype)


def seq_split_decode(query: torch.Tensor, layer, num_kv_heads: int, scaling: float, *, rank: int, world: int,
                     n_common_pages: int, group=None,
                     partial_fn: Optional[Callable] = None, merge_fn: Optional[Callable] = None) -> torch.Tensor:
    """Decode attention of `query` [B, H_Q, 1, D] over a sequence whose common packed pages
    [0, n_common_pages) are split over `world` ranks.  `layer` is this rank's KVCache_Layer (only its own
    page range needs to hold data).  Returns [B, 1, H_Q, D] on every rank.

    partial_fn / merge_fn default to the CUDA library; tests inject host versions."""
    import torch.distributed as dist

    lo, hi = split_pages(n_common_pages, world)[rank]
    part = (partial_fn or _cuda_partial)(query, layer, num_kv_heads, scaling, lo, hi, rank_flags(rank, world))
    part = part.contiguous()
    flat = torch.empty((world * part.shape[0],) + tuple(part.shape[1:]), dtype=part.dtype, device=part.device)
    if world > 1:
        dist.all_gather_into_tensor(flat, part, group=group)      # rank r's rows land at [r*B, (r+1)*B)
    else:
        flat.copy_(part)
    parts = flat.view((world,) + tuple(part.shape))
    return (merge_fn or _cuda_merge)(parts, query.dtype)
