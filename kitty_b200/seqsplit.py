"""Sequence-split decode attention: one sequence's packed pages spread over ranks.

The reference has no multi-GPU path (utils_kv_per_layer.py:16).  Here rank r
reduces a contiguous range of the common packed pages; rank 0 also takes the
sink tokens, the last rank the tail (extra key pages, Q-buffers, value ring) —
the last rank is the one that receives appended tokens and performs flushes.
Every rank emits (acc[128], max, sum) per query head, the [B, H_Q, 130] fp32
partials are all-gathered (NCCL over NVLink on GPUs) and merged identically on
every rank.  The exchange is 520 bytes per query head per rank: latency-bound.
Two ways to do it: one NCCL all-gather plus the merge kernel (default), or a
`PartialExchange`, where the merge kernel itself stores the partials into every
rank's buffer over NVLink and waits for the others (kitty_lse_exchange_merge) —
no collective launch at all.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch


def split_pages(n_pages: int, world: int, tail_weight: int = 0) -> list[tuple[int, int]]:
    """Contiguous page ranges [lo, hi) per rank.  With tail_weight = 0 the ranges are balanced (earlier ranks get
    the remainder).  The last rank also reduces the tail of the sequence (fp16 Q-buffers and value ring, up to
    ~290 tokens per head read with far less parallelism than packed pages); tail_weight says how many packed
    pages that work is worth, and the last rank gets that many pages fewer (never less than none)."""
    n_pages, tail_weight = max(n_pages, 0), max(tail_weight, 0)

    def balanced(n, parts):
        base, rem = divmod(n, parts)
        return [base + (1 if r < rem else 0) for r in range(parts)]

    if world == 1:
        return [(0, n_pages)]
    sizes = balanced(n_pages + tail_weight, world)
    if sizes[-1] >= tail_weight:
        sizes[-1] -= tail_weight
    else:                                          # the tail alone outweighs a share: the last rank takes no pages
        sizes = balanced(n_pages, world - 1) + [0]
    out, lo = [], 0
    for sz in sizes:
        out.append((lo, lo + sz))
        lo += sz
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


class PartialExchange:
    """Peer-addressable buffers for kitty_lse_exchange_merge: one symmetric-memory allocation per rank, every
    rank's copy mapped into every process (torch.distributed._symmetric_memory), zeroed once.  `rows` = B * H_Q."""

    def __init__(self, rows: int, device, group=None, wait_ns: int = 0):
        import ctypes

        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm

        from . import _lib

        group = group if group is not None else dist.group.WORLD
        self.rank, self.world, self.rows = dist.get_rank(group), dist.get_world_size(group), rows
        off = ctypes.c_int64(0)
        nbytes = _lib.lib().kitty_lse_exchange_bytes(rows, self.world, ctypes.byref(off))
        if nbytes < 0:
            _lib.check(int(nbytes), "kitty_lse_exchange_bytes")
        self.buf = symm.empty((int(nbytes) + 3) // 4, dtype=torch.float32, device=device)
        self.buf.zero_()
        self.handle = symm.rendezvous(self.buf, group.group_name)
        self.peer_table = int(self.handle.buffer_ptrs_dev)        # device array of `world` buffer addresses
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self.seq = 0
        self.wait_ns = int(wait_ns)                               # 0: the library's default limit (1 s)
        torch.cuda.synchronize(device)
        dist.barrier(group)                                       # every buffer is zero before anyone writes

    @classmethod
    def from_buffers(cls, rows: int, rank: int, buffers: list, wait_ns: int = 0) -> "PartialExchange":
        """An exchange over buffers the caller already holds (`buffers[r]` = rank r's zero-filled exchange buffer as
        addressable from this process, each of kitty_lse_exchange_bytes(rows, len(buffers)) bytes).  No process
        group is touched."""
        self = cls.__new__(cls)
        self.rank, self.world, self.rows = rank, len(buffers), rows
        self.buf, self.handle = buffers[rank], None
        self._buffers = list(buffers)
        dev = buffers[rank].device
        self._table = torch.tensor([b.data_ptr() for b in buffers], dtype=torch.int64, device=dev)
        self.peer_table = self._table.data_ptr()
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self.seq = 0
        self.wait_ns = int(wait_ns)
        return self

    def merge(self, part: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        """part: this rank's fp32 [B, H_Q, 130] partial.  Returns [B, 1, H_Q, 128] (identical on every rank)."""
        from . import _lib

        assert part.dtype == torch.float32 and part.is_contiguous() and part.shape[0] * part.shape[1] == self.rows
        B, H_Q, W = part.shape
        out = torch.empty((B, 1, H_Q, W - 2), dtype=out_dtype, device=part.device)
        self.seq += 1
        rc = _lib.lib().kitty_lse_exchange_merge(part.data_ptr(), self.rows, self.peer_table, self.rank, self.world,
                                                 self.seq, out.data_ptr(), _lib.dtype_code(out_dtype),
                                                 self.status.data_ptr(), self.wait_ns, _lib.stream_ptr(part.device))
        _lib.check(rc, "kitty_lse_exchange_merge")
        return out

    def check(self) -> None:
        """Synchronise and raise if a bounded wait of an earlier merge ran out."""
        from . import _lib

        if int(self.status.item()) != 0:
            raise _lib.KittyError(_lib.KITTY_E_TIMEOUT, "kitty_lse_exchange_merge (a peer's partial did not arrive "
                                                        "within the wait limit; rows it was needed for are unwritten)")


def seq_split_decode(query: torch.Tensor, layer, num_kv_heads: int, scaling: float, *, rank: int, world: int,
                     n_common_pages: int, group=None, exchange: Optional[PartialExchange] = None, tail_weight: int = 0,
                     partial_fn: Optional[Callable] = None, merge_fn: Optional[Callable] = None) -> torch.Tensor:
    """Decode attention of `query` [B, H_Q, 1, D] over a sequence whose common packed pages
    [0, n_common_pages) are split over `world` ranks.  `layer` is this rank's KVCache_Layer (only its own
    page range needs to hold data).  Returns [B, 1, H_Q, D] on every rank.

    partial_fn / merge_fn default to the CUDA library; tests inject host versions."""
    import torch.distributed as dist

    if world == 1 and partial_fn is None:
        from .attention import decode_attention

        return decode_attention(query, layer, num_kv_heads, scaling)      # nothing to combine
    lo, hi = split_pages(n_common_pages, world, tail_weight)[rank]
    if exchange is not None and partial_fn is None:
        from .attention import decode_attention

        # one call: this rank's part, then the merge kernel exchanges the partials over peer memory
        return decode_attention(query, layer, num_kv_heads, scaling, page_begin=lo, page_end=hi,
                                flags=rank_flags(rank, world), exchange=exchange)
    part = (partial_fn or _cuda_partial)(query, layer, num_kv_heads, scaling, lo, hi, rank_flags(rank, world))
    part = part.contiguous()
    if exchange is not None:
        return exchange.merge(part, query.dtype)
    flat = torch.empty((world * part.shape[0],) + tuple(part.shape[1:]), dtype=part.dtype, device=part.device)
    if world > 1:
        try:
            dist.all_gather_into_tensor(flat, part, group=group)      # rank r's rows land at [r*B, (r+1)*B)
        except RuntimeError as e:
            # a rank that never contributed its partial: the collective ends with the process group's timeout
            from . import _lib

            raise _lib.KittyError(_lib.KITTY_E_TIMEOUT, "sequence-split all-gather (a rank's partial did not arrive: "
                                  f"{str(e).splitlines()[0][:160]})") from e
    else:
        flat.copy_(part)
    parts = flat.view((world,) + tuple(part.shape))
    return (merge_fn or _cuda_merge)(parts, query.dtype)


def seq_split_step(cache, key_states: torch.Tensor, value_states: torch.Tensor, query: torch.Tensor, scaling: float, *,
                   rank: int, world: int, exchange: Optional[PartialExchange], layer_idx: int = 0,
                   tail_weight: int = 0) -> torch.Tensor:
    """One decode token of a single-layer cache on one rank of a sequence split, in ONE library call per layer:
    append + this rank's part of the attention + exchange of the partials over peer memory + flush-if-due, all from
    the device-resident step state (KittyCache.plan_step / step_layer / finish_step).  Every rank holds the
    counters and the small fp16 buffers; packed pages are only read inside the rank's own range.  With world == 1
    (exchange None) it is the ordinary one-call step.  For a model, call plan_step once per token and step_layer per
    layer instead."""
    lay = cache.kv_cache[layer_idx]
    lo, hi = split_pages(lay.PageCount_V, world, tail_weight)[rank]
    cache.plan_step(query.shape[0], query.shape[1], page_begin=lo, page_end=hi, flags=rank_flags(rank, world),
                    exchange=exchange if world > 1 else None)
    out = cache.step_layer(layer_idx, key_states, value_states, query, scaling)
    cache.finish_step()
    return out
