"""kitty_attention_forward with the reference's signature
(src/kitty/kvcache/kernels/kitty_attention.py:403-526): decode attention of one
query token per sequence over [sink | packed pages | Q-buffers | value ring].
One fused pass (split over the sequence, online softmax) instead of the
reference's QK kernel, softmax and SV kernel with logits round-tripping memory.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from . import _lib
from .layer_state import KVCache_Layer

MAX_KV_GROUP = 16


def decode_attention(query: torch.Tensor, kv_cache: KVCache_Layer, num_kv_heads: int, scaling: float, *,
                     out: Optional[torch.Tensor] = None, page_begin: int = 0, page_end: int = -1, flags: int = 3,
                     partial_out: Optional[torch.Tensor] = None, impl: int = 0, exchange=None) -> Optional[torch.Tensor]:
    """Launch the decode-attention kernels.  With `partial_out` (fp32 [B, H_Q, 130]) the un-normalised partial
    result of the selected part of the sequence is written there and nothing is returned.  With `exchange` (a
    seqsplit.PartialExchange) the call reduces this rank's part and its merge kernel combines it with the other
    ranks' parts over peer memory: the returned tensor is the complete result."""
    assert query.is_contiguous(), "Query tensor must be contiguous."
    B, H_Q, t_query, D = query.size()
    assert t_query == 1, "Only decoding step with t_query=1 is supported."
    assert H_Q % num_kv_heads == 0 and num_kv_heads == kv_cache.H_KV
    group = H_Q // num_kv_heads
    assert group <= MAX_KV_GROUP, f"KV_GROUP ({group}) exceeds MAX_KV_GROUP ({MAX_KV_GROUP})."
    if not query.is_cuda:
        raise ValueError("kitty_b200 has no CPU path: the query must be on a CUDA device")
    ws = kv_cache.workspace(B, H_Q)
    out_ptr, out_code = None, _lib.KITTY_F16
    if partial_out is None:
        if out is None:
            out = torch.empty((B, t_query, H_Q, D), dtype=query.dtype, device=query.device)
        assert out.is_contiguous()
        out_ptr, out_code = out.data_ptr(), _lib.dtype_code(out.dtype)
    else:
        assert partial_out.dtype == torch.float32 and partial_out.is_contiguous()
        assert tuple(partial_out.shape) == (B, H_Q, D + 2)
    if kv_cache.row_counts is not None:
        # ragged batch: every row has its own counters (whole sequence of every row; no split over GPUs)
        assert partial_out is None and exchange is None and (page_begin, page_end, flags) == (0, -1, 3)
        host, dev = kv_cache.row_ptrs()
        rc = _lib.lib().kitty_decode_attn_rows(kv_cache.c_layer(), host, dev, query.data_ptr(),
                                               _lib.dtype_code(query.dtype), B, H_Q, float(scaling), out_ptr, out_code,
                                               ws.data_ptr(), ws.numel(), impl, _lib.stream_ptr(query.device))
        _lib.check(rc, "kitty_decode_attn_rows")
        return out
    layer, counts = kv_cache.c_layer(), kv_cache.c_counts()
    if exchange is not None:
        assert partial_out is None and B * H_Q == exchange.rows
        exchange.seq += 1
        rc = _lib.lib().kitty_decode_attn_exchange(layer, counts, query.data_ptr(), _lib.dtype_code(query.dtype), B, H_Q,
                                                   float(scaling), out_ptr, out_code, ws.data_ptr(), ws.numel(),
                                                   page_begin, page_end, flags, impl, exchange.peer_table,
                                                   exchange.rank, exchange.world, exchange.seq,
                                                   exchange.status.data_ptr(), exchange.wait_ns,
                                                   _lib.stream_ptr(query.device))
        _lib.check(rc, "kitty_decode_attn_exchange")
        return out
    rc = _lib.lib().kitty_decode_attn(layer, counts, query.data_ptr(), _lib.dtype_code(query.dtype), B, H_Q,
                                      float(scaling), out_ptr, out_code, ws.data_ptr(), ws.numel(), page_begin,
                                      page_end, flags, None if partial_out is None else partial_out.data_ptr(), impl,
                                      _lib.stream_ptr(query.device))
    _lib.check(rc, "kitty_decode_attn")
    return out


def kitty_attention_forward(module: nn.Module, query: torch.Tensor, kv_cache: KVCache_Layer, scaling: float):
    """Returns (attn_output [B, 1, H_Q, D] in the query's dtype, None)."""
    B, H_Q, t_query, D = query.size()
    assert H_Q == module.num_attention_heads, "H_Q must match num_attention_heads."
    return decode_attention(query, kv_cache, module.num_key_value_heads, scaling), None


def lse_merge(partials: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """Combine fp32 partials [n_parts, B, H_Q, 130] (e.g. all-gathered over ranks) into [B, 1, H_Q, 128]."""
    assert partials.dtype == torch.float32 and partials.is_contiguous() and partials.dim() == 4
    n, B, H_Q, W = partials.shape
    out = torch.empty((B, 1, H_Q, W - 2), dtype=out_dtype, device=partials.device)
    rc = _lib.lib().kitty_lse_merge(partials.data_ptr(), n, B * H_Q, out.data_ptr(), _lib.dtype_code(out_dtype),
                                    _lib.stream_ptr(partials.device))
    _lib.check(rc, "kitty_lse_merge")
    return out


def workspace_status(kv_cache: KVCache_Layer) -> int:
    """Synchronise and read the sticky device status word of the layer's workspace (0 = fine)."""
    import ctypes

    if kv_cache._workspace is None:
        return 0
    st = ctypes.c_int32(0)
    _lib.lib().kitty_workspace_status(kv_cache._workspace.data_ptr(), ctypes.byref(st),
                                      _lib.stream_ptr(kv_cache.device))
    return int(st.value)
