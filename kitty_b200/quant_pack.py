"""quantize_pack_k / quantize_pack_v with the reference's signatures
(src/kitty/kvcache/kernels/kitty_quant_pack.py:253-356), backed by the CUDA
library.  No copy of the source slice is made: the kernels read the strided
[B, H, T, D] tensor in place, once.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _lib


def _src_args(x: torch.Tensor):
    if x.dim() != 4:
        raise ValueError("expected a [B, H, T, D] tensor")
    if not x.is_cuda:
        raise ValueError("kitty_b200 has no CPU path: the tensor must be on a CUDA device")
    if x.stride(3) != 1:
        x = x.contiguous()
    return x, _lib.dtype_code(x.dtype), x.stride(0), x.stride(1), x.stride(2)


def quantize_pack_k(key_states: torch.Tensor, key_states_t_offset: int, key_states_page_count: int,
                    page_table_k: torch.Tensor, page_offset_k: int, cache: torch.Tensor,
                    cache_metadata: torch.Tensor, page_size: int, d_boost: int, *,
                    channel_idx: Optional[torch.Tensor] = None, selection: str = "fused",
                    div_mode: int = _lib.DIV_IEEE) -> Optional[torch.Tensor]:
    """Quantize and pack key pages.

    selection 'fused' (default): boosted channels are ranked inside the kernel (ties by ascending channel).
    selection 'torch': the index bytes are computed with `abs().mean(-2).topk()` on the device, exactly the
    reference's host prologue (kitty_quant_pack.py:275-288), and supplied to the kernel.
    channel_idx: uint8 [B, H, pages, D] supplied index bytes (overrides `selection`).
    Returns the index bytes used when selection != 'fused', else None.
    """
    B, H, T, D = key_states.shape
    if page_size != 128 or D != 128 or d_boost != 32:
        raise ValueError("kitty_b200 kernels are built for page_size=128, D=128, d_boost=32")
    assert key_states_t_offset + page_size * key_states_page_count <= T
    x, dt, sb, sh, st = _src_args(key_states)
    mode = _lib.SELECT_FUSED
    idx_ptr = None
    if channel_idx is None and selection == "torch":
        pages = x[:, :, key_states_t_offset:key_states_t_offset + page_size * key_states_page_count, :]
        pages = pages.reshape(B, H, key_states_page_count, page_size, D)
        _, top = pages.abs().mean(dim=-2).topk(d_boost, dim=-1)
        channel_idx = torch.full((B, H, key_states_page_count, D), d_boost, dtype=torch.uint8, device=x.device)
        channel_idx.scatter_(-1, top, torch.arange(d_boost, device=x.device, dtype=torch.uint8).expand_as(top))
    elif channel_idx is None and selection != "fused":
        raise ValueError("selection must be 'fused' or 'torch'")
    if channel_idx is not None:
        channel_idx = channel_idx.to(device=x.device, dtype=torch.uint8).contiguous()
        assert tuple(channel_idx.shape) == (B, H, key_states_page_count, D)
        mode, idx_ptr = _lib.SELECT_SUPPLIED, channel_idx.data_ptr()
    assert page_table_k.dtype == torch.int64 and page_table_k.stride(1) == 1
    assert cache.dtype == torch.uint8 and cache.stride(1) == 1 and cache_metadata.is_contiguous()
    rc = _lib.lib().kitty_quant_pack_k(x.data_ptr(), dt, sb, sh, st, B, H, key_states_t_offset, key_states_page_count,
                                       page_table_k.data_ptr(), page_table_k.stride(0), page_offset_k,
                                       cache.data_ptr(), cache.stride(0), cache_metadata.data_ptr(), idx_ptr, mode,
                                       div_mode, _lib.stream_ptr(x.device))
    _lib.check(rc, "kitty_quant_pack_k")
    return channel_idx


def quantize_pack_v(value_states: torch.Tensor, value_states_t_offset: int, value_states_page_count: int,
                    page_table_v: torch.Tensor, page_offset_v: int, cache: torch.Tensor,
                    cache_metadata: torch.Tensor, page_size: int, *, div_mode: int = _lib.DIV_IEEE) -> None:
    """Quantize and pack value pages (per-token 2-bit)."""
    B, H, T, D = value_states.shape
    if page_size != 128 or D != 128:
        raise ValueError("kitty_b200 kernels are built for page_size=128, D=128")
    assert value_states_t_offset + page_size * value_states_page_count <= T
    x, dt, sb, sh, st = _src_args(value_states)
    assert page_table_v.dtype == torch.int64 and page_table_v.stride(1) == 1
    assert cache.dtype == torch.uint8 and cache.stride(1) == 1 and cache_metadata.is_contiguous()
    rc = _lib.lib().kitty_quant_pack_v(x.data_ptr(), dt, sb, sh, st, B, H, value_states_t_offset,
                                       value_states_page_count, page_table_v.data_ptr(), page_table_v.stride(0),
                                       page_offset_v, cache.data_ptr(), cache.stride(0), cache_metadata.data_ptr(),
                                       div_mode, _lib.stream_ptr(x.device))
    _lib.check(rc, "kitty_quant_pack_v")


def quantize_pack_kv(key_states: torch.Tensor, key_states_t_offset: int, key_states_page_count: int,
                     page_table_k: torch.Tensor, page_offset_k: int, key_cache: torch.Tensor,
                     key_cache_metadata: torch.Tensor, value_states: torch.Tensor, value_states_t_offset: int,
                     value_states_page_count: int, page_table_v: torch.Tensor, page_offset_v: int,
                     value_cache: torch.Tensor, value_cache_metadata: torch.Tensor, page_size: int, d_boost: int, *,
                     selection: str = "fused", div_mode: int = _lib.DIV_IEEE) -> None:
    """quantize_pack_k followed by quantize_pack_v as the reference's prefill issues them (kvcache/kitty.py:143, :175),
    in one library call: with 16-bit input, in-kernel selection and IEEE division both run in ONE launch in which the
    value tiles fill the SMs that the last wave of key tiles leaves free.  Results are bit-identical to the two
    separate calls; any other combination of options makes the two calls."""
    B, H, _, D = key_states.shape
    one_call = (selection == "fused" and key_states_page_count > 0 and value_states_page_count > 0
                and key_states.dtype == value_states.dtype and tuple(value_states.shape[:2]) == (B, H))
    if not one_call:
        if key_states_page_count > 0:
            quantize_pack_k(key_states, key_states_t_offset, key_states_page_count, page_table_k, page_offset_k,
                            key_cache, key_cache_metadata, page_size, d_boost, selection=selection, div_mode=div_mode)
        if value_states_page_count > 0:
            quantize_pack_v(value_states, value_states_t_offset, value_states_page_count, page_table_v, page_offset_v,
                            value_cache, value_cache_metadata, page_size, div_mode=div_mode)
        return
    if page_size != 128 or D != 128 or d_boost != 32 or value_states.shape[3] != 128:
        raise ValueError("kitty_b200 kernels are built for page_size=128, D=128, d_boost=32")
    assert key_states_t_offset + page_size * key_states_page_count <= key_states.shape[2]
    assert value_states_t_offset + page_size * value_states_page_count <= value_states.shape[2]
    k, dt, ksb, ksh, kst = _src_args(key_states)
    v, _, vsb, vsh, vst = _src_args(value_states)
    for pt in (page_table_k, page_table_v):
        assert pt.dtype == torch.int64 and pt.stride(1) == 1
    for c, m in ((key_cache, key_cache_metadata), (value_cache, value_cache_metadata)):
        assert c.dtype == torch.uint8 and c.stride(1) == 1 and m.is_contiguous()
    rc = _lib.lib().kitty_quant_pack_kv(k.data_ptr(), v.data_ptr(), dt, ksb, ksh, kst, vsb, vsh, vst, B, H,
                                        key_states_t_offset, key_states_page_count, page_table_k.data_ptr(),
                                        page_table_k.stride(0), page_offset_k, key_cache.data_ptr(),
                                        key_cache.stride(0), key_cache_metadata.data_ptr(), None, _lib.SELECT_FUSED,
                                        value_states_t_offset, value_states_page_count, page_table_v.data_ptr(),
                                        page_table_v.stride(0), page_offset_v, value_cache.data_ptr(),
                                        value_cache.stride(0), value_cache_metadata.data_ptr(), div_mode,
                                        _lib.stream_ptr(k.device))
    _lib.check(rc, "kitty_quant_pack_kv")
