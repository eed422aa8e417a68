"""KittyCache: the reference's HF-Transformers cache object
(src/kitty/kvcache/kitty.py:24-258) on top of the CUDA library.

Same surface — `update` (True during prefill), `quantize_prefill`,
`quantize_decode`, `get_seq_length`, `.kv_cache[layer]`, `get_kvcache_kitty` — and
the same state machine.  What changes is how the work is issued: the decode
append is one kernel instead of 2-4 indexed copies, the prefill's five slice
copies are one kernel, key and value flushes share a launch, and the prompt is
quantized in place from the strided projection output without `.contiguous()`
copies.
"""
from __future__ import annotations

from typing import Any, Optional

import torch
from transformers.cache_utils import Cache

from . import _lib
from .layer_state import KVCache_Layer
from .quant_pack import quantize_pack_k, quantize_pack_v


class KittyCache(Cache):
    is_compileable = False

    def __init__(self, config, max_batch_size: int, max_length: int, device="cuda", selection: str = "fused",
                 div_mode: int = _lib.DIV_IEEE, num_pages: Optional[int] = None, page_order=None) -> None:
        try:
            super().__init__(layers=[])
        except TypeError:           # older transformers: Cache.__init__() takes no arguments
            super().__init__()
        text_cfg = config.get_text_config() if hasattr(config, "get_text_config") else config
        self.num_hidden_layers = text_cfg.num_hidden_layers
        self.head_dim = getattr(text_cfg, "head_dim", None) or text_cfg.hidden_size // text_cfg.num_attention_heads
        self.num_key_value_heads = text_cfg.num_key_value_heads
        self.page_size = 128
        self.d_boosted = self.head_dim // 4
        self.sink_length = 32
        self.low_bit = 2
        self.high_bit = 4
        self.selection = selection
        self.div_mode = div_mode
        self._kitty_max_batch, self._kitty_max_length = max_batch_size, max_length
        self.fuse_eager_steps = True      # patched attention modules use plan_step/step_layer/finish_step for decode tokens
        self._step_dev: Optional[torch.Tensor] = None       # device block of the device-resident decode step
        self._step_host = None
        self._step_exchange = None                          # seqsplit.PartialExchange of the token being planned
        self.kv_cache: list[KVCache_Layer] = [
            KVCache_Layer(MAX_BS=max_batch_size, MAX_LEN=max_length, H_KV=self.num_key_value_heads, D=self.head_dim,
                          D_BOOSTED=self.d_boosted, LOW_BIT=self.low_bit, HIGH_BIT=self.high_bit,
                          PAGE_SIZE=self.page_size, S=self.sink_length, device=device, num_pages=num_pages,
                          page_order=page_order)
            for _ in range(self.num_hidden_layers)]
        for lay in self.kv_cache[1:]:
            lay._ws_box = self.kv_cache[0]._ws_box     # one decode workspace for all layers (calls are stream-ordered)

    # ------------------------------------------------------------------ #
    def update(self, key_states: torch.Tensor, value_states: torch.Tensor, layer_idx: int,
               cache_kwargs: Optional[dict[str, Any]] = None) -> bool:
        """Prefill (first call of a layer): remember the prompt's K/V and return True.
        Decode: append one token per sequence and return False."""
        lay = self.kv_cache[layer_idx]
        if lay.Sink_Count == 0:
            lay.key_states, lay.value_states = key_states, value_states
            return True
        assert key_states.shape[-2] == 1 and value_states.shape[-2] == 1, \
            "Decode: key_states and value_states should have sequence length of 1."
        B = key_states.shape[0]
        if key_states.stride(-1) != 1:
            key_states = key_states.contiguous()
        if value_states.stride(-1) != 1:
            value_states = value_states.contiguous()
        if value_states.dtype != key_states.dtype:
            value_states = value_states.to(key_states.dtype)
        sink_full = lay.Sink_Count >= lay.S
        if sink_full:
            assert lay.Q_Buffer_Count_K < lay.PAGE_SIZE
            assert lay.Local_Count_V <= lay.PAGE_SIZE
            if lay.Local_Count_V == lay.PAGE_SIZE:
                assert lay.Q_Buffer_Count_V < lay.PAGE_SIZE
        rc = _lib.lib().kitty_append(lay.c_layer(), lay.c_counts(), key_states.data_ptr(), value_states.data_ptr(),
                                     _lib.dtype_code(key_states.dtype), key_states.stride(0), key_states.stride(1),
                                     value_states.stride(0), value_states.stride(1), B,
                                     _lib.stream_ptr(key_states.device))
        _lib.check(rc, "kitty_append")
        if not sink_full:
            lay.Sink_Count += 1
        else:
            lay.Q_Buffer_Count_K += 1
            if lay.Local_Count_V < lay.PAGE_SIZE:
                lay.Local_Count_V += 1
            else:
                lay.Q_Buffer_Count_V += 1
                lay.Write_Offset_Local_V = (lay.Write_Offset_Local_V + 1) % lay.PAGE_SIZE
        return False

    def quantize_prefill(self, layer_idx: int = 0) -> None:
        lay = self.kv_cache[layer_idx]
        if lay.key_states is None or lay.value_states is None:
            raise ValueError("No key_states or value_states to quantize. Please call update() first.")
        k, v = lay.key_states, lay.value_states
        if k.stride(-1) != 1:
            k = k.contiguous()
        if v.stride(-1) != 1:
            v = v.contiguous()
        if v.dtype != k.dtype:
            v = v.to(k.dtype)
        B, _, L, _ = k.shape
        P = lay.PAGE_SIZE
        sink = min(lay.S, L)
        qbuf_k = (L - sink) % P
        pages_k = (L - sink - qbuf_k) // P
        local_v = min(P, L - sink)
        qbuf_v = (L - sink - local_v) % P
        pages_v = (L - sink - local_v - qbuf_v) // P
        lay.ensure_pages(pages_k + 1, pages_v + 1)          # the prompt's pages and the one the next flush fills
        rc = _lib.lib().kitty_prefill_tails(lay.c_layer(), k.data_ptr(), v.data_ptr(), _lib.dtype_code(k.dtype),
                                            k.stride(0), k.stride(1), k.stride(2), v.stride(0), v.stride(1),
                                            v.stride(2), B, L, sink, qbuf_k, local_v, qbuf_v,
                                            _lib.stream_ptr(k.device))
        _lib.check(rc, "kitty_prefill_tails")
        lay.Sink_Count = sink
        lay.Q_Buffer_Count_K = qbuf_k
        lay.Local_Count_V = local_v
        lay.Q_Buffer_Count_V = qbuf_v
        if pages_k > 0:
            quantize_pack_k(k, sink, pages_k, lay.PageTable_K, 0, lay.KeyCache, lay.KeyCache_metadata, P,
                            lay.D_BOOSTED, selection=self.selection, div_mode=self.div_mode)
            lay.PageCount_K += pages_k
        if pages_v > 0:
            quantize_pack_v(v, sink, pages_v, lay.PageTable_V, 0, lay.ValueCache, lay.ValueCache_metadata, P,
                            div_mode=self.div_mode)
            lay.PageCount_V += pages_v
        lay.key_states = None
        lay.value_states = None

    def quantize_decode(self, layer_idx: int = 0) -> None:
        """A Q-buffer that holds a full page becomes the next packed page (keys and values independently)."""
        lay = self.kv_cache[layer_idx]
        fk = lay.Q_Buffer_Count_K == lay.PAGE_SIZE
        fv = lay.Q_Buffer_Count_V == lay.PAGE_SIZE
        if not (fk or fv):
            return
        if fk and self.selection == "torch":
            quantize_pack_k(lay.Q_Buffer_K, 0, 1, lay.PageTable_K, lay.PageCount_K, lay.KeyCache,
                            lay.KeyCache_metadata, lay.PAGE_SIZE, lay.D_BOOSTED, selection="torch",
                            div_mode=self.div_mode)
            fk_launch = False
        else:
            fk_launch = fk
        if fk_launch or fv:
            rc = _lib.lib().kitty_flush(lay.c_layer(), lay.c_counts(), lay.MAX_BS, int(fk_launch), int(fv),
                                        _lib.SELECT_FUSED, self.div_mode, _lib.stream_ptr(lay.device))
            _lib.check(rc, "kitty_flush")
        if fk:
            lay.PageCount_K += 1
            lay.Q_Buffer_Count_K = 0
        if fv:
            lay.PageCount_V += 1
            lay.Q_Buffer_Count_V = 0
        lay.ensure_pages(lay.PageCount_K + 1, lay.PageCount_V + 1)      # keep the next flush's page assigned

    def reset(self) -> None:
        """Forget every sequence (pooled mode: the page rows go back to the pools).  The reference builds a new
        cache per generate() call instead (latency_benchmarking/benchmark_kitty.py:154-160)."""
        for lay in self.kv_cache:
            lay.release_pages()

    # -- decode step with device-resident state (for CUDA-graph capture) ----------------- #
    # The three calls of a decode step (update, kitty_attention_forward, quantize_decode) pass the
    # counters by value, so their launches differ from token to token.  In this mode the counters and
    # the split-KV plan of the token live in one 160-byte device block that every kernel reads:
    #     cache.plan_step(B, H_Q)            host, once per token (one tiny launch writes the block)
    #     cache.step_layer(i, k, v, q, ...)  per layer; four launches with step-independent arguments
    #     cache.finish_step()                host, once per token: counters := state after the flushes
    # step_layer may be captured in a CUDA graph and replayed for every later token.
    def plan_step(self, batch: int, h_q: int, page_begin: int = 0, page_end: int = -1, flags: int = 3,
                  exchange=None) -> "_lib.KittyStepState":
        """Plan one decode token.  page_begin / page_end / flags select this rank's part of a sequence split over
        GPUs (defaults: the whole sequence); with `exchange` (a seqsplit.PartialExchange) the layers' step_layer
        calls of this token combine the ranks' partials over peer memory, one exchange per layer."""
        import ctypes

        if self.selection != "fused":
            raise ValueError("the device-resident decode step selects channels inside the flush kernel "
                             "(selection='fused')")
        lay0 = self.kv_cache[0]
        ref = self._counter_tuple(lay0)
        for lay in self.kv_cache[1:]:
            if self._counter_tuple(lay) != ref:
                raise ValueError("the layers of the cache are not at the same position")
        if self._step_dev is None:
            self._step_dev = torch.zeros(ctypes.sizeof(_lib.KittyStepState), dtype=torch.uint8, device=lay0.device)
        st = _lib.KittyStepState()
        seq0 = 0
        if exchange is not None:
            seq0 = exchange.seq + 1                      # layer i of this token uses sequence number seq0 + i
            exchange.seq += self.num_hidden_layers
        rc = _lib.lib().kitty_plan_step_split(lay0.c_layer(), lay0.c_counts(), batch, h_q, page_begin, page_end, flags,
                                              seq0, ctypes.byref(st), self._step_dev.data_ptr(),
                                              _lib.stream_ptr(lay0.device))
        _lib.check(rc, "kitty_plan_step_split")
        self._step_host = st
        self._step_exchange = exchange
        return st

    def step_layer(self, layer_idx: int, key_states: torch.Tensor, value_states: torch.Tensor, query: torch.Tensor,
                   scaling: float, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """append + attention + flush-if-due of one layer from the planned state.  key/value [B, H, 1, 128],
        query [B, H_Q, 1, 128] contiguous.  Returns [B, 1, H_Q, 128] in the query's dtype."""
        if self._step_dev is None:
            raise RuntimeError("call plan_step() first")
        lay = self.kv_cache[layer_idx]
        B, H_Q, t_query, D = query.shape
        assert t_query == 1 and query.is_contiguous()
        assert key_states.shape[-2] == 1 and value_states.shape[-2] == 1
        assert key_states.stride(-1) == 1 and value_states.stride(-1) == 1 and key_states.dtype == value_states.dtype
        if out is None:
            out = torch.empty((B, 1, H_Q, D), dtype=query.dtype, device=query.device)
        ws = lay.workspace(lay.MAX_BS, H_Q)
        args = (lay.c_layer(), self._step_dev.data_ptr(), key_states.data_ptr(), value_states.data_ptr(),
                _lib.dtype_code(key_states.dtype), key_states.stride(0), key_states.stride(1), value_states.stride(0),
                value_states.stride(1), query.data_ptr(), _lib.dtype_code(query.dtype), B, H_Q, float(scaling),
                out.data_ptr(), _lib.dtype_code(out.dtype), ws.data_ptr(), ws.numel(), self.div_mode)
        xch = getattr(self, "_step_exchange", None)
        if xch is None:
            rc = _lib.lib().kitty_decode_step(*args, _lib.stream_ptr(query.device))
            _lib.check(rc, "kitty_decode_step")
        else:
            assert B * H_Q == xch.rows
            rc = _lib.lib().kitty_decode_step_exchange(*args, xch.peer_table, xch.rank, xch.world, layer_idx,
                                                       xch.status.data_ptr(), xch.wait_ns,
                                                       _lib.stream_ptr(query.device))
            _lib.check(rc, "kitty_decode_step_exchange")
        return out

    def finish_step(self) -> None:
        st = self._step_host
        if st is None:
            raise RuntimeError("call plan_step() first")
        n = st.next
        for lay in self.kv_cache:
            lay.PageCount_K, lay.PageCount_V, lay.Sink_Count = n.PageCount_K, n.PageCount_V, n.Sink_Count
            lay.Q_Buffer_Count_K, lay.Q_Buffer_Count_V = n.Q_Buffer_Count_K, n.Q_Buffer_Count_V
            lay.Local_Count_V, lay.Write_Offset_Local_V = n.Local_Count_V, n.Write_Offset_Local_V
            lay.ensure_pages(lay.PageCount_K + 1, lay.PageCount_V + 1)
        self._step_host = None
        self._step_exchange = None

    @staticmethod
    def _counter_tuple(lay) -> tuple:
        return (lay.PageCount_K, lay.PageCount_V, lay.Sink_Count, lay.Q_Buffer_Count_K, lay.Q_Buffer_Count_V,
                lay.Local_Count_V, lay.Write_Offset_Local_V)

    def get_seq_length(self, layer_idx: int = 0) -> int:
        return self.kv_cache[layer_idx].get_total_length()

    # -- what transformers' generate() asks of a cache ------------------------------------ #
    def get_mask_sizes(self, cache_position, layer_idx: int = 0):
        query_length = cache_position.shape[0] if hasattr(cache_position, "shape") else int(cache_position)
        return self.get_seq_length(layer_idx) + query_length, 0

    def get_max_cache_shape(self, layer_idx: int = 0) -> int:
        return self._kitty_max_length

    def __len__(self) -> int:
        return self.num_hidden_layers


def get_kvcache_kitty(config, max_batch_size: int, max_length: int, **kwargs) -> KittyCache:
    return KittyCache(config=config, max_batch_size=max_batch_size, max_length=max_length, **kwargs)
