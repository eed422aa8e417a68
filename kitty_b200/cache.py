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

import numpy as np
import torch
from transformers.cache_utils import Cache

from . import _lib
from .layer_state import KVCache_Layer
from .quant_pack import quantize_pack_k, quantize_pack_kv, quantize_pack_v


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
        lengths = (cache_kwargs or {}).get("lengths")
        if lay.Sink_Count == 0 and lay.row_counts is None:
            lay.key_states, lay.value_states = key_states, value_states
            lay.prompt_lengths = None if lengths is None else [int(x) for x in lengths]
            return True
        if key_states.shape[-2] != 1 or lengths is not None:
            # a further piece of the prompt (chunked prefill), possibly of a different length per row
            n = key_states.shape[-2]
            if lay.row_counts is None and (lengths is None or all(int(x) == n for x in lengths)):
                self._append_chunk_uniform(lay, key_states, value_states)
            else:
                self._append_chunk(lay, key_states, value_states, lengths)
            return False
        if lay.row_counts is not None:
            self._append_rows(lay, key_states, value_states, None)
            return False
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

    # -- ragged batches and prompts that arrive in pieces -------------------------------------------- #
    # The reference detects the prompt by Sink_Count == 0 and keeps one set of counters per layer
    # (kvcache/kitty.py:89-95, utils_kv_per_layer.py:53-80): all rows the same length, the prompt in one piece.
    # Here update(..., cache_kwargs={"lengths": [...]}) gives every row its own length (keys / values right-padded
    # to the longest), and a later update() with more than one token appends a further piece of the prompt.  The
    # layer then carries one set of counters per row (KVCache_Layer.row_counts) and the *_rows entry points run.
    @staticmethod
    def _advance_append(rc: np.ndarray, active: np.ndarray, S: int, P: int) -> None:
        """Counters after one appended token per active row (kvcache/kitty.py:102-123, row-wise)."""
        sink_room = active & (rc[:, 2] < S)
        rest = active & ~sink_room
        rc[sink_room, 2] += 1
        rc[rest, 3] += 1
        ring_room = rest & (rc[:, 5] < P)
        evict = rest & ~ring_room
        rc[ring_room, 5] += 1
        rc[evict, 4] += 1
        rc[evict, 6] = (rc[evict, 6] + 1) % P

    @staticmethod
    def _advance_flush(rc: np.ndarray, P: int) -> None:
        """Counters after the flushes that are due (kvcache/kitty.py:201-234, row-wise)."""
        fk, fv = rc[:, 3] == P, rc[:, 4] == P
        rc[fk, 0] += 1
        rc[fk, 3] = 0
        rc[fv, 1] += 1
        rc[fv, 4] = 0

    def _append_rows(self, lay, key_states, value_states, active) -> None:
        """One token per row (rows where `active` is False take none), per-row counters."""
        B = key_states.shape[0]
        if key_states.stride(-1) != 1:
            key_states = key_states.contiguous()
        if value_states.stride(-1) != 1:
            value_states = value_states.contiguous()
        if value_states.dtype != key_states.dtype:
            value_states = value_states.to(key_states.dtype)
        rc = lay.row_counts
        act = np.ones(lay.MAX_BS, dtype=bool) if active is None else np.asarray(active, dtype=bool).copy()
        act[B:] = False
        rc[:, 7] = np.where(act, 0, 1)                       # `reserved` != 0: the kernel skips the row
        assert (rc[act, 3] < lay.PAGE_SIZE).all() and (rc[act, 4] < lay.PAGE_SIZE).all()
        lay.sync_rows()
        host, dev = lay.row_ptrs()
        rc_ = _lib.lib().kitty_append_rows(lay.c_layer(), host, dev, key_states.data_ptr(), value_states.data_ptr(),
                                           _lib.dtype_code(key_states.dtype), key_states.stride(0),
                                           key_states.stride(1), value_states.stride(0), value_states.stride(1), B,
                                           _lib.stream_ptr(key_states.device))
        _lib.check(rc_, "kitty_append_rows")
        self._advance_append(rc, act, lay.S, lay.PAGE_SIZE)
        rc[:, 7] = 0
        lay.sync_rows()

    def _flush_rows(self, lay) -> None:
        rc = lay.row_counts
        if not ((rc[:, 3] == lay.PAGE_SIZE) | (rc[:, 4] == lay.PAGE_SIZE)).any():
            return
        if self.selection != "fused":
            raise ValueError("per-row counters select channels inside the flush kernel (selection='fused')")
        host, dev = lay.row_ptrs()
        rc_ = _lib.lib().kitty_flush_rows(lay.c_layer(), host, dev, lay.MAX_BS, _lib.SELECT_FUSED, self.div_mode,
                                          _lib.stream_ptr(lay.device))
        _lib.check(rc_, "kitty_flush_rows")
        self._advance_flush(rc, lay.PAGE_SIZE)
        lay.sync_rows()
        lay.ensure_pages(lay.PageCount_K + 1, lay.PageCount_V + 1)

    def _append_chunk(self, lay, key_states, value_states, lengths) -> None:
        """A further piece of the prompt: n tokens per row (lengths[b] <= n of them for row b), appended in order.
        The state afterwards is the one n decode steps would have left: tokens pass through the sink, the Q-buffers
        and the value ring, and every Q-buffer that fills up becomes a page.  One append (and, when due, one flush)
        launch per token position."""
        B, _, n, _ = key_states.shape
        lens = np.full(lay.MAX_BS, 0, dtype=np.int64)
        lens[:B] = n if lengths is None else np.asarray([int(x) for x in lengths], dtype=np.int64)
        assert (lens <= n).all() and (lens >= 0).all()
        lay.make_ragged()
        lay.ensure_pages(lay.PageCount_K + 2 + n // lay.PAGE_SIZE, lay.PageCount_V + 2 + n // lay.PAGE_SIZE)
        for t in range(int(lens.max())):
            self._append_rows(lay, key_states[:, :, t:t + 1], value_states[:, :, t:t + 1], lens > t)
            self._flush_rows(lay)

    def _append_chunk_uniform(self, lay, key_states, value_states) -> None:
        """A further piece of the prompt, the same n tokens for every row of a layer whose rows share one set of
        counters: the whole piece in a few launches.  The state afterwards is bit for bit the one n decode steps
        (append, then flush when a Q-buffer is full) leave behind: the tokens are cast to fp16 as the append kernel
        casts them; what fits goes to the sink; keys join the key Q-buffer, and every full 128 tokens of
        [Q-buffer, piece] become a page; values enter the ring of the last 128 tokens at the slot the append kernel
        would have used (oldest token at Write_Offset_Local_V), the tokens they push out join the value Q-buffer, and
        every full 128 of those become a page.  The layer keeps its single set of counters."""
        P, S = lay.PAGE_SIZE, lay.S
        B = key_states.shape[0]
        n = key_states.shape[2]
        # capacity first, before anything is written: the pages this piece completes must exist
        rest = n - min(n, S - lay.Sink_Count)
        new_k = (lay.Q_Buffer_Count_K + rest) // P
        pushed = max(0, rest - (P - lay.Local_Count_V))
        new_v = (lay.Q_Buffer_Count_V + pushed) // P
        if lay.PageCount_K + new_k > lay.MAX_PAGE or lay.PageCount_V + new_v > lay.MAX_PAGE:
            raise _lib.KittyError(_lib.KITTY_E_BADARG, "KittyCache.update: the piece does not fit the cache's pages")
        kh = key_states.to(torch.float16)
        vh = value_states.to(torch.float16)
        take = min(n, S - lay.Sink_Count)
        if take > 0:
            lay.Sink_Buffer_K[:B, :, lay.Sink_Count:lay.Sink_Count + take] = kh[:, :, :take]
            lay.Sink_Buffer_V[:B, :, lay.Sink_Count:lay.Sink_Count + take] = vh[:, :, :take]
            lay.Sink_Count += take
            kh, vh, n = kh[:, :, take:], vh[:, :, take:], n - take
        if n == 0:
            return
        lay.ensure_pages(lay.PageCount_K + n // P + 2, lay.PageCount_V + n // P + 2)
        # keys: [key Q-buffer, piece]
        qk = lay.Q_Buffer_Count_K
        stream_k = torch.cat([lay.Q_Buffer_K[:B, :, :qk], kh], dim=2) if qk else kh
        pages_k, rem_k = divmod(stream_k.shape[2], P)
        # values: first the ring fills up, then every further token pushes the oldest one out
        fill = min(n, P - lay.Local_Count_V)
        if fill > 0:
            lay.Local_Buffer_V[:B, :, lay.Local_Count_V:lay.Local_Count_V + fill] = vh[:, :, :fill]
            lay.Local_Count_V += fill
        m = n - fill
        stream_v, pages_v, rem_v = None, 0, lay.Q_Buffer_Count_V
        if m > 0:
            w = lay.Write_Offset_Local_V
            ring = lay.Local_Buffer_V[:B]
            ordered = torch.roll(ring, shifts=-w, dims=2) if w else ring            # oldest first
            seq = torch.cat([ordered, vh[:, :, fill:]], dim=2)                       # P + m tokens, oldest first
            w = (w + m) % P
            keep = seq[:, :, m:]
            lay.Local_Buffer_V[:B] = torch.roll(keep, shifts=w, dims=2) if w else keep
            lay.Write_Offset_Local_V = w
            qv = lay.Q_Buffer_Count_V
            stream_v = torch.cat([lay.Q_Buffer_V[:B, :, :qv], seq[:, :, :m]], dim=2) if qv else seq[:, :, :m]
            pages_v, rem_v = divmod(stream_v.shape[2], P)
        # the full pages of both streams in one library call
        if pages_k or pages_v:
            quantize_pack_kv(stream_k, 0, pages_k, lay.PageTable_K, lay.PageCount_K, lay.KeyCache,
                             lay.KeyCache_metadata, stream_v if stream_v is not None else stream_k, 0, pages_v,
                             lay.PageTable_V, lay.PageCount_V, lay.ValueCache, lay.ValueCache_metadata, P,
                             lay.D_BOOSTED, selection=self.selection, div_mode=self.div_mode)
            lay.PageCount_K += pages_k
            lay.PageCount_V += pages_v
        if rem_k:
            lay.Q_Buffer_K[:B, :, :rem_k] = stream_k[:, :, pages_k * P:]
        lay.Q_Buffer_Count_K = rem_k
        if stream_v is not None:
            if rem_v:
                lay.Q_Buffer_V[:B, :, :rem_v] = stream_v[:, :, pages_v * P:]
            lay.Q_Buffer_Count_V = rem_v
        lay.ensure_pages(lay.PageCount_K + 1, lay.PageCount_V + 1)

    def _quantize_prefill_ragged(self, lay, k, v) -> None:
        """Prompt with one length per row: each row is partitioned and quantized as a batch of one (the kernels see a
        view of the layer that starts at the row)."""
        B, _, Lmax, _ = k.shape
        lens = lay.prompt_lengths
        assert len(lens) == B and all(0 < L <= Lmax for L in lens)
        P = lay.PAGE_SIZE
        rc = np.zeros((lay.MAX_BS, 8), dtype=np.int32)
        lay.ensure_pages((max(lens) - lay.S) // P + 1, (max(lens) - lay.S) // P + 1)
        for b, L in enumerate(lens):
            sink = min(lay.S, L)
            qbuf_k = (L - sink) % P
            pages_k = (L - sink - qbuf_k) // P
            local_v = min(P, L - sink)
            qbuf_v = (L - sink - local_v) % P
            pages_v = (L - sink - local_v - qbuf_v) // P
            sub = _lib.KittyLayer.from_buffer_copy(lay.c_layer())
            sub.max_bs = 1
            for name in ("Sink_Buffer_K", "Sink_Buffer_V", "Q_Buffer_K", "Q_Buffer_V", "Local_Buffer_V"):
                setattr(sub, name, getattr(lay, name)[b].data_ptr())
            kb_, vb_ = k[b:b + 1], v[b:b + 1]
            rc_ = _lib.lib().kitty_prefill_tails(sub, kb_.data_ptr(), vb_.data_ptr(), _lib.dtype_code(k.dtype),
                                                 kb_.stride(0), kb_.stride(1), kb_.stride(2), vb_.stride(0),
                                                 vb_.stride(1), vb_.stride(2), 1, L, sink, qbuf_k, local_v, qbuf_v,
                                                 _lib.stream_ptr(k.device))
            _lib.check(rc_, "kitty_prefill_tails")
            if pages_k > 0:
                quantize_pack_k(kb_, sink, pages_k, lay.PageTable_K[b:b + 1], 0, lay.KeyCache, lay.KeyCache_metadata, P,
                                lay.D_BOOSTED, selection=self.selection, div_mode=self.div_mode)
            if pages_v > 0:
                quantize_pack_v(vb_, sink, pages_v, lay.PageTable_V[b:b + 1], 0, lay.ValueCache,
                                lay.ValueCache_metadata, P, div_mode=self.div_mode)
            rc[b, :7] = (pages_k, pages_v, sink, qbuf_k, qbuf_v, local_v, 0)
        lay.row_counts = rc
        lay._row_dev = torch.zeros((lay.MAX_BS, 8), dtype=torch.int32, device=lay.device)
        lay.sync_rows()
        lay.prompt_lengths = None
        lay.key_states = lay.value_states = None

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
        if lay.prompt_lengths is not None:
            return self._quantize_prefill_ragged(lay, k, v)
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
        # keys and values in one library call (one launch where the options allow it)
        quantize_pack_kv(k, sink, pages_k, lay.PageTable_K, 0, lay.KeyCache, lay.KeyCache_metadata,
                         v, sink, pages_v, lay.PageTable_V, 0, lay.ValueCache, lay.ValueCache_metadata, P,
                         lay.D_BOOSTED, selection=self.selection, div_mode=self.div_mode)
        lay.PageCount_K += pages_k
        lay.PageCount_V += pages_v
        lay.key_states = None
        lay.value_states = None

    def quantize_decode(self, layer_idx: int = 0) -> None:
        """A Q-buffer that holds a full page becomes the next packed page (keys and values independently)."""
        lay = self.kv_cache[layer_idx]
        if lay.row_counts is not None:
            return self._flush_rows(lay)
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
        if lay0.row_counts is not None:
            raise ValueError("the device-resident decode step keeps one set of counters for the batch; a ragged batch "
                             "uses update() / kitty_attention_forward() / quantize_decode()")
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
