"""Per-layer device buffers of the Kitty cache.

Field names, shapes, dtypes and the byte layout of the packed pages are those of
the reference's `KVCache_Layer` (src/kitty/kvcache/utils_kv_per_layer.py:18-95),
so code written against that object keeps working.  Differences: the device is a
constructor argument instead of the literal 'cuda', the identity page tables are
filled with one `arange` instead of a Python loop of single-element writes, and
the object carries the C structs the kernels take.
"""
from __future__ import annotations

import math
from typing import Optional

import numpy as np
import torch

from . import _lib

PAGE_SIZE = 128
SINK = 32


class PagePool:
    """Free list of page rows of one cache tensor (host side).  The reference allocates MAX_BS * ceil(MAX_LEN / 128)
    rows per layer and an identity page table (utils_kv_per_layer.py:48-59); behind the same table a pool can hold
    fewer rows than that worst case and hand them out as sequences grow.  `order` fixes the hand-out order
    (tests pass a permutation so that the mapping is not the identity)."""

    def __init__(self, num_pages: int, order: Optional[list] = None):
        ids = list(range(num_pages)) if order is None else list(order)
        if sorted(ids) != list(range(num_pages)):
            raise ValueError("order must be a permutation of range(num_pages)")
        self.num_pages = num_pages
        self._free = ids[::-1]            # pop() hands out ids in `order`

    def available(self) -> int:
        return len(self._free)

    def alloc(self, n: int) -> list:
        if n > len(self._free):
            raise MemoryError(f"page pool exhausted: {n} pages wanted, {len(self._free)} of {self.num_pages} free")
        return [self._free.pop() for _ in range(n)]

    def free(self, ids) -> None:
        ids = [int(i) for i in ids]
        if any(i < 0 or i >= self.num_pages for i in ids) or set(ids) & set(self._free) or len(set(ids)) != len(ids):
            raise ValueError("freeing a page that is not allocated")
        self._free.extend(reversed(ids))


class KVCache_Layer:
    def __init__(self, MAX_BS: int, MAX_LEN: int, H_KV: int, D: int, D_BOOSTED: int, LOW_BIT: int, HIGH_BIT: int,
                 PAGE_SIZE: int, S: int, device="cuda", num_pages: Optional[int] = None,
                 page_order: Optional[list] = None):
        if (PAGE_SIZE, D, D_BOOSTED, S, LOW_BIT, HIGH_BIT) != (128, 128, 32, 32, 2, 4):
            raise ValueError("kitty_b200 kernels are built for PAGE_SIZE=128, D=128, D_BOOSTED=32, S=32, 2/4 bit; got "
                             f"{(PAGE_SIZE, D, D_BOOSTED, S, LOW_BIT, HIGH_BIT)}")
        dev = torch.device(device)
        if dev.type != "cuda":
            raise ValueError("kitty_b200 buffers live on a CUDA device (there is no CPU path)")
        self.BITS_PER_BYTE = 8
        self.HIGH_BIT, self.LOW_BIT = HIGH_BIT, LOW_BIT
        self.MAX_BS, self.MAX_LEN, self.H_KV, self.D = MAX_BS, MAX_LEN, H_KV, D
        self.D_BOOSTED, self.PAGE_SIZE, self.S = D_BOOSTED, PAGE_SIZE, S
        self.device = dev
        self.MAX_PAGE = math.ceil(MAX_LEN / PAGE_SIZE)
        row = PAGE_SIZE * LOW_BIT // 8                       # bytes of one channel row (keys) / token row (values)
        self.bytes_per_page_K = H_KV * (row * (D + D_BOOSTED) + D)
        self.bytes_per_page_V = H_KV * row * PAGE_SIZE
        # Static mode (num_pages None, the reference's): one row per (sequence, page) and identity tables.
        # Pooled mode: num_pages rows per cache tensor, table entries assigned by ensure_pages() as the
        # sequences grow; the kernels only ever see the tables.
        self.pooled = num_pages is not None
        n = num_pages if self.pooled else MAX_BS * self.MAX_PAGE
        self.pool_K = PagePool(n, page_order) if self.pooled else None
        self.pool_V = PagePool(n, page_order) if self.pooled else None
        self._assigned_K = 0              # pages [0, _assigned_*) of every sequence have a row
        self._assigned_V = 0
        z = dict(device=dev)
        self.KeyCache = torch.zeros((n, self.bytes_per_page_K), dtype=torch.uint8, **z)
        self.KeyCache_metadata = torch.zeros((n, H_KV, D, 2), dtype=torch.float16, **z)
        self.ValueCache = torch.zeros((n, self.bytes_per_page_V), dtype=torch.uint8, **z)
        self.ValueCache_metadata = torch.zeros((n, H_KV, PAGE_SIZE, 2), dtype=torch.float16, **z)
        if self.pooled:
            self.PageTable_K = torch.zeros((MAX_BS, self.MAX_PAGE), dtype=torch.int64, **z)
            self.PageTable_V = torch.zeros((MAX_BS, self.MAX_PAGE), dtype=torch.int64, **z)
        else:
            self.PageTable_K = torch.arange(n, dtype=torch.int64, **z).view(MAX_BS, self.MAX_PAGE).contiguous()
            self.PageTable_V = self.PageTable_K.clone()
        self.PageCount_K = 0
        self.PageCount_V = 0
        self.Sink_Buffer_K = torch.zeros((MAX_BS, H_KV, S, D), dtype=torch.float16, **z)
        self.Sink_Buffer_V = torch.zeros((MAX_BS, H_KV, S, D), dtype=torch.float16, **z)
        self.Sink_Count = 0
        self.Q_Buffer_K = torch.zeros((MAX_BS, H_KV, PAGE_SIZE, D), dtype=torch.float16, **z)
        self.Q_Buffer_V = torch.zeros((MAX_BS, H_KV, PAGE_SIZE, D), dtype=torch.float16, **z)
        self.Q_Buffer_Count_K = 0
        self.Q_Buffer_Count_V = 0
        self.Local_Buffer_V = torch.zeros((MAX_BS, H_KV, PAGE_SIZE, D), dtype=torch.float16, **z)
        self.Local_Count_V = 0
        self.Write_Offset_Local_V = 0
        self.key_states: Optional[torch.Tensor] = None
        self.value_states: Optional[torch.Tensor] = None
        # Ragged batches.  The reference keeps one set of counters for the whole batch (the ints above,
        # utils_kv_per_layer.py:53-80).  When the rows of a batch differ in length, `row_counts` holds one set per
        # row — int32 [MAX_BS, 8] in the field order of struct kitty_counts — with a device mirror for the kernels,
        # and the ints above hold the largest value over the rows.
        self.row_counts: Optional[np.ndarray] = None
        self._row_dev: Optional[torch.Tensor] = None
        self.prompt_lengths = None        # lengths given with a ragged prompt, until quantize_prefill() consumes them
        self._c_layer = None
        self._c_counts = None
        # scratch of the decode kernels, in a one-element box so that the layers of a cache can share one buffer
        # (their calls are serialised on the stream): KittyCache points every layer at the same box
        self._ws_box: list = [None]
        self._workspace_need: dict = {}

    # -- reference surface ------------------------------------------------- #
    def get_total_length(self) -> int:
        if self.row_counts is not None:           # ragged: the longest row
            return int(self.row_lengths().max())
        seqlen_k = self.PageCount_K * self.PAGE_SIZE + self.Sink_Count + self.Q_Buffer_Count_K
        seqlen_v = self.PageCount_V * self.PAGE_SIZE + self.Sink_Count + self.Q_Buffer_Count_V + self.Local_Count_V
        assert seqlen_k == seqlen_v, f"seqlen_K: {seqlen_k}, seqlen_V: {seqlen_v}"
        return seqlen_k

    # -- per-row counters (ragged batches) -------------------------------------- #
    ROW_FIELDS = ("PageCount_K", "PageCount_V", "Sink_Count", "Q_Buffer_Count_K", "Q_Buffer_Count_V", "Local_Count_V",
                  "Write_Offset_Local_V")

    def make_ragged(self) -> None:
        """Switch to per-row counters, every row starting from the shared ones."""
        if self.row_counts is None:
            rc = np.zeros((self.MAX_BS, 8), dtype=np.int32)
            for i, name in enumerate(self.ROW_FIELDS):
                rc[:, i] = getattr(self, name)
            self.row_counts = rc
            self._row_dev = torch.zeros((self.MAX_BS, 8), dtype=torch.int32, device=self.device)
            self.sync_rows()

    def row_lengths(self) -> np.ndarray:
        rc = self.row_counts
        k = rc[:, 0] * self.PAGE_SIZE + rc[:, 2] + rc[:, 3]
        v = rc[:, 1] * self.PAGE_SIZE + rc[:, 2] + rc[:, 4] + rc[:, 5]
        assert (k == v).all(), f"seqlen_K: {k}, seqlen_V: {v}"
        return k

    def sync_rows(self) -> None:
        """Copy the per-row counters to the device mirror (in stream order: a kernel launched afterwards sees them,
        one launched before does not) and refresh the shared ints with the largest value over the rows."""
        self._row_dev.copy_(torch.from_numpy(self.row_counts.copy()))
        for i, name in enumerate(self.ROW_FIELDS):
            setattr(self, name, int(self.row_counts[:, i].max()))

    def row_ptrs(self):
        """(host pointer, device pointer) of the per-row counters for the C entry points."""
        return self.row_counts.ctypes.data, self._row_dev.data_ptr()

    # -- pooled page rows ----------------------------------------------------- #
    def ensure_pages(self, pages_k: int, pages_v: int) -> None:
        """Pooled mode: make sure pages [0, pages_k) / [0, pages_v) of every sequence have a cache row (capped at
        MAX_PAGE).  New table entries are written with one small host-to-device copy per tensor, in stream order
        before the kernels that use them.  A no-op in static mode."""
        if not self.pooled:
            return
        for which, want in (("K", min(pages_k, self.MAX_PAGE)), ("V", min(pages_v, self.MAX_PAGE))):
            have = getattr(self, "_assigned_" + which)
            if want <= have:
                continue
            pool = getattr(self, "pool_" + which)
            ids = pool.alloc((want - have) * self.MAX_BS)
            block = torch.tensor(ids, dtype=torch.int64).view(want - have, self.MAX_BS).t().contiguous()
            getattr(self, "PageTable_" + which)[:, have:want].copy_(block.to(self.device, non_blocking=False))
            setattr(self, "_assigned_" + which, want)

    def release_pages(self) -> None:
        """Pooled mode: give every assigned row back and clear the counters (the sequences are finished)."""
        if self.pooled:
            for which in ("K", "V"):
                have = getattr(self, "_assigned_" + which)
                if have:
                    ids = getattr(self, "PageTable_" + which)[:, :have].t().reshape(-1).tolist()
                    getattr(self, "pool_" + which).free(ids)
                setattr(self, "_assigned_" + which, 0)
        self.PageCount_K = self.PageCount_V = 0
        self.Sink_Count = self.Q_Buffer_Count_K = self.Q_Buffer_Count_V = 0
        self.Local_Count_V = self.Write_Offset_Local_V = 0
        self.key_states = self.value_states = None
        self.row_counts = self._row_dev = self.prompt_lengths = None

    # -- C-ABI views --------------------------------------------------------- #
    def c_layer(self) -> "_lib.KittyLayer":
        """struct kitty_layer pointing at this layer's tensors (built once; the tensors are never reallocated)."""
        if self._c_layer is None:
            L = _lib.KittyLayer()
            L.max_bs, L.max_page, L.h_kv, L.head_dim = self.MAX_BS, self.MAX_PAGE, self.H_KV, self.D
            L.d_boost, L.page_size, L.sink_size, L.reserved = self.D_BOOSTED, self.PAGE_SIZE, self.S, 0
            for name in ("KeyCache", "KeyCache_metadata", "ValueCache", "ValueCache_metadata", "PageTable_K",
                         "PageTable_V", "Sink_Buffer_K", "Sink_Buffer_V", "Q_Buffer_K", "Q_Buffer_V",
                         "Local_Buffer_V"):
                t = getattr(self, name)
                assert t.is_contiguous()
                setattr(L, name, t.data_ptr())
            self._c_layer = L
        return self._c_layer

    def c_counts(self) -> "_lib.KittyCounts":
        """struct kitty_counts with the current counters (one struct per layer, refilled on every call: the C
        entry points copy it before they return)."""
        c = self._c_counts
        if c is None:
            c = self._c_counts = _lib.KittyCounts()
        c.PageCount_K, c.PageCount_V, c.Sink_Count = self.PageCount_K, self.PageCount_V, self.Sink_Count
        c.Q_Buffer_Count_K, c.Q_Buffer_Count_V = self.Q_Buffer_Count_K, self.Q_Buffer_Count_V
        c.Local_Count_V, c.Write_Offset_Local_V, c.reserved = self.Local_Count_V, self.Write_Offset_Local_V, 0
        return c

    def workspace(self, batch: int, h_q: int) -> torch.Tensor:
        """Zero-initialised scratch for the decode kernels, allocated on first use and kept."""
        need = self._workspace_need.get((batch, h_q))
        if need is None:
            need = _lib.lib().kitty_decode_workspace_bytes(batch, self.H_KV, h_q, self.MAX_PAGE)
            if need < 0:
                _lib.check(int(need), "kitty_decode_workspace_bytes")
            self._workspace_need[(batch, h_q)] = need
        if self._workspace is None or self._workspace.numel() < need:
            self._ws_box[0] = torch.zeros(int(need), dtype=torch.uint8, device=self.device)
        return self._workspace

    @property
    def _workspace(self) -> Optional[torch.Tensor]:
        return self._ws_box[0]
