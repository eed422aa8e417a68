"""Host-side state machine of KittyCache, run on CPU against a recording stand-in
for the CUDA library: the counters must follow the oracle's (i.e. the
reference's) transitions and the right entry points must be called."""
import types

import numpy as np
import pytest
import torch

from oracle import kitty_oracle as ko
from tests.helpers import COUNTERS


class FakeLayer:
    """Counters and geometry only; no device buffers."""

    def __init__(self, MAX_BS, MAX_LEN, H_KV, D, D_BOOSTED, LOW_BIT, HIGH_BIT, PAGE_SIZE, S, device="cuda",
                 num_pages=None, page_order=None):
        self.ensured = []
        self.MAX_BS, self.MAX_LEN, self.H_KV, self.D, self.D_BOOSTED = MAX_BS, MAX_LEN, H_KV, D, D_BOOSTED
        self.PAGE_SIZE, self.S, self.device = PAGE_SIZE, S, torch.device("cpu")
        self.MAX_PAGE = -(-MAX_LEN // PAGE_SIZE)
        for c in COUNTERS:
            setattr(self, c, 0)
        self.key_states = self.value_states = None
        self._ws_box = [None]
        self.row_counts = self.prompt_lengths = None
        for n in ("PageTable_K", "PageTable_V", "KeyCache", "KeyCache_metadata", "ValueCache", "ValueCache_metadata",
                  "Q_Buffer_K", "Q_Buffer_V"):
            setattr(self, n, None)

    def c_layer(self):
        return None

    # the per-row counter helpers are plain host code: borrow them from the real layer class
    from kitty_b200.layer_state import KVCache_Layer as _Real
    ROW_FIELDS = _Real.ROW_FIELDS
    make_ragged, row_lengths, sync_rows, row_ptrs = _Real.make_ragged, _Real.row_lengths, _Real.sync_rows, _Real.row_ptrs

    def ensure_pages(self, pages_k, pages_v):
        self.ensured.append((pages_k, pages_v))

    def c_counts(self):
        return tuple(getattr(self, c) for c in COUNTERS)

    def get_total_length(self):
        k = self.PageCount_K * 128 + self.Sink_Count + self.Q_Buffer_Count_K
        v = self.PageCount_V * 128 + self.Sink_Count + self.Q_Buffer_Count_V + self.Local_Count_V
        assert k == v
        return k


@pytest.fixture
def fake(monkeypatch):
    import kitty_b200.cache as cache_mod
    from kitty_b200 import _lib

    calls = []

    class Rec:
        def __getattr__(self, name):
            def f(*a):
                calls.append((name, a))
                return 0
            return f

    monkeypatch.setattr(cache_mod, "KVCache_Layer", FakeLayer)
    monkeypatch.setattr(_lib, "lib", lambda: Rec())
    monkeypatch.setattr(_lib, "stream_ptr", lambda d: 0)
    monkeypatch.setattr(cache_mod, "quantize_pack_k", lambda *a, **k: calls.append(("pack_k", a)))
    monkeypatch.setattr(cache_mod, "quantize_pack_v", lambda *a, **k: calls.append(("pack_v", a)))

    def pack_kv(k, k_off, pk, ptk, pok, kc, km, v, v_off, pv, ptv, pov, vc, vm, P, d_boost, **kw):
        # the prefill's one call for both: recorded as the two calls it stands for
        if pk > 0:
            calls.append(("pack_k", (k, k_off, pk, ptk, pok, kc, km, P, d_boost)))
        if pv > 0:
            calls.append(("pack_v", (v, v_off, pv, ptv, pov, vc, vm, P)))

    monkeypatch.setattr(cache_mod, "quantize_pack_kv", pack_kv)
    return cache_mod, calls


@pytest.mark.parametrize("L", [1, 20, 32, 33, 159, 160, 161, 288, 289, 32 + 3 * 128 + 57])
def test_counters_follow_the_reference_state_machine(fake, L):
    cache_mod, calls = fake
    cfg = types.SimpleNamespace(num_hidden_layers=2, head_dim=128, num_key_value_heads=2, num_attention_heads=8,
                                hidden_size=1024)
    steps = 300
    cache = cache_mod.KittyCache(cfg, 1, L + steps + 8)
    oc = ko.OracleKittyCache(2, 2, 128, 1, L + steps + 8, select=lambda pages, dt: torch.zeros(pages.shape[:-2] + (128,), dtype=torch.uint8).numpy())
    k = torch.zeros(1, 2, L, 128, dtype=torch.float16)
    for layer in (0, 1):
        assert cache.update(k, k, layer) is True and oc.update(k, k, layer) is True
        cache.quantize_prefill(layer)
        oc.quantize_prefill(layer)
        assert cache.kv_cache[layer].key_states is None
    tok = torch.zeros(1, 2, 1, 128, dtype=torch.float16)
    for s in range(steps):
        for layer in (0, 1):
            assert cache.update(tok, tok, layer) is False
            oc.update(tok, tok, layer)
            cache.quantize_decode(layer)
            oc.quantize_decode(layer)
            got = [getattr(cache.kv_cache[layer], c) for c in COUNTERS]
            want = [getattr(oc.kv_cache[layer], c) for c in COUNTERS]
            assert got == want, (s, layer, got, want)
        assert cache.get_seq_length(0) == L + s + 1
    names = [c[0] for c in calls]
    assert names.count("kitty_prefill_tails") == 2
    assert names.count("kitty_append") == 2 * steps
    p = ko.prefill_partition(L)
    assert names.count("pack_k") == (2 if p["pages_k"] else 0)
    flushes = [c for c in calls if c[0] == "kitty_flush"]
    final = oc.kv_cache[0]
    k_flushed = sum(1 for c in flushes if c[1][3]) // 2
    v_flushed = sum(1 for c in flushes if c[1][4]) // 2
    assert k_flushed == final.PageCount_K - p["pages_k"] and v_flushed == final.PageCount_V - p["pages_v"]


def test_a_further_piece_of_the_prompt_is_appended_token_by_token(fake):
    """A second multi-token update() is a further piece of the prompt: the layer switches to per-row counters, one
    kitty_append_rows per token position (rows that have run out of tokens are marked inactive), kitty_flush_rows
    when a Q-buffer is full — and the counters of every row equal the oracle's after the same number of tokens."""
    cache_mod, calls = fake
    cfg = types.SimpleNamespace(num_hidden_layers=1, head_dim=128, num_key_value_heads=1, num_attention_heads=4,
                                hidden_size=512)
    cache = cache_mod.KittyCache(cfg, 2, 1024)
    k = torch.zeros(2, 1, 40, 128, dtype=torch.float16)
    assert cache.update(k, k, 0) is True
    cache.quantize_prefill(0)
    calls.clear()
    chunk = torch.zeros(2, 1, 300, 128, dtype=torch.float16)
    assert cache.update(chunk, chunk, 0, {"lengths": [300, 130]}) is False
    names = [n for n, _ in calls]
    assert names.count("kitty_append_rows") == 300
    assert names.count("kitty_flush_rows") == 2          # token 120: a key page of both rows; token 248: row 0's second
                                                         # key page and first value page, in one launch
    lay = cache.kv_cache[0]
    for b, n in enumerate((300, 130)):
        oc = ko.OracleKittyCache(1, 1, 128, 1, 1024)
        oc.update(np.zeros((1, 1, 40, 128), np.float32), np.zeros((1, 1, 40, 128), np.float32), 0)
        oc.quantize_prefill(0)
        for _ in range(n):
            oc.update(np.zeros((1, 1, 1, 128), np.float32), np.zeros((1, 1, 1, 128), np.float32), 0)
            oc.quantize_decode(0)
        assert [int(x) for x in lay.row_counts[b, :7]] == [getattr(oc.kv_cache[0], c) for c in COUNTERS]
    assert cache.get_seq_length(0) == 340
    with pytest.raises(ValueError):
        cache.quantize_prefill(0)
    assert cache.get_mask_sizes(torch.arange(1), 0) == (341, 0)
    assert len(cache) == 2 - 1 and cache.get_max_cache_shape() == 1024


def test_page_pool_hands_out_and_takes_back():
    from kitty_b200.layer_state import PagePool

    pool = PagePool(6, order=[4, 0, 5, 1, 3, 2])
    assert pool.alloc(3) == [4, 0, 5] and pool.available() == 3
    pool.free([0, 4])
    assert pool.available() == 5
    assert sorted(pool.alloc(5)) == [0, 1, 2, 3, 4]
    with pytest.raises(MemoryError):
        pool.alloc(1)
    with pytest.raises(ValueError):
        PagePool(3, order=[0, 0, 1])
    pool.free([5])
    with pytest.raises(ValueError):
        pool.free([5])                 # already free


def _py_step(c):
    """kvcache/kitty.py:102-123 (append) then :201-234 (flush) on a dict of counters."""
    a = dict(c)
    if a["Sink_Count"] < 32:
        a["Sink_Count"] += 1
    else:
        a["Q_Buffer_Count_K"] += 1
        if a["Local_Count_V"] < 128:
            a["Local_Count_V"] += 1
        else:
            a["Q_Buffer_Count_V"] += 1
            a["Write_Offset_Local_V"] = (a["Write_Offset_Local_V"] + 1) % 128
    n = dict(a)
    fk, fv = n["Q_Buffer_Count_K"] == 128, n["Q_Buffer_Count_V"] == 128
    if fk:
        n["PageCount_K"] += 1
        n["Q_Buffer_Count_K"] = 0
    if fv:
        n["PageCount_V"] += 1
        n["Q_Buffer_Count_V"] = 0
    return a, n, fk, fv


@pytest.mark.parametrize("prompt,h_kv,h_q", [(1, 2, 8), (40, 2, 8), (32 + 128 * 3 + 100, 1, 7)])
def test_plan_step_follows_the_reference_state_machine(prompt, h_kv, h_q):
    """kitty_plan_step is host arithmetic (no device needed when no device block is given): its counters after the
    append and after the flushes must be the reference's, and its item counts must describe the plan."""
    import ctypes

    from kitty_b200 import _lib
    from oracle import kitty_oracle as ko

    p = ko.prefill_partition(prompt)
    c = {"PageCount_K": p["pages_k"], "PageCount_V": p["pages_v"], "Sink_Count": p["sink"],
         "Q_Buffer_Count_K": p["qbuf_k"], "Q_Buffer_Count_V": p["qbuf_v"], "Local_Count_V": p["local_v"],
         "Write_Offset_Local_V": 0}
    L = _lib.KittyLayer()
    L.max_bs, L.max_page, L.h_kv, L.head_dim, L.d_boost, L.page_size, L.sink_size = 4, 64, h_kv, 128, 32, 128, 32
    B = 3
    seen_flush_k = seen_flush_v = 0
    for _ in range(700):
        counts = _lib.KittyCounts()
        for k, v in c.items():
            setattr(counts, k, v)
        st = _lib.KittyStepState()
        rc = _lib.lib().kitty_plan_step(ctypes.byref(L), ctypes.byref(counts), B, h_q, ctypes.byref(st), None, None)
        assert rc == 0
        a, n, fk, fv = _py_step(c)
        assert {k: getattr(st.after, k) for k in c} == a
        assert {k: getattr(st.next, k) for k in c} == n
        assert (st.flush_k, st.flush_v) == (int(fk), int(fv))
        tail = (a["PageCount_K"] - a["PageCount_V"]) * 128 + a["Q_Buffer_Count_K"]
        assert st.pb == 0 and st.pe == a["PageCount_V"] and st.has_tail == int(tail > 0) and st.has_sink == 1
        edge_tokens = a["Sink_Count"] + tail
        assert st.edge_parts == -(-edge_tokens // st.edge_part_tok) and st.edge_part_tok % 64 == 0
        assert st.n_slots == st.edge_parts + st.nchunk and st.chunk_slot0 == st.edge_parts
        n_gt = 1 if h_q // h_kv <= 4 else -(-(h_q // h_kv) // 8)
        assert st.n_items == B * h_kv * n_gt * st.nchunk and st.n_edge == B * h_kv * st.edge_parts
        assert st.nchunk * st.ch >= a["PageCount_V"] and (st.nchunk == 0) == (a["PageCount_V"] == 0)
        seen_flush_k += fk
        seen_flush_v += fv
        c = n
    assert seen_flush_k >= 4 and seen_flush_v >= 4
    bad = _lib.KittyCounts()
    bad.Sink_Count, bad.Q_Buffer_Count_K = 10, 5          # tokens in the Q-buffer before the sink is full
    st = _lib.KittyStepState()
    assert _lib.lib().kitty_plan_step(ctypes.byref(L), ctypes.byref(bad), B, h_q, ctypes.byref(st), None, None) == -1


def test_split_pages_is_a_contiguous_partition_for_any_tail_weight():
    from kitty_b200.seqsplit import split_pages

    for n in (0, 1, 7, 10, 100, 1022):
        for world in (1, 2, 3, 4, 8):
            for tw in (0, 3, 32, 5000):
                r = split_pages(n, world, tw)
                assert len(r) == world and r[0][0] == 0 and r[-1][1] == n
                assert all(a[1] == b[0] for a, b in zip(r, r[1:])) and all(lo <= hi for lo, hi in r)
    assert [hi - lo for lo, hi in split_pages(1022, 8)] == [128] * 6 + [127] * 2
    sizes = [hi - lo for lo, hi in split_pages(1022, 8, 32)]
    assert sizes[-1] == sizes[0] - 33 and max(sizes[:-1]) - min(sizes[:-1]) <= 1


def test_plan_step_split_covers_the_sequence_exactly_once():
    """kitty_plan_step_split for the ranks of a sequence split: the page ranges of the ranks tile the common pages, the
    sink belongs to rank 0 only and the tail to the last rank only, every rank plans the same append and flushes, and
    the exchange sequence number is carried in the state."""
    import ctypes

    from kitty_b200 import _lib
    from kitty_b200.seqsplit import rank_flags, split_pages
    from oracle import kitty_oracle as ko

    p = ko.prefill_partition(32 + 128 * 37 + 100)
    counts = _lib.KittyCounts()
    for k, v in {"PageCount_K": p["pages_k"], "PageCount_V": p["pages_v"], "Sink_Count": p["sink"],
                 "Q_Buffer_Count_K": p["qbuf_k"], "Q_Buffer_Count_V": p["qbuf_v"], "Local_Count_V": p["local_v"],
                 "Write_Offset_Local_V": 0}.items():
        setattr(counts, k, v)
    L = _lib.KittyLayer()
    L.max_bs, L.max_page, L.h_kv, L.head_dim, L.d_boost, L.page_size, L.sink_size = 2, 64, 4, 128, 32, 128, 32
    world = 5
    covered, states = [], []
    for rank, (lo, hi) in enumerate(split_pages(p["pages_v"], world)):
        st = _lib.KittyStepState()
        rc = _lib.lib().kitty_plan_step_split(ctypes.byref(L), ctypes.byref(counts), 1, 28, lo, hi, rank_flags(rank, world),
                                              17, ctypes.byref(st), None, None)
        assert rc == 0
        assert (st.pb, st.pe) == (lo, hi) and st.xchg_seq == 17
        assert st.has_sink == int(rank == 0) and st.has_tail == int(rank == world - 1)
        assert st.n_items == 4 * st.nchunk and st.nchunk * st.ch >= hi - lo
        covered += list(range(st.pb, st.pe))
        states.append(st)
    assert covered == list(range(p["pages_v"]))
    for st in states[1:]:
        assert [getattr(st.next, f) for f, _ in _lib.KittyCounts._fields_] == \
               [getattr(states[0].next, f) for f, _ in _lib.KittyCounts._fields_]
        assert (st.flush_k, st.flush_v) == (states[0].flush_k, states[0].flush_v)
    st = _lib.KittyStepState()
    assert _lib.lib().kitty_plan_step_split(ctypes.byref(L), ctypes.byref(counts), 1, 28, 0, -1, 3, -1, ctypes.byref(st),
                                            None, None) == _lib.KITTY_E_BADARG


class _TokenSim:
    """Token-by-token model of one layer's queues (kvcache/kitty.py:102-123 and 201-234): tokens are numbers."""

    def __init__(self, S=32, P=128):
        self.S, self.P = S, P
        self.sink, self.qk, self.qv, self.pages_k, self.pages_v = [], [], [], [], []
        self.ring, self.w = [], 0

    def push(self, t):
        if len(self.sink) < self.S:
            self.sink.append(t)
            return
        self.qk.append(t)
        if len(self.ring) < self.P:
            self.ring.append(t)
        else:
            self.qv.append(self.ring[self.w])
            self.ring[self.w] = t
            self.w = (self.w + 1) % self.P
        if len(self.qk) == self.P:
            self.pages_k.append(self.qk)
            self.qk = []
        if len(self.qv) == self.P:
            self.pages_v.append(self.qv)
            self.qv = []


@pytest.mark.parametrize("history,pieces", [
    (20, [5, 300, 2]),            # the piece straddles the sink; the ring fills and wraps
    (40, [88, 129, 640]),         # ring not yet full, then exactly full, then several pages at once
    (32 + 128 + 77, [200, 51]),   # ring already wrapped (write offset != 0)
])
def test_a_uniform_piece_of_the_prompt_goes_through_in_bulk(fake, history, pieces):
    """update() with n > 1 tokens for every row of a layer with one set of counters takes the bulk path: sink, key
    Q-buffer, value ring (slots and write offset) and value Q-buffer end up exactly as after n single-token appends,
    the pages receive exactly the tokens the flushes would have packed, and the layer keeps its single counters."""
    cache_mod, calls = fake
    cfg = types.SimpleNamespace(num_hidden_layers=1, head_dim=128, num_key_value_heads=1, num_attention_heads=4,
                                hidden_size=512)
    cache = cache_mod.KittyCache(cfg, 1, 4096)
    lay = cache.kv_cache[0]
    f16 = dict(dtype=torch.float16)
    lay.Sink_Buffer_K, lay.Sink_Buffer_V = torch.zeros(1, 1, 32, 128, **f16), torch.zeros(1, 1, 32, 128, **f16)
    lay.Q_Buffer_K, lay.Q_Buffer_V = torch.zeros(1, 1, 128, 128, **f16), torch.zeros(1, 1, 128, 128, **f16)
    lay.Local_Buffer_V = torch.zeros(1, 1, 128, 128, **f16)
    sim = _TokenSim()
    for t in range(1, history + 1):
        sim.push(t)

    def load_state():
        lay.Sink_Count, lay.Q_Buffer_Count_K, lay.Q_Buffer_Count_V = len(sim.sink), len(sim.qk), len(sim.qv)
        lay.Local_Count_V, lay.Write_Offset_Local_V = len(sim.ring), sim.w
        lay.PageCount_K, lay.PageCount_V = len(sim.pages_k), len(sim.pages_v)
        for buf, vals in ((lay.Sink_Buffer_K, sim.sink), (lay.Sink_Buffer_V, sim.sink), (lay.Q_Buffer_K, sim.qk),
                          (lay.Q_Buffer_V, sim.qv), (lay.Local_Buffer_V, sim.ring)):
            buf.zero_()
            if vals:
                buf[0, 0, :len(vals)] = torch.tensor(vals, **f16)[:, None]
    load_state()
    packed = {"pack_k": [list(p) for p in sim.pages_k], "pack_v": [list(p) for p in sim.pages_v]}
    nxt = history + 1
    for n in pieces:
        calls.clear()
        toks = torch.arange(nxt, nxt + n, dtype=torch.float32)
        chunk = toks[None, None, :, None].expand(1, 1, n, 128).to(torch.float32 if n % 2 else torch.float16)
        assert cache.update(chunk, chunk, 0) is False
        for t in range(nxt, nxt + n):
            sim.push(t)
        nxt += n
        for name, a in calls:
            if name in packed:
                stream, t_off, pages, _, page_off = a[:5]
                assert t_off == 0 and page_off == len(packed[name])
                for p in range(pages):
                    packed[name].append([int(x) for x in stream[0, 0, 128 * p:128 * (p + 1), 0].float().tolist()])
        assert lay.row_counts is None
        assert not any(nm in ("kitty_append", "kitty_append_rows", "kitty_flush_rows") for nm, _ in calls)
        assert (lay.Sink_Count, lay.Q_Buffer_Count_K, lay.Q_Buffer_Count_V, lay.Local_Count_V, lay.Write_Offset_Local_V,
                lay.PageCount_K, lay.PageCount_V) == (len(sim.sink), len(sim.qk), len(sim.qv), len(sim.ring), sim.w,
                                                      len(sim.pages_k), len(sim.pages_v))
        for buf, vals in ((lay.Sink_Buffer_K, sim.sink), (lay.Sink_Buffer_V, sim.sink), (lay.Q_Buffer_K, sim.qk),
                          (lay.Q_Buffer_V, sim.qv), (lay.Local_Buffer_V, sim.ring)):
            assert [int(x) for x in buf[0, 0, :len(vals), 0].tolist()] == vals
        assert packed["pack_k"] == sim.pages_k and packed["pack_v"] == sim.pages_v
    assert cache.get_seq_length(0) == nxt - 1


def test_a_piece_that_does_not_fit_is_refused_before_anything_is_written(fake, monkeypatch):
    cache_mod, calls = fake
    from kitty_b200 import _lib
    monkeypatch.setattr(_lib, "strerror", lambda status: "bad argument")
    cfg = types.SimpleNamespace(num_hidden_layers=1, head_dim=128, num_key_value_heads=1, num_attention_heads=4,
                                hidden_size=512)
    cache = cache_mod.KittyCache(cfg, 1, 512)            # 4 pages
    lay = cache.kv_cache[0]
    k = torch.zeros(1, 1, 40, 128, dtype=torch.float16)
    assert cache.update(k, k, 0) is True
    cache.quantize_prefill(0)
    before = [getattr(lay, c) for c in COUNTERS]
    calls.clear()
    piece = torch.zeros(1, 1, 700, 128, dtype=torch.float16)
    with pytest.raises(_lib.KittyError):
        cache.update(piece, piece, 0)
    assert [getattr(lay, c) for c in COUNTERS] == before and not calls
