"""Ragged batches and prompts that arrive in pieces: every batch row with its own counters.  The reference keeps one
set of counters per layer (utils_kv_per_layer.py:53-80) and takes the prompt in one piece (kvcache/kitty.py:89-95);
here a batch of rows with different lengths must behave, row by row, exactly like single-row caches — checked
against one oracle cache per row, bit for bit on every buffer and within the attention tolerance on the outputs."""
import types

import numpy as np
import pytest
import torch

from oracle import kitty_oracle as ko
from tests.helpers import COUNTERS, make_kv

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
ATTN_TOL = 1e-2


@pytest.fixture(scope="module")
def kb():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import kitty_b200

    return kitty_b200


def _cfg(h_kv, h_q):
    return types.SimpleNamespace(num_hidden_layers=1, head_dim=128, num_key_value_heads=h_kv, num_attention_heads=h_q,
                                 hidden_size=128 * h_q)


def _bits(a):
    a = np.ascontiguousarray(a)
    return a.view(np.int16) if a.dtype == np.float16 else a


def _assert_row_equals_oracle(lay, b, olay):
    """Row b of the device layer against a single-row oracle layer: counters, fp16 buffers, and the row's pages."""
    rc = lay.row_counts[b]
    assert [int(x) for x in rc[:7]] == [getattr(olay, c) for c in COUNTERS], (b, rc)
    for name in ("Sink_Buffer_K", "Sink_Buffer_V", "Q_Buffer_K", "Q_Buffer_V", "Local_Buffer_V"):
        got, want = getattr(lay, name)[b].cpu().numpy(), np.asarray(getattr(olay, name))[0]
        if name.startswith("Sink"):
            n = olay.Sink_Count
        elif name == "Q_Buffer_K":
            n = olay.Q_Buffer_Count_K
        elif name == "Q_Buffer_V":
            n = olay.Q_Buffer_Count_V
        else:
            n = 128 if olay.Local_Count_V == 128 else olay.Local_Count_V
        assert np.array_equal(_bits(got[:, :n]), _bits(want[:, :n])), (b, name)
    for which, pages in (("Key", olay.PageCount_K), ("Value", olay.PageCount_V)):
        ids = getattr(lay, "PageTable_" + which[0])[b, :pages].cpu().numpy()
        oids = np.asarray(getattr(olay, "PageTable_" + which[0]))[0, :pages]
        got, want = getattr(lay, which + "Cache").cpu().numpy()[ids], np.asarray(getattr(olay, which + "Cache"))[oids]
        assert np.array_equal(got, want), (b, which)
        gm = getattr(lay, which + "Cache_metadata").cpu().numpy()[ids]
        wm = np.asarray(getattr(olay, which + "Cache_metadata"))[oids]
        assert np.array_equal(_bits(gm), _bits(wm)), (b, which, "metadata")


@pytest.mark.parametrize("h_kv,h_q,lens", [
    (2, 8, [32 + 3 * 128 + 100, 20, 32 + 128]),          # a row inside the sink, a row with one page exactly
    (1, 7, [700, 32 + 5 * 128 + 127]),                   # groups of 7: the two-group integer kernel
    (1, 12, [161, 32 + 2 * 128 + 60]),                   # groups of 12: the fp16 streaming kernel
])
def test_ragged_batch_equals_one_oracle_cache_per_row(kb, h_kv, h_q, lens):
    B, Lmax, steps = len(lens), max(lens), 140
    k, v = make_kv(B, h_kv, Lmax, 128, 300 + h_q, torch.float16)
    cache = kb.KittyCache(_cfg(h_kv, h_q), B, Lmax + steps + 8, device=DEV)
    oracles = [ko.OracleKittyCache(1, h_kv, 128, 1, Lmax + steps + 8) for _ in lens]
    assert cache.update(k.to(DEV), v.to(DEV), 0, {"lengths": lens}) is True
    cache.quantize_prefill(0)
    for b, L in enumerate(lens):
        oracles[b].update(k[b:b + 1, :, :L], v[b:b + 1, :, :L], 0)
        oracles[b].quantize_prefill(0)
    lay = cache.kv_cache[0]
    assert lay.row_counts is not None and cache.get_seq_length(0) == Lmax
    for b in range(B):
        _assert_row_equals_oracle(lay, b, oracles[b].kv_cache[0])
    g = torch.Generator().manual_seed(11)
    mod = types.SimpleNamespace(num_attention_heads=h_q, num_key_value_heads=h_kv)
    scaling = 128 ** -0.5
    for s in range(steps):
        kt, vt = torch.randn(B, h_kv, 1, 128, generator=g).half(), torch.randn(B, h_kv, 1, 128, generator=g).half()
        q = torch.randn(B, h_q, 1, 128, generator=g).half()
        assert cache.update(kt.to(DEV), vt.to(DEV), 0) is False
        for b in range(B):
            oracles[b].update(kt[b:b + 1], vt[b:b + 1], 0)
        if s % 9 == 0 or s > steps - 4:
            out, _ = kb.kitty_attention_forward(mod, q.to(DEV), lay, scaling)
            outs = {0: out}
            if s % 27 == 0:
                outs[1] = kb.decode_attention(q.to(DEV), lay, h_kv, scaling, impl=1)
                outs[2] = kb.decode_attention(q.to(DEV), lay, h_kv, scaling, impl=2)
            for b in range(B):
                want = ko.decode_attention(oracles[b].kv_cache[0], q[b:b + 1], h_q, scaling)
                for impl, o in outs.items():
                    err = ko.rel_err(o[b:b + 1].float().cpu().numpy(), want)
                    assert err <= ATTN_TOL, (s, b, impl, err)
        cache.quantize_decode(0)
        for b in range(B):
            oracles[b].quantize_decode(0)
    assert cache.get_seq_length(0) == Lmax + steps
    for b in range(B):
        _assert_row_equals_oracle(lay, b, oracles[b].kv_cache[0])
    assert kb.workspace_status(lay) == 0


def test_prompt_in_pieces_equals_token_by_token_and_one_piece(kb):
    """A prompt given as three update() calls (the later ones of a different length per row) leaves every row in the
    state token-by-token appends leave in the oracle; its pages equal those of the same tokens given in one piece."""
    h_kv, h_q, B = 2, 8, 2
    first, second, third = 200, [150, 90], [77, 300]
    total = [first + second[b] + third[b] for b in range(B)]
    k, v = make_kv(B, h_kv, max(total), 128, 17, torch.float16)
    cache = kb.KittyCache(_cfg(h_kv, h_q), B, max(total) + 64, device=DEV)
    assert cache.update(k[:, :, :first].to(DEV), v[:, :, :first].to(DEV), 0) is True
    cache.quantize_prefill(0)
    # second piece: rows take 150 and 90 tokens out of a 150-token tensor; third piece: 77 and 300 out of 300
    off = [first, first]
    for piece in (second, third):
        n = max(piece)
        kc = torch.zeros(B, h_kv, n, 128, dtype=torch.float16)
        vc = torch.zeros(B, h_kv, n, 128, dtype=torch.float16)
        for b in range(B):
            kc[b, :, :piece[b]] = k[b, :, off[b]:off[b] + piece[b]]
            vc[b, :, :piece[b]] = v[b, :, off[b]:off[b] + piece[b]]
            off[b] += piece[b]
        assert cache.update(kc.to(DEV), vc.to(DEV), 0, {"lengths": piece}) is False
    lay = cache.kv_cache[0]
    assert list(lay.row_lengths()[:B]) == total
    for b in range(B):
        oc = ko.OracleKittyCache(1, h_kv, 128, 1, max(total) + 64)
        oc.update(k[b:b + 1, :, :first], v[b:b + 1, :, :first], 0)
        oc.quantize_prefill(0)
        for t in range(first, total[b]):
            oc.update(k[b:b + 1, :, t:t + 1], v[b:b + 1, :, t:t + 1], 0)
            oc.quantize_decode(0)
        _assert_row_equals_oracle(lay, b, oc.kv_cache[0])
        one = ko.OracleKittyCache(1, h_kv, 128, 1, max(total) + 64)
        one.update(k[b:b + 1, :, :total[b]], v[b:b + 1, :, :total[b]], 0)
        one.quantize_prefill(0)
        ol, il = oc.kv_cache[0], one.kv_cache[0]
        assert (ol.PageCount_K, ol.PageCount_V) == (il.PageCount_K, il.PageCount_V)
        assert np.array_equal(ol.KeyCache[:ol.PageCount_K], il.KeyCache[:il.PageCount_K])
        assert np.array_equal(ol.ValueCache[:ol.PageCount_V], il.ValueCache[:il.PageCount_V])
    # and the attention of the next token agrees with the oracle row by row
    g = torch.Generator().manual_seed(5)
    q = torch.randn(B, h_q, 1, 128, generator=g).half()
    out = kb.decode_attention(q.to(DEV), lay, h_kv, 0.088)
    for b in range(B):
        oc = ko.OracleKittyCache(1, h_kv, 128, 1, max(total) + 64)
        oc.update(k[b:b + 1, :, :total[b]], v[b:b + 1, :, :total[b]], 0)
        oc.quantize_prefill(0)
        want = ko.decode_attention(oc.kv_cache[0], q[b:b + 1], h_q, 0.088)
        assert ko.rel_err(out[b:b + 1].float().cpu().numpy(), want) <= ATTN_TOL


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_uniform_pieces_take_the_bulk_path_and_equal_token_by_token(kb, dtype):
    """Pieces of the same length for every row of a layer with one set of counters: a few launches per piece, the
    layer keeps its single counters, and every buffer and page equals the oracle's after token-by-token appends (the
    oracle, like the append kernel, stores appended tokens as fp16 — which is what distinguishes this from a longer
    prefill when the model runs in bf16)."""
    h_kv, h_q, B = 2, 8, 2
    first, pieces = 20, [5, 300, 129, 700]
    total = first + sum(pieces)
    k, v = make_kv(B, h_kv, total, 128, 23, dtype)
    cache = kb.KittyCache(_cfg(h_kv, h_q), B, total + 64, device=DEV)
    assert cache.update(k[:, :, :first].to(DEV), v[:, :, :first].to(DEV), 0) is True
    cache.quantize_prefill(0)
    off = first
    for n in pieces:
        assert cache.update(k[:, :, off:off + n].to(DEV), v[:, :, off:off + n].to(DEV), 0) is False
        off += n
    lay = cache.kv_cache[0]
    assert lay.row_counts is None and cache.get_seq_length(0) == total
    lay.make_ragged()                       # only to reuse the row-wise comparison below
    for b in range(B):
        oc = ko.OracleKittyCache(1, h_kv, 128, 1, total + 64)
        oc.update(k[b:b + 1, :, :first], v[b:b + 1, :, :first], 0)
        oc.quantize_prefill(0)
        for t in range(first, total):
            oc.update(k[b:b + 1, :, t:t + 1], v[b:b + 1, :, t:t + 1], 0)
            oc.quantize_decode(0)
        _assert_row_equals_oracle(lay, b, oc.kv_cache[0])
    assert kb.workspace_status(lay) == 0


def test_ragged_entry_points_reject_bad_rows(kb):
    import ctypes

    from kitty_b200 import _lib

    cache = kb.KittyCache(_cfg(1, 4), 2, 600, device=DEV)
    k, v = make_kv(2, 1, 300, 128, 3, torch.float16)
    cache.update(k.to(DEV), v.to(DEV), 0, {"lengths": [300, 120]})
    cache.quantize_prefill(0)
    lay = cache.kv_cache[0]
    bad = lay.row_counts.copy()
    bad[1, 4] += 1                                    # row 1: key and value lengths disagree
    q = torch.zeros(2, 4, 1, 128, dtype=torch.float16, device=DEV)
    ws = lay.workspace(2, 4)
    rc = _lib.lib().kitty_decode_attn_rows(lay.c_layer(), bad.ctypes.data, lay._row_dev.data_ptr(), q.data_ptr(), 0, 2,
                                           4, 1.0, q.data_ptr(), 0, ws.data_ptr(), ws.numel(), 0, None)
    assert rc == _lib.KITTY_E_BADARG
    rc = _lib.lib().kitty_decode_attn_rows(lay.c_layer(), None, lay._row_dev.data_ptr(), q.data_ptr(), 0, 2, 4, 1.0,
                                           q.data_ptr(), 0, ws.data_ptr(), ws.numel(), 0, None)
    assert rc == _lib.KITTY_E_BADARG
    with pytest.raises(ValueError):
        cache.plan_step(2, 4)                          # the device-resident step keeps one set of counters
