"""Parity of the CUDA path (called through the C-ABI library) with the oracle and
with the reference-generated golden fixtures.  Needs a B200: run with -m gpu."""
import types

import numpy as np
import pytest
import torch

from oracle import kitty_oracle as ko
from tests.helpers import BUFFERS, COUNTERS, load, make_kv, tensor_from_raw

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
ATTN_TOL = 1e-2      # max|a-b| / max|b| for attention outputs (the stated bf16-level tolerance)
QUANT = ["quant_f16_outlier8", "quant_bf16_loguniform", "quant_f32_outlier8", "quant_f16_degenerate"]
TORCH_DT = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}


@pytest.fixture(scope="module")
def kb():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import kitty_b200

    return kitty_b200


def _buffers(B, H, maxp):
    z = dict(device=DEV)
    return (torch.zeros(B * maxp, H * 5248, dtype=torch.uint8, **z), torch.zeros(B * maxp, H, 128, 2, dtype=torch.float16, **z),
            torch.zeros(B * maxp, H * 4096, dtype=torch.uint8, **z), torch.zeros(B * maxp, H, 128, 2, dtype=torch.float16, **z),
            torch.arange(B * maxp, dtype=torch.int64, **z).view(B, maxp))


def _f16_bits(t):
    return t.cpu().contiguous().view(torch.int16).numpy()


# --------------------------------------------------------------------------- #
# quantize / pack
# --------------------------------------------------------------------------- #
@pytest.mark.parametrize("name", QUANT)
def test_quant_matches_reference_bytes_with_supplied_index(kb, name):
    """With the reference's own index bytes the kernels must reproduce the
    reference's cache bytes and fp16 metadata exactly."""
    fx = load(name)
    dt = str(fx["dtype"])
    x = tensor_from_raw(fx["x"], dt).to(DEV)
    B, H, T, D = x.shape
    P, poff, t0 = int(fx["pages"]), int(fx["page_offset"]), int(fx["t_offset"])
    kc, km, vc, vm, pt = _buffers(B, H, 4)
    ref_k = fx["KeyCache"].reshape(-1, H, 5248)
    idx = np.stack([ref_k[poff + p, :, 5120:] for p in range(P)], 1)[None]
    kb.quantize_pack_k(x, t0, P, pt, poff, kc, km, 128, 32, channel_idx=torch.from_numpy(idx.copy()))
    kb.quantize_pack_v(x, t0, P, pt, poff, vc, vm, 128)
    assert np.array_equal(kc.cpu().numpy(), fx["KeyCache"])
    assert np.array_equal(_f16_bits(km), fx["KeyCache_metadata"].view(np.int16))
    assert np.array_equal(vc.cpu().numpy(), fx["ValueCache"])
    assert np.array_equal(_f16_bits(vm), fx["ValueCache_metadata"].view(np.int16))


@pytest.mark.parametrize("dtype,kind,seed", [("f16", "outlier8", 5), ("bf16", "loguniform", 6), ("f32", "outlier8", 7),
                                             ("f16", "loguniform", 8), ("bf16", "outlier8", 9)])
def test_quant_fused_selection_bit_exact_with_oracle(kb, dtype, kind, seed):
    """In-kernel score + rank + quantize + pack on strided input, against the
    oracle's order-independent score and lowest-channel-first tie rule."""
    B, H, P = 2, 3, 5
    T = 32 + P * 128 + 17
    k, v = make_kv(B, H, T, 128, seed, TORCH_DT[dtype], kind)
    # strided source: [B, T, H, D] storage viewed as [B, H, T, D], as a model's projection output is
    ks = k.transpose(1, 2).contiguous().to(DEV).transpose(1, 2)
    vs = v.transpose(1, 2).contiguous().to(DEV).transpose(1, 2)
    kc, km, vc, vm, pt = _buffers(B, H, 8)
    idx_out = torch.full((B, H, P, 128), 255, dtype=torch.uint8, device=DEV)
    from kitty_b200 import _lib

    rc = _lib.lib().kitty_quant_pack_k(ks.data_ptr(), _lib.dtype_code(ks.dtype), ks.stride(0), ks.stride(1), ks.stride(2),
                                       B, H, 32, P, pt.data_ptr(), pt.stride(0), 2, kc.data_ptr(), kc.stride(0),
                                       km.data_ptr(), idx_out.data_ptr(), _lib.SELECT_FUSED, _lib.DIV_IEEE,
                                       torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    kb.quantize_pack_v(vs, 32, P, pt, 2, vc, vm, 128)
    pages = ko.as_f32(k)[:, :, 32:32 + P * 128].reshape(B, H, P, 128, 128)
    idx = ko.rank_channels(ko.channel_score(pages, dtype, "exact"), 32, "stable")
    assert np.array_equal(idx_out.cpu().numpy(), idx)
    rec, meta = ko.quantize_k_pages(pages.reshape(-1, 128, 128), idx.reshape(-1, 128), 32)
    rec, meta = rec.reshape(B, H, P, 5248), meta.reshape(B, H, P, 128, 2)
    vpages = ko.as_f32(v)[:, :, 32:32 + P * 128].reshape(-1, 128, 128)
    vrec, vmeta = ko.quantize_v_pages(vpages)
    vrec, vmeta = vrec.reshape(B, H, P, 4096), vmeta.reshape(B, H, P, 128, 2)
    kc_h, km_h, vc_h, vm_h = kc.cpu().numpy().reshape(-1, H, 5248), _f16_bits(km), vc.cpu().numpy().reshape(-1, H, 4096), _f16_bits(vm)
    for b in range(B):
        for p in range(P):
            pid = b * 8 + 2 + p
            assert np.array_equal(kc_h[pid], rec[b, :, p]), (b, p)
            assert np.array_equal(km_h[pid], meta[b, :, p].view(np.int16))
            assert np.array_equal(vc_h[pid], vrec[b, :, p])
            assert np.array_equal(vm_h[pid], vmeta[b, :, p].view(np.int16))
    # pages outside [2, 2+P) untouched
    assert not kc_h[0].any() and not kc_h[1].any() and not kc_h[7].any()


@pytest.mark.parametrize("dtype", ["f16", "bf16"])
def test_quant_degenerate_pages_bit_exact_with_oracle(kb, dtype):
    """Pages that stress the boundary computation and the selection: all zeros; one constant per channel (range 0, the
    scale floor); every channel with max = -min (the middle boundary sits at zero, where the 16-bit grid is finer
    than fp32 next to min); values far below the scale floor; values near the top of the type's range; all channels
    equal (every score ties: lower channel first); a page of two values only."""
    g = torch.Generator().manual_seed(41)
    H, P = 2, 7
    x = torch.zeros(1, H, P * 128, 128)
    pg = lambda i: x[:, :, 128 * i:128 * (i + 1)]
    pg(1)[:] = (torch.arange(128) * 0.25 - 9.0)[None, None, None, :]
    a = torch.randn(1, H, 64, 128, generator=g) * torch.exp(torch.rand(1, H, 1, 128, generator=g) * 3.0)
    a[:, :, 0] = a.abs().amax(2) * 1.5                      # the largest magnitude of the channel, with both signs below
    pg(2)[:] = torch.cat([a, -a], dim=2)
    pg(3)[:] = torch.randn(1, H, 128, 128, generator=g) * 1e-7
    pg(4)[:] = torch.randn(1, H, 128, 128, generator=g) * (6000.0 if dtype == "f16" else 1e30)
    pg(5)[:] = torch.randn(1, H, 128, 1, generator=g).expand(1, H, 128, 128)
    pg(6)[:] = torch.where(torch.rand(1, H, 128, 128, generator=g) < 0.5, torch.tensor(-1.0), torch.tensor(3.0))
    xd = x.to(TORCH_DT[dtype])
    kc, km, vc, vm, pt = _buffers(1, H, 8)
    idx_out = torch.full((1, H, P, 128), 255, dtype=torch.uint8, device=DEV)
    from kitty_b200 import _lib

    xs = xd.to(DEV)
    rc = _lib.lib().kitty_quant_pack_k(xs.data_ptr(), _lib.dtype_code(xs.dtype), xs.stride(0), xs.stride(1), xs.stride(2),
                                       1, H, 0, P, pt.data_ptr(), pt.stride(0), 0, kc.data_ptr(), kc.stride(0),
                                       km.data_ptr(), idx_out.data_ptr(), _lib.SELECT_FUSED, _lib.DIV_IEEE,
                                       torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    kb.quantize_pack_v(xs, 0, P, pt, 0, vc, vm, 128)
    pages = ko.as_f32(xd).reshape(1, H, P, 128, 128)
    idx = ko.rank_channels(ko.channel_score(pages, dtype, "exact"), 32, "stable")
    assert np.array_equal(idx_out.cpu().numpy(), idx)
    rec, meta = ko.quantize_k_pages(pages.reshape(-1, 128, 128), idx.reshape(-1, 128), 32)
    rec, meta = rec.reshape(H, P, 5248), meta.reshape(H, P, 128, 2)
    vrec, vmeta = ko.quantize_v_pages(pages.reshape(-1, 128, 128))
    vrec, vmeta = vrec.reshape(H, P, 4096), vmeta.reshape(H, P, 128, 2)
    kc_h, km_h = kc.cpu().numpy().reshape(-1, H, 5248), _f16_bits(km)
    vc_h, vm_h = vc.cpu().numpy().reshape(-1, H, 4096), _f16_bits(vm)
    for p in range(P):
        assert np.array_equal(kc_h[p], rec[:, p]), p
        assert np.array_equal(km_h[p], meta[:, p].view(np.int16)), p
        assert np.array_equal(vc_h[p], vrec[:, p]), p
        assert np.array_equal(vm_h[p], vmeta[:, p].view(np.int16)), p


@pytest.mark.parametrize("dtype,strided,pk,pv", [("bf16", False, 5, 5), ("f16", True, 4, 3), ("bf16", True, 2, 6),
                                                 ("f32", False, 3, 3)])
def test_quant_keys_and_values_in_one_call_equal_the_two_calls(kb, dtype, strided, pk, pv):
    """kitty_quant_pack_kv (one launch for 16-bit input) against kitty_quant_pack_k + kitty_quant_pack_v: every byte
    of the four destination buffers, with different page counts, offsets and page-table offsets for keys and values."""
    B, H = 2, 3
    T = 40 + max(pk, pv) * 128 + 9
    k, v = make_kv(B, H, T, 128, 31, TORCH_DT[dtype], "loguniform")
    if strided:
        ks = k.transpose(1, 2).contiguous().to(DEV).transpose(1, 2)
        vs = v.transpose(1, 2).contiguous().to(DEV).transpose(1, 2)
    else:
        ks, vs = k.to(DEV), v.to(DEV)
    one = _buffers(B, H, 8)
    two = _buffers(B, H, 8)
    kb.quantize_pack_kv(ks, 32, pk, one[4], 1, one[0], one[1], vs, 40, pv, one[4], 2, one[2], one[3], 128, 32)
    kb.quantize_pack_k(ks, 32, pk, two[4], 1, two[0], two[1], 128, 32)
    kb.quantize_pack_v(vs, 40, pv, two[4], 2, two[2], two[3], 128)
    for a, b in zip(one[:4], two[:4]):
        assert torch.equal(a.view(torch.uint8), b.view(torch.uint8))
    assert one[0].any() and one[2].any()
    # the same through the C entry point with SUPPLIED index bytes (those the in-kernel selection just produced)
    from kitty_b200 import _lib

    idx = torch.full((B, H, pk, 128), 255, dtype=torch.uint8, device=DEV)
    kb.quantize_pack_k(ks, 32, pk, two[4], 1, two[0], two[1], 128, 32)
    rc = _lib.lib().kitty_quant_pack_k(ks.data_ptr(), _lib.dtype_code(ks.dtype), ks.stride(0), ks.stride(1), ks.stride(2),
                                       B, H, 32, pk, two[4].data_ptr(), two[4].stride(0), 1, two[0].data_ptr(),
                                       two[0].stride(0), two[1].data_ptr(), idx.data_ptr(), _lib.SELECT_FUSED,
                                       _lib.DIV_IEEE, torch.cuda.current_stream().cuda_stream)
    assert rc == 0 and int(idx.max()) <= 32
    three = _buffers(B, H, 8)
    rc = _lib.lib().kitty_quant_pack_kv(ks.data_ptr(), vs.data_ptr(), _lib.dtype_code(ks.dtype), ks.stride(0), ks.stride(1),
                                        ks.stride(2), vs.stride(0), vs.stride(1), vs.stride(2), B, H, 32, pk,
                                        three[4].data_ptr(), three[4].stride(0), 1, three[0].data_ptr(),
                                        three[0].stride(0), three[1].data_ptr(), idx.data_ptr(), _lib.SELECT_SUPPLIED,
                                        40, pv, three[4].data_ptr(), three[4].stride(0), 2, three[2].data_ptr(),
                                        three[2].stride(0), three[3].data_ptr(), _lib.DIV_IEEE,
                                        torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    for a, b in zip(three[:4], two[:4]):
        assert torch.equal(a.view(torch.uint8), b.view(torch.uint8))
    # a bad argument in the value half is reported before the key half is launched
    rc = _lib.lib().kitty_quant_pack_kv(ks.data_ptr(), vs.data_ptr(), _lib.dtype_code(ks.dtype), ks.stride(0), ks.stride(1),
                                        ks.stride(2), vs.stride(0), vs.stride(1), vs.stride(2), B, H, 32, pk,
                                        three[4].data_ptr(), three[4].stride(0), 1, three[0].data_ptr(),
                                        three[0].stride(0), three[1].data_ptr(), None, _lib.SELECT_FUSED,
                                        40, pv, None, three[4].stride(0), 2, three[2].data_ptr(),
                                        three[2].stride(0), three[3].data_ptr(), _lib.DIV_IEEE,
                                        torch.cuda.current_stream().cuda_stream)
    assert rc == _lib.KITTY_E_BADARG


def test_quant_torch_selection_is_tie_equivalent(kb):
    """selection='torch' (the reference's host prologue run on the device) and the
    fused rule agree on the score found at every rank."""
    B, H, P = 1, 4, 6
    k, _ = make_kv(B, H, P * 128, 128, 21, torch.float16, "loguniform")
    kd = k.to(DEV)
    kc, km, _, _, pt = _buffers(B, H, 8)
    idx_t = kb.quantize_pack_k(kd, 0, P, pt, 0, kc, km, 128, 32, selection="torch").cpu().numpy()
    pages = ko.as_f32(k).reshape(B, H, P, 128, 128)
    s = ko.channel_score(pages, "f16", "exact")
    idx_f = ko.rank_channels(s, 32, "stable")
    st = ko.channel_score(pages, "f16", "torch")
    rows = (s == st).all(-1)
    assert rows.mean() > 0.9
    assert ko.selection_equivalent(s[rows], idx_f[rows], idx_t[rows], 32)


def test_quant_div_full_mode_differs_rarely(kb):
    """div.full.f32 is within 2 ulp of IEEE: codes may differ only at exact rounding ties."""
    k, _ = make_kv(1, 2, 512, 128, 33, torch.float16, "outlier8")
    kd = k.to(DEV)
    from kitty_b200 import _lib

    a = _buffers(1, 2, 4)
    b = _buffers(1, 2, 4)
    kb.quantize_pack_v(kd, 0, 4, a[4], 0, a[2], a[3], 128)
    kb.quantize_pack_v(kd, 0, 4, b[4], 0, b[2], b[3], 128, div_mode=_lib.DIV_FULL)
    assert torch.equal(a[3], b[3])
    diff = (a[2] != b[2]).float().mean().item()
    assert diff < 1e-3


# --------------------------------------------------------------------------- #
# cache state machine + attention
# --------------------------------------------------------------------------- #
def _cfg(layers, h_kv, h_q):
    return types.SimpleNamespace(num_hidden_layers=layers, head_dim=128, num_key_value_heads=h_kv,
                                 num_attention_heads=h_q, hidden_size=128 * h_q)


def _assert_same_state(lay, olay, what=BUFFERS):
    for n in what:
        a, b = getattr(lay, n).cpu().numpy(), np.asarray(getattr(olay, n))
        if a.dtype == np.float16:
            a, b = a.view(np.int16), b.view(np.int16)
        assert np.array_equal(a, b), n
    assert [getattr(lay, c) for c in COUNTERS] == [getattr(olay, c) for c in COUNTERS]


@pytest.mark.parametrize("name", ["cache_g4", "cache_g7_short"])
def test_cache_replay_against_oracle_and_reference(kb, name):
    """Replay the fixture's prefill + decode steps.  Every buffer must equal the
    oracle's bit for bit after every flush; attention must match the oracle and
    the reference's recorded outputs within ATTN_TOL."""
    fx = load(name)
    k0, v0 = tensor_from_raw(fx["k_prefill"], "f16"), tensor_from_raw(fx["v_prefill"], "f16")
    B, H, L, D = k0.shape
    h_q, scaling = int(fx["h_q"]), float(fx["scaling"])
    steps = fx["k_steps"].shape[0]
    cache = kb.KittyCache(_cfg(1, H, h_q), B, L + steps + 8, device=DEV)
    ocache = ko.OracleKittyCache(1, H, D, B, L + steps + 8)
    mod = types.SimpleNamespace(num_attention_heads=h_q, num_key_value_heads=H)
    assert cache.update(k0.to(DEV), v0.to(DEV), 0) is True and ocache.update(k0, v0, 0) is True
    cache.quantize_prefill(0)
    ocache.quantize_prefill(0)
    lay, olay = cache.kv_cache[0], ocache.kv_cache[0]
    _assert_same_state(lay, olay)
    # everything that does not depend on the order of equal scores also equals the reference's own state
    non_k = [n for n in BUFFERS if n not in ("KeyCache", "KeyCache_metadata")]
    for n in non_k:
        a, b = getattr(lay, n).cpu().numpy(), fx["prefill_" + n]
        assert np.array_equal(a.view(np.int16) if a.dtype == np.float16 else a, b.view(np.int16) if b.dtype == np.float16 else b), n
    probes = list(fx["probe_steps"])
    for s in range(steps):
        k, v = tensor_from_raw(fx["k_steps"][s], "f16"), tensor_from_raw(fx["v_steps"][s], "f16")
        assert cache.update(k.to(DEV), v.to(DEV), 0) is False
        ocache.update(k, v, 0)
        assert cache.get_seq_length(0) == ocache.get_seq_length(0)
        if s in probes or s % 37 == 5:
            q = tensor_from_raw(fx["q_steps"][s], "f16")
            out, w = kb.kitty_attention_forward(mod, q.to(DEV), lay, scaling)
            assert w is None and out.shape == (B, 1, h_q, D) and out.dtype == torch.float16
            want = ko.decode_attention(olay, q, h_q, scaling)
            assert ko.rel_err(out.float().cpu().numpy(), want) <= ATTN_TOL
            for impl in (1, 2):
                out1 = kb.decode_attention(q.to(DEV), lay, H, scaling, impl=impl)
                assert ko.rel_err(out1.float().cpu().numpy(), want) <= ATTN_TOL
            if s in probes:
                ref = ko.as_f32(tensor_from_raw(fx["attn_out"][probes.index(s)], "f16"))
                assert ko.rel_err(out.float().cpu().numpy(), ref) <= ATTN_TOL
        flush = lay.Q_Buffer_Count_K == 128 or lay.Q_Buffer_Count_V == 128
        cache.quantize_decode(0)
        ocache.quantize_decode(0)
        if flush or s == steps - 1:
            _assert_same_state(lay, olay)
    for n in non_k:
        a, b = getattr(lay, n).cpu().numpy(), fx["final_" + n]
        assert np.array_equal(a.view(np.int16) if a.dtype == np.float16 else a, b.view(np.int16) if b.dtype == np.float16 else b), n
    from kitty_b200.attention import workspace_status

    assert workspace_status(lay) == 0


@pytest.mark.parametrize("h_kv,h_q,B,L,dtype", [
    (8, 32, 1, 2048, torch.float32),     # the CPU-runnable configuration: fp32 N(0,1), 2048 cached tokens
    (2, 8, 3, 32 + 9 * 128 + 1, torch.bfloat16),
    (1, 7, 2, 32 + 6 * 128 + 127, torch.bfloat16),
    (2, 2, 1, 32 + 4 * 128, torch.float16),      # group of 1
    (1, 16, 1, 32 + 5 * 128 + 3, torch.float16),  # group of 16: two tiles of 8 query heads
    (2, 24, 1, 700, torch.float16),              # group of 12
    (2, 16, 2, 32 + 7 * 128 + 31, torch.bfloat16),   # group of 8: two full operand groups of the integer kernel
    (1, 5, 2, 32 + 10 * 128 + 99, torch.float16),    # group of 5: second operand group holds one head
    (3, 18, 1, 32 + 5 * 128 + 64, torch.bfloat16),   # group of 6
    (8, 32, 9, 32 + 3 * 128 + 5, torch.float16),     # 72 (batch, kv-head) row groups
    (1, 4, 2, 20, torch.float16),                # shorter than the sink
    (1, 4, 2, 33, torch.float16),
    (1, 4, 1, 160, torch.float16),               # exactly sink + one page: no packed value page yet
    (1, 4, 1, 161, torch.float16),
])
def test_attention_after_prefill_and_a_few_steps(kb, h_kv, h_q, B, L, dtype):
    k, v = make_kv(B, h_kv, L, 128, 100 + L, dtype)
    cache = kb.KittyCache(_cfg(1, h_kv, h_q), B, L + 64, device=DEV)
    dn = {torch.float16: "f16", torch.bfloat16: "bf16", torch.float32: "f32"}[dtype]
    ocache = ko.OracleKittyCache(1, h_kv, 128, B, L + 64)
    cache.update(k.to(DEV), v.to(DEV), 0)
    ocache.update(k, v, 0, dtype=dn)
    cache.quantize_prefill(0)
    ocache.quantize_prefill(0)
    lay, olay = cache.kv_cache[0], ocache.kv_cache[0]
    _assert_same_state(lay, olay)
    g = torch.Generator().manual_seed(L)
    scaling = 128 ** -0.5
    for s in range(3):
        kt, vt = torch.randn(B, h_kv, 1, 128, generator=g).to(dtype), torch.randn(B, h_kv, 1, 128, generator=g).to(dtype)
        q = torch.randn(B, h_q, 1, 128, generator=g).to(dtype)
        cache.update(kt.to(DEV), vt.to(DEV), 0)
        ocache.update(kt, vt, 0, dtype=dn)
        want = ko.decode_attention(olay, q, h_q, scaling)
        for impl in (0, 1, 2):      # default kernels, plain cross-check kernel, fp16 streaming kernel
            out = kb.decode_attention(q.to(DEV), lay, h_kv, scaling, impl=impl)
            assert out.dtype == dtype
            err = ko.rel_err(out.float().cpu().numpy(), want)
            assert err <= ATTN_TOL, (impl, s, err)
        cache.quantize_decode(0)
        ocache.quantize_decode(0)
    _assert_same_state(lay, olay)


def test_sequence_split_partials_merge_to_the_full_result(kb):
    """Three 'ranks' each reduce a contiguous range of pages (sink on the first,
    tail on the last); merging their partials equals the single-call result."""
    h_kv, h_q, B, L = 2, 14, 2, 32 + 11 * 128 + 40
    k, v = make_kv(B, h_kv, L, 128, 77, torch.bfloat16)
    cache = kb.KittyCache(_cfg(1, h_kv, h_q), B, L + 8, device=DEV)
    cache.update(k.to(DEV), v.to(DEV), 0)
    cache.quantize_prefill(0)
    lay = cache.kv_cache[0]
    g = torch.Generator().manual_seed(3)
    kt, vt = torch.randn(B, h_kv, 1, 128, generator=g).bfloat16(), torch.randn(B, h_kv, 1, 128, generator=g).bfloat16()
    cache.update(kt.to(DEV), vt.to(DEV), 0)
    q = torch.randn(B, h_q, 1, 128, generator=g).bfloat16().to(DEV)
    full = kb.decode_attention(q, lay, h_kv, 128 ** -0.5)
    pv = lay.PageCount_V
    cuts = [0, 3, 4, pv]
    parts = torch.empty(3, B, h_q, 130, dtype=torch.float32, device=DEV)
    for r in range(3):
        flags = (1 if r == 0 else 0) | (2 if r == 2 else 0)
        kb.decode_attention(q, lay, h_kv, 128 ** -0.5, page_begin=cuts[r], page_end=cuts[r + 1], flags=flags,
                            partial_out=parts[r])
    merged = kb.lse_merge(parts, torch.bfloat16)
    assert ko.rel_err(merged.float().cpu().numpy(), full.float().cpu().numpy()) <= 1e-2
    # an empty range yields an empty partial that does not disturb the merge
    empty = torch.empty(B, h_q, 130, dtype=torch.float32, device=DEV)
    kb.decode_attention(q, lay, h_kv, 128 ** -0.5, page_begin=2, page_end=2, flags=0, partial_out=empty)
    merged2 = kb.lse_merge(torch.cat([parts, empty[None]]).contiguous(), torch.bfloat16)
    assert torch.equal(merged, merged2)


def test_argument_errors(kb):
    from kitty_b200 import _lib

    cache = kb.KittyCache(_cfg(1, 2, 8), 1, 512, device=DEV)
    lay = cache.kv_cache[0]
    q = torch.zeros(1, 8, 1, 128, dtype=torch.float16, device=DEV)
    with pytest.raises(_lib.KittyError):            # empty cache: nothing to attend to
        kb.decode_attention(q, lay, 2, 1.0)
    with pytest.raises(AssertionError):             # two query tokens
        kb.decode_attention(torch.zeros(1, 8, 2, 128, dtype=torch.float16, device=DEV), lay, 2, 1.0)
    with pytest.raises(ValueError):
        cache.quantize_prefill(0)                   # before update()
    k, v = make_kv(1, 2, 300, 128, 1)
    cache.update(k.to(DEV), v.to(DEV), 0)
    cache.quantize_prefill(0)
    ws = torch.zeros(512, dtype=torch.uint8, device=DEV)
    rc = _lib.lib().kitty_decode_attn(lay.c_layer(), lay.c_counts(), q.data_ptr(), 0, 1, 8, 1.0, q.data_ptr(), 0,
                                      ws.data_ptr(), ws.numel(), 0, -1, 3, None, 0, None)
    assert rc == _lib.KITTY_E_WORKSPACE
    bad = lay.c_counts()
    bad.Q_Buffer_Count_V += 1                        # key/value lengths disagree
    rc = _lib.lib().kitty_decode_attn(lay.c_layer(), bad, q.data_ptr(), 0, 1, 8, 1.0, q.data_ptr(), 0,
                                      lay.workspace(1, 8).data_ptr(), lay.workspace(1, 8).numel(), 0, -1, 3, None, 0, None)
    assert rc == _lib.KITTY_E_BADARG
    with pytest.raises(_lib.KittyError):            # further pieces of the prompt until the cache's 4 pages are full
        cache.update(k.to(DEV), v.to(DEV), 0)
        cache.update(k.to(DEV), v.to(DEV), 0)


# --------------------------------------------------------------------------- #
# full-size properties (sizes of the 32K-token kernel sweep)
# --------------------------------------------------------------------------- #
def test_full_size_32k_properties(kb):
    """At 32768 cached tokens (255 key pages / 254 value pages): the streaming
    kernel agrees with the plain kernel, a split over pages merges to the same
    result, and one (batch, head) agrees with the oracle."""
    h_kv, h_q, B, L = 8, 32, 2, 32768
    g = torch.Generator().manual_seed(2024)
    k = torch.randn(B, h_kv, L, 128, generator=g)
    for h in range(h_kv):
        k[:, h, :, torch.randperm(128, generator=g)[:4]] *= 8.0
    v = torch.randn(B, h_kv, L, 128, generator=g)
    k, v = k.bfloat16(), v.bfloat16()
    cache = kb.KittyCache(_cfg(1, h_kv, h_q), B, L + 256, device=DEV)
    cache.update(k.to(DEV), v.to(DEV), 0)
    cache.quantize_prefill(0)
    lay = cache.kv_cache[0]
    assert (lay.PageCount_K, lay.PageCount_V, lay.Q_Buffer_Count_K, lay.Q_Buffer_Count_V) == (255, 254, 96, 96)
    kt, vt = torch.randn(B, h_kv, 1, 128, generator=g).bfloat16(), torch.randn(B, h_kv, 1, 128, generator=g).bfloat16()
    cache.update(kt.to(DEV), vt.to(DEV), 0)
    q = torch.randn(B, h_q, 1, 128, generator=g).bfloat16().to(DEV)
    sc = 128 ** -0.5
    fast = kb.decode_attention(q, lay, h_kv, sc).float().cpu().numpy()
    plain = kb.decode_attention(q, lay, h_kv, sc, impl=1).float().cpu().numpy()
    assert ko.rel_err(fast, plain) <= ATTN_TOL
    fp16k = kb.decode_attention(q, lay, h_kv, sc, impl=2).float().cpu().numpy()
    assert ko.rel_err(fp16k, plain) <= ATTN_TOL
    parts = torch.empty(4, B, h_q, 130, dtype=torch.float32, device=DEV)
    cuts = [0, 64, 128, 192, 254]
    for r in range(4):
        kb.decode_attention(q, lay, h_kv, sc, page_begin=cuts[r], page_end=cuts[r + 1],
                            flags=(1 if r == 0 else 0) | (2 if r == 3 else 0), partial_out=parts[r])
    merged = kb.lse_merge(parts, torch.bfloat16).float().cpu().numpy()
    assert ko.rel_err(merged, fast) <= ATTN_TOL
    # oracle on one (batch, head): rebuild an oracle layer view from the device buffers
    view = types.SimpleNamespace(D=128, D_BOOSTED=32, H_KV=h_kv, **{n: getattr(lay, n).cpu().numpy() for n in BUFFERS},
                                 **{c: getattr(lay, c) for c in COUNTERS})
    b, h = 1, 5
    K, V = ko.gather_kv(view, b, h)
    qh = q[b, h * 4:(h + 1) * 4, 0].float().cpu().numpy()
    m, l, acc = ko.attention_partial(qh, K, V, sc)
    assert ko.rel_err(fast[b, 0, h * 4:(h + 1) * 4], acc / l[:, None]) <= ATTN_TOL
    # quantized pages themselves: a sample of pages bit-exact with the oracle
    pages = ko.as_f32(k)[b, h, 32:32 + 3 * 128].reshape(3, 128, 128)
    idx = ko.rank_channels(ko.channel_score(pages, "bf16", "exact"), 32, "stable")
    rec, meta = ko.quantize_k_pages(pages, idx, 32)
    got = lay.KeyCache.cpu().numpy().reshape(-1, h_kv, 5248)
    for p in range(3):
        assert np.array_equal(got[b * lay.MAX_PAGE + p, h], rec[p])


def test_exchange_merge_single_rank_equals_lse_merge(kb):
    """World of one: the peer-memory combine publishes to its own buffer, waits for its own flag and
    normalises — the same result as kitty_lse_merge of one part, over several calls (both buffer halves)."""
    import ctypes

    from kitty_b200 import _lib

    rows = 28
    off = ctypes.c_int64(0)
    nbytes = _lib.lib().kitty_lse_exchange_bytes(rows, 1, ctypes.byref(off))
    assert nbytes == 2 * rows * 130 * 4 + 2 * rows * 4 and off.value == 2 * rows * 130 * 4
    buf = torch.zeros(nbytes // 4, dtype=torch.float32, device=DEV)
    table = torch.tensor([buf.data_ptr()], dtype=torch.int64, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    g = torch.Generator().manual_seed(4)
    for seq in range(1, 5):
        part = torch.randn(1, rows, 130, generator=g).to(DEV)
        part[..., 129] = part[..., 129].abs() + 0.5
        out = torch.empty(1, 1, rows, 128, dtype=torch.float32, device=DEV)
        rc = _lib.lib().kitty_lse_exchange_merge(part.data_ptr(), rows, table.data_ptr(), 0, 1, seq, out.data_ptr(),
                                                 _lib.KITTY_F32, status.data_ptr(), 0, _lib.stream_ptr(torch.device(DEV)))
        assert rc == 0
        want = kb.lse_merge(part.view(1, 1, rows, 130).contiguous(), torch.float32)
        assert torch.allclose(out, want, rtol=1e-6, atol=0)
    assert int(status.item()) == 0
    assert _lib.lib().kitty_lse_exchange_merge(part.data_ptr(), 2000, table.data_ptr(), 0, 1, 9, out.data_ptr(),
                                               _lib.KITTY_F32, None, 0, None) == _lib.KITTY_E_BADARG


def test_full_size_131k_group_of_7_properties(kb):
    """The long-context shape (28 query / 4 KV heads, batch 1, 131072 cached tokens: 1023 key pages, 1022 value
    pages): the fp16 streaming kernel agrees with the plain kernel, an 8-way split over the pages merges to the same
    result, and one head agrees with the oracle."""
    h_kv, h_q, B, L = 4, 28, 1, 131072
    g = torch.Generator().manual_seed(77)
    k = torch.randn(B, h_kv, L, 128, generator=g)
    for h in range(h_kv):
        k[:, h, :, torch.randperm(128, generator=g)[:4]] *= 8.0
    v = torch.randn(B, h_kv, L, 128, generator=g)
    k, v = k.bfloat16(), v.bfloat16()
    cache = kb.KittyCache(_cfg(1, h_kv, h_q), B, L + 256, device=DEV)
    cache.update(k.to(DEV), v.to(DEV), 0)
    cache.quantize_prefill(0)
    lay = cache.kv_cache[0]
    assert (lay.PageCount_K, lay.PageCount_V, lay.Q_Buffer_Count_K, lay.Q_Buffer_Count_V) == (1023, 1022, 96, 96)
    kt, vt = torch.randn(B, h_kv, 1, 128, generator=g).bfloat16(), torch.randn(B, h_kv, 1, 128, generator=g).bfloat16()
    cache.update(kt.to(DEV), vt.to(DEV), 0)
    q = torch.randn(B, h_q, 1, 128, generator=g).bfloat16().to(DEV)
    sc = 128 ** -0.5
    fast = kb.decode_attention(q, lay, h_kv, sc).float().cpu().numpy()
    plain = kb.decode_attention(q, lay, h_kv, sc, impl=1).float().cpu().numpy()
    assert ko.rel_err(fast, plain) <= ATTN_TOL
    from kitty_b200.seqsplit import rank_flags, split_pages

    parts = torch.empty(8, B, h_q, 130, dtype=torch.float32, device=DEV)
    for r, (lo, hi) in enumerate(split_pages(lay.PageCount_V, 8)):
        kb.decode_attention(q, lay, h_kv, sc, page_begin=lo, page_end=hi, flags=rank_flags(r, 8), partial_out=parts[r])
    merged = kb.lse_merge(parts, torch.bfloat16).float().cpu().numpy()
    assert ko.rel_err(merged, fast) <= ATTN_TOL
    view = types.SimpleNamespace(D=128, D_BOOSTED=32, H_KV=h_kv, **{n: getattr(lay, n).cpu().numpy() for n in BUFFERS},
                                 **{c: getattr(lay, c) for c in COUNTERS})
    h = 2
    K, V = ko.gather_kv(view, 0, h)
    qh = q[0, h * 7:(h + 1) * 7, 0].float().cpu().numpy()
    m, l, acc = ko.attention_partial(qh, K, V, sc)
    assert ko.rel_err(fast[0, 0, h * 7:(h + 1) * 7], acc / l[:, None]) <= ATTN_TOL
    assert kb.workspace_status(lay) == 0


def test_attention_with_exchange_in_a_world_of_one(kb):
    """kitty_decode_attn_exchange with a single rank (its merge kernel publishes to its own buffer and waits for its
    own flag) returns what kitty_decode_attn returns, for both streaming kernels and on consecutive calls."""
    import ctypes

    from kitty_b200 import _lib

    for h_kv, h_q in ((2, 8), (1, 7)):
        B, L = 2, 32 + 128 * 5 + 77
        cache = kb.KittyCache(_cfg(1, h_kv, h_q), B, L + 64, device=DEV)
        k, v = make_kv(B, h_kv, L, 128, 21, torch.float16)
        cache.update(k.to(DEV), v.to(DEV), 0)
        cache.quantize_prefill(0)
        lay = cache.kv_cache[0]
        rows = B * h_q
        off = ctypes.c_int64(0)
        nbytes = _lib.lib().kitty_lse_exchange_bytes(rows, 1, ctypes.byref(off))
        xch = types.SimpleNamespace(rows=rows, rank=0, world=1, seq=0, wait_ns=0,
                                    buf=torch.zeros(nbytes // 4, dtype=torch.float32, device=DEV),
                                    status=torch.zeros(1, dtype=torch.int32, device=DEV))
        table = torch.tensor([xch.buf.data_ptr()], dtype=torch.int64, device=DEV)
        xch.peer_table = table.data_ptr()
        g = torch.Generator().manual_seed(5)
        for step in range(3):
            kt, vt = torch.randn(B, h_kv, 1, 128, generator=g).half(), torch.randn(B, h_kv, 1, 128, generator=g).half()
            cache.update(kt.to(DEV), vt.to(DEV), 0)
            q = torch.randn(B, h_q, 1, 128, generator=g).half().to(DEV)
            want = kb.decode_attention(q, lay, h_kv, 0.088)
            got = kb.decode_attention(q, lay, h_kv, 0.088, exchange=xch)
            assert torch.equal(got, want), (h_q, step)
        assert xch.seq == 3 and int(xch.status.item()) == 0


def test_full_size_bulk_quantize_properties(kb):
    """One layer call of the bulk-quantize workload (65536 tokens x 8 KV heads, bf16, per-channel scales log-uniform
    in [1, 16]).  Properties that hold for every page at any size: each key page boosts exactly 32 channels whose
    slots are a permutation of 0..31 and whose scores are the 32 largest; every dequantized element is within half a
    step (plus the fp16 rounding of scale and minimum) of its input; and all 4096 page-heads of the call, keys and
    values, are bit-exact with the oracle."""
    H, T, P = 8, 65536, 512
    g = torch.Generator(device=DEV).manual_seed(31)
    sc = torch.exp(torch.rand(1, H, 1, 128, generator=g, device=DEV) * float(np.log(16.0)))
    k = (torch.randn(1, H, T, 128, generator=g, device=DEV) * sc).to(torch.bfloat16)
    v = (torch.randn(1, H, T, 128, generator=g, device=DEV) * sc).to(torch.bfloat16)
    kc, km, vc, vm, pt = _buffers(1, H, P)
    kb.quantize_pack_k(k, 0, P, pt, 0, kc, km, 128, 32)
    kb.quantize_pack_v(v, 0, P, pt, 0, vc, vm, 128)
    shifts = torch.tensor([0, 2, 4, 6], device=DEV, dtype=torch.uint8)

    def fields(b):                                       # [..., n] bytes -> [..., 4n] 2-bit fields, LSB first
        return ((b.unsqueeze(-1) >> shifts) & 3).flatten(-2)

    # ---- keys ---- //
    rec = kc.view(P, H, 5248)
    idx = rec[..., 5120:].to(torch.int64)                                          # [P, H, 128] slot or 32
    boosted = idx < 32
    assert bool((boosted.sum(-1) == 32).all())
    slots = torch.where(boosted, idx, torch.full_like(idx, 99)).sort(-1).values[..., :32]
    assert bool((slots == torch.arange(32, device=DEV)).all())
    x = k[0].float().view(H, P, 128, 128).permute(1, 0, 3, 2)                      # [P, H, channel, token]
    score = x.abs().mean(-1)
    kth = score.topk(32, dim=-1).values[..., -1:]
    assert bool((score[boosted].view(P, H, 32) >= kth * (1 - 1e-2)).all())         # scores are rounded to bf16 (spacing 2^-7): ties at the cut
    lo = fields(rec[..., :4096].reshape(P, H, 128, 32)).float()                    # [P, H, 128, 128]
    hi_rows = fields(rec[..., 4096:5120].reshape(P, H, 32, 32)).float()            # [P, H, slot, token]
    hi = torch.gather(hi_rows, 2, idx.clamp(max=31).unsqueeze(-1).expand(-1, -1, -1, 128)) * boosted.unsqueeze(-1)
    code = lo + 4.0 * hi
    assert bool((code[~boosted] <= 3).all())
    scale, mn = km.view(P, H, 128, 2)[..., 0].float().unsqueeze(-1), km.view(P, H, 128, 2)[..., 1].float().unsqueeze(-1)
    err = (code * scale + mn - x).abs()
    bound = 0.5 * scale + 16 * 2.0 ** -11 * scale + 2.0 ** -10 * mn.abs() + 1e-6
    assert bool((err <= bound).all())
    # ---- values ---- //
    vcode = fields(vc.view(P, H, 128, 32)).float()                                 # [P, H, token, channel]
    vscale = vm.view(P, H, 128, 2)[..., 0].float().unsqueeze(-1)
    vmn = vm.view(P, H, 128, 2)[..., 1].float().unsqueeze(-1)
    xv = v[0].float().view(H, P, 128, 128).permute(1, 0, 2, 3)
    verr = (vcode * vscale + vmn - xv).abs()
    assert bool((verr <= 0.5 * vscale + 4 * 2.0 ** -11 * vscale + 2.0 ** -10 * vmn.abs() + 1e-6).all())
    # ---- every page-head of the call against the oracle, bit for bit: codes, high plane, index bytes, fp16 (scale, min) ---- //
    kp = ko.as_f32(k[0].cpu()).reshape(H, P, 128, 128)
    oi = ko.rank_channels(ko.channel_score(kp, "bf16", "exact"), 32, "stable")
    orec, ometa = ko.quantize_k_pages(kp.reshape(-1, 128, 128), oi.reshape(-1, 128), 32)
    orec, ometa = orec.reshape(H, P, 5248).transpose(1, 0, 2), ometa.reshape(H, P, 128, 2).transpose(1, 0, 2, 3)
    assert np.array_equal(rec.cpu().numpy(), orec)
    assert np.array_equal(_f16_bits(km.view(P, H, 128, 2)), np.ascontiguousarray(ometa).view(np.int16))
    vp = ko.as_f32(v[0].cpu()).reshape(H * P, 128, 128)
    ovrec, ovmeta = ko.quantize_v_pages(vp)
    ovrec, ovmeta = ovrec.reshape(H, P, 4096).transpose(1, 0, 2), ovmeta.reshape(H, P, 128, 2).transpose(1, 0, 2, 3)
    assert np.array_equal(vc.view(P, H, 4096).cpu().numpy(), ovrec)
    assert np.array_equal(_f16_bits(vm.view(P, H, 128, 2)), np.ascontiguousarray(ovmeta).view(np.int16))
