"""The oracle must reproduce what the reference's own kernels produced
(fixtures written by tests/golden/make_golden.py)."""
import numpy as np
import pytest

from oracle import kitty_oracle as ko
from tests.helpers import BUFFERS, COUNTERS, load, tensor_from_raw

QUANT = ["quant_f16_outlier8", "quant_bf16_loguniform", "quant_f32_outlier8", "quant_f16_degenerate"]


def _pages(fx):
    dt = str(fx["dtype"])
    x = ko.as_f32(tensor_from_raw(fx["x"], dt))
    B, H, T, D = x.shape
    t0, P = int(fx["t_offset"]), int(fx["pages"])
    return dt, x[:, :, t0:t0 + P * 128].reshape(B, H, P, 128, D), int(fx["page_offset"])


@pytest.mark.parametrize("name", QUANT)
def test_quantize_bit_exact_with_reference(name):
    fx = load(name)
    dt, pages, poff = _pages(fx)
    B, H, P, _, D = pages.shape
    lay = ko.layout_k(D, 32)
    ref_k = fx["KeyCache"].reshape(-1, H, lay["head_bytes"])
    ref_idx = np.stack([ref_k[poff + p, :, lay["off_idx"]:] for p in range(P)], 1)[None]      # [1,H,P,D]
    # selection exactly as the reference executes it on this host
    idx = ko.rank_channels(ko.channel_score(pages, dt, "torch"), 32, "torch")
    assert np.array_equal(idx, ref_idx)
    rec, meta = ko.quantize_k_pages(pages.reshape(-1, 128, D), ref_idx.reshape(-1, D), 32)
    rec, meta = rec.reshape(B, H, P, -1), meta.reshape(B, H, P, D, 2)
    vrec, vmeta = ko.quantize_v_pages(pages.reshape(-1, 128, D))
    vrec, vmeta = vrec.reshape(B, H, P, -1), vmeta.reshape(B, H, P, 128, 2)
    for p in range(P):
        assert np.array_equal(rec[0, :, p], ref_k[poff + p])
        assert np.array_equal(meta[0, :, p].view(np.uint16), fx["KeyCache_metadata"][poff + p].view(np.uint16))
        assert np.array_equal(vrec[0, :, p].reshape(-1), fx["ValueCache"][poff + p])
        assert np.array_equal(vmeta[0, :, p].view(np.uint16), fx["ValueCache_metadata"][poff + p].view(np.uint16))
    # untouched pages stay zero
    assert not fx["KeyCache"][0].any() and not fx["KeyCache"][poff + P:].any()


@pytest.mark.parametrize("name", QUANT)
def test_exact_stable_selection_is_tie_equivalent(name):
    """The order-independent score and the lowest-channel-first tie rule pick
    the same scores at every rank as torch's mean/topk."""
    fx = load(name)
    dt, pages, _ = _pages(fx)
    s_torch = ko.channel_score(pages, dt, "torch")
    s_exact = ko.channel_score(pages, dt, "exact")
    if dt == "f32":
        # fp32 sums differ in the last place with the order of summation; ranks do not
        assert np.allclose(s_torch, s_exact, rtol=4e-7, atol=0)
        assert np.array_equal(ko.rank_channels(s_exact, 32, "stable"), ko.rank_channels(s_torch, 32, "torch"))
        return
    assert np.mean(s_torch != s_exact) < 2e-3
    same = s_torch == s_exact
    rows = same.all(-1)
    a = ko.rank_channels(s_exact, 32, "stable")
    b = ko.rank_channels(s_torch, 32, "torch")
    assert ko.selection_equivalent(s_exact[rows], a[rows], b[rows], 32)


def _replay(name):
    fx = load(name)
    k0, v0 = tensor_from_raw(fx["k_prefill"], "f16"), tensor_from_raw(fx["v_prefill"], "f16")
    B, H, L, D = k0.shape
    steps = fx["k_steps"].shape[0]
    cache = ko.OracleKittyCache(1, H, D, B, L + steps + 8, score_mode="torch", tie_rule="torch")
    return fx, cache, k0, v0


def _same_state(lay, fx, prefix):
    for n in BUFFERS:
        a, b = np.asarray(getattr(lay, n)), fx[prefix + n]
        if a.dtype == np.float16:
            a, b = a.view(np.uint16), b.view(np.uint16)
        assert np.array_equal(a, b), n
    got = [getattr(lay, c) for c in COUNTERS]
    assert got == list(fx[prefix + "counters"]), (got, fx[prefix + "counters"])


@pytest.mark.parametrize("name", ["cache_g4", "cache_g7_short"])
def test_cache_state_machine_and_attention(name):
    fx, cache, k0, v0 = _replay(name)
    lay = cache.kv_cache[0]
    assert cache.update(k0, v0, 0) is True
    cache.quantize_prefill(0)
    _same_state(lay, fx, "prefill_")
    h_q, scaling = int(fx["h_q"]), float(fx["scaling"])
    probes = list(fx["probe_steps"])
    worst = 0.0
    for s in range(fx["k_steps"].shape[0]):
        k = tensor_from_raw(fx["k_steps"][s], "f16")
        v = tensor_from_raw(fx["v_steps"][s], "f16")
        assert cache.update(k, v, 0) is False
        if s in probes:
            i = probes.index(s)
            assert cache.get_seq_length(0) == int(fx["attn_len"][i])
            q = tensor_from_raw(fx["q_steps"][s], "f16")
            out = ko.decode_attention(lay, q, h_q, scaling)
            ref = ko.as_f32(tensor_from_raw(fx["attn_out"][i], "f16"))
            # the reference rounds logits and probabilities to fp16; the oracle keeps float64
            worst = max(worst, ko.rel_err(out, ref))
        cache.quantize_decode(0)
    _same_state(lay, fx, "final_")
    assert worst <= 5e-3, worst


def test_prefill_partition_examples():
    # sink / K pages / K tail / V pages / V tail / ring for the benchmark lengths
    p = ko.prefill_partition(2048)
    assert (p["pages_k"], p["qbuf_k"], p["pages_v"], p["qbuf_v"], p["local_v"]) == (15, 96, 14, 96, 128)
    assert ko.prefill_partition(32768)["pages_k"] == 255 and ko.prefill_partition(32768)["pages_v"] == 254
    assert ko.prefill_partition(131072)["pages_k"] == 1023
    for L in [1, 31, 32, 33, 159, 160, 161, 288, 289]:
        p = ko.prefill_partition(L)
        assert p["sink"] + p["pages_k"] * 128 + p["qbuf_k"] == L
        assert p["sink"] + p["pages_v"] * 128 + p["qbuf_v"] + p["local_v"] == L
