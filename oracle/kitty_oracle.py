"""CPU oracle for the Kitty quantized KV-cache hot path.  TEST INFRASTRUCTURE ONLY.

This module restates, in numpy (IEEE fp32 arithmetic on the host), the algorithm
of the reference's quantize/pack kernels, its packed page format, its cache
state machine and its decode attention.  It is the checker for the CUDA library
and is never on the product path: only the test-suite, the smoke check and the
benchmark's CPU-baseline leg import it.

Parity status: PINNED.  tests/golden/ holds outputs of the reference's own
kernels (run on CPU through the Triton interpreter by tests/golden/make_golden.py)
and tests/test_oracle_golden.py requires this module to reproduce them
bit-for-bit (codes, high plane, index bytes, fp16 scale/min) and, for
attention, to the tolerance written in that test.

Reference files restated here (paths inside the reference project):
  src/kitty/kvcache/kernels/kitty_quant_pack.py   K/V quantize + pack, selection
  src/kitty/kvcache/utils_kv_per_layer.py         buffers and byte layout
  src/kitty/kvcache/kitty.py                      prefill / decode state machine
  src/kitty/kvcache/kernels/kitty_attention.py    decode attention
"""
from __future__ import annotations

import numpy as np

PAGE = 128          # tokens per page / quantization group   (kitty.py:43)
SINK = 32           # full-precision sink tokens             (kitty.py:45)
LOW_LEVELS = 3.0    # 2-bit codes 0..3                        (kitty_quant_pack.py:80)
HIGH_LEVELS = 15.0  # 4-bit codes 0..15                       (kitty_quant_pack.py:79)
SCALE_FLOOR = np.float32(1e-6)                              # (kitty_quant_pack.py:82)


# --------------------------------------------------------------------------- #
# dtype helpers
# --------------------------------------------------------------------------- #
def as_f32(t) -> np.ndarray:
    """Exact up-cast of a torch tensor / numpy array (fp16, bf16, fp32) to fp32."""
    if isinstance(t, np.ndarray):
        return t.astype(np.float32)
    import torch

    return t.detach().to("cpu", torch.float32).numpy()


def round_to_dtype(v64: np.ndarray, dtype: str) -> np.ndarray:
    """Round float64 values to `dtype` ('f16' | 'bf16' | 'f32') with ONE
    round-to-nearest-even step and return them as float64."""
    v64 = np.asarray(v64, dtype=np.float64)
    if dtype == "f32":
        return v64.astype(np.float32).astype(np.float64)
    bits = {"f16": 11, "bf16": 8}[dtype]
    m, e = np.frexp(v64)                       # v = m * 2**e, 0.5 <= |m| < 1
    out = np.ldexp(np.rint(m * (1 << bits)), e - bits)
    if dtype == "f16":                          # fixed spacing 2**-24 below 2**-14
        sub = np.abs(v64) < 2.0 ** -14
        out = np.where(sub, np.rint(v64 * 2.0 ** 24) * 2.0 ** -24, out)
    return out


def layout_k(D: int, d_boost: int):
    """Byte offsets inside one head's key record (kitty_quant_pack.py:42-45)."""
    row = PAGE * 2 // 8
    return dict(row=row, off_hi=row * D, off_idx=row * (D + d_boost),
                head_bytes=row * (D + d_boost) + D)


def layout_v(D: int):
    """Value record: one row of D/4 bytes per token (kitty_quant_pack.py:180-181)."""
    row = D * 2 // 8
    return dict(row=row, head_bytes=row * PAGE)


# --------------------------------------------------------------------------- #
# channel selection                       (kitty_quant_pack.py:280-288)
# --------------------------------------------------------------------------- #
def channel_score(x: np.ndarray, dtype: str, mode: str = "exact") -> np.ndarray:
    """Mean |x| over the page's tokens, rounded to the input dtype.

    x: [..., PAGE, D] fp32 (exact up-cast of the input).  Returns float64.
    mode 'exact': the infinitely precise mean rounded once — independent of any
    summation order, which is the contract the CUDA kernel implements.
    mode 'torch': literally `abs().mean(dim=-2)` in the input dtype on the host,
    as the reference calls it; used to pin this file to the golden vectors.
    """
    if mode == "torch":
        import torch

        tdt = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}[dtype]
        t = torch.from_numpy(np.ascontiguousarray(x)).to(tdt)
        return t.abs().mean(dim=-2).to(torch.float64).numpy()
    s = np.abs(x.astype(np.float64)).sum(axis=-2)      # exact for 16-bit inputs
    return round_to_dtype(s / x.shape[-2], dtype)


def rank_channels(score: np.ndarray, d_boost: int, rule: str = "stable") -> np.ndarray:
    """Dense→sparse index bytes: slot r (< d_boost) for the channel of rank r in
    descending score order, d_boost for every other channel.

    rule 'stable': equal scores are ordered by ascending channel number (the
    CUDA kernel's rule).  rule 'torch': `torch.topk` on the host, whose order
    among equal scores is unspecified (what the reference executes).
    """
    D = score.shape[-1]
    flat = score.reshape(-1, D)
    idx = np.full(flat.shape, d_boost, dtype=np.uint8)
    if d_boost == 0:
        return idx.reshape(score.shape)
    if rule == "torch":
        import torch

        _, top = torch.from_numpy(flat.copy()).topk(d_boost, dim=-1)
        top = top.numpy()
    else:
        top = np.argsort(-flat, axis=-1, kind="stable")[:, :d_boost]
    rows = np.arange(flat.shape[0])[:, None]
    idx[rows, top] = np.arange(d_boost, dtype=np.uint8)[None, :]
    return idx.reshape(score.shape)


def selection_equivalent(score: np.ndarray, idx_a: np.ndarray, idx_b: np.ndarray, d_boost: int) -> bool:
    """True when two index rows differ only by the order of equal scores: the
    score found at every rank is the same in both."""
    D = score.shape[-1]
    s = score.reshape(-1, D)
    a = idx_a.reshape(-1, D)
    b = idx_b.reshape(-1, D)
    for r in range(s.shape[0]):
        sa = np.full(d_boost, np.nan)
        sb = np.full(d_boost, np.nan)
        ma, mb = a[r] < d_boost, b[r] < d_boost
        sa[a[r][ma]] = s[r][ma]
        sb[b[r][mb]] = s[r][mb]
        if not np.array_equal(sa, sb):
            return False
    return True


# --------------------------------------------------------------------------- #
# quantize + pack
# --------------------------------------------------------------------------- #
def _pack4(codes: np.ndarray) -> np.ndarray:
    """Pack 2-bit codes along the last axis, 4 per byte, first code in the low
    bits (kitty_quant_pack.py:116-119)."""
    c = codes.reshape(*codes.shape[:-1], codes.shape[-1] // 4, 4).astype(np.uint8)
    return (c[..., 0] | (c[..., 1] << 2) | (c[..., 2] << 4) | (c[..., 3] << 6)).astype(np.uint8)


def _unpack4(packed: np.ndarray) -> np.ndarray:
    sh = np.array([0, 2, 4, 6], dtype=np.uint8)
    out = (packed[..., None] >> sh) & 3
    return out.reshape(*packed.shape[:-1], packed.shape[-1] * 4)


def quantize_k_pages(x: np.ndarray, idx: np.ndarray, d_boost: int):
    """Channel-wise quantization of key pages (kitty_quant_pack.py:75-125).

    x   [N, PAGE, D] fp32, idx [N, D] uint8.
    Returns (record [N, head_bytes] uint8, meta [N, D, 2] fp16).
    """
    x = x.astype(np.float32)
    N, P, D = x.shape
    lay = layout_k(D, d_boost)
    boosted = idx < d_boost                                   # [N, D]
    mx = x.max(axis=1)
    mn = x.min(axis=1)
    rng = (mx - mn).astype(np.float32)
    scale = np.where(boosted, rng / np.float32(HIGH_LEVELS), rng / np.float32(LOW_LEVELS)).astype(np.float32)
    scale = np.where(scale < SCALE_FLOOR, SCALE_FLOOR, scale).astype(np.float32)
    xf = ((x - mn[:, None, :]).astype(np.float32) / scale[:, None, :]).astype(np.float32)
    q = np.floor((xf + np.float32(0.5)).astype(np.float32))
    top = np.where(boosted, np.float32(HIGH_LEVELS), np.float32(LOW_LEVELS))[:, None, :]
    q = np.minimum(np.maximum(q, np.float32(0.0)), top).astype(np.uint8)   # [N, P, D]

    rec = np.zeros((N, lay["head_bytes"]), dtype=np.uint8)
    qt = q.transpose(0, 2, 1)                                 # [N, D, P]
    lo = _pack4(qt & 3)                                       # [N, D, P/4]
    rec[:, : lay["off_hi"]] = lo.reshape(N, -1)
    hi = _pack4((qt >> 2) & 3)                                # [N, D, P/4]
    hi_rows = rec[:, lay["off_hi"]: lay["off_idx"]].reshape(N, d_boost, lay["row"]) if d_boost else None
    if d_boost:
        n_i, d_i = np.nonzero(boosted)
        hi_rows[n_i, idx[n_i, d_i]] = hi[n_i, d_i]            # row = slot (kitty_quant_pack.py:137-144)
    rec[:, lay["off_idx"]:] = idx
    meta = np.stack([scale.astype(np.float16), mn.astype(np.float16)], axis=-1)
    return rec, meta


def quantize_v_pages(x: np.ndarray):
    """Per-token quantization of value pages (kitty_quant_pack.py:201-249).

    x [N, PAGE, D] fp32.  Returns (record [N, PAGE*D/4] uint8, meta [N, PAGE, 2] fp16).
    """
    x = x.astype(np.float32)
    N, P, D = x.shape
    mx = x.max(axis=2)
    mn = x.min(axis=2)
    scale = ((mx - mn).astype(np.float32) / np.float32(LOW_LEVELS)).astype(np.float32)
    scale = np.where(scale < SCALE_FLOOR, SCALE_FLOOR, scale).astype(np.float32)
    xf = ((x - mn[:, :, None]).astype(np.float32) / scale[:, :, None]).astype(np.float32)
    q = np.floor((xf + np.float32(0.5)).astype(np.float32))
    q = np.minimum(np.maximum(q, np.float32(0.0)), np.float32(LOW_LEVELS)).astype(np.uint8)
    rec = _pack4(q).reshape(N, -1)                            # token-major rows of D/4 bytes
    meta = np.stack([scale.astype(np.float16), mn.astype(np.float16)], axis=-1)
    return rec, meta


def dequantize_k_record(rec: np.ndarray, meta: np.ndarray, D: int, d_boost: int) -> np.ndarray:
    """[PAGE, D] fp16 keys rebuilt as the reference's decode kernel does:
    fp16(code) * scale + min in fp16 (kitty_attention.py:141-165)."""
    lay = layout_k(D, d_boost)
    lo = _unpack4(rec[: lay["off_hi"]].reshape(D, lay["row"]))          # [D, PAGE]
    idx = rec[lay["off_idx"]: lay["off_idx"] + D]
    hi_rows = rec[lay["off_hi"]: lay["off_idx"]].reshape(d_boost, lay["row"]) if d_boost else None
    code = lo.astype(np.uint8)
    if d_boost:
        b = idx < d_boost
        hi = np.zeros_like(lo)
        hi[b] = _unpack4(hi_rows[idx[b]])
        code = lo | (hi << 2)
    c16 = code.astype(np.float16)
    k = (c16 * meta[:, 0:1]).astype(np.float16) + meta[:, 1:2]
    return k.astype(np.float16).T                                       # [PAGE, D]


def dequantize_v_record(rec: np.ndarray, meta: np.ndarray, D: int) -> np.ndarray:
    """[PAGE, D] fp16 values (kitty_attention.py:312-320)."""
    code = _unpack4(rec.reshape(PAGE, D // 4)).astype(np.float16)
    v = (code * meta[:, 0:1]).astype(np.float16) + meta[:, 1:2]
    return v.astype(np.float16)


# --------------------------------------------------------------------------- #
# cache state machine
# --------------------------------------------------------------------------- #
def prefill_partition(L: int):
    """How a prompt of L tokens is split (kitty.py:131-136, 161-163)."""
    sink = min(SINK, L)
    qbuf_k = max(0, L - sink) % PAGE
    pages_k = (L - sink - qbuf_k) // PAGE
    local_v = max(0, min(PAGE, L - sink))
    qbuf_v = max(0, L - sink - local_v) % PAGE
    pages_v = (L - sink - local_v - qbuf_v) // PAGE
    return dict(sink=sink, qbuf_k=qbuf_k, pages_k=pages_k, local_v=local_v, qbuf_v=qbuf_v, pages_v=pages_v)


class OracleLayer:
    """Host copy of one layer's buffers with the reference's names and shapes
    (utils_kv_per_layer.py:18-83)."""

    def __init__(self, max_bs: int, max_len: int, h_kv: int, D: int, d_boost: int | None = None):
        self.MAX_BS, self.MAX_LEN, self.H_KV, self.D = max_bs, max_len, h_kv, D
        self.D_BOOSTED = D // 4 if d_boost is None else d_boost
        self.PAGE_SIZE, self.S = PAGE, SINK
        self.MAX_PAGE = -(-max_len // PAGE)
        lk, lv = layout_k(D, self.D_BOOSTED), layout_v(D)
        self.bytes_per_page_K = h_kv * lk["head_bytes"]
        self.bytes_per_page_V = h_kv * lv["head_bytes"]
        n = max_bs * self.MAX_PAGE
        self.KeyCache = np.zeros((n, self.bytes_per_page_K), np.uint8)
        self.KeyCache_metadata = np.zeros((n, h_kv, D, 2), np.float16)
        self.ValueCache = np.zeros((n, self.bytes_per_page_V), np.uint8)
        self.ValueCache_metadata = np.zeros((n, h_kv, PAGE, 2), np.float16)
        self.PageTable_K = np.arange(n, dtype=np.int64).reshape(max_bs, self.MAX_PAGE)
        self.PageTable_V = self.PageTable_K.copy()
        self.PageCount_K = self.PageCount_V = 0
        self.Sink_Buffer_K = np.zeros((max_bs, h_kv, SINK, D), np.float16)
        self.Sink_Buffer_V = np.zeros_like(self.Sink_Buffer_K)
        self.Sink_Count = 0
        self.Q_Buffer_K = np.zeros((max_bs, h_kv, PAGE, D), np.float16)
        self.Q_Buffer_V = np.zeros_like(self.Q_Buffer_K)
        self.Q_Buffer_Count_K = self.Q_Buffer_Count_V = 0
        self.Local_Buffer_V = np.zeros_like(self.Q_Buffer_K)
        self.Local_Count_V = 0
        self.Write_Offset_Local_V = 0
        self.key_states = None        # (fp32 array, dtype name) stashed by update()
        self.value_states = None

    def get_total_length(self) -> int:
        k = self.PageCount_K * PAGE + self.Sink_Count + self.Q_Buffer_Count_K
        v = self.PageCount_V * PAGE + self.Sink_Count + self.Q_Buffer_Count_V + self.Local_Count_V
        assert k == v, f"seqlen_K: {k}, seqlen_V: {v}"
        return k


class OracleKittyCache:
    """The reference cache's behaviour on host arrays (kitty.py:24-241).

    score_mode / tie_rule choose how boosted channels are picked:
    ('torch', 'torch') is what the reference executes on this host,
    ('exact', 'stable') is the order-independent contract of the CUDA kernels.
    A callable `select` (x_pages, dtype) -> idx overrides both.
    """

    def __init__(self, num_layers, h_kv, D, max_bs, max_len, score_mode="exact", tie_rule="stable", select=None):
        self.kv_cache = [OracleLayer(max_bs, max_len, h_kv, D) for _ in range(num_layers)]
        self.score_mode, self.tie_rule, self.select = score_mode, tie_rule, select

    # -- quantize helpers -------------------------------------------------- #
    def _pick(self, pages: np.ndarray, dtype: str, d_boost: int) -> np.ndarray:
        if self.select is not None:
            return self.select(pages, dtype)
        return rank_channels(channel_score(pages, dtype, self.score_mode), d_boost, self.tie_rule)

    def _pack_k(self, lay: OracleLayer, x: np.ndarray, dtype: str, t_off: int, n_pages: int, page_off: int):
        """quantize_pack_k (kitty_quant_pack.py:253-312): x [B, H, T, D] fp32."""
        B, H, _, D = x.shape
        pages = x[:, :, t_off: t_off + n_pages * PAGE, :].reshape(B, H, n_pages, PAGE, D)
        idx = self._pick(pages, dtype, lay.D_BOOSTED)                       # [B, H, n, D]
        rec, meta = quantize_k_pages(pages.reshape(-1, PAGE, D), idx.reshape(-1, D), lay.D_BOOSTED)
        hb = rec.shape[1]
        rec = rec.reshape(B, H, n_pages, hb)
        meta = meta.reshape(B, H, n_pages, D, 2)
        for b in range(B):
            for p in range(n_pages):
                pid = lay.PageTable_K[b, page_off + p]
                lay.KeyCache[pid] = rec[b, :, p].reshape(-1)
                lay.KeyCache_metadata[pid] = meta[b, :, p]

    def _pack_v(self, lay: OracleLayer, x: np.ndarray, t_off: int, n_pages: int, page_off: int):
        """quantize_pack_v (kitty_quant_pack.py:315-356)."""
        B, H, _, D = x.shape
        pages = x[:, :, t_off: t_off + n_pages * PAGE, :].reshape(B, H, n_pages, PAGE, D)
        rec, meta = quantize_v_pages(pages.reshape(-1, PAGE, D))
        rec = rec.reshape(B, H, n_pages, -1)
        meta = meta.reshape(B, H, n_pages, PAGE, 2)
        for b in range(B):
            for p in range(n_pages):
                pid = lay.PageTable_V[b, page_off + p]
                lay.ValueCache[pid] = rec[b, :, p].reshape(-1)
                lay.ValueCache_metadata[pid] = meta[b, :, p]

    # -- public surface ---------------------------------------------------- #
    def update(self, key_states, value_states, layer_idx: int, dtype: str = "f16") -> bool:
        """kitty.py:63-124.  key/value_states: [B, H, T, D] (any float array)."""
        lay = self.kv_cache[layer_idx]
        k, v = as_f32(key_states), as_f32(value_states)
        if lay.Sink_Count == 0:
            lay.key_states, lay.value_states = (k, dtype), (v, dtype)
            return True
        assert k.shape[-2] == 1 and v.shape[-2] == 1
        k16, v16 = k[:, :, 0, :].astype(np.float16), v[:, :, 0, :].astype(np.float16)
        if lay.Sink_Count < lay.S:
            lay.Sink_Buffer_K[:, :, lay.Sink_Count] = k16
            lay.Sink_Buffer_V[:, :, lay.Sink_Count] = v16
            lay.Sink_Count += 1
            return False
        assert lay.Q_Buffer_Count_K < PAGE
        lay.Q_Buffer_K[:, :, lay.Q_Buffer_Count_K] = k16
        lay.Q_Buffer_Count_K += 1
        if lay.Local_Count_V < PAGE:
            lay.Local_Buffer_V[:, :, lay.Local_Count_V] = v16
            lay.Local_Count_V += 1
        else:
            assert lay.Q_Buffer_Count_V < PAGE
            w = lay.Write_Offset_Local_V
            lay.Q_Buffer_V[:, :, lay.Q_Buffer_Count_V] = lay.Local_Buffer_V[:, :, w]
            lay.Q_Buffer_Count_V += 1
            lay.Local_Buffer_V[:, :, w] = v16
            lay.Write_Offset_Local_V = (w + 1) % PAGE
        return False

    def quantize_prefill(self, layer_idx: int = 0) -> None:
        """kitty.py:126-192."""
        lay = self.kv_cache[layer_idx]
        if lay.key_states is None or lay.value_states is None:
            raise ValueError("No key_states or value_states to quantize. Please call update() first.")
        (k, kd), (v, _) = lay.key_states, lay.value_states
        L = k.shape[-2]
        p = prefill_partition(L)
        s = p["sink"]
        lay.Sink_Buffer_K[:, :, :s] = k[:, :, :s].astype(np.float16)
        lay.Sink_Buffer_V[:, :, :s] = v[:, :, :s].astype(np.float16)
        lay.Sink_Count = s
        if p["qbuf_k"]:
            lay.Q_Buffer_K[:, :, : p["qbuf_k"]] = k[:, :, L - p["qbuf_k"]:].astype(np.float16)
            lay.Q_Buffer_Count_K = p["qbuf_k"]
        if p["pages_k"]:
            self._pack_k(lay, k, kd, s, p["pages_k"], 0)
            lay.PageCount_K += p["pages_k"]
        if p["local_v"]:
            lay.Local_Buffer_V[:, :, : p["local_v"]] = v[:, :, L - p["local_v"]:].astype(np.float16)
            lay.Local_Count_V = p["local_v"]
        if p["qbuf_v"]:
            a = L - p["local_v"] - p["qbuf_v"]
            lay.Q_Buffer_V[:, :, : p["qbuf_v"]] = v[:, :, a: a + p["qbuf_v"]].astype(np.float16)
            lay.Q_Buffer_Count_V = p["qbuf_v"]
        if p["pages_v"]:
            self._pack_v(lay, v, s, p["pages_v"], 0)
            lay.PageCount_V += p["pages_v"]
        lay.key_states = lay.value_states = None

    def quantize_decode(self, layer_idx: int = 0) -> None:
        """kitty.py:194-236: a full Q-buffer becomes the next page."""
        lay = self.kv_cache[layer_idx]
        if lay.Q_Buffer_Count_K == PAGE:
            self._pack_k(lay, lay.Q_Buffer_K.astype(np.float32), "f16", 0, 1, lay.PageCount_K)
            lay.PageCount_K += 1
            lay.Q_Buffer_Count_K = 0
        if lay.Q_Buffer_Count_V == PAGE:
            self._pack_v(lay, lay.Q_Buffer_V.astype(np.float32), 0, 1, lay.PageCount_V)
            lay.PageCount_V += 1
            lay.Q_Buffer_Count_V = 0

    def get_seq_length(self, layer_idx: int = 0) -> int:
        return self.kv_cache[layer_idx].get_total_length()


# --------------------------------------------------------------------------- #
# decode attention                         (kitty_attention.py:16-526)
# --------------------------------------------------------------------------- #
def gather_kv(lay, b: int, h: int):
    """Dequantized fp16 K [T, D] and V [T, D] of one (batch, kv-head) in the
    token order the reference's kernels walk: K = sink | pages | Q-buffer,
    V = sink | pages | Q-buffer | ring in age order."""
    D, db = lay.D, lay.D_BOOSTED
    lk, lv = layout_k(D, db), layout_v(D)

    def arr(x):
        return np.asarray(x)

    ks = [arr(lay.Sink_Buffer_K)[b, h, : lay.Sink_Count]]
    for i in range(lay.PageCount_K):
        pid = int(arr(lay.PageTable_K)[b, i])
        rec = arr(lay.KeyCache)[pid, h * lk["head_bytes"]: (h + 1) * lk["head_bytes"]]
        ks.append(dequantize_k_record(rec, arr(lay.KeyCache_metadata)[pid, h], D, db))
    ks.append(arr(lay.Q_Buffer_K)[b, h, : lay.Q_Buffer_Count_K])
    vs = [arr(lay.Sink_Buffer_V)[b, h, : lay.Sink_Count]]
    for i in range(lay.PageCount_V):
        pid = int(arr(lay.PageTable_V)[b, i])
        rec = arr(lay.ValueCache)[pid, h * lv["head_bytes"]: (h + 1) * lv["head_bytes"]]
        vs.append(dequantize_v_record(rec, arr(lay.ValueCache_metadata)[pid, h], D))
    vs.append(arr(lay.Q_Buffer_V)[b, h, : lay.Q_Buffer_Count_V])
    order = (np.arange(PAGE) + lay.Write_Offset_Local_V) % PAGE       # kitty_attention.py:373-374
    vs.append(arr(lay.Local_Buffer_V)[b, h][order][: lay.Local_Count_V])
    return np.concatenate(ks, 0), np.concatenate(vs, 0)


def attention_partial(q: np.ndarray, K: np.ndarray, V: np.ndarray, scaling: float):
    """(max, sum, unnormalised acc) of softmax(q K^T * scaling) V in float64, for
    a slice of the sequence.  q [G, D]."""
    s = (q.astype(np.float64) @ K.astype(np.float64).T) * scaling
    m = s.max(axis=-1) if s.shape[-1] else np.full(q.shape[0], -np.inf)
    p = np.exp(s - m[:, None]) if s.shape[-1] else np.zeros_like(s)
    return m, p.sum(-1), p @ V.astype(np.float64)


def merge_partials(parts):
    """Log-sum-exp combination of (m, l, acc) partials → normalised output."""
    m = np.max(np.stack([p[0] for p in parts]), axis=0)
    l = sum(p[1] * np.exp(p[0] - m) for p in parts)
    acc = sum(p[2] * np.exp(p[0] - m)[:, None] for p in parts)
    return acc / l[:, None]


def decode_attention(lay, query, h_q: int, scaling: float) -> np.ndarray:
    """Decode attention of one query token over the whole cache, as
    kitty_attention_forward computes it but in float64 after the fp16
    dequantization.  query [B, H_Q, 1, D] → [B, 1, H_Q, D] float64."""
    q = as_f32(query)
    B, _, _, D = q.shape
    G = h_q // lay.H_KV
    out = np.zeros((B, 1, h_q, D))
    for b in range(B):
        for h in range(lay.H_KV):
            K, V = gather_kv(lay, b, h)
            m, l, acc = attention_partial(q[b, h * G: (h + 1) * G, 0], K, V, scaling)
            out[b, 0, h * G: (h + 1) * G] = acc / l[:, None]
    return out


def rel_err(a: np.ndarray, b: np.ndarray) -> float:
    """max|a-b| / max|b| — the attention tolerance metric."""
    return float(np.max(np.abs(np.asarray(a, np.float64) - np.asarray(b, np.float64))) / np.max(np.abs(b)))
