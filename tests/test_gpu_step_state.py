"""The decode step with device-resident state (kitty_plan_step + kitty_decode_step) must leave the
cache and the attention output bit-identical to the three reference-shaped calls
(update -> kitty_attention_forward -> quantize_decode), eagerly and when replayed from a CUDA graph.
Needs a B200: run with -m gpu."""
import types

import pytest
import torch

from tests.helpers import BUFFERS, COUNTERS, make_kv

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def kb():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import kitty_b200

    return kitty_b200


def _cfg(layers, h_kv, h_q):
    return types.SimpleNamespace(num_hidden_layers=layers, head_dim=128, num_key_value_heads=h_kv,
                                 num_attention_heads=h_q, hidden_size=128 * h_q)


def _prefilled(kb, cfg, B, L, seed, max_len):
    cache = kb.get_kvcache_kitty(cfg, B, max_len, device=DEV)
    for i in range(cfg.num_hidden_layers):
        k, v = make_kv(B, cfg.num_key_value_heads, L, 128, seed + i)
        assert cache.update(k.to(DEV), v.to(DEV), i) is True
        cache.quantize_prefill(i)
    return cache


def _same(a, b):
    for la, lb in zip(a.kv_cache, b.kv_cache):
        assert [getattr(la, c) for c in COUNTERS] == [getattr(lb, c) for c in COUNTERS]
        for n in BUFFERS:
            assert torch.equal(getattr(la, n), getattr(lb, n)), n


def _inputs(B, h_kv, h_q, step, layer):
    g = torch.Generator().manual_seed(1000 * step + layer)
    k = torch.randn(B, h_kv, 1, 128, generator=g).half().to(DEV)
    v = torch.randn(B, h_kv, 1, 128, generator=g).half().to(DEV)
    q = torch.randn(B, h_q, 1, 128, generator=g).half().to(DEV)
    return k, v, q


@pytest.mark.parametrize("L,steps,h_kv,h_q", [(10, 60, 2, 8), (32 + 128 * 2 + 120, 24, 2, 8), (32 + 128 + 127, 140, 2, 8),
                                              (32 + 128 * 2 + 120, 24, 1, 7), (20, 50, 1, 12)])
def test_step_state_path_is_bit_identical(kb, L, steps, h_kv, h_q):
    """Short prompt (sink and ring still filling), a key flush after 8 steps, and a run long enough for a value
    flush: same outputs, same buffers, same counters after every step.  Groups of 4 query heads per KV head take
    the int8 streaming kernel, 7 and 12 the fp16 one."""
    B, layers = 3, 2
    cfg = _cfg(layers, h_kv, h_q)
    ref = _prefilled(kb, cfg, B, L, 5, 1024)
    dyn = _prefilled(kb, cfg, B, L, 5, 1024)
    mod = types.SimpleNamespace(num_attention_heads=h_q, num_key_value_heads=h_kv)
    flushed_k = flushed_v = 0
    for s in range(steps):
        st = dyn.plan_step(B, h_q)
        flushed_k += st.flush_k
        flushed_v += st.flush_v
        for i in range(layers):
            k, v, q = _inputs(B, h_kv, h_q, s, i)
            assert ref.update(k, v, i) is False
            want, _ = kb.kitty_attention_forward(mod, q, ref.kv_cache[i], 0.09)
            ref.quantize_decode(i)
            got = dyn.step_layer(i, k, v, q, 0.09)
            assert torch.equal(got, want), (s, i)
        dyn.finish_step()
        _same(dyn, ref)
        assert kb.workspace_status(dyn.kv_cache[0]) == 0
    if L > 32:
        assert flushed_k >= 1
    if steps >= 140:
        assert flushed_v >= 1


def test_step_state_graph_replay(kb):
    """One captured step (two layers) replayed across a key flush and into the next page."""
    B, h_kv, h_q, layers = 2, 2, 8, 2
    L = 32 + 128 * 3 + 122
    cfg = _cfg(layers, h_kv, h_q)
    ref = _prefilled(kb, cfg, B, L, 9, 1024)
    dyn = _prefilled(kb, cfg, B, L, 9, 1024)
    mod = types.SimpleNamespace(num_attention_heads=h_q, num_key_value_heads=h_kv)
    sk = [torch.zeros(B, h_kv, 1, 128, dtype=torch.float16, device=DEV) for _ in range(layers)]
    sv = [torch.zeros_like(t) for t in sk]
    sq = [torch.zeros(B, h_q, 1, 128, dtype=torch.float16, device=DEV) for _ in range(layers)]
    so = [torch.zeros(B, 1, h_q, 128, dtype=torch.float16, device=DEV) for _ in range(layers)]

    def run_layers():
        for i in range(layers):
            dyn.step_layer(i, sk[i], sv[i], sq[i], 0.09, out=so[i])

    graph = None
    for s in range(20):
        ins = [_inputs(B, h_kv, h_q, s, i) for i in range(layers)]
        for i, (k, v, q) in enumerate(ins):
            sk[i].copy_(k), sv[i].copy_(v), sq[i].copy_(q)
        dyn.plan_step(B, h_q)
        if s < 2:
            run_layers()
        elif graph is None:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                run_layers()
            graph.replay()
        else:
            graph.replay()
        dyn.finish_step()
        for i, (k, v, q) in enumerate(ins):
            ref.update(k, v, i)
            want, _ = kb.kitty_attention_forward(mod, q, ref.kv_cache[i], 0.09)
            ref.quantize_decode(i)
            assert torch.equal(so[i], want), (s, i)
        _same(dyn, ref)
    assert ref.kv_cache[0].PageCount_K == 4          # 3 pages from the prompt + the flush at step 6


def test_plan_step_rejects_what_it_cannot_run(kb):
    cfg = _cfg(1, 1, 32)                     # 32 query heads per KV head: more than any kernel takes
    cache = kb.get_kvcache_kitty(cfg, 1, 512, device=DEV)
    with pytest.raises(kb.KittyError):
        cache.plan_step(1, 32)
    cfg = _cfg(2, 2, 8)
    cache = kb.get_kvcache_kitty(cfg, 1, 512, device=DEV)
    cache.kv_cache[1].Sink_Count = 3         # layers out of step
    with pytest.raises(ValueError):
        cache.plan_step(1, 8)


def test_graphed_decoder_follows_the_eager_adapter(kb):
    """Tiny Llama: tokens from the graph-replayed decoder equal those of the eager patched model."""
    from transformers import LlamaConfig, LlamaForCausalLM

    from kitty_b200.hf_adapter import GraphedDecoder, greedy_decode, patch_model

    torch.manual_seed(0)
    cfg = LlamaConfig(hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=8,
                      num_key_value_heads=2, head_dim=128, vocab_size=1000, max_position_embeddings=2048)
    m = LlamaForCausalLM(cfg).to(torch.bfloat16).eval().cuda()
    patch_model(m)
    ids = torch.randint(0, 1000, (2, 32 + 128 * 2 + 120), device="cuda")
    want = greedy_decode(m, ids, 24, kb.get_kvcache_kitty(cfg, 2, 1024, device=DEV))
    cache = kb.get_kvcache_kitty(cfg, 2, 1024, device=DEV)
    dec = GraphedDecoder(m, cache, 2)
    got = dec.generate(ids, 24)
    assert dec.graph is not None
    assert cache.get_seq_length(0) == ids.shape[1] + 23
    assert torch.equal(got, want)


def test_pooled_pages_match_identity_tables(kb):
    """A cache whose page rows come from a shuffled pool (fewer rows than the static worst case) must give the same
    attention outputs and hold the same page bytes, seen through its tables, as the reference-style static cache —
    across prefill, decode steps with key and value flushes, and a reset followed by a second batch."""
    B, h_kv, h_q, layers, max_len = 2, 2, 8, 1, 4096            # static: 2 * 32 rows per tensor
    cfg = _cfg(layers, h_kv, h_q)
    mod = types.SimpleNamespace(num_attention_heads=h_q, num_key_value_heads=h_kv)
    g = torch.Generator().manual_seed(3)
    order = torch.randperm(12, generator=g).tolist()
    pooled = kb.get_kvcache_kitty(cfg, B, max_len, device=DEV, num_pages=12, page_order=order)
    for round_ in range(2):
        L = 32 + 128 * 2 + 120 + 7 * round_
        static = kb.get_kvcache_kitty(cfg, B, max_len, device=DEV)
        k, v = make_kv(B, h_kv, L, 128, 40 + round_)
        for c in (static, pooled):
            assert c.update(k.to(DEV), v.to(DEV), 0) is True
            c.quantize_prefill(0)
        for s in range(140):
            kk, vv, q = _inputs(B, h_kv, h_q, s + 1000 * round_, 0)
            outs = []
            for c in (static, pooled):
                c.update(kk, vv, 0)
                outs.append(kb.kitty_attention_forward(mod, q, c.kv_cache[0], 0.09)[0])
                c.quantize_decode(0)
            assert torch.equal(outs[0], outs[1]), (round_, s)
        ls, lp = static.kv_cache[0], pooled.kv_cache[0]
        assert [getattr(ls, n) for n in COUNTERS] == [getattr(lp, n) for n in COUNTERS]
        assert ls.PageCount_K >= 4 and ls.PageCount_V >= 3
        for cache_name, table_name, count in (("KeyCache", "PageTable_K", ls.PageCount_K),
                                              ("ValueCache", "PageTable_V", ls.PageCount_V)):
            rows_s = getattr(ls, cache_name)[getattr(ls, table_name)[:, :count].reshape(-1)]
            rows_p = getattr(lp, cache_name)[getattr(lp, table_name)[:, :count].reshape(-1)]
            assert torch.equal(rows_s, rows_p), cache_name
        assert not torch.equal(lp.PageTable_K[:, :ls.PageCount_K], ls.PageTable_K[:, :ls.PageCount_K])
        assert lp.pool_K.available() == 12 - B * (ls.PageCount_K + 1)
        pooled.reset()
        assert lp.pool_K.available() == 12 and lp.pool_V.available() == 12 and pooled.get_seq_length(0) == 0
    small = kb.get_kvcache_kitty(cfg, B, max_len, device=DEV, num_pages=4)
    k, v = make_kv(B, h_kv, 32 + 128 * 3, 128, 50)
    small.update(k.to(DEV), v.to(DEV), 0)
    with pytest.raises(MemoryError):
        small.quantize_prefill(0)
