"""The attention patch for stock HuggingFace models: wiring on CPU (fake cache),
end to end on a GPU (tiny random Llama)."""
import pytest
import torch


def _tiny(dtype=torch.float32):
    from transformers import LlamaConfig, LlamaForCausalLM

    torch.manual_seed(0)
    cfg = LlamaConfig(hidden_size=512, intermediate_size=1024, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, head_dim=128, vocab_size=1000, max_position_embeddings=4096)
    return cfg, LlamaForCausalLM(cfg).eval().to(dtype)


class _PrefillOnlyCache:
    def __init__(self):
        self.quantized = []

    def update(self, k, v, i):
        assert k.shape[1] == 2 and k.shape[-1] == 128
        return True

    def quantize_prefill(self, i):
        self.quantized.append(i)

    def get_seq_length(self, i=0):
        return 0

    def get_mask_sizes(self, cache_position, i=0):
        return (cache_position.shape[0] if hasattr(cache_position, "shape") else int(cache_position)), 0


def test_patched_prefill_equals_stock_model_on_cpu():
    from kitty_b200.hf_adapter import patch_model

    cfg, m = _tiny()
    _, stock = _tiny()
    stock.load_state_dict(m.state_dict())
    assert patch_model(m) == 2
    ids = torch.randint(0, 1000, (2, 24))
    c = _PrefillOnlyCache()
    with torch.no_grad():
        a = m.model(input_ids=ids, position_ids=torch.arange(24).unsqueeze(0), past_key_values=c, use_cache=True).last_hidden_state
        b = stock.model(input_ids=ids).last_hidden_state
    assert c.quantized == [0, 1]
    assert torch.allclose(a, b, atol=1e-5)


@pytest.mark.gpu
def test_greedy_decode_matches_stock_model_while_nothing_is_quantized():
    """Prompt of 100 tokens + 20 steps stays inside sink + Q-buffer + ring (all fp16): the patched model with the
    Kitty cache must follow the stock model with HF's own cache."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import kitty_b200 as kb
    from kitty_b200.hf_adapter import greedy_decode, patch_model

    cfg, m = _tiny(torch.float16)
    _, stock = _tiny(torch.float16)
    stock.load_state_dict(m.state_dict())
    m, stock = m.cuda(), stock.cuda()
    patch_model(m)
    ids = torch.randint(0, 1000, (3, 100), device="cuda")
    cache = kb.get_kvcache_kitty(cfg, 3, 512, device="cuda:0")
    got = greedy_decode(m, ids, 20, cache)
    want = stock.generate(ids, max_new_tokens=20, do_sample=False, eos_token_id=None, pad_token_id=0)[:, 100:]
    assert cache.get_seq_length(0) == 119
    agree = (got == want).float().mean().item()
    assert agree >= 0.9, agree        # random-init logits are nearly flat: allow a few fp16 near-ties


@pytest.mark.gpu
def test_greedy_decode_long_prompt_runs_through_flushes():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import kitty_b200 as kb
    from kitty_b200.hf_adapter import greedy_decode, patch_model

    cfg, m = _tiny(torch.bfloat16)
    m = m.cuda()
    patch_model(m)
    ids = torch.randint(0, 1000, (2, 700), device="cuda")
    cache = kb.get_kvcache_kitty(cfg, 2, 1024, device="cuda:0")
    out = greedy_decode(m, ids, 140, cache)
    assert out.shape == (2, 140) and int(out.min()) >= 0
    lay = cache.kv_cache[1]
    assert cache.get_seq_length(1) == 700 + 139
    assert lay.PageCount_K == (700 + 139 - 32) // 128 and lay.PageCount_V == lay.PageCount_K - 1


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_rope_kernel_is_bit_identical_to_the_elementwise_sequence(dtype):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from kitty_b200.hf_adapter import _rope, rope_decode_token

    g = torch.Generator().manual_seed(8)
    B, h_q, h_kv, D = 3, 8, 2, 128
    q = torch.randn(B, 1, h_q, D, generator=g).to(dtype).cuda()
    k = torch.randn(B, 1, h_kv, D, generator=g).to(dtype).cuda()
    for rows in (1, B):                                   # one position for all rows, or one per row
        ang = torch.rand(rows, 1, D // 2, generator=g) * 6.28
        ang = torch.cat([ang, ang], dim=-1)
        cos, sin = ang.cos().to(dtype).cuda(), ang.sin().to(dtype).cuda()
        want_q, want_k = _rope(q.transpose(1, 2), k.transpose(1, 2), cos, sin)
        got_q, got_k = rope_decode_token(q, k, cos, sin)
        assert got_q.is_contiguous() and got_k.is_contiguous()
        assert torch.equal(got_q, want_q) and torch.equal(got_k, want_k)


@pytest.mark.gpu
def test_eager_decode_with_one_call_per_layer_equals_three_calls():
    """The patched attention forward takes decode tokens through plan_step / step_layer / finish_step; switching
    that off (update -> kitty_attention_forward -> quantize_decode) must give the same tokens and the same cache."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import kitty_b200 as kb
    from kitty_b200.hf_adapter import greedy_decode, patch_model
    from tests.helpers import BUFFERS, COUNTERS

    cfg, m = _tiny(torch.bfloat16)
    m = m.cuda()
    patch_model(m)
    ids = torch.randint(0, 1000, (2, 32 + 128 * 2 + 120), device="cuda")
    outs, caches = [], []
    for fuse in (True, False):
        cache = kb.get_kvcache_kitty(cfg, 2, 1024, device="cuda:0")
        cache.fuse_eager_steps = fuse
        outs.append(greedy_decode(m, ids, 30, cache))
        caches.append(cache)
    assert torch.equal(outs[0], outs[1])
    for la, lb in zip(caches[0].kv_cache, caches[1].kv_cache):
        assert [getattr(la, c) for c in COUNTERS] == [getattr(lb, c) for c in COUNTERS]
        assert la.PageCount_K == 3            # the flush at step 8 went through both paths
        for n in BUFFERS:
            assert torch.equal(getattr(la, n), getattr(lb, n)), n


def test_patched_prefill_honours_the_padding_mask_on_cpu():
    """A left-padded batch: the stock model masks the padding; the patched forward must hand the same mask to its
    prompt attention (it used to run plain causal attention and silently attend to the padding)."""
    from kitty_b200.hf_adapter import patch_model

    cfg, m = _tiny()
    _, stock = _tiny()
    stock.load_state_dict(m.state_dict())
    patch_model(m)
    ids = torch.randint(0, 1000, (2, 24))
    mask = torch.ones(2, 24, dtype=torch.long)
    mask[1, :7] = 0                                            # sequence 1 starts with 7 padding tokens
    pos = (mask.cumsum(-1) - 1).clamp(min=0)
    with torch.no_grad():
        a = m.model(input_ids=ids, attention_mask=mask, position_ids=pos, past_key_values=_PrefillOnlyCache(),
                    use_cache=True).last_hidden_state
        b = stock.model(input_ids=ids, attention_mask=mask, position_ids=pos).last_hidden_state
        c = m.model(input_ids=ids, position_ids=pos, past_key_values=_PrefillOnlyCache(), use_cache=True).last_hidden_state
    real = mask.bool()
    assert torch.allclose(a[real], b[real], atol=1e-5)
    assert not torch.allclose(c[1, 7:], b[1, 7:], atol=1e-3)   # without the mask the padded row differs: the test bites


def test_patched_forward_accepts_the_singular_cache_keyword_and_rejects_sliding_windows():
    from kitty_b200.hf_adapter import patch_model

    cfg, m = _tiny()
    patch_model(m)
    attn = m.model.layers[0].self_attn
    hs = torch.randn(1, 5, 512)
    pos = m.model.rotary_emb(hs, torch.arange(5).unsqueeze(0))
    c = _PrefillOnlyCache()
    with torch.no_grad():
        out, _ = attn(hs, position_embeddings=pos, past_key_value=c)
    assert out.shape == (1, 5, 512) and c.quantized == [0]
    attn.sliding_window = 4096
    with pytest.raises(NotImplementedError):
        attn(hs, position_embeddings=pos, past_key_value=c)
