"""Use KittyCache with stock HuggingFace decoder models (Llama / Qwen3 style attention).

The reference ships a forked modeling file whose attention forward calls the
cache (src/kitty/models/qwen3/modeling_qwen3.py:203-255): update() -> prefill
attention + quantize_prefill(), or kitty_attention_forward() + quantize_decode().
`patch_model` installs that same call sequence on the attention modules of an
unmodified transformers model, so no forked model code is needed.
"""
from __future__ import annotations

import types

import torch
import torch.nn.functional as F

from .attention import kitty_attention_forward


def _rotate_half(x):
    x1, x2 = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2:]
    return torch.cat((-x2, x1), dim=-1)


def _rope(q, k, cos, sin):
    cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
    return (q * cos) + (_rotate_half(q) * sin), (k * cos) + (_rotate_half(k) * sin)


def rope_decode_token(q: torch.Tensor, k: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor):
    """Rotary embedding of one decode token in one launch (kitty_rope_qk), bit-identical to `_rope` on the transposed
    tensors.  q [B, 1, H_Q, D], k [B, 1, H, D] as the projections produce them; cos / sin [B or 1, 1, D].
    Returns q [B, H_Q, 1, D] and k [B, H, 1, D], contiguous."""
    from . import _lib

    B, t, h_q, D = q.shape
    h_kv = k.shape[2]
    assert t == 1 and D == 128 and q.is_contiguous() and k.is_contiguous()
    cos2, sin2 = cos.reshape(-1, D), sin.reshape(-1, D)
    if cos2.dtype != q.dtype:
        cos2, sin2 = cos2.to(q.dtype), sin2.to(q.dtype)
    cos2, sin2 = cos2.contiguous(), sin2.contiguous()
    assert cos2.shape[0] in (1, B) and sin2.shape == cos2.shape
    q_out = torch.empty((B, h_q, 1, D), dtype=q.dtype, device=q.device)
    k_out = torch.empty((B, h_kv, 1, D), dtype=k.dtype, device=k.device)
    rc = _lib.lib().kitty_rope_qk(q.data_ptr(), k.data_ptr(), cos2.data_ptr(), sin2.data_ptr(), q_out.data_ptr(),
                                  k_out.data_ptr(), _lib.dtype_code(q.dtype), B, h_q, h_kv,
                                  D if cos2.shape[0] == B and B > 1 else 0, _lib.stream_ptr(q.device))
    _lib.check(rc, "kitty_rope_qk")
    return q_out, k_out


def _prefill_attention(q, k, v, attention_mask, scaling):
    """Prompt attention on the full-precision K/V (models/qwen3/modeling_qwen3.py:228-242 hands the mask to the
    attention interface).  attention_mask: None (plain causal), or the model's 4-D mask — boolean (True = attend)
    or additive float — covering [B, 1, L, L]; a padded batch arrives that way."""
    if attention_mask is None:
        return F.scaled_dot_product_attention(q, k, v, is_causal=q.shape[-2] > 1, scale=scaling, enable_gqa=True)
    if attention_mask.dim() != 4:
        raise ValueError("the patched attention expects the model's 4-D attention mask, got shape "
                         f"{tuple(attention_mask.shape)}")
    mask = attention_mask[..., : k.shape[-2]]
    if mask.dtype != torch.bool:
        mask = mask.to(q.dtype)
    return F.scaled_dot_product_attention(q, k, v, attn_mask=mask, is_causal=False, scale=scaling, enable_gqa=True)


def kitty_attention_module_forward(self, hidden_states, position_embeddings=None, attention_mask=None,
                                   past_key_values=None, past_key_value=None, **kwargs):
    """Replacement for `<Model>Attention.forward` (projection layout of Llama / Qwen3).  The cache may arrive as
    `past_key_values` or, as in the reference's signature and older transformers, `past_key_value`.  Decode tokens
    ignore the mask, as the reference's decode path does (kernels/kitty_attention.py:403-526 takes none)."""
    if past_key_values is None:
        past_key_values = past_key_value
    if getattr(self, "sliding_window", None) is not None:
        raise NotImplementedError("the Kitty cache keeps every token: sliding-window attention layers are not supported")
    input_shape = hidden_states.shape[:-1]
    hidden_shape = (*input_shape, -1, self.head_dim)
    q = self.q_proj(hidden_states).view(hidden_shape)
    k = self.k_proj(hidden_states).view(hidden_shape)
    if getattr(self, "q_norm", None) is not None:          # Qwen3: RMSNorm on the head dimension
        q, k = self.q_norm(q), self.k_norm(k)
    v = self.v_proj(hidden_states).view(hidden_shape).transpose(1, 2)
    cos, sin = position_embeddings
    if q.shape[1] == 1 and q.is_cuda and q.shape[-1] == 128 and q.is_contiguous() and k.is_contiguous():
        q, k = rope_decode_token(q, k, cos, sin)          # one launch, same bits as the element-wise sequence
    else:
        q, k = _rope(q.transpose(1, 2), k.transpose(1, 2), cos, sin)
    assert past_key_values is not None, "the patched attention needs a KittyCache"
    cache = past_key_values
    if _fused_step_ok(cache, self.layer_idx, q, k, v):
        # decode token, all layers in step: one library call per layer (append + attention + flush-if-due from the
        # device-resident state) instead of three; same bits as the three calls
        if self.layer_idx == 0:
            cache.plan_step(q.shape[0], q.shape[1])
        out = cache.step_layer(self.layer_idx, k, v, q, self.scaling)
        if self.layer_idx == cache.num_hidden_layers - 1:
            cache.finish_step()
        return self.o_proj(out.reshape(*input_shape, -1)), None
    is_prefill = past_key_values.update(k, v, self.layer_idx)
    if is_prefill:
        out = _prefill_attention(q, k, v, attention_mask, self.scaling).transpose(1, 2)
        past_key_values.quantize_prefill(self.layer_idx)
    else:
        out, _ = kitty_attention_forward(self, q.contiguous(), past_key_values.kv_cache[self.layer_idx], self.scaling)
        past_key_values.quantize_decode(self.layer_idx)
    out = out.reshape(*input_shape, -1).contiguous()
    return self.o_proj(out), None


def _fused_step_ok(cache, layer_idx: int, q, k, v) -> bool:
    """The one-call decode step applies when the token is a decode token of a cache that selects channels in the
    kernel, the layers are visited in order from layer 0, and the tensors have the layout step_layer takes."""
    if not getattr(cache, "fuse_eager_steps", False) or getattr(cache, "selection", None) != "fused":
        return False
    if q.shape[-2] != 1 or not (q.is_contiguous() and k.stride(-1) == 1 and v.stride(-1) == 1 and k.dtype == v.dtype):
        return False
    if layer_idx == 0:
        lay0 = cache.kv_cache[0]
        # layer 0 always starts a new step; a ragged batch (per-row counters) takes the three-call path
        return lay0.Sink_Count > 0 and lay0.row_counts is None and q.shape[1] // lay0.H_KV <= 16
    return cache._step_host is not None           # a step planned at layer 0 is under way


def patch_model(model) -> int:
    """Install the Kitty call sequence on every self-attention module of `model`.  Returns how many were patched."""
    n = 0
    cfg = model.config.get_text_config() if hasattr(model.config, "get_text_config") else model.config
    for mod in model.modules():
        if all(hasattr(mod, a) for a in ("q_proj", "k_proj", "v_proj", "o_proj", "layer_idx")):
            mod.num_attention_heads = cfg.num_attention_heads
            mod.num_key_value_heads = cfg.num_key_value_heads
            mod.forward = types.MethodType(kitty_attention_module_forward, mod)
            n += 1
    return n


@torch.no_grad()
def greedy_decode(model, input_ids: torch.Tensor, steps: int, cache):
    """Prefill `input_ids` [B, L] then `steps` greedy tokens with `cache` (a KittyCache).  Returns [B, steps] ids.
    The method of the reference's latency benchmark (latency_benchmarking/benchmark_kitty.py:154-183):
    fresh cache, greedy, fixed length, no EOS stop."""
    B, L = input_ids.shape
    dev = input_ids.device
    pos = torch.arange(L, device=dev).unsqueeze(0)
    hs = model.model(input_ids=input_ids, position_ids=pos, past_key_values=cache, use_cache=True,
                     attention_mask=None).last_hidden_state
    tok = model.lm_head(hs[:, -1:, :]).argmax(-1)
    out = [tok]
    for s in range(1, steps):
        pos = torch.full((1, 1), L + s - 1, device=dev, dtype=torch.long)
        hs = model.model(input_ids=tok, position_ids=pos, past_key_values=cache, use_cache=True,
                         attention_mask=None).last_hidden_state
        tok = model.lm_head(hs).argmax(-1)
        out.append(tok)
    return torch.cat(out, dim=1)


class GraphedDecoder:
    """Greedy decode steps of a patched Llama / Qwen3 style model replayed from one CUDA graph.

    The reference's decode step costs ~10 kernel launches per layer issued from Python
    (kvcache/kitty.py:89-123, kernels/kitty_attention.py:403-526), which bounds its small-batch
    latency.  Here the whole token (embedding, every layer with `KittyCache.step_layer`, final norm,
    lm_head, argmax, position increment) is captured once; each later token is `plan_step()` (host
    arithmetic + one tiny launch), one graph launch, and `finish_step()`.  The graph stays valid for
    the life of the cache because the cache kernels read their counters from a device block.
    """

    def __init__(self, model, cache, batch: int, warmup: int = 2):
        self.model, self.cache, self.batch = model, cache, batch
        self.inner = model.model
        self.h_q = model.config.get_text_config().num_attention_heads if hasattr(model.config, "get_text_config") \
            else model.config.num_attention_heads
        dev = next(model.parameters()).device
        self.tok = torch.zeros((batch, 1), dtype=torch.long, device=dev)
        self.pos = torch.zeros((1, 1), dtype=torch.long, device=dev)
        self.graph = None
        self.warmup = warmup

    def _attention(self, attn, hidden_states, cos, sin):
        input_shape = hidden_states.shape[:-1]
        hidden_shape = (*input_shape, -1, attn.head_dim)
        q = attn.q_proj(hidden_states).view(hidden_shape)
        k = attn.k_proj(hidden_states).view(hidden_shape)
        if getattr(attn, "q_norm", None) is not None:
            q, k = attn.q_norm(q), attn.k_norm(k)
        v = attn.v_proj(hidden_states).view(hidden_shape).transpose(1, 2)      # [B, H, 1, D]: contiguous for one token
        q, k = rope_decode_token(q, k, cos, sin)                                # [B, H_Q, 1, D], [B, H, 1, D]
        out = self.cache.step_layer(attn.layer_idx, k, v, q, attn.scaling)
        return attn.o_proj(out.reshape(*input_shape, -1))

    def _token(self):
        """One decode step on the static buffers: tok <- argmax(model(tok at pos)); pos += 1."""
        m = self.inner
        hs = m.embed_tokens(self.tok)
        cos, sin = m.rotary_emb(hs, self.pos)
        for layer in m.layers:
            hs = hs + self._attention(layer.self_attn, layer.input_layernorm(hs), cos, sin)
            hs = hs + layer.mlp(layer.post_attention_layernorm(hs))
        nxt = self.model.lm_head(m.norm(hs)).argmax(-1)
        self.tok.copy_(nxt)
        self.pos.add_(1)

    @torch.no_grad()
    def step(self) -> torch.Tensor:
        """Advance every sequence by one token.  Returns the static [B, 1] token buffer (clone it to keep it)."""
        self.cache.plan_step(self.batch, self.h_q)
        if self.graph is None and self.warmup > 0:
            self.warmup -= 1                       # eager steps first: lazy initialisation must not be captured
            self._token()
        elif self.graph is None:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._token()
            self.graph = g
            g.replay()                             # capture records without running
        else:
            self.graph.replay()
        self.cache.finish_step()
        return self.tok

    @torch.no_grad()
    def generate(self, input_ids: torch.Tensor, steps: int) -> torch.Tensor:
        """Prefill (eager, through the patched modules) and `steps` greedy tokens.  Returns [B, steps]."""
        B, L = input_ids.shape
        pos = torch.arange(L, device=input_ids.device).unsqueeze(0)
        hs = self.inner(input_ids=input_ids, position_ids=pos, past_key_values=self.cache, use_cache=True,
                        attention_mask=None).last_hidden_state
        self.tok.copy_(self.model.lm_head(hs[:, -1:, :]).argmax(-1))
        self.pos.fill_(L)
        out = [self.tok.clone()]
        for _ in range(1, steps):
            out.append(self.step().clone())
        return torch.cat(out, dim=1)
