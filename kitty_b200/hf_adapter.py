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


def kitty_attention_module_forward(self, hidden_states, position_embeddings=None, attention_mask=None,
                                   past_key_values=None, **kwargs):
    """Replacement for `<Model>Attention.forward` (projection layout of Llama / Qwen3)."""
    input_shape = hidden_states.shape[:-1]
    hidden_shape = (*input_shape, -1, self.head_dim)
    q = self.q_proj(hidden_states).view(hidden_shape)
    k = self.k_proj(hidden_states).view(hidden_shape)
    if getattr(self, "q_norm", None) is not None:          # Qwen3: RMSNorm on the head dimension
        q, k = self.q_norm(q), self.k_norm(k)
    q, k = q.transpose(1, 2), k.transpose(1, 2)
    v = self.v_proj(hidden_states).view(hidden_shape).transpose(1, 2)
    cos, sin = position_embeddings
    q, k = _rope(q, k, cos, sin)
    assert past_key_values is not None, "the patched attention needs a KittyCache"
    is_prefill = past_key_values.update(k, v, self.layer_idx)
    if is_prefill:
        out = F.scaled_dot_product_attention(q, k, v, is_causal=q.shape[-2] > 1, scale=self.scaling, enable_gqa=True)
        out = out.transpose(1, 2)
        past_key_values.quantize_prefill(self.layer_idx)
    else:
        out, _ = kitty_attention_forward(self, q.contiguous(), past_key_values.kv_cache[self.layer_idx], self.scaling)
        past_key_values.quantize_decode(self.layer_idx)
    out = out.reshape(*input_shape, -1).contiguous()
    return self.o_proj(out), None


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
