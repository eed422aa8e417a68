"""kitty_b200 — B200 (sm_100a) implementation of Kitty's quantized KV-cache hot path.

Importing the package does not load the CUDA library; the first call does, and
raises if it has not been built (python -m kitty_b200.build).
"""
from ._lib import KittyError
from .attention import decode_attention, kitty_attention_forward, lse_merge, workspace_status
from .cache import KittyCache, get_kvcache_kitty
from .layer_state import KVCache_Layer
from .quant_pack import quantize_pack_k, quantize_pack_kv, quantize_pack_v

__all__ = ["KittyCache", "get_kvcache_kitty", "KVCache_Layer", "kitty_attention_forward", "decode_attention",
           "lse_merge", "quantize_pack_k", "quantize_pack_kv", "quantize_pack_v", "workspace_status", "KittyError"]
