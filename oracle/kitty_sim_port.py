"""CPU baseline: the reference's PyTorch (fake-quant) path.  TEST/BENCH INFRASTRUCTURE ONLY.

The reference ships a second, pure-PyTorch implementation of the same cache for
its accuracy runs (src/kitty_sim): keys are fake-quantized channel-wise per
128-token group with the top-|x| channels promoted to 4 bit, values per token,
and attention is plain eager attention over the dequantized tensors.  That is
the reference's CPU-runnable path; this file restates it so that the benchmark
can time it on the GPU box's host cores, where the reference checkout does not
exist.  It is never imported by the product package.  Pinned: tests/test_sim_port_golden.py
compares it bit for bit with outputs of the reference's own simulator (tests/golden/sim_port.npz).

Restated from (paths inside the reference project):
  src/kitty_sim/utils_quant.py:12-114      build_promote_mask, fake_quant_groupwise_lastdim
  src/kitty_sim/kitty_simulate.py:170-252  KittyKVCache.update (prefill / decode bookkeeping)
  src/kitty/models/qwen3/modeling_qwen3.py:132-167  repeat_kv + eager attention
"""
from __future__ import annotations

import torch


def promote_mask_magnitude(key_t: torch.Tensor, ratio: float) -> torch.Tensor:
    """key_t [B, H, D, T] -> bool [B, H, D]: the channels with the largest mean |x| (utils_quant.py:30-53)."""
    B, H, D, _ = key_t.shape
    k = max(0, min(int(D * ratio + 1e-6), D))
    mask = torch.zeros((B, H, D), dtype=torch.bool)
    if k == 0:
        return mask
    if k >= D:
        return ~mask
    _, top = key_t.abs().mean(dim=-1).topk(k, dim=-1)
    mask.scatter_(-1, top, True)
    return mask


def fake_quant_lastdim(x: torch.Tensor, group: int, bit: int, mask: torch.Tensor | None = None,
                       promote_bit: int = 4) -> torch.Tensor:
    """Quantize-dequantize along the last dim in groups (utils_quant.py:63-114): clamp, round half to even."""
    B, H, D, T = x.shape
    g = x.contiguous().view(B, H, D, T // group, group)
    mn = g.min(dim=-1, keepdim=True).values
    mx = g.max(dim=-1, keepdim=True).values
    eps = 1e-4 if x.dtype in (torch.float16, torch.bfloat16) else 1e-6
    rng = (mx - mn).clamp(min=eps)
    if mask is not None:
        m = mask.view(B, H, D, 1, 1)
        scale = torch.where(m, rng / (2 ** promote_bit - 1), rng / (2 ** bit - 1))
        top = torch.where(m, torch.full_like(scale, 2 ** promote_bit - 1), torch.full_like(scale, 2 ** bit - 1))
    else:
        scale = rng / (2 ** bit - 1)
        top = torch.full_like(scale, 2 ** bit - 1)
    q = ((g - mn) / scale).clamp(torch.zeros_like(top), top).round()
    return (q * scale + mn).view(B, H, D, T).to(x.dtype)


class SimKittyCache:
    """One layer of the simulated cache (kitty_simulate.py:170-252) with the real cache's hyper-parameters:
    sink 32, group/buffer 128, 2-bit keys and values, 25 % of the key channels promoted to 4 bit."""

    def __init__(self, sink=32, buffer=128, group=128, kbits=2, vbits=2, ratio=0.25, promote_bit=4):
        self.sink, self.buffer, self.group = sink, buffer, group
        self.kbits, self.vbits, self.ratio, self.promote_bit = kbits, vbits, ratio, promote_bit
        self.k = self.v = None

    def _quant_k(self, sl: torch.Tensor) -> torch.Tensor:
        t = sl.transpose(2, 3).contiguous()
        mask = promote_mask_magnitude(t, self.ratio)
        return fake_quant_lastdim(t, self.group, self.kbits, mask, self.promote_bit).transpose(2, 3).contiguous()

    def update(self, k: torch.Tensor, v: torch.Tensor):
        if self.k is None:                                   # prefill
            self.k, self.v = k.detach().clone(), v.detach().clone()
            keys, values = self.k.detach().clone(), self.v.detach().clone()   # post-quant: the prompt step sees full precision
            L = self.k.shape[-2]
            if L > self.sink + self.buffer:
                n = L - self.sink
                n_q = n - n % self.buffer
                for i in range(self.sink, self.sink + n_q, self.buffer):
                    self.k[:, :, i:i + self.buffer] = self._quant_k(self.k[:, :, i:i + self.buffer])
                end = self.sink + n - self.buffer            # values: everything but the newest `buffer` tokens
                self.v[:, :, self.sink:end] = fake_quant_lastdim(self.v[:, :, self.sink:end], self.group, self.vbits)
            return keys, values
        self.k = torch.cat([self.k, k], dim=-2)
        self.v = torch.cat([self.v, v], dim=-2)
        keys, values = self.k.detach().clone(), self.v.detach().clone()      # post-quant: this step sees full precision
        n = self.k.shape[-2] - self.sink - self.buffer
        if n > 0 and n % self.buffer == 1:
            self.k[:, :, -self.buffer - 1:-1] = self._quant_k(self.k[:, :, -self.buffer - 1:-1])
        if n > 0:
            s = self.v[:, :, -self.buffer - 1:-self.buffer]
            self.v[:, :, -self.buffer - 1:-self.buffer] = fake_quant_lastdim(s, self.group, self.vbits)
        return keys, values


def eager_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scaling: float) -> torch.Tensor:
    """q [B, H_Q, 1, D], k/v [B, H_KV, T, D] -> [B, 1, H_Q, D] (modeling_qwen3.py:132-167, no mask at decode)."""
    B, H_KV, T, D = k.shape
    rep = q.shape[1] // H_KV
    kk = k[:, :, None].expand(B, H_KV, rep, T, D).reshape(B, H_KV * rep, T, D)
    vv = v[:, :, None].expand(B, H_KV, rep, T, D).reshape(B, H_KV * rep, T, D)
    w = torch.matmul(q, kk.transpose(2, 3)) * scaling
    w = torch.nn.functional.softmax(w, dim=-1, dtype=torch.float32).to(q.dtype)
    return torch.matmul(w, vv).transpose(1, 2).contiguous()


def decode_step(cache: SimKittyCache, q, k, v, scaling: float) -> torch.Tensor:
    keys, values = cache.update(k, v)
    return eager_attention(q, keys, values, scaling)
