"""Generate tests/golden/sim_port.npz by EXECUTING THE REFERENCE's PyTorch simulator (src/kitty_sim) on the CPU.

    python tests/golden/make_sim_golden.py /path/to/Kitty

The fixture pins oracle/kitty_sim_port.py, the restatement of that simulator which the benchmark times as the
reference's CPU path.  Two things are adapted at run time so that the reference imports under the installed
transformers, and nothing else: `transformers.cache_utils.CacheConfig` (removed upstream) is stubbed with a class
that stores `cache_implementation`, and the `key_cache` / `value_cache` lists that `DynamicCache` no longer creates
are added to the cache object after construction.  Every array in the fixture is an input to or an output of the
reference's own functions: build_promote_mask, fake_quant_groupwise_lastdim (utils_quant.py) and KittyKVCache.update
(kitty_simulate.py), with the real cache's hyper-parameters (sink 32, buffer/group 128, 2-bit K and V, 25 % of the
key channels promoted to 4 bit, magnitude selection, KIVI-style value cache, PostQuant).
"""
from __future__ import annotations

import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def load_sim(ref_root: str):
    import transformers.cache_utils as cu

    if not hasattr(cu, "CacheConfig"):
        class CacheConfig:                       # the removed base class: it only stored the implementation name
            def __init__(self, cache_implementation=None):
                self.cache_implementation = cache_implementation

        cu.CacheConfig = CacheConfig
    src = os.path.join(ref_root, "src")
    sys.path.insert(0, src)
    spec = importlib.util.spec_from_file_location("kitty_sim_utils_quant", os.path.join(src, "kitty_sim", "utils_quant.py"))
    uq = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(uq)
    import kitty_sim.kitty_simulate as ks

    return uq, ks


def main():
    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("KITTY_REFERENCE", "")
    uq, ks = load_sim(ref_root)
    g = torch.Generator().manual_seed(0)
    out = {}
    # ---- the two functions on one key slice and one value slice ---- #
    ksl = torch.randn(1, 1, 128, 128, generator=g)                      # [B, nh, D, T]
    ksl[:, :, torch.randperm(128, generator=g)[:4]] *= 8.0
    mask = uq.build_promote_mask(ksl, 0.25, 1)
    out["fq_key_in"] = ksl.numpy()
    out["fq_mask"] = mask.numpy()
    out["fq_key_out"] = uq.fake_quant_groupwise_lastdim(ksl, 128, 2, mask, 4).numpy()
    vsl = torch.randn(1, 1, 64, 128, generator=g)
    out["fq_val_in"] = vsl.numpy()
    out["fq_val_out"] = uq.fake_quant_groupwise_lastdim(vsl, 128, 2).numpy()
    h16 = torch.randn(1, 1, 16, 128, generator=g).half()
    out["fq_f16_in"] = h16.view(torch.int16).numpy()
    out["fq_f16_out"] = uq.fake_quant_groupwise_lastdim(h16, 128, 2).view(torch.int16).numpy()
    # ---- the cache state machine: prefill, then decode steps past one key quantization ---- #
    cfg = ks.KittyKVCacheConfig(sink_length=32, buffer_length=128, group_size=128, kbits=2, vbits=2, promote_ratio=0.25,
                                promote_bit=4, channel_selection=1, VCache_BitDecoding=False, PostQuant=True)
    cache = ks.KittyKVCache(cfg)
    if not hasattr(cache, "key_cache"):
        cache.key_cache, cache.value_cache = [], []
    B, H, L, D, steps = 1, 1, 32 + 128 + 120, 128, 12
    k0, v0 = torch.randn(B, H, L, D, generator=g), torch.randn(B, H, L, D, generator=g)
    k0[:, :, :, torch.randperm(D, generator=g)[:4]] *= 8.0
    kr, vr = cache.update(k0, v0, 0)
    out["k_prefill"], out["v_prefill"] = k0.numpy(), v0.numpy()
    assert torch.equal(kr, k0) and torch.equal(vr, v0)         # PostQuant: the prompt step sees full precision
    out["prefill_key_cache"], out["prefill_value_cache"] = cache.key_cache[0].numpy().copy(), cache.value_cache[0].numpy().copy()
    ks_, vs_, kret, vret = [], [], [], []
    for s in range(steps):
        kt, vt = torch.randn(B, H, 1, D, generator=g), torch.randn(B, H, 1, D, generator=g)
        kr, vr = cache.update(kt, vt, 0)
        ks_.append(kt.numpy()); vs_.append(vt.numpy())
        if s in (8, 9):                          # step 8 appends the token that triggers the key quantization
            kret.append(kr.numpy()); vret.append(vr.numpy())
    out["k_steps"], out["v_steps"] = np.stack(ks_), np.stack(vs_)
    out["probe_steps"] = np.array([8, 9])
    for i, (a, b) in enumerate(zip(kret, vret)):
        out[f"keys_returned_{i}"], out[f"values_returned_{i}"] = a, b
    out["final_key_cache"], out["final_value_cache"] = cache.key_cache[0].numpy(), cache.value_cache[0].numpy()
    np.savez_compressed(os.path.join(HERE, "sim_port.npz"), **out)
    print("wrote sim_port.npz:", {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
