"""Generate the golden fixtures in this folder by EXECUTING THE REFERENCE.

Run once, in a container that has the reference checkout (pass its path as the
first argument or in $KITTY_REFERENCE) and no GPU:

    python tests/golden/make_golden.py /path/to/Kitty

The reference's Triton kernels are run on the CPU through the Triton
interpreter (TRITON_INTERPRET=1).  Its sources are copied, at run time only,
into a temporary folder where three things are adapted and nothing else:
  * `transformers.cache_utils.CacheConfig` (removed from current transformers)
    is stubbed before import, and KittyCache objects are built without calling
    `Cache.__init__` (which now requires arguments);
  * allocations on device 'cuda' are redirected to the CPU;
  * the uint8 slot index is widened to int32 before it is multiplied by the
    32-byte row stride (kitty_quant_pack.py:141, kitty_attention.py:154).  Under
    current Triton the product stays uint8 and wraps, so the 32 high-plane rows
    alias onto 8; the widened form yields the 32 distinct rows the buffer is
    sized for (utils_kv_per_layer.py:35).
The fixtures are small .npz files; every array in them is an input to or an
output of the reference's own functions.
"""
from __future__ import annotations

import os
import shutil
import sys
import tempfile
import types

os.environ["TRITON_INTERPRET"] = "1"

import numpy as np  # noqa: E402
import torch  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def load_reference(ref_root: str):
    src = os.path.join(ref_root, "src", "kitty")
    tmp = tempfile.mkdtemp(prefix="kitty_ref_")
    dst = os.path.join(tmp, "kitty")
    shutil.copytree(os.path.join(src, "kvcache"), os.path.join(dst, "kvcache"))
    patches = {
        "kvcache/kernels/kitty_quant_pack.py": [
            ("+ dense_sparse_idx[None, :] * K_STRIDE_D", "+ dense_sparse_idx[None, :].to(tl.int32) * K_STRIDE_D")],
        "kvcache/kernels/kitty_attention.py": [
            ("+ boost_idx[:, None] * K_STRIDE_D", "+ boost_idx[:, None].to(tl.int32) * K_STRIDE_D")],
    }
    for rel, subs in patches.items():
        p = os.path.join(dst, rel)
        text = open(p).read()
        for old, new in subs:
            assert text.count(old) == 1, (rel, old)
            text = text.replace(old, new)
        open(p, "w").write(text)
    import transformers.cache_utils as cu

    if not hasattr(cu, "CacheConfig"):
        cu.CacheConfig = type("CacheConfig", (), {})
    sys.path.insert(0, tmp)
    real_zeros = torch.zeros

    def zeros_on_cpu(*a, **kw):
        if str(kw.get("device", "")).startswith("cuda"):
            kw["device"] = "cpu"
        return real_zeros(*a, **kw)

    torch.zeros = zeros_on_cpu
    import kitty.kvcache.kitty as ref_cache
    import kitty.kvcache.kernels.kitty_attention as ref_attn
    import kitty.kvcache.kernels.kitty_quant_pack as ref_qp
    from kitty.kvcache.utils_kv_per_layer import KVCache_Layer

    return types.SimpleNamespace(cache=ref_cache, attn=ref_attn, qp=ref_qp, Layer=KVCache_Layer)


def new_ref_cache(ref, n_layers, h_kv, D, max_bs, max_len):
    c = ref.cache.KittyCache.__new__(ref.cache.KittyCache)
    c.kv_cache = [ref.Layer(MAX_BS=max_bs, MAX_LEN=max_len, H_KV=h_kv, D=D, D_BOOSTED=D // 4, LOW_BIT=2,
                            HIGH_BIT=4, PAGE_SIZE=128, S=32) for _ in range(n_layers)]
    c.num_hidden_layers, c.head_dim, c.num_key_value_heads = n_layers, D, h_kv
    c.page_size, c.d_boosted, c.sink_length, c.low_bit, c.high_bit = 128, D // 4, 32, 2, 4
    return c


def raw16(t: torch.Tensor) -> np.ndarray:
    """16-bit tensor → its bit pattern (uint16), so bf16 survives an .npz."""
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def layer_arrays(lay, prefix=""):
    names = ["KeyCache", "KeyCache_metadata", "ValueCache", "ValueCache_metadata", "PageTable_K", "PageTable_V",
             "Sink_Buffer_K", "Sink_Buffer_V", "Q_Buffer_K", "Q_Buffer_V", "Local_Buffer_V"]
    out = {prefix + n: getattr(lay, n).numpy().copy() for n in names}
    out[prefix + "counters"] = np.array([lay.PageCount_K, lay.PageCount_V, lay.Sink_Count, lay.Q_Buffer_Count_K,
                                         lay.Q_Buffer_Count_V, lay.Local_Count_V, lay.Write_Offset_Local_V], np.int64)
    return out


# --------------------------------------------------------------------------- #
def gen_quant(ref, name, dtype, seed, kind):
    """One call of quantize_pack_k and quantize_pack_v on [B=1, H=2, 32+2*128, 128]."""
    g = torch.Generator().manual_seed(seed)
    B, H, P, D = 1, 2, 2, 128
    T = 32 + P * 128
    x = torch.randn(B, H, T, D, generator=g)
    if kind == "outlier8":            # 4 channels per head scaled x8
        for h in range(H):
            x[:, h, :, torch.randperm(D, generator=g)[:4]] *= 8.0
    elif kind == "loguniform":        # per-(head, channel) scale exp(U(0, ln 16))
        x = x * torch.exp(torch.rand(1, H, 1, D, generator=g) * np.log(16.0))
    elif kind == "degenerate":        # a constant channel, an all-zero page, a tiny-range token
        x[:, 0, :, 5] = 0.75
        x[:, 1, 32:160, :] = 0.0
        x[:, 0, 40, :] = 1e-7 * torch.arange(D)
    x = x.to(dtype)
    maxp = 4
    kc = torch.zeros(B * maxp, H * 5248, dtype=torch.uint8)
    km = torch.zeros(B * maxp, H, D, 2, dtype=torch.half)
    vc = torch.zeros(B * maxp, H * 4096, dtype=torch.uint8)
    vm = torch.zeros(B * maxp, H, 128, 2, dtype=torch.half)
    pt = torch.arange(B * maxp, dtype=torch.int64).view(B, maxp)
    ref.qp.quantize_pack_k(x, 32, P, pt, 1, kc, km, 128, 32)
    ref.qp.quantize_pack_v(x, 32, P, pt, 1, vc, vm, 128)
    arrays = dict(KeyCache=kc.numpy(), KeyCache_metadata=km.numpy(), ValueCache=vc.numpy(),
                  ValueCache_metadata=vm.numpy(), t_offset=np.int64(32), pages=np.int64(P), page_offset=np.int64(1))
    arrays["x"] = x.numpy() if dtype == torch.float32 else raw16(x)
    arrays["dtype"] = np.array({torch.float16: "f16", torch.bfloat16: "bf16", torch.float32: "f32"}[dtype])
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **arrays)
    print("wrote", name)


def gen_cache(ref, name, seed, h_kv, h_q, B, L, steps, probe_steps):
    """Prefill L tokens then `steps` decode steps through the reference cache and
    its decode attention (fp16, as the reference requires)."""
    g = torch.Generator().manual_seed(seed)
    D = 128
    cache = new_ref_cache(ref, 1, h_kv, D, B, L + steps + 8)
    mod = types.SimpleNamespace(num_attention_heads=h_q, num_key_value_heads=h_kv)
    scaling = D ** -0.5
    k0 = torch.randn(B, h_kv, L, D, generator=g)
    for h in range(h_kv):
        k0[:, h, :, torch.randperm(D, generator=g)[:4]] *= 8.0
    v0 = torch.randn(B, h_kv, L, D, generator=g)
    k0, v0 = k0.half(), v0.half()
    assert cache.update(k0, v0, 0) is True
    cache.quantize_prefill(0)
    arrays = dict(k_prefill=raw16(k0), v_prefill=raw16(v0), h_q=np.int64(h_q), scaling=np.float64(scaling))
    arrays.update(layer_arrays(cache.kv_cache[0], "prefill_"))
    ks, vs, qs, outs, lens = [], [], [], [], []
    for s in range(steps):
        k = torch.randn(B, h_kv, 1, D, generator=g).half()
        v = torch.randn(B, h_kv, 1, D, generator=g).half()
        q = torch.randn(B, h_q, 1, D, generator=g).half()
        assert cache.update(k, v, 0) is False
        if s in probe_steps:
            o, _ = ref.attn.kitty_attention_forward(mod, q, cache.kv_cache[0], scaling)
            outs.append(raw16(o))
            lens.append(cache.get_seq_length(0))
        cache.quantize_decode(0)
        ks.append(raw16(k)); vs.append(raw16(v)); qs.append(raw16(q))
    arrays.update(k_steps=np.stack(ks), v_steps=np.stack(vs), q_steps=np.stack(qs), attn_out=np.stack(outs),
                  attn_len=np.array(lens), probe_steps=np.array(sorted(probe_steps)))
    arrays.update(layer_arrays(cache.kv_cache[0], "final_"))
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **arrays)
    print("wrote", name, "final length", cache.get_seq_length(0))


def main():
    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("KITTY_REFERENCE", "")
    if not os.path.isdir(os.path.join(ref_root, "src", "kitty")):
        raise SystemExit("usage: make_golden.py <path to the reference checkout>")
    ref = load_reference(ref_root)
    gen_quant(ref, "quant_f16_outlier8", torch.float16, 0, "outlier8")
    gen_quant(ref, "quant_bf16_loguniform", torch.bfloat16, 1, "loguniform")
    gen_quant(ref, "quant_f32_outlier8", torch.float32, 2, "outlier8")
    gen_quant(ref, "quant_f16_degenerate", torch.float16, 3, "degenerate")
    # G=4: prompt with ragged tails; decode across a K flush (step 70) and a V flush.
    gen_cache(ref, "cache_g4", 10, h_kv=2, h_q=8, B=2, L=32 + 2 * 128 + 57, steps=150,
              probe_steps={0, 1, 70, 71, 100, 149})
    # G=7, short prompt: sink not yet full, ring still filling.
    gen_cache(ref, "cache_g7_short", 11, h_kv=1, h_q=7, B=1, L=20, steps=300, probe_steps={0, 11, 12, 139, 140, 267, 299})


if __name__ == "__main__":
    main()
