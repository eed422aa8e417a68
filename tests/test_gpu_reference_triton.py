"""The reference's own Triton kernels on the GPU (from the copy under baseline/_ref that oracle/make_ref_copy.py
writes: slot index widened to int32, nothing else changed) against the CUDA library, on the same cache object.
Skipped where that copy or a working Triton build is missing — the pinned oracle tests do not depend on it."""
import os
import sys
import types

import pytest
import torch

from tests.helpers import make_kv

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")


@pytest.fixture(scope="module")
def ref():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    if not os.path.isdir(os.path.join(REF, "kitty")):
        pytest.skip("baseline/_ref/kitty is absent")
    if REF not in sys.path:
        sys.path.insert(0, REF)
    try:
        import kitty.kvcache.kernels.kitty_attention as ra
        import kitty.kvcache.kernels.kitty_quant_pack as rq
    except Exception as e:      # noqa: BLE001
        pytest.skip(f"the reference kernels do not import here: {e}")
    return types.SimpleNamespace(attn=ra, qp=rq)


@pytest.mark.parametrize("h_kv,h_q", [(2, 8), (1, 7)])
def test_attention_agrees_with_the_reference_kernels_on_the_same_cache(ref, h_kv, h_q):
    import kitty_b200 as kb

    B, L = 2, 32 + 6 * 128 + 70
    cfg = types.SimpleNamespace(num_hidden_layers=1, head_dim=128, num_key_value_heads=h_kv, num_attention_heads=h_q,
                                hidden_size=128 * h_q)
    k, v = make_kv(B, h_kv, L, 128, 88, torch.float16)
    cache = kb.KittyCache(cfg, B, L + 200, device=DEV)
    cache.update(k.to(DEV), v.to(DEV), 0)
    cache.quantize_prefill(0)
    lay = cache.kv_cache[0]
    mod = types.SimpleNamespace(num_attention_heads=h_q, num_key_value_heads=h_kv)
    g = torch.Generator().manual_seed(4)
    for step in range(140):                      # through a flush and a rotated value ring
        kt, vt = torch.randn(B, h_kv, 1, 128, generator=g).half(), torch.randn(B, h_kv, 1, 128, generator=g).half()
        cache.update(kt.to(DEV), vt.to(DEV), 0)
        if step % 23 == 0 or step > 136:
            q = torch.randn(B, h_q, 1, 128, generator=g).half().to(DEV)
            try:
                want, _ = ref.attn.kitty_attention_forward(mod, q, lay, 128 ** -0.5)
            except Exception as e:      # noqa: BLE001
                pytest.skip(f"the reference kernels do not build for this GPU: {str(e).splitlines()[0][:200]}")
            got, _ = kb.kitty_attention_forward(mod, q, lay, 128 ** -0.5)
            err = float((got.float() - want.float()).abs().max() / want.float().abs().max())
            assert err <= 1e-2, (step, err)
        cache.quantize_decode(0)


def test_quantized_bytes_agree_with_the_reference_kernels(ref):
    """With the reference's index bytes (abs().mean().topk() on this GPU) and the division Triton compiles
    (div.full.f32), the library's key and value pages equal the reference kernels' output."""
    import kitty_b200 as kb
    from kitty_b200 import _lib

    B, H, P = 1, 4, 24
    k, v = make_kv(B, H, P * 128, 128, 12, torch.float16, "loguniform")
    k, v = k.to(DEV), v.to(DEV)
    z = dict(device=DEV)

    def bufs():
        return (torch.zeros(P, H * 5248, dtype=torch.uint8, **z), torch.zeros(P, H, 128, 2, dtype=torch.float16, **z),
                torch.zeros(P, H * 4096, dtype=torch.uint8, **z), torch.zeros(P, H, 128, 2, dtype=torch.float16, **z))

    pt = torch.arange(P, dtype=torch.int64, **z).view(1, P)
    rkc, rkm, rvc, rvm = bufs()
    try:
        ref.qp.quantize_pack_k(k, 0, P, pt, 0, rkc, rkm, 128, 32)
        ref.qp.quantize_pack_v(v, 0, P, pt, 0, rvc, rvm, 128)
    except Exception as e:      # noqa: BLE001
        pytest.skip(f"the reference kernels do not build for this GPU: {str(e).splitlines()[0][:200]}")
    kc, km, vc, vm = bufs()
    idx = rkc.view(P, H, 5248)[..., 5120:].permute(1, 0, 2).unsqueeze(0).contiguous()      # the reference's index bytes
    kb.quantize_pack_k(k, 0, P, pt, 0, kc, km, 128, 32, channel_idx=idx, div_mode=_lib.DIV_FULL)
    kb.quantize_pack_v(v, 0, P, pt, 0, vc, vm, 128, div_mode=_lib.DIV_FULL)
    same = {"key_bytes": float((kc == rkc).float().mean()), "key_metadata": float((km == rkm).float().mean()),
            "value_bytes": float((vc == rvc).float().mean()), "value_metadata": float((vm == rvm).float().mean())}
    assert all(x >= 0.9999 for x in same.values()), same
