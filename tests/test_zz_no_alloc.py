"""The allocation-free decode entry point (collected last on purpose).

`kitty_decode_attn_static` serves callers that may not allocate device memory and
have no workspace to lend — for example a process whose GPU memory is entirely
owned by another allocator, or a latency-critical loop that must stay away from
cudaMalloc's driver lock.  Its partial results live in a fixed array inside the
library.  The test calls it through the C ABI, twice in a row on different
states of the cache (the second call reuses the array the first one dirtied),
and requires the same output as the ordinary entry point.
"""
import ctypes
import types

import pytest
import torch

from tests.helpers import make_kv

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _call_static(lib, lay, q, h_q, scaling, status):
    out = torch.empty((q.shape[0], 1, h_q, 128), dtype=q.dtype, device=q.device)
    code = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}[q.dtype]
    rc = lib.kitty_decode_attn_static(lay.c_layer(), lay.c_counts(), q.data_ptr(), code, q.shape[0], h_q,
                                      float(scaling), out.data_ptr(), code, 0, -1, 3, None, 0, status.data_ptr(),
                                      torch.cuda.current_stream().cuda_stream)
    return rc, out


@pytest.mark.parametrize("h_kv,h_q", [(2, 8), (1, 7)])
def test_static_scratch_entry_matches_workspace_entry_twice(h_kv, h_q):
    """Same plan, same kernels, only the scratch address differs: the two entry points must agree bit for bit, for the
    integer streaming kernel (groups of 4 heads) and the fp16 one (groups of 7)."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import kitty_b200 as kb
    from kitty_b200 import _lib

    lib = _lib.lib()
    B, L = 3, 32 + 21 * 128 + 77
    cfg = types.SimpleNamespace(num_hidden_layers=1, head_dim=128, num_key_value_heads=h_kv, num_attention_heads=h_q,
                                hidden_size=128 * h_q)
    k, v = make_kv(B, h_kv, L, 128, 4242, torch.bfloat16)
    cache = kb.KittyCache(cfg, B, L + 16, device=DEV)
    cache.update(k.to(DEV), v.to(DEV), 0)
    cache.quantize_prefill(0)
    lay = cache.kv_cache[0]
    g = torch.Generator().manual_seed(7)
    scaling = 128 ** -0.5
    status = torch.full((1,), -1, dtype=torch.int32, device=DEV)
    for step in range(2):
        kt = torch.randn(B, h_kv, 1, 128, generator=g).bfloat16().to(DEV)
        vt = torch.randn(B, h_kv, 1, 128, generator=g).bfloat16().to(DEV)
        q = torch.randn(B, h_q, 1, 128, generator=g).bfloat16().to(DEV)
        cache.update(kt, vt, 0)
        want = kb.decode_attention(q, lay, h_kv, scaling)            # caller-owned workspace
        rc, got = _call_static(lib, lay, q, h_q, scaling, status)    # built-in scratch
        assert rc == 0, _lib.strerror(rc)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        assert torch.equal(got, want), (step, (got.float() - want.float()).abs().max().item())
        cache.quantize_decode(0)


def test_static_scratch_entry_rejects_what_does_not_fit():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import kitty_b200 as kb
    from kitty_b200 import _lib

    lib = _lib.lib()
    # 640 sequences x 8 KV heads x 16 query heads each: one slot per (sequence, head) already exceeds 8 MiB
    h_kv, h_q, B = 8, 128, 640
    cfg = types.SimpleNamespace(num_hidden_layers=1, head_dim=128, num_key_value_heads=h_kv, num_attention_heads=h_q,
                                hidden_size=128 * h_q)
    cache = kb.KittyCache(cfg, B, 256, device=DEV)
    k = torch.zeros(B, h_kv, 40, 128, dtype=torch.float16, device=DEV)
    cache.update(k, k, 0)
    cache.quantize_prefill(0)
    q = torch.zeros(B, h_q, 1, 128, dtype=torch.float16, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    rc, _ = _call_static(lib, cache.kv_cache[0], q, h_q, 1.0, status)
    assert rc == _lib.KITTY_E_STATIC_LIMIT
    assert "KITTY_STATIC_SCRATCH_BYTES" in _lib.strerror(rc)
