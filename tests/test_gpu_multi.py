"""Sequence-split decode on 2 GPUs against the single-GPU call, both ways of combining the partials: NCCL
all-gather + kitty_lse_merge, and the peer-memory exchange inside the merge kernel (kitty_lse_exchange_merge).
Skipped when fewer than 2 GPUs are visible."""
import os
import socket
import types

import pytest
import torch
import torch.multiprocessing as mp

from tests.helpers import make_kv

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, q_out):
    import torch.distributed as dist

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    import kitty_b200 as kb
    from kitty_b200.seqsplit import PartialExchange, rank_flags, seq_split_decode, split_pages

    h_kv, h_q, B, L = 4, 28, 1, 32 + 40 * 128 + 50          # the long-context shape: 28 query / 4 KV heads
    cfg = types.SimpleNamespace(num_hidden_layers=1, head_dim=128, num_key_value_heads=h_kv, num_attention_heads=h_q,
                                hidden_size=128 * h_q)
    k, v = make_kv(B, h_kv, L, 128, 9, torch.bfloat16)
    cache = kb.KittyCache(cfg, B, L + 8, device=dev)          # every rank holds the same cache; each reads only its range
    cache.update(k.to(dev), v.to(dev), 0)
    cache.quantize_prefill(0)
    g = torch.Generator().manual_seed(2)
    cache.update(torch.randn(B, h_kv, 1, 128, generator=g).bfloat16().to(dev),
                 torch.randn(B, h_kv, 1, 128, generator=g).bfloat16().to(dev), 0)
    q = torch.randn(B, h_q, 1, 128, generator=g).bfloat16().to(dev)
    lay = cache.kv_cache[0]
    full = kb.decode_attention(q, lay, h_kv, 128 ** -0.5)
    out = seq_split_decode(q, lay, h_kv, 128 ** -0.5, rank=rank, world=world, n_common_pages=lay.PageCount_V)
    torch.cuda.synchronize(dev)
    err = (out.float() - full.float()).abs().max().item() / full.float().abs().max().item()
    # the same step with the partials exchanged by the merge kernel itself, several calls in a row
    xch = PartialExchange(B * h_q, dev)
    err_x = 0.0
    for _ in range(5):
        out_x = seq_split_decode(q, lay, h_kv, 128 ** -0.5, rank=rank, world=world, n_common_pages=lay.PageCount_V,
                                 exchange=xch)
        torch.cuda.synchronize(dev)
        err_x = max(err_x, (out_x.float() - out.float()).abs().max().item() / out.float().abs().max().item())
        # and in two calls: partial of this rank's range, then the stand-alone exchange + merge
        lo, hi = split_pages(lay.PageCount_V, world)[rank]
        part = torch.empty(B, h_q, 130, dtype=torch.float32, device=dev)
        kb.decode_attention(q, lay, h_kv, 128 ** -0.5, page_begin=lo, page_end=hi, flags=rank_flags(rank, world),
                            partial_out=part)
        out_y = xch.merge(part, q.dtype)
        torch.cuda.synchronize(dev)
        err_x = max(err_x, (out_y.float() - out.float()).abs().max().item() / out.float().abs().max().item())
    xch.check()
    # the whole layer step in one call per rank (device-resident counters, exchange inside): same tokens appended on
    # every rank, results equal to the three-call path on a twin cache, through a flush
    from kitty_b200.seqsplit import seq_split_step

    twin = kb.KittyCache(cfg, B, L + 64, device=dev)
    step_cache = kb.KittyCache(cfg, B, L + 64, device=dev)
    for c in (twin, step_cache):
        c.update(k.to(dev), v.to(dev), 0)
        c.quantize_prefill(0)
    err_s = 0.0
    for s_ in range(90):                                   # the Q-buffers hold 50 tokens: a key flush at step 78
        kt = torch.randn(B, h_kv, 1, 128, generator=g).bfloat16().to(dev)
        vt = torch.randn(B, h_kv, 1, 128, generator=g).bfloat16().to(dev)
        qt = torch.randn(B, h_q, 1, 128, generator=g).bfloat16().to(dev)
        twin.update(kt, vt, 0)
        want = kb.decode_attention(qt, twin.kv_cache[0], h_kv, 128 ** -0.5)
        twin.quantize_decode(0)
        got = seq_split_step(step_cache, kt, vt, qt, 128 ** -0.5, rank=rank, world=world, exchange=xch)
        if s_ % 11 == 0 or s_ > 75:
            torch.cuda.synchronize(dev)
            err_s = max(err_s, (got.float() - want.float()).abs().max().item() / want.float().abs().max().item())
    torch.cuda.synchronize(dev)
    xch.check()
    assert step_cache.kv_cache[0].PageCount_K == twin.kv_cache[0].PageCount_K == 41
    assert torch.equal(step_cache.kv_cache[0].KeyCache, twin.kv_cache[0].KeyCache)
    q_out.put((rank, err, max(err_x, err_s)))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.timeout(600)
def test_two_gpu_sequence_split():
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=500) for _ in procs]
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert all(e <= 1e-2 for _, e, _ in res), res
    assert all(ex <= 4e-3 for _, _, ex in res), res       # same partials; the sums may differ in the last bf16 bit
