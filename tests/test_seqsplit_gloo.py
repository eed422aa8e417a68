"""Sequence-split decode across 2 ranks on CPU (gloo): the host plumbing — page
ranges, sink/tail flags, all-gather order, merge — with the oracle standing in
for the device kernels.  The merged result must equal single-rank attention."""
import os
import socket
import types

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

from oracle import kitty_oracle as ko
from tests.helpers import make_kv

LOG2E = 1.4426950408889634


def test_split_pages_and_flags():
    from kitty_b200.seqsplit import rank_flags, split_pages

    assert split_pages(1022, 8) == [(0, 128), (128, 256), (256, 384), (384, 512), (512, 640), (640, 768), (768, 895), (895, 1022)]
    assert split_pages(3, 4) == [(0, 1), (1, 2), (2, 3), (3, 3)]
    assert split_pages(0, 2) == [(0, 0), (0, 0)]
    for n, w in [(254, 2), (7, 3), (1022, 8)]:
        r = split_pages(n, w)
        assert r[0][0] == 0 and r[-1][1] == n and all(a[1] == b[0] for a, b in zip(r, r[1:]))
    assert [rank_flags(r, 4) for r in range(4)] == [1, 0, 0, 2] and rank_flags(0, 1) == 3


def _oracle_partial(lay, h_kv, h_q):
    """partial_fn with the C entry point's meaning, computed by the oracle (base-2 max, as the kernels emit)."""
    def fn(query, layer, num_kv_heads, scaling, lo, hi, flags):
        q = ko.as_f32(query)
        B, G = q.shape[0], h_q // h_kv
        out = np.zeros((B, h_q, 130), np.float32)
        for b in range(B):
            for h in range(h_kv):
                K, V = ko.gather_kv(lay, b, h)
                s0 = lay.Sink_Count
                pv = lay.PageCount_V
                sel = []
                if flags & 1:
                    sel += list(range(0, s0))
                sel += list(range(s0 + 128 * lo, s0 + 128 * hi))
                if flags & 2:
                    sel += list(range(s0 + 128 * pv, K.shape[0]))
                sel = np.array(sel, dtype=np.int64)
                m, l, acc = ko.attention_partial(q[b, h * G:(h + 1) * G, 0], K[sel], V[sel], scaling)
                out[b, h * G:(h + 1) * G, :128] = acc
                out[b, h * G:(h + 1) * G, 128] = m * LOG2E
                out[b, h * G:(h + 1) * G, 129] = l
        return torch.from_numpy(out)
    return fn


def _host_merge(parts, dtype):
    p = parts.numpy().astype(np.float64)
    M = p[..., 128].max(0)
    w = np.exp2(p[..., 128] - M)
    acc = (p[..., :128] * w[..., None]).sum(0)
    l = (p[..., 129] * w).sum(0)
    return torch.from_numpy((acc / l[..., None])[:, None].astype(np.float32))


def _worker(rank, world, port, q_out):
    import torch.distributed as dist

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from kitty_b200.seqsplit import seq_split_decode

    h_kv, h_q, B, L = 2, 14, 2, 32 + 7 * 128 + 50
    k, v = make_kv(B, h_kv, L, 128, 5, torch.float16)
    oc = ko.OracleKittyCache(1, h_kv, 128, B, L + 8)
    oc.update(k, v, 0)
    oc.quantize_prefill(0)
    g = torch.Generator().manual_seed(1)
    oc.update(torch.randn(B, h_kv, 1, 128, generator=g).half(), torch.randn(B, h_kv, 1, 128, generator=g).half(), 0)
    q = torch.randn(B, h_q, 1, 128, generator=g).half()
    lay = oc.kv_cache[0]
    out = seq_split_decode(q, lay, h_kv, 128 ** -0.5, rank=rank, world=world, n_common_pages=lay.PageCount_V,
                           partial_fn=_oracle_partial(lay, h_kv, h_q), merge_fn=_host_merge)
    want = ko.decode_attention(lay, q, h_q, 128 ** -0.5)
    q_out.put((rank, float(np.abs(out.numpy() - want).max() / np.abs(want).max())))
    dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_two_rank_sequence_split_matches_single_rank():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    assert sorted(r for r, _ in res) == [0, 1]
    assert all(e < 1e-5 for _, e in res), res


def _withhold_worker(rank, world, port, q_out, release):
    """Rank 1 computes its partial and then never joins the all-gather (it waits on the host until rank 0 has
    reported): rank 0's collective must end with the process group's timeout and surface as KITTY_E_TIMEOUT."""
    import datetime

    import torch.distributed as dist

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    from kitty_b200 import _lib
    from kitty_b200.seqsplit import seq_split_decode

    h_kv, h_q, B, L = 1, 4, 1, 32 + 3 * 128 + 9
    k, v = make_kv(B, h_kv, L, 128, 6, torch.float16)
    oc = ko.OracleKittyCache(1, h_kv, 128, B, L + 8)
    oc.update(k, v, 0)
    oc.quantize_prefill(0)
    q = torch.randn(B, h_q, 1, 128, generator=torch.Generator().manual_seed(2)).half()
    lay = oc.kv_cache[0]
    if rank == 1:
        release.wait(120)          # withholds its contribution; leaves only after rank 0 has seen the failure
        q_out.put((rank, "withheld"))
        return
    try:
        seq_split_decode(q, lay, h_kv, 128 ** -0.5, rank=rank, world=world, n_common_pages=lay.PageCount_V,
                         partial_fn=_oracle_partial(lay, h_kv, h_q), merge_fn=_host_merge)
        q_out.put((rank, "no error"))
    except _lib.KittyError as e:
        q_out.put((rank, e.status))
    finally:
        release.set()


@pytest.mark.timeout(300)
def test_withheld_partial_is_reported_as_timeout():
    from kitty_b200 import _lib

    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q, release = ctx.Queue(), ctx.Event()
    procs = [ctx.Process(target=_withhold_worker, args=(r, 2, port, q, release)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=240) for _ in procs)
    for p in procs:
        p.join(60)
        if p.is_alive():
            p.kill()
    assert res[1] == "withheld"
    assert res[0] == _lib.KITTY_E_TIMEOUT, res
