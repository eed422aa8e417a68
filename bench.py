"""Benchmark of the quantized-KV decode hot path.

Workload (the 32K-token single-layer decode-attention configuration): one layer,
32 query / 8 KV heads, head_dim 128, 32768 cached tokens per sequence (255 packed
key pages, 254 packed value pages, fp16 tails), bf16 Gaussian K with 4 outlier
channels per head (x8), batch rows sharded over the GPUs (weak scaling: every
GPU holds `--batch` sequences).  One step = one decode step of that layer
through the cache object: append the new token's K/V, fused dequant decode
attention, flush a full Q-buffer if there is one.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch B] [--impl reference] [--no-extras]
    python bench.py --workload quantize            # bulk prefill quantize/pack throughput alone
    python bench.py --workload e2e [--no-graph]    # Llama-3-8B-shaped decoder, greedy decode with the cache, alone
    python bench.py --workload seqsplit [--exchange peer] [--seq-batch B]   # 131072-token sequence split over the ranks, alone

Prints one JSON line (rank 0).  `value` is device-timed with the step inputs
already in HBM; `e2e` runs the same step through the public API from pinned
host tensors with the result copied back every step (median of 5 repeats of the
K steps).  The same line carries one short record for each of the other
workloads, each with its own CUDA-event timing and byte count: `sweep`
(attention call at batch 1 / 8 / 32), `quantize` (bulk prefill quantize/pack),
`model_e2e` (decoder model, greedy decode) and `reference_gpu` (the reference's
own Triton kernels on the same GPU, when their copy under baseline/_ref exists)
on one GPU, and `seqsplit` (the 131072-token sequence split over the ranks) when
launched on more than one.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

H_KV, H_Q, D, CTX = 8, 32, 128, 32768
K_PAGE_BYTES, V_PAGE_BYTES = 5760, 4608     # packed record + fp16 metadata per (page, kv-head)
# dram__bytes_read.sum + dram__bytes_write.sum of decode_paged_i8_kernel per page pair, from one ncu capture of the
# batch-8 case of this workload (180.75 MB for the launch less the 6.66 MB of its 64 edges = 174.09 MB over 16256
# pairs).  A figure from a past capture: it has to be re-taken whenever the streaming kernel's data path changes.
DRAM_BYTES_PER_PAGE_PAIR = 10709


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batch", type=int, default=128, help="sequences per GPU")
    ap.add_argument("--ctx", type=int, default=CTX)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="only the headline decode workload: skip the sweep / quantize / model_e2e / seqsplit records")
    ap.add_argument("--workload", default="decode", choices=["decode", "quantize", "e2e", "seqsplit"],
                    help="decode (the headline metric), quantize (bulk prefill quantize/pack throughput) or e2e "
                         "(Llama-3-8B-shaped random-init decoder: batch 16, 4096-token prompts, 256 greedy steps)")
    ap.add_argument("--layers", type=int, default=32, help="decoder layers of the e2e workload")
    ap.add_argument("--graph", action=argparse.BooleanOptionalAction, default=True,
                    help="e2e workload: replay the decode step from a CUDA graph (GraphedDecoder); --no-graph runs the "
                         "eager patched model")
    ap.add_argument("--e2e-batch", type=int, default=16, help="batch of the e2e workload")
    ap.add_argument("--e2e-steps", type=int, default=256, help="greedy steps of the e2e workload")
    ap.add_argument("--seq-batch", type=int, default=1, help="seqsplit workload: sequences (the named config has 1)")
    ap.add_argument("--tail-weight", type=int, default=0,
                    help="seqsplit workload: packed pages the last rank's tail is counted as when the pages are split")
    ap.add_argument("--exchange", default="nccl", choices=["nccl", "peer", "step", "graph"],
                    help="seqsplit workload: combine the partials with an NCCL all-gather + merge kernel, or inside "
                         "the merge kernel over peer memory")
    return ap.parse_args()


# --------------------------------------------------------------------------- #
# byte accounting (per sequence = per batch row, all 8 KV heads)
# --------------------------------------------------------------------------- #
def partition(ctx: int) -> dict:
    """How a prompt of ctx tokens is laid out by the cache (sink, packed pages, fp16 tails)."""
    sink = min(32, ctx)
    qbuf_k = (ctx - sink) % 128
    local_v = min(128, ctx - sink)
    qbuf_v = (ctx - sink - local_v) % 128
    return dict(sink=sink, qbuf_k=qbuf_k, pages_k=(ctx - sink - qbuf_k) // 128, local_v=local_v, qbuf_v=qbuf_v,
                pages_v=(ctx - sink - local_v - qbuf_v) // 128)


def packed_bytes(pages_k: int, pages_v: int) -> int:
    return H_KV * (pages_k * K_PAGE_BYTES + pages_v * V_PAGE_BYTES)


def attention_bytes(lay) -> int:
    """Algorithmic bytes of one attention call per sequence: packed pages + fp16 tails + page tables + q/out."""
    g = H_Q // H_KV
    tails = (2 * lay.Sink_Count + lay.Q_Buffer_Count_K + lay.Q_Buffer_Count_V + lay.Local_Count_V) * 256
    per_head = (lay.PageCount_K * K_PAGE_BYTES + lay.PageCount_V * V_PAGE_BYTES + tails
                + (lay.PageCount_K + lay.PageCount_V) * 8 + 2 * g * 256)
    return H_KV * per_head


# --------------------------------------------------------------------------- #
# clocks during the timed region (read-only NVML queries)
# --------------------------------------------------------------------------- #
class ClockSampler:
    def __init__(self, index: int, interval_s: float = 0.001):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self.interval_s = interval_s
        self._stop = threading.Event()
        self._t = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20,
                 "hw_power_brake_slowdown": 0x80}
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h) if hasattr(
                    nv, "nvmlDeviceGetCurrentClocksEventReasons") else nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for n, bit in names.items():
                    if r & bit:
                        self.reasons.add(n)
            except Exception:
                pass
            self._stop.wait(self.interval_s)

    def __enter__(self):
        if self.nv is not None:
            self._t = threading.Thread(target=self._run, daemon=True)
            self._t.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._t is not None:
            self._t.join()

    def summary(self):
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


# --------------------------------------------------------------------------- #
# reference arm / CPU baseline: the reference's PyTorch path on the host cores
# --------------------------------------------------------------------------- #
def cpu_reference(ctx: int, steps: int, warmup: int, budget_s: float = 25.0):
    """Times decode steps of the reference's PyTorch (fake-quant + eager attention) path, fp32, on all host
    cores, for ONE sequence of the workload (8 KV heads, `ctx` cached tokens)."""
    from oracle import kitty_sim_port as sp

    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    torch.set_num_threads(cores)
    g = torch.Generator().manual_seed(0)
    k = torch.randn(1, H_KV, ctx, D, generator=g)
    for h in range(H_KV):
        k[:, h, :, torch.randperm(D, generator=g)[:4]] *= 8.0
    v = torch.randn(1, H_KV, ctx, D, generator=g)
    cache = sp.SimKittyCache()
    cache.update(k, v)
    del k, v
    scaling = D ** -0.5
    times = []
    t_begin = time.perf_counter()
    for s in range(warmup + steps):
        q = torch.randn(1, H_Q, 1, D, generator=g)
        kt, vt = torch.randn(1, H_KV, 1, D, generator=g), torch.randn(1, H_KV, 1, D, generator=g)
        t0 = time.perf_counter()
        sp.decode_step(cache, q, kt, vt, scaling)
        dt = time.perf_counter() - t0
        if s >= warmup:
            times.append(dt)
        if s >= warmup + 2 and time.perf_counter() - t_begin > budget_s:
            break
    p = partition(ctx)
    per_step = sum(times) / len(times)
    gbs = packed_bytes(p["pages_k"], p["pages_v"]) / per_step / 1e9
    return {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port",
            "sample": f"1 sequence (8 KV heads, {ctx} tokens), {len(times)} decode steps, fp32, torch on {cores} threads; "
                      "bytes counted as the packed-KV bytes of that sequence",
            "ms_per_step": per_step * 1e3, "steps": len(times), "tokens_per_s": 1.0 / per_step}


# --------------------------------------------------------------------------- #
def build_cache(kb, batch, ctx, extra, device, seed, dtype=torch.bfloat16, layers=1):
    cfg = argparse.Namespace(num_hidden_layers=layers, head_dim=D, num_key_value_heads=H_KV, num_attention_heads=H_Q,
                             hidden_size=H_Q * D)
    cache = kb.KittyCache(cfg, batch, ctx + extra + 256, device=device)
    g = torch.Generator(device=device).manual_seed(seed)
    from kitty_b200 import _lib

    p = partition(ctx)
    for lay in cache.kv_cache:
        # the prompt is generated and quantized in slices of 16 sequences to bound transient memory
        for b0 in range(0, batch, 16):
            b1 = min(batch, b0 + 16)
            k = torch.randn(b1 - b0, H_KV, ctx, D, generator=g, device=device, dtype=torch.float32)
            for h in range(H_KV):
                k[:, h, :, torch.randperm(D, generator=g, device=device)[:4]] *= 8.0
            k = k.to(dtype)
            v = torch.randn(b1 - b0, H_KV, ctx, D, generator=g, device=device, dtype=torch.float32).to(dtype)
            sub = _lib.KittyLayer.from_buffer_copy(lay.c_layer())
            for name in ("Sink_Buffer_K", "Sink_Buffer_V", "Q_Buffer_K", "Q_Buffer_V", "Local_Buffer_V"):
                setattr(sub, name, getattr(lay, name)[b0].data_ptr())
            rc = _lib.lib().kitty_prefill_tails(sub, k.data_ptr(), v.data_ptr(), _lib.dtype_code(dtype), k.stride(0), k.stride(1),
                                                k.stride(2), v.stride(0), v.stride(1), v.stride(2), b1 - b0, ctx, p["sink"],
                                                p["qbuf_k"], p["local_v"], p["qbuf_v"], _lib.stream_ptr(k.device))
            _lib.check(rc, "kitty_prefill_tails")
            kb.quantize_pack_k(k, p["sink"], p["pages_k"], lay.PageTable_K[b0:b1], 0, lay.KeyCache, lay.KeyCache_metadata, 128, 32)
            kb.quantize_pack_v(v, p["sink"], p["pages_v"], lay.PageTable_V[b0:b1], 0, lay.ValueCache, lay.ValueCache_metadata, 128)
            del k, v
        lay.Sink_Count, lay.Q_Buffer_Count_K, lay.Local_Count_V, lay.Q_Buffer_Count_V = p["sink"], p["qbuf_k"], p["local_v"], p["qbuf_v"]
        lay.PageCount_K, lay.PageCount_V = p["pages_k"], p["pages_v"]
    torch.cuda.synchronize(device)
    return cache


def hbm_peak():
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        return json.load(open(peaks_path))["hbm_gbs"], "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback"


def quantize_record(device, steps: int = 3, warmup: int = 3, layers: int = 32) -> dict:
    """Bulk prefill quantize/pack: 65536 tokens x 8 KV heads x head_dim 128 per layer call, bf16 Gaussian K/V with
    per-(head, channel) scales log-uniform in [1, 16]; `layers` layer calls per step (distinct inputs cycle through 4
    buffers of 134 MB each for K and for V, larger than L2).  K calls, V calls and the mixed K+V sequence are each
    timed with CUDA events."""
    import kitty_b200 as kb

    T, nbuf = 65536, 4
    g = torch.Generator(device=device).manual_seed(5)
    ks, vs = [], []
    for _ in range(nbuf):
        sc = torch.exp(torch.rand(1, H_KV, 1, D, generator=g, device=device) * 2.772588722239781)
        ks.append((torch.randn(1, H_KV, T, D, generator=g, device=device) * sc).to(torch.bfloat16))
        vs.append(torch.randn(1, H_KV, T, D, generator=g, device=device).to(torch.bfloat16))
    pages = T // 128
    z = dict(device=device)
    kc = torch.zeros(pages, H_KV * 5248, dtype=torch.uint8, **z)
    km = torch.zeros(pages, H_KV, 128, 2, dtype=torch.float16, **z)
    vc = torch.zeros(pages, H_KV * 4096, dtype=torch.uint8, **z)
    vm = torch.zeros(pages, H_KV, 128, 2, dtype=torch.float16, **z)
    pt = torch.arange(pages, dtype=torch.int64, **z).view(1, pages)

    def run(do_k, do_v):
        for l in range(layers):
            if do_k and do_v == "one call":
                # the prefill's call: keys and values of a layer in one launch (kitty_quant_pack_kv)
                kb.quantize_pack_kv(ks[l % nbuf], 0, pages, pt, 0, kc, km, vs[l % nbuf], 0, pages, pt, 0, vc, vm, 128, 32)
                continue
            if do_k:
                kb.quantize_pack_k(ks[l % nbuf], 0, pages, pt, 0, kc, km, 128, 32)
            if do_v:
                kb.quantize_pack_v(vs[l % nbuf], 0, pages, pt, 0, vc, vm, 128)

    def timed(do_k, do_v):
        for _ in range(warmup):
            run(do_k, do_v)
        torch.cuda.synchronize(device)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            run(do_k, do_v)
        e1.record()
        e1.synchronize()
        return e0.elapsed_time(e1) / steps

    ms_kv, ms_two, ms_k, ms_v = timed(True, "one call"), timed(True, True), timed(True, False), timed(False, True)
    units = layers * pages * H_KV
    peak, peak_src = hbm_peak()
    gbs = lambda b, ms: b / (ms * 1e-3) / 1e9
    kv, two = gbs(units * (38528 + 37376), ms_kv), gbs(units * (38528 + 37376), ms_two)
    k, v = gbs(units * 38528, ms_k), gbs(units * 37376, ms_v)
    return {"metric": "prefill_quantize_pack_throughput", "value": kv, "unit": "GB/s", "ms_per_step": ms_kv,
            "steps": steps, "warmup": warmup, "gpu_launches": layers * steps,
            "workload": f"65536 tokens x {layers} layer calls x 8 KV heads x head_dim 128, bf16, K and V; in-kernel channel "
                        "selection; algorithmic bytes 38528 (K) / 37376 (V) per page-head; value = keys and values of a "
                        "layer in one call (kitty_quant_pack_kv: one launch, as the cache's prefill issues it)",
            "roofline": {"bound": "hbm", "achieved": kv, "peak": peak, "unit": "GB/s", "frac": kv / peak, "traffic": None,
                         "peak_source": peak_src,
                         "pack_kv_kernel": {"GBps": kv, "frac": kv / peak, "ms_per_layer_call": ms_kv / layers},
                         "two_launches": {"GBps": two, "frac": two / peak, "ms_per_layer_call": ms_two / layers},
                         "pack_k_kernel": {"GBps": k, "frac": k / peak, "ms_per_layer_call": ms_k / layers},
                         "pack_v_kernel": {"GBps": v, "frac": v / peak, "ms_per_layer_call": ms_v / layers}}}


def quantize_workload(args):
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(device)
    r = quantize_record(device, steps=args.steps, warmup=max(3, args.warmup))
    r.update({"n_gpus": 1, "higher_is_better": True, "dtype": "f32", "data": "synthetic",
              "config": {"workload": r.pop("workload")}})
    print(json.dumps(r))


def model_record(device, layers: int = 32, B: int = 16, steps: int = 256, graph: bool = True, runs: int = 1) -> dict:
    """Random-init Llama-3-8B-shaped decoder (hidden 4096, 32q/8kv heads, head_dim 128, inter 14336, vocab 128256),
    bf16, batch 16, prompts of 4096 uniform-random token ids (seed 0), 256 greedy decode steps with a fresh
    KittyCache per run — the method of the reference's latency benchmark (fresh cache, greedy, fixed length;
    latency_benchmarking/benchmark_kitty.py:154-183)."""
    from transformers import LlamaConfig, LlamaForCausalLM

    import kitty_b200 as kb
    from kitty_b200.hf_adapter import GraphedDecoder, patch_model

    L = 4096
    cfg = LlamaConfig(hidden_size=4096, intermediate_size=14336, num_hidden_layers=layers, num_attention_heads=32,
                      num_key_value_heads=8, head_dim=128, vocab_size=128256, max_position_embeddings=8192,
                      rope_theta=500000.0, tie_word_embeddings=False)
    torch.manual_seed(0)
    old = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    with torch.device(device):
        model = LlamaForCausalLM(cfg).eval()
    torch.set_default_dtype(old)
    patch_model(model)
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, 128256, (B, L), generator=g).to(device)
    steady = []

    def run():
        cache = kb.get_kvcache_kitty(cfg, B, L + steps + 8, device=device)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        with torch.no_grad():
            pos = torch.arange(L, device=device).unsqueeze(0)
            hs = model.model(input_ids=ids, position_ids=pos, past_key_values=cache, use_cache=True).last_hidden_state
            tok = model.lm_head(hs[:, -1:, :]).argmax(-1)
            torch.cuda.synchronize()
            t1 = time.perf_counter()
            th = t1
            if graph:
                dec = GraphedDecoder(model, cache, B)
                dec.tok.copy_(tok)
                dec.pos.fill_(L)
                for s_ in range(1, steps):
                    if s_ == steps // 2:
                        torch.cuda.synchronize()
                        th = time.perf_counter()
                    dec.step()
            else:
                for s_ in range(1, steps):
                    if s_ == steps // 2:
                        torch.cuda.synchronize()
                        th = time.perf_counter()
                    p = torch.full((1, 1), L + s_ - 1, device=device, dtype=torch.long)
                    hs = model.model(input_ids=tok, position_ids=p, past_key_values=cache, use_cache=True).last_hidden_state
                    tok = model.lm_head(hs).argmax(-1)
            torch.cuda.synchronize()
        t2 = time.perf_counter()
        del cache
        steady.append((t2 - th) / (steps - steps // 2) * 1e3)
        return t1 - t0, t2 - t1

    run()                                   # warm-up generate (fresh cache per run, as the reference benchmark does)
    pre, dec = zip(*[run() for _ in range(max(1, runs))])
    dec_s, pre_s = min(dec), min(pre)
    del model
    torch.cuda.empty_cache()
    return {"metric": "e2e_decode_tokens_per_s", "value": B * (steps - 1) / dec_s, "unit": "tokens/s",
            "ms_per_step": dec_s / (steps - 1) * 1e3, "steady_ms_per_step": min(steady[1:]), "steps": steps,
            "prefill_s": pre_s, "decode_s": dec_s, "generate_s": pre_s + dec_s, "dtype": "bf16", "timing": "host clock "
            "around the whole greedy decode, device synchronised on both sides",
            "workload": f"random-init Llama-3-8B shape, {layers} layers, batch {B}, prompt 4096, {steps} greedy steps, "
                        "KittyCache" + (", decode steps replayed from one CUDA graph (capture included)" if graph else "")}


def e2e_workload(args):
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(device)
    r = model_record(device, args.layers, args.e2e_batch, args.e2e_steps, args.graph, runs=max(1, min(args.steps, 3)))
    r.update({"n_gpus": 1, "higher_is_better": True, "data": "synthetic", "config": {"workload": r.pop("workload")}})
    print(json.dumps(r))


def sweep_record(kb, device, ctx: int, batches=(1, 8, 32)) -> dict:
    """The attention call alone (kitty_attention_forward) at small batches, L2 flushed before every call."""
    mod = argparse.Namespace(num_attention_heads=H_Q, num_key_value_heads=H_KV)
    peak, _ = hbm_peak()
    sweep = {}
    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    for b in batches:
        c2 = build_cache(kb, b, ctx, 64, device, seed=7)
        l2 = c2.kv_cache[0]
        q = torch.randn(b, H_Q, 1, D, device=device).to(torch.bfloat16)
        c2.update(torch.randn(b, H_KV, 1, D, device=device).to(torch.bfloat16),
                  torch.randn(b, H_KV, 1, D, device=device).to(torch.bfloat16), 0)
        for _ in range(5):
            kb.kitty_attention_forward(mod, q, l2, D ** -0.5)
        a, z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        times = []
        for _ in range(30):
            flush_buf.zero_()                      # evict the cache from L2 between iterations
            a.record()
            kb.kitty_attention_forward(mod, q, l2, D ** -0.5)
            z.record()
            z.synchronize()
            times.append(a.elapsed_time(z))
        us = statistics.median(times) * 1e3
        alg = b * attention_bytes(l2)
        sweep[f"batch{b}"] = {"us_per_call": us, "algorithmic_bytes": alg, "GBps": alg / (us * 1e-6) / 1e9,
                              "frac_of_peak": alg / (us * 1e-6) / 1e9 / peak}
        del c2
    sweep["how"] = "median of 30 calls, CUDA events around the call, a 256 MB buffer written before each (L2 flushed)"
    return sweep


def reference_gpu_record(kb, device, ctx: int, batches=(8, 32)) -> dict:
    """The reference's own GPU path on this GPU: its Triton kernels from the copy under baseline/_ref (written by
    oracle/make_ref_copy.py: the slot index widened to int32, nothing else changed), fp16 as the reference requires.
    Attention: kitty_attention_forward of the reference on the very layer object the CUDA library uses (same field
    names, shapes and dtypes), next to the library's call — output difference and time of both, L2 flushed before
    every call.  Quantize: the reference's quantize_pack_k / quantize_pack_v (host prologue included) on one layer
    call of the bulk workload, next to the library's."""
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "kitty")):
        return {"unavailable": "baseline/_ref/kitty is absent (python oracle/make_ref_copy.py <reference checkout> writes it)"}
    if ref_dir not in sys.path:
        sys.path.insert(0, ref_dir)
    try:
        import kitty.kvcache.kernels.kitty_attention as ra
        import kitty.kvcache.kernels.kitty_quant_pack as rq
    except Exception as e:           # noqa: BLE001 - whatever the import raises is the record
        return {"unavailable": f"import failed: {type(e).__name__}: {str(e).splitlines()[0][:200]}"}
    mod = argparse.Namespace(num_attention_heads=H_Q, num_key_value_heads=H_KV)
    scaling = D ** -0.5
    rec = {"how": "reference = its Triton kernels compiled by the installed Triton for this GPU; fp16 q/k/v; median of "
                  "20 calls, CUDA events, a 256 MB buffer written before each call (L2 flushed)"}
    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=device)

    def timed(fn, n=20):
        for _ in range(3):
            fn()
        a, z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ts = []
        for _ in range(n):
            flush_buf.zero_()
            a.record()
            fn()
            z.record()
            z.synchronize()
            ts.append(a.elapsed_time(z))
        return statistics.median(ts) * 1e3

    try:
        att = {}
        for b in batches:
            c2 = build_cache(kb, b, ctx, 64, device, seed=7, dtype=torch.float16)
            l2 = c2.kv_cache[0]
            c2.update(torch.randn(b, H_KV, 1, D, device=device).half(), torch.randn(b, H_KV, 1, D, device=device).half(), 0)
            q = torch.randn(b, H_Q, 1, D, device=device).half()
            out_ref, _ = ra.kitty_attention_forward(mod, q, l2, scaling)
            out, _ = kb.kitty_attention_forward(mod, q, l2, scaling)
            err = float((out.float() - out_ref.float()).abs().max() / out_ref.float().abs().max())
            us_ref = timed(lambda: ra.kitty_attention_forward(mod, q, l2, scaling))
            us = timed(lambda: kb.kitty_attention_forward(mod, q, l2, scaling))
            att[f"batch{b}"] = {"reference_us": us_ref, "ours_us": us, "speedup": us_ref / us, "max_rel_diff": err}
            del c2
        rec["attention_32k"] = att
        # one layer call of the bulk quantize workload, fp16
        T, pages = 65536, 512
        g = torch.Generator(device=device).manual_seed(5)
        sc = torch.exp(torch.rand(1, H_KV, 1, D, generator=g, device=device) * 2.772588722239781)
        k = (torch.randn(1, H_KV, T, D, generator=g, device=device) * sc).half()
        v = torch.randn(1, H_KV, T, D, generator=g, device=device).half()
        z = dict(device=device)
        bufs = [(torch.zeros(pages, H_KV * 5248, dtype=torch.uint8, **z), torch.zeros(pages, H_KV, 128, 2, dtype=torch.float16, **z),
                 torch.zeros(pages, H_KV * 4096, dtype=torch.uint8, **z), torch.zeros(pages, H_KV, 128, 2, dtype=torch.float16, **z))
                for _ in range(2)]
        pt = torch.arange(pages, dtype=torch.int64, **z).view(1, pages)
        (rkc, rkm, rvc, rvm), (kc, km, vc, vm) = bufs
        from kitty_b200 import _lib

        rq.quantize_pack_k(k, 0, pages, pt, 0, rkc, rkm, 128, 32)
        rq.quantize_pack_v(v, 0, pages, pt, 0, rvc, rvm, 128)
        kb.quantize_pack_k(k, 0, pages, pt, 0, kc, km, 128, 32, selection="torch", div_mode=_lib.DIV_FULL)
        kb.quantize_pack_v(v, 0, pages, pt, 0, vc, vm, 128, div_mode=_lib.DIV_FULL)
        units = pages * H_KV
        rk = timed(lambda: rq.quantize_pack_k(k, 0, pages, pt, 0, rkc, rkm, 128, 32), 10)
        rv = timed(lambda: rq.quantize_pack_v(v, 0, pages, pt, 0, rvc, rvm, 128), 10)
        ok_ = timed(lambda: kb.quantize_pack_k(k, 0, pages, pt, 0, kc, km, 128, 32), 10)
        ov = timed(lambda: kb.quantize_pack_v(v, 0, pages, pt, 0, vc, vm, 128), 10)
        rec["quantize_layer_call"] = {
            "reference_k_us": rk, "ours_k_us": ok_, "k_speedup": rk / ok_, "reference_k_GBps": units * 38528 / rk / 1e3,
            "reference_v_us": rv, "ours_v_us": ov, "v_speedup": rv / ov, "reference_v_GBps": units * 37376 / rv / 1e3,
            "same_bytes_with_reference_division_and_selection": {
                "key_bytes": float((rkc == kc).float().mean()), "key_metadata": float((rkm == km).float().mean()),
                "value_bytes": float((rvc == vc).float().mean()), "value_metadata": float((rvm == vm).float().mean())},
            "note": "byte comparison: library run with the index bytes of abs().mean().topk() on this GPU and with "
                    "div.full.f32, the division Triton compiles; timing: library in its default mode (in-kernel "
                    "selection, IEEE division)"}
    except Exception as e:           # noqa: BLE001 - e.g. the Triton build for this GPU failed: record why
        rec["unavailable"] = f"{type(e).__name__}: {str(e).splitlines()[0][:300]}"
    return rec


def seqsplit_measure(kb, device, rank, world, dist, steps, warmup, seq_batch, exchange, tail_weight):
    """Per-layer-step latency (us, max over ranks) of the long-context shape: 28 query / 4 KV heads, 131072 cached
    tokens, the common pages split in contiguous ranges over `world` ranks (sink on rank 0, tail on the last rank).
    NL layers' caches take turns so that every step reads cold pages (NL x 43 MB per sequence > L2) and the steps
    are queued back to back, as the layers of a model are; the same seeds on every rank: same sequences."""
    global H_KV, H_Q
    from kitty_b200.seqsplit import PartialExchange, rank_flags, seq_split_decode, split_pages

    saved = (H_KV, H_Q)
    H_KV, H_Q = 4, 28
    try:
        ctx = 131072
        W, K, SB = max(3, warmup), steps, seq_batch
        REP = 5                                        # the median of REP repeats of K steps is reported
        NL = 8 if SB * 8 * 43 <= 4000 else 4
        if exchange in ("step", "graph"):
            # one cache of NL layers, as a model has: the token is planned once and every layer is one library call
            model_cache = build_cache(kb, SB, ctx, (W + REP * K) // NL + 4, device, seed=4321, layers=NL)
            caches = [model_cache]
        else:
            caches = [build_cache(kb, SB, ctx, (W + REP * K) // NL + 2, device, seed=4321 + j) for j in range(NL)]
        lay = caches[0].kv_cache[0]
        g = torch.Generator(device=device).manual_seed(17)
        qs = torch.randn(W + REP * K, SB, H_Q, 1, D, generator=g, device=device).to(torch.bfloat16)
        ks = torch.randn(W + REP * K, SB, H_KV, 1, D, generator=g, device=device).to(torch.bfloat16)
        vs = torch.randn(W + REP * K, SB, H_KV, 1, D, generator=g, device=device).to(torch.bfloat16)
        xch = PartialExchange(SB * H_Q, device) if (exchange in ("peer", "step", "graph") and world > 1) else None
        graph = [None, 0]                              # the captured token, eager tokens done

        def token_graphed():
            """One token = NL layer steps of the NL-layer cache, replayed from a CUDA graph as a model's decode step
            is (hf_adapter.GraphedDecoder): plan on the host, one graph launch, counters advanced on the host.  The
            captured layer calls read static inputs; counters, plan and exchange sequence come from the device block
            that plan_step() rewrites, so the same graph serves every token."""
            cache = caches[0]
            lo, hi = split_pages(cache.kv_cache[0].PageCount_V, world, tail_weight)[rank]
            cache.plan_step(SB, H_Q, page_begin=lo, page_end=hi, flags=rank_flags(rank, world),
                            exchange=xch if world > 1 else None)

            def layers():
                for li in range(NL):
                    cache.step_layer(li, ks[li], vs[li], qs[li], D ** -0.5)
            if graph[0] is None and graph[1] < 2:
                graph[1] += 1
                layers()                               # eager first: lazy initialisation must not be captured
            elif graph[0] is None:
                g_ = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g_):
                    layers()
                graph[0] = g_
                g_.replay()                            # capture records without running
            else:
                graph[0].replay()
            cache.finish_step()

        def step(i):
            if exchange == "step":
                # one library call per layer step, counters and plan in a device block written once per token
                cache, li = caches[0], i % NL
                if li == 0:
                    lo, hi = split_pages(cache.kv_cache[0].PageCount_V, world, tail_weight)[rank]
                    cache.plan_step(SB, H_Q, page_begin=lo, page_end=hi, flags=rank_flags(rank, world),
                                    exchange=xch if world > 1 else None)
                out = cache.step_layer(li, ks[i], vs[i], qs[i], D ** -0.5)
                if li == NL - 1:
                    cache.finish_step()
                return out
            cache = caches[i % NL]
            layer = cache.kv_cache[0]
            cache.update(ks[i], vs[i], 0)
            out = seq_split_decode(qs[i], layer, H_KV, D ** -0.5, rank=rank, world=world,
                                   n_common_pages=layer.PageCount_V, exchange=xch, tail_weight=tail_weight)
            cache.quantize_decode(0)
            return out

        if exchange == "graph":
            for _ in range(W // NL + 3):
                token_graphed()
        else:
            for i in range(W):
                step(i)
        reps = []
        for r in range(REP):
            torch.cuda.synchronize(device)
            if dist is not None and world > 1:
                dist.barrier()
            torch.cuda.synchronize(device)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            if exchange == "graph":
                for _ in range(K // NL):
                    token_graphed()
            else:
                for i in range(K):
                    step(W + r * K + i)
            e1.record()
            e1.synchronize()
            reps.append(e0.elapsed_time(e1) * (K / ((K // NL) * NL) if exchange == "graph" else 1.0))
        t = torch.tensor(reps, device=device, dtype=torch.float64)
        if dist is not None and world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)          # per repeat: the slowest rank
        if xch is not None:
            xch.check()
        packed = SB * H_KV * (lay.PageCount_K * K_PAGE_BYTES + lay.PageCount_V * V_PAGE_BYTES)
        return float(t.median()) / K * 1e3, packed, NL
    finally:
        H_KV, H_Q = saved


def seqsplit_record(kb, device, rank, world, dist, steps: int = 48, warmup: int = 8) -> dict:
    """The long-context configuration on `world` GPUs: per-layer-step latency with the two ways of combining the
    partials, next to the same sequence reduced by one GPU alone (rank 0's figure; the other ranks wait)."""
    rec = {"workload": "1 layer step, 28q/4kv heads, 131072 cached tokens, sequence split over the ranks in contiguous "
                       "page ranges; 8 layers' caches in turn (cold pages every step), steps queued back to back; CUDA "
                       "events, max over ranks, median of 5 repeats of the steps", "n_gpus": world, "steps": steps,
           "unit": "us"}
    peak, _ = hbm_peak()
    for sb in (1, 8):
        one = torch.zeros(2, device=device, dtype=torch.float64)
        if rank == 0:
            us1, packed, _ = seqsplit_measure(kb, device, 0, 1, None, steps, warmup, sb, "step", 0)
            one[0] = us1
            one[1], _, _ = seqsplit_measure(kb, device, 0, 1, None, steps, warmup, sb, "graph", 0)
        if world > 1:
            dist.all_reduce(one, op=dist.ReduceOp.MAX)
        us1 = float(one[0])
        r = {"one_gpu_us": us1, "one_gpu_graph_us": float(one[1])}
        for ex in ("graph", "step", "peer", "nccl"):
            us, packed, _ = seqsplit_measure(kb, device, rank, world, dist, steps, warmup, sb, ex, 0)
            base = float(one[1]) if ex == "graph" else us1      # like with like: graph replay against graph replay
            r[f"{ex}_us"] = us
            r[f"{ex}_speedup_vs_one_gpu"] = base / us
            r[f"{ex}_strong_scaling_efficiency"] = base / us / world
            r[f"{ex}_packed_kv_GBps_aggregate"] = packed / (us * 1e-6) / 1e9
        r["packed_kv_bytes"] = packed
        r["one_gpu_frac_of_peak"] = packed / (us1 * 1e-6) / 1e9 / peak
        rec[f"batch{sb}"] = r
    rec["collective"] = {"graph": "none: as 'step', with the layer steps of one token replayed from a CUDA graph (plan on "
                                  "the host, one graph launch per token, as hf_adapter.GraphedDecoder runs a model), so "
                                  "that no rank waits for another rank's host; the one-GPU figure next to it "
                                  "(one_gpu_graph_us) is replayed from a graph too",
                         "step": "none: as 'peer', with the whole layer step (append, attention, exchange, flush) in one "
                                 "library call from device-resident counters (kitty_decode_step_exchange) on one "
                                 "8-layer cache whose token is planned once for all layers, as in a model; the one-GPU "
                                 "figure uses the same one-call step (kitty_decode_step)",
                         "peer": "none: the attention call's merge step stores the partials into every rank's buffer over "
                                 "NVLink and waits (bounded) for the others (kitty_decode_attn_exchange)",
                         "nccl": "all_gather of [28,130] fp32 per rank + kitty_lse_merge"}
    return rec


def seqsplit_workload(args):
    """The sequence-split workload alone.  Launch under torchrun for N > 1."""
    import kitty_b200 as kb

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(device)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=device)
    us, packed, NL = seqsplit_measure(kb, device, rank, world, dist, args.steps, args.warmup, args.seq_batch,
                                      args.exchange, args.tail_weight)
    if rank == 0:
        print(json.dumps({"metric": "seqsplit_layer_step_latency", "value": us, "unit": "us", "n_gpus": world,
                          "steps": args.steps, "warmup": max(3, args.warmup), "higher_is_better": False, "dtype": "f16",
                          "data": "synthetic", "packed_kv_GBps_aggregate": packed / (us * 1e-6) / 1e9,
                          "config": {"workload": f"1 layer, 28q/4kv heads, batch {args.seq_batch}, 131072 cached tokens, "
                                                 f"sequence split over {world} GPU(s) (tail weight {args.tail_weight}), "
                                                 f"{NL} layers' caches in turn (cold pages every step), steps queued back to back",
                                     "collective": "peer-memory exchange inside the attention call" if args.exchange != "nccl"
                                     and world > 1 else "all_gather of [28,130] fp32 per rank + merge",
                                     "calls_per_step": 1 if args.exchange in ("step", "graph") else 3}}))
    if dist is not None:
        dist.destroy_process_group()


def decode_config(ctx: int, B: int, world: int) -> dict:
    """The `config` of the headline line, identical in both arms (the reference arm times a bounded sample of it)."""
    p = partition(ctx)
    return {"workload": f"decode step, 1 layer, 32q/8kv heads, head_dim 128, {ctx} cached tokens, bf16 q/k/v, "
                        "2-bit K (25% channels 4-bit) / 2-bit V pages",
            "batch_per_gpu": B, "global_batch": B * world, "parallelism": f"batch-sharded x{world}, no collective",
            "l2": f"inputs larger than L2 ({B * packed_bytes(p['pages_k'], p['pages_v']) / 1e6:.0f} MB of packed pages per GPU per step)"}


def main():
    args = parse()
    if args.workload == "seqsplit" and args.impl == "ours":
        return seqsplit_workload(args)
    if args.workload == "quantize" and args.impl == "ours":
        return quantize_workload(args)
    if args.workload == "e2e" and args.impl == "ours":
        return e2e_workload(args)
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        if rank != 0:
            return
        r = cpu_reference(args.ctx, args.steps, args.warmup, budget_s=120.0)
        line = {"impl": "reference", "metric": "decode_attn_packed_kv_throughput", "value": r["value"], "unit": "GB/s",
                "n_gpus": args.gpus, "steps": r["steps"], "warmup": args.warmup, "ms_per_step": r["ms_per_step"],
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": decode_config(args.ctx, args.batch, args.gpus),
                "sample_note": "each step is ONE sequence of the configuration's batch (the reference's PyTorch path in "
                               "fp32 on the host cores); throughput is per byte of packed KV, so the sample scales",
                "cpu_baseline": {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")},
                "decode_tokens_per_s": r["tokens_per_s"],
                "e2e": {"value": r["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (kitty_b200 has no CPU path)")
    import kitty_b200 as kb
    from kitty_b200 import _lib

    _lib.lib()
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=device)

    B, W, K = args.batch, args.warmup, args.steps
    if W < 3:
        W = 3
    E2E_REPEATS = 5
    total = (W + K) + (W + E2E_REPEATS * K)     # device-timed pass, then the end-to-end pass
    cache = build_cache(kb, B, args.ctx, total, device, seed=1234 + rank)
    lay = cache.kv_cache[0]
    mod = argparse.Namespace(num_attention_heads=H_Q, num_key_value_heads=H_KV)
    scaling = D ** -0.5
    g = torch.Generator(device=device).manual_seed(99 + rank)
    n_dev = W + K
    qs = torch.randn(n_dev, B, H_Q, 1, D, generator=g, device=device).to(torch.bfloat16)
    ks = torch.randn(n_dev, B, H_KV, 1, D, generator=g, device=device).to(torch.bfloat16)
    vs = torch.randn(n_dev, B, H_KV, 1, D, generator=g, device=device).to(torch.bfloat16)
    launches = {"n": 0}
    flush_log = []

    def step(q, k, v):
        cache.update(k, v, 0)
        out, _ = kb.kitty_attention_forward(mod, q, lay, scaling)
        flush = lay.Q_Buffer_Count_K == 128 or lay.Q_Buffer_Count_V == 128
        cache.quantize_decode(0)
        launches["n"] += 3 + (1 if flush else 0)      # append, streaming (pages + edges), merge (+ flush)
        flush_log.append(flush)
        return out

    def barrier():
        torch.cuda.synchronize(device)
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize(device)

    # ---------------- device-timed pass: inputs resident in HBM ---------------- #
    for i in range(W):
        step(qs[i], ks[i], vs[i])
    barrier()
    launches["n"] = 0
    flush_log.clear()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    attn_ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(K)]
    packed = attn_alg = 0
    with ClockSampler(local_rank) as clocks:
        ev0.record()
        for i in range(K):
            q, k, v = qs[W + i], ks[W + i], vs[W + i]
            cache.update(k, v, 0)
            packed += B * packed_bytes(lay.PageCount_K, lay.PageCount_V)
            attn_alg += B * attention_bytes(lay)
            attn_ev[i][0].record()
            kb.kitty_attention_forward(mod, q, lay, scaling)
            attn_ev[i][1].record()
            flush = lay.Q_Buffer_Count_K == 128 or lay.Q_Buffer_Count_V == 128
            cache.quantize_decode(0)
            launches["n"] += 3 + (1 if flush else 0)
            flush_log.append(flush)
        ev1.record()
        barrier()
    ms = ev0.elapsed_time(ev1)
    attn_ms = sum(a.elapsed_time(b) for a, b in attn_ev)
    gpu_launches = launches["n"]
    flush_steps_value = [i for i, f in enumerate(flush_log) if f]
    t = torch.tensor([ms, attn_ms], device=device, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, attn_ms = float(t[0]), float(t[1])
    value = world * packed / (ms * 1e-3) / 1e9
    tokens_per_s = world * B * K / (ms * 1e-3)
    del qs, ks, vs

    # ---------------- end-to-end pass: pinned host inputs, result copied back every step ---------------- #
    # one pinned buffer per step, [q | k | v] back to back: a single host-to-device copy.  E2E_REPEATS repeats of the
    # K steps are timed one by one (host clock, barrier on both sides) and the median repeat is reported: a step here
    # is bound by host latency (copy in, launch, copy out, synchronise), which is noisy over a few milliseconds.
    nq, nk = B * H_Q * D, B * H_KV * D
    n_e2e = W + E2E_REPEATS * K
    gh = torch.Generator().manual_seed(7 + rank)
    hin = torch.randn(n_e2e, nq + 2 * nk, generator=gh).to(torch.bfloat16).pin_memory()
    hout = torch.empty(B, 1, H_Q, D, dtype=torch.bfloat16).pin_memory()

    def e2e_step(i):
        x = hin[i].to(device, non_blocking=True)
        q = x[:nq].view(B, H_Q, 1, D)
        k = x[nq:nq + nk].view(B, H_KV, 1, D)
        v = x[nq + nk:].view(B, H_KV, 1, D)
        out = step(q, k, v)
        hout.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()       # the caller reads the result of every step

    for i in range(W):
        e2e_step(i)
    barrier()
    flush_log.clear()
    rep_s, rep_bytes = [], []
    with ClockSampler(local_rank, interval_s=0.005) as clocks_e:      # second timed region: its samples join the first region's
        for r in range(E2E_REPEATS):
            nbytes = 0
            t0 = time.perf_counter()
            for i in range(K):
                e2e_step(W + r * K + i)
                nbytes += B * packed_bytes(lay.PageCount_K, lay.PageCount_V)
            barrier()
            rep_s.append(time.perf_counter() - t0)
            rep_bytes.append(nbytes)
    clocks.samples += clocks_e.samples
    clocks.reasons |= clocks_e.reasons
    te = torch.tensor(rep_s, device=device, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(te, op=dist.ReduceOp.MAX)
    rep_s = [float(x) for x in te]
    mid = sorted(range(E2E_REPEATS), key=lambda r: rep_s[r])[E2E_REPEATS // 2]
    e2e_s, packed_e = rep_s[mid], rep_bytes[mid]
    flush_steps_e2e = [i for i, f in enumerate(flush_log) if f]
    h2d = B * (H_Q + 2 * H_KV) * D * 2
    d2h = B * H_Q * D * 2
    from kitty_b200.attention import workspace_status

    if workspace_status(lay) != 0:
        raise SystemExit("device-side bounded wait ran out during the benchmark")
    pages_v = lay.PageCount_V
    del cache, lay, hin
    torch.cuda.empty_cache()

    # ---------------- records of the other workloads (own timing each) ---------------- #
    extras = {}
    if not args.no_extras:
        if world == 1:
            extras["sweep"] = sweep_record(kb, device, args.ctx)
            extras["quantize"] = quantize_record(device)
            torch.cuda.empty_cache()
            extras["model_e2e"] = model_record(device)
            extras["reference_gpu"] = reference_gpu_record(kb, device, args.ctx)
        else:
            extras["seqsplit"] = seqsplit_record(kb, device, rank, world, dist)

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    peak, peak_src = hbm_peak()
    achieved = (attn_alg / K) / (attn_ms / K * 1e-3) / 1e9     # per attention call, this rank
    line = {
        "metric": "decode_attn_packed_kv_throughput", "value": value, "unit": "GB/s", "n_gpus": world, "steps": K,
        "warmup": W, "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16", "data": "synthetic",
        "dtype_note": "arithmetic type of the path: q/k/v arrive as bf16, the cache's full-precision buffers and the "
                      "(scale, min) metadata are fp16 as in the reference, dequantisation and softmax accumulate in fp32",
        "config": decode_config(args.ctx, B, world),
        "flush_steps": {"value": flush_steps_value, "e2e": flush_steps_e2e,
                        "note": "indices of the timed steps in which a full Q-buffer was quantized into a page (the "
                                "Q-buffers hold 96 tokens after the prompt, so the first flush is the 32nd step after "
                                "it); e2e: indices over all 5 repeats"},
        "decode_tokens_per_s": tokens_per_s,
        "e2e": {"value": world * packed_e / e2e_s / 1e9, "unit": "GB/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": e2e_s / K * 1e3, "decode_tokens_per_s": world * B * K / e2e_s,
                "repeats": E2E_REPEATS, "repeat_ms_per_step": [x / K * 1e3 for x in rep_s], "statistic": "median repeat"},
        "gpu_launches": gpu_launches,
        "clocks": clocks.summary(),
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": B * H_KV * pages_v * DRAM_BYTES_PER_PAGE_PAIR, "peak_source": peak_src,
                     "kernel": "decode attention call = decode_paged_i8_kernel (page pairs and edges, >97 % of the "
                               "step's device time in the ncu launch list) + merge_kernel; achieved = algorithmic bytes of "
                               "the call / CUDA-event time of the call; traffic = ncu DRAM bytes of the streaming "
                               "kernel per page pair (batch-8 capture) x page pairs of one launch",
                     "algorithmic_bytes_per_call": attn_alg / K, "ms_per_call": attn_ms / K},
    }
    if world == 1 and not args.no_cpu_baseline:
        r = cpu_reference(args.ctx, 40, 2, budget_s=20.0)
        line["cpu_baseline"] = {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")}
    line.update(extras)
    print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
