"""The restated CPU baseline (oracle/kitty_sim_port.py) against outputs of the reference's own simulator
(tests/golden/sim_port.npz, written by tests/golden/make_sim_golden.py from src/kitty_sim): bit-equal fake-quant
outputs, promote masks and cache contents through a prompt and decode steps past a key quantization."""
import numpy as np
import torch

from oracle import kitty_sim_port as sp
from tests.helpers import load


def test_fake_quant_and_mask_match_the_reference():
    fx = load("sim_port")
    k = torch.from_numpy(fx["fq_key_in"])
    mask = sp.promote_mask_magnitude(k, 0.25)
    assert np.array_equal(mask.numpy(), fx["fq_mask"]) and int(mask.sum()) == 32
    assert np.array_equal(sp.fake_quant_lastdim(k, 128, 2, mask, 4).numpy(), fx["fq_key_out"])
    v = torch.from_numpy(fx["fq_val_in"])
    assert np.array_equal(sp.fake_quant_lastdim(v, 128, 2).numpy(), fx["fq_val_out"])
    h = torch.from_numpy(fx["fq_f16_in"]).view(torch.float16)          # 16-bit input: range floor 1e-4, fp16 arithmetic
    assert np.array_equal(sp.fake_quant_lastdim(h, 128, 2).view(torch.int16).numpy(), fx["fq_f16_out"])


def test_cache_state_machine_matches_the_reference():
    fx = load("sim_port")
    cache = sp.SimKittyCache()
    k0, v0 = torch.from_numpy(fx["k_prefill"]), torch.from_numpy(fx["v_prefill"])
    kr, vr = cache.update(k0, v0)
    assert torch.equal(kr, k0) and torch.equal(vr, v0)                 # the prompt step sees full precision
    assert np.array_equal(cache.k.numpy(), fx["prefill_key_cache"])
    assert np.array_equal(cache.v.numpy(), fx["prefill_value_cache"])
    probes = list(fx["probe_steps"])
    for s in range(fx["k_steps"].shape[0]):
        kr, vr = cache.update(torch.from_numpy(fx["k_steps"][s]), torch.from_numpy(fx["v_steps"][s]))
        if s in probes:
            i = probes.index(s)
            assert np.array_equal(kr.numpy(), fx[f"keys_returned_{i}"]), s
            assert np.array_equal(vr.numpy(), fx[f"values_returned_{i}"]), s
    assert np.array_equal(cache.k.numpy(), fx["final_key_cache"])
    assert np.array_equal(cache.v.numpy(), fx["final_value_cache"])
    # something was quantized on the way: the stored keys are not the inputs any more
    assert not np.array_equal(fx["final_key_cache"][:, :, :280], fx["k_prefill"])
