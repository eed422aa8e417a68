"""Shared helpers for the tests: fixture decoding and seeded input generators."""
import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
COUNTERS = ["PageCount_K", "PageCount_V", "Sink_Count", "Q_Buffer_Count_K", "Q_Buffer_Count_V", "Local_Count_V",
            "Write_Offset_Local_V"]
BUFFERS = ["KeyCache", "KeyCache_metadata", "ValueCache", "ValueCache_metadata", "PageTable_K", "PageTable_V",
           "Sink_Buffer_K", "Sink_Buffer_V", "Q_Buffer_K", "Q_Buffer_V", "Local_Buffer_V"]


def load(name):
    return np.load(os.path.join(GOLDEN, name + ".npz"))


def tensor_from_raw(raw, dtype: str) -> torch.Tensor:
    """uint16 bit patterns (or fp32 values) from a fixture → torch tensor of that dtype."""
    if dtype == "f32":
        return torch.from_numpy(np.ascontiguousarray(raw))
    t = torch.from_numpy(np.ascontiguousarray(raw).view(np.int16))
    return t.view(torch.float16 if dtype == "f16" else torch.bfloat16)


def make_kv(B, H, T, D, seed, dtype=torch.float16, kind="outlier8"):
    """Seeded synthetic keys/values: Gaussian, with either 4 channels per head
    scaled x8 or per-(head, channel) scales drawn log-uniform in [1, 16]."""
    g = torch.Generator().manual_seed(seed)
    k = torch.randn(B, H, T, D, generator=g)
    if kind == "outlier8":
        for h in range(H):
            k[:, h, :, torch.randperm(D, generator=g)[:4]] *= 8.0
    elif kind == "loguniform":
        k = k * torch.exp(torch.rand(1, H, 1, D, generator=g) * float(np.log(16.0)))
    v = torch.randn(B, H, T, D, generator=g)
    return k.to(dtype), v.to(dtype)
