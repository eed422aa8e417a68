"""Write a runnable copy of the reference's Triton kernels into baseline/_ref/ (git-ignored; it travels to the GPU box
with the working tree).  TEST/BENCH INFRASTRUCTURE ONLY — nothing in kitty_b200/ imports it.

    python oracle/make_ref_copy.py /path/to/Kitty

Three files of the reference are copied unchanged except for one token each in the two kernel files: the uint8 slot
index is widened to int32 before it is multiplied by the 32-byte row stride (kvcache/kernels/kitty_quant_pack.py:141,
kvcache/kernels/kitty_attention.py:154).  Under current Triton the product stays uint8 and wraps, so the 32 high-plane
rows alias onto 8; the widened form addresses the 32 distinct rows the buffer is sized for
(kvcache/utils_kv_per_layer.py:35).  The package __init__ files are written empty, because the reference's own import
kvcache/kitty.py, which needs a transformers class that no longer exists.

With the copy in place the benchmark can time the reference's own GPU path (kitty_attention_forward, quantize_pack_k,
quantize_pack_v) on the same B200 and the same cache contents as the CUDA library, and a GPU test compares the two.
"""
from __future__ import annotations

import os
import shutil
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DEST = os.path.join(ROOT, "baseline", "_ref")

PATCHES = {
    "kvcache/kernels/kitty_quant_pack.py": [
        ("+ dense_sparse_idx[None, :] * K_STRIDE_D", "+ dense_sparse_idx[None, :].to(tl.int32) * K_STRIDE_D")],
    "kvcache/kernels/kitty_attention.py": [
        ("+ boost_idx[:, None] * K_STRIDE_D", "+ boost_idx[:, None].to(tl.int32) * K_STRIDE_D")],
    "kvcache/utils_kv_per_layer.py": [],
}


def make(ref_root: str) -> str:
    src = os.path.join(ref_root, "src", "kitty")
    if not os.path.isdir(src):
        raise FileNotFoundError(f"{src}: not a checkout of the reference")
    pkg = os.path.join(DEST, "kitty")
    if os.path.isdir(pkg):
        shutil.rmtree(pkg)
    for rel, subs in PATCHES.items():
        text = open(os.path.join(src, rel)).read()
        for old, new in subs:
            assert text.count(old) == 1, (rel, old)
            text = text.replace(old, new)
        dst = os.path.join(pkg, rel)
        os.makedirs(os.path.dirname(dst), exist_ok=True)
        open(dst, "w").write(text)
    for d in ("", "kvcache", "kvcache/kernels"):
        open(os.path.join(pkg, d, "__init__.py"), "w").close()
    return pkg


if __name__ == "__main__":
    print(make(sys.argv[1] if len(sys.argv) > 1 else os.environ.get("KITTY_REFERENCE", "/root/reference")))
