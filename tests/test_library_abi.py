"""The C-ABI library loads and exports every symbol the public header declares
(no compute calls: runs without a GPU)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "kitty_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(kitty_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    from kitty_b200 import _lib

    assert _declared() == sorted(_lib.EXPORTS)


def test_library_exports_every_declared_symbol():
    from kitty_b200 import _lib, build

    build.build()
    L = ctypes.CDLL(_lib.LIB_PATH)
    for name in _declared():
        assert hasattr(L, name), name
    assert _lib.lib().kitty_version() >= 100
    for code in (0, -1, -2, -3, -4, -5):
        assert _lib.strerror(code) != "unknown status"
    assert _lib.strerror(-99) == "unknown status"


def test_struct_sizes_match_the_header():
    from kitty_b200 import _lib

    assert ctypes.sizeof(_lib.KittyCounts) == 32
    assert ctypes.sizeof(_lib.KittyStepState) == 168          # 3 x kitty_counts + 18 ints (the header says so)
    assert ctypes.sizeof(_lib.KittyLayer) == 8 * 4 + 11 * 8


def test_argument_errors_need_no_gpu():
    from kitty_b200 import _lib

    L = _lib.lib()
    assert L.kitty_decode_workspace_bytes(1, 8, 30, 16) == _lib.KITTY_E_BADARG      # h_q not a multiple of h_kv
    assert L.kitty_decode_workspace_bytes(1, 1, 17, 16) == _lib.KITTY_E_BADSHAPE    # group > 16
    assert L.kitty_decode_workspace_bytes(1, 8, 32, 256) > 256
    assert L.kitty_quant_pack_v(None, 0, 0, 0, 0, 1, 1, 0, 1, None, 0, 0, None, 0, None, 0, None) == _lib.KITTY_E_BADARG
    with pytest.raises(_lib.KittyError):
        _lib.check(_lib.KITTY_E_WORKSPACE, "x")


def test_no_cpu_path():
    import torch
    from kitty_b200 import KVCache_Layer, quantize_pack_v

    with pytest.raises(ValueError):
        KVCache_Layer(1, 256, 1, 128, 32, 2, 4, 128, 32, device="cpu")
    x = torch.zeros(1, 1, 128, 128, dtype=torch.float16)
    with pytest.raises(ValueError):
        quantize_pack_v(x, 0, 1, torch.zeros(1, 1, dtype=torch.int64), 0, torch.zeros(1, 4096, dtype=torch.uint8),
                        torch.zeros(1, 1, 128, 2, dtype=torch.float16), 128)
