"""ctypes binding of libkitty_b200.so (declarations in include/kitty_b200.h).

There is no CPU or PyTorch fallback: if the shared library is missing or a call
fails, the error is raised to the caller.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "lib", "libkitty_b200.so")

KITTY_OK, KITTY_E_BADARG, KITTY_E_BADSHAPE, KITTY_E_WORKSPACE, KITTY_E_CUDA, KITTY_E_TIMEOUT = 0, -1, -2, -3, -4, -5
KITTY_E_STATIC_LIMIT = -6
STATIC_SCRATCH_BYTES = 8 << 20
KITTY_F16, KITTY_BF16, KITTY_F32 = 0, 1, 2
SELECT_FUSED, SELECT_SUPPLIED = 0, 1
DIV_IEEE, DIV_FULL = 0, 1

EXPORTS = [
    "kitty_version", "kitty_strerror", "kitty_quant_pack_k", "kitty_quant_pack_v", "kitty_quant_pack_kv",
    "kitty_prefill_tails",
    "kitty_append", "kitty_flush", "kitty_decode_workspace_bytes", "kitty_workspace_status", "kitty_decode_attn",
    "kitty_lse_merge", "kitty_decode_attn_static", "kitty_plan_step", "kitty_decode_step",
    "kitty_lse_exchange_bytes", "kitty_lse_exchange_merge", "kitty_decode_attn_exchange", "kitty_rope_qk",
    "kitty_plan_step_split", "kitty_decode_step_exchange", "kitty_append_rows", "kitty_flush_rows",
    "kitty_decode_attn_rows",
]


class KittyLayer(C.Structure):
    """struct kitty_layer"""
    _fields_ = [(n, C.c_int32) for n in
                ("max_bs", "max_page", "h_kv", "head_dim", "d_boost", "page_size", "sink_size", "reserved")] + \
               [(n, C.c_void_p) for n in
                ("KeyCache", "KeyCache_metadata", "ValueCache", "ValueCache_metadata", "PageTable_K", "PageTable_V",
                 "Sink_Buffer_K", "Sink_Buffer_V", "Q_Buffer_K", "Q_Buffer_V", "Local_Buffer_V")]


class KittyCounts(C.Structure):
    """struct kitty_counts"""
    _fields_ = [(n, C.c_int32) for n in
                ("PageCount_K", "PageCount_V", "Sink_Count", "Q_Buffer_Count_K", "Q_Buffer_Count_V", "Local_Count_V",
                 "Write_Offset_Local_V", "reserved")]


class KittyStepState(C.Structure):
    """struct kitty_step_state"""
    _fields_ = [("before", KittyCounts), ("after", KittyCounts), ("next", KittyCounts)] + \
               [(n, C.c_int32) for n in ("pb", "pe", "ch", "nchunk", "has_sink", "has_tail", "n_slots", "n_tiles",
                                         "chunk_slot0", "edge_slot", "n_items", "n_edge", "flush_k", "flush_v",
                                         "edge_parts", "edge_part_tok", "xchg_seq", "reserved")]


class KittyError(RuntimeError):
    def __init__(self, status: int, where: str):
        self.status = status
        super().__init__(f"{where}: {strerror(status)} (status {status})")


_lib = None


def lib() -> C.CDLL:
    """The loaded library; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing. Build the CUDA library first: python -m kitty_b200.build "
            "(kitty_b200 has no CPU fallback).")
    L = C.CDLL(LIB_PATH)
    i32, i64, vp = C.c_int32, C.c_int64, C.c_void_p
    L.kitty_version.restype = C.c_int
    L.kitty_strerror.restype = C.c_char_p
    L.kitty_strerror.argtypes = [C.c_int]
    L.kitty_quant_pack_k.restype = C.c_int
    L.kitty_quant_pack_k.argtypes = [vp, C.c_int, i64, i64, i64, i32, i32, i64, i32, vp, i64, i32, vp, i64, vp, vp,
                                     C.c_int, C.c_int, vp]
    L.kitty_quant_pack_v.restype = C.c_int
    L.kitty_quant_pack_v.argtypes = [vp, C.c_int, i64, i64, i64, i32, i32, i64, i32, vp, i64, i32, vp, i64, vp,
                                     C.c_int, vp]
    L.kitty_quant_pack_kv.restype = C.c_int
    L.kitty_quant_pack_kv.argtypes = [vp, vp, C.c_int, i64, i64, i64, i64, i64, i64, i32, i32,
                                      i64, i32, vp, i64, i32, vp, i64, vp, vp, C.c_int,
                                      i64, i32, vp, i64, i32, vp, i64, vp, C.c_int, vp]
    L.kitty_prefill_tails.restype = C.c_int
    L.kitty_prefill_tails.argtypes = [C.POINTER(KittyLayer), vp, vp, C.c_int, i64, i64, i64, i64, i64, i64, i32, i64,
                                      i32, i32, i32, i32, vp]
    L.kitty_append.restype = C.c_int
    L.kitty_append.argtypes = [C.POINTER(KittyLayer), C.POINTER(KittyCounts), vp, vp, C.c_int, i64, i64, i64, i64, i32,
                               vp]
    L.kitty_flush.restype = C.c_int
    L.kitty_flush.argtypes = [C.POINTER(KittyLayer), C.POINTER(KittyCounts), i32, C.c_int, C.c_int, C.c_int, C.c_int,
                              vp]
    L.kitty_decode_workspace_bytes.restype = i64
    L.kitty_decode_workspace_bytes.argtypes = [i32, i32, i32, i32]
    L.kitty_workspace_status.restype = C.c_int
    L.kitty_workspace_status.argtypes = [vp, C.POINTER(i32), vp]
    L.kitty_decode_attn.restype = C.c_int
    L.kitty_decode_attn.argtypes = [C.POINTER(KittyLayer), C.POINTER(KittyCounts), vp, C.c_int, i32, i32, C.c_float,
                                    vp, C.c_int, vp, i64, i32, i32, i32, vp, C.c_int, vp]
    L.kitty_decode_attn_static.restype = C.c_int
    L.kitty_decode_attn_static.argtypes = [C.POINTER(KittyLayer), C.POINTER(KittyCounts), vp, C.c_int, i32, i32,
                                           C.c_float, vp, C.c_int, i32, i32, i32, vp, C.c_int, vp, vp]
    L.kitty_plan_step.restype = C.c_int
    L.kitty_plan_step.argtypes = [C.POINTER(KittyLayer), C.POINTER(KittyCounts), i32, i32, C.POINTER(KittyStepState),
                                  vp, vp]
    L.kitty_decode_step.restype = C.c_int
    L.kitty_decode_step.argtypes = [C.POINTER(KittyLayer), vp, vp, vp, C.c_int, i64, i64, i64, i64, vp, C.c_int, i32,
                                    i32, C.c_float, vp, C.c_int, vp, i64, C.c_int, vp]
    L.kitty_plan_step_split.restype = C.c_int
    L.kitty_plan_step_split.argtypes = [C.POINTER(KittyLayer), C.POINTER(KittyCounts), i32, i32, i32, i32, i32, i32,
                                        C.POINTER(KittyStepState), vp, vp]
    L.kitty_decode_step_exchange.restype = C.c_int
    L.kitty_decode_step_exchange.argtypes = [C.POINTER(KittyLayer), vp, vp, vp, C.c_int, i64, i64, i64, i64, vp, C.c_int,
                                             i32, i32, C.c_float, vp, C.c_int, vp, i64, C.c_int, vp, i32, i32, i32, vp,
                                             i64, vp]
    L.kitty_append_rows.restype = C.c_int
    L.kitty_append_rows.argtypes = [C.POINTER(KittyLayer), vp, vp, vp, vp, C.c_int, i64, i64, i64, i64, i32, vp]
    L.kitty_flush_rows.restype = C.c_int
    L.kitty_flush_rows.argtypes = [C.POINTER(KittyLayer), vp, vp, i32, C.c_int, C.c_int, vp]
    L.kitty_decode_attn_rows.restype = C.c_int
    L.kitty_decode_attn_rows.argtypes = [C.POINTER(KittyLayer), vp, vp, vp, C.c_int, i32, i32, C.c_float, vp, C.c_int,
                                         vp, i64, C.c_int, vp]
    L.kitty_decode_attn_exchange.restype = C.c_int
    L.kitty_decode_attn_exchange.argtypes = [C.POINTER(KittyLayer), C.POINTER(KittyCounts), vp, C.c_int, i32, i32,
                                             C.c_float, vp, C.c_int, vp, i64, i32, i32, i32, C.c_int, vp, i32, i32, i32,
                                             vp, i64, vp]
    L.kitty_rope_qk.restype = C.c_int
    L.kitty_rope_qk.argtypes = [vp, vp, vp, vp, vp, vp, C.c_int, i32, i32, i32, i64, vp]
    L.kitty_lse_exchange_bytes.restype = i64
    L.kitty_lse_exchange_bytes.argtypes = [i64, i32, C.POINTER(i64)]
    L.kitty_lse_exchange_merge.restype = C.c_int
    L.kitty_lse_exchange_merge.argtypes = [vp, i64, vp, i32, i32, i32, vp, C.c_int, vp, i64, vp]
    L.kitty_lse_merge.restype = C.c_int
    L.kitty_lse_merge.argtypes = [vp, i32, i64, vp, C.c_int, vp]
    _lib = L
    return L


def strerror(status: int) -> str:
    return lib().kitty_strerror(int(status)).decode()


def check(status: int, where: str) -> None:
    if status != KITTY_OK:
        raise KittyError(int(status), where)


def dtype_code(dtype) -> int:
    import torch

    try:
        return {torch.float16: KITTY_F16, torch.bfloat16: KITTY_BF16, torch.float32: KITTY_F32}[dtype]
    except KeyError:
        raise TypeError(f"kitty_b200 supports float16, bfloat16 and float32 tensors, got {dtype}") from None


def stream_ptr(device) -> int:
    import torch

    return torch.cuda.current_stream(device).cuda_stream
