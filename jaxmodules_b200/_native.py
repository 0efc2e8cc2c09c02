"""ctypes binding of libbma.so (the C ABI declared in include/bma.h).

There is no fallback: if the library has not been built, importing the symbols raises, and
every compute entry point needs a CUDA device.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

_LIB_PATH = Path(__file__).resolve().parent / "libbma.so"

BMA_OK = 0
BMA_ERR_ARG, BMA_ERR_UNSUPPORTED, BMA_ERR_WORKSPACE, BMA_ERR_CUDA, BMA_ERR_LIMIT = -1, -2, -3, -4, -5
BMA_ERR_DEVICE_CHECK = 1
BMA_DTYPE_F32, BMA_DTYPE_BF16 = 0, 1
BMA_MASK_CAUSAL, BMA_MASK_BAND, BMA_MASK_BLOCK_WINDOW, BMA_MASK_SEGMENT, BMA_MASK_BITMAP, BMA_MASK_TILES = 1, 2, 4, 8, 16, 32
BMA_MASK_COMPILE_CONSERVATIVE = 256
BMA_BACKEND_AUTO, BMA_BACKEND_SIMT, BMA_BACKEND_TCGEN05 = 0, 1, 2


class MaskSpec(C.Structure):
    _fields_ = [
        ("flags", C.c_int32),
        ("q_valid", C.c_int32), ("k_valid", C.c_int32),
        ("q_offset", C.c_int32), ("k_offset", C.c_int32),
        ("band_left", C.c_int32), ("band_right", C.c_int32),
        ("win_block", C.c_int32), ("win_left", C.c_int32), ("win_right", C.c_int32), ("win_nblk", C.c_int32),
        ("bitmap_B", C.c_int32), ("bitmap_H", C.c_int32), ("bitmap_q", C.c_int32), ("bitmap_words", C.c_int32),
        ("reserved_", C.c_int32),
        ("seg_q", C.c_void_p), ("seg_k", C.c_void_p),
        ("seg_q_stride", C.c_int64), ("seg_k_stride", C.c_int64),
        ("bitmap", C.c_void_p),
        ("tiles_B", C.c_int32), ("tiles_H", C.c_int32), ("tiles_q", C.c_int32), ("tiles_k", C.c_int32),
        ("tile_class", C.c_void_p), ("tile_slot", C.c_void_p), ("tile_bits", C.c_void_p),
    ]


class BlockLists(C.Structure):
    _fields_ = [
        ("B", C.c_int32), ("H", C.c_int32), ("NQ", C.c_int32), ("NKV", C.c_int32),
        ("q_block", C.c_int32), ("kv_block", C.c_int32),
        ("kv_num", C.c_void_p), ("kv_idx", C.c_void_p),
        ("full_kv_num", C.c_void_p), ("full_kv_idx", C.c_void_p),
        ("q_num", C.c_void_p), ("q_idx", C.c_void_p),
        ("full_q_num", C.c_void_p), ("full_q_idx", C.c_void_p),
    ]


PROGRAM_MAX_INSTR, PROGRAM_MAX_TABLES = 60, 4
OPS = ["CONST", "NEG", "ABS", "NOT", "INV", "ADD", "SUB", "MUL", "FLOORDIV", "MOD", "MIN", "MAX",
       "LT", "LE", "GT", "GE", "EQ", "NE", "AND", "OR", "XOR", "SHL", "SHR", "SELECT", "LOAD1", "LOAD2"]
OP = {name: i for i, name in enumerate(OPS)}


class MaskProgram(C.Structure):
    """bma_mask_program of include/bma.h."""
    _fields_ = [
        ("n_instr", C.c_int32), ("n_tables", C.c_int32),
        ("code", C.c_int32 * (4 * PROGRAM_MAX_INSTR)),
        ("tables", C.c_void_p * PROGRAM_MAX_TABLES),
        ("table_rows", C.c_int64 * PROGRAM_MAX_TABLES),
        ("table_cols", C.c_int64 * PROGRAM_MAX_TABLES),
        ("table_stride", C.c_int64 * PROGRAM_MAX_TABLES),
    ]


class Tensor(C.Structure):
    _fields_ = [
        ("ptr", C.c_void_p),
        ("stride_b", C.c_int64), ("stride_l", C.c_int64), ("stride_h", C.c_int64),
        ("dtype", C.c_int32), ("reserved_", C.c_int32),
    ]


class AttnArgs(C.Structure):
    _fields_ = [
        ("B", C.c_int32), ("N", C.c_int32), ("L", C.c_int32), ("Hq", C.c_int32), ("Hkv", C.c_int32), ("d", C.c_int32),
        ("scale", C.c_float), ("backend", C.c_int32),
        ("q", Tensor), ("k", Tensor), ("v", Tensor),
        ("o", Tensor), ("lse", C.c_void_p),
        ("d_o", Tensor), ("delta", C.c_void_p),
        ("dq", Tensor), ("dk", Tensor), ("dv", Tensor),
        ("key_bias", C.c_void_p),
    ]


# name -> (restype, argtypes); the single source for the loader and for the symbol test
SIGNATURES = {
    "bma_version": (C.c_int, []),
    "bma_launch_count": (C.c_ulonglong, []),
    "bma_error_string": (C.c_char_p, [C.c_int]),
    "bma_mask_compile_workspace_bytes": (C.c_size_t, [C.POINTER(MaskSpec), C.c_int32, C.c_int32, C.c_int32, C.c_int32]),
    "bma_mask_compile": (C.c_int, [C.POINTER(MaskSpec), C.c_int32, C.c_int32, C.POINTER(BlockLists), C.c_void_p,
                                   C.c_size_t, C.c_void_p]),
    "bma_mask_compile_static_limit": (C.c_size_t, []),
    "bma_mask_compile_static": (C.c_int, [C.POINTER(MaskSpec), C.c_int32, C.c_int32, C.POINTER(BlockLists), C.c_void_p]),
    "bma_mask_table_build": (C.c_int, [C.POINTER(MaskProgram), C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                       C.c_void_p, C.c_void_p]),
    "bma_mask_tiles_build": (C.c_int, [C.POINTER(MaskProgram), C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                       C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p]),
    "bma_attn_plan": (C.c_int, [C.POINTER(AttnArgs), C.POINTER(C.c_int32), C.POINTER(C.c_int32), C.POINTER(C.c_int32)]),
    "bma_attn_bwd_plan": (C.c_int, [C.POINTER(AttnArgs), C.POINTER(C.c_int32), C.POINTER(C.c_int32), C.POINTER(C.c_int32)]),
    "bma_attn_fwd": (C.c_int, [C.POINTER(AttnArgs), C.POINTER(MaskSpec), C.POINTER(BlockLists), C.c_void_p]),
    "bma_attn_bwd_preprocess": (C.c_int, [C.POINTER(AttnArgs), C.c_void_p, C.c_void_p]),
    "bma_attn_bwd_workspace_bytes": (C.c_size_t, [C.POINTER(AttnArgs)]),
    "bma_block_lists_visited": (C.c_int, [C.POINTER(BlockLists), C.c_void_p, C.c_void_p]),
    "bma_attn_bwd_scratch_bytes": (C.c_size_t, [C.POINTER(AttnArgs), C.POINTER(BlockLists), C.c_void_p]),
    "bma_attn_bwd_scratch_min_bytes": (C.c_size_t, [C.POINTER(AttnArgs), C.POINTER(BlockLists), C.c_void_p]),
    "bma_attn_bwd": (C.c_int, [C.POINTER(AttnArgs), C.POINTER(MaskSpec), C.POINTER(BlockLists), C.c_void_p, C.c_size_t,
                               C.c_void_p, C.c_void_p, C.c_void_p]),
    "bma_debug_expire_wait": (C.c_int, [C.c_uint64, C.c_int32, C.c_void_p]),
    "bma_attn_merge": (C.c_int, [C.POINTER(AttnArgs), C.c_void_p]),
    "bma_device_status": (C.c_int, [C.c_void_p, C.POINTER(C.c_int32)]),
}

_lib = None


class BmaError(RuntimeError):
    def __init__(self, status: int, where: str):
        self.status = status
        text = lib().bma_error_string(status).decode()
        super().__init__(f"{where}: status {status}: {text}")


def lib_path() -> Path:
    return Path(os.environ.get("BMA_LIBRARY", str(_LIB_PATH)))


def lib():
    """The loaded library; raises if it was not built (python -m jaxmodules_b200.build)."""
    global _lib
    if _lib is None:
        p = lib_path()
        if not p.exists():
            raise RuntimeError(
                f"{p} is missing: build the CUDA library with `python -m jaxmodules_b200.build` "
                "(there is no CPU or PyTorch fallback)")
        handle = C.CDLL(str(p))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(status: int, where: str):
    if status != BMA_OK:
        raise BmaError(status, where)
