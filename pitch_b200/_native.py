"""ctypes binding of ``libpitch_b200.so`` (declarations: ``include/pitch_b200.h``).

There is no CPU implementation behind this module: if the shared library is
missing the import of any compute entry point raises ``KernelUnavailable``.
Build it with ``python -m pitch_b200.build``.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, Structure, c_char_p, c_float, c_int, c_int32, c_int64, c_uint32, c_uint64, c_void_p
from pathlib import Path

from .errors import KernelUnavailable, from_status

LIB_PATH = Path(__file__).resolve().parent / "_lib" / "libpitch_b200.so"

ABI_VERSION = 2
TURBO_QUANT, POLAR_QUANT = 0, 1
F32, F16, BF16 = 0, 1, 2
PLANE_TURBO, PLANE_POLAR, PLANE_CHANNEL = 0, 1, 2


class Buffer(Structure):
    """``pitch_buffer``: device allocation + byte offset."""
    _fields_ = [("base", c_void_p), ("length", c_int64), ("offset", c_int64)]


class Plane(Structure):
    """``pitch_plane``."""
    _fields_ = [("kind", c_int32), ("bits", c_int32), ("group_size", c_int32), ("seed", c_uint32),
                ("codes", c_void_p), ("codes_seg_stride", c_int64),
                ("side", c_void_p), ("side_seg_stride", c_int64),
                ("out", c_void_p), ("out_seg_stride", c_int64),
                ("codes_bytes", c_int64), ("side_bytes", c_int64), ("out_bytes", c_int64)]


class AppendSrc(Structure):
    """``pitch_append_src``."""
    _fields_ = [("input", c_void_p), ("input_seg_stride", c_int64),
                ("residual", c_void_p), ("residual_seg_stride", c_int64),
                ("input_bytes", c_int64), ("residual_bytes", c_int64)]


class RopeBias(Structure):
    """``pitch_rope_bias``."""
    _fields_ = [("bias", c_void_p), ("bias_seg_stride", c_int64), ("cos_table", c_void_p), ("sin_table", c_void_p),
                ("positions", c_int64)]


class CacheDesc(Structure):
    """``pitch_cache_desc``."""
    _fields_ = [("dim", c_int32), ("out_dtype", c_int32), ("segments", c_int64), ("tokens", c_int64),
                ("n_planes", c_int32), ("reserved", c_int32), ("planes", Plane * 4),
                ("key_bias", POINTER(RopeBias)), ("capacity", c_int64)]


class CacheState(Structure):
    """``pitch_cache_state`` (lives in device memory; this mirror only gives its size and layout)."""
    _fields_ = [("tokens", c_int64), ("status", c_int32), ("arrivals", c_uint32)]


class AttentionArgs(Structure):
    """``pitch_attention_args``."""
    _fields_ = [("queries", c_void_p), ("out", c_void_p), ("workspace", c_void_p), ("workspace_bytes", c_int64),
                ("n_queries", c_int32), ("scale", c_float), ("precision", c_int32), ("reserved", c_int32)]


# name -> (restype, argtypes); every symbol include/pitch_b200.h declares
PROTOTYPES = {
    "pitch_abi_version": (c_int, []),
    "pitch_status_string": (c_char_p, [c_int]),
    "pitch_last_error": (c_char_p, []),
    "pitch_code_stride": (c_int, [c_int, c_int]),
    "pitch_set_codebook": (c_int, [c_int, c_int, POINTER(c_float)]),
    "pitch_has_codebook": (c_int, [c_int, c_int]),
    "pitch_enqueue_encode": (c_int, [c_int, c_int, c_int, c_uint32, c_int, Buffer, Buffer, Buffer, c_int64, c_void_p]),
    "pitch_enqueue_decode": (c_int, [c_int, c_int, c_int, c_uint32, c_int, Buffer, Buffer, Buffer, c_int64, c_void_p]),
    "pitch_enqueue_channel_encode": (c_int, [c_int, c_int, c_int, c_int, Buffer, Buffer, Buffer, c_int64, c_void_p]),
    "pitch_enqueue_channel_decode": (c_int, [c_int, c_int, c_int, c_int, Buffer, Buffer, Buffer, c_int64, c_void_p]),
    "pitch_enqueue_rotate": (c_int, [c_int, c_int, c_uint32, Buffer, Buffer, c_int64, c_void_p]),
    "pitch_enqueue_pack_codes": (c_int, [c_int, c_int, Buffer, Buffer, c_int64, c_void_p]),
    "pitch_enqueue_unpack_codes": (c_int, [c_int, c_int, Buffer, Buffer, c_int64, c_void_p]),
    "pitch_enqueue_cache_decode": (c_int, [POINTER(CacheDesc), c_void_p]),
    "pitch_enqueue_cache_append": (c_int, [POINTER(CacheDesc), POINTER(AppendSrc), c_int, c_int64, c_void_p]),
    "pitch_enqueue_cache_append_noalloc": (c_int, [POINTER(CacheDesc), POINTER(AppendSrc), c_int, c_int64, c_void_p]),
    "pitch_enqueue_cache_step": (c_int, [POINTER(CacheDesc), POINTER(AppendSrc), c_int, c_void_p, c_void_p]),
    "pitch_enqueue_cache_newest": (c_int, [POINTER(CacheDesc), c_void_p, c_void_p, c_int64, c_void_p]),
    "pitch_cache_attention_workspace": (c_int64, [POINTER(CacheDesc), c_int]),
    "pitch_enqueue_cache_attention": (c_int, [POINTER(CacheDesc), POINTER(AttentionArgs), c_void_p]),
    "pitch_enqueue_rope_bias": (c_int, [c_int, c_int, c_int, c_void_p, c_int64, c_int64, c_int64, c_int64,
                                        POINTER(RopeBias), c_void_p]),
    "pitch_enqueue_checksum": (c_int, [Buffer, c_int64, c_void_p, c_void_p]),
}

_lib = None


def lib():
    """The loaded library; raises ``KernelUnavailable`` when it has not been built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise KernelUnavailable(
                f"{LIB_PATH} is missing: build the CUDA extension with `python -m pitch_b200.build` "
                "(there is no CPU fallback)")
        try:
            L = ctypes.CDLL(str(LIB_PATH))
        except OSError as e:  # pragma: no cover - depends on the machine
            raise KernelUnavailable(f"cannot load {LIB_PATH}: {e}") from e
        for name, (res, args) in PROTOTYPES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        if L.pitch_abi_version() != ABI_VERSION:
            raise KernelUnavailable(f"{LIB_PATH} has ABI version {L.pitch_abi_version()}, this package needs {ABI_VERSION}: "
                                    "rebuild it with `python -m pitch_b200.build --force`")
        _lib = L
    return _lib


def check(status: int) -> None:
    """Raises the exception that corresponds to a non-zero ``pitch_status``."""
    if status != 0:
        detail = lib().pitch_last_error().decode(errors="replace")
        raise from_status(status, detail)
