"""ctypes wrapper of ``oracle/kernel_f32.c`` (CPU oracle #2, float32 arithmetic).

TEST INFRASTRUCTURE ONLY.  Functions take and return NumPy arrays; packed
codes are uint8 arrays of ``count * stride`` bytes, like the GPU buffers.
"""
from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import numpy as np

from . import spec_np

_HERE = Path(__file__).resolve().parent
_SO = _HERE / "_build" / "libpitch_oracle.so"
_lib = None

_f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
_u8p = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")
_u16p = np.ctypeslib.ndpointer(np.uint16, flags="C_CONTIGUOUS")
_i64, _int, _u32 = ctypes.c_int64, ctypes.c_int, ctypes.c_uint32


def build(force: bool = False) -> Path:
    """Compiles the C oracle with the Makefile beside it (gcc, a second or two)."""
    src = _HERE / "kernel_f32.c"
    if force or not _SO.exists() or _SO.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(_HERE), "-B" if force else "-s"], check=True,
                       stdout=subprocess.DEVNULL)
    return _SO


def lib():
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(str(_SO))
        L.pitch_oracle_edges.argtypes = [_f32p, _int, _f32p]
        L.pitch_oracle_turbo_encode.argtypes = [_f32p, _i64, _int, _int, _u32, _f32p, _u8p, _f32p]
        L.pitch_oracle_turbo_decode.argtypes = [_u8p, _f32p, _i64, _int, _int, _u32, _f32p, _f32p]
        L.pitch_oracle_polar_encode.argtypes = [_f32p, _i64, _int, _int, _u32, _u8p, _f32p]
        L.pitch_oracle_polar_encode_metal.argtypes = [_f32p, _i64, _int, _int, _u32, _u8p, _f32p]
        L.pitch_oracle_polar_decode.argtypes = [_u8p, _f32p, _i64, _int, _int, _u32, _f32p]
        L.pitch_oracle_channel_encode.argtypes = [_f32p, _i64, _int, _int, _int, _u8p, _u16p]
        L.pitch_oracle_channel_decode.argtypes = [_u8p, _u16p, _i64, _int, _int, _int, _f32p]
        L.pitch_oracle_f32_to_f16.argtypes = [ctypes.c_float]
        L.pitch_oracle_f32_to_f16.restype = ctypes.c_uint16
        L.pitch_oracle_f16_to_f32.argtypes = [ctypes.c_uint16]
        L.pitch_oracle_f16_to_f32.restype = ctypes.c_float
        _lib = L
    return _lib


def _book(d, b):
    return np.ascontiguousarray(spec_np.turbo_codebook(d, b).astype(np.float32))


def encode(method: str, X, bits: int, seed: int = spec_np.DEFAULT_SEED, metal_literal: bool = False):
    """Returns (packed codes uint8 (n*stride,), scales float32 (n,)).  ``metal_literal`` selects, for
    PolarQuant, the variant that follows the Metal kernel's divisions per pair to the letter."""
    X = np.ascontiguousarray(X, dtype=np.float32)
    n, d = X.shape
    codes = np.zeros(n * spec_np.code_stride_bytes(d, bits), dtype=np.uint8)
    scales = np.zeros(n, dtype=np.float32)
    if method == "turboQuant":
        lib().pitch_oracle_turbo_encode(X, n, d, bits, seed & 0xFFFFFFFF, _book(d, bits), codes, scales)
    elif metal_literal:
        lib().pitch_oracle_polar_encode_metal(X, n, d, bits, seed & 0xFFFFFFFF, codes, scales)
    else:
        lib().pitch_oracle_polar_encode(X, n, d, bits, seed & 0xFFFFFFFF, codes, scales)
    return codes, scales


def decode(method: str, codes, scales, d: int, bits: int, seed: int = spec_np.DEFAULT_SEED):
    """Packed codes + float32 scales -> float32 (n, d)."""
    codes = np.ascontiguousarray(codes, dtype=np.uint8)
    scales = np.ascontiguousarray(scales, dtype=np.float32)
    n = scales.shape[0]
    out = np.zeros((n, d), dtype=np.float32)
    if method == "turboQuant":
        lib().pitch_oracle_turbo_decode(codes, scales, n, d, bits, seed & 0xFFFFFFFF, _book(d, bits), out)
    else:
        lib().pitch_oracle_polar_decode(codes, scales, n, d, bits, seed & 0xFFFFFFFF, out)
    return out


def channel_encode(X, bits: int, G: int = 64):
    """Returns (packed codes uint8, ranges uint16 (groups, 2, d) = fp16 bit patterns)."""
    X = np.ascontiguousarray(X, dtype=np.float32)
    n, d = X.shape
    groups = -(-n // G)
    codes = np.zeros(n * spec_np.code_stride_bytes(d, bits), dtype=np.uint8)
    ranges = np.zeros((groups, 2, d), dtype=np.uint16)
    lib().pitch_oracle_channel_encode(X, n, d, bits, G, codes, ranges)
    return codes, ranges


def channel_decode(codes, ranges, n: int, d: int, bits: int, G: int = 64):
    codes = np.ascontiguousarray(codes, dtype=np.uint8)
    ranges = np.ascontiguousarray(ranges, dtype=np.uint16)
    out = np.zeros((n, d), dtype=np.float32)
    lib().pitch_oracle_channel_decode(codes, ranges, n, d, bits, G, out)
    return out
