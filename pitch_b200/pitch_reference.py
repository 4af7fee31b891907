"""Drop-in for the reference's executable specification, backed by the CUDA kernels.

Same names, signatures, return shapes and dtypes as ``reference/pitch_reference.py``
(``import pitch_b200.pitch_reference as R`` in place of ``import pitch_reference as R``):
codes come back unpacked as int64 ``(n, d)`` arrays, scales as float64, per-channel
ranges as float16 ``(groups, 2, d)``.  Inputs are NumPy arrays (or anything
``np.asarray`` accepts); they are rounded to float32 before they reach the GPU,
which is what the reference's fixtures feed the specification.  The arithmetic
runs in float32 on the device (the specification uses float64 for the per-vector
methods): packed codes agree except at float32 boundary ties, decoded values to
about 1e-6 relative.

Only index bookkeeping (hash, signs, strides, bit accounting) is computed on the
host; everything that touches vector data calls the C ABI.
"""
from __future__ import annotations

import numpy as np

from . import _native
from .codebooks import turbo_codebook  # noqa: F401  (part of the specification's surface)
from .codec import PITCH, as_buffer, stream_handle
from .config import DEFAULT_SEED, ChannelQuantConfig, QuantConfig, QuantMethod, code_stride_bytes

SUPPORTED_BITS = range(2, 9)
SUPPORTED_DIMS = [2 ** k for k in range(1, 11)]
CHANNEL_DEFAULT_GROUP = 64
FP16_MAX = 65504.0


def _torch():
    import torch
    return torch


# ---------------------------------------------------------------------------- index helpers (host)
def pcg_hash(v):
    """reference/pitch_reference.py:11-15."""
    m = np.uint64(0xFFFFFFFF)
    v = np.asarray(v, dtype=np.uint64) & m
    s = (v * np.uint64(747796405) + np.uint64(2891336453)) & m
    w = (((s >> ((s >> np.uint64(28)) + np.uint64(4))) ^ s) * np.uint64(277803737)) & m
    return ((w >> np.uint64(22)) ^ w) & m


def rand_signs(seed: int, d: int) -> np.ndarray:
    """reference/pitch_reference.py:17-19."""
    h = pcg_hash((np.uint64(int(seed) & 0xFFFFFFFF) + np.arange(d, dtype=np.uint64)) & np.uint64(0xFFFFFFFF))
    return np.where(h & np.uint64(1), 1.0, -1.0)


def bits_per_coordinate(d: int, b: int) -> float:
    """reference/pitch_reference.py:134-135."""
    return (code_stride_bytes(d, b) + 4) * 8 / d


def channel_group_count(n: int, G: int) -> int:
    return (n + G - 1) // G


def channel_bits_per_coordinate(d: int, b: int, G: int = CHANNEL_DEFAULT_GROUP) -> float:
    """reference/pitch_reference.py:177-178."""
    return code_stride_bytes(d, b) * 8 / d + 32 / G


# ---------------------------------------------------------------------------- device helpers
def _to_device_f32(X):
    torch = _torch()
    p = PITCH.shared()
    x = np.ascontiguousarray(np.asarray(X), dtype=np.float32)
    if x.ndim != 2:
        raise ValueError("expected a 2-D array (n, d)")
    return p, torch.from_numpy(x).to(p.device), x.shape


def _rotation(mode: int, X, seed: int):
    torch = _torch()
    p, d_in, (n, d) = _to_device_f32(X)
    out = torch.empty_like(d_in)
    st = _native.lib().pitch_enqueue_rotate(mode, d, int(seed) & 0xFFFFFFFF, as_buffer(d_in, 0, "input"),
                                            as_buffer(out, 0, "output"), n, stream_handle(None, p.device))
    _native.check(st)
    return out.cpu().numpy().astype(np.float64)


def wht(x):
    """Unnormalised Walsh-Hadamard transform of each row (reference/pitch_reference.py:21-31)."""
    return _rotation(0, x, 0)


def rotate(X, seed):
    return _rotation(1, X, seed)


def unrotate(Y, seed):
    return _rotation(2, Y, seed)


def pack_codes(codes, b: int) -> bytes:
    """(n, d) integer codes -> packed bytes (reference/pitch_reference.py:68-79)."""
    torch = _torch()
    p = PITCH.shared()
    c = np.ascontiguousarray(np.asarray(codes), dtype=np.int32)
    n, d = c.shape
    d_c = torch.from_numpy(c).to(p.device)
    packed = torch.empty(n * code_stride_bytes(d, b), dtype=torch.uint8, device=p.device)
    p.enqueue_pack_codes(d_c, packed, n, d, b)
    return packed.cpu().numpy().tobytes()


def unpack_codes(buf, n: int, d: int, b: int) -> np.ndarray:
    """Packed bytes -> (n, d) int64 codes (reference/pitch_reference.py:81-90)."""
    torch = _torch()
    p = PITCH.shared()
    raw = np.frombuffer(bytes(buf), dtype=np.uint8, count=n * code_stride_bytes(d, b)).copy()
    packed = torch.from_numpy(raw).to(p.device)
    out = torch.empty((n, d), dtype=torch.int32, device=p.device)
    p.enqueue_unpack_codes(packed, out, n, d, b)
    return out.cpu().numpy().astype(np.int64)


def _device_unpack(p, packed, n, d, b):
    torch = _torch()
    out = torch.empty((n, d), dtype=torch.int32, device=p.device)
    p.enqueue_unpack_codes(packed, out, n, d, b)
    return out.cpu().numpy().astype(np.int64)


def _device_pack(p, codes, b):
    torch = _torch()
    c = np.ascontiguousarray(np.asarray(codes), dtype=np.int32)
    if c.ndim != 2:
        raise ValueError("expected a 2-D array of codes (n, d)")
    n, d = c.shape
    packed = torch.empty(n * code_stride_bytes(d, b), dtype=torch.uint8, device=p.device)
    p.enqueue_pack_codes(torch.from_numpy(c).to(p.device), packed, n, d, b)
    return packed, n, d


# ---------------------------------------------------------------------------- per-vector codecs
def _encode(method: QuantMethod, X, b: int, seed: int):
    torch = _torch()
    p, d_in, (n, d) = _to_device_f32(X)
    cfg = QuantConfig(method, d, b, int(seed) & 0xFFFFFFFF)
    codes = torch.empty(n * cfg.code_stride, dtype=torch.uint8, device=p.device)
    scales = torch.empty(n, dtype=torch.float32, device=p.device)
    p.enqueue_encode(d_in, codes, scales, n, cfg)
    return _device_unpack(p, codes, n, d, b), scales.cpu().numpy().astype(np.float64)


def _decode(method: QuantMethod, codes, scales, b: int, seed: int):
    torch = _torch()
    p = PITCH.shared()
    packed, n, d = _device_pack(p, codes, b)
    cfg = QuantConfig(method, d, b, int(seed) & 0xFFFFFFFF)
    s = torch.from_numpy(np.ascontiguousarray(np.asarray(scales), dtype=np.float32).reshape(-1)).to(p.device)
    if s.numel() != n:
        raise ValueError(f"expected {n} scales, found {s.numel()}")
    out = torch.empty((n, d), dtype=torch.float32, device=p.device)
    p.enqueue_decode(packed, s, out, n, cfg)
    return out.cpu().numpy().astype(np.float64)


def turbo_encode(X, b: int, seed: int = DEFAULT_SEED):
    """Returns (codes (n,d) int64, norms (n,) float64).  reference/pitch_reference.py:92-102."""
    return _encode(QuantMethod.turboQuant, X, b, seed)


def turbo_decode(codes, norms, b: int, seed: int = DEFAULT_SEED):
    """reference/pitch_reference.py:104-107."""
    return _decode(QuantMethod.turboQuant, codes, norms, b, seed)


def polar_encode(X, b: int, seed: int = DEFAULT_SEED):
    """Returns (codes, rmax).  reference/pitch_reference.py:109-121."""
    return _encode(QuantMethod.polarQuant, X, b, seed)


def polar_decode(codes, rmax, b: int, seed: int = DEFAULT_SEED):
    """reference/pitch_reference.py:123-129."""
    return _decode(QuantMethod.polarQuant, codes, rmax, b, seed)


ENCODERS = {"turboQuant": turbo_encode, "polarQuant": polar_encode}
DECODERS = {"turboQuant": turbo_decode, "polarQuant": polar_decode}


# ---------------------------------------------------------------------------- per-channel keys
def channel_encode(X, b: int, G: int = CHANNEL_DEFAULT_GROUP):
    """Returns (codes (n,d) int64, ranges float16 (groups, 2, d)).  reference/pitch_reference.py:145-162."""
    torch = _torch()
    x = np.asarray(X, dtype=np.float32)
    if not np.isfinite(x).all() or np.abs(x).max() > FP16_MAX:
        raise ValueError("inputs must be finite with magnitude at most 65504 (fp16 range)")
    p, d_in, (n, d) = _to_device_f32(x)
    cfg = ChannelQuantConfig(d, b, G)
    groups = cfg.group_count(n)
    codes = torch.empty(n * cfg.code_stride, dtype=torch.uint8, device=p.device)
    ranges = torch.empty((groups, 2, d), dtype=torch.float16, device=p.device)
    p.enqueue_per_channel_encode(d_in, codes, ranges, n, cfg)
    return _device_unpack(p, codes, n, d, b), ranges.cpu().numpy()


def channel_decode(codes, ranges, b: int, G: int = CHANNEL_DEFAULT_GROUP):
    """Returns float32 (n, d).  reference/pitch_reference.py:165-174."""
    torch = _torch()
    p = PITCH.shared()
    packed, n, d = _device_pack(p, codes, b)
    cfg = ChannelQuantConfig(d, b, G)
    r = np.ascontiguousarray(np.asarray(ranges), dtype=np.float16)
    d_r = torch.from_numpy(r).to(p.device)
    out = torch.empty((n, d), dtype=torch.float32, device=p.device)
    p.enqueue_per_channel_decode(packed, d_r, out, n, cfg)
    return out.cpu().numpy()
