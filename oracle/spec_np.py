"""CPU oracle #1: a NumPy restatement of PITCH's executable specification.

TEST INFRASTRUCTURE ONLY.  Nothing in the product package may import this
module; it is the checker the CUDA kernels are compared against (tests, the
smoke check and the CPU-baseline leg of the benchmark).

Every function restates one function of the reference's
``reference/pitch_reference.py`` (cited per function as file:line) in
independent code.  Arithmetic precision follows the specification exactly:
rotation, norms and polar maths in float64 on float32-valued inputs, the
per-channel codec entirely in float32.

Parity status: PINNED.  ``tests/test_oracle_golden.py`` replays all 40
per-vector and all 17 per-channel golden cases of the reference's own test
fixtures (``Tests/PITCHTests/Fixtures/parity.json`` and
``channel_parity.json``, repackaged as ``tests/golden/*.npz``) and requires
byte-identical codes, scales/ranges and reconstructions.
"""
from __future__ import annotations

import json
import math
from pathlib import Path

import numpy as np

DEFAULT_SEED = 0x50495443            # reference/pitch_reference.py:7
SUPPORTED_BITS = tuple(range(2, 9))  # reference/pitch_reference.py:8
SUPPORTED_DIMS = tuple(1 << k for k in range(1, 11))  # reference/pitch_reference.py:9
CHANNEL_DEFAULT_GROUP = 64           # reference/pitch_reference.py:137
FP16_MAX = 65504.0                   # reference/pitch_reference.py:138

_M32 = np.uint64(0xFFFFFFFF)

_DATA = Path(__file__).resolve().parent.parent / "pitch_b200" / "data" / "codebooks_f32.npz"
_books: dict[str, np.ndarray] | None = None


# --------------------------------------------------------------------------- rotation
def pcg_hash(v):
    """32-bit PCG-style output hash (reference/pitch_reference.py:11-15)."""
    v = np.asarray(v, dtype=np.uint64) & _M32
    s = (v * np.uint64(747796405) + np.uint64(2891336453)) & _M32
    rot = (s >> np.uint64(28)) + np.uint64(4)
    w = (((s >> rot) ^ s) * np.uint64(277803737)) & _M32
    return ((w >> np.uint64(22)) ^ w) & _M32


def rand_signs(seed: int, d: int) -> np.ndarray:
    """Diagonal of +-1: +1 where the hash of (seed+i) mod 2^32 is odd
    (reference/pitch_reference.py:17-19)."""
    idx = (np.arange(d, dtype=np.uint64) + np.uint64(seed & 0xFFFFFFFF)) & _M32
    odd = (pcg_hash(idx) & np.uint64(1)).astype(bool)
    out = np.full(d, -1.0)
    out[odd] = 1.0
    return out


def wht(x: np.ndarray) -> np.ndarray:
    """Unnormalised Walsh-Hadamard transform along the last axis, stages
    h = 1, 2, 4, ... (reference/pitch_reference.py:21-31).  float64."""
    y = np.array(x, dtype=np.float64)
    n, d = y.shape
    h = 1
    while h < d:
        v = y.reshape(n, d // (2 * h), 2, h)
        top = v[:, :, 0, :] + v[:, :, 1, :]
        bot = v[:, :, 0, :] - v[:, :, 1, :]
        y = np.stack((top, bot), axis=2).reshape(n, d)
        h *= 2
    return y


def rotate(X, seed):
    """wht(X * signs) / sqrt(d)  (reference/pitch_reference.py:33)."""
    d = X.shape[1]
    return wht(X * rand_signs(seed, d)) / math.sqrt(d)


def unrotate(Y, seed):
    """wht(Y) * signs / sqrt(d)  (reference/pitch_reference.py:34)."""
    d = Y.shape[1]
    return wht(Y) * rand_signs(seed, d) / math.sqrt(d)


# --------------------------------------------------------------------------- codebooks
def turbo_codebook(d: int, b: int) -> np.ndarray:
    """float32 Lloyd-Max centroids for key "{d}_{b}", widened to float64
    (reference/pitch_reference.py:55-63).  The table is the reference's
    ``reference/codebooks.json`` stored as float32 arrays."""
    global _books
    if _books is None:
        with np.load(_DATA) as z:
            _books = {k: z[k].astype(np.float32) for k in z.files}
    return _books[f"{d}_{b}"].astype(np.float64)


def turbo_edges(d: int, b: int) -> np.ndarray:
    """Decision boundaries: float32 midpoints 0.5f*(c[i]+c[i+1]), widened
    (reference/pitch_reference.py:99-100)."""
    c = turbo_codebook(d, b).astype(np.float32)
    return (np.float32(0.5) * (c[1:] + c[:-1])).astype(np.float64)


# --------------------------------------------------------------------------- packing
def code_stride_bytes(d: int, b: int) -> int:
    """Bytes of packed codes per vector, rounded up to whole 32-bit words
    (reference/pitch_reference.py:65-66)."""
    return 4 * ((d * b + 31) // 32)


def pack_codes(codes: np.ndarray, b: int) -> bytes:
    """LSB-first b-bit stream per vector in little-endian 32-bit words; code i
    occupies bits [i*b, i*b+b) (reference/pitch_reference.py:68-79)."""
    codes = np.asarray(codes)
    n, d = codes.shape
    nbits = code_stride_bytes(d, b) * 8
    bits = np.zeros((n, nbits), dtype=np.uint8)
    c = codes.astype(np.uint64)
    for k in range(b):
        bits[:, k:d * b:b] = ((c >> np.uint64(k)) & np.uint64(1)).astype(np.uint8)
    return np.packbits(bits, axis=1, bitorder="little").tobytes()


def unpack_codes(buf: bytes, n: int, d: int, b: int) -> np.ndarray:
    """Inverse of pack_codes (reference/pitch_reference.py:81-90)."""
    stride = code_stride_bytes(d, b)
    raw = np.frombuffer(buf, dtype=np.uint8, count=n * stride).reshape(n, stride)
    bits = np.unpackbits(raw, axis=1, bitorder="little")
    codes = np.zeros((n, d), dtype=np.int64)
    for k in range(b):
        codes |= bits[:, k:d * b:b].astype(np.int64) << k
    return codes


# --------------------------------------------------------------------------- TurboQuant
def turbo_encode(X, b: int, seed: int = DEFAULT_SEED):
    """norm, unit vector, rotate, count of edges strictly below each coordinate
    (reference/pitch_reference.py:92-102).  Returns (codes (n,d) int64, norms (n,) f64)."""
    X = np.asarray(X, dtype=np.float64)
    d = X.shape[1]
    norms = np.linalg.norm(X, axis=1)
    div = norms.copy()
    div[div <= 0] = 1.0
    U = rotate(X / div[:, None], seed)
    codes = np.searchsorted(turbo_edges(d, b), U, side="left")
    return codes.astype(np.int64), norms


def turbo_decode(codes, norms, b: int, seed: int = DEFAULT_SEED):
    """centroid lookup, inverse rotation, times norm
    (reference/pitch_reference.py:104-107)."""
    codes = np.asarray(codes)
    d = codes.shape[1]
    Y = turbo_codebook(d, b)[codes]
    return unrotate(Y, seed) * np.asarray(norms, dtype=np.float64)[:, None]


# --------------------------------------------------------------------------- PolarQuant variant
def polar_encode(X, b: int, seed: int = DEFAULT_SEED):
    """rotate (no normalisation); pairs -> (r, theta); radius on 2^b-1 steps of
    [0, rmax], angle on 2^b circular bins (reference/pitch_reference.py:109-121)."""
    Y = rotate(np.asarray(X, dtype=np.float64), seed)
    re, im = Y[:, 0::2], Y[:, 1::2]
    r = np.hypot(re, im)
    theta = np.mod(np.arctan2(im, re), 2 * np.pi)
    levels = 2 ** b - 1
    bins = 2 ** b
    rmax = r.max(axis=1)
    div = np.where(rmax > 0, rmax, 1.0)[:, None]
    rq = np.clip(np.floor(r / div * levels + 0.5), 0, levels)
    tq = np.mod(np.floor(theta / (2 * np.pi) * bins + 0.5), bins)
    codes = np.empty(Y.shape, dtype=np.int64)
    codes[:, 0::2] = rq
    codes[:, 1::2] = tq
    return codes, rmax


def polar_decode(codes, rmax, b: int, seed: int = DEFAULT_SEED):
    """(reference/pitch_reference.py:123-129)."""
    codes = np.asarray(codes)
    levels = 2 ** b - 1
    bins = 2 ** b
    r = codes[:, 0::2] / levels * np.asarray(rmax, dtype=np.float64)[:, None]
    theta = codes[:, 1::2] / bins * 2 * np.pi
    Y = np.empty(codes.shape, dtype=np.float64)
    Y[:, 0::2] = r * np.cos(theta)
    Y[:, 1::2] = r * np.sin(theta)
    return unrotate(Y, seed)


ENCODERS = {"turboQuant": turbo_encode, "polarQuant": polar_encode}   # reference/pitch_reference.py:131
DECODERS = {"turboQuant": turbo_decode, "polarQuant": polar_decode}   # reference/pitch_reference.py:132


def bits_per_coordinate(d: int, b: int) -> float:
    """(reference/pitch_reference.py:134-135)."""
    return (code_stride_bytes(d, b) + 4) * 8 / d


# --------------------------------------------------------------------------- per-channel keys
def channel_group_count(n: int, G: int) -> int:
    """(reference/pitch_reference.py:141-142)."""
    return -(-n // G)


def channel_encode(X, b: int, G: int = CHANNEL_DEFAULT_GROUP):
    """Per group of G tokens and per channel: fp16-rounded min/max, float32
    step, float32 round-half-up quantisation (reference/pitch_reference.py:145-162)."""
    X = np.asarray(X, dtype=np.float32)
    n, d = X.shape
    if not np.isfinite(X).all() or np.abs(X).max() > FP16_MAX:
        raise ValueError("inputs must be finite with magnitude at most 65504 (fp16 range)")
    top = np.float32(2 ** b - 1)
    groups = channel_group_count(n, G)
    codes = np.empty((n, d), dtype=np.int64)
    ranges = np.empty((groups, 2, d), dtype=np.float16)
    for g in range(groups):
        blk = X[g * G:(g + 1) * G]
        lo16 = blk.min(axis=0).astype(np.float16)
        hi16 = blk.max(axis=0).astype(np.float16)
        lo = lo16.astype(np.float32)
        step = (hi16.astype(np.float32) - lo) / top
        step = np.where(step == 0, np.float32(1), step).astype(np.float32)
        q = np.floor((blk - lo) / step + np.float32(0.5))
        codes[g * G:(g + 1) * G] = np.clip(q, 0, top).astype(np.int64)
        ranges[g, 0] = lo16
        ranges[g, 1] = hi16
    return codes, ranges


def channel_decode(codes, ranges, b: int, G: int = CHANNEL_DEFAULT_GROUP):
    """code * step + lo in float32, two roundings (reference/pitch_reference.py:165-174)."""
    codes = np.asarray(codes)
    n, d = codes.shape
    top = np.float32(2 ** b - 1)
    out = np.empty((n, d), dtype=np.float32)
    for g in range(channel_group_count(n, G)):
        lo = ranges[g, 0].astype(np.float32)
        step = (ranges[g, 1].astype(np.float32) - lo) / top
        step = np.where(step == 0, np.float32(1), step).astype(np.float32)
        out[g * G:(g + 1) * G] = codes[g * G:(g + 1) * G].astype(np.float32) * step + lo
    return out


def rotated_bias(bias, cos_table, sin_table):
    """R_t b for every position t of the rotary tables: ``b * cos + rotate_half(b) * sin`` with
    ``rotate_half(b) = (-b[d/2:], b[:d/2])`` (reference/mechanism_eval.py:82-91, ``rotated_bias``),
    in float32 with one rounding per operation.  bias (d,), tables (T, d) -> (T, d) float32."""
    b = np.asarray(bias, dtype=np.float32)
    d = b.shape[0]
    rh = np.concatenate([-b[d // 2:], b[:d // 2]]).astype(np.float32)
    c = np.asarray(cos_table, dtype=np.float32)
    s = np.asarray(sin_table, dtype=np.float32)
    return (b[None, :] * c).astype(np.float32) + (rh[None, :] * s).astype(np.float32)


def channel_bits_per_coordinate(d: int, b: int, G: int = CHANNEL_DEFAULT_GROUP) -> float:
    """(reference/pitch_reference.py:177-178)."""
    return code_stride_bytes(d, b) * 8 / d + 32 / G
