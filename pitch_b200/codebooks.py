"""TurboQuant codebooks: float32 Lloyd-Max centroids per (dim, bits).

The values are data published with the reference (``reference/codebooks.json``,
mirrored in ``Sources/PITCH/TurboCodebooks.swift``); they are loaded, never
regenerated, because codes are only meaningful against the same table.
``turbo_codebook`` keeps the name and return type of the specification
(reference/pitch_reference.py:55-63).
"""
from __future__ import annotations

import json
import threading
from pathlib import Path

import numpy as np

_DATA = Path(__file__).resolve().parent / "data" / "codebooks_f32.npz"
_lock = threading.Lock()
_books: dict[tuple[int, int], np.ndarray] | None = None
_registered = False


def _load() -> dict[tuple[int, int], np.ndarray]:
    global _books
    with _lock:
        if _books is None:
            with np.load(_DATA) as z:
                _books = {tuple(int(t) for t in k.split("_")): np.ascontiguousarray(z[k], dtype=np.float32)
                          for k in z.files}
    return _books


def turbo_codebook(d: int, b: int) -> np.ndarray:
    """2^b ascending centroids for (d, b), float32 values widened to float64."""
    try:
        return _load()[(d, b)].astype(np.float64)
    except KeyError:
        raise KeyError(f"{d}_{b}") from None


def codebook_f32(d: int, b: int) -> np.ndarray:
    return _load()[(d, b)]


def load_codebooks_json(path) -> None:
    """Replaces the table with the contents of a ``codebooks.json`` in the reference's format
    ({"<dim>_<bits>": [centroids...]}) and re-registers it with the native library."""
    global _books, _registered
    table = json.loads(Path(path).read_text())
    books = {}
    for key, values in table.items():
        d, b = (int(t) for t in key.split("_"))
        c = np.asarray(values, dtype=np.float32)
        if c.shape != (1 << b,):
            raise ValueError(f"codebook {key}: expected {1 << b} centroids, found {c.size}")
        books[(d, b)] = np.ascontiguousarray(c)
    with _lock:
        _books = books
        _registered = False
    register_all()


def register_all() -> None:
    """Hands every codebook to the native library (host-side copy; idempotent)."""
    global _registered
    if _registered:
        return
    from . import _native
    import ctypes
    L = _native.lib()
    for (d, b), c in _load().items():
        _native.check(L.pitch_set_codebook(d, b, c.ctypes.data_as(ctypes.POINTER(ctypes.c_float))))
    _registered = True
