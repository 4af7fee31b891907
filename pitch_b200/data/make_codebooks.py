#!/usr/bin/env python3
"""Repackages PITCH's TurboQuant codebook table as float32 arrays.

The table is input data of the codec, not code: 70 Lloyd-Max codebooks keyed
"{dim}_{bits}" (dim a power of two 2...1024, bits 2...8), each 2^bits float32
centroids, ascending and antisymmetric.  They are published with the reference
as ``reference/codebooks.json`` (produced by ``reference/gen_fixtures.py:24-33``
from ``reference/pitch_reference.py:36-53``).  The kernels must use exactly
these values, so they are loaded, never regenerated.

    python pitch_b200/data/make_codebooks.py /path/to/reference/codebooks.json

writes ``codebooks_f32.npz`` next to this script.  ``pitch_b200.codebooks``
also reads a codebooks.json directly (``load_codebooks_json``).
"""
import json
import sys
from pathlib import Path

import numpy as np


def main(src: str) -> None:
    table = json.loads(Path(src).read_text())
    out = {}
    for key, values in table.items():
        d, b = (int(t) for t in key.split("_"))
        c = np.asarray(values, dtype=np.float32)
        assert c.shape == (1 << b,), key
        assert np.all(np.diff(c) > 0), f"{key}: not ascending"
        assert np.array_equal(c, -c[::-1]), f"{key}: not antisymmetric"
        assert [float(v) for v in c] == values, f"{key}: not float32-exact"
        out[key] = c
    dst = Path(__file__).resolve().parent / "codebooks_f32.npz"
    np.savez_compressed(dst, **out)
    print(f"wrote {len(out)} codebooks to {dst} ({dst.stat().st_size} bytes)")


if __name__ == "__main__":
    main(sys.argv[1])
