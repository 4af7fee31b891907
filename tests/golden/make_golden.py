#!/usr/bin/env python3
"""Builds the golden vectors under tests/golden/ from the reference itself.

Run in a container that has the reference checkout (it cannot travel to the
GPU machines; the .npz files this writes can):

    python tests/golden/make_golden.py /path/to/PITCH

What it does
 1. imports the reference's executable specification
    (``reference/pitch_reference.py``) unchanged;
 2. reads the reference's own golden fixtures
    (``Tests/PITCHTests/Fixtures/parity.json`` - 40 per-vector cases, and
    ``channel_parity.json`` - 17 per-channel cases), replays the pipeline of
    ``reference/gen_fixtures.py:63-141`` with the imported specification and
    REQUIRES byte-identical codes, scales / ranges and reconstructions;
 3. stores those fixtures as arrays (``parity.npz``, ``channel_parity.npz``);
 4. runs the imported specification on further seeded inputs that the
    fixtures do not cover (every dim x bits x method, bits 5-7, odd channel
    dims and group sizes, the benchmark configurations at reduced size) and
    stores inputs and outputs (``spec_extra.npz``).

Key layout: ``<case>/<field>`` inside each npz; ``__cases__`` is a JSON list
describing every case.
"""
import base64
import json
import sys
from pathlib import Path

import numpy as np

sys.dont_write_bytecode = True
HERE = Path(__file__).resolve().parent


def b64(s, dtype):
    return np.frombuffer(base64.b64decode(s), dtype=dtype).copy()


def save(name, arrays, cases):
    arrays["__cases__"] = np.frombuffer(json.dumps(cases).encode(), dtype=np.uint8)
    path = HERE / name
    np.savez_compressed(path, **arrays)
    print(f"wrote {len(cases)} cases to {path} ({path.stat().st_size} bytes)")


def main(root: str) -> None:
    root = Path(root)
    sys.path.insert(0, str(root / "reference"))
    import pitch_reference as R  # the reference, unchanged

    # ------------------------------------------------------------------ per-vector fixtures
    fx = json.loads((root / "Tests/PITCHTests/Fixtures/parity.json").read_text())
    arrays, cases = {}, []
    groups = {}
    for g in fx["groups"]:
        X = b64(g["input"], "<f4").reshape(g["count"], g["dim"])
        groups[g["name"]] = X
        arrays[f"input/{g['name']}"] = X
    for i, c in enumerate(fx["cases"]):
        X32 = groups[c["group"]]
        n, d = X32.shape
        codes_ref = b64(c["codes"], np.uint8)
        scales_ref = b64(c["scales"], "<f4")
        recon_ref = b64(c["reconstruction"], "<f4").reshape(n, d)
        # replay gen_fixtures.py:76-94 with the imported specification
        codes, scales = R.ENCODERS[c["method"]](X32.astype(np.float64), c["bits"], c["seed"])
        scales32 = np.asarray(scales, dtype=np.float32)
        recon = R.DECODERS[c["method"]](codes, scales32.astype(np.float64), c["bits"], c["seed"])
        assert R.pack_codes(codes, c["bits"]) == codes_ref.tobytes(), ("codes", i)
        assert scales32.tobytes() == scales_ref.tobytes(), ("scales", i)
        assert np.asarray(recon, dtype="<f4").tobytes() == recon_ref.tobytes(), ("recon", i)
        key = f"case{i:02d}"
        arrays[f"{key}/codes"] = codes_ref
        arrays[f"{key}/scales"] = scales_ref
        arrays[f"{key}/reconstruction"] = recon_ref
        cases.append(dict(key=key, group=c["group"], method=c["method"], bits=c["bits"],
                          seed=c["seed"], relative_error=c["relative_error"]))
    assert len(cases) == 40
    save("parity.npz", arrays, cases)

    # ------------------------------------------------------------------ per-channel fixtures
    fx = json.loads((root / "Tests/PITCHTests/Fixtures/channel_parity.json").read_text())
    arrays, cases = {}, []
    groups = {}
    for g in fx["groups"]:
        X = b64(g["input"], "<f4").reshape(g["count"], g["dim"])
        groups[g["name"]] = X
        arrays[f"input/{g['name']}"] = X
    for i, c in enumerate(fx["cases"]):
        X = groups[c["group"]]
        n, d = X.shape
        G = c["group_size"]
        codes_ref = b64(c["codes"], np.uint8)
        ranges_ref = b64(c["ranges"], "<u2").reshape(-1, 2, d)
        recon_ref = b64(c["reconstruction"], "<f4").reshape(n, d)
        codes, ranges = R.channel_encode(X, c["bits"], G)
        recon = R.channel_decode(codes, ranges, c["bits"], G)
        assert R.pack_codes(codes, c["bits"]) == codes_ref.tobytes(), ("codes", i)
        assert ranges.view("<u2").tobytes() == ranges_ref.tobytes(), ("ranges", i)
        assert np.asarray(recon, dtype="<f4").tobytes() == recon_ref.tobytes(), ("recon", i)
        key = f"case{i:02d}"
        arrays[f"{key}/codes"] = codes_ref
        arrays[f"{key}/ranges"] = ranges_ref
        arrays[f"{key}/reconstruction"] = recon_ref
        cases.append(dict(key=key, group=c["group"], bits=c["bits"], group_size=G, mse=c["mse"]))
    assert len(cases) == 17
    save("channel_parity.npz", arrays, cases)

    # ------------------------------------------------------------------ further cases from the spec
    arrays, cases = {}, []
    rng = np.random.default_rng(20261125)

    def lognormal_vectors(n, d):
        g = rng.standard_normal((n, d))
        s = rng.lognormal(0.0, 0.5, size=(n, 1))
        return (g * s).astype(np.float32)

    # every supported (dim, bits) for both per-vector methods
    for d in R.SUPPORTED_DIMS:
        X32 = lognormal_vectors(4, d)
        X32[3] = 0.0                                   # a zero vector in every group
        arrays[f"input/sweep{d}"] = X32
        for method in ("turboQuant", "polarQuant"):
            for bits in R.SUPPORTED_BITS:
                seed = R.DEFAULT_SEED if bits % 2 == 0 else (0x9E3779B9 + d * 131 + bits)
                codes, scales = R.ENCODERS[method](X32.astype(np.float64), bits, seed)
                scales32 = np.asarray(scales, dtype=np.float32)
                recon = R.DECODERS[method](codes, scales32.astype(np.float64), bits, seed)
                key = f"sweep/{method}/{d}_{bits}"
                arrays[f"{key}/codes"] = np.frombuffer(R.pack_codes(codes, bits), dtype=np.uint8)
                arrays[f"{key}/scales"] = scales32
                arrays[f"{key}/reconstruction"] = np.asarray(recon, dtype=np.float32)
                cases.append(dict(key=key, kind="vector", group=f"sweep{d}", method=method,
                                  bits=bits, seed=int(seed)))

    # benchmark configurations at reduced size (config 1: d=64 b=4; config 3: d=128 b=3/4; config 5: d=128)
    for name, n, d in (("cfg1", 192, 64), ("cfg3", 96, 128)):
        X32 = lognormal_vectors(n, d)
        arrays[f"input/{name}"] = X32
        for method in ("turboQuant", "polarQuant"):
            for bits in (3, 4):
                codes, scales = R.ENCODERS[method](X32.astype(np.float64), bits, R.DEFAULT_SEED)
                scales32 = np.asarray(scales, dtype=np.float32)
                recon = R.DECODERS[method](codes, scales32.astype(np.float64), bits, R.DEFAULT_SEED)
                key = f"{name}/{method}/{bits}"
                arrays[f"{key}/codes"] = np.frombuffer(R.pack_codes(codes, bits), dtype=np.uint8)
                arrays[f"{key}/scales"] = scales32
                arrays[f"{key}/reconstruction"] = np.asarray(recon, dtype=np.float32)
                cases.append(dict(key=key, kind="vector", group=name, method=method,
                                  bits=bits, seed=int(R.DEFAULT_SEED)))

    # per-channel: odd dims, group sizes, partial groups, biased keys with outlier channels (config 2 shape)
    def biased_keys(n, d):
        X = rng.standard_normal((n, d)) + rng.normal(0.0, 2.0, size=(1, d))
        out = rng.choice(d, size=min(4, d), replace=False)
        X[:, out] *= 20.0
        return X.astype(np.float32)

    chan = [("ch1", 70, 1, 64), ("ch7", 33, 7, 8), ("ch64", 130, 64, 64), ("ch64g1", 5, 64, 1),
            ("ch100", 70, 100, 32), ("ch1024", 20, 1024, 16), ("ch128", 96, 128, 64)]
    for name, n, d, G in chan:
        X = biased_keys(n, d)
        if d >= 2:
            X[:, 1] = 1.5                              # a constant channel (step -> 1)
        arrays[f"input/{name}"] = X
        for bits in R.SUPPORTED_BITS:
            codes, ranges = R.channel_encode(X, bits, G)
            recon = R.channel_decode(codes, ranges, bits, G)
            key = f"{name}/{bits}"
            arrays[f"{key}/codes"] = np.frombuffer(R.pack_codes(codes, bits), dtype=np.uint8)
            arrays[f"{key}/ranges"] = ranges.view(np.uint16)
            arrays[f"{key}/reconstruction"] = recon
            cases.append(dict(key=key, kind="channel", group=name, bits=bits, group_size=G))

    # helper functions of the spec: hash, signs, strides
    arrays["helpers/pcg_hash_in"] = np.array([0, 1, 2, 0x50495443, 0xFFFFFFFF, 12345], dtype=np.uint64)
    arrays["helpers/pcg_hash_out"] = np.asarray(R.pcg_hash(arrays["helpers/pcg_hash_in"]), dtype=np.uint64)
    arrays["helpers/signs_default_1024"] = R.rand_signs(R.DEFAULT_SEED, 1024).astype(np.int8)
    arrays["helpers/signs_12345_16"] = R.rand_signs(12345, 16).astype(np.int8)
    arrays["helpers/signs_wrap_64"] = R.rand_signs(0xFFFFFFF0, 64).astype(np.int8)
    arrays["helpers/stride"] = np.array([[d, b, R.code_stride_bytes(d, b)]
                                         for d in (1, 2, 7, 64, 96, 100, 128, 1024) for b in R.SUPPORTED_BITS])
    save("spec_extra.npz", arrays, cases)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <path to the reference checkout>")
    main(sys.argv[1])
