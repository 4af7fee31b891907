"""Pins both CPU oracles against the reference's golden vectors (no GPU).

Oracle #1 (NumPy, float64 spec) must reproduce every golden case byte for byte.
Oracle #2 (C, float32 kernel arithmetic) must meet the tolerances the
reference's own parity tests apply to its float32 kernels
(Tests/PITCHTests/ParityTests.swift:67-81, PerChannelTests.swift:82-97).
"""
import numpy as np
import pytest

from conftest import max_rel_l2
from oracle import kernel_f32, spec_np


def _unpack(buf, n, d, b):
    return spec_np.unpack_codes(bytes(buf), n, d, b)


# ---------------------------------------------------------------- oracle #1, reference fixtures
def test_fixture_inventory(golden_parity, golden_channel):
    assert len(golden_parity.cases) == 40                      # ParityTests.swift:43
    assert {c["method"] for c in golden_parity.cases} == {"turboQuant", "polarQuant"}
    assert len(golden_channel.cases) == 17                     # PerChannelTests.swift:62
    assert {c["group_size"] for c in golden_channel.cases} == {16, 64}


def test_spec_port_reproduces_per_vector_fixtures(golden_parity):
    for c in golden_parity.cases:
        X32 = golden_parity[f"input/{c['group']}"]
        codes, scales = spec_np.ENCODERS[c["method"]](X32.astype(np.float64), c["bits"], c["seed"])
        scales32 = np.asarray(scales, dtype=np.float32)
        recon = spec_np.DECODERS[c["method"]](codes, scales32.astype(np.float64), c["bits"], c["seed"])
        k = c["key"]
        assert spec_np.pack_codes(codes, c["bits"]) == golden_parity[f"{k}/codes"].tobytes(), k
        assert scales32.tobytes() == golden_parity[f"{k}/scales"].tobytes(), k
        assert recon.astype(np.float32).tobytes() == golden_parity[f"{k}/reconstruction"].tobytes(), k
        rel = float((((X32 - recon) ** 2).sum(1) / (X32.astype(np.float64) ** 2).sum(1)).mean())
        assert rel == pytest.approx(c["relative_error"], rel=1e-12)


def test_spec_port_reproduces_per_channel_fixtures(golden_channel):
    for c in golden_channel.cases:
        X = golden_channel[f"input/{c['group']}"]
        codes, ranges = spec_np.channel_encode(X, c["bits"], c["group_size"])
        recon = spec_np.channel_decode(codes, ranges, c["bits"], c["group_size"])
        k = c["key"]
        assert spec_np.pack_codes(codes, c["bits"]) == golden_channel[f"{k}/codes"].tobytes(), k
        assert ranges.view(np.uint16).tobytes() == golden_channel[f"{k}/ranges"].tobytes(), k
        assert recon.tobytes() == golden_channel[f"{k}/reconstruction"].tobytes(), k


def test_spec_port_reproduces_extra_cases(golden_extra):
    for c in golden_extra.cases:
        X = golden_extra[f"input/{c['group']}"]
        k = c["key"]
        if c["kind"] == "vector":
            codes, scales = spec_np.ENCODERS[c["method"]](X.astype(np.float64), c["bits"], c["seed"])
            scales32 = np.asarray(scales, dtype=np.float32)
            recon = spec_np.DECODERS[c["method"]](codes, scales32.astype(np.float64), c["bits"], c["seed"])
            assert spec_np.pack_codes(codes, c["bits"]) == golden_extra[f"{k}/codes"].tobytes(), k
            assert scales32.tobytes() == golden_extra[f"{k}/scales"].tobytes(), k
            assert recon.astype(np.float32).tobytes() == golden_extra[f"{k}/reconstruction"].tobytes(), k
        else:
            codes, ranges = spec_np.channel_encode(X, c["bits"], c["group_size"])
            recon = spec_np.channel_decode(codes, ranges, c["bits"], c["group_size"])
            assert spec_np.pack_codes(codes, c["bits"]) == golden_extra[f"{k}/codes"].tobytes(), k
            assert ranges.view(np.uint16).tobytes() == golden_extra[f"{k}/ranges"].tobytes(), k
            assert recon.tobytes() == golden_extra[f"{k}/reconstruction"].tobytes(), k


def test_spec_port_helpers(golden_extra):
    assert np.array_equal(spec_np.pcg_hash(golden_extra["helpers/pcg_hash_in"]),
                          golden_extra["helpers/pcg_hash_out"])
    assert np.array_equal(spec_np.rand_signs(spec_np.DEFAULT_SEED, 1024),
                          golden_extra["helpers/signs_default_1024"])
    assert np.array_equal(spec_np.rand_signs(12345, 16), golden_extra["helpers/signs_12345_16"])
    assert np.array_equal(spec_np.rand_signs(0xFFFFFFF0, 64), golden_extra["helpers/signs_wrap_64"])
    for d, b, stride in golden_extra["helpers/stride"]:
        assert spec_np.code_stride_bytes(int(d), int(b)) == stride


def test_pack_unpack_round_trip():
    rng = np.random.default_rng(5)
    for d in (1, 2, 7, 64, 96, 100, 1024):
        for b in spec_np.SUPPORTED_BITS:
            codes = rng.integers(0, 1 << b, size=(5, d))
            buf = spec_np.pack_codes(codes, b)
            assert len(buf) == 5 * spec_np.code_stride_bytes(d, b)
            assert np.array_equal(spec_np.unpack_codes(buf, 5, d, b), codes)


# ---------------------------------------------------------------- oracle #2 (float32) vs fixtures
def _vector_cases(g):
    return [c for c in g.cases if c.get("kind", "vector") == "vector"]


@pytest.mark.parametrize("which", ["parity", "extra"])
def test_f32_oracle_per_vector(which, golden_parity, golden_extra):
    g = golden_parity if which == "parity" else golden_extra
    total = mism = 0
    for c in _vector_cases(g):
        X = g[f"input/{c['group']}"]
        n, d = X.shape
        k, b = c["key"], c["bits"]
        codes, scales = kernel_f32.encode(c["method"], X, b, c["seed"])
        ref_codes, ref_scales = g[f"{k}/codes"], g[f"{k}/scales"]
        diff = _unpack(codes, n, d, b) != _unpack(ref_codes, n, d, b)
        assert diff.sum() <= max(2, diff.size // 500), (k, int(diff.sum()))        # ParityTests.swift:67
        assert np.all(np.abs(scales - ref_scales) <= 1e-5 * np.maximum(1, np.abs(ref_scales))), k  # :69
        dec = kernel_f32.decode(c["method"], ref_codes, ref_scales, d, b, c["seed"])
        assert max_rel_l2(dec, g[f"{k}/reconstruction"]) < 1e-5, k                   # :73-76
        total += diff.size
        mism += int(diff.sum())
    # float32-vs-float64 boundary ties are rare: well under one code in ten thousand overall
    assert mism <= max(4, total // 10000), (mism, total)


@pytest.mark.parametrize("which", ["parity", "extra"])
def test_f32_oracle_metal_literal_polar_variant(which, golden_parity, golden_extra):
    """The PolarQuant encoder written as the Metal kernel writes it (a division per pair,
    PITCHKernels.metal:207-214) meets the reference's float32-vs-float64 tolerance on the golden
    vectors, and differs from the division-free variant on a handful of codes only."""
    g = golden_parity if which == "parity" else golden_extra
    total = mism = between = 0
    for c in _vector_cases(g):
        if c["method"] != "polarQuant":
            continue
        X = g[f"input/{c['group']}"]
        n, d = X.shape
        k, b = c["key"], c["bits"]
        codes, scales = kernel_f32.encode("polarQuant", X, b, c["seed"], metal_literal=True)
        other, other_scales = kernel_f32.encode("polarQuant", X, b, c["seed"])
        assert scales.tobytes() == other_scales.tobytes(), k
        diff = _unpack(codes, n, d, b) != _unpack(g[f"{k}/codes"], n, d, b)
        assert diff.sum() <= max(2, diff.size // 500), (k, int(diff.sum()))        # ParityTests.swift:67
        total += diff.size
        mism += int(diff.sum())
        between += int((_unpack(codes, n, d, b) != _unpack(other, n, d, b)).sum())
    assert total > 0 and mism <= max(4, total // 10000) and between <= max(4, total // 10000), (mism, between, total)


@pytest.mark.parametrize("which", ["channel", "extra"])
def test_f32_oracle_per_channel_is_bit_exact(which, golden_channel, golden_extra):
    g = golden_channel if which == "channel" else golden_extra
    cases = [c for c in g.cases if c.get("kind", "channel") == "channel"]
    assert cases
    for c in cases:
        X = g[f"input/{c['group']}"]
        n, d = X.shape
        k, b, G = c["key"], c["bits"], c["group_size"]
        codes, ranges = kernel_f32.channel_encode(X, b, G)
        assert ranges.tobytes() == g[f"{k}/ranges"].tobytes(), k                      # PerChannelTests.swift:82
        assert codes.tobytes() == g[f"{k}/codes"].tobytes(), k
        dec = kernel_f32.channel_decode(g[f"{k}/codes"], g[f"{k}/ranges"], n, d, b, G)
        assert dec.tobytes() == g[f"{k}/reconstruction"].tobytes(), k


def test_f32_oracle_half_conversion():
    L = kernel_f32.lib()
    vals = np.concatenate([np.random.default_rng(0).standard_normal(2000) * 100,
                           [0.0, -0.0, 65504.0, -65504.0, 6e-8, 1e-7, 6.1e-5, 65519.9, 1.0009765625]])
    for v in vals.astype(np.float32):
        assert L.pitch_oracle_f32_to_f16(float(v)) == int(np.float16(v).view(np.uint16)), v
    for h in (0x3C00, 0xC000, 0x7BFF, 0x0001, 0x0400, 0x83FF):                      # PerChannelTests.swift:214-221
        assert L.pitch_oracle_f16_to_f32(h) == float(np.uint16(h).view(np.float16))


def test_rotated_bias_oracle_reproduces_the_reference():
    """``oracle.spec_np.rotated_bias`` against the output of the reference's own ``rotated_bias``
    (reference/mechanism_eval.py:82-91), produced by tests/golden/make_bias_golden.py: bit for bit."""
    from conftest import Golden
    from oracle import spec_np
    g = Golden("rotated_bias.npz")
    assert len(g.cases) == 3
    for c in g.cases:
        k = c["key"]
        bias, cos, sin, want = g[f"{k}/bias"], g[f"{k}/cos"], g[f"{k}/sin"], g[f"{k}/rotated_bias"]
        assert want.shape == (c["heads"], c["positions"], c["dim"]) and want.dtype == np.float32
        for h in range(c["heads"]):
            assert spec_np.rotated_bias(bias[h], cos, sin).tobytes() == want[h].tobytes(), (k, h)
