"""Behaviour of the codec API on the GPU, re-expressing the reference's Swift suites:
CodecTests.swift, BatchAPITests.swift, PerChannelTests.swift, RotationWorstCaseTests.swift.
Inputs are seeded NumPy generators (the Swift generators are not reproducible here), so the
thresholds, not the vectors, come from those suites."""
import math

import numpy as np
import pytest

from conftest import max_rel_l2, mean_rel_err

pytestmark = pytest.mark.gpu

METHODS = ["turboQuant", "polarQuant"]


@pytest.fixture(scope="module")
def q():
    from pitch_b200 import PITCH
    return PITCH()


def gaussian(count, dim, seed):
    return np.random.default_rng(seed).standard_normal((count, dim)).astype(np.float32)


def uniform(count, dim, seed):
    return np.random.default_rng(seed).uniform(-1, 1, size=(count, dim)).astype(np.float32)


def offset_keys(count, dim, seed):
    x = gaussian(count, dim, seed)
    x[:, :min(4, dim)] += np.array([40, -25, 18, -12], dtype=np.float32)[:min(4, dim)]
    return x


def round_trip_error(q, method, bits, dim, count=64, gauss=False):
    x = gaussian(count, dim, 1) if gauss else uniform(count, dim, 1)
    return mean_rel_err(x, q.decode(q.encode(x, dim=dim, bits=bits, method=method)).reshape(count, dim))


# ---------------------------------------------------------------- accuracy (CodecTests.swift:12-74)
ACCURACY = [("turboQuant", 2, 0.14), ("turboQuant", 3, 0.045), ("turboQuant", 4, 0.013), ("turboQuant", 8, 1.5e-4),
            ("polarQuant", 2, 0.30), ("polarQuant", 3, 0.075), ("polarQuant", 4, 0.02), ("polarQuant", 8, 7.5e-5)]


@pytest.mark.parametrize("method,bits,threshold", ACCURACY)
@pytest.mark.parametrize("dim", [64, 512])
def test_round_trip_accuracy(q, method, bits, threshold, dim):
    assert round_trip_error(q, method, bits, dim) < threshold


@pytest.mark.parametrize("bits", range(2, 9))
def test_turboquant_meets_theorem_1(q, bits):
    e = round_trip_error(q, "turboQuant", bits, 64, count=16384, gauss=True)
    lower = 4.0 ** -bits
    assert lower <= e <= math.sqrt(3) * math.pi / 2 * lower


@pytest.mark.parametrize("method", METHODS)
def test_error_falls_with_bits(q, method):
    e = [round_trip_error(q, method, b, 256) for b in (2, 3, 4, 8)]
    assert e[0] > 2 * e[1] and e[1] > 2 * e[2] and e[2] > 50 * e[3]


def test_polar_angle_codebook_uses_all_codes(q):
    assert round_trip_error(q, "polarQuant", 3, 1024, count=16, gauss=True) < 0.070


@pytest.mark.parametrize("method", METHODS)
@pytest.mark.parametrize("dim", [2, 1024])
def test_extreme_dimensions_round_trip(q, method, dim):
    x = gaussian(8, dim, 3)
    out = q.decode(q.encode(x, dim=dim, bits=8, method=method))
    assert out.size == x.size and np.isfinite(out).all()
    assert mean_rel_err(x, out.reshape(8, dim)) < 0.01


# ---------------------------------------------------------------- behaviour (CodecTests.swift:76-158)
@pytest.mark.parametrize("method", METHODS)
def test_zero_vector_decodes_to_zero(q, method):
    batch = q.encode(np.zeros(64, dtype=np.float32), bits=4, method=method)
    assert np.all(q.decode(batch) == 0)
    if method == "turboQuant":      # the edge at exactly 0 is not strictly below 0: code 2^(b-1) - 1
        assert set(batch.codes) == {0x77}


@pytest.mark.parametrize("method", METHODS)
def test_scale_invariance(q, method):
    x = gaussian(4, 128, 4)
    a = q.decode(q.encode(x, dim=128, bits=4, method=method)).reshape(4, 128)
    b = q.decode(q.encode(x * 1000, dim=128, bits=4, method=method)).reshape(4, 128)
    assert max_rel_l2(b / 1000, a) < 1e-4


@pytest.mark.parametrize("method", METHODS)
def test_seed_determinism_and_effect(q, method):
    x = uniform(8, 256, 5)
    a = q.encode(x, dim=256, bits=4, method=method, seed=42)
    assert a == q.encode(x, dim=256, bits=4, method=method, seed=42)
    assert q.encode(x, dim=256, bits=4, method=method, seed=1).codes != q.encode(x, dim=256, bits=4, method=method, seed=2).codes


def test_seed_precedence(q):
    from pitch_b200 import PITCH, DEFAULT_SEED
    x = uniform(1, 64, 7)
    assert q.encode(x, bits=4, method="turboQuant").config.seed == DEFAULT_SEED
    assert PITCH(seed=7).encode(x, bits=4, method="turboQuant").config.seed == 7
    assert q.encode(x, bits=4, method="turboQuant", seed=99).config.seed == 99


@pytest.mark.parametrize("dim", [0, 1, 3, 100, 2048])
def test_invalid_dimension(q, dim):
    from pitch_b200 import PITCHError
    with pytest.raises(PITCHError):
        q.encode(np.ones(max(dim, 1), dtype=np.float32), dim=dim, bits=4, method="turboQuant")


@pytest.mark.parametrize("bits", [0, 1, 9, 16])
def test_invalid_bit_width(q, bits):
    from pitch_b200 import InvalidBitWidth
    with pytest.raises(InvalidBitWidth):
        q.encode(np.ones(64, dtype=np.float32), bits=bits, method="polarQuant")


def test_empty_and_partial_input(q):
    from pitch_b200 import PITCHError
    with pytest.raises(PITCHError):
        q.encode(np.zeros(0, dtype=np.float32), dim=64, bits=4, method="turboQuant")
    with pytest.raises(PITCHError):
        q.encode(np.ones(100, dtype=np.float32), dim=64, bits=4, method="turboQuant")


@pytest.mark.parametrize("bad", [float("nan"), float("inf"), float("-inf"), 1e30, -1e18])
@pytest.mark.parametrize("position", [0, 37, 4095])
def test_invalid_values(q, bad, position):
    from pitch_b200 import PITCHError
    x = np.full(4096, 0.5, dtype=np.float32)
    x[position] = bad
    with pytest.raises(PITCHError):
        q.encode(x, dim=64, bits=4, method="turboQuant")


@pytest.mark.parametrize("method", METHODS)
def test_largest_allowed_magnitude_round_trips(q, method):
    x = np.full(1024, 1e17, dtype=np.float32)
    out = q.decode(q.encode(x, bits=8, method=method))
    assert np.isfinite(out).all() and mean_rel_err(x[None], out[None]) < 0.01


# ---------------------------------------------------------------- rotation worst case
def test_one_hot_inputs_exceed_theorem_1(q):
    d = 64
    x = np.eye(d, dtype=np.float32)
    err = mean_rel_err(x, q.decode(q.encode(x, dim=d, bits=2, method="turboQuant")).reshape(d, d))
    assert abs(err - 0.25) < 1e-3 and err > math.sqrt(3) * math.pi / 2 / 16


def test_outlier_channel_within_bound(q):
    rng = np.random.default_rng(8)
    d, n = 64, 2048
    x = rng.standard_normal((n, d)).astype(np.float32)
    x[np.arange(n), rng.integers(0, d, n)] *= 30
    err = mean_rel_err(x, q.decode(q.encode(x, dim=d, bits=2, method="turboQuant")).reshape(n, d))
    assert err < math.sqrt(3) * math.pi / 2 / 16


# ---------------------------------------------------------------- batch API (BatchAPITests.swift)
@pytest.mark.parametrize("method", METHODS)
def test_batch_equals_individual_encodes(q, method):
    x = gaussian(16, 128, 10)
    batch = q.encode(x, dim=128, bits=3, method=method)
    for i in range(16):
        assert batch.vectors(i, i + 1) == q.encode(x[i], bits=3, method=method)


@pytest.mark.parametrize("method", METHODS)
def test_append_and_slice(q, method):
    from pitch_b200 import PITCHError
    whole = q.encode(gaussian(10, 64, 11), dim=64, bits=4, method=method)
    built = whole.vectors(0, 3)
    built.append(whole.vectors(3, 10))
    assert built == whole and built.count == 10
    other = q.encode(gaussian(1, 64, 13), bits=3, method=method)
    with pytest.raises(PITCHError):
        built.append(other)


@pytest.mark.parametrize("method", METHODS)
def test_decode_into_caller_buffer_at_offset(q, method):
    import torch
    dim, count, pad = 256, 4, 32
    batch = q.encode(gaussian(count, dim, 14), dim=dim, bits=4, method=method)
    expected = q.decode(batch)
    buf = torch.full((pad + count * dim + pad,), -12345.0, dtype=torch.float32, device=q.device)
    q.decode_into(batch, buf, offset=pad * 4)
    a = buf.cpu().numpy()
    assert np.array_equal(a[pad:pad + count * dim], expected)
    assert np.all(a[:pad] == -12345.0) and np.all(a[pad + count * dim:] == -12345.0)


@pytest.mark.parametrize("method", METHODS)
def test_gpu_resident_pipeline_matches_array_api(q, method):
    import torch
    dim, count = 128, 32
    cfg = q.config(method, dim, 4)
    x = gaussian(count, dim, 15)
    dev = q.device
    d_in = torch.from_numpy(x).to(dev)
    codes = torch.empty(count * cfg.code_stride, dtype=torch.uint8, device=dev)
    scales = torch.empty(count, dtype=torch.float32, device=dev)
    out = torch.empty(count * dim, dtype=torch.float32, device=dev)
    stream = q.make_stream()
    stream.wait_stream(torch.cuda.current_stream(dev))
    q.enqueue_encode(d_in, codes, scales, count, cfg, stream=stream)
    q.enqueue_decode(codes, scales, out, count, cfg, stream=stream)
    stream.synchronize()
    assert np.array_equal(out.cpu().numpy(), q.decode(q.encode(x, config=cfg)))


def test_enqueue_rejects_bad_buffers(q):
    import torch
    from pitch_b200 import InvalidInput
    dev = q.device
    cfg = q.config("turboQuant", 64, 4)
    x = torch.ones(64 * 4, dtype=torch.float32, device=dev)
    codes = torch.empty(cfg.code_stride * 3, dtype=torch.uint8, device=dev)       # needs 4
    scales = torch.empty(4, dtype=torch.float32, device=dev)
    with pytest.raises(InvalidInput):
        q.enqueue_encode(x, codes, scales, 4, cfg)
    pcfg = q.config("polarQuant", 64, 4)
    with pytest.raises(InvalidInput):                                               # misaligned offset
        q.enqueue_decode(torch.empty(1024, dtype=torch.uint8, device=dev), torch.empty(16, dtype=torch.float32, device=dev),
                         torch.empty(1024, dtype=torch.float32, device=dev), 1, pcfg, codes_offset=2)
    with pytest.raises(InvalidInput):                                               # count < 1
        q.enqueue_encode(x, torch.empty(128, dtype=torch.uint8, device=dev), scales, 0, cfg)
    with pytest.raises(InvalidInput):                                               # host memory
        q.enqueue_encode(torch.ones(64), torch.empty(128, dtype=torch.uint8, device=dev), scales, 1, cfg)


@pytest.mark.parametrize("method", METHODS)
def test_json_round_trip(q, method):
    from pitch_b200 import CompressedBatch
    batch = q.encode(gaussian(5, 128, 16), dim=128, bits=3, method=method)
    restored = CompressedBatch.from_json(batch.to_json())
    assert restored == batch and np.array_equal(q.decode(restored), q.decode(batch))


def test_batch_accounting(q):
    batch = q.encode(gaussian(100, 64, 18), dim=64, bits=3, method="turboQuant")
    assert batch.payload_byte_count == 2400 and batch.side_information_byte_count == 416
    assert batch.stored_byte_count == 2816 and batch.original_byte_count == 25600


# ---------------------------------------------------------------- per-channel (PerChannelTests.swift:102-228)
@pytest.mark.parametrize("dim", [64, 96, 128])
def test_error_within_half_a_step(q, dim):
    count, bits = 200, 4
    x = offset_keys(count, dim, dim)
    block = q.encode_per_channel(x, dim=dim, bits=bits)
    y = q.decode_per_channel(block).reshape(count, dim)
    r = block.ranges.view(np.float16).astype(np.float32).reshape(-1, 2, dim)
    g = np.arange(count) // 64
    lo, hi = r[g, 0], r[g, 1]
    step = (hi - lo) / 15
    slack = 1e-3 * np.maximum(np.abs(lo), np.abs(hi)) + 1e-6
    assert np.all(np.abs(x - y) <= 0.5 * step + slack)


def test_per_channel_beats_turboquant_on_offset_keys(q):
    x = offset_keys(256, 64, 3)
    ch = q.decode_per_channel(q.encode_per_channel(x, dim=64, bits=4)).reshape(256, 64)
    tq = q.decode(q.encode(x, dim=64, bits=4, method="turboQuant")).reshape(256, 64)
    assert ((x - ch) ** 2).mean() < 0.5 * ((x - tq) ** 2).mean()


def test_constant_channel_is_exact(q):
    x = gaussian(64, 8, 5)
    x[:, 0] = 1.5
    y = q.decode_per_channel(q.encode_per_channel(x, dim=8, bits=2)).reshape(64, 8)
    assert np.all(y[:, 0] == 1.5)


def test_partial_final_group(q):
    block = q.encode_per_channel(offset_keys(150, 64, 9), dim=64, bits=4)
    assert block.count == 150 and block.group_count == 3 and block.ranges.size == 3 * 2 * 64


def test_groupwise_encode_matches_whole_block(q):
    import torch
    dim, count = 64, 150
    cfg = q.channel_config(dim, 4)
    x = offset_keys(count, dim, 11)
    dev = q.device
    d_in = torch.from_numpy(x).to(dev)
    codes = torch.empty(count * cfg.code_stride, dtype=torch.uint8, device=dev)
    groups = cfg.group_count(count)
    ranges = torch.empty(groups * cfg.range_stride, dtype=torch.uint8, device=dev)
    out = torch.empty(count * dim, dtype=torch.float32, device=dev)
    for g in range(groups):
        first = g * cfg.group_size
        n = min(cfg.group_size, count - first)
        q.enqueue_per_channel_encode(d_in, codes, ranges, n, cfg, input_offset=first * dim * 4,
                                     codes_offset=first * cfg.code_stride, ranges_offset=g * cfg.range_stride)
    q.enqueue_per_channel_decode(codes, ranges, out, count, cfg)
    whole = q.decode_per_channel(q.encode_per_channel(x, config=cfg))
    assert np.array_equal(out.cpu().numpy(), whole)


def test_block_append_requires_group_boundary(q):
    from pitch_b200 import PITCHError
    x = offset_keys(64, 16, 2)
    a = q.encode_per_channel(x, dim=16, bits=4)
    a.append(q.encode_per_channel(x[:10], dim=16, bits=4))
    assert a.count == 74 and a.group_count == 2
    with pytest.raises(PITCHError):
        a.append(q.encode_per_channel(x, dim=16, bits=4))


def test_per_channel_rejects_invalid_arguments(q):
    from pitch_b200 import PITCHError
    for args in ([[1, 2, 3]], [[1, float("nan")]], [[1, 70000]]):
        with pytest.raises(PITCHError):
            q.encode_per_channel(np.array(args[0], dtype=np.float32), dim=2, bits=4)


def test_per_channel_storage_and_json(q):
    from pitch_b200 import ChannelCompressedBlock, ChannelQuantConfig
    c = ChannelQuantConfig(64, 4)
    block = q.encode_per_channel(offset_keys(128, 64, 1), config=c)
    assert block.stored_byte_count == 128 * 32 + 2 * 256 + 16
    b2 = q.encode_per_channel(offset_keys(70, 32, 4), dim=32, bits=3, group_size=32)
    assert ChannelCompressedBlock.from_json(b2.to_json()) == b2


def test_concurrent_host_threads_on_their_own_streams(q):
    """The C entry points are re-entrant: two host threads enqueue on two streams at once and each
    gets exactly what a single thread gets."""
    import threading
    import torch
    from pitch_b200 import ChannelQuantConfig, QuantConfig
    dev = q.device
    cfgs = [QuantConfig("turboQuant", 64, 4), QuantConfig("polarQuant", 128, 3), QuantConfig("turboQuant", 256, 5)]
    ccfg = ChannelQuantConfig(64, 4, 64)
    n = 4096

    def work(seed, stream, result):
        g = torch.Generator(device=dev)
        g.manual_seed(seed)
        outs = []
        with torch.cuda.stream(stream) if stream is not None else torch.cuda.stream(torch.cuda.current_stream(dev)):
            for rep in range(20):
                for cfg in cfgs:
                    x = torch.randn((n, cfg.dim), generator=g, device=dev)
                    codes = torch.empty(n * cfg.code_stride, dtype=torch.uint8, device=dev)
                    sc = torch.empty(n, device=dev)
                    y = torch.empty_like(x)
                    q.enqueue_encode(x, codes, sc, n, cfg, stream=stream)
                    q.enqueue_decode(codes, sc, y, n, cfg, stream=stream)
                    outs.append((codes, sc, y))
                x = torch.randn((n, 64), generator=g, device=dev)
                codes = torch.empty(n * ccfg.code_stride, dtype=torch.uint8, device=dev)
                rng_ = torch.empty(ccfg.group_count(n) * 2 * 64, dtype=torch.float16, device=dev)
                y = torch.empty_like(x)
                q.enqueue_per_channel_encode(x, codes, rng_, n, ccfg, stream=stream)
                q.enqueue_per_channel_decode(codes, rng_, y, n, ccfg, stream=stream)
                outs.append((codes, rng_, y))
            if stream is not None:
                stream.synchronize()
        result.extend(outs)

    serial = [[], []]
    for i in range(2):
        work(100 + i, None, serial[i])
    torch.cuda.synchronize()
    parallel = [[], []]
    streams = [torch.cuda.Stream(dev), torch.cuda.Stream(dev)]
    threads = [threading.Thread(target=work, args=(100 + i, streams[i], parallel[i])) for i in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    torch.cuda.synchronize()
    for i in range(2):
        assert len(serial[i]) == len(parallel[i]) == 80
        for a, b in zip(serial[i], parallel[i]):
            assert all(torch.equal(u, v) for u, v in zip(a, b))
