"""CPU-only tests: the C ABI library loads and exports every declared symbol, host-side value
types and containers behave like the reference's, sharding and the checksum gather work on two
gloo ranks.  No compute entry point is called here (there is no GPU and no CPU fallback)."""
import ctypes
import re
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def lib():
    from pitch_b200 import build as native_build
    native_build.build()
    from pitch_b200 import _native
    return _native.lib()


def test_library_exports_every_declared_symbol(lib):
    from pitch_b200 import _native
    header = (ROOT / "include" / "pitch_b200.h").read_text()
    declared = set(re.findall(r"^\s*(?:int|int64_t|const char\*)\s+(pitch_\w+)\s*\(", header, flags=re.M))
    assert declared, "no declarations found in the header"
    assert declared == set(_native.PROTOTYPES), declared ^ set(_native.PROTOTYPES)
    for name in declared:
        assert hasattr(lib, name), name
    assert lib.pitch_abi_version() == 2
    assert lib.pitch_status_string(3) == b"invalid dimension"


def test_stride_and_codebook_table(lib):
    from pitch_b200 import codebooks, code_stride_bytes
    for d, b, want in ((64, 3, 24), (64, 4, 32), (128, 3, 48), (1024, 4, 512), (2, 3, 4), (96, 3, 36), (1, 2, 4)):
        assert lib.pitch_code_stride(d, b) == want == code_stride_bytes(d, b)      # BatchAPITests.swift:160-175
    codebooks.register_all()
    assert lib.pitch_has_codebook(64, 4) == 1 and lib.pitch_has_codebook(100, 4) == 0
    c = codebooks.turbo_codebook(64, 4)
    assert c.dtype == np.float64 and c.shape == (16,) and np.array_equal(c, -c[::-1]) and np.all(np.diff(c) > 0)
    bad = (ctypes.c_float * 4)(0.0, 1.0, 0.5, 2.0)
    assert lib.pitch_set_codebook(64, 2, bad) == 1                                 # not ascending -> invalid input
    assert b"ascending" in lib.pitch_last_error()
    assert lib.pitch_set_codebook(100, 2, bad) == 3 and lib.pitch_set_codebook(64, 9, bad) == 2


def test_validation_happens_before_any_device_work(lib):
    """Argument errors are reported with the reference's status codes even without a GPU."""
    from pitch_b200 import _native
    B = _native.Buffer
    ok = B(0x1000, 1 << 20, 0)
    f = lib.pitch_enqueue_encode
    assert f(0, 100, 4, 0, 0, ok, ok, ok, 1, None) == 3            # invalidDimension
    assert f(0, 64, 9, 0, 0, ok, ok, ok, 1, None) == 2             # invalidBitWidth
    assert f(0, 64, 4, 0, 0, ok, ok, ok, 0, None) == 1             # count must be at least 1
    assert f(0, 64, 4, 0, 0, ok, B(0x1000, 1 << 20, 2), ok, 1, None) == 1   # offset not a multiple of 4
    assert b"multiple of 4" in lib.pitch_last_error()
    assert f(0, 64, 4, 0, 0, ok, B(0x1000, 64, 0), ok, 4, None) == 1        # codes buffer too small
    assert b"needs 128" in lib.pitch_last_error()
    assert f(0, 64, 4, 0, 0, B(None, 0, 0), ok, ok, 1, None) == 1
    g = lib.pitch_enqueue_channel_decode
    assert g(0, 4, 64, 0, ok, ok, ok, 1, None) == 1 and g(2048, 4, 64, 0, ok, ok, ok, 1, None) == 1
    assert g(64, 1, 64, 0, ok, ok, ok, 1, None) == 2 and g(64, 4, 0, 0, ok, ok, ok, 1, None) == 1


def _cache_desc(dim=64, segments=48, tokens=32768, k=(2, 4, 64), v=(0, 4, 0)):
    from pitch_b200 import _native
    d = _native.CacheDesc()
    d.dim, d.out_dtype, d.segments, d.tokens, d.n_planes = dim, 2, segments, tokens, 2
    for pl, (kind, bits, group) in zip(d.planes, (k, v)):
        pl.kind, pl.bits, pl.group_size = kind, bits, group
        pl.codes = pl.side = pl.out = 0x10000
        pl.codes_seg_stride = pl.side_seg_stride = pl.out_seg_stride = 1 << 30
        pl.codes_bytes = pl.side_bytes = pl.out_bytes = 1 << 40
    return d


def test_cache_entry_points_check_extents_before_any_device_work(lib):
    """Codec.check for the whole-cache calls (Sources/PITCH/Core/Codec.swift:37-47): every plane's
    buffers must cover the segments and tokens addressed; refusals come before any launch."""
    import ctypes as C
    from pitch_b200 import _native
    dec, app, step = lib.pitch_enqueue_cache_decode, lib.pitch_enqueue_cache_append, lib.pitch_enqueue_cache_step
    err = lib.pitch_last_error

    def src_for(d, n_new=1, residual=True):
        src = (_native.AppendSrc * 4)()
        for i in range(2):
            src[i].input, src[i].input_seg_stride, src[i].input_bytes = 0x20000, d.dim * 4 * n_new, 1 << 30
            if residual and d.planes[i].kind == 2:
                src[i].residual, src[i].residual_seg_stride, src[i].residual_bytes = 0x30000, (d.planes[i].group_size + 2) * d.dim * 4, 1 << 30
        return src

    # decode: each buffer of each plane, one byte short of what 48 segments x 32768 tokens need
    for plane, field, what in ((0, "codes_bytes", b"codes buffer"), (1, "codes_bytes", b"codes buffer"),
                               (0, "side_bytes", b"side-information"), (1, "side_bytes", b"side-information"),
                               (0, "out_bytes", b"output buffer"), (1, "out_bytes", b"output buffer")):
        d = _cache_desc()
        pl = d.planes[plane]
        need = {"codes_bytes": 32768 * 32, "side_bytes": 512 * 2 * 64 * 2 if plane == 0 else 32768 * 4, "out_bytes": 32768 * 64 * 2}[field]
        setattr(pl, field, 47 * (1 << 30) + need - 1)
        assert dec(C.byref(d), None) == 1 and what in err() and str(47 * (1 << 30) + need).encode() in err(), err()
    d = _cache_desc()
    d.planes[1].out_seg_stride = 32768 * 64 * 2 - 16
    assert dec(C.byref(d), None) == 1 and b"segment stride" in err()
    d = _cache_desc()
    d.planes[0].side = 0x10008
    assert dec(C.byref(d), None) == 1 and b"multiples of 16" in err()
    d = _cache_desc()
    d.planes[1].out = 0
    assert dec(C.byref(d), None) == 1 and b"null pointer" in err()
    d = _cache_desc()
    d.capacity = 32000                                      # the cache was sized for fewer tokens than the call addresses
    assert dec(C.byref(d), None) == 1 and b"sized for 32000" in err()
    d = _cache_desc(tokens=100)
    d.capacity = 32768                                      # extents are checked against the capacity, not the tokens held
    d.planes[0].codes_bytes = 47 * (1 << 30) + 100 * 32
    assert dec(C.byref(d), None) == 1 and b"codes buffer" in err()

    # append / step: the cache must have room for the new tokens, inputs and residual must be long enough
    d = _cache_desc(tokens=32768)
    d.planes[1].side_bytes = 47 * (1 << 30) + 32768 * 4     # room for exactly the tokens held
    assert app(C.byref(d), src_for(d), 0, 1, None) == 1 and b"side-information" in err()
    assert step(C.byref(d), src_for(d), 0, None, None) == 1 and b"side-information" in err()
    d = _cache_desc(tokens=63)
    assert app(C.byref(d), src_for(d, 2), 0, 2, None) == 1 and b"one group" in err()
    d = _cache_desc(tokens=10)
    src = src_for(d)
    src[1].input_bytes = 47 * 256 + 255
    assert app(C.byref(d), src, 0, 1, None) == 1 and b"input buffer" in err()
    src = src_for(d)
    src[0].residual_bytes = 47 * 66 * 256 + 66 * 256 - 1
    assert app(C.byref(d), src, 0, 1, None) == 1 and b"residual buffer" in err()
    src = src_for(d, residual=False)
    assert app(C.byref(d), src, 0, 1, None) == 1 and b"residual buffer is null" in err()
    src = src_for(d)
    src[0].input = 0x20002
    assert step(C.byref(d), src, 0, None, None) == 1 and b"multiples of 4" in err()
    # a device-side counter needs the capacity in the descriptor and an aligned counter
    assert step(C.byref(d), src_for(d), 0, 0x40000, None) == 1 and b"capacity" in err()
    d.capacity = 32768
    assert step(C.byref(d), src_for(d), 0, 0x40008, None) == 1 and b"16-byte aligned" in err()
    # the allocation-free append range-checks every factor of the residual size before multiplying
    d = _cache_desc(tokens=0)
    d.segments = 1 << 40
    assert lib.pitch_enqueue_cache_append_noalloc(C.byref(d), src_for(d), 0, 1, None) == 1 and b"segments" in err()
    d = _cache_desc(tokens=0, k=(2, 4, 1 << 20))
    assert lib.pitch_enqueue_cache_append_noalloc(C.byref(d), src_for(d), 0, 1, None) == 1 and b"group size" in err()


def test_newest_token_gather_checks_its_arguments(lib):
    import ctypes as C
    f = lib.pitch_enqueue_cache_newest
    d = _cache_desc()
    need = 2 * 48 * 64 * 2
    assert f(C.byref(d), None, None, need, None) == 1 and b"destination" in lib.pitch_last_error()
    assert f(C.byref(d), None, 0x50008, need, None) == 1 and b"aligned" in lib.pitch_last_error()
    assert f(C.byref(d), None, 0x50000, need - 1, None) == 1 and b"needs 12288" in lib.pitch_last_error()
    assert f(C.byref(_cache_desc(tokens=0)), None, 0x50000, need, None) == 1 and b"no token" in lib.pitch_last_error()
    assert f(C.byref(d), 0x60000, 0x50000, need, None) == 1 and b"capacity" in lib.pitch_last_error()   # counter without capacity
    d.planes[1].out_bytes = 47 * (1 << 30) + 32768 * 64 * 2 - 1
    assert f(C.byref(d), None, 0x50000, need, None) == 1 and b"output buffer" in lib.pitch_last_error()
    assert f(None, None, 0x50000, need, None) == 1


def test_attention_workspace_and_shape_rules(lib):
    """Pure host logic of the cache attention entry point: run partitioning and refusals."""
    import ctypes as C
    from pitch_b200 import _native
    ws = lib.pitch_cache_attention_workspace
    d = _cache_desc()
    # 48 x 1024 tiles over 2368 resident warps -> runs of 21 tiles, 49 runs per segment
    assert ws(C.byref(d), 7) == 48 * 49 * 7 * 66 * 4
    assert ws(C.byref(_cache_desc(segments=1, tokens=31)), 8) == 1 * 1 * 8 * 66 * 4
    assert ws(C.byref(_cache_desc(segments=2, tokens=5000)), 1) == 2 * 40 * 1 * 66 * 4      # at least 4 tiles per run
    assert ws(C.byref(_cache_desc(k=(0, 4, 0))), 7) == 48 * 49 * 7 * 66 * 4             # TurboQuant keys: same run layout
    # dim 128 (TurboQuant keys only): 8 warps per multiprocessor -> runs of 43 tiles, 24 per segment, 2 + 128 floats each;
    # 10 with bf16 operands and 4-bit codes -> runs of 35 tiles, 30 per segment: room for either
    assert ws(C.byref(_cache_desc(dim=128, k=(0, 4, 0))), 8) == 48 * 30 * 8 * 130 * 4
    assert ws(C.byref(_cache_desc(dim=128, k=(0, 3, 0), v=(0, 3, 0))), 8) == 48 * 24 * 8 * 130 * 4   # 3-bit cache at dim 128
    for bad in (_cache_desc(dim=128), _cache_desc(dim=128, k=(0, 4, 0), v=(0, 3, 0)), _cache_desc(dim=128, k=(0, 3, 0)), _cache_desc(k=(2, 4, 48)), _cache_desc(k=(2, 2, 64)), _cache_desc(k=(0, 3, 0)), _cache_desc(k=(1, 4, 0)),
                _cache_desc(v=(1, 4, 0)), _cache_desc(v=(0, 3, 0)), _cache_desc(tokens=0)):
        assert ws(C.byref(bad), 4) == -1 and lib.pitch_last_error()
    assert ws(C.byref(d), 0) == -1 and ws(C.byref(d), 9) == -1
    args = _native.AttentionArgs(0x10000, 0x20000, 0x30000, 16, 7, 0.125)
    assert lib.pitch_enqueue_cache_attention(C.byref(d), C.byref(args), None) == 1          # workspace too small
    assert b"workspace" in lib.pitch_last_error()
    args = _native.AttentionArgs(0x10000, 0x20000, 0x30000, 1 << 30, 7, 0.0)
    assert lib.pitch_enqueue_cache_attention(C.byref(d), C.byref(args), None) == 1 and b"scale" in lib.pitch_last_error()


def test_rope_bias_argument_rules(lib):
    import ctypes as C
    from pitch_b200 import _native
    f = lib.pitch_enqueue_rope_bias
    rope = _native.RopeBias(0x1000, 256, 0x2000, 0x3000, 100)
    assert f(12, 0, 1, 0x4000, 1024, 1, 0, 4, C.byref(rope), None) == 3                      # dim not a multiple of 8
    assert f(64, 5, 1, 0x4000, 1024, 1, 0, 4, C.byref(rope), None) == 1                      # unknown dtype
    assert f(64, 0, 1, 0x4000, 1024, 1, 98, 4, C.byref(rope), None) == 1 and b"rotary tables" in lib.pitch_last_error()
    assert f(64, 0, 1, 0x4004, 1024, 1, 0, 4, C.byref(rope), None) == 1 and b"aligned" in lib.pitch_last_error()
    assert f(64, 0, 1, 0x4000, 1024, 1, 0, 4, None, None) == 1
    assert f(64, 0, 1, 0x4000, 512, 2, 0, 4, C.byref(rope), None) == 1 and b"stride" in lib.pitch_last_error()


def test_missing_library_fails_loudly(tmp_path, monkeypatch):
    from pitch_b200 import KernelUnavailable, _native
    monkeypatch.setattr(_native, "_lib", None)
    monkeypatch.setattr(_native, "LIB_PATH", tmp_path / "nope.so")
    with pytest.raises(KernelUnavailable):
        _native.lib()


def test_product_never_imports_the_oracle():
    for path in (ROOT / "pitch_b200").rglob("*.py"):
        text = path.read_text()
        assert not re.search(r"^\s*(from|import)\s+oracle\b", text, flags=re.M), path
    for path in (ROOT / "pitch_b200" / "csrc").glob("*"):
        assert "oracle" not in path.read_text(), path


# ---------------------------------------------------------------- configs (QuantConfig / ChannelQuantConfig)
def test_quant_config_validation_and_accounting():
    from pitch_b200 import InvalidBitWidth, InvalidDimension, QuantConfig, QuantMethod
    for dim in (0, 1, 3, 100, 2048):
        with pytest.raises(InvalidDimension):
            QuantConfig("turboQuant", dim, 4)
    for bits in (0, 1, 9, 16):
        with pytest.raises(InvalidBitWidth):
            QuantConfig("polarQuant", 64, bits)
    t = QuantConfig(QuantMethod.turboQuant, 64, 3)
    assert (t.code_stride, t.bytes_per_vector, t.bits_per_coordinate) == (24, 28, 3.5)
    p = QuantConfig("polarQuant", 1024, 4)
    assert p.bytes_per_vector == 516 and abs(p.compression_ratio - 4096 / 516) < 1e-12
    kv = QuantConfig("turboQuant", np.int64(64), 4)
    assert abs(kv.compression_ratio_vs_float16 - 16 / 4.5) < 1e-12 and kv.seed == 0x50495443
    assert QuantConfig.from_json(kv.to_json()) == kv


def test_channel_config_validation_and_accounting():
    from pitch_b200 import ChannelQuantConfig, PITCHError
    for args in ((0, 4), (2048, 4), (64, 1), (64, 4, 0), (64, 4, 70000)):
        with pytest.raises(PITCHError):
            ChannelQuantConfig(*args)
    c = ChannelQuantConfig(64, 4)
    assert c.bits_per_coordinate == 4.5 and ChannelQuantConfig(128, 4).bits_per_coordinate == 4.5
    assert ChannelQuantConfig(128, 4, 128).bits_per_coordinate == 4.25
    assert c.group_count(150) == 3 and c.range_stride == 256 and ChannelQuantConfig(96, 3).code_stride == 36


# ---------------------------------------------------------------- containers
def test_compressed_batch_rules():
    from pitch_b200 import CompressedBatch, PITCHError, QuantConfig
    cfg = QuantConfig("turboQuant", 64, 4)
    for codes, scales in ((bytes(28), [1]), (bytes(32), [1, 2]), (bytes(32), [float("nan")]), (b"", []), (bytes(32), [-1])):
        with pytest.raises(PITCHError):
            CompressedBatch(cfg, codes, scales)
    a = CompressedBatch(cfg, bytes(range(64)), [1.0, 2.0])
    b = a.vectors(1, 2)
    assert b.count == 1 and b.codes == bytes(range(32, 64)) and b.scales[0] == 2.0
    c = a.vectors(0, 1)
    c.append(b)
    assert c == a
    with pytest.raises(PITCHError):
        a.vectors(1, 1)
    with pytest.raises(PITCHError):
        a.append(CompressedBatch(QuantConfig("turboQuant", 64, 3), bytes(24), [1.0]))
    assert CompressedBatch.from_json(a.to_json()) == a
    import json
    obj = json.loads(a.to_json())
    assert set(obj) == {"formatVersion", "config", "codes", "scales"} and obj["formatVersion"] == 3
    assert obj["config"] == {"method": "turboQuant", "dim": 64, "bits": 4, "seed": 0x50495443}
    obj["formatVersion"] = 4
    with pytest.raises(PITCHError):
        CompressedBatch.from_json(json.dumps(obj))
    with pytest.raises(PITCHError):
        CompressedBatch.from_json('{"formatVersion":3,"config":{"method":"turboQuant","dim":100,"bits":4,"seed":1},"codes":"","scales":[1]}')
    assert a.stored_byte_count == 64 + 8 + 16 and a.original_byte_count == 512


def test_channel_block_rules():
    from pitch_b200 import ChannelCompressedBlock, ChannelQuantConfig, PITCHError, half_to_float
    cfg = ChannelQuantConfig(4, 4)
    with pytest.raises(PITCHError):
        ChannelCompressedBlock(cfg, bytes(4), [0, 0])                                  # ranges too short
    with pytest.raises(PITCHError):
        ChannelCompressedBlock(cfg, bytes(4), [0x4000, 0, 0, 0, 0x3C00, 0, 0, 0])      # min 2.0 above max 1.0
    blk = ChannelCompressedBlock(cfg, bytes(4), [0x3C00, 0, 0, 0, 0x4000, 0, 0, 0])
    assert blk.range(0, 0) == (1.0, 2.0) and blk.count == 1 and blk.group_count == 1
    assert ChannelCompressedBlock.from_json(blk.to_json()) == blk
    with pytest.raises(PITCHError):
        blk.append(blk)                                                                  # partial group
    for h, want in ((0x3C00, 1.0), (0xC000, -2.0), (0x7BFF, 65504.0), (0x0001, 2.0 ** -24)):
        assert half_to_float(h) == want
    assert half_to_float(0x7C00) == float("inf") and np.isnan(half_to_float(0x7E00))


# ---------------------------------------------------------------- sharding + gloo gather
def test_shard_segments_cover_without_overlap():
    from pitch_b200.shard import shard_segments
    for world in (1, 2, 4, 8):
        shards = [shard_segments(24, 2, world, r) for r in range(world)]
        assert [s.segments for s in shards] == [48 // world] * world
        covered = [i for s in shards for i in s.segment_range]
        assert covered == list(range(48))
        shards = [shard_segments(80, 8, world, r, by="segment") for r in range(world)]
        assert sum(s.segments for s in shards) == 640 and shards[-1].segment_range[-1] == 639
    uneven = [shard_segments(5, 1, 3, r, by="segment") for r in range(3)]
    assert [list(s.segment_range) for s in uneven] == [[0, 1], [2, 3], [4]]
    with pytest.raises(ValueError):
        shard_segments(24, 2, 5, 0)


_GLOO = r"""
import os, sys, datetime
sys.path.insert(0, {root!r})
import torch.distributed as dist
from pitch_b200.shard import gather_int64, shard_segments
rank, world, mode = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3]
os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=sys.argv[4], RANK=str(rank), WORLD_SIZE=str(world))
dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=8))
sh = shard_segments(24, 2, world, rank)
if mode == "die" and rank == 1:
    raise SystemExit(3)                      # a rank that never reaches the gather
got = gather_int64([0xFFFFFFFFFFFFFFF0 + rank, sh.first_segment, sh.segments])
assert got == [[0xFFFFFFFFFFFFFFF0 + r, r * 24, 24] for r in range(world)], got
print("ok", rank)
dist.destroy_process_group()
"""


def _spawn(mode, port):
    code = _GLOO.format(root=str(ROOT))
    return [subprocess.Popen([sys.executable, "-c", code, str(r), "2", mode, str(port)], stdout=subprocess.PIPE,
                             stderr=subprocess.PIPE, text=True) for r in range(2)]


def test_checksum_gather_on_two_gloo_ranks():
    procs = _spawn("ok", 29731)
    outs = [p.communicate(timeout=120) for p in procs]
    assert [p.returncode for p in procs] == [0, 0], outs
    assert all("ok" in o[0] for o in outs)


def test_gather_fails_cleanly_when_a_rank_is_missing():
    procs = _spawn("die", 29733)
    outs = [p.communicate(timeout=120) for p in procs]
    assert procs[1].returncode == 3
    assert procs[0].returncode not in (0, None), outs     # the survivor gets an error, it does not hang


# ---------------------------------------------------------------- benchmark bookkeeping
def test_bench_byte_accounting_matches_the_published_workload():
    """Algorithmic bytes of one whole-cache decode of configuration 4 (the figures the benchmark's roofline is computed from)."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("bench", ROOT / "bench.py")
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    rd, wr = bench.step_bytes(48, 32768)
    assert (rd, wr) == (113_246_208, 402_653_184) and rd + wr == 515_899_392
    rd1, wr1 = bench.step_bytes(1, 65)                       # a partial second group still costs a full range block
    assert rd1 == 65 * 32 + 2 * 256 + 65 * 32 + 65 * 4 and wr1 == 2 * 65 * 64 * 2
