"""Whole-cache decode and append (the per-step hot loop): the fused launch must give exactly
what the stand-alone decoders give, which in turn are pinned to the oracles elsewhere."""
import numpy as np
import pytest

from conftest import max_rel_l2
from oracle import kernel_f32, spec_np

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def q():
    from pitch_b200 import PITCH
    return PITCH()


def make_inputs(rng, S, T, d):
    K = rng.standard_normal((S, T, d)) + rng.normal(0.0, 2.0, size=(S, 1, d))
    V = rng.standard_normal((S, T, d))
    return K.astype(np.float32), V.astype(np.float32)


@pytest.mark.parametrize("out_dtype", ["bfloat16", "float16", "float32"])
def test_fused_decode_d64_b4_matches_oracles(q, out_dtype):
    """Config 4's shape at reduced size: K per-channel b=4 G=64, V TurboQuant b=4, d=64."""
    import torch
    from pitch_b200 import ChannelQuantConfig, KVCache, QuantConfig
    rng = np.random.default_rng(4)
    S, T, d = 6, 333, 64                     # partial last tile, partial last group
    K, V = make_inputs(rng, S, T, d)
    cache = KVCache(S, d, 400, ChannelQuantConfig(d, 4, 64), QuantConfig("turboQuant", d, 4),
                    out_dtype=out_dtype, pitch=q)
    cache.prefill(torch.from_numpy(K).to(q.device), torch.from_numpy(V).to(q.device))
    assert cache.tokens == T
    ko, vo = cache.decode()
    torch.cuda.synchronize()
    tdt = getattr(torch, out_dtype)
    for s in range(S):
        kc, kr = spec_np.channel_encode(K[s], 4, 64)
        k_ref = torch.from_numpy(spec_np.channel_decode(kc, kr, 4, 64)).to(tdt)
        assert torch.equal(ko[s].cpu(), k_ref), s                      # bit-exact, after rounding to out_dtype
        vc, vn = kernel_f32.encode("turboQuant", V[s], 4)
        got_codes = cache.planes[1].codes[s, :T * 32].cpu().numpy()
        assert got_codes.tobytes() == vc.tobytes(), s
        v32 = kernel_f32.decode("turboQuant", vc, vn, d, 4)
        if out_dtype == "float32":
            assert max_rel_l2(vo[s].cpu().numpy(), v32) < 2e-6
            spec = spec_np.turbo_decode(spec_np.unpack_codes(vc.tobytes(), T, d, 4), vn.astype(np.float64), 4)
            assert max_rel_l2(vo[s].cpu().numpy(), spec) < 1e-5
        else:
            # half outputs: equal to the rounded float32 oracle except where the two float32 values
            # straddle a rounding boundary (different but equally valid summation order)
            ref16 = torch.from_numpy(v32).to(tdt)
            mism = (vo[s].cpu() != ref16).float().mean().item()
            assert mism < 2e-3, (s, mism)
            assert max_rel_l2(vo[s].cpu().float().numpy(), v32) < (5e-3 if out_dtype == "bfloat16" else 6e-4)
    # untouched beyond the tokens held
    assert torch.count_nonzero(cache.planes[0].out[:, T:]) == 0 and torch.count_nonzero(cache.planes[1].out[:, T:]) == 0


def test_fused_equals_standalone_decoders(q):
    import torch
    from pitch_b200 import ChannelQuantConfig, KVCache, QuantConfig
    rng = np.random.default_rng(5)
    S, T, d = 4, 515, 64
    K, V = make_inputs(rng, S, T, d)
    kcfg, vcfg = ChannelQuantConfig(d, 4, 64), QuantConfig("turboQuant", d, 4)
    cache = KVCache(S, d, T, kcfg, vcfg, out_dtype="bfloat16", pitch=q)
    cache.prefill(torch.from_numpy(K).to(q.device), torch.from_numpy(V).to(q.device))
    ko, vo = cache.decode()
    for s in range(S):
        k1 = torch.empty((T, d), dtype=torch.bfloat16, device=q.device)
        v1 = torch.empty((T, d), dtype=torch.bfloat16, device=q.device)
        pk, pv = cache.planes
        q.enqueue_per_channel_decode(pk.codes[s], pk.side[s].reshape(-1), k1, T, kcfg)
        q.enqueue_decode(pv.codes[s], pv.side[s], v1, T, vcfg)
        assert torch.equal(k1, ko[s]) and torch.equal(v1, vo[s])


@pytest.mark.parametrize("kcfg_name,vcfg_name,d", [("turbo3", "turbo3", 128), ("turbo4", "turbo4", 128),
                                                     ("chan4", "turbo3", 128), ("chan4g32", "turbo3", 64),
                                                     ("chan4g32", "polar4", 64), ("chan3", "turbo5", 32)])
def test_other_cache_shapes(q, kcfg_name, vcfg_name, d):
    """Config 5's shape (K and V both TurboQuant, d=128, b in {3,4}), per-channel keys at d=128 and
    3-bit values (all on the one-launch path), and combinations that take one launch per segment."""
    import torch
    from pitch_b200 import ChannelQuantConfig, KVCache, QuantConfig

    def cfg(name):
        return {"turbo3": QuantConfig("turboQuant", d, 3), "turbo4": QuantConfig("turboQuant", d, 4),
                "turbo5": QuantConfig("turboQuant", d, 5), "polar4": QuantConfig("polarQuant", d, 4),
                "chan4": ChannelQuantConfig(d, 4, 64), "chan4g32": ChannelQuantConfig(d, 4, 32),
                "chan3": ChannelQuantConfig(d, 3, 64)}[name]
    rng = np.random.default_rng(6)
    S, T = 3, 200
    K, V = make_inputs(rng, S, T, d)
    kc, vc = cfg(kcfg_name), cfg(vcfg_name)
    cache = KVCache(S, d, T, kc, vc, out_dtype="float16", pitch=q)
    cache.prefill(torch.from_numpy(K).to(q.device), torch.from_numpy(V).to(q.device))
    outs = cache.decode()
    torch.cuda.synchronize()
    for x, c, o in zip((K, V), (kc, vc), outs):
        for s in range(S):
            if isinstance(c, ChannelQuantConfig):
                codes, r = spec_np.channel_encode(x[s], c.bits, c.group_size)
                ref = spec_np.channel_decode(codes, r, c.bits, c.group_size)
                assert torch.equal(o[s].cpu(), torch.from_numpy(ref).half())
            else:
                codes, sc = kernel_f32.encode(c.method.value, x[s], c.bits)
                ref = kernel_f32.decode(c.method.value, codes, sc, d, c.bits)
                assert max_rel_l2(o[s].cpu().float().numpy(), ref) < 6e-4


def test_append_equals_bulk_encode(q):
    """Growing cache: tokens appended one (or a few) at a time have exactly the codes, norms and
    ranges of a bulk encode of the same tokens (README.md:62-85 pattern;
    PerChannelTests.swift:143-172 for the group-wise equivalence)."""
    import torch
    from pitch_b200 import ChannelQuantConfig, KVCache, QuantConfig
    rng = np.random.default_rng(7)
    S, T, d = 5, 150, 64
    K, V = make_inputs(rng, S, T, d)
    kcfg, vcfg = ChannelQuantConfig(d, 4, 64), QuantConfig("turboQuant", d, 4)
    Kd, Vd = torch.from_numpy(K).to(q.device), torch.from_numpy(V).to(q.device)
    bulk = KVCache(S, d, T, kcfg, vcfg, pitch=q)
    bulk.prefill(Kd, Vd)
    grown = KVCache(S, d, T, kcfg, vcfg, pitch=q)
    grown.prefill(Kd[:, :70].contiguous(), Vd[:, :70].contiguous())
    t = 70
    for step in (1, 1, 3, 1, 70, 4):                       # crosses a group boundary inside the 70
        grown.append(Kd[:, t:t + step].contiguous(), Vd[:, t:t + step].contiguous())
        t += step
    assert t == T and grown.tokens == T
    torch.cuda.synchronize()
    for pb, pg in zip(bulk.planes, grown.planes):
        assert torch.equal(pb.codes, pg.codes) and torch.equal(pb.side, pg.side)
    assert bulk.checksums() == grown.checksums() or True   # decoded buffers compared below
    ob, og = bulk.decode(), grown.decode()
    assert torch.equal(ob[0], og[0]) and torch.equal(ob[1], og[1])
    assert bulk.checksums() == grown.checksums()


def test_append_general_dims_and_dtypes(q):
    import torch
    from pitch_b200 import ChannelQuantConfig, KVCache, QuantConfig
    rng = np.random.default_rng(8)
    for d, kcfg, vcfg, dt in ((128, QuantConfig("turboQuant", 128, 3), QuantConfig("polarQuant", 128, 4), torch.float16),
                              (16, ChannelQuantConfig(16, 5, 8), QuantConfig("turboQuant", 16, 8), torch.bfloat16),
                              (1024, QuantConfig("polarQuant", 1024, 2), QuantConfig("turboQuant", 1024, 6), torch.float32)):
        S, T = 2, 21
        K, V = make_inputs(rng, S, T, d)
        Kd, Vd = torch.from_numpy(K).to(q.device).to(dt), torch.from_numpy(V).to(q.device).to(dt)
        bulk = KVCache(S, d, 64, kcfg, vcfg, out_dtype="float32", pitch=q)
        bulk.prefill(Kd, Vd)
        grown = KVCache(S, d, 64, kcfg, vcfg, out_dtype="float32", pitch=q)
        for t in range(T):
            grown.append(Kd[:, t:t + 1].contiguous(), Vd[:, t:t + 1].contiguous())
        torch.cuda.synchronize()
        for pb, pg in zip(bulk.planes, grown.planes):
            if pb.is_channel or pb.config.method.value == "turboQuant":
                assert torch.equal(pb.codes, pg.codes), (d, pb.name)
            else:                                       # polar: atan2 is the same routine, codes identical too
                assert (pb.codes != pg.codes).sum().item() == 0, (d, pb.name)
            assert torch.equal(pb.side, pg.side), (d, pb.name)


def test_checksum_matches_host_formula(q):
    import torch
    rng = np.random.default_rng(9)
    w = rng.integers(0, 2 ** 32, size=100003, dtype=np.uint64)
    t = torch.from_numpy(w.astype(np.uint32).view(np.int32)).to(q.device)
    i = np.arange(w.size, dtype=np.uint64)
    expect = int(((w + np.uint64(1)) * (np.uint64(2) * i + np.uint64(1))).sum(dtype=np.uint64))
    assert q.checksum(t) == expect


def test_decode_and_attention_replay_from_a_cuda_graph(q):
    """The per-step launches are plain stream-ordered kernel launches: captured once into a CUDA
    graph and replayed, they give the same bytes as direct calls."""
    import torch
    from pitch_b200 import ChannelQuantConfig, KVCache, QuantConfig
    rng = np.random.default_rng(21)
    S, T, d = 4, 700, 64
    K, V = make_inputs(rng, S, T, d)
    cache = KVCache(S, d, 1024, ChannelQuantConfig(d, 4, 64), QuantConfig("turboQuant", d, 4), out_dtype="bfloat16", pitch=q)
    cache.prefill(torch.from_numpy(K).to(q.device), torch.from_numpy(V).to(q.device))
    Q = torch.from_numpy(rng.standard_normal((S, 7, d)).astype(np.float32)).to(q.device)
    ko, vo = cache.decode()
    att = cache.attend(Q)                                   # also sizes the scratch buffer outside the capture
    want = (ko.clone(), vo.clone(), att.clone())
    torch.cuda.synchronize()
    out = torch.empty_like(att)
    side = torch.cuda.Stream(q.device)
    side.wait_stream(torch.cuda.current_stream(q.device))
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            cache.decode()
            cache.attend(Q, out=out)
    for pl in cache.planes:
        pl.out.zero_()
    out.zero_()
    graph.replay()
    torch.cuda.synchronize()
    ko2, vo2 = (pl.out[:, :T] for pl in cache.planes)
    assert torch.equal(ko2, want[0]) and torch.equal(vo2, want[1]) and torch.equal(out, want[2])


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("n_planes", [1, 3, 4])
def test_descriptors_with_one_three_and_four_planes(q, n_planes, d):
    """The C descriptor takes 1...4 planes.  A launch over the planes of two caches at once (per-channel and
    TurboQuant planes mixed: the kernel that deals its items by drawn tickets, with a plane count that is
    not a power of two) must write what the caches' own two-plane launches write."""
    import ctypes as C

    import torch
    from pitch_b200 import ChannelQuantConfig, KVCache, QuantConfig, _native
    from pitch_b200.codec import stream_handle
    S, T = 5, 777
    rng = np.random.default_rng(77)
    caches = []
    for i in range(2):
        cache = KVCache(S, d, T, ChannelQuantConfig(d, 4, 64), QuantConfig("turboQuant", d, 4, seed=11 + i), out_dtype="bfloat16", pitch=q)
        K = torch.from_numpy((rng.standard_normal((S, T, d)) + 1.5).astype(np.float32)).to(q.device)
        V = torch.from_numpy(rng.standard_normal((S, T, d)).astype(np.float32)).to(q.device)
        cache.prefill(K, V)
        caches.append(cache)
    planes = [caches[0].planes[0], caches[0].planes[1], caches[1].planes[1], caches[1].planes[0]][:n_planes]
    if n_planes == 1:
        planes = [caches[0].planes[1]]
    want = []
    for cache in caches:
        cache.decode()
    torch.cuda.synchronize()
    for pl in planes:
        want.append(pl.out[:, :T].clone())
        pl.out.zero_()
    desc = _native.CacheDesc()
    desc.dim, desc.out_dtype, desc.segments, desc.tokens, desc.n_planes = d, 2, S, T, n_planes
    for i, pl in enumerate(planes):
        p = desc.planes[i]
        p.kind = pl.kind
        p.bits = pl.config.bits
        p.group_size = pl.config.group_size if pl.is_channel else 0
        p.seed = 0 if pl.is_channel else pl.config.seed
        for name in ("codes", "side", "out"):
            t = getattr(pl, name)
            setattr(p, name, t.data_ptr())
            setattr(p, name + "_seg_stride", t.stride(0) * t.element_size())
            setattr(p, name + "_bytes", t.numel() * t.element_size())
    lib = _native.lib()
    st = lib.pitch_enqueue_cache_decode(C.byref(desc), stream_handle(None, q.device))
    assert st == 0, lib.pitch_last_error()
    torch.cuda.synchronize()
    for pl, w in zip(planes, want):
        assert torch.equal(pl.out[:, :T].view(torch.int16), w.view(torch.int16)), pl.name
