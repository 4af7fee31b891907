"""Attention computed straight from the compressed cache against attention over the cache as the
specification port decodes it (float64), and against torch attention over the GPU-decoded float32
cache at a full-length context.  Tolerance: 2e-5 relative L2 per (segment, query) row -- float32
accumulation over up to 32,768 tokens in a different order, base-2 exponentials."""
import numpy as np
import pytest

from oracle import spec_np

pytestmark = pytest.mark.gpu

TOL = 2e-5


@pytest.fixture(scope="module")
def q():
    from pitch_b200 import PITCH
    return PITCH()


def build_cache(q, S, T, G, seed, capacity=None):
    import torch
    from pitch_b200 import ChannelQuantConfig, KVCache, QuantConfig
    rng = np.random.default_rng(seed)
    d = 64
    K = (rng.standard_normal((S, T, d)) + rng.normal(0.0, 2.0, size=(S, 1, d))).astype(np.float32)
    V = (rng.standard_normal((S, T, d)) * np.exp(0.5 * rng.standard_normal((S, T, 1)))).astype(np.float32)
    cache = KVCache(S, d, capacity or T, ChannelQuantConfig(d, 4, G), QuantConfig("turboQuant", d, 4),
                    out_dtype="float32", pitch=q)
    cache.prefill(torch.from_numpy(K).to(q.device), torch.from_numpy(V).to(q.device))
    assert cache.tokens == T
    return cache, rng


def spec_decoded(cache, s):
    """Keys and values of segment s as the specification decodes the stored bytes (float64)."""
    T, d = cache.tokens, cache.dim
    pk, pv = cache.planes
    G = pk.config.group_size
    groups = -(-T // G)
    kc = spec_np.unpack_codes(pk.codes[s, :T * 32].cpu().numpy().tobytes(), T, d, 4)
    kr = pk.side[s, :groups].cpu().numpy()                       # [groups, 2, d] float16
    K = spec_np.channel_decode(kc, kr, 4, G).astype(np.float64)
    vc = pv.codes[s, :T * 32].cpu().numpy()
    vn = pv.side[s, :T].cpu().numpy().astype(np.float64)
    V = spec_np.turbo_decode(spec_np.unpack_codes(vc.tobytes(), T, d, 4), vn, 4)
    return K, np.asarray(V, dtype=np.float64)


def attention64(Q, K, V, scale):
    s = (Q @ K.T) * scale
    s -= s.max(axis=1, keepdims=True)
    p = np.exp(s)
    return (p / p.sum(axis=1, keepdims=True)) @ V


def rows_rel_l2(got, ref):
    return float(np.max(np.linalg.norm(got - ref, axis=-1) / np.linalg.norm(ref, axis=-1)))


@pytest.mark.parametrize("S,T,R,G,scale", [(3, 333, 7, 64, None), (2, 5000, 1, 32, None), (1, 31, 8, 64, None),
                                            (2, 2048 + 17, 4, 128, 0.5), (5, 1024, 2, 64, None), (1, 1, 3, 64, None),
                                            (2, 9000, 5, 64, 1.0), (1, 300, 6, 96, None)])
def test_matches_attention_over_spec_decoded_cache(q, S, T, R, G, scale):
    import torch
    cache, rng = build_cache(q, S, T, G, seed=100 + T)
    Q = rng.standard_normal((S, R, 64)).astype(np.float32)
    out = cache.attend(torch.from_numpy(Q).to(q.device), scale=scale)
    torch.cuda.synchronize()
    got = out.cpu().numpy().astype(np.float64)
    assert np.isfinite(got).all()
    sc = 64 ** -0.5 if scale is None else scale
    for s in range(S):
        K, V = spec_decoded(cache, s)
        ref = attention64(Q[s].astype(np.float64), K, V, sc)
        assert rows_rel_l2(got[s], ref) < TOL, (s, rows_rel_l2(got[s], ref))


@pytest.mark.parametrize("S,T,R,G", [(3, 333, 7, 64), (2, 9000, 5, 64), (1, 31, 8, 64), (2, 2048 + 17, 4, 128)])
def test_bf16_operand_mode_is_as_accurate_as_attention_over_the_bf16_cache(q, S, T, R, G):
    """``precision="bfloat16"``: operands as a bf16 pipeline has them.  Its error against float64
    attention over the specification-decoded cache must stay within a few bf16 roundings (8e-3), and must
    not exceed (by more than a small factor) the error of what it replaces: torch attention over
    the cache decoded to bf16."""
    import torch
    cache, rng = build_cache(q, S, T, G, seed=300 + T)
    Q = rng.standard_normal((S, R, 64)).astype(np.float32)
    Qd = torch.from_numpy(Q).to(q.device)
    fast = cache.attend(Qd, precision="bfloat16").cpu().numpy().astype(np.float64)
    exact = cache.attend(Qd).cpu().numpy().astype(np.float64)
    ko, vo = cache.decode()
    sdpa = torch.nn.functional.scaled_dot_product_attention(Qd.bfloat16().unsqueeze(0), ko.bfloat16().unsqueeze(0),
                                                            vo.bfloat16().unsqueeze(0))[0].float().cpu().numpy().astype(np.float64)
    for s in range(S):
        K, V = spec_decoded(cache, s)
        ref = attention64(Q[s].astype(np.float64), K, V, 64 ** -0.5)
        e_fast, e_exact, e_sdpa = rows_rel_l2(fast[s], ref), rows_rel_l2(exact[s], ref), rows_rel_l2(sdpa[s], ref)
        assert e_exact < TOL
        assert e_fast < 8e-3, (s, e_fast)
        assert e_fast < 1.5 * e_sdpa + 1e-3, (s, e_fast, e_sdpa)
    with pytest.raises(Exception):
        cache.attend(Qd, precision="float8")


def build_turbo_cache(q, S, T, seed, d=64, bits=4):
    """Keys and values both TurboQuant (with different rotation seeds)."""
    import torch
    from pitch_b200 import KVCache, QuantConfig
    rng = np.random.default_rng(seed)
    K = (rng.standard_normal((S, T, d)) * np.exp(0.4 * rng.standard_normal((S, T, 1)))).astype(np.float32)
    V = (rng.standard_normal((S, T, d)) * np.exp(0.5 * rng.standard_normal((S, T, 1)))).astype(np.float32)
    cache = KVCache(S, d, T, QuantConfig("turboQuant", d, bits, seed=777), QuantConfig("turboQuant", d, bits), out_dtype="float32", pitch=q)
    cache.prefill(torch.from_numpy(K).to(q.device), torch.from_numpy(V).to(q.device))
    return cache, rng


def spec_decoded_turbo(cache, s):
    T, d = cache.tokens, cache.dim
    out = []
    for pl in cache.planes:
        b = pl.config.bits
        c = pl.codes[s, :T * (d * b // 8)].cpu().numpy()
        n = pl.side[s, :T].cpu().numpy().astype(np.float64)
        out.append(np.asarray(spec_np.turbo_decode(spec_np.unpack_codes(c.tobytes(), T, d, b), n, b, pl.config.seed), dtype=np.float64))
    return out


def bf16_pipeline(cache, Qd, scale):
    """What ``precision="bfloat16"`` stands in for: torch attention in bf16 over the cache decoded to bf16."""
    import torch
    ko, vo = cache.decode()
    out = torch.nn.functional.scaled_dot_product_attention(Qd.bfloat16().unsqueeze(0), ko.bfloat16().unsqueeze(0),
                                                           vo.bfloat16().unsqueeze(0), scale=scale)
    return out[0].float().cpu().numpy().astype(np.float64)


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("S,T,R,scale", [(3, 333, 7, None), (2, 5000, 1, None), (1, 31, 8, None), (2, 9000, 5, 1.0), (1, 1, 3, None)])
def test_turboquant_keys_match_attention_over_spec_decoded_cache(q, S, T, R, scale, d):
    """A cache whose keys are TurboQuant too (dimension 64, and 128 as in a Llama-3-70B-shaped cache):
    the query is rotated once instead of un-rotating every key."""
    import torch
    cache, rng = build_turbo_cache(q, S, T, seed=400 + T, d=d)
    Q = rng.standard_normal((S, R, d)).astype(np.float32)
    Qd = torch.from_numpy(Q).to(q.device)
    got = cache.attend(Qd, scale=scale).cpu().numpy().astype(np.float64)
    fast = cache.attend(Qd, scale=scale, precision="bfloat16").cpu().numpy().astype(np.float64)
    assert np.isfinite(got).all() and np.isfinite(fast).all()
    sc = d ** -0.5 if scale is None else scale
    sdpa = bf16_pipeline(cache, Qd, sc)
    for s in range(S):
        K, V = spec_decoded_turbo(cache, s)
        ref = attention64(Q[s].astype(np.float64), K, V, sc)
        # centroids enter the score product as two bf16 parts (2^-17): a softmax scale of 1.0 (scores eight
        # times larger than usual) carries that into the weights
        assert rows_rel_l2(got[s], ref) < (TOL if scale is None else 1e-4), (s, rows_rel_l2(got[s], ref))
        # bf16 operands (centroids and weights each in one bf16): the error class of torch attention over the
        # cache decoded to bf16 (a few bf16 roundings; observed up to twice its error on short contexts)
        e_fast, e_sdpa = rows_rel_l2(fast[s], ref), rows_rel_l2(sdpa[s], ref)
        assert e_fast < 2.5 * e_sdpa + 2e-3, (s, e_fast, e_sdpa)


@pytest.mark.parametrize("S,T,R,scale", [(3, 333, 7, None), (2, 5000, 1, None), (1, 31, 8, None), (2, 9000, 5, 1.0), (1, 1, 3, None),
                                          (1, 32768, 8, None)])
def test_three_bit_cache_at_dimension_128(q, S, T, R, scale):
    """The 3-bit Llama-3-70B-shaped cache: codes of a vector are 48 bytes, a pair of codes straddles bytes."""
    import torch
    cache, rng = build_turbo_cache(q, S, T, seed=500 + T, d=128, bits=3)
    Q = rng.standard_normal((S, R, 128)).astype(np.float32)
    Qd = torch.from_numpy(Q).to(q.device)
    got = cache.attend(Qd, scale=scale).cpu().numpy().astype(np.float64)
    fast = cache.attend(Qd, scale=scale, precision="bfloat16").cpu().numpy().astype(np.float64)
    assert np.isfinite(got).all() and np.isfinite(fast).all()
    sc = 128 ** -0.5 if scale is None else scale
    sdpa = bf16_pipeline(cache, Qd, sc)
    for s in range(S):
        K, V = spec_decoded_turbo(cache, s)
        ref = attention64(Q[s].astype(np.float64), K, V, sc)
        assert rows_rel_l2(got[s], ref) < (TOL if scale is None else 1e-4), (s, rows_rel_l2(got[s], ref))
        e_fast, e_sdpa = rows_rel_l2(fast[s], ref), rows_rel_l2(sdpa[s], ref)
        assert e_fast < 2.5 * e_sdpa + 2e-3, (s, e_fast, e_sdpa)


def test_grows_with_the_cache(q):
    """Attention after every append of a growing cache (partial groups, tiles and slices)."""
    import torch
    from pitch_b200 import ChannelQuantConfig, KVCache, QuantConfig
    rng = np.random.default_rng(7)
    S, d, R = 2, 64, 7
    cache = KVCache(S, d, 256, ChannelQuantConfig(d, 4, 64), QuantConfig("turboQuant", d, 4), out_dtype="float32", pitch=q)
    Q = torch.from_numpy(rng.standard_normal((S, R, d)).astype(np.float32)).to(q.device)
    for step in range(70):
        k = torch.from_numpy(rng.standard_normal((S, 1, d)).astype(np.float32) + 1.0).to(q.device)
        v = torch.from_numpy(rng.standard_normal((S, 1, d)).astype(np.float32)).to(q.device)
        cache.append(k, v)
        if step % 9 and step < 64:
            continue
        out = cache.attend(Q).cpu().numpy().astype(np.float64)
        for s in range(S):
            K, V = spec_decoded(cache, s)
            ref = attention64(Q[s].cpu().numpy().astype(np.float64), K, V, d ** -0.5)
            assert rows_rel_l2(out[s], ref) < TOL, (step, s)


def test_full_context_against_decoded_cache(q):
    """32,768 tokens, 7 query heads per KV head (the benchmark's shape, fewer segments): fused
    attention against float64 attention over the float32 cache the decode kernel writes."""
    import torch
    S, T, R = 4, 32768, 7
    cache, rng = build_cache(q, S, T, 64, seed=11)
    Q = torch.from_numpy(rng.standard_normal((S, R, 64)).astype(np.float32)).to(q.device)
    out = cache.attend(Q)
    ko, vo = cache.decode()
    s = torch.einsum("srd,std->srt", Q.double(), ko.double()) * 64 ** -0.5
    ref = torch.einsum("srt,std->srd", torch.softmax(s, dim=-1), vo.double())
    err = (torch.linalg.norm(out.double() - ref, dim=-1) / torch.linalg.norm(ref, dim=-1)).max().item()
    assert err < TOL, err
    # a sharp softmax (large scale): still finite and close
    out2 = cache.attend(Q, scale=4.0)
    ref2 = torch.einsum("srt,std->srd", torch.softmax(s * (4.0 / 64 ** -0.5), dim=-1), vo.double())
    err2 = (torch.linalg.norm(out2.double() - ref2, dim=-1) / torch.linalg.norm(ref2, dim=-1)).max().item()
    assert torch.isfinite(out2).all() and err2 < 1e-4, err2


def test_two_calls_share_the_workspace(q):
    import torch
    cache, rng = build_cache(q, 3, 700, 64, seed=12)
    Q1 = torch.from_numpy(rng.standard_normal((3, 7, 64)).astype(np.float32)).to(q.device)
    Q2 = torch.from_numpy(rng.standard_normal((3, 2, 64)).astype(np.float32)).to(q.device)
    a1 = cache.attend(Q1).clone()
    a2 = cache.attend(Q2).clone()
    b1 = cache.attend(Q1)
    assert torch.equal(a1, b1)                                     # deterministic, scratch content irrelevant
    assert torch.allclose(a2, cache.attend(Q1[:, :2].contiguous() * 0 + Q2), rtol=0, atol=0)


def test_unsupported_shapes_are_refused(q):
    import torch
    from pitch_b200 import ChannelQuantConfig, KVCache, QuantConfig
    from pitch_b200.errors import InvalidInput
    dev = q.device
    cases = [(64, ChannelQuantConfig(64, 4, 48), QuantConfig("turboQuant", 64, 4)),      # group not a multiple of 32
             (64, ChannelQuantConfig(64, 2, 64), QuantConfig("turboQuant", 64, 4)),      # 2-bit keys
             (64, ChannelQuantConfig(64, 4, 64), QuantConfig("polarQuant", 64, 4)),      # PolarQuant values
             (128, ChannelQuantConfig(128, 4, 64), QuantConfig("turboQuant", 128, 4)),   # per-channel keys at dim 128
             (64, QuantConfig("turboQuant", 64, 3), QuantConfig("turboQuant", 64, 3)),   # 3 bits at dim 64
             (128, QuantConfig("turboQuant", 128, 4), QuantConfig("turboQuant", 128, 3))]  # keys and values of different widths
    for d, kc, vc in cases:
        cache = KVCache(2, d, 128, kc, vc, pitch=q)
        x = torch.randn((2, 128, d), device=dev)
        cache.prefill(x, x)
        with pytest.raises(InvalidInput):
            cache.attend(torch.randn((2, 4, d), device=dev))
    cache, _ = build_cache(q, 2, 100, 64, seed=1)
    with pytest.raises(InvalidInput):
        cache.attend(torch.randn((2, 9, 64), device=dev))               # more than 8 queries
    with pytest.raises(InvalidInput):
        cache.attend(torch.randn((2, 4, 64), device=dev), scale=0.0)
    with pytest.raises(InvalidInput):
        cache.attend(torch.randn((2, 4, 64), device=dev, dtype=torch.float16))
    empty = KVCache(2, 64, 128, ChannelQuantConfig(64, 4, 64), QuantConfig("turboQuant", 64, 4), pitch=q)
    with pytest.raises(InvalidInput):
        empty.attend(torch.randn((2, 4, 64), device=dev))
