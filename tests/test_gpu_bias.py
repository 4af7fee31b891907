"""Exact key-bias removal around the codecs: the element-wise pass is bit-exact against the oracle's
float32 restatement of ``rotated_bias`` (reference/mechanism_eval.py:82-91); a cache built with
``key_bias`` decodes to what the specification gives for (keys - R_t b) plus R_t b, and a biased key
distribution that per-vector TurboQuant reconstructs poorly is reconstructed well again."""
import numpy as np
import pytest

from conftest import max_rel_l2
from oracle import spec_np

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def q():
    from pitch_b200 import PITCH
    return PITCH()


def rotary_tables(positions, dim, base=10000.0):
    """Full-width tables as a transformer applies them: frequencies repeated over both halves."""
    inv = base ** (-np.arange(0, dim, 2, dtype=np.float64) / dim)
    ang = np.arange(positions, dtype=np.float64)[:, None] * inv[None, :]
    ang = np.concatenate([ang, ang], axis=1)
    return np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)


@pytest.mark.parametrize("dtype", ["float32", "float16", "bfloat16"])
@pytest.mark.parametrize("S,count,dim,first", [(3, 77, 64, 5), (2, 1000, 128, 0), (1, 3, 8, 0), (4, 33, 1024, 2)])
def test_elementwise_pass_is_bit_exact(q, dtype, S, count, dim, first):
    import torch
    rng = np.random.default_rng(dim + count)
    tdt = getattr(torch, dtype)
    x = torch.from_numpy(rng.standard_normal((S, count, dim)).astype(np.float32)).to(tdt)
    bias = (3.0 * rng.standard_normal((S, dim))).astype(np.float32)
    cos, sin = rotary_tables(first + count + 4, dim)
    dev = q.device
    tb, tc, ts = (torch.from_numpy(a).to(dev) for a in (bias, cos, sin))
    for subtract in (True, False):
        data = x.to(dev).clone()
        q.enqueue_rope_bias(data, tb, tc, ts, first_position=first, subtract=subtract)
        x32 = x.float().numpy()
        ref = np.empty_like(x32)
        for s in range(S):
            rb = spec_np.rotated_bias(bias[s], cos, sin)[first:first + count]
            ref[s] = x32[s] - rb if subtract else x32[s] + rb
        assert torch.equal(data.cpu(), torch.from_numpy(ref).to(tdt)), (dtype, subtract)


def test_elementwise_pass_reproduces_the_reference_rotated_bias(q):
    """The kernel against the reference's own ``rotated_bias`` (reference/mechanism_eval.py:82-91,
    fixtures of tests/golden/make_bias_golden.py): adding R_t b to zeros must give the reference's
    R_t b bit for bit, and subtracting it again must give zeros."""
    import torch
    from conftest import Golden
    g = Golden("rotated_bias.npz")
    for c in g.cases:
        k = c["key"]
        dev = q.device
        bias, cos, sin = (torch.from_numpy(g[f"{k}/{n}"]).to(dev) for n in ("bias", "cos", "sin"))
        want = torch.from_numpy(g[f"{k}/rotated_bias"])
        data = torch.zeros((c["heads"], c["positions"], c["dim"]), device=dev)
        q.enqueue_rope_bias(data, bias, cos, sin, subtract=False)
        assert torch.equal(data.cpu(), want), k
        q.enqueue_rope_bias(data, bias, cos, sin, subtract=True)
        assert torch.count_nonzero(data) == 0, k


def test_strided_segments_leave_the_gap_untouched(q):
    import torch
    dev = q.device
    rng = np.random.default_rng(3)
    buf = torch.from_numpy(rng.standard_normal((2, 50, 64)).astype(np.float32)).to(dev)
    before = buf.clone()
    cos, sin = rotary_tables(64, 64)
    q.enqueue_rope_bias(buf[:, :20], torch.ones((2, 64), device=dev), torch.from_numpy(cos).to(dev),
                        torch.from_numpy(sin).to(dev), subtract=False)
    assert torch.equal(buf[:, 20:], before[:, 20:]) and not torch.equal(buf[:, :20], before[:, :20])


def test_cache_with_key_bias(q):
    import torch
    from pitch_b200 import KVCache, QuantConfig
    rng = np.random.default_rng(9)
    S, T, d = 3, 300, 64
    dev = q.device
    cos, sin = rotary_tables(384, d)
    bias = (8.0 * rng.standard_normal((S, d))).astype(np.float32)          # a bias well above the keys' spread
    content = rng.standard_normal((S, T, d)).astype(np.float32)
    K = np.stack([content[s] + spec_np.rotated_bias(bias[s], cos, sin)[:T] for s in range(S)]).astype(np.float32)
    V = rng.standard_normal((S, T, d)).astype(np.float32)
    cfg = QuantConfig("turboQuant", d, 4)
    tK, tV = torch.from_numpy(K).to(dev), torch.from_numpy(V).to(dev)
    kb = tuple(torch.from_numpy(a).to(dev) for a in (bias, cos, sin))

    plain = KVCache(S, d, T, cfg, cfg, out_dtype="float32", pitch=q)
    plain.prefill(tK, tV)
    k_plain = plain.decode()[0].cpu().numpy()

    cache = KVCache(S, d, T, cfg, cfg, out_dtype="float32", pitch=q, key_bias=kb)
    cache.prefill(tK[:, :200].contiguous(), tV[:, :200].contiguous())
    for t in range(200, T):                                                # then token by token
        cache.append(tK[:, t:t + 1].contiguous(), tV[:, t:t + 1].contiguous())
    k_hat = cache.decode()[0].cpu().numpy()
    for s in range(S):
        rb = spec_np.rotated_bias(bias[s], cos, sin)[:T]
        codes, norms = spec_np.turbo_encode((K[s] - rb).astype(np.float32), 4)
        ref = spec_np.turbo_decode(codes, norms, 4) + rb
        assert max_rel_l2(k_hat[s], ref) < 1e-5, s
        # what the fix is for: the content under the bias is reconstructed far better
        err_fix = np.linalg.norm(k_hat[s] - K[s]) / np.linalg.norm(content[s])
        err_plain = np.linalg.norm(k_plain[s] - K[s]) / np.linalg.norm(content[s])
        assert err_fix < 0.15 and err_plain > 4 * err_fix, (err_fix, err_plain)
    # values are untouched by the option
    assert torch.equal(cache.decode()[1], plain.decode()[1])


def _bias_pair(q, S, d, cap, kcfg, vcfg, out_dtype, seed):
    """Two caches with the same key bias: one handles it inside the decode / step launch, the
    other with separate element-wise launches (the arrangement the other tests pin to the oracle)."""
    import torch
    from pitch_b200 import KVCache
    rng = np.random.default_rng(seed)
    cos, sin = rotary_tables(cap, d, base=1000000.0)
    kb = tuple(torch.from_numpy(a).to(q.device) for a in ((6.0 * rng.standard_normal((S, d))).astype(np.float32), cos, sin))
    fused = KVCache(S, d, cap, kcfg, vcfg, out_dtype=out_dtype, pitch=q, key_bias=kb)
    split = KVCache(S, d, cap, kcfg, vcfg, out_dtype=out_dtype, pitch=q, key_bias=kb, fuse_key_bias=False)
    assert fused._fuse_bias and not split._fuse_bias
    return fused, split, rng


def _same_cache(a, b, what):
    import torch
    assert a.tokens == b.tokens
    for pa, pb in zip(a.planes, b.planes):
        assert torch.equal(pa.codes, pb.codes), f"{what}: {pa.name} codes at {a.tokens} tokens"
        assert torch.equal(pa.side.view(torch.int16), pb.side.view(torch.int16)), f"{what}: {pa.name} side information"
        view = torch.int16 if pa.out.element_size() == 2 else torch.int32
        diff = pa.out[:, :a.tokens].view(view) != pb.out[:, :b.tokens].view(view)
        assert not bool(diff.any()), f"{what}: decoded {pa.name} differ at {int(diff.sum())} places, {a.tokens} tokens"


@pytest.mark.parametrize("out_dtype,in_dtype", [("bfloat16", "float32"), ("float16", "bfloat16"), ("float32", "float16")])
@pytest.mark.parametrize("shape", ["turbo64", "turbo128b3", "channel64", "channel128"])
def test_key_bias_inside_the_launch_equals_separate_passes(q, shape, out_dtype, in_dtype):
    """README.md:100 of the reference asks for the bias removal inside the kernels: decode and step
    with the option must give, bit for bit, what decode / append give with the bias handled by
    separate passes before and after."""
    import torch
    from pitch_b200 import ChannelQuantConfig, QuantConfig
    d, kcfg, vcfg = {"turbo64": (64, QuantConfig("turboQuant", 64, 4), QuantConfig("turboQuant", 64, 4)),
                     "turbo128b3": (128, QuantConfig("turboQuant", 128, 3), QuantConfig("turboQuant", 128, 3)),
                     "channel64": (64, ChannelQuantConfig(64, 4, 64), QuantConfig("turboQuant", 64, 4)),
                     "channel128": (128, ChannelQuantConfig(128, 4, 32), QuantConfig("turboQuant", 128, 3))}[shape]
    S, T0, steps, cap = 21, 77, 100, 256                     # 42 (segment, plane) pairs: more than the 16 warps of a CTA
    fused, split, rng = _bias_pair(q, S, d, cap, kcfg, vcfg, out_dtype, 31)
    tin = getattr(torch, in_dtype)
    K = torch.from_numpy((rng.standard_normal((S, T0 + steps, d)) * 2 + 5).astype(np.float32)).to(q.device).to(tin)
    V = torch.from_numpy(rng.standard_normal((S, T0 + steps, d)).astype(np.float32)).to(q.device).to(tin)
    for c in (fused, split):
        c.prefill(K[:, :T0].contiguous(), V[:, :T0].contiguous())
        c.decode()
    torch.cuda.synchronize()
    _same_cache(fused, split, shape + " decode")
    for t in range(T0, T0 + steps):
        k, v = K[:, t:t + 1].contiguous(), V[:, t:t + 1].contiguous()
        fused.step(k, v)
        split.step(k, v)                                     # append (bias taken off a copy) + decode + separate pass
        if t % 9 == 0 or t > T0 + steps - 3:
            torch.cuda.synchronize()
            _same_cache(fused, split, shape + " step")
    torch.cuda.synchronize()
    _same_cache(fused, split, shape + " step")


def test_key_bias_inside_the_launch_over_many_token_blocks(q):
    """More token blocks than multiprocessors: every CTA walks several blocks and the table rows of
    the next block arrive while the current one is decoded."""
    import torch
    from pitch_b200 import ChannelQuantConfig, QuantConfig
    S, d, T = 3, 64, 9000
    fused, split, rng = _bias_pair(q, S, d, 9216, ChannelQuantConfig(d, 4, 64), QuantConfig("turboQuant", d, 4), "bfloat16", 32)
    K = torch.from_numpy((rng.standard_normal((S, T + 3, d)) + 4).astype(np.float32)).to(q.device)
    V = torch.from_numpy(rng.standard_normal((S, T + 3, d)).astype(np.float32)).to(q.device)
    for c in (fused, split):
        c.prefill(K[:, :T].contiguous(), V[:, :T].contiguous())
    for t in range(T, T + 3):
        fused.step(K[:, t:t + 1].contiguous(), V[:, t:t + 1].contiguous())
        split.step(K[:, t:t + 1].contiguous(), V[:, t:t + 1].contiguous())
    torch.cuda.synchronize()
    _same_cache(fused, split, "many blocks")
    # float32 output takes the single-buffer arrangement of the table rows
    f32, s32, rng = _bias_pair(q, 2, d, 9216, QuantConfig("turboQuant", d, 4), QuantConfig("turboQuant", d, 4), "float32", 33)
    for c in (f32, s32):
        c.prefill(K[:2, :T].contiguous(), V[:2, :T].contiguous())
        c.decode()
    torch.cuda.synchronize()
    _same_cache(f32, s32, "many blocks, float32")


def test_bad_arguments(q):
    import torch
    from pitch_b200.errors import InvalidDimension, InvalidInput
    dev = q.device
    cos, sin = (torch.from_numpy(a).to(dev) for a in rotary_tables(16, 64))
    data = torch.zeros((1, 20, 64), device=dev)
    with pytest.raises(InvalidInput):                                       # positions beyond the tables
        q.enqueue_rope_bias(data, torch.zeros((1, 64), device=dev), cos, sin, subtract=True)
    with pytest.raises(InvalidInput):
        q.enqueue_rope_bias(data[:, :4], torch.zeros((2, 64), device=dev), cos, sin, subtract=True)
    c12, s12 = (torch.from_numpy(a).to(dev) for a in rotary_tables(16, 12))
    with pytest.raises(InvalidDimension):
        q.enqueue_rope_bias(torch.zeros((1, 4, 12), device=dev), torch.zeros((1, 12), device=dev), c12, s12, subtract=True)
