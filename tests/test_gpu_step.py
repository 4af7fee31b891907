"""The one-launch generation step (``pitch_enqueue_cache_step`` / ``KVCache.step``): append one
token per segment and decode the whole cache in a single kernel.

The bar is equality: after every step the cache must hold exactly the codes, side information
and residual that ``append`` writes, and the decoded planes must equal ``decode``'s, bit for bit
(README.md:62-77 of the reference describes the two-call pattern the step replaces; the append
arithmetic is that of the bulk encoders, which the other suites pin against the specification).
The walks below cross item boundaries (2048 coordinates), per-channel group boundaries and start
from an empty cache; the last test checks the stepped cache against the CPU oracles directly."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def q():
    from pitch_b200 import PITCH
    return PITCH()


def _configs():
    from pitch_b200 import ChannelQuantConfig, QuantConfig
    t = lambda d, b: QuantConfig("turboQuant", d, b)
    c = lambda d, g: ChannelQuantConfig(d, 4, g)
    return {
        "cfg4 K per-channel G64 + V turbo b4, d64": (64, c(64, 64), t(64, 4)),
        "K per-channel G32 + V turbo b3, d64": (64, c(64, 32), t(64, 3)),
        "K per-channel G128 + V turbo b4, d64": (64, c(64, 128), t(64, 4)),
        "cfg5 K turbo + V turbo b4, d128": (128, t(128, 4), t(128, 4)),
        "cfg5 K turbo + V turbo b3, d128": (128, t(128, 3), t(128, 3)),
        "K per-channel G16 + V turbo b4, d128": (128, c(128, 16), t(128, 4)),
        "K per-channel G64 + V per-channel G32, d128": (128, c(128, 64), c(128, 32)),
        "K turbo + V turbo b3, d64": (64, t(64, 3), t(64, 3)),
    }


def _data(S, T, d, seed, dtype, dev):
    import torch
    rng = np.random.default_rng(seed)
    K = (rng.standard_normal((S, T, d)) + rng.normal(0, 2, (S, 1, d))).astype(np.float32)
    K[:, :, 3] *= 20.0                                                  # an outlier channel, as a biased key projection has
    V = (rng.standard_normal((S, T, d)) * np.exp(0.5 * rng.standard_normal((S, T, 1)))).astype(np.float32)
    V[0, T // 2] = 0.0                                                  # a zero vector on the way
    return torch.from_numpy(K).to(dev).to(dtype), torch.from_numpy(V).to(dev).to(dtype)


def _assert_same(a, b, what):
    import torch
    assert a.tokens == b.tokens, what
    for pa, pb in zip(a.planes, b.planes):
        assert torch.equal(pa.codes, pb.codes), f"{what}: {pa.name} codes differ at {a.tokens} tokens"
        assert torch.equal(pa.side.view(torch.int16), pb.side.view(torch.int16)), f"{what}: {pa.name} side information differs at {a.tokens} tokens"
        if pa.residual is not None:
            G = pa.config.group_size
            used = a.tokens - (a.tokens - 1) // G * G                    # rows of the newest group in use
            assert torch.equal(pa.residual[:, :used], pb.residual[:, :used]), f"{what}: {pa.name} residual rows differ"
            assert torch.equal(pa.residual[:, G:], pb.residual[:, G:]), f"{what}: {pa.name} running range differs"
        assert torch.equal(pa.out[:, :a.tokens].view(torch.int16 if pa.out.element_size() == 2 else torch.int32),
                           pb.out[:, :b.tokens].view(torch.int16 if pb.out.element_size() == 2 else torch.int32)), \
            f"{what}: decoded {pa.name} differ at {a.tokens} tokens"


@pytest.mark.parametrize("name", list(_configs()))
@pytest.mark.parametrize("out_dtype,in_dtype", [("bfloat16", "float32"), ("float16", "bfloat16"), ("float32", "float16")])
def test_step_equals_append_then_decode(q, name, out_dtype, in_dtype):
    import torch
    from pitch_b200 import KVCache
    d, kcfg, vcfg = _configs()[name]
    S, T0, steps = 5, 0, 150
    tin = getattr(torch, in_dtype)
    K, V = _data(S, T0 + steps, d, 11, tin, q.device)
    ref = KVCache(S, d, 256, kcfg, vcfg, out_dtype=out_dtype, pitch=q)
    new = KVCache(S, d, 256, kcfg, vcfg, out_dtype=out_dtype, pitch=q)
    assert new._fused, "these shapes are the ones the one-launch step covers"
    for t in range(T0, T0 + steps):
        k, v = K[:, t:t + 1].contiguous(), V[:, t:t + 1].contiguous()
        ref.append(k, v)
        ref.decode()
        ko, vo = new.step(k, v)
        assert ko.shape == (S, t + 1, d) and vo.shape == (S, t + 1, d)
        if t % 7 == 0 or t >= T0 + steps - 3 or (t + 1) % 16 == 0:
            torch.cuda.synchronize()
            _assert_same(ref, new, name)
    torch.cuda.synchronize()
    _assert_same(ref, new, name)


def test_step_after_prefill_mixes_with_append(q):
    """A stepped cache is interchangeable with an appended one at any moment: prefill, step, a
    multi-token append, step again."""
    import torch
    from pitch_b200 import ChannelQuantConfig, KVCache, QuantConfig
    S, d = 7, 64
    kcfg, vcfg = ChannelQuantConfig(d, 4, 64), QuantConfig("turboQuant", d, 4)
    K, V = _data(S, 400, d, 12, torch.float32, q.device)
    ref = KVCache(S, d, 512, kcfg, vcfg, pitch=q)
    new = KVCache(S, d, 512, kcfg, vcfg, pitch=q)
    ref.prefill(K[:, :203].contiguous(), V[:, :203].contiguous())
    new.prefill(K[:, :203].contiguous(), V[:, :203].contiguous())
    t = 203
    for piece in (1, 1, 1, -30, 1, 1, -23, 1, -64, 1, 1):               # negative: an append of that many tokens
        n = abs(piece)
        k, v = K[:, t:t + n].contiguous(), V[:, t:t + n].contiguous()
        ref.append(k, v)
        if piece > 0:
            new.step(k, v)
        else:
            new.append(k, v)
        t += n
    ref.decode()
    new.decode()
    torch.cuda.synchronize()
    _assert_same(ref, new, "mixed")


def test_step_falls_back_to_two_launches_off_the_fused_shapes(q):
    import torch
    from pitch_b200 import ChannelQuantConfig, KVCache, QuantConfig
    S, d = 3, 32
    kcfg, vcfg = ChannelQuantConfig(d, 3, 16), QuantConfig("polarQuant", d, 5)
    K, V = _data(S, 40, d, 13, torch.float32, q.device)
    ref = KVCache(S, d, 128, kcfg, vcfg, out_dtype="float32", pitch=q)
    new = KVCache(S, d, 128, kcfg, vcfg, out_dtype="float32", pitch=q)
    assert not new._fused
    for t in range(40):
        k, v = K[:, t:t + 1].contiguous(), V[:, t:t + 1].contiguous()
        ref.append(k, v)
        new.step(k, v)
    ref.decode()
    torch.cuda.synchronize()
    _assert_same(ref, new, "fallback")


def test_step_with_device_counter_replays_from_one_cuda_graph(q):
    """With the token count in device memory no launch parameter changes from step to step: one
    captured graph is replayed token after token, and a full cache refuses the step."""
    import torch
    from pitch_b200 import ChannelQuantConfig, InvalidInput, KVCache, QuantConfig
    S, d = 4, 64
    kcfg, vcfg = ChannelQuantConfig(d, 4, 64), QuantConfig("turboQuant", d, 4)
    K, V = _data(S, 256, d, 14, torch.float32, q.device)
    ref = KVCache(S, d, 256, kcfg, vcfg, pitch=q)
    new = KVCache(S, d, 256, kcfg, vcfg, pitch=q)
    ref.prefill(K[:, :100].contiguous(), V[:, :100].contiguous())
    new.prefill(K[:, :100].contiguous(), V[:, :100].contiguous())
    kbuf, vbuf = torch.empty((S, 1, d), device=q.device), torch.empty((S, 1, d), device=q.device)
    graph = new.capture_step(kbuf, vbuf)
    assert new.tokens == 100 and new.counter() == (100, 0)
    for t in range(100, 256):
        kbuf.copy_(K[:, t:t + 1])
        vbuf.copy_(V[:, t:t + 1])
        new.replay(graph)
        ref.append(K[:, t:t + 1].contiguous(), V[:, t:t + 1].contiguous())
        if t in (100, 127, 128, 191, 255):
            ref.decode()
            torch.cuda.synchronize()
            _assert_same(ref, new, "graph replay")
            assert new.counter() == (t + 1, 0)
    # the cache is full: the host refuses ...
    with pytest.raises(InvalidInput):
        new.replay(graph)
    # ... and so does the kernel when the graph is launched all the same: nothing changes, status is set
    before = [pl.codes.clone() for pl in new.planes]
    graph.replay()
    torch.cuda.synchronize()
    assert new.counter() == (256, 1)
    for pl, b in zip(new.planes, before):
        assert torch.equal(pl.codes, b)
    # direct calls keep working with the counter in place, and host-side changes reach it
    new.truncate(192)
    ref.truncate(192)
    assert new.counter() == (192, 0)
    for t in range(192, 200):
        k, v = K[:, t:t + 1].contiguous(), V[:, t:t + 1].contiguous()
        new.step(k, v)
        ref.append(k, v)
    ref.decode()
    torch.cuda.synchronize()
    _assert_same(ref, new, "direct calls with a counter")
    assert new.counter() == (200, 0)


def test_whole_generation_step_from_host_to_host_as_one_graph(q):
    """What a serving loop does per token, captured once: the new token comes from pinned host memory,
    the step runs, the newly decoded token of every plane and segment is gathered (its position read from
    the device-side counter) and goes back to pinned host memory."""
    import torch
    from pitch_b200 import ChannelQuantConfig, InvalidInput, KVCache, QuantConfig
    S, d = 6, 64
    kcfg, vcfg = ChannelQuantConfig(d, 4, 64), QuantConfig("turboQuant", d, 4)
    K, V = _data(S, 200, d, 15, torch.float32, q.device)
    Kh, Vh = K.cpu(), V.cpu()
    cache = KVCache(S, d, 256, kcfg, vcfg, pitch=q)
    with pytest.raises(InvalidInput):
        cache.newest()                                                   # nothing held yet
    cache.prefill(K[:, :70].contiguous(), V[:, :70].contiguous())
    # direct call, host-side count
    cache.decode()
    got = cache.newest()
    torch.cuda.synchronize()
    assert got.shape == (2, S, d) and got.dtype == torch.bfloat16
    assert torch.equal(got[0], cache.planes[0].out[:, 69]) and torch.equal(got[1], cache.planes[1].out[:, 69])
    with pytest.raises(InvalidInput):
        cache.newest(out=torch.empty((2, S, d), device=q.device))        # wrong dtype
    host_in = torch.empty((2, S, 1, d)).pin_memory()
    host_out = torch.empty((2, S, d), dtype=torch.bfloat16).pin_memory()
    dev_in = torch.empty((2, S, 1, d), device=q.device)
    dev_new = torch.empty((2, S, d), dtype=torch.bfloat16, device=q.device)

    def one_step():
        dev_in.copy_(host_in, non_blocking=True)
        cache.step(dev_in[0], dev_in[1], views=False)
        cache.newest(out=dev_new)
        host_out.copy_(dev_new, non_blocking=True)

    graph = cache.capture(one_step)
    assert cache.tokens == 70
    ref = KVCache(S, d, 256, kcfg, vcfg, pitch=q)
    ref.prefill(K[:, :70].contiguous(), V[:, :70].contiguous())
    for t in range(70, 200):
        host_in[0].copy_(Kh[:, t:t + 1])
        host_in[1].copy_(Vh[:, t:t + 1])
        cache.replay(graph)
        torch.cuda.synchronize()
        ref.append(K[:, t:t + 1].contiguous(), V[:, t:t + 1].contiguous())
        if t % 13 == 0 or t in (127, 128, 199):
            ko, vo = ref.decode()
            torch.cuda.synchronize()
            assert torch.equal(host_out[0], ko[:, t].cpu()), t
            assert torch.equal(host_out[1], vo[:, t].cpu()), t
    ref.decode()
    torch.cuda.synchronize()
    _assert_same(ref, cache, "host-to-host graph")
    with pytest.raises(InvalidInput):
        cache.capture(lambda: None)                                      # no step inside


def test_stepped_cache_against_the_cpu_oracles(q):
    """The stepped cache itself against the specification: per-channel keys bit-exact (codes,
    ranges, decoded values after rounding to bf16), TurboQuant value codes bit-exact against the
    float32 restatement of the kernel arithmetic, ties against the float64 specification counted."""
    import torch
    from oracle import kernel_f32, spec_np
    from pitch_b200 import ChannelQuantConfig, KVCache, QuantConfig
    S, d, T = 3, 64, 333
    rng = np.random.default_rng(15)
    K = (rng.standard_normal((S, T, d)) + rng.normal(0, 2, (S, 1, d))).astype(np.float32)
    V = rng.standard_normal((S, T, d)).astype(np.float32)
    Kd, Vd = torch.from_numpy(K).to(q.device), torch.from_numpy(V).to(q.device)
    cache = KVCache(S, d, 384, ChannelQuantConfig(d, 4, 64), QuantConfig("turboQuant", d, 4), pitch=q)
    cache.prefill(Kd[:, :100].contiguous(), Vd[:, :100].contiguous())
    for t in range(100, T):
        ko, vo = cache.step(Kd[:, t:t + 1].contiguous(), Vd[:, t:t + 1].contiguous())
    torch.cuda.synchronize()
    ties = 0
    for s in range(S):
        kc, kr = spec_np.channel_encode(K[s], 4, 64)
        assert cache.planes[0].codes[s, :T * 32].cpu().numpy().tobytes() == spec_np.pack_codes(kc, 4)
        groups = kr.shape[0]
        assert np.array_equal(cache.planes[0].side[s, :groups].cpu().numpy().view(np.uint16), kr.view(np.uint16))
        assert torch.equal(ko[s].cpu(), torch.from_numpy(spec_np.channel_decode(kc, kr, 4, 64)).bfloat16())
        vc, vn = kernel_f32.encode("turboQuant", V[s], 4)
        got = cache.planes[1].codes[s, :T * 32].cpu().numpy()
        assert got.tobytes() == vc.tobytes()
        assert np.array_equal(cache.planes[1].side[s, :T].cpu().numpy(), vn)
        sc, sn = spec_np.turbo_encode(V[s].astype(np.float64), 4)
        mine = spec_np.unpack_codes(got.tobytes(), T, d, 4)
        diff = mine != sc
        ties += int(diff.sum())
        assert np.all(np.abs(mine.astype(int) - sc.astype(int))[diff] == 1)
        ref = kernel_f32.decode("turboQuant", vc, vn, d, 4)
        rel = np.sqrt(((vo[s].cpu().float().numpy() - ref) ** 2).sum(1) / np.maximum((ref ** 2).sum(1), 1e-30)).max()
        assert rel < 5e-3                                                # bf16 rounding of the output
    assert ties <= 4, ties
    print(f"boundary ties against the float64 specification: {ties} of {S * T * d} codes")
