"""The allocation-free append entry point (collected last on purpose: a run that stops at the
first failure has then already run every other test).

Some hosts cannot give the library a residual buffer: a serving loop that forbids device
allocations once generation has started, or a foreign-function caller that owns nothing but the
cache buffers it passes in.  ``pitch_enqueue_cache_append_noalloc`` keeps the per-channel
residual in a fixed array inside the library instead.  It must write exactly what
``pitch_enqueue_cache_append`` writes - codes, norms and fp16 ranges bit for bit (integer and
fp16 data: the tolerance of the other cache tests is equality) - on consecutive calls, which is
what shows that the state carried in the built-in array from one call to the next is right.
"""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _call_noalloc(cache, keys, values):
    """One call of the C entry point, built by hand: (descriptor, sources without residual)."""
    from pitch_b200 import _native
    from pitch_b200.codec import native_dtype, stream_handle
    desc = cache._desc(cache.tokens)
    src = (_native.AppendSrc * 4)()
    for i, x in enumerate((keys, values)):
        src[i].input = x.data_ptr()
        src[i].input_seg_stride = x.stride(0) * x.element_size()
        src[i].input_bytes = x.numel() * x.element_size()
    st = _native.lib().pitch_enqueue_cache_append_noalloc(ctypes.byref(desc), src, native_dtype(keys.dtype),
                                                          int(keys.shape[1]), stream_handle(None, cache.device))
    return st


def _same(a, b):
    import torch
    for pa, pb in zip(a.planes, b.planes):
        if not (torch.equal(pa.codes, pb.codes) and torch.equal(pa.side, pb.side)):
            return False
    return True


def test_noalloc_append_matches_append_on_consecutive_calls():
    import torch
    from pitch_b200 import ChannelQuantConfig, KVCache, PITCH, QuantConfig, _native
    q = PITCH()
    rng = np.random.default_rng(99)
    S, d, G = 6, 64, 64
    K = (rng.standard_normal((S, 200, d)) + rng.normal(0, 2, (S, 1, d))).astype(np.float32)
    V = rng.standard_normal((S, 200, d)).astype(np.float32)
    Kd, Vd = torch.from_numpy(K).to(q.device), torch.from_numpy(V).to(q.device)
    kcfg, vcfg = ChannelQuantConfig(d, 4, G), QuantConfig("turboQuant", d, 4)
    ref = KVCache(S, d, 256, kcfg, vcfg, pitch=q)        # existing entry point, caller-owned residual
    new = KVCache(S, d, 256, kcfg, vcfg, pitch=q)        # allocation-free entry point
    ref.prefill(Kd[:, :128].contiguous(), Vd[:, :128].contiguous())     # two whole groups: both start on a boundary
    new.prefill(Kd[:, :128].contiguous(), Vd[:, :128].contiguous())
    t = 128
    for n_new in (1, 1, 5, 1, 56, 1, 7):                 # consecutive calls; the 56 completes the group, then a new one
        k, v = Kd[:, t:t + n_new].contiguous(), Vd[:, t:t + n_new].contiguous()
        ref.append(k, v)
        assert _call_noalloc(new, k, v) == 0, _native.lib().pitch_last_error()
        new.tokens += n_new
        t += n_new
        torch.cuda.synchronize()
        assert _same(ref, new), f"differs after the call that brought the cache to {t} tokens"
    # the decoded caches agree too
    ra, rb = ref.decode(), new.decode()
    assert torch.equal(ra[0], rb[0]) and torch.equal(ra[1], rb[1])
    # the caller's own residual tensors were never touched by the allocation-free path
    assert torch.count_nonzero(new.planes[0].residual) == 0


def test_noalloc_append_python_helper_and_limits():
    import torch
    from pitch_b200 import ChannelQuantConfig, KVCache, PITCH, PITCHError, QuantConfig, _native
    from pitch_b200.noalloc import RESIDUAL_FLOATS, append_noalloc
    q = PITCH()
    rng = np.random.default_rng(100)
    S, d = 3, 32
    kcfg, vcfg = ChannelQuantConfig(d, 3, 16), QuantConfig("polarQuant", d, 5)
    X = torch.from_numpy(rng.standard_normal((S, 40, d)).astype(np.float32)).to(q.device)
    a = KVCache(S, d, 128, kcfg, vcfg, pitch=q)
    b = KVCache(S, d, 128, kcfg, vcfg, pitch=q)
    a.append(X, X)
    append_noalloc(b, X[:, :9].contiguous(), X[:, :9].contiguous())      # split differently on purpose
    append_noalloc(b, X[:, 9:].contiguous(), X[:, 9:].contiguous())
    torch.cuda.synchronize()
    assert a.tokens == b.tokens == 40 and _same(a, b)
    # another cache may not take over in the middle of a group ...
    c = KVCache(S, d, 128, kcfg, vcfg, pitch=q)
    c.append(X[:, :5].contiguous(), X[:, :5].contiguous())
    assert _call_noalloc(c, X[:, 5:6].contiguous(), X[:, 5:6].contiguous()) == 4          # configuration mismatch
    assert b"one cache at a time" in _native.lib().pitch_last_error()
    # ... and a cache that does not fit the built-in array is refused with a clear message
    big_groups = 65536
    segs = RESIDUAL_FLOATS // ((big_groups + 2) * d) + 1
    big = KVCache(segs, d, 128, ChannelQuantConfig(d, 4, big_groups), vcfg, pitch=q)
    Y = torch.zeros((segs, 1, d), device=q.device)
    with pytest.raises(PITCHError, match="built-in buffer holds"):
        append_noalloc(big, Y, Y)


def test_noalloc_append_removes_the_key_bias_like_append():
    """A cache built with ``key_bias`` takes the rotated bias off the new keys before encoding them;
    the allocation-free helper must do the same, or ``decode`` would add back a bias that was never
    removed.  Codes, norms and ranges must equal those of ``KVCache.append``, and so must the decoded keys."""
    import torch
    from pitch_b200 import ChannelQuantConfig, KVCache, PITCH, QuantConfig
    from pitch_b200.noalloc import append_noalloc
    q = PITCH()
    rng = np.random.default_rng(101)
    S, d, T = 4, 64, 150
    inv = 10000.0 ** (-np.arange(0, d, 2, dtype=np.float64) / d)
    ang = np.arange(256, dtype=np.float64)[:, None] * inv[None, :]
    ang = np.concatenate([ang, ang], axis=1)
    kb = tuple(torch.from_numpy(a).to(q.device) for a in ((5.0 * rng.standard_normal((S, d))).astype(np.float32),
                                                          np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)))
    K = torch.from_numpy((rng.standard_normal((S, T, d)) + 3).astype(np.float32)).to(q.device)
    V = torch.from_numpy(rng.standard_normal((S, T, d)).astype(np.float32)).to(q.device)
    for kcfg in (ChannelQuantConfig(d, 4, 64), QuantConfig("turboQuant", d, 4)):
        ref = KVCache(S, d, 256, kcfg, QuantConfig("turboQuant", d, 4), pitch=q, key_bias=kb)
        new = KVCache(S, d, 256, kcfg, QuantConfig("turboQuant", d, 4), pitch=q, key_bias=kb)
        t = 0
        for n_new in (64, 1, 30, 1, 33, 21):
            k, v = K[:, t:t + n_new].contiguous(), V[:, t:t + n_new].contiguous()
            ref.append(k, v)
            append_noalloc(new, k, v)
            t += n_new
        torch.cuda.synchronize()
        assert ref.tokens == new.tokens == T and _same(ref, new)
        ra, rb = ref.decode(), new.decode()
        assert torch.equal(ra[0], rb[0]) and torch.equal(ra[1], rb[1])
