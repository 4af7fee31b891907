"""Appending to a ``KVCache`` through the allocation-free entry point.

``append_noalloc`` does what ``KVCache.append`` does (key-bias removal included), but the float32 residual of the per-channel
planes (the newest, still growing group of every segment) is kept in a fixed array inside the
native library instead of a tensor the caller allocated.  It exists for hosts that are not
allowed, or not able, to allocate device memory: a serving loop whose device memory is one
pre-sized arena with driver allocations forbidden once generation starts, or a foreign-function
caller that owns only the cache buffers it passes in.

Limits (see ``pitch_enqueue_cache_append_noalloc`` in ``include/pitch_b200.h``): at most
``RESIDUAL_FLOATS`` floats, counted as ``segments * (group_size + 2) * dim`` per per-channel
plane; one cache per GPU at a time, switched only on a group boundary; calls on one GPU must be
stream-ordered, overlapping calls race on the shared array.  The first call on a GPU looks the
array up once and should come before any stream capture.
"""
from __future__ import annotations

import ctypes

from . import _native
from .cache import KVCache
from .codec import native_dtype, stream_handle
from .errors import InvalidInput

RESIDUAL_FLOATS = 2 * 1024 * 1024      # PITCH_NOALLOC_RESIDUAL_FLOATS


def append_noalloc(cache: KVCache, keys, values, stream=None) -> None:
    """Encodes ``[segments, n_new, dim]`` keys and values at positions ``[tokens, tokens + n_new)``
    of ``cache`` without touching ``cache``'s own residual tensors."""
    keys, values = cache._check_new(keys, "keys"), cache._check_new(values, "values")
    if keys.shape != values.shape or keys.dtype != values.dtype:
        raise InvalidInput("keys and values must have the same shape and dtype")
    n_new = int(keys.shape[1])
    if n_new < 1:
        raise InvalidInput("n_new must be at least 1")
    if cache.tokens + n_new > cache.capacity:
        raise InvalidInput(f"cache holds {cache.tokens} of {cache.capacity} tokens; cannot append {n_new}")
    if cache.key_bias is not None:
        # same as KVCache.append: the rotated key bias of each position comes off a copy of the keys
        with cache._stream_context(stream):
            keys = keys.clone()
        cache.pitch.enqueue_rope_bias(keys, *cache.key_bias, first_position=cache.tokens, subtract=True, stream=stream)
    limit = min([pl.config.group_size for pl in cache.planes if pl.is_channel] + [65535])
    done = 0
    while done < n_new:
        room = limit - (cache.tokens % limit) if limit != 65535 else limit
        step = min(room, n_new - done)
        desc = cache._desc(cache.tokens)
        src = (_native.AppendSrc * 4)()
        for i, x in enumerate((keys, values)):
            esz = x.element_size()
            src[i].input = x.data_ptr() + done * cache.dim * esz
            src[i].input_seg_stride = x.stride(0) * esz
            src[i].input_bytes = x.numel() * esz - done * cache.dim * esz
        st = _native.lib().pitch_enqueue_cache_append_noalloc(ctypes.byref(desc), src, native_dtype(keys.dtype), step,
                                                              stream_handle(stream, cache.device))
        _native.check(st)
        cache.tokens += step
        done += step
    cache._push_counter()
