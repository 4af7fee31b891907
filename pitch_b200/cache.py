"""A compressed KV cache held by one GPU, with one-launch whole-cache decode.

The reference describes the pattern but leaves it to the caller (README.md:62-85): per
generated token, ``enqueueEncode`` the new token of every head at its offset, then
``enqueueDecode`` the whole cache; per-channel keys are encoded group by group, the
newest partial group being re-encoded as it grows.  ``KVCache`` packages that pattern:

* a *segment* is one (layer, KV head); a cache sharded over GPUs gives each rank a
  contiguous range of segments and no rank ever touches another rank's memory;
* a *plane* is one tensor of the cache (keys or values) with its codec: per-channel
  (``ChannelQuantConfig``) or per-vector (``QuantConfig``, TurboQuant or PolarQuant);
* ``append`` encodes new tokens for all segments and planes (one launch);
* ``decode`` reconstructs every token of every segment and plane (one launch);
* ``step`` does both for one new token per segment in a single launch - the per-token path.

Layout in device memory, per plane, segment-major and token-major:
codes ``[segments][capacity * code_stride]`` bytes, side information
``[segments][capacity]`` float32 (norm / rmax) or ``[segments][groups][2][dim]`` fp16
(minima then maxima), output ``[segments][capacity][dim]`` of ``out_dtype``.
"""
from __future__ import annotations

import contextlib
import ctypes
from dataclasses import dataclass

from . import _native, codebooks
from .codec import PITCH, native_dtype, stream_handle, torch_dtype
from .config import ChannelQuantConfig, QuantConfig, QuantMethod
from .errors import InvalidInput


def _torch():
    import torch
    return torch


@dataclass
class _Plane:
    name: str
    config: object           # QuantConfig | ChannelQuantConfig
    codes: object            # uint8 [segments, capacity * stride]
    side: object             # float32 [segments, capacity] | float16 [segments, groups, 2, dim]
    out: object              # out_dtype [segments, capacity, dim]
    residual: object | None  # float32 [segments, group_size + 2, dim] for per-channel planes (tokens, running min, max)

    @property
    def is_channel(self) -> bool:
        return isinstance(self.config, ChannelQuantConfig)

    @property
    def kind(self) -> int:
        if self.is_channel:
            return _native.PLANE_CHANNEL
        return _native.PLANE_TURBO if self.config.method is QuantMethod.turboQuant else _native.PLANE_POLAR


class KVCache:
    """Compressed keys and values for ``segments`` (layer x KV head) sequences of up to
    ``capacity`` tokens of dimension ``dim``."""

    def __init__(self, segments: int, dim: int, capacity: int, key_config, value_config, *,
                 out_dtype="bfloat16", device=None, pitch: PITCH | None = None, key_bias=None,
                 fuse_key_bias: bool = True):
        """``key_bias=(bias, cos_table, sin_table)`` turns on exact key-bias removal
        (reference/mechanism_eval.py:4-7): ``bias`` float32 ``[segments, dim]`` is the key
        projection's bias per KV head, the tables float32 ``[positions, dim]`` are the model's
        rotary tables.  The rotated bias of a token's position is subtracted from the keys before
        they are encoded and added back to the decoded keys, at no storage cost.  On cache shapes
        the one-launch kernel covers, ``decode`` and ``step`` do this inside their launch;
        ``fuse_key_bias=False`` keeps it as separate element-wise launches (same results)."""
        torch = _torch()
        self.pitch = pitch if pitch is not None else PITCH(device)
        self.device = self.pitch.device
        if segments < 1 or capacity < 1:
            raise InvalidInput("segments and capacity must be at least 1")
        for cfg in (key_config, value_config):
            if cfg.dim != dim:
                raise InvalidInput(f"codec dimension {cfg.dim} differs from the cache's {dim}")
        self.segments, self.dim = int(segments), int(dim)
        self.capacity = (int(capacity) + 127) // 128 * 128      # keeps every segment stride 16-byte aligned
        self.out_dtype = torch_dtype(out_dtype)
        self.tokens = 0
        self._desc_cache = None
        self._state = None                  # device-side token counter (use_device_counter)
        self._float_dtypes = (torch.float32, torch.float16, torch.bfloat16)
        self.planes = [self._make_plane("keys", key_config), self._make_plane("values", value_config)]
        self._piece_limit = min([pl.config.group_size for pl in self.planes if pl.is_channel] + [65535])
        self.key_bias = None
        self._fused = self._fused_ok()
        self._fuse_bias = False
        self._rope = None
        if key_bias is not None:
            bias, cos_table, sin_table = key_bias
            if tuple(bias.shape) != (self.segments, self.dim) or cos_table.shape[0] < self.capacity:
                raise InvalidInput(f"key_bias needs bias [{self.segments}, {self.dim}] and tables with at least {self.capacity} rows")
            for t, name in ((bias, "bias"), (cos_table, "cos_table"), (sin_table, "sin_table")):
                if not (t.is_cuda and t.is_contiguous() and t.dtype == torch.float32 and t.dim() == 2 and t.shape[1] == self.dim):
                    raise InvalidInput(f"key_bias {name} must be a contiguous float32 CUDA tensor with {self.dim} columns")
            self.key_bias = (bias, cos_table, sin_table)
            self._fuse_bias = bool(fuse_key_bias) and self._fused
            self._rope = _native.RopeBias(bias.data_ptr(), self.dim * 4, cos_table.data_ptr(), sin_table.data_ptr(),
                                          int(cos_table.shape[0]))
        codebooks.register_all()

    def _make_plane(self, name: str, cfg) -> _Plane:
        torch = _torch()
        S, C, d, dev = self.segments, self.capacity, self.dim, self.device
        codes = torch.zeros((S, C * cfg.code_stride), dtype=torch.uint8, device=dev)
        out = torch.zeros((S, C, d), dtype=self.out_dtype, device=dev)
        if isinstance(cfg, ChannelQuantConfig):
            groups = cfg.group_count(C)
            side = torch.zeros((S, groups, 2, d), dtype=torch.float16, device=dev)
            residual = torch.zeros((S, cfg.group_size + 2, d), dtype=torch.float32, device=dev)
        else:
            side = torch.zeros((S, C), dtype=torch.float32, device=dev)
            residual = None
        return _Plane(name, cfg, codes, side, out, residual)

    # ------------------------------------------------------------------ descriptors
    def _desc(self, tokens: int, with_bias: bool = False) -> _native.CacheDesc:
        """The C descriptor of this cache.  Buffers never move, so it is filled once and only the
        token count changes from call to call (this runs on the per-token path).  ``with_bias``
        selects the twin that also carries the key-bias tables (what ``decode`` and ``step`` pass
        when the bias is handled inside their launch)."""
        if with_bias:
            if self._desc_cache is None:
                self._desc(tokens)
            d = self._desc_bias
            d.tokens = tokens
            return d
        d = self._desc_cache
        if d is None:
            d = _native.CacheDesc()
            d.dim = self.dim
            d.out_dtype = native_dtype(self.out_dtype)
            d.segments = self.segments
            d.n_planes = len(self.planes)
            d.capacity = self.capacity
            for i, pl in enumerate(self.planes):
                q = d.planes[i]
                q.kind = pl.kind
                q.bits = pl.config.bits
                q.group_size = pl.config.group_size if pl.is_channel else 0
                q.seed = 0 if pl.is_channel else pl.config.seed
                q.codes = pl.codes.data_ptr()
                q.codes_seg_stride = pl.codes.stride(0) * pl.codes.element_size()
                q.codes_bytes = pl.codes.numel() * pl.codes.element_size()
                q.side = pl.side.data_ptr()
                q.side_seg_stride = pl.side.stride(0) * pl.side.element_size()
                q.side_bytes = pl.side.numel() * pl.side.element_size()
                q.out = pl.out.data_ptr()
                q.out_seg_stride = pl.out.stride(0) * pl.out.element_size()
                q.out_bytes = pl.out.numel() * pl.out.element_size()
            self._desc_cache = d
            self._desc_ref = ctypes.byref(d)
            src = (_native.AppendSrc * 4)()
            for i, pl in enumerate(self.planes):
                if pl.residual is not None:
                    src[i].residual = pl.residual.data_ptr()
                    src[i].residual_seg_stride = pl.residual.stride(0) * 4
                    src[i].residual_bytes = pl.residual.numel() * 4
            self._src_cache = src
            self._src_geometry = None
            self._lib = _native.lib()
            # twin descriptor with the key-bias tables
            b = _native.CacheDesc.from_buffer_copy(d)
            if self._rope is not None:
                b.key_bias = ctypes.pointer(self._rope)
            self._desc_bias = b
            self._desc_bias_ref = ctypes.byref(b)
        d.tokens = tokens
        return d

    def _fill_src(self, keys, values, first: int, n: int):
        """Points the cached ``pitch_append_src`` array at tokens ``[first, first + n)`` of the inputs.
        Strides and extents are rewritten only when the inputs' geometry changed since the last call
        (this runs once per generated token)."""
        src = self._src_cache
        esz = keys.element_size()
        off = first * self.dim * esz
        geometry = (keys.stride(0), values.stride(0), keys.numel(), values.numel(), esz, off)
        src[0].input = keys.data_ptr() + off
        src[1].input = values.data_ptr() + off
        if geometry != self._src_geometry:
            for i, x in enumerate((keys, values)):
                src[i].input_seg_stride = x.stride(0) * esz
                src[i].input_bytes = x.numel() * esz - off
            self._src_geometry = geometry
        return src

    def _stream_context(self, stream):
        """Context manager that makes ``stream`` (a torch stream, a raw handle or None) torch's
        current stream, so that tensors made inside are ordered and owned like the kernels."""
        torch = _torch()
        if stream is None:
            return contextlib.nullcontext()
        if isinstance(stream, int):
            stream = torch.cuda.ExternalStream(stream, device=self.device)
        return torch.cuda.stream(stream)

    # ------------------------------------------------------------------ writing
    def _check_new(self, x, name: str):
        torch = _torch()
        if not (isinstance(x, torch.Tensor) and x.is_cuda and x.is_contiguous()):
            raise InvalidInput(f"{name} must be a contiguous CUDA tensor")
        if x.dim() != 3 or x.shape[0] != self.segments or x.shape[2] != self.dim:
            raise InvalidInput(f"{name} must have shape [segments={self.segments}, n_new, dim={self.dim}]")
        if x.dtype not in self._float_dtypes:
            torch_dtype(x.dtype)          # raises with the list of accepted types
        return x

    def append(self, keys, values, stream=None) -> None:
        """Encodes ``n_new`` tokens per segment (tensors ``[segments, n_new, dim]``, float32 /
        float16 / bfloat16, same dtype for both) at positions ``[tokens, tokens + n_new)``.
        Stream-ordered; never waits."""
        keys, values = self._check_new(keys, "keys"), self._check_new(values, "values")
        if keys.shape != values.shape or keys.dtype != values.dtype:
            raise InvalidInput("keys and values must have the same shape and dtype")
        n_new = int(keys.shape[1])
        if n_new < 1:
            raise InvalidInput("n_new must be at least 1")
        if self.tokens + n_new > self.capacity:
            raise InvalidInput(f"cache holds {self.tokens} of {self.capacity} tokens; cannot append {n_new}")
        if self.key_bias is not None:
            with self._stream_context(stream):          # the copy is made, and later freed, on the launching stream
                keys = keys.clone()
            self.pitch.enqueue_rope_bias(keys, *self.key_bias, first_position=self.tokens, subtract=True, stream=stream)
        limit = self._piece_limit           # new tokens of one launch must fall into one per-channel group
        done = 0
        while done < n_new:
            room = limit - (self.tokens % limit) if limit != 65535 else limit
            step = min(room, n_new - done)
            self._append_piece(keys, values, done, step, stream)
            self.tokens += step
            done += step
        self._push_counter()

    def _append_piece(self, keys, values, first: int, n: int, stream) -> None:
        self._desc(self.tokens)
        src = self._fill_src(keys, values, first, n)
        st = self._lib.pitch_enqueue_cache_append(self._desc_ref, src, native_dtype(keys.dtype), n,
                                                  stream_handle(stream, self.device))
        if st:
            _native.check(st)

    # ------------------------------------------------------------------ the per-token path
    def step(self, keys, values, stream=None, views: bool = True):
        """One generation step: appends ONE new token per segment (tensors ``[segments, 1, dim]``)
        and decodes the whole cache, new token included, in a single launch; returns the decoded
        views like ``decode`` (``views=False``: returns None and leaves it to the caller to slice
        ``planes[i].out[:, :tokens]``, which saves a few microseconds per token).  Results are exactly
        those of ``append`` followed by ``decode``.  Cache shapes the one-launch kernel does not cover
        run as those two calls."""
        if not self._fused or (self.key_bias is not None and not self._fuse_bias):
            self.append(keys, values, stream)
            return self.decode(stream)
        keys, values = self._check_new(keys, "keys"), self._check_new(values, "values")
        if keys.shape[1] != 1 or keys.shape != values.shape or keys.dtype != values.dtype:
            raise InvalidInput("step takes one new token per segment: keys and values of shape [segments, 1, dim], same dtype")
        if self.tokens >= self.capacity:
            raise InvalidInput(f"cache holds {self.tokens} of {self.capacity} tokens; cannot append 1")
        self._desc(self.tokens, self._fuse_bias)
        src = self._fill_src(keys, values, 0, 1)
        st = self._lib.pitch_enqueue_cache_step(self._desc_bias_ref if self._fuse_bias else self._desc_ref, src, native_dtype(keys.dtype),
                                                self._state.data_ptr() if self._state is not None else None,
                                                stream_handle(stream, self.device))
        if st:
            _native.check(st)
        self.tokens += 1
        return tuple(pl.out[:, :self.tokens] for pl in self.planes) if views else None

    def _fused_ok(self) -> bool:
        """Whether the one-launch step kernel covers this cache (dim 64 or 128; TurboQuant planes of
        one width, 3 or 4 bits; per-channel planes of 4 bits with whole items per group)."""
        if self.dim not in (64, 128):
            return False
        widths = set()
        for pl in self.planes:
            if pl.is_channel:
                if pl.config.bits != 4 or pl.config.group_size % (2048 // self.dim):
                    return False
            elif pl.kind != _native.PLANE_TURBO or pl.config.bits not in (3, 4):
                return False
            else:
                widths.add(pl.config.bits)
        return len(widths) <= 1

    def use_device_counter(self) -> None:
        """Keeps the token count in device memory as well (``pitch_cache_state``): ``step`` then
        launches with parameters that do not depend on the count, so one captured CUDA graph of a
        step can be replayed token after token (``capture_step`` / ``replay``).  Needs a cache shape
        the one-launch step covers and no key-bias removal."""
        torch = _torch()
        if not self._fused or (self.key_bias is not None and not self._fuse_bias):
            raise InvalidInput("the device-side token counter needs a cache shape the one-launch step covers")
        if self._state is None:
            self._state = torch.zeros(2, dtype=torch.int64, device=self.device)     # tokens | status, arrivals
        self._push_counter()

    def _push_counter(self) -> None:
        if self._state is not None:
            torch = _torch()
            self._state.copy_(torch.tensor([self.tokens, 0], dtype=torch.int64))

    def counter(self) -> tuple[int, int]:
        """(tokens, status) as the device-side counter holds them (waits for the stream)."""
        if self._state is None:
            raise InvalidInput("no device-side counter: call use_device_counter() first")
        tokens, rest = (int(v) for v in self._state.cpu())
        return tokens, rest & 0xFFFFFFFF

    def capture_step(self, keys, values):
        """Captures one ``step`` reading the new token from the given tensors (whose storage the
        caller refills before every replay) into a CUDA graph.  Returns the graph; run it with
        ``replay``."""
        return self.capture(lambda: self.step(keys, values, views=False))

    def capture(self, enqueue):
        """Captures what ``enqueue()`` puts on the current stream into a CUDA graph: exactly one
        ``step``, and around it whatever belongs to a generation step - the copy of the new token from
        pinned host memory, ``newest``, the copy of its result back to the host.  All tensors it touches
        must stay alive and in place.  Returns the graph; run it with ``replay``."""
        torch = _torch()
        self.use_device_counter()
        if self.tokens >= 1:
            self.decode()                        # first use of the kernel configures it: keep that out of the capture
        torch.cuda.synchronize(self.device)
        graph = torch.cuda.CUDAGraph()
        held = self.tokens
        with torch.cuda.graph(graph, capture_error_mode="thread_local"):
            enqueue()
        if self.tokens != held + 1:
            self.tokens = held
            raise InvalidInput("the captured function must make exactly one step")
        self.tokens = held                       # capturing queues nothing
        return graph

    def newest(self, out=None, stream=None):
        """The decoded token at the newest position of every plane and segment, gathered into one
        contiguous tensor ``[planes, segments, dim]`` of the output dtype (``pitch_enqueue_cache_newest``).
        With the device-side counter in use the position is read on the device, so the call can be part
        of a captured step."""
        torch = _torch()
        if self.tokens < 1:
            raise InvalidInput("the cache is empty")
        dt = self.planes[0].out.dtype
        shape = (len(self.planes), self.segments, self.dim)
        if out is None:
            with self._stream_context(stream):
                out = torch.empty(shape, dtype=dt, device=self.device)
        elif (tuple(out.shape) != shape or out.dtype != dt or not out.is_contiguous() or not out.is_cuda
              or out.device != self.planes[0].out.device):
            raise InvalidInput(f"out must be a contiguous CUDA tensor of shape {shape} and dtype {dt} on the cache's device")
        self._desc(self.tokens, False)
        st = self._lib.pitch_enqueue_cache_newest(self._desc_ref, self._state.data_ptr() if self._state is not None else None,
                                                  out.data_ptr(), out.numel() * out.element_size(), stream_handle(stream, self.device))
        if st:
            _native.check(st)
        return out

    def replay(self, graph, views: bool = True):
        """Replays a graph made by ``capture_step`` / ``capture``: one more token per segment.  Returns the
        decoded planes as ``step`` does (``views=False``: nothing, for a loop that reads its results elsewhere)."""
        if self.tokens >= self.capacity:
            raise InvalidInput(f"cache holds {self.tokens} of {self.capacity} tokens; cannot append 1")
        graph.replay()
        self.tokens += 1
        return tuple(pl.out[:, :self.tokens] for pl in self.planes) if views else None

    def prefill(self, keys, values, stream=None) -> None:
        """Bulk-encodes ``[segments, T, dim]`` tensors into an empty cache with the stand-alone
        encoders (whole groups for per-channel planes), then appends what is left of a final
        partial group so that it stays re-encodable."""
        keys, values = self._check_new(keys, "keys"), self._check_new(values, "values")
        if self.tokens != 0:
            raise InvalidInput("prefill needs an empty cache")
        T = int(keys.shape[1])
        if T > self.capacity:
            raise InvalidInput(f"{T} tokens exceed the capacity {self.capacity}")
        groups = [pl.config.group_size for pl in self.planes if pl.is_channel]
        bulk = T if not groups else T // max(groups) * max(groups)
        if len(set(groups)) > 1:
            raise InvalidInput("per-channel planes of one cache must share a group size")
        p = self.pitch
        key_bias, self.key_bias = self.key_bias, None          # applied once here, not again by append() below
        if key_bias is not None:
            with self._stream_context(stream):
                keys = keys.clone()
            p.enqueue_rope_bias(keys, *key_bias, first_position=0, subtract=True, stream=stream)
        esz = keys.element_size()
        for pl, x in zip(self.planes, (keys, values)):
            if bulk == 0:
                break
            for s in range(self.segments):
                in_off = s * x.stride(0) * esz
                c_off = s * pl.codes.stride(0)
                s_off = s * pl.side.stride(0) * pl.side.element_size()
                if pl.is_channel:
                    p.enqueue_per_channel_encode(x, pl.codes, pl.side, bulk, pl.config, input_offset=in_off,
                                                 codes_offset=c_off, ranges_offset=s_off, stream=stream)
                else:
                    p.enqueue_encode(x, pl.codes, pl.side, bulk, pl.config, input_offset=in_off,
                                     codes_offset=c_off, scales_offset=s_off, stream=stream)
        self.tokens = bulk
        try:
            if bulk < T:
                self.append(keys[:, bulk:].contiguous(), values[:, bulk:].contiguous(), stream)
        finally:
            self.key_bias = key_bias
        self._push_counter()

    def truncate(self, tokens: int) -> None:
        """Forgets every token from ``tokens`` on (host-side bookkeeping only).  The new length
        must be a multiple of the per-channel group size so that no partial group is cut."""
        if not 0 <= tokens <= self.tokens:
            raise InvalidInput(f"cannot truncate {self.tokens} tokens to {tokens}")
        for pl in self.planes:
            if pl.is_channel and tokens % pl.config.group_size:
                raise InvalidInput("truncate to a multiple of the group size")
        self.tokens = int(tokens)
        self._push_counter()

    # ------------------------------------------------------------------ reading
    def decode(self, stream=None):
        """Queues the reconstruction of all ``tokens`` tokens of every segment and plane and
        returns views ``[segments, tokens, dim]`` of the key and value output buffers (valid
        once the stream reaches this point)."""
        if self.tokens < 1:
            raise InvalidInput("the cache is empty")
        self._desc(self.tokens, self._fuse_bias)
        st = self._lib.pitch_enqueue_cache_decode(self._desc_bias_ref if self._fuse_bias else self._desc_ref,
                                                  stream_handle(stream, self.device))
        if st:
            _native.check(st)
        if self.key_bias is not None and not self._fuse_bias:
            self.pitch.enqueue_rope_bias(self.planes[0].out[:, :self.tokens], *self.key_bias, first_position=0,
                                         subtract=False, stream=stream)
        return tuple(pl.out[:, :self.tokens] for pl in self.planes)

    def attend(self, queries, scale: float | None = None, out=None, stream=None, precision: str = "float32"):
        """Single-token attention over the compressed cache without decoding it to memory:
        ``queries`` is float32 ``[segments, n_queries, dim]`` (``n_queries`` <= 8: the query
        heads that share a KV head); returns float32 ``[segments, n_queries, dim]`` with
        ``softmax_t(scale * q . K_t) . V_t`` over the ``tokens`` tokens held.  ``scale`` defaults
        to ``1/sqrt(dim)``.  Supported: dim 64 with per-channel 4-bit keys (group size a multiple of
        32) or TurboQuant 4-bit keys, dim 128 with TurboQuant keys and values of 4 or of 3 bits;
        TurboQuant 4-bit values otherwise.  ``precision="float32"`` keeps products float32-accurate
        (about 1e-5 against attention over the float32-decoded cache); ``"bfloat16"`` uses operands
        as a bf16 pipeline has them (as accurate as attention over the cache decoded to bf16: a few
        bf16 roundings, up to about 5e-3) at half the tensor-core work.  Stream-ordered; the scratch buffer is kept by the
        cache and reused, so calls on one cache must be stream-ordered with respect to each other."""
        torch = _torch()
        if self.tokens < 1:
            raise InvalidInput("the cache is empty")
        if self.key_bias is not None:
            raise InvalidInput("attention from the compressed cache does not support key-bias removal")
        if not (isinstance(queries, torch.Tensor) and queries.is_cuda and queries.is_contiguous()
                and queries.dtype == torch.float32):
            raise InvalidInput("queries must be a contiguous float32 CUDA tensor")
        if queries.dim() != 3 or queries.shape[0] != self.segments or queries.shape[2] != self.dim:
            raise InvalidInput(f"queries must have shape [segments={self.segments}, n_queries, dim={self.dim}]")
        n_q = int(queries.shape[1])
        if out is None:
            out = torch.empty_like(queries)
        elif not (isinstance(out, torch.Tensor) and out.is_cuda and out.is_contiguous() and out.dtype == torch.float32
                  and out.shape == queries.shape):
            raise InvalidInput("out must be a contiguous float32 CUDA tensor shaped like queries")
        self._desc(self.tokens)
        need = self._lib.pitch_cache_attention_workspace(self._desc_ref, n_q)
        if need < 0:
            _native.check(1)               # invalid input; the library holds the reason
        ws = getattr(self, "_attention_ws", None)
        if ws is None or ws.numel() < need:
            ws = torch.empty(max(need, 1 << 20), dtype=torch.uint8, device=self.device)
            self._attention_ws = ws
        if precision not in ("float32", "bfloat16"):
            raise InvalidInput(f"precision {precision!r} must be 'float32' or 'bfloat16'")
        args = _native.AttentionArgs(queries.data_ptr(), out.data_ptr(), ws.data_ptr(), ws.numel(), n_q,
                                     float(scale) if scale is not None else self.dim ** -0.5,
                                     1 if precision == "bfloat16" else 0, 0)
        st = self._lib.pitch_enqueue_cache_attention(self._desc_ref, ctypes.byref(args), stream_handle(stream, self.device))
        if st:
            _native.check(st)
        return out

    # ------------------------------------------------------------------ accounting
    def stored_bytes(self, tokens: int | None = None) -> int:
        """Bytes of packed codes plus side information for ``tokens`` tokens per segment."""
        t = self.tokens if tokens is None else tokens
        total = 0
        for pl in self.planes:
            total += t * pl.config.code_stride
            total += pl.config.group_count(t) * pl.config.range_stride if pl.is_channel else t * 4
        return total * self.segments

    def decoded_bytes(self, tokens: int | None = None) -> int:
        t = self.tokens if tokens is None else tokens
        return len(self.planes) * self.segments * t * self.dim * self.planes[0].out.element_size()

    def checksums(self) -> dict:
        """Position-weighted 64-bit checksums of the stored codes and of the decoded outputs,
        per plane (only the bytes of the ``tokens`` tokens currently held)."""
        out = {}
        for pl in self.planes:
            c = pl.codes[:, :self.tokens * pl.config.code_stride].contiguous()
            o = pl.out[:, :self.tokens].contiguous()
            out[pl.name] = {"codes": self.pitch.checksum(c), "decoded": self.pitch.checksum(o)}
        return out
