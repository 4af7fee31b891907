"""The codec facade: array API and GPU-resident (stream-ordered) API.

``PITCH`` keeps the surface of the reference's Swift class
(Sources/PITCH/PITCH.swift:15-189 and the extension in
Sources/PITCH/PerChannel.swift:182-290), snake-cased:

    encode / decode / decode_into                    array API (host arrays in and out; waits)
    enqueue_encode / enqueue_decode                  caller's device buffers, caller's stream, no wait
    encode_per_channel / decode_per_channel(_into)   per-channel keys, array API
    enqueue_per_channel_encode / _decode             per-channel keys, device buffers

MTLBuffer -> a CUDA torch tensor used as raw bytes (any dtype, contiguous);
MTLCommandBuffer -> a CUDA stream (``torch.cuda.Stream``, a raw handle, or the
tensor device's current stream).  PyTorch only carries memory and streams:
every byte of codec work is done by the kernels behind the C ABI.
"""
from __future__ import annotations

import ctypes

import numpy as np

from . import _native, codebooks
from ._native import Buffer
from .config import DEFAULT_SEED, ChannelQuantConfig, QuantConfig, QuantMethod
from .containers import ChannelCompressedBlock, CompressedBatch
from .errors import DeviceNotSupported, InvalidInput

_DTYPE_NAMES = {"float32": _native.F32, "float16": _native.F16, "bfloat16": _native.BF16}


def _torch():
    import torch
    return torch


_NATIVE_BY_TORCH: dict = {}


def native_dtype(dtype) -> int:
    """``pitch_dtype`` of a torch dtype / its name; float32 for anything that is not a float type
    (raw byte buffers)."""
    try:
        return _NATIVE_BY_TORCH[dtype]
    except (KeyError, TypeError):
        pass
    name = str(dtype).replace("torch.", "")
    code = _DTYPE_NAMES.get(name, _native.F32)
    try:
        _NATIVE_BY_TORCH[dtype] = code
    except TypeError:
        pass
    return code


def torch_dtype(dtype):
    torch = _torch()
    if isinstance(dtype, torch.dtype):
        if str(dtype).replace("torch.", "") not in _DTYPE_NAMES:
            raise InvalidInput(f"unsupported element type {dtype}; use float32, float16 or bfloat16")
        return dtype
    try:
        return {"float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16,
                "f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}[str(dtype)]
    except KeyError:
        raise InvalidInput(f"unsupported element type {dtype!r}; use float32, float16 or bfloat16") from None


def as_buffer(t, offset: int, name: str) -> Buffer:
    """(tensor, byte offset) -> ``pitch_buffer``.  The tensor is used as raw bytes."""
    torch = _torch()
    if not isinstance(t, torch.Tensor):
        raise InvalidInput(f"{name} must be a torch tensor on a CUDA device")
    if not t.is_cuda:
        raise InvalidInput(f"{name} buffer is not device memory")
    if not t.is_contiguous():
        raise InvalidInput(f"{name} must be contiguous")
    return Buffer(t.data_ptr(), t.numel() * t.element_size(), int(offset))


_raw_stream = None


def stream_handle(stream, device) -> int:
    """The ``cudaStream_t`` to launch on: ``stream`` (a torch stream or a raw handle), or the
    device's current torch stream."""
    global _raw_stream
    if stream is None:
        torch = _torch()
        if _raw_stream is None:
            # the raw-handle query is several times cheaper than building a Stream object per call
            _raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", False)
        if _raw_stream and device.index is not None:
            return _raw_stream(device.index)
        return torch.cuda.current_stream(device).cuda_stream
    if isinstance(stream, int):
        return stream
    return stream.cuda_stream


class PITCH:
    """KV-cache codec on one CUDA device."""

    default_seed = DEFAULT_SEED

    def __init__(self, device=None, seed: int = DEFAULT_SEED):
        torch = _torch()
        _native.lib()                      # fail loudly when the extension is missing
        if not torch.cuda.is_available():
            raise DeviceNotSupported("CUDA is not available on this machine")
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        if self.device.type != "cuda":
            raise DeviceNotSupported(f"{self.device} is not a CUDA device")
        if self.device.index is None:
            self.device = torch.device("cuda", torch.cuda.current_device())
        self.seed = int(seed) & 0xFFFFFFFF
        codebooks.register_all()

    _shared = None

    @classmethod
    def shared(cls) -> "PITCH":
        """Instance on the current CUDA device with the default seed (PITCH.shared)."""
        if cls._shared is None:
            cls._shared = cls()
        return cls._shared

    # ------------------------------------------------------------------ configuration
    def config(self, method, dim: int, bits: int) -> QuantConfig:
        return QuantConfig(QuantMethod.parse(method), dim, bits, self.seed)

    def channel_config(self, dim: int, bits: int, group_size: int = 64) -> ChannelQuantConfig:
        return ChannelQuantConfig(dim, bits, group_size)

    def make_stream(self):
        """A stream on this device, for callers that do not have one (makeCommandBuffer)."""
        return _torch().cuda.Stream(self.device)

    # ------------------------------------------------------------------ GPU-resident API
    def enqueue_encode(self, input, codes, scales, count: int, config: QuantConfig, *, input_offset: int = 0,
                       codes_offset: int = 0, scales_offset: int = 0, stream=None, dtype=None) -> None:
        """Queues compression of ``count`` contiguous vectors on ``stream`` and returns at once.

        Writes ``count * config.code_stride`` bytes of codes and ``count`` float32 scales; results
        are valid when the stream reaches this point.  Offsets are in bytes, multiples of 4.
        ``dtype`` is the element type of ``input`` (default: the tensor's dtype when it is
        float32 / float16 / bfloat16, else float32).  Values are not inspected: they must be
        finite with magnitude at most ``QuantConfig.max_input_magnitude``.
        """
        dt = native_dtype(input.dtype if dtype is None else torch_dtype(dtype))
        st = _native.lib().pitch_enqueue_encode(
            config.method.native, config.dim, config.bits, config.seed, dt,
            as_buffer(input, input_offset, "input"), as_buffer(codes, codes_offset, "codes"),
            as_buffer(scales, scales_offset, "scales"), int(count), stream_handle(stream, input.device))
        _native.check(st)

    def enqueue_decode(self, codes, scales, output, count: int, config: QuantConfig, *, codes_offset: int = 0,
                       scales_offset: int = 0, output_offset: int = 0, stream=None, dtype=None) -> None:
        """Queues reconstruction of ``count`` vectors into ``output`` (``count * dim`` elements)."""
        dt = native_dtype(output.dtype if dtype is None else torch_dtype(dtype))
        st = _native.lib().pitch_enqueue_decode(
            config.method.native, config.dim, config.bits, config.seed, dt,
            as_buffer(codes, codes_offset, "codes"), as_buffer(scales, scales_offset, "scales"),
            as_buffer(output, output_offset, "output"), int(count), stream_handle(stream, output.device))
        _native.check(st)

    def enqueue_per_channel_encode(self, input, codes, ranges, count: int, config: ChannelQuantConfig, *,
                                   input_offset: int = 0, codes_offset: int = 0, ranges_offset: int = 0,
                                   stream=None, dtype=None) -> None:
        """Queues per-channel compression of ``count`` tokens (token-major).  Groups start at the
        first token of the call; the last group may be partial.  Writes
        ``ceil(count / group_size) * config.range_stride`` bytes of fp16 ranges."""
        dt = native_dtype(input.dtype if dtype is None else torch_dtype(dtype))
        st = _native.lib().pitch_enqueue_channel_encode(
            config.dim, config.bits, config.group_size, dt, as_buffer(input, input_offset, "input"),
            as_buffer(codes, codes_offset, "codes"), as_buffer(ranges, ranges_offset, "ranges"), int(count),
            stream_handle(stream, input.device))
        _native.check(st)

    def enqueue_per_channel_decode(self, codes, ranges, output, count: int, config: ChannelQuantConfig, *,
                                   codes_offset: int = 0, ranges_offset: int = 0, output_offset: int = 0,
                                   stream=None, dtype=None) -> None:
        dt = native_dtype(output.dtype if dtype is None else torch_dtype(dtype))
        st = _native.lib().pitch_enqueue_channel_decode(
            config.dim, config.bits, config.group_size, dt, as_buffer(codes, codes_offset, "codes"),
            as_buffer(ranges, ranges_offset, "ranges"), as_buffer(output, output_offset, "output"), int(count),
            stream_handle(stream, output.device))
        _native.check(st)

    def enqueue_pack_codes(self, codes_i32, packed, count: int, dim: int, bits: int, *, stream=None) -> None:
        st = _native.lib().pitch_enqueue_pack_codes(dim, bits, as_buffer(codes_i32, 0, "codes_i32"),
                                                    as_buffer(packed, 0, "packed"), int(count),
                                                    stream_handle(stream, packed.device))
        _native.check(st)

    def enqueue_unpack_codes(self, packed, codes_i32, count: int, dim: int, bits: int, *, stream=None) -> None:
        st = _native.lib().pitch_enqueue_unpack_codes(dim, bits, as_buffer(packed, 0, "packed"),
                                                      as_buffer(codes_i32, 0, "codes_i32"), int(count),
                                                      stream_handle(stream, packed.device))
        _native.check(st)

    def checksum(self, tensor, nbytes: int | None = None, *, stream=None) -> int:
        """64-bit position-weighted checksum of a device buffer (waits for the result)."""
        torch = _torch()
        n = tensor.numel() * tensor.element_size() if nbytes is None else nbytes
        acc = torch.zeros(1, dtype=torch.int64, device=tensor.device)
        st = _native.lib().pitch_enqueue_checksum(as_buffer(tensor, 0, "buffer"), int(n), acc.data_ptr(),
                                                  stream_handle(stream, tensor.device))
        _native.check(st)
        return int(acc.item()) & 0xFFFFFFFFFFFFFFFF

    def enqueue_rope_bias(self, data, bias, cos_table, sin_table, *, first_position: int = 0, subtract: bool,
                          stream=None) -> None:
        """Exact key-bias removal (reference/mechanism_eval.py:82-91, ``rotated_bias``): in place,
        ``data[s, v] -= / += bias[s] * cos[p] + rotate_half(bias[s]) * sin[p]`` with
        ``p = first_position + v``.  ``data`` is ``[segments, count, dim]`` (float32 / float16 /
        bfloat16; the segment stride may exceed ``count * dim``), ``bias`` float32
        ``[segments, dim]``, the tables float32 ``[positions, dim]`` (the model's own rotary
        tables).  ``subtract=True`` before encoding, ``False`` after decoding."""
        torch = _torch()
        for t, name in ((data, "data"), (bias, "bias"), (cos_table, "cos_table"), (sin_table, "sin_table")):
            if not (isinstance(t, torch.Tensor) and t.is_cuda):
                raise InvalidInput(f"{name} must be a CUDA tensor")
        if data.dim() != 3 or data.stride(2) != 1 or data.stride(1) != data.shape[2]:
            raise InvalidInput("data must be [segments, count, dim] with contiguous vectors")
        S, count, dim = (int(v) for v in data.shape)
        for t, name in ((bias, "bias"), (cos_table, "cos_table"), (sin_table, "sin_table")):
            if t.dtype != torch.float32 or not t.is_contiguous() or t.dim() != 2 or t.shape[1] != dim:
                raise InvalidInput(f"{name} must be a contiguous float32 tensor with {dim} columns")
        if bias.shape[0] != S or cos_table.shape != sin_table.shape:
            raise InvalidInput("bias needs one row per segment; cos and sin tables must have the same shape")
        rope = _native.RopeBias(bias.data_ptr(), dim * 4, cos_table.data_ptr(), sin_table.data_ptr(), int(cos_table.shape[0]))
        st = _native.lib().pitch_enqueue_rope_bias(dim, native_dtype(data.dtype), 1 if subtract else 0, data.data_ptr(),
                                                   data.stride(0) * data.element_size(), S, int(first_position), count,
                                                   ctypes.byref(rope), stream_handle(stream, data.device))
        _native.check(st)

    # ------------------------------------------------------------------ array API, per-vector
    @staticmethod
    def _host_floats(vectors, what: str) -> np.ndarray:
        torch = _torch()
        if isinstance(vectors, torch.Tensor):
            vectors = vectors.detach().to("cpu", torch.float32).numpy()
        x = np.ascontiguousarray(vectors, dtype=np.float32).reshape(-1)
        return x

    @staticmethod
    def _validate_values(x: np.ndarray, limit: float, why: str) -> None:
        # PITCH.validateValues, Sources/PITCH/PITCH.swift:172-181 / PerChannel.swift:273-282
        if not np.isfinite(x).all():
            raise InvalidInput("input contains NaN or infinity")
        largest = float(np.abs(x).max()) if x.size else 0.0
        if largest > limit:
            raise InvalidInput(f"input magnitude {largest} exceeds {limit}; {why}")

    def encode(self, vectors, dim: int | None = None, bits: int | None = None, method=None, seed: int | None = None,
               config: QuantConfig | None = None) -> CompressedBatch:
        """Compresses ``len(vectors) / dim`` vectors stored contiguously (host data in, host
        container out).  ``dim`` defaults to the length of a one-dimensional input or the last
        axis of a two-dimensional one."""
        torch = _torch()
        if config is None:
            if dim is None:
                shape = np.shape(vectors)
                dim = int(shape[-1]) if len(shape) >= 1 else 0
            config = QuantConfig(QuantMethod.parse(method), dim, bits, self.seed if seed is None else seed)
        x = self._host_floats(vectors, "vectors")
        if x.size == 0 or x.size % config.dim:
            raise InvalidInput(f"{x.size} floats is not a whole number of {config.dim}-dim vectors")
        self._validate_values(x, QuantConfig.max_input_magnitude,
                              "the kernels' float32 sum of squares would overflow")
        count = x.size // config.dim
        with torch.cuda.device(self.device):
            d_in = torch.from_numpy(x).to(self.device)
            d_codes = torch.empty(count * config.code_stride, dtype=torch.uint8, device=self.device)
            d_scales = torch.empty(count, dtype=torch.float32, device=self.device)
            self.enqueue_encode(d_in, d_codes, d_scales, count, config)
            codes = d_codes.cpu().numpy().tobytes()
            scales = d_scales.cpu().numpy()
        return CompressedBatch(config, codes, scales, _unchecked=True)

    def decode(self, batch: CompressedBatch) -> np.ndarray:
        """Reconstructs every vector of the batch, contiguously: float32 array of count*dim."""
        torch = _torch()
        out = torch.empty(batch.count * batch.config.dim, dtype=torch.float32, device=self.device)
        self.decode_into(batch, out, 0)
        return out.cpu().numpy()

    def decode_into(self, batch: CompressedBatch, buffer, offset: int = 0, dtype=None) -> None:
        """Reconstructs the batch into a device ``buffer`` starting at byte ``offset``, then waits."""
        torch = _torch()
        batch.validate()
        with torch.cuda.device(self.device):
            d_codes = torch.frombuffer(bytearray(batch.codes), dtype=torch.uint8).to(self.device)
            d_scales = torch.from_numpy(batch.scales).to(self.device)
            self.enqueue_decode(d_codes, d_scales, buffer, batch.count, batch.config, output_offset=offset,
                                dtype=dtype)
            torch.cuda.current_stream(self.device).synchronize()

    # ------------------------------------------------------------------ array API, per-channel
    def encode_per_channel(self, vectors, dim: int | None = None, bits: int | None = None, group_size: int = 64,
                           config: ChannelQuantConfig | None = None) -> ChannelCompressedBlock:
        """Compresses ``len(vectors) / dim`` tokens stored contiguously, token-major."""
        torch = _torch()
        if config is None:
            if dim is None:
                dim = int(np.shape(vectors)[-1])
            config = ChannelQuantConfig(dim, bits, group_size)
        x = self._host_floats(vectors, "vectors")
        if x.size == 0 or x.size % config.dim:
            raise InvalidInput(f"{x.size} floats is not a whole number of {config.dim}-dim tokens")
        self._validate_values(x, ChannelQuantConfig.max_input_magnitude, "per-channel ranges are stored in fp16")
        count = x.size // config.dim
        groups = config.group_count(count)
        with torch.cuda.device(self.device):
            d_in = torch.from_numpy(x).to(self.device)
            d_codes = torch.empty(count * config.code_stride, dtype=torch.uint8, device=self.device)
            d_ranges = torch.empty(groups * 2 * config.dim, dtype=torch.float16, device=self.device)
            self.enqueue_per_channel_encode(d_in, d_codes, d_ranges, count, config)
            codes = d_codes.cpu().numpy().tobytes()
            ranges = d_ranges.cpu().numpy().view(np.uint16)
        return ChannelCompressedBlock(config, codes, ranges, _unchecked=True)

    def decode_per_channel(self, block: ChannelCompressedBlock) -> np.ndarray:
        torch = _torch()
        out = torch.empty(block.count * block.config.dim, dtype=torch.float32, device=self.device)
        self.decode_per_channel_into(block, out, 0)
        return out.cpu().numpy()

    def decode_per_channel_into(self, block: ChannelCompressedBlock, buffer, offset: int = 0, dtype=None) -> None:
        torch = _torch()
        block.validate()
        with torch.cuda.device(self.device):
            d_codes = torch.frombuffer(bytearray(block.codes), dtype=torch.uint8).to(self.device)
            d_ranges = torch.from_numpy(block.ranges.view(np.float16)).to(self.device)
            self.enqueue_per_channel_decode(d_codes, d_ranges, buffer, block.count, block.config,
                                            output_offset=offset, dtype=dtype)
            torch.cuda.current_stream(self.device).synchronize()
