"""Validated parameter records of the codec.

``QuantConfig`` mirrors Sources/PITCH/Models/QuantConfig.swift:11-61,
``ChannelQuantConfig`` mirrors Sources/PITCH/PerChannel.swift:15-70 and
``QuantMethod`` mirrors Sources/PITCH/Models/QuantMethod.swift:8-11.
"""
from __future__ import annotations

import enum
import operator
from dataclasses import dataclass

from .errors import InvalidBitWidth, InvalidDimension, InvalidInput

DEFAULT_SEED = 0x50495443            # PITCH.defaultSeed, Sources/PITCH/PITCH.swift:18
SUPPORTED_BITS = range(2, 9)
MAX_DIMENSION = 1024


class QuantMethod(str, enum.Enum):
    turboQuant = "turboQuant"
    polarQuant = "polarQuant"

    @classmethod
    def parse(cls, value) -> "QuantMethod":
        if isinstance(value, cls):
            return value
        try:
            return cls(value)
        except ValueError:
            raise InvalidInput(f"unknown method {value!r}") from None

    @property
    def native(self) -> int:
        return 0 if self is QuantMethod.turboQuant else 1


def _as_int(v):
    """Python int for any integral value (NumPy integers included), else None."""
    try:
        return operator.index(v)
    except TypeError:
        return None


def code_stride_bytes(dim: int, bits: int) -> int:
    """Bytes of packed codes per vector or token: whole 32-bit words."""
    return (dim * bits + 31) // 32 * 4


@dataclass(frozen=True)
class QuantConfig:
    """Everything needed to interpret a batch of per-vector codes."""
    method: QuantMethod
    dim: int
    bits: int
    seed: int = DEFAULT_SEED

    max_input_magnitude = 1e17       # QuantConfig.maxInputMagnitude

    def __post_init__(self):
        object.__setattr__(self, "method", QuantMethod.parse(self.method))
        d, b = _as_int(self.dim), _as_int(self.bits)
        if d is None or d < 2 or d > MAX_DIMENSION or d & (d - 1):
            raise InvalidDimension(self.dim)
        if b is None or b not in SUPPORTED_BITS:
            raise InvalidBitWidth(self.bits)
        object.__setattr__(self, "dim", d)
        object.__setattr__(self, "bits", b)
        if not 0 <= int(self.seed) <= 0xFFFFFFFF:
            raise InvalidInput(f"seed {self.seed} does not fit in 32 bits")
        object.__setattr__(self, "seed", int(self.seed))

    @property
    def code_stride(self) -> int:
        return code_stride_bytes(self.dim, self.bits)

    @property
    def bytes_per_vector(self) -> int:
        return self.code_stride + 4

    @property
    def bits_per_coordinate(self) -> float:
        return self.bytes_per_vector * 8 / self.dim

    @property
    def compression_ratio(self) -> float:
        return 32.0 / self.bits_per_coordinate

    @property
    def compression_ratio_vs_float16(self) -> float:
        return 16.0 / self.bits_per_coordinate

    def to_json(self) -> dict:
        return {"method": self.method.value, "dim": self.dim, "bits": self.bits, "seed": self.seed}

    @classmethod
    def from_json(cls, obj: dict) -> "QuantConfig":
        return cls(QuantMethod.parse(obj["method"]), int(obj["dim"]), int(obj["bits"]), int(obj["seed"]))


@dataclass(frozen=True)
class ChannelQuantConfig:
    """Per-channel key quantisation: any dim 1...1024, groups of ``group_size`` tokens."""
    dim: int
    bits: int
    group_size: int = 64

    default_group_size = 64
    max_input_magnitude = 65504.0    # fp16 range; ChannelQuantConfig.maxInputMagnitude

    def __post_init__(self):
        d, b, g = _as_int(self.dim), _as_int(self.bits), _as_int(self.group_size)
        if d is None or not 1 <= d <= MAX_DIMENSION:
            raise InvalidInput(f"per-channel dimension {self.dim} must be in 1...{MAX_DIMENSION}")
        if b is None or b not in SUPPORTED_BITS:
            raise InvalidBitWidth(self.bits)
        if g is None or not 1 <= g <= 65536:
            raise InvalidInput(f"group size {self.group_size} must be in 1...65536")
        object.__setattr__(self, "dim", d)
        object.__setattr__(self, "bits", b)
        object.__setattr__(self, "group_size", g)

    @property
    def code_stride(self) -> int:
        return code_stride_bytes(self.dim, self.bits)

    @property
    def range_stride(self) -> int:
        """Bytes of fp16 ranges per group: ``dim`` minima then ``dim`` maxima."""
        return self.dim * 2 * 2

    def group_count(self, tokens: int) -> int:
        return (tokens + self.group_size - 1) // self.group_size

    @property
    def bits_per_coordinate(self) -> float:
        return self.code_stride * 8 / self.dim + self.range_stride * 8 / (self.dim * self.group_size)

    @property
    def compression_ratio(self) -> float:
        return 32.0 / self.bits_per_coordinate

    @property
    def compression_ratio_vs_float16(self) -> float:
        return 16.0 / self.bits_per_coordinate

    def to_json(self) -> dict:
        return {"dim": self.dim, "bits": self.bits, "groupSize": self.group_size}

    @classmethod
    def from_json(cls, obj: dict) -> "ChannelQuantConfig":
        return cls(int(obj["dim"]), int(obj["bits"]), int(obj["groupSize"]))
