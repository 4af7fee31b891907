"""Host-side containers for compressed data and their JSON wire format.

``CompressedBatch`` mirrors Sources/PITCH/Models/CompressedBatch.swift:13-121 and
``ChannelCompressedBlock`` mirrors Sources/PITCH/PerChannel.swift:72-168: same
fields, validation, append / slice rules, storage accounting (including the
16-byte header) and the same JSON keys (``formatVersion`` 3 and 1, ``codes`` as
base64, ``scales`` as numbers, ``ranges`` as uint16 bit patterns), so blobs
interchange with the Swift library's ``Codable`` output.
"""
from __future__ import annotations

import base64
import json

import numpy as np

from .config import ChannelQuantConfig, QuantConfig
from .errors import ConfigurationMismatch, InvalidInput

HEADER_BYTE_COUNT = 16


class CompressedBatch:
    """Vectors sharing one QuantConfig: vector i's codes are bytes
    [i*code_stride, (i+1)*code_stride) of ``codes``; its side information is ``scales[i]``."""
    format_version = 3
    header_byte_count = HEADER_BYTE_COUNT

    def __init__(self, config: QuantConfig, codes, scales, _unchecked: bool = False):
        self.config = config
        self.codes = bytes(codes)
        self.scales = np.ascontiguousarray(scales, dtype=np.float32).reshape(-1)
        if not _unchecked:
            self.validate()

    @property
    def count(self) -> int:
        return int(self.scales.shape[0])

    def validate(self) -> None:
        if self.scales.size == 0:
            raise InvalidInput("a batch must contain at least one vector")
        expected = self.count * self.config.code_stride
        if len(self.codes) != expected:
            raise InvalidInput(f"codes is {len(self.codes)} bytes; expected {expected} for {self.count} vectors")
        if not (np.isfinite(self.scales).all() and (self.scales >= 0).all()):
            raise InvalidInput("scales must be finite and non-negative")

    def append(self, other: "CompressedBatch") -> None:
        if other.config != self.config:
            raise ConfigurationMismatch("cannot append a batch with a different config")
        self.codes += other.codes
        self.scales = np.concatenate([self.scales, other.scales])

    def vectors(self, start: int, stop: int) -> "CompressedBatch":
        """The vectors in [start, stop) as a new batch."""
        if start < 0 or stop > self.count or start >= stop:
            raise InvalidInput(f"range {start}..<{stop} is outside 0..<{self.count}")
        s = self.config.code_stride
        return CompressedBatch(self.config, self.codes[start * s:stop * s], self.scales[start:stop].copy(),
                               _unchecked=True)

    def __eq__(self, other):
        return (isinstance(other, CompressedBatch) and self.config == other.config and self.codes == other.codes
                and self.scales.tobytes() == other.scales.tobytes())

    # ---- storage accounting (CompressedBatch.swift:70-92) ----
    @property
    def payload_byte_count(self) -> int:
        return len(self.codes)

    @property
    def side_information_byte_count(self) -> int:
        return self.count * 4 + HEADER_BYTE_COUNT

    @property
    def stored_byte_count(self) -> int:
        return self.payload_byte_count + self.side_information_byte_count

    @property
    def original_byte_count(self) -> int:
        return self.count * self.config.dim * 4

    @property
    def compression_ratio(self) -> float:
        return self.original_byte_count / self.stored_byte_count

    @property
    def compression_ratio_vs_float16(self) -> float:
        return self.compression_ratio / 2

    @property
    def bits_per_coordinate(self) -> float:
        return self.stored_byte_count * 8 / (self.count * self.config.dim)

    # ---- JSON (CompressedBatch.swift:95-121) ----
    def to_json(self) -> str:
        return json.dumps({"formatVersion": self.format_version, "config": self.config.to_json(),
                           "codes": base64.b64encode(self.codes).decode(),
                           "scales": [float(s) for s in self.scales]})

    @classmethod
    def from_json(cls, text) -> "CompressedBatch":
        obj = json.loads(text)
        version = obj["formatVersion"]
        if version != cls.format_version:
            raise InvalidInput(f"Unsupported PITCH format version {version}; expected {cls.format_version}")
        return cls(QuantConfig.from_json(obj["config"]), base64.b64decode(obj["codes"]),
                   np.asarray(obj["scales"], dtype=np.float32))


class ChannelCompressedBlock:
    """One head's keys, token-major: packed codes plus fp16 ranges (uint16 bit patterns,
    layout [group][min|max][channel])."""
    format_version = 1
    header_byte_count = HEADER_BYTE_COUNT

    def __init__(self, config: ChannelQuantConfig, codes, ranges, _unchecked: bool = False):
        self.config = config
        self.codes = bytes(codes)
        self.ranges = np.ascontiguousarray(ranges, dtype=np.uint16).reshape(-1)
        if not _unchecked:
            self.validate()

    @property
    def count(self) -> int:
        return len(self.codes) // self.config.code_stride

    @property
    def group_count(self) -> int:
        return self.config.group_count(self.count)

    def validate(self) -> None:
        s = self.config.code_stride
        if len(self.codes) == 0 or len(self.codes) % s:
            raise InvalidInput(f"codes is {len(self.codes)} bytes; expected a positive multiple of {s}")
        expected = self.group_count * 2 * self.config.dim
        if self.ranges.size != expected:
            raise InvalidInput(f"ranges has {self.ranges.size} values; expected {expected} for {self.count} tokens")
        r = self.ranges.view(np.float16).astype(np.float32).reshape(self.group_count, 2, self.config.dim)
        bad = ~(np.isfinite(r[:, 0]) & np.isfinite(r[:, 1]) & (r[:, 0] <= r[:, 1]))
        if bad.any():
            g, ch = np.argwhere(bad)[0]
            raise InvalidInput(f"group {g} channel {ch}: range [{r[g, 0, ch]}, {r[g, 1, ch]}] is invalid")

    def range(self, group: int, channel: int) -> tuple[float, float]:
        d = self.config.dim
        h = self.ranges.view(np.float16)
        return float(h[group * 2 * d + channel]), float(h[group * 2 * d + d + channel])

    def append(self, other: "ChannelCompressedBlock") -> None:
        if other.config != self.config:
            raise ConfigurationMismatch("cannot append a block with a different config")
        if self.count % self.config.group_size:
            raise InvalidInput(f"cannot append after a partial group ({self.count} tokens, "
                               f"group size {self.config.group_size})")
        self.codes += other.codes
        self.ranges = np.concatenate([self.ranges, other.ranges])

    def __eq__(self, other):
        return (isinstance(other, ChannelCompressedBlock) and self.config == other.config
                and self.codes == other.codes and self.ranges.tobytes() == other.ranges.tobytes())

    # ---- storage accounting (PerChannel.swift:130-140) ----
    @property
    def payload_byte_count(self) -> int:
        return len(self.codes)

    @property
    def side_information_byte_count(self) -> int:
        return self.ranges.size * 2 + HEADER_BYTE_COUNT

    @property
    def stored_byte_count(self) -> int:
        return self.payload_byte_count + self.side_information_byte_count

    @property
    def original_byte_count(self) -> int:
        return self.count * self.config.dim * 4

    @property
    def compression_ratio(self) -> float:
        return self.original_byte_count / self.stored_byte_count

    @property
    def compression_ratio_vs_float16(self) -> float:
        return self.compression_ratio / 2

    @property
    def bits_per_coordinate(self) -> float:
        return self.stored_byte_count * 8 / (self.count * self.config.dim)

    # ---- JSON (PerChannel.swift:143-168) ----
    def to_json(self) -> str:
        return json.dumps({"formatVersion": self.format_version, "config": self.config.to_json(),
                           "codes": base64.b64encode(self.codes).decode(),
                           "ranges": [int(r) for r in self.ranges]})

    @classmethod
    def from_json(cls, text) -> "ChannelCompressedBlock":
        obj = json.loads(text)
        version = obj["formatVersion"]
        if version != cls.format_version:
            raise InvalidInput(f"Unsupported PITCH per-channel format version {version}; "
                               f"expected {cls.format_version}")
        return cls(ChannelQuantConfig.from_json(obj["config"]), base64.b64decode(obj["codes"]),
                   np.asarray(obj["ranges"], dtype=np.uint16))


def half_to_float(h: int) -> float:
    """IEEE binary16 bit pattern -> float (PerChannel.swift:171-180)."""
    return float(np.array([h], dtype=np.uint16).view(np.float16)[0])
