"""Exceptions: one class per case of the reference's ``PITCHError``
(Sources/PITCH/Core/PITCHError.swift:10-19) and per ``pitch_status`` of the C ABI."""
from __future__ import annotations


class PITCHError(Exception):
    """Base class; ``status`` is the C ABI's ``pitch_status`` code."""
    status = -1


class InvalidInput(PITCHError, ValueError):
    status = 1          # .invalidInput


class InvalidBitWidth(PITCHError, ValueError):
    status = 2          # .invalidBitWidth

    def __init__(self, bits):
        self.bits = bits
        super().__init__(f"Invalid bit width {bits}. Must be in 2...8.")


class InvalidDimension(PITCHError, ValueError):
    status = 3          # .invalidDimension

    def __init__(self, dim):
        self.dim = dim
        super().__init__(f"Invalid dimension {dim}. Must be a power of two in [2, 1024].")


class ConfigurationMismatch(PITCHError, ValueError):
    status = 4          # .configurationMismatch


class KernelUnavailable(PITCHError, RuntimeError):
    status = 5          # .shaderCompilationFailed: the native library or a kernel image is missing


class EncodingFailed(PITCHError, RuntimeError):
    status = 6          # .encodingFailed


class DecodingFailed(PITCHError, RuntimeError):
    status = 7          # .decodingFailed


class DeviceNotSupported(PITCHError, RuntimeError):
    status = 8          # .metalNotSupported: no usable CUDA device


def from_status(status: int, detail: str) -> PITCHError:
    """Exception for a non-zero status returned by the C ABI."""
    if status == 1:
        return InvalidInput(detail)
    if status in (2, 3):
        # the ABI's message carries the offending value; keep it verbatim
        err = (InvalidBitWidth if status == 2 else InvalidDimension).__new__(
            InvalidBitWidth if status == 2 else InvalidDimension)
        Exception.__init__(err, detail)
        return err
    cls = {4: ConfigurationMismatch, 5: KernelUnavailable, 6: EncodingFailed,
           7: DecodingFailed, 8: DeviceNotSupported}.get(status, PITCHError)
    return cls(detail or f"status {status}")
