"""pitch_b200: B200-native (sm_100a) KV-cache codec with the API of SwiftCham/PITCH.

* ``PITCH`` - the facade (array API and stream-ordered GPU-resident API).
* ``pitch_b200.pitch_reference`` - drop-in for the reference's NumPy specification module.
* ``KVCache`` - a compressed cache sharded by (layer, KV head) with one-launch whole-cache decode.

All compute runs in hand-written CUDA kernels behind the C ABI in
``include/pitch_b200.h``; there is no CPU fallback.
"""
from .config import DEFAULT_SEED, ChannelQuantConfig, QuantConfig, QuantMethod, code_stride_bytes
from .containers import ChannelCompressedBlock, CompressedBatch, half_to_float
from .errors import (ConfigurationMismatch, DecodingFailed, DeviceNotSupported, EncodingFailed, InvalidBitWidth,
                     InvalidDimension, InvalidInput, KernelUnavailable, PITCHError)

__all__ = [
    "PITCH", "KVCache", "DEFAULT_SEED", "QuantMethod", "QuantConfig", "ChannelQuantConfig", "CompressedBatch",
    "ChannelCompressedBlock", "code_stride_bytes", "half_to_float", "PITCHError", "InvalidInput",
    "InvalidBitWidth", "InvalidDimension", "ConfigurationMismatch", "KernelUnavailable", "EncodingFailed",
    "DecodingFailed", "DeviceNotSupported",
]


def __getattr__(name):
    # torch is only needed by the classes that touch the GPU; keep `import pitch_b200` light
    if name == "PITCH":
        from .codec import PITCH
        return PITCH
    if name == "KVCache":
        from .cache import KVCache
        return KVCache
    raise AttributeError(name)
