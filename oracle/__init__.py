"""CPU oracles for the KV-cache codec (test infrastructure only).

``spec_np``    - NumPy restatement of the reference's float64 specification.
``kernel_f32`` - ctypes wrapper of a C restatement of the float32 kernel arithmetic.

Only the test suite, the smoke check and the CPU-baseline leg of the benchmark
may import this package; the product package never does.
"""
