"""B200-native quantized-matmul hot path behind jax-metallib's operator boundary.

``libqmm.so`` (hand-written sm_100a kernels behind a C ABI, declared in
``include/qmm.h``) is the product; this package is the host-side mirror of the
reference's operator API (``quantized``) plus wrappers for the StableHLO-level
quantized matmuls (``ops``).  Importing the package does not load the library;
the first operator call does, and raises if it is missing.
"""

__all__ = ["ops", "quantized", "synthetic"]
