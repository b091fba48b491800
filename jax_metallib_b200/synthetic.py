"""Seeded synthetic inputs for the five quantized-matmul workloads.

No dataset is involved: every tensor is drawn from the distribution the
workload definition names, with ``numpy.random.default_rng(1000*config+index)``
(host generators, used by the parity tests at sizes a CPU can check) or a
seeded ``torch.Generator`` on the device (bench-sized tensors that would not
fit through the host).  Model names are shape lists only; weights are random.
"""

from __future__ import annotations

import numpy as np

try:
    import ml_dtypes

    _BF16 = ml_dtypes.bfloat16
except Exception:  # pragma: no cover
    _BF16 = None


def _rng(config: int, index: int = 0) -> np.random.Generator:
    return np.random.default_rng(1000 * config + index)


def to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """float32 -> bf16 bit patterns (uint16), round-to-nearest-even."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def config1(M=32, K=1024, N=1024):
    """int8 per-channel weight-only, f32 activations."""
    r = _rng(1)
    x = r.standard_normal((M, K)).astype(np.float32)
    w = r.integers(-127, 128, size=(K, N), dtype=np.int64).astype(np.int8)
    scale = r.uniform(0.005, 0.02, size=(N,)).astype(np.float32)
    return dict(x=x, w=w, scale=scale)


def config2(M=2048, K=4096, N=4096):
    """int8 x int8 -> int32 with f32 row/column rescale."""
    r = _rng(2)
    a = r.integers(-127, 128, size=(M, K), dtype=np.int64).astype(np.int8)
    b = r.integers(-127, 128, size=(K, N), dtype=np.int64).astype(np.int8)
    row = r.uniform(0.01, 0.05, size=(M,)).astype(np.float32)
    col = r.uniform(0.005, 0.02, size=(N,)).astype(np.float32)
    return dict(a=a, b=b, row=row, col=col)


def config3(M=1, K=4096, N=14336, group=128, index=0):
    """int4 asymmetric group-wise weight-only at decode shapes.

    Returns bf16 tensors as uint16 bit patterns plus their f32 values."""
    r = _rng(3, index)
    x = r.standard_normal((M, K)).astype(np.float32)
    x_bits = to_bf16_bits(x)
    q = r.integers(0, 16, size=(K, N), dtype=np.int64).astype(np.uint8)
    wq = (q[0::2] | (q[1::2] << 4)).astype(np.uint8)  # [K/2, N], low nibble = even k
    s = r.uniform(0.002, 0.01, size=(K // group, N)).astype(np.float32)
    s_bits = to_bf16_bits(s)
    z = r.integers(0, 16, size=(K // group, N), dtype=np.int64).astype(np.uint8)
    z_packed = (z[:, 0::2] | (z[:, 1::2] << 4)).astype(np.uint8)
    return dict(x_bits=x_bits, x=bf16_bits_to_f32(x_bits), wq=wq, s_bits=s_bits, s=bf16_bits_to_f32(s_bits), z=z,
                z_packed=z_packed, group=group)


def config5_layer_shapes(d_model=8192, ffn=28672, qkv=10240):
    """(name, K, N) of the four linears of one Llama-3-70B-shaped layer; gate and
    up are one fused [d_model, 2*ffn] projection."""
    return [("qkv", d_model, qkv), ("o", d_model, d_model), ("gate_up", d_model, 2 * ffn), ("down", ffn, d_model)]


def config5_small(M=256, K=512, N=384, index=0):
    """Reduced-shape instance of the int8 per-channel bf16 linears (host arrays)."""
    r = _rng(5, index)
    x = r.standard_normal((M, K)).astype(np.float32)
    x_bits = to_bf16_bits(x)
    w = r.integers(-127, 128, size=(K, N), dtype=np.int64).astype(np.int8)
    scale = r.uniform(0.005, 0.02, size=(N,)).astype(np.float32)
    return dict(x_bits=x_bits, x=bf16_bits_to_f32(x_bits), w=w, scale=scale)


# ---- device-side generators for bench-sized tensors -------------------------

def torch_generator(device, config: int, index: int = 0):
    import torch

    g = torch.Generator(device=device)
    g.manual_seed(1000 * config + index)
    return g


def device_int8(shape, device, gen):
    """Uniform integers in [-127, 127] as int8, generated on the device."""
    import torch

    return torch.randint(-127, 128, shape, dtype=torch.int8, device=device, generator=gen)


def device_uniform(shape, lo, hi, device, gen, dtype=None):
    import torch

    t = torch.rand(shape, dtype=torch.float32, device=device, generator=gen) * (hi - lo) + lo
    return t if dtype is None else t.to(dtype)


def device_normal(shape, device, gen, dtype=None):
    import torch

    t = torch.randn(shape, dtype=torch.float32, device=device, generator=gen)
    return t if dtype is None else t.to(dtype)
