"""Operator API of the quantized-matmul path, with the reference's signatures.

Mirrors ``src/jax_plugins/silicon/quantized.py`` of jax-metallib:
``mx_quantize`` / ``mx_dequantize`` / ``quantized_matmul`` (:125, :212, :995)
and ``affine_quantize`` / ``affine_dequantize`` / ``affine_quantized_matmul``
(:276, :408, :1077): same names, keyword arguments, packing formats, shapes,
dtypes and ``ValueError`` behaviour.  As in the reference, quantise/dequantise
run on the host in NumPy (they are offline weight preparation); the two matmul
functions launch the fused dequant-GEMM kernels of ``libqmm.so``.

Differences, on purpose: where the reference falls back to CPU dequantise +
matmul when its GPU launcher is unavailable or the dtype is unsupported
(:1028-1031, :1045-1049, :1107-1112), this implementation raises — the CUDA
library is the only execution path.  Inputs may be NumPy arrays (copied to the
device and back, like the reference's ``metal.execute`` host copies,
src/jax_plugins/silicon/metal.py:259-331) or CUDA torch tensors (returned as
torch tensors, no host copies).
"""

from __future__ import annotations

import numpy as np

from . import _lib

_MX_MODES = {
    "mxfp4": {"bits": 4, "group_size": 32, "scale_type": "e8m0"},
    "mxfp8": {"bits": 8, "group_size": 32, "scale_type": "e8m0"},
    "nvfp4": {"bits": 4, "group_size": 16, "scale_type": "e4m3"},
}
_AFFINE_DEFAULTS = {"bits": 4, "group_size": 64}

# ---------------------------------------------------------------------------
# element codecs (table driven)
# ---------------------------------------------------------------------------
_E2M1_VALUES = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)
# midpoints between neighbouring magnitudes and the code an exact midpoint takes (the even one)
_E2M1_MID = (_E2M1_VALUES[:-1] + _E2M1_VALUES[1:]) / 2
_E2M1_MID_CODE = np.array([0, 2, 2, 4, 4, 6, 6], dtype=np.uint8)


def _fp4_e2m1_quantize(x):
    x = np.asarray(x, dtype=np.float32)
    a = np.abs(x)
    below = (a[..., None] > _E2M1_MID).sum(axis=-1).astype(np.uint8)  # midpoints strictly below |x|
    code = below.copy()
    for mid, c in zip(_E2M1_MID, _E2M1_MID_CODE):
        code = np.where(a == mid, c, code)
    return ((np.signbit(x).astype(np.uint8) << 3) | code).astype(np.uint8)


def _fp4_e2m1_dequantize(bits):
    bits = np.asarray(bits)
    mag = _E2M1_VALUES[(bits & 0x7).astype(np.intp)]
    return np.where(bits & 0x8, -mag, mag).astype(np.float32)


def _e4m3_table() -> np.ndarray:
    codes = np.arange(128)
    e, m = codes >> 3, codes & 7
    vals = np.where(e == 0, m * 2.0**-9, (8 + m) * 2.0 ** (e - 10.0))
    vals = vals.astype(np.float32)
    vals[127] = np.nan
    return vals


_E4M3_ABS = _e4m3_table()  # index = 7-bit magnitude code


def _fp8_e4m3_dequantize(bits):
    bits = np.asarray(bits, dtype=np.uint8)
    mag = _E4M3_ABS[(bits & 0x7F).astype(np.intp)]
    return np.where(bits & 0x80, -mag, mag).astype(np.float32)


def _fp8_e4m3_quantize(x):
    x = np.asarray(x, dtype=np.float32)
    neg = np.signbit(x)
    a = np.abs(np.clip(x, -448.0, 448.0))
    a = np.where(np.isnan(a), np.float32(448.0), a)
    finite = _E4M3_ABS[:127]
    hi = np.minimum(np.searchsorted(finite, a, side="left"), 126)
    lo = np.maximum(hi - 1, 0)
    up = (finite[hi] - a < a - finite[lo]) | ((finite[hi] - a == a - finite[lo]) & (hi % 2 == 0))
    return (np.where(up, hi, lo).astype(np.uint8) | (neg.astype(np.uint8) << 7)).astype(np.uint8)


def _fp8_e8m0_quantize(x):
    x = np.asarray(x)
    if x.dtype not in (np.float32, np.float64):
        x = x.astype(np.float32)
    bad = ~np.isfinite(x)
    tiny = x.dtype.type(np.finfo(np.float32).tiny)
    n = np.clip(np.round(np.log2(np.where(bad, x.dtype.type(1), np.maximum(x, tiny)))).astype(np.int32), -127, 127)
    return np.where(bad, 0xFF, n + 127).astype(np.uint8)


def _fp8_e8m0_dequantize(bits):
    bits = np.asarray(bits, dtype=np.uint8)
    v = np.ldexp(np.float32(1.0), np.minimum(bits.astype(np.int32) - 127, 127)).astype(np.float32)
    return np.where(bits == 0xFF, np.float32(np.nan), v).astype(np.float32)


# ---------------------------------------------------------------------------
# array plumbing
# ---------------------------------------------------------------------------

def _is_torch(x) -> bool:
    return type(x).__module__.split(".")[0] == "torch"


def _np(x, dtype=None) -> np.ndarray:
    if _is_torch(x):
        x = x.detach().cpu().numpy()
    return np.asarray(x, dtype=dtype)


def _mode(mode):
    if mode not in _MX_MODES:
        raise ValueError(f"Unknown mode '{mode}'. Must be one of {list(_MX_MODES.keys())}")
    return _MX_MODES[mode]


def _bits_ok(bits):
    if bits not in (2, 3, 4, 8):
        raise ValueError(f"bits must be 2, 3, 4, or 8; got {bits}")


# ---------------------------------------------------------------------------
# MX formats
# ---------------------------------------------------------------------------

def mx_quantize(w, *, mode: str = "mxfp4") -> tuple:
    """Quantise ``w[..., K]`` to an MX format; returns ``(packed uint8, scales uint8)``.

    fp4 modes pack two elements per byte (element i in the low nibble), so
    ``packed`` is ``[..., K//2]``; fp8 is ``[..., K]``; ``scales`` is
    ``[..., K//group_size]`` (reference: quantized.py:125-209)."""
    cfg = _mode(mode)
    w = _np(w, np.float32)
    K = w.shape[-1]
    gs = cfg["group_size"]
    if K % gs != 0:
        raise ValueError(f"Last dimension ({K}) must be divisible by group_size ({gs})")
    grp = w.reshape(-1, K // gs, gs)
    gmax = np.abs(grp).max(axis=-1)
    top = np.float32(6.0 if cfg["bits"] == 4 else 448.0)
    with np.errstate(invalid="ignore"):
        raw = np.where(gmax != 0, gmax / top, np.float32(0)).astype(np.float32)
    if cfg["scale_type"] == "e8m0":
        sbits = _fp8_e8m0_quantize(raw)
        sval = _fp8_e8m0_dequantize(sbits)
    else:
        sbits = _fp8_e4m3_quantize(raw)
        sval = _fp8_e4m3_dequantize(sbits)
    with np.errstate(invalid="ignore", divide="ignore"):
        unit = np.where(sval[..., None] != 0, grp / sval[..., None], np.float32(0)).astype(np.float32)
    if cfg["bits"] == 4:
        codes = _fp4_e2m1_quantize(unit).reshape(-1, K)
        packed = (codes[:, 0::2] | (codes[:, 1::2] << 4)).astype(np.uint8).reshape(*w.shape[:-1], K // 2)
    else:
        packed = _fp8_e4m3_quantize(unit).reshape(*w.shape[:-1], K)
    return packed, sbits.reshape(*w.shape[:-1], K // gs)


def mx_dequantize(packed, scales, *, mode: str = "mxfp4", shape=None, dtype=np.float32):
    """Inverse of :func:`mx_quantize` (reference: quantized.py:212-273)."""
    cfg = _mode(mode)
    packed = _np(packed, np.uint8)
    scales = _np(scales, np.uint8)
    if cfg["bits"] == 4 and shape is None:
        raise ValueError("shape is required for FP4 dequantization")
    K = shape[-1] if shape is not None else packed.shape[-1]
    gs = cfg["group_size"]
    rows = packed.reshape(-1, packed.shape[-1])
    if cfg["bits"] == 4:
        codes = np.empty((rows.shape[0], rows.shape[1] * 2), dtype=np.uint8)
        codes[:, 0::2] = rows & 0xF
        codes[:, 1::2] = rows >> 4
        elems = _fp4_e2m1_dequantize(codes[:, :K])
    else:
        elems = _fp8_e4m3_dequantize(rows[:, :K])
    sv = (_fp8_e8m0_dequantize(scales) if cfg["scale_type"] == "e8m0" else _fp8_e4m3_dequantize(scales))
    sv = sv.reshape(-1, K // gs)
    out = (elems.reshape(-1, K // gs, gs) * sv[:, :, None]).reshape(-1, K)
    if shape is not None:
        out = out.reshape(shape)
    return out.astype(dtype)


# ---------------------------------------------------------------------------
# affine formats
# ---------------------------------------------------------------------------

def _pack_bits(q: np.ndarray, bits: int) -> np.ndarray:
    """``q[rows, K]`` small integers -> little-endian bit stream in uint32 words."""
    rows, K = q.shape
    per = {2: 16, 4: 8}.get(bits)
    if per:
        shifts = (np.arange(per, dtype=np.uint32) * bits)[None, None, :]
        v = q.reshape(rows, K // per, per).astype(np.uint32) << shifts
        return np.bitwise_or.reduce(v, axis=-1).astype(np.uint32)
    # 3-bit: 32 values -> 96 bits -> 3 words
    bitsarr = ((q.reshape(rows, K // 32, 32, 1).astype(np.uint32) >> np.arange(3, dtype=np.uint32)) & 1)
    stream = bitsarr.reshape(rows, K // 32, 3, 32)  # 96 bits, little endian, split in 3 words
    weights = (np.uint64(1) << np.arange(32, dtype=np.uint64))
    return (stream.astype(np.uint64) * weights).sum(axis=-1).astype(np.uint32).reshape(rows, K * 3 // 32)


def _unpack_bits(words: np.ndarray, bits: int, K: int) -> np.ndarray:
    rows = words.shape[0]
    if bits in (2, 4):
        per = 32 // bits
        shifts = (np.arange(per, dtype=np.uint32) * bits)[None, None, :]
        v = (words.astype(np.uint32)[:, :, None] >> shifts) & np.uint32((1 << bits) - 1)
        return v.reshape(rows, -1)[:, :K].astype(np.int32)
    w3 = words.astype(np.uint32).reshape(rows, -1, 3, 1)
    stream = ((w3 >> np.arange(32, dtype=np.uint32)) & 1).reshape(rows, -1, 32, 3)  # [.., value, bit]
    v = (stream * np.array([1, 2, 4], dtype=np.uint32)).sum(axis=-1)
    return v.reshape(rows, -1)[:, :K].astype(np.int32)


def affine_quantize(w, *, bits: int = 4, group_size: int = 64) -> tuple:
    """Per-group min/max affine quantisation; returns ``(packed, scales f32, biases f32)``.

    4-bit packs 8 values per uint32 (value j at bits 4j), 8-bit is uint8, 3-bit
    packs 32 values per 3 words, 2-bit 16 per word (reference: quantized.py:276-405)."""
    _bits_ok(bits)
    w = _np(w, np.float32)
    K = w.shape[-1]
    if K % group_size != 0:
        raise ValueError(f"Last dimension ({K}) must be divisible by group_size ({group_size})")
    levels = (1 << bits) - 1
    grp = w.reshape(-1, K // group_size, group_size)
    lo = grp.min(axis=-1)
    hi = grp.max(axis=-1)
    step = np.where(hi != lo, (hi.astype(np.float64) - lo.astype(np.float64)) / levels, 1.0)
    step32 = step.astype(np.float32)
    q = np.clip(np.round((grp - lo[..., None]) / step32[..., None]).astype(np.int32), 0, levels)
    q = q.reshape(-1, K)
    lead = w.shape[:-1]
    if bits == 8:
        packed = q.astype(np.uint8).reshape(*lead, K)
    else:
        words = _pack_bits(q, bits)
        packed = words.reshape(*lead, words.shape[-1])
    gshape = (*lead, K // group_size)
    return packed, step32.reshape(gshape), lo.astype(np.float32).reshape(gshape)


def affine_dequantize(packed, scales, biases, *, bits: int = 4, group_size: int = 64, shape=None, dtype=np.float32):
    """``scale * q + bias`` per group (reference: quantized.py:408-482)."""
    _bits_ok(bits)
    packed = _np(packed)
    scales = _np(scales, np.float32)
    biases = _np(biases, np.float32)
    if bits != 8 and shape is None:
        raise ValueError("shape is required for sub-byte dequantization")
    K = shape[-1] if shape is not None else packed.shape[-1]
    rows = packed.reshape(-1, packed.shape[-1])
    q = rows[:, :K].astype(np.int32) if bits == 8 else _unpack_bits(rows, bits, K)
    ng = K // group_size
    out = scales.reshape(-1, ng, 1) * q.reshape(-1, ng, group_size).astype(np.float32) + biases.reshape(-1, ng, 1)
    out = out.reshape(-1, K)
    if shape is not None:
        out = out.reshape(shape)
    return out.astype(dtype)


# ---------------------------------------------------------------------------
# fused matmuls (CUDA only)
# ---------------------------------------------------------------------------

def _to_device(a, torch, device, dtype=None):
    if _is_torch(a):
        t = a.to(device)
    else:
        t = torch.from_numpy(np.ascontiguousarray(a)).to(device)
    if dtype is not None and t.dtype != dtype:
        t = t.to(dtype)
    return t.contiguous()


def _launch_matmul(x, call, N, K, out_dtype):
    """Shared driver: flatten batch dims, run the kernel in x's dtype, cast, restore dims."""
    import torch

    if not torch.cuda.is_available():
        raise RuntimeError("quantized matmul needs a CUDA device: this build has no CPU fallback")
    _lib.load()
    is_t = _is_torch(x)
    device = x.device if (is_t and x.is_cuda) else torch.device("cuda", torch.cuda.current_device())
    xt = _to_device(x, torch, device)
    if xt.dtype == torch.float32:
        tag = _lib.QMM_F32
    elif xt.dtype == torch.float16:
        tag = _lib.QMM_F16
    else:
        raise TypeError(f"activations must be float32 or float16, got {xt.dtype}")
    if xt.shape[-1] != K:
        raise ValueError(f"x has inner dimension {xt.shape[-1]}, expected K={K}")
    x2 = xt.reshape(-1, K)
    M = x2.shape[0]
    y = torch.empty((M, N), dtype=xt.dtype, device=device)
    call(x2, y, M, tag, device, torch)
    y = y.reshape(*xt.shape[:-1], N)
    if is_t:
        if out_dtype is not None and not isinstance(out_dtype, torch.dtype):
            out_dtype = getattr(torch, np.dtype(out_dtype).name)
        return y if out_dtype is None else y.to(out_dtype)
    out = y.cpu().numpy()
    return out if out_dtype is None else out.astype(out_dtype)


def quantized_matmul(x, w_packed, scales, *, mode: str = "mxfp4", K: int, out_dtype=None):
    """``x[..., M, K] @ dequant(w_packed[N, K//pack], scales[N, K//group])^T`` (reference: quantized.py:995-1074)."""
    cfg = _mode(mode)
    N = w_packed.shape[0]
    if K % cfg["group_size"] != 0:
        raise ValueError(f"K ({K}) must be divisible by group_size ({cfg['group_size']})")

    def call(x2, y, M, tag, device, torch):
        wp = _to_device(w_packed, torch, device, torch.uint8)
        sc = _to_device(scales, torch, device, torch.uint8)
        pack = 2 if cfg["bits"] == 4 else 1
        if wp.shape != (N, K // pack) or sc.shape != (N, K // cfg["group_size"]):
            raise ValueError(f"packed weights {tuple(wp.shape)} / scales {tuple(sc.shape)} do not match N={N}, K={K}")
        _lib.check(_lib.load().qmm_mx_matmul(x2.data_ptr(), wp.data_ptr(), sc.data_ptr(), y.data_ptr(), M, N, K,
                                             _lib.MX_MODE_IDS[mode], tag, torch.cuda.current_stream().cuda_stream))

    return _launch_matmul(x, call, N, K, out_dtype)


def affine_quantized_matmul(x, w_packed, scales, biases, *, bits: int = 4, group_size: int = 64, K: int,
                            out_dtype=None):
    """``x[..., M, K] @ dequant(w_packed, scales, biases)^T`` for 4- and 8-bit affine weights
    (reference: quantized.py:1077-1152)."""
    _bits_ok(bits)
    if bits not in (4, 8):
        raise ValueError(f"fused affine matmul kernels exist for bits 4 and 8; got {bits}")
    if K % group_size != 0:
        raise ValueError(f"K ({K}) must be divisible by group_size ({group_size})")
    N = w_packed.shape[0]

    def call(x2, y, M, tag, device, torch):
        if bits == 4:
            wp_np = w_packed if _is_torch(w_packed) else np.ascontiguousarray(w_packed, dtype=np.uint32).view(np.int32)
            wp = _to_device(wp_np, torch, device)
            want = (N, K // 8)
        else:
            wp = _to_device(w_packed, torch, device, torch.uint8)
            want = (N, K)
        sc = _to_device(scales, torch, device, torch.float32)
        bi = _to_device(biases, torch, device, torch.float32)
        if tuple(wp.shape) != want or sc.shape != (N, K // group_size) or bi.shape != sc.shape:
            raise ValueError(f"packed weights {tuple(wp.shape)} / scales {tuple(sc.shape)} do not match N={N}, K={K}")
        _lib.check(_lib.load().qmm_affine_matmul(x2.data_ptr(), wp.data_ptr(), sc.data_ptr(), bi.data_ptr(),
                                                 y.data_ptr(), M, N, K, bits, group_size, tag,
                                                 torch.cuda.current_stream().cuda_stream))

    return _launch_matmul(x, call, N, K, out_dtype)
