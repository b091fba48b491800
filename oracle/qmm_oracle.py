"""CPU oracle for the quantized-matmul hot path.  TEST INFRASTRUCTURE ONLY.

This module is the checker, never the product: only ``tests/``, the smoke
check and the ``cpu_baseline`` / ``--impl reference`` legs of ``bench.py`` may
import it.  The shipped path (``jax_metallib_b200``) never calls into it and
raises when its CUDA library is missing.

It restates, in vectorised NumPy, the arithmetic the reference pins for this
path.  Each function cites the reference file:line it follows (paths are
relative to the reference project root):

* element codecs and (de)quantisers of the operator API:
  ``src/jax_plugins/silicon/quantized.py:53-122`` (E2M1 / E4M3 / E8M0),
  ``:125-273`` (MX), ``:276-482`` (affine);
* the fused dequant-GEMM kernels' arithmetic order (``scale*q + bias`` in f32,
  product in f32, f32 accumulate, one final cast):
  ``src/jax_plugins/silicon/quantized.py:528-753`` and ``:772-957``;
* StableHLO semantics of the dequant chain: integer dot exact in int32
  (``src/pjrt_plugin/ops/binary_ops.mm:438-475``), ``convert`` int->float exact
  and float->bf16 round-to-nearest-even with NaN -> sign|0x7FC0
  (``src/pjrt_plugin/ops/shape_ops.mm:726-731,768-770``), logical right shift
  (``src/pjrt_plugin/ops/bitwise_ops.mm:250-292``), dot accumulating in f32 and
  rounding once to the declared result type
  (``src/pjrt_plugin/ops/binary_ops.mm:775-805``).

Pinning: ``tests/golden/make_golden.py`` imports the reference's own
``quantized.py`` (through a NumPy stand-in for ``jax.numpy``) and stores its
outputs; ``tests/test_oracle_golden.py`` checks this restatement against those
fixtures and against the known-answer tables of the reference's
``tests/test_quantized.py``.  The StableHLO-level dequant chain
(convert -> scale/zero-point -> dot_general at int4/int8 weight formats) has no
reference test and the reference's oracle for it (XLA:CPU inside jaxlib 0.11)
is not installable offline: for those functions parity is UNPINNED and the
contract is the stated tolerance against fp32 dequantise-then-dot.
"""

from __future__ import annotations

import numpy as np

try:  # ml_dtypes ships with the image; only used for convenience views
    import ml_dtypes

    BF16 = ml_dtypes.bfloat16
except Exception:  # pragma: no cover
    ml_dtypes = None
    BF16 = None

# --------------------------------------------------------------------------
# bf16 helpers (bit-level, so they do not depend on ml_dtypes rounding)
# --------------------------------------------------------------------------


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """float32 -> bf16 bit pattern, round-to-nearest-even, NaN -> sign|0x7FC0.

    Follows the rounding the reference applies for f32->bf16 ``convert``
    (src/pjrt_plugin/ops/shape_ops.mm:768-770).
    """
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    rounded = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    out = np.where(nan, ((u >> 16) & 0x8000) | 0x7FC0, rounded)
    return out.astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def round_to_bf16(x: np.ndarray) -> np.ndarray:
    """float32 values rounded to the nearest bf16, returned as float32."""
    return bf16_bits_to_f32(f32_to_bf16_bits(x))


def max_rel_err(out: np.ndarray, ref: np.ndarray) -> float:
    """max|out-ref| / max|ref| — the reference's own definition
    (tests/test_f32_gemm_precision.py:36-37)."""
    out = np.asarray(out, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    denom = max(float(np.max(np.abs(ref))), 1e-30)
    return float(np.max(np.abs(out - ref))) / denom


# --------------------------------------------------------------------------
# StableHLO-level configurations (int8 per-channel, int8 dot, int4 g128, sharded int8 per-channel)
# --------------------------------------------------------------------------


def w8_perchannel_dequant(w_i8: np.ndarray, scale: np.ndarray) -> np.ndarray:
    """``W.astype(f32) * scale[None, :]`` — convert is exact, multiply in f32
    (src/pjrt_plugin/ops/shape_ops.mm:793-829, ops/binary_ops.mm:165-193)."""
    return w_i8.astype(np.float32) * np.asarray(scale, dtype=np.float32)[None, :]


def w8_perchannel_matmul(x: np.ndarray, w_i8: np.ndarray, scale: np.ndarray) -> np.ndarray:
    """fp32 dequantise-then-dot oracle for ``x @ (W.astype(f32) * scale[None,:])``.

    The dot is carried in float64 and rounded once to f32, so that the oracle
    itself is not a source of accumulation-order noise.
    """
    w = w8_perchannel_dequant(w_i8, scale)
    return (np.asarray(x, dtype=np.float64) @ w.astype(np.float64)).astype(np.float32)


def i8_dot_i32(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """Exact integer dot with an int32 accumulator that wraps mod 2**32
    (src/pjrt_plugin/ops/binary_ops.mm:438-475; tests/test_int_dot.py).

    Works for int8 and uint8 operands.  The product is formed in float64 GEMM
    chunks: every partial sum of a K<=2**20 chunk of 8-bit products is below
    2**53, so the float64 result is exact; chunks are then added in int64 and
    wrapped.
    """
    a = np.asarray(a)
    b = np.asarray(b)
    K = a.shape[-1]
    acc = np.zeros(a.shape[:-1] + (b.shape[-1],), dtype=np.int64)
    step = 1 << 16
    for k0 in range(0, K, step):
        part = a[..., k0 : k0 + step].astype(np.float64) @ b[k0 : k0 + step].astype(np.float64)
        acc += part.astype(np.int64)
    return (acc & 0xFFFFFFFF).astype(np.uint32).view(np.int32) if acc.size else acc.astype(np.int32)


def i8_dot_rescale(acc_i32: np.ndarray, row: np.ndarray, col: np.ndarray) -> np.ndarray:
    """``acc.astype(f32) * row[:, None] * col[None, :]`` in exactly that order,
    every step rounded to f32 (StableHLO convert, multiply, multiply)."""
    f = acc_i32.astype(np.float32)
    f = f * np.asarray(row, dtype=np.float32)[:, None]
    f = f * np.asarray(col, dtype=np.float32)[None, :]
    return f


def w4_unpack_k_pairs(wq_u8: np.ndarray) -> np.ndarray:
    """``[K/2, N]`` bytes -> ``[K, N]`` nibbles; the low nibble holds the even k
    (the reference's low-nibble-first convention,
    src/jax_plugins/silicon/quantized.py:189-191,264; and/shift_right_logical
    as in src/pjrt_plugin/ops/bitwise_ops.mm:33-51,250-292)."""
    wq_u8 = np.asarray(wq_u8, dtype=np.uint8)
    lo = wq_u8 & 0xF
    hi = wq_u8 >> 4
    k2, n = wq_u8.shape
    return np.stack([lo, hi], axis=1).reshape(2 * k2, n)


def unpack_u4_pairs_last(z_packed: np.ndarray) -> np.ndarray:
    """``[..., N/2]`` bytes -> ``[..., N]`` nibbles, low nibble = even index."""
    z_packed = np.asarray(z_packed, dtype=np.uint8)
    lo = z_packed & 0xF
    hi = z_packed >> 4
    return np.stack([lo, hi], axis=-1).reshape(z_packed.shape[:-1] + (2 * z_packed.shape[-1],))


def pack_u4_pairs_last(z: np.ndarray) -> np.ndarray:
    z = np.asarray(z, dtype=np.uint8)
    return (z[..., 0::2] | (z[..., 1::2] << 4)).astype(np.uint8)


def w4_groupwise_dequant(wq_u8, scales_f32, zeros_u8, group: int = 128) -> np.ndarray:
    """``w[k,n] = (q[k,n] - z[k//g,n]) * s[k//g,n]`` in f32.

    ``scales_f32`` holds the bf16 scale values widened to f32 (exact)."""
    q = w4_unpack_k_pairs(wq_u8).astype(np.float32)
    K, N = q.shape
    s = np.asarray(scales_f32, dtype=np.float32)
    z = np.asarray(zeros_u8).astype(np.float32)
    q = q.reshape(K // group, group, N)
    w = (q - z[:, None, :]) * s[:, None, :]
    return w.reshape(K, N)


def w4a16_matmul(x_f32, wq_u8, scales_f32, zeros_u8, group: int = 128) -> np.ndarray:
    """fp32 dequantise-then-dot oracle for the int4 group-wise config; returns
    the un-rounded f32 result (callers compare a bf16 device result against it
    with the 1e-2 max-relative-error contract)."""
    w = w4_groupwise_dequant(wq_u8, scales_f32, zeros_u8, group)
    return (np.asarray(x_f32, dtype=np.float64) @ w.astype(np.float64)).astype(np.float32)


# --------------------------------------------------------------------------
# Operator-API element codecs (src/jax_plugins/silicon/quantized.py:53-122)
# --------------------------------------------------------------------------

_E2M1_POS = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)
# Decision boundaries between neighbouring magnitudes; a value exactly on a
# boundary goes to the even magnitude code (quantized.py:58-65).
_E2M1_BOUNDS = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], dtype=np.float32)


def e2m1_encode(x: np.ndarray) -> np.ndarray:
    x = np.asarray(x, dtype=np.float32)
    a = np.abs(x)
    # count boundaries strictly below a, then fix ties toward the even code
    code = np.searchsorted(_E2M1_BOUNDS, a, side="left").astype(np.int32)  # a == bound -> lower code
    on_bound = np.zeros(a.shape, dtype=bool)
    for i, b in enumerate(_E2M1_BOUNDS):
        on_bound |= a == b
        # at the boundary between code i and i+1 choose the even one
        even = i if i % 2 == 0 else i + 1
        code = np.where(a == b, even, code)
    code = np.where(np.isnan(a), 0, code)  # comparisons with NaN are all false
    sign = np.signbit(x).astype(np.uint8) << 3
    return (sign | code.astype(np.uint8)).astype(np.uint8)


def e2m1_decode(bits: np.ndarray) -> np.ndarray:
    bits = np.asarray(bits)
    sign = np.where(bits & 0x8, np.float32(-1.0), np.float32(1.0))
    return (sign * _E2M1_POS[(bits & 0x7).astype(np.int64)]).astype(np.float32)


def e4m3_decode(bits: np.ndarray) -> np.ndarray:
    """E4M3FN: bias 7, no infinities, code 0x7F/0xFF is NaN
    (quantized.py:94-102; MSL dequant_fp8_e4m3 :501-507)."""
    bits = np.asarray(bits, dtype=np.uint8)
    mag = (bits & 0x7F).astype(np.int32)
    e = mag >> 3
    m = mag & 7
    normal = np.ldexp((8 + m).astype(np.float32), e - 10)  # (1+m/8)*2^(e-7)
    sub = np.ldexp(m.astype(np.float32), -9)  # m/8 * 2^-6
    val = np.where(e == 0, sub, normal).astype(np.float32)
    val = np.where(bits & 0x80, -val, val)
    return np.where(mag == 0x7F, np.float32(np.nan), val).astype(np.float32)


_E4M3_POS = e4m3_decode(np.arange(0x7F, dtype=np.uint8))  # 0 .. 448, ascending


def e4m3_encode(x: np.ndarray) -> np.ndarray:
    """Nearest finite E4M3 code, ties to the even code, saturating at 0x7E;
    NaN encodes as +/-448 (quantized.py:76-91)."""
    x = np.asarray(x, dtype=np.float32)
    sign = np.signbit(x).astype(np.uint8)
    a = np.abs(np.clip(x, -448.0, 448.0))
    a = np.where(np.isnan(a), np.float32(448.0), a)
    hi = np.minimum(np.searchsorted(_E4M3_POS, a, side="left"), 0x7E)
    lo = np.maximum(hi - 1, 0)
    d_lo = a - _E4M3_POS[lo]
    d_hi = _E4M3_POS[hi] - a
    take_hi = (d_hi < d_lo) | ((d_hi == d_lo) & (hi % 2 == 0))
    mag = np.where(take_hi, hi, lo).astype(np.uint8)
    return (mag | (sign << 7)).astype(np.uint8)


def e8m0_encode(x: np.ndarray) -> np.ndarray:
    """Power-of-two scale code: round(log2 x) clipped to +/-127, +127 bias;
    non-finite -> 0xFF (quantized.py:108-115)."""
    x = np.asarray(x)  # log2 is evaluated in the input's own precision, as the reference does
    if x.dtype not in (np.float32, np.float64):
        x = x.astype(np.float32)
    bad = ~np.isfinite(x)
    safe = np.where(bad, x.dtype.type(1.0), np.maximum(x, x.dtype.type(np.finfo(np.float32).tiny)))
    n = np.clip(np.round(np.log2(safe)).astype(np.int32), -127, 127)
    return np.where(bad, 0xFF, n + 127).astype(np.uint8)


def e8m0_decode(bits: np.ndarray) -> np.ndarray:
    """2**(code-127); code 0xFF is NaN (quantized.py:118-122)."""
    bits = np.asarray(bits, dtype=np.uint8)
    e = np.minimum(bits.astype(np.int32) - 127, 127)
    v = np.ldexp(np.ones(bits.shape, dtype=np.float32), e)
    return np.where(bits == 0xFF, np.float32(np.nan), v).astype(np.float32)


MX_MODES = {
    "mxfp4": dict(bits=4, group=32, scale="e8m0"),
    "mxfp8": dict(bits=8, group=32, scale="e8m0"),
    "nvfp4": dict(bits=4, group=16, scale="e4m3"),
}


def _check_mode(mode):
    if mode not in MX_MODES:
        raise ValueError(f"Unknown mode '{mode}'. Must be one of {list(MX_MODES)}")
    return MX_MODES[mode]


def mx_quantize(w, *, mode="mxfp4"):
    """Group-wise MX quantisation (quantized.py:125-209): per group the raw
    scale is max|w| / max_repr (6 for fp4, 448 for fp8; 0 for an all-zero
    group), stored as E8M0 or E4M3; elements are w / decoded_scale (0 where
    the decoded scale is 0) encoded as E2M1 or E4M3; fp4 packs element i in the
    low nibble and i+1 in the high nibble."""
    cfg = _check_mode(mode)
    w = np.asarray(w, dtype=np.float32)
    K = w.shape[-1]
    g = cfg["group"]
    if K % g:
        raise ValueError(f"Last dimension ({K}) must be divisible by group_size ({g})")
    flat = w.reshape(-1, K // g, g)
    gmax = np.max(np.abs(flat), axis=-1)  # NaN propagates like np.max
    max_repr = np.float32(6.0 if cfg["bits"] == 4 else 448.0)
    with np.errstate(invalid="ignore", divide="ignore"):
        raw = np.where(gmax != 0, gmax / max_repr, np.float32(0.0))
    if cfg["scale"] == "e8m0":
        sc_bits = e8m0_encode(raw)
        sc = e8m0_decode(sc_bits)
    else:
        sc_bits = e4m3_encode(raw.astype(np.float32))
        sc = e4m3_decode(sc_bits)
    with np.errstate(invalid="ignore", divide="ignore"):
        norm = np.where(sc[..., None] != 0, flat / sc[..., None], np.float32(0.0)).astype(np.float32)
    if cfg["bits"] == 4:
        q = e2m1_encode(norm).reshape(flat.shape[0], K)
        packed = (q[:, 0::2] | (q[:, 1::2] << 4)).astype(np.uint8)
        packed = packed.reshape(w.shape[:-1] + (K // 2,))
    else:
        packed = e4m3_encode(norm).reshape(w.shape[:-1] + (K,))
    return packed, sc_bits.reshape(w.shape[:-1] + (K // g,))


def mx_dequantize(packed, scales, *, mode="mxfp4", shape=None, dtype=np.float32):
    """Inverse of :func:`mx_quantize` (quantized.py:212-273): value = decoded
    scale * decoded element, in f32."""
    cfg = _check_mode(mode)
    packed = np.asarray(packed, dtype=np.uint8)
    scales = np.asarray(scales, dtype=np.uint8)
    if cfg["bits"] == 4 and shape is None:
        raise ValueError("shape is required for FP4 dequantization")
    K = shape[-1] if shape is not None else packed.shape[-1]
    g = cfg["group"]
    p2 = packed.reshape(-1, packed.shape[-1])
    if cfg["bits"] == 4:
        nib = np.stack([p2 & 0xF, p2 >> 4], axis=-1).reshape(p2.shape[0], -1)[:, :K]
        el = e2m1_decode(nib)
    else:
        el = e4m3_decode(p2[:, :K])
    sc = e8m0_decode(scales) if cfg["scale"] == "e8m0" else e4m3_decode(scales)
    sc = sc.reshape(-1, K // g)
    out = (sc[:, :, None] * el.reshape(el.shape[0], K // g, g)).reshape(el.shape[0], K).astype(np.float32)
    if shape is not None:
        out = out.reshape(shape)
    return out.astype(dtype)


def _check_bits(bits):
    if bits not in (2, 3, 4, 8):
        raise ValueError(f"bits must be 2, 3, 4, or 8; got {bits}")


def affine_quantize(w, *, bits=4, group_size=64):
    """Per-group min/max affine quantisation (quantized.py:276-405):
    scale = (max-min)/(2**bits-1) computed in Python floats (float64) and
    stored as f32 (1.0 for a flat group), bias = min, q = clip(round((w-bias)/
    scale), 0, 2**bits-1) with the division carried in float64 against the
    float64 scale; 4-bit packs value j of each 8 at bits 4j of a uint32."""
    _check_bits(bits)
    w = np.asarray(w, dtype=np.float32)
    K = w.shape[-1]
    if K % group_size:
        raise ValueError(f"Last dimension ({K}) must be divisible by group_size ({group_size})")
    nb = (1 << bits) - 1
    flat = w.reshape(-1, K // group_size, group_size)
    wmin = flat.min(axis=-1).astype(np.float64)
    wmax = flat.max(axis=-1).astype(np.float64)
    scale64 = np.where(wmax != wmin, (wmax - wmin) / nb, 1.0)
    # the reference divides the f32 group by Python floats: NumPy keeps the
    # array dtype (f32) for array-with-python-scalar arithmetic
    bias32 = wmin.astype(np.float32)
    q = np.round((flat - bias32[..., None]) / scale64.astype(np.float32)[..., None])
    q = np.clip(q.astype(np.int32), 0, nb).reshape(flat.shape[0], K).astype(np.uint32)
    lead = w.shape[:-1]
    if bits == 8:
        packed = q.astype(np.uint8).reshape(lead + (K,))
    elif bits == 4:
        v = (q & 0xF).reshape(-1, K // 8, 8)
        packed = np.zeros(v.shape[:2], dtype=np.uint32)
        for j in range(8):
            packed |= v[:, :, j] << np.uint32(4 * j)
        packed = packed.reshape(lead + (K // 8,))
    elif bits == 2:
        v = (q & 0x3).reshape(-1, K // 16, 16)
        packed = np.zeros(v.shape[:2], dtype=np.uint32)
        for j in range(16):
            packed |= v[:, :, j] << np.uint32(2 * j)
        packed = packed.reshape(lead + (K // 16,))
    else:  # 3-bit: 32 values in 3 words, little-endian bit stream
        v = (q & 0x7).reshape(-1, K // 32, 32).astype(np.uint64)
        stream = np.zeros(v.shape[:2] + (2,), dtype=np.uint64)  # 96 bits in two u64 (64 + 32)
        lo = np.zeros(v.shape[:2], dtype=np.uint64)
        hi = np.zeros(v.shape[:2], dtype=np.uint64)
        for j in range(32):
            pos = 3 * j
            if pos < 64:
                lo |= v[:, :, j] << np.uint64(pos)
                if pos > 61:
                    hi |= v[:, :, j] >> np.uint64(64 - pos)
            else:
                hi |= v[:, :, j] << np.uint64(pos - 64)
        del stream
        words = np.stack(
            [lo & np.uint64(0xFFFFFFFF), lo >> np.uint64(32), hi & np.uint64(0xFFFFFFFF)], axis=-1
        ).astype(np.uint32)
        packed = words.reshape(lead + (K * 3 // 32,))
    gshape = lead + (K // group_size,)
    return packed, scale64.astype(np.float32).reshape(gshape), bias32.reshape(gshape)


def affine_unpack(packed, *, bits, K):
    """Packed words -> integer codes ``[rows, K]`` (quantized.py:445-470)."""
    _check_bits(bits)
    p = np.asarray(packed)
    p2 = p.reshape(-1, p.shape[-1])
    if bits == 8:
        return p2[:, :K].astype(np.int32)
    p2 = p2.astype(np.uint32)
    if bits == 4:
        sh = (4 * np.arange(8, dtype=np.uint32))[None, None, :]
        return ((p2[:, :, None] >> sh) & 0xF).reshape(p2.shape[0], -1)[:, :K].astype(np.int32)
    if bits == 2:
        sh = (2 * np.arange(16, dtype=np.uint32))[None, None, :]
        return ((p2[:, :, None] >> sh) & 0x3).reshape(p2.shape[0], -1)[:, :K].astype(np.int32)
    w = p2.reshape(p2.shape[0], -1, 3).astype(np.uint64)
    lo = w[:, :, 0] | (w[:, :, 1] << np.uint64(32))
    hi = w[:, :, 2]
    out = np.zeros(w.shape[:2] + (32,), dtype=np.int32)
    for j in range(32):
        pos = 3 * j
        if pos < 64:
            val = lo >> np.uint64(pos)
            if pos > 61:
                val = val | (hi << np.uint64(64 - pos))
        else:
            val = hi >> np.uint64(pos - 64)
        out[:, :, j] = (val & np.uint64(7)).astype(np.int32)
    return out.reshape(out.shape[0], -1)[:, :K]


def affine_dequantize(packed, scales, biases, *, bits=4, group_size=64, shape=None, dtype=np.float32):
    """``scale * q + bias`` per group in f32 (quantized.py:408-482)."""
    _check_bits(bits)
    p = np.asarray(packed)
    if bits != 8 and shape is None:
        raise ValueError("shape is required for sub-byte dequantization")
    K = shape[-1] if shape is not None else p.shape[-1]
    q = affine_unpack(p, bits=bits, K=K).astype(np.float32)
    ng = K // group_size
    s = np.asarray(scales, dtype=np.float32).reshape(-1, ng)
    b = np.asarray(biases, dtype=np.float32).reshape(-1, ng)
    out = (s[:, :, None] * q.reshape(q.shape[0], ng, group_size) + b[:, :, None]).reshape(q.shape[0], K)
    if shape is not None:
        out = out.reshape(shape)
    return out.astype(dtype)


def affine_qmm(x, packed, scales, biases, *, bits=4, group_size=64, K, out_dtype=None):
    """Restatement of the fused affine dequant-GEMM kernels' arithmetic
    (quantized.py:772-957): activation widened to f32, weight = scale*q+bias
    in f32, product and accumulation in f32 (float64 here, rounded once),
    result cast to the activation dtype and then to ``out_dtype``
    (:1137-1152)."""
    x = np.asarray(x)
    N = np.asarray(packed).shape[0]
    w = affine_dequantize(packed, scales, biases, bits=bits, group_size=group_size, shape=(N, K))
    x2 = x.reshape(-1, K).astype(np.float64)
    y = (x2 @ w.astype(np.float64).T).astype(np.float32).astype(x.dtype)
    y = y.reshape(x.shape[:-1] + (N,))
    return y.astype(out_dtype if out_dtype is not None else x.dtype)


def mx_qmm(x, packed, scales, *, mode="mxfp4", K, out_dtype=None):
    """Restatement of the fused MX dequant-GEMM kernels (quantized.py:528-753):
    weight = decoded scale * decoded element in f32, NaN codes propagate."""
    _check_mode(mode)
    x = np.asarray(x)
    N = np.asarray(packed).shape[0]
    w = mx_dequantize(packed, scales, mode=mode, shape=(N, K))
    x2 = x.reshape(-1, K).astype(np.float64)
    with np.errstate(invalid="ignore"):
        y = (x2 @ w.astype(np.float64).T).astype(np.float32).astype(x.dtype)
    y = y.reshape(x.shape[:-1] + (N,))
    return y.astype(out_dtype if out_dtype is not None else x.dtype)
