"""Generate ``reference_quantized.npz`` from the reference's own CPU helpers.

Run where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/reference

The reference's ``src/jax_plugins/silicon/quantized.py`` is imported unmodified
(through ``oracle/ref_shim.py``'s NumPy stand-in for ``jax.numpy``) and its
outputs on seeded inputs are stored.  Seeds and shapes follow the reference's
``tests/test_quantized.py`` (``default_rng(42)``, normal * 0.1, the (M, N, K)
triples it uses) plus edge cases (zero groups, flat groups, NaN weights, NaN
scale codes).  The committed ``.npz`` is what the CPU tests compare the oracle
against, and what the GPU tests compare the CUDA path against.
"""

from __future__ import annotations

import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle.ref_shim import load_reference_quantized  # noqa: E402


def main(reference_root: str) -> None:
    R = load_reference_quantized(reference_root)
    out = {}
    # element codec tables
    codes = np.arange(256, dtype=np.uint8)
    out["e4m3_decode_table"] = R._fp8_e4m3_dequantize(codes)
    out["e8m0_decode_table"] = R._fp8_e8m0_dequantize(codes)
    out["e2m1_decode_table"] = R._fp4_e2m1_dequantize(codes[:16])
    rng = np.random.default_rng(7)
    probe = np.concatenate(
        [
            rng.standard_normal(512).astype(np.float32) * 3,
            rng.standard_normal(512).astype(np.float32) * 200,
            rng.standard_normal(256).astype(np.float32) * 0.01,
            np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 0.0, -0.0, 100.0, 448, 480, 1 / 512, 2 / 512,
                      3 / 512, 280, 304, 432, np.inf, -np.inf, np.nan], dtype=np.float32),
        ]
    )
    probe = np.concatenate([probe, -probe])
    out["codec_probe"] = probe
    out["e2m1_encode_probe"] = R._fp4_e2m1_quantize(probe)
    out["e4m3_encode_probe"] = R._fp8_e4m3_quantize(probe)
    pos = np.abs(probe)
    out["e8m0_encode_probe"] = R._fp8_e8m0_quantize(pos)

    # MX quantise / dequantise / matmul at the reference test shapes
    for mode in ("mxfp4", "mxfp8", "nvfp4"):
        for (M, N, K) in ((4, 8, 64), (8, 16, 64), (16, 32, 128)):
            rng = np.random.default_rng(42)
            x = rng.standard_normal((M, K)).astype(np.float32) * 0.1
            w = rng.standard_normal((N, K)).astype(np.float32) * 0.1
            tag = f"mx_{mode}_{M}x{N}x{K}"
            p, s = R.mx_quantize(w, mode=mode)
            out[tag + "_x"] = x
            out[tag + "_w"] = w
            out[tag + "_packed"] = np.asarray(p)
            out[tag + "_scales"] = np.asarray(s)
            out[tag + "_dequant"] = np.asarray(R.mx_dequantize(p, s, mode=mode, shape=w.shape))
            out[tag + "_matmul_f32"] = np.asarray(R.quantized_matmul(x, p, s, mode=mode, K=K))
            out[tag + "_matmul_f16"] = np.asarray(R.quantized_matmul(x.astype(np.float16), p, s, mode=mode, K=K))
        # edge: zero group + NaN weight
        w = np.random.default_rng(3).standard_normal((4, 64)).astype(np.float32)
        w[1, :32] = 0.0
        w[2, 5] = np.nan
        p, s = R.mx_quantize(w, mode=mode)
        out[f"mx_{mode}_edge_w"] = w
        out[f"mx_{mode}_edge_packed"] = np.asarray(p)
        out[f"mx_{mode}_edge_scales"] = np.asarray(s)
        out[f"mx_{mode}_edge_dequant"] = np.asarray(R.mx_dequantize(p, s, mode=mode, shape=w.shape))

    # affine quantise / dequantise / matmul
    for bits in (2, 3, 4, 8):
        for gs in (32, 64, 128):
            rng = np.random.default_rng(42)
            M, N, K = 8, 16, 128
            x = rng.standard_normal((M, K)).astype(np.float32) * 0.1
            w = rng.standard_normal((N, K)).astype(np.float32) * 0.1
            w[3, :gs] = 0.25  # a flat group: scale 1.0, bias 0.25
            tag = f"affine_b{bits}_g{gs}"
            p, s, b = R.affine_quantize(w, bits=bits, group_size=gs)
            out[tag + "_x"] = x
            out[tag + "_w"] = w
            out[tag + "_packed"] = np.asarray(p)
            out[tag + "_scales"] = np.asarray(s)
            out[tag + "_biases"] = np.asarray(b)
            out[tag + "_dequant"] = np.asarray(
                R.affine_dequantize(p, s, b, bits=bits, group_size=gs, shape=w.shape)
            )
            if bits in (4, 8):
                out[tag + "_matmul_f32"] = np.asarray(
                    R.affine_quantized_matmul(x, p, s, b, bits=bits, group_size=gs, K=K)
                )
                out[tag + "_matmul_f16"] = np.asarray(
                    R.affine_quantized_matmul(x.astype(np.float16), p, s, b, bits=bits, group_size=gs, K=K)
                )
    # the exact known answer of tests/test_quantized.py:528-541
    w = np.ones((2, 64), dtype=np.float32)
    p, s, b = R.affine_quantize(w, bits=4, group_size=64)
    out["affine_ones_packed"] = np.asarray(p)
    out["affine_ones_scales"] = np.asarray(s)
    out["affine_ones_biases"] = np.asarray(b)
    out["affine_ones_matmul"] = np.asarray(
        R.affine_quantized_matmul(np.ones((1, 64), np.float16), p, s, b, bits=4, group_size=64, K=64,
                                  out_dtype=np.float32)
    )
    path = os.path.join(HERE, "reference_quantized.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, len(out), "arrays", os.path.getsize(path), "bytes")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: make_golden.py <checkout of the reference project>")
    main(sys.argv[1])
