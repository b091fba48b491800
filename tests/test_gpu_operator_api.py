"""The operator API on the GPU, against the reference's own outputs (golden
fixtures) and the known answers of the reference's tests/test_quantized.py."""

import numpy as np
import pytest
import torch

from jax_metallib_b200 import quantized as Q
from oracle import qmm_oracle as O

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("mode", ["mxfp4", "mxfp8", "nvfp4"])
@pytest.mark.parametrize("shape", ["4x8x64", "8x16x64", "16x32x128"])
def test_mx_matmul_matches_reference_outputs(cuda, golden, mode, shape):
    tag = f"mx_{mode}_{shape}"
    x, p, s = golden[tag + "_x"], golden[tag + "_packed"], golden[tag + "_scales"]
    K = x.shape[1]
    out = Q.quantized_matmul(x, p, s, mode=mode, K=K)
    assert isinstance(out, np.ndarray) and out.dtype == np.float32
    np.testing.assert_allclose(out, golden[tag + "_matmul_f32"], rtol=1e-5, atol=1e-6)
    out16 = Q.quantized_matmul(x.astype(np.float16), p, s, mode=mode, K=K)
    assert out16.dtype == np.float16
    np.testing.assert_allclose(out16.astype(np.float32), O.mx_qmm(x.astype(np.float16), p, s, mode=mode, K=K)
                               .astype(np.float32), rtol=2e-3, atol=1e-3)
    # tolerance of the reference's own test against the float matmul (tests/test_quantized.py:228-253)
    ref = x @ golden[tag + "_w"].T
    np.testing.assert_allclose(out, ref, rtol=0.5, atol=0.1 if "fp4" in mode else 0.06)


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("gs", [32, 64, 128])
def test_affine_matmul_matches_reference_outputs(cuda, golden, bits, gs):
    tag = f"affine_b{bits}_g{gs}"
    x, p, s, b = golden[tag + "_x"], golden[tag + "_packed"], golden[tag + "_scales"], golden[tag + "_biases"]
    out = Q.affine_quantized_matmul(x, p, s, b, bits=bits, group_size=gs, K=128)
    np.testing.assert_allclose(out, golden[tag + "_matmul_f32"], rtol=1e-5, atol=1e-6)
    out16 = Q.affine_quantized_matmul(x.astype(np.float16), p, s, b, bits=bits, group_size=gs, K=128)
    assert out16.dtype == np.float16
    np.testing.assert_allclose(out16.astype(np.float32), golden[tag + "_matmul_f16"].astype(np.float32),
                               rtol=4e-3, atol=2e-3)


def test_known_answers_of_the_reference_tests(cuda):
    # all-ones 4-bit affine: exactly [[64, 64]] (tests/test_quantized.py:528-541)
    p, s, b = Q.affine_quantize(np.ones((2, 64), np.float32), bits=4, group_size=64)
    out = Q.affine_quantized_matmul(np.ones((1, 64), np.float16), p, s, b, bits=4, group_size=64, K=64,
                                    out_dtype=np.float32)
    assert out.dtype == np.float32
    np.testing.assert_array_equal(out, [[64.0, 64.0]])
    # NaN propagation (tests/test_quantized.py:303-335)
    x = np.ones((1, 32), np.float32)
    out = Q.quantized_matmul(x, np.array([[0x7F] + [0] * 31], np.uint8), np.array([[127]], np.uint8), mode="mxfp8", K=32)
    assert np.isnan(out[0, 0])
    for mode, nb in (("mxfp4", 16), ("mxfp8", 32)):
        out = Q.quantized_matmul(x, np.full((1, nb), 0x11, np.uint8), np.array([[0xFF]], np.uint8), mode=mode, K=32)
        assert np.isnan(out[0, 0])
    out = Q.quantized_matmul(np.ones((1, 16), np.float32), np.full((1, 8), 0x11, np.uint8),
                             np.array([[0x7F]], np.uint8), mode="nvfp4", K=16)
    assert np.isnan(out[0, 0])
    # f16 activations widened to an f32 result (tests/test_quantized.py:510-526)
    w = np.ones((2, 64), np.float32)
    p, s = Q.mx_quantize(w, mode="mxfp8")
    out = Q.quantized_matmul(np.ones((1, 64), np.float16), p, s, mode="mxfp8", K=64, out_dtype=np.float32)
    assert out.dtype == np.float32
    np.testing.assert_allclose(out, np.ones((1, 64), np.float32) @ Q.mx_dequantize(p, s, mode="mxfp8", shape=w.shape).T,
                               atol=0.1, rtol=0.01)


@pytest.mark.parametrize("mode", ["mxfp4", "mxfp8", "nvfp4"])
def test_larger_and_batched_shapes(cuda, mode):
    rng = np.random.default_rng(42)
    M, N, K = 64, 128, 256
    x = rng.standard_normal((2, 3, M, K)).astype(np.float32) * 0.1
    w = rng.standard_normal((N, K)).astype(np.float32) * 0.1
    p, s = Q.mx_quantize(w, mode=mode)
    xt = torch.from_numpy(x).cuda()
    out = Q.quantized_matmul(xt, torch.from_numpy(p).cuda(), torch.from_numpy(s).cuda(), mode=mode, K=K)
    assert isinstance(out, torch.Tensor) and out.shape == (2, 3, M, N) and out.is_cuda
    ref = O.mx_qmm(x, p, s, mode=mode, K=K)
    np.testing.assert_allclose(out.cpu().numpy(), ref, rtol=1e-4, atol=1e-5)
    assert not np.isnan(out.cpu().numpy()).any() and np.any(out.cpu().numpy() != 0)


def test_affine_large_k_and_rows(cuda):
    rng = np.random.default_rng(7)
    M, N, K = 19, 96, 4096
    x = rng.standard_normal((M, K)).astype(np.float32)
    w = rng.standard_normal((N, K)).astype(np.float32) * 0.05
    for bits in (4, 8):
        p, s, b = Q.affine_quantize(w, bits=bits, group_size=128)
        out = Q.affine_quantized_matmul(x, p, s, b, bits=bits, group_size=128, K=K)
        ref = O.affine_qmm(x, p, s, b, bits=bits, group_size=128, K=K)
        assert O.max_rel_err(out, ref) <= 1e-5


@pytest.mark.parametrize("M", [1, 5, 8, 9, 16])
@pytest.mark.parametrize("bits,gs,K,N", [(4, 64, 4096, 208), (4, 128, 4096, 4096), (4, 64, 192, 16), (4, 256, 1024, 80),
                                         (4, 64, 64, 32), (8, 32, 4096, 208), (8, 64, 4096, 4096), (8, 32, 96, 16),
                                         (8, 128, 1024, 80), (8, 32, 32, 32),
                                         # shapes of the TMA-ring kernel: several tiles per CTA, K cut 2 to 16 ways,
                                         # groups of 1, 2 and 4 steps, a last CTA with fewer tiles
                                         (4, 64, 4096, 14336), (4, 128, 4096, 2368), (4, 256, 8192, 512), (4, 64, 1024, 2384),
                                         (4, 64, 14336, 4096), (8, 32, 2048, 1024), (8, 64, 4096, 14336), (8, 128, 8192, 2400)])
def test_affine_f16_decode_sizes(cuda, M, bits, gs, K, N):
    """f16 activations with at most 16 rows and groups of a multiple of 64 (4-bit) or 32 (8-bit) take
    the tensor-core kernel (codes fed to the MMA as f16 subnormals, scale and bias applied per group);
    same result as the dequantise-then-multiply arithmetic of the reference's fused kernels up to f32
    summation order."""
    rng = np.random.default_rng(M * 1000 + K + N + bits)
    x = rng.standard_normal((M, K)).astype(np.float16)
    w = rng.standard_normal((N, K)).astype(np.float32) * 0.05
    p, s, b = Q.affine_quantize(w, bits=bits, group_size=gs)
    out = Q.affine_quantized_matmul(x, p, s, b, bits=bits, group_size=gs, K=K)
    assert out.dtype == np.float16 and out.shape == (M, N)
    ref = O.affine_qmm(x.astype(np.float32), p, s, b, bits=bits, group_size=gs, K=K)
    # one f16 rounding of the result (2^-11 relative) on top of f32 accumulation
    np.testing.assert_allclose(out.astype(np.float32), ref, rtol=1e-3, atol=1e-3 * float(np.abs(ref).max()))
    # f32 activations take the general kernel: the two routes agree
    wide = Q.affine_quantized_matmul(x.astype(np.float32), p, s, b, bits=bits, group_size=gs, K=K)
    np.testing.assert_allclose(out.astype(np.float32), wide, rtol=1e-3, atol=1e-3 * float(np.abs(ref).max()))


@pytest.mark.parametrize("bits", [4, 8])
def test_affine_f16_tiny_and_large_activations(cuda, bits):
    """Activation magnitudes at both ends of f16: the subnormal trick scales no activation, so
    neither underflow nor overflow is introduced."""
    rng = np.random.default_rng(3)
    K, N, gs = 512, 64, 64
    w = rng.standard_normal((N, K)).astype(np.float32)
    p, s, b = Q.affine_quantize(w, bits=bits, group_size=gs)
    for scale in (2.0 ** -20, 1.0, 200.0):
        x = (rng.standard_normal((3, K)) * scale).astype(np.float16)
        out = Q.affine_quantized_matmul(x, p, s, b, bits=bits, group_size=gs, K=K).astype(np.float32)
        ref = O.affine_qmm(x.astype(np.float32), p, s, b, bits=bits, group_size=gs, K=K)
        assert np.isfinite(out).all()
        np.testing.assert_allclose(out, ref, rtol=2e-3, atol=2e-3 * float(np.abs(ref).max()))


@pytest.mark.parametrize("M", [1, 5, 8, 9, 16])
@pytest.mark.parametrize("mode,K,N", [("mxfp4", 4096, 14336), ("mxfp4", 512, 16), ("mxfp4", 8192, 2384), ("mxfp4", 1024, 208),
                                      ("mxfp8", 4096, 14336), ("mxfp8", 512, 16), ("mxfp8", 8192, 2384), ("mxfp8", 1536, 208),
                                      ("nvfp4", 4096, 14336), ("nvfp4", 256, 16), ("nvfp4", 8192, 2384), ("nvfp4", 768, 208)])
def test_mx_f16_decode_sizes(cuda, M, mode, K, N):
    """f16 activations with at most 16 rows and K a multiple of 16 scale groups take the tensor-core kernel
    (codes placed in f16 as they are, power-of-two factor applied once); same result as the
    dequantise-then-multiply arithmetic of the reference's fused kernels up to f32 summation order."""
    rng = np.random.default_rng(M * 1000 + K + N)
    x = rng.standard_normal((M, K)).astype(np.float16)
    w = (rng.standard_normal((N, K)) * np.exp(rng.standard_normal((N, 1)))).astype(np.float32) * 0.05
    p, s = Q.mx_quantize(w, mode=mode)
    out = Q.quantized_matmul(x, p, s, mode=mode, K=K)
    assert out.dtype == np.float16 and out.shape == (M, N)
    ref = O.mx_qmm(x.astype(np.float32), p, s, mode=mode, K=K)
    np.testing.assert_allclose(out.astype(np.float32), ref, rtol=1e-3, atol=1e-3 * float(np.abs(ref).max()))
    wide = Q.quantized_matmul(x.astype(np.float32), p, s, mode=mode, K=K)    # f32 activations: the general kernel
    np.testing.assert_allclose(out.astype(np.float32), wide, rtol=1e-3, atol=1e-3 * float(np.abs(ref).max()))


@pytest.mark.parametrize("mode", ["mxfp4", "mxfp8", "nvfp4"])
def test_mx_f16_special_codes(cuda, mode):
    """NaN element codes (e4m3 0x7F / 0xFF), NaN scale codes (e8m0 0xFF, e4m3 0x7F) and the e8m0 code 0
    (2^-127) on the tensor-core route: NaN reaches exactly the output columns of the weight rows that
    hold one, for every activation row; everything else is unchanged."""
    rng = np.random.default_rng(11)
    K, N, M = 1024, 64, 3
    group = 16 if mode == "nvfp4" else 32
    x = rng.standard_normal((M, K)).astype(np.float16)
    w = rng.standard_normal((N, K)).astype(np.float32) * 0.1
    p, s = Q.mx_quantize(w, mode=mode)
    p, s = p.copy(), s.copy()
    nan_rows = set()
    if mode == "mxfp8":
        p[5, 700] = 0x7F
        p[40, 3] = 0xFF
        nan_rows |= {5, 40}
    if mode == "nvfp4":
        s[9, 17] = 0x7F
        s[33, K // group - 1] = 0xFF
        nan_rows |= {9, 33}
    else:
        s[12, 5] = 0xFF
        nan_rows |= {12}
        s[20, 7] = 0          # 2^-127: the group contributes (next to) nothing
    out = Q.quantized_matmul(x, p, s, mode=mode, K=K).astype(np.float32)
    ref = O.mx_qmm(x.astype(np.float32), p, s, mode=mode, K=K)
    for n in range(N):
        if n in nan_rows:
            assert np.isnan(out[:, n]).all(), n
            assert np.isnan(ref[:, n]).all(), n
        else:
            assert np.isfinite(out[:, n]).all(), n
    keep = [n for n in range(N) if n not in nan_rows]
    np.testing.assert_allclose(out[:, keep], ref[:, keep], rtol=1e-3, atol=1e-3 * float(np.abs(ref[:, keep]).max()))
