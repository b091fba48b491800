"""Parity of the CUDA path (through the C ABI) against the CPU oracle.

Bit-exact for the int32 accumulators of the integer dots; max relative error
(max|out-ref| / max|ref|) <= 2e-3 for f32 outputs and <= 1e-2 for bf16 outputs
against the fp32 dequantise-then-dot oracle.
"""

import numpy as np
import pytest
import torch

from jax_metallib_b200 import _lib, ops, synthetic
from oracle import qmm_oracle as O

pytestmark = pytest.mark.gpu

TOL_F32 = 2e-3
TOL_BF16 = 1e-2


def dev(a, cuda, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).to(cuda)
    return t if dtype is None else t.view(dtype)


def bf16_to_np(t: torch.Tensor) -> np.ndarray:
    return synthetic.bf16_bits_to_f32(t.view(torch.int16).cpu().numpy().view(np.uint16))


def test_native_library_is_loaded(cuda):
    lib = _lib.load()
    assert b"sm_100a" in lib.qmm_version()
    assert lib.qmm_device_status() == 0


# ---------------------------------------------------------------- config 1
@pytest.mark.parametrize("shape", [(32, 1024, 1024), (5, 100, 37), (1, 64, 8), (70, 2048, 96), (33, 129, 65)])
def test_w8a32_perchannel(cuda, shape):
    M, K, N = shape
    c = synthetic.config1(M, K, N)
    y = ops.w8a32_perchannel(dev(c["x"], cuda), dev(c["w"], cuda), dev(c["scale"], cuda)).cpu().numpy()
    ref = O.w8_perchannel_matmul(c["x"], c["w"], c["scale"])
    assert y.shape == ref.shape and y.dtype == np.float32
    assert O.max_rel_err(y, ref) <= TOL_F32
    assert O.max_rel_err(y, ref) <= 1e-5  # f32 FMA arithmetic: far inside the contract


def test_w8a32_rank3_and_empty(cuda):
    c = synthetic.config1(6, 128, 64)
    x3 = dev(c["x"].reshape(2, 3, 128), cuda)
    y = ops.w8a32_perchannel(x3, dev(c["w"], cuda), dev(c["scale"], cuda))
    assert y.shape == (2, 3, 64)
    ref = O.w8_perchannel_matmul(c["x"], c["w"], c["scale"]).reshape(2, 3, 64)
    assert O.max_rel_err(y.cpu().numpy(), ref) <= 1e-5
    e = ops.w8a32_perchannel(torch.empty((0, 128), device=cuda), dev(c["w"], cuda), dev(c["scale"], cuda))
    assert e.shape == (0, 64)


# ---------------------------------------------------------------- config 2
@pytest.mark.parametrize("shape", [(128, 128, 256), (256, 512, 512), (384, 1024, 640), (200, 272, 336),
                                   (2048, 4096, 4096)])
def test_i8_dot_bit_exact_and_rescale(cuda, shape):
    M, K, N = shape
    c = synthetic.config2(M, K, N)
    acc, out = ops.i8_dot(dev(c["a"], cuda), dev(c["b"], cuda), dev(c["row"], cuda), dev(c["col"], cuda))
    ref_acc = O.i8_dot_i32(c["a"], c["b"])
    np.testing.assert_array_equal(acc.cpu().numpy(), ref_acc)
    ref_out = O.i8_dot_rescale(ref_acc, c["row"], c["col"])
    got = out.cpu().numpy()
    assert O.max_rel_err(got, ref_out) <= TOL_F32
    np.testing.assert_array_equal(got, ref_out)  # same op order, each step rounded to f32: identical bits


@pytest.mark.parametrize("au,bu", [(False, True), (True, False), (True, True)])
def test_i8_dot_unsigned_operands(cuda, au, bu):
    rng = np.random.default_rng(0)
    a = rng.integers(0 if au else -128, 256 if au else 128, size=(256, 384)).astype(np.uint8 if au else np.int8)
    b = rng.integers(0 if bu else -128, 256 if bu else 128, size=(384, 256)).astype(np.uint8 if bu else np.int8)
    acc, _ = ops.i8_dot(dev(a, cuda), dev(b, cuda))
    np.testing.assert_array_equal(acc.cpu().numpy(), O.i8_dot_i32(a, b))


@pytest.mark.parametrize("dtype", [np.int8, np.uint8])
def test_i8_dot_small_shapes_of_the_reference_tests(cuda, dtype):
    # tests/test_int_dot.py:25-52 (seed 0, [-300,300) wrapped) and tests/test_dot_preferred_dtype.py:44-53
    rng = np.random.default_rng(0)
    for (m, k, n) in [(5, 7, 3), (1, 7, 3), (33, 40, 17), (256, 512, 128), (31, 40, 1)]:
        a = rng.integers(-300, 300, size=(m, k), dtype=np.int64).astype(dtype)
        b = rng.integers(-300, 300, size=(k, n), dtype=np.int64).astype(dtype)
        acc, _ = ops.i8_dot(dev(a, cuda), dev(b, cuda))
        np.testing.assert_array_equal(acc.cpu().numpy(), O.i8_dot_i32(a, b))


def test_i8_dot_extreme_values(cuda):
    a = np.full((128, 4096), -128, np.int8)
    b = np.full((4096, 256), -128, np.int8)
    acc, _ = ops.i8_dot(dev(a, cuda), dev(b, cuda))
    assert (acc.cpu().numpy() == 4096 * 16384).all()
    b[:] = 127
    acc, _ = ops.i8_dot(dev(a, cuda), dev(b, cuda))
    assert (acc.cpu().numpy() == -128 * 127 * 4096).all()


# ---------------------------------------------------------------- config 3
def _w4_check(cuda, M, K, N, packed, index=0):
    c = synthetic.config3(M, K, N, index=index)
    z = c["z_packed"] if packed else c["z"]
    y = ops.w4a16_g128(dev(c["x_bits"].view(np.int16), cuda, torch.bfloat16), dev(c["wq"], cuda),
                       dev(c["s_bits"].view(np.int16), cuda, torch.bfloat16), dev(z, cuda), zeros_packed=packed)
    torch.cuda.synchronize()
    assert _lib.load().qmm_device_status() == 0
    ref = O.w4a16_matmul(c["x"], c["wq"], c["s"], c["z"])
    got = bf16_to_np(y)
    assert got.shape == ref.shape
    err = O.max_rel_err(got, ref)
    assert err <= TOL_BF16, err
    return got, ref


@pytest.mark.parametrize("M", [1, 4, 16])
@pytest.mark.parametrize("packed", [False, True])
def test_w4a16_decode_full_shape(cuda, M, packed):
    got, ref = _w4_check(cuda, M, 4096, 14336, packed)
    # element-wise version with an absolute floor
    floor = 1e-2 * np.max(np.abs(ref))
    assert np.all(np.abs(got - ref) <= 8e-3 * np.abs(ref) + floor)


@pytest.mark.parametrize("shape", [(1, 128, 128), (3, 256, 128), (8, 128, 384), (9, 512, 256), (17, 384, 256),
                                   (32, 1024, 512), (8, 4096, 1024), (8, 14336, 4096), (2, 4096, 4096)])
def test_w4a16_decode_other_shapes(cuda, shape):
    M, K, N = shape
    _w4_check(cuda, M, K, N, packed=(M % 2 == 0), index=M)


def test_w4a16_workspace_is_left_clean_and_results_repeat(cuda):
    c = synthetic.config3(4, 4096, 14336)
    args = (dev(c["x_bits"].view(np.int16), cuda, torch.bfloat16), dev(c["wq"], cuda),
            dev(c["s_bits"].view(np.int16), cuda, torch.bfloat16), dev(c["z"], cuda))
    need = _lib.load().qmm_w4a16_g128_workspace_bytes(4, 14336, 4096)
    ws = torch.zeros(need, dtype=torch.uint8, device=cuda)
    y1 = ops.w4a16_g128(*args, workspace=ws).clone()
    counters = ws[: 2048 * 8 * 4].view(torch.int32)  # the header: one arrival counter per (column block, warp)
    assert int(counters.abs().sum()) == 0
    y2 = ops.w4a16_g128(*args, workspace=ws)
    assert torch.equal(y1, y2)  # fixed summation order: bitwise repeatable


def test_w4a16_rejects_what_it_does_not_cover(cuda):
    c = synthetic.config3(1, 256, 128)
    x = dev(c["x_bits"].view(np.int16), cuda, torch.bfloat16)
    wq, s, z = dev(c["wq"], cuda), dev(c["s_bits"].view(np.int16), cuda, torch.bfloat16), dev(c["z"], cuda)
    lib = _lib.load()
    st = lib.qmm_w4a16_g128(x.data_ptr(), wq.data_ptr(), s.data_ptr(), z.data_ptr(), 0, x.data_ptr(), 1, 128, 256, 64,
                            None, 0, 0, None)  # a group size the kernels do not cover
    assert lib.qmm_status_name(st) == b"QMM_ERR_UNSUPPORTED"
    with pytest.raises(_lib.QmmError) as e:
        ops.w4a16_g128(x, wq, s, z, workspace=torch.zeros(256, dtype=torch.uint8, device=cuda)[:16])
    assert e.value.status_name == "QMM_ERR_WORKSPACE"


# ---------------------------------------------------------------- int4 g128 at prefill sizes (tcgen05)
def _w4_prefill_check(cuda, M, K, N, packed, seed):
    """Device-generated operands; sampled rows (four per 256-row tile) over all columns against the oracle."""
    gen = synthetic.torch_generator(cuda, 3, seed)
    G = K // 128
    x = synthetic.device_normal((M, K), cuda, gen, torch.bfloat16)
    wq = torch.randint(0, 256, (K // 2, N), dtype=torch.uint8, device=cuda, generator=gen)
    sc = synthetic.device_uniform((G, N), 0.002, 0.01, cuda, gen, torch.bfloat16)
    z = torch.randint(0, 16, (G, N), dtype=torch.uint8, device=cuda, generator=gen)
    zarg = (z[:, 0::2] | (z[:, 1::2] << 4)).contiguous() if packed else z
    y = ops.w4a16_g128(x, wq, sc, zarg, zeros_packed=packed)
    torch.cuda.synchronize()
    assert _lib.load().qmm_device_status() == 0
    rows = np.array(sorted({min(M - 1, t * 256 + o) for t in range((M + 255) // 256) for o in (3, 100, 131, 250)}))
    rows_t = torch.from_numpy(rows).to(cuda)
    got = bf16_to_np(y[rows_t].contiguous())
    xs = bf16_to_np(x[rows_t].contiguous())
    wq_h, z_h = wq.cpu().numpy(), z.cpu().numpy()
    s_h = bf16_to_np(sc)
    ref = np.empty((len(rows), N), np.float32)
    for c0 in range(0, N, 2048):
        ref[:, c0:c0 + 2048] = O.w4a16_matmul(xs, wq_h[:, c0:c0 + 2048], s_h[:, c0:c0 + 2048], z_h[:, c0:c0 + 2048])
    err = O.max_rel_err(got, ref)
    assert err <= TOL_BF16, err
    return err


@pytest.mark.parametrize("M", [64, 512, 4096])
def test_w4a16_prefill_full_shape(cuda, M):
    _w4_prefill_check(cuda, M, 4096, 14336, packed=(M != 512), seed=M)


@pytest.mark.parametrize("shape", [(33, 128, 128), (100, 256, 384), (257, 1024, 640), (300, 14336, 4096)])
def test_w4a16_prefill_other_shapes(cuda, shape):
    M, K, N = shape
    _w4_prefill_check(cuda, M, K, N, packed=(M % 2 == 0), seed=M + K)


def test_w4a16_prefill_agrees_with_the_decode_kernel_at_the_boundary(cuda):
    # M = 32 runs the decode kernel, M = 33 the GEMM: the rows they share agree within the contract
    gen = synthetic.torch_generator(cuda, 3, 99)
    K, N = 1024, 512
    x = synthetic.device_normal((33, K), cuda, gen, torch.bfloat16)
    wq = torch.randint(0, 256, (K // 2, N), dtype=torch.uint8, device=cuda, generator=gen)
    sc = synthetic.device_uniform((K // 128, N), 0.002, 0.01, cuda, gen, torch.bfloat16)
    z = torch.randint(0, 16, (K // 128, N), dtype=torch.uint8, device=cuda, generator=gen)
    a = ops.w4a16_g128(x[:32].contiguous(), wq, sc, z)
    b = ops.w4a16_g128(x, wq, sc, z)
    assert O.max_rel_err(bf16_to_np(b[:32].contiguous()), bf16_to_np(a)) <= TOL_BF16


# ---------------------------------------------------------------- config 5 (one rank)
@pytest.mark.parametrize("shape", [(256, 512, 384), (128, 64, 128), (512, 1024, 256), (300, 200, 144),
                                   (4096, 8192, 1024), (1024, 28672, 512)])
def test_w8a16_perchannel(cuda, shape):
    M, K, N = shape
    c = synthetic.config5_small(M, K, N)
    y = ops.w8a16_perchannel(dev(c["x_bits"].view(np.int16), cuda, torch.bfloat16), dev(c["w"], cuda),
                             dev(c["scale"], cuda))
    torch.cuda.synchronize()
    assert _lib.load().qmm_device_status() == 0
    ref = O.w8_perchannel_matmul(c["x"], c["w"], c["scale"])
    err = O.max_rel_err(bf16_to_np(y), ref)
    assert err <= TOL_BF16, err
    # exact products, f32 accumulation, one rounding: within one bf16 ulp of the oracle
    assert np.all(np.abs(bf16_to_np(y) - ref) <= np.abs(ref) * 2.0**-7 + 1e-3 * np.max(np.abs(ref)))


def test_w8a16_writes_a_column_shard_in_place(cuda):
    c = synthetic.config5_small(256, 256, 256)
    x = dev(c["x_bits"].view(np.int16), cuda, torch.bfloat16)
    w, sc = dev(c["w"], cuda), dev(c["scale"], cuda)
    full = ops.w8a16_perchannel(x, w, sc)
    out = torch.zeros((256, 512), dtype=torch.bfloat16, device=cuda)
    ops.w8a16_perchannel(x, w[:, :128].contiguous(), sc[:128].contiguous(), out=out, out_col_offset=256)
    assert torch.equal(out[:, 256:384], full[:, :128])
    assert float(out[:, :256].abs().sum()) == 0 and float(out[:, 384:].abs().sum()) == 0


def _w8a16_rows_check(cuda, M, K, N, seed):
    """Run the kernel on device-generated operands of a bench-sized launch and check four rows of
    every 256-row tile (both row halves of a tile, so every kind of cut tail part is hit) over all
    columns against the oracle."""
    gen = synthetic.torch_generator(cuda, 5, seed)
    x = synthetic.device_normal((M, K), cuda, gen, torch.bfloat16)
    w = synthetic.device_int8((K, N), cuda, gen)
    sc = synthetic.device_uniform((N,), 0.005, 0.02, cuda, gen)
    y = ops.w8a16_perchannel(x, w, sc)
    torch.cuda.synchronize()
    assert _lib.load().qmm_device_status() == 0
    rows = np.array(sorted({min(M - 1, t * 256 + o) for t in range((M + 255) // 256) for o in (3, 100, 131, 250)}))
    rows_t = torch.from_numpy(rows).to(cuda)
    got = bf16_to_np(y[rows_t].contiguous())
    xs = bf16_to_np(x[rows_t].contiguous())
    w_h, sc_h = w.cpu().numpy(), sc.cpu().numpy()
    ref = np.empty((len(rows), N), np.float32)
    for c0 in range(0, N, 4096):  # column chunks bound the oracle's float64 copy of the weights
        ref[:, c0:c0 + 4096] = O.w8_perchannel_matmul(xs, w_h[:, c0:c0 + 4096], sc_h[c0:c0 + 4096])
    err = O.max_rel_err(got, ref)
    assert err <= TOL_BF16, err
    assert np.all(np.abs(got - ref) <= np.abs(ref) * 2.0**-7 + 1e-3 * np.max(np.abs(ref)))


# The four launches of a Llama-3-70B-shaped layer (the benchmark's headline workload) at full width
# and at the column-shard widths of 2, 4 and 8 ranks: every launch has more tiles than SMs or a tail
# that is cut into parts, which the reduced shapes above do not reach.
@pytest.mark.parametrize("name,K,N", [(f"{n}/{p}", k, w // p) for n, k, w in synthetic.config5_layer_shapes()
                                      for p in (1, 2, 4, 8)])
def test_w8a16_bench_launch_shapes(cuda, name, K, N):
    _w8a16_rows_check(cuda, 4096, K, N, seed=K // 64 + N)


@pytest.mark.parametrize("limit", [140, 37, 1, 7, 9, 6, 3])
def test_w8a16_and_int8_dot_under_a_cta_limit(cuda, limit):
    """Fewer persistent CTAs than SMs (SMs left to a collective): same results, bit for bit.

    The w8a16 shape has 20 tiles: limit 7 gives two full rounds and then six whole tail tiles,
    9 a tail cut in quarters, 6 a tail cut in halves, 3 a quarter-cut tail of which a CTA takes a
    run of several parts."""
    lib = _lib.load()
    c = synthetic.config5_small(1024, 512, 1280)
    x = dev(c["x_bits"].view(np.int16), cuda, torch.bfloat16)
    w, sc = dev(c["w"], cuda), dev(c["scale"], cuda)
    rng = np.random.default_rng(77)
    a = torch.from_numpy(rng.integers(-128, 128, (512, 256), dtype=np.int8)).to(cuda)
    b = torch.from_numpy(rng.integers(-128, 128, (256, 768), dtype=np.int8)).to(cuda)
    full = ops.w8a16_perchannel(x, w, sc)
    acc_full, _ = ops.i8_dot(a, b)
    try:
        _lib.check(lib.qmm_set_cta_limit(limit))
        limited = ops.w8a16_perchannel(x, w, sc)
        acc_limited, _ = ops.i8_dot(a, b)
        torch.cuda.synchronize()
    finally:
        _lib.check(lib.qmm_set_cta_limit(0))
    assert lib.qmm_device_status() == 0
    assert torch.equal(full, limited)
    assert torch.equal(acc_full, acc_limited)
    assert lib.qmm_set_cta_limit(-1) != 0


def test_w8a16_small_shape_route(cuda):
    c = synthetic.config5_small(7, 50, 30)
    y = ops.w8a16_perchannel(dev(c["x_bits"].view(np.int16), cuda, torch.bfloat16), dev(c["w"], cuda),
                             dev(c["scale"], cuda))
    assert O.max_rel_err(bf16_to_np(y), O.w8_perchannel_matmul(c["x"], c["w"], c["scale"])) <= TOL_BF16
