"""Textual StableHLO in, fused kernels out: the compile/execute path on the GPU,
checked against the CPU oracle at the shapes the fixtures declare."""

import os

import numpy as np
import pytest
import torch

from jax_metallib_b200 import synthetic
from jax_metallib_b200.stablehlo import Executable
from oracle import qmm_oracle as O

pytestmark = pytest.mark.gpu
FIX = os.path.join(os.path.dirname(os.path.abspath(__file__)), "fixtures")


def load(name):
    return open(os.path.join(FIX, name)).read()


def dev(a, cuda, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).to(cuda)
    return t if dtype is None else t.view(dtype)


def bf16_np(t):
    return synthetic.bf16_bits_to_f32(t.view(torch.int16).cpu().numpy().view(np.uint16))


def test_config1_module(cuda):
    exe = Executable(load("cfg1_w8a32.mlir"))
    c = synthetic.config1()
    out = torch.empty((32, 1024), dtype=torch.float32, device=cuda)
    exe([dev(c["x"], cuda), dev(c["w"], cuda), dev(c["scale"], cuda)], [out])
    assert O.max_rel_err(out.cpu().numpy(), O.w8_perchannel_matmul(c["x"], c["w"], c["scale"])) <= 2e-3


def test_config2_module_returns_accumulator_and_rescaled_output(cuda):
    exe = Executable(load("cfg2_i8dot_rescale.mlir"))
    c = synthetic.config2()
    acc = torch.empty((2048, 4096), dtype=torch.int32, device=cuda)
    out = torch.empty((2048, 4096), dtype=torch.float32, device=cuda)
    exe([dev(c["a"], cuda), dev(c["b"], cuda), dev(c["row"], cuda), dev(c["col"], cuda)], [acc, out])
    ref = O.i8_dot_i32(c["a"], c["b"])
    np.testing.assert_array_equal(acc.cpu().numpy(), ref)
    assert O.max_rel_err(out.cpu().numpy(), O.i8_dot_rescale(ref, c["row"], c["col"])) <= 2e-3


def test_config3_module_with_packed_ui4_zero_points(cuda):
    exe = Executable(load("cfg3_w4a16.mlir"))
    c = synthetic.config3(4, 4096, 14336)
    out = torch.empty((4, 14336), dtype=torch.bfloat16, device=cuda)
    args = [dev(c["x_bits"].view(np.int16), cuda, torch.bfloat16), dev(c["wq"], cuda),
            dev(c["s_bits"].view(np.int16), cuda, torch.bfloat16), dev(c["z_packed"], cuda)]
    exe(args, [out])
    exe(args, [out])  # the plan's workspace is reusable
    assert O.max_rel_err(bf16_np(out), O.w4a16_matmul(c["x"], c["wq"], c["s"], c["z"])) <= 1e-2


def test_config5_module(cuda):
    exe = Executable(load("cfg5_w8a16.mlir"))
    c = synthetic.config5_small(4096, 8192, 1024)
    out = torch.empty((4096, 1024), dtype=torch.bfloat16, device=cuda)
    exe([dev(c["x_bits"].view(np.int16), cuda, torch.bfloat16), dev(c["w"], cuda), dev(c["scale"], cuda)], [out])
    assert O.max_rel_err(bf16_np(out), O.w8_perchannel_matmul(c["x"], c["w"], c["scale"])) <= 1e-2


# ---------------------------------------------------------------- around the fused patterns
def _run(name, cuda, host_args, out_specs, bf16_args=()):
    exe = Executable(load(name))
    args = [dev(a, cuda, torch.bfloat16) if i in bf16_args else dev(a, cuda) for i, a in enumerate(host_args)]
    outs = [torch.full(shape, -7, dtype=dt, device=cuda) for shape, dt in out_specs]
    exe(args, outs)
    torch.cuda.synchronize()
    return exe, outs


def test_unfused_chain_computes_the_same_values_op_by_op(cuda):
    rng = np.random.default_rng(21)
    x = rng.standard_normal((32, 256)).astype(np.float32)
    w = rng.integers(-127, 128, size=(256, 128)).astype(np.int8)
    s = rng.uniform(0.005, 0.02, size=(128,)).astype(np.float32)
    exe, (y, wd) = _run("unfused_escaping_intermediate.mlir", cuda, [x, w, s],
                        [((32, 128), torch.float32), ((256, 128), torch.float32)])
    assert [t["event"] for t in exe.trace()].count("fused") == 0
    np.testing.assert_array_equal(wd.cpu().numpy(), O.w8_perchannel_dequant(w, s))  # convert and multiply are exact f32 ops
    assert O.max_rel_err(y.cpu().numpy(), O.w8_perchannel_matmul(x, w, s)) <= 2e-3
    # a [N, K] weight: dequantised, transposed, multiplied
    x = rng.standard_normal((16, 256)).astype(np.float32)
    wt = rng.integers(-127, 128, size=(128, 256)).astype(np.int8)
    _, (y,) = _run("unfused_transposed_weight.mlir", cuda, [x, wt, s], [((16, 128), torch.float32)])
    assert O.max_rel_err(y.cpu().numpy(), O.w8_perchannel_matmul(x, wt.T.copy(), s)) <= 2e-3
    # the same contraction written as [M, K] x [N, K] in bf16
    xb = synthetic.to_bf16_bits(x)
    _, (y,) = _run("unfused_contract_rhs_dim1.mlir", cuda, [xb.view(np.int16), wt, s], [((16, 128), torch.bfloat16)],
                   bf16_args=(0,))
    ref = O.w8_perchannel_matmul(synthetic.bf16_bits_to_f32(xb), wt.T.copy(), s)
    assert O.max_rel_err(bf16_np(y), ref) <= 1e-2


def test_legacy_dot_constants_bias_and_trailing_convert(cuda):
    rng = np.random.default_rng(22)
    x = rng.standard_normal((32, 256)).astype(np.float32)
    w = rng.integers(-127, 128, size=(256, 128)).astype(np.int8)
    s = rng.uniform(0.005, 0.02, size=(128,)).astype(np.float32)
    _, (y,) = _run("legacy_dot_w8a32.mlir", cuda, [x, w, s], [((32, 128), torch.float32)])
    assert O.max_rel_err(y.cpu().numpy(), O.w8_perchannel_matmul(x, w, s)) <= 2e-3
    # weight and scale are dense constants of the module, the bias is added by a standalone kernel
    x = rng.integers(-4, 5, size=(8, 4)).astype(np.float32)
    bias = np.array([1.0, -2.0, 0.5], np.float32)
    wc = np.array([[1, -2, 3], [4, 5, -6], [-7, 8, 9], [10, -11, 12]], np.float32)
    sc = np.array([0.5, 0.25, 2.0], np.float32)
    _, (y,) = _run("const_weight_bias_add.mlir", cuda, [x, bias], [((8, 3), torch.float32)])
    np.testing.assert_array_equal(y.cpu().numpy(), (x @ wc) * sc + bias)  # small integers: exact in f32
    c = synthetic.config5_small(256, 512, 384)
    _, (y,) = _run("cfg5_f32_accumulate_then_convert.mlir", cuda, [c["x_bits"].view(np.int16), c["w"], c["scale"]],
                   [((256, 384), torch.bfloat16)], bf16_args=(0,))
    assert O.max_rel_err(bf16_np(y), O.w8_perchannel_matmul(c["x"], c["w"], c["scale"])) <= 1e-2


def test_int8_typed_dot_wraps_and_shape_ops(cuda):
    rng = np.random.default_rng(0)  # tests/test_int_dot.py: an i8 result wraps mod 2^8 after an int32 accumulate
    a = rng.integers(-300, 300, size=(5, 7), dtype=np.int64).astype(np.int8)
    b = rng.integers(-300, 300, size=(7, 3), dtype=np.int64).astype(np.int8)
    _, (y,) = _run("int8_result_wraps.mlir", cuda, [a, b], [((5, 3), torch.int8)])
    np.testing.assert_array_equal(y.cpu().numpy(), (a.astype(np.int32) @ b.astype(np.int32)).astype(np.int8))
    p = rng.integers(0, 1 << 20, size=(6, 8)).astype(np.int32)
    q = rng.integers(0, 1 << 20, size=(6, 2)).astype(np.int32)
    _, (y,) = _run("unfused_slice_concat.mlir", cuda, [p, q], [((6, 6), torch.int32)])
    np.testing.assert_array_equal(y.cpu().numpy(), np.concatenate([p[:, 1:8:2], q], axis=1) >> 3)


def test_custom_call_route_runs_the_named_kernels(cuda):
    from jax_metallib_b200 import custom_call as cc

    c = synthetic.config5_small(256, 512, 384)
    text = cc.module_text(["tensor<256x512xbf16>", "tensor<512x384xi8>", "tensor<384xf32>"], "tensor<256x384xbf16>",
                          cc.backend_config("w8a16_perchannel"))
    exe = Executable(text)
    out = torch.empty((256, 384), dtype=torch.bfloat16, device=cuda)
    exe([dev(c["x_bits"].view(np.int16), cuda, torch.bfloat16), dev(c["w"], cuda), dev(c["scale"], cuda)], [out])
    assert O.max_rel_err(bf16_np(out), O.w8_perchannel_matmul(c["x"], c["w"], c["scale"])) <= 1e-2
    c = synthetic.config2(128, 256, 384)
    text = cc.module_text(["tensor<128x256xi8>", "tensor<256x384xi8>", "tensor<128xf32>", "tensor<384xf32>"],
                          "tensor<128x384xf32>", cc.backend_config("i8i8_i32"))
    out = torch.empty((128, 384), dtype=torch.float32, device=cuda)
    Executable(text)([dev(c["a"], cuda), dev(c["b"], cuda), dev(c["row"], cuda), dev(c["col"], cuda)], [out])
    np.testing.assert_array_equal(out.cpu().numpy(), O.i8_dot_rescale(O.i8_dot_i32(c["a"], c["b"]), c["row"], c["col"]))
    c = synthetic.config3(4, 1024, 512)
    text = cc.module_text(["tensor<4x1024xbf16>", "tensor<512x512xui8>", "tensor<8x512xbf16>", "tensor<8x256xui8>"],
                          "tensor<4x512xbf16>", cc.backend_config("w4a16_g128", zeros_packed=True))
    out = torch.empty((4, 512), dtype=torch.bfloat16, device=cuda)
    Executable(text)([dev(c["x_bits"].view(np.int16), cuda, torch.bfloat16), dev(c["wq"], cuda),
                      dev(c["s_bits"].view(np.int16), cuda, torch.bfloat16), dev(c["z_packed"], cuda)], [out])
    assert O.max_rel_err(bf16_np(out), O.w4a16_matmul(c["x"], c["wq"], c["s"], c["z"])) <= 1e-2


def test_scan_over_two_layers_runs_on_views_of_the_stacked_weights(cuda):
    exe = Executable(load("scan_two_layers_w8a16.mlir"))
    rng = np.random.default_rng(31)
    xb = synthetic.to_bf16_bits(rng.standard_normal((256, 512)).astype(np.float32))
    w = rng.integers(-127, 128, size=(2, 512, 512)).astype(np.int8)
    s = rng.uniform(0.001, 0.004, size=(2, 512)).astype(np.float32)
    out = torch.empty((256, 512), dtype=torch.bfloat16, device=cuda)
    exe([dev(xb.view(np.int16), cuda, torch.bfloat16), dev(w, cuda), dev(s, cuda)], [out])
    torch.cuda.synchronize()
    h = O.round_to_bf16(O.w8_perchannel_matmul(synthetic.bf16_bits_to_f32(xb), w[0], s[0]))  # layer 0's bf16 output
    ref = O.w8_perchannel_matmul(h, w[1], s[1])
    assert O.max_rel_err(bf16_np(out), ref) <= 1e-2
