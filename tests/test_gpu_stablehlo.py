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
