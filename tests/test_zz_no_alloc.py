"""The allocation-free variant of the int4 decode matmul.

Some hosts of this library cannot hand it a workspace: code that runs under a
runtime which has already claimed almost all device memory (where a fresh
cudaMalloc may fail), or a token-by-token decode loop that cannot afford the
device-wide synchronisation an allocation brings.  For them
``qmm_w4a16_g128_static_scratch`` keeps its split-K scratch in a fixed array
inside the library.  This test calls it through the C ABI, twice in a row (the
second call finds the array as the first one left it), and compares every
output with the ordinary entry point, which gets a caller-provided workspace.
Both run the same kernel with the same summation order, so the outputs must
agree bit for bit — well inside the 1e-2 contract the other decode tests use.

The file name sorts last so that a run stopped at the first failure has
already executed every other test.
"""

import ctypes

import numpy as np
import pytest
import torch

from jax_metallib_b200 import _lib, synthetic
from oracle import qmm_oracle as O

pytestmark = pytest.mark.gpu

TOL_BF16 = 1e-2
SCRATCH_LIMIT = 8 << 20  # QMM_STATIC_SCRATCH_BYTES in include/qmm.h


def _dev(a, cuda, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).to(cuda)
    return t if dtype is None else t.view(dtype)


def _bf16_to_np(t):
    return synthetic.bf16_bits_to_f32(t.view(torch.int16).cpu().numpy().view(np.uint16))


@pytest.mark.parametrize("shape,packed", [((4, 4096, 14336), True), ((16, 4096, 14336), False), ((8, 1024, 512), True)])
def test_static_scratch_matches_workspace_entry_point_twice(cuda, shape, packed):
    M, K, N = shape
    lib = _lib.load()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    need = lib.qmm_w4a16_g128_workspace_bytes(M, N, K)
    assert 0 < need <= SCRATCH_LIMIT
    ws = torch.zeros(need, dtype=torch.uint8, device=cuda)
    ref_np = None
    for call in range(2):  # two calls in a row, fresh inputs each time
        c = synthetic.config3(M, K, N, index=10 + call)
        x = _dev(c["x_bits"].view(np.int16), cuda, torch.bfloat16)
        wq = _dev(c["wq"], cuda)
        s = _dev(c["s_bits"].view(np.int16), cuda, torch.bfloat16)
        z = _dev(c["z_packed"] if packed else c["z"], cuda)
        want = torch.empty((M, N), dtype=torch.bfloat16, device=cuda)
        got = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=cuda)
        _lib.check(lib.qmm_w4a16_g128(x.data_ptr(), wq.data_ptr(), s.data_ptr(), z.data_ptr(), int(packed),
                                      want.data_ptr(), M, N, K, 128, ws.data_ptr(), ws.numel(), 0, stream))
        _lib.check(lib.qmm_w4a16_g128_static_scratch(x.data_ptr(), wq.data_ptr(), s.data_ptr(), z.data_ptr(),
                                                     int(packed), got.data_ptr(), M, N, K, 128, stream))
        torch.cuda.synchronize()
        assert lib.qmm_device_status() == 0
        a, b = _bf16_to_np(got), _bf16_to_np(want)
        assert O.max_rel_err(a, b) <= TOL_BF16
        assert torch.equal(got, want)  # same kernel, same fixed summation order
        ref_np = O.w4a16_matmul(c["x"], c["wq"], c["s"], c["z"])
        assert O.max_rel_err(a, ref_np) <= TOL_BF16
    assert ref_np is not None


def test_static_scratch_refuses_shapes_beyond_its_limit(cuda):
    lib = _lib.load()
    M, K, N = 32, 4096, 28672
    assert lib.qmm_w4a16_g128_workspace_bytes(M, N, K) > SCRATCH_LIMIT
    c = synthetic.config3(M, 256, 128)  # small tensors: the size check comes before any launch
    x = _dev(c["x_bits"].view(np.int16), cuda, torch.bfloat16)
    wq, s, z = _dev(c["wq"], cuda), _dev(c["s_bits"].view(np.int16), cuda, torch.bfloat16), _dev(c["z"], cuda)
    y = torch.empty((M, 128), dtype=torch.bfloat16, device=cuda)
    st = lib.qmm_w4a16_g128_static_scratch(x.data_ptr(), wq.data_ptr(), s.data_ptr(), z.data_ptr(), 0, y.data_ptr(),
                                           M, N, K, 128, None)
    assert lib.qmm_status_name(st) == b"QMM_ERR_WORKSPACE"
    msg = _lib.last_error()
    assert "built-in" in msg and str(SCRATCH_LIMIT) in msg


def test_static_scratch_calls_leave_free_device_memory_unchanged(cuda):
    """What the name of the entry point promises: once the library's device image is loaded (the
    first call on a device does that), further calls neither take nor give back device memory."""
    lib = _lib.load()
    M, K, N = 4, 1024, 512
    c = synthetic.config3(M, K, N, index=21)
    x = _dev(c["x_bits"].view(np.int16), cuda, torch.bfloat16)
    wq, s, z = _dev(c["wq"], cuda), _dev(c["s_bits"].view(np.int16), cuda, torch.bfloat16), _dev(c["z_packed"], cuda)
    y = torch.empty((M, N), dtype=torch.bfloat16, device=cuda)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def call():
        _lib.check(lib.qmm_w4a16_g128_static_scratch(x.data_ptr(), wq.data_ptr(), s.data_ptr(), z.data_ptr(), 1,
                                                     y.data_ptr(), M, N, K, 128, stream))

    call()  # resolves the array's address and loads the kernel
    torch.cuda.synchronize()
    for _attempt in range(3):  # another process on the device may move the figure; it must hold at least once
        free_before, _ = torch.cuda.mem_get_info(cuda)
        for _ in range(3):
            call()
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info(cuda)
        if free_after == free_before:
            break
    assert free_after == free_before
