"""Launch options of the weight-only int8 GEMM (``qmm_w8a16_perchannel_ex``) and the bounded
signal wait, through the C ABI on one GPU.  The multicast store needs two GPUs and is covered by
``tests/test_gpu_tp_exchange.py``."""

import ctypes

import numpy as np
import pytest
import torch

from jax_metallib_b200 import _lib, ops, synthetic
from oracle import qmm_oracle as O

pytestmark = pytest.mark.gpu


def _operands(cuda, M, K, N, seed):
    gen = synthetic.torch_generator(cuda, 5, seed)
    x = synthetic.device_normal((M, K), cuda, gen, torch.bfloat16)
    w = synthetic.device_int8((K, N), cuda, gen)
    sc = synthetic.device_uniform((N,), 0.005, 0.02, cuda, gen)
    return x, w, sc


def test_independent_launches_overlap_without_changing_results(cuda):
    # a chain of launches that do not wait for one another: every output equals the ordered launch's
    lib = _lib.load()
    probs = [_operands(cuda, 1024, 512, n, 100 + i) for i, n in enumerate((1280, 768, 2560, 1024, 1280, 256))]
    want = [ops.w8a16_perchannel(x, w, sc) for x, w, sc in probs]
    torch.cuda.synchronize()
    outs = [torch.full_like(y, float("nan")) for y in want]
    for _ in range(3):
        for (x, w, sc), out in zip(probs, outs):
            ops.w8a16_perchannel(x, w, sc, out=out, independent=True)
    torch.cuda.synchronize()
    assert lib.qmm_device_status() == 0
    for a, b in zip(outs, want):
        assert torch.equal(a, b)
    x, w, sc = probs[0]
    ref = O.w8_perchannel_matmul(x.float().cpu().numpy(), w.cpu().numpy(), sc.cpu().numpy())
    assert O.max_rel_err(outs[0].float().cpu().numpy(), ref) <= 1e-2


def test_completion_signal_counts_launches_and_wait_passes(cuda):
    lib = _lib.load()
    x, w, sc = _operands(cuda, 512, 256, 1536, 7)
    y = torch.empty((512, 1536), dtype=torch.bfloat16, device=cuda)
    words = torch.zeros(2, dtype=torch.int32, device=cuda)  # [0] signal, [1] arrival counter
    ext = _lib.GemmExt(0, words.data_ptr(), words.data_ptr() + 4)
    stream = torch.cuda.current_stream().cuda_stream
    for _ in range(3):
        _lib.check(lib.qmm_w8a16_perchannel_ex(x.data_ptr(), w.data_ptr(), sc.data_ptr(), y.data_ptr(), 512, 1536, 256,
                                               1536, ctypes.byref(ext), stream))
    # the signal is already on its way (same GPU, earlier in the stream): the wait returns at once
    _lib.check(lib.qmm_wait_signals(words.data_ptr(), 1, 3, 0, stream))
    torch.cuda.synchronize()
    assert words.tolist() == [3, 0]  # three launches signalled; the arrival counter wrapped back to zero
    assert lib.qmm_device_status() == 0
    assert torch.equal(y, ops.w8a16_perchannel(x, w, sc))


def test_signal_wait_gives_up_with_a_status_instead_of_hanging(cuda):
    # a word that nothing sets: the wait runs out after 50 ms, records a timeout and the context stays usable
    lib = _lib.load()
    word = torch.zeros(1, dtype=torch.int32, device=cuda)
    try:
        _lib.check(lib.qmm_wait_signals(word.data_ptr(), 1, 1, 50_000_000, torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()
        st = lib.qmm_device_status()
        assert st & 0xFFFF == 5 and st >> 16 == 60  # QMM_ERR_TIMEOUT, site tag of the signal wait
        x, w, sc = _operands(cuda, 256, 128, 256, 9)
        with pytest.raises(_lib.QmmError) as e:  # launches are refused while the word is set
            ops.w8a16_perchannel(x, w, sc)
        assert e.value.status_name == "QMM_ERR_TIMEOUT"
    finally:
        lib.qmm_clear_device_status()
    assert lib.qmm_device_status() == 0
    y = ops.w8a16_perchannel(x, w, sc)
    torch.cuda.synchronize()
    assert torch.isfinite(y.float()).all()


def test_ext_rejects_bad_options(cuda):
    lib = _lib.load()
    x, w, sc = _operands(cuda, 256, 128, 256, 11)
    y = torch.empty((256, 256), dtype=torch.bfloat16, device=cuda)
    ext = _lib.GemmExt(0x80)
    st = lib.qmm_w8a16_perchannel_ex(x.data_ptr(), w.data_ptr(), sc.data_ptr(), y.data_ptr(), 256, 256, 128, 256,
                                     ctypes.byref(ext), None)
    assert lib.qmm_status_name(st) == b"QMM_ERR_INVALID_ARGUMENT" and "flag" in _lib.last_error()
    word = torch.zeros(1, dtype=torch.int32, device=cuda)
    ext = _lib.GemmExt(0, word.data_ptr(), None)
    st = lib.qmm_w8a16_perchannel_ex(x.data_ptr(), w.data_ptr(), sc.data_ptr(), y.data_ptr(), 256, 256, 128, 256,
                                     ctypes.byref(ext), None)
    assert lib.qmm_status_name(st) == b"QMM_ERR_INVALID_ARGUMENT"
    # the CUDA-core route (a shape TMA cannot describe) cannot signal
    ext = _lib.GemmExt(0, word.data_ptr(), word.data_ptr())
    st = lib.qmm_w8a16_perchannel_ex(x.data_ptr(), w.data_ptr(), sc.data_ptr(), y.data_ptr(), 7, 30, 50, 30,
                                     ctypes.byref(ext), None)
    assert lib.qmm_status_name(st) == b"QMM_ERR_UNSUPPORTED"
