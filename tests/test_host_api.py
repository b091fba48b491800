"""Host-side logic of the operator API and the C-ABI library (no GPU needed)."""

import ctypes
import os
import re

import numpy as np
import pytest

from jax_metallib_b200 import _lib
from jax_metallib_b200 import quantized as Q

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_loads_and_exports_every_declared_symbol():
    inc = os.path.join(ROOT, "include")
    header = "".join(open(os.path.join(inc, f)).read() for f in sorted(os.listdir(inc)) if f.endswith(".h"))
    declared = set(re.findall(r"QMM_API\s+[\w\s\*]+?\b(qmm_\w+)\s*\(", header))
    assert len(declared) >= 100
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} is declared in include/qmm.h but not exported"
    assert declared <= set(_lib.SIGNATURES), "every declared entry point has a ctypes signature"
    assert b"sm_100a" in _lib.load().qmm_version()


def test_per_device_bookkeeping_selftest():
    # function attributes (dynamic shared-memory opt-in) are set once per device ordinal, not once per process
    assert _lib.load().qmm_selftest_host() == 0


def test_error_reporting_without_a_gpu():
    lib = _lib.load()
    # argument validation happens before any CUDA call
    st = lib.qmm_w4a16_g128(None, None, None, None, 0, None, 1, 128, 128, 128, None, 0, 0, None)
    assert st == 1 and lib.qmm_status_name(st) == b"QMM_ERR_INVALID_ARGUMENT"
    assert "null" in _lib.last_error()
    buf = ctypes.create_string_buffer(8)
    full = lib.qmm_last_error(buf, 8)
    assert full > 7 and len(buf.value) == 7  # truncated, NUL-terminated
    assert lib.qmm_w4a16_g128_workspace_bytes(1, 100, 4096) == 0  # N not a multiple of 128
    assert lib.qmm_w4a16_g128_workspace_bytes(1, 14336, 4096) > 0
    with pytest.raises(_lib.QmmError) as e:
        _lib.check(lib.qmm_affine_matmul(1, 1, 1, 1, 1, 1, 1, 64, 3, 64, 0, None))
    assert e.value.status_name == "QMM_ERR_UNSUPPORTED"


def test_gather_copy_entry_points_validate_before_any_cuda_call():
    """qmm_multicast_copy / qmm_peer_copy: null, misaligned and out-of-range arguments are refused
    with QMM_ERR_INVALID_ARGUMENT (no launch is attempted, so this runs without a GPU)."""
    lib = _lib.load()
    buf = (ctypes.c_uint8 * 256)()
    base = ctypes.addressof(buf)
    base += (-base) % 16
    assert lib.qmm_multicast_copy(None, base, 64, base, base, 0, None) == 1
    assert lib.qmm_multicast_copy(base, base + 16, 40, base + 32, base + 36, 0, None) == 1      # bytes not a multiple of 16
    assert lib.qmm_multicast_copy(base + 4, base + 16, 64, base + 32, base + 36, 0, None) == 1  # misaligned source
    assert lib.qmm_multicast_copy(base, base + 16, 64, base + 32, base + 36, -1, None) == 1
    assert lib.qmm_multicast_copy(base, base + 16, 0, base + 32, base + 36, 0, None) == 0       # nothing to copy
    dst = (ctypes.c_void_p * 2)(base + 64, base + 128)
    sig = (ctypes.c_void_p * 2)(base + 192, base + 196)
    assert lib.qmm_peer_copy(base, dst, sig, 0, 64, base + 200, base + 204, 0, None) == 1        # no peers
    assert lib.qmm_peer_copy(base, dst, sig, 16, 64, base + 200, base + 204, 0, None) == 1       # more than QMM_MAX_PEERS
    bad = (ctypes.c_void_p * 2)(base + 64, None)
    assert lib.qmm_peer_copy(base, bad, sig, 2, 64, base + 200, base + 204, 0, None) == 1
    assert "peer 1" in _lib.last_error()
    assert lib.qmm_peer_copy(base, dst, sig, 2, 0, base + 200, base + 204, 0, None) == 0


def test_codecs_match_reference_fixtures(golden):
    p = golden["codec_probe"]
    np.testing.assert_array_equal(Q._fp4_e2m1_quantize(p), golden["e2m1_encode_probe"])
    np.testing.assert_array_equal(Q._fp8_e4m3_quantize(p), golden["e4m3_encode_probe"])
    np.testing.assert_array_equal(Q._fp8_e8m0_quantize(np.abs(p)), golden["e8m0_encode_probe"])
    codes = np.arange(256, dtype=np.uint8)
    np.testing.assert_array_equal(Q._fp8_e4m3_dequantize(codes), golden["e4m3_decode_table"])
    np.testing.assert_array_equal(Q._fp8_e8m0_dequantize(codes), golden["e8m0_decode_table"])
    np.testing.assert_array_equal(Q._fp4_e2m1_dequantize(codes[:16]), golden["e2m1_decode_table"])


@pytest.mark.parametrize("mode", ["mxfp4", "mxfp8", "nvfp4"])
def test_mx_roundtrip_shapes_and_fixtures(golden, mode):
    for shape in ("4x8x64", "8x16x64", "16x32x128"):
        tag = f"mx_{mode}_{shape}"
        w = golden[tag + "_w"]
        p, s = Q.mx_quantize(w, mode=mode)
        assert p.dtype == np.uint8 and s.dtype == np.uint8
        np.testing.assert_array_equal(p, golden[tag + "_packed"])
        np.testing.assert_array_equal(s, golden[tag + "_scales"])
        np.testing.assert_array_equal(Q.mx_dequantize(p, s, mode=mode, shape=w.shape), golden[tag + "_dequant"])
    cfg = Q._MX_MODES[mode]
    p, s = Q.mx_quantize(np.ones((16, 128), np.float32), mode=mode)
    assert p.shape == (16, 128 // (2 if cfg["bits"] == 4 else 1)) and s.shape == (16, 128 // cfg["group_size"])
    p, s = Q.mx_quantize(np.zeros((2, 64), np.float32), mode=mode)
    np.testing.assert_array_equal(Q.mx_dequantize(p, s, mode=mode, shape=(2, 64)), 0.0)
    # roundtrip tolerance of tests/test_quantized.py:167-186
    w = np.random.default_rng(42).standard_normal((4, 64)).astype(np.float32) * 0.1
    p, s = Q.mx_quantize(w, mode=mode)
    np.testing.assert_allclose(Q.mx_dequantize(p, s, mode=mode, shape=w.shape), w,
                               atol=0.15 if "fp4" in mode else 0.1, rtol=0.8)


@pytest.mark.parametrize("bits", [2, 3, 4, 8])
def test_affine_roundtrip_and_fixtures(golden, bits):
    for gs in (32, 64, 128):
        tag = f"affine_b{bits}_g{gs}"
        w = golden[tag + "_w"]
        p, s, b = Q.affine_quantize(w, bits=bits, group_size=gs)
        assert p.dtype == golden[tag + "_packed"].dtype
        np.testing.assert_array_equal(p, golden[tag + "_packed"])
        np.testing.assert_array_equal(s, golden[tag + "_scales"])
        np.testing.assert_array_equal(b, golden[tag + "_biases"])
        np.testing.assert_array_equal(Q.affine_dequantize(p, s, b, bits=bits, group_size=gs, shape=w.shape),
                                      golden[tag + "_dequant"])
    if bits in (4, 8):
        p, s, b = Q.affine_quantize(np.ones((16, 128), np.float32), bits=bits, group_size=64)
        assert p.shape == ((16, 16) if bits == 4 else (16, 128))
        assert p.dtype == (np.uint32 if bits == 4 else np.uint8)
        assert s.shape == (16, 2) and b.shape == (16, 2)


def test_value_errors_match_reference_behaviour():
    w = np.ones((2, 48), np.float32)
    with pytest.raises(ValueError, match="Unknown mode"):
        Q.mx_quantize(w, mode="fp3")
    with pytest.raises(ValueError, match="divisible by group_size"):
        Q.mx_quantize(w, mode="mxfp4")
    with pytest.raises(ValueError, match="shape is required"):
        Q.mx_dequantize(np.zeros((2, 16), np.uint8), np.zeros((2, 1), np.uint8), mode="mxfp4")
    with pytest.raises(ValueError, match="bits must be"):
        Q.affine_quantize(w, bits=5)
    with pytest.raises(ValueError, match="divisible by group_size"):
        Q.affine_quantize(w, bits=4, group_size=64)
    with pytest.raises(ValueError, match="shape is required"):
        Q.affine_dequantize(np.zeros((2, 8), np.uint32), np.ones((2, 1)), np.zeros((2, 1)), bits=4)
    with pytest.raises(ValueError, match="Unknown mode"):
        Q.quantized_matmul(np.ones((1, 32), np.float32), np.zeros((1, 16), np.uint8), np.zeros((1, 1), np.uint8),
                           mode="bogus", K=32)


def test_matmul_refuses_to_run_without_cuda():
    import torch

    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    w = np.ones((2, 64), np.float32)
    p, s, b = Q.affine_quantize(w, bits=4, group_size=64)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        Q.affine_quantized_matmul(np.ones((1, 64), np.float32), p, s, b, bits=4, group_size=64, K=64)


# ---- runtime events: host-side objects, no GPU involved -------------------------------------------
def test_event_bounded_await_set_and_callbacks():
    """A caller-facing wait gives up after its timeout with a DEADLINE_EXCEEDED-class status and leaves
    the event pending (src/pjrt_plugin/core/completion_event.h:62-83, api/pjrt_event.cc:46-59)."""
    import time

    from jax_metallib_b200 import runtime

    lib = _lib.load()
    ev = runtime.Event()
    assert not ev.is_ready()
    t0 = time.time()
    with pytest.raises(_lib.QmmError) as e:
        ev.await_(60)  # nothing sets it: the wait runs out on the host
    assert e.value.status_name == "QMM_ERR_TIMEOUT" and 0.05 <= time.time() - t0 < 5.0
    assert lib.qmm_rt_status_to_pjrt_code(e.value.status) == 4  # DEADLINE_EXCEEDED
    assert not ev.is_ready()  # still pending
    seen = []
    ev.on_ready(lambda status, msg: seen.append((status, msg)))
    assert seen == []
    ev.set()
    assert ev.is_ready() and seen == [(0, "")]
    ev.await_(10)
    ev.on_ready(lambda status, msg: seen.append("late"))  # ready already: runs at once
    assert seen[-1] == "late"
    ev.set(3, "second completion is ignored")
    assert ev.error() == 0
    bad = runtime.Event()
    bad.set(3, "upload failed")
    with pytest.raises(_lib.QmmError) as e:
        bad.await_(10)
    assert "upload failed" in str(e.value) and e.value.status == 3


def test_runtime_timeout_env_is_read_per_wait(monkeypatch):
    import time

    from jax_metallib_b200 import runtime

    ev = runtime.Event()
    monkeypatch.setenv("QMM_RT_COMPLETION_TIMEOUT_MS", "40")
    t0 = time.time()
    with pytest.raises(_lib.QmmError):
        ev.await_()
    assert time.time() - t0 < 5.0
