"""The runtime layer (client / buffer / event / executable) through its C ABI on the GPU.

What the reference pins for its PJRT objects is checked here at the level below the PJRT table:
distinct clients with their own handles and user data (tests/test_pjrt_client_ownership.py:118-158),
strided and zero-element uploads (src/pjrt_plugin/core/mps_client.mm:133-215), range-checked raw reads
(core/mps_buffer.mm:393-423), failures of a host read reported through its event
(api/pjrt_buffer.cc:217-234), and execution of the StableHLO fixtures with outputs returned at once
behind a producer event (api/pjrt_executable.cc:253-298), each compared with the CPU oracle."""

import ctypes
import os

import numpy as np
import pytest

from jax_metallib_b200 import _lib, runtime, synthetic
from oracle import qmm_oracle as O

pytestmark = pytest.mark.gpu
FIX = os.path.join(os.path.dirname(os.path.abspath(__file__)), "fixtures")


def load(name):
    return open(os.path.join(FIX, name)).read()


@pytest.fixture(scope="module")
def client(cuda):
    c = runtime.Client()
    yield c
    c.destroy()


def test_every_client_is_distinct_and_owns_its_handles_and_user_data(cuda):
    lib = _lib.load()
    a, b = runtime.Client(), runtime.Client()
    assert a._h != b._h and a.num_devices >= 1 and a.platform_name == "qmm_b200"
    assert "sm_100a" in a.platform_version
    assert a.device_handle(0) != b.device_handle(0) and a.memory_handle(0) != b.memory_handle(0)
    assert lib.qmm_rt_memory_device(a.memory_handle(0)) == a.device_handle(0)
    assert lib.qmm_rt_memory_kind(a.memory_handle(0)) == b"device"
    assert "SMs" in a.device_debug_string(0)
    dev = ctypes.c_void_p()
    assert lib.qmm_rt_client_lookup_device(a._h, 0, ctypes.byref(dev)) == 0 and dev.value == a.device_handle(0)
    assert lib.qmm_rt_client_lookup_device(a._h, 9999, ctypes.byref(dev)) != 0
    assign = (ctypes.c_int * 1)()
    assert lib.qmm_rt_client_default_device_assignment(a._h, 1, 1, assign, 1) == 0 and assign[0] == 0
    # keyed user data: isolated per client, destroyed exactly once with its owner
    destroyed = []
    deleter_t = ctypes.CFUNCTYPE(None, ctypes.c_void_p)
    deleter = deleter_t(lambda p: destroyed.append(p))
    d = ctypes.cast(deleter, ctypes.c_void_p)
    assert lib.qmm_rt_memory_set_user_data(a.memory_handle(0), 7, 0x1001, d) == 0
    assert lib.qmm_rt_memory_set_user_data(b.memory_handle(0), 7, 0x2002, d) == 0
    assert lib.qmm_rt_memory_get_user_data(a.memory_handle(0), 7) == 0x1001
    assert lib.qmm_rt_memory_get_user_data(b.memory_handle(0), 7) == 0x2002
    assert not lib.qmm_rt_memory_get_user_data(a.memory_handle(0), 8)
    assert lib.qmm_rt_memory_set_user_data(a.memory_handle(0), 7, 0x1003, d) == 0  # replaces: old datum destroyed
    assert destroyed == [0x1001]
    a.destroy()
    assert destroyed == [0x1001, 0x1003]
    assert lib.qmm_rt_memory_get_user_data(b.memory_handle(0), 7) == 0x2002  # the other client is untouched
    b.destroy()
    assert destroyed == [0x1001, 0x1003, 0x2002]


def test_strided_and_zero_element_uploads_and_raw_reads(client):
    rng = np.random.default_rng(3)
    base = rng.standard_normal((6, 10, 8)).astype(np.float32)
    for view in (base, base.transpose(2, 0, 1), base[:, ::3, 1:7:2], base[1], base[..., 0], base[::-1]):
        buf, done = client.buffer_from_host(view, want_event=True)
        done.await_(5000)
        assert buf.shape == view.shape and buf.nbytes == view.size * 4
        np.testing.assert_array_equal(buf.to_numpy(), np.ascontiguousarray(view))
        buf.destroy()
    used0, limit = client.memory_stats(0)
    empty = client.buffer_from_host(np.zeros((5, 0, 3), np.float32))
    assert empty.shape == (5, 0, 3) and empty.nbytes == 0 and empty.device_pointer != 0
    assert empty.to_numpy().shape == (5, 0, 3)
    assert client.memory_stats(0)[0] > used0 and limit > 1 << 30
    empty.destroy()
    assert client.memory_stats(0)[0] == used0
    # raw reads are range-checked and report failure through the event
    src = np.arange(64, dtype=np.int32)
    buf = client.buffer_from_host(src)
    out = np.zeros(8, np.int32)
    ev = buf.copy_raw_to_host(out, 32, 32)
    ev.await_(5000)
    np.testing.assert_array_equal(out, src[8:16])
    ev = buf.copy_raw_to_host(out, 250, 32)
    with pytest.raises(_lib.QmmError) as e:
        ev.await_(5000)
    assert "out of range" in str(e.value)
    small = np.zeros(4, np.int32)
    ev = buf.to_host(small)  # a destination that is too small: the call succeeds, the event carries the error
    with pytest.raises(_lib.QmmError):
        ev.await_(5000)
    # delete: the handle survives, reads are refused, destroy is still fine
    buf.delete()
    assert buf.is_deleted()
    ev = buf.to_host(np.zeros(64, np.int32))
    with pytest.raises(_lib.QmmError) as e:
        ev.await_(5000)
    assert "deleted" in str(e.value)
    buf.destroy()


def test_ready_events_callbacks_and_external_references(client):
    lib = _lib.load()
    x = np.arange(1 << 20, dtype=np.float32)
    buf = client.buffer_from_host(x)
    ev = buf.ready_event()
    seen = []
    ev.on_ready(lambda status, msg: seen.append(status))
    ev.await_(5000)
    assert ev.is_ready() and ev.error() == 0
    for _ in range(200):  # the callback runs on the completion thread
        if seen:
            break
        import time
        time.sleep(0.005)
    assert seen == [0]
    # an external reference keeps the storage alive across delete
    assert lib.qmm_rt_buffer_increase_external_refs(buf._h) == 0
    ptr = buf.device_pointer
    buf.delete()
    assert buf.is_deleted() and buf.device_pointer == ptr
    assert lib.qmm_rt_buffer_decrease_external_refs(buf._h) == 0
    assert buf.device_pointer == 0
    assert lib.qmm_rt_buffer_decrease_external_refs(buf._h) != 0
    buf.destroy()


def test_view_of_device_memory_and_error_buffer(client):
    import torch

    lib = _lib.load()
    t = torch.arange(256, dtype=torch.float32, device="cuda:0")
    torch.cuda.synchronize()
    released = []
    cb_t = ctypes.CFUNCTYPE(None, ctypes.c_void_p, ctypes.c_void_p)
    cb = cb_t(lambda p, arg: released.append(p))
    dims = (ctypes.c_int64 * 2)(16, 16)
    h = ctypes.c_void_p()
    assert lib.qmm_rt_buffer_view_of_device_memory(client._h, t.data_ptr(), _lib.QMM_F32, dims, 2, client.device_handle(0),
                                                   ctypes.cast(cb, ctypes.c_void_p), None, ctypes.byref(h)) == 0
    view = runtime.Buffer(client, h.value)
    np.testing.assert_array_equal(view.to_numpy(), t.cpu().numpy().reshape(16, 16))
    view.destroy()
    assert released == [t.data_ptr()]
    assert lib.qmm_rt_buffer_create_error(client._h, 3, b"poisoned", _lib.QMM_F32, dims, 2, client.device_handle(0),
                                          ctypes.byref(h)) == 0
    bad = runtime.Buffer(client, h.value)
    with pytest.raises(_lib.QmmError) as e:
        bad.ready_event().await_(1000)
    assert "poisoned" in str(e.value)
    bad.destroy()


def _bf16(a):
    return synthetic.bf16_bits_to_f32(a)


def test_execute_config1_and_config5_fixtures(client):
    exe = client.compile(load("cfg1_w8a32.mlir"))
    assert exe.name == "jit_f" and exe.num_args == 3 and exe.num_outputs == 1
    assert exe.output_info(0) == (_lib.QMM_F32, (32, 1024)) and exe.arg_info(1) == (_lib.QMM_S8, (1024, 1024))
    assert exe.flops == 2.0 * 32 * 1024 * 1024 and len(exe.fingerprint) == 16
    assert '"event":"fused"' in exe.trace()
    c = synthetic.config1()
    args = [client.buffer_from_host(c[k]) for k in ("x", "w", "scale")]
    (out,), done = exe.execute(args)
    y = out.to_numpy()
    done.await_(10000)
    assert done.is_ready()
    assert O.max_rel_err(y, O.w8_perchannel_matmul(c["x"], c["w"], c["scale"])) <= 2e-3
    # wrong shape / wrong count / deleted argument are refused before anything is launched
    with pytest.raises(_lib.QmmError):
        exe.execute(args[:2])
    wrong = client.buffer_from_host(np.zeros((16, 1024), np.float32))
    with pytest.raises(_lib.QmmError):
        exe.execute([wrong, args[1], args[2]])
    args[2].delete()
    with pytest.raises(_lib.QmmError) as e:
        exe.execute(args)
    assert "deleted" in str(e.value)
    # serialise -> load: same fingerprint, same result
    blob = exe.serialize()
    exe2 = client.deserialize_and_load(blob)
    assert exe2.fingerprint == exe.fingerprint
    with pytest.raises(_lib.QmmError):
        client.deserialize_and_load(blob[:-5])
    args[2] = client.buffer_from_host(c["scale"])
    (out2,), _ = exe2.execute(args)
    np.testing.assert_array_equal(out2.to_numpy(), y)

    exe5 = client.compile(load("cfg5_w8a16.mlir"))
    c = synthetic.config5_small(4096, 8192, 1024)
    a5 = [client.buffer_from_host(c["x_bits"], dtype=_lib.QMM_BF16), client.buffer_from_host(c["w"]),
          client.buffer_from_host(c["scale"])]
    (o5,), _ = exe5.execute(a5)
    assert o5.dtype == _lib.QMM_BF16 and o5.shape == (4096, 1024)
    assert O.max_rel_err(_bf16(o5.to_numpy()), O.w8_perchannel_matmul(c["x"], c["w"], c["scale"])) <= 1e-2


def test_execute_config2_and_config3_fixtures(client):
    exe = client.compile(load("cfg2_i8dot_rescale.mlir"))
    assert exe.num_outputs == 2 and exe.output_info(0)[0] == _lib.QMM_S32
    c = synthetic.config2()
    args = [client.buffer_from_host(c[k]) for k in ("a", "b", "row", "col")]
    (acc, out), done = exe.execute(args)
    ref = O.i8_dot_i32(c["a"], c["b"])
    np.testing.assert_array_equal(acc.to_numpy(), ref)
    assert O.max_rel_err(out.to_numpy(), O.i8_dot_rescale(ref, c["row"], c["col"])) <= 2e-3
    only = client.compile(load("cfg2_i8dot_only.mlir"))  # ui8 [256,512] x i8 [512,128]
    assert only.arg_info(0) == (_lib.QMM_U8, (256, 512))
    rng = np.random.default_rng(2)
    a_u = rng.integers(0, 256, size=(256, 512)).astype(np.uint8)
    b_s = rng.integers(-128, 128, size=(512, 128)).astype(np.int8)
    (acc2,), _ = only.execute([client.buffer_from_host(a_u), client.buffer_from_host(b_s)])
    np.testing.assert_array_equal(acc2.to_numpy(), O.i8_dot_i32(a_u, b_s))
    with pytest.raises(_lib.QmmError):  # an argument of the wrong element type is refused
        only.execute([client.buffer_from_host(a_u.view(np.int8)), client.buffer_from_host(b_s)])

    exe3 = client.compile(load("cfg3_w4a16.mlir"))
    c = synthetic.config3(4, 4096, 14336)
    a3 = [client.buffer_from_host(c["x_bits"], dtype=_lib.QMM_BF16), client.buffer_from_host(c["wq"]),
          client.buffer_from_host(c["s_bits"], dtype=_lib.QMM_BF16),
          client.buffer_from_host(c["z_packed"], dtype=_lib.QMM_U4, shape=(32, 14336))]
    ref3 = O.w4a16_matmul(c["x"], c["wq"], c["s"], c["z"])
    for _ in range(2):  # the executable's scratch is reused across launches
        (o3,), _ = exe3.execute(a3)
        assert O.max_rel_err(_bf16(o3.to_numpy()), ref3) <= 1e-2


def test_compile_refuses_what_it_cannot_read(client):
    with pytest.raises(_lib.QmmError) as e:
        client.compile(b"ML\xefR\x01StableHLO_v1.0.0\x00garbage")
    assert e.value.status_name == "QMM_ERR_UNSUPPORTED" and "bytecode" in str(e.value)
    with pytest.raises(_lib.QmmError) as e:
        client.compile("HloModule m", fmt="hlo")
    assert e.value.status_name == "QMM_ERR_UNSUPPORTED"
    with pytest.raises(_lib.QmmError) as e:
        client.compile(load("reject_unfused_add.mlir"))
    assert "stablehlo.tanh" in str(e.value)


def test_execute_a_layer_module_of_four_linears(client):
    # four fused steps in one program: the later ones are launched as independent of the first
    from jax_metallib_b200.stablehlo import weight_only_linears_module

    M = 512
    specs = [(M, 512, 1280, 0), (M, 512, 1024, 0), (M, 512, 3584, 0), (M, 1792, 512, 1)]
    exe = client.compile(weight_only_linears_module(specs))
    rng = np.random.default_rng(12)
    acts = {a: synthetic.to_bf16_bits(rng.standard_normal((M, k)).astype(np.float32)) for _, k, _, a in specs}
    args = [client.buffer_from_host(acts[0], dtype=_lib.QMM_BF16), client.buffer_from_host(acts[1], dtype=_lib.QMM_BF16)]
    host = []
    for _, k, n, a in specs:
        w = rng.integers(-127, 128, size=(k, n), dtype=np.int64).astype(np.int8)
        s = rng.uniform(0.005, 0.02, size=(n,)).astype(np.float32)
        host.append((a, w, s))
        args += [client.buffer_from_host(w), client.buffer_from_host(s)]
    for _ in range(3):  # outputs are freed and their memory reused by the next launch
        outs, done = exe.execute(args)
        got = [o.to_numpy() for o in outs]
        for o in outs:
            o.destroy()
    done.await_(10000)
    for (a, w, s), y in zip(host, got):
        ref = O.w8_perchannel_matmul(_bf16(acts[a]), w, s)
        assert O.max_rel_err(_bf16(y), ref) <= 1e-2
