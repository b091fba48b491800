"""Python face of the runtime layer (``include/qmm_rt.h``): client, buffers, events, executables.

This is what a PJRT plugin's callbacks would call from C (the reference's glue is
src/pjrt_plugin/api/*.cc over core/mps_client.mm, core/mps_buffer.mm,
core/completion_event.h); from Python it gives the same flow without jax:

    client = Client()
    exe = client.compile(stablehlo_text)                 # PJRT_Client_Compile
    args = [client.buffer_from_host(a) for a in arrays]  # PJRT_Client_BufferFromHostBuffer
    outs, done = exe.execute(args)                       # PJRT_LoadedExecutable_Execute
    y = outs[0].to_numpy()                               # PJRT_Buffer_ToHostBuffer + PJRT_Event_Await

Host arrays are NumPy arrays; bf16 travels as ``uint16`` bit patterns (or ``ml_dtypes.bfloat16``),
4-bit tensors as packed ``uint8`` with ``dtype=QMM_U4`` and the logical shape given explicitly.
Everything runs on the GPU through ``libqmm.so``; there is no CPU fallback.
"""

from __future__ import annotations

import ctypes
from ctypes import c_int, c_int64, c_size_t, c_void_p

import numpy as np

from . import _lib

_NP_TO_QMM = {np.dtype(np.float32): _lib.QMM_F32, np.dtype(np.float16): _lib.QMM_F16, np.dtype(np.int8): _lib.QMM_S8,
              np.dtype(np.uint8): _lib.QMM_U8, np.dtype(np.int32): _lib.QMM_S32, np.dtype(np.uint32): _lib.QMM_U32}
_QMM_TO_NP = {_lib.QMM_F32: np.float32, _lib.QMM_F16: np.float16, _lib.QMM_BF16: np.uint16, _lib.QMM_S8: np.int8,
              _lib.QMM_U8: np.uint8, _lib.QMM_S32: np.int32, _lib.QMM_U32: np.uint32, _lib.QMM_U4: np.uint8}


def _qmm_dtype(a: np.ndarray, dtype) -> int:
    if dtype is not None:
        return int(dtype)
    if a.dtype.name == "bfloat16":
        return _lib.QMM_BF16
    try:
        return _NP_TO_QMM[a.dtype]
    except KeyError:
        raise TypeError(f"no device element type for NumPy dtype {a.dtype}") from None


class Event:
    """A completion event (``PJRT_Event``).  Owns its handle."""

    def __init__(self, handle: int | None = None):
        self._lib = _lib.load()
        if handle is None:
            h = c_void_p()
            _lib.check(self._lib.qmm_rt_event_create(ctypes.byref(h)))
            handle = h.value
        self._h = handle
        self._callbacks = []  # keeps ctypes thunks alive

    def is_ready(self) -> bool:
        return bool(self._lib.qmm_rt_event_is_ready(self._h))

    def set(self, status: int = 0, message: str = "") -> None:
        _lib.check(self._lib.qmm_rt_event_set(self._h, status, message.encode()))

    def await_(self, timeout_ms: int = 0) -> None:
        """Bounded wait; raises ``QmmError`` with status ``QMM_ERR_TIMEOUT`` when it runs out."""
        _lib.check(self._lib.qmm_rt_event_await(self._h, timeout_ms))

    def error(self) -> int:
        return self._lib.qmm_rt_event_error(self._h)

    def on_ready(self, fn) -> None:
        cb_t = ctypes.CFUNCTYPE(None, c_int, ctypes.c_char_p, c_void_p)
        thunk = cb_t(lambda status, msg, _arg: fn(status, (msg or b"").decode()))
        self._callbacks.append(thunk)
        _lib.check(self._lib.qmm_rt_event_on_ready(self._h, ctypes.cast(thunk, c_void_p), None))

    def destroy(self) -> None:
        if self._h:
            self._lib.qmm_rt_event_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.destroy()
        except Exception:  # noqa: BLE001
            pass


class Buffer:
    """A device buffer (``PJRT_Buffer``).  Owns its handle."""

    def __init__(self, client: "Client", handle: int):
        self.client = client
        self._lib = client._lib
        self._h = handle

    @property
    def dtype(self) -> int:
        return self._lib.qmm_rt_buffer_dtype(self._h)

    @property
    def shape(self) -> tuple:
        r = self._lib.qmm_rt_buffer_rank(self._h)
        p = ctypes.cast(self._lib.qmm_rt_buffer_dims(self._h), ctypes.POINTER(c_int64))
        return tuple(int(p[i]) for i in range(r))

    @property
    def nbytes(self) -> int:
        return self._lib.qmm_rt_buffer_size_bytes(self._h)

    @property
    def device_pointer(self) -> int:
        return self._lib.qmm_rt_buffer_device_pointer(self._h) or 0

    @property
    def device_id(self) -> int:
        return self._lib.qmm_rt_device_id(self._lib.qmm_rt_buffer_device(self._h))

    def ready_event(self) -> Event:
        h = c_void_p()
        _lib.check(self._lib.qmm_rt_buffer_ready_event(self._h, ctypes.byref(h)))
        return Event(h.value)

    def to_host(self, out: np.ndarray) -> Event:
        """Start the copy into ``out`` (C-contiguous, large enough); the returned event completes with it."""
        if not out.flags.c_contiguous:
            raise ValueError("the destination must be C-contiguous")
        h = c_void_p()
        need = c_size_t()
        _lib.check(self._lib.qmm_rt_buffer_to_host(self._h, out.ctypes.data, out.nbytes, ctypes.byref(need),
                                                   ctypes.byref(h)))
        return Event(h.value)

    def to_numpy(self, timeout_ms: int = 0) -> np.ndarray:
        shape = self.shape
        np_dtype = _QMM_TO_NP[self.dtype]
        if self.dtype == _lib.QMM_U4:
            shape = shape[:-1] + (shape[-1] // 2,)
        out = np.empty(shape, dtype=np_dtype)
        ev = self.to_host(out)
        ev.await_(timeout_ms)
        return out

    def copy_raw_to_host(self, out: np.ndarray, offset: int, size: int) -> Event:
        h = c_void_p()
        _lib.check(self._lib.qmm_rt_buffer_copy_raw_to_host(self._h, out.ctypes.data, offset, size, ctypes.byref(h)))
        return Event(h.value)

    def copy_to_device(self, device_index: int) -> "Buffer":
        dev = self._lib.qmm_rt_client_device(self.client._h, device_index)
        h = c_void_p()
        _lib.check(self._lib.qmm_rt_buffer_copy_to_device(self._h, dev, ctypes.byref(h)))
        return Buffer(self.client, h.value)

    def delete(self) -> None:
        _lib.check(self._lib.qmm_rt_buffer_delete(self._h))

    def is_deleted(self) -> bool:
        return bool(self._lib.qmm_rt_buffer_is_deleted(self._h))

    def destroy(self) -> None:
        if self._h:
            self._lib.qmm_rt_buffer_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            if self.client._h:
                self.destroy()
        except Exception:  # noqa: BLE001
            pass


class Executable:
    """A compiled, loaded program (``PJRT_LoadedExecutable``)."""

    def __init__(self, client: "Client", handle: int):
        self.client = client
        self._lib = client._lib
        self._h = handle

    @property
    def name(self) -> str:
        return self._lib.qmm_rt_executable_name(self._h).decode()

    @property
    def fingerprint(self) -> str:
        return self._lib.qmm_rt_executable_fingerprint(self._h).decode()

    @property
    def num_outputs(self) -> int:
        return self._lib.qmm_rt_executable_num_outputs(self._h)

    @property
    def num_args(self) -> int:
        return self._lib.qmm_rt_executable_num_args(self._h)

    def output_info(self, i: int):
        r = self._lib.qmm_rt_executable_output_rank(self._h, i)
        p = ctypes.cast(self._lib.qmm_rt_executable_output_dims(self._h, i), ctypes.POINTER(c_int64))
        return self._lib.qmm_rt_executable_output_dtype(self._h, i), tuple(int(p[k]) for k in range(r))

    def arg_info(self, i: int):
        r = self._lib.qmm_rt_executable_arg_rank(self._h, i)
        p = ctypes.cast(self._lib.qmm_rt_executable_arg_dims(self._h, i), ctypes.POINTER(c_int64))
        return self._lib.qmm_rt_executable_arg_dtype(self._h, i), tuple(int(p[k]) for k in range(r))

    @property
    def flops(self) -> float:
        return self._lib.qmm_rt_executable_flops(self._h)

    def trace(self) -> str:
        n = self._lib.qmm_rt_executable_trace(self._h, None, 0)
        buf = ctypes.create_string_buffer(n + 1)
        self._lib.qmm_rt_executable_trace(self._h, buf, n + 1)
        return buf.value.decode()

    def serialize(self) -> bytes:
        blob = c_void_p()
        size = c_size_t()
        _lib.check(self._lib.qmm_rt_executable_serialize(self._h, ctypes.byref(blob), ctypes.byref(size)))
        try:
            return ctypes.string_at(blob.value, size.value)
        finally:
            self._lib.qmm_rt_serialized_free(blob)

    def execute(self, args, want_event: bool = True):
        """One device: ``args`` is a list of buffers.  Returns ``(outputs, device_complete_event)``."""
        outs, evs = self.execute_sharded([list(args)], want_events=want_event)
        return outs[0], (evs[0] if evs else None)

    def execute_sharded(self, argument_lists, want_events: bool = True):
        """``argument_lists[d][a]``: one list per device.  Returns ``(outputs[d][o], events[d])``."""
        nd = len(argument_lists)
        na = len(argument_lists[0]) if nd else 0
        nout = self.num_outputs
        ArgList = c_void_p * max(1, na)
        OutList = c_void_p * max(1, nout)
        arg_arrays = [ArgList(*[b._h for b in lst]) for lst in argument_lists]
        out_arrays = [OutList() for _ in range(nd)]
        arg_ptrs = (c_void_p * nd)(*[ctypes.cast(a, c_void_p) for a in arg_arrays])
        out_ptrs = (c_void_p * nd)(*[ctypes.cast(o, c_void_p) for o in out_arrays])
        evs = (c_void_p * nd)() if want_events else None
        _lib.check(self._lib.qmm_rt_executable_execute(self._h, arg_ptrs, nd, na, out_ptrs, evs))
        outs = [[Buffer(self.client, out_arrays[d][o]) for o in range(nout)] for d in range(nd)]
        return outs, ([Event(evs[d]) for d in range(nd)] if want_events else None)

    def destroy(self) -> None:
        if self._h:
            self._lib.qmm_rt_executable_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            if self.client._h:
                self.destroy()
        except Exception:  # noqa: BLE001
            pass


class Client:
    """A runtime client (``PJRT_Client``): owns the devices and memories of the process."""

    def __init__(self):
        self._lib = _lib.load()
        h = c_void_p()
        _lib.check(self._lib.qmm_rt_client_create(ctypes.byref(h)))
        self._h = h.value

    @property
    def platform_name(self) -> str:
        return self._lib.qmm_rt_client_platform_name(self._h).decode()

    @property
    def platform_version(self) -> str:
        return self._lib.qmm_rt_client_platform_version(self._h).decode()

    @property
    def num_devices(self) -> int:
        return self._lib.qmm_rt_client_num_devices(self._h)

    def device_handle(self, index: int) -> int:
        return self._lib.qmm_rt_client_device(self._h, index)

    def memory_handle(self, index: int) -> int:
        return self._lib.qmm_rt_client_memory(self._h, index)

    def device_debug_string(self, index: int) -> str:
        return self._lib.qmm_rt_device_debug_string(self.device_handle(index)).decode()

    def memory_stats(self, index: int):
        used, limit = c_int64(), c_int64()
        _lib.check(self._lib.qmm_rt_device_memory_stats(self.device_handle(index), ctypes.byref(used), ctypes.byref(limit)))
        return used.value, limit.value

    def buffer_from_host(self, array: np.ndarray, device_index: int = 0, dtype=None, shape=None, want_event=False):
        """Upload a NumPy array (any strides).  ``dtype`` overrides the element type (``QMM_BF16``
        for ``uint16`` bit patterns, ``QMM_U4`` for packed nibbles, with ``shape`` the logical shape)."""
        a = np.asarray(array)
        q = _qmm_dtype(a, dtype)
        if q == _lib.QMM_U4:
            if shape is None:
                shape = a.shape[:-1] + (a.shape[-1] * 2,)
            a = np.ascontiguousarray(a)
            strides = None
        else:
            if shape is None:
                shape = a.shape
            strides = (c_int64 * max(1, a.ndim))(*a.strides) if a.ndim else None
        dims = (c_int64 * max(1, len(shape)))(*shape)
        h, ev = c_void_p(), c_void_p()
        _lib.check(self._lib.qmm_rt_buffer_from_host(self._h, a.ctypes.data if a.size else None, q, dims, len(shape),
                                                     strides, self.device_handle(device_index), ctypes.byref(h),
                                                     ctypes.byref(ev)))
        buf = Buffer(self, h.value)
        buf._keepalive = a  # the source must stay valid until the transfer is done
        event = Event(ev.value)
        if want_event:
            return buf, event
        event.destroy()
        return buf

    def view_of_device_memory(self, device_ptr: int, dtype: int, shape, device_index: int = 0, keepalive=None) -> Buffer:
        """Wrap device memory the caller owns (``PJRT_Client_CreateViewOfDeviceBuffer``); no copy.
        ``keepalive`` is held by the returned buffer (e.g. the tensor that owns the memory)."""
        dims = (c_int64 * max(1, len(shape)))(*shape)
        h = c_void_p()
        _lib.check(self._lib.qmm_rt_buffer_view_of_device_memory(self._h, device_ptr, dtype, dims, len(shape),
                                                                 self.device_handle(device_index), None, None,
                                                                 ctypes.byref(h)))
        buf = Buffer(self, h.value)
        buf._keepalive = keepalive
        return buf

    def compile(self, program, fmt: str = "mlir") -> Executable:
        data = program if isinstance(program, (bytes, bytearray)) else program.encode()
        h = c_void_p()
        _lib.check(self._lib.qmm_rt_client_compile(self._h, bytes(data), len(data), fmt.encode(), ctypes.byref(h)))
        return Executable(self, h.value)

    def deserialize_and_load(self, blob: bytes) -> Executable:
        h = c_void_p()
        _lib.check(self._lib.qmm_rt_executable_deserialize_and_load(self._h, blob, len(blob), ctypes.byref(h)))
        return Executable(self, h.value)

    def destroy(self) -> None:
        if self._h:
            self._lib.qmm_rt_client_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.destroy()
        except Exception:  # noqa: BLE001
            pass
