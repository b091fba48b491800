"""ctypes binding of ``libqmm.so``.

The library is the product: if it is missing or fails to load, every operator
raises.  There is no CPU or framework fallback behind these calls.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_int, c_int64, c_size_t, c_uint, c_void_p

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("QMM_LIBRARY_PATH", os.path.join(HERE, "libqmm.so"))

QMM_F32, QMM_F16, QMM_BF16, QMM_S8, QMM_U8, QMM_S32, QMM_U4, QMM_U32 = range(8)
QMM_MXFP4, QMM_MXFP8, QMM_NVFP4 = range(3)
QMM_W4_STATIC_WEIGHTS = 1
QMM_ATTN_STATIC_CACHE = 1
MX_MODE_IDS = {"mxfp4": QMM_MXFP4, "mxfp8": QMM_MXFP8, "nvfp4": QMM_NVFP4}

# name -> (restype, argtypes); mirrors include/qmm.h
SIGNATURES = {
    "qmm_version": (c_char_p, []),
    "qmm_status_name": (c_char_p, [c_int]),
    "qmm_last_error": (c_size_t, [c_char_p, c_size_t]),
    "qmm_device_status": (c_int, []),
    "qmm_selftest_host": (c_int, []),
    "qmm_clear_device_status": (None, []),
    "qmm_w8a32_perchannel": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p]),
    "qmm_w8a16_perchannel": (
        c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_void_p]),
    "qmm_w8a16_perchannel_ex": (
        c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_void_p, c_void_p]),
    "qmm_wait_signals": (c_int, [c_void_p, c_int, ctypes.c_uint32, ctypes.c_uint64, c_void_p]),
    "qmm_multicast_copy": (c_int, [c_void_p, c_void_p, ctypes.c_size_t, c_void_p, c_void_p, c_int, c_void_p]),
    "qmm_peer_copy": (c_int, [c_void_p, c_void_p, c_void_p, c_int, ctypes.c_size_t, c_void_p, c_void_p, c_int, c_void_p]),
    "qmm_i8i8_i32": (
        c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int, c_int,
                c_void_p]),
    "qmm_w4a16_g128_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int64]),
    "qmm_w4a16_g128": (
        c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int64, c_int64, c_int64, c_int64, c_void_p,
                c_size_t, c_uint, c_void_p]),
    "qmm_w4a16_g128_static_scratch": (
        c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int64, c_int64, c_int64, c_int64,
                c_void_p]),
    "qmm_affine_matmul": (
        c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int, c_int64, c_int,
                c_void_p]),
    "qmm_set_cta_limit": (c_int, [c_int]),
    "qmm_take_rows_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, ctypes.c_uint16, c_void_p]),
    "qmm_add_rmsnorm_bf16": (
        c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, ctypes.c_float, c_void_p]),
    "qmm_rope_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, ctypes.c_float, c_int64,
                              c_int64, c_void_p]),
    "qmm_silu_mul_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p]),
    "qmm_attention_decode_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int64, c_int64]),
    "qmm_attention_decode_bf16": (
        c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64,
                ctypes.c_float, c_int64, c_int64, c_void_p, c_size_t, ctypes.c_uint, c_void_p]),
    "qmm_bf16_matmul_small_m": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p]),
    "qmm_plan_compile": (c_int, [c_char_p, c_size_t, ctypes.POINTER(c_void_p)]),
    "qmm_plan_destroy": (None, [c_void_p]),
    "qmm_plan_num_steps": (c_int, [c_void_p]),
    "qmm_plan_num_fused_steps": (c_int, [c_void_p]),
    "qmm_plan_num_args": (c_int, [c_void_p]),
    "qmm_plan_num_results": (c_int, [c_void_p]),
    "qmm_plan_workspace_bytes": (c_size_t, [c_void_p]),
    "qmm_plan_arg_info": (c_int, [c_void_p, c_int, ctypes.POINTER(c_int), ctypes.POINTER(c_int64), ctypes.POINTER(c_int)]),
    "qmm_plan_result_info": (c_int, [c_void_p, c_int, ctypes.POINTER(c_int), ctypes.POINTER(c_int64),
                                     ctypes.POINTER(c_int)]),
    "qmm_plan_name": (c_char_p, [c_void_p]),
    "qmm_plan_num_replicas": (c_int, [c_void_p]),
    "qmm_plan_num_partitions": (c_int, [c_void_p]),
    "qmm_plan_flops": (ctypes.c_double, [c_void_p]),
    "qmm_plan_trace": (c_size_t, [c_void_p, c_char_p, c_size_t]),
    "qmm_plan_execute": (
        c_int, [c_void_p, ctypes.POINTER(c_void_p), c_int, ctypes.POINTER(c_void_p), c_int, c_void_p, c_size_t,
                c_void_p]),
    "qmm_mx_matmul": (
        c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int, c_int, c_void_p]),
}


# name -> (restype, argtypes); mirrors include/qmm_rt.h
RT_SIGNATURES = {
    "qmm_rt_status_to_pjrt_code": (c_int, [c_int]),
    "qmm_rt_client_create": (c_int, [c_void_p]),
    "qmm_rt_client_destroy": (c_int, [c_void_p]),
    "qmm_rt_default_client": (c_void_p, []),
    "qmm_rt_client_platform_name": (c_char_p, [c_void_p]),
    "qmm_rt_client_platform_version": (c_char_p, [c_void_p]),
    "qmm_rt_client_process_index": (c_int, [c_void_p]),
    "qmm_rt_client_num_devices": (c_int, [c_void_p]),
    "qmm_rt_client_device": (c_void_p, [c_void_p, c_int]),
    "qmm_rt_client_lookup_device": (c_int, [c_void_p, c_int, c_void_p]),
    "qmm_rt_client_num_memories": (c_int, [c_void_p]),
    "qmm_rt_client_memory": (c_void_p, [c_void_p, c_int]),
    "qmm_rt_client_default_device_assignment": (c_int, [c_void_p, c_int, c_int, c_void_p, c_size_t]),
    "qmm_rt_device_id": (c_int, [c_void_p]),
    "qmm_rt_device_process_index": (c_int, [c_void_p]),
    "qmm_rt_device_local_hardware_id": (c_int, [c_void_p]),
    "qmm_rt_device_is_addressable": (c_int, [c_void_p]),
    "qmm_rt_device_kind": (c_char_p, [c_void_p]),
    "qmm_rt_device_debug_string": (c_char_p, [c_void_p]),
    "qmm_rt_device_to_string": (c_char_p, [c_void_p]),
    "qmm_rt_device_default_memory": (c_void_p, [c_void_p]),
    "qmm_rt_device_memory_stats": (c_int, [c_void_p, c_void_p, c_void_p]),
    "qmm_rt_memory_id": (c_int, [c_void_p]),
    "qmm_rt_memory_kind": (c_char_p, [c_void_p]),
    "qmm_rt_memory_kind_id": (c_int, [c_void_p]),
    "qmm_rt_memory_debug_string": (c_char_p, [c_void_p]),
    "qmm_rt_memory_to_string": (c_char_p, [c_void_p]),
    "qmm_rt_memory_device": (c_void_p, [c_void_p]),
    "qmm_rt_memory_set_user_data": (c_int, [c_void_p, ctypes.c_uint64, c_void_p, c_void_p]),
    "qmm_rt_memory_get_user_data": (c_void_p, [c_void_p, ctypes.c_uint64]),
    "qmm_rt_event_create": (c_int, [c_void_p]),
    "qmm_rt_event_set": (c_int, [c_void_p, c_int, c_char_p]),
    "qmm_rt_event_destroy": (c_int, [c_void_p]),
    "qmm_rt_event_is_ready": (c_int, [c_void_p]),
    "qmm_rt_event_error": (c_int, [c_void_p]),
    "qmm_rt_event_await": (c_int, [c_void_p, c_int]),
    "qmm_rt_event_on_ready": (c_int, [c_void_p, c_void_p, c_void_p]),
    "qmm_rt_buffer_from_host": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "qmm_rt_buffer_create_uninitialized": (c_int, [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p]),
    "qmm_rt_buffer_view_of_device_memory": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "qmm_rt_buffer_create_error": (c_int, [c_void_p, c_int, c_char_p, c_int, c_void_p, c_int, c_void_p, c_void_p]),
    "qmm_rt_buffer_dtype": (c_int, [c_void_p]),
    "qmm_rt_buffer_rank": (c_int, [c_void_p]),
    "qmm_rt_buffer_dims": (c_void_p, [c_void_p]),
    "qmm_rt_buffer_size_bytes": (c_size_t, [c_void_p]),
    "qmm_rt_buffer_device": (c_void_p, [c_void_p]),
    "qmm_rt_buffer_memory": (c_void_p, [c_void_p]),
    "qmm_rt_buffer_is_on_cpu": (c_int, [c_void_p]),
    "qmm_rt_buffer_delete": (c_int, [c_void_p]),
    "qmm_rt_buffer_is_deleted": (c_int, [c_void_p]),
    "qmm_rt_buffer_destroy": (c_int, [c_void_p]),
    "qmm_rt_buffer_ready_event": (c_int, [c_void_p, c_void_p]),
    "qmm_rt_buffer_to_host": (c_int, [c_void_p, c_void_p, c_size_t, c_void_p, c_void_p]),
    "qmm_rt_buffer_copy_raw_to_host": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_void_p]),
    "qmm_rt_buffer_copy_to_device": (c_int, [c_void_p, c_void_p, c_void_p]),
    "qmm_rt_buffer_device_pointer": (c_void_p, [c_void_p]),
    "qmm_rt_buffer_increase_external_refs": (c_int, [c_void_p]),
    "qmm_rt_buffer_decrease_external_refs": (c_int, [c_void_p]),
    "qmm_rt_client_compile": (c_int, [c_void_p, c_void_p, c_size_t, c_char_p, c_void_p]),
    "qmm_rt_executable_destroy": (c_int, [c_void_p]),
    "qmm_rt_executable_delete": (c_int, [c_void_p]),
    "qmm_rt_executable_is_deleted": (c_int, [c_void_p]),
    "qmm_rt_executable_name": (c_char_p, [c_void_p]),
    "qmm_rt_executable_num_replicas": (c_int, [c_void_p]),
    "qmm_rt_executable_num_partitions": (c_int, [c_void_p]),
    "qmm_rt_executable_num_outputs": (c_int, [c_void_p]),
    "qmm_rt_executable_num_args": (c_int, [c_void_p]),
    "qmm_rt_executable_code_size": (c_int64, [c_void_p]),
    "qmm_rt_executable_fingerprint": (c_char_p, [c_void_p]),
    "qmm_rt_executable_program": (c_char_p, [c_void_p, c_void_p]),
    "qmm_rt_executable_output_dtype": (c_int, [c_void_p, c_int]),
    "qmm_rt_executable_output_rank": (c_int, [c_void_p, c_int]),
    "qmm_rt_executable_output_dims": (c_void_p, [c_void_p, c_int]),
    "qmm_rt_executable_output_memory_kind": (c_char_p, [c_void_p, c_int]),
    "qmm_rt_executable_arg_dtype": (c_int, [c_void_p, c_int]),
    "qmm_rt_executable_arg_rank": (c_int, [c_void_p, c_int]),
    "qmm_rt_executable_arg_dims": (c_void_p, [c_void_p, c_int]),
    "qmm_rt_executable_flops": (ctypes.c_double, [c_void_p]),
    "qmm_rt_executable_trace": (c_size_t, [c_void_p, c_void_p, c_size_t]),
    "qmm_rt_executable_serialize": (c_int, [c_void_p, c_void_p, c_void_p]),
    "qmm_rt_serialized_free": (None, [c_void_p]),
    "qmm_rt_executable_deserialize_and_load": (c_int, [c_void_p, c_void_p, c_size_t, c_void_p]),
    "qmm_rt_executable_client": (c_void_p, [c_void_p]),
    "qmm_rt_executable_execute": (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p]),
}
SIGNATURES.update(RT_SIGNATURES)

QMM_GEMM_INDEPENDENT = 1
QMM_GEMM_STORE_MULTIMEM = 2


class GemmExt(ctypes.Structure):
    """``qmm_gemm_ext`` of include/qmm.h."""

    _fields_ = [("struct_size", c_size_t), ("flags", ctypes.c_uint32), ("done_signal", c_void_p),
                ("arrive_counter", c_void_p)]

    def __init__(self, flags=0, done_signal=None, arrive_counter=None):
        super().__init__(ctypes.sizeof(GemmExt), flags, done_signal, arrive_counter)


class QmmError(RuntimeError):
    def __init__(self, status: int, name: str, message: str):
        super().__init__(f"{name} ({status}): {message}")
        self.status = status
        self.status_name = name


_lib = None


def load():
    """Load the library once; raise loudly if the CUDA extension is absent."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m jax_metallib_b200.build` "
            "(there is no CPU fallback for the quantized-matmul path)"
        )
    lib = ctypes.CDLL(LIB_PATH, mode=ctypes.RTLD_LOCAL)
    for name, (res, args) in SIGNATURES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as e:  # pragma: no cover
            raise ImportError(f"{LIB_PATH} does not export {name}") from e
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def last_error() -> str:
    lib = load()
    buf = ctypes.create_string_buffer(512)
    lib.qmm_last_error(buf, 512)
    return buf.value.decode("utf-8", "replace")


def check(status: int) -> None:
    if status != 0:
        lib = load()
        raise QmmError(status, lib.qmm_status_name(status).decode(), last_error())
