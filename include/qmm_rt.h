/*
 * qmm_rt.h — the runtime objects of libqmm.so: client, devices, memories,
 * buffers, events and executables, as a C ABI.
 *
 * This is the layer a PJRT plugin table sits on.  The reference fills the
 * PJRT_Api table in src/pjrt_plugin/api/pjrt_api.cc:160-322 with callbacks that
 * unwrap handle structs and call into its client / buffer / executable classes
 * (src/pjrt_plugin/core/mps_client.mm, mps_buffer.mm, mps_executable.mm,
 * completion_event.h).  The PJRT C API header is not part of this source tree,
 * so the table itself is only built where jaxlib's headers exist; everything
 * the callbacks need is exported here, one function per callback the reference
 * fills, each naming that callback.  A table entry is then a few lines: unwrap
 * the args struct, call the function below, turn a non-zero status into a
 * PJRT_Error with qmm_last_error() and qmm_rt_status_to_pjrt_code().
 *
 * Conventions.  Every function returns 0 (QMM_OK) or a qmm_status code; the
 * message of the calling thread's last failure is available from
 * qmm_last_error().  Nothing throws across this boundary.  Ownership follows
 * PJRT: a client owns its devices and memories (their handles stay valid until
 * qmm_rt_client_destroy); the caller owns buffers, events and executables and
 * destroys them through the functions below; strings and arrays returned by a
 * getter are borrowed from the handle they were asked of.  Functions may be
 * called from any thread.  Device work is asynchronous: outputs are returned at
 * once with a producer event; host reads wait for it; waits a caller makes are
 * bounded.
 */
#ifndef QMM_RT_H_
#define QMM_RT_H_

#include "qmm.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct qmm_rt_client qmm_rt_client;
typedef struct qmm_rt_device qmm_rt_device;
typedef struct qmm_rt_memory qmm_rt_memory;
typedef struct qmm_rt_buffer qmm_rt_buffer;
typedef struct qmm_rt_event qmm_rt_event;
typedef struct qmm_rt_executable qmm_rt_executable;

/* The status codes of this library as the PJRT / absl error codes a plugin
 * reports them with (INVALID_ARGUMENT 3, DEADLINE_EXCEEDED 4, UNIMPLEMENTED 12,
 * INTERNAL 13, ...), as the reference does in MakeError
 * (src/pjrt_plugin/api/pjrt_memory.cc:22-57). */
QMM_API int qmm_rt_status_to_pjrt_code(int status);

/* ---------------------------------------------------------------- client --
 * PJRT_Client_Create / _Destroy (src/pjrt_plugin/api/pjrt_client.cc:22-80):
 * every create returns a distinct client with its own device and memory
 * handles (tests/test_pjrt_client_ownership.py:118-158).  A client covers
 * every CUDA device visible to the process; each device gets its own streams.
 * qmm_rt_default_client() is the lazily created client that callbacks fall
 * back to when handed a null client (api/pjrt_api.cc:21-31); it is never
 * destroyed. */
QMM_API int qmm_rt_client_create(qmm_rt_client** client);
QMM_API int qmm_rt_client_destroy(qmm_rt_client* client);
QMM_API qmm_rt_client* qmm_rt_default_client(void);
/* PJRT_Client_PlatformName / _PlatformVersion / _ProcessIndex */
QMM_API const char* qmm_rt_client_platform_name(const qmm_rt_client* client);
QMM_API const char* qmm_rt_client_platform_version(const qmm_rt_client* client);
QMM_API int qmm_rt_client_process_index(const qmm_rt_client* client);
/* PJRT_Client_Devices / _AddressableDevices (the same list: one process) */
QMM_API int qmm_rt_client_num_devices(const qmm_rt_client* client);
QMM_API qmm_rt_device* qmm_rt_client_device(const qmm_rt_client* client, int index);
/* PJRT_Client_LookupDevice / _LookupAddressableDevice: by global id / local hardware id */
QMM_API int qmm_rt_client_lookup_device(const qmm_rt_client* client, int id, qmm_rt_device** device);
/* PJRT_Client_AddressableMemories */
QMM_API int qmm_rt_client_num_memories(const qmm_rt_client* client);
QMM_API qmm_rt_memory* qmm_rt_client_memory(const qmm_rt_client* client, int index);
/* PJRT_Client_DefaultDeviceAssignment: assignment[r * num_partitions + p] = device id */
QMM_API int qmm_rt_client_default_device_assignment(const qmm_rt_client* client, int num_replicas,
                                                    int num_partitions, int* assignment, size_t capacity);

/* ---------------------------------------------------------------- device --
 * PJRT_Device_* and PJRT_DeviceDescription_* (src/pjrt_plugin/api/pjrt_device.cc). */
QMM_API int qmm_rt_device_id(const qmm_rt_device* device);
QMM_API int qmm_rt_device_process_index(const qmm_rt_device* device);
QMM_API int qmm_rt_device_local_hardware_id(const qmm_rt_device* device);
QMM_API int qmm_rt_device_is_addressable(const qmm_rt_device* device);
QMM_API const char* qmm_rt_device_kind(const qmm_rt_device* device);
QMM_API const char* qmm_rt_device_debug_string(const qmm_rt_device* device);
QMM_API const char* qmm_rt_device_to_string(const qmm_rt_device* device);
QMM_API qmm_rt_memory* qmm_rt_device_default_memory(const qmm_rt_device* device);
/* PJRT_Device_MemoryStats: bytes this client holds on the device and the device's capacity */
QMM_API int qmm_rt_device_memory_stats(const qmm_rt_device* device, int64_t* bytes_in_use,
                                       int64_t* bytes_limit);

/* ---------------------------------------------------------------- memory --
 * PJRT_Memory_* (src/pjrt_plugin/api/pjrt_memory.cc:60-200).  One memory space
 * ("device", HBM) per device.  Memory handles carry keyed user data with
 * destructors, isolated per client and destroyed exactly once with the owner
 * (api/pjrt_memory.cc:115-152, tests/test_pjrt_client_ownership.py:118-158);
 * a destructor runs outside the handle's lock. */
QMM_API int qmm_rt_memory_id(const qmm_rt_memory* memory);
QMM_API const char* qmm_rt_memory_kind(const qmm_rt_memory* memory);
QMM_API int qmm_rt_memory_kind_id(const qmm_rt_memory* memory);
QMM_API const char* qmm_rt_memory_debug_string(const qmm_rt_memory* memory);
QMM_API const char* qmm_rt_memory_to_string(const qmm_rt_memory* memory);
QMM_API qmm_rt_device* qmm_rt_memory_device(const qmm_rt_memory* memory);
typedef void (*qmm_rt_user_data_deleter)(void* data);
QMM_API int qmm_rt_memory_set_user_data(qmm_rt_memory* memory, uint64_t key, void* data,
                                        qmm_rt_user_data_deleter deleter);
QMM_API void* qmm_rt_memory_get_user_data(qmm_rt_memory* memory, uint64_t key);

/* ----------------------------------------------------------------- event --
 * PJRT_Event_* (src/pjrt_plugin/api/pjrt_event.cc:20-98) over a completion
 * state like src/pjrt_plugin/core/completion_event.h:32-213: ready flag, error
 * text, callbacks that run once (on the completing thread, or at once when the
 * event is ready already).  qmm_rt_event_await is the caller-facing wait: it
 * gives up after the timeout (QMM_RT_COMPLETION_TIMEOUT_MS, default 30000,
 * read per wait; or timeout_ms when > 0), returns QMM_ERR_TIMEOUT (PJRT
 * DEADLINE_EXCEEDED) and leaves the event pending: the device work goes on. */
QMM_API int qmm_rt_event_create(qmm_rt_event** event);                         /* PJRT_Event_Create */
QMM_API int qmm_rt_event_set(qmm_rt_event* event, int status, const char* message); /* PJRT_Event_Set */
QMM_API int qmm_rt_event_destroy(qmm_rt_event* event);                         /* PJRT_Event_Destroy */
QMM_API int qmm_rt_event_is_ready(const qmm_rt_event* event);                  /* PJRT_Event_IsReady */
QMM_API int qmm_rt_event_error(const qmm_rt_event* event);                     /* PJRT_Event_Error: status it completed with */
QMM_API int qmm_rt_event_await(qmm_rt_event* event, int timeout_ms);           /* PJRT_Event_Await */
typedef void (*qmm_rt_event_callback)(int status, const char* message, void* user_arg);
QMM_API int qmm_rt_event_on_ready(qmm_rt_event* event, qmm_rt_event_callback callback, void* user_arg);

/* ---------------------------------------------------------------- buffer --
 * PJRT_Client_BufferFromHostBuffer (src/pjrt_plugin/api/pjrt_client.cc:254-293,
 * src/pjrt_plugin/core/mps_client.mm:114-291): dims in elements, byte_strides
 * NULL for a dense row-major source; a strided source is gathered into a dense
 * buffer; a zero-element shape gets a placeholder allocation and copies
 * nothing.  Device memory comes from the device's stream-ordered pool.  The
 * host data may be reused once *done_with_host (optional) is ready.  QMM_U4
 * buffers hold two elements per byte (low nibble first): the innermost
 * dimension must be even and the host source dense. */
QMM_API int qmm_rt_buffer_from_host(qmm_rt_client* client, const void* data, int dtype,
                                    const int64_t* dims, int rank, const int64_t* byte_strides,
                                    qmm_rt_device* device, qmm_rt_buffer** buffer,
                                    qmm_rt_event** done_with_host);
/* PJRT_Client_CreateUninitializedBuffer */
QMM_API int qmm_rt_buffer_create_uninitialized(qmm_rt_client* client, int dtype, const int64_t* dims,
                                               int rank, qmm_rt_device* device, qmm_rt_buffer** buffer);
/* PJRT_Client_CreateViewOfDeviceBuffer (api/pjrt_client.cc:308-318): wraps device
 * memory the caller owns; on_delete(device_ptr, user_arg) runs when the buffer
 * lets go of it. */
typedef void (*qmm_rt_on_delete)(void* device_ptr, void* user_arg);
QMM_API int qmm_rt_buffer_view_of_device_memory(qmm_rt_client* client, void* device_ptr, int dtype,
                                                const int64_t* dims, int rank, qmm_rt_device* device,
                                                qmm_rt_on_delete on_delete, void* user_arg,
                                                qmm_rt_buffer** buffer);
/* PJRT_Client_CreateErrorBuffer: a buffer whose ready event carries the error */
QMM_API int qmm_rt_buffer_create_error(qmm_rt_client* client, int status, const char* message, int dtype,
                                       const int64_t* dims, int rank, qmm_rt_device* device,
                                       qmm_rt_buffer** buffer);
/* PJRT_Buffer_ElementType / _Dimensions / _UnpaddedDimensions / _OnDeviceSizeInBytes /
 * _Device / _Memory / _IsOnCpu */
QMM_API int qmm_rt_buffer_dtype(const qmm_rt_buffer* buffer);
QMM_API int qmm_rt_buffer_rank(const qmm_rt_buffer* buffer);
QMM_API const int64_t* qmm_rt_buffer_dims(const qmm_rt_buffer* buffer);
QMM_API size_t qmm_rt_buffer_size_bytes(const qmm_rt_buffer* buffer);
QMM_API qmm_rt_device* qmm_rt_buffer_device(const qmm_rt_buffer* buffer);
QMM_API qmm_rt_memory* qmm_rt_buffer_memory(const qmm_rt_buffer* buffer);
QMM_API int qmm_rt_buffer_is_on_cpu(const qmm_rt_buffer* buffer);
/* PJRT_Buffer_Delete / _IsDeleted / _Destroy (src/pjrt_plugin/core/mps_buffer.mm:656-669):
 * the storage is released behind the buffer's producer, as a stream-ordered
 * free, so the device is never still writing what is handed back and the host
 * does not block. */
QMM_API int qmm_rt_buffer_delete(qmm_rt_buffer* buffer);
QMM_API int qmm_rt_buffer_is_deleted(const qmm_rt_buffer* buffer);
QMM_API int qmm_rt_buffer_destroy(qmm_rt_buffer* buffer);
/* PJRT_Buffer_ReadyEvent: a new event (caller destroys it) that completes when the
 * buffer's contents are defined. */
QMM_API int qmm_rt_buffer_ready_event(qmm_rt_buffer* buffer, qmm_rt_event** event);
/* PJRT_Buffer_ToHostBuffer (src/pjrt_plugin/api/pjrt_buffer.cc:217-234): dst == NULL only
 * asks for the size.  The copy waits for the producer; a failure is reported
 * through the returned event, not through the return value. */
QMM_API int qmm_rt_buffer_to_host(qmm_rt_buffer* buffer, void* dst, size_t dst_size, size_t* needed,
                                  qmm_rt_event** event);
/* PJRT_Buffer_CopyRawToHost / _CopyRawToHostFuture (src/pjrt_plugin/core/mps_buffer.mm:393-423):
 * byte range [offset, offset + size), range-checked. */
QMM_API int qmm_rt_buffer_copy_raw_to_host(qmm_rt_buffer* buffer, void* dst, int64_t offset, int64_t size,
                                           qmm_rt_event** event);
/* PJRT_Buffer_CopyToDevice / _CopyToMemory */
QMM_API int qmm_rt_buffer_copy_to_device(qmm_rt_buffer* buffer, qmm_rt_device* device, qmm_rt_buffer** copy);
/* PJRT_Buffer_UnsafePointer / _OpaqueDeviceMemoryDataPointer */
QMM_API void* qmm_rt_buffer_device_pointer(const qmm_rt_buffer* buffer);
/* PJRT_Buffer_IncreaseExternalReferenceCount / _DecreaseExternalReferenceCount: while the count
 * is positive, delete and destroy keep the storage alive. */
QMM_API int qmm_rt_buffer_increase_external_refs(qmm_rt_buffer* buffer);
QMM_API int qmm_rt_buffer_decrease_external_refs(qmm_rt_buffer* buffer);

/* ------------------------------------------------------------ executable --
 * PJRT_Client_Compile (src/pjrt_plugin/api/pjrt_client.cc:172-250): format is
 * "mlir" (StableHLO text; MLIR bytecode is recognised by its magic and refused
 * with a message that says how to get text) — "hlo" / "hlo_with_config" are
 * refused as in the reference's unsupported paths.  Compilation is
 * qmm_plan_compile: the dequantisation chains of the program become single
 * kernel launches; an op outside the supported set is an error naming it. */
QMM_API int qmm_rt_client_compile(qmm_rt_client* client, const char* program, size_t size,
                                  const char* format, qmm_rt_executable** executable);
/* PJRT_Executable_Destroy / PJRT_LoadedExecutable_Destroy / _Delete / _IsDeleted */
QMM_API int qmm_rt_executable_destroy(qmm_rt_executable* executable);
QMM_API int qmm_rt_executable_delete(qmm_rt_executable* executable);
QMM_API int qmm_rt_executable_is_deleted(const qmm_rt_executable* executable);
/* PJRT_Executable_Name / _NumReplicas / _NumPartitions / _NumOutputs /
 * _SizeOfGeneratedCodeInBytes / _Fingerprint / _OptimizedProgram (the program text) */
QMM_API const char* qmm_rt_executable_name(const qmm_rt_executable* executable);
QMM_API int qmm_rt_executable_num_replicas(const qmm_rt_executable* executable);
QMM_API int qmm_rt_executable_num_partitions(const qmm_rt_executable* executable);
QMM_API int qmm_rt_executable_num_outputs(const qmm_rt_executable* executable);
QMM_API int qmm_rt_executable_num_args(const qmm_rt_executable* executable);
QMM_API int64_t qmm_rt_executable_code_size(const qmm_rt_executable* executable);
QMM_API const char* qmm_rt_executable_fingerprint(const qmm_rt_executable* executable);
QMM_API const char* qmm_rt_executable_program(const qmm_rt_executable* executable, size_t* size);
/* PJRT_Executable_OutputElementTypes / _OutputDimensions / _OutputMemoryKinds
 * (and the same for parameters: _ParameterMemoryKinds) */
QMM_API int qmm_rt_executable_output_dtype(const qmm_rt_executable* executable, int index);
QMM_API int qmm_rt_executable_output_rank(const qmm_rt_executable* executable, int index);
QMM_API const int64_t* qmm_rt_executable_output_dims(const qmm_rt_executable* executable, int index);
QMM_API const char* qmm_rt_executable_output_memory_kind(const qmm_rt_executable* executable, int index);
QMM_API int qmm_rt_executable_arg_dtype(const qmm_rt_executable* executable, int index);
QMM_API int qmm_rt_executable_arg_rank(const qmm_rt_executable* executable, int index);
QMM_API const int64_t* qmm_rt_executable_arg_dims(const qmm_rt_executable* executable, int index);
/* PJRT_Executable_GetCostAnalysis: floating-point / integer operations of the fused matmuls */
QMM_API double qmm_rt_executable_flops(const qmm_rt_executable* executable);
/* The plan trace (one QMM_PLAN_JSON line per decision), see qmm_plan_trace. */
QMM_API size_t qmm_rt_executable_trace(const qmm_rt_executable* executable, char* buf, size_t cap);
/* PJRT_Executable_Serialize / PJRT_Executable_DeserializeAndLoad
 * (src/pjrt_plugin/api/pjrt_executable.cc:161-187,303-340): the blob is a
 * versioned header, the fingerprint and the program text; loading re-plans it
 * and checks the fingerprint.  qmm_rt_serialized_free releases a blob. */
QMM_API int qmm_rt_executable_serialize(const qmm_rt_executable* executable, char** blob, size_t* size);
QMM_API void qmm_rt_serialized_free(char* blob);
QMM_API int qmm_rt_executable_deserialize_and_load(qmm_rt_client* client, const char* blob, size_t size,
                                                   qmm_rt_executable** executable);
/* PJRT_LoadedExecutable_AddressableDevices / _GetDeviceAssignment: the executable runs on any
 * device of its client; replica r of an execute call runs on argument list r's device. */
QMM_API qmm_rt_client* qmm_rt_executable_client(const qmm_rt_executable* executable);
/* PJRT_LoadedExecutable_Execute (src/pjrt_plugin/api/pjrt_executable.cc:253-298):
 * argument_lists[d][a] for d < num_devices, a < num_args; output_lists[d][o]
 * receives new buffers (caller destroys them) which are returned at once, each
 * with the launch's completion as its producer; device_complete_events (may be
 * NULL) receives one event per device.  The device of list d is the device of
 * its first argument (all arguments of a list must live on one device). */
QMM_API int qmm_rt_executable_execute(qmm_rt_executable* executable, qmm_rt_buffer* const* const* argument_lists,
                                      int num_devices, int num_args, qmm_rt_buffer** const* output_lists,
                                      qmm_rt_event** device_complete_events);

#ifdef __cplusplus
}
#endif
#endif /* QMM_RT_H_ */
