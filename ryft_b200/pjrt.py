"""Host-side mirror of the ryft-pjrt surface over the PJRT C API, via ctypes.

The reference's users write (crates/ryft-pjrt/src/plugins.rs:120-141, clients.rs, programs.rs, buffers.rs, events.rs):

    plugin = load_plugin(path)                  # dlopen + GetPjrtApi + PJRT_Plugin_Initialize
    client = plugin.client(options)             # PJRT_Client_Create
    exe = client.compile(Program.mlir(text), CompilationOptions(...))
    buf = client.buffer(bytes, BufferType.F32, dims, device=device)
    outs = exe.execute([ExecutionDeviceInputs([buf, ...])])   # one entry per addressable device
    outs[0].done.await_(); host = outs[0].outputs[0].copy_to_host().await_()

This module offers the same names and argument meaning in Python and issues exactly the C calls ryft-pjrt issues
(same argument structs, `struct_size` set, two-call protocols honoured), so a parity test reads like the reference's
own tests (e.g. crates/ryft-pjrt/src/programs.rs:2781-2829).  No Rust toolchain is needed to exercise the plugin.
"""
from __future__ import annotations

import ctypes as C
import enum
import os
import re
import threading
from dataclasses import dataclass, field
from pathlib import Path
from typing import Callable, Dict, List, Optional, Sequence

import numpy as np

_REPO = Path(__file__).resolve().parent.parent
_HEADER = _REPO / "include" / "b2x_pjrt_c_api.h"
_DEFAULT_PLUGIN = Path(__file__).resolve().parent / "lib" / "libpjrt-plugin-cuda-13.so"


class PjrtError(RuntimeError):
    """A PJRT_Error returned by the plugin (code = absl status code, crates/ryft-pjrt/src/errors.rs:440-457)."""

    CODES = {0: "OK", 1: "CANCELLED", 2: "UNKNOWN", 3: "INVALID_ARGUMENT", 4: "DEADLINE_EXCEEDED", 5: "NOT_FOUND",
             6: "ALREADY_EXISTS", 7: "PERMISSION_DENIED", 8: "RESOURCE_EXHAUSTED", 9: "FAILED_PRECONDITION", 10: "ABORTED",
             11: "OUT_OF_RANGE", 12: "UNIMPLEMENTED", 13: "INTERNAL", 14: "UNAVAILABLE", 15: "DATA_LOSS", 16: "UNAUTHENTICATED"}

    def __init__(self, code: int, message: str):
        super().__init__(f"{self.CODES.get(code, code)}: {message}")
        self.code = code
        self.code_name = self.CODES.get(code, str(code))
        self.message = message


class BufferType(enum.IntEnum):
    """PJRT_Buffer_Type (crates/ryft-pjrt/src/buffers.rs:2568-2600)."""
    INVALID = 0; PRED = 1; S8 = 2; S16 = 3; S32 = 4; S64 = 5; U8 = 6; U16 = 7; U32 = 8; U64 = 9
    F16 = 10; F32 = 11; F64 = 12; BF16 = 13


def _np_to_buffer_type(dt) -> BufferType:
    name = np.dtype(dt).name
    table = {"bool": BufferType.PRED, "int8": BufferType.S8, "int16": BufferType.S16, "int32": BufferType.S32,
             "int64": BufferType.S64, "uint8": BufferType.U8, "uint16": BufferType.U16, "uint32": BufferType.U32,
             "uint64": BufferType.U64, "float16": BufferType.F16, "float32": BufferType.F32, "float64": BufferType.F64,
             "bfloat16": BufferType.BF16}
    return table[name]


def buffer_type_to_np(t: BufferType):
    if t == BufferType.BF16:
        import ml_dtypes
        return np.dtype(ml_dtypes.bfloat16)
    table = {BufferType.PRED: np.bool_, BufferType.S8: np.int8, BufferType.S16: np.int16, BufferType.S32: np.int32,
             BufferType.S64: np.int64, BufferType.U8: np.uint8, BufferType.U16: np.uint16, BufferType.U32: np.uint32,
             BufferType.U64: np.uint64, BufferType.F16: np.float16, BufferType.F32: np.float32, BufferType.F64: np.float64}
    return np.dtype(table[t])


# ---- C layouts ------------------------------------------------------------------------------------------------------
_vp, _sz, _i, _i64, _b, _cp, _u = C.c_void_p, C.c_size_t, C.c_int, C.c_int64, C.c_bool, C.c_char_p, C.c_uint


def _args(name: str, fields):
    return type(name, (C.Structure,), {"_fields_": [("struct_size", _sz), ("extension_start", _vp)] + list(fields)})


EXTENSION_TYPE_STREAM = 3          # crates/ryft-pjrt/src/lib.rs:183
EXTENSION_TYPE_LAYOUTS = 4         # crates/ryft-pjrt/src/lib.rs:184
EXTENSION_TYPE_MEMORY_DESCRIPTIONS = 6   # crates/ryft-pjrt/src/lib.rs:186
EXTENSION_TYPE_ABI_VERSION = 20    # crates/ryft-pjrt/src/lib.rs:200
EXTENSION_TYPE_STEP_TIMING = 0x62327801


class _GetStreamArgs(C.Structure):
    _fields_ = [("struct_size", _sz), ("device", _vp), ("stream", C.c_ssize_t)]


class _WaitStreamArgs(C.Structure):
    _fields_ = [("struct_size", _sz), ("stream", C.c_ssize_t), ("buffer", _vp)]


class _StepTimingArgs(C.Structure):
    _fields_ = [("struct_size", _sz), ("executable", _vp), ("device_index", _sz), ("enable", _i), ("collect", _i), ("num_steps", _sz),
                ("num_executions", _sz), ("step_ms", C.POINTER(C.c_float)), ("labels", C.POINTER(C.c_char_p)), ("flops", C.POINTER(C.c_double)),
                ("bytes", C.POINTER(C.c_double)), ("kernel_launches", C.POINTER(_i)), ("replay", _i), ("replay_ms", C.c_float), ("replay_host_ms", C.c_float)]


class _NamedValueUnion(C.Union):
    _fields_ = [("string_value", _vp), ("int64_value", _i64), ("int64_array_value", C.POINTER(_i64)), ("float_value", C.c_float),
                ("bool_value", _b)]


class NamedValueC(C.Structure):
    _fields_ = [("struct_size", _sz), ("extension_start", _vp), ("name", _vp), ("name_size", _sz), ("type", _u),
                ("value", _NamedValueUnion), ("value_size", _sz)]


A = {
    "Error_Destroy": _args("Error_Destroy", [("error", _vp)]),
    "Error_Message": _args("Error_Message", [("error", _vp), ("message", _vp), ("message_size", _sz)]),
    "Error_GetCode": _args("Error_GetCode", [("error", _vp), ("code", _u)]),
    "Plugin_Initialize": _args("Plugin_Initialize", []),
    "Plugin_Attributes": _args("Plugin_Attributes", [("attributes", C.POINTER(NamedValueC)), ("num_attributes", _sz)]),
    "Event_Create": _args("Event_Create", [("event", _vp)]),
    "Event_Set": _args("Event_Set", [("event", _vp), ("error_code", _u), ("error_message", _cp), ("error_message_size", _sz)]),
    "Event_Destroy": _args("Event_Destroy", [("event", _vp)]),
    "Event_IsReady": _args("Event_IsReady", [("event", _vp), ("is_ready", _b)]),
    "Event_Error": _args("Event_Error", [("event", _vp)]),
    "Event_Await": _args("Event_Await", [("event", _vp)]),
    "Event_OnReady": _args("Event_OnReady", [("event", _vp), ("callback", _vp), ("user_arg", _vp)]),
    "Client_Create": _args("Client_Create", [("create_options", C.POINTER(NamedValueC)), ("num_options", _sz), ("kv_get_callback", _vp),
                                              ("kv_get_user_arg", _vp), ("kv_put_callback", _vp), ("kv_put_user_arg", _vp), ("client", _vp),
                                              ("kv_try_get_callback", _vp), ("kv_try_get_user_arg", _vp)]),
    "Client_Destroy": _args("Client_Destroy", [("client", _vp)]),
    "Client_PlatformName": _args("Client_PlatformName", [("client", _vp), ("platform_name", _vp), ("platform_name_size", _sz)]),
    "Client_PlatformVersion": _args("Client_PlatformVersion", [("client", _vp), ("platform_version", _vp), ("platform_version_size", _sz)]),
    "Client_ProcessIndex": _args("Client_ProcessIndex", [("client", _vp), ("process_index", _i)]),
    "Client_Devices": _args("Client_Devices", [("client", _vp), ("devices", C.POINTER(_vp)), ("num_devices", _sz)]),
    "Client_AddressableDevices": _args("Client_AddressableDevices", [("client", _vp), ("addressable_devices", C.POINTER(_vp)), ("num_addressable_devices", _sz)]),
    "Client_LookupDevice": _args("Client_LookupDevice", [("client", _vp), ("id", _i), ("device", _vp)]),
    "Client_AddressableMemories": _args("Client_AddressableMemories", [("client", _vp), ("addressable_memories", C.POINTER(_vp)), ("num_addressable_memories", _sz)]),
    "Client_DefaultDeviceAssignment": _args("Client_DefaultDeviceAssignment", [("client", _vp), ("num_replicas", _i), ("num_partitions", _i),
                                                                                ("default_assignment_size", _sz), ("default_assignment", C.POINTER(_i))]),
    "Client_Compile": _args("Client_Compile", [("client", _vp), ("program", _vp), ("compile_options", _vp), ("compile_options_size", _sz), ("executable", _vp)]),
    "Client_BufferFromHostBuffer": _args("Client_BufferFromHostBuffer", [
        ("client", _vp), ("data", _vp), ("type", _u), ("dims", C.POINTER(_i64)), ("num_dims", _sz), ("byte_strides", C.POINTER(_i64)),
        ("num_byte_strides", _sz), ("host_buffer_semantics", _u), ("device", _vp), ("memory", _vp), ("device_layout", _vp),
        ("done_with_host_buffer", _vp), ("buffer", _vp)]),
    "Client_CreateViewOfDeviceBuffer": _args("Client_CreateViewOfDeviceBuffer", [
        ("client", _vp), ("device_buffer_ptr", _vp), ("dims", C.POINTER(_i64)), ("num_dims", _sz), ("element_type", _u), ("layout", _vp),
        ("device", _vp), ("on_delete_callback", _vp), ("on_delete_callback_arg", _vp), ("stream", C.c_ssize_t), ("buffer", _vp), ("memory", _vp)]),
    "Client_CreateErrorBuffer": _args("Client_CreateErrorBuffer", [
        ("client", _vp), ("error_code", _u), ("error_message", _cp), ("error_message_size", _sz), ("shape_dims", C.POINTER(_i64)),
        ("shape_num_dims", _sz), ("shape_element_type", _u), ("shape_layout", _vp), ("memory", _vp), ("buffer", _vp), ("payload", _vp), ("payload_size", _sz)]),
    "Device_GetDescription": _args("Device_GetDescription", [("device", _vp), ("device_description", _vp)]),
    "Device_IsAddressable": _args("Device_IsAddressable", [("device", _vp), ("is_addressable", _b)]),
    "Device_LocalHardwareId": _args("Device_LocalHardwareId", [("device", _vp), ("local_hardware_id", _i)]),
    "Device_DefaultMemory": _args("Device_DefaultMemory", [("device", _vp), ("memory", _vp)]),
    "Device_AddressableMemories": _args("Device_AddressableMemories", [("device", _vp), ("memories", C.POINTER(_vp)), ("num_memories", _sz)]),
    "Device_MemoryStats": _args("Device_MemoryStats", [("device", _vp), ("bytes_in_use", _i64)] + sum(
        [[(n, _i64), (n + "_is_set", _b)] for n in ("peak_bytes_in_use", "num_allocs", "largest_alloc_size", "bytes_limit", "bytes_reserved",
                                                     "peak_bytes_reserved", "bytes_reservable_limit", "largest_free_block_bytes", "pool_bytes",
                                                     "peak_pool_bytes")], [])),
    "Device_PoisonExecution": _args("Device_PoisonExecution", [("device", _vp), ("launch_id", C.c_int32), ("error_code", _u), ("error_message", _cp),
                                                                ("error_message_size", _sz), ("poisoned", _b), ("payload", _vp), ("payload_size", _sz)]),
    "DeviceDescription_Id": _args("DeviceDescription_Id", [("device_description", _vp), ("id", _i)]),
    "DeviceDescription_ProcessIndex": _args("DeviceDescription_ProcessIndex", [("device_description", _vp), ("process_index", _i)]),
    "DeviceDescription_Kind": _args("DeviceDescription_Kind", [("device_description", _vp), ("device_kind", _vp), ("device_kind_size", _sz)]),
    "DeviceDescription_ToString": _args("DeviceDescription_ToString", [("device_description", _vp), ("to_string", _vp), ("to_string_size", _sz)]),
    "DeviceDescription_DebugString": _args("DeviceDescription_DebugString", [("device_description", _vp), ("debug_string", _vp), ("debug_string_size", _sz)]),
    "DeviceDescription_Attributes": _args("DeviceDescription_Attributes", [("device_description", _vp), ("num_attributes", _sz), ("attributes", C.POINTER(NamedValueC))]),
    "Memory_Id": _args("Memory_Id", [("memory", _vp), ("id", _i)]),
    "Memory_Kind": _args("Memory_Kind", [("memory", _vp), ("kind", _vp), ("kind_size", _sz)]),
    "Memory_AddressableByDevices": _args("Memory_AddressableByDevices", [("memory", _vp), ("devices", C.POINTER(_vp)), ("num_devices", _sz)]),
    "Executable_Destroy": _args("Executable_Destroy", [("executable", _vp)]),
    "Executable_Name": _args("Executable_Name", [("executable", _vp), ("executable_name", _vp), ("executable_name_size", _sz)]),
    "Executable_NumReplicas": _args("Executable_NumReplicas", [("executable", _vp), ("num_replicas", _sz)]),
    "Executable_NumPartitions": _args("Executable_NumPartitions", [("executable", _vp), ("num_partitions", _sz)]),
    "Executable_NumOutputs": _args("Executable_NumOutputs", [("executable", _vp), ("num_outputs", _sz)]),
    "Executable_OutputElementTypes": _args("Executable_OutputElementTypes", [("executable", _vp), ("output_types", C.POINTER(_u)), ("num_output_types", _sz)]),
    "Executable_OutputDimensions": _args("Executable_OutputDimensions", [("executable", _vp), ("num_outputs", _sz), ("dims", C.POINTER(_i64)), ("dim_sizes", C.POINTER(_sz))]),
    "Executable_OutputMemoryKinds": _args("Executable_OutputMemoryKinds", [("executable", _vp), ("num_outputs", _sz), ("memory_kinds", C.POINTER(_vp)), ("memory_kind_sizes", C.POINTER(_sz))]),
    "Executable_Fingerprint": _args("Executable_Fingerprint", [("executable", _vp), ("executable_fingerprint", _vp), ("executable_fingerprint_size", _sz)]),
    "Executable_GetCostAnalysis": _args("Executable_GetCostAnalysis", [("executable", _vp), ("num_properties", _sz), ("properties", C.POINTER(NamedValueC))]),
    "Executable_Serialize": _args("Executable_Serialize", [("executable", _vp), ("serialized_bytes", _vp), ("serialized_bytes_size", _sz),
                                                            ("serialized_executable", _vp), ("serialized_executable_deleter", _vp)]),
    "Executable_OptimizedProgram": _args("Executable_OptimizedProgram", [("executable", _vp), ("program", _vp)]),
    "Executable_GetCompiledMemoryStats": _args("Executable_GetCompiledMemoryStats", [("executable", _vp)] + [(n, _i64) for n in (
        "generated_code_size_in_bytes", "argument_size_in_bytes", "output_size_in_bytes", "alias_size_in_bytes", "temp_size_in_bytes",
        "host_generated_code_size_in_bytes", "host_argument_size_in_bytes", "host_output_size_in_bytes", "host_alias_size_in_bytes",
        "host_temp_size_in_bytes", "peak_memory_in_bytes", "total_size_in_bytes", "total_allocation_bytes", "indefinite_allocations",
        "peak_unpadded_heap_bytes")]),
    "Executable_DeserializeAndLoad": _args("Executable_DeserializeAndLoad", [
        ("client", _vp), ("serialized_executable", _vp), ("serialized_executable_size", _sz), ("loaded_executable", _vp),
        ("overridden_serialized_compile_options", _vp), ("overridden_serialized_compile_options_size", _sz)]),
    "LoadedExecutable_Destroy": _args("LoadedExecutable_Destroy", [("executable", _vp)]),
    "LoadedExecutable_GetExecutable": _args("LoadedExecutable_GetExecutable", [("loaded_executable", _vp), ("executable", _vp)]),
    "LoadedExecutable_AddressableDevices": _args("LoadedExecutable_AddressableDevices", [("executable", _vp), ("addressable_devices", C.POINTER(_vp)), ("num_addressable_devices", _sz)]),
    "LoadedExecutable_AddressableDeviceLogicalIds": _args("LoadedExecutable_AddressableDeviceLogicalIds", [("executable", _vp), ("ids", C.POINTER(_i * 2)), ("num", _sz)]),
    "LoadedExecutable_GetDeviceAssignment": _args("LoadedExecutable_GetDeviceAssignment", [("executable", _vp), ("serialized_bytes", _vp), ("serialized_bytes_size", _sz),
                                                                                            ("serialized_device_assignment", _vp), ("deleter", _vp)]),
    "LoadedExecutable_Delete": _args("LoadedExecutable_Delete", [("executable", _vp)]),
    "LoadedExecutable_IsDeleted": _args("LoadedExecutable_IsDeleted", [("executable", _vp), ("is_deleted", _b)]),
    "LoadedExecutable_Execute": _args("LoadedExecutable_Execute", [("executable", _vp), ("options", _vp), ("argument_lists", C.POINTER(C.POINTER(_vp))),
                                                                    ("num_devices", _sz), ("num_args", _sz), ("output_lists", C.POINTER(C.POINTER(_vp))),
                                                                    ("device_complete_events", C.POINTER(_vp)), ("execute_device", _vp)]),
    "Buffer_Destroy": _args("Buffer_Destroy", [("buffer", _vp)]),
    "Buffer_Delete": _args("Buffer_Delete", [("buffer", _vp)]),
    "Buffer_IsDeleted": _args("Buffer_IsDeleted", [("buffer", _vp), ("is_deleted", _b)]),
    "Buffer_ElementType": _args("Buffer_ElementType", [("buffer", _vp), ("type", _u)]),
    "Buffer_Dimensions": _args("Buffer_Dimensions", [("buffer", _vp), ("dims", C.POINTER(_i64)), ("num_dims", _sz)]),
    "Buffer_OnDeviceSizeInBytes": _args("Buffer_OnDeviceSizeInBytes", [("buffer", _vp), ("on_device_size_in_bytes", _sz)]),
    "Buffer_Device": _args("Buffer_Device", [("buffer", _vp), ("device", _vp)]),
    "Buffer_Memory": _args("Buffer_Memory", [("buffer", _vp), ("memory", _vp)]),
    "Buffer_IsOnCpu": _args("Buffer_IsOnCpu", [("buffer", _vp), ("is_on_cpu", _b)]),
    "Buffer_ReadyEvent": _args("Buffer_ReadyEvent", [("buffer", _vp), ("event", _vp)]),
    "Buffer_ToHostBuffer": _args("Buffer_ToHostBuffer", [("src", _vp), ("host_layout", _vp), ("dst", _vp), ("dst_size", _sz), ("event", _vp)]),
    "Buffer_CopyRawToHost": _args("Buffer_CopyRawToHost", [("buffer", _vp), ("dst", _vp), ("offset", _i64), ("transfer_size", _i64), ("event", _vp)]),
    "Buffer_CopyToDevice": _args("Buffer_CopyToDevice", [("buffer", _vp), ("dst_device", _vp), ("dst_buffer", _vp)]),
    "Buffer_OpaqueDeviceMemoryDataPointer": _args("Buffer_OpaqueDeviceMemoryDataPointer", [("buffer", _vp), ("device_memory_ptr", _vp)]),
}


class ShapeSpecC(C.Structure):
    """PJRT_ShapeSpec (crates/ryft-pjrt/src/transfers.rs:800-812)."""
    _fields_ = [("struct_size", _sz), ("extension_start", _vp), ("dims", C.POINTER(_i64)), ("num_dims", _sz), ("element_type", _i)]


_TM = "AsyncHostToDeviceTransferManager_"
A.update({
    "Client_CreateBuffersForAsyncHostToDevice": _args("CreateBuffersForAsyncH2D", [("client", _vp), ("shape_specs", C.POINTER(ShapeSpecC)), ("num_shape_specs", _sz),
                                                                                   ("device_layouts", _vp), ("num_device_layouts", _sz), ("memory", _vp),
                                                                                   ("transfer_manager", _vp)]),
    _TM + "Device": _args("TmDevice", [("transfer_manager", _vp), ("device_out", _vp)]),
    _TM + "BufferCount": _args("TmBufferCount", [("transfer_manager", _vp), ("buffer_count", _sz)]),
    _TM + "BufferSize": _args("TmBufferSize", [("transfer_manager", _vp), ("buffer_index", _i), ("buffer_size", _sz)]),
    _TM + "RetrieveBuffer": _args("TmRetrieveBuffer", [("transfer_manager", _vp), ("buffer_index", _i), ("buffer_out", _vp)]),
    _TM + "TransferData": _args("TmTransferData", [("transfer_manager", _vp), ("buffer_index", _i), ("data", _vp), ("offset", _i64), ("transfer_size", _i64),
                                                   ("is_last_transfer", C.c_bool), ("done_with_h2d_transfer", _vp)]),
    _TM + "TransferLiteral": _args("TmTransferLiteral", [("transfer_manager", _vp), ("buffer_index", _i), ("data", _vp), ("shape_dims", C.POINTER(_i64)),
                                                         ("shape_num_dims", _sz), ("shape_element_type", _i), ("shape_layout", _vp), ("done_with_h2d_transfer", _vp)]),
    _TM + "SetBufferError": _args("TmSetBufferError", [("transfer_manager", _vp), ("buffer_index", _i), ("error_code", _i), ("error_message", C.c_char_p),
                                                       ("error_message_size", _sz)]),
    _TM + "AddMetadata": _args("TmAddMetadata", [("transfer_manager", _vp), ("transfer_metadata", _vp), ("num_metadata", _sz)]),
    _TM + "Destroy": _args("TmDestroy", [("transfer_manager", _vp)]),
})


class ProgramC(C.Structure):
    _fields_ = [("struct_size", _sz), ("extension_start", _vp), ("code", _vp), ("code_size", _sz), ("format", _vp), ("format_size", _sz)]


class ExecuteOptionsC(C.Structure):
    _fields_ = [("struct_size", _sz), ("extension_start", _vp), ("send_callbacks", _vp), ("recv_callbacks", _vp), ("num_send_ops", _sz),
                ("num_recv_ops", _sz), ("launch_id", _i), ("non_donatable_input_indices", C.POINTER(_i64)), ("num_non_donatable_input_indices", _sz),
                ("context", _vp), ("call_location", _cp), ("num_tasks", _sz), ("task_ids", _vp), ("incarnation_ids", _vp), ("multi_slice_config", _vp)]


class ApiVersionC(C.Structure):
    _fields_ = [("struct_size", _sz), ("extension_start", _vp), ("major_version", _i), ("minor_version", _i)]


def api_function_names() -> List[str]:
    """Function-pointer order of PJRT_Api, read from include/b2x_pjrt_c_api.h (one source of truth for the layout)."""
    text = _HEADER.read_text()
    body = text[text.index("typedef struct PJRT_Api {"):text.index("} PJRT_Api;")]
    names = []
    for line in body.splitlines():
        m = re.search(r"B2X_PJRT_FN\((\w+)\)|PJRT_Fn (\w+);|\(\*(PJRT_\w+)\)\(", line)
        if m:
            names.append(next(g for g in m.groups() if g))
    return names


_FN = C.CFUNCTYPE(_vp, _vp)
_VOIDFN = C.CFUNCTYPE(None, _vp)


class Api:
    """The PJRT_Api function table (crates/ryft-pjrt/src/lib.rs:214-364)."""

    def __init__(self, ptr: int):
        self.ptr = ptr
        names = api_function_names()
        self.names = names
        head = C.cast(ptr, C.POINTER(_sz))
        self.struct_size = head[0]
        ver = ApiVersionC.from_address(ptr + 16)
        self.version = (ver.major_version, ver.minor_version)
        base = ptr + 16 + C.sizeof(ApiVersionC)
        self.fns: Dict[str, int] = {}
        for i, n in enumerate(names):
            off = 16 + C.sizeof(ApiVersionC) + 8 * i
            self.fns[n] = C.c_void_p.from_address(base + 8 * i).value if off < self.struct_size else None

    def has(self, name: str) -> bool:
        return bool(self.fns.get("PJRT_" + name))

    def extension(self, type_id: int) -> Optional[int]:
        """Address of the extension struct with the given type id in the PJRT_Api::extension_start chain
        (crates/ryft-pjrt/src/lib.rs:205-212), or None; absence maps to Unimplemented in ryft."""
        node = C.c_void_p.from_address(self.ptr + 8).value
        while node:
            ext_type = C.c_uint.from_address(node + 8).value
            if ext_type == type_id:
                return node
            node = C.c_void_p.from_address(node + 16).value
        return None

    def call(self, name: str, args) -> None:
        """Invokes PJRT_<name>(&args); a NULL entry maps to UNIMPLEMENTED like ryft's macros do
        (crates/ryft-pjrt/src/macros.rs:36-44)."""
        fp = self.fns.get("PJRT_" + name)
        if not fp:
            raise PjrtError(12, f"PJRT_{name} is not implemented by this plugin")
        args.struct_size = C.sizeof(args)
        if name in ("Error_Destroy", "Error_Message"):
            _VOIDFN(fp)(C.addressof(args))
            return
        err = _FN(fp)(C.addressof(args))
        if err:
            raise self._take_error(err)

    def _take_error(self, err: int) -> PjrtError:
        m = A["Error_Message"](); m.error = err
        self.call("Error_Message", m)
        msg = C.string_at(m.message, m.message_size).decode("utf-8", "replace")
        g = A["Error_GetCode"](); g.error = err
        self.call("Error_GetCode", g)
        d = A["Error_Destroy"](); d.error = err
        self.call("Error_Destroy", d)
        return PjrtError(int(g.code), msg)


def _str(ptr, size) -> str:
    return C.string_at(ptr, size).decode("utf-8", "replace") if ptr else ""


def _named_values(ptr, n) -> Dict[str, object]:
    out = {}
    for i in range(n):
        v = ptr[i]
        name = _str(v.name, v.name_size)
        if v.type == 0:
            out[name] = _str(v.value.string_value, v.value_size)
        elif v.type == 1:
            out[name] = int(v.value.int64_value)
        elif v.type == 2:
            out[name] = [int(v.value.int64_array_value[j]) for j in range(v.value_size)]
        elif v.type == 3:
            out[name] = float(v.value.float_value)
        else:
            out[name] = bool(v.value.bool_value)
    return out


# ---- CompilationOptions (protobuf wire format written by hand) --------------------------------------------------------
def _varint(v: int) -> bytes:
    out = bytearray()
    v &= (1 << 64) - 1
    while v >= 0x80:
        out.append((v & 0x7F) | 0x80)
        v >>= 7
    out.append(v)
    return bytes(out)


def _field(tag: int, wire: int, payload: bytes) -> bytes:
    return _varint((tag << 3) | wire) + payload


@dataclass
class CompilationOptions:
    """Subset of xla.CompileOptionsProto that the executor honours (crates/ryft-xla-sys/src/protos.rs:3298-3346,
    2391-2417): replica_count, partition_count, device_assignment, device_ordinal, matrix_unit_operand_precision."""
    replica_count: int = 1
    partition_count: int = 1
    device_assignment: Optional[List[int]] = None  # replica -> device id
    device_ordinal: int = -1
    precision: int = 0
    use_spmd_partitioning: bool = False

    def encode(self) -> bytes:
        ebo = b""
        if self.device_ordinal >= 0:
            ebo += _field(1, 0, _varint(self.device_ordinal))
        ebo += _field(4, 0, _varint(self.replica_count))
        ebo += _field(5, 0, _varint(self.partition_count))
        if self.use_spmd_partitioning:
            ebo += _field(6, 0, _varint(1))
        if self.device_assignment is not None:
            packed = b"".join(_varint(d) for d in self.device_assignment)
            comp = _field(1, 2, _varint(len(packed)) + packed)
            da = _field(1, 0, _varint(self.replica_count)) + _field(2, 0, _varint(1)) + _field(3, 2, _varint(len(comp)) + comp)
            ebo += _field(9, 2, _varint(len(da)) + da)
        out = _field(3, 2, _varint(len(ebo)) + ebo)
        if self.precision:
            out += _field(10, 0, _varint(self.precision))
        return out


@dataclass
class Program:
    """`Program::Mlir { bytecode }` (crates/ryft-pjrt/src/programs.rs:19-62); `code` may be MLIR text."""
    code: bytes
    format: str = "mlir"

    @staticmethod
    def mlir(text) -> "Program":
        return Program(text.encode() if isinstance(text, str) else bytes(text))


# ---- object wrappers ---------------------------------------------------------------------------------------------------
class Event:
    """`Event<()>` (crates/ryft-pjrt/src/events.rs:18-198)."""

    def __init__(self, api: Api, handle: int, result: Optional[Callable[[], object]] = None, keep=None):
        self.api, self.handle, self._result, self._keep = api, handle, result, keep

    @staticmethod
    def create(api: Api) -> "Event":
        a = A["Event_Create"](); api.call("Event_Create", a)
        return Event(api, a.event)

    def set(self, code: int = 0, message: str = "") -> None:
        a = A["Event_Set"](); a.event = self.handle; a.error_code = code
        m = message.encode(); a.error_message = m; a.error_message_size = len(m)
        self.api.call("Event_Set", a)

    def ready(self) -> bool:
        a = A["Event_IsReady"](); a.event = self.handle
        self.api.call("Event_IsReady", a)
        return bool(a.is_ready)

    def await_(self):
        a = A["Event_Await"](); a.event = self.handle
        self.api.call("Event_Await", a)
        return self._result() if self._result else None

    def error(self) -> Optional[PjrtError]:
        a = A["Event_Error"](); a.event = self.handle
        try:
            self.api.call("Event_Error", a)
        except PjrtError as e:
            return e
        return None

    def on_ready(self, fn: Callable[[Optional[PjrtError]], None]) -> None:
        api = self.api
        holder = {}

        def tramp(err, _arg):
            e = api._take_error(err) if err else None
            try:
                fn(e)
            finally:
                _LIVE_CALLBACKS.pop(holder["key"], None)
        cb = C.CFUNCTYPE(None, _vp, _vp)(tramp)
        holder["key"] = id(cb)
        _LIVE_CALLBACKS[id(cb)] = cb
        a = A["Event_OnReady"](); a.event = self.handle; a.callback = C.cast(cb, _vp); a.user_arg = None
        self.api.call("Event_OnReady", a)

    def __del__(self):
        try:
            if self.handle:
                a = A["Event_Destroy"](); a.event = self.handle
                self.api.call("Event_Destroy", a)
                self.handle = None
        except Exception:
            pass


_LIVE_CALLBACKS: Dict[int, object] = {}


class Device:
    def __init__(self, client: "Client", handle: int):
        self.client, self.api, self.handle = client, client.api, handle
        a = A["Device_GetDescription"](); a.device = handle
        self.api.call("Device_GetDescription", a)
        self._desc = a.device_description

    def _desc_call(self, name, out_ptr, out_size):
        a = A[name](); a.device_description = self._desc
        self.api.call(name, a)
        return _str(getattr(a, out_ptr), getattr(a, out_size))

    @property
    def id(self) -> int:
        a = A["DeviceDescription_Id"](); a.device_description = self._desc
        self.api.call("DeviceDescription_Id", a)
        return int(a.id)

    @property
    def process_index(self) -> int:
        a = A["DeviceDescription_ProcessIndex"](); a.device_description = self._desc
        self.api.call("DeviceDescription_ProcessIndex", a)
        return int(a.process_index)

    def memory_descriptions(self):
        """Memory-descriptions extension (crates/ryft-pjrt/src/extensions/memory_descriptions.rs): the memory kinds of
        this device's description as (kind, kind_id) pairs, and the index of the default one."""
        ext = self.api.extension(EXTENSION_TYPE_MEMORY_DESCRIPTIONS)
        if not ext:
            raise PjrtError(12, "the plugin has no memory-descriptions extension")
        a = _args("MemoryDescriptions", [("device_description", _vp), ("memory_descriptions", _vp), ("num_memory_descriptions", _sz),
                                         ("default_memory_index", C.c_ssize_t)])()
        a.struct_size = C.sizeof(a); a.device_description = self._desc
        err = _FN(C.c_void_p.from_address(ext + 24).value)(C.addressof(a))
        if err:
            raise self.api._take_error(err)
        out = []
        ptrs = (C.c_void_p * a.num_memory_descriptions).from_address(a.memory_descriptions) if a.num_memory_descriptions else []
        for i in range(a.num_memory_descriptions):
            k = _args("MemoryDescriptionKind", [("memory_description", _vp), ("kind", _vp), ("kind_size", _sz), ("kind_id", _i)])()
            k.struct_size = C.sizeof(k); k.memory_description = ptrs[i]
            err = _FN(C.c_void_p.from_address(ext + 32).value)(C.addressof(k))
            if err:
                raise self.api._take_error(err)
            out.append((_str(k.kind, k.kind_size), int(k.kind_id)))
        return out, int(a.default_memory_index)

    @property
    def kind(self) -> str: return self._desc_call("DeviceDescription_Kind", "device_kind", "device_kind_size")
    def to_string(self) -> str: return self._desc_call("DeviceDescription_ToString", "to_string", "to_string_size")
    def debug_string(self) -> str: return self._desc_call("DeviceDescription_DebugString", "debug_string", "debug_string_size")

    def attributes(self) -> Dict[str, object]:
        a = A["DeviceDescription_Attributes"](); a.device_description = self._desc
        self.api.call("DeviceDescription_Attributes", a)
        return _named_values(a.attributes, a.num_attributes)

    def is_addressable(self) -> bool:
        a = A["Device_IsAddressable"](); a.device = self.handle
        self.api.call("Device_IsAddressable", a)
        return bool(a.is_addressable)

    def local_hardware_id(self) -> int:
        a = A["Device_LocalHardwareId"](); a.device = self.handle
        self.api.call("Device_LocalHardwareId", a)
        return int(a.local_hardware_id)

    def default_memory(self) -> int:
        a = A["Device_DefaultMemory"](); a.device = self.handle
        self.api.call("Device_DefaultMemory", a)
        return a.memory

    def memory_statistics(self) -> Dict[str, int]:
        a = A["Device_MemoryStats"](); a.device = self.handle
        self.api.call("Device_MemoryStats", a)
        return {"bytes_in_use": a.bytes_in_use, "peak_bytes_in_use": a.peak_bytes_in_use, "num_allocs": a.num_allocs, "bytes_limit": a.bytes_limit}

    def compute_stream(self) -> int:
        """Stream extension (crates/ryft-pjrt/src/extensions/stream.rs): the CUDA stream executions on this device are
        enqueued on, as an integer handle."""
        ext = self.api.extension(EXTENSION_TYPE_STREAM)
        if not ext:
            raise PjrtError(12, "the plugin has no stream extension")
        fn = C.c_void_p.from_address(ext + 24).value
        a = _GetStreamArgs(); a.struct_size = C.sizeof(a); a.device = self.handle
        err = _FN(fn)(C.addressof(a))
        if err:
            raise self.api._take_error(err)
        return int(a.stream)

    def poison_execution(self, launch_id: int, code: int, message: str) -> bool:
        a = A["Device_PoisonExecution"](); a.device = self.handle; a.launch_id = launch_id; a.error_code = code
        m = message.encode(); a.error_message = m; a.error_message_size = len(m)
        self.api.call("Device_PoisonExecution", a)
        return bool(a.poisoned)

    def __eq__(self, other): return isinstance(other, Device) and other.handle == self.handle
    def __hash__(self): return hash(self.handle)


class Buffer:
    """`Buffer` (crates/ryft-pjrt/src/buffers.rs)."""

    def __init__(self, client: "Client", handle: int, keep=None):
        self.client, self.api, self.handle, self._keep = client, client.api, handle, keep

    def layout(self) -> "Layout":
        """Memory layout of this buffer through the layouts extension (crates/ryft-pjrt/src/extensions/layouts.rs:610-629)."""
        a = _args("LayoutBuffer", [("buffer", _vp), ("layout", _vp)])()
        a.buffer = self.handle
        Layout._call(self.client.api, Layout._BUFFER, a)
        return Layout(self.client.api, a.layout, borrowed=False)

    def element_type(self) -> BufferType:
        a = A["Buffer_ElementType"](); a.buffer = self.handle
        self.api.call("Buffer_ElementType", a)
        return BufferType(a.type)

    def dimensions(self) -> List[int]:
        a = A["Buffer_Dimensions"](); a.buffer = self.handle
        self.api.call("Buffer_Dimensions", a)
        return [int(a.dims[i]) for i in range(a.num_dims)]

    def on_device_size_in_bytes(self) -> int:
        a = A["Buffer_OnDeviceSizeInBytes"](); a.buffer = self.handle
        self.api.call("Buffer_OnDeviceSizeInBytes", a)
        return int(a.on_device_size_in_bytes)

    def device(self) -> Device:
        a = A["Buffer_Device"](); a.buffer = self.handle
        self.api.call("Buffer_Device", a)
        return Device(self.client, a.device)

    def is_on_cpu(self) -> bool:
        a = A["Buffer_IsOnCpu"](); a.buffer = self.handle
        self.api.call("Buffer_IsOnCpu", a)
        return bool(a.is_on_cpu)

    def device_pointer(self) -> int:
        a = A["Buffer_OpaqueDeviceMemoryDataPointer"](); a.buffer = self.handle
        self.api.call("Buffer_OpaqueDeviceMemoryDataPointer", a)
        return int(a.device_memory_ptr or 0)

    def ready(self) -> Event:
        a = A["Buffer_ReadyEvent"](); a.buffer = self.handle
        self.api.call("Buffer_ReadyEvent", a)
        return Event(self.api, a.event)

    def wait_until_ready_on_stream(self, stream: int) -> None:
        """Stream extension: makes `stream` wait for this buffer's definition event."""
        ext = self.api.extension(EXTENSION_TYPE_STREAM)
        if not ext:
            raise PjrtError(12, "the plugin has no stream extension")
        fn = C.c_void_p.from_address(ext + 32).value
        a = _WaitStreamArgs(); a.struct_size = C.sizeof(a); a.stream = stream; a.buffer = self.handle
        err = _FN(fn)(C.addressof(a))
        if err:
            raise self.api._take_error(err)

    def copy_to_host(self, out: Optional[np.ndarray] = None) -> Event:
        """Two-call protocol of `Buffer::copy_to_host` (crates/ryft-pjrt/src/buffers.rs:1237-1295): size query, then copy.
        Awaiting the returned event yields the bytes (or `out`)."""
        a = A["Buffer_ToHostBuffer"](); a.src = self.handle; a.dst = None
        self.api.call("Buffer_ToHostBuffer", a)
        n = int(a.dst_size)
        if out is None:
            host = np.empty(n, dtype=np.uint8)
        else:
            host = out
            assert host.nbytes >= n and host.flags.c_contiguous
        a2 = A["Buffer_ToHostBuffer"](); a2.src = self.handle; a2.dst = host.ctypes.data; a2.dst_size = host.nbytes
        self.api.call("Buffer_ToHostBuffer", a2)
        return Event(self.api, a2.event, result=(lambda: host.tobytes()) if out is None else (lambda: host), keep=host)

    def to_numpy(self) -> np.ndarray:
        dt = buffer_type_to_np(self.element_type())
        dims = self.dimensions()
        out = np.empty(dims, dtype=dt)
        self.copy_to_host(out.reshape(-1).view(np.uint8) if out.size else np.empty(0, np.uint8)).await_()
        return out

    def copy_raw_to_host(self, offset: int, size: int) -> Event:
        host = np.empty(max(size, 0), dtype=np.uint8)
        a = A["Buffer_CopyRawToHost"](); a.buffer = self.handle; a.dst = host.ctypes.data; a.offset = offset; a.transfer_size = size
        self.api.call("Buffer_CopyRawToHost", a)
        return Event(self.api, a.event, result=lambda: host.tobytes(), keep=host)

    def copy_to_device(self, device: Device) -> "Buffer":
        a = A["Buffer_CopyToDevice"](); a.buffer = self.handle; a.dst_device = device.handle
        self.api.call("Buffer_CopyToDevice", a)
        return Buffer(self.client, a.dst_buffer)

    def delete(self) -> None:
        a = A["Buffer_Delete"](); a.buffer = self.handle
        self.api.call("Buffer_Delete", a)

    def is_deleted(self) -> bool:
        a = A["Buffer_IsDeleted"](); a.buffer = self.handle
        self.api.call("Buffer_IsDeleted", a)
        return bool(a.is_deleted)

    def __del__(self):
        try:
            if self.handle and self.client.handle:
                a = A["Buffer_Destroy"](); a.buffer = self.handle
                self.api.call("Buffer_Destroy", a)
                self.handle = None
        except Exception:
            pass


@dataclass
class ExecutionDeviceInputs:
    """Arguments for one addressable device (crates/ryft-pjrt/src/programs.rs:745-748)."""
    inputs: Sequence[Buffer]


@dataclass
class ExecutionDeviceOutputs:
    done: Event
    outputs: List[Buffer]


class Executable:
    def __init__(self, api: Api, handle: int):
        self.api, self.handle = api, handle

    def _get(self, name, *fields):
        a = A[name](); a.executable = self.handle
        self.api.call(name, a)
        return a

    def _layouts(self, slot: int) -> List["Layout"]:
        a = _args("LayoutExecutable", [("executable", _vp), ("count", _sz), ("layouts", _vp)])()
        a.executable = self.handle
        Layout._call(self.api, slot, a)
        ptrs = (C.c_void_p * a.count).from_address(a.layouts) if a.count else []
        keep = [Layout(self.api, ptrs[i], borrowed=True) for i in range(a.count)]
        for l in keep:
            l._owner = self          # borrowed from the executable: keep it alive
        return keep

    def input_layouts(self) -> List["Layout"]:
        """`Executable::input_layouts` (crates/ryft-pjrt/src/extensions/layouts.rs:247-263)."""
        return self._layouts(Layout._EXE_PARAMETERS)

    def output_layouts(self) -> List["Layout"]:
        """`Executable::output_layouts` (crates/ryft-pjrt/src/extensions/layouts.rs:266-283)."""
        return self._layouts(Layout._EXE_OUTPUTS)

    def name(self) -> str:
        a = self._get("Executable_Name"); return _str(a.executable_name, a.executable_name_size)
    def num_replicas(self) -> int: return int(self._get("Executable_NumReplicas").num_replicas)
    def num_partitions(self) -> int: return int(self._get("Executable_NumPartitions").num_partitions)
    def num_outputs(self) -> int: return int(self._get("Executable_NumOutputs").num_outputs)

    def output_element_types(self) -> List[BufferType]:
        a = self._get("Executable_OutputElementTypes")
        return [BufferType(a.output_types[i]) for i in range(a.num_output_types)]

    def output_dimensions(self) -> List[List[int]]:
        a = self._get("Executable_OutputDimensions")
        out, k = [], 0
        for i in range(a.num_outputs):
            r = a.dim_sizes[i]
            out.append([int(a.dims[k + j]) for j in range(r)])
            k += r
        return out

    def output_memory_kinds(self) -> List[str]:
        a = self._get("Executable_OutputMemoryKinds")
        return [_str(a.memory_kinds[i], a.memory_kind_sizes[i]) for i in range(a.num_outputs)]

    def abi_version(self) -> "ExecutableAbiVersion":
        """`Executable::abi_version` (crates/ryft-pjrt/src/extensions/abi_version.rs:51-62)."""
        a = _AbiVersion._struct([("executable", _vp), ("abi_version", _vp)]); a.executable = self.handle
        _AbiVersion._call(self.api, _AbiVersion._EXECUTABLE, a)
        return ExecutableAbiVersion(self.api, a.abi_version)

    def fingerprint(self) -> str:
        a = self._get("Executable_Fingerprint"); return _str(a.executable_fingerprint, a.executable_fingerprint_size)

    def cost_analysis(self) -> Dict[str, object]:
        a = self._get("Executable_GetCostAnalysis"); return _named_values(a.properties, a.num_properties)

    def compiled_memory_statistics(self) -> Dict[str, int]:
        a = self._get("Executable_GetCompiledMemoryStats")
        return {"argument_size_in_bytes": a.argument_size_in_bytes, "output_size_in_bytes": a.output_size_in_bytes,
                "temp_size_in_bytes": a.temp_size_in_bytes}

    def serialize(self) -> bytes:
        a = self._get("Executable_Serialize")
        data = C.string_at(a.serialized_bytes, a.serialized_bytes_size)
        if a.serialized_executable_deleter:
            _VOIDFN(a.serialized_executable_deleter)(a.serialized_executable)
        return data

    def optimized_program(self) -> Program:
        p = ProgramC(); p.struct_size = C.sizeof(p); p.code = None
        a = A["Executable_OptimizedProgram"](); a.executable = self.handle; a.program = C.addressof(p)
        self.api.call("Executable_OptimizedProgram", a)
        buf = C.create_string_buffer(p.code_size)
        p.code = C.addressof(buf)
        self.api.call("Executable_OptimizedProgram", a)
        return Program(buf.raw[:p.code_size], _str(p.format, p.format_size))

    def __del__(self):
        try:
            if self.handle:
                a = A["Executable_Destroy"](); a.executable = self.handle
                self.api.call("Executable_Destroy", a)
                self.handle = None
        except Exception:
            pass


class LoadedExecutable:
    """`LoadedExecutable` (crates/ryft-pjrt/src/programs.rs:636-995)."""

    def __init__(self, client: "Client", handle: int):
        self.client, self.api, self.handle = client, client.api, handle

    def executable(self) -> Executable:
        a = A["LoadedExecutable_GetExecutable"](); a.loaded_executable = self.handle
        self.api.call("LoadedExecutable_GetExecutable", a)
        return Executable(self.api, a.executable)

    def addressable_devices(self) -> List[Device]:
        a = A["LoadedExecutable_AddressableDevices"](); a.executable = self.handle
        self.api.call("LoadedExecutable_AddressableDevices", a)
        return [Device(self.client, a.addressable_devices[i]) for i in range(a.num_addressable_devices)]

    def addressable_device_logical_ids(self) -> List[tuple]:
        a = A["LoadedExecutable_AddressableDeviceLogicalIds"](); a.executable = self.handle
        self.api.call("LoadedExecutable_AddressableDeviceLogicalIds", a)
        return [(int(a.ids[i][0]), int(a.ids[i][1])) for i in range(a.num)]

    def device_assignment(self) -> bytes:
        a = A["LoadedExecutable_GetDeviceAssignment"](); a.executable = self.handle
        self.api.call("LoadedExecutable_GetDeviceAssignment", a)
        data = C.string_at(a.serialized_bytes, a.serialized_bytes_size)
        if a.deleter:
            _VOIDFN(a.deleter)(a.serialized_device_assignment)
        return data

    def step_timing(self, enable: int = -1, collect: bool = False, device_index: int = 0) -> List[dict]:
        """Step-timing extension of this plugin: per plan step, the label, algorithmic flops and bytes per launch,
        kernels launched per step and (when `collect`) the device milliseconds summed over the executions recorded
        since timing was enabled."""
        a = self._step_timing_call(enable, collect, device_index, 0)
        out = []
        for i in range(a.num_steps):
            out.append({"label": a.labels[i].decode(), "flops": a.flops[i], "bytes": a.bytes[i], "kernel_launches": a.kernel_launches[i],
                        "ms": a.step_ms[i], "executions": int(a.num_executions)})
        return out

    def replay(self, times: int, device_index: int = 0) -> float:
        """Enqueues the plan `times` more times back to back with the arguments and outputs of the last execution that was
        launched while step timing was enabled (the caller keeps those buffers alive) and returns the device milliseconds
        of all repetitions together: the kernels' own time, without the host work of an execution between launches."""
        a = self._step_timing_call(-1, False, device_index, times)
        self.last_replay_host_ms = float(a.replay_host_ms)   # close to the device time: the host's enqueue rate was the limit
        return float(a.replay_ms)

    def _step_timing_call(self, enable: int, collect: bool, device_index: int, replay: int) -> "_StepTimingArgs":
        ext = self.api.extension(EXTENSION_TYPE_STEP_TIMING)
        if not ext:
            raise PjrtError(12, "the plugin has no step-timing extension")
        fn = C.c_void_p.from_address(ext + 24).value
        a = _StepTimingArgs(); a.struct_size = C.sizeof(a); a.executable = self.handle; a.device_index = device_index
        a.enable = enable; a.collect = 1 if collect else 0; a.replay = replay
        err = _FN(fn)(C.addressof(a))
        if err:
            raise self.api._take_error(err)
        return a

    def delete(self) -> None:
        a = A["LoadedExecutable_Delete"](); a.executable = self.handle
        self.api.call("LoadedExecutable_Delete", a)

    def is_deleted(self) -> bool:
        a = A["LoadedExecutable_IsDeleted"](); a.executable = self.handle
        self.api.call("LoadedExecutable_IsDeleted", a)
        return bool(a.is_deleted)

    def execute(self, inputs: Sequence[ExecutionDeviceInputs], launch_id: int = 0, execute_device: Optional[Device] = None) -> List[ExecutionDeviceOutputs]:
        """`LoadedExecutable::execute` (crates/ryft-pjrt/src/programs.rs:769-963): the same client-side validation
        messages, then PJRT_LoadedExecutable_Execute with pre-allocated output and event slots."""
        # the device count and the output count of a loaded executable never change: asked once, not per launch
        shape = getattr(self, "_launch_shape", None)
        if shape is None:
            shape = self._launch_shape = (len(self.addressable_devices()), self.executable().num_outputs())
        n_devices, num_outputs = shape
        if execute_device is None and len(inputs) != n_devices:
            raise PjrtError(3, f"the number of provided execution inputs ({len(inputs)}) does not match the number of addressable "
                               f"devices of the executable ({n_devices})")
        num_args = len(inputs[0].inputs) if inputs else 0
        for i, di in enumerate(inputs):
            if len(di.inputs) != num_args:
                raise PjrtError(3, f"device {i} was given {len(di.inputs)} arguments but device 0 was given {num_args}")
        nd = len(inputs)
        arg_rows = [(_vp * max(num_args, 1))(*[b.handle for b in di.inputs]) for di in inputs]
        arg_lists = (C.POINTER(_vp) * nd)(*[C.cast(r, C.POINTER(_vp)) for r in arg_rows])
        out_rows = [(_vp * max(num_outputs, 1))() for _ in range(nd)]
        out_lists = (C.POINTER(_vp) * nd)(*[C.cast(r, C.POINTER(_vp)) for r in out_rows])
        events = (_vp * nd)()
        opts = ExecuteOptionsC(); opts.struct_size = C.sizeof(opts); opts.launch_id = launch_id
        nd_idx = (_i64 * max(num_args, 1))(*range(num_args))
        opts.non_donatable_input_indices = C.cast(nd_idx, C.POINTER(_i64)); opts.num_non_donatable_input_indices = num_args
        a = A["LoadedExecutable_Execute"]()
        a.executable = self.handle; a.options = C.addressof(opts)
        a.argument_lists = C.cast(arg_lists, C.POINTER(C.POINTER(_vp))); a.num_devices = nd; a.num_args = num_args
        a.output_lists = C.cast(out_lists, C.POINTER(C.POINTER(_vp))); a.device_complete_events = C.cast(events, C.POINTER(_vp))
        a.execute_device = execute_device.handle if execute_device else None
        self.api.call("LoadedExecutable_Execute", a)
        res = []
        for d in range(nd):
            outs = [Buffer(self.client, out_rows[d][o]) for o in range(num_outputs)]
            res.append(ExecutionDeviceOutputs(Event(self.api, events[d]), outs))
        return res

    def __del__(self):
        try:
            if self.handle and self.client.handle:
                a = A["LoadedExecutable_Destroy"](); a.executable = self.handle
                self.api.call("LoadedExecutable_Destroy", a)
                self.handle = None
        except Exception:
            pass


class _AbiVersion:
    """Common part of `RuntimeAbiVersion` and `ExecutableAbiVersion` (crates/ryft-pjrt/src/extensions/abi_version.rs:
    233-416): an owned handle of the ABI-version extension.  The extension's argument structs carry no
    `extension_start` field (abi_version.rs:525-752)."""

    # slots of PJRT_AbiVersion_Extension after the 24-byte base (abi_version.rs:754-769)
    (_CLIENT_RUNTIME, _EXECUTABLE, _RT_DESTROY, _RT_WITH_RUNTIME, _RT_WITH_EXECUTABLE, _RT_TO_PROTO, _RT_PLATFORM, _EX_DESTROY,
     _EX_TO_PROTO, _EX_PLATFORM, _RT_FROM_PROTO, _EX_FROM_PROTO) = range(12)
    _DESTROY_SLOT = _TO_PROTO_SLOT = _PLATFORM_SLOT = -1

    def __init__(self, api: "Api", handle: int):
        self.api, self.handle = api, handle

    @staticmethod
    def _struct(fields):
        return type("AbiArgs", (C.Structure,), {"_fields_": [("struct_size", _sz)] + list(fields)})()

    @staticmethod
    def _call(api: "Api", slot: int, args) -> None:
        ext = api.extension(EXTENSION_TYPE_ABI_VERSION)
        if not ext:
            raise PjrtError(12, "the plugin has no ABI-version extension")
        fp = C.c_void_p.from_address(ext + 24 + 8 * slot).value
        if not fp:
            raise PjrtError(12, "this function of the ABI-version extension is not implemented by the plugin")
        args.struct_size = C.sizeof(args)
        err = _FN(fp)(C.addressof(args))
        if err:
            raise api._take_error(err)

    def platform_id(self) -> int:
        a = self._struct([("abi_version", _vp), ("platform_id", C.c_uint64)]); a.abi_version = self.handle
        self._call(self.api, self._PLATFORM_SLOT, a)
        return a.platform_id

    def serialize(self) -> bytes:
        """The serialized `{1: platform, 2: version payload}` message (crates/ryft-xla-sys/src/protos.rs:3812-3838)."""
        a = self._struct([("abi_version", _vp), ("serialized_proto", _vp), ("serialized_proto_size", _sz), ("serialized_proto_holder", _vp),
                          ("serialized_proto_deleter", _vp)])
        a.abi_version = self.handle
        self._call(self.api, self._TO_PROTO_SLOT, a)
        data = C.string_at(a.serialized_proto, a.serialized_proto_size)
        if a.serialized_proto_deleter:
            C.CFUNCTYPE(None, _vp)(a.serialized_proto_deleter)(a.serialized_proto_holder)
        return data

    def proto(self) -> Dict[str, object]:
        """The message decoded into `{"platform": int, "version": bytes}`."""
        data, pos, out = self.serialize(), 0, {"platform": 0, "version": b""}

        def varint():
            nonlocal pos
            v = shift = 0
            while True:
                b = data[pos]; pos += 1
                v |= (b & 0x7F) << shift; shift += 7
                if not b & 0x80:
                    return v
        while pos < len(data):
            tag = varint()
            if tag == (1 << 3):
                out["platform"] = varint()
            elif tag == (2 << 3) | 2:
                n = varint(); out["version"] = data[pos:pos + n]; pos += n
            else:
                raise PjrtError(13, f"unexpected field tag {tag} in an ABI version message")
        return out

    def __eq__(self, other) -> bool:
        return type(other) is type(self) and self.serialize() == other.serialize()

    def __hash__(self) -> int:
        return hash(self.serialize())

    def __del__(self):
        if getattr(self, "handle", None):
            try:
                a = self._struct([("abi_version", _vp)]); a.abi_version = self.handle
                self._call(self.api, self._DESTROY_SLOT, a)
            except Exception:
                pass
            self.handle = None


class ExecutableAbiVersion(_AbiVersion):
    """`ExecutableAbiVersion` (crates/ryft-pjrt/src/extensions/abi_version.rs:339-416)."""
    _DESTROY_SLOT, _TO_PROTO_SLOT, _PLATFORM_SLOT = _AbiVersion._EX_DESTROY, _AbiVersion._EX_TO_PROTO, _AbiVersion._EX_PLATFORM

    @staticmethod
    def deserialize(api: "Api", data: bytes) -> "ExecutableAbiVersion":
        """`Api::deserialize_executable_abi_version` (abi_version.rs:212-230)."""
        buf = C.create_string_buffer(data, len(data))
        a = _AbiVersion._struct([("serialized_proto", _vp), ("serialized_proto_size", _sz), ("abi_version", _vp)])
        a.serialized_proto = C.cast(buf, _vp); a.serialized_proto_size = len(data)
        _AbiVersion._call(api, _AbiVersion._EX_FROM_PROTO, a)
        return ExecutableAbiVersion(api, a.abi_version)


class RuntimeAbiVersion(_AbiVersion):
    """`RuntimeAbiVersion` (crates/ryft-pjrt/src/extensions/abi_version.rs:233-336).  The compatibility checks return
    None and raise `PjrtError` when the versions do not fit, like the reference's `Result<(), Error>`."""
    _DESTROY_SLOT, _TO_PROTO_SLOT, _PLATFORM_SLOT = _AbiVersion._RT_DESTROY, _AbiVersion._RT_TO_PROTO, _AbiVersion._RT_PLATFORM

    @staticmethod
    def deserialize(api: "Api", data: bytes) -> "RuntimeAbiVersion":
        """`Api::deserialize_runtime_abi_version` (abi_version.rs:184-202)."""
        buf = C.create_string_buffer(data, len(data))
        a = _AbiVersion._struct([("serialized_proto", _vp), ("serialized_proto_size", _sz), ("abi_version", _vp)])
        a.serialized_proto = C.cast(buf, _vp); a.serialized_proto_size = len(data)
        _AbiVersion._call(api, _AbiVersion._RT_FROM_PROTO, a)
        return RuntimeAbiVersion(api, a.abi_version)

    def is_compatible_with_runtime(self, other: "RuntimeAbiVersion") -> None:
        a = self._struct([("abi_version", _vp), ("other_abi_version", _vp)]); a.abi_version = self.handle; a.other_abi_version = other.handle
        self._call(self.api, self._RT_WITH_RUNTIME, a)

    def is_compatible_with_executable(self, other: ExecutableAbiVersion) -> None:
        a = self._struct([("abi_version", _vp), ("executable_abi_version", _vp)]); a.abi_version = self.handle
        a.executable_abi_version = other.handle
        self._call(self.api, self._RT_WITH_EXECUTABLE, a)


class Layout:
    """`Layout` of the layouts extension (crates/ryft-pjrt/src/extensions/layouts.rs:94-190): an opaque memory layout
    handle that renders as its minor-to-major order, e.g. "{2,1,0}".  Borrowed layouts (those an executable lends out)
    are not destroyed."""

    # slots of PJRT_Layouts_Extension after the 24-byte base (layouts.rs:798-807)
    _DESTROY, _SERIALIZE, _CLIENT_DEFAULT, _BUFFER, _TOPOLOGY_DEFAULT, _EXE_OUTPUTS, _EXE_PARAMETERS = range(7)

    def __init__(self, api: "Api", handle: int, borrowed: bool):
        self.api, self.handle, self.borrowed = api, handle, borrowed

    @staticmethod
    def _fn(api: "Api", slot: int):
        ext = api.extension(EXTENSION_TYPE_LAYOUTS)
        if not ext:
            raise PjrtError(12, "the plugin has no layouts extension")
        fp = C.c_void_p.from_address(ext + 24 + 8 * slot).value
        if not fp:
            raise PjrtError(12, "this function of the layouts extension is not implemented by the plugin")
        return _FN(fp)

    @staticmethod
    def _call(api: "Api", slot: int, args) -> None:
        args.struct_size = C.sizeof(args)
        err = Layout._fn(api, slot)(C.addressof(args))
        if err:
            raise api._take_error(err)

    def serialize(self) -> str:
        a = _args("LayoutSerialize", [("layout", _vp), ("serialized_bytes", _vp), ("serialized_bytes_size", _sz), ("serialized_layout", _vp),
                                      ("serialized_layout_deleter", _vp)])()
        a.layout = self.handle
        Layout._call(self.api, Layout._SERIALIZE, a)
        text = C.string_at(a.serialized_bytes, a.serialized_bytes_size).decode()
        if a.serialized_layout_deleter:
            C.CFUNCTYPE(None, _vp)(a.serialized_layout_deleter)(a.serialized_layout)
        return text

    def minor_to_major(self) -> List[int]:
        body = self.serialize().strip("{}").split(":")[0]
        return [int(x) for x in body.split(",")] if body else []

    def __str__(self) -> str:
        return self.serialize()

    def __repr__(self) -> str:
        return f"Layout[{self.serialize()}]"

    def __eq__(self, other) -> bool:
        return isinstance(other, Layout) and self.serialize() == other.serialize()

    def __del__(self):
        if not self.borrowed and self.handle:
            try:
                a = _args("LayoutDestroy", [("layout", _vp)])()
                a.layout = self.handle
                Layout._call(self.api, Layout._DESTROY, a)
            except Exception:
                pass
            self.handle = None


class HostToDeviceTransferManager:
    """`HostToDeviceTransferManager` (crates/ryft-pjrt/src/transfers.rs:39-349): device buffers created up front and
    filled later, chunk by chunk; a buffer becomes ready with its last chunk.  Host data passed to `transfer_data` /
    `transfer_literal` is kept alive by the returned event until the copy has read it."""

    def __init__(self, client: "Client", handle: int):
        self.client, self.api, self.handle = client, client.api, handle

    def _call(self, name: str, **fields):
        a = A[_TM + name](); a.transfer_manager = self.handle
        for k, v in fields.items():
            setattr(a, k, v)
        self.api.call(_TM + name, a)
        return a

    def device(self) -> "Device":
        return Device(self.client, self._call("Device").device_out)

    def buffer_count(self) -> int:
        return int(self._call("BufferCount").buffer_count)

    def buffer_on_device_size_in_bytes(self, index: int) -> int:
        return int(self._call("BufferSize", buffer_index=index).buffer_size)

    def retrieve_buffer(self, index: int) -> "Buffer":
        return Buffer(self.client, self._call("RetrieveBuffer", buffer_index=index).buffer_out)

    def transfer_data(self, index: int, data: bytes, offset: int, is_last_transfer: bool) -> "Event":
        buf = C.create_string_buffer(bytes(data), len(data))
        a = self._call("TransferData", buffer_index=index, data=C.addressof(buf), offset=offset, transfer_size=len(data), is_last_transfer=is_last_transfer)
        return Event(self.api, a.done_with_h2d_transfer, keep=buf)

    def transfer_literal(self, index: int, data: bytes, buffer_type: int, dims: Sequence[int]) -> "Event":
        buf = C.create_string_buffer(bytes(data), len(data))
        d = (_i64 * max(len(dims), 1))(*dims)
        a = self._call("TransferLiteral", buffer_index=index, data=C.addressof(buf), shape_dims=C.cast(d, C.POINTER(_i64)), shape_num_dims=len(dims),
                       shape_element_type=int(buffer_type))
        return Event(self.api, a.done_with_h2d_transfer, keep=(buf, d))

    def set_error(self, index: int, code: int, message: str) -> None:
        m = message.encode()
        self._call("SetBufferError", buffer_index=index, error_code=code, error_message=m, error_message_size=len(m))

    def add_metadata(self, metadata: Dict[str, object]) -> None:
        self._call("AddMetadata", transfer_metadata=None, num_metadata=0)   # the plugin has nothing to attach metadata to

    def close(self) -> None:
        if self.handle:
            self._call("Destroy")
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class KeyValueStore:
    """Interface of the store behind the client's kv callbacks (crates/ryft-pjrt/src/clients.rs:575-640)."""

    def get(self, key: str, timeout_ms: int) -> bytes: raise NotImplementedError
    def put(self, key: str, value: bytes) -> None: raise NotImplementedError


class DictKeyValueStore(KeyValueStore):
    """In-process store (the shape of the reference's TestKeyValueStore, crates/ryft-pjrt/src/clients.rs:1299-1322)."""

    def __init__(self):
        self._d: Dict[str, bytes] = {}
        self._cv = threading.Condition()

    def get(self, key, timeout_ms):
        with self._cv:
            if not self._cv.wait_for(lambda: key in self._d, timeout_ms / 1000.0):
                raise TimeoutError(key)
            return self._d[key]

    def put(self, key, value):
        with self._cv:
            self._d[key] = value
            self._cv.notify_all()


class TorchStoreKeyValueStore(KeyValueStore):
    """Backs the callbacks with a torch.distributed store (one process per GPU under torchrun)."""

    def __init__(self, store):
        self.store = store

    def get(self, key, timeout_ms):
        self.store.wait([key])
        return bytes(self.store.get(key))

    def put(self, key, value):
        self.store.set(key, value)


class KvCallbacks:
    """The two C callbacks `PJRT_Client_Create` takes for a distributed key-value store
    (`PJRT_KeyValueGetCallback` / `PJRT_KeyValuePutCallback`, crates/ryft-pjrt/src/clients.rs:849-964), backed by a
    `KeyValueStore`.  The plugin calls them from its own threads; a returned value stays alive until the plugin calls
    the deleter it was handed."""

    GET = _args("KvGet", [("key", _vp), ("key_size", _sz), ("timeout_in_ms", _i), ("callback_error", _vp), ("user_arg", _vp),
                           ("value", _vp), ("value_size", _sz), ("value_deleter_callback", _vp)])
    PUT = _args("KvPut", [("key", _vp), ("key_size", _sz), ("value", _vp), ("value_size", _sz), ("callback_error", _vp), ("user_arg", _vp)])

    def __init__(self, store: KeyValueStore):
        self.store = store
        self.live = {}

        def deleter(ptr):
            self.live.pop(ptr, None)
        self._deleter = C.CFUNCTYPE(None, _vp)(deleter)

        def kv_get(p):
            g = KvCallbacks.GET.from_address(p)
            val = store.get(_str(g.key, g.key_size), g.timeout_in_ms)
            buf = C.create_string_buffer(val, len(val))
            addr = C.addressof(buf)
            self.live[addr] = buf
            g.value = addr; g.value_size = len(val); g.value_deleter_callback = C.cast(self._deleter, _vp)
            return None

        def kv_put(p):
            g = KvCallbacks.PUT.from_address(p)
            store.put(_str(g.key, g.key_size), C.string_at(g.value, g.value_size))
            return None
        self._get = C.CFUNCTYPE(_vp, _vp)(kv_get)
        self._put = C.CFUNCTYPE(_vp, _vp)(kv_put)
        self.get_ptr = C.cast(self._get, _vp)
        self.put_ptr = C.cast(self._put, _vp)


class Client:
    """`Client` (crates/ryft-pjrt/src/clients.rs)."""

    def __init__(self, plugin: "Plugin", options: Optional[Dict[str, object]] = None, kv_store: Optional[KeyValueStore] = None):
        self.plugin, self.api = plugin, plugin.api
        self.handle = None
        options = options or {}
        nvs = (NamedValueC * max(len(options), 1))()
        self._keep = []
        for i, (k, v) in enumerate(options.items()):
            nv = nvs[i]
            nv.struct_size = C.sizeof(NamedValueC)
            kb = k.encode(); kbuf = C.create_string_buffer(kb); self._keep.append(kbuf)
            nv.name = C.cast(kbuf, _vp); nv.name_size = len(kb)
            if isinstance(v, bool):
                nv.type = 4; nv.value.bool_value = v; nv.value_size = 1
            elif isinstance(v, int):
                nv.type = 1; nv.value.int64_value = v; nv.value_size = 1
            elif isinstance(v, float):
                nv.type = 3; nv.value.float_value = v; nv.value_size = 1
            elif isinstance(v, str):
                vb = C.create_string_buffer(v.encode()); self._keep.append(vb)
                nv.type = 0; nv.value.string_value = C.cast(vb, _vp); nv.value_size = len(v.encode())
            else:
                arr = (_i64 * len(v))(*v); self._keep.append(arr)
                nv.type = 2; nv.value.int64_array_value = C.cast(arr, C.POINTER(_i64)); nv.value_size = len(v)
        a = A["Client_Create"]()
        a.create_options = C.cast(nvs, C.POINTER(NamedValueC)); a.num_options = len(options)
        if kv_store is not None:
            self._install_kv(a, kv_store)
        self.api.call("Client_Create", a)
        self.handle = a.client

    def _install_kv(self, a, store: KeyValueStore):
        self._kv = KvCallbacks(store)
        a.kv_get_callback = self._kv.get_ptr
        a.kv_put_callback = self._kv.put_ptr

    def abi_version(self) -> "RuntimeAbiVersion":
        """`Client::abi_version` (crates/ryft-pjrt/src/extensions/abi_version.rs:72-83)."""
        a = _AbiVersion._struct([("client", _vp), ("abi_version", _vp)]); a.client = self.handle
        _AbiVersion._call(self.api, _AbiVersion._CLIENT_RUNTIME, a)
        return RuntimeAbiVersion(self.api, a.abi_version)

    def default_layout(self, element_type: int, dims) -> "Layout":
        """`Client::default_layout` (crates/ryft-pjrt/src/extensions/layouts.rs:198-219)."""
        arr = (_i64 * max(len(dims), 1))(*dims)
        a = _args("LayoutClientDefault", [("client", _vp), ("element_type", _i), ("dims", _vp), ("num_dims", _sz), ("layout", _vp)])()
        a.client = self.handle; a.element_type = int(element_type); a.dims = C.cast(arr, _vp); a.num_dims = len(dims)
        Layout._call(self.api, Layout._CLIENT_DEFAULT, a)
        return Layout(self.api, a.layout, borrowed=False)

    def platform_name(self) -> str:
        a = A["Client_PlatformName"](); a.client = self.handle
        self.api.call("Client_PlatformName", a); return _str(a.platform_name, a.platform_name_size)

    def platform_version(self) -> str:
        a = A["Client_PlatformVersion"](); a.client = self.handle
        self.api.call("Client_PlatformVersion", a); return _str(a.platform_version, a.platform_version_size)

    def process_index(self) -> int:
        a = A["Client_ProcessIndex"](); a.client = self.handle
        self.api.call("Client_ProcessIndex", a); return int(a.process_index)

    def devices(self) -> List[Device]:
        a = A["Client_Devices"](); a.client = self.handle
        self.api.call("Client_Devices", a)
        return [Device(self, a.devices[i]) for i in range(a.num_devices)]

    def addressable_devices(self) -> List[Device]:
        a = A["Client_AddressableDevices"](); a.client = self.handle
        self.api.call("Client_AddressableDevices", a)
        return [Device(self, a.addressable_devices[i]) for i in range(a.num_addressable_devices)]

    def lookup_device(self, device_id: int) -> Device:
        a = A["Client_LookupDevice"](); a.client = self.handle; a.id = device_id
        self.api.call("Client_LookupDevice", a)
        return Device(self, a.device)

    def default_device_assignment(self, num_replicas: int, num_partitions: int) -> List[int]:
        n = num_replicas * num_partitions
        out = (_i * max(n, 1))()
        a = A["Client_DefaultDeviceAssignment"](); a.client = self.handle; a.num_replicas = num_replicas; a.num_partitions = num_partitions
        a.default_assignment_size = n; a.default_assignment = C.cast(out, C.POINTER(_i))
        self.api.call("Client_DefaultDeviceAssignment", a)
        return [int(out[i]) for i in range(n)]

    def compile(self, program: Program, options: Optional[CompilationOptions] = None) -> LoadedExecutable:
        """`Client::compile` (crates/ryft-pjrt/src/programs.rs:1245-1263)."""
        options = options or CompilationOptions()
        code = C.create_string_buffer(program.code, len(program.code))
        fmt = program.format.encode()
        fbuf = C.create_string_buffer(fmt, len(fmt))
        p = ProgramC(); p.struct_size = C.sizeof(p)
        p.code = C.addressof(code); p.code_size = len(program.code); p.format = C.addressof(fbuf); p.format_size = len(fmt)
        opts = options.encode()
        obuf = C.create_string_buffer(opts, len(opts))
        a = A["Client_Compile"](); a.client = self.handle; a.program = C.addressof(p)
        a.compile_options = C.addressof(obuf); a.compile_options_size = len(opts)
        self.api.call("Client_Compile", a)
        return LoadedExecutable(self, a.executable)

    def deserialize_and_load(self, data: bytes) -> LoadedExecutable:
        buf = C.create_string_buffer(data, len(data))
        a = A["Executable_DeserializeAndLoad"](); a.client = self.handle
        a.serialized_executable = C.addressof(buf); a.serialized_executable_size = len(data)
        self.api.call("Executable_DeserializeAndLoad", a)
        return LoadedExecutable(self, a.loaded_executable)

    def buffer(self, data, buffer_type: Optional[BufferType] = None, dims: Optional[Sequence[int]] = None, device: Optional[Device] = None,
               semantics: int = 0, byte_strides: Optional[Sequence[int]] = None) -> Buffer:
        """`Client::buffer` (crates/ryft-pjrt/src/buffers.rs:2099-2150): device = NULL, memory = the device's default
        memory, host semantics kImmutableOnlyDuringCall for borrowed bytes.  `data` is bytes, a numpy array, or an
        integer host address paired with `nbytes` semantics through a numpy/torch array's pointer."""
        keep = None
        if isinstance(data, np.ndarray):
            arr = data if (byte_strides is not None or data.flags.c_contiguous) else data.copy(order="C")
            keep = arr
            ptr = arr.ctypes.data
            if buffer_type is None: buffer_type = _np_to_buffer_type(arr.dtype)
            if dims is None: dims = arr.shape
        elif isinstance(data, (bytes, bytearray)):
            keep = C.create_string_buffer(bytes(data), len(data))
            ptr = C.addressof(keep)
        else:
            ptr = int(data)
        assert buffer_type is not None and dims is not None
        device = device or self.addressable_devices()[0]
        d = (_i64 * max(len(dims), 1))(*dims)
        a = A["Client_BufferFromHostBuffer"]()
        a.client = self.handle; a.data = ptr; a.type = int(buffer_type)
        a.dims = C.cast(d, C.POINTER(_i64)); a.num_dims = len(dims)
        if byte_strides is not None:
            s = (_i64 * max(len(byte_strides), 1))(*byte_strides)
            a.byte_strides = C.cast(s, C.POINTER(_i64)); a.num_byte_strides = len(byte_strides)
        a.host_buffer_semantics = semantics
        a.device = None; a.memory = device.default_memory()
        self.api.call("Client_BufferFromHostBuffer", a)
        done = Event(self.api, a.done_with_host_buffer)
        buf = Buffer(self, a.buffer, keep=keep if semantics != 0 else None)
        buf.done_with_host_buffer = done
        return buf

    def view_of_device_buffer(self, ptr: int, buffer_type: BufferType, dims: Sequence[int], device: Optional[Device] = None, stream: int = 0, keep=None) -> Buffer:
        """`Client::borrowed_on_device_buffer` (crates/ryft-pjrt/src/buffers.rs:2285-2319): zero-copy import."""
        device = device or self.addressable_devices()[0]
        d = (_i64 * max(len(dims), 1))(*dims)
        a = A["Client_CreateViewOfDeviceBuffer"]()
        a.client = self.handle; a.device_buffer_ptr = ptr; a.dims = C.cast(d, C.POINTER(_i64)); a.num_dims = len(dims)
        a.element_type = int(buffer_type); a.device = device.handle; a.stream = stream
        self.api.call("Client_CreateViewOfDeviceBuffer", a)
        return Buffer(self, a.buffer, keep=keep)

    def host_to_device_transfer_manager(self, specifications: Sequence[tuple], device: Optional[Device] = None) -> "HostToDeviceTransferManager":
        """`Client::host_to_device_transfer_manager` (crates/ryft-pjrt/src/transfers.rs:351-420); `specifications` are
        (buffer type, dims) pairs, the buffers are created in `device`'s default memory."""
        device = device or self.addressable_devices()[0]
        specs = (ShapeSpecC * max(len(specifications), 1))()
        keep = []
        for i, (bt, dims) in enumerate(specifications):
            d = (_i64 * max(len(dims), 1))(*dims); keep.append(d)
            specs[i].struct_size = C.sizeof(ShapeSpecC); specs[i].dims = C.cast(d, C.POINTER(_i64)); specs[i].num_dims = len(dims); specs[i].element_type = int(bt)
        a = A["Client_CreateBuffersForAsyncHostToDevice"](); a.client = self.handle
        a.shape_specs = C.cast(specs, C.POINTER(ShapeSpecC)); a.num_shape_specs = len(specifications); a.memory = device.default_memory()
        self.api.call("Client_CreateBuffersForAsyncHostToDevice", a)
        return HostToDeviceTransferManager(self, a.transfer_manager)

    def error_buffer(self, code: int, message: str, buffer_type: BufferType, dims: Sequence[int], device: Optional[Device] = None) -> Buffer:
        device = device or self.addressable_devices()[0]
        d = (_i64 * max(len(dims), 1))(*dims)
        m = message.encode()
        a = A["Client_CreateErrorBuffer"](); a.client = self.handle; a.error_code = code; a.error_message = m; a.error_message_size = len(m)
        a.shape_dims = C.cast(d, C.POINTER(_i64)); a.shape_num_dims = len(dims); a.shape_element_type = int(buffer_type)
        a.memory = device.default_memory()
        self.api.call("Client_CreateErrorBuffer", a)
        return Buffer(self, a.buffer)

    def close(self) -> None:
        if self.handle:
            a = A["Client_Destroy"](); a.client = self.handle
            self.handle = None
            self.api.call("Client_Destroy", a)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Plugin:
    """`Plugin` (crates/ryft-pjrt/src/plugins.rs:14-60)."""

    def __init__(self, path: os.PathLike):
        self.path = str(path)
        if not Path(self.path).exists():
            raise FileNotFoundError(
                f"{self.path} is missing: build the native library first (python -m ryft_b200.build); there is no fallback")
        self.lib = C.CDLL(self.path, mode=C.RTLD_LOCAL)
        get = self.lib.GetPjrtApi
        get.restype = _vp
        self.api = Api(get())
        self.api.call("Plugin_Initialize", A["Plugin_Initialize"]())

    def version(self): return self.api.version

    def attributes(self) -> Dict[str, object]:
        a = A["Plugin_Attributes"]()
        self.api.call("Plugin_Attributes", a)
        return _named_values(a.attributes, a.num_attributes)

    def attribute(self, name: str):
        attrs = self.attributes()
        if name not in attrs:
            raise PjrtError(5, f"no plugin attribute named '{name}'")
        return attrs[name]

    def client(self, options: Optional[Dict[str, object]] = None, kv_store: Optional[KeyValueStore] = None) -> Client:
        return Client(self, options, kv_store)


_PLUGINS: Dict[str, Plugin] = {}
_PLUGINS_LOCK = threading.Lock()


def load_plugin(path: os.PathLike) -> Plugin:
    """`load_plugin` (crates/ryft-pjrt/src/plugins.rs:120-122): plugins are cached by canonical path."""
    key = str(Path(path).resolve())
    with _PLUGINS_LOCK:
        if key not in _PLUGINS:
            _PLUGINS[key] = Plugin(key)
        return _PLUGINS[key]


def load_cuda_13_plugin() -> Plugin:
    """`load_cuda_13_plugin` (crates/ryft-pjrt/src/plugins.rs:138-141), resolved to the in-tree build."""
    return load_plugin(os.environ.get("PJRT_PLUGIN_CUDA_13_LIB", str(_DEFAULT_PLUGIN)))
