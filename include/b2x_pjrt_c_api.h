/*
 * PJRT C API surface (version 0.104) served by the B200 StableHLO executor plugin.
 *
 * The plugin is a shared library whose single exported symbol is `GetPjrtApi`
 * (reference: crates/ryft-pjrt/src/plugins.rs:67-79 resolves exactly that symbol;
 * crates/ryft-xla-sys/pjrt_plugin_version_script.lds:1-7 is the export list).
 * Every layout below is laid out field for field after the `#[repr(C)]`
 * definitions in the reference's `ffi` modules, which are the only layout
 * source available (the upstream C header is not part of the reference tree).
 * Each group names the reference file and line of the definition it mirrors.
 *
 * Conventions (crates/ryft-pjrt/src/macros.rs:27-108):
 *   - every `*_Args` starts with `struct_size` and `extension_start`;
 *   - every function returns `PJRT_Error*` (NULL = success) except
 *     `PJRT_Error_Destroy` and `PJRT_Error_Message`, which return void;
 *   - a NULL function pointer, or one beyond `PJRT_Api::struct_size`, means
 *     "unimplemented" to the caller.
 */
#ifndef B2X_PJRT_C_API_H_
#define B2X_PJRT_C_API_H_

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PJRT_API_MAJOR 0   /* crates/ryft-pjrt/src/versions.rs:33 */
#define PJRT_API_MINOR 104 /* crates/ryft-pjrt/src/versions.rs:34 */

/* ---- base types: crates/ryft-pjrt/src/lib.rs:179-212 ---------------------------------- */
typedef unsigned int PJRT_Extension_Type;
typedef struct PJRT_Extension_Base {
  size_t struct_size;
  PJRT_Extension_Type extension_type;
  struct PJRT_Extension_Base* next;
} PJRT_Extension_Base;

/* crates/ryft-pjrt/src/versions.rs:36-48 */
typedef struct PJRT_Api_Version {
  size_t struct_size;
  PJRT_Extension_Base* extension_start;
  int major_version;
  int minor_version;
} PJRT_Api_Version;

/* Opaque handles. */
typedef struct PJRT_Error PJRT_Error;
typedef struct PJRT_Event PJRT_Event;
typedef struct PJRT_Client PJRT_Client;
typedef struct PJRT_Device PJRT_Device;
typedef struct PJRT_DeviceDescription PJRT_DeviceDescription;
typedef struct PJRT_Memory PJRT_Memory;
typedef struct PJRT_Buffer PJRT_Buffer;
typedef struct PJRT_Executable PJRT_Executable;
typedef struct PJRT_LoadedExecutable PJRT_LoadedExecutable;
typedef struct PJRT_ExecuteContext PJRT_ExecuteContext;
typedef struct PJRT_TopologyDescription PJRT_TopologyDescription;
typedef struct PJRT_SerializedExecutable PJRT_SerializedExecutable;
typedef struct PJRT_SerializedCompileOptions PJRT_SerializedCompileOptions;
typedef struct PJRT_DeviceAssignmentSerialized PJRT_DeviceAssignmentSerialized;
typedef struct PJRT_Device_Attributes PJRT_Device_Attributes;
typedef struct PJRT_AsyncTrackingEvent PJRT_AsyncTrackingEvent;
typedef struct PJRT_MultiSlice_Config PJRT_MultiSlice_Config;

/* ---- named values: crates/ryft-pjrt/src/values.rs:214-259 ------------------------------ */
typedef unsigned int PJRT_NamedValue_Type;
enum {
  PJRT_NamedValue_kString = 0,
  PJRT_NamedValue_kInt64 = 1,
  PJRT_NamedValue_kInt64List = 2,
  PJRT_NamedValue_kFloat = 3,
  PJRT_NamedValue_kBool = 4
};
typedef struct PJRT_NamedValue {
  size_t struct_size;
  PJRT_Extension_Base* extension_start;
  const char* name;
  size_t name_size;
  PJRT_NamedValue_Type type;
  union {
    const char* string_value;
    int64_t int64_value;
    const int64_t* int64_array_value;
    float float_value;
    bool bool_value;
  };
  size_t value_size; /* element count for strings and lists, 1 otherwise */
} PJRT_NamedValue;

/* ---- errors: crates/ryft-pjrt/src/errors.rs:417-526 ------------------------------------ */
typedef unsigned int PJRT_Error_Code; /* absl codes 0..16, errors.rs:440-457 */
enum {
  PJRT_Error_Code_OK = 0,
  PJRT_Error_Code_CANCELLED = 1,
  PJRT_Error_Code_UNKNOWN = 2,
  PJRT_Error_Code_INVALID_ARGUMENT = 3,
  PJRT_Error_Code_DEADLINE_EXCEEDED = 4,
  PJRT_Error_Code_NOT_FOUND = 5,
  PJRT_Error_Code_ALREADY_EXISTS = 6,
  PJRT_Error_Code_PERMISSION_DENIED = 7,
  PJRT_Error_Code_RESOURCE_EXHAUSTED = 8,
  PJRT_Error_Code_FAILED_PRECONDITION = 9,
  PJRT_Error_Code_ABORTED = 10,
  PJRT_Error_Code_OUT_OF_RANGE = 11,
  PJRT_Error_Code_UNIMPLEMENTED = 12,
  PJRT_Error_Code_INTERNAL = 13,
  PJRT_Error_Code_UNAVAILABLE = 14,
  PJRT_Error_Code_DATA_LOSS = 15,
  PJRT_Error_Code_UNAUTHENTICATED = 16
};
typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_Error* error; } PJRT_Error_Destroy_Args;
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  const PJRT_Error* error; const char* message; size_t message_size; /* out, borrowed */
} PJRT_Error_Message_Args;
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  const PJRT_Error* error; PJRT_Error_Code code; /* out */
} PJRT_Error_GetCode_Args;
typedef void (*PJRT_Error_PayloadVisitor)(const char* key, size_t key_size, const char* value, size_t value_size,
                                          void* user_arg);
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  const PJRT_Error* error; PJRT_Error_PayloadVisitor visitor; void* user_arg;
} PJRT_Error_ForEachPayload_Args;
/* Passed to caller-supplied callbacks so that they can hand a PJRT_Error back (errors.rs:522-526). */
typedef PJRT_Error* (*PJRT_CallbackError)(PJRT_Error_Code code, const char* message, size_t message_size);

/* ---- plugin: crates/ryft-pjrt/src/plugins.rs:178-205 ----------------------------------- */
typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; } PJRT_Plugin_Initialize_Args;
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  const PJRT_NamedValue* attributes; size_t num_attributes; /* out, borrowed */
} PJRT_Plugin_Attributes_Args;

/* ---- events: crates/ryft-pjrt/src/events.rs:380-506 ------------------------------------ */
typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_Event* event; } PJRT_Event_Create_Args;
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  PJRT_Event* event; PJRT_Error_Code error_code; const char* error_message; size_t error_message_size;
} PJRT_Event_Set_Args;
typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_Event* event; bool is_ready; } PJRT_Event_IsReady_Args;
/* The callback takes ownership of `error` (events.rs:100-108) and may run on any plugin thread. */
typedef void (*PJRT_Event_OnReadyCallback)(PJRT_Error* error, void* user_arg);
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  PJRT_Event* event; PJRT_Event_OnReadyCallback callback; void* user_arg;
} PJRT_Event_OnReady_Args;
typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_Event* event; } PJRT_Event_Await_Args;
typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_Event* event; } PJRT_Event_Error_Args;
typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_Event* event; } PJRT_Event_Destroy_Args;

/* ---- client: crates/ryft-pjrt/src/clients.rs:841-1275 ---------------------------------- */
typedef void (*PJRT_KeyValue_ValueDeleter)(char* value);
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  const char* key; size_t key_size; int timeout_in_ms;
  PJRT_CallbackError* callback_error; void* user_arg;
  char* value; size_t value_size; PJRT_KeyValue_ValueDeleter value_deleter_callback; /* out */
} PJRT_KeyValueGetCallback_Args;
typedef PJRT_Error* (*PJRT_KeyValueGetCallback)(PJRT_KeyValueGetCallback_Args* args);
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  const char* key; size_t key_size;
  PJRT_CallbackError* callback_error; void* user_arg;
  char* value; size_t value_size; PJRT_KeyValue_ValueDeleter value_deleter_callback; /* out */
} PJRT_KeyValueTryGetCallback_Args;
typedef PJRT_Error* (*PJRT_KeyValueTryGetCallback)(PJRT_KeyValueTryGetCallback_Args* args);
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  const char* key; size_t key_size; const char* value; size_t value_size;
  PJRT_CallbackError* callback_error; void* user_arg;
} PJRT_KeyValuePutCallback_Args;
typedef PJRT_Error* (*PJRT_KeyValuePutCallback)(PJRT_KeyValuePutCallback_Args* args);

typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  const PJRT_NamedValue* create_options; size_t num_options;
  PJRT_KeyValueGetCallback kv_get_callback; void* kv_get_user_arg;
  PJRT_KeyValuePutCallback kv_put_callback; void* kv_put_user_arg;
  PJRT_Client* client; /* out */
  PJRT_KeyValueTryGetCallback kv_try_get_callback; void* kv_try_get_user_arg;
} PJRT_Client_Create_Args;
typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_Client* client; } PJRT_Client_Destroy_Args;
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  PJRT_Client* client; const char* platform_name; size_t platform_name_size;
} PJRT_Client_PlatformName_Args;
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  PJRT_Client* client; const char* platform_version; size_t platform_version_size;
} PJRT_Client_PlatformVersion_Args;
typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_Client* client; int process_index; } PJRT_Client_ProcessIndex_Args;
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  PJRT_Client* client; PJRT_Device* const* devices; size_t num_devices;
} PJRT_Client_Devices_Args;
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  PJRT_Client* client; PJRT_Device* const* addressable_devices; size_t num_addressable_devices;
} PJRT_Client_AddressableDevices_Args;
typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_Client* client; int id; PJRT_Device* device; } PJRT_Client_LookupDevice_Args;
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  PJRT_Client* client; int local_hardware_id; PJRT_Device* addressable_device;
} PJRT_Client_LookupAddressableDevice_Args;
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  PJRT_Client* client; PJRT_Memory* const* addressable_memories; size_t num_addressable_memories;
} PJRT_Client_AddressableMemories_Args;
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  PJRT_Client* client; int num_replicas; int num_partitions;
  size_t default_assignment_size; int* default_assignment; /* caller-allocated, replica-major */
} PJRT_Client_DefaultDeviceAssignment_Args;
typedef unsigned int PJRT_ProcessState;
typedef struct {
  size_t struct_size; int task_id; uint64_t incarnation_id; PJRT_ProcessState state;
  int error_code; const char* error_message; size_t error_message_size;
} PJRT_ProcessInfo;
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  PJRT_Client* client; PJRT_ProcessInfo* process_infos; size_t num_process_infos;
} PJRT_Client_UpdateGlobalProcessInfo_Args;

/* ---- devices and descriptions: crates/ryft-pjrt/src/devices.rs:777-1170 ---------------- */
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  PJRT_Device* device; PJRT_DeviceDescription* device_description;
} PJRT_Device_GetDescription_Args;
typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_Device* device; bool is_addressable; } PJRT_Device_IsAddressable_Args;
typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_Device* device; int local_hardware_id; } PJRT_Device_LocalHardwareId_Args;
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  PJRT_Device* device; PJRT_Memory* const* memories; size_t num_memories;
} PJRT_Device_AddressableMemories_Args;
typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_Device* device; PJRT_Memory* memory; } PJRT_Device_DefaultMemory_Args;
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  PJRT_Device* device;
  int64_t bytes_in_use;
  int64_t peak_bytes_in_use; bool peak_bytes_in_use_is_set;
  int64_t num_allocs; bool num_allocs_is_set;
  int64_t largest_alloc_size; bool largest_alloc_size_is_set;
  int64_t bytes_limit; bool bytes_limit_is_set;
  int64_t bytes_reserved; bool bytes_reserved_is_set;
  int64_t peak_bytes_reserved; bool peak_bytes_reserved_is_set;
  int64_t bytes_reservable_limit; bool bytes_reservable_limit_is_set;
  int64_t largest_free_block_bytes; bool largest_free_block_bytes_is_set;
  int64_t pool_bytes; bool pool_bytes_is_set;
  int64_t peak_pool_bytes; bool peak_pool_bytes_is_set;
} PJRT_Device_MemoryStats_Args;
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  PJRT_Device* device; const PJRT_NamedValue* attributes; size_t num_attributes;
  PJRT_Device_Attributes* device_attributes; void (*attributes_deleter)(PJRT_Device_Attributes*);
} PJRT_Device_GetAttributes_Args;
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  PJRT_Device* device; int32_t launch_id; PJRT_Error_Code error_code;
  const char* error_message; size_t error_message_size; bool poisoned; /* out */
  const PJRT_NamedValue* payload; size_t payload_size;
} PJRT_Device_PoisonExecution_Args;
typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_DeviceDescription* device_description; int id; } PJRT_DeviceDescription_Id_Args;
typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_DeviceDescription* device_description; int process_index; } PJRT_DeviceDescription_ProcessIndex_Args;
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  PJRT_DeviceDescription* device_description; size_t num_attributes; const PJRT_NamedValue* attributes;
} PJRT_DeviceDescription_Attributes_Args;
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  PJRT_DeviceDescription* device_description; const char* device_kind; size_t device_kind_size;
} PJRT_DeviceDescription_Kind_Args;
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  PJRT_DeviceDescription* device_description; const char* debug_string; size_t debug_string_size;
} PJRT_DeviceDescription_DebugString_Args;
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  PJRT_DeviceDescription* device_description; const char* to_string; size_t to_string_size;
} PJRT_DeviceDescription_ToString_Args;

/* ---- memories: crates/ryft-pjrt/src/memories.rs:205-335 -------------------------------- */
typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_Memory* memory; int id; } PJRT_Memory_Id_Args;
typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_Memory* memory; int kind_id; } PJRT_Memory_Kind_Id_Args;
typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_Memory* memory; const char* kind; size_t kind_size; } PJRT_Memory_Kind_Args;
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  PJRT_Memory* memory; PJRT_Device* const* devices; size_t num_devices;
} PJRT_Memory_AddressableByDevices_Args;
typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_Memory* memory; const char* to_string; size_t to_string_size; } PJRT_Memory_ToString_Args;
typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_Memory* memory; const char* debug_string; size_t debug_string_size; } PJRT_Memory_DebugString_Args;

/* ---- buffers: crates/ryft-pjrt/src/buffers.rs:2568-3590 -------------------------------- */
typedef unsigned int PJRT_Buffer_Type; /* buffers.rs:2568-2600 */
enum {
  PJRT_Buffer_Type_INVALID = 0, PJRT_Buffer_Type_PRED = 1, PJRT_Buffer_Type_S8 = 2, PJRT_Buffer_Type_S16 = 3,
  PJRT_Buffer_Type_S32 = 4, PJRT_Buffer_Type_S64 = 5, PJRT_Buffer_Type_U8 = 6, PJRT_Buffer_Type_U16 = 7,
  PJRT_Buffer_Type_U32 = 8, PJRT_Buffer_Type_U64 = 9, PJRT_Buffer_Type_F16 = 10, PJRT_Buffer_Type_F32 = 11,
  PJRT_Buffer_Type_F64 = 12, PJRT_Buffer_Type_BF16 = 13, PJRT_Buffer_Type_C64 = 14, PJRT_Buffer_Type_C128 = 15,
  PJRT_Buffer_Type_TOKEN = 23
};
typedef unsigned int PJRT_Buffer_MemoryLayout_Type;
enum { PJRT_Buffer_MemoryLayout_Type_Tiled = 0, PJRT_Buffer_MemoryLayout_Type_Strides = 1 };
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  const int64_t* minor_to_major; size_t minor_to_major_size;
  const int64_t* tile_dims; const size_t* tile_dim_sizes; size_t num_tiles;
} PJRT_Buffer_MemoryLayout_Tiled;
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  const int64_t* byte_strides; size_t num_byte_strides;
} PJRT_Buffer_MemoryLayout_Strides;
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  union { PJRT_Buffer_MemoryLayout_Tiled tiled; PJRT_Buffer_MemoryLayout_Strides strides; };
  PJRT_Buffer_MemoryLayout_Type type;
} PJRT_Buffer_MemoryLayout;
typedef unsigned int PJRT_HostBufferSemantics; /* buffers.rs:3250-3254 */
enum {
  PJRT_HostBufferSemantics_kImmutableOnlyDuringCall = 0,
  PJRT_HostBufferSemantics_kImmutableUntilTransferCompletes = 1,
  PJRT_HostBufferSemantics_kImmutableZeroCopy = 2,
  PJRT_HostBufferSemantics_kMutableZeroCopy = 3
};
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  PJRT_Client* client; const void* data; PJRT_Buffer_Type type;
  const int64_t* dims; size_t num_dims;
  const int64_t* byte_strides; size_t num_byte_strides; /* NULL => dense major-to-minor */
  PJRT_HostBufferSemantics host_buffer_semantics;
  PJRT_Device* device; PJRT_Memory* memory; /* ryft passes device == NULL and a memory (buffers.rs:2113-2133) */
  PJRT_Buffer_MemoryLayout* device_layout;
  PJRT_Event* done_with_host_buffer; PJRT_Buffer* buffer; /* out */
} PJRT_Client_BufferFromHostBuffer_Args;
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  PJRT_Client* client; const int64_t* shape_dims; size_t shape_num_dims; PJRT_Buffer_Type shape_element_type;
  PJRT_Buffer_MemoryLayout* shape_layout; PJRT_Device* device; PJRT_Memory* memory; PJRT_Buffer* buffer; /* out */
} PJRT_Client_CreateUninitializedBuffer_Args;
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  PJRT_Client* client; void* device_buffer_ptr; const int64_t* dims; size_t num_dims; PJRT_Buffer_Type element_type;
  PJRT_Buffer_MemoryLayout* layout; PJRT_Device* device;
  void (*on_delete_callback)(void* device_buffer_ptr, void* user_arg); void* on_delete_callback_arg;
  intptr_t stream; PJRT_Buffer* buffer; /* out */ PJRT_Memory* memory;
} PJRT_Client_CreateViewOfDeviceBuffer_Args;
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  PJRT_Client* client; PJRT_Error_Code error_code; const char* error_message; size_t error_message_size;
  const int64_t* shape_dims; size_t shape_num_dims; PJRT_Buffer_Type shape_element_type;
  PJRT_Buffer_MemoryLayout* shape_layout; PJRT_Memory* memory; PJRT_Buffer* buffer; /* out */
  const PJRT_NamedValue* payload; size_t payload_size;
} PJRT_Client_CreateErrorBuffer_Args;
typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_Client* client; void* data; size_t size; } PJRT_Client_DmaMap_Args;
typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_Client* client; void* data; } PJRT_Client_DmaUnmap_Args;

typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_Buffer* buffer; } PJRT_Buffer_Destroy_Args;
typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_Buffer* buffer; PJRT_Buffer_Type type; } PJRT_Buffer_ElementType_Args;
typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_Buffer* buffer; const int64_t* dims; size_t num_dims; } PJRT_Buffer_Dimensions_Args;
typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_Buffer* buffer; const int64_t* unpadded_dims; size_t num_dims; } PJRT_Buffer_UnpaddedDimensions_Args;
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  PJRT_Buffer* buffer; const size_t* dynamic_dim_indices; size_t num_dynamic_dims;
} PJRT_Buffer_DynamicDimensionIndices_Args;
typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_Buffer* buffer; PJRT_Buffer_MemoryLayout layout; } PJRT_Buffer_GetMemoryLayout_Args;
typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_Buffer* buffer; size_t on_device_size_in_bytes; } PJRT_Buffer_OnDeviceSizeInBytes_Args;
typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_Buffer* buffer; PJRT_Device* device; } PJRT_Buffer_Device_Args;
typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_Buffer* buffer; PJRT_Memory* memory; } PJRT_Buffer_Memory_Args;
typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_Buffer* buffer; } PJRT_Buffer_Delete_Args;
typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_Buffer* buffer; bool is_deleted; } PJRT_Buffer_IsDeleted_Args;
typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_Buffer* buffer; PJRT_Device* dst_device; PJRT_Buffer* dst_buffer; } PJRT_Buffer_CopyToDevice_Args;
typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_Buffer* buffer; PJRT_Memory* dst_memory; PJRT_Buffer* dst_buffer; } PJRT_Buffer_CopyToMemory_Args;
/* Two-call protocol (buffers.rs:1237-1295): dst == NULL => only dst_size is written. */
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  PJRT_Buffer* src; PJRT_Buffer_MemoryLayout* host_layout; void* dst; size_t dst_size; PJRT_Event* event;
} PJRT_Buffer_ToHostBuffer_Args;
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  PJRT_Buffer* buffer; void* dst; int64_t offset; int64_t transfer_size; PJRT_Event* event;
} PJRT_Buffer_CopyRawToHost_Args;
typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_Buffer* buffer; bool is_on_cpu; } PJRT_Buffer_IsOnCpu_Args;
typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_Buffer* buffer; PJRT_Event* event; } PJRT_Buffer_ReadyEvent_Args;
typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_Buffer* buffer; uintptr_t buffer_pointer; } PJRT_Buffer_UnsafePointer_Args;
typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_Buffer* buffer; } PJRT_Buffer_IncreaseExternalReferenceCount_Args;
typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_Buffer* buffer; } PJRT_Buffer_DecreaseExternalReferenceCount_Args;
typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_Buffer* buffer; void* device_memory_ptr; } PJRT_Buffer_OpaqueDeviceMemoryDataPointer_Args;
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  PJRT_Buffer* buffer; PJRT_Buffer_Type element_type; const int64_t* dims; size_t num_dims;
  PJRT_Buffer_MemoryLayout* device_layout; PJRT_Buffer* out_buffer;
} PJRT_Buffer_Bitcast_Args;

/* ---- programs and executables: crates/ryft-pjrt/src/programs.rs:1499-2446 -------------- */
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  char* code; size_t code_size;       /* MLIR text, or bytecode starting with "ML\xEFR" */
  const char* format; size_t format_size; /* "mlir" (length-delimited, programs.rs:1249) */
} PJRT_Program;
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  PJRT_Client* client; const PJRT_Program* program;
  const char* compile_options; size_t compile_options_size; /* serialized CompileOptionsProto */
  PJRT_LoadedExecutable* executable; /* out */
} PJRT_Client_Compile_Args;
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  const PJRT_TopologyDescription* topology; const PJRT_Program* program;
  const char* compile_options; size_t compile_options_size; PJRT_Client* client; PJRT_Executable* executable;
} PJRT_Compile_Args;
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  PJRT_Client* client; PJRT_Executable* executable; const char* compile_options; size_t compile_options_size;
  PJRT_LoadedExecutable* loaded_executable;
} PJRT_Client_Load_Args;
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  PJRT_Client* client; const char* serialized_executable; size_t serialized_executable_size;
  PJRT_LoadedExecutable* loaded_executable;
  const char* overridden_serialized_compile_options; size_t overridden_serialized_compile_options_size;
} PJRT_Executable_DeserializeAndLoad_Args;

typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_Executable* executable; } PJRT_Executable_Destroy_Args;
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  PJRT_Executable* executable; const char* executable_name; size_t executable_name_size;
} PJRT_Executable_Name_Args;
typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_Executable* executable; size_t num_replicas; } PJRT_Executable_NumReplicas_Args;
typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_Executable* executable; size_t num_partitions; } PJRT_Executable_NumPartitions_Args;
typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_Executable* executable; size_t num_outputs; } PJRT_Executable_NumOutputs_Args;
typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_Executable* executable; int64_t size_in_bytes; } PJRT_Executable_SizeOfGeneratedCodeInBytes_Args;
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  PJRT_Executable* executable; size_t num_properties; const PJRT_NamedValue* properties;
} PJRT_Executable_GetCostAnalysis_Args;
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  PJRT_Executable* executable; size_t num_outputs; const char* const* memory_kinds; const size_t* memory_kind_sizes;
} PJRT_Executable_OutputMemoryKinds_Args;
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  PJRT_Executable* executable; size_t num_parameters; const char* const* memory_kinds; const size_t* memory_kind_sizes;
} PJRT_Executable_ParameterMemoryKinds_Args;
typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_Executable* executable; PJRT_Program* program; } PJRT_Executable_OptimizedProgram_Args;
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  const PJRT_Executable* executable; const char* serialized_bytes; size_t serialized_bytes_size;
  PJRT_SerializedExecutable* serialized_executable; void (*serialized_executable_deleter)(PJRT_SerializedExecutable*);
} PJRT_Executable_Serialize_Args;
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  const PJRT_Executable* executable; const char* serialized_bytes; size_t serialized_bytes_size;
  PJRT_SerializedCompileOptions* serialized_compile_options;
  void (*serialized_compile_options_deleter)(PJRT_SerializedCompileOptions*);
} PJRT_Executable_GetCompileOptions_Args;
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  PJRT_Executable* executable; PJRT_Buffer_Type* output_types; size_t num_output_types;
} PJRT_Executable_OutputElementTypes_Args;
/* dims of all outputs concatenated; dim_sizes[i] = rank of output i (decode: programs.rs:172-196). */
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  PJRT_Executable* executable; size_t num_outputs; const int64_t* dims; const size_t* dim_sizes;
} PJRT_Executable_OutputDimensions_Args;
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  PJRT_Executable* executable; const char* executable_fingerprint; size_t executable_fingerprint_size;
} PJRT_Executable_Fingerprint_Args;
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  PJRT_Executable* executable;
  int64_t generated_code_size_in_bytes, argument_size_in_bytes, output_size_in_bytes, alias_size_in_bytes,
      temp_size_in_bytes, host_generated_code_size_in_bytes, host_argument_size_in_bytes, host_output_size_in_bytes,
      host_alias_size_in_bytes, host_temp_size_in_bytes, peak_memory_in_bytes, total_size_in_bytes,
      total_allocation_bytes, indefinite_allocations, peak_unpadded_heap_bytes;
} PJRT_Executable_GetCompiledMemoryStats_Args;

typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_LoadedExecutable* executable; } PJRT_LoadedExecutable_Destroy_Args;
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  PJRT_LoadedExecutable* loaded_executable; PJRT_Executable* executable; /* out, caller destroys */
} PJRT_LoadedExecutable_GetExecutable_Args;
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  PJRT_LoadedExecutable* executable; PJRT_Device* const* addressable_devices; size_t num_addressable_devices;
} PJRT_LoadedExecutable_AddressableDevices_Args;
typedef struct { int replica; int partition; } PJRT_LogicalDeviceIds;
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  PJRT_LoadedExecutable* executable; const PJRT_LogicalDeviceIds* addressable_device_logical_ids;
  size_t num_addressable_device_logical_ids;
} PJRT_LoadedExecutable_AddressableDeviceLogicalIds_Args;
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  PJRT_LoadedExecutable* executable; const char* serialized_bytes; size_t serialized_bytes_size; /* DeviceAssignmentProto */
  PJRT_DeviceAssignmentSerialized* serialized_device_assignment;
  void (*serialized_device_assignment_deleter)(PJRT_DeviceAssignmentSerialized*);
} PJRT_LoadedExecutable_GetDeviceAssignment_Args;
typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_LoadedExecutable* executable; } PJRT_LoadedExecutable_Delete_Args;
typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_LoadedExecutable* executable; bool is_deleted; } PJRT_LoadedExecutable_IsDeleted_Args;
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  PJRT_LoadedExecutable* executable; const char* executable_fingerprint; size_t executable_fingerprint_size;
} PJRT_LoadedExecutable_Fingerprint_Args;
typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_ExecuteContext* context; } PJRT_ExecuteContext_Create_Args;
typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_ExecuteContext* context; } PJRT_ExecuteContext_Destroy_Args;
typedef struct PJRT_SendCallbackInfo PJRT_SendCallbackInfo;
typedef struct PJRT_RecvCallbackInfo PJRT_RecvCallbackInfo;
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  PJRT_SendCallbackInfo** send_callbacks; PJRT_RecvCallbackInfo** recv_callbacks;
  size_t num_send_ops; size_t num_recv_ops;
  int launch_id;
  const int64_t* non_donatable_input_indices; size_t num_non_donatable_input_indices;
  PJRT_ExecuteContext* context; const char* call_location;
  size_t num_tasks; int* task_ids; int64_t* incarnation_ids; PJRT_MultiSlice_Config* multi_slice_config;
} PJRT_ExecuteOptions;
/* argument_lists[num_devices][num_args]; the caller pre-allocates output_lists[num_devices][num_outputs] and,
 * optionally, device_complete_events[num_devices]; the plugin fills every slot (programs.rs:886-962). */
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start;
  PJRT_LoadedExecutable* executable; PJRT_ExecuteOptions* options;
  PJRT_Buffer* const* const* argument_lists; size_t num_devices; size_t num_args;
  PJRT_Buffer** const* output_lists; PJRT_Event** device_complete_events; PJRT_Device* execute_device;
} PJRT_LoadedExecutable_Execute_Args;

/* ---- function table: order of crates/ryft-pjrt/src/lib.rs:222-363 ---------------------- */
/* Asynchronous host-to-device transfer manager (crates/ryft-pjrt/src/transfers.rs:537-850): device buffers are created
 * first and filled later in chunks; a buffer becomes ready when its last chunk (or a whole-buffer literal) has arrived,
 * or carries the error set on it. */
typedef struct PJRT_AsyncHostToDeviceTransferManager PJRT_AsyncHostToDeviceTransferManager;
typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; const int64_t* dims; size_t num_dims; PJRT_Buffer_Type element_type; } PJRT_ShapeSpec;
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_Client* client; PJRT_ShapeSpec* shape_specs; size_t num_shape_specs;
  PJRT_Buffer_MemoryLayout** device_layouts; size_t num_device_layouts; PJRT_Memory* memory;
  PJRT_AsyncHostToDeviceTransferManager* transfer_manager;  /* out */
} PJRT_Client_CreateBuffersForAsyncHostToDevice_Args;
typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_AsyncHostToDeviceTransferManager* transfer_manager; PJRT_Device* device_out; }
    PJRT_AsyncHostToDeviceTransferManager_Device_Args;
typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_AsyncHostToDeviceTransferManager* transfer_manager; size_t buffer_count; }
    PJRT_AsyncHostToDeviceTransferManager_BufferCount_Args;
typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_AsyncHostToDeviceTransferManager* transfer_manager; int buffer_index;
                 size_t buffer_size; } PJRT_AsyncHostToDeviceTransferManager_BufferSize_Args;
typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_AsyncHostToDeviceTransferManager* transfer_manager; int buffer_index;
                 PJRT_Buffer* buffer_out; } PJRT_AsyncHostToDeviceTransferManager_RetrieveBuffer_Args;
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_AsyncHostToDeviceTransferManager* transfer_manager; int buffer_index;
  const void* data; int64_t offset; int64_t transfer_size; bool is_last_transfer; PJRT_Event* done_with_h2d_transfer;  /* out */
} PJRT_AsyncHostToDeviceTransferManager_TransferData_Args;
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_AsyncHostToDeviceTransferManager* transfer_manager; int buffer_index;
  const void* data; const int64_t* shape_dims; size_t shape_num_dims; PJRT_Buffer_Type shape_element_type; PJRT_Buffer_MemoryLayout* shape_layout;
  PJRT_Event* done_with_h2d_transfer;  /* out */
} PJRT_AsyncHostToDeviceTransferManager_TransferLiteral_Args;
typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_AsyncHostToDeviceTransferManager* transfer_manager; int buffer_index;
                 PJRT_Error_Code error_code; const char* error_message; size_t error_message_size; } PJRT_AsyncHostToDeviceTransferManager_SetBufferError_Args;
typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_AsyncHostToDeviceTransferManager* transfer_manager;
                 const PJRT_NamedValue* transfer_metadata; size_t num_metadata; } PJRT_AsyncHostToDeviceTransferManager_AddMetadata_Args;
typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_AsyncHostToDeviceTransferManager* transfer_manager; }
    PJRT_AsyncHostToDeviceTransferManager_Destroy_Args;

typedef PJRT_Error* (*PJRT_Fn)(void* args); /* placeholder type for entries this plugin leaves NULL */
#define B2X_PJRT_FN(name) PJRT_Error* (*name)(name##_Args*)
typedef struct PJRT_Api {
  size_t struct_size;
  PJRT_Extension_Base* extension_start;
  PJRT_Api_Version pjrt_api_version;
  void (*PJRT_Error_Destroy)(PJRT_Error_Destroy_Args*);
  void (*PJRT_Error_Message)(PJRT_Error_Message_Args*);
  B2X_PJRT_FN(PJRT_Error_GetCode);
  B2X_PJRT_FN(PJRT_Plugin_Initialize);
  B2X_PJRT_FN(PJRT_Plugin_Attributes);
  B2X_PJRT_FN(PJRT_Event_Destroy);
  B2X_PJRT_FN(PJRT_Event_IsReady);
  B2X_PJRT_FN(PJRT_Event_Error);
  B2X_PJRT_FN(PJRT_Event_Await);
  B2X_PJRT_FN(PJRT_Event_OnReady);
  B2X_PJRT_FN(PJRT_Client_Create);
  B2X_PJRT_FN(PJRT_Client_Destroy);
  B2X_PJRT_FN(PJRT_Client_PlatformName);
  B2X_PJRT_FN(PJRT_Client_ProcessIndex);
  B2X_PJRT_FN(PJRT_Client_PlatformVersion);
  B2X_PJRT_FN(PJRT_Client_Devices);
  B2X_PJRT_FN(PJRT_Client_AddressableDevices);
  B2X_PJRT_FN(PJRT_Client_LookupDevice);
  B2X_PJRT_FN(PJRT_Client_LookupAddressableDevice);
  B2X_PJRT_FN(PJRT_Client_AddressableMemories);
  B2X_PJRT_FN(PJRT_Client_Compile);
  B2X_PJRT_FN(PJRT_Client_DefaultDeviceAssignment);
  B2X_PJRT_FN(PJRT_Client_BufferFromHostBuffer);
  B2X_PJRT_FN(PJRT_DeviceDescription_Id);
  B2X_PJRT_FN(PJRT_DeviceDescription_ProcessIndex);
  B2X_PJRT_FN(PJRT_DeviceDescription_Attributes);
  B2X_PJRT_FN(PJRT_DeviceDescription_Kind);
  B2X_PJRT_FN(PJRT_DeviceDescription_DebugString);
  B2X_PJRT_FN(PJRT_DeviceDescription_ToString);
  B2X_PJRT_FN(PJRT_Device_GetDescription);
  B2X_PJRT_FN(PJRT_Device_IsAddressable);
  B2X_PJRT_FN(PJRT_Device_LocalHardwareId);
  B2X_PJRT_FN(PJRT_Device_AddressableMemories);
  B2X_PJRT_FN(PJRT_Device_DefaultMemory);
  B2X_PJRT_FN(PJRT_Device_MemoryStats);
  B2X_PJRT_FN(PJRT_Memory_Id);
  B2X_PJRT_FN(PJRT_Memory_Kind);
  B2X_PJRT_FN(PJRT_Memory_DebugString);
  B2X_PJRT_FN(PJRT_Memory_ToString);
  B2X_PJRT_FN(PJRT_Memory_AddressableByDevices);
  B2X_PJRT_FN(PJRT_Executable_Destroy);
  B2X_PJRT_FN(PJRT_Executable_Name);
  B2X_PJRT_FN(PJRT_Executable_NumReplicas);
  B2X_PJRT_FN(PJRT_Executable_NumPartitions);
  B2X_PJRT_FN(PJRT_Executable_NumOutputs);
  B2X_PJRT_FN(PJRT_Executable_SizeOfGeneratedCodeInBytes);
  B2X_PJRT_FN(PJRT_Executable_GetCostAnalysis);
  B2X_PJRT_FN(PJRT_Executable_OutputMemoryKinds);
  B2X_PJRT_FN(PJRT_Executable_OptimizedProgram);
  B2X_PJRT_FN(PJRT_Executable_Serialize);
  B2X_PJRT_FN(PJRT_LoadedExecutable_Destroy);
  B2X_PJRT_FN(PJRT_LoadedExecutable_GetExecutable);
  B2X_PJRT_FN(PJRT_LoadedExecutable_AddressableDevices);
  B2X_PJRT_FN(PJRT_LoadedExecutable_Delete);
  B2X_PJRT_FN(PJRT_LoadedExecutable_IsDeleted);
  B2X_PJRT_FN(PJRT_LoadedExecutable_Execute);
  B2X_PJRT_FN(PJRT_Executable_DeserializeAndLoad);
  B2X_PJRT_FN(PJRT_LoadedExecutable_Fingerprint);
  B2X_PJRT_FN(PJRT_Buffer_Destroy);
  B2X_PJRT_FN(PJRT_Buffer_ElementType);
  B2X_PJRT_FN(PJRT_Buffer_Dimensions);
  B2X_PJRT_FN(PJRT_Buffer_UnpaddedDimensions);
  B2X_PJRT_FN(PJRT_Buffer_DynamicDimensionIndices);
  B2X_PJRT_FN(PJRT_Buffer_GetMemoryLayout);
  B2X_PJRT_FN(PJRT_Buffer_OnDeviceSizeInBytes);
  B2X_PJRT_FN(PJRT_Buffer_Device);
  B2X_PJRT_FN(PJRT_Buffer_Memory);
  B2X_PJRT_FN(PJRT_Buffer_Delete);
  B2X_PJRT_FN(PJRT_Buffer_IsDeleted);
  B2X_PJRT_FN(PJRT_Buffer_CopyToDevice);
  B2X_PJRT_FN(PJRT_Buffer_ToHostBuffer);
  B2X_PJRT_FN(PJRT_Buffer_IsOnCpu);
  B2X_PJRT_FN(PJRT_Buffer_ReadyEvent);
  B2X_PJRT_FN(PJRT_Buffer_UnsafePointer);
  B2X_PJRT_FN(PJRT_Buffer_IncreaseExternalReferenceCount);
  B2X_PJRT_FN(PJRT_Buffer_DecreaseExternalReferenceCount);
  B2X_PJRT_FN(PJRT_Buffer_OpaqueDeviceMemoryDataPointer);
  PJRT_Fn PJRT_CopyToDeviceStream_Destroy;
  PJRT_Fn PJRT_CopyToDeviceStream_AddChunk;
  PJRT_Fn PJRT_CopyToDeviceStream_TotalBytes;
  PJRT_Fn PJRT_CopyToDeviceStream_GranuleSize;
  PJRT_Fn PJRT_CopyToDeviceStream_CurrentBytes;
  PJRT_Fn PJRT_TopologyDescription_Create;
  PJRT_Fn PJRT_TopologyDescription_Destroy;
  PJRT_Fn PJRT_TopologyDescription_PlatformName;
  PJRT_Fn PJRT_TopologyDescription_PlatformVersion;
  PJRT_Fn PJRT_TopologyDescription_GetDeviceDescriptions;
  PJRT_Fn PJRT_TopologyDescription_Serialize;
  PJRT_Fn PJRT_TopologyDescription_Attributes;
  PJRT_Fn PJRT_Compile;
  B2X_PJRT_FN(PJRT_Executable_OutputElementTypes);
  B2X_PJRT_FN(PJRT_Executable_OutputDimensions);
  B2X_PJRT_FN(PJRT_Buffer_CopyToMemory);
  B2X_PJRT_FN(PJRT_Client_CreateViewOfDeviceBuffer);
  B2X_PJRT_FN(PJRT_Executable_Fingerprint);
  PJRT_Fn PJRT_Client_TopologyDescription;
  B2X_PJRT_FN(PJRT_Executable_GetCompiledMemoryStats);
  B2X_PJRT_FN(PJRT_Memory_Kind_Id);
  B2X_PJRT_FN(PJRT_ExecuteContext_Create);
  B2X_PJRT_FN(PJRT_ExecuteContext_Destroy);
  B2X_PJRT_FN(PJRT_Buffer_CopyRawToHost);
  B2X_PJRT_FN(PJRT_AsyncHostToDeviceTransferManager_Destroy);
  B2X_PJRT_FN(PJRT_AsyncHostToDeviceTransferManager_TransferData);
  B2X_PJRT_FN(PJRT_Client_CreateBuffersForAsyncHostToDevice);
  B2X_PJRT_FN(PJRT_AsyncHostToDeviceTransferManager_RetrieveBuffer);
  B2X_PJRT_FN(PJRT_AsyncHostToDeviceTransferManager_Device);
  B2X_PJRT_FN(PJRT_AsyncHostToDeviceTransferManager_BufferCount);
  B2X_PJRT_FN(PJRT_AsyncHostToDeviceTransferManager_BufferSize);
  B2X_PJRT_FN(PJRT_AsyncHostToDeviceTransferManager_SetBufferError);
  B2X_PJRT_FN(PJRT_AsyncHostToDeviceTransferManager_AddMetadata);
  B2X_PJRT_FN(PJRT_Client_DmaMap);
  B2X_PJRT_FN(PJRT_Client_DmaUnmap);
  B2X_PJRT_FN(PJRT_Client_CreateUninitializedBuffer);
  B2X_PJRT_FN(PJRT_Client_UpdateGlobalProcessInfo);
  PJRT_Fn PJRT_TopologyDescription_Deserialize;
  PJRT_Fn PJRT_Client_CreateAliasBuffer;
  PJRT_Fn PJRT_Client_FulfillAliasBuffer;
  B2X_PJRT_FN(PJRT_LoadedExecutable_GetDeviceAssignment);
  B2X_PJRT_FN(PJRT_Client_CreateErrorBuffer);
  B2X_PJRT_FN(PJRT_AsyncHostToDeviceTransferManager_TransferLiteral);
  PJRT_Fn PJRT_Buffer_CopyRawToHostFuture;
  B2X_PJRT_FN(PJRT_Device_PoisonExecution);
  PJRT_Fn PJRT_Device_CreateAsyncTrackingEvent;
  PJRT_Fn PJRT_AsyncTrackingEvent_Destroy;
  B2X_PJRT_FN(PJRT_Executable_GetCompileOptions);
  PJRT_Fn PJRT_Buffer_DonateWithControlDependency;
  B2X_PJRT_FN(PJRT_Event_Create);
  B2X_PJRT_FN(PJRT_Event_Set);
  B2X_PJRT_FN(PJRT_Device_GetAttributes);
  B2X_PJRT_FN(PJRT_Client_Load);
  B2X_PJRT_FN(PJRT_LoadedExecutable_AddressableDeviceLogicalIds);
  B2X_PJRT_FN(PJRT_Buffer_Bitcast);
  B2X_PJRT_FN(PJRT_Error_ForEachPayload);
  PJRT_Fn PJRT_TopologyDescription_Fingerprint;
  B2X_PJRT_FN(PJRT_Executable_ParameterMemoryKinds);
} PJRT_Api;

/* ---- extensions reachable from PJRT_Api::extension_start (linked list of PJRT_Extension_Base) ---------------------- */

/* Stream extension, type id 3 (crates/ryft-pjrt/src/extensions/stream.rs:123-160; ids: crates/ryft-pjrt/src/lib.rs:179-203).
 * `PJRT_Get_Stream_For_External_Ready_Events` returns the device's compute stream, the stream every kernel of an
 * execution is launched on, so that a caller can order its own work, or CUDA timing events, against executions.
 * `PJRT_Wait_Until_Buffer_Ready_On_Stream` makes `stream` wait for the buffer's definition event. */
#define PJRT_Extension_Type_Stream 3
typedef struct { size_t struct_size; PJRT_Device* device; intptr_t stream; /* out */ } PJRT_Get_Stream_For_External_Ready_Events_Args;
typedef struct { size_t struct_size; intptr_t stream; PJRT_Buffer* buffer; } PJRT_Wait_Until_Buffer_Ready_On_Stream_Args;
typedef struct PJRT_Stream_Extension {
  PJRT_Extension_Base base;
  PJRT_Error* (*get_stream)(PJRT_Get_Stream_For_External_Ready_Events_Args*);
  PJRT_Error* (*wait_stream)(PJRT_Wait_Until_Buffer_Ready_On_Stream_Args*);
} PJRT_Stream_Extension;

/* Layouts extension (crates/ryft-pjrt/src/extensions/layouts.rs:596-807, version 4).  Every buffer of this plugin is
 * dense and major-to-minor, so a layout is just the minor_to_major permutation {n-1, ..., 0}; it serializes to the
 * rendered text form the reference parses (`SerializedLayout::proto`, layouts.rs:401-550), e.g. "{2,1,0}".
 * Layouts returned by Client_GetDefaultLayout and Buffer_MemoryLayout are owned by the caller (MemoryLayout_Destroy);
 * those returned by the Executable_Get*Layouts calls are borrowed from the executable (layouts.rs:247-283). */
#define PJRT_Extension_Type_Layouts 4
typedef struct PJRT_Layouts_MemoryLayout PJRT_Layouts_MemoryLayout;
typedef struct PJRT_Layouts_SerializedLayout PJRT_Layouts_SerializedLayout;
typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_Buffer* buffer; PJRT_Layouts_MemoryLayout* layout; /* out */ }
    PJRT_Layouts_PJRT_Buffer_MemoryLayout_Args;
typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_Layouts_MemoryLayout* layout; } PJRT_Layouts_MemoryLayout_Destroy_Args;
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_Layouts_MemoryLayout* layout;
  const char* serialized_bytes; size_t serialized_bytes_size;          /* out, valid while serialized_layout lives */
  PJRT_Layouts_SerializedLayout* serialized_layout;                     /* out */
  void (*serialized_layout_deleter)(PJRT_Layouts_SerializedLayout*);    /* out */
} PJRT_Layouts_MemoryLayout_Serialize_Args;
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_Client* client; PJRT_Buffer_Type element_type;
  const int64_t* dims; size_t num_dims; PJRT_Layouts_MemoryLayout* layout; /* out */
} PJRT_Layouts_PJRT_Client_GetDefaultLayout_Args;
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start; void* topology_description; PJRT_Buffer_Type element_type;
  const int64_t* dims; size_t num_dims; PJRT_Layouts_MemoryLayout* layout; /* out */
} PJRT_Layouts_PJRT_Topology_GetDefaultLayout_Args;
typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_Executable* executable; size_t num_parameters; /* out */
                 PJRT_Layouts_MemoryLayout** layouts; /* out */ } PJRT_Layouts_PJRT_Executable_GetParameterLayouts_Args;
typedef struct { size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_Executable* executable; size_t num_outputs; /* out */
                 PJRT_Layouts_MemoryLayout** layouts; /* out */ } PJRT_Layouts_PJRT_Executable_GetOutputLayouts_Args;
typedef struct PJRT_Layouts_Extension {
  PJRT_Extension_Base base;
  PJRT_Error* (*PJRT_Layouts_MemoryLayout_Destroy)(PJRT_Layouts_MemoryLayout_Destroy_Args*);
  PJRT_Error* (*PJRT_Layouts_MemoryLayout_Serialize)(PJRT_Layouts_MemoryLayout_Serialize_Args*);
  PJRT_Error* (*PJRT_Layouts_PJRT_Client_GetDefaultLayout)(PJRT_Layouts_PJRT_Client_GetDefaultLayout_Args*);
  PJRT_Error* (*PJRT_Layouts_PJRT_Buffer_MemoryLayout)(PJRT_Layouts_PJRT_Buffer_MemoryLayout_Args*);
  PJRT_Error* (*PJRT_Layouts_PJRT_Topology_GetDefaultLayout)(PJRT_Layouts_PJRT_Topology_GetDefaultLayout_Args*);   /* NULL: no topologies */
  PJRT_Error* (*PJRT_Layouts_PJRT_Executable_GetOutputLayouts)(PJRT_Layouts_PJRT_Executable_GetOutputLayouts_Args*);
  PJRT_Error* (*PJRT_Layouts_PJRT_Executable_GetParameterLayouts)(PJRT_Layouts_PJRT_Executable_GetParameterLayouts_Args*);
} PJRT_Layouts_Extension;

/* Memory-descriptions extension (crates/ryft-pjrt/src/extensions/memory_descriptions.rs:215-285, version 1): the memory
 * kinds a described device offers.  Every device of this plugin has one, "device" (HBM), which is also its default. */
#define PJRT_Extension_Type_MemoryDescriptions 6
typedef struct PJRT_MemoryDescription PJRT_MemoryDescription;
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start; PJRT_DeviceDescription* device_description;
  const PJRT_MemoryDescription* const* memory_descriptions; size_t num_memory_descriptions; ptrdiff_t default_memory_index;  /* out */
} PJRT_DeviceDescription_MemoryDescriptions_Args;
typedef struct {
  size_t struct_size; PJRT_Extension_Base* extension_start; const PJRT_MemoryDescription* memory_description;
  const char* kind; size_t kind_size; int kind_id;  /* out */
} PJRT_MemoryDescription_Kind_Args;
typedef struct PJRT_MemoryDescriptions_Extension {
  PJRT_Extension_Base base;
  PJRT_Error* (*PJRT_DeviceDescription_MemoryDescriptions)(PJRT_DeviceDescription_MemoryDescriptions_Args*);
  PJRT_Error* (*PJRT_MemoryDescription_Kind)(PJRT_MemoryDescription_Kind_Args*);
} PJRT_MemoryDescriptions_Extension;

/* ABI-version extension (crates/ryft-pjrt/src/extensions/abi_version.rs:499-770, version 1): the serialization
 * generation of the runtime and of an executable, and whether they fit together.  The Args of this extension carry no
 * `extension_start` field.  The protobuf form is `{1: uint64 platform, 2: bytes version}`
 * (crates/ryft-xla-sys/src/protos.rs:3812-3838); this plugin's `version` payload is two varints:
 * serialization generation, SM architecture (100). */
#define PJRT_Extension_Type_AbiVersion 20
#define B2X_ABI_PLATFORM_ID 0x6232785f63756461ull /* "b2x_cuda" */
typedef struct PJRT_RuntimeAbiVersion PJRT_RuntimeAbiVersion;
typedef struct PJRT_ExecutableAbiVersion PJRT_ExecutableAbiVersion;
typedef struct PJRT_SerializedProto PJRT_SerializedProto;
typedef struct { size_t struct_size; PJRT_Client* client; PJRT_RuntimeAbiVersion* abi_version; /* out */ } PJRT_Client_RuntimeAbiVersion_Args;
typedef struct { size_t struct_size; PJRT_Executable* executable; PJRT_ExecutableAbiVersion* abi_version; /* out */ } PJRT_Executable_GetAbiVersion_Args;
typedef struct { size_t struct_size; PJRT_RuntimeAbiVersion* abi_version; } PJRT_RuntimeAbiVersion_Destroy_Args;
typedef struct { size_t struct_size; const PJRT_RuntimeAbiVersion* abi_version; const PJRT_RuntimeAbiVersion* other_abi_version; } PJRT_RuntimeAbiVersion_IsCompatibleWithRuntime_Args;
typedef struct { size_t struct_size; const PJRT_RuntimeAbiVersion* abi_version; const PJRT_ExecutableAbiVersion* executable_abi_version; } PJRT_RuntimeAbiVersion_IsCompatibleWithExecutable_Args;
typedef struct {
  size_t struct_size; const PJRT_RuntimeAbiVersion* abi_version;
  const char* serialized_proto; size_t serialized_proto_size;                                     /* out */
  PJRT_SerializedProto* serialized_proto_holder; void (*serialized_proto_deleter)(PJRT_SerializedProto*);  /* out */
} PJRT_RuntimeAbiVersion_ToProto_Args;
typedef struct { size_t struct_size; const PJRT_RuntimeAbiVersion* abi_version; uint64_t platform_id; /* out */ } PJRT_RuntimeAbiVersion_PlatformId_Args;
typedef struct { size_t struct_size; PJRT_ExecutableAbiVersion* abi_version; } PJRT_ExecutableAbiVersion_Destroy_Args;
typedef struct {
  size_t struct_size; const PJRT_ExecutableAbiVersion* abi_version;
  const char* serialized_proto; size_t serialized_proto_size;                                     /* out */
  PJRT_SerializedProto* serialized_proto_holder; void (*serialized_proto_deleter)(PJRT_SerializedProto*);  /* out */
} PJRT_ExecutableAbiVersion_ToProto_Args;
typedef struct { size_t struct_size; const PJRT_ExecutableAbiVersion* abi_version; uint64_t platform_id; /* out */ } PJRT_ExecutableAbiVersion_PlatformId_Args;
typedef struct { size_t struct_size; const char* serialized_proto; size_t serialized_proto_size; PJRT_RuntimeAbiVersion* abi_version; /* out */ } PJRT_RuntimeAbiVersion_FromProto_Args;
typedef struct { size_t struct_size; const char* serialized_proto; size_t serialized_proto_size; PJRT_ExecutableAbiVersion* abi_version; /* out */ } PJRT_ExecutableAbiVersion_FromProto_Args;
typedef struct PJRT_AbiVersion_Extension {
  PJRT_Extension_Base base;
  PJRT_Error* (*PJRT_Client_RuntimeAbiVersion)(PJRT_Client_RuntimeAbiVersion_Args*);
  PJRT_Error* (*PJRT_Executable_GetAbiVersion)(PJRT_Executable_GetAbiVersion_Args*);
  PJRT_Error* (*PJRT_RuntimeAbiVersion_Destroy)(PJRT_RuntimeAbiVersion_Destroy_Args*);
  PJRT_Error* (*PJRT_RuntimeAbiVersion_IsCompatibleWithRuntime)(PJRT_RuntimeAbiVersion_IsCompatibleWithRuntime_Args*);
  PJRT_Error* (*PJRT_RuntimeAbiVersion_IsCompatibleWithExecutable)(PJRT_RuntimeAbiVersion_IsCompatibleWithExecutable_Args*);
  PJRT_Error* (*PJRT_RuntimeAbiVersion_ToProto)(PJRT_RuntimeAbiVersion_ToProto_Args*);
  PJRT_Error* (*PJRT_RuntimeAbiVersion_PlatformId)(PJRT_RuntimeAbiVersion_PlatformId_Args*);
  PJRT_Error* (*PJRT_ExecutableAbiVersion_Destroy)(PJRT_ExecutableAbiVersion_Destroy_Args*);
  PJRT_Error* (*PJRT_ExecutableAbiVersion_ToProto)(PJRT_ExecutableAbiVersion_ToProto_Args*);
  PJRT_Error* (*PJRT_ExecutableAbiVersion_PlatformId)(PJRT_ExecutableAbiVersion_PlatformId_Args*);
  PJRT_Error* (*PJRT_RuntimeAbiVersion_FromProto)(PJRT_RuntimeAbiVersion_FromProto_Args*);
  PJRT_Error* (*PJRT_ExecutableAbiVersion_FromProto)(PJRT_ExecutableAbiVersion_FromProto_Args*);
} PJRT_AbiVersion_Extension;

/* Step-timing extension (no counterpart in the reference; private type id).  When enabled for a loaded executable,
 * every later execution brackets each plan step with CUDA events on the stream the step runs on.  `collect` waits
 * for the recorded executions, sums the device time per step and resets the record.  Arrays are borrowed from the
 * executable and stay valid until the next call. */
#define B2X_Extension_Type_StepTiming 0x62327801u
typedef struct {
  size_t struct_size;
  PJRT_LoadedExecutable* executable;
  size_t device_index;        /* index into the executable's addressable devices */
  int enable;                 /* in: 1 = start recording, 0 = stop, -1 = leave as is */
  int collect;                /* in: non-zero = gather the timings recorded so far */
  size_t num_steps;           /* out */
  size_t num_executions;      /* out: executions summed in step_ms */
  const float* step_ms;       /* out: total device milliseconds per step over those executions */
  const char* const* labels;  /* out: one NUL-terminated label per step ("gemm ...", "reduce ...") */
  const double* flops;        /* out: algorithmic FLOPs of one launch of the step */
  const double* bytes;        /* out: algorithmic bytes of one launch of the step */
  const int* kernel_launches; /* out: kernels this library launches per step (0 for NCCL collectives and copies) */
  /* Read only when struct_size covers them.  replay > 0: enqueue the plan `replay` more times back to back with the
   * arguments and outputs of the device's last recorded execution (recording must be enabled when that execution is
   * launched, and the caller keeps its buffers alive), one pair of CUDA events around all of them: the device time of
   * the kernels without the host work of an execution between launches.  Refused for plans with collectives. */
  int replay;                 /* in */
  float replay_ms;            /* out: device milliseconds of all `replay` repetitions together */
  float replay_host_ms;       /* out: host milliseconds spent enqueueing them (close to replay_ms = the host was the limit) */
} B2X_StepTiming_Args;
typedef struct B2X_StepTiming_Extension {
  PJRT_Extension_Base base;
  PJRT_Error* (*step_timing)(B2X_StepTiming_Args*);
} B2X_StepTiming_Extension;

/* The one exported symbol of the plugin (crates/ryft-pjrt/src/plugins.rs:67-79). */
const PJRT_Api* GetPjrtApi(void);

#ifdef __cplusplus
}
#endif
#endif /* B2X_PJRT_C_API_H_ */
