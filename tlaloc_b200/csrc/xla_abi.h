// The slice of two stable C ABIs this library speaks, declared here so the library builds without an XLA
// checkout: XLA's typed-FFI call frame (xla/ffi/api/c_api.h, API 0.5) and the head of PJRT_Api plus its GPU
// custom-call extension (xla/pjrt/c/pjrt_c_api.h, pjrt_c_api_gpu_extension.h version 3).  Only the members
// this library reads or writes are named; layouts (field order, widths, x86-64/aarch64 LP64 alignment) follow
// the upstream headers, and tests/test_ffi_abi.py checks every offset and size used here against the headers
// the reference vendors (triton/third_party/xla) whenever those are present.  The reference's JVM side keeps
// the same offsets by hand (runtime-pjrt/.../ffm/XlaFfiCallFrame.kt:25-42, PjrtFfiRegistry.kt:34-56).
#pragma once

#include <stddef.h>
#include <stdint.h>

extern "C" {

// ---- typed FFI ---------------------------------------------------------------------------------------------

enum AbiFfiExtensionType : int32_t { kAbiFfiExtensionMetadata = 1 };
enum AbiFfiStage : int32_t {
  kAbiFfiInstantiate = 0,
  kAbiFfiPrepare = 1,
  kAbiFfiInitialize = 2,
  kAbiFfiExecute = 3,
  kAbiFfiRecord = 4
};
enum AbiFfiErrorCode : int32_t { kAbiFfiInvalidArgument = 3, kAbiFfiInternal = 13 };
enum AbiFfiAttrType : int32_t { kAbiFfiAttrArray = 1, kAbiFfiAttrDictionary = 2, kAbiFfiAttrScalar = 3, kAbiFfiAttrString = 4 };
constexpr int kAbiFfiApiMajor = 0;
constexpr int kAbiFfiApiMinor = 5;
constexpr uint32_t kAbiFfiTraitCommandBufferCompatible = 1u << 0;

struct AbiFfiExtensionBase {  // XLA_FFI_InternalExtension
  size_t struct_size;
  int32_t type;
  AbiFfiExtensionBase* next;
};

struct AbiFfiApiVersion {  // XLA_FFI_Api_Version
  size_t struct_size;
  AbiFfiExtensionBase* extension_start;
  int major_version;
  int minor_version;
};

struct AbiFfiMetadata {  // XLA_FFI_Metadata
  size_t struct_size;
  AbiFfiApiVersion api_version;
  uint32_t traits;
  int64_t state_type_id;
};

struct AbiFfiMetadataExtension {  // XLA_FFI_Metadata_Extension
  AbiFfiExtensionBase base;
  AbiFfiMetadata* metadata;
};

struct AbiFfiByteSpan {
  const char* ptr;
  size_t len;
};

struct AbiFfiScalar {
  int32_t dtype;
  void* value;
};

struct AbiFfiBuffer {  // XLA_FFI_Buffer
  size_t struct_size;
  AbiFfiExtensionBase* extension_start;
  int32_t dtype;
  void* data;
  int64_t rank;
  int64_t* dims;
};

struct AbiFfiArgs {  // XLA_FFI_Args and XLA_FFI_Rets share this shape
  size_t struct_size;
  AbiFfiExtensionBase* extension_start;
  int64_t size;
  int32_t* types;
  void** values;
};

struct AbiFfiAttrs {  // XLA_FFI_Attrs: sorted by name
  size_t struct_size;
  AbiFfiExtensionBase* extension_start;
  int64_t size;
  int32_t* types;
  AbiFfiByteSpan** names;
  void** values;
};

struct AbiFfiError;
struct AbiFfiContext;
struct AbiFfiApi;

struct AbiFfiCallFrame {  // XLA_FFI_CallFrame
  size_t struct_size;
  AbiFfiExtensionBase* extension_start;
  const AbiFfiApi* api;
  AbiFfiContext* ctx;
  int32_t stage;
  AbiFfiArgs args;
  AbiFfiArgs rets;
  AbiFfiAttrs attrs;
  void* future;
};

struct AbiFfiErrorCreateArgs {  // XLA_FFI_Error_Create_Args
  size_t struct_size;
  AbiFfiExtensionBase* extension_start;
  const char* message;
  int32_t errc;
};

struct AbiFfiStreamGetArgs {  // XLA_FFI_Stream_Get_Args
  size_t struct_size;
  AbiFfiExtensionBase* extension_start;
  AbiFfiContext* ctx;
  void* stream;
};

struct AbiFfiApi {  // XLA_FFI_Api, up to the last entry this library calls
  size_t struct_size;
  AbiFfiExtensionBase* extension_start;
  AbiFfiApiVersion api_version;
  const void* internal_api;
  AbiFfiError* (*error_create)(AbiFfiErrorCreateArgs*);
  void (*error_get_details)(void*);
  void (*error_destroy)(void*);
  AbiFfiError* (*handler_register)(void*);
  AbiFfiError* (*stream_get)(AbiFfiStreamGetArgs*);
};

typedef AbiFfiError* (*AbiFfiHandler)(AbiFfiCallFrame*);

// ---- PJRT --------------------------------------------------------------------------------------------------

enum AbiPjrtExtensionType : int32_t { kAbiPjrtExtensionGpuCustomCall = 0 };

struct AbiPjrtExtensionBase {  // PJRT_Extension_Base
  size_t struct_size;
  int32_t type;
  AbiPjrtExtensionBase* next;
};

struct AbiPjrtApiVersion {
  size_t struct_size;
  AbiPjrtExtensionBase* extension_start;
  int major_version;
  int minor_version;
};

struct AbiPjrtError;

struct AbiPjrtErrorDestroyArgs {
  size_t struct_size;
  AbiPjrtExtensionBase* extension_start;
  AbiPjrtError* error;
};

struct AbiPjrtErrorMessageArgs {
  size_t struct_size;
  AbiPjrtExtensionBase* extension_start;
  const AbiPjrtError* error;
  const char* message;
  size_t message_size;
};

struct AbiPjrtApiHead {  // the first members of PJRT_Api
  size_t struct_size;
  AbiPjrtExtensionBase* extension_start;
  AbiPjrtApiVersion pjrt_api_version;
  void (*error_destroy)(AbiPjrtErrorDestroyArgs*);
  void (*error_message)(AbiPjrtErrorMessageArgs*);
};

struct AbiPjrtGpuRegisterCustomCallArgs {  // PJRT_Gpu_Register_Custom_Call_Args (extension version 3)
  size_t struct_size;
  const char* function_name;
  size_t function_name_size;
  int api_version;  // 1 = typed FFI
  void* handler_instantiate;
  void* handler_prepare;
  void* handler_initialize;
  void* handler_execute;
  uint32_t traits;
};

struct AbiPjrtGpuCustomCall {  // PJRT_Gpu_Custom_Call
  AbiPjrtExtensionBase base;
  AbiPjrtError* (*custom_call)(AbiPjrtGpuRegisterCustomCallArgs*);
  bool custom_call_handles_traits;
};

}  // extern "C"

// struct_size values XLA's own PJRT_STRUCT_SIZE / XLA_FFI_STRUCT_SIZE macros give (offset of the last field + its size).
#define TLALOC_ABI_SIZE_THROUGH(type, field) (offsetof(type, field) + sizeof(((type*)0)->field))
