"""CPU checks of the host side: the library loads and exports what the header declares, the ABI structs match
the headers the reference vendors, the operand parser refuses what the reference refuses."""
import ctypes
import os
import threading
import subprocess
import tempfile

import numpy as np
import pytest

from tlaloc_b200 import _native as N
from tlaloc_b200 import build as B
from tlaloc_b200.attrs import parse_paged_attention

REF_XLA = "/root/reference/triton/third_party/xla"


def test_library_loads_and_exports_every_declared_symbol():
    lib = N.lib()
    names = N.declared_symbols()
    assert "tlaloc_b200_paged_attention" in names and "TlalocRegisterKernels" in names and len(names) >= 17
    for name in names:
        assert hasattr(lib, name), name
        assert name in N._SIGNATURES, f"{name} has no ctypes signature"
    assert lib.tlaloc_b200_abi_version() == 1
    seen = []
    t = threading.Thread(target=lambda: seen.append(lib.tlaloc_b200_last_error()))  # the message is per thread:
    t.start()                                                                        # a new thread has none yet
    t.join()
    assert seen == [b""]


def test_argument_refusals_need_no_gpu():
    lib = N.lib()
    # a null pointer, a bad dtype and a bad shape are refused before any CUDA call
    rc = lib.tlaloc_b200_paged_attention(None, N.F32, None, None, N.F32, None, None, None, 0, None, N.F32, None, None, 1,
                                         1, 1, 1, 1, 1, 1, 1, 1, 1.0, 0, None)
    assert rc == N.INVALID_ARGUMENT and b"null" in lib.tlaloc_b200_last_error()
    one = ctypes.c_void_p(16)
    rc = lib.tlaloc_b200_paged_attention(one, N.F32, one, one, N.F32, one, one, None, 0, one, N.F32, None, one, 1,
                                         3, 4, 8, 6, 2, 3, 3, 2, 0.5, 0, None)  # 4 heads over 3 kv heads
    assert rc == N.INVALID_ARGUMENT and b"multiple of numKvHeads" in lib.tlaloc_b200_last_error()
    rc = lib.tlaloc_b200_paged_attention(one, N.F32, one, one, N.F32, one, one, None, 0, one, N.F32, None, one, 1,
                                         3, 4, 8, 6, 2, 2, 3, 2, 0.5, 0, None)  # 3 rows over 2 tables
    assert rc == N.INVALID_ARGUMENT and b"one per row" in lib.tlaloc_b200_last_error()
    rc = lib.tlaloc_b200_paged_attention(one, N.S8, one, one, N.F32, one, one, None, 0, one, N.F32, None, one, 1,
                                         2, 4, 8, 6, 2, 2, 3, 2, 0.5, 0, None)
    assert rc == N.INVALID_ARGUMENT and b"f32 or bf16" in lib.tlaloc_b200_last_error()
    rc = lib.tlaloc_b200_int8_gemm(one, N.F32, one, one, None, one, N.F32, None, 0, 0, 8, 8, 0, None)
    assert rc == N.INVALID_ARGUMENT
    rc = lib.tlaloc_b200_rope_kv_write(one, one, one, one, one, one, one, one, N.F32, one, one, N.F32, 1, 4, 2, 3, 8, 8, 12, 6, 6, None)
    assert rc == N.INVALID_ARGUMENT and b"odd" in lib.tlaloc_b200_last_error()
    assert lib.tlaloc_b200_paged_attention_splits(32, 8, 32, 512, 16) == 32
    assert lib.tlaloc_b200_paged_attention_scratch_bytes(32, 32, 128, 32) == 32 * 32 * 32 * 130 * 4
    assert lib.tlaloc_b200_ffi_handler(b"tlaloc_paged_attention") and lib.tlaloc_b200_ffi_handler(b"nope") is None


class _T:
    def __init__(self, shape, dtype="float32"):
        self.shape, self.dtype = shape, dtype


def test_parser_refuses_what_the_reference_refuses():
    """ir/src/commonTest/.../PagedAttentionTest.kt:518-567 and PagedAttentionAttrs.kt:145-286."""
    q, k = _T((2, 4, 3)), _T((6, 2, 2, 3))
    t, l = _T((2, 3), "int32"), _T((2,), "int32")
    p = parse_paged_attention(q, k, k, t, l, scale=0.5)
    assert (p.group, p.rows_per_table, p.max_context_len, p.first_live(5)) == (2, 1, 6, 0)
    assert parse_paged_attention(q, k, k, t, l, scale=0.5, sliding_window=2).first_live(5) == 3
    p3 = parse_paged_attention(_T((6, 4, 3)), k, k, t, _T((6,), "int32"), scale=0.5)
    assert p3.rows_per_table == 3 and p3.table_of(5) == 1

    def refused(match, *a, **kw):
        with pytest.raises(ValueError, match=match):
            parse_paged_attention(*a, **kw)

    refused("sliding_window", q, k, k, t, l, scale=0.5, sliding_window=0)
    refused("one per row", _T((3, 4, 3)), k, k, t, _T((3,), "int32"), scale=0.5)
    refused("scale", q, k, k, t, l, scale=None)
    refused("finite", q, k, k, t, l, scale=float("inf"))
    refused("refused by name", q, k, k, t, l, scale=0.5, block_size=2)
    refused("refused by name", q, k, k, t, l, scale=0.5, numKvHeads=2)
    refused("rank-3", _T((2, 12)), k, k, t, l, scale=0.5)
    refused("valueCache shape", q, k, _T((6, 2, 2, 4)), t, l, scale=0.5)
    refused("integer tensor", q, k, k, _T((2, 3), "float32"), l, scale=0.5)
    refused("multiple of numKvHeads", _T((2, 3, 3)), k, k, t, l, scale=0.5)
    refused("keep has 4 chunks", q, k, k, t, l, scale=0.5, keep=_T((2, 4), "int32"))
    refused("return_lse", q, k, k, t, l, scale=0.5, return_lse=True, sliding_window=2)
    assert parse_paged_attention(q, k, k, t, l, scale=0.5, keep=_T((2, 3), "int32")).keep_chunk == 2


@pytest.mark.skipif(not os.path.isdir(REF_XLA), reason="the XLA headers the reference vendors are not mounted")
def test_abi_structs_match_the_vendored_xla_headers():
    """Every offset and size tlaloc_b200/csrc/xla_abi.h relies on, against xla/ffi/api/c_api.h and the PJRT headers."""
    checks = [
        ("AbiFfiCallFrame", "XLA_FFI_CallFrame", ["struct_size", "extension_start", "api", "ctx", "stage", "args", "rets", "attrs", "future"]),
        ("AbiFfiBuffer", "XLA_FFI_Buffer", ["struct_size", "extension_start", "dtype", "data", "rank", "dims"]),
        ("AbiFfiArgs", "XLA_FFI_Args", ["struct_size", "extension_start", "size", "types", ("values", "args")]),
        ("AbiFfiArgs", "XLA_FFI_Rets", ["struct_size", "extension_start", "size", "types", ("values", "rets")]),
        ("AbiFfiAttrs", "XLA_FFI_Attrs", ["struct_size", "extension_start", "size", "types", "names", ("values", "attrs")]),
        ("AbiFfiExtensionBase", "XLA_FFI_InternalExtension", ["struct_size", "type", "next"]),
        ("AbiFfiMetadata", "XLA_FFI_Metadata", ["struct_size", "api_version", "traits", "state_type_id"]),
        ("AbiFfiMetadataExtension", "XLA_FFI_Metadata_Extension", [("base", "extension_base"), "metadata"]),
        ("AbiFfiApiVersion", "XLA_FFI_Api_Version", ["struct_size", "extension_start", "major_version", "minor_version"]),
        ("AbiFfiScalar", "XLA_FFI_Scalar", ["dtype", "value"]),
        ("AbiFfiByteSpan", "XLA_FFI_ByteSpan", ["ptr", "len"]),
        ("AbiFfiErrorCreateArgs", "XLA_FFI_Error_Create_Args", ["struct_size", "extension_start", "message", "errc"]),
        ("AbiFfiStreamGetArgs", "XLA_FFI_Stream_Get_Args", ["struct_size", "extension_start", "ctx", "stream"]),
        ("AbiFfiApi", "XLA_FFI_Api", ["struct_size", "extension_start", "api_version", "internal_api",
                                       ("error_create", "XLA_FFI_Error_Create"), ("error_destroy", "XLA_FFI_Error_Destroy"),
                                       ("stream_get", "XLA_FFI_Stream_Get")]),
        ("AbiPjrtExtensionBase", "PJRT_Extension_Base", ["struct_size", "type", "next"]),
        ("AbiPjrtApiHead", "PJRT_Api", ["struct_size", "extension_start", "pjrt_api_version",
                                         ("error_destroy", "PJRT_Error_Destroy"), ("error_message", "PJRT_Error_Message")]),
        ("AbiPjrtErrorMessageArgs", "PJRT_Error_Message_Args", ["struct_size", "extension_start", "error", "message", "message_size"]),
        ("AbiPjrtErrorDestroyArgs", "PJRT_Error_Destroy_Args", ["struct_size", "extension_start", "error"]),
        ("AbiPjrtGpuRegisterCustomCallArgs", "PJRT_Gpu_Register_Custom_Call_Args",
         ["struct_size", "function_name", "function_name_size", "api_version", "handler_instantiate", "handler_prepare",
          "handler_initialize", "handler_execute", "traits"]),
        ("AbiPjrtGpuCustomCall", "PJRT_Gpu_Custom_Call", ["base", "custom_call", "custom_call_handles_traits"]),
    ]
    lines = ['#include <cstddef>', '#include "xla/ffi/api/c_api.h"', '#include "xla/pjrt/c/pjrt_c_api.h"',
             '#include "xla/pjrt/c/pjrt_c_api_gpu_extension.h"', f'#include "{B.CSRC}/xla_abi.h"']
    for mine, theirs, fields in checks:
        for f in fields:
            a, b = f if isinstance(f, tuple) else (f, f)
            lines.append(f'static_assert(offsetof({mine}, {a}) == offsetof({theirs}, {b}), "{mine}.{a}");')
            lines.append(f'static_assert(sizeof((({mine}*)0)->{a}) == sizeof((({theirs}*)0)->{b}), "{mine}.{a} size");')
    consts = [("kAbiFfiExtensionMetadata", "XLA_FFI_Extension_Metadata"), ("kAbiFfiInitialize", "XLA_FFI_ExecutionStage_INITIALIZE"),
              ("kAbiFfiExecute", "XLA_FFI_ExecutionStage_EXECUTE"), ("kAbiFfiInvalidArgument", "XLA_FFI_Error_Code_INVALID_ARGUMENT"),
              ("kAbiFfiInternal", "XLA_FFI_Error_Code_INTERNAL"), ("kAbiFfiAttrScalar", "XLA_FFI_AttrType_SCALAR"),
              ("kAbiFfiApiMajor", "XLA_FFI_API_MAJOR"), ("kAbiFfiApiMinor", "XLA_FFI_API_MINOR"),
              ("kAbiFfiTraitCommandBufferCompatible", "XLA_FFI_HANDLER_TRAITS_COMMAND_BUFFER_COMPATIBLE"),
              ("kAbiPjrtExtensionGpuCustomCall", "PJRT_Extension_Type_Gpu_Custom_Call"),
              ("TLALOC_B200_F32", "XLA_FFI_DataType_F32"), ("TLALOC_B200_BF16", "XLA_FFI_DataType_BF16"),
              ("TLALOC_B200_S8", "XLA_FFI_DataType_S8"), ("TLALOC_B200_S32", "XLA_FFI_DataType_S32"),
              ("TLALOC_ABI_SIZE_THROUGH(AbiFfiErrorCreateArgs, errc)", "XLA_FFI_Error_Create_Args_STRUCT_SIZE"),
              ("TLALOC_ABI_SIZE_THROUGH(AbiFfiStreamGetArgs, stream)", "XLA_FFI_Stream_Get_Args_STRUCT_SIZE"),
              ("TLALOC_ABI_SIZE_THROUGH(AbiPjrtGpuRegisterCustomCallArgs, traits)", "PJRT_Gpu_Register_Custom_Call_Args_STRUCT_SIZE"),
              ("TLALOC_ABI_SIZE_THROUGH(AbiPjrtErrorMessageArgs, message_size)", "PJRT_Error_Message_Args_STRUCT_SIZE"),
              ("TLALOC_ABI_SIZE_THROUGH(AbiPjrtErrorDestroyArgs, error)", "PJRT_Error_Destroy_Args_STRUCT_SIZE")]
    lines.append(f'#include "{B.INCLUDE}/tlaloc_b200.h"')
    for mine, theirs in consts:
        lines.append(f'static_assert((long)({mine}) == (long)({theirs}), "{theirs}");')
    lines.append("int main() { return 0; }")
    with tempfile.TemporaryDirectory() as d:
        src = os.path.join(d, "abi_check.cc")
        with open(src, "w") as f:
            f.write("\n".join(lines))
        r = subprocess.run(["g++", "-std=c++17", "-fsyntax-only", "-I", REF_XLA, src], capture_output=True, text=True)
        assert r.returncode == 0, r.stderr[-3000:]


def test_peer_sum_refuses_bad_arguments_before_touching_the_gpu():
    """The tensor-parallel sum validates on the host first; world 1 is a no-op (no device is needed for either)."""
    lib = N.lib()
    bases = (ctypes.c_void_p * 2)(0x1000, 0x2000)
    state = ctypes.c_void_p(0x3000)
    call = lib.tlaloc_b200_peer_allreduce_f32
    assert call(bases, 0, 0, state, 0, 9, 4, None) == N.INVALID_ARGUMENT and b"world 9" in lib.tlaloc_b200_last_error()
    assert call(bases, 0, 0, state, 2, 2, 4, None) == N.INVALID_ARGUMENT and b"rank 2" in lib.tlaloc_b200_last_error()
    assert call(bases, 0, 0, state, 0, 2, 6, None) == N.INVALID_ARGUMENT  # count not a multiple of 4
    assert call(bases, 8, 0, state, 0, 2, 4, None) == N.INVALID_ARGUMENT  # values not 16-byte aligned
    assert call(None, 0, 0, state, 0, 2, 4, None) == N.INVALID_ARGUMENT
    misaligned = (ctypes.c_void_p * 2)(0x1000, 0x2004)
    assert call(misaligned, 0, 0, state, 0, 2, 4, None) == N.INVALID_ARGUMENT and b"rank 1" in lib.tlaloc_b200_last_error()
    assert call(bases, 0, 0, state, 0, 1, 4, None) == N.OK  # one rank: nothing to exchange, nothing launched
    assert call(bases, 0, 0, state, 0, 2, 0, None) == N.OK

    from tlaloc_b200.peer import PeerBuffers

    with pytest.raises(ValueError):
        PeerBuffers([(4, 4)], rank=0, world=9)


def test_fused_peer_sum_and_norm_refuses_bad_shapes_before_touching_the_gpu():
    lib = N.lib()
    bases = (ctypes.c_void_p * 2)(0x1000, 0x2000)
    state = ctypes.c_void_p(0x3000)
    call = lib.tlaloc_b200_peer_allreduce_rmsnorm_f32
    assert call(bases, 0, 4096, 8192, state, None, 1e-5, 0, 1, 4, 256, None) == N.INVALID_ARGUMENT  # one rank: use rmsnorm
    assert call(bases, 0, 4096, 8192, state, None, 1e-5, 0, 2, 3, 256, None) == N.INVALID_ARGUMENT  # rows do not divide
    assert b"3 rows" in lib.tlaloc_b200_last_error()
    assert call(bases, 0, 4096, 8192, state, None, 1e-5, 0, 2, 4, 250, None) == N.INVALID_ARGUMENT  # cols not a multiple of 16
    assert call(bases, 0, 4096, 8192, state, None, 1e-5, 0, 2, 4, 65536, None) == N.INVALID_ARGUMENT  # a row too long for registers
    assert call(bases, 0, 4100, 8192, state, None, 1e-5, 0, 2, 4, 256, None) == N.INVALID_ARGUMENT  # norm region misaligned
    assert call(bases, 0, 4096, 8192, state, ctypes.c_void_p(0x4004), 1e-5, 0, 2, 4, 256, None) == N.INVALID_ARGUMENT  # gain misaligned
