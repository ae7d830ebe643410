"""The drop-in boundary without a GPU: TlalocRegisterKernels against a fake PJRT_Api, and the typed-FFI handlers'
protocol and refusals against hand-built call frames (the reference's pattern: XlaFfiCallFrameTest.kt:55-100,
PjrtCustomCallRegistrationSpikeTest.kt:14-30)."""
import ctypes as C

import ffi_frames as F
from tlaloc_b200 import _native as N

TARGETS = ["tlaloc_paged_attention", "tlaloc_int8_gemm", "tlaloc_kv_cache_write"]


def test_register_kernels_registers_typed_ffi_handlers_with_the_gpu_custom_call_extension():
    lib = N.lib()
    fake = F.FakePjrt()
    assert lib.TlalocRegisterKernels(C.addressof(fake.api)) is None
    assert [r[0] for r in fake.registered] == TARGETS
    for name, api_version, init, execute, size in fake.registered:
        assert api_version == 1 and init == execute == lib.tlaloc_b200_ffi_handler(name.encode()) and init
        assert size == C.sizeof(F.RegisterArgs) - 4  # struct_size runs through `traits`, the last field (no tail padding)


def test_register_kernels_reports_a_missing_extension_and_a_refused_registration():
    lib = N.lib()
    assert b"no GPU custom-call extension" in lib.TlalocRegisterKernels(C.addressof(F.FakePjrt(with_extension=False).api))
    fake = F.FakePjrt(fail_on="tlaloc_int8_gemm")
    msg = lib.TlalocRegisterKernels(C.addressof(fake.api))
    assert b"registering tlaloc_int8_gemm" in msg and b"already registered" in msg
    assert fake.destroyed == [0xBAD] and [r[0] for r in fake.registered] == ["tlaloc_paged_attention"]
    assert b"null" in lib.TlalocRegisterKernels(None)


def test_metadata_query_is_answered_and_other_stages_are_no_ops():
    lib = N.lib()
    for t in TARGETS:
        h = F.handler(lib, t)
        xla = F.FakeXla()
        md = F.Metadata(struct_size=C.sizeof(F.Metadata))
        assert h(C.byref(xla.frame(F.EXECUTE, metadata=md))) is None
        assert (md.api_version.major, md.api_version.minor, md.traits) == (0, 5, 1)  # command-buffer compatible
        for stage in (F.INSTANTIATE, F.PREPARE):
            assert h(C.byref(xla.frame(stage))) is None
        assert xla.errors == []


def _pa_frame(xla, q_dims=(2, 4, 8), k_dims=(6, 2, 2, 8), t_dims=(2, 3), scratch_dims=(1, 2, 4, 10), q_dtype=F.F32,
              attrs=None, nargs=5):
    ptr = 256
    a = [xla.buffer(q_dtype, ptr, q_dims), xla.buffer(F.F32, ptr, k_dims), xla.buffer(F.F32, ptr, k_dims),
         xla.buffer(F.S32, ptr, t_dims), xla.buffer(F.S32, ptr, (q_dims[0],))][:nargs]
    r = [xla.buffer(q_dtype, ptr, q_dims), xla.buffer(F.F32, ptr, scratch_dims)]
    if attrs is None:
        attrs = {"scale": (F.F32, C.c_float(0.5))}
    return xla.frame(F.EXECUTE, a, r, attrs)


def test_paged_attention_handler_refuses_bad_frames_by_name():
    h = F.handler(N.lib(), "tlaloc_paged_attention")

    def refused(match, **kw):
        xla = F.FakeXla()
        assert h(C.byref(_pa_frame(xla, **kw))) is not None
        code, msg = xla.errors[-1]
        assert code == F.INVALID_ARGUMENT and msg.startswith("tlaloc_paged_attention: ") and match in msg, msg

    refused("takes 5 operands", nargs=4)
    refused("needs an f32 'scale' attribute", attrs={})
    refused("needs an f32 'scale' attribute", attrs={"scale": (F.S32, C.c_int32(1))})
    refused("sliding_window", attrs={"scale": (F.F32, C.c_float(0.5)), "sliding_window": (F.S32, C.c_int32(0))})
    refused("ranks", q_dims=(2, 32))
    refused("scratch must be f32 [S, R, H, D + 2]", scratch_dims=(1, 2, 4, 8))
    refused("headDim", k_dims=(6, 2, 2, 16))
    refused("multiple of numKvHeads", k_dims=(6, 2, 3, 8))          # refused by the C ABI below the handler
    refused("one per row", q_dims=(3, 4, 8), scratch_dims=(1, 3, 4, 10))  # 3 rows over 2 tables
    refused("f32 or bf16", q_dtype=F.S8)


def test_int8_gemm_and_kv_write_handlers_refuse_bad_frames_by_name():
    lib = N.lib()
    h = F.handler(lib, "tlaloc_int8_gemm")
    xla = F.FakeXla()
    ptr = 256
    x, w, s, y = xla.buffer(F.BF16, ptr, (4, 64)), xla.buffer(F.S8, ptr, (64, 32)), xla.buffer(F.F32, ptr, (32,)), xla.buffer(F.F32, ptr, (4, 32))
    assert h(C.byref(xla.frame(F.EXECUTE, [x, w], [y]))) is not None and "takes 3 operands" in xla.errors[-1][1]
    bad_w = xla.buffer(F.S8, ptr, (32, 64))  # the weight the wrong way round ([out, in]): refused, never silently transposed
    assert h(C.byref(xla.frame(F.EXECUTE, [x, bad_w, s], [y]))) is not None and "codes [K, N] (in, out)" in xla.errors[-1][1]
    f32_w = xla.buffer(F.F32, ptr, (64, 32))
    assert h(C.byref(xla.frame(F.EXECUTE, [x, f32_w, s], [y]))) is not None and "codes must be s8" in xla.errors[-1][1]
    h = F.handler(lib, "tlaloc_kv_cache_write")
    pool, rows, slots = xla.buffer(F.F32, ptr, (4, 16, 2, 8)), xla.buffer(F.F32, ptr, (3, 2, 8)), xla.buffer(F.S32, ptr, (3,))
    assert h(C.byref(xla.frame(F.EXECUTE, [pool, rows], [pool]))) is not None and "takes 3 operands" in xla.errors[-1][1]
    bad_rows = xla.buffer(F.F32, ptr, (3, 4, 8))
    assert h(C.byref(xla.frame(F.EXECUTE, [pool, bad_rows, slots], [pool]))) is not None and "[T, Hkv, D]" in xla.errors[-1][1]
    assert all(code == F.INVALID_ARGUMENT for code, _ in xla.errors)
    assert F.handler(lib, "tlaloc_moe_fp4") is None  # out of scope: not exported
