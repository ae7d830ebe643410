"""Hand-built XLA typed-FFI call frames and a fake PJRT_Api, in ctypes.

The pattern of the reference's own ABI test (runtime-pjrt/.../ffm/XlaFfiCallFrameTest.kt:55-100): no XLA plugin is
needed to drive a handler, only a frame laid out as xla/ffi/api/c_api.h lays it out.  Field order follows
tlaloc_b200/csrc/xla_abi.h, which tests/test_host_cpu.py checks against the vendored XLA headers.
"""
import ctypes as C

F32, BF16, S8, S32, S64 = 11, 16, 2, 4, 5
INSTANTIATE, PREPARE, INITIALIZE, EXECUTE = 0, 1, 2, 3
INVALID_ARGUMENT, INTERNAL = 3, 13


class ExtBase(C.Structure):
    pass


ExtBase._fields_ = [("struct_size", C.c_size_t), ("type", C.c_int32), ("next", C.POINTER(ExtBase))]


class ApiVersion(C.Structure):
    _fields_ = [("struct_size", C.c_size_t), ("extension_start", C.c_void_p), ("major", C.c_int), ("minor", C.c_int)]


class Metadata(C.Structure):
    _fields_ = [("struct_size", C.c_size_t), ("api_version", ApiVersion), ("traits", C.c_uint32), ("state_type_id", C.c_int64)]


class MetadataExt(C.Structure):
    _fields_ = [("base", ExtBase), ("metadata", C.POINTER(Metadata))]


class ByteSpan(C.Structure):
    _fields_ = [("ptr", C.c_char_p), ("len", C.c_size_t)]


class Scalar(C.Structure):
    _fields_ = [("dtype", C.c_int32), ("value", C.c_void_p)]


class Buffer(C.Structure):
    _fields_ = [("struct_size", C.c_size_t), ("extension_start", C.c_void_p), ("dtype", C.c_int32), ("data", C.c_void_p),
                ("rank", C.c_int64), ("dims", C.POINTER(C.c_int64))]


class Args(C.Structure):
    _fields_ = [("struct_size", C.c_size_t), ("extension_start", C.c_void_p), ("size", C.c_int64),
                ("types", C.POINTER(C.c_int32)), ("values", C.POINTER(C.c_void_p))]


class Attrs(C.Structure):
    _fields_ = [("struct_size", C.c_size_t), ("extension_start", C.c_void_p), ("size", C.c_int64),
                ("types", C.POINTER(C.c_int32)), ("names", C.POINTER(C.POINTER(ByteSpan))), ("values", C.POINTER(C.c_void_p))]


class ErrorCreateArgs(C.Structure):
    _fields_ = [("struct_size", C.c_size_t), ("extension_start", C.c_void_p), ("message", C.c_char_p), ("errc", C.c_int32)]


class StreamGetArgs(C.Structure):
    _fields_ = [("struct_size", C.c_size_t), ("extension_start", C.c_void_p), ("ctx", C.c_void_p), ("stream", C.c_void_p)]


ERROR_CREATE = C.CFUNCTYPE(C.c_void_p, C.POINTER(ErrorCreateArgs))
STREAM_GET = C.CFUNCTYPE(C.c_void_p, C.POINTER(StreamGetArgs))
VOIDFN = C.CFUNCTYPE(None, C.c_void_p)
PTRFN = C.CFUNCTYPE(C.c_void_p, C.c_void_p)


class Api(C.Structure):
    _fields_ = [("struct_size", C.c_size_t), ("extension_start", C.c_void_p), ("api_version", ApiVersion),
                ("internal_api", C.c_void_p), ("error_create", ERROR_CREATE), ("error_get_details", VOIDFN),
                ("error_destroy", VOIDFN), ("handler_register", PTRFN), ("stream_get", STREAM_GET)]


class CallFrame(C.Structure):
    _fields_ = [("struct_size", C.c_size_t), ("extension_start", C.POINTER(ExtBase)), ("api", C.POINTER(Api)),
                ("ctx", C.c_void_p), ("stage", C.c_int32), ("args", Args), ("rets", Args), ("attrs", Attrs),
                ("future", C.c_void_p)]


HANDLER = C.CFUNCTYPE(C.c_void_p, C.POINTER(CallFrame))


class FakeXla:
    """The two XLA_FFI_Api entries the handlers call: errors are collected, the stream is whatever the test sets."""

    def __init__(self, stream=0):
        self.errors, self.stream, self._keep = [], stream, []

        def error_create(a):
            self.errors.append((a.contents.errc, a.contents.message.decode()))
            return len(self.errors)  # any non-null token

        def stream_get(a):
            a.contents.stream = self.stream
            return None

        self._ec, self._sg = ERROR_CREATE(error_create), STREAM_GET(stream_get)
        self.api = Api(struct_size=C.sizeof(Api), error_create=self._ec, stream_get=self._sg)
        self.api.api_version.major, self.api.api_version.minor = 0, 5

    def buffer(self, dtype, data_ptr, dims):
        arr = (C.c_int64 * max(1, len(dims)))(*dims)
        b = Buffer(struct_size=C.sizeof(Buffer), dtype=dtype, data=data_ptr, rank=len(dims), dims=arr)
        self._keep += [arr, b]
        return b

    def frame(self, stage, args=(), rets=(), attrs=None, metadata=None):
        """attrs: {name: (dtype, ctypes scalar)}; sorted by name as XLA delivers them."""
        f = CallFrame(struct_size=C.sizeof(CallFrame), api=C.pointer(self.api), stage=stage)

        def pack(bufs, dst):
            n = len(bufs)
            types = (C.c_int32 * max(1, n))(*([1] * n))
            vals = (C.c_void_p * max(1, n))(*[C.addressof(b) for b in bufs])
            dst.struct_size, dst.size, dst.types, dst.values = C.sizeof(Args), n, types, vals
            self._keep += [types, vals, list(bufs)]

        pack(list(args), f.args)
        pack(list(rets), f.rets)
        attrs = attrs or {}
        names = sorted(attrs)
        n = len(names)
        types = (C.c_int32 * max(1, n))(*([3] * n))
        spans = [ByteSpan(name.encode(), len(name)) for name in names]
        span_ptrs = (C.POINTER(ByteSpan) * max(1, n))(*[C.pointer(s) for s in spans])
        scalars = []
        for name in names:
            dt, val = attrs[name]
            scalars.append(Scalar(dtype=dt, value=C.addressof(val)))
        vals = (C.c_void_p * max(1, n))(*[C.addressof(s) for s in scalars])
        f.attrs.struct_size, f.attrs.size, f.attrs.types, f.attrs.names, f.attrs.values = C.sizeof(Attrs), n, types, span_ptrs, vals
        self._keep += [types, spans, span_ptrs, scalars, vals, attrs]
        if metadata is not None:
            ext = MetadataExt()
            ext.base.struct_size, ext.base.type, ext.metadata = C.sizeof(MetadataExt), 1, C.pointer(metadata)
            f.extension_start = C.cast(C.pointer(ext), C.POINTER(ExtBase))
            self._keep.append(ext)
        self._keep.append(f)
        return f


def handler(lib, target: str):
    ptr = lib.tlaloc_b200_ffi_handler(target.encode())
    return HANDLER(ptr) if ptr else None


# ---- a fake PJRT_Api with one GPU custom-call extension that records registrations ----------------------------


class PjrtExtBase(C.Structure):
    pass


PjrtExtBase._fields_ = [("struct_size", C.c_size_t), ("type", C.c_int32), ("next", C.POINTER(PjrtExtBase))]


class RegisterArgs(C.Structure):
    _fields_ = [("struct_size", C.c_size_t), ("function_name", C.c_char_p), ("function_name_size", C.c_size_t),
                ("api_version", C.c_int), ("handler_instantiate", C.c_void_p), ("handler_prepare", C.c_void_p),
                ("handler_initialize", C.c_void_p), ("handler_execute", C.c_void_p), ("traits", C.c_uint32)]


REGISTER = C.CFUNCTYPE(C.c_void_p, C.POINTER(RegisterArgs))


class GpuCustomCall(C.Structure):
    _fields_ = [("base", PjrtExtBase), ("custom_call", REGISTER), ("custom_call_handles_traits", C.c_bool)]


class ErrMessageArgs(C.Structure):
    _fields_ = [("struct_size", C.c_size_t), ("extension_start", C.c_void_p), ("error", C.c_void_p),
                ("message", C.c_char_p), ("message_size", C.c_size_t)]


class ErrDestroyArgs(C.Structure):
    _fields_ = [("struct_size", C.c_size_t), ("extension_start", C.c_void_p), ("error", C.c_void_p)]


ERR_MESSAGE = C.CFUNCTYPE(None, C.POINTER(ErrMessageArgs))
ERR_DESTROY = C.CFUNCTYPE(None, C.POINTER(ErrDestroyArgs))


class PjrtApiHead(C.Structure):
    _fields_ = [("struct_size", C.c_size_t), ("extension_start", C.POINTER(PjrtExtBase)), ("version", ApiVersion),
                ("error_destroy", ERR_DESTROY), ("error_message", ERR_MESSAGE), ("pad", C.c_void_p * 64)]


class FakePjrt:
    def __init__(self, with_extension=True, fail_on=None):
        self.registered, self.destroyed, self.fail_on = [], [], fail_on
        self._msg = b"a custom call of that name is already registered"

        def register(a):
            name = a.contents.function_name[:a.contents.function_name_size].decode()
            if name == self.fail_on:
                return 0xBAD
            self.registered.append((name, a.contents.api_version, a.contents.handler_initialize, a.contents.handler_execute,
                                    a.contents.struct_size))
            return None

        def message(a):
            a.contents.message, a.contents.message_size = self._msg, len(self._msg)

        def destroy(a):
            self.destroyed.append(a.contents.error)

        self._r, self._m, self._d = REGISTER(register), ERR_MESSAGE(message), ERR_DESTROY(destroy)
        self.ext = GpuCustomCall(custom_call=self._r, custom_call_handles_traits=True)
        self.ext.base.struct_size, self.ext.base.type = C.sizeof(GpuCustomCall), 0
        self.other = PjrtExtBase(struct_size=C.sizeof(PjrtExtBase), type=3)  # some other extension first in the chain
        if with_extension:
            self.other.next = C.cast(C.pointer(self.ext), C.POINTER(PjrtExtBase))
        self.api = PjrtApiHead(struct_size=C.sizeof(PjrtApiHead), extension_start=C.pointer(self.other),
                               error_destroy=self._d, error_message=self._m)
