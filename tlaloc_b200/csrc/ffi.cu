// The library's reference-facing surface: XLA typed-FFI handlers over the C ABI, and TlalocRegisterKernels, the
// entry point the reference's loaders call (triton/backend/pjrt_runtime.cc:139-164 from C++,
// runtime-pjrt/.../ffm/PjrtFfiRegistry.kt:192-204 from the JVM).
//
// Handler protocol, as the reference's handlers follow it (triton/kernels/paged_attention.cu:1334-1446):
//   1. a frame carrying a metadata extension is XLA asking for the handler's FFI version and traits: answer, return;
//   2. stage INITIALIZE: set the kernels' attributes, outside any CUDA graph capture;
//   3. any stage but EXECUTE: nothing to do;
//   4. EXECUTE: validate operands/results/attrs, take XLA's stream, enqueue on it; never allocate or synchronise.
// Handlers are thread-safe: they keep no state beyond the once-only kernel set-up, which is mutex-guarded.
#include <atomic>
#include <cstring>
#include <string>

#include "common.cuh"
#include "xla_abi.h"

namespace tlaloc_b200 {

char* ErrorBuffer()
{
  static thread_local char buf[kErrorBufferBytes] = {0};
  return buf;
}

namespace {
std::atomic<long long> g_launches{0};
std::atomic<int> g_order_faithful{0};
}  // namespace

void CountLaunches(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
bool OrderFaithful() { return g_order_faithful.load(std::memory_order_relaxed) != 0; }

namespace {

AbiFfiError* MakeError(const AbiFfiApi* api, int32_t code, const std::string& msg)
{
  AbiFfiErrorCreateArgs a;
  std::memset(&a, 0, sizeof(a));
  a.struct_size = TLALOC_ABI_SIZE_THROUGH(AbiFfiErrorCreateArgs, errc);
  a.message = msg.c_str();
  a.errc = code;
  return api->error_create(&a);
}

// A C-ABI status as an XLA error (null for success).
AbiFfiError* FromStatus(const AbiFfiApi* api, const char* target, int status)
{
  if (status == kOk) return nullptr;
  return MakeError(api, status == kInternal ? kAbiFfiInternal : kAbiFfiInvalidArgument,
                   std::string(target) + ": " + tlaloc_b200_last_error());
}

// Answers XLA's metadata query if the frame carries one.
bool AnswerMetadata(AbiFfiCallFrame* frame)
{
  for (AbiFfiExtensionBase* ext = frame->extension_start; ext != nullptr; ext = ext->next) {
    if (ext->type == kAbiFfiExtensionMetadata) {
      AbiFfiMetadata* md = reinterpret_cast<AbiFfiMetadataExtension*>(ext)->metadata;
      md->api_version.major_version = kAbiFfiApiMajor;
      md->api_version.minor_version = kAbiFfiApiMinor;
      md->traits = kAbiFfiTraitCommandBufferCompatible;
      return true;
    }
  }
  return false;
}

AbiFfiError* Initialize(const AbiFfiApi* api, const char* target)
{
  return FromStatus(api, target, tlaloc_b200_init());
}

AbiFfiError* GetStream(AbiFfiCallFrame* frame, void** stream)
{
  AbiFfiStreamGetArgs sa;
  std::memset(&sa, 0, sizeof(sa));
  sa.struct_size = TLALOC_ABI_SIZE_THROUGH(AbiFfiStreamGetArgs, stream);
  sa.ctx = frame->ctx;
  if (AbiFfiError* err = frame->api->stream_get(&sa)) return err;
  *stream = sa.stream;
  return nullptr;
}

const AbiFfiBuffer* Arg(const AbiFfiCallFrame* f, int i) { return static_cast<const AbiFfiBuffer*>(f->args.values[i]); }
const AbiFfiBuffer* Ret(const AbiFfiCallFrame* f, int i) { return static_cast<const AbiFfiBuffer*>(f->rets.values[i]); }

bool NameIs(const AbiFfiByteSpan* n, const char* s) { return n->len == std::strlen(s) && std::memcmp(n->ptr, s, n->len) == 0; }

// A scalar attribute as an integer, from s32 or s64.
bool ScalarInt(const AbiFfiScalar* sc, int64_t* out)
{
  if (sc->dtype == TLALOC_B200_S32) {
    *out = *static_cast<const int32_t*>(sc->value);
    return true;
  }
  if (sc->dtype == 5 /* S64 */) {
    *out = *static_cast<const int64_t*>(sc->value);
    return true;
  }
  return false;
}

bool FitsInt(int64_t v) { return v >= 0 && v <= 0x7fffffff; }

// tlaloc_paged_attention: operands query [R,H,D], keyCache, valueCache [P,bs,Hkv,D], blockTables s32 [Tb,M],
// seqLens s32 [R], optional keep s32 [R,C]; results out [R,H,D], scratch f32 [S,R,H,D+2], optional lse f32 [R,H].
// Attributes: scale (f32, required), sliding_window (s32/s64, optional), prefill_f16 (accepted and ignored: this
// library has one precision).  The wire format is the reference's (triton/kernels/paged_attention.cu:5-17,
// stablehlo/.../StablehloEmitter.kt:3461-3490) widened to bf16 queries and outputs.
AbiFfiError* PagedAttentionHandler(AbiFfiCallFrame* frame)
{
  const char* target = "tlaloc_paged_attention";
  if (AnswerMetadata(frame)) return nullptr;
  const AbiFfiApi* api = frame->api;
  if (frame->stage == kAbiFfiInitialize) return Initialize(api, target);
  if (frame->stage != kAbiFfiExecute) return nullptr;
  auto invalid = [&](const std::string& m) { return MakeError(api, kAbiFfiInvalidArgument, std::string(target) + ": " + m); };
  if ((frame->args.size != 5 && frame->args.size != 6) || (frame->rets.size != 2 && frame->rets.size != 3)) {
    return invalid("takes 5 operands (6 with a keep mask) and returns 2 results (3 with the log-sum-exp)");
  }
  const AbiFfiBuffer *q = Arg(frame, 0), *k = Arg(frame, 1), *v = Arg(frame, 2), *t = Arg(frame, 3), *l = Arg(frame, 4);
  const AbiFfiBuffer* keep = frame->args.size == 6 ? Arg(frame, 5) : nullptr;
  const AbiFfiBuffer *out = Ret(frame, 0), *scratch = Ret(frame, 1);
  const AbiFfiBuffer* lse = frame->rets.size == 3 ? Ret(frame, 2) : nullptr;
  float scale = 0.f;
  bool has_scale = false;
  int64_t window = 0;
  for (int64_t i = 0; i < frame->attrs.size; ++i) {
    if (frame->attrs.types[i] != kAbiFfiAttrScalar) continue;
    const AbiFfiScalar* sc = static_cast<const AbiFfiScalar*>(frame->attrs.values[i]);
    if (NameIs(frame->attrs.names[i], "scale") && sc->dtype == TLALOC_B200_F32) {
      scale = *static_cast<const float*>(sc->value);
      has_scale = true;
    } else if (NameIs(frame->attrs.names[i], "sliding_window")) {
      if (!ScalarInt(sc, &window) || window < 1 || !FitsInt(window)) return invalid("'sliding_window' must be a whole number >= 1");
    }
  }
  if (!has_scale) return invalid("needs an f32 'scale' attribute");
  if (q->rank != 3 || k->rank != 4 || v->rank != 4 || t->rank != 2 || l->rank != 1 || out->rank != 3 || scratch->rank != 4) {
    return invalid("unexpected operand or result ranks");
  }
  for (int d = 0; d < 4; ++d) {
    if (k->dims[d] != v->dims[d]) return invalid("valueCache shape must match keyCache");
  }
  if (k->dtype != v->dtype) return invalid("valueCache dtype must match keyCache");
  if (t->dtype != TLALOC_B200_S32 || l->dtype != TLALOC_B200_S32) return invalid("blockTables and seqLens must be s32");
  if (k->dims[3] != q->dims[2]) return invalid("keyCache headDim must match query headDim");
  if (l->dims[0] != q->dims[0]) return invalid("seqLens must have one entry per query row");
  for (int d = 0; d < 3; ++d) {
    if (out->dims[d] != q->dims[d]) return invalid("result shape must match the query shape");
  }
  for (int d = 0; d < 3; ++d) {
    if (!FitsInt(q->dims[d])) return invalid("query dims out of range");
  }
  for (int d = 0; d < 4; ++d) {
    if (!FitsInt(k->dims[d])) return invalid("pool dims out of range");
  }
  if (!FitsInt(t->dims[0]) || !FitsInt(t->dims[1]) || !FitsInt(scratch->dims[0])) return invalid("table or scratch dims out of range");
  if (scratch->dtype != TLALOC_B200_F32 || scratch->dims[1] != q->dims[0] || scratch->dims[2] != q->dims[1] ||
      scratch->dims[3] != q->dims[2] + 2 || scratch->dims[0] < 1) {
    return invalid("scratch must be f32 [S, R, H, D + 2]");
  }
  int keep_chunks = 0;
  if (keep != nullptr) {
    if (keep->rank != 2 || keep->dtype != TLALOC_B200_S32 || keep->dims[0] != q->dims[0] || keep->dims[1] < 1 || !FitsInt(keep->dims[1])) {
      return invalid("keep must be s32 [R, C] with C dividing the context");
    }
    keep_chunks = static_cast<int>(keep->dims[1]);
  }
  if (lse != nullptr && (lse->rank != 2 || lse->dtype != TLALOC_B200_F32 || lse->dims[0] != q->dims[0] || lse->dims[1] != q->dims[1])) {
    return invalid("the log-sum-exp result must be f32 [R, H]");
  }
  void* stream = nullptr;
  if (AbiFfiError* err = GetStream(frame, &stream)) return err;
  const int status = tlaloc_b200_paged_attention(
      q->data, q->dtype, k->data, v->data, k->dtype, static_cast<const int32_t*>(t->data),
      static_cast<const int32_t*>(l->data), keep ? static_cast<const int32_t*>(keep->data) : nullptr, keep_chunks,
      out->data, out->dtype, lse ? static_cast<float*>(lse->data) : nullptr, static_cast<float*>(scratch->data),
      static_cast<int32_t>(scratch->dims[0]), static_cast<int32_t>(q->dims[0]), static_cast<int32_t>(q->dims[1]),
      static_cast<int32_t>(q->dims[2]), static_cast<int32_t>(k->dims[0]), static_cast<int32_t>(k->dims[1]),
      static_cast<int32_t>(k->dims[2]), static_cast<int32_t>(t->dims[1]), static_cast<int32_t>(t->dims[0]), scale,
      static_cast<int32_t>(window), stream);
  return FromStatus(api, target, status);
}

// tlaloc_int8_gemm: operands x [M,K] (f32|bf16), codes s8 [K,N], scales f32 [N], optional residual f32 [M,N];
// results y [M,N] (f32|bf16), optional scratch (any f32 buffer; needed for an f32 x and for i8_mma).  Attributes
// exact (s32, optional, nonzero = the order-faithful kernel) and i8_mma (s32, optional, nonzero = 17 to 128 rows on the
// int8 tensor-core kernel, TLALOC_B200_GEMM_I8_MMA).  The custom-call form of HfDecoderGraph.proj over an int8
// weight, which the reference leaves to XLA as convert + dot_general + multiply.
AbiFfiError* Int8GemmHandler(AbiFfiCallFrame* frame)
{
  const char* target = "tlaloc_int8_gemm";
  if (AnswerMetadata(frame)) return nullptr;
  const AbiFfiApi* api = frame->api;
  if (frame->stage == kAbiFfiInitialize) return Initialize(api, target);
  if (frame->stage != kAbiFfiExecute) return nullptr;
  auto invalid = [&](const std::string& m) { return MakeError(api, kAbiFfiInvalidArgument, std::string(target) + ": " + m); };
  if ((frame->args.size != 3 && frame->args.size != 4) || (frame->rets.size != 1 && frame->rets.size != 2)) {
    return invalid("takes 3 operands (4 with a residual) and returns 1 result (2 with scratch)");
  }
  const AbiFfiBuffer *x = Arg(frame, 0), *w = Arg(frame, 1), *s = Arg(frame, 2);
  const AbiFfiBuffer* res = frame->args.size == 4 ? Arg(frame, 3) : nullptr;
  const AbiFfiBuffer* y = Ret(frame, 0);
  const AbiFfiBuffer* scratch = frame->rets.size == 2 ? Ret(frame, 1) : nullptr;
  if (x->rank != 2 || w->rank != 2 || s->rank != 1 || y->rank != 2) return invalid("x, codes and y must be rank 2 and scales rank 1");
  if (w->dtype != TLALOC_B200_S8 || s->dtype != TLALOC_B200_F32) return invalid("codes must be s8 and scales f32");
  if (w->dims[0] != x->dims[1] || s->dims[0] != w->dims[1] || y->dims[0] != x->dims[0] || y->dims[1] != w->dims[1]) {
    return invalid("shapes must be x [M, K], codes [K, N] (in, out), scales [N], y [M, N]");
  }
  if (!FitsInt(x->dims[0]) || !FitsInt(x->dims[1]) || !FitsInt(w->dims[1])) return invalid("dims out of range");
  if (res != nullptr && (res->rank != 2 || res->dtype != TLALOC_B200_F32 || res->dims[0] != y->dims[0] || res->dims[1] != y->dims[1])) {
    return invalid("the residual must be f32 [M, N]");
  }
  int64_t exact = 0, i8_mma = 0;
  for (int64_t i = 0; i < frame->attrs.size; ++i) {
    if (frame->attrs.types[i] != kAbiFfiAttrScalar) continue;
    if (NameIs(frame->attrs.names[i], "exact")) {
      if (!ScalarInt(static_cast<const AbiFfiScalar*>(frame->attrs.values[i]), &exact)) return invalid("'exact' must be s32");
    } else if (NameIs(frame->attrs.names[i], "i8_mma")) {
      if (!ScalarInt(static_cast<const AbiFfiScalar*>(frame->attrs.values[i]), &i8_mma)) return invalid("'i8_mma' must be s32");
    }
  }
  size_t scratch_bytes = 0;
  if (scratch != nullptr) {
    scratch_bytes = DtypeBytes(scratch->dtype);
    for (int64_t d = 0; d < scratch->rank; ++d) scratch_bytes *= static_cast<size_t>(scratch->dims[d]);
  }
  void* stream = nullptr;
  if (AbiFfiError* err = GetStream(frame, &stream)) return err;
  const int status = tlaloc_b200_int8_gemm(
      x->data, x->dtype, static_cast<const int8_t*>(w->data), static_cast<const float*>(s->data),
      res ? static_cast<const float*>(res->data) : nullptr, y->data, y->dtype,
      scratch ? static_cast<float*>(scratch->data) : nullptr, scratch_bytes, static_cast<int32_t>(x->dims[0]),
      static_cast<int32_t>(x->dims[1]), static_cast<int32_t>(w->dims[1]),
      (exact != 0 ? TLALOC_B200_GEMM_EXACT : 0) | (i8_mma != 0 ? TLALOC_B200_GEMM_I8_MMA : 0), stream);
  return FromStatus(api, target, status);
}

// tlaloc_kv_cache_write: operands pool [P,bs,Hkv,D], newKv [T,Hkv,D], slotMapping s32 [T]; result pool (aliased to
// operand 0 by the program's output_operand_aliases; when XLA hands a distinct buffer the pool is copied first).
AbiFfiError* KvCacheWriteHandler(AbiFfiCallFrame* frame)
{
  const char* target = "tlaloc_kv_cache_write";
  if (AnswerMetadata(frame)) return nullptr;
  const AbiFfiApi* api = frame->api;
  if (frame->stage == kAbiFfiInitialize) return Initialize(api, target);
  if (frame->stage != kAbiFfiExecute) return nullptr;
  auto invalid = [&](const std::string& m) { return MakeError(api, kAbiFfiInvalidArgument, std::string(target) + ": " + m); };
  if (frame->args.size != 3 || frame->rets.size != 1) return invalid("takes 3 operands and returns 1 result");
  const AbiFfiBuffer *pool = Arg(frame, 0), *rows = Arg(frame, 1), *slots = Arg(frame, 2), *out = Ret(frame, 0);
  if (pool->rank != 4 || rows->rank != 3 || slots->rank != 1 || out->rank != 4) return invalid("unexpected operand or result ranks");
  if (slots->dtype != TLALOC_B200_S32 || slots->dims[0] != rows->dims[0]) return invalid("slotMapping must be s32 [T]");
  if (rows->dims[1] != pool->dims[2] || rows->dims[2] != pool->dims[3]) return invalid("newKv must be [T, Hkv, D] of the pool's heads");
  if (out->dtype != pool->dtype) return invalid("the result pool must have the operand pool's dtype");
  size_t elems = 1;
  for (int d = 0; d < 4; ++d) {
    if (out->dims[d] != pool->dims[d] || !FitsInt(pool->dims[d])) return invalid("the result pool must have the operand pool's shape");
    elems *= static_cast<size_t>(pool->dims[d]);
  }
  if (!FitsInt(pool->dims[0] * pool->dims[1]) || !FitsInt(rows->dims[1] * rows->dims[2])) return invalid("pool too large");
  void* stream = nullptr;
  if (AbiFfiError* err = GetStream(frame, &stream)) return err;
  if (out->data != pool->data) {
    const cudaError_t e = cudaMemcpyAsync(out->data, pool->data, elems * DtypeBytes(pool->dtype), cudaMemcpyDeviceToDevice,
                                          static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return MakeError(api, kAbiFfiInternal, std::string(target) + ": " + cudaGetErrorString(e));
  }
  const int status = tlaloc_b200_kv_cache_write(out->data, out->dtype, rows->data, rows->dtype,
                                                static_cast<const int32_t*>(slots->data), static_cast<int32_t>(rows->dims[0]),
                                                static_cast<int32_t>(rows->dims[1] * rows->dims[2]),
                                                static_cast<int32_t>(pool->dims[0] * pool->dims[1]), stream);
  return FromStatus(api, target, status);
}

}  // namespace
}  // namespace tlaloc_b200

using namespace tlaloc_b200;

namespace tlaloc_b200 {
bool PdlEnabled()
{
  static const bool on = [] {
    const char* e = std::getenv("TLALOC_B200_PDL");
    return e == nullptr || std::atoi(e) != 0;
  }();
  return on;
}
}  // namespace tlaloc_b200

extern "C" int tlaloc_b200_abi_version(void) { return TLALOC_B200_ABI_VERSION; }

extern "C" const char* tlaloc_b200_last_error(void) { return ErrorBuffer(); }

extern "C" long long tlaloc_b200_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

extern "C" int tlaloc_b200_device_status(void)
{
  const int a = ReadTcStatus(), b = ReadI8Status(), c = ReadPaStatus();
  return a < 0 || b < 0 || c < 0 ? -1 : (a | b | c);
}

extern "C" int tlaloc_b200_set_order_faithful(int on)
{
  return g_order_faithful.exchange(on != 0 ? 1 : 0, std::memory_order_relaxed);
}

extern "C" int tlaloc_b200_init(void)
{
  cudaError_t e = PreparePagedAttentionKernels();
  if (e == cudaSuccess) e = PrepareInt8GemmKernels();
  if (e == cudaSuccess) e = PrepareInt8GemmTcKernels();
  if (e == cudaSuccess) e = PrepareInt8GemmI8Kernels();
  if (e != cudaSuccess) return CudaFail("kernel set-up", e);
  return kOk;
}

// The handlers by name, for callers that register them one at a time (a JVM's registerExecuteHandler route,
// runtime-pjrt/.../ffm/PjrtFfiRegistry.kt:168-182) and for tests that drive them with hand-built call frames.
extern "C" __attribute__((visibility("default"))) void* tlaloc_b200_ffi_handler(const char* target)
{
  if (target == nullptr) return nullptr;
  if (std::strcmp(target, "tlaloc_paged_attention") == 0) return reinterpret_cast<void*>(&PagedAttentionHandler);
  if (std::strcmp(target, "tlaloc_int8_gemm") == 0) return reinterpret_cast<void*>(&Int8GemmHandler);
  if (std::strcmp(target, "tlaloc_kv_cache_write") == 0) return reinterpret_cast<void*>(&KvCacheWriteHandler);
  return nullptr;
}

extern "C" __attribute__((visibility("default"))) const char* TlalocRegisterKernels(const struct PJRT_Api* opaque_api)
{
  static std::string error;
  if (opaque_api == nullptr) {
    error = "the PJRT_Api pointer is null";
    return error.c_str();
  }
  const AbiPjrtApiHead* api = reinterpret_cast<const AbiPjrtApiHead*>(opaque_api);
  AbiPjrtGpuCustomCall* ext = nullptr;
  for (AbiPjrtExtensionBase* e = api->extension_start; e != nullptr; e = e->next) {
    if (e->type == kAbiPjrtExtensionGpuCustomCall) ext = reinterpret_cast<AbiPjrtGpuCustomCall*>(e);
  }
  if (ext == nullptr) {
    error = "the PJRT plugin has no GPU custom-call extension";
    return error.c_str();
  }
  const char* names[] = {"tlaloc_paged_attention", "tlaloc_int8_gemm", "tlaloc_kv_cache_write"};
  for (const char* name : names) {
    AbiPjrtGpuRegisterCustomCallArgs a;
    std::memset(&a, 0, sizeof(a));
    a.struct_size = TLALOC_ABI_SIZE_THROUGH(AbiPjrtGpuRegisterCustomCallArgs, traits);
    a.function_name = name;
    a.function_name_size = std::strlen(name);
    a.api_version = 1;  // typed FFI
    // The same handler at INITIALIZE: kernel attributes are set there, outside any graph capture.
    a.handler_initialize = tlaloc_b200_ffi_handler(name);
    a.handler_execute = a.handler_initialize;
    a.traits = kAbiFfiTraitCommandBufferCompatible;
    AbiPjrtError* err = ext->custom_call(&a);
    if (err == nullptr) continue;
    AbiPjrtErrorMessageArgs m;
    std::memset(&m, 0, sizeof(m));
    m.struct_size = TLALOC_ABI_SIZE_THROUGH(AbiPjrtErrorMessageArgs, message_size);
    m.error = err;
    api->error_message(&m);
    error = std::string("registering ") + name + ": " + std::string(m.message ? m.message : "", m.message ? m.message_size : 0);
    AbiPjrtErrorDestroyArgs d;
    std::memset(&d, 0, sizeof(d));
    d.struct_size = TLALOC_ABI_SIZE_THROUGH(AbiPjrtErrorDestroyArgs, error);
    d.error = err;
    api->error_destroy(&d);
    return error.c_str();
  }
  return nullptr;
}
