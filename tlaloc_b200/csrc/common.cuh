// Shared by the kernels of libtlaloc_kernels.so (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <mutex>

#include "../../include/tlaloc_b200.h"

struct CUtensorMap_st;  // the driver API's tensor map (cuda.h), named here without including it

namespace tlaloc_b200 {

// Status codes of the C ABI (include/tlaloc_b200.h).
constexpr int kOk = TLALOC_B200_OK;
constexpr int kInvalid = TLALOC_B200_INVALID_ARGUMENT;
constexpr int kInternal = TLALOC_B200_INTERNAL;
constexpr int kUnsupported = TLALOC_B200_UNSUPPORTED;

// The calling thread's last error message (returned by tlaloc_b200_last_error).
char* ErrorBuffer();
constexpr int kErrorBufferBytes = 512;

inline int Fail(int code, const char* fmt, ...)
{
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(ErrorBuffer(), kErrorBufferBytes, fmt, ap);
  va_end(ap);
  return code;
}

inline int CudaFail(const char* what, cudaError_t e)
{
  return Fail(kInternal, "%s: %s", what, cudaGetErrorString(e));
}

inline bool IsFloatType(int dt) { return dt == TLALOC_B200_F32 || dt == TLALOC_B200_BF16; }
// What a KV pool may hold: the float types plus e4m3fn.
inline bool IsPoolType(int dt) { return IsFloatType(dt) || dt == TLALOC_B200_F8E4M3FN; }
inline size_t DtypeBytes(int dt) { return dt == TLALOC_B200_F32 || dt == TLALOC_B200_S32 ? 4 : dt == TLALOC_B200_BF16 ? 2 : 1; }

__device__ __forceinline__ float ToF32(float x) { return x; }
__device__ __forceinline__ float ToF32(__nv_bfloat16 x) { return __bfloat162float(x); }
__device__ __forceinline__ float ToF32(int8_t x) { return static_cast<float>(x); }
__device__ __forceinline__ float ToF32(__nv_fp8_e4m3 x) { return static_cast<float>(x); }

template <typename T>
__device__ __forceinline__ T FromF32(float x);
template <>
__device__ __forceinline__ float FromF32<float>(float x) { return x; }
template <>
__device__ __forceinline__ __nv_bfloat16 FromF32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
// e4m3fn as a KV pool stores it: clamped to +-448, rounded to nearest even; NaN stays NaN (0x7F).
template <>
__device__ __forceinline__ __nv_fp8_e4m3 FromF32<__nv_fp8_e4m3>(float x)
{
  __nv_fp8_e4m3 r;
  r.__x = __nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3);
  return r;
}

// tlaloc_b200_set_order_faithful: every operator evaluates in the reference interpreter's own order (parity runs).
bool OrderFaithful();

// Kernels launched by this library since it was loaded (tlaloc_b200_launch_count); a plain statistic.
void CountLaunches(int n);

// Programmatic dependent launch.  A decode step is ~800 small launches in one stream, and the gap between a kernel's
// last CTA and the next kernel's first one is a few microseconds each.  Every kernel of the library is launched with
// the programmatic-serialization attribute and starts with GridDependencySync(): the kernel may be scheduled (and run
// whatever comes before that call: shared-memory carve-up, mbarrier and TMEM setup) while its predecessor drains, and
// the call then waits until the predecessor grid has COMPLETED and its writes are visible.  So no global memory is
// read or written before it, and correctness is exactly that of plain stream order.  The one exception, taken only
// when the caller states that the weights are constant (TLALOC_B200_GEMM_WEIGHTS_CONST): the projection kernels fetch
// their first stages of codes ahead of the call, since no kernel in flight can be writing them.  The trigger for the kernel's
// own successors is issued right after the wait, never before it, so at most one kernel is ever waiting behind a
// running one.  A launch without the attribute (another library's kernel, $TLALOC_B200_PDL=0) makes the call a no-op.
__device__ __forceinline__ void GridDependencySync()
{
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
bool PdlEnabled();
// The launch attributes every kernel gets; `attrs` must have room for 2.  Returns the count.
inline int ChainAttributes(cudaLaunchAttribute* attrs, int cluster_y = 0)
{
  int n = 0;
  if (cluster_y > 0) {
    attrs[n].id = cudaLaunchAttributeClusterDimension;
    attrs[n].val.clusterDim.x = 1;
    attrs[n].val.clusterDim.y = static_cast<unsigned>(cluster_y);
    attrs[n].val.clusterDim.z = 1;
    ++n;
  }
  if (PdlEnabled()) {
    attrs[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  return n;
}
template <typename... KArgs, typename... Args>
cudaError_t LaunchChained(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args)
{
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attrs[2];
  cfg.numAttrs = ChainAttributes(attrs);
  cfg.attrs = attrs;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Kernel attribute set-up (the dynamic shared memory opt-in) is per device: a process that drives several GPUs (a PJRT
// client's usual layout) must repeat it on each.  Run(f) calls f(device) once per device, with that device current,
// under a mutex; a failed set-up is retried by the next call.
constexpr int kMaxDevices = 64;
struct OncePerDevice {
  std::mutex mu;
  bool done[kMaxDevices] = {};
  template <typename F>
  cudaError_t Run(F f)
  {
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return e;
    if (device < 0 || device >= kMaxDevices) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(mu);
    if (done[device]) return cudaSuccess;
    e = f(device);
    if (e == cudaSuccess) done[device] = true;
    return e;
  }
};

// Per-device kernel attribute set-up of each translation unit; called from tlaloc_b200_init and from the typed-FFI
// handlers' INITIALIZE stage, so that no launch inside a CUDA graph capture has to change a function attribute.
cudaError_t PreparePagedAttentionKernels();
cudaError_t PrepareInt8GemmKernels();
cudaError_t PrepareInt8GemmTcKernels();

// The tensor-core projection (int8_gemm_tc.cu): rows [0, m) of y = (x @ codes) * scales (+ residual), x bf16.
cudaError_t LaunchInt8GemmTc(const __nv_bfloat16* x, const int8_t* codes, const float* scales, const float* residual,
                             void* y, int y_dtype, int m, int k, int n, cudaStream_t st, int* launches, bool weights_const,
                             bool swiglu = false);
// 1 if a bounded device-side wait has timed out since the last call (synchronous read), 0 if not, -1 on a CUDA error.
int ReadTcStatus();
// The same projection with the codes fed to the tensor core as int8 and the activations as two int8 planes
// (int8_gemm_i8.cu); m <= 128 rows per call.
cudaError_t PrepareInt8GemmI8Kernels();
bool Int8GemmI8Applies(const void* codes, int m, int k, int n);
size_t Int8GemmI8ScratchBytes(int m, int k);
cudaError_t LaunchInt8GemmI8(const void* x, int x_dtype, const int8_t* codes, const float* scales, const float* residual,
                             void* y, int y_dtype, void* scratch, int m, int k, int n, cudaStream_t st, int* launches,
                             bool weights_const, bool swiglu, bool have_planes);
// The quantizer alone: the planes of x [m, k] into `planes` (Int8GemmI8ScratchBytes(m, k) bytes).
cudaError_t LaunchQuantizeRowsI8(const void* x, int x_dtype, void* planes, int m, int k, cudaStream_t st);
int ReadI8Status();
bool EncodeKvPoolMap(::CUtensorMap_st* map, const void* base, int head_dim, int kv_heads, unsigned long long positions, int elem_bytes);
bool TensorMapEncoderReady();
int ReadPaStatus();

// The activation planes of the int8 tensor-core projection: row m of x as q = rint(x / s[m]) = 256 hi + lo with s[m] the
// smallest power of two that keeps |q| <= 127 * 256.  Layout in the projection's scratch for an [m, k] activation:
// hi int8 [m, k], lo int8 [m, k], s f32 [m].  Any kernel that produces a projection's input may write them itself
// (RMSNorm, the one-barrier sum over ranks) and the projection is then called with TLALOC_B200_GEMM_X_PLANES.
constexpr int kI8QMax = 127 * 256;
// 1 / s for a row whose largest magnitude is amax (bad: the row holds an infinity or a NaN); *step = s, or NaN for a bad row.
__device__ __forceinline__ float I8RowInvStep(float amax, bool bad, float* step)
{
  int e = 0;
  if (amax > 0.f) {
    int p;
    frexpf(amax, &p);  // amax = f 2^p, f in [0.5, 1)
    e = min(max(p - 15, -126), 126);
    if (ldexpf(amax, -e) > static_cast<float>(kI8QMax)) ++e;
  }
  *step = bad ? __int_as_float(0x7fc00000) : ldexpf(1.f, e);
  return bad ? 0.f : ldexpf(1.f, -e);
}
__device__ __forceinline__ void I8Split(float v, float inv, int& hi, int& lo)
{
  int q = __float2int_rn(v * inv);  // inv is 0 for a bad row: q = 0 (or the NaN conversion's 0)
  q = min(max(q, -kI8QMax), kI8QMax);
  hi = (q + 128) >> 8;
  lo = q - (hi << 8);
}
// Four consecutive values as one word of each plane.
__device__ __forceinline__ void I8Split4(float a, float b, float c, float d, float inv, uint32_t& hi_word, uint32_t& lo_word)
{
  int h0, l0, h1, l1, h2, l2, h3, l3;
  I8Split(a, inv, h0, l0);
  I8Split(b, inv, h1, l1);
  I8Split(c, inv, h2, l2);
  I8Split(d, inv, h3, l3);
  hi_word = (h0 & 255u) | ((h1 & 255u) << 8) | ((h2 & 255u) << 16) | (static_cast<uint32_t>(h3) << 24);
  lo_word = (l0 & 255u) | ((l1 & 255u) << 8) | ((l2 & 255u) << 16) | (static_cast<uint32_t>(l3) << 24);
}
__device__ __forceinline__ float Bf16Value(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

inline bool Aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace tlaloc_b200
