// Shared by the kernels of libtlaloc_kernels.so (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/tlaloc_b200.h"

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
inline size_t DtypeBytes(int dt) { return dt == TLALOC_B200_F32 || dt == TLALOC_B200_S32 ? 4 : dt == TLALOC_B200_BF16 ? 2 : 1; }

__device__ __forceinline__ float ToF32(float x) { return x; }
__device__ __forceinline__ float ToF32(__nv_bfloat16 x) { return __bfloat162float(x); }
__device__ __forceinline__ float ToF32(int8_t x) { return static_cast<float>(x); }

template <typename T>
__device__ __forceinline__ T FromF32(float x);
template <>
__device__ __forceinline__ float FromF32<float>(float x) { return x; }
template <>
__device__ __forceinline__ __nv_bfloat16 FromF32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

// Kernels launched by this library since it was loaded (tlaloc_b200_launch_count); a plain statistic.
void CountLaunches(int n);

// Once-per-process kernel attribute setup (dynamic shared memory opt-in) of each
// translation unit; called from tlaloc_b200_init and from the typed-FFI
// handlers' INITIALIZE stage, so that no launch inside a CUDA graph capture
// has to change a function attribute.
cudaError_t PreparePagedAttentionKernels();
cudaError_t PrepareInt8GemmKernels();
cudaError_t PrepareInt8GemmTcKernels();

// The tensor-core projection (int8_gemm_tc.cu): rows [0, m) of y = (x @ codes) * scales (+ residual), x bf16.
cudaError_t LaunchInt8GemmTc(const __nv_bfloat16* x, const int8_t* codes, const float* scales, const float* residual,
                             void* y, int y_dtype, int m, int k, int n, cudaStream_t st, int* launches);
// 1 if a bounded device-side wait has timed out since the last call (synchronous read), 0 if not, -1 on a CUDA error.
int ReadTcStatus();

}  // namespace tlaloc_b200
