// The small ops of a Llama decode step around the two hot kernels (ir/.../inference/HfDecoderGraph.kt:
// embedding :904-909, rmsNorm :663-699, rope :792-818 + the two KV_CACHE_WRITEs of attention() :1230-1231,
// SwiGLU :979-988, greedy next token).  All are single-pass, HBM-bound element-wise or row-reduction kernels;
// RoPE, the KV write and the query's narrowing are one launch.
#include "common.cuh"

namespace tlaloc_b200 {
namespace {

template <typename TT>
__global__ void EmbeddingKernel(const TT* table, const int* ids, float* out, int vocab, int dim)
{
  GridDependencySync();
  const int p = blockIdx.x;
  int v = __ldg(ids + p);
  v = v < 0 ? 0 : (v >= vocab ? vocab - 1 : v);
  const TT* src = table + static_cast<size_t>(v) * dim;
  for (int d = threadIdx.x; d < dim; d += blockDim.x) out[static_cast<size_t>(p) * dim + d] = ToF32(src[d]);
}

__device__ __forceinline__ float BlockSum(float v, float* red)
{
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float r = 0.f;
  for (int w = 0; w < nw; ++w) r += red[w];
  return r;
}

// One CTA per row: x * rsqrt(mean(x^2) + eps) * gain.  mean = sum / n, rsqrt in double then narrowed, and the two
// multiplies kept separate, as the interpreter evaluates the graph's nodes (DxirInterpreter.kt:567-572,1791-1807).
// Rows of up to 8192 values (a multiple of 4) are read once with 16-byte loads, all in flight together, and kept
// in registers for the second pass; other rows take the two-pass loop.
__device__ __forceinline__ float BlockMax(float v, float* red)
{
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float r = red[0];
  for (int w = 1; w < nw; ++w) r = fmaxf(r, red[w]);
  return r;
}

// PLANES: the row is also written as the int8 tensor-core projection's activation planes (of the bf16-rounded result,
// which is what the projection would quantize): hi and lo int8 [rows, n] and the row step; only on the register path
// (the host launches the quantizer separately otherwise).
template <typename OT, bool PLANES>
__global__ void __launch_bounds__(256) RmsNormKernel(const float* x, const float* gain, OT* out, int n, float eps, int8_t* hi,
                                                     int8_t* lo, float* steps)
{
  GridDependencySync();
  __shared__ float red[8];
  const float* xr = x + static_cast<size_t>(blockIdx.x) * n;
  OT* o = out + static_cast<size_t>(blockIdx.x) * n;
  if ((n & 3) == 0 && n <= 8192 && (reinterpret_cast<uintptr_t>(xr) & 15) == 0 && (reinterpret_cast<uintptr_t>(gain) & 15) == 0) {
    const int n4 = n >> 2;
    float4 v[8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int j = threadIdx.x + i * 256;
      v[i] = j < n4 ? reinterpret_cast<const float4*>(xr)[j] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) ss = fmaf(v[i].x, v[i].x, fmaf(v[i].y, v[i].y, fmaf(v[i].z, v[i].z, fmaf(v[i].w, v[i].w, ss))));
    ss = BlockSum(ss, red);
    const float rsq = static_cast<float>(1.0 / sqrt(static_cast<double>(ss / static_cast<float>(n) + eps)));
    float amax = 0.f;
    bool bad = false;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int j = threadIdx.x + i * 256;
      if (j < n4) {
        float4 g = gain != nullptr ? reinterpret_cast<const float4*>(gain)[j] : make_float4(1.f, 1.f, 1.f, 1.f);
        const float a = __fmul_rn(v[i].x, rsq), b = __fmul_rn(v[i].y, rsq), c = __fmul_rn(v[i].z, rsq), d = __fmul_rn(v[i].w, rsq);
        const float r0 = gain != nullptr ? __fmul_rn(a, g.x) : a, r1 = gain != nullptr ? __fmul_rn(b, g.y) : b;
        const float r2 = gain != nullptr ? __fmul_rn(c, g.z) : c, r3 = gain != nullptr ? __fmul_rn(d, g.w) : d;
        o[4 * j] = FromF32<OT>(r0);
        o[4 * j + 1] = FromF32<OT>(r1);
        o[4 * j + 2] = FromF32<OT>(r2);
        o[4 * j + 3] = FromF32<OT>(r3);
        if constexpr (PLANES) {
          v[i] = make_float4(Bf16Value(r0), Bf16Value(r1), Bf16Value(r2), Bf16Value(r3));
          const float m4 = fmaxf(fmaxf(fabsf(v[i].x), fabsf(v[i].y)), fmaxf(fabsf(v[i].z), fabsf(v[i].w)));
          bad = bad || !(m4 <= 3.4e38f);
          amax = fmaxf(amax, m4);
        }
      }
    }
    if constexpr (PLANES) {
      amax = BlockMax(amax, red);
      const bool row_bad = __syncthreads_or(bad ? 1 : 0) != 0;
      float step;
      const float inv = I8RowInvStep(amax, row_bad, &step);
      if (threadIdx.x == 0) steps[blockIdx.x] = step;
      uint32_t* hrow = reinterpret_cast<uint32_t*>(hi + static_cast<size_t>(blockIdx.x) * n);
      uint32_t* lrow = reinterpret_cast<uint32_t*>(lo + static_cast<size_t>(blockIdx.x) * n);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int j = threadIdx.x + i * 256;
        if (j < n4) {
          uint32_t hw, lw;
          I8Split4(v[i].x, v[i].y, v[i].z, v[i].w, inv, hw, lw);
          hrow[j] = hw;
          lrow[j] = lw;
        }
      }
    }
    return;
  }
  float ss = 0.f;
  for (int j = threadIdx.x; j < n; j += blockDim.x) {
    const float v = xr[j];
    ss = fmaf(v, v, ss);
  }
  ss = BlockSum(ss, red);
  const float mean = ss / static_cast<float>(n);
  const float rsq = static_cast<float>(1.0 / sqrt(static_cast<double>(mean + eps)));
  for (int j = threadIdx.x; j < n; j += blockDim.x) {
    float v = __fmul_rn(xr[j], rsq);
    if (gain != nullptr) v = __fmul_rn(v, gain[j]);
    o[j] = FromF32<OT>(v);
  }
}

// The interpreter's own evaluation of the same graph nodes (parity mode): sq = x * x, mean = (sum of sq in index
// order, f32) / n, + eps, rsqrt in double, (x * rsq) * gain; one thread sums a row.
template <typename OT>
__global__ void __launch_bounds__(256) RmsNormOrderFaithfulKernel(const float* x, const float* gain, OT* out, int n, float eps)
{
  GridDependencySync();
  __shared__ float s_rsq;
  const float* xr = x + static_cast<size_t>(blockIdx.x) * n;
  OT* o = out + static_cast<size_t>(blockIdx.x) * n;
  if (threadIdx.x == 0) {
    float acc = 0.f;
    for (int j = 0; j < n; ++j) acc = __fadd_rn(acc, __fmul_rn(xr[j], xr[j]));
    const float shifted = __fadd_rn(__fdiv_rn(acc, static_cast<float>(n)), eps);
    s_rsq = static_cast<float>(1.0 / sqrt(static_cast<double>(shifted)));
  }
  __syncthreads();
  const float rsq = s_rsq;
  for (int j = threadIdx.x; j < n; j += blockDim.x) {
    float v = __fmul_rn(xr[j], rsq);
    if (gain != nullptr) v = __fmul_rn(v, gain[j]);
    o[j] = FromF32<OT>(v);
  }
}

// Grid (tokens, H + 2*Hkv): head slot h < H rotates a query head into q_out; the next Hkv rotate a key head into
// the key pool at the token's slot; the last Hkv copy a value head into the value pool.  x*cos + rotate_half(x)*sin
// with each product and the sum rounded to f32 (HfDecoderGraph.kt:792-818).
constexpr int kRopeHeadsPerCta = 8;

// One warp per (token, head slot); lane j takes the channel pairs (j, j + hd/2), (j + 32, j + 32 + hd/2), ...: both
// members of a pair need both inputs, and consecutive lanes touch consecutive addresses.
template <typename QT, typename KVT>
__global__ void __launch_bounds__(32 * kRopeHeadsPerCta)
RopeKvWriteKernel(const float* q, const float* k, const float* v, const int* positions, const float* cos_t,
                  const float* sin_t, const int* slots, QT* q_out, KVT* kc, KVT* vc, int H, int Hkv, int hd,
                  int num_slots, int max_pos, int ldq, int ldk, int ldv)
{
  GridDependencySync();
  const int t = blockIdx.x, hs = blockIdx.y * kRopeHeadsPerCta + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (hs >= H + 2 * Hkv) return;
  const int half = hd >> 1;
  if (hs < H + Hkv) {
    int pos = __ldg(positions + t);
    pos = pos < 0 ? 0 : (pos >= max_pos ? max_pos - 1 : pos);
    const float* c = cos_t + static_cast<size_t>(pos) * hd;
    const float* s = sin_t + static_cast<size_t>(pos) * hd;
    if (hs < H) {
      const float* x = q + static_cast<size_t>(t) * ldq + hs * hd;
      QT* o = q_out + (static_cast<size_t>(t) * H + hs) * hd;
      for (int j = lane; j < half; j += 32) {
        const float lo = x[j], hi = x[j + half];
        o[j] = FromF32<QT>(__fadd_rn(__fmul_rn(lo, c[j]), __fmul_rn(-hi, s[j])));
        o[j + half] = FromF32<QT>(__fadd_rn(__fmul_rn(hi, c[j + half]), __fmul_rn(lo, s[j + half])));
      }
      return;
    }
    const int slot = __ldg(slots + t);
    if (slot < 0 || slot >= num_slots) return;  // padding lane (negative) or a slot past the pool: no write
    const int h = hs - H;
    const float* x = k + static_cast<size_t>(t) * ldk + h * hd;
    KVT* o = kc + (static_cast<size_t>(slot) * Hkv + h) * hd;
    for (int j = lane; j < half; j += 32) {
      const float lo = x[j], hi = x[j + half];
      o[j] = FromF32<KVT>(__fadd_rn(__fmul_rn(lo, c[j]), __fmul_rn(-hi, s[j])));
      o[j + half] = FromF32<KVT>(__fadd_rn(__fmul_rn(hi, c[j + half]), __fmul_rn(lo, s[j + half])));
    }
    return;
  }
  const int slot = __ldg(slots + t);
  if (slot < 0 || slot >= num_slots) return;
  const int h = hs - H - Hkv;
  const float* x = v + static_cast<size_t>(t) * ldv + h * hd;
  KVT* o = vc + (static_cast<size_t>(slot) * Hkv + h) * hd;
  for (int j = lane; j < hd; j += 32) o[j] = FromF32<KVT>(x[j]);
}

__device__ __forceinline__ float SiluMul(float g, float u) { return __fmul_rn(g / (1.f + expf(-g)), u); }
// SILU as the interpreter evaluates it: in double, narrowed once (DxirInterpreter.kt:567-592).
__device__ __forceinline__ float SiluMulOrderFaithful(float g, float u)
{
  const double gd = static_cast<double>(g);
  return __fmul_rn(static_cast<float>(gd / (1.0 + exp(-gd))), u);
}
template <typename OT>
__global__ void SwigluOrderFaithfulKernel(const float* gate, const float* up, int ld, OT* out, int rows, int n)
{
  GridDependencySync();
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= static_cast<size_t>(rows) * n) return;
  const int r = static_cast<int>(i / n), c = static_cast<int>(i - static_cast<size_t>(r) * n);
  out[i] = FromF32<OT>(SiluMulOrderFaithful(gate[static_cast<size_t>(r) * ld + c], up[static_cast<size_t>(r) * ld + c]));
}

// Four columns per thread when the rows allow 16-byte accesses (VEC), else one.
template <typename OT, bool VEC>
__global__ void SwigluKernel(const float* gate, const float* up, int ld, OT* out, int rows, int n)
{
  GridDependencySync();
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (VEC) {
    const int n4 = n >> 2;
    if (i >= static_cast<size_t>(rows) * n4) return;
    const int r = static_cast<int>(i / n4), c = static_cast<int>(i - static_cast<size_t>(r) * n4) * 4;
    const float4 g = *reinterpret_cast<const float4*>(gate + static_cast<size_t>(r) * ld + c);
    const float4 u = *reinterpret_cast<const float4*>(up + static_cast<size_t>(r) * ld + c);
    OT* o = out + static_cast<size_t>(r) * n + c;
    o[0] = FromF32<OT>(SiluMul(g.x, u.x));
    o[1] = FromF32<OT>(SiluMul(g.y, u.y));
    o[2] = FromF32<OT>(SiluMul(g.z, u.z));
    o[3] = FromF32<OT>(SiluMul(g.w, u.w));
  } else {
    if (i >= static_cast<size_t>(rows) * n) return;
    const int r = static_cast<int>(i / n), c = static_cast<int>(i - static_cast<size_t>(r) * n);
    out[i] = FromF32<OT>(SiluMul(gate[static_cast<size_t>(r) * ld + c], up[static_cast<size_t>(r) * ld + c]));
  }
}

// One CTA per row; the first index of the maximum wins (DxirInterpreter.kt:2414-2426).
__global__ void __launch_bounds__(256) ArgmaxKernel(const float* x, int* out, int n)
{
  GridDependencySync();
  __shared__ float bv[8];
  __shared__ int bi[8];
  const float* xr = x + static_cast<size_t>(blockIdx.x) * n;
  float best = -INFINITY;
  int idx = 0x7fffffff;
  for (int j = threadIdx.x; j < n; j += blockDim.x) {
    const float v = xr[j];
    if (v > best || (v == best && j < idx)) {
      best = v;
      idx = j;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (ov > best || (ov == best && oi < idx)) {
      best = ov;
      idx = oi;
    }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) {
    bv[warp] = best;
    bi[warp] = idx;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < static_cast<int>(blockDim.x >> 5); ++w) {
      if (bv[w] > best || (bv[w] == best && bi[w] < idx)) {
        best = bv[w];
        idx = bi[w];
      }
    }
    // A row of NaNs (or an empty comparison) leaves idx unset: the interpreter's answer is index 0.
    out[blockIdx.x] = idx == 0x7fffffff ? 0 : idx;
  }
}

}  // namespace
}  // namespace tlaloc_b200

using namespace tlaloc_b200;

extern "C" int tlaloc_b200_embedding(const void* table, int32_t table_dtype, const int32_t* ids, float* out,
                                     int32_t positions, int32_t vocab, int32_t dim, void* stream)
{
  if (!table || !ids || !out) return Fail(kInvalid, "EMBEDDING: a required device pointer is null");
  if (!IsFloatType(table_dtype)) return Fail(kInvalid, "EMBEDDING: the table must be f32 or bf16");
  if (positions < 0 || vocab < 1 || dim < 1) return Fail(kInvalid, "EMBEDDING: bad sizes");
  if (positions == 0) return kOk;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e;
  if (table_dtype == TLALOC_B200_F32) {
    e = LaunchChained(EmbeddingKernel<float>, positions, 256, 0, st, static_cast<const float*>(table), ids, out, vocab, dim);
  } else {
    e = LaunchChained(EmbeddingKernel<__nv_bfloat16>, positions, 256, 0, st, static_cast<const __nv_bfloat16*>(table), ids, out, vocab, dim);
  }
  if (e != cudaSuccess) return CudaFail("EMBEDDING launch", e);
  CountLaunches(1);
  return kOk;
}

extern "C" int tlaloc_b200_rmsnorm(const float* x, const float* gain, void* out, int32_t out_dtype, int32_t rows,
                                   int32_t n, float eps, void* stream)
{
  if (!x || !out) return Fail(kInvalid, "RMSNORM: a required device pointer is null");
  if (!IsFloatType(out_dtype)) return Fail(kInvalid, "RMSNORM: out must be f32 or bf16");
  if (rows < 0 || n < 1) return Fail(kInvalid, "RMSNORM: bad sizes");
  if (rows == 0) return kOk;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e;
  if (OrderFaithful()) {
    e = out_dtype == TLALOC_B200_F32
            ? LaunchChained(RmsNormOrderFaithfulKernel<float>, rows, 256, 0, st, x, gain, static_cast<float*>(out), n, eps)
            : LaunchChained(RmsNormOrderFaithfulKernel<__nv_bfloat16>, rows, 256, 0, st, x, gain, static_cast<__nv_bfloat16*>(out), n, eps);
  } else if (out_dtype == TLALOC_B200_F32) {
    e = LaunchChained(RmsNormKernel<float, false>, rows, 256, 0, st, x, gain, static_cast<float*>(out), n, eps, nullptr, nullptr, nullptr);
  } else {
    e = LaunchChained(RmsNormKernel<__nv_bfloat16, false>, rows, 256, 0, st, x, gain, static_cast<__nv_bfloat16*>(out), n, eps, nullptr,
                      nullptr, nullptr);
  }
  if (e != cudaSuccess) return CudaFail("RMSNORM launch", e);
  CountLaunches(1);
  return kOk;
}

extern "C" int tlaloc_b200_rmsnorm_planes(const float* x, const float* gain, void* out, void* planes, size_t planes_bytes,
                                          int32_t rows, int32_t n, float eps, void* stream)
{
  const char* op = "RMSNORM_PLANES";
  if (!x || !out || !planes) return Fail(kInvalid, "%s: a required device pointer is null", op);
  if (rows < 0 || n < 1) return Fail(kInvalid, "%s: bad sizes", op);
  if (rows == 0) return kOk;
  if (!Aligned16(planes) || n % 16 != 0) return Fail(kInvalid, "%s: the planes must be 16-byte aligned and n a multiple of 16", op);
  if (planes_bytes < Int8GemmI8ScratchBytes(rows, n)) {
    return Fail(kInvalid, "%s: the planes of %d x %d need %zu bytes, got %zu", op, rows, n, Int8GemmI8ScratchBytes(rows, n), planes_bytes);
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // One launch when the row stays in registers; otherwise (long or unaligned rows, parity mode) the norm, then the
  // projection's own quantizer on its bf16 result.
  if (OrderFaithful() || n > 8192 || !Aligned16(x) || !Aligned16(gain)) {
    const int status = tlaloc_b200_rmsnorm(x, gain, out, TLALOC_B200_BF16, rows, n, eps, stream);
    if (status != kOk) return status;
    const cudaError_t qe = LaunchQuantizeRowsI8(out, TLALOC_B200_BF16, planes, rows, n, st);
    if (qe != cudaSuccess) return CudaFail("RMSNORM_PLANES quantizer launch", qe);
    CountLaunches(1);
    return kOk;
  }
  int8_t* hi = static_cast<int8_t*>(planes);
  int8_t* lo = hi + static_cast<size_t>(rows) * n;
  float* steps = reinterpret_cast<float*>(lo + static_cast<size_t>(rows) * n);
  const cudaError_t e = LaunchChained(RmsNormKernel<__nv_bfloat16, true>, rows, 256, 0, st, x, gain, static_cast<__nv_bfloat16*>(out), n,
                                      eps, hi, lo, steps);
  if (e != cudaSuccess) return CudaFail("RMSNORM_PLANES launch", e);
  CountLaunches(1);
  return kOk;
}

extern "C" int tlaloc_b200_rope_kv_write(const float* q, const float* k, const float* v, const int32_t* positions,
                                         const float* cos_table, const float* sin_table,
                                         const int32_t* slot_mapping, void* q_out, int32_t q_out_dtype,
                                         void* key_cache, void* value_cache, int32_t kv_dtype, int32_t num_tokens,
                                         int32_t num_heads, int32_t num_kv_heads, int32_t head_dim, int32_t num_slots,
                                         int32_t max_pos, int32_t ld_q, int32_t ld_k, int32_t ld_v, void* stream)
{
  const char* op = "ROPE_KV_WRITE";
  if (!q || !k || !v || !positions || !cos_table || !sin_table || !slot_mapping || !q_out || !key_cache || !value_cache) {
    return Fail(kInvalid, "%s: a required device pointer is null", op);
  }
  if (!IsFloatType(q_out_dtype) || !IsPoolType(kv_dtype)) return Fail(kInvalid, "%s: q_out must be f32 or bf16, the pools f32, bf16 or f8e4m3fn", op);
  if (head_dim < 2 || head_dim % 2 != 0) {
    return Fail(kInvalid, "%s: head_dim %d is odd; RoPE rotates pairs of channels (rotate_half)", op, head_dim);
  }
  if (num_tokens < 0 || num_heads < 1 || num_kv_heads < 1 || num_slots < 1 || max_pos < 1) return Fail(kInvalid, "%s: bad sizes", op);
  if (ld_q < num_heads * head_dim || ld_k < num_kv_heads * head_dim || ld_v < num_kv_heads * head_dim) {
    return Fail(kInvalid, "%s: a row stride is shorter than its row", op);
  }
  if (num_tokens == 0) return kOk;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const dim3 grid(num_tokens, (num_heads + 2 * num_kv_heads + kRopeHeadsPerCta - 1) / kRopeHeadsPerCta);
  const int threads = 32 * kRopeHeadsPerCta;
  cudaError_t e;
#define TLALOC_LAUNCH(QT, KVT)                                                                                      \
  e = LaunchChained(RopeKvWriteKernel<QT, KVT>, grid, threads, 0, st, q, k, v, positions, cos_table, sin_table,     \
                    slot_mapping, static_cast<QT*>(q_out), static_cast<KVT*>(key_cache),                           \
                    static_cast<KVT*>(value_cache), num_heads, num_kv_heads, head_dim, num_slots, max_pos, ld_q,   \
                    ld_k, ld_v)
  if (q_out_dtype == TLALOC_B200_F32 && kv_dtype == TLALOC_B200_F32) TLALOC_LAUNCH(float, float);
  else if (q_out_dtype == TLALOC_B200_F32 && kv_dtype == TLALOC_B200_BF16) TLALOC_LAUNCH(float, __nv_bfloat16);
  else if (q_out_dtype == TLALOC_B200_F32) TLALOC_LAUNCH(float, __nv_fp8_e4m3);
  else if (kv_dtype == TLALOC_B200_F32) TLALOC_LAUNCH(__nv_bfloat16, float);
  else if (kv_dtype == TLALOC_B200_BF16) TLALOC_LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else TLALOC_LAUNCH(__nv_bfloat16, __nv_fp8_e4m3);
#undef TLALOC_LAUNCH
  if (e != cudaSuccess) return CudaFail("ROPE_KV_WRITE launch", e);
  CountLaunches(1);
  return kOk;
}

extern "C" int tlaloc_b200_swiglu(const float* gate, const float* up, int32_t ld, void* out, int32_t out_dtype,
                                  int32_t rows, int32_t n, void* stream)
{
  if (!gate || !up || !out) return Fail(kInvalid, "SWIGLU: a required device pointer is null");
  if (!IsFloatType(out_dtype)) return Fail(kInvalid, "SWIGLU: out must be f32 or bf16");
  if (rows < 0 || n < 1 || ld < n) return Fail(kInvalid, "SWIGLU: bad sizes");
  if (rows == 0) return kOk;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool vec = n % 4 == 0 && ld % 4 == 0 && (reinterpret_cast<uintptr_t>(gate) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(up) & 15) == 0;
  const size_t total = static_cast<size_t>(rows) * (vec ? n / 4 : n);
  const unsigned blocks = static_cast<unsigned>((total + 255) / 256);
  cudaError_t e;
  if (OrderFaithful()) {
    const unsigned fb = static_cast<unsigned>((static_cast<size_t>(rows) * n + 255) / 256);
    e = out_dtype == TLALOC_B200_F32
            ? LaunchChained(SwigluOrderFaithfulKernel<float>, fb, 256, 0, st, gate, up, ld, static_cast<float*>(out), rows, n)
            : LaunchChained(SwigluOrderFaithfulKernel<__nv_bfloat16>, fb, 256, 0, st, gate, up, ld, static_cast<__nv_bfloat16*>(out), rows, n);
  } else if (out_dtype == TLALOC_B200_F32) {
    e = vec ? LaunchChained(SwigluKernel<float, true>, blocks, 256, 0, st, gate, up, ld, static_cast<float*>(out), rows, n)
            : LaunchChained(SwigluKernel<float, false>, blocks, 256, 0, st, gate, up, ld, static_cast<float*>(out), rows, n);
  } else {
    e = vec ? LaunchChained(SwigluKernel<__nv_bfloat16, true>, blocks, 256, 0, st, gate, up, ld, static_cast<__nv_bfloat16*>(out), rows, n)
            : LaunchChained(SwigluKernel<__nv_bfloat16, false>, blocks, 256, 0, st, gate, up, ld, static_cast<__nv_bfloat16*>(out), rows, n);
  }
  if (e != cudaSuccess) return CudaFail("SWIGLU launch", e);
  CountLaunches(1);
  return kOk;
}

extern "C" int tlaloc_b200_argmax(const float* logits, int32_t* out, int32_t rows, int32_t n, void* stream)
{
  if (!logits || !out) return Fail(kInvalid, "ARGMAX: a required device pointer is null");
  if (rows < 0 || n < 1) return Fail(kInvalid, "ARGMAX: bad sizes");
  if (rows == 0) return kOk;
  const cudaError_t e = LaunchChained(ArgmaxKernel, rows, 256, 0, static_cast<cudaStream_t>(stream), logits, out, n);
  if (e != cudaSuccess) return CudaFail("ARGMAX launch", e);
  CountLaunches(1);
  return kOk;
}
