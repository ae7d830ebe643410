// The int8 weight-only projection y = (cast(x) @ cast(codes)) * scale for sm_100a
// (HfDecoderGraph.proj over WeightQuant.INT8, ir/.../inference/HfDecoderGraph.kt:625-655).
//
//   Int8GemvKernel   decode rows (M <= 32 per launch; more rows run as several launches).  HBM-bound: every
//                    weight byte is read once, straight from global memory into registers with 16-byte
//                    coalesced loads of the reference's own [K, N] layout (no repacking).  A CTA owns 128
//                    output columns and one slice of K; its eight warps split the slice's 16-row steps.  The
//                    int8 codes become exact bf16 pairs in registers (one byte-permute, two logic ops and one
//                    packed bf16 add per pair), the activations wait in shared memory as bf16 (double-buffered
//                    cp.async chunks), and the products run on mma.sync m16n8k16 bf16 with fp32 accumulators.
//                    The K slices of one column tile form a thread-block cluster and are summed through
//                    distributed shared memory in rank order, so there is no global scratch, no second
//                    kernel, and the result does not depend on timing.  The per-column scale (and an optional
//                    residual) is applied to the finished sum, as the graph multiplies after the dot.
//   GemmExactKernel  the interpreter's MATMUL order (DxirInterpreter.kt:739-765): f32, k ascending, separate
//                    multiply and add, zero activations skipped.  Bit-identical to the CPU oracle; slow.
#include <cooperative_groups.h>

#include <mutex>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace tlaloc_b200 {
namespace {

struct GemmParams {
  const __nv_bfloat16* x;  // [M, K] bf16
  const int8_t* w;         // [K, N]
  const float* scales;     // [N] or null
  const float* residual;   // [M, N] or null
  void* y;                 // [M, N]
  int M, K, N;
  int Kc;  // K per CTA (multiple of 16 * kGvWarps)
  int ks;  // K slices (cluster size along y)
};

constexpr int kGvThreads = 256;
constexpr int kGvWarps = 8;
constexpr int kGvCols = 128;
constexpr int kGvChunk = 1024;            // k per activation chunk in shared memory
constexpr int kGvXStride = kGvChunk + 8;  // bf16 elements per staged row (16 bytes of padding: conflict-free ldmatrix)
constexpr int kGvRedStride = kGvCols + 4;

__device__ __forceinline__ uint32_t SmemAddr(const void* ptr)
{
  return static_cast<uint32_t>(__cvta_generic_to_shared(ptr));
}
__device__ __forceinline__ void CpAsync16(uint32_t dst, const void* src, int src_bytes)
{
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void CpAsyncCommit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void CpAsyncWait()
{
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}
__device__ __forceinline__ void LdMatrixX4(uint32_t (&r)[4], uint32_t addr)
{
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void MmaBf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
{
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// Streaming 16-byte load of weights: read once, kept out of L1.
__device__ __forceinline__ uint4 LoadW(const int8_t* ptr)
{
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(ptr));
  return v;
}
// Bytes `b` of two words (codes of two consecutive k for one column) as an exact bf16 pair, lower k in the low
// half.  For a code v with bits s:lo7, 0x4300|lo7 is the bf16 128 + lo7 and 0xC300|s<<7 is -128 or -256; their
// sum is v, exactly.
template <int B>
__device__ __forceinline__ uint32_t CodesToBf16x2(uint32_t w_lo_k, uint32_t w_hi_k)
{
  const uint32_t q = __byte_perm(w_lo_k, w_hi_k, B | (B << 4) | ((4 + B) << 8) | ((4 + B) << 12));
  const uint32_t t = (q & 0x007F007Fu) | 0x43004300u;
  const uint32_t c = (q & 0x00800080u) | 0xC300C300u;
  uint32_t r;
  asm("add.rn.bf16x2 %0, %1, %2;\n" : "=r"(r) : "r"(t), "r"(c));
  return r;
}

template <int MT>
struct GvLayout {
  static constexpr int kRows = MT * 16;
  static constexpr int kXBytes = kRows * kGvXStride * 2;  // one activation chunk
  static constexpr int kRedBytes = kGvWarps * kRows * kGvRedStride * 4;
  static constexpr int kTileBytes = kRows * kGvRedStride * 4;
  // The two activation buffers and the warps' partial tiles share one space (the partials come last).
  static constexpr int kMainBytes = 2 * kXBytes > kRedBytes ? 2 * kXBytes : kRedBytes;
  static constexpr int kBytes = kMainBytes + kTileBytes;
};

template <int MT, int U, typename YT>
__global__ void __launch_bounds__(kGvThreads, 1) Int8GemvKernel(GemmParams p)
{
  using L = GvLayout<MT>;
  extern __shared__ __align__(128) unsigned char smem[];
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(smem);  // [2][kRows][kGvXStride]
  float* red = reinterpret_cast<float*>(smem);                 // [kGvWarps][kRows][kGvRedStride] (after the loop)
  float* tile = reinterpret_cast<float*>(smem + L::kMainBytes);  // [kRows][kGvRedStride]

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int gid = lane >> 2, tig = lane & 3;
  const int col0 = blockIdx.x * kGvCols;
  const int kb = blockIdx.y * p.Kc;
  const int ke = min(p.K, kb + p.Kc);
  const int nsteps = ke > kb ? (ke - kb + 15) >> 4 : 0;          // this CTA's 16-row steps
  const int nchunks = (nsteps * 16 + kGvChunk - 1) / kGvChunk;    // activation chunks
  constexpr int kStepsPerWarpChunk = kGvChunk / 16 / kGvWarps;    // 8
  constexpr int kGroupsPerChunk = kStepsPerWarpChunk / U;
  const int my_col = col0 + gid * 16;
  const bool col_ok = my_col < p.N;

  // Activation chunk c -> buffer c & 1: rows m < M copy 16-byte pieces of x[m, kb + c*chunk ...), the rest zero.
  auto stage_x = [&](int c) {
    __nv_bfloat16* dst = xs + (c & 1) * (L::kRows * kGvXStride);
    const int k_lo = kb + c * kGvChunk;
    for (int idx = tid; idx < L::kRows * (kGvChunk / 8); idx += kGvThreads) {
      const int m = idx / (kGvChunk / 8), piece = idx - m * (kGvChunk / 8);
      const int k = k_lo + piece * 8;
      // K is a multiple of 8 on this path, so a piece is wholly inside or outside [0, K).
      const bool valid = m < p.M && k < ke;
      const __nv_bfloat16* src = p.x + (valid ? static_cast<size_t>(m) * p.K + k : 0);
      CpAsync16(SmemAddr(dst + m * kGvXStride + piece * 8), src, valid ? 16 : 0);
    }
  };
  // The weights of step j (16 rows of K) for this lane: rows 2*tig + {0, 1, 8, 9}, 16 columns from my_col.
  auto load_w = [&](int j, uint4 (&r)[4]) {
    const int k0 = kb + 16 * j + 2 * tig;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int row = k0 + (q & 1) + (q >> 1) * 8;
      if (j < nsteps && row < ke && col_ok) r[q] = LoadW(p.w + static_cast<size_t>(row) * p.N + my_col);
      else r[q] = make_uint4(0u, 0u, 0u, 0u);
    }
  };

  float acc[MT][16][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int nt = 0; nt < 16; ++nt) acc[mt][nt][0] = acc[mt][nt][1] = acc[mt][nt][2] = acc[mt][nt][3] = 0.f;

  auto compute = [&](int j, const uint4 (&r)[4], const __nv_bfloat16* xbuf) {
    if (j >= nsteps) return;
    const int kl = (16 * j) % kGvChunk;  // step's first k inside its chunk
    uint32_t a[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      const int row = mt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
      LdMatrixX4(a[mt], SmemAddr(xbuf + row * kGvXStride + kl + (lane >> 4) * 8));
    }
    const uint32_t wa[4] = {r[0].x, r[0].y, r[0].z, r[0].w}, wb[4] = {r[1].x, r[1].y, r[1].z, r[1].w};
    const uint32_t wc[4] = {r[2].x, r[2].y, r[2].z, r[2].w}, wd[4] = {r[3].x, r[3].y, r[3].z, r[3].w};
#pragma unroll
    for (int wi = 0; wi < 4; ++wi) {
      uint32_t b0[4], b1[4];
      b0[0] = CodesToBf16x2<0>(wa[wi], wb[wi]);
      b0[1] = CodesToBf16x2<1>(wa[wi], wb[wi]);
      b0[2] = CodesToBf16x2<2>(wa[wi], wb[wi]);
      b0[3] = CodesToBf16x2<3>(wa[wi], wb[wi]);
      b1[0] = CodesToBf16x2<0>(wc[wi], wd[wi]);
      b1[1] = CodesToBf16x2<1>(wc[wi], wd[wi]);
      b1[2] = CodesToBf16x2<2>(wc[wi], wd[wi]);
      b1[3] = CodesToBf16x2<3>(wc[wi], wd[wi]);
#pragma unroll
      for (int bi = 0; bi < 4; ++bi) {
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) MmaBf16(acc[mt][wi * 4 + bi], a[mt], b0[bi], b1[bi]);
      }
    }
  };

  // Warp `warp` takes steps warp, warp + 8, ...; U of them form a group whose weights are loaded together,
  // one group ahead of the one being multiplied.
  uint4 wcur[U][4], wnxt[U][4];
  auto load_group = [&](int g, uint4 (&buf)[U][4]) {
#pragma unroll
    for (int u = 0; u < U; ++u) load_w(warp + kGvWarps * (g * U + u), buf[u]);
  };
  auto compute_group = [&](int g, const uint4 (&buf)[U][4], const __nv_bfloat16* xbuf) {
#pragma unroll
    for (int u = 0; u < U; ++u) compute(warp + kGvWarps * (g * U + u), buf[u], xbuf);
  };

  if (nchunks > 0) {
    stage_x(0);
    CpAsyncCommit();
    load_group(0, wcur);
  }
  for (int c = 0; c < nchunks; ++c) {
    if (c + 1 < nchunks) stage_x(c + 1);
    CpAsyncCommit();
    CpAsyncWait<1>();
    __syncthreads();  // chunk c is in shared memory for every warp
    const __nv_bfloat16* xbuf = xs + (c & 1) * (L::kRows * kGvXStride);
    static_assert(kGroupsPerChunk % 2 == 0, "groups alternate between two register sets");
#pragma unroll 1
    for (int gg = 0; gg < kGroupsPerChunk; gg += 2) {
      const int g = c * kGroupsPerChunk + gg;
      load_group(g + 1, wnxt);
      compute_group(g, wcur, xbuf);
      load_group(g + 2, wcur);
      compute_group(g + 1, wnxt, xbuf);
    }
    __syncthreads();  // before chunk c + 2 overwrites this buffer
  }
  CpAsyncWait<0>();
  __syncthreads();

  // The eight warps' partial tiles -> shared memory -> one tile, summed in warp order.
  {
    float* mine = red + warp * (L::kRows * kGvRedStride);
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
      for (int nt = 0; nt < 16; ++nt) {
        // accumulator columns 2*tig, 2*tig+1 of n-tile nt are output columns col0 + (2*tig + e)*16 + nt
        const int m0 = mt * 16 + gid;
        mine[m0 * kGvRedStride + (2 * tig) * 16 + nt] = acc[mt][nt][0];
        mine[m0 * kGvRedStride + (2 * tig + 1) * 16 + nt] = acc[mt][nt][1];
        mine[(m0 + 8) * kGvRedStride + (2 * tig) * 16 + nt] = acc[mt][nt][2];
        mine[(m0 + 8) * kGvRedStride + (2 * tig + 1) * 16 + nt] = acc[mt][nt][3];
      }
    }
  }
  __syncthreads();
  for (int e = tid; e < L::kRows * kGvCols; e += kGvThreads) {
    const int m = e / kGvCols, c = e - m * kGvCols;
    float v = 0.f;
#pragma unroll
    for (int w = 0; w < kGvWarps; ++w) v += red[w * (L::kRows * kGvRedStride) + m * kGvRedStride + c];
    tile[m * kGvRedStride + c] = v;
  }
  // The K slices of this column tile are the ranks of one cluster: rank r finishes every ks-th row.
  cg::cluster_group cluster = cg::this_cluster();
  const unsigned rank = cluster.block_rank(), nranks = cluster.num_blocks();
  cluster.sync();
  YT* y = static_cast<YT*>(p.y);
  for (int m = rank; m < p.M; m += nranks) {
    for (int c = tid; c < kGvCols; c += kGvThreads) {
      const int col = col0 + c;
      if (col >= p.N) continue;
      float v = 0.f;
      for (unsigned q = 0; q < nranks; ++q) v += cluster.map_shared_rank(tile, q)[m * kGvRedStride + c];
      if (p.scales != nullptr) v *= __ldg(p.scales + col);
      if (p.residual != nullptr) v += __ldg(p.residual + static_cast<size_t>(m) * p.N + col);
      y[static_cast<size_t>(m) * p.N + col] = FromF32<YT>(v);
    }
  }
  cluster.sync();  // no CTA leaves while a peer may still read its tile
}

// ------------------------------------------------------------------------------------------

template <typename XT>
__global__ void ToBf16Kernel(const XT* x, __nv_bfloat16* out, size_t n)
{
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) out[i] = __float2bfloat16_rn(ToF32(x[i]));
}

// y[i, j] = (sum over p ascending of x[i, p] * w[p, j], f32, separate multiply and add, x == 0 skipped) * scale[j]
// (+ residual).  Grid (ceil(N / 256), M).
template <typename XT, typename WT, typename YT>
__global__ void __launch_bounds__(256) GemmExactKernel(const XT* x, const WT* w, const float* scales,
                                                       const float* residual, YT* y, int M, int K, int N,
                                                       int round_x)
{
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  const int i = blockIdx.y;
  if (j >= N) return;
  float acc = 0.f;
  for (int p = 0; p < K; ++p) {
    float a = ToF32(x[static_cast<size_t>(i) * K + p]);
    if (round_x) a = __bfloat162float(__float2bfloat16_rn(a));
    if (a == 0.f) continue;
    acc = __fadd_rn(acc, __fmul_rn(a, ToF32(w[static_cast<size_t>(p) * N + j])));
  }
  if (scales != nullptr) acc = __fmul_rn(acc, scales[j]);
  if (residual != nullptr) acc = __fadd_rn(acc, residual[static_cast<size_t>(i) * N + j]);
  y[static_cast<size_t>(i) * N + j] = FromF32<YT>(acc);
}

template <int MT, int U, typename YT>
cudaError_t PrepareGemv()
{
  return cudaFuncSetAttribute(Int8GemvKernel<MT, U, YT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              GvLayout<MT>::kBytes);
}

template <int MT, int U, typename YT>
cudaError_t LaunchGemv(const GemmParams& p, cudaStream_t stream)
{
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((p.N + kGvCols - 1) / kGvCols, p.ks, 1);
  cfg.blockDim = dim3(kGvThreads, 1, 1);
  cfg.dynamicSmemBytes = GvLayout<MT>::kBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = p.ks;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, Int8GemvKernel<MT, U, YT>, p);
}

// K slices for a shape: enough CTAs to fill the 148 SMs a few times over, each slice at least one full round of
// the eight warps; 1, 2, 4 or 8 (the portable cluster sizes).  $TLALOC_B200_GEMV_KS overrides.
int ChooseSlices(int k, int n)
{
  static const int forced = [] {
    const char* e = std::getenv("TLALOC_B200_GEMV_KS");
    return e != nullptr ? std::atoi(e) : 0;
  }();
  if (forced == 1 || forced == 2 || forced == 4 || forced == 8) return forced;
  const int tiles = (n + kGvCols - 1) / kGvCols;
  int ks = 1;
  while (ks < 8 && tiles * ks < 3 * 148 && k / (ks * 2) >= 16 * kGvWarps * 2) ks *= 2;
  return ks;
}

}  // namespace

cudaError_t PrepareInt8GemmKernels()
{
  static std::mutex mu;
  static bool done = false;
  std::lock_guard<std::mutex> lock(mu);
  if (done) return cudaSuccess;
  cudaError_t e = PrepareGemv<1, 4, float>();
  if (e == cudaSuccess) e = PrepareGemv<1, 4, __nv_bfloat16>();
  if (e == cudaSuccess) e = PrepareGemv<2, 2, float>();
  if (e == cudaSuccess) e = PrepareGemv<2, 2, __nv_bfloat16>();
  if (e == cudaSuccess) done = true;
  return e;
}

}  // namespace tlaloc_b200

using namespace tlaloc_b200;

namespace {

bool FastShape(int k, int n) { return n % 16 == 0 && k % 8 == 0 && k >= 16; }

template <typename XT, typename WT>
cudaError_t LaunchExact(const void* x, const void* w, const float* scales, const float* residual, void* y,
                        int y_dtype, int m, int k, int n, int round_x, cudaStream_t st)
{
  const dim3 grid((n + 255) / 256, m);
  if (y_dtype == TLALOC_B200_F32) {
    GemmExactKernel<<<grid, 256, 0, st>>>(static_cast<const XT*>(x), static_cast<const WT*>(w), scales, residual,
                                          static_cast<float*>(y), m, k, n, round_x);
  } else {
    GemmExactKernel<<<grid, 256, 0, st>>>(static_cast<const XT*>(x), static_cast<const WT*>(w), scales, residual,
                                          static_cast<__nv_bfloat16*>(y), m, k, n, round_x);
  }
  return cudaGetLastError();
}

}  // namespace

extern "C" size_t tlaloc_b200_int8_gemm_scratch_bytes(int32_t m, int32_t k, int32_t n)
{
  (void)n;
  if (m <= 0 || k <= 0) return 0;
  // Room for a bf16 copy of an f32 activation matrix.
  return sizeof(__nv_bfloat16) * static_cast<size_t>(m) * k;
}

extern "C" int tlaloc_b200_int8_gemm(const void* x, int32_t x_dtype, const int8_t* codes, const float* scales,
                                     const float* residual, void* y, int32_t y_dtype, float* scratch,
                                     size_t scratch_bytes, int32_t m, int32_t k, int32_t n, int32_t flags,
                                     void* stream)
{
  const char* op = "INT8_PROJ";
  if (!x || !codes || !y) return Fail(kInvalid, "%s: a required device pointer is null", op);
  if (!IsFloatType(x_dtype) || !IsFloatType(y_dtype)) return Fail(kInvalid, "%s: x and y must be f32 or bf16", op);
  if (m < 1 || k < 1 || n < 1) return Fail(kInvalid, "%s: needs positive [M, K] x [K, N], got M %d K %d N %d", op, m, k, n);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e;
  if ((flags & TLALOC_B200_GEMM_EXACT) != 0 || !FastShape(k, n)) {
    const int round_x = x_dtype == TLALOC_B200_F32 && (flags & TLALOC_B200_GEMM_X_F32_EXACT) == 0;
    e = x_dtype == TLALOC_B200_F32
            ? LaunchExact<float, int8_t>(x, codes, scales, residual, y, y_dtype, m, k, n, round_x, st)
            : LaunchExact<__nv_bfloat16, int8_t>(x, codes, scales, residual, y, y_dtype, m, k, n, 0, st);
    if (e != cudaSuccess) return CudaFail("INT8_PROJ exact launch", e);
    CountLaunches(1);
    return kOk;
  }
  e = PrepareInt8GemmKernels();
  if (e != cudaSuccess) return CudaFail("INT8_PROJ set-up", e);
  const __nv_bfloat16* xb = static_cast<const __nv_bfloat16*>(x);
  if (x_dtype == TLALOC_B200_F32) {
    const size_t need = sizeof(__nv_bfloat16) * static_cast<size_t>(m) * k;
    if (scratch == nullptr || scratch_bytes < need) {
      return Fail(kInvalid, "%s: an f32 x needs %zu bytes of scratch for its bf16 copy, got %zu", op, need, scratch_bytes);
    }
    const size_t count = static_cast<size_t>(m) * k;
    ToBf16Kernel<<<static_cast<unsigned>((count + 255) / 256), 256, 0, st>>>(static_cast<const float*>(x),
                                                                            reinterpret_cast<__nv_bfloat16*>(scratch), count);
    e = cudaGetLastError();
    if (e != cudaSuccess) return CudaFail("INT8_PROJ activation cast", e);
    CountLaunches(1);
    xb = reinterpret_cast<const __nv_bfloat16*>(scratch);
  }
  GemmParams p;
  p.w = codes;
  p.scales = scales;
  p.K = k;
  p.N = n;
  p.ks = ChooseSlices(k, n);
  const int per = (k + p.ks - 1) / p.ks;
  p.Kc = (per + 16 * kGvWarps - 1) / (16 * kGvWarps) * (16 * kGvWarps);
  const size_t ybytes = DtypeBytes(y_dtype);
  for (int m0 = 0; m0 < m; m0 += 32) {
    const int rows = std::min(32, m - m0);
    p.M = rows;
    p.x = xb + static_cast<size_t>(m0) * k;
    p.residual = residual ? residual + static_cast<size_t>(m0) * n : nullptr;
    p.y = static_cast<unsigned char*>(y) + static_cast<size_t>(m0) * n * ybytes;
    if (rows <= 16) {
      e = y_dtype == TLALOC_B200_F32 ? LaunchGemv<1, 4, float>(p, st) : LaunchGemv<1, 4, __nv_bfloat16>(p, st);
    } else {
      e = y_dtype == TLALOC_B200_F32 ? LaunchGemv<2, 2, float>(p, st) : LaunchGemv<2, 2, __nv_bfloat16>(p, st);
    }
    if (e != cudaSuccess) return CudaFail("INT8_PROJ launch", e);
    CountLaunches(1);
  }
  return kOk;
}

extern "C" int tlaloc_b200_dense_gemm_exact(const void* x, int32_t x_dtype, const void* w, int32_t w_dtype, float* y,
                                            int32_t m, int32_t k, int32_t n, int32_t flags, void* stream)
{
  const char* op = "MATMUL";
  if (!x || !w || !y) return Fail(kInvalid, "%s: a required device pointer is null", op);
  if (!IsFloatType(x_dtype) || !IsFloatType(w_dtype)) return Fail(kInvalid, "%s: x and w must be f32 or bf16", op);
  if (m < 1 || k < 1 || n < 1) return Fail(kInvalid, "%s: needs positive [M, K] x [K, N], got M %d K %d N %d", op, m, k, n);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // An f32 x meets a bf16 weight as bf16 (HfDecoderGraph.kt:641-647) unless the caller keeps it f32.
  const int round_x = x_dtype == TLALOC_B200_F32 && w_dtype == TLALOC_B200_BF16 && (flags & TLALOC_B200_GEMM_X_F32_EXACT) == 0;
  cudaError_t e;
  if (x_dtype == TLALOC_B200_F32 && w_dtype == TLALOC_B200_F32) {
    e = LaunchExact<float, float>(x, w, nullptr, nullptr, y, TLALOC_B200_F32, m, k, n, 0, st);
  } else if (x_dtype == TLALOC_B200_F32) {
    e = LaunchExact<float, __nv_bfloat16>(x, w, nullptr, nullptr, y, TLALOC_B200_F32, m, k, n, round_x, st);
  } else if (w_dtype == TLALOC_B200_F32) {
    e = LaunchExact<__nv_bfloat16, float>(x, w, nullptr, nullptr, y, TLALOC_B200_F32, m, k, n, 0, st);
  } else {
    e = LaunchExact<__nv_bfloat16, __nv_bfloat16>(x, w, nullptr, nullptr, y, TLALOC_B200_F32, m, k, n, 0, st);
  }
  if (e != cudaSuccess) return CudaFail("MATMUL exact launch", e);
  CountLaunches(1);
  return kOk;
}
