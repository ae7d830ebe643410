// The int8 weight-only projection y = (cast(x) @ cast(codes)) * scale for sm_100a
// (HfDecoderGraph.proj over WeightQuant.INT8, ir/.../inference/HfDecoderGraph.kt:625-655).
//
//   Int8GemvKernel   decode rows (M <= 32 per launch; by default only up to 16 rows come here, 17 and more go to the
//                    tensor-core kernels of int8_gemm_tc.cu and int8_gemm_i8.cu).  HBM-bound: every
//                    weight byte is read once, from the reference's own [K, N] layout (no repacking).  A CTA owns
//                    128 output columns and one slice of K; each of its four warps is an independent cp.async
//                    pipeline over its own 32-row stages (a 32 x 128 int8 weight tile plus the matching 32-wide
//                    strip of the bf16 activations, XOR-swizzled in shared memory), so there is no CTA-wide barrier
//                    in the loop and four CTAs fit an SM.  The MMA runs transposed: the 16 output columns a lane
//                    pair-set owns are the M dimension and the (<= 8 per n-tile) activation rows the N dimension, so
//                    one 16-row step costs 8 mma.sync m16n8k16 per n-tile.  The int8 codes become exact bf16 pairs in
//                    registers (one byte-permute, two logic ops and one packed bf16 add per pair); products are
//                    exact, accumulation fp32.  The K slices of one column tile form a thread-block cluster and are
//                    summed through distributed shared memory in rank order: no global scratch, no second kernel,
//                    and a result that does not depend on timing.  The per-column scale (and an optional residual)
//                    is applied to the finished sum, as the graph multiplies after the dot.
//   GemmExactKernel  the interpreter's MATMUL order (DxirInterpreter.kt:739-765): f32, k ascending, separate
//                    multiply and add, zero activations skipped.  Bit-identical to the CPU oracle; slow.
#include <cooperative_groups.h>

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
  int Kc;  // K per CTA (a multiple of kGvStageK * kGvWarps)
  int ks;  // K slices (cluster size along y)
  int weights_const;  // no kernel still in flight writes codes or scales: the first weight stages are fetched before the dependency wait
};

constexpr int kGvThreads = 128;
constexpr int kGvWarps = 4;
constexpr int kGvCols = 128;
constexpr int kGvStageK = 32;  // k rows per pipeline stage
constexpr int kGvStages = 3;
constexpr int kGvWBytes = kGvStageK * kGvCols;  // the stage's weight tile
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
__device__ __forceinline__ void LdMatrixX2(uint32_t (&r)[2], uint32_t addr)
{
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
__device__ __forceinline__ uint4 LdShared16(uint32_t addr)
{
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ void MmaBf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
{
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// Bytes `B` of two words (codes of two consecutive k for one column) as an exact bf16 pair, lower k in the low
// half.  For a code v with bits s:lo7, 0x4300|lo7 is the bf16 128 + lo7 and 0xC300|s<<7 is -128 or -256; their
// sum is v, exactly.
template <int B>
__device__ __forceinline__ uint32_t CodesToBf16x2(uint32_t w_lo_k, uint32_t w_hi_k)
{
  const uint32_t q = __byte_perm(w_lo_k, w_hi_k, B | (B << 4) | ((4 + B) << 8) | ((4 + B) << 12));
  uint32_t t, c;  // (q & mask) | magic as one three-input logic op each
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;\n" : "=r"(t) : "r"(q), "r"(0x007F007Fu), "r"(0x43004300u));
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;\n" : "=r"(c) : "r"(q), "r"(0x00800080u), "r"(0xC300C300u));
  uint32_t r;
  asm("fma.rn.bf16x2 %0, %1, %2, %3;\n" : "=r"(r) : "r"(t), "r"(0x3F803F80u), "r"(c));
  return r;
}

template <int NT>
struct GvLayout {
  static constexpr int kRows = NT * 8;                     // activation rows a launch covers
  static constexpr int kXBytes = kRows * kGvStageK * 2;    // the stage's activation strip, [rows][32] bf16
  static constexpr int kStageBytes = kGvWBytes + kXBytes;
  static constexpr int kWarpBytes = kGvStages * kStageBytes;
  static constexpr int kPipeBytes = kGvWarps * kWarpBytes;
  // After the loop the same space holds the four warps' partial tiles and the CTA's summed tile.
  static constexpr int kTileBytes = kRows * kGvRedStride * 4;
  static constexpr int kRedBytes = (kGvWarps + 1) * kTileBytes;
  static constexpr int kBytes = kPipeBytes > kRedBytes ? kPipeBytes : kRedBytes;
};

template <int NT, typename YT>
__global__ void __launch_bounds__(kGvThreads) Int8GemvKernel(GemmParams p)
{
  if (!p.weights_const) GridDependencySync();
  using L = GvLayout<NT>;
  extern __shared__ __align__(128) unsigned char smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int gid = lane >> 2, tig = lane & 3;
  const int col0 = blockIdx.x * kGvCols;
  const int kb = blockIdx.y * p.Kc;
  const int ke = min(p.K, kb + p.Kc);
  const int nstages = ke > kb ? (ke - kb + kGvStageK - 1) / kGvStageK : 0;
  const int my_n = warp < nstages ? (nstages - warp + kGvWarps - 1) / kGvWarps : 0;
  const uint32_t my_pipe_addr = SmemAddr(smem + warp * L::kWarpBytes);

  // Copies of one stage (k rows [k0, k0 + 32) of this warp), all lane-invariant parts computed once.
  //   weights: copy i of lane (l3 = lane >> 3, ch = lane & 7) moves row l3 + 4i, 16-byte chunk ch, to chunk
  //            ch ^ (row & 6): (row & 6) is (l3 & 2) for even i and (l3 & 2) | 4 for odd i;
  //   activations: copy i moves row (lane >> 2) + 8i, 16-byte piece lane & 3, to piece ^ ((row >> 1) & 3).
  // The reads further down are then conflict-free.  K is a multiple of 8 and N of 16 on this path, so a chunk is
  // wholly inside or outside the matrix; outside is zero-filled.
  const int l3 = lane >> 3, ch = lane & 7;
  const bool col_ok = col0 + ch * 16 < p.N;
  const uint32_t wdst_even = l3 * kGvCols + ((ch ^ (l3 & 2)) << 4);
  const uint32_t wdst_odd = (l3 + 4) * kGvCols + ((ch ^ ((l3 & 2) | 4)) << 4);
  const size_t w_row4 = static_cast<size_t>(4) * p.N;
  const int8_t* w_lane = p.w + static_cast<size_t>(kb + warp * kGvStageK + l3) * p.N + col0 + (col_ok ? ch * 16 : 0);
  const size_t w_stage = static_cast<size_t>(kGvWarps * kGvStageK) * p.N;
  const int xm = lane >> 2, xpiece = lane & 3;
  const uint32_t xdst = kGvWBytes + xm * (kGvStageK * 2) + ((xpiece ^ ((xm >> 1) & 3)) << 4);
  const __nv_bfloat16* x_lane = p.x + static_cast<size_t>(xm) * p.K + kb + warp * kGvStageK + xpiece * 8;

  // A stage's copies in two parts: the weights, which with weights_const depend on no earlier kernel, and the activations.
  auto issue_w = [&](int it) {
    const int k0 = kb + (warp + kGvWarps * it) * kGvStageK;
    const uint32_t dst = my_pipe_addr + (it % kGvStages) * L::kStageBytes;
    const int8_t* src = w_lane + it * w_stage;
    if (k0 + kGvStageK <= ke) {  // the whole stage is inside K
      const int bytes = col_ok ? 16 : 0;
#pragma unroll
      for (int i = 0; i < 8; i += 2) {
        CpAsync16(dst + wdst_even + i * (4 * kGvCols), src + i * w_row4, bytes);
        CpAsync16(dst + wdst_odd + i * (4 * kGvCols), src + (i + 1) * w_row4, bytes);
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const bool valid = col_ok && k0 + l3 + 4 * i < ke;
        CpAsync16(dst + ((i & 1) ? wdst_odd - 4 * kGvCols : wdst_even) + i * (4 * kGvCols), valid ? src + i * w_row4 : p.w, valid ? 16 : 0);
      }
    }
  };
  auto issue_x = [&](int it) {
    const int k0 = kb + (warp + kGvWarps * it) * kGvStageK;
    const uint32_t dst = my_pipe_addr + (it % kGvStages) * L::kStageBytes;
    if (k0 + kGvStageK <= ke) {
#pragma unroll
      for (int i = 0; i < NT; ++i) {
        const bool valid = xm + 8 * i < p.M;
        CpAsync16(dst + xdst + i * (8 * kGvStageK * 2), x_lane + (valid ? static_cast<size_t>(8 * i) * p.K + it * (kGvWarps * kGvStageK) : 0),
                  valid ? 16 : 0);
      }
    } else {
#pragma unroll
      for (int i = 0; i < NT; ++i) {
        const bool valid = xm + 8 * i < p.M && k0 + xpiece * 8 < ke;
        CpAsync16(dst + xdst + i * (8 * kGvStageK * 2),
                  valid ? x_lane + static_cast<size_t>(8 * i) * p.K + it * (kGvWarps * kGvStageK) : p.x, valid ? 16 : 0);
      }
    }
  };
  auto issue = [&](int it) {
    issue_w(it);
    issue_x(it);
  };

  if (p.weights_const) {
    // The weights of the first stages are on their way while the previous kernel drains; the first commit group then
    // holds all of them together with the first stage's activations.
    for (int it = 0; it < kGvStages - 1; ++it)
      if (it < my_n) issue_w(it);
    GridDependencySync();
    for (int it = 0; it < kGvStages - 1; ++it) {
      if (it < my_n) issue_x(it);
      CpAsyncCommit();
    }
  } else {
    for (int it = 0; it < kGvStages - 1; ++it) {
      if (it < my_n) issue(it);
      CpAsyncCommit();
    }
  }

  // acc[j][nt]: output columns col0 + gid*16 + 2j (c0, c1) and + 2j + 1 (c2, c3), activation rows nt*8 + 2tig, + 1.
  float acc[8][NT][4];
#pragma unroll
  for (int j = 0; j < 8; ++j)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) acc[j][nt][0] = acc[j][nt][1] = acc[j][nt][2] = acc[j][nt][3] = 0.f;

  // Reads of a stage.  Weights: this lane's 16 columns (chunk gid) of rows 2tig + {0, 1, 8, 9} of each 16-row step;
  // for all of them (row & 6) == 2tig.  Activations (ldmatrix): row lane & 7 of the n-tile, piece 2h + ((lane >> 3) & 1).
  const uint32_t wread = (2 * tig) * kGvCols + ((gid ^ (2 * tig)) << 4);
  const int xr = lane & 7, xsw = (xr >> 1) & 3, xp0 = (lane >> 3) & 1;
  const uint32_t xread0 = kGvWBytes + xr * (kGvStageK * 2) + ((xp0 ^ xsw) << 4);
  const uint32_t xread1 = kGvWBytes + xr * (kGvStageK * 2) + (((xp0 + 2) ^ xsw) << 4);

  for (int it = 0; it < my_n; ++it) {
    if (it + kGvStages - 1 < my_n) issue(it + kGvStages - 1);
    CpAsyncCommit();
    CpAsyncWait<kGvStages - 1>();
    __syncwarp();
    const uint32_t st_addr = my_pipe_addr + (it % kGvStages) * L::kStageBytes;
#pragma unroll
    for (int h = 0; h < kGvStageK / 16; ++h) {
      // x^T as B fragments: b0b1 = x[row gid][16h + 2tig, +1], b2b3 = x[row gid][16h + 8 + 2tig, +1].
      uint32_t b[NT][2];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) LdMatrixX2(b[nt], st_addr + (h ? xread1 : xread0) + nt * (8 * kGvStageK * 2));
      const uint32_t wbase = st_addr + wread + h * (16 * kGvCols);
      const uint4 ra = LdShared16(wbase), rb = LdShared16(wbase + kGvCols);
      const uint4 rc = LdShared16(wbase + 8 * kGvCols), rd = LdShared16(wbase + 9 * kGvCols);
      const uint32_t wa[4] = {ra.x, ra.y, ra.z, ra.w}, wb[4] = {rb.x, rb.y, rb.z, rb.w};
      const uint32_t wc[4] = {rc.x, rc.y, rc.z, rc.w}, wd[4] = {rd.x, rd.y, rd.z, rd.w};
#pragma unroll
      for (int wi = 0; wi < 4; ++wi) {
        // Bytes 0, 1 of word wi are columns 4wi, 4wi + 1 (MMA j = 2wi); bytes 2, 3 are MMA j = 2wi + 1.
        uint32_t a0[4], a1[4];
        a0[0] = CodesToBf16x2<0>(wa[wi], wb[wi]);
        a0[1] = CodesToBf16x2<1>(wa[wi], wb[wi]);
        a0[2] = CodesToBf16x2<0>(wc[wi], wd[wi]);
        a0[3] = CodesToBf16x2<1>(wc[wi], wd[wi]);
        a1[0] = CodesToBf16x2<2>(wa[wi], wb[wi]);
        a1[1] = CodesToBf16x2<3>(wa[wi], wb[wi]);
        a1[2] = CodesToBf16x2<2>(wc[wi], wd[wi]);
        a1[3] = CodesToBf16x2<3>(wc[wi], wd[wi]);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          MmaBf16(acc[2 * wi][nt], a0, b[nt][0], b[nt][1]);
          MmaBf16(acc[2 * wi + 1][nt], a1, b[nt][0], b[nt][1]);
        }
      }
    }
    __syncwarp();  // the stage is free for the copy the next iteration issues
  }
  CpAsyncWait<0>();
  __syncthreads();  // every warp is done with the pipeline space

  // The four warps' partial tiles -> shared memory -> one tile, summed in warp order.
  float* red = reinterpret_cast<float*>(smem);                  // [kGvWarps][kRows][kGvRedStride]
  float* tile = red + kGvWarps * (L::kRows * kGvRedStride);     // [kRows][kGvRedStride]
  {
    float* mine = red + warp * (L::kRows * kGvRedStride);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const int m = nt * 8 + 2 * tig, c = gid * 16 + 2 * j;
        mine[m * kGvRedStride + c] = acc[j][nt][0];
        mine[(m + 1) * kGvRedStride + c] = acc[j][nt][1];
        mine[m * kGvRedStride + c + 1] = acc[j][nt][2];
        mine[(m + 1) * kGvRedStride + c + 1] = acc[j][nt][3];
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
    const int col = col0 + tid;
    if (col < p.N) {
      float v = 0.f;
      for (unsigned q = 0; q < nranks; ++q) v += cluster.map_shared_rank(tile, q)[m * kGvRedStride + tid];
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
  GridDependencySync();
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
  GridDependencySync();
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

// The fused gate|up projection + SwiGLU in the interpreter's order, for shapes the tensor-core kernel does not take:
// column j of the result reads gate column (j / 128) * 256 + j % 128 and up column 128 further on.
template <typename XT, typename YT>
__global__ void __launch_bounds__(256) GemmSwigluExactKernel(const XT* x, const int8_t* w, const float* scales, YT* y, int M, int K,
                                                             int N, int round_x, int faithful)
{
  GridDependencySync();
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  const int i = blockIdx.y;
  const int half = N >> 1;
  if (j >= half) return;
  const int cg = (j >> 7) * 256 + (j & 127), cu = cg + 128;
  float g = 0.f, u = 0.f;
  for (int p = 0; p < K; ++p) {
    float a = ToF32(x[static_cast<size_t>(i) * K + p]);
    if (round_x) a = __bfloat162float(__float2bfloat16_rn(a));
    if (a == 0.f) continue;
    g = __fadd_rn(g, __fmul_rn(a, ToF32(w[static_cast<size_t>(p) * N + cg])));
    u = __fadd_rn(u, __fmul_rn(a, ToF32(w[static_cast<size_t>(p) * N + cu])));
  }
  if (scales != nullptr) {
    g = __fmul_rn(g, scales[cg]);
    u = __fmul_rn(u, scales[cu]);
  }
  float silu;
  if (faithful) {
    const double gd = static_cast<double>(g);
    silu = static_cast<float>(gd / (1.0 + exp(-gd)));
  } else {
    silu = g / (1.f + expf(-g));
  }
  y[static_cast<size_t>(i) * half + j] = FromF32<YT>(__fmul_rn(silu, u));
}

template <int NT, typename YT>
cudaError_t PrepareGemv()
{
  return cudaFuncSetAttribute(Int8GemvKernel<NT, YT>, cudaFuncAttributeMaxDynamicSharedMemorySize, GvLayout<NT>::kBytes);
}

template <int NT, typename YT>
cudaError_t LaunchGemv(const GemmParams& p, cudaStream_t stream)
{
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((p.N + kGvCols - 1) / kGvCols, p.ks, 1);
  cfg.blockDim = dim3(kGvThreads, 1, 1);
  cfg.dynamicSmemBytes = GvLayout<NT>::kBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  cfg.numAttrs = ChainAttributes(attr, p.ks);
  cfg.attrs = attr;
  return cudaLaunchKernelEx(&cfg, Int8GemvKernel<NT, YT>, p);
}

// K slices for a shape (1, 2, 4 or 8: the portable cluster sizes): the count that wastes the least of the last
// wave of CTAs over the 148 SMs (four CTAs each), among those that leave every warp at least four stages.
// $TLALOC_B200_GEMV_KS overrides.
int ChooseSlices(int k, int n)
{
  static const int forced = [] {
    const char* e = std::getenv("TLALOC_B200_GEMV_KS");
    return e != nullptr ? std::atoi(e) : 0;
  }();
  if (forced == 1 || forced == 2 || forced == 4 || forced == 8) return forced;
  const int tiles = (n + kGvCols - 1) / kGvCols;
  const int slots = 148 * 4;
  int best = 1;
  double best_eff = -1.0;
  for (int ks = 1; ks <= 8; ks *= 2) {
    if (ks > 1 && k / ks < kGvStageK * kGvWarps * 4) break;
    const int items = tiles * ks;
    const int waves = (items + slots - 1) / slots;
    const double eff = static_cast<double>(items) / (static_cast<double>(waves) * slots);
    if (eff > best_eff + 0.02) {
      best_eff = eff;
      best = ks;
    }
  }
  return best;
}

}  // namespace

cudaError_t PrepareInt8GemmKernels()
{
  static OncePerDevice once;
  return once.Run([](int) {
    cudaError_t e = PrepareGemv<1, float>();
    if (e == cudaSuccess) e = PrepareGemv<1, __nv_bfloat16>();
    if (e == cudaSuccess) e = PrepareGemv<2, float>();
    if (e == cudaSuccess) e = PrepareGemv<2, __nv_bfloat16>();
    if (e == cudaSuccess) e = PrepareGemv<4, float>();
    if (e == cudaSuccess) e = PrepareGemv<4, __nv_bfloat16>();
    return e;
  });
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
    return LaunchChained(GemmExactKernel<XT, WT, float>, grid, 256, 0, st, static_cast<const XT*>(x),
                         static_cast<const WT*>(w), scales, residual, static_cast<float*>(y), m, k, n, round_x);
  }
  return LaunchChained(GemmExactKernel<XT, WT, __nv_bfloat16>, grid, 256, 0, st, static_cast<const XT*>(x),
                       static_cast<const WT*>(w), scales, residual, static_cast<__nv_bfloat16*>(y), m, k, n, round_x);
}

template <typename YT>
cudaError_t LaunchGemvRows(const GemmParams& p, int rows, cudaStream_t st)
{
  if (rows <= 8) return LaunchGemv<1, YT>(p, st);
  if (rows <= 16) return LaunchGemv<2, YT>(p, st);
  return LaunchGemv<4, YT>(p, st);
}

}  // namespace

// Scratch: the bf16 copy of an f32 x, or the two int8 planes of the activations and their row steps.
extern "C" size_t tlaloc_b200_int8_gemm_scratch_bytes(int32_t m, int32_t k, int32_t n)
{
  (void)n;
  if (m <= 0 || k <= 0) return 0;
  return (Int8GemmI8ScratchBytes(m, k) + 255) / 256 * 256;
}

namespace {
int TcMinRows()
{
  static const int tc_min = [] {
    const char* v = std::getenv("TLALOC_B200_GEMM_TC_MIN");
    return v != nullptr ? std::atoi(v) : 17;
  }();
  return tc_min;
}
// 17 to 128 rows, the caller's consent and room in the scratch: the int8 tensor-core kernel.
bool UseI8(const int8_t* codes, const void* scratch, size_t scratch_bytes, int m, int k, int n, int flags)
{
  return (flags & TLALOC_B200_GEMM_I8_MMA) != 0 && m >= TcMinRows() && Int8GemmI8Applies(codes, m, k, n) && scratch != nullptr && Aligned16(scratch) &&
         scratch_bytes >= Int8GemmI8ScratchBytes(m, k);
}
}  // namespace

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
  // The fast kernels move x and the codes in 16-byte pieces: a view that starts off a 16-byte boundary (x + 4 elements,
  // a weight slice at an odd column) takes the order-faithful kernel instead, which has no alignment needs.
  const bool aligned = Aligned16(codes) && (x_dtype == TLALOC_B200_F32 || Aligned16(x));
  if ((flags & TLALOC_B200_GEMM_EXACT) != 0 || OrderFaithful() || !FastShape(k, n) || !aligned) {
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
  if (UseI8(codes, scratch, scratch_bytes, m, k, n, flags)) {
    int launches = 0;
    e = LaunchInt8GemmI8(x, x_dtype, codes, scales, residual, y, y_dtype, scratch, m, k, n, st, &launches,
                         (flags & TLALOC_B200_GEMM_WEIGHTS_CONST) != 0, false, (flags & TLALOC_B200_GEMM_X_PLANES) != 0);
    if (e != cudaSuccess) return CudaFail("INT8_PROJ int8 tensor-core launch", e);
    CountLaunches(launches);
    return kOk;
  }
  const __nv_bfloat16* xb = static_cast<const __nv_bfloat16*>(x);
  if (x_dtype == TLALOC_B200_F32) {
    const size_t need = sizeof(__nv_bfloat16) * static_cast<size_t>(m) * k;
    if (scratch == nullptr || scratch_bytes < need) {
      return Fail(kInvalid, "%s: an f32 x needs %zu bytes of scratch for its bf16 copy, got %zu", op, need, scratch_bytes);
    }
    if (!Aligned16(scratch)) return Fail(kInvalid, "%s: scratch must be 16-byte aligned", op);
    const size_t count = static_cast<size_t>(m) * k;
    e = LaunchChained(ToBf16Kernel<float>, static_cast<unsigned>((count + 255) / 256), 256, 0, st,
                      static_cast<const float*>(x), reinterpret_cast<__nv_bfloat16*>(scratch), count);
    if (e != cudaSuccess) return CudaFail("INT8_PROJ activation cast", e);
    CountLaunches(1);
    xb = reinterpret_cast<const __nv_bfloat16*>(scratch);
  }
  const int tc_min = TcMinRows();
  // 17 rows and more: the tcgen05 kernel (measured at 32 rows: 123 vs 193 us at 57344 x 8192, 190 vs 216 us at the
  // 128256 x 4096 head; at 17 rows 166 vs 198 us; at 8 rows the row-vector kernel is faster, 103 vs ~165 us)
  if (m >= tc_min) {
    e = PrepareInt8GemmTcKernels();
    if (e != cudaSuccess) return CudaFail("INT8_PROJ set-up", e);
    int launches = 0;
    e = LaunchInt8GemmTc(xb, codes, scales, residual, y, y_dtype, m, k, n, st, &launches,
                         (flags & TLALOC_B200_GEMM_WEIGHTS_CONST) != 0);
    if (e != cudaSuccess) return CudaFail("INT8_PROJ tensor-core launch", e);
    CountLaunches(launches);
    return kOk;
  }
  GemmParams p;
  p.w = codes;
  p.scales = scales;
  p.K = k;
  p.N = n;
  p.ks = ChooseSlices(k, n);
  p.weights_const = (flags & TLALOC_B200_GEMM_WEIGHTS_CONST) != 0 ? 1 : 0;
  const int per = (k + p.ks - 1) / p.ks;
  const int unit = kGvStageK * kGvWarps;
  p.Kc = (per + unit - 1) / unit * unit;
  const size_t ybytes = DtypeBytes(y_dtype);
  for (int m0 = 0; m0 < m; m0 += 32) {
    const int rows = std::min(32, m - m0);
    p.M = rows;
    p.x = xb + static_cast<size_t>(m0) * k;
    p.residual = residual ? residual + static_cast<size_t>(m0) * n : nullptr;
    p.y = static_cast<unsigned char*>(y) + static_cast<size_t>(m0) * n * ybytes;
    e = y_dtype == TLALOC_B200_F32 ? LaunchGemvRows<float>(p, rows, st) : LaunchGemvRows<__nv_bfloat16>(p, rows, st);
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

extern "C" int tlaloc_b200_int8_gemm_swiglu(const void* x, int32_t x_dtype, const int8_t* codes, const float* scales, void* y,
                                            int32_t y_dtype, float* scratch, size_t scratch_bytes, int32_t m, int32_t k, int32_t n,
                                            int32_t flags, void* stream)
{
  const char* op = "INT8_PROJ_SWIGLU";
  if (!x || !codes || !y) return Fail(kInvalid, "%s: a required device pointer is null", op);
  if (!IsFloatType(x_dtype) || !IsFloatType(y_dtype)) return Fail(kInvalid, "%s: x and y must be f32 or bf16", op);
  if (m < 1 || k < 1 || n < 256 || n % 256 != 0) {
    return Fail(kInvalid, "%s: needs [M, K] x [K, N] with N a multiple of 256 (gate|up blocks of 128 + 128), got M %d K %d N %d", op, m, k, n);
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int tc_min = TcMinRows();
  const bool aligned = Aligned16(codes) && (x_dtype == TLALOC_B200_F32 || Aligned16(x)) && (reinterpret_cast<uintptr_t>(y) & 7) == 0;
  cudaError_t e;
  if ((flags & TLALOC_B200_GEMM_EXACT) != 0 || OrderFaithful() || !FastShape(k, n) || !aligned || m < tc_min) {
    const int faithful = (flags & TLALOC_B200_GEMM_EXACT) != 0 || OrderFaithful();
    const int round_x = x_dtype == TLALOC_B200_F32 && (flags & TLALOC_B200_GEMM_X_F32_EXACT) == 0;
    const dim3 grid((n / 2 + 255) / 256, m);
#define TLALOC_SWIGLU_EXACT(XT, YT, RX)                                                                                  \
  e = LaunchChained(GemmSwigluExactKernel<XT, YT>, grid, 256, 0, st, static_cast<const XT*>(x), codes, scales,         \
                    static_cast<YT*>(y), m, k, n, RX, faithful)
    if (x_dtype == TLALOC_B200_F32 && y_dtype == TLALOC_B200_F32) TLALOC_SWIGLU_EXACT(float, float, round_x);
    else if (x_dtype == TLALOC_B200_F32) TLALOC_SWIGLU_EXACT(float, __nv_bfloat16, round_x);
    else if (y_dtype == TLALOC_B200_F32) TLALOC_SWIGLU_EXACT(__nv_bfloat16, float, 0);
    else TLALOC_SWIGLU_EXACT(__nv_bfloat16, __nv_bfloat16, 0);
#undef TLALOC_SWIGLU_EXACT
    if (e != cudaSuccess) return CudaFail("INT8_PROJ_SWIGLU exact launch", e);
    CountLaunches(1);
    return kOk;
  }
  if (UseI8(codes, scratch, scratch_bytes, m, k, n, flags)) {
    int launches = 0;
    e = LaunchInt8GemmI8(x, x_dtype, codes, scales, nullptr, y, y_dtype, scratch, m, k, n, st, &launches,
                         (flags & TLALOC_B200_GEMM_WEIGHTS_CONST) != 0, true, (flags & TLALOC_B200_GEMM_X_PLANES) != 0);
    if (e != cudaSuccess) return CudaFail("INT8_PROJ_SWIGLU int8 tensor-core launch", e);
    CountLaunches(launches);
    return kOk;
  }
  const __nv_bfloat16* xb = static_cast<const __nv_bfloat16*>(x);
  if (x_dtype == TLALOC_B200_F32) {
    const size_t need = sizeof(__nv_bfloat16) * static_cast<size_t>(m) * k;
    if (scratch == nullptr || scratch_bytes < need || !Aligned16(scratch)) {
      return Fail(kInvalid, "%s: an f32 x needs %zu bytes of 16-byte aligned scratch for its bf16 copy, got %zu", op, need, scratch_bytes);
    }
    const size_t count = static_cast<size_t>(m) * k;
    e = LaunchChained(ToBf16Kernel<float>, static_cast<unsigned>((count + 255) / 256), 256, 0, st, static_cast<const float*>(x),
                      reinterpret_cast<__nv_bfloat16*>(scratch), count);
    if (e != cudaSuccess) return CudaFail("INT8_PROJ_SWIGLU activation cast", e);
    CountLaunches(1);
    xb = reinterpret_cast<const __nv_bfloat16*>(scratch);
  }
  e = PrepareInt8GemmTcKernels();
  if (e != cudaSuccess) return CudaFail("INT8_PROJ_SWIGLU set-up", e);
  int launches = 0;
  e = LaunchInt8GemmTc(xb, codes, scales, nullptr, y, y_dtype, m, k, n, st, &launches, (flags & TLALOC_B200_GEMM_WEIGHTS_CONST) != 0, true);
  if (e != cudaSuccess) return CudaFail("INT8_PROJ_SWIGLU tensor-core launch", e);
  CountLaunches(launches);
  return kOk;
}
