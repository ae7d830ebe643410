// The int8 weight-only projection for batches of rows (17 <= M <= 256 per launch) on the 5th-generation tensor
// cores: y = (cast(x) @ cast(codes)) * scale (HfDecoderGraph.proj, ir/.../inference/HfDecoderGraph.kt:625-655).
//
// Formulation: D^T[n, m] = sum_k W^T[n, k] X^T[k, m].  The 128 output columns of an accumulator are the MMA's M
// dimension (TMEM lanes), the MPAD activation rows its N dimension (TMEM columns); a CTA owns 256 output columns
// (two accumulators) and one slice of K, walked in blocks of 64 rows:
//   1. cp.async stages the block's raw int8 weights [64][256] (the reference's own [K, N] layout) and the matching
//      bf16 activation strip [MPAD][64], the latter straight into the canonical K-major 128-byte-swizzled operand
//      layout; several blocks are in flight.
//   2. all 512 threads turn the int8 codes into exact bf16 (byte-permute, two logic ops, one packed fma per pair) and
//      store them as the MN-major 128-byte-swizzled A operand: W's rows are contiguous along N, which is exactly
//      MN-major, so 16 codes become two 16-byte stores and nothing is transposed.
//   3. one thread issues tcgen05.mma (kind::f16, bf16 x bf16 -> f32 in TMEM), 4 K-steps x 2 accumulators per block, and
//      commits to an mbarrier that frees the block's buffers two blocks later; conversion of the next block overlaps.
// Epilogue: tcgen05.ld brings the accumulators to registers (lane = output column); with one K slice they are
// scaled and stored directly (32 lanes = 128 contiguous bytes of a row); with several, the slices of a column tile
// form a thread-block cluster and meet in distributed shared memory, summed in rank order (deterministic).
// Every mbarrier wait is bounded: on a time-out the kernel records it in a status word, frees its TMEM and returns.
#include <cooperative_groups.h>

#include <mutex>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace tlaloc_b200 {
namespace {

struct TcParams {
  const __nv_bfloat16* x;  // [M, K]
  const int8_t* w;         // [K, N]
  const float* scales;
  const float* residual;
  void* y;
  int M, K, N;
  int Kc, ks;
};

constexpr int kTcThreads = 512;                  // converter threads (16 warps)
constexpr int kTcLaunchThreads = kTcThreads + 32;  // plus one warp whose elected lane issues the MMAs
constexpr int kTcBN = 256;  // output columns per CTA: two accumulators of 128
constexpr int kTcBK = 64;   // k rows per block
constexpr int kTcRawBytes = kTcBK * kTcBN;
constexpr int kTcABytes = 2 * 128 * kTcBK * 2;  // both accumulators' bf16 A tiles of one block
constexpr int kTcTileStride = kTcBN + 4;
constexpr uint32_t kTcSpinLimit = 1u << 20;

__device__ int g_tc_status = 0;  // nonzero after an mbarrier wait timed out (sticky until read)

template <int MPAD>
struct TcLayout {
  static constexpr int kXBytes = MPAD * kTcBK * 2;
  static constexpr int kStageBytes = kTcRawBytes + kXBytes;
  static constexpr int kStages = MPAD <= 64 ? 6 : (MPAD == 128 ? 5 : 3);
  static constexpr int kAOffset = kStages * kStageBytes;
  static constexpr int kBarOffset = kAOffset + 2 * kTcABytes;  // four mbarriers, then the TMEM base address
  static constexpr int kPipeBytes = kBarOffset + 64;
  static constexpr int kTileBytes = MPAD <= 128 ? MPAD * kTcTileStride * 4 : 0;  // cluster reduction tile (aliases the pipeline)
  static constexpr int kBytes = (kPipeBytes > kTileBytes ? kPipeBytes : kTileBytes) + 1024;  // slack to align to 1024
  static constexpr int kTmemCols = 2 * MPAD < 32 ? 32 : 2 * MPAD;
  static_assert(kStageBytes % 1024 == 0, "operand tiles start on 1024-byte boundaries");
};

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
__device__ __forceinline__ uint4 LdShared16(uint32_t addr)
{
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ void StShared16(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d)
{
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};\n" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
// Two codes of one word (bytes selected by SEL into the low byte of each half) as an exact bf16 pair: for a code v
// with bits s:lo7, 0x4300|lo7 is the bf16 128 + lo7 and 0xC300|s<<7 is -128 or -256; their sum is v.
template <int SEL>
__device__ __forceinline__ uint32_t CodePairToBf16x2(uint32_t w)
{
  const uint32_t q = __byte_perm(w, 0u, SEL);
  uint32_t t, c, r;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;\n" : "=r"(t) : "r"(q), "r"(0x007F007Fu), "r"(0x43004300u));
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;\n" : "=r"(c) : "r"(q), "r"(0x00800080u), "r"(0xC300C300u));
  asm("fma.rn.bf16x2 %0, %1, %2, %3;\n" : "=r"(r) : "r"(t), "r"(0x3F803F80u), "r"(c));
  return r;
}

__device__ __forceinline__ void MbarInit(uint32_t bar, uint32_t count)
{
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count) : "memory");
}
// One lane polls for the warp (32 pollers per warp would spend the SM's issue slots on the wait itself).
__device__ __forceinline__ bool MbarWait(uint32_t bar, uint32_t parity);
__device__ __forceinline__ bool MbarWaitWarp(uint32_t bar, uint32_t parity, int lane)
{
  int ok = 1;
  if (lane == 0) ok = MbarWait(bar, parity) ? 1 : 0;
  ok = __shfl_sync(0xffffffffu, ok, 0);
  return ok != 0;
}
// Waits for the phase with the given parity; gives up after kTcSpinLimit polls.  Returns false on a time-out.
__device__ __forceinline__ bool MbarWait(uint32_t bar, uint32_t parity)
{
  for (uint32_t i = 0; i < kTcSpinLimit; ++i) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}\n"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    if (done) return true;
  }
  return false;
}

// Shared-memory matrix descriptor of a 128-byte-swizzled operand tile: start address, leading and stride byte offsets
// (all in 16-byte units), descriptor version 1, layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t SmemDesc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes)
{
  return static_cast<uint64_t>((addr >> 4) & 0x3FFFu) | (static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16) |
         (static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32) | (1ull << 46) | (2ull << 61);
}
// kind::f16 instruction descriptor: f32 accumulator, bf16 A and B, A MN-major, B K-major, M = 128, N = n.
__host__ __device__ constexpr uint32_t InstrDesc(int n)
{
  return (1u << 4) | (1u << 7) | (1u << 10) | (1u << 15) | (static_cast<uint32_t>(n >> 3) << 17) | (8u << 24);
}
__device__ __forceinline__ void TcMma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void TcCommit(uint32_t bar)
{
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void TcLd8(uint32_t taddr, uint32_t (&r)[8])
{
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr));
}

template <int MPAD, typename YT>
__global__ void __launch_bounds__(kTcLaunchThreads, 1) Int8GemmTcKernel(TcParams p)
{
  using L = TcLayout<MPAD>;
  extern __shared__ unsigned char smem_raw[];
  // 1024-byte alignment of the operand tiles (the swizzle is a function of address bits 4..9).
  const uint32_t smem_base = (SmemAddr(smem_raw) + 1023u) & ~1023u;
  unsigned char* smem = smem_raw + (smem_base - SmemAddr(smem_raw));
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int col0 = blockIdx.x * kTcBN;
  const int kb0 = blockIdx.y * p.Kc;
  const int ke = min(p.K, kb0 + p.Kc);
  const int nblocks = ke > kb0 ? (ke - kb0 + kTcBK - 1) / kTcBK : 0;
  // mma_done[2]: the MMAs of a block have completed (frees its A buffer and its stage); conv_done[2]: the sixteen
  // converter warps have finished a block's A tile and landed its activation strip.
  const uint32_t mma_done0 = smem_base + L::kBarOffset, conv_done0 = mma_done0 + 16;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + L::kBarOffset + 32);

  if (tid == 0) {
    MbarInit(mma_done0, 1);
    MbarInit(mma_done0 + 8, 1);
    MbarInit(conv_done0, kTcThreads / 32);
    MbarInit(conv_done0 + 8, kTcThreads / 32);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_base + L::kBarOffset + 32),
                 "r"(static_cast<uint32_t>(L::kTmemCols))
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  // One block's copies.  Weights: chunk c = tid + 512 i is row c / 16, 16 columns from (c % 16) * 16, stored as is.
  // Activations: chunk c is row c / 8, 8 k from (c % 8) * 8, stored at ((row / 8) * 8 + row % 8) * 128 bytes with the
  // 16-byte chunk index XORed with row % 8 (the K-major 128-byte swizzle).  Outside the matrix: zero-filled.
  auto issue = [&](int b) {
    const int k0 = kb0 + b * kTcBK;
    const uint32_t st = smem_base + (b % L::kStages) * L::kStageBytes;
#pragma unroll
    for (int i = 0; i < kTcRawBytes / 16 / kTcThreads; ++i) {
      const int c = tid + kTcThreads * i;
      const int row = c >> 4, c16 = c & 15;
      const bool valid = k0 + row < ke && col0 + c16 * 16 < p.N;
      CpAsync16(st + row * kTcBN + c16 * 16, valid ? p.w + static_cast<size_t>(k0 + row) * p.N + col0 + c16 * 16 : p.w, valid ? 16 : 0);
    }
#pragma unroll
    for (int i = 0; i < (L::kXBytes / 16 + kTcThreads - 1) / kTcThreads; ++i) {
      const int c = tid + kTcThreads * i;
      if (c < L::kXBytes / 16) {
        const int m = c >> 3, ch = c & 7;
        const bool valid = m < p.M && k0 + ch * 8 < ke;
        CpAsync16(st + kTcRawBytes + (m >> 3) * 1024 + (m & 7) * 128 + ((ch ^ (m & 7)) << 4),
                  valid ? p.x + static_cast<size_t>(m) * p.K + k0 + ch * 8 : p.x, valid ? 16 : 0);
      }
    }
  };

  bool ok = true;
  constexpr uint32_t idesc = InstrDesc(MPAD);
  if (warp < kTcThreads / 32) {
    // Converter warps.  A thread converts exactly the weight chunks it copied, so its own cp.async completion is all
    // it waits for; the loop has no CTA-wide barrier.
    for (int b = 0; b < L::kStages - 2; ++b) {
      if (b < nblocks) issue(b);
      CpAsyncCommit();
    }
    for (int b = 0; b < nblocks; ++b) {
      // Block b - 2 used the same A buffer and the stage about to be refilled: its MMAs must have completed.
      if (b >= 2) ok = MbarWaitWarp(mma_done0 + (b & 1) * 8, ((b - 2) >> 1) & 1, lane) && ok;
      if (b + L::kStages - 2 < nblocks) issue(b + L::kStages - 2);
      CpAsyncCommit();
      CpAsyncWait<L::kStages - 2>();
      // int8 -> bf16, into the MN-major swizzled A tiles: element (n, k) of accumulator n / 128 lives at
      // (n % 128 / 64) * 8192 + (k / 8) * 1024 + (k % 8) * 128 + (((n % 64) / 8) ^ (k % 8)) * 16 + (n % 8) * 2.
      const uint32_t st = smem_base + (b % L::kStages) * L::kStageBytes;
      const uint32_t a_tile = smem_base + L::kAOffset + (b & 1) * kTcABytes;
#pragma unroll
      for (int i = 0; i < kTcRawBytes / 16 / kTcThreads; ++i) {
        const int c = tid + kTcThreads * i;
        const int row = c >> 4, c16 = c & 15;
        const uint4 v = LdShared16(st + row * kTcBN + c16 * 16);
        const uint32_t o0 = CodePairToBf16x2<0x1100>(v.x), o1 = CodePairToBf16x2<0x3322>(v.x);
        const uint32_t o2 = CodePairToBf16x2<0x1100>(v.y), o3 = CodePairToBf16x2<0x3322>(v.y);
        const uint32_t o4 = CodePairToBf16x2<0x1100>(v.z), o5 = CodePairToBf16x2<0x3322>(v.z);
        const uint32_t o6 = CodePairToBf16x2<0x1100>(v.w), o7 = CodePairToBf16x2<0x3322>(v.w);
        const int k_in = row & 7;
        const uint32_t dst = a_tile + (c16 >> 3) * 16384 + ((c16 >> 2) & 1) * 8192 + (row >> 3) * 1024 + k_in * 128;
        const int chunk = 2 * (c16 & 3);
        StShared16(dst + ((chunk ^ k_in) << 4), o0, o1, o2, o3);
        StShared16(dst + (((chunk + 1) ^ k_in) << 4), o4, o5, o6, o7);
      }
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");  // these writes (and the cp.async strip) -> tensor core
      __syncwarp();
      if (lane == 0) {
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(conv_done0 + (b & 1) * 8) : "memory");
      }
    }
    CpAsyncWait<0>();
    if (nblocks > 0) {
      const int last = nblocks - 1;
      ok = MbarWaitWarp(mma_done0 + (last & 1) * 8, (last >> 1) & 1, lane) && ok;
      if (nblocks > 1) ok = MbarWaitWarp(mma_done0 + ((last - 1) & 1) * 8, ((last - 1) >> 1) & 1, lane) && ok;
    }
  } else if (lane == 0) {
    // The MMA thread: for each block, wait for the converters, then 4 K-steps x 2 accumulators and a commit.
    for (int b = 0; b < nblocks; ++b) {
      ok = MbarWait(conv_done0 + (b & 1) * 8, (b >> 1) & 1) && ok;
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      const uint32_t x_tile = smem_base + (b % L::kStages) * L::kStageBytes + kTcRawBytes;
      const uint32_t a_tile = smem_base + L::kAOffset + (b & 1) * kTcABytes;
#pragma unroll
      for (int j = 0; j < kTcBK / 16; ++j) {
        const uint64_t b_desc = SmemDesc(x_tile + j * 32, 16, 1024);
#pragma unroll
        for (int nb = 0; nb < 2; ++nb) {
          const uint64_t a_desc = SmemDesc(a_tile + nb * 16384 + j * 2048, 8192, 1024);
          TcMma(tmem_base + nb * MPAD, a_desc, b_desc, idesc, (b > 0 || j > 0) ? 1u : 0u);
        }
      }
      TcCommit(mma_done0 + (b & 1) * 8);
    }
  }
  if (!ok) atomicExch(&g_tc_status, 1);
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  __syncthreads();  // the pipeline space is free

  // Epilogue.  Warp w reads TMEM lanes 32 (w % 4) .. + 31 (output columns) of both accumulators, for its quarter
  // (w / 4) of the activation rows.
  cg::cluster_group cluster = cg::this_cluster();
  const unsigned rank = cluster.block_rank(), nranks = cluster.num_blocks();
  const int lg = warp & 3, wq = warp >> 2;
  constexpr int kRowsPerWarp = MPAD / 4;
  float* tile = reinterpret_cast<float*>(smem);
  YT* y = static_cast<YT*>(p.y);
#pragma unroll
  for (int nb = 0; nb < (warp < kTcThreads / 32 ? 2 : 0); ++nb) {
    const int n_local = nb * 128 + lg * 32 + lane;
    const int col = col0 + n_local;
    const float scale = (p.scales != nullptr && col < p.N) ? __ldg(p.scales + col) : 1.f;
#pragma unroll
    for (int m0 = 0; m0 < kRowsPerWarp; m0 += 8) {
      const int m_base = wq * kRowsPerWarp + m0;
      uint32_t r[8];
      if (nblocks > 0) {
        TcLd8(tmem_base + (static_cast<uint32_t>(lg * 32) << 16) + nb * MPAD + m_base, r);
        asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) r[e] = 0u;
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const int m = m_base + e;
        const float v = __uint_as_float(r[e]);
        if (MPAD > 128 || nranks == 1) {
          if (m < p.M && col < p.N) {
            float o = v * scale;
            if (p.residual != nullptr) o += __ldg(p.residual + static_cast<size_t>(m) * p.N + col);
            y[static_cast<size_t>(m) * p.N + col] = FromF32<YT>(o);
          }
        } else {
          tile[m * kTcTileStride + n_local] = v;
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  if (MPAD <= 128 && nranks > 1) {
    // The K slices of this column tile are the ranks of one cluster: rank r finishes every nranks-th row.
    cluster.sync();
    for (int m = rank + nranks * (tid >> 8); m < p.M && tid < kTcThreads; m += 2 * nranks) {
      const int n_local = tid & 255, col = col0 + n_local;
      if (col < p.N) {
        float v = 0.f;
        for (unsigned q = 0; q < nranks; ++q) v += cluster.map_shared_rank(tile, q)[m * kTcTileStride + n_local];
        if (p.scales != nullptr) v *= __ldg(p.scales + col);
        if (p.residual != nullptr) v += __ldg(p.residual + static_cast<size_t>(m) * p.N + col);
        y[static_cast<size_t>(m) * p.N + col] = FromF32<YT>(v);
      }
    }
    cluster.sync();  // no CTA leaves while a peer may still read its tile
  } else {
    __syncthreads();
  }
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(static_cast<uint32_t>(L::kTmemCols)) : "memory");
  }
}

template <int MPAD, typename YT>
cudaError_t PrepareTc()
{
  return cudaFuncSetAttribute(Int8GemmTcKernel<MPAD, YT>, cudaFuncAttributeMaxDynamicSharedMemorySize, TcLayout<MPAD>::kBytes);
}

template <int MPAD, typename YT>
cudaError_t LaunchTc(const TcParams& p, cudaStream_t stream)
{
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((p.N + kTcBN - 1) / kTcBN, p.ks, 1);
  cfg.blockDim = dim3(kTcLaunchThreads, 1, 1);
  cfg.dynamicSmemBytes = TcLayout<MPAD>::kBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = p.ks;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, Int8GemmTcKernel<MPAD, YT>, p);
}

// K slices (1, 2, 4 or 8): the count that wastes the least of the last wave over the 148 SMs (one CTA each), among
// those that leave every slice at least eight blocks.  $TLALOC_B200_GEMM_KS overrides.
int ChooseTcSlices(int k, int n, int mpad)
{
  static const int forced = [] {
    const char* e = std::getenv("TLALOC_B200_GEMM_KS");
    return e != nullptr ? std::atoi(e) : 0;
  }();
  if (mpad > 128) return 1;
  if (forced == 1 || forced == 2 || forced == 4 || forced == 8) return forced;
  const int tiles = (n + kTcBN - 1) / kTcBN;
  int best = 1;
  double best_eff = -1.0;
  for (int ks = 1; ks <= 8; ks *= 2) {
    if (ks > 1 && k / ks < kTcBK * 8) break;
    const int items = tiles * ks;
    const int waves = (items + 147) / 148;
    const double eff = static_cast<double>(items) / (static_cast<double>(waves) * 148);
    if (eff > best_eff + 0.12) {  // more slices also cost a larger cluster reduction: ask for a clear gain
      best_eff = eff;
      best = ks;
    }
  }
  return best;
}

template <typename YT>
cudaError_t LaunchTcRows(const TcParams& p, int rows, cudaStream_t st)
{
  if (rows <= 32) return LaunchTc<32, YT>(p, st);
  if (rows <= 64) return LaunchTc<64, YT>(p, st);
  if (rows <= 128) return LaunchTc<128, YT>(p, st);
  return LaunchTc<256, YT>(p, st);
}

}  // namespace

cudaError_t PrepareInt8GemmTcKernels()
{
  static std::mutex mu;
  static bool done = false;
  std::lock_guard<std::mutex> lock(mu);
  if (done) return cudaSuccess;
  cudaError_t e = PrepareTc<32, float>();
  if (e == cudaSuccess) e = PrepareTc<32, __nv_bfloat16>();
  if (e == cudaSuccess) e = PrepareTc<64, float>();
  if (e == cudaSuccess) e = PrepareTc<64, __nv_bfloat16>();
  if (e == cudaSuccess) e = PrepareTc<128, float>();
  if (e == cudaSuccess) e = PrepareTc<128, __nv_bfloat16>();
  if (e == cudaSuccess) e = PrepareTc<256, float>();
  if (e == cudaSuccess) e = PrepareTc<256, __nv_bfloat16>();
  if (e == cudaSuccess) done = true;
  return e;
}

// Rows [0, m) of the projection on the tensor-core kernel, at most 256 rows per launch.  x is bf16.
cudaError_t LaunchInt8GemmTc(const __nv_bfloat16* x, const int8_t* codes, const float* scales, const float* residual,
                             void* y, int y_dtype, int m, int k, int n, cudaStream_t st, int* launches)
{
  TcParams p;
  p.w = codes;
  p.scales = scales;
  p.K = k;
  p.N = n;
  const size_t ybytes = DtypeBytes(y_dtype);
  for (int m0 = 0; m0 < m; m0 += 256) {
    const int rows = std::min(256, m - m0);
    const int mpad = rows <= 32 ? 32 : rows <= 64 ? 64 : rows <= 128 ? 128 : 256;
    p.ks = ChooseTcSlices(k, n, mpad);
    const int per = (k + p.ks - 1) / p.ks;
    p.Kc = (per + kTcBK - 1) / kTcBK * kTcBK;
    p.M = rows;
    p.x = x + static_cast<size_t>(m0) * k;
    p.residual = residual ? residual + static_cast<size_t>(m0) * n : nullptr;
    p.y = static_cast<unsigned char*>(y) + static_cast<size_t>(m0) * n * ybytes;
    const cudaError_t e = y_dtype == TLALOC_B200_F32 ? LaunchTcRows<float>(p, rows, st) : LaunchTcRows<__nv_bfloat16>(p, rows, st);
    if (e != cudaSuccess) return e;
    ++*launches;
  }
  return cudaSuccess;
}

int ReadTcStatus()
{
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_tc_status, sizeof(int)) != cudaSuccess) return -1;
  if (v != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_tc_status, &zero, sizeof(int));
  }
  return v;
}

}  // namespace tlaloc_b200
