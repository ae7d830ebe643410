// The int8 weight-only projection for batches of rows (17 <= M <= 256 per launch) on the 5th-generation tensor
// cores: y = (cast(x) @ cast(codes)) * scale (HfDecoderGraph.proj, ir/.../inference/HfDecoderGraph.kt:625-655).
//
// Formulation: D[m, n] = sum_k X[m, k] W[k, n].  The activation rows are the MMA's M dimension (TMEM lanes, always
// 128 of them, the unused ones ignored), 256 output columns its N dimension (TMEM columns); a CTA owns those 256
// columns and one slice of K, walked in blocks of 64 rows.  The sixteen converter warps form four groups; group g
// owns blocks g, g + 4, ... and for each of them:
//   1. requests the block's bf16 activation strip [MPAD][64] with cp.async, straight into the canonical K-major
//      128-byte-swizzled operand layout;
//   2. turns the block's int8 codes, which its threads loaded from global memory STRAIGHT INTO REGISTERS one group
//      period earlier (the reference's own [K, N] layout: a warp reads two 256-byte runs), into exact bf16
//      (byte-permute, two logic ops, one packed fma per pair) and stores them as the MN-major 128-byte-swizzled B
//      operand: W's rows are contiguous along N, which is exactly MN-major, so 16 codes become two 16-byte stores and
//      nothing is transposed.  Each chunk's registers are refilled with the group's next block as soon as they are
//      consumed.  Raw codes never touch shared memory: shared-memory bandwidth (operand reads by the tensor core +
//      these stores + the strips) is the scarce resource here, and a raw staging buffer would add a third again;
//   3. arrives on the block's mbarrier.  One thread of a seventeenth warp waits for it and issues tcgen05.mma
//      (kind::f16, bf16 x bf16 -> f32 in TMEM), 4 K-steps of 128 x 256 x 16, then commits to the mbarrier that hands
//      the buffers back to the group.
// Why groups: with all sixteen warps sharing every block, each warp's serial chain (wait, request, convert, fence,
// arrive: ~1400 cycles, mostly instruction latency) was paid once per block and set the pace; a group pays the fixed
// part once per FOUR blocks and the groups' chains overlap.
// Epilogue: tcgen05.ld brings the accumulator to registers (lane = activation row, eight output columns at a time);
// with one K slice they are scaled and stored directly (32 bytes per thread); with several, the slices of a column
// tile form a thread-block cluster and meet in distributed shared memory, summed in rank order (deterministic).
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

constexpr int kTcThreads = 512;                    // converter threads (16 warps)
constexpr int kTcLaunchThreads = kTcThreads + 32;  // plus one warp whose elected lane issues the MMAs
constexpr int kTcBN = 256;                         // output columns per CTA: the N of one MMA
constexpr int kTcBK = 64;                          // k rows per block
constexpr int kTcWBytes = kTcBN * kTcBK * 2;       // one block's weights as bf16
constexpr int kTcTileStride = kTcBN + 4;
constexpr uint32_t kTcSpinLimit = 1u << 22;

__device__ int g_tc_status = 0;  // nonzero after an mbarrier wait timed out (sticky until read)

// Shared memory: [activation strips, kBufs][bf16 weight tiles, kBufs][mbarriers, TMEM base].  An MMA always reads
// 128 activation rows; with MPAD < 128 the rows past MPAD are whatever follows in shared memory, which only reaches
// accumulator lanes that are never read.
template <int MPAD>
struct TcLayout {
  static constexpr int kXBytes = MPAD * kTcBK * 2;
  // Converter groups: group g converts blocks g, g + kGroups, ...  There are as many buffers as groups, so a buffer
  // always belongs to the same group and the parity a group waits for can only be the barrier's latest phase.
  static constexpr int kGroups = MPAD > 128 ? 2 : 4;
  static constexpr int kBufs = kGroups;  // blocks in flight between the converters and the tensor core
  static constexpr int kGroupWarps = kTcThreads / 32 / kGroups;
  static constexpr int kGroupThreads = 32 * kGroupWarps;
  static constexpr int kRowsPerPass = 2 * kGroupWarps;        // k rows a group's warps cover with one load each
  static constexpr int kChunks = kTcBK / kRowsPerPass;        // 16-code chunks per thread per block
  static constexpr int kXRowsPerPass = kGroupThreads / 8;     // activation rows a group's threads cover with one copy each
  static constexpr int kWOffset = kBufs * kXBytes;
  static constexpr int kBarOffset = kWOffset + kBufs * kTcWBytes;  // mma_done[kBufs], conv_done[kBufs], then the TMEM base
  static constexpr int kPipeBytes = kBarOffset + 128;
  static constexpr int kTileBytes = MPAD <= 128 ? MPAD * kTcTileStride * 4 : 0;  // cluster reduction tile (aliases the pipeline)
  static constexpr int kBytes = (kPipeBytes > kTileBytes ? kPipeBytes : kTileBytes) + 1024;  // slack to align to 1024
  static constexpr int kAccs = MPAD > 128 ? 2 : 1;  // accumulators of 128 activation rows x 256 columns
  static constexpr int kTmemCols = kAccs * kTcBN;
  static_assert(kXBytes % 1024 == 0, "operand tiles start on 1024-byte boundaries");
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
// 16 weight codes straight from global memory to registers (streamed: no L1 allocation); zeros when not valid.
__device__ __forceinline__ uint4 LdWeights16(const int8_t* ptr, bool valid)
{
  uint4 v = make_uint4(0u, 0u, 0u, 0u);
  if (valid) {
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(ptr));
  }
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
// kind::f16 instruction descriptor: f32 accumulator, bf16 A and B, A K-major, B MN-major, M = 128, N = 256.
__host__ __device__ constexpr uint32_t InstrDesc()
{
  return (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | (static_cast<uint32_t>(kTcBN >> 3) << 17) | (8u << 24);
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

// Eight consecutive outputs of one row; 16-byte stores when the address allows.
__device__ __forceinline__ void StoreRow8(float* dst, const float (&o)[8])
{
  if ((reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
    reinterpret_cast<float4*>(dst)[0] = make_float4(o[0], o[1], o[2], o[3]);
    reinterpret_cast<float4*>(dst)[1] = make_float4(o[4], o[5], o[6], o[7]);
  } else {
#pragma unroll
    for (int e = 0; e < 8; ++e) dst[e] = o[e];
  }
}
__device__ __forceinline__ void StoreRow8(__nv_bfloat16* dst, const float (&o)[8])
{
  if ((reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
    uint4 v;
    __nv_bfloat162 h;
    h = __floats2bfloat162_rn(o[0], o[1]); v.x = *reinterpret_cast<uint32_t*>(&h);
    h = __floats2bfloat162_rn(o[2], o[3]); v.y = *reinterpret_cast<uint32_t*>(&h);
    h = __floats2bfloat162_rn(o[4], o[5]); v.z = *reinterpret_cast<uint32_t*>(&h);
    h = __floats2bfloat162_rn(o[6], o[7]); v.w = *reinterpret_cast<uint32_t*>(&h);
    *reinterpret_cast<uint4*>(dst) = v;
  } else {
#pragma unroll
    for (int e = 0; e < 8; ++e) dst[e] = __float2bfloat16_rn(o[e]);
  }
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
  // mma_done[i]: the MMAs of the block in buffer i have completed (frees its weight tile and activation strip);
  // conv_done[i]: the four warps of the block's converter group have filled weight tile i and landed the strip.
  const uint32_t mma_done0 = smem_base + L::kBarOffset, conv_done0 = mma_done0 + 8 * L::kBufs;
  const uint32_t tmem_slot_addr = smem_base + L::kBarOffset + 64;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + L::kBarOffset + 64);

  if (tid == 0) {
    for (int i = 0; i < L::kBufs; ++i) {
      MbarInit(mma_done0 + 8 * i, 1);
      MbarInit(conv_done0 + 8 * i, L::kGroupWarps);
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(tmem_slot_addr),
                 "r"(static_cast<uint32_t>(L::kTmemCols))
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  bool ok = true;
  if (warp < kTcThreads / 32) {
    // Converter warps, in kGroups groups; a group takes every kGroups-th block and does ALL of it, so the fixed costs
    // of a block (barrier wait, strip request, proxy fence, arrival) are paid by a few warps instead of sixteen and
    // the groups' phases interleave on the schedulers instead of coinciding.
    // Within a block a warp owns k rows 2 wg + r + kRowsPerPass * i, all 256 columns: lane = atom * 8 + r * 4 + j
    // holds 16 codes of columns atom * 64 + 16 j.  Global loads: two 256-byte runs per warp instruction.  Shared
    // stores: a quarter-warp writes two adjacent k rows of one 64-column atom, whose swizzled 16-byte slots have
    // opposite parity, so the eight stores of a phase hit eight different bank groups.
    constexpr int kG = L::kGroups, kChunks = L::kChunks, kRP = L::kRowsPerPass, kXR = L::kXRowsPerPass;
    const int grp = warp / L::kGroupWarps, wg = warp % L::kGroupWarps, gtid = tid % L::kGroupThreads;
    const int j = lane & 3, r = (lane >> 2) & 1, atom = lane >> 3;
    const int row0 = 2 * wg + r, k_in = row0 & 7;  // rows row0 + kRP * i; kRP is a multiple of 8, so k % 8 is fixed
    const int ccol = atom * 64 + j * 16;
    const bool col_ok = col0 + ccol < p.N;
    const int8_t* wp = p.w + static_cast<size_t>(kb0 + row0) * p.N + col0 + ccol;
    const size_t pass = static_cast<size_t>(kRP) * p.N, blk = static_cast<size_t>(kTcBK) * p.N;
    // element (n, k) of the MN-major 128-byte-swizzled tile lives at
    // (n / 64) * 8192 + (k / 8) * 1024 + (k % 8) * 128 + (((n % 64) / 8) ^ (k % 8)) * 16 + (n % 8) * 2
    const uint32_t dst_off = atom * 8192 + (row0 >> 3) * 1024 + k_in * 128;
    const uint32_t s0 = static_cast<uint32_t>((2 * j) ^ k_in) << 4, s1 = static_cast<uint32_t>((2 * j + 1) ^ k_in) << 4;
    // The activation strip [MPAD][64] bf16 goes straight into the K-major 128-byte-swizzled operand layout: chunk
    // c = gtid + kGroupThreads * i is row c / 8, 8 k from (c % 8) * 8, stored at (row / 8) * 1024 + (row % 8) * 128 with the
    // 16-byte chunk index XORed with row % 8.  Outside the matrix: zero-filled.
    const int xm0 = gtid >> 3, xch = gtid & 7;
    const uint32_t xdst0 = (xm0 >> 3) * 1024 + (xm0 & 7) * 128 + ((xch ^ (xm0 & 7)) << 4);
    const __nv_bfloat16* xsrc0 = p.x + static_cast<size_t>(xm0) * p.K + kb0 + xch * 8;
    const size_t xstep = static_cast<size_t>(kXR) * p.K;

    uint4 wreg[kChunks];
#pragma unroll
    for (int i = 0; i < kChunks; ++i)
      wreg[i] = LdWeights16(wp + static_cast<size_t>(grp) * blk + i * pass, col_ok && kb0 + grp * kTcBK + row0 + kRP * i < ke);
    for (int b = grp; b < nblocks; b += kG) {
      const int buf = b % L::kBufs;
      // Block b - kBufs used this weight tile and this strip buffer.
      if (b >= L::kBufs) ok = MbarWaitWarp(mma_done0 + buf * 8, ((b / L::kBufs) - 1) & 1, lane) && ok;
      const int k0 = kb0 + b * kTcBK;
      {
        const uint32_t st = smem_base + buf * L::kXBytes + xdst0;
        const __nv_bfloat16* src = xsrc0 + b * kTcBK;
        const bool k_ok = k0 + xch * 8 < ke;
#pragma unroll
        for (int i = 0; i < MPAD / kXR; ++i) {
          const bool valid = k_ok && xm0 + kXR * i < p.M;
          CpAsync16(st + i * (kXR * 128), valid ? src + i * xstep : p.x, valid ? 16 : 0);
        }
        CpAsyncCommit();
      }
      const uint32_t bt = smem_base + L::kWOffset + buf * kTcWBytes + dst_off;
      const int8_t* next = wp + static_cast<size_t>(b + kG) * blk;
      const int next_k = k0 + kG * kTcBK + row0;  // at or past ke when this was the group's last block
#pragma unroll
      for (int i = 0; i < kChunks; ++i) {
        const uint4 v = wreg[i];
        const uint32_t o0 = CodePairToBf16x2<0x1100>(v.x), o1 = CodePairToBf16x2<0x3322>(v.x);
        const uint32_t o2 = CodePairToBf16x2<0x1100>(v.y), o3 = CodePairToBf16x2<0x3322>(v.y);
        const uint32_t o4 = CodePairToBf16x2<0x1100>(v.z), o5 = CodePairToBf16x2<0x3322>(v.z);
        const uint32_t o6 = CodePairToBf16x2<0x1100>(v.w), o7 = CodePairToBf16x2<0x3322>(v.w);
        StShared16(bt + i * (kRP * 128) + s0, o0, o1, o2, o3);
        StShared16(bt + i * (kRP * 128) + s1, o4, o5, o6, o7);
        wreg[i] = LdWeights16(next + i * pass, col_ok && next_k + kRP * i < ke);  // the group's next block, a period ahead
      }
      CpAsyncWait<0>();  // this thread's part of the strip has landed
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");  // these writes (and the cp.async strip) -> tensor core
      __syncwarp();
      if (lane == 0) {
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(conv_done0 + buf * 8) : "memory");
      }
    }
  } else if (lane == 0) {
    // The MMA thread: for each block, wait for its converter group, then 4 K-steps of 128 x 256 x 16 per accumulator
    // and a commit.  A = the activation strip (K-major), B = the converted weights (MN-major).  Descriptors differ
    // from block to block only in the 14-bit start-address field, so they are built once and advanced by adds.
    constexpr uint32_t idesc = InstrDesc();
    const uint64_t a_desc0 = SmemDesc(smem_base, 16, 1024), b_desc0 = SmemDesc(smem_base + L::kWOffset, 8192, 1024);
    for (int b = 0; b < nblocks; ++b) {
      const int buf = b % L::kBufs;
      ok = MbarWait(conv_done0 + buf * 8, (b / L::kBufs) & 1) && ok;
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      const uint64_t a_desc = a_desc0 + static_cast<uint64_t>((buf * L::kXBytes) >> 4);
      const uint64_t b_desc = b_desc0 + static_cast<uint64_t>((buf * kTcWBytes) >> 4);
#pragma unroll
      for (int ks = 0; ks < kTcBK / 16; ++ks) {
#pragma unroll
        for (int acc = 0; acc < L::kAccs; ++acc)
          TcMma(tmem_base + acc * kTcBN, a_desc + static_cast<uint64_t>((acc * 16384 + ks * 32) >> 4),
                b_desc + static_cast<uint64_t>((ks * 2048) >> 4), idesc, (b > 0 || ks > 0) ? 1u : 0u);
      }
      TcCommit(mma_done0 + buf * 8);
    }
    // The last commit covers every MMA before it.  Its phase is unambiguous here: the converters of the last block
    // had already waited for the same barrier's previous phase.
    if (nblocks > 0) ok = MbarWait(mma_done0 + ((nblocks - 1) % L::kBufs) * 8, ((nblocks - 1) / L::kBufs) & 1) && ok;
  }
  if (!ok) atomicExch(&g_tc_status, 1);
  if (warp < kTcThreads / 32) CpAsyncWait<0>();
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();  // every MMA has completed; the pipeline space is free
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");

  // Epilogue.  TMEM lane = activation row, TMEM column = output column.  Warp w reads lanes 32 (w % 4) .. + 31 and the
  // quarter w / 4 of the 256 columns, eight columns at a time.
  cg::cluster_group cluster = cg::this_cluster();
  const unsigned rank = cluster.block_rank(), nranks = cluster.num_blocks();
  const int lg = warp & 3, wq = warp >> 2;
  float* tile = reinterpret_cast<float*>(smem);
  YT* y = static_cast<YT*>(p.y);
  const bool direct = MPAD > 128 || nranks == 1;
  if (warp < kTcThreads / 32 && lg * 32 < (MPAD < 128 ? MPAD : 128)) {
#pragma unroll
    for (int acc = 0; acc < L::kAccs; ++acc) {
      const int m = acc * 128 + lg * 32 + lane;
#pragma unroll 2
      for (int c0 = wq * 64; c0 < wq * 64 + 64; c0 += 8) {
        uint32_t rr[8];
        if (nblocks > 0) {
          TcLd8(tmem_base + (static_cast<uint32_t>(lg * 32) << 16) + acc * kTcBN + c0, rr);
          asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
        } else {
#pragma unroll
          for (int e = 0; e < 8; ++e) rr[e] = 0u;
        }
        if (direct) {
          const int col = col0 + c0;  // N is a multiple of 16: eight columns are inside or outside together
          if (m < p.M && col < p.N) {
            float o[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) o[e] = __uint_as_float(rr[e]) * (p.scales != nullptr ? __ldg(p.scales + col + e) : 1.f);
            const size_t at = static_cast<size_t>(m) * p.N + col;
            if (p.residual != nullptr) {
              if ((reinterpret_cast<uintptr_t>(p.residual + at) & 15) == 0) {
                const float4 r0 = __ldg(reinterpret_cast<const float4*>(p.residual + at));
                const float4 r1 = __ldg(reinterpret_cast<const float4*>(p.residual + at + 4));
                o[0] += r0.x; o[1] += r0.y; o[2] += r0.z; o[3] += r0.w;
                o[4] += r1.x; o[5] += r1.y; o[6] += r1.z; o[7] += r1.w;
              } else {
#pragma unroll
                for (int e = 0; e < 8; ++e) o[e] += __ldg(p.residual + at + e);
              }
            }
            StoreRow8(y + at, o);
          }
        } else {
          float4* dst = reinterpret_cast<float4*>(tile + m * kTcTileStride + c0);
          dst[0] = make_float4(__uint_as_float(rr[0]), __uint_as_float(rr[1]), __uint_as_float(rr[2]), __uint_as_float(rr[3]));
          dst[1] = make_float4(__uint_as_float(rr[4]), __uint_as_float(rr[5]), __uint_as_float(rr[6]), __uint_as_float(rr[7]));
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

// CTAs of the kernel that can be resident at once when launched as clusters of ks (index [MPAD class][ks]); filled by
// PrepareInt8GemmTcKernels from the occupancy calculator, because clusters must fit inside a GPC and so do not always
// reach all 148 SMs (clusters of 8 reach 120).
int g_tc_slots[3][9];

template <int MPAD>
void FillTcSlots(int cls)
{
  for (int ks = 1; ks <= 8; ++ks) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(148, ks, 1);
    cfg.blockDim = dim3(kTcLaunchThreads, 1, 1);
    cfg.dynamicSmemBytes = TcLayout<MPAD>::kBytes;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = ks;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, Int8GemmTcKernel<MPAD, float>, &cfg) != cudaSuccess || clusters <= 0) {
      cudaGetLastError();
      clusters = (ks <= 2 ? 148 : ks <= 4 ? 128 : 112) / ks;  // a cautious guess when the query is not available
    }
    g_tc_slots[cls][ks] = clusters * ks;
  }
}

// K slices (1..8) of a launch: the count with the lowest modelled time, in units of one 64-row block of one CTA:
//   waves(ks) * (blocks per slice + fixed cost of a CTA [+ cost of the cluster reduction])
// with waves = ceil(column tiles * ks / resident CTAs).  The constants come from timing the kernel at one full wave
// over a range of K (fixed cost ~10 blocks) and from the reduction's traffic.  $TLALOC_B200_GEMM_KS overrides.
int ChooseTcSlices(int k, int n, int mpad, double* cost_out = nullptr)
{
  static const int forced = [] {
    const char* e = std::getenv("TLALOC_B200_GEMM_KS");
    return e != nullptr ? std::atoi(e) : 0;
  }();
  const int tiles = (n + kTcBN - 1) / kTcBN;
  const int nb = (k + kTcBK - 1) / kTcBK;
  if (mpad > 128) {  // no cluster reduction for two accumulators; a block costs about 1.7x one of a single accumulator
    if (cost_out != nullptr) *cost_out = 1.7 * ((tiles + 147) / 148) * (nb + 10.0);
    return 1;
  }
  if (forced >= 1 && forced <= 8) return forced;
  const int cls = mpad <= 32 ? 0 : mpad <= 64 ? 1 : 2;
  int best = 1;
  double best_cost = 1e30;
  for (int ks = 1; ks <= 8; ++ks) {
    if (ks > 1 && nb / ks < 4) break;
    const int slots = g_tc_slots[cls][ks] > 0 ? g_tc_slots[cls][ks] : 148 / ks * ks;
    const int waves = (tiles * ks + slots - 1) / slots;
    const double per_cta = (nb + ks - 1) / ks + 10.0 + (ks > 1 ? 8.0 + 1.5 * ks : 0.0);
    const double cost = waves * per_cta;
    if (cost < best_cost * 0.97) {  // prefer fewer slices unless the gain is real
      best_cost = cost;
      best = ks;
    }
  }
  if (cost_out != nullptr) *cost_out = best_cost;
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
  if (e == cudaSuccess) {
    FillTcSlots<32>(0);
    FillTcSlots<64>(1);
    FillTcSlots<128>(2);
    done = true;
  }
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
  for (int m0 = 0; m0 < m;) {
    int rows = std::min(256, m - m0);
    if (rows > 128) {
      // Two accumulators share one pass over the weights but cannot split K; with few column tiles two passes of 128
      // rows, each split over K, keep more SMs busy.
      double c256 = 0.0, c128 = 0.0;
      ChooseTcSlices(k, n, 256, &c256);
      ChooseTcSlices(k, n, 128, &c128);
      if (2.0 * c128 < c256) rows = 128;
    }
    const int mpad = rows <= 32 ? 32 : rows <= 64 ? 64 : rows <= 128 ? 128 : 256;
    p.ks = ChooseTcSlices(k, n, mpad);
    const int nb = (k + kTcBK - 1) / kTcBK;
    p.Kc = (nb + p.ks - 1) / p.ks * kTcBK;  // whole blocks per slice; trailing slices may be empty
    p.M = rows;
    p.x = x + static_cast<size_t>(m0) * k;
    p.residual = residual ? residual + static_cast<size_t>(m0) * n : nullptr;
    p.y = static_cast<unsigned char*>(y) + static_cast<size_t>(m0) * n * ybytes;
    const cudaError_t e = y_dtype == TLALOC_B200_F32 ? LaunchTcRows<float>(p, rows, st) : LaunchTcRows<__nv_bfloat16>(p, rows, st);
    if (e != cudaSuccess) return e;
    ++*launches;
    m0 += rows;
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
