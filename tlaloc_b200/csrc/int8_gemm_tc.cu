// The int8 weight-only projection for batches of rows (17 and more; at most 256 per launch) on the 5th-generation tensor
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
//      (two logic ops and one packed fma per pair, plus one shift per word) and stores them as the MN-major 128-byte-swizzled B
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
// Epilogue: tcgen05.ld brings the accumulator to registers (lane = activation row, 64 output columns per thread) and
// a row-major tile in shared memory turns that into 1 KB coalesced row stores with scale and residual applied; with
// several K slices, the slices of a column tile form a thread-block cluster and their tiles meet in distributed
// shared memory, summed in rank order (deterministic).  The dependency wait of the programmatic launch sits after the
// on-chip set-up (and, for constant weights, after the first weight loads have been requested).
// Every mbarrier wait is bounded: on a time-out the kernel records it in a status word, frees its TMEM and returns.
#include <cooperative_groups.h>

#include <mutex>
#include <string>
#include <type_traits>

#include "common.cuh"
#include "tc_common.cuh"

namespace cg = cooperative_groups;

namespace tlaloc_b200 {
namespace {

using namespace tc;

struct TcParams {
  const __nv_bfloat16* x;  // [M, K]
  const int8_t* w;         // [K, N]
  const float* scales;
  const float* residual;
  void* y;
  int M, K, N;
  int Kc, ks;
  int weights_const;  // codes and scales are not written by the preceding kernel: fetch them before the dependency wait
  int swiglu;         // the columns are gate|up blocks of 128 + 128: y [M, N / 2] = silu(gate) * up (no residual)
};

constexpr int kTcThreads = 512;                    // converter threads (16 warps)
constexpr int kTcLaunchThreads = kTcThreads + 32;  // plus one warp whose first lane issues the MMAs
constexpr int kTcBK = 64;                          // k rows per block
constexpr int kTcWBytes = kTcBN * kTcBK * 2;       // one block's weights as bf16

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
  static constexpr int kPipeEnd = kWOffset + kBufs * kTcWBytes;
  static constexpr int kTileRows = MPAD < 128 ? MPAD : 128;
  static constexpr int kTileBytes = kTileRows * kTcTileStride * 4;  // epilogue tile of one accumulator; aliases the pipeline
  // mma_done[kBufs], conv_done[kBufs], the TMEM base and the abort word, then the tile's 256 scales: past both the
  // pipeline and the tile
  static constexpr int kBarOffset = (kPipeEnd > kTileBytes ? kPipeEnd : kTileBytes + 15) / 16 * 16;
  static constexpr int kScaleOffset = kBarOffset + 128;
  static constexpr int kBytes = kScaleOffset + kTcBN * 4 + 1024;  // slack to align to 1024
  static constexpr int kAccs = MPAD > 128 ? 2 : 1;  // accumulators of 128 activation rows x 256 columns
  static constexpr int kTmemCols = kAccs * kTcBN;
  static_assert(kXBytes % 1024 == 0, "operand tiles start on 1024-byte boundaries");
};

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
__device__ __forceinline__ uint4 LdWeights16Always(const int8_t* ptr)
{
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(ptr));
  return v;
}
__device__ __forceinline__ void StShared16(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d)
{
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};\n" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
// Two codes in the LOW bytes of the two halves of q (the high bytes are ignored) as an exact bf16 pair: for a code v
// with bits s:lo7, 0x4300|lo7 is the bf16 128 + lo7 and 0xC300|s<<7 is -128 or -256; their sum is v.
__device__ __forceinline__ uint32_t LowBytesToBf16x2(uint32_t q)
{
  uint32_t t, c, r;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;\n" : "=r"(t) : "r"(q), "r"(0x007F007Fu), "r"(0x43004300u));
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;\n" : "=r"(c) : "r"(q), "r"(0x00800080u), "r"(0xC300C300u));
  asm("fma.rn.bf16x2 %0, %1, %2, %3;\n" : "=r"(r) : "r"(t), "r"(0x3F803F80u), "r"(c));
  return r;
}
// The four codes c0..c3 of one word as the pairs (c0, c2) and (c1, c3): the even bytes already sit in the low byte of
// each half, the odd ones after one shift, so no byte permute is needed.  The weight tile therefore holds its columns
// in the order 0 2 1 3 within every group of four; the epilogue swaps them back on the way out of TMEM.
__device__ __forceinline__ void WordToBf16(uint32_t w, uint32_t& even, uint32_t& odd)
{
  even = LowBytesToBf16x2(w);
  odd = LowBytesToBf16x2(w >> 8);
}

// kind::f16 instruction descriptor: f32 accumulator, bf16 A and B (the two operand formats must agree: a bf16 A with an
// f16 B raises an illegal-instruction error), A K-major, B MN-major, M = 128, N = 256.
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
  volatile uint32_t* abort_word = tmem_slot + 1;  // raised by the first wait that gives up

  if (tid == 0) {
    *abort_word = 0u;
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

  // Converter warps, in kGroups groups; a group takes every kGroups-th block and does ALL of it, so the fixed costs
  // of a block (barrier wait, strip request, proxy fence, arrival) are paid by a few warps instead of sixteen and
  // the groups' phases interleave on the schedulers instead of coinciding.
  // Within a block a warp owns k rows 2 wg + r + kRowsPerPass * i, all 256 columns: lane = atom * 8 + r * 4 + j
  // holds 16 codes of columns atom * 64 + 16 j.  Global loads: two 256-byte runs per warp instruction.  Shared
  // stores: a quarter-warp writes two adjacent k rows of one 64-column atom, whose swizzled 16-byte slots have
  // opposite parity.
  constexpr int kG = L::kGroups, kChunks = L::kChunks, kRP = L::kRowsPerPass, kXR = L::kXRowsPerPass;
  const bool conv = warp < kTcThreads / 32;
  const int grp = warp / L::kGroupWarps, wg = warp % L::kGroupWarps, gtid = tid % L::kGroupThreads;
  const int j = lane & 3, r = (lane >> 2) & 1, atom = lane >> 3;
  const int row0 = 2 * wg + r, k_in = row0 & 7;  // rows row0 + kRP * i; kRP is a multiple of 8, so k % 8 is fixed
  const int ccol = atom * 64 + j * 16;
  const bool col_ok = conv && col0 + ccol < p.N;
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
  float* s_scales = reinterpret_cast<float*>(smem + L::kScaleOffset);
  const int x_rows = p.M > xm0 ? (p.M - xm0 + kXR - 1) / kXR : 0;  // strip rows this thread copies: xm0 + kXR * i < M
  const bool tile_full = col0 + kTcBN <= p.N;

  // Everything above touched only shared memory and TMEM.  The weights and scales are the first global reads; when
  // the caller says no preceding kernel writes them they are requested BEFORE the dependency wait, so the coldest
  // loads of the launch travel while the predecessor drains.  The activations always come after it.
  uint4 wreg[kChunks];
  if (!p.weights_const) GridDependencySync();
#pragma unroll
  for (int i = 0; i < kChunks; ++i)
    wreg[i] = LdWeights16(wp + static_cast<size_t>(grp) * blk + i * pass, col_ok && kb0 + grp * kTcBK + row0 + kRP * i < ke);
  // this thread's scale: requested now, parked in shared memory after the main loop (nobody waits for it here)
  const float my_scale = (tid < kTcBN && p.scales != nullptr && col0 + tid < p.N) ? __ldg(p.scales + col0 + tid) : 1.f;
  if (p.weights_const) GridDependencySync();

  bool ok = true;
  if (conv) {
    for (int b = grp; b < nblocks; b += kG) {
      const int buf = b % L::kBufs;
      // Block b - kBufs used this weight tile and this strip buffer.
      if (b >= L::kBufs) ok = MbarWaitWarp(mma_done0 + buf * 8, ((b / L::kBufs) - 1) & 1, lane, abort_word) && ok;
      const int k0 = kb0 + b * kTcBK;
      {
        const uint32_t st = smem_base + buf * L::kXBytes + xdst0;
        const __nv_bfloat16* src = xsrc0 + b * kTcBK;
        if (k0 + kTcBK <= ke) {
          // A full block: only rows that exist are requested.  The rows past M keep whatever the buffer held; they
          // feed accumulator lanes that are never read.  (A partial block must zero-fill its missing k instead:
          // garbage there would meet the zero weights of those k and 0 x NaN is NaN.)
#pragma unroll
          for (int i = 0; i < MPAD / kXR; ++i)
            if (i < x_rows) CpAsync16(st + i * (kXR * 128), src + i * xstep, 16);
        } else {
          const bool k_ok = k0 + xch * 8 < ke;
#pragma unroll
          for (int i = 0; i < MPAD / kXR; ++i) {
            const bool valid = k_ok && i < x_rows;
            CpAsync16(st + i * (kXR * 128), valid ? src + i * xstep : p.x, valid ? 16 : 0);
          }
        }
        CpAsyncCommit();
      }
      const uint32_t bt = smem_base + L::kWOffset + buf * kTcWBytes + dst_off;
      const int8_t* next = wp + static_cast<size_t>(b + kG) * blk;
      const int next_k = k0 + kG * kTcBK + row0;  // at or past ke when this was the group's last block
      auto convert_block = [&](auto fast) {
#pragma unroll
        for (int i = 0; i < kChunks; ++i) {
          const uint4 v = wreg[i];
          uint32_t o0, o1, o2, o3, o4, o5, o6, o7;
          WordToBf16(v.x, o0, o1);
          WordToBf16(v.y, o2, o3);
          WordToBf16(v.z, o4, o5);
          WordToBf16(v.w, o6, o7);
          StShared16(bt + i * (kRP * 128) + s0, o0, o1, o2, o3);
          StShared16(bt + i * (kRP * 128) + s1, o4, o5, o6, o7);
          // the group's next block, one group period ahead
          if constexpr (decltype(fast)::value) wreg[i] = LdWeights16Always(next + i * pass);
          else wreg[i] = LdWeights16(next + i * pass, col_ok && next_k + kRP * i < ke);
        }
      };
      // Uniform over the CTA: the next block exists, is a whole block, and the tile has all its 256 columns.
      if (tile_full && k0 + (kG + 1) * kTcBK <= ke) convert_block(std::true_type{});
      else convert_block(std::false_type{});
      CpAsyncWait<0>();  // this thread's part of the strip has landed
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");  // these writes (and the cp.async strip) -> tensor core
      __syncwarp();
      if (lane == 0) {
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(conv_done0 + buf * 8) : "memory");
      }
    }
  } else {
    // The MMA thread (one lane; nothing else may sit between a block's arrival and its MMAs): for each block, wait for
    // its converter group, then 4 K-steps of 128 x 256 x 16 per accumulator and a commit.  A = the activation strip
    // (K-major), B = the converted weights (MN-major).  Descriptors differ from block to block only in the 14-bit
    // start-address field, so they are built once and advanced by adds.
    if (lane == 0) {
      constexpr uint32_t idesc = InstrDesc();
      const uint64_t a_desc0 = SmemDesc(smem_base, 16, 1024), b_desc0 = SmemDesc(smem_base + L::kWOffset, 8192, 1024);
      for (int b = 0; b < nblocks; ++b) {
        const int buf = b % L::kBufs;
        ok = MbarWait(conv_done0 + buf * 8, (b / L::kBufs) & 1, abort_word) && ok;
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
      if (nblocks > 0) ok = MbarWait(mma_done0 + ((nblocks - 1) % L::kBufs) * 8, ((nblocks - 1) / L::kBufs) & 1, abort_word) && ok;
    }
  }
  if (!ok) atomicExch(&g_tc_status, 1);
  if (conv) CpAsyncWait<0>();
  if (tid < kTcBN) s_scales[tid] = my_scale;
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();  // every MMA has completed; the pipeline space is free
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");

  // Epilogue.  TMEM lane = activation row, TMEM column = output column, but a row of the output is contiguous along
  // the columns: storing straight from the tcgen05.ld registers would touch 32 different rows per warp instruction
  // (measured: 12k cycles for a 128 x 256 tile).  So the accumulator first goes to a row-major tile in shared memory
  // (warp w reads lanes 32 (w % 4) .. + 31 and the quarter w / 4 of the columns: two tcgen05.ld of 32 columns, one
  // wait, sixteen 16-byte stores without bank conflicts), and leaves it row by row, 1 KB per row, coalesced.
  cg::cluster_group cluster = cg::this_cluster();
  const unsigned rank = cluster.block_rank(), nranks = cluster.num_blocks();
  const int lg = warp & 3, wq = warp >> 2;
  float* tile = reinterpret_cast<float*>(smem);
  const EpilogueOut out{p.residual, p.y, p.M, p.N, p.swiglu};
  const bool vec_ok = (reinterpret_cast<uintptr_t>(p.y) & 15) == 0 && (reinterpret_cast<uintptr_t>(p.residual) & 15) == 0;
#pragma unroll
  for (int acc = 0; acc < L::kAccs; ++acc) {
    if (conv && lg * 32 < L::kTileRows) {
      const int m = lg * 32 + lane;
      uint32_t rr[64];
      if (nblocks > 0) {
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(lg * 32) << 16) + acc * kTcBN + wq * 64;
        TcLd32(taddr, rr);
        TcLd32(taddr + 32, rr + 32);
        asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
      } else {
#pragma unroll
        for (int e = 0; e < 64; ++e) rr[e] = 0u;
      }
      float4* dst = reinterpret_cast<float4*>(tile + m * kTcTileStride + wq * 64);
#pragma unroll
      for (int c = 0; c < 16; ++c)
        dst[c] = make_float4(__uint_as_float(rr[4 * c]), __uint_as_float(rr[4 * c + 2]), __uint_as_float(rr[4 * c + 1]),
                             __uint_as_float(rr[4 * c + 3]));  // TMEM holds the columns as 0 2 1 3 (see WordToBf16)
    }
    if (nranks == 1) {
      __syncthreads();
      if (conv) EpilogueRows<L::kTileRows, YT>(tile, s_scales, out, col0, acc * 128, tid, vec_ok);
      if (acc + 1 < L::kAccs) __syncthreads();  // the tile is reused by the second accumulator
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  if (nranks > 1) {  // only launched with one accumulator
    cluster.sync();
    if (conv) EpilogueCluster<YT>(cluster, tile, s_scales, out, col0, tid);
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
  cudaLaunchAttribute attr[2];
  cfg.numAttrs = ChainAttributes(attr, p.ks);
  cfg.attrs = attr;
  return cudaLaunchKernelEx(&cfg, Int8GemmTcKernel<MPAD, YT>, p);
}

// CTAs of the kernel that can be resident at once when launched as clusters of ks (index [device][MPAD class][ks]);
// filled per device by PrepareInt8GemmTcKernels from the occupancy calculator, because clusters must fit inside a GPC
// and so do not always reach all 148 SMs (clusters of 8 reach 120).
int g_tc_slots[kMaxDevices][3][9];

template <int MPAD>
void FillTcSlots(int device, int cls)
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
    g_tc_slots[device][cls][ks] = clusters * ks;
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
  if (mpad > 128) {  // no cluster reduction for two accumulators; a block costs about twice one of a single accumulator
    if (cost_out != nullptr) *cost_out = 2.0 * ((tiles + 147) / 148) * (nb + 10.0);
    return 1;
  }
  if (forced >= 1 && forced <= 8) return forced;
  const int cls = mpad <= 32 ? 0 : mpad <= 64 ? 1 : 2;
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) device = 0;
  int best = 1;
  double best_cost = 1e30;
  for (int ks = 1; ks <= 8; ++ks) {
    if (ks > 1 && nb / ks < 4) break;
    const int slots = g_tc_slots[device][cls][ks] > 0 ? g_tc_slots[device][cls][ks] : 148 / ks * ks;
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
  static OncePerDevice once;
  return once.Run([](int device) {
    cudaError_t e = PrepareTc<32, float>();
    if (e == cudaSuccess) e = PrepareTc<32, __nv_bfloat16>();
    if (e == cudaSuccess) e = PrepareTc<64, float>();
    if (e == cudaSuccess) e = PrepareTc<64, __nv_bfloat16>();
    if (e == cudaSuccess) e = PrepareTc<128, float>();
    if (e == cudaSuccess) e = PrepareTc<128, __nv_bfloat16>();
    if (e == cudaSuccess) e = PrepareTc<256, float>();
    if (e == cudaSuccess) e = PrepareTc<256, __nv_bfloat16>();
    if (e == cudaSuccess) {
      FillTcSlots<32>(device, 0);
      FillTcSlots<64>(device, 1);
      FillTcSlots<128>(device, 2);
    }
    return e;
  });
}

// Rows [0, m) of the projection on the tensor-core kernel, at most 256 rows per launch.  x is bf16.
cudaError_t LaunchInt8GemmTc(const __nv_bfloat16* x, const int8_t* codes, const float* scales, const float* residual,
                             void* y, int y_dtype, int m, int k, int n, cudaStream_t st, int* launches, bool weights_const,
                             bool swiglu)
{
  TcParams p;
  p.weights_const = weights_const ? 1 : 0;
  p.swiglu = swiglu ? 1 : 0;
  p.w = codes;
  p.scales = scales;
  p.K = k;
  p.N = n;
  const size_t ybytes = DtypeBytes(y_dtype);
  const int nb = (k + kTcBK - 1) / kTcBK;
  for (int m0 = 0; m0 < m;) {
    int rows = std::min(256, m - m0);
    if (rows > 128) {
      // Two accumulators share one pass over the weights but cannot split K; with few column tiles two passes of 128
      // rows, each split over K, keep more SMs busy.
      double c256 = 0.0, c128 = 0.0;
      ChooseTcSlices(k, n, 128, &c128);
      ChooseTcSlices(k, n, 256, &c256);
      if (2.0 * c128 < c256) rows = 128;
    }
    const int mpad = rows <= 32 ? 32 : rows <= 64 ? 64 : rows <= 128 ? 128 : 256;
    p.ks = ChooseTcSlices(k, n, mpad);
    p.Kc = (nb + p.ks - 1) / p.ks * kTcBK;  // whole blocks per slice; trailing slices may be empty
    p.M = rows;
    p.x = x + static_cast<size_t>(m0) * k;
    p.residual = residual ? residual + static_cast<size_t>(m0) * n : nullptr;
    p.y = static_cast<unsigned char*>(y) + static_cast<size_t>(m0) * (swiglu ? n / 2 : n) * ybytes;
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
