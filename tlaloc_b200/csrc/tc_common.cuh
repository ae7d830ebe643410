// Pieces shared by the tensor-core projection kernels: mbarrier waits with a time limit, shared-memory matrix
// descriptors, TMEM loads, and the epilogue that turns a 128 x 256 f32 tile in shared memory into output rows
// (scale, residual, SwiGLU, the sum over the K slices of a cluster).
#pragma once

#include <cooperative_groups.h>

#include "common.cuh"

namespace tlaloc_b200 {
namespace tc {

namespace cg = cooperative_groups;

constexpr int kTcBN = 256;  // output columns per CTA: the N of one MMA
constexpr int kTcTileStride = kTcBN + 4;
constexpr uint32_t kTcSpinLimit = 1u << 22;

__device__ __forceinline__ uint32_t SmemAddr(const void* ptr)
{
  return static_cast<uint32_t>(__cvta_generic_to_shared(ptr));
}
__device__ __forceinline__ void MbarInit(uint32_t bar, uint32_t count)
{
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count) : "memory");
}
// Waits for the phase with the given parity.  Bounded twice over: a wait gives up after kTcWaitNs of wall time, and the
// first wait of a CTA that gives up raises the CTA's abort word in shared memory, which every other wait polls, so a
// pipeline that has stopped costs one time limit and not one per block.  Returns false when it gave up.
constexpr unsigned long long kTcWaitNs = 200ull * 1000ull * 1000ull;  // 0.2 s: a block takes under a microsecond
__device__ __forceinline__ bool MbarWait(uint32_t bar, uint32_t parity, volatile uint32_t* abort_word)
{
  unsigned long long t0 = 0;
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
    if ((i & 31u) == 31u) {
      if (*abort_word != 0u) return false;
      unsigned long long now;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
      if (t0 == 0) t0 = now;
      else if (now - t0 > kTcWaitNs) break;
    }
  }
  *abort_word = 1u;
  return false;
}
// One lane polls for the warp (32 pollers per warp would spend the SM's issue slots on the wait itself).
__device__ __forceinline__ bool MbarWaitWarp(uint32_t bar, uint32_t parity, int lane, volatile uint32_t* abort_word)
{
  int ok = 1;
  if (lane == 0) ok = MbarWait(bar, parity, abort_word) ? 1 : 0;
  ok = __shfl_sync(0xffffffffu, ok, 0);
  return ok != 0;
}

// Shared-memory matrix descriptor of a 128-byte-swizzled operand tile: start address, leading and stride byte offsets
// (all in 16-byte units), descriptor version 1, layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t SmemDesc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes)
{
  return static_cast<uint64_t>((addr >> 4) & 0x3FFFu) | (static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16) |
         (static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void TcCommit(uint32_t bar)
{
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void TcLd32(uint32_t taddr, uint32_t* r)
{
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
        "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
// Four consecutive outputs of one row.
__device__ __forceinline__ void StoreRow4(float* dst, float4 v, bool vec)
{
  if (vec) {
    *reinterpret_cast<float4*>(dst) = v;
  } else {
    dst[0] = v.x; dst[1] = v.y; dst[2] = v.z; dst[3] = v.w;
  }
}
__device__ __forceinline__ void StoreRow4(__nv_bfloat16* dst, float4 v, bool vec)
{
  if (vec) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<const uint32_t*>(&lo);
    u.y = *reinterpret_cast<const uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(dst) = u;
  } else {
    dst[0] = __float2bfloat16_rn(v.x); dst[1] = __float2bfloat16_rn(v.y);
    dst[2] = __float2bfloat16_rn(v.z); dst[3] = __float2bfloat16_rn(v.w);
  }
}

// SiLU(gate) * up as the decode step's SwiGLU kernel computes it (f32, the library exponential).
__device__ __forceinline__ float SiluMulF32(float g, float u) { return __fmul_rn(g / (1.f + expf(-g)), u); }

// The cluster reduction of a gate|up tile: thread n_local < 128 owns gate column n_local and up column 128 + n_local
// of the tile, sums both over the ranks in rank order, and writes silu(gate * scale) * (up * scale) to column
// col_out of the [M, N / 2] result.
template <int NR, typename YT>
__device__ __forceinline__ void ClusterReduceRowsSwiglu(cg::cluster_group& cluster, float* tile, YT* y, int M, int ld_out,
                                                        float scale_g, float scale_u, int n_local, int col_out, int rank, int half)
{
  constexpr int kRows = NR <= 4 ? 16 / NR : 8 / NR;
  constexpr int step = 2 * NR;
  for (int m0 = rank + NR * half; m0 < M; m0 += kRows * step) {
    float tg[NR][kRows], tu[NR][kRows];
#pragma unroll
    for (int q = 0; q < NR; ++q) {
      const float* peer = cluster.map_shared_rank(tile, q) + n_local;
#pragma unroll
      for (int u = 0; u < kRows; ++u) {
        const int m = m0 + u * step;
        tg[q][u] = m < M ? peer[m * kTcTileStride] : 0.f;
        tu[q][u] = m < M ? peer[m * kTcTileStride + 128] : 0.f;
      }
    }
#pragma unroll
    for (int u = 0; u < kRows; ++u) {
      const int m = m0 + u * step;
      float g = tg[0][u], v = tu[0][u];
#pragma unroll
      for (int q = 1; q < NR; ++q) {
        g += tg[q][u];
        v += tu[q][u];
      }
      if (m < M) y[static_cast<size_t>(m) * ld_out + col_out] = FromF32<YT>(SiluMulF32(g * scale_g, v * scale_u));
    }
  }
}

// The K slices of a column tile are the NR ranks of one cluster, each holding its partial tile in shared memory.
// Rank r finishes every NR-th row: a thread owns one column and takes its rows a few at a time, ALL of a trip's
// NR x rows loads from distributed shared memory in flight before the first add (one remote latency per trip, not
// one per rank); each row is summed in rank order, so the result does not depend on which CTA finishes first.
template <int NR, typename YT>
__device__ __forceinline__ void ClusterReduceRows(cg::cluster_group& cluster, float* tile, const float* residual, YT* y,
                                                  int M, int N, float scale, int n_local, int col, int rank, int half)
{
  constexpr int kRows = NR <= 4 ? 32 / NR : 16 / NR;
  constexpr int step = 2 * NR;
  for (int m0 = rank + NR * half; m0 < M; m0 += kRows * step) {
    float t[NR][kRows], res[kRows];
#pragma unroll
    for (int u = 0; u < kRows; ++u) {
      const int m = m0 + u * step;
      res[u] = (residual != nullptr && m < M) ? __ldg(residual + static_cast<size_t>(m) * N + col) : 0.f;
    }
#pragma unroll
    for (int q = 0; q < NR; ++q) {
      const float* peer = cluster.map_shared_rank(tile, q) + n_local;
#pragma unroll
      for (int u = 0; u < kRows; ++u) {
        const int m = m0 + u * step;
        t[q][u] = m < M ? peer[m * kTcTileStride] : 0.f;
      }
    }
#pragma unroll
    for (int u = 0; u < kRows; ++u) {
      const int m = m0 + u * step;
      float v = t[0][u];
#pragma unroll
      for (int q = 1; q < NR; ++q) v += t[q][u];
      if (m < M) y[static_cast<size_t>(m) * N + col] = FromF32<YT>(v * scale + res[u]);
    }
  }
}


struct EpilogueOut {
  const float* residual;  // [M, N] f32 added to the result, or null
  void* y;                // [M, N], or [M, N / 2] with swiglu
  int M, N;
  int swiglu;  // the columns are gate|up blocks of 128 + 128: y = silu(gate) * up (no residual)
};

// A CTA that owns all of K writes its tile: rows [0, kTileRows) of the row-major f32 tile are output rows
// row_base + m, columns col0 .. col0 + 255; 512 threads.  s_scales holds the tile's 256 column scales.
template <int kTileRows, typename YT>
__device__ __forceinline__ void EpilogueRows(const float* tile, const float* s_scales, const EpilogueOut& o, int col0,
                                             int row_base, int tid, bool vec_ok)
{
  YT* y = static_cast<YT*>(o.y);
  if (o.swiglu) {
    // gate|up tile (always whole: N is a multiple of 256 here): 32 threads per row, four output columns each
    const int g4 = (tid & 31) * 4;
    const float4 sg = *reinterpret_cast<const float4*>(s_scales + g4), su = *reinterpret_cast<const float4*>(s_scales + 128 + g4);
    const int ld_out = o.N >> 1;
#pragma unroll 4
    for (int m = tid >> 5; m < kTileRows; m += 16) {
      const int row = row_base + m;
      if (row >= o.M) break;
      const float4 g = *reinterpret_cast<const float4*>(tile + m * kTcTileStride + g4);
      const float4 u = *reinterpret_cast<const float4*>(tile + m * kTcTileStride + 128 + g4);
      const float4 v = make_float4(SiluMulF32(g.x * sg.x, u.x * su.x), SiluMulF32(g.y * sg.y, u.y * su.y),
                                   SiluMulF32(g.z * sg.z, u.z * su.z), SiluMulF32(g.w * sg.w, u.w * su.w));
      StoreRow4(y + static_cast<size_t>(row) * ld_out + (col0 >> 1) + g4, v, vec_ok);
    }
    return;
  }
  // 64 threads per row (four columns each), eight rows per pass.  N is a multiple of 16: four columns are inside or
  // outside together.
  const int c4 = (tid & 63) * 4;
  if (col0 + c4 >= o.N) return;
  const float4 sc = *reinterpret_cast<const float4*>(s_scales + c4);
#pragma unroll 4
  for (int m = tid >> 6; m < kTileRows; m += 8) {
    const int row = row_base + m;
    if (row >= o.M) break;
    float4 v = *reinterpret_cast<const float4*>(tile + m * kTcTileStride + c4);
    const size_t at = static_cast<size_t>(row) * o.N + col0 + c4;
    v.x *= sc.x; v.y *= sc.y; v.z *= sc.z; v.w *= sc.w;
    if (o.residual != nullptr) {
      if (vec_ok) {
        const float4 rs = __ldg(reinterpret_cast<const float4*>(o.residual + at));
        v.x += rs.x; v.y += rs.y; v.z += rs.z; v.w += rs.w;
      } else {
        v.x += __ldg(o.residual + at); v.y += __ldg(o.residual + at + 1);
        v.z += __ldg(o.residual + at + 2); v.w += __ldg(o.residual + at + 3);
      }
    }
    StoreRow4(y + at, v, vec_ok);
  }
}

// The K slices of a column tile, one per CTA of the cluster, meet: call between two cluster.sync() with 512 threads.
template <typename YT>
__device__ __forceinline__ void EpilogueCluster(cg::cluster_group& cluster, float* tile, const float* s_scales,
                                                const EpilogueOut& o, int col0, int tid)
{
  YT* y = static_cast<YT*>(o.y);
  const int nranks = static_cast<int>(cluster.num_blocks()), rk = static_cast<int>(cluster.block_rank());
  const int n_local = tid & 255, col = col0 + n_local, half = tid >> 8;
  if (o.swiglu) {
    if (n_local >= 128) return;
    const float sg = s_scales[n_local], su = s_scales[128 + n_local];
    const int ld_out = o.N >> 1, col_out = (col0 >> 1) + n_local;
    switch (nranks) {
      case 2: ClusterReduceRowsSwiglu<2>(cluster, tile, y, o.M, ld_out, sg, su, n_local, col_out, rk, half); break;
      case 3: ClusterReduceRowsSwiglu<3>(cluster, tile, y, o.M, ld_out, sg, su, n_local, col_out, rk, half); break;
      case 4: ClusterReduceRowsSwiglu<4>(cluster, tile, y, o.M, ld_out, sg, su, n_local, col_out, rk, half); break;
      case 5: ClusterReduceRowsSwiglu<5>(cluster, tile, y, o.M, ld_out, sg, su, n_local, col_out, rk, half); break;
      case 6: ClusterReduceRowsSwiglu<6>(cluster, tile, y, o.M, ld_out, sg, su, n_local, col_out, rk, half); break;
      case 7: ClusterReduceRowsSwiglu<7>(cluster, tile, y, o.M, ld_out, sg, su, n_local, col_out, rk, half); break;
      default: ClusterReduceRowsSwiglu<8>(cluster, tile, y, o.M, ld_out, sg, su, n_local, col_out, rk, half); break;
    }
    return;
  }
  if (col >= o.N) return;
  const float scale = s_scales[n_local];
  switch (nranks) {
    case 2: ClusterReduceRows<2>(cluster, tile, o.residual, y, o.M, o.N, scale, n_local, col, rk, half); break;
    case 3: ClusterReduceRows<3>(cluster, tile, o.residual, y, o.M, o.N, scale, n_local, col, rk, half); break;
    case 4: ClusterReduceRows<4>(cluster, tile, o.residual, y, o.M, o.N, scale, n_local, col, rk, half); break;
    case 5: ClusterReduceRows<5>(cluster, tile, o.residual, y, o.M, o.N, scale, n_local, col, rk, half); break;
    case 6: ClusterReduceRows<6>(cluster, tile, o.residual, y, o.M, o.N, scale, n_local, col, rk, half); break;
    case 7: ClusterReduceRows<7>(cluster, tile, o.residual, y, o.M, o.N, scale, n_local, col, rk, half); break;
    default: ClusterReduceRows<8>(cluster, tile, o.residual, y, o.M, o.N, scale, n_local, col, rk, half); break;
  }
}

}  // namespace tc
}  // namespace tlaloc_b200
