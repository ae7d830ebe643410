// Paged-attention decode for sm_100a: context-split slice kernels + a combine pass.
//
// PAGED_ATTENTION as the reference defines it (ir/.../PagedAttentionAttrs.kt:79-286,
// interpreter ir/.../passes/DxirInterpreter.kt:2049-2140): row r of the query attends
// positions [first, seq_lens[r]) of the pages its block table names, query head h
// reading kv head h / group.
//
// Work decomposition (both slice kernels): one CTA per (context slice, kv head, block
// table).  A CTA serves every query that reads that kv head through that table
// (rows_per_table x group of them), so each K/V byte of the slice is fetched from HBM
// once.  Each CTA leaves one record {max, sum, acc[D]} per query in the caller's
// scratch [S, R, H, D + 2]; PaCombine merges the records of a row's live slices.
// Slices that hold no live position of any of the CTA's rows exit without writing:
// the combine pass derives a row's live slice range from seq_lens itself.
//
//   PaSliceMma      bf16 pools, D in {64, 128}, <= 16 queries per CTA.  Four warps,
//                   each an independent cp.async pipeline over its own 16-position
//                   groups (16-byte coalesced copies of each position's 2*D-byte row,
//                   gathered through the block table, XOR-swizzled in shared memory);
//                   the 16 positions of a group are the M rows of mma.sync m16n8k16 bf16
//                   (S = K.Q^T with Q^T held in registers as B fragments for the whole
//                   slice; O^T += V^T.P with P moved between fragment layouts by
//                   movmatrix), the queries the N columns, fp32 accumulators; the
//                   probabilities (and an f32 query) are carried as hi + lo bf16 parts so
//                   the result keeps ~16 bits; online softmax in the log2 domain.
//                   HBM-bound once the per-group instruction count is low enough: with the
//                   queries as M rows the kernel was bound by instruction issue instead.
//   PaSliceGeneric  any D <= 256, any block size, f32 or bf16 pools, keep masks, up to
//                   any number of queries (in passes of 8): plain fp32 FMA, warp per
//                   position for the scores and thread per head dimension for the values.
#include <cuda.h>
#include <mutex>

#include "common.cuh"
#include "tc_common.cuh"

namespace tlaloc_b200 {
namespace {

struct PaParams {
  const void* q;
  const void* kc;
  const void* vc;
  const int* tables;
  const int* lens;
  const int* keep;
  float* scratch;
  void* out;
  float* lse;
  int R, H, Hkv, D, bs, M, Tb, P;
  int S;      // context slices in use
  int slice;  // positions per slice
  int group, rpt, NQ;
  int window, keep_chunks, keep_chunk;
  int bs_shift;  // log2(bs) when bs is a power of two, else -1
  float scale;
};

__device__ __forceinline__ int ClampI(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }

__device__ __forceinline__ bool Kept(const PaParams& p, int row, int pos)
{
  return p.keep == nullptr || __ldg(p.keep + static_cast<size_t>(row) * p.keep_chunks + pos / p.keep_chunk) != 0;
}

__device__ __forceinline__ float* Record(const PaParams& p, int s, int row, int head)
{
  return p.scratch + ((static_cast<size_t>(s) * p.R + row) * p.H + head) * (p.D + 2);
}

// ------------------------------------------------------------------------------------------
// The generic slice kernel.

constexpr int kGenThreads = 128;
constexpr int kGenTile = 128;  // positions per tile
constexpr int kGenQ = 8;       // queries per pass

template <typename QT, typename KVT>
__global__ void __launch_bounds__(kGenThreads) PaSliceGeneric(PaParams p)
{
  GridDependencySync();
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* qs = reinterpret_cast<float*>(smem_raw);                      // [kGenQ][D]
  float* sc = qs + kGenQ * p.D;                                        // [kGenQ][kGenTile]
  long long* off = reinterpret_cast<long long*>(sc + kGenQ * kGenTile);  // [kGenTile]
  __shared__ float m_s[kGenQ], l_s[kGenQ], alpha_s[kGenQ];
  __shared__ int len_s[kGenQ], first_s[kGenQ], row_s[kGenQ], head_s[kGenQ];

  const int s = blockIdx.x, kv = blockIdx.y, tb = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int D = p.D, ctx = p.M * p.bs;
  const int c0 = s * p.slice;
  const int c1max = min(c0 + p.slice, ctx);
  const QT* q = static_cast<const QT*>(p.q);
  const KVT* kc = static_cast<const KVT*>(p.kc);
  const KVT* vc = static_cast<const KVT*>(p.vc);

  for (int q0 = 0; q0 < p.NQ; q0 += kGenQ) {
    const int nq = min(kGenQ, p.NQ - q0);
    __syncthreads();
    if (tid < kGenQ) {
      int row = 0, head = 0, len = 0, first = 0;
      if (tid < nq) {
        const int i = q0 + tid;
        row = tb * p.rpt + i / p.group;
        head = kv * p.group + i % p.group;
        len = ClampI(__ldg(p.lens + row), 0, ctx);
        first = p.window > 0 ? max(0, len - p.window) : 0;
      }
      row_s[tid] = row;
      head_s[tid] = head;
      len_s[tid] = len;
      first_s[tid] = first;
      m_s[tid] = -INFINITY;
      l_s[tid] = 0.f;
      alpha_s[tid] = 0.f;
    }
    __syncthreads();
    int maxlen = 0, minfirst = ctx;
    for (int i = 0; i < nq; ++i) {
      maxlen = max(maxlen, len_s[i]);
      minfirst = min(minfirst, first_s[i]);
    }
    const int c1 = min(c1max, maxlen);
    const int t_begin = max(c0, minfirst);
    if (t_begin >= c1) continue;  // no live position for these rows here: no record (see PaCombine)
    for (int idx = tid; idx < kGenQ * D; idx += kGenThreads) {
      const int i = idx / D, d = idx - i * D;
      qs[idx] = i < nq ? ToF32(q[(static_cast<size_t>(row_s[i]) * p.H + head_s[i]) * D + d]) : 0.f;
    }
    float acc[kGenQ][2];
#pragma unroll
    for (int i = 0; i < kGenQ; ++i) acc[i][0] = acc[i][1] = 0.f;

    for (int t0 = t_begin; t0 < c1; t0 += kGenTile) {
      __syncthreads();
      const int tn = min(kGenTile, c1 - t0);
      if (tid < tn) {
        const int t = t0 + tid;
        const int blk = ClampI(__ldg(p.tables + static_cast<size_t>(tb) * p.M + t / p.bs), 0, p.P - 1);
        off[tid] = ((static_cast<long long>(blk) * p.bs + t % p.bs) * p.Hkv + kv) * D;
      }
      __syncthreads();
      // Scores: a warp per position, lanes across the head dimension.
      for (int j = warp; j < tn; j += kGenThreads / 32) {
        const KVT* kr = kc + off[j];
        float part[kGenQ];
#pragma unroll
        for (int i = 0; i < kGenQ; ++i) part[i] = 0.f;
        for (int d = lane; d < D; d += 32) {
          const float kd = ToF32(kr[d]);
#pragma unroll
          for (int i = 0; i < kGenQ; ++i) part[i] = fmaf(qs[i * D + d], kd, part[i]);
        }
        float mine = 0.f;
#pragma unroll
        for (int i = 0; i < kGenQ; ++i) {
          float v = part[i];
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
          if (lane == i) mine = v;
        }
        if (lane < kGenQ) {
          const int t = t0 + j;
          const bool live = lane < nq && t >= first_s[lane] && t < len_s[lane] && Kept(p, row_s[lane], t);
          sc[lane * kGenTile + j] = live ? mine * p.scale : -INFINITY;
        }
      }
      __syncthreads();
      // Online softmax: a warp per query.
      for (int i = warp; i < nq; i += kGenThreads / 32) {
        float tmax = -INFINITY;
        for (int j = lane; j < tn; j += 32) tmax = fmaxf(tmax, sc[i * kGenTile + j]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, o));
        const float m_old = m_s[i], m_new = fmaxf(m_old, tmax);
        float sum = 0.f;
        for (int j = lane; j < tn; j += 32) {
          const float x = sc[i * kGenTile + j];
          const float e = x == -INFINITY ? 0.f : expf(x - m_new);
          sc[i * kGenTile + j] = e;
          sum += e;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        if (lane == 0) {
          const float alpha = m_old == -INFINITY ? 0.f : expf(m_old - m_new);
          l_s[i] = l_s[i] * alpha + sum;
          m_s[i] = m_new;
          alpha_s[i] = alpha;
        }
      }
      __syncthreads();
      // Values: a thread per head dimension (two when D > 128), coalesced across the row.
#pragma unroll
      for (int dd = 0; dd < 2; ++dd) {
        const int d = tid + dd * kGenThreads;
        if (d < D) {
#pragma unroll
          for (int i = 0; i < kGenQ; ++i) acc[i][dd] *= alpha_s[i];
          for (int j = 0; j < tn; ++j) {
            const float v = ToF32(vc[off[j] + d]);
#pragma unroll
            for (int i = 0; i < kGenQ; ++i)
              if (i < nq) acc[i][dd] = fmaf(sc[i * kGenTile + j], v, acc[i][dd]);
          }
        }
      }
    }
#pragma unroll
    for (int i = 0; i < kGenQ; ++i) {
      if (i < nq) {
        float* rec = Record(p, s, row_s[i], head_s[i]);
        if (tid == 0) {
          rec[0] = m_s[i];
          rec[1] = l_s[i];
        }
#pragma unroll
        for (int dd = 0; dd < 2; ++dd) {
          const int d = tid + dd * kGenThreads;
          if (d < D) rec[2 + d] = acc[i][dd];
        }
      }
    }
  }
}

// ------------------------------------------------------------------------------------------
// The tensor-core slice kernel (bf16 pools).
//
// Orientation: the 16 positions of a group are the M dimension of every MMA and the (<= 8 per n-tile) queries
// the N dimension, so a group costs D/16 MMAs for S^T = K Q^T and D/16 (x2: hi and lo parts of P) for
// O^T = V^T P^T, and nothing is padded beyond 8 queries.  Q^T lives in registers as B fragments for the whole
// kernel; K is read from shared memory as A fragments (ldmatrix), V^T as A fragments (ldmatrix.trans); the
// probabilities go from accumulator layout to B-fragment layout with movmatrix.

constexpr int kMmaThreads = 128;
constexpr int kMmaWarps = 4;
constexpr int kMmaQ = 16;  // the most queries per (table, kv head) this kernel takes: two n-tiles of 8
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

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
__device__ __forceinline__ void LdMatrixX4Trans(uint32_t (&r)[4], uint32_t addr)
{
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ uint32_t MovMatrixTrans(uint32_t a)
{
  uint32_t d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(d) : "r"(a));
  return d;
}
__device__ __forceinline__ void MmaBf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
{
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float Exp2(float x)
{
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
// Two floats as bf16 hi parts (lower index in the low half) and the bf16 of what is left.
__device__ __forceinline__ void SplitPack(float x, float y, uint32_t& hi, uint32_t& lo)
{
  const __nv_bfloat16 xh = __float2bfloat16_rn(x), yh = __float2bfloat16_rn(y);
  const __nv_bfloat16 xl = __float2bfloat16_rn(x - __bfloat162float(xh));
  const __nv_bfloat16 yl = __float2bfloat16_rn(y - __bfloat162float(yh));
  hi = static_cast<uint32_t>(__bfloat16_as_ushort(xh)) | (static_cast<uint32_t>(__bfloat16_as_ushort(yh)) << 16);
  lo = static_cast<uint32_t>(__bfloat16_as_ushort(xl)) | (static_cast<uint32_t>(__bfloat16_as_ushort(yl)) << 16);
}

// Dynamic shared memory of PaSliceMma, in bytes: the four warps' stages, then the slice's block-table entries.
template <int D, int NS>
struct MmaLayout {
  static constexpr int kRowBytes = D * 2;
  static constexpr int kTileBytes = 16 * kRowBytes;  // 16 positions of K (or V)
  static constexpr int kStageBytes = 2 * kTileBytes;
  static constexpr int kWarpBytes = NS * kStageBytes;
  static constexpr int kTabOffset = kMmaWarps * kWarpBytes;
  static_assert(kWarpBytes >= static_cast<int>(sizeof(float)) * kMmaQ * (D + 2), "a warp's stages hold its partial record");
  static size_t Bytes(int tab_entries) { return kTabOffset + sizeof(int) * static_cast<size_t>(tab_entries); }
};

// QT: the query's element type (an f32 query is carried as hi + lo bf16 parts); NT: n-tiles of 8 queries.
// TMA: the K and V tiles arrive as boxes of a tensor map over the pool (one lane issues them, an mbarrier per warp and
// stage counts their bytes) instead of 16-byte cp.async copies issued by every lane; the tile then lies in shared memory
// as 128-byte rows (one 2 KB sub-tile per 64 channels) under the 128-byte swizzle.  Needs a group of 16 positions to
// lie inside one block (block size a power of two >= 16).
__device__ int g_pa_status;  // 1: a wait for a K/V tile ran out (the launch's result is then not valid)

__device__ __forceinline__ void TmaLoad3d(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint32_t bar)
{
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];\n" ::"r"(dst),
               "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(z), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void PaMbarExpectTx(uint32_t bar, uint32_t bytes)
{
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}

template <typename QT, int D, int NS, int NT, bool TMA>
__device__ __forceinline__ void PaSliceMmaBody(const PaParams& p, const CUtensorMap* map_k, const CUtensorMap* map_v)
{
  GridDependencySync();
  constexpr bool QLO = sizeof(QT) == 4;
  using L = MmaLayout<D, NS>;
  constexpr int CPR = L::kRowBytes / 16;  // 16-byte chunks per row
  constexpr int KS = D / 16;              // k-steps of Q K^T, m-tiles of V^T P^T
  extern __shared__ __align__(1024) unsigned char smem[];
  unsigned char* stages = smem;
  int* tab = reinterpret_cast<int*>(smem + L::kTabOffset);
  __shared__ __align__(8) unsigned long long tile_bars[kMmaWarps * NS];
  __shared__ uint32_t abort_word;

  const int s = blockIdx.x, kv = blockIdx.y, tb = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int gid = lane >> 2, tig = lane & 3;
  const int ctx = p.M * p.bs;
  const int c0 = s * p.slice;

  // The slice's block-table entries are requested first and for the whole slice, whatever the rows' lengths turn out
  // to be, so that this load and the lengths travel together instead of one after the other (entries past the live
  // range are clamped and never used).
  const int c_end = min(c0 + p.slice, ctx);
  const int b0 = p.bs_shift >= 0 ? (c0 >> p.bs_shift) : c0 / p.bs;
  const int b_last = c_end > c0 ? (p.bs_shift >= 0 ? ((c_end - 1) >> p.bs_shift) : (c_end - 1) / p.bs) : b0 - 1;
  for (int j = tid; j <= b_last - b0; j += kMmaThreads) {
    tab[j] = ClampI(__ldg(p.tables + static_cast<size_t>(tb) * p.M + b0 + j), 0, p.P - 1);
  }
  // Every thread derives the CTA's live range from its rows' lengths.
  int maxlen = 0, minfirst = ctx;
  for (int r = 0; r < p.rpt; ++r) {
    const int len = ClampI(__ldg(p.lens + tb * p.rpt + r), 0, ctx);
    maxlen = max(maxlen, len);
    minfirst = min(minfirst, p.window > 0 ? max(0, len - p.window) : 0);
  }
  const int c1 = min(min(c0 + p.slice, ctx), maxlen);
  const int t_begin = max(c0, minfirst) & ~15;  // groups start on multiples of 16 (the slice start is one)
  if (t_begin >= c1) return;
  const int ngroups = (c1 - t_begin + 15) >> 4;


  // This lane's queries: column 2*tig + e of n-tile nt is query nt*8 + 2*tig + e (row / head as below).
  int qlen[NT][2], qfirst[NT][2];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int i = nt * 8 + 2 * tig + e;
      int len = 0, first = 0;
      if (i < p.NQ) {
        const int full = ClampI(__ldg(p.lens + tb * p.rpt + i / p.group), 0, ctx);
        first = p.window > 0 ? max(0, full - p.window) : 0;
        len = min(full, c1);
      }
      qlen[nt][e] = len;
      qfirst[nt][e] = first;
    }
  }
  // Q^T as B fragments: for k-step kk, b0b1 = Q[query gid][16kk + 2tig, +1], b2b3 = Q[query gid][16kk + 8 + 2tig, +1].
  uint32_t qh[NT][KS][2], ql[QLO ? NT : 1][QLO ? KS : 1][2];
  {
    const QT* q = static_cast<const QT*>(p.q);
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const int i = nt * 8 + gid;
      const bool have = i < p.NQ;
      const QT* src = q + (static_cast<size_t>(tb * p.rpt + (have ? i / p.group : 0)) * p.H + kv * p.group + (have ? i % p.group : 0)) * D;
#pragma unroll
      for (int kk = 0; kk < KS; ++kk) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int d = 16 * kk + 8 * h + 2 * tig;
          const float x = have ? ToF32(src[d]) : 0.f, y = have ? ToF32(src[d + 1]) : 0.f;
          uint32_t hi, lo;
          SplitPack(x, y, hi, lo);
          qh[nt][kk][h] = hi;
          if (QLO) ql[nt][kk][h] = lo;
        }
      }
    }
  }
  if (TMA) {
    if (threadIdx.x == 0) abort_word = 0;
    if ((threadIdx.x & 31) == 0) {
      for (int st = 0; st < NS; ++st) tc::MbarInit(SmemAddr(&tile_bars[(threadIdx.x >> 5) * NS + st]), 1);
      asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
  }
  __syncthreads();  // tab is staged

  const __nv_bfloat16* kc = static_cast<const __nv_bfloat16*>(p.kc);
  const __nv_bfloat16* vc = static_cast<const __nv_bfloat16*>(p.vc);
  unsigned char* my_stages = stages + warp * L::kWarpBytes;
  const uint32_t my_stages_addr = SmemAddr(my_stages);
  const int my_n = warp < ngroups ? (ngroups - warp + kMmaWarps - 1) / kMmaWarps : 0;
  const size_t row_elems = static_cast<size_t>(p.Hkv) * D;  // elements between consecutive positions of a block
  const bool one_block_per_group = p.bs_shift >= 4;          // block size a power of two >= 16: a group never straddles blocks

  // One group of 16 positions: each lane copies 16-byte chunks of the K and V rows; a row's chunk c lands at
  // chunk c ^ (row & 7) so that the ldmatrix reads below are conflict-free.  Rows at or past c1 are zero-filled.
  const uint32_t my_bars = SmemAddr(&tile_bars[warp * NS]);
  auto issue = [&](int it) {
    const int t_base = t_begin + ((warp + kMmaWarps * it) << 4);
    const uint32_t dst_base = my_stages_addr + (it % NS) * L::kStageBytes;
    if (TMA) {
      if (lane == 0) {
        const int blk = tab[(t_base >> p.bs_shift) - b0];
        const int pos = (blk << p.bs_shift) + (t_base & (p.bs - 1));  // the group's first position in the pool
        const uint32_t bar = my_bars + 8 * (it % NS);
        PaMbarExpectTx(bar, L::kStageBytes);
#pragma unroll
        for (int h = 0; h < D / 64; ++h) {
          TmaLoad3d(dst_base + h * 2048, map_k, 64 * h, kv, pos, bar);
          TmaLoad3d(dst_base + L::kTileBytes + h * 2048, map_v, 64 * h, kv, pos, bar);
        }
      }
      return;
    }
    size_t group_off = 0;
    if (one_block_per_group) {
      const int blk = tab[(t_base >> p.bs_shift) - b0];
      group_off = ((static_cast<size_t>(blk) << p.bs_shift) + (t_base & (p.bs - 1))) * row_elems + static_cast<size_t>(kv) * D;
    }
#pragma unroll
    for (int i = 0; i < 16 * CPR / 32; ++i) {
      const int c = lane + 32 * i;
      const int r = c / CPR, col = c % CPR;
      const int t = t_base + r;
      const bool valid = t < c1;
      size_t off = 0;
      if (valid) {
        if (one_block_per_group) {
          off = group_off + r * row_elems + col * 8;
        } else {
          const int blk_i = p.bs_shift >= 0 ? (t >> p.bs_shift) : t / p.bs;
          const int slot = t - blk_i * p.bs;
          off = ((static_cast<size_t>(tab[blk_i - b0]) * p.bs + slot) * p.Hkv + kv) * D + col * 8;
        }
      }
      const uint32_t dst = dst_base + r * L::kRowBytes + ((col ^ (r & 7)) << 4);
      CpAsync16(dst, kc + off, valid ? 16 : 0);
      CpAsync16(dst + L::kTileBytes, vc + off, valid ? 16 : 0);
    }
  };

  for (int it = 0; it < NS - 1; ++it) {
    if (it < my_n) issue(it);
    if (!TMA) CpAsyncCommit();
  }

  float o[NT][KS][4];
  float m_run[NT][2], l_run[NT][2];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    m_run[nt][0] = m_run[nt][1] = -INFINITY;
    l_run[nt][0] = l_run[nt][1] = 0.f;
#pragma unroll
    for (int mt = 0; mt < KS; ++mt) o[nt][mt][0] = o[nt][mt][1] = o[nt][mt][2] = o[nt][mt][3] = 0.f;
  }
  const float sl2 = p.scale * kLog2e;
  const int row_k = (lane & 7) + ((lane >> 3) & 1) * 8;  // K as A: matrices 1, 3 are positions 8..15; 2, 3 the next 8 dims
  const int row_v = (lane & 7) + (lane >> 4) * 8;        // V^T as A: matrices 2, 3 are positions 8..15; 1, 3 the next 8 dims

  for (int it = 0; it < my_n; ++it) {
    const int t_base = t_begin + ((warp + kMmaWarps * it) << 4);
    const uint32_t k_addr = my_stages_addr + (it % NS) * L::kStageBytes;
    const uint32_t v_addr = k_addr + L::kTileBytes;
    if (TMA) {
      if (it + NS - 1 < my_n) issue(it + NS - 1);
      if (!tc::MbarWait(my_bars + 8 * (it % NS), (it / NS) & 1, &abort_word)) {
        g_pa_status = 1;
        break;
      }
      if (t_base + 16 > c1) {
        // The box brought whole rows of the block; positions at or past the live end weigh nothing, but their V rows
        // may hold anything (0 x NaN): zero them.  A row is 128 bytes of each sub-tile whatever the swizzle.
        const int r0 = c1 - t_base;
        for (int idx = lane; idx < (16 - r0) * (D / 64) * 8; idx += 32) {
          const int r = r0 + idx / ((D / 64) * 8), rem = idx % ((D / 64) * 8);
          *reinterpret_cast<uint4*>(my_stages + (it % NS) * L::kStageBytes + L::kTileBytes + (rem >> 3) * 2048 + r * 128 + (rem & 7) * 16) =
              make_uint4(0u, 0u, 0u, 0u);
        }
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");  // before a later box lands in the same space
        __syncwarp();
      }
    } else {
      if (it + NS - 1 < my_n) issue(it + NS - 1);
      CpAsyncCommit();
      CpAsyncWait<NS - 1>();
      __syncwarp();
    }

    // Four accumulation chains per score tile, added at the end: a quarter of the dependent MMAs in a row.
    float sch[4][NT][4];
#pragma unroll
    for (int c = 0; c < 4; ++c)
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) sch[c][nt][0] = sch[c][nt][1] = sch[c][nt][2] = sch[c][nt][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < KS; ++kk) {
      uint32_t a[4];
      if (TMA) {
        const int ci = 2 * kk + (lane >> 4);
        LdMatrixX4(a, k_addr + (ci >> 3) * 2048 + row_k * 128 + (((ci & 7) ^ (row_k & 7)) << 4));
      } else {
        LdMatrixX4(a, k_addr + row_k * L::kRowBytes + (((2 * kk + (lane >> 4)) ^ (row_k & 7)) << 4));
      }
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        if (QLO) {
          MmaBf16(sch[2 * (kk & 1)][nt], a, qh[nt][kk][0], qh[nt][kk][1]);
          MmaBf16(sch[2 * (kk & 1) + 1][nt], a, ql[nt][kk][0], ql[nt][kk][1]);
        } else {
          MmaBf16(sch[kk & 3][nt], a, qh[nt][kk][0], qh[nt][kk][1]);
        }
      }
    }
    float sacc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
      for (int x = 0; x < 4; ++x) sacc[nt][x] = (sch[0][nt][x] + sch[1][nt][x]) + (sch[2][nt][x] + sch[3][nt][x]);
    }
    // sacc[nt]: [0], [1] = position t_base + gid against queries 2tig, 2tig + 1; [2], [3] = position t_base + gid + 8.
    uint32_t pb_hi[NT][2], pb_lo[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        const int e = x & 1;
        const int tok = t_base + gid + (x >> 1) * 8;
        const bool live = tok < qlen[nt][e] && tok >= qfirst[nt][e];
        const float v = live ? sacc[nt][x] * sl2 : -INFINITY;
        sacc[nt][x] = v;
        tmax[e] = fmaxf(tmax[e], v);
      }
      float alpha[2];
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        float t = tmax[e];
        t = fmaxf(t, __shfl_xor_sync(0xffffffffu, t, 4));
        t = fmaxf(t, __shfl_xor_sync(0xffffffffu, t, 8));
        t = fmaxf(t, __shfl_xor_sync(0xffffffffu, t, 16));
        const float mn = fmaxf(m_run[nt][e], t);
        alpha[e] = mn == -INFINITY ? 1.f : Exp2(m_run[nt][e] - mn);
        const float base = mn == -INFINITY ? 0.f : mn;
        m_run[nt][e] = mn;
        const float p0 = Exp2(sacc[nt][e] - base), p1 = Exp2(sacc[nt][2 + e] - base);
        sacc[nt][e] = p0;
        sacc[nt][2 + e] = p1;
        l_run[nt][e] = l_run[nt][e] * alpha[e] + p0 + p1;
      }
#pragma unroll
      for (int mt = 0; mt < KS; ++mt) {
        o[nt][mt][0] *= alpha[0];
        o[nt][mt][1] *= alpha[1];
        o[nt][mt][2] *= alpha[0];
        o[nt][mt][3] *= alpha[1];
      }
      // P (positions x queries, accumulator layout) -> P^T as B fragments: transpose the two 8x8 blocks.
      uint32_t h0, l0, h1, l1;
      SplitPack(sacc[nt][0], sacc[nt][1], h0, l0);
      SplitPack(sacc[nt][2], sacc[nt][3], h1, l1);
      pb_hi[nt][0] = MovMatrixTrans(h0);
      pb_hi[nt][1] = MovMatrixTrans(h1);
      pb_lo[nt][0] = MovMatrixTrans(l0);
      pb_lo[nt][1] = MovMatrixTrans(l1);
    }
#pragma unroll
    for (int mt = 0; mt < KS; ++mt) {
      uint32_t a[4];
      if (TMA) {
        const int ci = 2 * mt + ((lane >> 3) & 1);
        LdMatrixX4Trans(a, v_addr + (ci >> 3) * 2048 + row_v * 128 + (((ci & 7) ^ (row_v & 7)) << 4));
      } else {
        LdMatrixX4Trans(a, v_addr + row_v * L::kRowBytes + (((2 * mt + ((lane >> 3) & 1)) ^ (row_v & 7)) << 4));
      }
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        MmaBf16(o[nt][mt], a, pb_hi[nt][0], pb_hi[nt][1]);
        MmaBf16(o[nt][mt], a, pb_lo[nt][0], pb_lo[nt][1]);
      }
    }
    __syncwarp();  // the stage is free for the copy the next iteration issues
  }
  if (!TMA) CpAsyncWait<0>();
  __syncwarp();

  // Each warp leaves {m, l, o} of its positions in its own stage space; the CTA then merges the four.
  {
    float* wm = reinterpret_cast<float*>(my_stages);
    float* wl = wm + kMmaQ;
    float* wo = wl + kMmaQ;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        float l = l_run[nt][e];
        l += __shfl_xor_sync(0xffffffffu, l, 4);
        l += __shfl_xor_sync(0xffffffffu, l, 8);
        l += __shfl_xor_sync(0xffffffffu, l, 16);
        const int i = nt * 8 + 2 * tig + e;
        if (gid == 0) {
          wm[i] = m_run[nt][e];
          wl[i] = l;
        }
#pragma unroll
        for (int mt = 0; mt < KS; ++mt) {
          wo[i * D + 16 * mt + gid] = o[nt][mt][e];
          wo[i * D + 16 * mt + gid + 8] = o[nt][mt][2 + e];
        }
      }
    }
  }
  __syncthreads();
  for (int idx = tid; idx < p.NQ * D; idx += kMmaThreads) {
    const int i = idx / D, d = idx - i * D;
    float mx = -INFINITY;
#pragma unroll
    for (int w = 0; w < kMmaWarps; ++w) mx = fmaxf(mx, reinterpret_cast<const float*>(stages + w * L::kWarpBytes)[i]);
    float acc = 0.f, l = 0.f;
    if (mx != -INFINITY) {
#pragma unroll
      for (int w = 0; w < kMmaWarps; ++w) {
        const float* wm = reinterpret_cast<const float*>(stages + w * L::kWarpBytes);
        const float f = Exp2(wm[i] - mx);
        acc += f * wm[2 * kMmaQ + i * D + d];
        l += f * wm[kMmaQ + i];
      }
    }
    float* rec = Record(p, s, tb * p.rpt + i / p.group, kv * p.group + i % p.group);
    rec[2 + d] = acc;
    if (d == 0) {
      rec[0] = mx * kLn2;
      rec[1] = l;
    }
  }
}

template <typename QT, int D, int NS, int NT>
__global__ void __launch_bounds__(kMmaThreads) PaSliceMma(PaParams p)
{
  PaSliceMmaBody<QT, D, NS, NT, false>(p, nullptr, nullptr);
}

template <typename QT, int D, int NT>
__global__ void __launch_bounds__(kMmaThreads)
    PaSliceTma(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, PaParams p)
{
  PaSliceMmaBody<QT, D, 2, NT, true>(p, &map_k, &map_v);
}

// ------------------------------------------------------------------------------------------
// The tensor-core slice kernel for f8e4m3fn pools: the same decomposition as PaSliceMma with half the bytes per
// position.  An e4m3fn value is exact in f16 (4 significant bits, exponents 2^-9 .. 2^8), so the MMAs run on f16
// operands: the raw bytes are copied to shared memory as they lie (a position's head row is D bytes), ldmatrix
// moves them as if they were 16-bit elements (one "element" = two neighbouring channels) and cvt.f16x2.e4m3x2
// widens each pair in registers.  That fixes which channels a lane holds, which differs from the 16-bit layout:
//   K as A (positions x channels): a lane's register of chunk c holds channels 16c + 4tig .. + 3 of position gid,
//     so MMA k-slots 2tig, 2tig+1 / 2tig+8, 2tig+9 stand for channels 16c + 4tig, +1 / +2, +3, and the query's B
//     fragments are loaded with the same assignment (a dot product does not care in which order it is summed);
//   V^T as A (channels x positions, ldmatrix.trans): a lane's register holds channels 2gid, 2gid+1 of positions
//     2tig, 2tig+1; a byte permute pairs the two positions of each channel, so accumulator rows gid / gid+8 of
//     m-tile c stand for channels 16c + 2gid / 16c + 2gid + 1 (undone when the record is written).
// The query and the probabilities are carried as hi + lo f16 parts (22 bits); a query beyond f16's range (|q| > 65504)
// is clamped to it.

__device__ __forceinline__ void MmaF16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
{
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// The four e4m3fn bytes of a word as two f16 pairs (bytes 0, 1 and bytes 2, 3), exactly; the halves of the word are
// named as 16-bit registers, with no shift or mask of their own.
__device__ __forceinline__ void E4m3x4ToF16x2x2(uint32_t word, uint32_t& low_pair, uint32_t& high_pair)
{
  asm("{\n\t.reg .b16 lo, hi;\n\t"
      "mov.b32 {lo, hi}, %2;\n\t"
      "cvt.rn.f16x2.e4m3x2 %0, lo;\n\t"
      "cvt.rn.f16x2.e4m3x2 %1, hi;\n\t}\n"
      : "=r"(low_pair), "=r"(high_pair)
      : "r"(word));
}
// Two floats as f16 hi parts (lower index in the low half) and the f16 of what is left.
__device__ __forceinline__ void SplitPackF16(float x, float y, uint32_t& hi, uint32_t& lo)
{
  x = fminf(fmaxf(x, -65504.f), 65504.f);
  y = fminf(fmaxf(y, -65504.f), 65504.f);
  const __half xh = __float2half_rn(x), yh = __float2half_rn(y);
  const __half xl = __float2half_rn(x - __half2float(xh)), yl = __float2half_rn(y - __half2float(yh));
  hi = static_cast<uint32_t>(__half_as_ushort(xh)) | (static_cast<uint32_t>(__half_as_ushort(yh)) << 16);
  lo = static_cast<uint32_t>(__half_as_ushort(xl)) | (static_cast<uint32_t>(__half_as_ushort(yl)) << 16);
}

template <int D, int NS>
struct MmaLayoutF8 {
  static constexpr int kRowBytes = D;
  static constexpr int kTileBytes = 16 * kRowBytes;
  static constexpr int kStageBytes = 2 * kTileBytes;
  static constexpr int kWarpBytes = NS * kStageBytes;
  static constexpr int kTabOffset = kMmaWarps * kWarpBytes;
  static size_t Bytes(int tab_entries) { return kTabOffset + sizeof(int) * static_cast<size_t>(tab_entries); }
};

// TMA: as in PaSliceMmaBody, the tiles arrive as boxes (16 positions x D bytes of one head) of a byte tensor map over
// the pool; the map's swizzle (128-byte rows: SWIZZLE_128B, 64-byte rows: SWIZZLE_64B) is the layout the cp.async form
// builds by hand, so the reads below are the same for both.
template <typename QT, int D, int NS, int NT, bool TMA>
__device__ __forceinline__ void PaSliceMmaF8Body(const PaParams& p, const CUtensorMap* map_k, const CUtensorMap* map_v)
{
  GridDependencySync();
  constexpr bool QLO = sizeof(QT) == 4;  // a bf16 query is exact in f16 (within its range): no low part to carry
  using L = MmaLayoutF8<D, NS>;
  static_assert(L::kWarpBytes >= static_cast<int>(sizeof(float)) * (2 * kMmaQ + 8 * NT * D), "a warp's stages hold its partial record");
  constexpr int CPR = L::kRowBytes / 16;  // 16-byte chunks per row: 8 (D = 128) or 4 (D = 64)
  constexpr int KS = D / 16;              // k-steps of K Q^T, m-tiles of V^T P^T: one per chunk
  extern __shared__ __align__(1024) unsigned char smem[];
  unsigned char* stages = smem;
  int* tab = reinterpret_cast<int*>(smem + L::kTabOffset);
  __shared__ __align__(8) unsigned long long tile_bars[kMmaWarps * NS];
  __shared__ uint32_t abort_word;

  const int s = blockIdx.x, kv = blockIdx.y, tb = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int gid = lane >> 2, tig = lane & 3;
  const int ctx = p.M * p.bs;
  const int c0 = s * p.slice;

  const int c_end = min(c0 + p.slice, ctx);
  const int b0 = p.bs_shift >= 0 ? (c0 >> p.bs_shift) : c0 / p.bs;
  const int b_last = c_end > c0 ? (p.bs_shift >= 0 ? ((c_end - 1) >> p.bs_shift) : (c_end - 1) / p.bs) : b0 - 1;
  for (int j = tid; j <= b_last - b0; j += kMmaThreads) {
    tab[j] = ClampI(__ldg(p.tables + static_cast<size_t>(tb) * p.M + b0 + j), 0, p.P - 1);
  }
  int maxlen = 0, minfirst = ctx;
  for (int r = 0; r < p.rpt; ++r) {
    const int len = ClampI(__ldg(p.lens + tb * p.rpt + r), 0, ctx);
    maxlen = max(maxlen, len);
    minfirst = min(minfirst, p.window > 0 ? max(0, len - p.window) : 0);
  }
  const int c1 = min(min(c0 + p.slice, ctx), maxlen);
  const int t_begin = max(c0, minfirst) & ~15;
  if (t_begin >= c1) return;
  const int ngroups = (c1 - t_begin + 15) >> 4;

  int qlen[NT][2], qfirst[NT][2];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int i = nt * 8 + 2 * tig + e;
      int len = 0, first = 0;
      if (i < p.NQ) {
        const int full = ClampI(__ldg(p.lens + tb * p.rpt + i / p.group), 0, ctx);
        first = p.window > 0 ? max(0, full - p.window) : 0;
        len = min(full, c1);
      }
      qlen[nt][e] = len;
      qfirst[nt][e] = first;
    }
  }
  // Q^T as B fragments under the byte layout's channel assignment: for k-step kk, b0b1 = Q[query gid][16kk + 4tig, +1],
  // b2b3 = Q[query gid][16kk + 4tig + 2, +3]; hi and lo f16 parts.
  uint32_t qh[NT][KS][2], ql[QLO ? NT : 1][QLO ? KS : 1][2];
  {
    const QT* q = static_cast<const QT*>(p.q);
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const int i = nt * 8 + gid;
      const bool have = i < p.NQ;
      const QT* src = q + (static_cast<size_t>(tb * p.rpt + (have ? i / p.group : 0)) * p.H + kv * p.group + (have ? i % p.group : 0)) * D;
#pragma unroll
      for (int kk = 0; kk < KS; ++kk) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int d = 16 * kk + 4 * tig + 2 * h;
          const float x = have ? ToF32(src[d]) : 0.f, y = have ? ToF32(src[d + 1]) : 0.f;
          uint32_t hi, lo;
          SplitPackF16(x, y, hi, lo);
          qh[nt][kk][h] = hi;
          if (QLO) ql[nt][kk][h] = lo;
        }
      }
    }
  }
  if (TMA) {
    if (threadIdx.x == 0) abort_word = 0;
    if ((threadIdx.x & 31) == 0) {
      for (int st = 0; st < NS; ++st) tc::MbarInit(SmemAddr(&tile_bars[(threadIdx.x >> 5) * NS + st]), 1);
      asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
  }
  __syncthreads();  // tab is staged

  const unsigned char* kc = static_cast<const unsigned char*>(p.kc);
  const unsigned char* vc = static_cast<const unsigned char*>(p.vc);
  unsigned char* my_stages = stages + warp * L::kWarpBytes;
  const uint32_t my_stages_addr = SmemAddr(my_stages);
  const int my_n = warp < ngroups ? (ngroups - warp + kMmaWarps - 1) / kMmaWarps : 0;
  const size_t row_elems = static_cast<size_t>(p.Hkv) * D;  // bytes between consecutive positions of a block
  const bool one_block_per_group = p.bs_shift >= 4;

  // A row's 16-byte chunk c lands at chunk c ^ swz(row): with 128-byte rows swz = row & 7, with 64-byte rows (two rows
  // per 128 bytes) swz = (row >> 1) & 3; either way the eight rows an ldmatrix touches fall in eight different 16-byte
  // bank groups.
  auto swz = [](int r) { return CPR == 8 ? (r & 7) : ((r >> 1) & 3); };
  const uint32_t my_bars = SmemAddr(&tile_bars[warp * NS]);
  auto issue = [&](int it) {
    const int t_base = t_begin + ((warp + kMmaWarps * it) << 4);
    const uint32_t dst_base = my_stages_addr + (it % NS) * L::kStageBytes;
    if (TMA) {
      if (lane == 0) {
        const int blk = tab[(t_base >> p.bs_shift) - b0];
        const int pos = (blk << p.bs_shift) + (t_base & (p.bs - 1));  // the group's first position in the pool
        const uint32_t bar = my_bars + 8 * (it % NS);
        PaMbarExpectTx(bar, L::kStageBytes);
        TmaLoad3d(dst_base, map_k, 0, kv, pos, bar);
        TmaLoad3d(dst_base + L::kTileBytes, map_v, 0, kv, pos, bar);
      }
      return;
    }
    size_t group_off = 0;
    if (one_block_per_group) {
      const int blk = tab[(t_base >> p.bs_shift) - b0];
      group_off = ((static_cast<size_t>(blk) << p.bs_shift) + (t_base & (p.bs - 1))) * row_elems + static_cast<size_t>(kv) * D;
    }
#pragma unroll
    for (int i = 0; i < 16 * CPR / 32; ++i) {
      const int c = lane + 32 * i;
      const int r = c / CPR, col = c % CPR;
      const int t = t_base + r;
      const bool valid = t < c1;
      size_t off = 0;
      if (valid) {
        if (one_block_per_group) {
          off = group_off + r * row_elems + col * 16;
        } else {
          const int blk_i = p.bs_shift >= 0 ? (t >> p.bs_shift) : t / p.bs;
          const int slot = t - blk_i * p.bs;
          off = ((static_cast<size_t>(tab[blk_i - b0]) * p.bs + slot) * p.Hkv + kv) * D + col * 16;
        }
      }
      const uint32_t dst = dst_base + r * L::kRowBytes + ((col ^ swz(r)) << 4);
      CpAsync16(dst, kc + off, valid ? 16 : 0);
      CpAsync16(dst + L::kTileBytes, vc + off, valid ? 16 : 0);
    }
  };

  for (int it = 0; it < NS - 1; ++it) {
    if (it < my_n) issue(it);
    if (!TMA) CpAsyncCommit();
  }

  float o[NT][KS][4];
  float m_run[NT][2], l_run[NT][2];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    m_run[nt][0] = m_run[nt][1] = -INFINITY;
    l_run[nt][0] = l_run[nt][1] = 0.f;
#pragma unroll
    for (int mt = 0; mt < KS; ++mt) o[nt][mt][0] = o[nt][mt][1] = o[nt][mt][2] = o[nt][mt][3] = 0.f;
  }
  const float sl2 = p.scale * kLog2e;
  // ldmatrix addressing, the same for K and V: matrices 0, 1 = positions 0-7, 8-15 of chunk 2j; 2, 3 = of chunk 2j + 1.
  const int row_a = (lane & 7) + ((lane >> 3) & 1) * 8;
  const uint32_t row_off = row_a * L::kRowBytes;
  const int row_swz = swz(row_a), hi_chunk = lane >> 4;

  for (int it = 0; it < my_n; ++it) {
    const int t_base = t_begin + ((warp + kMmaWarps * it) << 4);
    const uint32_t k_addr = my_stages_addr + (it % NS) * L::kStageBytes;
    const uint32_t v_addr = k_addr + L::kTileBytes;
    if (it + NS - 1 < my_n) issue(it + NS - 1);
    if (TMA) {
      if (!tc::MbarWait(my_bars + 8 * (it % NS), (it / NS) & 1, &abort_word)) {
        g_pa_status = 1;
        break;
      }
      if (t_base + 16 > c1) {
        // positions at or past the live end weigh nothing, but their V rows may hold anything (0 x NaN): zero them
        const int r0 = c1 - t_base;
        for (int idx = lane; idx < (16 - r0) * CPR; idx += 32) {
          *reinterpret_cast<uint4*>(my_stages + (it % NS) * L::kStageBytes + L::kTileBytes + (r0 + idx / CPR) * L::kRowBytes + (idx % CPR) * 16) =
              make_uint4(0u, 0u, 0u, 0u);
        }
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");  // before a later box lands in the same space
        __syncwarp();
      }
    } else {
      CpAsyncCommit();
      CpAsyncWait<NS - 1>();
      __syncwarp();
    }

    // Four accumulation chains per score tile, added at the end: a quarter of the dependent MMAs in a row.
    float sch[4][NT][4];
#pragma unroll
    for (int c = 0; c < 4; ++c)
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) sch[c][nt][0] = sch[c][nt][1] = sch[c][nt][2] = sch[c][nt][3] = 0.f;
#pragma unroll
    for (int j = 0; j < KS / 2; ++j) {
      uint32_t r[4];
      LdMatrixX4(r, k_addr + row_off + (((2 * j + hi_chunk) ^ row_swz) << 4));
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int kk = 2 * j + half;
        const uint32_t lo_rows = r[2 * half], hi_rows = r[2 * half + 1];
        uint32_t a[4];
        E4m3x4ToF16x2x2(lo_rows, a[0], a[2]);
        E4m3x4ToF16x2x2(hi_rows, a[1], a[3]);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          if (QLO) {
            MmaF16(sch[2 * half][nt], a, qh[nt][kk][0], qh[nt][kk][1]);
            MmaF16(sch[2 * half + 1][nt], a, ql[nt][kk][0], ql[nt][kk][1]);
          } else {
            MmaF16(sch[kk & 3][nt], a, qh[nt][kk][0], qh[nt][kk][1]);
          }
        }
      }
    }
    float sacc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
      for (int x = 0; x < 4; ++x) sacc[nt][x] = (sch[0][nt][x] + sch[1][nt][x]) + (sch[2][nt][x] + sch[3][nt][x]);
    }
    uint32_t pb_hi[NT][2], pb_lo[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        const int e = x & 1;
        const int tok = t_base + gid + (x >> 1) * 8;
        const bool live = tok < qlen[nt][e] && tok >= qfirst[nt][e];
        const float v = live ? sacc[nt][x] * sl2 : -INFINITY;
        sacc[nt][x] = v;
        tmax[e] = fmaxf(tmax[e], v);
      }
      float alpha[2];
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        float t = tmax[e];
        t = fmaxf(t, __shfl_xor_sync(0xffffffffu, t, 4));
        t = fmaxf(t, __shfl_xor_sync(0xffffffffu, t, 8));
        t = fmaxf(t, __shfl_xor_sync(0xffffffffu, t, 16));
        const float mn = fmaxf(m_run[nt][e], t);
        alpha[e] = mn == -INFINITY ? 1.f : Exp2(m_run[nt][e] - mn);
        const float base = mn == -INFINITY ? 0.f : mn;
        m_run[nt][e] = mn;
        const float p0 = Exp2(sacc[nt][e] - base), p1 = Exp2(sacc[nt][2 + e] - base);
        sacc[nt][e] = p0;
        sacc[nt][2 + e] = p1;
        l_run[nt][e] = l_run[nt][e] * alpha[e] + p0 + p1;
      }
#pragma unroll
      for (int mt = 0; mt < KS; ++mt) {
        o[nt][mt][0] *= alpha[0];
        o[nt][mt][1] *= alpha[1];
        o[nt][mt][2] *= alpha[0];
        o[nt][mt][3] *= alpha[1];
      }
      uint32_t h0, l0, h1, l1;
      SplitPackF16(sacc[nt][0], sacc[nt][1], h0, l0);
      SplitPackF16(sacc[nt][2], sacc[nt][3], h1, l1);
      pb_hi[nt][0] = MovMatrixTrans(h0);
      pb_hi[nt][1] = MovMatrixTrans(h1);
      pb_lo[nt][0] = MovMatrixTrans(l0);
      pb_lo[nt][1] = MovMatrixTrans(l1);
    }
#pragma unroll
    for (int j = 0; j < KS / 2; ++j) {
      uint32_t r[4];
      LdMatrixX4Trans(r, v_addr + row_off + (((2 * j + hi_chunk) ^ row_swz) << 4));
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int mt = 2 * j + half;
        // bytes {p0 c0, p0 c1, p1 c0, p1 c1} -> {p0 c0, p1 c0 | p0 c1, p1 c1}: the two positions of each channel side by side
        const uint32_t lo_pos = __byte_perm(r[2 * half], 0u, 0x3120), hi_pos = __byte_perm(r[2 * half + 1], 0u, 0x3120);
        uint32_t a[4];
        E4m3x4ToF16x2x2(lo_pos, a[0], a[1]);
        E4m3x4ToF16x2x2(hi_pos, a[2], a[3]);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          MmaF16(o[nt][mt], a, pb_hi[nt][0], pb_hi[nt][1]);
          MmaF16(o[nt][mt], a, pb_lo[nt][0], pb_lo[nt][1]);
        }
      }
    }
    __syncwarp();
  }
  if (!TMA) CpAsyncWait<0>();
  __syncwarp();

  {
    float* wm = reinterpret_cast<float*>(my_stages);
    float* wl = wm + kMmaQ;
    float* wo = wl + kMmaQ;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        float l = l_run[nt][e];
        l += __shfl_xor_sync(0xffffffffu, l, 4);
        l += __shfl_xor_sync(0xffffffffu, l, 8);
        l += __shfl_xor_sync(0xffffffffu, l, 16);
        const int i = nt * 8 + 2 * tig + e;
        if (gid == 0) {
          wm[i] = m_run[nt][e];
          wl[i] = l;
        }
#pragma unroll
        for (int mt = 0; mt < KS; ++mt) {
          wo[i * D + 16 * mt + 2 * gid] = o[nt][mt][e];          // accumulator row gid: channel 16 mt + 2 gid
          wo[i * D + 16 * mt + 2 * gid + 1] = o[nt][mt][2 + e];  // accumulator row gid + 8: channel 16 mt + 2 gid + 1
        }
      }
    }
  }
  __syncthreads();
  for (int idx = tid; idx < p.NQ * D; idx += kMmaThreads) {
    const int i = idx / D, d = idx - i * D;
    float mx = -INFINITY;
#pragma unroll
    for (int w = 0; w < kMmaWarps; ++w) mx = fmaxf(mx, reinterpret_cast<const float*>(stages + w * L::kWarpBytes)[i]);
    float acc = 0.f, l = 0.f;
    if (mx != -INFINITY) {
#pragma unroll
      for (int w = 0; w < kMmaWarps; ++w) {
        const float* wm = reinterpret_cast<const float*>(stages + w * L::kWarpBytes);
        const float f = Exp2(wm[i] - mx);
        acc += f * wm[2 * kMmaQ + i * D + d];
        l += f * wm[kMmaQ + i];
      }
    }
    float* rec = Record(p, s, tb * p.rpt + i / p.group, kv * p.group + i % p.group);
    rec[2 + d] = acc;
    if (d == 0) {
      rec[0] = mx * kLn2;
      rec[1] = l;
    }
  }
}

template <typename QT, int D, int NS, int NT>
__global__ void __launch_bounds__(kMmaThreads) PaSliceMmaF8(PaParams p)
{
  PaSliceMmaF8Body<QT, D, NS, NT, false>(p, nullptr, nullptr);
}

template <typename QT, int D, int NS, int NT>
__global__ void __launch_bounds__(kMmaThreads)
    PaSliceTmaF8(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, PaParams p)
{
  PaSliceMmaF8Body<QT, D, NS, NT, true>(p, &map_k, &map_v);
}

// ------------------------------------------------------------------------------------------
// Combine: grid R*H.  Row r's live slices are [first / slice, ceil(len / slice)); their records merge as
// out = sum_s exp(m_s - max) acc_s / sum_s exp(m_s - max) l_s, in slice order (deterministic).

constexpr int kCombineThreads = 128;  // four warps, one (row, head) each
constexpr int kCombineBatch = 8;      // slices whose records are in flight together

__device__ __forceinline__ void StorePair(float* o, float a, float b) { *reinterpret_cast<float2*>(o) = make_float2(a, b); }
__device__ __forceinline__ void StorePair(__nv_bfloat16* o, float a, float b)
{
  *reinterpret_cast<__nv_bfloat162*>(o) = __floats2bfloat162_rn(a, b);
}

// Merges the records {max, sum, acc[D]} of a row's live slices, in slice order.  One warp per (row, head): lane l
// holds the max and sum of slice s_lo + l (32 slices at a time), the weights travel by shuffle, and every lane owns
// the channel pairs 2l, 2l + 1 (+ 64, ...).  The loads of a trip do not depend on one another, so a merge costs about
// two trips to L2 rather than one per slice.  D is even (RoPE pairs) or the scalar tail handles the last channel.
template <typename OT, int PAIRS>  // PAIRS channel pairs per lane: D <= 64 * PAIRS
__global__ void __launch_bounds__(kCombineThreads) PaCombine(PaParams p)
{
  GridDependencySync();
  const int lane = threadIdx.x & 31;
  const int rh = blockIdx.x * (kCombineThreads / 32) + (threadIdx.x >> 5);
  if (rh >= p.R * p.H) return;
  const int row = rh / p.H, head = rh - row * p.H;
  const int ctx = p.M * p.bs;
  const int len = ClampI(__ldg(p.lens + row), 0, ctx);
  const int first = p.window > 0 ? max(0, len - p.window) : 0;
  const int s_lo = first / p.slice, s_hi = min(p.S, (len + p.slice - 1) / p.slice);
  const size_t stride = static_cast<size_t>(p.R) * p.H * (p.D + 2);
  const float* base = Record(p, 0, row, head);
  const int pairs = p.D >> 1;
  const bool even = (p.D & 1) == 0 && (reinterpret_cast<uintptr_t>(p.scratch) & 7) == 0 && (reinterpret_cast<uintptr_t>(p.out) & 7) == 0;
  // Eight slices at a time: their records are requested together (a live slice's record is always written, so the
  // loads need not wait for the weights), then folded in slice order.
  auto load_batch = [&](int s0, int count, float2(&v)[kCombineBatch][PAIRS]) {
#pragma unroll
    for (int u = 0; u < kCombineBatch; ++u) {
      const float* rec = base + (s0 + u) * stride + 2;
#pragma unroll
      for (int j = 0; j < PAIRS; ++j) {
        const int pr = lane + 32 * j;
        v[u][j] = make_float2(0.f, 0.f);
        if (u < count && pr < pairs) {
          if (even) v[u][j] = *reinterpret_cast<const float2*>(rec + 2 * pr);  // records start on 8-byte boundaries only for even D
          else v[u][j] = make_float2(rec[2 * pr], rec[2 * pr + 1]);
        }
      }
    }
  };
  // One trip to memory brings this lane's slice header {max, sum} of the first 32 slices AND the first eight records.
  float hm = -INFINITY, hs = 0.f;
  if (s_lo + lane < s_hi) {
    hm = base[(s_lo + lane) * stride];
    hs = base[(s_lo + lane) * stride + 1];
  }
  float2 v[kCombineBatch][PAIRS];
  load_batch(s_lo, min(kCombineBatch, s_hi - s_lo), v);
  float mx = hm;
  for (int s = s_lo + 32 + lane; s < s_hi; s += 32) mx = fmaxf(mx, base[s * stride]);  // more than 32 slices: rare
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float denom = 0.f;
  float acc[2 * PAIRS];
#pragma unroll
  for (int i = 0; i < 2 * PAIRS; ++i) acc[i] = 0.f;
  for (int c0 = s_lo; c0 < s_hi; c0 += 32) {
    const int mine = c0 + lane;
    float w_l = 0.f, ws_l = 0.f;
    if (mine < s_hi) {
      const float m = c0 == s_lo ? hm : base[mine * stride];
      w_l = m == -INFINITY ? 0.f : expf(m - mx);
      ws_l = w_l != 0.f ? w_l * (c0 == s_lo ? hs : base[mine * stride + 1]) : 0.f;
    }
    const int n = min(32, s_hi - c0);
    for (int i0 = 0; i0 < n; i0 += kCombineBatch) {
      if (c0 != s_lo || i0 != 0) load_batch(c0 + i0, min(kCombineBatch, n - i0), v);
#pragma unroll
      for (int u = 0; u < kCombineBatch; ++u) {
        const int i = i0 + u;
        const float w = __shfl_sync(0xffffffffu, w_l, i & 31), ws = __shfl_sync(0xffffffffu, ws_l, i & 31);
        if (i < n && w != 0.f) {  // uniform over the warp
          denom += ws;
#pragma unroll
          for (int j = 0; j < PAIRS; ++j) {
            acc[2 * j] += w * v[u][j].x;
            acc[2 * j + 1] += w * v[u][j].y;
          }
        }
      }
    }
  }
  OT* out = static_cast<OT*>(p.out) + static_cast<size_t>(rh) * p.D;
  const bool empty = mx == -INFINITY || denom == 0.f;
#pragma unroll
  for (int j = 0; j < PAIRS; ++j) {
    const int pr = lane + 32 * j;
    if (pr < pairs) {
      const float a = empty ? 0.f : acc[2 * j] / denom, b = empty ? 0.f : acc[2 * j + 1] / denom;
      if (even) {
        StorePair(out + 2 * pr, a, b);
      } else {
        out[2 * pr] = FromF32<OT>(a);
        out[2 * pr + 1] = FromF32<OT>(b);
      }
    }
  }
  if ((p.D & 1) != 0 && lane == 0) {  // an odd head dimension: the last channel, not part of any pair
    float a = 0.f;
    if (!empty) {
      for (int s = s_lo; s < s_hi; ++s) {
        const float m = base[s * stride];
        const float w = m == -INFINITY ? 0.f : expf(m - mx);
        if (w != 0.f) a += w * base[s * stride + 2 + p.D - 1];
      }
      a /= denom;
    }
    out[p.D - 1] = FromF32<OT>(a);
  }
  if (lane == 0 && p.lse != nullptr) p.lse[rh] = empty ? -INFINITY : mx + logf(denom);
}

// ------------------------------------------------------------------------------------------
// Parity mode: the interpreter's own walk (DxirInterpreter.kt:2049-2140).  One CTA per (row, head): every score is a
// double dot over the head dimension in ascending order times the scale; the denominator is summed in position order
// by one thread; channel j accumulates (e / denom) * v in double over the positions in ascending order, multiply and
// add rounded separately; one narrowing to f32 at the end.  The scores of the whole row sit in shared memory.

constexpr int kFaithfulThreads = 256;
constexpr int kFaithfulMaxCtx = 5632;  // doubles that fit the default 48 KB of dynamic shared memory, less the rest

template <typename QT, typename KVT, typename OT>
__global__ void __launch_bounds__(kFaithfulThreads) PaOrderFaithful(PaParams p)
{
  GridDependencySync();
  extern __shared__ __align__(16) unsigned char smem_raw[];
  double* scores = reinterpret_cast<double*>(smem_raw);
  __shared__ double red[kFaithfulThreads / 32];
  __shared__ double s_mx, s_denom;
  const int rh = blockIdx.x, row = rh / p.H, head = rh - row * p.H;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int D = p.D, ctx = p.M * p.bs, kv = head / p.group, tb = row / p.rpt;
  const int len = ClampI(__ldg(p.lens + row), 0, ctx);
  const int first = p.window > 0 ? max(0, len - p.window) : 0;
  const QT* q = static_cast<const QT*>(p.q) + static_cast<size_t>(rh) * D;
  const KVT* kc = static_cast<const KVT*>(p.kc);
  const KVT* vc = static_cast<const KVT*>(p.vc);
  OT* out = static_cast<OT*>(p.out) + static_cast<size_t>(rh) * D;
  const double scale = static_cast<double>(p.scale);
  auto offset = [&](int t) {
    const int blk = ClampI(__ldg(p.tables + static_cast<size_t>(tb) * p.M + t / p.bs), 0, p.P - 1);
    return ((static_cast<size_t>(blk) * p.bs + t % p.bs) * p.Hkv + kv) * D;
  };
  double mx = -INFINITY;
  for (int t = first + tid; t < len; t += kFaithfulThreads) {
    double sc = -INFINITY;
    if (Kept(p, row, t)) {
      const KVT* kr = kc + offset(t);
      double dot = 0.0;
      for (int j = 0; j < D; ++j) dot = __dadd_rn(dot, __dmul_rn(static_cast<double>(ToF32(q[j])), static_cast<double>(ToF32(kr[j]))));
      sc = __dmul_rn(dot, scale);
      mx = fmax(mx, sc);
    }
    scores[t - first] = sc;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmax(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if (lane == 0) red[warp] = mx;
  __syncthreads();
  if (tid == 0) {
    double m = red[0];
    for (int w = 1; w < kFaithfulThreads / 32; ++w) m = fmax(m, red[w]);
    s_mx = m;
  }
  __syncthreads();
  mx = s_mx;
  for (int t = first + tid; t < len; t += kFaithfulThreads) {
    const double sc = scores[t - first];
    scores[t - first] = sc == -INFINITY ? 0.0 : exp(sc - mx);  // a masked position weighs nothing
  }
  __syncthreads();
  if (tid == 0) {
    double denom = 0.0;
    for (int t = first; t < len; ++t)
      if (Kept(p, row, t)) denom = __dadd_rn(denom, scores[t - first]);
    s_denom = denom;
  }
  __syncthreads();
  const double denom = s_denom;
  const bool empty = len <= first || mx == -INFINITY || denom == 0.0;
  for (int j = tid; j < D; j += kFaithfulThreads) {
    double acc = 0.0;
    if (!empty) {
      for (int t = first; t < len; ++t) {
        if (!Kept(p, row, t)) continue;
        const double w = scores[t - first] / denom;
        acc = __dadd_rn(acc, __dmul_rn(w, static_cast<double>(ToF32(vc[offset(t) + j]))));
      }
    }
    out[j] = FromF32<OT>(static_cast<float>(acc));
  }
  if (tid == 0 && p.lse != nullptr) p.lse[rh] = empty ? -INFINITY : static_cast<float>(mx + log(denom));
}

template <typename QT, typename KVT>
cudaError_t LaunchFaithful(const PaParams& p, int out_dtype, int span, cudaStream_t st)
{
  const size_t smem = sizeof(double) * static_cast<size_t>(span > 0 ? span : 1);
  const unsigned grid = static_cast<unsigned>(p.R * p.H);
  if (out_dtype == TLALOC_B200_F32) return LaunchChained(PaOrderFaithful<QT, KVT, float>, grid, kFaithfulThreads, smem, st, p);
  return LaunchChained(PaOrderFaithful<QT, KVT, __nv_bfloat16>, grid, kFaithfulThreads, smem, st, p);
}

// ------------------------------------------------------------------------------------------
// KV_CACHE_WRITE: one CTA per token row.

template <typename PT, typename NT>
__global__ void KvCacheWriteKernel(PT* pool, const NT* new_kv, const int* slots, int row_elems, int num_slots)
{
  GridDependencySync();
  const int i = blockIdx.x;
  const int slot = __ldg(slots + i);
  if (slot < 0 || slot >= num_slots) return;
  PT* dst = pool + static_cast<size_t>(slot) * row_elems;
  const NT* src = new_kv + static_cast<size_t>(i) * row_elems;
  for (int j = threadIdx.x; j < row_elems; j += blockDim.x) dst[j] = FromF32<PT>(ToF32(src[j]));
}

// ------------------------------------------------------------------------------------------
// Host side.

// Stages per warp: 2 by default (three CTAs per SM; occupancy matters more than depth here) ($TLALOC_B200_PA_STAGES = 2, 3 or 4).
int MmaStages()
{
  static const int v = [] {
    const char* e = std::getenv("TLALOC_B200_PA_STAGES");
    const int x = e != nullptr ? std::atoi(e) : 0;
    return x >= 2 && x <= 4 ? x : 2;
  }();
  return v;
}

// Room for the table entries of the longest slice a launch may choose (8192 positions of 8-position blocks).
constexpr int kMaxTabEntries = 1024 + 2;

template <typename QT, int D, int NS>
cudaError_t PrepareMmaNs()
{
  cudaError_t e = cudaFuncSetAttribute(PaSliceMma<QT, D, NS, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(MmaLayout<D, NS>::Bytes(kMaxTabEntries)));
  if (e == cudaSuccess) {
    e = cudaFuncSetAttribute(PaSliceMma<QT, D, NS, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(MmaLayout<D, NS>::Bytes(kMaxTabEntries)));
  }
  return e;
}

template <typename QT, int D>
cudaError_t PrepareMma()
{
  cudaError_t e = PrepareMmaNs<QT, D, 2>();
  if (e == cudaSuccess) e = PrepareMmaNs<QT, D, 3>();
  if (e == cudaSuccess) e = PrepareMmaNs<QT, D, 4>();
  return e;
}

template <typename QT, int D, int NS>
cudaError_t LaunchMmaNs(const PaParams& p, cudaStream_t stream)
{
  const size_t smem = MmaLayout<D, NS>::Bytes(p.slice / p.bs + 2);
  const dim3 grid(p.S, p.Hkv, p.Tb);
  if (p.NQ <= 8) return LaunchChained(PaSliceMma<QT, D, NS, 1>, grid, kMmaThreads, smem, stream, p);
  return LaunchChained(PaSliceMma<QT, D, NS, 2>, grid, kMmaThreads, smem, stream, p);
}

// The TMA-fed form of the bf16 kernel ($TLALOC_B200_PA_TMA=0 keeps the cp.async form).
bool MmaTmaEnabled()
{
  static const bool v = [] {
    const char* e = std::getenv("TLALOC_B200_PA_TMA");
    return e == nullptr || e[0] != '0';
  }();
  return v;
}

template <typename QT, int D>
cudaError_t PrepareTma()
{
  cudaError_t e = cudaFuncSetAttribute(PaSliceTma<QT, D, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(MmaLayout<D, 2>::Bytes(kMaxTabEntries)));
  if (e == cudaSuccess) {
    e = cudaFuncSetAttribute(PaSliceTma<QT, D, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(MmaLayout<D, 2>::Bytes(kMaxTabEntries)));
  }
  return e;
}

// False when the launch does not qualify (the caller then takes the cp.async form).
template <typename QT, int D>
bool LaunchTma(const PaParams& p, cudaStream_t stream, cudaError_t* err)
{
  if (!MmaTmaEnabled() || MmaStages() != 2 || p.bs_shift < 4) return false;
  CUtensorMap map_k, map_v;
  const unsigned long long positions = static_cast<unsigned long long>(p.P) * p.bs;
  if (!EncodeKvPoolMap(&map_k, p.kc, D, p.Hkv, positions, 2) || !EncodeKvPoolMap(&map_v, p.vc, D, p.Hkv, positions, 2)) return false;
  const size_t smem = MmaLayout<D, 2>::Bytes(p.slice / p.bs + 2);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.S, p.Hkv, p.Tb);
  cfg.blockDim = dim3(kMmaThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[2];
  cfg.numAttrs = ChainAttributes(attrs);
  cfg.attrs = attrs;
  *err = p.NQ <= 8 ? cudaLaunchKernelEx(&cfg, PaSliceTma<QT, D, 1>, map_k, map_v, p) : cudaLaunchKernelEx(&cfg, PaSliceTma<QT, D, 2>, map_k, map_v, p);
  return true;
}

template <typename QT, int D>
cudaError_t LaunchMma(const PaParams& p, cudaStream_t stream)
{
  cudaError_t tma_err = cudaSuccess;
  if (LaunchTma<QT, D>(p, stream, &tma_err)) return tma_err;
  switch (MmaStages()) {
    case 3: return LaunchMmaNs<QT, D, 3>(p, stream);
    case 4: return LaunchMmaNs<QT, D, 4>(p, stream);
    default: return LaunchMmaNs<QT, D, 2>(p, stream);
  }
}

constexpr int kF8Stages = 3;  // 48 KB per CTA: four CTAs per SM (83 vs 89 us on the operator configuration with four stages and three CTAs)

// Stages per warp of the f8 kernel ($TLALOC_B200_PA_F8_STAGES = 3 or 4; two would not hold a 16-query partial record).
int MmaF8Stages()
{
  static const int v = [] {
    const char* e = std::getenv("TLALOC_B200_PA_F8_STAGES");
    const int x = e != nullptr ? std::atoi(e) : 0;
    return x >= 3 && x <= 4 ? x : kF8Stages;
  }();
  return v;
}

template <typename QT, int D, int NS>
cudaError_t PrepareMmaF8Ns()
{
  const int bytes = static_cast<int>(MmaLayoutF8<D, NS>::Bytes(kMaxTabEntries));
  cudaError_t e = cudaFuncSetAttribute(PaSliceMmaF8<QT, D, NS, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e == cudaSuccess) e = cudaFuncSetAttribute(PaSliceMmaF8<QT, D, NS, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e == cudaSuccess) e = cudaFuncSetAttribute(PaSliceTmaF8<QT, D, NS, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e == cudaSuccess) e = cudaFuncSetAttribute(PaSliceTmaF8<QT, D, NS, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  return e;
}

template <typename QT, int D>
cudaError_t PrepareMmaF8()
{
  cudaError_t e = PrepareMmaF8Ns<QT, D, 3>();
  if (e == cudaSuccess) e = PrepareMmaF8Ns<QT, D, 4>();
  return e;
}

template <typename QT, int D, int NS>
cudaError_t LaunchMmaF8Ns(const PaParams& p, cudaStream_t stream)
{
  const size_t smem = MmaLayoutF8<D, NS>::Bytes(p.slice / p.bs + 2);
  const dim3 grid(p.S, p.Hkv, p.Tb);
  if (MmaTmaEnabled() && p.bs_shift >= 4) {  // a group of 16 positions lies inside one block: the tiles come as TMA boxes
    CUtensorMap map_k, map_v;
    const unsigned long long positions = static_cast<unsigned long long>(p.P) * p.bs;
    if (EncodeKvPoolMap(&map_k, p.kc, D, p.Hkv, positions, 1) && EncodeKvPoolMap(&map_v, p.vc, D, p.Hkv, positions, 1)) {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = grid;
      cfg.blockDim = dim3(kMmaThreads, 1, 1);
      cfg.dynamicSmemBytes = smem;
      cfg.stream = stream;
      cudaLaunchAttribute attrs[2];
      cfg.numAttrs = ChainAttributes(attrs);
      cfg.attrs = attrs;
      if (p.NQ <= 8) return cudaLaunchKernelEx(&cfg, PaSliceTmaF8<QT, D, NS, 1>, map_k, map_v, p);
      return cudaLaunchKernelEx(&cfg, PaSliceTmaF8<QT, D, NS, 2>, map_k, map_v, p);
    }
  }
  if (p.NQ <= 8) return LaunchChained(PaSliceMmaF8<QT, D, NS, 1>, grid, kMmaThreads, smem, stream, p);
  return LaunchChained(PaSliceMmaF8<QT, D, NS, 2>, grid, kMmaThreads, smem, stream, p);
}

template <typename QT, int D>
cudaError_t LaunchMmaF8(const PaParams& p, cudaStream_t stream)
{
  switch (MmaF8Stages()) {
    case 3: return LaunchMmaF8Ns<QT, D, 3>(p, stream);
    default: return LaunchMmaF8Ns<QT, D, 4>(p, stream);
  }
}

template <typename QT, typename KVT>
cudaError_t LaunchGeneric(const PaParams& p, cudaStream_t stream)
{
  const size_t smem = sizeof(float) * (kGenQ * p.D + kGenQ * kGenTile) + sizeof(long long) * kGenTile;
  return LaunchChained(PaSliceGeneric<QT, KVT>, dim3(p.S, p.Hkv, p.Tb), kGenThreads, smem, stream, p);
}

// Positions per slice of the tensor-core kernel when the scratch allows it; $TLALOC_B200_PA_SLICE overrides.
// A CTA pays about 3 us of latency before its first position (lengths and table entries, then the first K/V rows)
// and again to merge its warps and write its records, so slices should be as long as the grid can afford: 1024
// positions, doubled (up to 4096) while the launch would still have some 2000 CTAs at the longest context, i.e. a
// few waves of the 444 resident ones at typical lengths.  Measured on the 70B step (1024 (table, KV head) pairs,
// contexts up to 16K): 0.718 -> 0.670 -> 0.661 ms per layer at 1024 / 2048 / 4096; 512 pairs: 382 / 374 / 372 us; 256
// pairs: 203 / 200 / 222 us; 128 pairs (one KV head per rank): 117 / 128 us, and 256 pairs at contexts up to 8K also
// keep 1024.
int PreferredSlice(int ctx, long long pairs)
{
  static const int forced = [] {
    const char* e = std::getenv("TLALOC_B200_PA_SLICE");
    const int x = e != nullptr ? std::atoi(e) : 0;
    return x >= 16 ? x : 0;
  }();
  if (forced > 0) return forced;
  int slice = 1024;
  while (slice < 4096 && pairs * ((ctx + 2 * slice - 1) / (2 * slice)) >= 2000) slice *= 2;
  return slice;
}

}  // namespace

cudaError_t PreparePagedAttentionKernels()
{
  static OncePerDevice once;
  return once.Run([](int) {
    TensorMapEncoderReady();  // without it the bf16 kernel keeps its cp.async form
    cudaError_t e = PrepareMma<__nv_bfloat16, 64>();
    if (e == cudaSuccess) e = PrepareMma<__nv_bfloat16, 128>();
    if (e == cudaSuccess) e = PrepareMma<float, 64>();
    if (e == cudaSuccess) e = PrepareMma<float, 128>();
    if (e == cudaSuccess) e = PrepareTma<__nv_bfloat16, 64>();
    if (e == cudaSuccess) e = PrepareTma<__nv_bfloat16, 128>();
    if (e == cudaSuccess) e = PrepareTma<float, 64>();
    if (e == cudaSuccess) e = PrepareTma<float, 128>();
    if (e == cudaSuccess) e = PrepareMmaF8<__nv_bfloat16, 64>();
    if (e == cudaSuccess) e = PrepareMmaF8<__nv_bfloat16, 128>();
    if (e == cudaSuccess) e = PrepareMmaF8<float, 64>();
    if (e == cudaSuccess) e = PrepareMmaF8<float, 128>();
    return e;
  });
}

int ReadPaStatus()
{
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_pa_status, sizeof(int)) != cudaSuccess) return -1;
  if (v != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_pa_status, &zero, sizeof(int));
  }
  return v;
}

}  // namespace tlaloc_b200

using namespace tlaloc_b200;

extern "C" int tlaloc_b200_paged_attention_splits(int32_t num_rows, int32_t num_kv_heads, int32_t num_tables,
                                                  int32_t max_blocks_per_seq, int32_t block_size)
{
  (void)num_rows;
  (void)num_kv_heads;
  (void)num_tables;
  const int64_t ctx = static_cast<int64_t>(max_blocks_per_seq) * block_size;
  // The slice count the reference's emitter sizes its scratch result for (256 positions per slice,
  // stablehlo/.../StablehloEmitter.kt:104,3475-3478); the kernels use this many or fewer.
  return static_cast<int>(ctx <= 0 ? 1 : (ctx + 255) / 256);
}

extern "C" size_t tlaloc_b200_paged_attention_scratch_bytes(int32_t num_rows, int32_t num_heads, int32_t head_dim,
                                                            int32_t splits)
{
  if (num_rows <= 0 || num_heads <= 0 || head_dim <= 0 || splits <= 0) return 0;
  return sizeof(float) * static_cast<size_t>(splits) * num_rows * num_heads * (head_dim + 2);
}

extern "C" int tlaloc_b200_paged_attention(const void* query, int32_t q_dtype, const void* key_cache,
                                           const void* value_cache, int32_t kv_dtype, const int32_t* block_tables,
                                           const int32_t* seq_lens, const int32_t* keep, int32_t keep_chunks,
                                           void* out, int32_t out_dtype, float* lse, float* scratch, int32_t splits,
                                           int32_t num_rows, int32_t num_heads, int32_t head_dim, int32_t num_blocks,
                                           int32_t block_size, int32_t num_kv_heads, int32_t max_blocks_per_seq,
                                           int32_t num_tables, float scale, int32_t sliding_window, void* stream)
{
  const char* op = "PAGED_ATTENTION";
  if (!query || !key_cache || !value_cache || !block_tables || !seq_lens || !out || !scratch) {
    return Fail(kInvalid, "%s: a required device pointer is null", op);
  }
  if (!IsFloatType(q_dtype) || !IsPoolType(kv_dtype) || !IsFloatType(out_dtype)) {
    return Fail(kInvalid, "%s: query and out must be f32 or bf16, the pools f32, bf16 or f8e4m3fn (got dtypes %d, %d, %d)", op,
                q_dtype, kv_dtype, out_dtype);
  }
  if (num_rows < 1 || num_heads < 1 || head_dim < 1) {
    return Fail(kInvalid, "%s: query must be [numSeqs, numHeads, headDim] with positive dims, got [%d, %d, %d]", op,
                num_rows, num_heads, head_dim);
  }
  if (block_size < 1 || num_blocks < 1 || max_blocks_per_seq < 1) {
    return Fail(kInvalid, "%s: needs positive numBlocks/blockSize/maxBlocksPerSeq, got %d/%d/%d", op, num_blocks,
                block_size, max_blocks_per_seq);
  }
  if (num_kv_heads < 1 || num_heads % num_kv_heads != 0) {
    return Fail(kInvalid, "%s: numHeads %d must be a positive multiple of numKvHeads %d", op, num_heads,
                num_kv_heads);
  }
  if (num_tables < 1 || num_rows % num_tables != 0) {
    return Fail(kInvalid,
                "%s: blockTables has %d rows but query has %d rows; the tables must be one per row or one per equal "
                "group of consecutive rows",
                op, num_tables, num_rows);
  }
  if (!(scale == scale) || scale > 3.0e38f || scale < -3.0e38f) return Fail(kInvalid, "%s: scale must be finite", op);
  if (sliding_window < 0) return Fail(kInvalid, "%s: sliding_window must be a whole number >= 1 (0 = none)", op);
  const int64_t ctx64 = static_cast<int64_t>(max_blocks_per_seq) * block_size;
  if (ctx64 > (1 << 30)) return Fail(kUnsupported, "%s: context of %lld positions is too long", op, (long long)ctx64);
  const int ctx = static_cast<int>(ctx64);
  if (keep != nullptr && (keep_chunks < 1 || ctx % keep_chunks != 0)) {
    return Fail(kInvalid, "%s: keep has %d chunks, which do not divide the %d positions", op, keep_chunks, ctx);
  }
  if (splits < 1) return Fail(kInvalid, "%s: scratch must hold at least one slice", op);
  if (head_dim > 256) return Fail(kUnsupported, "%s: headDim %d > 256", op, head_dim);

  PaParams p;
  p.q = query;
  p.kc = key_cache;
  p.vc = value_cache;
  p.tables = block_tables;
  p.lens = seq_lens;
  p.keep = keep;
  p.scratch = scratch;
  p.out = out;
  p.lse = lse;
  p.R = num_rows;
  p.H = num_heads;
  p.Hkv = num_kv_heads;
  p.D = head_dim;
  p.bs = block_size;
  p.M = max_blocks_per_seq;
  p.Tb = num_tables;
  p.P = num_blocks;
  p.group = num_heads / num_kv_heads;
  p.rpt = num_rows / num_tables;
  p.NQ = p.rpt * p.group;
  p.window = sliding_window;
  p.keep_chunks = keep ? keep_chunks : 0;
  p.keep_chunk = keep ? ctx / keep_chunks : 1;
  p.bs_shift = (block_size & (block_size - 1)) == 0 ? __builtin_ctz(block_size) : -1;
  p.scale = scale;

  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (OrderFaithful()) {  // parity mode: the interpreter's walk, straight into out (no slices, no scratch use)
    const int span = sliding_window > 0 ? std::min(sliding_window, ctx) : ctx;
    if (span > kFaithfulMaxCtx) {
      return Fail(kUnsupported, "%s: parity mode holds a row's scores on chip, at most %d positions (got %d)", op, kFaithfulMaxCtx, span);
    }
    p.slice = ctx;
    p.S = 1;
    cudaError_t fe;
    if (q_dtype == TLALOC_B200_F32 && kv_dtype == TLALOC_B200_F32) fe = LaunchFaithful<float, float>(p, out_dtype, span, st);
    else if (q_dtype == TLALOC_B200_F32 && kv_dtype == TLALOC_B200_BF16) fe = LaunchFaithful<float, __nv_bfloat16>(p, out_dtype, span, st);
    else if (q_dtype == TLALOC_B200_F32) fe = LaunchFaithful<float, __nv_fp8_e4m3>(p, out_dtype, span, st);
    else if (kv_dtype == TLALOC_B200_F32) fe = LaunchFaithful<__nv_bfloat16, float>(p, out_dtype, span, st);
    else if (kv_dtype == TLALOC_B200_BF16) fe = LaunchFaithful<__nv_bfloat16, __nv_bfloat16>(p, out_dtype, span, st);
    else fe = LaunchFaithful<__nv_bfloat16, __nv_fp8_e4m3>(p, out_dtype, span, st);
    if (fe != cudaSuccess) return CudaFail("PAGED_ATTENTION parity-mode launch", fe);
    CountLaunches(1);
    return kOk;
  }
  // The tensor-core kernel copies K/V rows in 16-byte pieces: pools that start off a 16-byte boundary (a slice of a
  // larger allocation at an odd element) take the generic kernel, which has no alignment needs.
  // $TLALOC_B200_PA_F8_GENERIC=1 sends e4m3fn pools to the generic kernel (a debugging aid).
  static const bool f8_generic = [] {
    const char* v = std::getenv("TLALOC_B200_PA_F8_GENERIC");
    return v != nullptr && v[0] == '1';
  }();
  const bool f8 = kv_dtype == TLALOC_B200_F8E4M3FN;
  const bool mma = (kv_dtype == TLALOC_B200_BF16 || (f8 && !f8_generic)) && (head_dim == 64 || head_dim == 128) && p.NQ <= kMmaQ &&
                   keep == nullptr && (f8 ? block_size >= 16 : block_size >= 8) && Aligned16(key_cache) && Aligned16(value_cache);
  // Slice length: the preferred one (tensor-core kernel) or 256, stretched until `splits` slices cover the context.
  int slice = mma ? PreferredSlice(ctx, static_cast<long long>(num_tables) * num_kv_heads) : 256;
  if (static_cast<int64_t>(slice) * splits < ctx) slice = (ctx + splits - 1) / splits;
  if (mma) slice = std::min((slice + 15) / 16 * 16, 8192);
  if (static_cast<int64_t>(slice) * splits < ctx) {
    return Fail(kInvalid, "%s: scratch holds %d slices, too few for %d positions", op, splits, ctx);
  }
  p.slice = slice;
  p.S = (ctx + slice - 1) / slice;

  cudaError_t e = cudaSuccess;
  if (mma) {
    e = PreparePagedAttentionKernels();
    if (e != cudaSuccess) return CudaFail("PAGED_ATTENTION set-up", e);
    if (f8) {
      if (q_dtype == TLALOC_B200_BF16) e = head_dim == 64 ? LaunchMmaF8<__nv_bfloat16, 64>(p, st) : LaunchMmaF8<__nv_bfloat16, 128>(p, st);
      else e = head_dim == 64 ? LaunchMmaF8<float, 64>(p, st) : LaunchMmaF8<float, 128>(p, st);
    } else if (q_dtype == TLALOC_B200_BF16) {
      e = head_dim == 64 ? LaunchMma<__nv_bfloat16, 64>(p, st) : LaunchMma<__nv_bfloat16, 128>(p, st);
    } else {
      e = head_dim == 64 ? LaunchMma<float, 64>(p, st) : LaunchMma<float, 128>(p, st);
    }
  } else if (q_dtype == TLALOC_B200_F32 && kv_dtype == TLALOC_B200_F32) {
    e = LaunchGeneric<float, float>(p, st);
  } else if (q_dtype == TLALOC_B200_F32 && kv_dtype == TLALOC_B200_BF16) {
    e = LaunchGeneric<float, __nv_bfloat16>(p, st);
  } else if (q_dtype == TLALOC_B200_F32) {
    e = LaunchGeneric<float, __nv_fp8_e4m3>(p, st);
  } else if (kv_dtype == TLALOC_B200_F32) {
    e = LaunchGeneric<__nv_bfloat16, float>(p, st);
  } else if (kv_dtype == TLALOC_B200_BF16) {
    e = LaunchGeneric<__nv_bfloat16, __nv_bfloat16>(p, st);
  } else {
    e = LaunchGeneric<__nv_bfloat16, __nv_fp8_e4m3>(p, st);
  }
  if (e != cudaSuccess) return CudaFail("PAGED_ATTENTION slice launch", e);
  const unsigned cgrid = static_cast<unsigned>((p.R * p.H + kCombineThreads / 32 - 1) / (kCombineThreads / 32));
  if (out_dtype == TLALOC_B200_F32) {
    e = p.D <= 64    ? LaunchChained(PaCombine<float, 1>, cgrid, kCombineThreads, 0, st, p)
        : p.D <= 128 ? LaunchChained(PaCombine<float, 2>, cgrid, kCombineThreads, 0, st, p)
                     : LaunchChained(PaCombine<float, 4>, cgrid, kCombineThreads, 0, st, p);
  } else {
    e = p.D <= 64    ? LaunchChained(PaCombine<__nv_bfloat16, 1>, cgrid, kCombineThreads, 0, st, p)
        : p.D <= 128 ? LaunchChained(PaCombine<__nv_bfloat16, 2>, cgrid, kCombineThreads, 0, st, p)
                     : LaunchChained(PaCombine<__nv_bfloat16, 4>, cgrid, kCombineThreads, 0, st, p);
  }
  if (e != cudaSuccess) return CudaFail("PAGED_ATTENTION combine launch", e);
  CountLaunches(2);
  return kOk;
}

extern "C" int tlaloc_b200_kv_cache_write(void* pool, int32_t pool_dtype, const void* new_kv, int32_t new_dtype,
                                          const int32_t* slot_mapping, int32_t num_tokens, int32_t row_elems,
                                          int32_t num_slots, void* stream)
{
  const char* op = "KV_CACHE_WRITE";
  if (!pool || !new_kv || !slot_mapping) return Fail(kInvalid, "%s: a required device pointer is null", op);
  if (!IsPoolType(pool_dtype) || !IsFloatType(new_dtype)) return Fail(kInvalid, "%s: the pool must be f32, bf16 or f8e4m3fn, the rows f32 or bf16", op);
  if (num_tokens < 0 || row_elems < 1 || num_slots < 1) return Fail(kInvalid, "%s: bad sizes", op);
  if (num_tokens == 0) return kOk;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int threads = row_elems >= 256 ? 256 : 128;
  cudaError_t e;
#define TLALOC_KVW(PT, NT)                                                                                    \
  e = LaunchChained(KvCacheWriteKernel<PT, NT>, num_tokens, threads, 0, st, static_cast<PT*>(pool),           \
                    static_cast<const NT*>(new_kv), slot_mapping, row_elems, num_slots)
  if (pool_dtype == TLALOC_B200_F32 && new_dtype == TLALOC_B200_F32) TLALOC_KVW(float, float);
  else if (pool_dtype == TLALOC_B200_F32) TLALOC_KVW(float, __nv_bfloat16);
  else if (pool_dtype == TLALOC_B200_BF16 && new_dtype == TLALOC_B200_F32) TLALOC_KVW(__nv_bfloat16, float);
  else if (pool_dtype == TLALOC_B200_BF16) TLALOC_KVW(__nv_bfloat16, __nv_bfloat16);
  else if (new_dtype == TLALOC_B200_F32) TLALOC_KVW(__nv_fp8_e4m3, float);
  else TLALOC_KVW(__nv_fp8_e4m3, __nv_bfloat16);
#undef TLALOC_KVW
  if (e != cudaSuccess) return CudaFail("KV_CACHE_WRITE launch", e);
  CountLaunches(1);
  return kOk;
}

// ------------------------------------------------------------------------------------------
// Paged attention for callers that cannot allocate device memory.
//
// The split records live in one fixed array inside this library instead of a caller's buffer.  The array is a
// device symbol: in host code its name only stands for it, so the address the kernels receive is looked up with
// cudaGetSymbolAddress, once per device, with that device current.

namespace {

constexpr size_t kStaticScratchBytes = size_t(16) << 20;  // 16 MiB on every GPU that loads the library, until exit
static __device__ __align__(256) float g_static_scratch[kStaticScratchBytes / sizeof(float)];

std::mutex g_static_mu;
float* g_static_ptr[kMaxDevices] = {nullptr};

// The device address of g_static_scratch on the current device (resolved on the first call per device).
cudaError_t StaticScratch(float** out)
{
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return e;
  if (device < 0 || device >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(g_static_mu);
  if (g_static_ptr[device] == nullptr) {
    float* ptr = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_static_scratch);
    if (e != cudaSuccess) return e;
    g_static_ptr[device] = ptr;
  }
  *out = g_static_ptr[device];
  return cudaSuccess;
}

}  // namespace

extern "C" size_t tlaloc_b200_paged_attention_static_scratch_bytes(void) { return kStaticScratchBytes; }

extern "C" int tlaloc_b200_paged_attention_static(const void* query, int32_t q_dtype, const void* key_cache,
                                                  const void* value_cache, int32_t kv_dtype,
                                                  const int32_t* block_tables, const int32_t* seq_lens,
                                                  const int32_t* keep, int32_t keep_chunks, void* out,
                                                  int32_t out_dtype, float* lse, int32_t num_rows, int32_t num_heads,
                                                  int32_t head_dim, int32_t num_blocks, int32_t block_size,
                                                  int32_t num_kv_heads, int32_t max_blocks_per_seq,
                                                  int32_t num_tables, float scale, int32_t sliding_window,
                                                  void* stream)
{
  const char* op = "PAGED_ATTENTION (static scratch)";
  if (num_rows < 1 || num_heads < 1 || head_dim < 1 || block_size < 1 || max_blocks_per_seq < 1) {
    return Fail(kInvalid, "%s: needs positive query and table dims", op);
  }
  const int64_t ctx = static_cast<int64_t>(max_blocks_per_seq) * block_size;
  const size_t record_set = sizeof(float) * static_cast<size_t>(num_rows) * num_heads * (head_dim + 2);  // one slice
  const int64_t fit = static_cast<int64_t>(kStaticScratchBytes / record_set);
  const int64_t least = (ctx + 8191) / 8192;  // the longest slice a launch takes is 8192 positions
  if (fit < 1 || fit < least) {
    return Fail(kInvalid,
                "%s: %d rows x %d heads x head_dim %d over %lld positions needs %zu bytes of split records, more than "
                "the %zu-byte array built into the library; use tlaloc_b200_paged_attention with your own scratch",
                op, num_rows, num_heads, head_dim, (long long)ctx, record_set * static_cast<size_t>(least),
                kStaticScratchBytes);
  }
  const int64_t want = (ctx + 255) / 256;
  const int32_t splits = static_cast<int32_t>(std::min(fit, want));
  float* scratch = nullptr;
  const cudaError_t e = StaticScratch(&scratch);
  if (e != cudaSuccess) return CudaFail("PAGED_ATTENTION (static scratch) set-up", e);
  return tlaloc_b200_paged_attention(query, q_dtype, key_cache, value_cache, kv_dtype, block_tables, seq_lens, keep,
                                     keep_chunks, out, out_dtype, lse, scratch, splits, num_rows, num_heads, head_dim,
                                     num_blocks, block_size, num_kv_heads, max_blocks_per_seq, num_tables, scale,
                                     sliding_window, stream);
}
