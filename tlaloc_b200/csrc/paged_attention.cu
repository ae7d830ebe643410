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
//                   Q.K^T and P.V on mma.sync m16n8k16 bf16 with fp32 accumulators, the
//                   probabilities (and an f32 query) carried as hi + lo bf16 parts so
//                   the result keeps ~16 bits; warp-shuffle online softmax in the log2
//                   domain.  HBM-bound: the tensor work is two to three small MMAs per
//                   position, far below what the SM can issue while the copies land.
//   PaSliceGeneric  any D <= 256, any block size, f32 or bf16 pools, keep masks, up to
//                   any number of queries (in passes of 8): plain fp32 FMA, warp per
//                   position for the scores and thread per head dimension for the values.
#include <mutex>

#include "common.cuh"

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

constexpr int kMmaThreads = 128;
constexpr int kMmaWarps = 4;
constexpr int kMmaQ = 16;  // query rows of one m16 tile
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

// Dynamic shared memory of PaSliceMma, in bytes: the query tile(s), the four warps'
// stages, then the slice's block-table entries.
template <int D, bool QLO, int NS>
struct MmaLayout {
  static constexpr int kRowBytes = D * 2;
  static constexpr int kTileBytes = 16 * kRowBytes;  // 16 positions of K (or V), or the 16 query rows
  static constexpr int kStageBytes = 2 * kTileBytes;
  static constexpr int kWarpBytes = NS * kStageBytes;
  static constexpr int kQBytes = (QLO ? 2 : 1) * kTileBytes;
  static constexpr int kTabOffset = kQBytes + kMmaWarps * kWarpBytes;
  static_assert(kWarpBytes >= static_cast<int>(sizeof(float)) * kMmaQ * (D + 2), "a warp's stages hold its partial record");
  static size_t Bytes(int tab_entries) { return kTabOffset + sizeof(int) * static_cast<size_t>(tab_entries); }
};

template <typename QT, int D, int NS>
__global__ void __launch_bounds__(kMmaThreads) PaSliceMma(PaParams p)
{
  constexpr bool QLO = sizeof(QT) == 4;
  using L = MmaLayout<D, QLO, NS>;
  constexpr int CPR = L::kRowBytes / 16;  // 16-byte chunks per row
  extern __shared__ __align__(1024) unsigned char smem[];
  unsigned char* qhi = smem;
  unsigned char* qlo = smem + L::kTileBytes;
  unsigned char* stages = smem + L::kQBytes;
  int* tab = reinterpret_cast<int*>(smem + L::kTabOffset);
  __shared__ int qlen_s[kMmaQ], qfirst_s[kMmaQ];

  const int s = blockIdx.x, kv = blockIdx.y, tb = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int gid = lane >> 2, tig = lane & 3;
  const int ctx = p.M * p.bs;
  const int c0 = s * p.slice;

  // Every thread derives the CTA's live range from its (<= 16) rows' lengths.
  int maxlen = 0, minfirst = ctx;
  for (int r = 0; r < p.rpt; ++r) {
    const int len = ClampI(__ldg(p.lens + tb * p.rpt + r), 0, ctx);
    maxlen = max(maxlen, len);
    minfirst = min(minfirst, p.window > 0 ? max(0, len - p.window) : 0);
  }
  const int c1 = min(min(c0 + p.slice, ctx), maxlen);
  const int t_begin = max(c0, minfirst);
  if (t_begin >= c1) return;
  const int ngroups = (c1 - t_begin + 15) >> 4;

  if (tid < kMmaQ) {
    int len = 0, first = 0;
    if (tid < p.NQ) {
      const int full = ClampI(__ldg(p.lens + tb * p.rpt + tid / p.group), 0, ctx);
      first = p.window > 0 ? max(0, full - p.window) : 0;
      len = min(full, c1);
    }
    qlen_s[tid] = len;
    qfirst_s[tid] = first;
  }
  const int b0 = p.bs_shift >= 0 ? (t_begin >> p.bs_shift) : t_begin / p.bs;
  const int b1 = p.bs_shift >= 0 ? ((c1 - 1) >> p.bs_shift) : (c1 - 1) / p.bs;
  for (int j = tid; j <= b1 - b0; j += kMmaThreads) {
    tab[j] = ClampI(__ldg(p.tables + static_cast<size_t>(tb) * p.M + b0 + j), 0, p.P - 1);
  }
  // The query tile: rows i < NQ hold query i (row i / group of the table, head kv*group + i % group), the
  // rest zero; bf16 hi part (and lo part for an f32 query), chunk-swizzled like the K/V rows.
  {
    const QT* q = static_cast<const QT*>(p.q);
    for (int idx = tid; idx < kMmaQ * (D / 2); idx += kMmaThreads) {
      const int i = idx / (D / 2), d = (idx - i * (D / 2)) * 2;
      float x = 0.f, y = 0.f;
      if (i < p.NQ) {
        const QT* src = q + (static_cast<size_t>(tb * p.rpt + i / p.group) * p.H + kv * p.group + i % p.group) * D + d;
        x = ToF32(src[0]);
        y = ToF32(src[1]);
      }
      uint32_t hi, lo;
      SplitPack(x, y, hi, lo);
      const int byte = d * 2, chunk = byte >> 4, within = byte & 15;
      const int at = i * L::kRowBytes + ((chunk ^ (i & 7)) << 4) + within;
      *reinterpret_cast<uint32_t*>(qhi + at) = hi;
      if (QLO) *reinterpret_cast<uint32_t*>(qlo + at) = lo;
    }
  }
  __syncthreads();

  const __nv_bfloat16* kc = static_cast<const __nv_bfloat16*>(p.kc);
  const __nv_bfloat16* vc = static_cast<const __nv_bfloat16*>(p.vc);
  unsigned char* my_stages = stages + warp * L::kWarpBytes;
  const uint32_t my_stages_addr = SmemAddr(my_stages);
  const int my_n = warp < ngroups ? (ngroups - warp + kMmaWarps - 1) / kMmaWarps : 0;

  // One group of 16 positions: each lane copies 16-byte chunks of the K and V rows; a row's chunk c
  // lands at chunk c ^ (row & 7) so that the ldmatrix reads below are conflict-free.
  auto issue = [&](int it) {
    const int t_base = t_begin + ((warp + kMmaWarps * it) << 4);
    const uint32_t dst_base = my_stages_addr + (it % NS) * L::kStageBytes;
#pragma unroll
    for (int i = 0; i < 16 * CPR / 32; ++i) {
      const int c = lane + 32 * i;
      const int r = c / CPR, col = c % CPR;
      const int t = t_base + r;
      const bool valid = t < c1;
      size_t off = 0;
      if (valid) {
        const int blk_i = p.bs_shift >= 0 ? (t >> p.bs_shift) : t / p.bs;
        const int slot = t - blk_i * p.bs;
        off = ((static_cast<size_t>(tab[blk_i - b0]) * p.bs + slot) * p.Hkv + kv) * D + col * 8;
      }
      const uint32_t dst = dst_base + r * L::kRowBytes + ((col ^ (r & 7)) << 4);
      CpAsync16(dst, kc + off, valid ? 16 : 0);
      CpAsync16(dst + L::kTileBytes, vc + off, valid ? 16 : 0);
    }
  };

  for (int it = 0; it < NS - 1; ++it) {
    if (it < my_n) issue(it);
    CpAsyncCommit();
  }

  float o[D / 8][4];
#pragma unroll
  for (int n = 0; n < D / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
  const int len_lo = qlen_s[gid], len_hi = qlen_s[gid + 8];
  const int first_lo = qfirst_s[gid], first_hi = qfirst_s[gid + 8];
  const float sl2 = p.scale * kLog2e;
  const uint32_t qhi_addr = SmemAddr(qhi), qlo_addr = SmemAddr(qlo);
  const int row_a = (lane & 7) + ((lane >> 3) & 1) * 8;  // A (query) and V: matrices 1, 3 are rows 8..15
  const int row_b = (lane & 7) + (lane >> 4) * 8;        // K: matrices 2, 3 are positions 8..15

  for (int it = 0; it < my_n; ++it) {
    if (it + NS - 1 < my_n) issue(it + NS - 1);
    CpAsyncCommit();
    CpAsyncWait<NS - 1>();
    __syncwarp();
    const int t_base = t_begin + ((warp + kMmaWarps * it) << 4);
    const uint32_t k_addr = my_stages_addr + (it % NS) * L::kStageBytes;
    const uint32_t v_addr = k_addr + L::kTileBytes;

    float sacc[2][4];
#pragma unroll
    for (int j = 0; j < 2; ++j) sacc[j][0] = sacc[j][1] = sacc[j][2] = sacc[j][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      uint32_t a[4], b[4];
      LdMatrixX4(a, qhi_addr + row_a * L::kRowBytes + (((2 * kk + (lane >> 4)) ^ (row_a & 7)) << 4));
      LdMatrixX4(b, k_addr + row_b * L::kRowBytes + (((2 * kk + ((lane >> 3) & 1)) ^ (row_b & 7)) << 4));
      MmaBf16(sacc[0], a, b[0], b[1]);
      MmaBf16(sacc[1], a, b[2], b[3]);
      if (QLO) {
        LdMatrixX4(a, qlo_addr + row_a * L::kRowBytes + (((2 * kk + (lane >> 4)) ^ (row_a & 7)) << 4));
        MmaBf16(sacc[0], a, b[0], b[1]);
        MmaBf16(sacc[1], a, b[2], b[3]);
      }
    }
    // Scale into the log2 domain, mask, and fold the group into the running softmax state.
    float tmax_lo = -INFINITY, tmax_hi = -INFINITY;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int tok = t_base + 8 * j + 2 * tig + (e & 1);
        const bool live = e < 2 ? (tok < len_lo && tok >= first_lo) : (tok < len_hi && tok >= first_hi);
        const float v = live ? sacc[j][e] * sl2 : -INFINITY;
        sacc[j][e] = v;
        if (e < 2) tmax_lo = fmaxf(tmax_lo, v);
        else tmax_hi = fmaxf(tmax_hi, v);
      }
    }
    tmax_lo = fmaxf(tmax_lo, __shfl_xor_sync(0xffffffffu, tmax_lo, 1));
    tmax_lo = fmaxf(tmax_lo, __shfl_xor_sync(0xffffffffu, tmax_lo, 2));
    tmax_hi = fmaxf(tmax_hi, __shfl_xor_sync(0xffffffffu, tmax_hi, 1));
    tmax_hi = fmaxf(tmax_hi, __shfl_xor_sync(0xffffffffu, tmax_hi, 2));
    const float mn_lo = fmaxf(m_lo, tmax_lo), mn_hi = fmaxf(m_hi, tmax_hi);
    const float alpha_lo = mn_lo == -INFINITY ? 1.f : Exp2(m_lo - mn_lo);
    const float alpha_hi = mn_hi == -INFINITY ? 1.f : Exp2(m_hi - mn_hi);
    const float base_lo = mn_lo == -INFINITY ? 0.f : mn_lo, base_hi = mn_hi == -INFINITY ? 0.f : mn_hi;
    m_lo = mn_lo;
    m_hi = mn_hi;
    float ps_lo = 0.f, ps_hi = 0.f;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      sacc[j][0] = Exp2(sacc[j][0] - base_lo);
      sacc[j][1] = Exp2(sacc[j][1] - base_lo);
      sacc[j][2] = Exp2(sacc[j][2] - base_hi);
      sacc[j][3] = Exp2(sacc[j][3] - base_hi);
      ps_lo += sacc[j][0] + sacc[j][1];
      ps_hi += sacc[j][2] + sacc[j][3];
    }
    l_lo = l_lo * alpha_lo + ps_lo;
    l_hi = l_hi * alpha_hi + ps_hi;
#pragma unroll
    for (int n = 0; n < D / 8; ++n) {
      o[n][0] *= alpha_lo;
      o[n][1] *= alpha_lo;
      o[n][2] *= alpha_hi;
      o[n][3] *= alpha_hi;
    }
    uint32_t ph[4], pl[4];
    SplitPack(sacc[0][0], sacc[0][1], ph[0], pl[0]);
    SplitPack(sacc[0][2], sacc[0][3], ph[1], pl[1]);
    SplitPack(sacc[1][0], sacc[1][1], ph[2], pl[2]);
    SplitPack(sacc[1][2], sacc[1][3], ph[3], pl[3]);
#pragma unroll
    for (int c = 0; c < CPR; c += 2) {
      uint32_t b[4];
      LdMatrixX4Trans(b, v_addr + row_a * L::kRowBytes + (((c + (lane >> 4)) ^ (row_a & 7)) << 4));
      MmaBf16(o[c], ph, b[0], b[1]);
      MmaBf16(o[c + 1], ph, b[2], b[3]);
      MmaBf16(o[c], pl, b[0], b[1]);
      MmaBf16(o[c + 1], pl, b[2], b[3]);
    }
    __syncwarp();  // the stage is free for the copy the next iteration issues
  }
  CpAsyncWait<0>();
  __syncwarp();

  // Each warp leaves {m, l, o} of its positions in its own stage space; the CTA then merges the four.
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
  {
    float* wm = reinterpret_cast<float*>(my_stages);
    float* wl = wm + kMmaQ;
    float* wo = wl + kMmaQ;
    if (tig == 0) {
      wm[gid] = m_lo;
      wm[gid + 8] = m_hi;
      wl[gid] = l_lo;
      wl[gid + 8] = l_hi;
    }
#pragma unroll
    for (int n = 0; n < D / 8; ++n) {
      *reinterpret_cast<float2*>(wo + gid * D + n * 8 + 2 * tig) = make_float2(o[n][0], o[n][1]);
      *reinterpret_cast<float2*>(wo + (gid + 8) * D + n * 8 + 2 * tig) = make_float2(o[n][2], o[n][3]);
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

// ------------------------------------------------------------------------------------------
// Combine: grid R*H.  Row r's live slices are [first / slice, ceil(len / slice)); their records merge as
// out = sum_s exp(m_s - max) acc_s / sum_s exp(m_s - max) l_s, in slice order (deterministic).

constexpr int kCombineThreads = 128;

template <typename OT>
__global__ void __launch_bounds__(kCombineThreads) PaCombine(PaParams p)
{
  extern __shared__ float w_s[];  // [S]
  const int rh = blockIdx.x, row = rh / p.H, head = rh - row * p.H;
  const int tid = threadIdx.x;
  const int ctx = p.M * p.bs;
  const int len = ClampI(__ldg(p.lens + row), 0, ctx);
  const int first = p.window > 0 ? max(0, len - p.window) : 0;
  const int s_lo = first / p.slice, s_hi = min(p.S, (len + p.slice - 1) / p.slice);
  const size_t stride = static_cast<size_t>(p.R) * p.H * (p.D + 2);
  const float* base = Record(p, 0, row, head);
  float mx = -INFINITY;
  for (int s = s_lo; s < s_hi; ++s) mx = fmaxf(mx, base[s * stride]);
  float denom = 0.f;
  for (int s = s_lo; s < s_hi; ++s) {
    const float m = base[s * stride];
    const float w = m == -INFINITY ? 0.f : expf(m - mx);
    if (tid == 0) w_s[s] = w;
    if (w != 0.f) denom += w * base[s * stride + 1];
  }
  __syncthreads();
  OT* out = static_cast<OT*>(p.out) + static_cast<size_t>(rh) * p.D;
  const bool empty = mx == -INFINITY || denom == 0.f;
  for (int d = tid; d < p.D; d += kCombineThreads) {
    float a = 0.f;
    if (!empty) {
      for (int s = s_lo; s < s_hi; ++s) {
        const float w = w_s[s];
        if (w != 0.f) a += w * base[s * stride + 2 + d];
      }
      a /= denom;
    }
    out[d] = FromF32<OT>(a);
  }
  if (tid == 0 && p.lse != nullptr) p.lse[rh] = empty ? -INFINITY : mx + logf(denom);
}

// ------------------------------------------------------------------------------------------
// KV_CACHE_WRITE: one CTA per token row.

template <typename PT, typename NT>
__global__ void KvCacheWriteKernel(PT* pool, const NT* new_kv, const int* slots, int row_elems, int num_slots)
{
  const int i = blockIdx.x;
  const int slot = __ldg(slots + i);
  if (slot < 0 || slot >= num_slots) return;
  PT* dst = pool + static_cast<size_t>(slot) * row_elems;
  const NT* src = new_kv + static_cast<size_t>(i) * row_elems;
  for (int j = threadIdx.x; j < row_elems; j += blockDim.x) dst[j] = FromF32<PT>(ToF32(src[j]));
}

// ------------------------------------------------------------------------------------------
// Host side.

constexpr int kMmaStages = 3;

template <typename QT, int D>
cudaError_t PrepareMma()
{
  using L = MmaLayout<D, sizeof(QT) == 4, kMmaStages>;
  // Room for the table entries of the longest slice a launch may choose (8192 positions of 8-position blocks).
  return cudaFuncSetAttribute(PaSliceMma<QT, D, kMmaStages>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              static_cast<int>(L::Bytes(1024 + 2)));
}

template <typename QT, int D>
cudaError_t LaunchMma(const PaParams& p, cudaStream_t stream)
{
  using L = MmaLayout<D, sizeof(QT) == 4, kMmaStages>;
  const size_t smem = L::Bytes(p.slice / p.bs + 2);
  PaSliceMma<QT, D, kMmaStages><<<dim3(p.S, p.Hkv, p.Tb), kMmaThreads, smem, stream>>>(p);
  return cudaGetLastError();
}

template <typename QT, typename KVT>
cudaError_t LaunchGeneric(const PaParams& p, cudaStream_t stream)
{
  const size_t smem = sizeof(float) * (kGenQ * p.D + kGenQ * kGenTile) + sizeof(long long) * kGenTile;
  PaSliceGeneric<QT, KVT><<<dim3(p.S, p.Hkv, p.Tb), kGenThreads, smem, stream>>>(p);
  return cudaGetLastError();
}

// Positions per slice of the tensor-core kernel when the scratch allows it; $TLALOC_B200_PA_SLICE overrides.
int PreferredSlice()
{
  static const int v = [] {
    const char* e = std::getenv("TLALOC_B200_PA_SLICE");
    const int x = e != nullptr ? std::atoi(e) : 0;
    return x >= 16 ? x : 512;
  }();
  return v;
}

}  // namespace

cudaError_t PreparePagedAttentionKernels()
{
  static std::mutex mu;
  static bool done = false;
  std::lock_guard<std::mutex> lock(mu);
  if (done) return cudaSuccess;
  cudaError_t e = PrepareMma<__nv_bfloat16, 64>();
  if (e == cudaSuccess) e = PrepareMma<__nv_bfloat16, 128>();
  if (e == cudaSuccess) e = PrepareMma<float, 64>();
  if (e == cudaSuccess) e = PrepareMma<float, 128>();
  if (e == cudaSuccess) done = true;
  return e;
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
  if (!IsFloatType(q_dtype) || !IsFloatType(kv_dtype) || !IsFloatType(out_dtype)) {
    return Fail(kInvalid, "%s: query, pools and out must be f32 or bf16 (got dtypes %d, %d, %d)", op, q_dtype,
                kv_dtype, out_dtype);
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
  const bool mma = kv_dtype == TLALOC_B200_BF16 && (head_dim == 64 || head_dim == 128) && p.NQ <= kMmaQ &&
                   keep == nullptr && block_size >= 8;
  // Slice length: the preferred one (tensor-core kernel) or 256, stretched until `splits` slices cover the context.
  int slice = mma ? PreferredSlice() : 256;
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
    if (q_dtype == TLALOC_B200_BF16) {
      e = head_dim == 64 ? LaunchMma<__nv_bfloat16, 64>(p, st) : LaunchMma<__nv_bfloat16, 128>(p, st);
    } else {
      e = head_dim == 64 ? LaunchMma<float, 64>(p, st) : LaunchMma<float, 128>(p, st);
    }
  } else if (q_dtype == TLALOC_B200_F32 && kv_dtype == TLALOC_B200_F32) {
    e = LaunchGeneric<float, float>(p, st);
  } else if (q_dtype == TLALOC_B200_F32) {
    e = LaunchGeneric<float, __nv_bfloat16>(p, st);
  } else if (kv_dtype == TLALOC_B200_F32) {
    e = LaunchGeneric<__nv_bfloat16, float>(p, st);
  } else {
    e = LaunchGeneric<__nv_bfloat16, __nv_bfloat16>(p, st);
  }
  if (e != cudaSuccess) return CudaFail("PAGED_ATTENTION slice launch", e);
  const size_t csmem = sizeof(float) * p.S;
  if (out_dtype == TLALOC_B200_F32) {
    PaCombine<float><<<p.R * p.H, kCombineThreads, csmem, st>>>(p);
  } else {
    PaCombine<__nv_bfloat16><<<p.R * p.H, kCombineThreads, csmem, st>>>(p);
  }
  e = cudaGetLastError();
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
  if (!IsFloatType(pool_dtype) || !IsFloatType(new_dtype)) return Fail(kInvalid, "%s: pool and rows must be f32 or bf16", op);
  if (num_tokens < 0 || row_elems < 1 || num_slots < 1) return Fail(kInvalid, "%s: bad sizes", op);
  if (num_tokens == 0) return kOk;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int threads = row_elems >= 256 ? 256 : 128;
  if (pool_dtype == TLALOC_B200_F32 && new_dtype == TLALOC_B200_F32) {
    KvCacheWriteKernel<<<num_tokens, threads, 0, st>>>(static_cast<float*>(pool), static_cast<const float*>(new_kv),
                                                       slot_mapping, row_elems, num_slots);
  } else if (pool_dtype == TLALOC_B200_F32) {
    KvCacheWriteKernel<<<num_tokens, threads, 0, st>>>(static_cast<float*>(pool),
                                                       static_cast<const __nv_bfloat16*>(new_kv), slot_mapping,
                                                       row_elems, num_slots);
  } else if (new_dtype == TLALOC_B200_F32) {
    KvCacheWriteKernel<<<num_tokens, threads, 0, st>>>(static_cast<__nv_bfloat16*>(pool),
                                                       static_cast<const float*>(new_kv), slot_mapping, row_elems,
                                                       num_slots);
  } else {
    KvCacheWriteKernel<<<num_tokens, threads, 0, st>>>(static_cast<__nv_bfloat16*>(pool),
                                                       static_cast<const __nv_bfloat16*>(new_kv), slot_mapping,
                                                       row_elems, num_slots);
  }
  const cudaError_t e = cudaGetLastError();
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

constexpr int kMaxDevices = 64;
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
