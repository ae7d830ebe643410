// The int8 weight-only projection for 17 to 128 rows with the weights left as int8 all the way to the tensor core:
// y = (cast(x) @ cast(codes)) * scale (HfDecoderGraph.proj, ir/.../inference/HfDecoderGraph.kt:625-655).
//
// The bf16 form of this projection (int8_gemm_tc.cu) spends its time turning codes into bf16 on the ALUs and pushing them
// through shared memory twice.  (Opt-in: TLALOC_B200_GEMM_I8_MMA; the caller accepts the activation format below.)  Here the codes go global -> shared memory by TMA and are read by tcgen05.mma.kind::i8
// as they are; it is the ACTIVATIONS that change form.  A row of x (bf16; an f32 x is rounded to bf16 first, as the
// bf16 kernel does) is written as
//     x[m, k] ~ (256 hi[m, k] + lo[m, k]) * s[m],   s[m] a power of two, hi in [-127, 127], lo in [-128, 127]
// i.e. a 16-bit fixed-point number under a per-row power-of-two scale: every element within 2^8 of the row's largest
// magnitude is represented EXACTLY (a bf16 has 8 significant bits), smaller ones are rounded to the nearest multiple of
// s[m], an absolute error of at most 2^-16 of the row's largest magnitude.  Then
//     y[m, n] = (256 sum_k hi w + sum_k lo w) * s[m] * scale[n]
// with both sums exact in int32 (|sum| <= 128 * 127 * K), two MMAs per K step into two TMEM accumulators (up to 64
// rows: one MMA whose 128 lanes carry both planes).  Integer-valued
// activations come out exact; for others the difference from the f32-accumulating bf16 kernel is far below bf16's own
// rounding of the inputs.  A row holding an infinity or a NaN gets s = NaN, so its whole output row is NaN.
//
// Formulation: D[m, n] = sum_k X[m, k] W[k, n], activation rows = the MMA's M (TMEM lanes), 256 weight columns = its N.
// A CTA owns 256 columns and one slice of K, walked in blocks of 128 rows through a ring of three stages (65 to 128
// activation rows; four stages for up to 64 rows, five for up to 32, whose strips are smaller):
//   producer thread  one lane; per block four TMA loads (hi strip, lo strip: K-major 128-byte-swizzled [rows][128 k];
//                    the block's codes as two MN-major 128-byte-swizzled boxes [128 k][128 n]: W's rows are contiguous
//                    along N, which is MN-major, so nothing is transposed) onto the stage's mbarrier;
//   MMA thread       one lane; per block 4 K-steps x {hi, lo} of 128 x 256 x 32 (up to 64 rows: the two strips, which
//                    lie one after the other, are ONE 128-row A operand, so one MMA per K-step serves both planes and
//                    the codes leave shared memory once), then a commit that hands the stage back;
//   sixteen warps    sleep at the CTA barrier until the last MMA has completed, then run the epilogue shared with the
//                    bf16 kernel (tile in shared memory, scale / residual / SwiGLU, cluster sum over the K slices).
// Rows past M and k past K are outside the tensor maps and arrive as zeros.  Every mbarrier wait is bounded.
#include <cuda.h>

#include <mutex>

#include "common.cuh"
#include "tc_common.cuh"

namespace tlaloc_b200 {
namespace {

using namespace tc;

constexpr int kI8BK = 128;                 // k rows per block
constexpr int kI8AtomBytes = kI8BK * 128;  // 128 k rows x 128 columns of codes
constexpr int kI8Workers = 512;            // the epilogue's threads
constexpr int kI8Threads = kI8Workers + 64;  // plus the MMA warp and the producer warp

// Shared memory for launches of up to MROWS activation rows (32, 64 or 128): the ring of stages, each [hi strip][lo
// strip][two atoms of codes], then the mbarriers, the TMEM base, the abort word and the tile's scales.  The strips hold
// MROWS rows; the MMA always reads 128 (the rows past MROWS are whatever follows in the stage, and only reach
// accumulator lanes that are never read), so fewer rows leave room for more stages: 3 of 64 KB, 4 of 48 KB, 5 of 40 KB.
template <int MROWS>
struct I8Layout {
  static constexpr int kStripBytes = MROWS * kI8BK;
  static constexpr int kStageBytes = 2 * kStripBytes + 2 * kI8AtomBytes;
  static constexpr int kStages = MROWS > 64 ? 3 : MROWS > 32 ? 4 : 5;
  static constexpr int kPipeBytes = kStages * kStageBytes;
  static constexpr int kTileBytes = MROWS * kTcTileStride * 4;  // the epilogue's f32 tile; aliases the ring
  static constexpr int kBarOffset = kPipeBytes;
  static constexpr int kScaleOffset = kBarOffset + 128;
  static constexpr int kSmemBytes = kScaleOffset + kTcBN * 4 + 1024;  // slack to align to 1024
  static_assert(kPipeBytes >= kTileBytes, "the tile aliases the ring");
  static_assert(kStripBytes % 1024 == 0 && kStageBytes % 1024 == 0, "operand tiles start on 1024-byte boundaries");
  static_assert(16 * kStages <= 96, "the barriers sit below the TMEM slot");
};

__device__ int g_i8_status = 0;  // nonzero after an mbarrier wait timed out (sticky until read)

struct I8Params {
  const float* scales;
  const float* residual;
  const float* row_scale;  // [M]: s[m]
  void* y;
  int M, K, N;
  int Kc, ks;
  int weights_const;  // codes and scales are not written by the preceding kernel: fetch them before the dependency wait
  int swiglu;
};

// ---- activations -> hi / lo planes ----------------------------------------------------------------------------------
template <typename XT>
__device__ __forceinline__ float AsBf16Value(XT v);
template <>
__device__ __forceinline__ float AsBf16Value<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <>
__device__ __forceinline__ float AsBf16Value<float>(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// One CTA per row: the row's largest magnitude, the power-of-two step s, then q = x / s (exact: a power of two) rounded
// to the nearest integer and split as q = 256 hi + lo.
template <typename XT>
__global__ void __launch_bounds__(256) QuantizeRowsI8Kernel(const XT* __restrict__ x, int8_t* __restrict__ hi,
                                                            int8_t* __restrict__ lo, float* __restrict__ row_scale, int K)
{
  GridDependencySync();
  const int m = blockIdx.x, tid = threadIdx.x;
  const XT* row = x + static_cast<size_t>(m) * K;
  constexpr int kVec = 16 / sizeof(XT);  // elements per 16-byte load
  const bool vec = (reinterpret_cast<uintptr_t>(row) & 15) == 0 && K % kVec == 0;
  float amax = 0.f;
  bool bad = false;
  auto see = [&](float v) {
    const float a = fabsf(v);
    bad = bad || !(a <= 3.4e38f);
    amax = fmaxf(amax, a);
  };
  if (vec) {
    for (int i = tid * kVec; i < K; i += 256 * kVec) {
      const uint4 u = *reinterpret_cast<const uint4*>(row + i);
      const XT* e = reinterpret_cast<const XT*>(&u);
#pragma unroll
      for (int j = 0; j < kVec; ++j) see(AsBf16Value<XT>(e[j]));
    }
  } else {
    for (int i = tid; i < K; i += 256) see(AsBf16Value<XT>(row[i]));
  }
  __shared__ float s_max[8];
  __shared__ int s_bad[8];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const int any_bad = __any_sync(0xffffffffu, bad);
  if ((tid & 31) == 0) {
    s_max[tid >> 5] = amax;
    s_bad[tid >> 5] = any_bad;
  }
  __syncthreads();
  amax = s_max[0];
  int row_bad = s_bad[0];
#pragma unroll
  for (int w = 1; w < 8; ++w) {
    amax = fmaxf(amax, s_max[w]);
    row_bad |= s_bad[w];
  }
  float step;
  const float inv = I8RowInvStep(amax, row_bad != 0, &step);
  if (tid == 0) row_scale[m] = step;
  int8_t* hrow = hi + static_cast<size_t>(m) * K;
  int8_t* lrow = lo + static_cast<size_t>(m) * K;
  auto split = [&](float v, int8_t& h, int8_t& l) {
    int hq, lq;
    I8Split(v, inv, hq, lq);
    h = static_cast<int8_t>(hq);
    l = static_cast<int8_t>(lq);
  };
  if (vec) {
    for (int i = tid * kVec; i < K; i += 256 * kVec) {
      const uint4 u = *reinterpret_cast<const uint4*>(row + i);
      const XT* el = reinterpret_cast<const XT*>(&u);
      alignas(8) int8_t h[kVec], l[kVec];
#pragma unroll
      for (int j = 0; j < kVec; ++j) split(AsBf16Value<XT>(el[j]), h[j], l[j]);
      if constexpr (kVec == 8) {
        *reinterpret_cast<uint2*>(hrow + i) = *reinterpret_cast<const uint2*>(h);
        *reinterpret_cast<uint2*>(lrow + i) = *reinterpret_cast<const uint2*>(l);
      } else {
        *reinterpret_cast<uint32_t*>(hrow + i) = *reinterpret_cast<const uint32_t*>(h);
        *reinterpret_cast<uint32_t*>(lrow + i) = *reinterpret_cast<const uint32_t*>(l);
      }
    }
  } else {
    for (int i = tid; i < K; i += 256) split(AsBf16Value<XT>(row[i]), hrow[i], lrow[i]);
  }
}

// ---- the projection --------------------------------------------------------------------------------------------------
// kind::i8 instruction descriptor: s32 accumulator, signed 8-bit A and B, A K-major, B MN-major, M = 128, N = 256.
__host__ __device__ constexpr uint32_t InstrDescI8()
{
  return (2u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | (static_cast<uint32_t>(kTcBN >> 3) << 17) | (8u << 24);
}
__device__ __forceinline__ void TcMmaI8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void MbarExpectTx(uint32_t bar, uint32_t bytes)
{
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
// One box of a two-dimensional tensor map into shared memory; (x, y) = (innermost coordinate, row).  x times the element
// size is always a multiple of 128 bytes here.
__device__ __forceinline__ void TmaLoad2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar, uint64_t policy)
{
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;\n" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar), "l"(policy)
      : "memory");
}

template <int MROWS, typename YT>
__global__ void __launch_bounds__(kI8Threads, 1)
    Int8GemmI8Kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_hi,
                     const __grid_constant__ CUtensorMap map_lo, I8Params p)
{
  using L = I8Layout<MROWS>;
  constexpr int kI8Stages = L::kStages, kI8StripBytes = L::kStripBytes, kI8StageBytes = L::kStageBytes;
  constexpr int kI8BarOffset = L::kBarOffset, kI8ScaleOffset = L::kScaleOffset;
  constexpr bool kStacked = MROWS <= 64;  // both planes in one accumulator's lanes (see the MMA thread)
  extern __shared__ unsigned char smem_raw[];
  const uint32_t smem_base = (SmemAddr(smem_raw) + 1023u) & ~1023u;  // the swizzle is a function of address bits 4..9
  unsigned char* smem = smem_raw + (smem_base - SmemAddr(smem_raw));
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int col0 = blockIdx.x * kTcBN;
  const int kb0 = blockIdx.y * p.Kc;
  const int ke = min(p.K, kb0 + p.Kc);
  const int nblocks = ke > kb0 ? (ke - kb0 + kI8BK - 1) / kI8BK : 0;
  // full[i]: the four boxes of the block in stage i have landed; empty[i]: its MMAs have completed.
  const uint32_t full0 = smem_base + kI8BarOffset, empty0 = full0 + 8 * kI8Stages;
  const uint32_t tmem_slot_addr = smem_base + kI8BarOffset + 96;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + kI8BarOffset + 96);
  volatile uint32_t* abort_word = tmem_slot + 1;  // raised by the first wait that gives up
  float* s_scales = reinterpret_cast<float*>(smem + kI8ScaleOffset);

  if (tid == 0) {
    *abort_word = 0u;
    for (int i = 0; i < kI8Stages; ++i) {
      MbarInit(full0 + 8 * i, 1);
      MbarInit(empty0 + 8 * i, 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(tmem_slot_addr), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  bool ok = true;
  if (warp == kI8Workers / 32 + 1) {
    // The producer.  Constant weights are requested before the dependency wait (the coldest loads of the launch travel
    // while the predecessor drains); the activation planes, which the preceding kernel wrote, after it.
    if (lane == 0) {
      uint64_t stream_policy, keep_policy;
      asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;\n" : "=l"(stream_policy));
      asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;\n" : "=l"(keep_policy));
      auto load_w = [&](int b) {
        const int s = b % kI8Stages;
        const uint32_t dst = smem_base + s * kI8StageBytes + 2 * kI8StripBytes;
        TmaLoad2d(dst, &map_w, col0, kb0 + b * kI8BK, full0 + 8 * s, stream_policy);
        TmaLoad2d(dst + kI8AtomBytes, &map_w, col0 + 128, kb0 + b * kI8BK, full0 + 8 * s, stream_policy);
      };
      auto load_x = [&](int b) {
        const int s = b % kI8Stages;
        const uint32_t dst = smem_base + s * kI8StageBytes;
        TmaLoad2d(dst, &map_hi, kb0 + b * kI8BK, 0, full0 + 8 * s, keep_policy);
        TmaLoad2d(dst + kI8StripBytes, &map_lo, kb0 + b * kI8BK, 0, full0 + 8 * s, keep_policy);
      };
      const int first = min(nblocks, kI8Stages);
      if (!p.weights_const) GridDependencySync();
      for (int b = 0; b < first; ++b) {
        MbarExpectTx(full0 + 8 * (b % kI8Stages), kI8StageBytes);
        load_w(b);
      }
      if (p.weights_const) GridDependencySync();
      for (int b = 0; b < first; ++b) load_x(b);
      for (int b = first; b < nblocks; ++b) {
        const int s = b % kI8Stages;
        ok = MbarWait(empty0 + 8 * s, ((b / kI8Stages) - 1) & 1, abort_word) && ok;
        MbarExpectTx(full0 + 8 * s, kI8StageBytes);
        load_w(b);
        load_x(b);
      }
    }
    __syncwarp();
  } else if (warp == kI8Workers / 32) {
    // The MMA thread: per block, 4 K-steps of 32.  65 to 128 rows: the hi plane into accumulator columns 0..255, the lo
    // plane into 256..511, both against the same codes.  Up to 64 rows: the stage's two strips, which lie one after the
    // other, ARE one 128-row A operand (lanes [0, MROWS) the hi plane, [MROWS, 2 MROWS) the lo plane), so one MMA per
    // K-step serves both planes and the codes are fetched from shared memory once.
    if (lane == 0) {
      constexpr uint32_t idesc = InstrDescI8();
      const uint64_t hi0 = SmemDesc(smem_base, 16, 1024), lo0 = SmemDesc(smem_base + kI8StripBytes, 16, 1024);
      const uint64_t w0 = SmemDesc(smem_base + 2 * kI8StripBytes, kI8AtomBytes, 1024);
      for (int b = 0; b < nblocks; ++b) {
        const int s = b % kI8Stages;
        ok = MbarWait(full0 + 8 * s, (b / kI8Stages) & 1, abort_word) && ok;
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        const uint64_t stage = static_cast<uint64_t>((s * kI8StageBytes) >> 4);
#pragma unroll
        for (int ks = 0; ks < kI8BK / 32; ++ks) {
          const uint32_t acc = (b > 0 || ks > 0) ? 1u : 0u;
          const uint64_t wd = w0 + stage + static_cast<uint64_t>((ks * 32 * 128) >> 4);
          TcMmaI8(tmem_base, hi0 + stage + static_cast<uint64_t>((ks * 32) >> 4), wd, idesc, acc);
          if constexpr (!kStacked) TcMmaI8(tmem_base + kTcBN, lo0 + stage + static_cast<uint64_t>((ks * 32) >> 4), wd, idesc, acc);
        }
        TcCommit(empty0 + 8 * s);
      }
      // The last commit covers every MMA before it.
      if (nblocks > 0) ok = MbarWait(empty0 + 8 * ((nblocks - 1) % kI8Stages), ((nblocks - 1) / kI8Stages) & 1, abort_word) && ok;
    }
    __syncwarp();
  } else {
    if (!p.weights_const) GridDependencySync();
    if (tid < kTcBN) s_scales[tid] = (p.scales != nullptr && col0 + tid < p.N) ? __ldg(p.scales + col0 + tid) : 1.f;
    if (p.weights_const) GridDependencySync();  // the residual and the row scales belong to earlier kernels
  }
  if (!ok) atomicExch(&g_i8_status, 1);
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();  // every MMA has completed and every box has landed; the ring's space is free
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");

  // Epilogue: warp w reads TMEM lanes 32 (w % 4) .. + 31 (lane = activation row) and the quarter w / 4 of the columns,
  // 32 at a time from both accumulators, and writes (256 hi + lo) * s[row] as f32 to the row-major tile.
  cg::cluster_group cluster = cg::this_cluster();
  const unsigned nranks = cluster.num_blocks();
  const bool worker = warp < kI8Workers / 32;
  float* tile = reinterpret_cast<float*>(smem);
  const EpilogueOut out{p.residual, p.y, p.M, p.N, p.swiglu};
  const bool vec_ok = (reinterpret_cast<uintptr_t>(p.y) & 15) == 0 && (reinterpret_cast<uintptr_t>(p.residual) & 15) == 0;
  if constexpr (kStacked) {
    // Lanes [0, MROWS) hold the hi sums of rows 0.., lanes [MROWS, 2 MROWS) the lo sums of the same rows: the warps on
    // the lo lanes write lo * s[row] to the tile first, then the warps on the hi lanes add 256 hi * s[row] (s is a power
    // of two, so this rounds exactly like (256 hi + lo) * s).
    constexpr int kQuarters = MROWS / 32;  // lane quarters per plane
    const int lg = warp & 3, wq = warp >> 2;
    const int m = (lg % kQuarters) * 32 + lane;
    const float rs = (worker && m < p.M) ? __ldg(p.row_scale + m) : 0.f;
#pragma unroll
    for (int pass = 0; pass < 2; ++pass) {
      const bool mine = worker && (pass == 0 ? (lg >= kQuarters && lg < 2 * kQuarters) : lg < kQuarters);
      if (mine) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t a[32];
          if (nblocks > 0) {
            TcLd32(tmem_base + (static_cast<uint32_t>(lg * 32) << 16) + wq * 64 + h * 32, a);
            asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
          } else {
#pragma unroll
            for (int e = 0; e < 32; ++e) a[e] = 0u;
          }
          float4* dst = reinterpret_cast<float4*>(tile + m * kTcTileStride + wq * 64 + h * 32);
          const float w = pass == 0 ? rs : 256.f * rs;
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            float4 v = pass == 0 ? make_float4(0.f, 0.f, 0.f, 0.f) : dst[c];
            v.x = fmaf(static_cast<float>(static_cast<int>(a[4 * c])), w, v.x);
            v.y = fmaf(static_cast<float>(static_cast<int>(a[4 * c + 1])), w, v.y);
            v.z = fmaf(static_cast<float>(static_cast<int>(a[4 * c + 2])), w, v.z);
            v.w = fmaf(static_cast<float>(static_cast<int>(a[4 * c + 3])), w, v.w);
            dst[c] = v;
          }
        }
      }
      if (pass == 0) __syncthreads();
    }
  } else if (worker && (warp & 3) * 32 < MROWS) {
    const int lg = warp & 3, wq = warp >> 2;
    const int m = lg * 32 + lane;
    const float rs = m < p.M ? __ldg(p.row_scale + m) : 0.f;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      uint32_t a[32], b[32];
      if (nblocks > 0) {
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(lg * 32) << 16) + wq * 64 + h * 32;
        TcLd32(taddr, a);
        TcLd32(taddr + kTcBN, b);
        asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
      } else {
#pragma unroll
        for (int e = 0; e < 32; ++e) a[e] = b[e] = 0u;
      }
      float4* dst = reinterpret_cast<float4*>(tile + m * kTcTileStride + wq * 64 + h * 32);
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        float4 v;
        v.x = fmaf(static_cast<float>(static_cast<int>(a[4 * c])), 256.f, static_cast<float>(static_cast<int>(b[4 * c]))) * rs;
        v.y = fmaf(static_cast<float>(static_cast<int>(a[4 * c + 1])), 256.f, static_cast<float>(static_cast<int>(b[4 * c + 1]))) * rs;
        v.z = fmaf(static_cast<float>(static_cast<int>(a[4 * c + 2])), 256.f, static_cast<float>(static_cast<int>(b[4 * c + 2]))) * rs;
        v.w = fmaf(static_cast<float>(static_cast<int>(a[4 * c + 3])), 256.f, static_cast<float>(static_cast<int>(b[4 * c + 3]))) * rs;
        dst[c] = v;
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  if (nranks == 1) {
    __syncthreads();
    if (worker) EpilogueRows<MROWS, YT>(tile, s_scales, out, col0, 0, tid, vec_ok);
    __syncthreads();
  } else {
    cluster.sync();
    if (worker) EpilogueCluster<YT>(cluster, tile, s_scales, out, col0, tid);
    cluster.sync();  // no CTA leaves while a peer may still read its tile
  }
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

// ---- host -----------------------------------------------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn EncodeTiled()
{
  static EncodeTiledFn fn = [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult res;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &res) != cudaSuccess || res != cudaDriverEntryPointSuccess) {
      cudaGetLastError();
      ptr = nullptr;
    }
    return reinterpret_cast<EncodeTiledFn>(ptr);
  }();
  return fn;
}

// A [rows][inner] byte matrix with rows `pitch` bytes apart, read in boxes of 128 bytes x box_rows rows, 128-byte
// swizzle, zeros outside.
bool ByteMatrixMap(CUtensorMap* map, const void* base, uint64_t inner, uint64_t rows, uint64_t pitch, uint32_t box_rows)
{
  EncodeTiledFn encode = EncodeTiled();
  if (encode == nullptr) return false;
  const cuuint64_t dims[2] = {inner, rows};
  const cuuint64_t strides[1] = {pitch};
  const cuuint32_t box[2] = {128, box_rows};
  const cuuint32_t elem[2] = {1, 1};
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, elem,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int g_i8_slots[kMaxDevices][9];  // resident CTAs when launched as clusters of ks (one CTA per SM whatever the row class)

void FillI8Slots(int device)
{
  for (int ks = 1; ks <= 8; ++ks) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(148, ks, 1);
    cfg.blockDim = dim3(kI8Threads, 1, 1);
    cfg.dynamicSmemBytes = I8Layout<128>::kSmemBytes;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = ks;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, Int8GemmI8Kernel<128, float>, &cfg) != cudaSuccess || clusters <= 0) {
      cudaGetLastError();
      clusters = (ks <= 2 ? 148 : ks <= 4 ? 128 : 112) / ks;  // a cautious guess when the query is not available
    }
    g_i8_slots[device][ks] = clusters * ks;
  }
}

cudaError_t PrepareI8()
{
  static OncePerDevice once;
  return once.Run([](int device) {
    cudaError_t e = cudaSuccess;
#define TLALOC_I8_OPT_IN(MROWS, YT)                                                                                     \
  if (e == cudaSuccess)                                                                                                 \
    e = cudaFuncSetAttribute(Int8GemmI8Kernel<MROWS, YT>, cudaFuncAttributeMaxDynamicSharedMemorySize, I8Layout<MROWS>::kSmemBytes)
    TLALOC_I8_OPT_IN(32, float);
    TLALOC_I8_OPT_IN(32, __nv_bfloat16);
    TLALOC_I8_OPT_IN(64, float);
    TLALOC_I8_OPT_IN(64, __nv_bfloat16);
    TLALOC_I8_OPT_IN(128, float);
    TLALOC_I8_OPT_IN(128, __nv_bfloat16);
#undef TLALOC_I8_OPT_IN
    if (e == cudaSuccess) FillI8Slots(device);
    return e;
  });
}

// K slices (1..8): the lowest modelled time in units of one 128-row block of one CTA,
//   waves(ks) * (blocks per slice + fixed cost of a CTA [+ cost of the cluster reduction]).
// $TLALOC_B200_GEMM_KS overrides.
int ChooseI8Slices(int k, int n)
{
  static const int forced = [] {
    const char* e = std::getenv("TLALOC_B200_GEMM_KS");
    return e != nullptr ? std::atoi(e) : 0;
  }();
  if (forced >= 1 && forced <= 8) return forced;
  const int tiles = (n + kTcBN - 1) / kTcBN;
  const int nb = (k + kI8BK - 1) / kI8BK;
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) device = 0;
  int best = 1;
  double best_cost = 1e30;
  for (int ks = 1; ks <= 8; ++ks) {
    if (ks > 1 && nb / ks < 2) break;
    const int slots = g_i8_slots[device][ks] > 0 ? g_i8_slots[device][ks] : 148 / ks * ks;
    const int waves = (tiles * ks + slots - 1) / slots;
    const double per_cta = (nb + ks - 1) / ks + 6.0 + (ks > 1 ? 5.0 + 1.0 * ks : 0.0);
    const double cost = waves * per_cta;
    if (cost < best_cost * 0.97) {
      best_cost = cost;
      best = ks;
    }
  }
  return best;
}

template <int MROWS, typename YT>
cudaError_t LaunchI8(const CUtensorMap& mw, const CUtensorMap& mh, const CUtensorMap& ml, const I8Params& p, cudaStream_t stream)
{
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((p.N + kTcBN - 1) / kTcBN, p.ks, 1);
  cfg.blockDim = dim3(kI8Threads, 1, 1);
  cfg.dynamicSmemBytes = I8Layout<MROWS>::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  cfg.numAttrs = ChainAttributes(attr, p.ks);
  cfg.attrs = attr;
  return cudaLaunchKernelEx(&cfg, Int8GemmI8Kernel<MROWS, YT>, mw, mh, ml, p);
}

template <typename YT>
cudaError_t LaunchI8Rows(const CUtensorMap& mw, const CUtensorMap& mh, const CUtensorMap& ml, const I8Params& p, cudaStream_t stream)
{
  if (p.M <= 32) return LaunchI8<32, YT>(mw, mh, ml, p, stream);
  if (p.M <= 64) return LaunchI8<64, YT>(mw, mh, ml, p, stream);
  return LaunchI8<128, YT>(mw, mh, ml, p, stream);
}

}  // namespace

// Resolves the driver's tensor-map encoder; called from kernel set-up so that no launch has to do it inside a capture.
bool TensorMapEncoderReady() { return EncodeTiled() != nullptr; }

// A [positions][kv_heads][head_dim] pool of 2-byte (bf16) or 1-byte (f8) elements, read in boxes of 16 positions of one
// head: 64 bf16 channels under the 128-byte swizzle, or a whole row of D bytes under the swizzle of that width.
bool EncodeKvPoolMap(::CUtensorMap_st* map, const void* base, int head_dim, int kv_heads, unsigned long long positions, int elem_bytes)
{
  EncodeTiledFn encode = EncodeTiled();
  if (encode == nullptr || (elem_bytes != 1 && elem_bytes != 2)) return false;
  const cuuint64_t row = static_cast<cuuint64_t>(head_dim) * elem_bytes;
  const cuuint64_t dims[3] = {static_cast<cuuint64_t>(head_dim), static_cast<cuuint64_t>(kv_heads), positions};
  const cuuint64_t strides[2] = {row, row * kv_heads};
  const cuuint32_t box[3] = {elem_bytes == 2 ? 64u : static_cast<cuuint32_t>(head_dim), 1, 16};
  const cuuint32_t elem[3] = {1, 1, 1};
  const bool wide = elem_bytes == 2 || head_dim >= 128;  // the box's rows are 128 bytes (else 64)
  return encode(map, elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims,
                strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, wide ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

cudaError_t PrepareInt8GemmI8Kernels()
{
  EncodeTiled();  // resolves the driver entry point now rather than inside a later stream capture
  return PrepareI8();
}

size_t Int8GemmI8ScratchBytes(int m, int k) { return 2 * static_cast<size_t>(m) * k + 4 * static_cast<size_t>(m); }

bool Int8GemmI8Applies(const void* codes, int m, int k, int n)
{
  static const bool enabled = [] {
    const char* v = std::getenv("TLALOC_B200_GEMM_I8");
    return v == nullptr || std::atoi(v) != 0;
  }();
  return enabled && m >= 1 && m <= 128 && k % 16 == 0 && n % 16 == 0 && Aligned16(codes) && EncodeTiled() != nullptr;
}

// Rows [0, m), m <= 128, of the projection on the int8 tensor-core kernel.  scratch (16-byte aligned,
// Int8GemmI8ScratchBytes(m, k) bytes) receives the activation planes and the row steps.
cudaError_t LaunchInt8GemmI8(const void* x, int x_dtype, const int8_t* codes, const float* scales, const float* residual,
                             void* y, int y_dtype, void* scratch, int m, int k, int n, cudaStream_t st, int* launches,
                             bool weights_const, bool swiglu, bool have_planes)
{
  cudaError_t e = PrepareI8();
  if (e != cudaSuccess) return e;
  int8_t* hi = static_cast<int8_t*>(scratch);
  int8_t* lo = hi + static_cast<size_t>(m) * k;
  float* row_scale = reinterpret_cast<float*>(lo + static_cast<size_t>(m) * k);
  if (!have_planes) {
    e = LaunchQuantizeRowsI8(x, x_dtype, scratch, m, k, st);
    if (e != cudaSuccess) return e;
    ++*launches;
  }
  CUtensorMap mw, mh, ml;
  const uint32_t strip_rows = m <= 32 ? 32 : m <= 64 ? 64 : 128;  // the row class of the launch: I8Layout<MROWS>
  if (!ByteMatrixMap(&mw, codes, static_cast<uint64_t>(n), static_cast<uint64_t>(k), static_cast<uint64_t>(n), 128) ||
      !ByteMatrixMap(&mh, hi, static_cast<uint64_t>(k), static_cast<uint64_t>(m), static_cast<uint64_t>(k), strip_rows) ||
      !ByteMatrixMap(&ml, lo, static_cast<uint64_t>(k), static_cast<uint64_t>(m), static_cast<uint64_t>(k), strip_rows)) {
    return cudaErrorInvalidValue;
  }
  I8Params p;
  p.scales = scales;
  p.residual = residual;
  p.row_scale = row_scale;
  p.y = y;
  p.M = m;
  p.K = k;
  p.N = n;
  p.ks = ChooseI8Slices(k, n);
  const int nb = (k + kI8BK - 1) / kI8BK;
  p.Kc = (nb + p.ks - 1) / p.ks * kI8BK;
  p.weights_const = weights_const ? 1 : 0;
  p.swiglu = swiglu ? 1 : 0;
  e = y_dtype == TLALOC_B200_F32 ? LaunchI8Rows<float>(mw, mh, ml, p, st) : LaunchI8Rows<__nv_bfloat16>(mw, mh, ml, p, st);
  if (e != cudaSuccess) return e;
  ++*launches;
  return cudaSuccess;
}

cudaError_t LaunchQuantizeRowsI8(const void* x, int x_dtype, void* planes, int m, int k, cudaStream_t st)
{
  int8_t* hi = static_cast<int8_t*>(planes);
  int8_t* lo = hi + static_cast<size_t>(m) * k;
  float* row_scale = reinterpret_cast<float*>(lo + static_cast<size_t>(m) * k);
  return x_dtype == TLALOC_B200_F32
             ? LaunchChained(QuantizeRowsI8Kernel<float>, static_cast<unsigned>(m), 256, 0, st, static_cast<const float*>(x), hi, lo, row_scale, k)
             : LaunchChained(QuantizeRowsI8Kernel<__nv_bfloat16>, static_cast<unsigned>(m), 256, 0, st,
                             static_cast<const __nv_bfloat16*>(x), hi, lo, row_scale, k);
}

int ReadI8Status()
{
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_i8_status, sizeof(int)) != cudaSuccess) return -1;
  if (v != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_i8_status, &zero, sizeof(int));
  }
  return v;
}

}  // namespace tlaloc_b200
