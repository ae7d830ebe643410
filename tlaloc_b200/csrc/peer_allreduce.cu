// Sum all-reduce of a tensor-parallel partial result over NVLink peer memory (sm_100a).
//
// What it stands in for: the reference expresses the sum after the row-parallel projections (o_proj, down_proj) as
// one `stablehlo.all_reduce` with an add region over the replica group
// (stablehlo/src/commonMain/kotlin/io/tlaloc/stablehlo/StablehloEmitter.kt:3048-3072) and leaves the transport to
// XLA.  Here every rank's buffer is mapped into every other rank's address space (CUDA IPC), and ONE kernel per
// rank does the whole exchange in place:
//
//   1. arrive: tell every peer "my partial is written" (a release store of the epoch into the peer's flag word),
//      wait until every peer has told me the same;
//   2. reduce-scatter by plain peer loads: rank r owns the r-th slice; it loads that slice from every rank's
//      buffer (volatile 16-byte loads, 2*world in flight per thread), adds them IN RANK ORDER (so every rank holds
//      bit-identical sums whatever the arrival order) and
//   3. all-gather by peer stores: writes the reduced slice back into the same slice of every rank's buffer.
//      Nobody else reads or writes slice r of any buffer during the exchange, which is what makes in-place safe;
//   4. depart: the last CTA to finish tells every peer "my loads and stores are done" and waits for theirs, so that
//      when the kernel completes the local buffer holds the full sum and no peer still reads the partial.
//
// Every wait is bounded by the global nanosecond timer; a wait that runs out records a code in the state words and
// the kernel returns (later launches then skip their waits), so a lost rank leaves the context usable and the host
// reads the status.  No multimem, no TMA, no cluster multicast: plain loads and stores on peer pointers only.
#include <cstring>

#include <cooperative_groups.h>

#include "common.cuh"

namespace tlaloc_b200 {
namespace {

constexpr int kMaxRanks = TLALOC_B200_MAX_PEERS;
constexpr int kThreads = 512;
constexpr unsigned long long kDefaultWaitNs = 20ull * 1000ull * 1000ull * 1000ull;  // 20 s: a rank may still be loading weights

struct PeerTable
{
  float* data[kMaxRanks];      // this all-reduce's buffer on each rank (mapped here)
  uint32_t* flags[kMaxRanks];  // [2][world] words on each rank: flags[q][phase * world + r] is written by rank r
};

// Flag words are written and polled with relaxed system-scope accesses; ordering comes from one system-scope fence on
// the signalling side (cumulative over the CTA's earlier writes through the barrier before it) and, on the waiting
// side, from reading the payload only with loads that bypass L1.
__device__ __forceinline__ void StoreFlag(uint32_t* p, uint32_t v)
{
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t LoadFlag(const uint32_t* p)
{
  uint32_t v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float4 LoadPeer(const float* p)
{
  float4 v;
  asm volatile("ld.volatile.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ unsigned long long NowNs()
{
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Thread `q` (< world) waits until rank q's flag of this phase reaches `epoch`.  Returns false when time ran out.
__device__ __forceinline__ bool WaitFlag(const uint32_t* flag, uint32_t epoch, unsigned long long limit_ns)
{
  if (static_cast<int32_t>(LoadFlag(flag) - epoch) >= 0) return true;
  const unsigned long long t0 = NowNs();
  for (;;) {
    for (int i = 0; i < 64; ++i)
      if (static_cast<int32_t>(LoadFlag(flag) - epoch) >= 0) return true;
    if (NowNs() - t0 > limit_ns) return false;
    __nanosleep(200);
  }
}
// The wait limit: state[3] microseconds when the caller set it, else 20 s.
__device__ __forceinline__ unsigned long long WaitLimitNs(const uint32_t* state)
{
  const uint32_t us = reinterpret_cast<const volatile uint32_t*>(state)[3];
  return us != 0 ? 1000ull * us : kDefaultWaitNs;
}

// state[0] = epoch of the last finished all-reduce, state[1] = CTAs finished in this launch, state[2] = status
// (0 ok, else 1 + 16 * phase + the rank that never arrived), state[3] = wait limit in microseconds (0 = 20 s).
template <int W>
__global__ void __launch_bounds__(kThreads, 1) PeerAllReduceKernel(PeerTable t, uint32_t* state, int rank, int world_rt, size_t n4)
{
  GridDependencySync();
  const int world = W > 0 ? W : world_rt;
  __shared__ uint32_t s_epoch, s_last, s_dead;
  const int tid = threadIdx.x;
  if (tid == 0) {
    s_epoch = *reinterpret_cast<volatile uint32_t*>(state) + 1u;
    s_dead = reinterpret_cast<volatile uint32_t*>(state)[2];
    s_last = 0;
  }
  __syncthreads();
  const uint32_t epoch = s_epoch;
  const bool dead = s_dead != 0;
  const unsigned long long limit_ns = WaitLimitNs(state);

  // 1. arrive.  The producing kernel has completed (stream order), so its writes are already in this GPU's L2, which
  // is where a peer's loads are served from: the flag needs no fence of its own.
  if (blockIdx.x == 0 && tid < world) StoreFlag(t.flags[tid] + rank, epoch);
  if (!dead && tid < world) {
    if (!WaitFlag(t.flags[rank] + tid, epoch, limit_ns)) atomicCAS(state + 2, 0u, 1u + tid);
  }
  __syncthreads();

  // 2 + 3. my slice, in units of float4.
  const size_t lo = n4 * rank / world, hi = n4 * (rank + 1) / world;
  for (size_t i = lo + static_cast<size_t>(blockIdx.x) * kThreads + tid; i < hi; i += static_cast<size_t>(gridDim.x) * kThreads) {
    float4 v[kMaxRanks];
#pragma unroll
    for (int q = 0; q < kMaxRanks; ++q)
      if (q < world) v[q] = LoadPeer(t.data[q] + 4 * i);
    float4 s = v[0];
#pragma unroll
    for (int q = 1; q < kMaxRanks; ++q)
      if (q < world) { s.x += v[q].x; s.y += v[q].y; s.z += v[q].z; s.w += v[q].w; }
#pragma unroll
    for (int q = 0; q < kMaxRanks; ++q)
      if (q < world) *reinterpret_cast<float4*>(t.data[q] + 4 * i) = s;
  }

  // 4. depart.  Release chain: every thread's peer stores -> CTA barrier -> thread 0's device-scope fence and
  // counter increment -> the last CTA observes the full count -> one system-scope fence -> the flags.
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    s_last = atomicAdd(state + 1, 1u) == gridDim.x - 1 ? 1u : 0u;
    __threadfence();
  }
  __syncthreads();
  if (!s_last) return;
  if (tid < world) {
    __threadfence_system();
    StoreFlag(t.flags[tid] + world + rank, epoch);
    if (!dead && !WaitFlag(t.flags[rank] + world + tid, epoch, limit_ns)) atomicCAS(state + 2, 0u, 17u + tid);
  }
  __syncthreads();
  if (tid == 0) {
    state[1] = 0;
    state[0] = epoch;
  }
}

// The same exchange with the RMSNorm that follows it in the decode step folded in.  The values are a [rows, cols]
// matrix and rank r owns rows [r * rows / world, (r + 1) * rows / world): one CTA per row, the whole reduced row in
// registers (cols <= 8192), so the rank that reduces a row also normalises it and pushes BOTH the f32 sums and the
// bf16 normalised row to every peer.  Saves the norm kernel's pass over the sums and one launch per exchange.
// Arithmetic of the norm as RmsNormKernel (decode_ops.cu): sum of squares by fused multiply-adds and a block
// reduction, rsqrt in double, the two multiplies rounded separately.
struct PeerNormTable
{
  float* data[kMaxRanks];
  __nv_bfloat16* norm[kMaxRanks];
  uint32_t* flags[kMaxRanks];
};

constexpr int kNormParts = 4;  // CTAs that share a row: a cluster, so the row's sum of squares meets in shared memory
constexpr int kNormVec = 4;    // float4 per thread per row: cols <= 4 * kNormParts * kNormVec * 512

__device__ __forceinline__ float BlockMax512(float v, float* red)
{
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();  // red may still be read by the sum before
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = lane < kThreads / 32 ? red[lane] : 0.f;
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) t = fmaxf(t, __shfl_xor_sync(0xffffffffu, t, o));
  return __shfl_sync(0xffffffffu, t, 0);
}

__device__ __forceinline__ float BlockSum512(float v, float* red)
{
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();  // red may still be read from the previous row
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = lane < kThreads / 32 ? red[lane] : 0.f;
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  return __shfl_sync(0xffffffffu, t, 0);
}

// Grid (row CTAs, kNormParts), clusters (1, kNormParts, 1): blockIdx.y is the part of the row this CTA holds.
template <int W>
__global__ void __launch_bounds__(kThreads, 1)
PeerAllReduceNormKernel(PeerNormTable t, uint32_t* state, const float* gain, float eps, int rank, int world_rt, int rows, int cols,
                        float* own_rows, int planes)
{
  GridDependencySync();
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  const int world = W > 0 ? W : world_rt;
  __shared__ uint32_t s_epoch, s_last, s_dead;
  __shared__ float red[kThreads / 32];
  __shared__ float part[2];  // this CTA's share of a row's sum of squares, double-buffered over rows
  __shared__ float pmax[2];  // with planes: the largest magnitude of this CTA's share of the normalised row, likewise
  __shared__ int pbad[2];    // ... and whether it holds an infinity or a NaN
  const int tid = threadIdx.x;
  if (tid == 0) {
    s_epoch = *reinterpret_cast<volatile uint32_t*>(state) + 1u;
    s_dead = reinterpret_cast<volatile uint32_t*>(state)[2];
    s_last = 0;
  }
  __syncthreads();
  const uint32_t epoch = s_epoch;
  const bool dead = s_dead != 0;
  const unsigned long long limit_ns = WaitLimitNs(state);
  if (blockIdx.x == 0 && blockIdx.y == 0 && tid < world) StoreFlag(t.flags[tid] + rank, epoch);
  if (!dead && tid < world) {
    if (!WaitFlag(t.flags[rank] + tid, epoch, limit_ns)) atomicCAS(state + 2, 0u, 1u + tid);
  }
  __syncthreads();

  const int part4 = (cols >> 2) / kNormParts;  // float4 per part of a row
  const int c_lo = blockIdx.y * part4;
  const int r_lo = rows * rank / world, r_hi = rows * (rank + 1) / world;
  int trip = 0;
  for (int row = r_lo + blockIdx.x; row < r_hi; row += gridDim.x, ++trip) {
    const size_t base = static_cast<size_t>(row) * cols;
    float4 sum[kNormVec];
#pragma unroll
    for (int i = 0; i < kNormVec; ++i) {
      const int c = tid + i * kThreads;
      sum[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (c < part4) {
        float4 v[kMaxRanks];
#pragma unroll
        for (int q = 0; q < kMaxRanks; ++q)
          if (q < world) v[q] = LoadPeer(t.data[q] + base + 4 * (c_lo + c));
        float4 a = v[0];
        if (own_rows != nullptr) {  // the residual stream of this rank's rows comes first, then the partials in rank order
          const float4 r = *reinterpret_cast<const float4*>(own_rows + static_cast<size_t>(row - r_lo) * cols + 4 * (c_lo + c));
          a.x += r.x; a.y += r.y; a.z += r.z; a.w += r.w;
        }
#pragma unroll
        for (int q = 1; q < kMaxRanks; ++q)
          if (q < world) { a.x += v[q].x; a.y += v[q].y; a.z += v[q].z; a.w += v[q].w; }
        sum[i] = a;
      }
    }
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < kNormVec; ++i)
      ss = fmaf(sum[i].x, sum[i].x, fmaf(sum[i].y, sum[i].y, fmaf(sum[i].z, sum[i].z, fmaf(sum[i].w, sum[i].w, ss))));
    ss = BlockSum512(ss, red);
    if (tid == 0) part[trip & 1] = ss;
    cluster.sync();  // every part's share is written; the other buffer was last read a whole trip ago
    float total = 0.f;
#pragma unroll
    for (int q = 0; q < kNormParts; ++q) total += cluster.map_shared_rank(part, q)[trip & 1];  // fixed order: same bits in every part
    const float rsq = static_cast<float>(1.0 / sqrt(static_cast<double>(total / static_cast<float>(cols) + eps)));
    float amax = 0.f;
    bool bad = false;
#pragma unroll
    for (int i = 0; i < kNormVec; ++i) {
      const int c = tid + i * kThreads;
      if (c < part4) {
        const int cc = c_lo + c;
        const float4 g = gain != nullptr ? __ldg(reinterpret_cast<const float4*>(gain) + cc) : make_float4(1.f, 1.f, 1.f, 1.f);
        const float4 a = sum[i];
        float n0 = __fmul_rn(a.x, rsq), n1 = __fmul_rn(a.y, rsq), n2 = __fmul_rn(a.z, rsq), n3 = __fmul_rn(a.w, rsq);
        if (gain != nullptr) { n0 = __fmul_rn(n0, g.x); n1 = __fmul_rn(n1, g.y); n2 = __fmul_rn(n2, g.z); n3 = __fmul_rn(n3, g.w); }
        const __nv_bfloat162 lo = __floats2bfloat162_rn(n0, n1), hi = __floats2bfloat162_rn(n2, n3);
        uint2 packed;
        packed.x = *reinterpret_cast<const uint32_t*>(&lo);
        packed.y = *reinterpret_cast<const uint32_t*>(&hi);
        if (own_rows != nullptr) {
          // the sums stay here, in this rank's rows of the residual stream; only the normalised row travels
          *reinterpret_cast<float4*>(own_rows + static_cast<size_t>(row - r_lo) * cols + 4 * cc) = a;
          if (planes) {  // the bf16 values stay in registers until the row's step is known (below)
            sum[i] = make_float4(__low2float(lo), __high2float(lo), __low2float(hi), __high2float(hi));
            const float m4 = fmaxf(fmaxf(fabsf(sum[i].x), fabsf(sum[i].y)), fmaxf(fabsf(sum[i].z), fabsf(sum[i].w)));
            bad = bad || !(m4 <= 3.4e38f);
            amax = fmaxf(amax, m4);
          } else {
#pragma unroll
            for (int q = 0; q < kMaxRanks; ++q)
              if (q < world) *reinterpret_cast<uint2*>(t.norm[q] + base + 4 * cc) = packed;
          }
        } else {
#pragma unroll
          for (int q = 0; q < kMaxRanks; ++q) {
            if (q < world) {
              *reinterpret_cast<float4*>(t.data[q] + base + 4 * cc) = a;
              *reinterpret_cast<uint2*>(t.norm[q] + base + 4 * cc) = packed;
            }
          }
        }
      }
    }
    if (planes) {
      // The normalised row travels as the int8 tensor-core projection's activation planes instead of bf16: the row's
      // step needs the largest magnitude over all parts of the row, so the parts meet once more.  The receiving
      // rank's norm region then holds [rows][cols] hi bytes, [rows][cols] lo bytes and [rows] f32 steps.
      amax = BlockMax512(amax, red);
      const int cta_bad = __syncthreads_or(bad ? 1 : 0);
      if (tid == 0) {
        pmax[trip & 1] = amax;
        pbad[trip & 1] = cta_bad;
      }
      cluster.sync();
      float row_max = 0.f;
      int row_bad = 0;
#pragma unroll
      for (int q = 0; q < kNormParts; ++q) {
        row_max = fmaxf(row_max, cluster.map_shared_rank(pmax, q)[trip & 1]);
        row_bad |= cluster.map_shared_rank(pbad, q)[trip & 1];
      }
      float step;
      const float inv = I8RowInvStep(row_max, row_bad != 0, &step);
      const size_t plane_bytes = static_cast<size_t>(rows) * cols;
      if (blockIdx.y == 0 && tid < world) {
        reinterpret_cast<float*>(reinterpret_cast<char*>(t.norm[tid]) + 2 * plane_bytes)[row] = step;
      }
#pragma unroll
      for (int i = 0; i < kNormVec; ++i) {
        const int c = tid + i * kThreads;
        if (c < part4) {
          uint32_t hw, lw;
          I8Split4(sum[i].x, sum[i].y, sum[i].z, sum[i].w, inv, hw, lw);
          const size_t at = base + 4 * static_cast<size_t>(c_lo + c);
#pragma unroll
          for (int q = 0; q < kMaxRanks; ++q) {
            if (q < world) {
              char* region = reinterpret_cast<char*>(t.norm[q]);
              *reinterpret_cast<uint32_t*>(region + at) = hw;
              *reinterpret_cast<uint32_t*>(region + plane_bytes + at) = lw;
            }
          }
        }
      }
    }
  }
  cluster.sync();  // no CTA of a row's cluster leaves while another may still read its share

  __syncthreads();
  if (tid == 0) {
    __threadfence();
    s_last = atomicAdd(state + 1, 1u) == gridDim.x * gridDim.y - 1 ? 1u : 0u;
    __threadfence();
  }
  __syncthreads();
  if (!s_last) return;
  if (tid < world) {
    __threadfence_system();
    StoreFlag(t.flags[tid] + world + rank, epoch);
    if (!dead && !WaitFlag(t.flags[rank] + world + tid, epoch, limit_ns)) atomicCAS(state + 2, 0u, 17u + tid);
  }
  __syncthreads();
  if (tid == 0) {
    state[1] = 0;
    state[0] = epoch;
  }
}

// ------------------------------------------------------------------------------------------------------------
// The one-barrier form: out = residual + the sum over ranks of a partial matrix, with the following RMSNorm.
//
// Every rank reads every rank's partial (its own locally, the others over NVLink) and keeps the whole sum, added in
// rank order, in LOCAL memory: nothing is stored to a peer, so the only rendezvous is the one before the reads ("every
// partial is written").  There is no second barrier: a rank's partial buffer is next written two exchanges later (the
// caller alternates between two partial buffers), and by then every peer has passed the arrival of the exchange in
// between, which it enters only after its reads of this one have completed.  One CTA per row holds the row in
// registers (cols <= 8192): 8 ranks x 4 vectors per thread in flight, the sum, the residual add, the row's sum of
// squares, and the normalised bf16 row, all in one pass.  Per rank 7/8 of the matrix crosses NVLink inbound (as in
// the two-phase form) but one flag round trip and the all-gather's store latency are gone.
struct PeerSumTable
{
  const float* partial[kMaxRanks];
  uint32_t* flags[kMaxRanks];
};

template <int W>
__global__ void __launch_bounds__(kThreads, 1)
PeerSumRowsKernel(PeerSumTable t, uint32_t* state, const float* residual, float* out, __nv_bfloat16* norm_out, const float* gain,
                  float eps, int rank, int world_rt, int rows, int cols, int8_t* plane_hi, int8_t* plane_lo, float* plane_steps)
{
  GridDependencySync();
  const int world = W > 0 ? W : world_rt;
  __shared__ uint32_t s_epoch, s_dead;
  __shared__ float red[kThreads / 32];
  const int tid = threadIdx.x;
  if (tid == 0) {
    s_epoch = *reinterpret_cast<volatile uint32_t*>(state) + 1u;
    s_dead = reinterpret_cast<volatile uint32_t*>(state)[2];
  }
  __syncthreads();
  const uint32_t epoch = s_epoch;
  const bool dead = s_dead != 0;
  const unsigned long long limit_ns = WaitLimitNs(state);
  // arrive: my partial is written (the producing kernel has completed: stream order); every CTA then waits, on LOCAL
  // flag words, until every rank has said the same.
  if (blockIdx.x == 0 && tid < world) StoreFlag(t.flags[tid] + rank, epoch);
  if (!dead && tid < world) {
    if (!WaitFlag(t.flags[rank] + tid, epoch, limit_ns)) atomicCAS(state + 2, 0u, 1u + tid);
  }
  __syncthreads();

  const int row4 = cols >> 2;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const size_t base = static_cast<size_t>(row) * cols;
    float4 sum[kNormVec];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < kNormVec; ++i) {
      const int c = tid + i * kThreads;
      sum[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (c < row4) {
        float4 v[kMaxRanks];
#pragma unroll
        for (int q = 0; q < kMaxRanks; ++q)
          if (q < world) v[q] = LoadPeer(t.partial[q] + base + 4 * c);
        float4 a = residual != nullptr ? *reinterpret_cast<const float4*>(residual + base + 4 * c) : make_float4(0.f, 0.f, 0.f, 0.f);
        if (residual == nullptr) a = v[0];
        else { a.x += v[0].x; a.y += v[0].y; a.z += v[0].z; a.w += v[0].w; }
#pragma unroll
        for (int q = 1; q < kMaxRanks; ++q)
          if (q < world) { a.x += v[q].x; a.y += v[q].y; a.z += v[q].z; a.w += v[q].w; }
        sum[i] = a;
        *reinterpret_cast<float4*>(out + base + 4 * c) = a;
        ss = fmaf(a.x, a.x, fmaf(a.y, a.y, fmaf(a.z, a.z, fmaf(a.w, a.w, ss))));
      }
    }
    if (norm_out != nullptr) {
      float amax = 0.f;
      bool bad = false;
      const float total = BlockSum512(ss, red);
      const float rsq = static_cast<float>(1.0 / sqrt(static_cast<double>(total / static_cast<float>(cols) + eps)));
#pragma unroll
      for (int i = 0; i < kNormVec; ++i) {
        const int c = tid + i * kThreads;
        if (c < row4) {
          const float4 g = gain != nullptr ? __ldg(reinterpret_cast<const float4*>(gain) + c) : make_float4(1.f, 1.f, 1.f, 1.f);
          const float4 a = sum[i];
          float n0 = __fmul_rn(a.x, rsq), n1 = __fmul_rn(a.y, rsq), n2 = __fmul_rn(a.z, rsq), n3 = __fmul_rn(a.w, rsq);
          if (gain != nullptr) { n0 = __fmul_rn(n0, g.x); n1 = __fmul_rn(n1, g.y); n2 = __fmul_rn(n2, g.z); n3 = __fmul_rn(n3, g.w); }
          const __nv_bfloat162 lo = __floats2bfloat162_rn(n0, n1), hi = __floats2bfloat162_rn(n2, n3);
          uint2 packed;
          packed.x = *reinterpret_cast<const uint32_t*>(&lo);
          packed.y = *reinterpret_cast<const uint32_t*>(&hi);
          *reinterpret_cast<uint2*>(norm_out + base + 4 * c) = packed;
          if (plane_hi != nullptr) {  // the bf16 values, for the planes below (the f32 sums are already stored)
            sum[i] = make_float4(__low2float(lo), __high2float(lo), __low2float(hi), __high2float(hi));
            const float m4 = fmaxf(fmaxf(fabsf(sum[i].x), fabsf(sum[i].y)), fmaxf(fabsf(sum[i].z), fabsf(sum[i].w)));
            bad = bad || !(m4 <= 3.4e38f);
            amax = fmaxf(amax, m4);
          }
        }
      }
      if (plane_hi != nullptr) {
        // the normalised row also as the int8 tensor-core projection's activation planes
        amax = BlockMax512(amax, red);
        const bool row_bad = __syncthreads_or(bad ? 1 : 0) != 0;
        float step;
        const float inv = I8RowInvStep(amax, row_bad, &step);
        if (tid == 0) plane_steps[row] = step;
#pragma unroll
        for (int i = 0; i < kNormVec; ++i) {
          const int c = tid + i * kThreads;
          if (c < row4) {
            uint32_t hw, lw;
            I8Split4(sum[i].x, sum[i].y, sum[i].z, sum[i].w, inv, hw, lw);
            reinterpret_cast<uint32_t*>(plane_hi + base)[c] = hw;
            reinterpret_cast<uint32_t*>(plane_lo + base)[c] = lw;
          }
        }
      }
    }
  }
  // The last CTA to finish closes the epoch (no flags to send: nobody waits for this rank's reads).
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    if (atomicAdd(state + 1, 1u) == gridDim.x - 1) {
      state[1] = 0;
      __threadfence();
      state[0] = epoch;
    }
  }
}

}  // namespace

int LaunchPeerAllReduce(void* const* bases, size_t data_offset, size_t flag_offset, uint32_t* state, int rank, int world,
                        size_t count, cudaStream_t st)
{
  if (world < 1 || world > kMaxRanks) return Fail(kInvalid, "peer_allreduce: world %d outside [1, %d]", world, kMaxRanks);
  if (rank < 0 || rank >= world) return Fail(kInvalid, "peer_allreduce: rank %d outside [0, %d)", rank, world);
  if (!bases || !state) return Fail(kInvalid, "peer_allreduce: null base table or state");
  if (count % 4 != 0 || data_offset % 16 != 0 || flag_offset % 4 != 0)
    return Fail(kInvalid, "peer_allreduce: count %zu must be a multiple of 4 and the data offset %zu of 16 bytes", count, data_offset);
  if (count == 0 || world == 1) return kOk;
  PeerTable t{};
  for (int q = 0; q < world; ++q) {
    if (!bases[q] || reinterpret_cast<uintptr_t>(bases[q]) % 16 != 0)
      return Fail(kInvalid, "peer_allreduce: base of rank %d is null or not 16-byte aligned", q);
    t.data[q] = reinterpret_cast<float*>(static_cast<char*>(bases[q]) + data_offset);
    t.flags[q] = reinterpret_cast<uint32_t*>(static_cast<char*>(bases[q]) + flag_offset);
  }
  const size_t n4 = count / 4;
  const size_t slice = (n4 + world - 1) / world;
  int grid = static_cast<int>((slice + kThreads - 1) / kThreads);
  grid = grid < 1 ? 1 : grid > 148 ? 148 : grid;
  cudaError_t e;
  switch (world) {
    case 2: e = LaunchChained(PeerAllReduceKernel<2>, grid, kThreads, 0, st, t, state, rank, world, n4); break;
    case 4: e = LaunchChained(PeerAllReduceKernel<4>, grid, kThreads, 0, st, t, state, rank, world, n4); break;
    case 8: e = LaunchChained(PeerAllReduceKernel<8>, grid, kThreads, 0, st, t, state, rank, world, n4); break;
    default: e = LaunchChained(PeerAllReduceKernel<0>, grid, kThreads, 0, st, t, state, rank, world, n4); break;
  }
  if (e != cudaSuccess) return CudaFail("peer_allreduce launch", e);
  CountLaunches(1);
  return kOk;
}

int LaunchPeerAllReduceNorm(void* const* bases, size_t data_offset, size_t norm_offset, size_t flag_offset, uint32_t* state,
                            const float* gain, float eps, int rank, int world, int rows, int cols, float* own_rows, int planes,
                            cudaStream_t st)
{
  if (planes && own_rows == nullptr) return Fail(kInvalid, "peer_allreduce_rmsnorm: planes go with the row-distributed form only");
  if (own_rows != nullptr && !Aligned16(own_rows)) return Fail(kInvalid, "peer_reduce_rmsnorm_rows: own_rows must be 16-byte aligned");
  if (world < 2 || world > kMaxRanks) return Fail(kInvalid, "peer_allreduce_rmsnorm: world %d outside [2, %d]", world, kMaxRanks);
  if (rank < 0 || rank >= world) return Fail(kInvalid, "peer_allreduce_rmsnorm: rank %d outside [0, %d)", rank, world);
  if (!bases || !state) return Fail(kInvalid, "peer_allreduce_rmsnorm: null base table or state");
  if (rows < 1 || cols < 16 || cols % (4 * kNormParts) != 0 || cols > 4 * kNormParts * kNormVec * kThreads) {
    return Fail(kInvalid, "peer_allreduce_rmsnorm: %d x %d: rows >= 1, cols a multiple of 16 up to %d", rows, cols,
                4 * kNormParts * kNormVec * kThreads);
  }
  if (rows % world != 0) return Fail(kInvalid, "peer_allreduce_rmsnorm: %d rows do not divide over %d ranks", rows, world);
  if (data_offset % 16 != 0 || norm_offset % 16 != 0 || flag_offset % 4 != 0 || (reinterpret_cast<uintptr_t>(gain) & 15) != 0) {
    return Fail(kInvalid, "peer_allreduce_rmsnorm: offsets and the gain must be 16-byte aligned");
  }
  PeerNormTable t{};
  for (int q = 0; q < world; ++q) {
    if (!bases[q] || reinterpret_cast<uintptr_t>(bases[q]) % 16 != 0)
      return Fail(kInvalid, "peer_allreduce_rmsnorm: base of rank %d is null or not 16-byte aligned", q);
    t.data[q] = reinterpret_cast<float*>(static_cast<char*>(bases[q]) + data_offset);
    t.norm[q] = reinterpret_cast<__nv_bfloat16*>(static_cast<char*>(bases[q]) + norm_offset);
    t.flags[q] = reinterpret_cast<uint32_t*>(static_cast<char*>(bases[q]) + flag_offset);
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(rows / world < 36 ? rows / world : 36, kNormParts, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.stream = st;
  cudaLaunchAttribute attrs[2];
  cfg.numAttrs = ChainAttributes(attrs, kNormParts);
  cfg.attrs = attrs;
  cudaError_t e;
  switch (world) {
    case 2: e = cudaLaunchKernelEx(&cfg, PeerAllReduceNormKernel<2>, t, state, gain, eps, rank, world, rows, cols, own_rows, planes); break;
    case 4: e = cudaLaunchKernelEx(&cfg, PeerAllReduceNormKernel<4>, t, state, gain, eps, rank, world, rows, cols, own_rows, planes); break;
    case 8: e = cudaLaunchKernelEx(&cfg, PeerAllReduceNormKernel<8>, t, state, gain, eps, rank, world, rows, cols, own_rows, planes); break;
    default: e = cudaLaunchKernelEx(&cfg, PeerAllReduceNormKernel<0>, t, state, gain, eps, rank, world, rows, cols, own_rows, planes); break;
  }
  if (e != cudaSuccess) return CudaFail("peer_allreduce_rmsnorm launch", e);
  CountLaunches(1);
  return kOk;
}

int LaunchPeerSumRows(void* const* bases, size_t partial_offset, size_t flag_offset, uint32_t* state, const float* residual,
                      float* out, void* norm_out, const float* gain, float eps, int rank, int world, int rows, int cols,
                      void* planes, size_t planes_bytes, cudaStream_t st)
{
  const char* op = "peer_sum_rows";
  if (world < 1 || world > kMaxRanks) return Fail(kInvalid, "%s: world %d outside [1, %d]", op, world, kMaxRanks);
  if (rank < 0 || rank >= world) return Fail(kInvalid, "%s: rank %d outside [0, %d)", op, rank, world);
  if (!bases || !state || !out) return Fail(kInvalid, "%s: null base table, state or out", op);
  if (rows < 1 || cols < 4 || cols % 4 != 0 || cols > 4 * kNormVec * kThreads) {
    return Fail(kInvalid, "%s: %d x %d: rows >= 1, cols a multiple of 4 up to %d", op, rows, cols, 4 * kNormVec * kThreads);
  }
  if (partial_offset % 16 != 0 || flag_offset % 4 != 0 || !Aligned16(residual) || !Aligned16(out) || !Aligned16(norm_out) || !Aligned16(gain)) {
    return Fail(kInvalid, "%s: the partial offset, residual, out, norm_out and gain must be 16-byte aligned", op);
  }
  PeerSumTable t{};
  for (int q = 0; q < world; ++q) {
    if (!bases[q] || reinterpret_cast<uintptr_t>(bases[q]) % 16 != 0) return Fail(kInvalid, "%s: base of rank %d is null or not 16-byte aligned", op, q);
    t.partial[q] = reinterpret_cast<const float*>(static_cast<const char*>(bases[q]) + partial_offset);
    t.flags[q] = reinterpret_cast<uint32_t*>(static_cast<char*>(bases[q]) + flag_offset);
  }
  if (planes != nullptr && (norm_out == nullptr || !Aligned16(planes) || cols % 16 != 0 || planes_bytes < Int8GemmI8ScratchBytes(rows, cols))) {
    return Fail(kInvalid, "%s: planes need norm_out, 16-byte alignment, cols a multiple of 16 and %zu bytes (got %zu)", op,
                Int8GemmI8ScratchBytes(rows, cols), planes_bytes);
  }
  const int grid = rows < 148 ? rows : 148;
  __nv_bfloat16* nout = static_cast<__nv_bfloat16*>(norm_out);
  int8_t* phi = static_cast<int8_t*>(planes);
  int8_t* plo = phi != nullptr ? phi + static_cast<size_t>(rows) * cols : nullptr;
  float* pst = phi != nullptr ? reinterpret_cast<float*>(plo + static_cast<size_t>(rows) * cols) : nullptr;
  cudaError_t e;
  switch (world) {
    case 2: e = LaunchChained(PeerSumRowsKernel<2>, grid, kThreads, 0, st, t, state, residual, out, nout, gain, eps, rank, world, rows, cols, phi, plo, pst); break;
    case 4: e = LaunchChained(PeerSumRowsKernel<4>, grid, kThreads, 0, st, t, state, residual, out, nout, gain, eps, rank, world, rows, cols, phi, plo, pst); break;
    case 8: e = LaunchChained(PeerSumRowsKernel<8>, grid, kThreads, 0, st, t, state, residual, out, nout, gain, eps, rank, world, rows, cols, phi, plo, pst); break;
    default: e = LaunchChained(PeerSumRowsKernel<0>, grid, kThreads, 0, st, t, state, residual, out, nout, gain, eps, rank, world, rows, cols, phi, plo, pst); break;
  }
  if (e != cudaSuccess) return CudaFail("peer_sum_rows launch", e);
  CountLaunches(1);
  return kOk;
}

}  // namespace tlaloc_b200

using namespace tlaloc_b200;

static_assert(sizeof(cudaIpcMemHandle_t) == TLALOC_B200_IPC_HANDLE_BYTES, "the handle is shipped as 64 opaque bytes");

extern "C" int tlaloc_b200_peer_alloc(size_t bytes, void** ptr, unsigned char* handle)
{
  if (!ptr || !handle || bytes == 0) return Fail(kInvalid, "peer_alloc: null output or zero size");
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e != cudaSuccess) return CudaFail("peer_alloc cudaMalloc", e);
  e = cudaMemset(p, 0, bytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    cudaFree(p);
    return CudaFail("peer_alloc", e);
  }
  memcpy(handle, &h, sizeof(h));
  *ptr = p;
  return kOk;
}

extern "C" int tlaloc_b200_peer_open(const unsigned char* handle, void** ptr)
{
  if (!ptr || !handle) return Fail(kInvalid, "peer_open: null argument");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  cudaError_t e = cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
  return e == cudaSuccess ? kOk : CudaFail("peer_open cudaIpcOpenMemHandle", e);
}

extern "C" int tlaloc_b200_peer_close(void* ptr)
{
  cudaError_t e = cudaIpcCloseMemHandle(ptr);
  return e == cudaSuccess ? kOk : CudaFail("peer_close", e);
}

extern "C" int tlaloc_b200_peer_free(void* ptr)
{
  cudaError_t e = cudaFree(ptr);
  return e == cudaSuccess ? kOk : CudaFail("peer_free", e);
}

extern "C" int tlaloc_b200_peer_allreduce_f32(void* const* bases, size_t data_offset, size_t flag_offset, uint32_t* state,
                                              int32_t rank, int32_t world, size_t count, void* stream)
{
  return LaunchPeerAllReduce(bases, data_offset, flag_offset, state, rank, world, count, static_cast<cudaStream_t>(stream));
}

extern "C" int tlaloc_b200_peer_allreduce_rmsnorm_f32(void* const* bases, size_t data_offset, size_t norm_offset,
                                                      size_t flag_offset, uint32_t* state, const float* gain, float eps,
                                                      int32_t rank, int32_t world, int32_t rows, int32_t cols, void* stream)
{
  return LaunchPeerAllReduceNorm(bases, data_offset, norm_offset, flag_offset, state, gain, eps, rank, world, rows, cols,
                                 nullptr, 0, static_cast<cudaStream_t>(stream));
}

extern "C" int tlaloc_b200_peer_reduce_rmsnorm_rows_f32(void* const* bases, size_t data_offset, size_t norm_offset,
                                                        size_t flag_offset, uint32_t* state, float* own_rows, const float* gain,
                                                        float eps, int32_t rank, int32_t world, int32_t rows, int32_t cols,
                                                        int32_t planes, void* stream)
{
  if (!own_rows) return Fail(kInvalid, "peer_reduce_rmsnorm_rows: own_rows is null");
  return LaunchPeerAllReduceNorm(bases, data_offset, norm_offset, flag_offset, state, gain, eps, rank, world, rows, cols,
                                 own_rows, planes != 0 ? 1 : 0, static_cast<cudaStream_t>(stream));
}

extern "C" int tlaloc_b200_peer_sum_rows_f32(void* const* bases, size_t partial_offset, size_t flag_offset, uint32_t* state,
                                             const float* residual, float* out, void* norm_out, const float* gain, float eps,
                                             int32_t rank, int32_t world, int32_t rows, int32_t cols, void* planes,
                                             size_t planes_bytes, void* stream)
{
  return LaunchPeerSumRows(bases, partial_offset, flag_offset, state, residual, out, norm_out, gain, eps, rank, world, rows, cols,
                           planes, planes_bytes, static_cast<cudaStream_t>(stream));
}
