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

#include "common.cuh"

namespace tlaloc_b200 {
namespace {

constexpr int kMaxRanks = TLALOC_B200_MAX_PEERS;
constexpr int kThreads = 512;
constexpr unsigned long long kWaitNs = 20ull * 1000ull * 1000ull * 1000ull;  // 20 s: a rank may still be loading weights

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
__device__ __forceinline__ bool WaitFlag(const uint32_t* flag, uint32_t epoch)
{
  if (static_cast<int32_t>(LoadFlag(flag) - epoch) >= 0) return true;
  const unsigned long long t0 = NowNs();
  for (;;) {
    for (int i = 0; i < 64; ++i)
      if (static_cast<int32_t>(LoadFlag(flag) - epoch) >= 0) return true;
    if (NowNs() - t0 > kWaitNs) return false;
    __nanosleep(200);
  }
}

// state[0] = epoch of the last finished all-reduce, state[1] = CTAs finished in this launch, state[2] = status
// (0 ok, else 1 + 16 * phase + the rank that never arrived).
template <int W>
__global__ void __launch_bounds__(kThreads) PeerAllReduceKernel(PeerTable t, uint32_t* state, int rank, int world_rt, size_t n4)
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

  // 1. arrive.  The producing kernel has completed (stream order), so its writes are already in this GPU's L2, which
  // is where a peer's loads are served from: the flag needs no fence of its own.
  if (blockIdx.x == 0 && tid < world) StoreFlag(t.flags[tid] + rank, epoch);
  if (!dead && tid < world) {
    if (!WaitFlag(t.flags[rank] + tid, epoch)) atomicCAS(state + 2, 0u, 1u + tid);
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
    if (!dead && !WaitFlag(t.flags[rank] + world + tid, epoch)) atomicCAS(state + 2, 0u, 17u + tid);
  }
  __syncthreads();
  if (tid == 0) {
    state[1] = 0;
    state[0] = epoch;
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
