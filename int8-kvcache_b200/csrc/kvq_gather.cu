// Output all-gather of request-sharded decode over NVLink peer memory (kvq_peer_allgather, include/kvq_b200.h).
//
// Request sharding leaves one exchange on the path: every rank's attention output rows [T / N, Hq, D] are needed by
// all ranks (sampling, or the next layer under replicated weights). The rows are small (16 requests x 28 heads x 128
// bf16 = 114 KB per rank at 8 GPUs), so the exchange is pure latency: a library all-gather costs ~25 us per step next
// to a ~97 us attention call. Here every rank stores its rows straight into every peer's gather buffer (plain
// st.global through the NVLink peer mapping), then raises a flag in the peer's flag array, and waits for the flags
// of the rows it receives. No multimem, no bulk-async copies.
//
// Protocol (one launch per rank per step; every rank makes the same sequence of calls):
//   the step's epoch is one more than a counter in this rank's memory, which the last block of the launch to finish
//   advances, so the launch has no per-step argument and can be replayed from a CUDA graph;
//   block (p, c) copies slice c of this rank's rows to peer p's staging buffer of this epoch's parity at row offset
//   `rank`; every thread fences its stores to system scope, the block meets, and thread 0 releases
//   flag[p][rank * SLICES + c] = epoch; then the same block waits until this rank's own flag[rank][p * SLICES + c]
//   reaches epoch (peer p's slice c has landed here) and copies that slice from the staging buffer to the caller's
//   output (L1-bypassing loads: the lines were written by another GPU).
// Flags only grow, so they are never reset; a waiter that sees a later epoch passes, which is correct because the
// staging buffers alternate between steps and a rank can be at most one step ahead of the slowest rank: it cannot
// leave step k + 1 before every rank has signalled k + 1.
// Every wait is bounded (~2^31 clock cycles, about a second): on expiry the block sets *status = 1 and returns, so a
// missing peer shows up as an error code on the host, not as a hung GPU. Blocks never wait for other blocks of the
// same launch, so the grid does not have to be co-resident.
#include <algorithm>

#include "kvq_common.cuh"

namespace kvq {
namespace {

constexpr int MAX_RANKS = 8, SLICES = 8, GATHER_THREADS = 512;

struct PeerArgs {
  uint4* dst[2][MAX_RANKS];     // rank p's two staging buffers (this process's mapping of them)
  uint32_t* flags[MAX_RANKS];   // rank p's flag array, MAX_RANKS * SLICES words
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(GATHER_THREADS) peer_allgather_kernel(const uint4* __restrict__ src, int64_t n16, PeerArgs pa,
                                                                       uint4* __restrict__ out, int rank, int slices,
                                                                       uint32_t* counters, int* status) {
  __shared__ uint32_t s_epoch;
  __shared__ int s_ok;
  const int p = blockIdx.x, c = blockIdx.y, tid = threadIdx.x;
  // counters[0]: epoch of the last completed step; counters[1]: blocks of this launch that are done
  if (tid == 0) s_epoch = *reinterpret_cast<volatile uint32_t*>(counters) + 1;
  __syncthreads();
  const uint32_t epoch = s_epoch;
  const int which = epoch & 1;
  const int64_t per = (n16 + slices - 1) / slices, i0 = c * per, i1 = min(n16, i0 + per);
  uint4* dst = pa.dst[which][p] + static_cast<int64_t>(rank) * n16;
  for (int64_t i = i0 + tid; i < i1; i += GATHER_THREADS) dst[i] = src[i];
  __threadfence_system();   // this thread's stores are visible system-wide before the flag below
  __syncthreads();
  if (tid == 0) {
    st_release_sys(pa.flags[p] + rank * SLICES + c, epoch);
    // wait for slice c of peer p's rows to land in this rank's staging buffer
    const uint32_t* mine = pa.flags[rank] + p * SLICES + c;
    const long long t0 = clock64();
    bool ok = false;
    for (;;) {
      if (static_cast<int32_t>(ld_acquire_sys(mine) - epoch) >= 0) {
        ok = true;
        break;
      }
      if (clock64() - t0 > (1ll << 31)) break;
      __nanosleep(64);
    }
    if (!ok) atomicExch(status, 1);
    s_ok = ok;
  }
  __syncthreads();
  if (s_ok) {
    const uint4* got = pa.dst[which][rank] + static_cast<int64_t>(p) * n16;
    uint4* o = out + static_cast<int64_t>(p) * n16;
    for (int64_t i = i0 + tid; i < i1; i += GATHER_THREADS) o[i] = __ldcg(got + i);
  }
  // the last block to finish closes the step
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    const uint32_t nblocks = gridDim.x * gridDim.y;
    if (atomicAdd(counters + 1, 1u) == nblocks - 1) {
      counters[1] = 0;
      __threadfence();
      *reinterpret_cast<volatile uint32_t*>(counters) = epoch;
    }
  }
}

}  // namespace
}  // namespace kvq

extern "C" __attribute__((visibility("default"))) int kvq_peer_allgather(const void* src, size_t bytes_per_rank,
                                                                         void* const* stage0, void* const* stage1,
                                                                         uint32_t* const* flag_bufs, void* out, int world,
                                                                         int rank, uint32_t* counters, int* status,
                                                                         kvq_stream_t stream) {
  using namespace kvq;
  if (world < 1 || world > MAX_RANKS || rank < 0 || rank >= world) {
    set_error("peer all-gather: rank %d of %d (at most %d ranks)", rank, world, MAX_RANKS);
    return KVQ_ERR_INVALID_ARGUMENT;
  }
  if (!src || !stage0 || !stage1 || !flag_bufs || !out || !counters || !status) {
    set_error("peer all-gather: null pointer argument");
    return KVQ_ERR_INVALID_ARGUMENT;
  }
  if (bytes_per_rank == 0) return KVQ_OK;
  if (bytes_per_rank % 16 || (reinterpret_cast<uintptr_t>(src) & 15) || (reinterpret_cast<uintptr_t>(out) & 15)) {
    set_error("peer all-gather: rows must be 16-byte aligned and a multiple of 16 bytes per rank (got %zu bytes at %p -> %p)",
              bytes_per_rank, src, out);
    return KVQ_ERR_INVALID_ARGUMENT;
  }
  PeerArgs pa{};
  for (int p = 0; p < world; ++p) {
    if (!stage0[p] || !stage1[p] || !flag_bufs[p] || ((reinterpret_cast<uintptr_t>(stage0[p]) | reinterpret_cast<uintptr_t>(stage1[p])) & 15)) {
      set_error("peer all-gather: staging buffer or flag pointer of rank %d is null or misaligned", p);
      return KVQ_ERR_INVALID_ARGUMENT;
    }
    pa.dst[0][p] = static_cast<uint4*>(stage0[p]);
    pa.dst[1][p] = static_cast<uint4*>(stage1[p]);
    pa.flags[p] = flag_bufs[p];
  }
  const int64_t n16 = static_cast<int64_t>(bytes_per_rank / 16);
  // one slice per 32 KB of rows, at most SLICES: a single block moves ~100 KB in a few microseconds over NVLink
  const int slices = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(SLICES, (n16 + 2047) / 2048)));
  peer_allgather_kernel<<<dim3(world, slices), GATHER_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(src), n16, pa, static_cast<uint4*>(out), rank, slices, counters, status);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("peer all-gather launch: %s", cudaGetErrorString(e));
    return KVQ_ERR_CUDA;
  }
  return KVQ_OK;
}
