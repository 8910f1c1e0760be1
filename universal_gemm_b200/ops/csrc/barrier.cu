// Cross-rank signal barrier on symmetric counters (sm_100a, works on any CUDA GPU
// with peer access).
//
// Rank r owns uint32 slots[world].  A barrier adds 1 to slot r of every peer
// (red.release.sys over NVLink) and then waits until each of its own slots has
// reached the barrier's sequence number (a per-rank device counter that every
// launch advances, so all ranks agree on it as long as they call in the same order).  The wait is bounded: when the limit
// runs out the kernel stores UG_ERR_TIMEOUT_PEER in the status word and returns,
// so the context stays usable and the host can raise.
//
// Replaces nvshmem.barrier_all / dist.barrier around every GEMM in the reference
// (dtensor_example.py:121-124, benchmark/matmul_bench_worker.py:120-122,
// stationary_c_plan.py:571-580).
#include <cuda_runtime.h>
#include <stdint.h>

#include "ptx_sm100.cuh"
#include "ugemm_b200.h"

using namespace ugptx;

namespace {

constexpr int kBarrierThreads = 256;

__global__ void __launch_bounds__(kBarrierThreads) signal_barrier_kernel(
    const uint64_t* __restrict__ peer_slots, int world, int rank, uint32_t* seq_counter, uint32_t* status,
    uint64_t timeout_ns, uint32_t* clear_ptr, int num_clear) {
  // The barrier's sequence number lives in device memory and advances by one per launch, so a captured
  // launch can be replayed (a CUDA graph of barrier + GEMM + barrier) and still wait for the right round.
  __shared__ uint32_t s_seq;
  if (threadIdx.x == 0) s_seq = atomicAdd(seq_counter, 1u) + 1u;
  __syncthreads();
  const uint32_t seq = s_seq;
  // Plan-local words (chunk counters, piece cursor) go back to zero here, so the
  // fused kernel that follows in the stream starts from a clean slate.
  for (int i = threadIdx.x; i < num_clear; i += blockDim.x) clear_ptr[i] = 0u;

  for (int p = threadIdx.x; p < world; p += blockDim.x) {
    uint32_t* theirs = reinterpret_cast<uint32_t*>(peer_slots[p]) + rank;
    __threadfence_system();
    red_release_sys_add(theirs, 1u);
  }
  const uint32_t* mine = reinterpret_cast<const uint32_t*>(peer_slots[rank]);
  const uint64_t deadline = global_timer_ns() + timeout_ns;
  for (int p = threadIdx.x; p < world; p += blockDim.x) {
    uint32_t spins = 0;
    while (static_cast<int32_t>(ld_acquire_sys(mine + p) - seq) < 0) {
      __nanosleep(100);
      if ((++spins & 0x3fu) == 0u && global_timer_ns() > deadline) {
        atomicCAS(status, 0u, static_cast<uint32_t>(UG_ERR_TIMEOUT_PEER));
        break;
      }
    }
  }
  __threadfence_system();
}

// Point-to-point signalling for put + signal protocols: the sender's stores (stream-ordered before this
// kernel) become visible before the counter moves; the receiver's wait is bounded like the barrier's.
__global__ void signal_add_kernel(uint32_t* counter, uint32_t value) {
  __threadfence_system();
  red_release_sys_add(counter, value);
}

__global__ void signal_wait_kernel(const uint32_t* counter, uint32_t expected, uint32_t* status, uint64_t timeout_ns) {
  const uint64_t deadline = global_timer_ns() + timeout_ns;
  uint32_t spins = 0;
  while (static_cast<int32_t>(ld_acquire_sys(counter) - expected) < 0) {
    __nanosleep(100);
    if ((++spins & 0x3fu) == 0u && global_timer_ns() > deadline) {
      atomicCAS(status, 0u, static_cast<uint32_t>(UG_ERR_TIMEOUT_PEER));
      break;
    }
  }
  __threadfence_system();
}

}  // namespace

extern "C" int ug_signal_add(uint64_t counter, uint32_t value, void* stream) {
  signal_add_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(reinterpret_cast<uint32_t*>(counter), value);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int ug_signal_wait(uint64_t counter, uint32_t expected, uint64_t status, uint64_t timeout_ns, void* stream) {
  signal_wait_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(reinterpret_cast<const uint32_t*>(counter), expected,
                                                                      reinterpret_cast<uint32_t*>(status), timeout_ns);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int ug_signal_barrier(const uint64_t* peer_slots_dev, int world, int rank, uint64_t seq_counter,
                                 uint64_t status, uint64_t timeout_ns, uint64_t clear_ptr, int num_clear,
                                 void* stream) {
  if (world <= 0 || rank < 0 || rank >= world) return static_cast<int>(cudaErrorInvalidValue);
  signal_barrier_kernel<<<1, kBarrierThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      peer_slots_dev, world, rank, reinterpret_cast<uint32_t*>(seq_counter), reinterpret_cast<uint32_t*>(status), timeout_ns,
      reinterpret_cast<uint32_t*>(clear_ptr), num_clear);
  return static_cast<int>(cudaGetLastError());
}
