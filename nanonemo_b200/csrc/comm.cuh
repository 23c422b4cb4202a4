// Device-side building blocks of the NVLink collectives, shared by the collective kernels (comm.cu)
// and the GEMMs that fuse a collective into their prologue / epilogue (gemm_comm.cu): the table of
// peer pointers, system-scope release / acquire accesses, and the bounded cross-rank block barrier.
#pragma once
#include "common.cuh"

namespace nnbcomm {

constexpr int kMaxWorld = 16;
// Every cross-GPU wait is bounded by TIME (read from %globaltimer), 30 s unless the launcher passes another limit: long
// enough that ordinary host-side skew between ranks (a checkpoint write, a logging call on one rank) never trips it, short
// enough that a peer that has gone away ends the kernel instead of hanging the GPU. A poll-count bound can be added on top
// (the bounded-wait test uses a few thousand polls).
constexpr unsigned long long kDefaultTimeoutNs = 30ull * 1000000000ull;
// At most 256 threads (the launchers use 128 by default, see comm_threads() in comm.cu) and at most 85 registers: a collective
// block then fits on an SM BESIDE a resident GEMM or attention CTA, so a collective running on the side stream neither waits
// for a persistent GEMM to drain nor takes SMs away from it.
constexpr int kCommThreads = 256;

__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Deadline of one wait: `expired()` is called once per poll and looks at the clock every 64th time.
struct Deadline {
  unsigned long long t0, limit;
  uint32_t polls;
  __device__ __forceinline__ explicit Deadline(unsigned long long limit_ns = kDefaultTimeoutNs) : t0(globaltimer_ns()), limit(limit_ns), polls(0) {}
  __device__ __forceinline__ bool expired() { return ((++polls & 63u) == 0u) && (globaltimer_ns() - t0 > limit); }
};

struct Peers {
  void* data[kMaxWorld];
  uint32_t* flags[kMaxWorld];
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(uint32_t* p, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Cross-rank barrier among the blocks that use flag slot `slot_block` (normally blockIdx.x): signal
// every peer, then wait for every peer. Epochs only grow, so flags are never reset. Returns false if
// a wait ran out (status = {code, rank, peer, block, epoch} recorded once). Call from all threads of
// the block (needs at least `world` threads). n_slot_blocks must be the same for every kernel that shares
// the flag buffer (the launchers pass the block count the buffer was sized for, not their grid size).
__device__ __forceinline__ bool block_barrier(const Peers& P, int rank, int world, int phase, int slot_block, int n_slot_blocks,
                                              uint32_t epoch, int* status, uint32_t poll_limit = 0,
                                              unsigned long long timeout_ns = kDefaultTimeoutNs) {
  __shared__ int s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  __threadfence_system();
  __syncthreads();
  const int slot = (phase * n_slot_blocks + slot_block) * kMaxWorld;
  if ((int)threadIdx.x < world) {
    const int peer = threadIdx.x;
    st_release_sys(P.flags[peer] + slot + rank, epoch);
    const uint32_t* mine = P.flags[rank] + slot + peer;
    Deadline dl(timeout_ns);
    while ((int32_t)(ld_acquire_sys(mine) - epoch) < 0) {  // signed distance tolerates wrap-around
      if (dl.expired() || (poll_limit != 0 && dl.polls > poll_limit)) {
        s_fail = 1;
        if (status != nullptr && atomicCAS(status, 0, 10 + phase) == 0) {
          status[1] = rank; status[2] = peer; status[3] = slot_block; status[4] = (int)epoch;
        }
        break;
      }
      __nanosleep(64);
    }
  }
  __syncthreads();
  return s_fail == 0;
}

// Per-block epoch kept in device memory: block b of every rank bumps counter b once per launch, so the launch arguments do
// not change from call to call (a captured CUDA graph can replay the collective) and ranks stay in step because they
// launch the same kernels in the same order with the same grids.
__device__ __forceinline__ uint32_t next_block_epoch(uint32_t* epochs) {
  __shared__ uint32_t s_epoch;
  if (threadIdx.x == 0) {
    s_epoch = epochs[blockIdx.x] + 1;
    epochs[blockIdx.x] = s_epoch;
  }
  __syncthreads();
  return s_epoch;
}

static inline int fill_peers(Peers& P, void* const* data_ptrs, void* const* flag_ptrs, int world) {
  if (world < 1 || world > kMaxWorld) {
    nnb_set_error("comm: world size %d not supported (1..%d)", world, kMaxWorld);
    return -1;
  }
  for (int r = 0; r < kMaxWorld; ++r) {
    P.data[r] = r < world && data_ptrs ? data_ptrs[r] : nullptr;
    P.flags[r] = r < world ? static_cast<uint32_t*>(flag_ptrs[r]) : nullptr;
  }
  return 0;
}

}  // namespace nnbcomm
