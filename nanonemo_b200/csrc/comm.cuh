// Device-side building blocks of the NVLink collectives, shared by the collective kernels (comm.cu)
// and the GEMMs that fuse a collective into their prologue / epilogue (gemm_comm.cu): the table of
// peer pointers, system-scope release / acquire accesses, and the bounded cross-rank block barrier.
#pragma once
#include "common.cuh"

namespace nnbcomm {

constexpr int kMaxWorld = 16;
constexpr uint32_t kPollLimit = 1u << 22;
constexpr int kCommThreads = 512;

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
// the block (needs at least `world` threads).
__device__ __forceinline__ bool block_barrier(const Peers& P, int rank, int world, int phase, int slot_block, int n_slot_blocks,
                                              uint32_t epoch, int* status, uint32_t poll_limit = kPollLimit) {
  __shared__ int s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  __threadfence_system();
  __syncthreads();
  const int slot = (phase * n_slot_blocks + slot_block) * kMaxWorld;
  if ((int)threadIdx.x < world) {
    const int peer = threadIdx.x;
    st_release_sys(P.flags[peer] + slot + rank, epoch);
    const uint32_t* mine = P.flags[rank] + slot + peer;
    uint32_t polls = 0;
    while ((int32_t)(ld_acquire_sys(mine) - epoch) < 0) {  // signed distance tolerates wrap-around
      if (++polls > poll_limit) {
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
