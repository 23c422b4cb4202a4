// Collectives over NVLink 5 / NVSwitch written as kernels on symmetric memory: every rank holds the
// same buffer at the same offsets and the kernel is given all peers' device pointers, so it reduces,
// scatters and gathers with plain peer loads and stores (ld/st.global on a peer address) — or, when a
// multicast address is supplied, with multimem.ld_reduce / multimem.st so the switch does the sum and
// the broadcast. No NCCL call is involved.
//
//   nnb_allreduce_f32       in-place two-shot all-reduce of a range, fused with a scale (the 1/world
//                           gradient average): rank r reduces slice r from all peers and writes the
//                           result into every peer's buffer.
//   nnb_reduce_scatter_f32  rank r's slice of the sum (+ scale) into a local shard buffer, and the sum
//                           of squares of that shard for global-norm clipping.
//   nnb_allgather_bytes     every rank's shard into the local full buffer (pull).
//
// Synchronisation: a second symmetric buffer of uint32 flags, one slot per (phase, block, source
// rank), written with st.release.sys and polled locally with ld.acquire.sys; values are the call's
// epoch number, so flags never need resetting (and CUDA-graph replays would need none either).
// Block b of a rank only ever talks to block b of its peers, so the kernel needs no grid-wide sync.
// EVERY wait is bounded: after kPollLimit polls the block records {code, rank, peer, block, epoch} in
// the status words and carries on to the end, and the host raises after the next synchronisation.
// Nothing here waits on a kernel of the same GPU: one rank = one process = one GPU.
//
// The reference reaches NCCL through torch DDP / FSDP2 / DTensor (nanonemo/distributed/*.py).
#include "comm.cuh"

namespace {

using namespace nnbcomm;

__device__ __forceinline__ float4 ld_peer_f4(const float* p) {
  float4 v;
  asm volatile("ld.global.relaxed.sys.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float4 multimem_ld_reduce_f4(const float* mc) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(mc) : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st_f4(float* mc, float4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}

// WMAX = compile-time bound on the world size, U = independent 16-byte positions per thread: U x WMAX peer
// loads are issued before the first add, so each thread keeps 1 KB in flight over NVLink (the kernel is
// latency-bound otherwise: one load per peer per thread reached only a third of NCCL's bus bandwidth).
template <int WMAX, int U>
__global__ void __launch_bounds__(kCommThreads) allreduce_f32_kernel(Peers P, float* mc, int rank, int world, long long lo,
                                                                     long long n, float scale, uint32_t epoch, int* status) {
  const bool ok = block_barrier(P, rank, world, 0, blockIdx.x, gridDim.x, epoch, status);  // every peer's inputs are final
  const long long per = ((n + world - 1) / world + 3) & ~3LL;       // slice length, multiple of 4
  const long long s0 = min((long long)rank * per, n), s1 = min(s0 + per, n);
  const long long n4 = (s1 - s0) >> 2;
  const long long stride = (long long)gridDim.x * blockDim.x;
  if (ok) {
    for (long long i0 = blockIdx.x * (long long)blockDim.x + threadIdx.x; i0 < n4; i0 += stride * U) {
      float4 v[U][WMAX];
      if (mc != nullptr) {
#pragma unroll
        for (int u = 0; u < U; ++u)
          if (i0 + u * stride < n4) v[u][0] = multimem_ld_reduce_f4(mc + lo + s0 + 4 * (i0 + u * stride));
      } else {
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
          for (int r = 0; r < WMAX; ++r)
            if (r < world && i0 + u * stride < n4)
              v[u][r] = ld_peer_f4(static_cast<const float*>(P.data[r]) + lo + s0 + 4 * (i0 + u * stride));
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + u * stride;
        if (i >= n4) continue;
        const long long off = lo + s0 + 4 * i;
        float4 acc = v[u][0];
        if (mc == nullptr) {
#pragma unroll
          for (int r = 1; r < WMAX; ++r)  // fixed order: the result does not depend on who reduces
            if (r < world) { acc.x += v[u][r].x; acc.y += v[u][r].y; acc.z += v[u][r].z; acc.w += v[u][r].w; }
        }
        acc.x *= scale; acc.y *= scale; acc.z *= scale; acc.w *= scale;
        if (mc != nullptr) {
          multimem_st_f4(mc + off, acc);
        } else {
#pragma unroll
          for (int r = 0; r < WMAX; ++r)
            if (r < world) *reinterpret_cast<float4*>(static_cast<float*>(P.data[r]) + off) = acc;
        }
      }
    }
  }
  block_barrier(P, rank, world, 1, blockIdx.x, gridDim.x, epoch, status);  // every peer's results have landed here
}

// out[i] = scale * sum_r data[r][lo + rank*per + i]; sumsq_out += sum(out^2) (one atomic per block).
template <int WMAX, int U>
__global__ void __launch_bounds__(kCommThreads) reduce_scatter_f32_kernel(Peers P, float* out, float* sumsq_out, int rank, int world,
                                                                          long long lo, long long per, float scale,
                                                                          uint32_t epoch, int* status) {
  __shared__ float s_part[kCommThreads / 32];
  const bool ok = block_barrier(P, rank, world, 0, blockIdx.x, gridDim.x, epoch, status);
  const long long n4 = per >> 2;
  const long long stride = (long long)gridDim.x * blockDim.x;
  float ss = 0.f;
  if (ok) {
    for (long long i0 = blockIdx.x * (long long)blockDim.x + threadIdx.x; i0 < n4; i0 += stride * U) {
      float4 v[U][WMAX];
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int r = 0; r < WMAX; ++r)
          if (r < world && i0 + u * stride < n4)
            v[u][r] = ld_peer_f4(static_cast<const float*>(P.data[r]) + lo + (long long)rank * per + 4 * (i0 + u * stride));
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + u * stride;
        if (i >= n4) continue;
        float4 acc = v[u][0];
#pragma unroll
        for (int r = 1; r < WMAX; ++r)
          if (r < world) { acc.x += v[u][r].x; acc.y += v[u][r].y; acc.z += v[u][r].z; acc.w += v[u][r].w; }
        acc.x *= scale; acc.y *= scale; acc.z *= scale; acc.w *= scale;
        reinterpret_cast<float4*>(out)[i] = acc;
        ss += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
      }
    }
  }
  if (sumsq_out != nullptr) {
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x < 32) {
      float v = threadIdx.x < kCommThreads / 32 ? s_part[threadIdx.x] : 0.f;
      v = warp_sum(v);
      if (threadIdx.x == 0) atomicAdd(sumsq_out, v);
    }
  }
  // peers may overwrite their inputs only after everybody has read them
  block_barrier(P, rank, world, 1, blockIdx.x, gridDim.x, epoch, status);
}

// local_full[r*per_bytes .. ] = peer r's shard (its bytes [src_off, src_off + per_bytes) ), 16-byte units.
__global__ void __launch_bounds__(kCommThreads) allgather_kernel(Peers P, uint8_t* local_full, int rank, int world,
                                                                 long long src_off, long long per_bytes, uint32_t epoch,
                                                                 int* status) {
  const bool ok = block_barrier(P, rank, world, 0, blockIdx.x, gridDim.x, epoch, status);  // every peer's shard is final
  const long long n16 = per_bytes >> 4;
  if (ok) {
    for (int rr = 0; rr < world; ++rr) {
      const int r = (rank + rr) % world;  // start with the local shard, then spread the peers
      const uint4* src = reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(P.data[r]) + src_off);
      uint4* dst = reinterpret_cast<uint4*>(local_full + (long long)r * per_bytes);
      const long long stride = (long long)gridDim.x * blockDim.x;
      for (long long i0 = blockIdx.x * (long long)blockDim.x + threadIdx.x; i0 < n16; i0 += stride * 8) {
        uint4 v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u)
          if (i0 + u * stride < n16)
            asm volatile("ld.global.relaxed.sys.v4.u32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(v[u].x), "=r"(v[u].y), "=r"(v[u].z), "=r"(v[u].w) : "l"(src + i0 + u * stride) : "memory");
#pragma unroll
        for (int u = 0; u < 8; ++u)
          if (i0 + u * stride < n16) dst[i0 + u * stride] = v[u];
      }
    }
  }
  block_barrier(P, rank, world, 1, blockIdx.x, gridDim.x, epoch, status);  // shards may be rewritten once everybody has copied them
}

// Exercises the bounded wait: a "world" of two ranks whose flag buffers are both this GPU's buffer, so the
// slot that the (absent) second rank would write is never written. The wait gives up after `poll_limit`
// polls, records the status words and the kernel returns normally; the context stays usable.
__global__ void timeout_probe_kernel(Peers P, uint32_t epoch, uint32_t poll_limit, int* status, int* result) {
  const bool ok = block_barrier(P, 0, 2, 0, 0, 1, epoch, status, poll_limit);
  if (threadIdx.x == 0) *result = ok ? 1 : -1;
}

}  // namespace

extern "C" int nnb_comm_timeout_probe(void* flags, void* status, void* result, int epoch, int poll_limit, cudaStream_t st) {
  Peers P;
  void* both[2] = {flags, flags};
  if (fill_peers(P, nullptr, both, 2) != 0) return -1;
  NNB_REQUIRE(poll_limit > 0 && poll_limit <= (1 << 22), "timeout_probe: poll_limit out of range");
  timeout_probe_kernel<<<1, 64, 0, st>>>(P, (uint32_t)epoch, (uint32_t)poll_limit, static_cast<int*>(status), static_cast<int*>(result));
  NNB_LAUNCH_OK("timeout_probe");
  return 0;
}

// Flag buffer requirement: uint32 [2 phases][blocks][16] per rank, zero before the first call.
extern "C" int nnb_comm_flag_words(int blocks) { return 2 * blocks * kMaxWorld; }

extern "C" int nnb_allreduce_f32(void* const* data_ptrs, void* const* flag_ptrs, void* multicast_ptr, void* status, int rank,
                                 int world, long long lo, long long n, float scale, int epoch, int blocks, cudaStream_t st) {
  Peers P;
  if (fill_peers(P, data_ptrs, flag_ptrs, world) != 0) return -1;
  NNB_REQUIRE(lo % 4 == 0 && n % 4 == 0, "allreduce: range must be 16-byte aligned (lo=%lld n=%lld)", lo, n);
  NNB_REQUIRE(blocks > 0 && blocks <= 1024, "allreduce: bad block count %d", blocks);
  if (n == 0) return 0;
  NNB_REQUIRE(world <= 8, "allreduce: world %d > 8 not supported by the unrolled kernel", world);
  float* mc = static_cast<float*>(multicast_ptr);
  int* stw = static_cast<int*>(status);
  if (world <= 2) allreduce_f32_kernel<2, 8><<<blocks, kCommThreads, 0, st>>>(P, mc, rank, world, lo, n, scale, (uint32_t)epoch, stw);
  else if (world <= 4) allreduce_f32_kernel<4, 4><<<blocks, kCommThreads, 0, st>>>(P, mc, rank, world, lo, n, scale, (uint32_t)epoch, stw);
  else allreduce_f32_kernel<8, 2><<<blocks, kCommThreads, 0, st>>>(P, mc, rank, world, lo, n, scale, (uint32_t)epoch, stw);
  NNB_LAUNCH_OK("allreduce_f32");
  return 0;
}

extern "C" int nnb_reduce_scatter_f32(void* const* data_ptrs, void* const* flag_ptrs, void* out, void* sumsq_out, void* status,
                                      int rank, int world, long long lo, long long per, float scale, int epoch, int blocks,
                                      cudaStream_t st) {
  Peers P;
  if (fill_peers(P, data_ptrs, flag_ptrs, world) != 0) return -1;
  NNB_REQUIRE(lo % 4 == 0 && per % 4 == 0, "reduce_scatter: range must be 16-byte aligned");
  if (per == 0) return 0;
  NNB_REQUIRE(world <= 8, "reduce_scatter: world %d > 8 not supported by the unrolled kernel", world);
  float* o = static_cast<float*>(out);
  float* sq = static_cast<float*>(sumsq_out);
  int* stw = static_cast<int*>(status);
  if (world <= 2) reduce_scatter_f32_kernel<2, 8><<<blocks, kCommThreads, 0, st>>>(P, o, sq, rank, world, lo, per, scale, (uint32_t)epoch, stw);
  else if (world <= 4) reduce_scatter_f32_kernel<4, 4><<<blocks, kCommThreads, 0, st>>>(P, o, sq, rank, world, lo, per, scale, (uint32_t)epoch, stw);
  else reduce_scatter_f32_kernel<8, 2><<<blocks, kCommThreads, 0, st>>>(P, o, sq, rank, world, lo, per, scale, (uint32_t)epoch, stw);
  NNB_LAUNCH_OK("reduce_scatter_f32");
  return 0;
}

extern "C" int nnb_allgather_bytes(void* const* data_ptrs, void* const* flag_ptrs, void* local_full, void* status, int rank,
                                   int world, long long src_off, long long per_bytes, int epoch, int blocks, cudaStream_t st) {
  Peers P;
  if (fill_peers(P, data_ptrs, flag_ptrs, world) != 0) return -1;
  NNB_REQUIRE(src_off % 16 == 0 && per_bytes % 16 == 0 && nnb_aligned16(local_full), "allgather: 16-byte alignment required");
  if (per_bytes == 0) return 0;
  allgather_kernel<<<blocks, kCommThreads, 0, st>>>(P, static_cast<uint8_t*>(local_full), rank, world, src_off, per_bytes,
                                                    (uint32_t)epoch, static_cast<int*>(status));
  NNB_LAUNCH_OK("allgather");
  return 0;
}
