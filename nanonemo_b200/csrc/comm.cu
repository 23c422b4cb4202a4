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
// rank), written with st.release.sys and polled locally with ld.acquire.sys; values are epoch
// numbers that block b of every rank keeps in device memory and bumps once per launch, so flags never
// need resetting and the launch arguments are the same from call to call (a captured CUDA graph
// replays the collectives as they are).
// Block b of a rank only ever talks to block b of its peers, so the kernel needs no grid-wide sync.
// EVERY wait is bounded in time (30 s by default): when it runs out the block records
// {code, rank, peer, block, epoch} in the status words and carries on to the end; the training step
// reads the status word with its loss and raises on the host.
// Nothing here waits on a kernel of the same GPU: one rank = one process = one GPU.
//
// The reference reaches NCCL through torch DDP / FSDP2 / DTensor (nanonemo/distributed/*.py).
#include <cmath>
#include <cstdlib>

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

// WMAX = compile-time bound on the world size, U = independent 16-byte positions per thread: U x WMAX peer loads are issued
// before the first add. U x WMAX = 8 keeps the kernel within 85 registers (see kCommThreads); two 128-thread blocks per SM
// then have 296 x 128 x 128 B = 4.8 MB in flight, above the NVLink latency-bandwidth product (~3 us x 0.8 TB/s).
//
// Gradient all-reduce (data parallel): in-place two-shot all-reduce of [lo, lo + n) fused with the 1/world average; rank r
// reduces slice r, writes the result into every peer's buffer and, on the way, sums the squares of its slice. Each block
// stores its partial sum of squares into EVERY peer's `norm_parts` row for this bucket ([bucket][rank][block], plain peer
// stores before the closing barrier), so that after the last bucket every rank holds the same table and adds it up in the
// same order (nnb_sumsq_combine): the global gradient norm needs no pass over the gradient and no further collective, and
// it is bitwise identical on every rank.
template <int WMAX, int U>
__global__ void __launch_bounds__(kCommThreads, 3) allreduce_f32_kernel(Peers P, Peers NP, float* mc, int rank, int world, long long lo,
                                                                        long long n, float scale, uint32_t* epochs, int slot_blocks,
                                                                        int bucket, unsigned long long timeout_ns, int* status) {
  __shared__ float s_part[kCommThreads / 32];
  const uint32_t epoch = next_block_epoch(epochs);
  const bool ok = block_barrier(P, rank, world, 0, blockIdx.x, slot_blocks, epoch, status, 0, timeout_ns);  // every peer's inputs are final
  const long long per = ((n + world - 1) / world + 3) & ~3LL;       // slice length, multiple of 4
  const long long s0 = min((long long)rank * per, n), s1 = min(s0 + per, n);
  const long long n4 = (s1 - s0) >> 2;
  const long long stride = (long long)gridDim.x * blockDim.x;
  float ss = 0.f;
  if (ok && mc != nullptr) {
    // The switch adds the ranks' values (multimem.ld_reduce) and broadcasts the result (multimem.st): one load and one store
    // per 16 bytes whatever the world size, so the loads in flight come from unrolling over positions only.
    constexpr int UM = 8;
    for (long long i0 = blockIdx.x * (long long)blockDim.x + threadIdx.x; i0 < n4; i0 += stride * UM) {
      float4 v[UM];
#pragma unroll
      for (int u = 0; u < UM; ++u)
        if (i0 + u * stride < n4) v[u] = multimem_ld_reduce_f4(mc + lo + s0 + 4 * (i0 + u * stride));
#pragma unroll
      for (int u = 0; u < UM; ++u) {
        const long long i = i0 + u * stride;
        if (i >= n4) continue;
        float4 acc = v[u];
        acc.x *= scale; acc.y *= scale; acc.z *= scale; acc.w *= scale;
        ss += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
        multimem_st_f4(mc + lo + s0 + 4 * i, acc);
      }
    }
  } else if (ok) {
    for (long long i0 = blockIdx.x * (long long)blockDim.x + threadIdx.x; i0 < n4; i0 += stride * U) {
      float4 v[U][WMAX];
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int r = 0; r < WMAX; ++r)
          if (r < world && i0 + u * stride < n4)
            v[u][r] = ld_peer_f4(static_cast<const float*>(P.data[r]) + lo + s0 + 4 * (i0 + u * stride));
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + u * stride;
        if (i >= n4) continue;
        const long long off = lo + s0 + 4 * i;
        float4 acc = v[u][0];
#pragma unroll
        for (int r = 1; r < WMAX; ++r)  // fixed order: the result does not depend on who reduces
          if (r < world) { acc.x += v[u][r].x; acc.y += v[u][r].y; acc.z += v[u][r].z; acc.w += v[u][r].w; }
        acc.x *= scale; acc.y *= scale; acc.z *= scale; acc.w *= scale;
        ss += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
#pragma unroll
        for (int r = 0; r < WMAX; ++r)
          if (r < world) *reinterpret_cast<float4*>(static_cast<float*>(P.data[r]) + off) = acc;
      }
    }
  }
  if (NP.data[0] != nullptr) {
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x < 32) {
      float v = threadIdx.x < (blockDim.x >> 5) ? s_part[threadIdx.x] : 0.f;
      v = warp_sum(v);  // fixed tree: the same inputs give the same bits
      const long long slot = ((long long)bucket * world + rank) * slot_blocks + blockIdx.x;
      if ((int)threadIdx.x < world) static_cast<float*>(NP.data[threadIdx.x])[slot] = v;
    }
  }
  block_barrier(P, rank, world, 1, blockIdx.x, slot_blocks, epoch, status, 0, timeout_ns);  // every peer's results (and partial norms) have landed here
}

// out[0] = sum of parts[0 .. n) added in index order by one thread per 1/256th and a fixed tree: same table, same bits.
__global__ void __launch_bounds__(256) sumsq_combine_kernel(const float* __restrict__ parts, long long n, float* __restrict__ out) {
  __shared__ float s_part[8];
  float s = 0.f;
  for (long long i = threadIdx.x; i < n; i += 256) s += parts[i];
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) t += s_part[i];
    out[0] = t;
  }
}

// Sharded optimizer state of one unit for the reduce-scatter that applies AdamW in its epilogue (no clipping: the update of
// an element needs nothing but its own reduced gradient). All pointers address this rank's shard of the unit.
struct ShardAdamW {
  float* p;                      // fp32 master weights, null = plain reduce-scatter
  float* m;
  float* v;
  void* wire;                    // 16-bit copy that the next all-gather sends, or null
  const unsigned char* decay;    // one flag per 256 elements
  float lr, beta1, beta2, eps, wd, bc1, bc2_sqrt;
  int wire_bf16;
};

// out[i] = scale * sum_r data[r][lo + rank*per + i] (gradient reduce-scatter of one FSDP unit), plus the squared norm of the
// reduced shard: added to sumsq_out (one atomic per block) and / or stored per block into every peer's norm table (row
// `bucket`), as the all-reduce does, so the global norm needs no further collective. With A.p set, the AdamW update of the
// shard happens right here on the reduced values, which then never travel through memory as a gradient.
template <int WMAX, int U>
__global__ void __launch_bounds__(kCommThreads, 3) reduce_scatter_f32_kernel(Peers P, Peers NP, float* out, float* sumsq_out, int rank,
                                                                             int world, long long lo, long long per, float scale,
                                                                             uint32_t* epochs, int slot_blocks, int bucket, ShardAdamW A,
                                                                             unsigned long long timeout_ns, int* status) {
  __shared__ float s_part[kCommThreads / 32];
  const uint32_t epoch = next_block_epoch(epochs);
  const bool ok = block_barrier(P, rank, world, 0, blockIdx.x, slot_blocks, epoch, status, 0, timeout_ns);
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
        ss += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
        if (A.p == nullptr) {
          reinterpret_cast<float4*>(out)[i] = acc;
        } else {
          float4 pp = reinterpret_cast<float4*>(A.p)[i], mm = reinterpret_cast<float4*>(A.m)[i], vv = reinterpret_cast<float4*>(A.v)[i];
          const float decay = A.decay[i >> 6] ? 1.f - A.lr * A.wd : 1.f;
          const float step_size = A.lr / A.bc1;
          float* Pp = &pp.x; const float* G = &acc.x; float* Mo = &mm.x; float* V = &vv.x;
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            Pp[k] *= decay;
            Mo[k] = Mo[k] + (G[k] - Mo[k]) * (1.f - A.beta1);
            V[k] = V[k] * A.beta2 + G[k] * G[k] * (1.f - A.beta2);
            Pp[k] -= step_size * (Mo[k] / (sqrtf(V[k]) / A.bc2_sqrt + A.eps));
          }
          reinterpret_cast<float4*>(A.p)[i] = pp;
          reinterpret_cast<float4*>(A.m)[i] = mm;
          reinterpret_cast<float4*>(A.v)[i] = vv;
          if (A.wire != nullptr) {
            if (A.wire_bf16) {
              __nv_bfloat162* w = reinterpret_cast<__nv_bfloat162*>(A.wire) + 2 * i;
              w[0] = __floats2bfloat162_rn(pp.x, pp.y);
              w[1] = __floats2bfloat162_rn(pp.z, pp.w);
            } else {
              __half2* w = reinterpret_cast<__half2*>(A.wire) + 2 * i;
              w[0] = __floats2half2_rn(pp.x, pp.y);
              w[1] = __floats2half2_rn(pp.z, pp.w);
            }
          }
        }
      }
    }
  }
  if (sumsq_out != nullptr || NP.data[0] != nullptr) {
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x < 32) {
      float v = threadIdx.x < (blockDim.x >> 5) ? s_part[threadIdx.x] : 0.f;
      v = warp_sum(v);
      if (threadIdx.x == 0 && sumsq_out != nullptr) atomicAdd(sumsq_out, v);
      if (NP.data[0] != nullptr && (int)threadIdx.x < world)
        static_cast<float*>(NP.data[threadIdx.x])[((long long)bucket * world + rank) * slot_blocks + blockIdx.x] = v;
    }
  }
  // peers may overwrite their inputs only after everybody has read them
  block_barrier(P, rank, world, 1, blockIdx.x, slot_blocks, epoch, status, 0, timeout_ns);
}

// local_full[r*per_bytes .. ] = peer r's shard (its bytes [src_off, src_off + per_bytes) ), 16-byte units.
__global__ void __launch_bounds__(kCommThreads, 3) allgather_kernel(Peers P, uint8_t* local_full, int rank, int world,
                                                                    long long src_off, long long per_bytes, uint32_t* epochs,
                                                                    int slot_blocks, unsigned long long timeout_ns, int* status) {
  const uint32_t epoch = next_block_epoch(epochs);
  const bool ok = block_barrier(P, rank, world, 0, blockIdx.x, slot_blocks, epoch, status, 0, timeout_ns);  // every peer's shard is final
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
  block_barrier(P, rank, world, 1, blockIdx.x, slot_blocks, epoch, status, 0, timeout_ns);  // shards may be rewritten once everybody has copied them
}

// Small ranges fetched from the ranks that own them, in ONE launch: item i copies `bytes[i]` bytes at `src_off[i]` of rank
// `src_rank[i]`'s buffer to `dst[i]` (local). Used for the few parameters a unit's first kernel needs before the unit's own
// all-gather has run (the norm weight in front of a QKV projection that gathers its unit itself). One block per item.
struct FetchItem {
  long long src_off, bytes;
  uint8_t* dst;
  int src_rank, pad;
};

__global__ void __launch_bounds__(kCommThreads, 3) peer_fetch_kernel(Peers P, const FetchItem* __restrict__ items, int n_items, int rank,
                                                                     int world, uint32_t* epochs, int slot_blocks,
                                                                     unsigned long long timeout_ns, int* status) {
  const uint32_t epoch = next_block_epoch(epochs);
  const bool ok = block_barrier(P, rank, world, 0, blockIdx.x, slot_blocks, epoch, status, 0, timeout_ns);  // owners' buffers are final
  if (ok) {
    for (int it = blockIdx.x; it < n_items; it += gridDim.x) {
      const FetchItem f = items[it];
      const uint4* src = reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(P.data[f.src_rank]) + f.src_off);
      uint4* dst = reinterpret_cast<uint4*>(f.dst);
      for (long long i = threadIdx.x; i < (f.bytes >> 4); i += blockDim.x) {
        uint4 v;
        asm volatile("ld.global.relaxed.sys.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(src + i) : "memory");
        dst[i] = v;
      }
    }
  }
  block_barrier(P, rank, world, 1, blockIdx.x, slot_blocks, epoch, status, 0, timeout_ns);  // owners may rewrite once everybody has read
}

// ---- vocabulary-parallel embedding (tensor + sequence parallel): the table is sharded over the vocabulary, the residual
// stream over the tokens. Token i (of N = world * per) belongs to rank i / per; its row lives on the rank whose vocabulary
// slice [v0, v0 + V) holds idx[i]. Exactly one rank owns each row, so nothing is reduced: the forward PUSHES every owned row
// into the token owner's staging buffer (peer stores), the backward PULLS the gradient rows of the tokens it owns from the
// token owners' staging buffers (peer loads) and adds them into its slice of the table's gradient. Block b of every rank
// handles the staging rows r with r % gridDim.x == b, so the block-to-block flag barrier orders every row it touches.
// The staging buffer ([per, D] elements of TO, symmetric) is free again when either kernel ends (closing barrier).
template <typename TO>
__device__ __forceinline__ void ld_sys8(const TO* p, float (&v)[8]) {
  if constexpr (sizeof(TO) == 4) {
    const float4 a = ld_peer_f4(reinterpret_cast<const float*>(p)), b = ld_peer_f4(reinterpret_cast<const float*>(p) + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  } else {
    uint4 raw;
    asm volatile("ld.global.relaxed.sys.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(raw.x), "=r"(raw.y), "=r"(raw.z), "=r"(raw.w) : "l"(p) : "memory");
    const TO* h = reinterpret_cast<const TO*>(&raw);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = to_f32(h[i]);
  }
}

template <typename TO>
__global__ void __launch_bounds__(kCommThreads, 3) vp_embed_fwd_kernel(Peers P, const long long* __restrict__ idx, const float* __restrict__ W,
                                                                       TO* __restrict__ out, long long per, int D, long long v0, long long V,
                                                                       int rank, int world, uint32_t* epochs, int slot_blocks,
                                                                       unsigned long long timeout_ns, int* status) {
  const uint32_t epoch = next_block_epoch(epochs);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5, vec = D >> 3;
  const long long mine = per > blockIdx.x ? (per - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;  // staging rows of this block
  for (long long it = warp; it < mine * world; it += nwarps) {
    const int dest = (int)(it / mine);
    const long long r = blockIdx.x + (it - dest * mine) * gridDim.x;
    const long long tok = idx[dest * per + r] - v0;
    if (tok < 0 || tok >= V) continue;  // another rank's row
    const float* src = W + tok * D;
    TO* dst = static_cast<TO*>(P.data[dest]) + r * D;
    for (int c = lane; c < vec; c += 32) {
      float v[8];
      Chunk8<float>::load(src + c * 8, v);
      Chunk8<TO>::store(dst + c * 8, v);
    }
  }
  const bool ok = block_barrier(P, rank, world, 0, blockIdx.x, slot_blocks, epoch, status, 0, timeout_ns);  // every owner has written
  if (ok) {
    const TO* stage = static_cast<const TO*>(P.data[rank]);
    for (long long it = warp; it < mine; it += nwarps) {
      const long long r = blockIdx.x + it * gridDim.x;
      for (int c = lane; c < vec; c += 32) {
        float v[8];
        ld_sys8(stage + r * D + c * 8, v);
        Chunk8<TO>::store(out + r * D + c * 8, v);
      }
    }
  }
  block_barrier(P, rank, world, 1, blockIdx.x, slot_blocks, epoch, status, 0, timeout_ns);  // staging may be written again
}

template <typename TO>
__global__ void __launch_bounds__(kCommThreads, 3) vp_embed_bwd_kernel(Peers P, const long long* __restrict__ idx, const TO* __restrict__ g,
                                                                       float* __restrict__ dW, long long per, int D, long long v0, long long V,
                                                                       int rank, int world, uint32_t* epochs, int slot_blocks,
                                                                       unsigned long long timeout_ns, int* status) {
  const uint32_t epoch = next_block_epoch(epochs);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5, vec = D >> 3;
  const long long mine = per > blockIdx.x ? (per - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  TO* stage = static_cast<TO*>(P.data[rank]);
  for (long long it = warp; it < mine; it += nwarps) {  // this rank's gradient rows, where the peers can read them
    const long long r = blockIdx.x + it * gridDim.x;
    for (int c = lane; c < vec; c += 32)
      *reinterpret_cast<uint4*>(stage + r * D + c * 8) = *reinterpret_cast<const uint4*>(g + r * D + c * 8);
    if constexpr (sizeof(TO) == 4)
      for (int c = lane; c < vec; c += 32)
        *reinterpret_cast<uint4*>(stage + r * D + c * 8 + 4) = *reinterpret_cast<const uint4*>(g + r * D + c * 8 + 4);
  }
  const bool ok = block_barrier(P, rank, world, 0, blockIdx.x, slot_blocks, epoch, status, 0, timeout_ns);  // every rank has staged
  if (ok) {
    for (long long it = warp; it < mine * world; it += nwarps) {
      const int src_rank = (int)(it / mine);
      const long long r = blockIdx.x + (it - src_rank * mine) * gridDim.x;
      const long long tok = idx[src_rank * per + r] - v0;
      if (tok < 0 || tok >= V) continue;
      const TO* src = static_cast<const TO*>(P.data[src_rank]) + r * D;
      float* dst = dW + tok * D;
      for (int c = lane; c < vec; c += 32) {
        float v[8];
        ld_sys8(src + c * 8, v);
        asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + c * 8), "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]) : "memory");
        asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + c * 8 + 4), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7]) : "memory");
      }
    }
  }
  block_barrier(P, rank, world, 1, blockIdx.x, slot_blocks, epoch, status, 0, timeout_ns);  // staging may be written again
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

// Flag buffer requirement: uint32 [2 phases][blocks][16] per rank, zero before the first call; `epochs`: device uint32
// [blocks], zero before the first call, private to the rank. `blocks` is the count both were sized for; every kernel that
// shares them indexes its flag slots with it.
extern "C" int nnb_comm_flag_words(int blocks) { return 2 * blocks * kMaxWorld; }

// Threads per collective block (a multiple of 32 up to kCommThreads; NANONEMO_COMM_THREADS). The default of 128 keeps a block
// at about 10 K registers, so that it fits on an SM next to ANY compute kernel of the training step, including the
// 320-thread x 168-register attention backward and the GEMMs with two epilogue groups (53.8 K of the 64 K registers): a
// collective that cannot share the SM either waits for those kernels or, once resident, keeps their CTAs off the SM while it
// sits in a cross-GPU barrier. The launcher's `blocks` (two per SM by default) makes up for the smaller blocks wherever the
// resident compute kernel leaves room for both.
static inline int comm_threads() {
  static int threads = [] {
    const char* e = getenv("NANONEMO_COMM_THREADS");
    int t = e ? atoi(e) : 128;
    t = (t / 32) * 32;
    return t < 32 ? 32 : (t > kCommThreads ? kCommThreads : t);
  }();
  return threads;
}

static inline unsigned long long timeout_ns_of(double seconds) {
  return seconds > 0 ? (unsigned long long)(seconds * 1e9) : kDefaultTimeoutNs;
}

// norm_ptrs: null, or every rank's `norm_parts` buffer (fp32 [buckets][world][blocks], symmetric); `bucket` picks the row.
extern "C" int nnb_allreduce_f32(void* const* data_ptrs, void* const* flag_ptrs, void* const* norm_ptrs, void* multicast_ptr,
                                 void* status, void* epochs, int rank, int world, long long lo, long long n, float scale, int bucket,
                                 int blocks, double timeout_s, cudaStream_t st) {
  Peers P, NP;
  if (fill_peers(P, data_ptrs, flag_ptrs, world) != 0) return -1;
  if (fill_peers(NP, norm_ptrs, flag_ptrs, world) != 0) return -1;
  NNB_REQUIRE(lo % 4 == 0 && n % 4 == 0, "allreduce: range must be 16-byte aligned (lo=%lld n=%lld)", lo, n);
  NNB_REQUIRE(blocks > 0 && blocks <= 1024 && epochs != nullptr, "allreduce: bad block count %d or no epoch counters", blocks);
  if (n == 0) return 0;
  NNB_REQUIRE(world <= 8, "allreduce: world %d > 8 not supported by the unrolled kernel", world);
  float* mc = static_cast<float*>(multicast_ptr);
  int* stw = static_cast<int*>(status);
  uint32_t* ep = static_cast<uint32_t*>(epochs);
  const unsigned long long tns = timeout_ns_of(timeout_s);
  if (world <= 2) allreduce_f32_kernel<2, 4><<<blocks, comm_threads(), 0, st>>>(P, NP, mc, rank, world, lo, n, scale, ep, blocks, bucket, tns, stw);
  else if (world <= 4) allreduce_f32_kernel<4, 2><<<blocks, comm_threads(), 0, st>>>(P, NP, mc, rank, world, lo, n, scale, ep, blocks, bucket, tns, stw);
  else allreduce_f32_kernel<8, 1><<<blocks, comm_threads(), 0, st>>>(P, NP, mc, rank, world, lo, n, scale, ep, blocks, bucket, tns, stw);
  NNB_LAUNCH_OK("allreduce_f32");
  return 0;
}

// out[0] = sum of the first n entries of `parts` in a fixed order (the table the all-reduce kernels filled).
extern "C" int nnb_sumsq_combine(const void* parts, long long n, void* out, cudaStream_t st) {
  NNB_REQUIRE(n >= 0 && out != nullptr, "sumsq_combine: bad arguments");
  sumsq_combine_kernel<<<1, 256, 0, st>>>(static_cast<const float*>(parts), n, static_cast<float*>(out));
  NNB_LAUNCH_OK("sumsq_combine");
  return 0;
}

static int launch_reduce_scatter(void* const* data_ptrs, void* const* flag_ptrs, void* const* norm_ptrs, void* out, void* sumsq_out,
                                 void* status, void* epochs, int rank, int world, long long lo, long long per, float scale, int bucket,
                                 int blocks, double timeout_s, const ShardAdamW& A, cudaStream_t st) {
  Peers P, NP;
  if (fill_peers(P, data_ptrs, flag_ptrs, world) != 0) return -1;
  if (fill_peers(NP, norm_ptrs, flag_ptrs, world) != 0) return -1;
  NNB_REQUIRE(lo % 4 == 0 && per % 4 == 0, "reduce_scatter: range must be 16-byte aligned");
  NNB_REQUIRE(blocks > 0 && blocks <= 1024 && epochs != nullptr, "reduce_scatter: bad block count %d or no epoch counters", blocks);
  if (per == 0) return 0;
  NNB_REQUIRE(world <= 8, "reduce_scatter: world %d > 8 not supported by the unrolled kernel", world);
  float* o = static_cast<float*>(out);
  float* sq = static_cast<float*>(sumsq_out);
  int* stw = static_cast<int*>(status);
  uint32_t* ep = static_cast<uint32_t*>(epochs);
  const unsigned long long tns = timeout_ns_of(timeout_s);
  if (world <= 2) reduce_scatter_f32_kernel<2, 4><<<blocks, comm_threads(), 0, st>>>(P, NP, o, sq, rank, world, lo, per, scale, ep, blocks, bucket, A, tns, stw);
  else if (world <= 4) reduce_scatter_f32_kernel<4, 2><<<blocks, comm_threads(), 0, st>>>(P, NP, o, sq, rank, world, lo, per, scale, ep, blocks, bucket, A, tns, stw);
  else reduce_scatter_f32_kernel<8, 1><<<blocks, comm_threads(), 0, st>>>(P, NP, o, sq, rank, world, lo, per, scale, ep, blocks, bucket, A, tns, stw);
  NNB_LAUNCH_OK("reduce_scatter_f32");
  return 0;
}

// norm_ptrs: null, or every rank's norm table (see nnb_allreduce_f32); `bucket` picks the row this call fills.
extern "C" int nnb_reduce_scatter_f32(void* const* data_ptrs, void* const* flag_ptrs, void* const* norm_ptrs, void* out, void* sumsq_out,
                                      void* status, void* epochs, int rank, int world, long long lo, long long per, float scale,
                                      int bucket, int blocks, double timeout_s, cudaStream_t st) {
  ShardAdamW none{};
  NNB_REQUIRE(out != nullptr, "reduce_scatter: no output buffer");
  return launch_reduce_scatter(data_ptrs, flag_ptrs, norm_ptrs, out, sumsq_out, status, epochs, rank, world, lo, per, scale, bucket,
                               blocks, timeout_s, none, st);
}

// Reduce-scatter whose epilogue IS the sharded AdamW step (for training without gradient clipping): p / m / v: this rank's
// fp32 shard of the unit (per elements), wire: its 16-bit copy for the next parameter all-gather (or null), decay_flags: one
// byte per 256 elements. The reduced gradient is never written; its squared norm still goes to the norm table for logging.
extern "C" int nnb_reduce_scatter_adamw(void* const* data_ptrs, void* const* flag_ptrs, void* const* norm_ptrs, void* p, void* m, void* v,
                                        void* wire, const void* decay_flags, void* status, void* epochs, int rank, int world,
                                        long long lo, long long per, float scale, int bucket, int blocks, double timeout_s, float lr,
                                        float beta1, float beta2, float eps, float wd, int step, int wire_dtype, cudaStream_t st) {
  NNB_REQUIRE(p != nullptr && m != nullptr && v != nullptr && decay_flags != nullptr, "reduce_scatter_adamw: missing optimizer state");
  NNB_REQUIRE(per % 256 == 0 && step >= 1, "reduce_scatter_adamw: shard of %lld elements must be a multiple of 256, step >= 1", per);
  NNB_REQUIRE(wire == nullptr || wire_dtype == NNB_BF16 || wire_dtype == NNB_F16, "reduce_scatter_adamw: wire dtype code %d", wire_dtype);
  ShardAdamW A{static_cast<float*>(p), static_cast<float*>(m), static_cast<float*>(v), wire, static_cast<const unsigned char*>(decay_flags),
               lr, beta1, beta2, eps, wd, (float)(1.0 - pow((double)beta1, (double)step)),
               (float)sqrt(1.0 - pow((double)beta2, (double)step)), wire_dtype == NNB_BF16 ? 1 : 0};
  return launch_reduce_scatter(data_ptrs, flag_ptrs, norm_ptrs, nullptr, nullptr, status, epochs, rank, world, lo, per, scale, bucket,
                               blocks, timeout_s, A, st);
}

extern "C" int nnb_allgather_bytes(void* const* data_ptrs, void* const* flag_ptrs, void* local_full, void* status, void* epochs,
                                   int rank, int world, long long src_off, long long per_bytes, int blocks, double timeout_s,
                                   cudaStream_t st) {
  Peers P;
  if (fill_peers(P, data_ptrs, flag_ptrs, world) != 0) return -1;
  NNB_REQUIRE(src_off % 16 == 0 && per_bytes % 16 == 0 && nnb_aligned16(local_full), "allgather: 16-byte alignment required");
  NNB_REQUIRE(blocks > 0 && blocks <= 1024 && epochs != nullptr, "allgather: bad block count %d or no epoch counters", blocks);
  if (per_bytes == 0) return 0;
  allgather_kernel<<<blocks, comm_threads(), 0, st>>>(P, static_cast<uint8_t*>(local_full), rank, world, src_off, per_bytes,
                                                    static_cast<uint32_t*>(epochs), blocks, timeout_ns_of(timeout_s),
                                                    static_cast<int*>(status));
  NNB_LAUNCH_OK("allgather");
  return 0;
}

// items: device array of n_items records {int64 src_off, int64 bytes, void* dst, int32 src_rank, int32 pad} (32 bytes each);
// offsets, sizes and destinations 16-byte aligned. Uses min(n_items, blocks) blocks of the communicator's flag slots.
extern "C" int nnb_peer_fetch(void* const* data_ptrs, void* const* flag_ptrs, const void* items, int n_items, void* status, void* epochs,
                              int rank, int world, int blocks, double timeout_s, cudaStream_t st) {
  Peers P;
  if (fill_peers(P, data_ptrs, flag_ptrs, world) != 0) return -1;
  NNB_REQUIRE(blocks > 0 && blocks <= 1024 && epochs != nullptr && items != nullptr, "peer_fetch: bad arguments");
  if (n_items <= 0) return 0;
  static_assert(sizeof(FetchItem) == 32, "FetchItem layout is part of the interface");
  peer_fetch_kernel<<<min(n_items, blocks), comm_threads(), 0, st>>>(P, static_cast<const FetchItem*>(items), n_items, rank, world,
                                                                  static_cast<uint32_t*>(epochs), blocks, timeout_ns_of(timeout_s),
                                                                  static_cast<int*>(status));
  NNB_LAUNCH_OK("peer_fetch");
  return 0;
}

// Vocabulary-parallel embedding. stage_ptrs: every rank's staging buffer ([per, D] elements of the residual dtype, symmetric);
// idx: ALL world * per token ids (int64, the same on every rank); W / dW: this rank's fp32 rows [v0, v0 + V) of the table and
// of its gradient; out / g: this rank's `per` rows. D a multiple of 8, everything 16-byte aligned.
static int vp_embed_checks(const char* what, const void* idx, const void* w, const void* rows, long long per, int D, long long V, int blocks,
                           const void* epochs) {
  NNB_REQUIRE(D > 0 && D % 8 == 0, "%s: D=%d must be a positive multiple of 8", what, D);
  NNB_REQUIRE(per >= 0 && V > 0 && idx != nullptr && w != nullptr && rows != nullptr, "%s: bad arguments", what);
  NNB_REQUIRE(nnb_aligned16(w) && nnb_aligned16(rows), "%s: 16-byte alignment required", what);
  NNB_REQUIRE(blocks > 0 && blocks <= 1024 && epochs != nullptr, "%s: bad block count %d or no epoch counters", what, blocks);
  return 0;
}

extern "C" int nnb_vp_embedding_fwd(void* const* stage_ptrs, void* const* flag_ptrs, const void* idx, const void* W, void* out, long long per,
                                    int D, long long v0, long long V, int dtype, void* status, void* epochs, int rank, int world, int blocks,
                                    double timeout_s, cudaStream_t st) {
  Peers P;
  if (fill_peers(P, stage_ptrs, flag_ptrs, world) != 0) return -1;
  if (vp_embed_checks("vp_embedding_fwd", idx, W, out, per, D, V, blocks, epochs) != 0) return -1;
  NNB_DISPATCH(dtype, TO, {
    vp_embed_fwd_kernel<TO><<<blocks, comm_threads(), 0, st>>>(P, static_cast<const long long*>(idx), static_cast<const float*>(W), static_cast<TO*>(out),
                                                            per, D, v0, V, rank, world, static_cast<uint32_t*>(epochs), blocks,
                                                            timeout_ns_of(timeout_s), static_cast<int*>(status));
  });
  NNB_LAUNCH_OK("vp_embedding_fwd");
  return 0;
}

extern "C" int nnb_vp_embedding_bwd(void* const* stage_ptrs, void* const* flag_ptrs, const void* idx, const void* g, void* dW, long long per,
                                    int D, long long v0, long long V, int dtype, void* status, void* epochs, int rank, int world, int blocks,
                                    double timeout_s, cudaStream_t st) {
  Peers P;
  if (fill_peers(P, stage_ptrs, flag_ptrs, world) != 0) return -1;
  if (vp_embed_checks("vp_embedding_bwd", idx, dW, g, per, D, V, blocks, epochs) != 0) return -1;
  NNB_DISPATCH(dtype, TO, {
    vp_embed_bwd_kernel<TO><<<blocks, comm_threads(), 0, st>>>(P, static_cast<const long long*>(idx), static_cast<const TO*>(g), static_cast<float*>(dW),
                                                            per, D, v0, V, rank, world, static_cast<uint32_t*>(epochs), blocks,
                                                            timeout_ns_of(timeout_s), static_cast<int*>(status));
  });
  NNB_LAUNCH_OK("vp_embedding_bwd");
  return 0;
}
