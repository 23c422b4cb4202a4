// bf16/fp16 GEMM on the 5th-generation tensor cores: D[M,N] (+)= A[M,K] * B[N,K]^T, fp32 accumulate.
//
// Structure (one persistent CTA per SM, 192 threads, warp-specialised):
//   warp 0      TMA producer: cp.async.bulk.tensor loads of 128-byte swizzled A/B tiles into a ring of
//               shared-memory stages, completion on mbarriers (expect-tx bytes);
//   warp 1      MMA issuer: one elected thread issues tcgen05.mma (M=128, N=BN, K=16) from shared-memory
//               descriptors into a TMEM accumulator, tcgen05.commit releases the stage / publishes the tile;
//   warps 2..5  epilogue: tcgen05.ld of the accumulator (each warp its lane quarter), convert, write a
//               128-byte swizzled staging tile, TMA store (or TMA reduce-add for fp32 accumulation).
// The accumulator is double buffered in TMEM (2 x BN columns), so the epilogue of tile i overlaps the
// MMAs of tile i+1, and the producer runs ahead across tiles: with K = 768 a tile is only 12 k-blocks
// long and the pipeline must never drain between tiles.
//
// Operand layouts (all three training GEMMs without a transposed copy of anything):
//   A K-major  : A stored [M, K] row-major.        A MN-major : A stored [K, M] row-major (A^T).
//   B K-major  : B stored [N, K] row-major.        B MN-major : B stored [K, N] row-major (B^T).
//   fprop  y  = x W^T        : A = x  (K-major),  B = W  (K-major)
//   dgrad  dx = dy W         : A = dy (K-major),  B = W  (MN-major: W is [N_out, K_in] = [K_gemm, N_gemm])
//   wgrad  dW += dy^T x      : A = dy (MN-major), B = x  (MN-major), fp32 output, split-K with TMA reduce-add
// Work items are (m-block, n-block, k-split); every item of a split-K GEMM reduce-adds its partial tile
// into the fp32 output, so accumulating into an existing gradient buffer costs nothing extra.
//
// This replaces the cuBLAS calls behind nn.Linear in the reference (nanonemo/model/layers.py:80-83,
// 128-130); the reference ships no tensor-core GEMM of its own.
#include <cstdlib>

#include "comm.cuh"
#include "gemm2.cuh"
#include <type_traits>

#include "sm100.cuh"

namespace {

using namespace sm100;

constexpr int BM = 128;
constexpr int BK = 64;  // 64 x 16-bit = 128 bytes = one swizzle span
constexpr int kThreads = 192;
constexpr int kEpilogueThreads = 128;
constexpr int kStagingBytes = 2 * BM * 128;  // two 128-row x 128-byte staging tiles

// MX = block-scaled e4m3 operands (MXFP8): a stage is still 128 bytes of K per row (128 elements instead of 64) plus the
// e8m0 scales of its rows (512 bytes per 128 rows: 4 K-blocks of 32 x 128 rows); the scales take 8 more TMEM columns.
template <int BN, bool MX = false>
struct Cfg {
  static constexpr int kStageBytesA = BM * BK * 2;
  static constexpr int kStageBytesB = BN * BK * 2;
  static constexpr int kOperandBytes = kStageBytesA + kStageBytesB;
  static constexpr int kSfBytesA = MX ? 512 : 0, kSfBytesB = MX ? (BN / 128) * 512 : 0;
  static constexpr int kStageBytes = kOperandBytes + (MX ? 1024 : 0);  // stage stride keeps the 1024-byte alignment
  static constexpr int kTxBytes = kOperandBytes + kSfBytesA + kSfBytesB;
  static constexpr int kStages = MX ? 5 : ((BN == 256) ? 4 : (BN == 192 ? 4 : 6));
  static constexpr int kSfCol = 2 * BN;  // TMEM columns [2 BN, 2 BN + 4) scales of A, [2 BN + 4, 2 BN + 8) scales of B
  static constexpr int kTmemCols = (2 * BN + (MX ? 8 : 0) <= 256) ? 256 : 512;  // allocations are powers of two
  static constexpr int kSmemBytes = kStages * kStageBytes + kStagingBytes + 1024 /*align*/ + 256 /*barriers*/;
  static_assert(!MX || BN == 128, "the block-scaled path is built for 128-wide tiles (two accumulators + scales must fit 512 columns)");
};

struct Params {
  int M, N, K;
  int m_blocks, n_blocks, k_splits, kblocks_total, kblocks_per_split;
  int group_m;          // tile order: groups of group_m m-blocks are swept n-block by n-block (1 = row by row)
  int a_mn, b_mn;       // operand majors
  int out_f32;          // output dtype: 0 = 16-bit (same as inputs), 1 = fp32
  int reduce_add;       // epilogue uses TMA reduce-add (fp32 only)
  uint32_t idesc;
  int out_bf16;         // 16-bit output format: 1 = bf16, 0 = fp16
  const uint8_t* sfa;   // MX: e8m0 scales of A in 512-byte chunks [m-block][k-block] (see nnb_mxfp8_quantize_sw)
  const uint8_t* sfb;   // MX: same for the rows of B, chunk index [n / 128][k-block]
  int* status;          // device int[4]: {code, role, block, item}; code 0 = ok
  // ---- fused collectives (mode 0: none)
  //  mode 1  GEMM -> reduce-scatter: output rows are sharded over `world` ranks (mblocks_per_rank m-blocks each);
  //          every tile is TMA-reduce-added straight into the OWNER rank's buffer over NVLink (tmDs.m[owner]).
  //  mode 2  all-gather -> GEMM: A rows are sharded over the ranks in a symmetric buffer; the first `gather_ctas`
  //          CTAs pull the peers' shards into the local buffer m-block by m-block and publish a ready flag per
  //          m-block; the other CTAs start on the local rows and wait (bounded) for a flag before a remote block.
  //  mode 3  parameter all-gather -> GEMM (FSDP): B is one weight inside a UNIT of parameters whose 16-bit bytes are sharded
  //          evenly over the ranks (symmetric "wire" buffers). The first `gather_ctas` CTAs copy every rank's shard of the
  //          whole unit into the local unsharded buffer chunk by chunk, the chunks that hold B first, and publish a flag
  //          per chunk; the producer of a compute CTA waits (bounded) for the chunks under its B tile. When the kernel
  //          ends the whole unit is local, so the block's other linears just read it.
  int mode, world, rank, mblocks_per_rank, gather_ctas;
  long long g_src_off, g_per_bytes, g_b_off;  // mode 3: shard offset in the wire buffers, bytes per rank, offset of B in the unit
  uint8_t* g_dst;                             // mode 3: local unsharded unit buffer
  int g_chunk_bytes, g_chunks_per_rank;       // mode 3: copy / flag granularity
  uint32_t epoch;
  uint32_t* local_flags;  // device uint32: [0] go flag, [1] finished-CTA counter, [2 + m_blk] m-block ready flags
  long long a_row_bytes;  // mode 2: bytes of one row of A (rows are contiguous)
  int* comm_status;       // device int[8] for the collective part
  nnbcomm::Peers peers;   // flags of every rank; data = every rank's A buffer (mode 2)
};

struct DMaps {
  CUtensorMap m[8];       // mode 1: one output map per rank; otherwise m[0]
};

template <int BN, bool MX>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ DMaps tmDs, const Params p) {
  using C = Cfg<BN, MX>;
  constexpr int kBlockK = MX ? 2 * BK : BK;  // elements of K per stage (always 128 bytes per row)
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stage_base = smem;
  uint8_t* staging = smem + C::kStages * C::kStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(staging + kStagingBytes);
  // barrier layout: full[kStages], empty[kStages], tmem_full[2], tmem_empty[2]
  const uint32_t bar_full = smem_u32(bars), bar_empty = bar_full + 8 * C::kStages;
  const uint32_t bar_tfull = bar_empty + 8 * C::kStages, bar_tempty = bar_tfull + 16;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * C::kStages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* epi_abort = abort_flag + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(bar_tfull + 8 * a, 1);
      mbar_init(bar_tempty + 8 * a, kEpilogueThreads / 32);
    }
    *abort_flag = 0;
    *epi_abort = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), C::kTmemCols);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    tma_prefetch_desc(&tmDs.m[0]);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int items = p.m_blocks * p.n_blocks * p.k_splits;
  int fail_role = 0, fail_item = -1;
  // compute CTAs: index cta0 of nctas (in mode 2 the first gather_ctas CTAs only move data)
  const int first_compute = (p.mode == 2 || p.mode == 3) ? p.gather_ctas : 0;
  const int cta0 = (int)blockIdx.x - first_compute, nctas = (int)gridDim.x - first_compute;
  // m-block visited at position `ord`: mode 2 starts with this rank's own rows, then follows the gather order
  auto m_of = [&](int ord) { return p.mode == 2 ? (p.rank * p.mblocks_per_rank + ord) % p.m_blocks : ord; };
  // tile index -> (position of the m-block, n-block). Consecutive tiles — the ones the persistent CTAs work on at the same
  // time — cover group_m m-blocks x (CTAs / group_m) n-blocks, so a wave re-uses a few MB of A and B from L2 instead of
  // streaming every n-block of B for a single m-block.
  auto tile_coords = [&](int tile, int& m_ord, int& n_blk) {
    const int per_group = p.group_m * p.n_blocks, g = tile / per_group, r = tile - g * per_group;
    const int gm = min(p.group_m, p.m_blocks - g * p.group_m);
    m_ord = g * p.group_m + r % gm;
    n_blk = r / gm;
  };

  if (p.mode == 1 && blockIdx.x == 0) {
    // every rank's output buffer has been zeroed (stream order on each rank) before anybody adds into it
    const bool ok = nnbcomm::block_barrier(p.peers, p.rank, p.world, 0, 0, 1, p.epoch, p.comm_status);
    if (threadIdx.x == 0) nnbcomm::st_release_gpu(p.local_flags, ok ? p.epoch : p.epoch - 1);
  }

  if (p.mode == 3 && cta0 < 0) {
    // ------------------------------------------------------------------ unit gather CTAs (FSDP parameter all-gather)
    const int G = p.gather_ctas, me = blockIdx.x;
    bool ok = nnbcomm::block_barrier(p.peers, p.rank, p.world, 0, me, G, p.epoch, p.comm_status);  // every rank's shard is final
    // chunk id = r * chunks_per_rank + k covers bytes [k CB, min((k + 1) CB, per)) of rank r's shard. This CTA copies the
    // chunks with id % G == me: first the ones that intersect B (the GEMM is waiting for those), then the others.
    uint16_t* my_chunks = reinterpret_cast<uint16_t*>(staging);   // staging tiles are unused by a gather CTA
    __shared__ int s_total;
    const long long CB = p.g_chunk_bytes, per = p.g_per_bytes;
    const long long b0 = p.g_b_off, b1 = p.g_b_off + (long long)p.N * p.K * 2;
    if (threadIdx.x == 0) {
      int n = 0;
      const int total_chunks = p.world * p.g_chunks_per_rank;
      for (int pass = 0; pass < 2; ++pass)
        for (int step = 0; step < p.world; ++step) {
          const int r = (p.rank + step) % p.world;  // own shard first, then the peers in ring order
          for (int k = 0; k < p.g_chunks_per_rank; ++k) {
            const int id = r * p.g_chunks_per_rank + k;
            if (id % G != me || id >= total_chunks) continue;
            const long long c0 = (long long)r * per + k * CB, c1 = min(c0 + CB, (long long)(r + 1) * per);
            const bool in_b = c0 < b1 && c1 > b0;
            if (in_b == (pass == 0) && n < (int)(kStagingBytes / 2)) my_chunks[n++] = (uint16_t)id;
          }
        }
      s_total = n;
    }
    __syncthreads();
    if (threadIdx.x == 0 && ok) {
      const int total = s_total;
      constexpr int S = C::kStages;
      constexpr int kLag = 2;
      auto locate = [&](int i, long long& src_off, long long& dst_off, uint32_t& bytes, int& r) {
        const int id = my_chunks[i];
        r = id / p.g_chunks_per_rank;
        const long long k = id % p.g_chunks_per_rank;
        bytes = (uint32_t)min(CB, per - k * CB);
        src_off = p.g_src_off + k * CB;
        dst_off = (long long)r * per + k * CB;
      };
      auto publish = [&](int j) {
        asm volatile("fence.proxy.async;" ::: "memory");
        __threadfence();
        nnbcomm::st_release_gpu(p.local_flags + 2 + my_chunks[j], p.epoch);
      };
      for (int i = 0; i < total + (S - kLag) && ok; ++i) {
        if (i < total) {
          long long so, d_o; uint32_t bytes; int r;
          locate(i, so, d_o, bytes, r);
          const uint32_t st = i % S;
          mbar_expect_tx(bar_full + 8 * st, bytes);
          asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                       ::"r"(smem_u32(stage_base + st * C::kStageBytes)), "l"(static_cast<const uint8_t*>(p.peers.data[r]) + so),
                         "r"(bytes), "r"(bar_full + 8 * st) : "memory");
        }
        const int j = i - (S - kLag);
        if (j >= 0 && j < total) {
          long long so, d_o; uint32_t bytes; int r;
          locate(j, so, d_o, bytes, r);
          const uint32_t st = j % S;
          if (!mbar_wait(bar_full + 8 * st, (j / S) & 1, abort_flag)) { ok = false; break; }
          asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(p.g_dst + d_o),
                       "r"(smem_u32(stage_base + st * C::kStageBytes)), "r"(bytes) : "memory");
          tma_commit_group();
          tma_wait_group<kLag - 1>();  // the stage the next load overwrites has been read; everything older is complete in memory
          if (j - (kLag - 1) >= 0) publish(j - (kLag - 1));
        }
      }
      tma_wait_group<0>();
      if (ok)
        for (int j = max(0, total - (kLag - 1)); j < total; ++j) publish(j);
    }
    __syncthreads();
    // this rank's shard may be rewritten (by the optimizer) only after every peer has copied it
    nnbcomm::block_barrier(p.peers, p.rank, p.world, 1, me, G, p.epoch, p.comm_status);
  } else if (p.mode == 2 && cta0 < 0) {
    // ------------------------------------------------------------------ gather CTAs (all threads copy)
    const int G = p.gather_ctas, me = blockIdx.x;
    bool ok = nnbcomm::block_barrier(p.peers, p.rank, p.world, 0, me, G, p.epoch, p.comm_status);  // peers' shards are final
    // One thread drives bulk asynchronous copies through the (otherwise unused) operand stages of this CTA:
    // peer memory -> shared memory (cp.async.bulk, completion on an mbarrier) -> local memory (bulk store), so a
    // handful of CTAs keep megabytes in flight over NVLink. An m-block's ready flag is published once its last
    // store group has completed.
    if (threadIdx.x == 0 && ok) {
      const long long mb_bytes = (long long)BM * p.a_row_bytes;
      int chunk_rows = BM;
      while (chunk_rows > 1 && (long long)chunk_rows * p.a_row_bytes > C::kStageBytes) chunk_rows >>= 1;
      const uint32_t chunk_bytes = (uint32_t)(chunk_rows * p.a_row_bytes);
      const int chunks_per_mb = BM / chunk_rows;
      const int my_mbs = (p.mblocks_per_rank - me + G - 1) / G;            // m-blocks of each peer handled here
      const int total = (p.world - 1) * my_mbs * chunks_per_mb;           // chunks to move
      constexpr int S = C::kStages;
      constexpr int kLag = 2;                                             // stores trail the loads by S - kLag chunks
      auto locate = [&](int i, long long& off, int& flag_idx, bool& last) {
        const int c = i % chunks_per_mb, mbi = (i / chunks_per_mb) % my_mbs, step = 1 + i / (chunks_per_mb * my_mbs);
        const int r = (p.rank + step) % p.world, mb = me + mbi * G;
        off = (long long)(r * p.mblocks_per_rank + mb) * mb_bytes + (long long)c * chunk_bytes;
        flag_idx = r * p.mblocks_per_rank + mb;
        last = c == chunks_per_mb - 1;
        return r;
      };
      auto store_chunk = [&](int j) -> bool {
        long long off; int fi; bool last;
        locate(j, off, fi, last);
        const uint32_t s = j % S;
        if (!mbar_wait(bar_full + 8 * s, (j / S) & 1, abort_flag)) return false;
        asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(static_cast<uint8_t*>(p.peers.data[p.rank]) + off),
                     "r"(smem_u32(stage_base + s * C::kStageBytes)), "r"(chunk_bytes) : "memory");
        tma_commit_group();
        return true;
      };
      auto publish_if_last = [&](int j) {
        long long off; int fi; bool last;
        locate(j, off, fi, last);
        if (last) {
          asm volatile("fence.proxy.async;" ::: "memory");
          __threadfence();
          nnbcomm::st_release_gpu(p.local_flags + 2 + fi, p.epoch);
        }
      };
      for (int i = 0; i < total + (S - kLag) && ok; ++i) {
        if (i < total) {
          long long off; int fi; bool last;
          const int r = locate(i, off, fi, last);
          const uint32_t s = i % S;
          mbar_expect_tx(bar_full + 8 * s, chunk_bytes);
          asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                       ::"r"(smem_u32(stage_base + s * C::kStageBytes)), "l"(static_cast<const uint8_t*>(p.peers.data[r]) + off),
                         "r"(chunk_bytes), "r"(bar_full + 8 * s) : "memory");
        }
        const int j = i - (S - kLag);
        if (j >= 0 && j < total) {
          if (!store_chunk(j)) { ok = false; break; }
          // at most kLag - 1 store groups stay pending: the stage the next load overwrites has been read, and
          // everything older is complete in memory
          tma_wait_group<kLag - 1>();
          if (j - (kLag - 1) >= 0) publish_if_last(j - (kLag - 1));
        }
      }
      tma_wait_group<0>();
      for (int j = max(0, total - (kLag - 1)); j < total; ++j) publish_if_last(j);
    }
    __syncthreads();
    // my shard may be overwritten only after every peer has copied it
    nnbcomm::block_barrier(p.peers, p.rank, p.world, 1, me, G, p.epoch, p.comm_status);
  } else if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int item = cta0; item < items && ok; item += nctas) {
        const int ks = item % p.k_splits, tile = item / p.k_splits;
        int m_ord, n_blk;
        tile_coords(tile, m_ord, n_blk);
        const int m_blk = m_of(m_ord);
        const int kb0 = ks * p.kblocks_per_split, kb1 = min(kb0 + p.kblocks_per_split, p.kblocks_total);
        if (p.mode == 2 && m_blk / p.mblocks_per_rank != p.rank) {
          // rows of a peer: wait until a gather CTA has landed this m-block in the local buffer
          const uint32_t* flag = p.local_flags + 2 + m_blk;
          nnbcomm::Deadline dl;
          while ((int32_t)(nnbcomm::ld_acquire_gpu(flag) - p.epoch) < 0) {
            if (dl.expired() || *abort_flag) { ok = false; *abort_flag = 1; fail_role = 4; fail_item = item; break; }
            __nanosleep(32);
          }
          if (!ok) break;
          asm volatile("fence.proxy.async;" ::: "memory");  // generic-proxy writes of the gather CTAs -> TMA reads
        }
        if (p.mode == 3) {
          // rows [n0, n1) of B are bytes [x0, x1) of the unit: wait for every chunk under them
          const long long row_bytes = (long long)p.K * 2;
          long long x = p.g_b_off + (long long)n_blk * BN * row_bytes;
          const long long x1 = p.g_b_off + (long long)min((n_blk + 1) * BN, p.N) * row_bytes;
          while (x < x1 && ok) {
            const long long r = x / p.g_per_bytes, k = (x - r * p.g_per_bytes) / p.g_chunk_bytes;
            const uint32_t* flag = p.local_flags + 2 + r * p.g_chunks_per_rank + k;
            nnbcomm::Deadline dl;
            while ((int32_t)(nnbcomm::ld_acquire_gpu(flag) - p.epoch) < 0) {
              if (dl.expired() || *abort_flag) { ok = false; *abort_flag = 1; fail_role = 4; fail_item = item; break; }
              __nanosleep(32);
            }
            x = min((r + 1) * p.g_per_bytes, r * p.g_per_bytes + (k + 1) * (long long)p.g_chunk_bytes);
          }
          if (!ok) break;
          asm volatile("fence.proxy.async;" ::: "memory");  // bulk-copy writes of the gather CTAs -> TMA reads
        }
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const uint32_t s = it % C::kStages, ph = (it / C::kStages) & 1;
          if (!mbar_wait(bar_empty + 8 * s, ph ^ 1, abort_flag)) { ok = false; fail_role = 1; fail_item = item; break; }
          const uint32_t full = bar_full + 8 * s;
          mbar_expect_tx(full, C::kTxBytes);
          const uint32_t sa = smem_u32(stage_base + s * C::kStageBytes), sb = sa + C::kStageBytesA;
          if constexpr (MX) {
            tma_load_2d(sa, &tmA, full, kb * kBlockK, m_blk * BM);
            tma_load_2d(sb, &tmB, full, kb * kBlockK, n_blk * BN);
            bulk_load(sa + C::kOperandBytes, p.sfa + ((long long)m_blk * p.kblocks_total + kb) * 512, 512, full);
#pragma unroll
            for (int j = 0; j < BN / 128; ++j)
              bulk_load(sa + C::kOperandBytes + 512 + 512 * j, p.sfb + ((long long)(n_blk * (BN / 128) + j) * p.kblocks_total + kb) * 512, 512, full);
            continue;
          }
          if (!p.a_mn) {
            tma_load_2d(sa, &tmA, full, kb * BK, m_blk * BM);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d(sa + j * (BK * 128), &tmA, full, m_blk * BM + j * 64, kb * BK);
          }
          if (!p.b_mn) {
            tma_load_2d(sb, &tmB, full, kb * BK, n_blk * BN);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_load_2d(sb + j * (BK * 128), &tmB, full, n_blk * BN + j * 64, kb * BK);
          }
        }
      }
      if (!ok) {
        // give the copies already in flight a bounded chance to land before the CTA exits
        const uint32_t first = it > (uint32_t)C::kStages ? it - C::kStages : 0;
        for (uint32_t j = first; j < it; ++j)
          for (uint32_t spin = 0; spin < (1u << 16) && !mbar_try_wait(bar_full + 8 * (j % C::kStages), (j / C::kStages) & 1); ++spin) {}
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      uint32_t it = 0, tile_iter = 0;
      bool ok = true;
      const uint32_t a_step = p.a_mn ? (16 * 128) >> 4 : 32 >> 4;  // descriptor start-address step per UMMA_K = 16
      const uint32_t b_step = p.b_mn ? (16 * 128) >> 4 : 32 >> 4;
      const uint32_t a_lbo = p.a_mn ? BK * 128 : 16, b_lbo = p.b_mn ? BK * 128 : 16;
      for (int item = cta0; item < items && ok; item += nctas, ++tile_iter) {
        const int ks = item % p.k_splits;
        const int kb0 = ks * p.kblocks_per_split, kb1 = min(kb0 + p.kblocks_per_split, p.kblocks_total);
        const uint32_t acc = tile_iter & 1, acc_ph = (tile_iter >> 1) & 1;
        if (!mbar_wait(bar_tempty + 8 * acc, acc_ph ^ 1, abort_flag)) { ok = false; fail_role = 2; fail_item = item; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const uint32_t s = it % C::kStages, ph = (it / C::kStages) & 1;
          if (!mbar_wait(bar_full + 8 * s, ph, abort_flag)) { ok = false; fail_role = 2; fail_item = item; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(stage_base + s * C::kStageBytes), sb = sa + C::kStageBytesA;
          const uint64_t da = make_smem_desc(sa, a_lbo, 1024), db = make_smem_desc(sb, b_lbo, 1024);
          if constexpr (MX) {
            // scales of this stage: shared memory -> tensor memory (tcgen05 operations of one thread execute in order, so the
            // copy neither overtakes the previous stage's MMAs nor is overtaken by the ones below)
            const uint32_t sf_tmem = tmem_base + C::kSfCol;
            tmem_cp_32x128b_warpx4(sf_tmem, make_smem_desc_noswizzle(sa + C::kOperandBytes, 0, 128));
#pragma unroll
            for (int j = 0; j < BN / 128; ++j)
              tmem_cp_32x128b_warpx4(sf_tmem + 4 + 4 * j, make_smem_desc_noswizzle(sa + C::kOperandBytes + 512 + 512 * j, 0, 128));
#pragma unroll
            for (uint32_t k = 0; k < 4; ++k)  // 4 x K = 32 (32 bytes of every 128-byte row); scale byte k of each column
              umma_mxf8(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), p.idesc | (k << 4) | (k << 29),
                        sf_tmem | (k << 30), (sf_tmem + 4) | (k << 30), (kb > kb0 || k > 0) ? 1u : 0u);
          } else {
#pragma unroll
            for (int k = 0; k < BK / 16; ++k)
              umma_f16(d_tmem, da + (uint64_t)(k * a_step), db + (uint64_t)(k * b_step), p.idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          umma_commit(bar_empty + 8 * s);  // the stage is free once these MMAs have read it
        }
        if (ok) umma_commit(bar_tfull + 8 * acc);  // accumulator complete
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;                 // TMEM lane quarter this warp may read
    const int row = q * 32 + lane;          // row of the tile owned by this thread
    const int et = threadIdx.x - 64;        // 0..127
    uint32_t tile_iter = 0, gchunk = 0;  // gchunk: staging buffers alternate across tiles too
    int pending_stores = 0;
    bool go = p.mode != 1;  // mode 1: the first reduce waits until every rank has zeroed its output
    for (int item = cta0; item < items; item += nctas, ++tile_iter) {
      const int tile = item / p.k_splits;
      int m_ord, n_blk;
      tile_coords(tile, m_ord, n_blk);
      const int m_blk = m_of(m_ord);
      // where the tile goes: mode 1 = the owner rank's buffer (peer memory), row offset inside its shard
      const int owner = p.mode == 1 ? m_blk / p.mblocks_per_rank : 0;
      const int d_row = p.mode == 1 ? (m_blk - owner * p.mblocks_per_rank) * BM : m_blk * BM;
      const CUtensorMap* tmD = &tmDs.m[owner];
      const uint32_t acc = tile_iter & 1, acc_ph = (tile_iter >> 1) & 1;
      const bool ok = mbar_wait(bar_tfull + 8 * acc, acc_ph, abort_flag);
      if (!ok) { fail_role = 3; fail_item = item; }
      if (et == 0) *epi_abort = *abort_flag;
      named_barrier_sync(1, kEpilogueThreads);
      if (*epi_abort) break;
      tc_fence_after();
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN;
      const int cols_per_chunk = p.out_f32 ? 32 : 64;  // 128 bytes of output per row and chunk
      const int chunks = BN / cols_per_chunk;
      for (int c = 0; c < chunks; ++c) {
        const int col0 = c * cols_per_chunk;
        if (n_blk * BN + col0 >= p.N) break;  // this chunk is entirely outside the matrix (uniform)
        uint8_t* buf = staging + (gchunk & 1) * (BM * 128);
        ++gchunk;
        if (et == 0 && pending_stores >= 2) tma_wait_group_read<1>();  // the store that last read `buf` is done
        if (!go) {
          if (et == 0) {
            nnbcomm::Deadline dl;
            bool late = false;
            while ((int32_t)(nnbcomm::ld_acquire_gpu(p.local_flags) - p.epoch) < 0 && !(late = dl.expired())) __nanosleep(64);
            if (late) *abort_flag = 1;
          }
          go = true;
        }
        named_barrier_sync(1, kEpilogueThreads);
        uint8_t* my_row = buf + row * 128;
        const int sw = row & 7;
        if (p.out_f32) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(t_row + col0, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *reinterpret_cast<uint4*>(my_row + ((j ^ sw) << 4)) = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
        } else {
          uint32_t r0[32], r1[32];
          tmem_ld_32x32b_x32(t_row + col0, r0);
          tmem_ld_32x32b_x32(t_row + col0 + 32, r1);
          tmem_ld_wait();
          // one branch around the whole conversion (not one per pair): each arm is straight-line code
          auto convert_row = [&](auto is_bf16) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              uint32_t w[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const int i = (j & 3) * 8 + 2 * e;
                w[e] = sm100::pack2_16<!decltype(is_bf16)::value>(__uint_as_float(j < 4 ? r0[i] : r1[i]), __uint_as_float(j < 4 ? r0[i + 1] : r1[i + 1]));
              }
              *reinterpret_cast<uint4*>(my_row + ((j ^ sw) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
            }
          };
          if (p.out_bf16 != 0) convert_row(std::true_type{});
          else convert_row(std::false_type{});
        }
        fence_proxy_async_smem();
        named_barrier_sync(1, kEpilogueThreads);
        if (et == 0) {
          if (p.reduce_add) tma_reduce_add_2d(tmD, smem_u32(buf), n_blk * BN + col0, d_row);
          else tma_store_2d(tmD, smem_u32(buf), n_blk * BN + col0, d_row);
          tma_commit_group();
        }
        if (pending_stores < 2) ++pending_stores;
      }
      // all TMEM reads of this accumulator are complete: hand it back to the MMA warp
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_tempty + 8 * acc);
    }
    if (et == 0) tma_wait_group<0>();  // every output byte has left shared memory and is visible
  }

  if (fail_item >= 0 && p.status != nullptr) {
    if (atomicCAS(p.status, 0, 1) == 0) {
      p.status[1] = fail_role;
      p.status[2] = blockIdx.x;
      p.status[3] = fail_item;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
  if (p.mode == 1) {
    // The last CTA of this rank to finish meets the last CTAs of the peers: when the kernel ends on a rank,
    // every rank's contributions to its shard have landed.
    __shared__ int s_last;
    if (threadIdx.x == 0) {
      __threadfence_system();
      s_last = atomicAdd(p.local_flags + 1, 1u) == gridDim.x - 1;
    }
    __syncthreads();
    if (s_last) {
      nnbcomm::block_barrier(p.peers, p.rank, p.world, 1, 0, 1, p.epoch, p.comm_status);
      if (threadIdx.x == 0) p.local_flags[1] = 0u;
    }
  }
}

template <int BN, bool MX = false>
int launch(const CUtensorMap& tmA, const CUtensorMap& tmB, const DMaps& tmDs, const Params& p, int grid, cudaStream_t st) {
  auto kern = gemm_tcgen05_kernel<BN, MX>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<BN, MX>::kSmemBytes) != cudaSuccess) {
      nnb_set_error("gemm: cannot reserve %d bytes of shared memory", Cfg<BN, MX>::kSmemBytes);
      return -3;
    }
    configured = true;
  }
  kern<<<grid, kThreads, Cfg<BN, MX>::kSmemBytes, st>>>(tmA, tmB, tmDs, p);
  return 0;
}

}  // namespace

namespace {

struct CommArgs {           // mode 0 when null
  int mode, world, rank, gather_ctas;
  void* const* data_ptrs;   // mode 1: every rank's output shard buffer; mode 2: every rank's full A buffer
  void* const* flag_ptrs;   // symmetric uint32 flag buffers (nnb_comm_flag_words(max(1, gather_ctas)))
  void* local_flags;        // device uint32 [2 + m_blocks], zero before the first call
  void* comm_status;        // device int[8]
  int epoch;
  // mode 3 (data_ptrs = every rank's wire buffer): the unit's shard starts at src_off bytes in each of them and is per_bytes
  // long; dst = local unsharded unit buffer; B sits b_off bytes into the unit
  long long src_off = 0, per_bytes = 0, b_off = 0;
  void* dst = nullptr;
};

int gemm_impl(const void* A, const void* B, void* D, int M, int N, int K, long long lda, long long ldb, long long ldd, int a_mn,
              int b_mn, int dtype, int out_f32, int accumulate, int k_splits, int bn_hint, int max_ctas, void* status,
              const CommArgs* comm, cudaStream_t st) {
  NNB_REQUIRE(M > 0 && N > 0 && K > 0, "gemm: empty problem %dx%dx%d", M, N, K);
  NNB_REQUIRE(dtype == NNB_BF16 || dtype == NNB_F16, "gemm: inputs must be bf16 or fp16 (dtype code %d)", dtype);
  const int mode = comm ? comm->mode : 0;
  NNB_REQUIRE(!accumulate || out_f32 || mode == 1, "gemm: accumulate needs an fp32 output");
  const CUtensorMapDataType in_dt = dtype == NNB_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const int sms = max_ctas > 0 ? min(max_ctas, nnb_num_sms()) : nnb_num_sms();
  // CTA-pair kernel (gemm2.cu): 256 x 256 tiles over two SMs. Measured faster than the single-CTA tiles at every shape of
  // the 114M model (1-20 %: K = 768 with any N, or N = 768 with any K), slower when N and K are both large (the 1.3B
  // shapes: 32768 x 2048 x 5632 runs at 1166 vs 1428 TFLOP/s; 8192^3 at 1233 vs 1274), where the single-CTA kernel stays.
  static const bool pair_enabled = [] { const char* e = getenv("NANONEMO_GEMM_PAIR"); return !(e && e[0] == '0'); }();
  const bool big_cube = M >= 2048 && N >= 2048 && K >= 2048;
  if (mode == 0 && (bn_hint == 512 || (bn_hint == 0 && pair_enabled && M >= 256 && N >= 256 && !big_cube))) {
    const NnbGemm2Args g{A, B, D, M, N, K, lda, ldb, ldd, a_mn, b_mn, dtype, out_f32, accumulate, k_splits, max_ctas, status};
    const int rc = nnb_gemm2_launch(g, st);
    if (rc <= 0) return rc;  // 1 = shape not served: fall through to the single-CTA kernel
    bn_hint = 0;
  }
  const int m_blocks_ = (M + BM - 1) / BM;
  // Tile width: the widest tile is the most efficient per FLOP, but the number of tiles should fill whole
  // waves of `sms` persistent CTAs. cost = waves x tile width (a tile's time is proportional to its width).
  int BN = 256;
  if (bn_hint == 128 || bn_hint == 192 || bn_hint == 256) {
    BN = bn_hint;
  } else if (N <= 128) {
    BN = 128;
  } else {
    double best = 1e30;
    const int cands[2] = {256, 128};  // 192-wide tiles measured slower even where they fill the waves better (kept behind bn_hint)
    const double eff[2] = {1.0, 1.10};  // narrower tiles re-read A more often: small penalty
    for (int i = 0; i < 2; ++i) {
      const int bn = cands[i];
      const long long tiles = (long long)m_blocks_ * ((N + bn - 1) / bn);
      const double cost = (double)((tiles + sms - 1) / sms) * bn * eff[i];
      if (cost < best) { best = cost; BN = bn; }
    }
    if (out_f32) BN = 256;  // split-K GEMMs balance with the split count instead
  }

  Params p{};
  p.M = M; p.N = N; p.K = K;
  p.m_blocks = (M + BM - 1) / BM;
  p.n_blocks = (N + BN - 1) / BN;
  p.kblocks_total = (K + BK - 1) / BK;
  int splits = 1;
  if (out_f32 && mode == 0) {
    if (k_splits > 0) splits = k_splits;
    else {
      // makespan of `tiles * s` equal items on `sms` persistent CTAs is ceil(tiles * s / sms) / s of the
      // whole K loop; take the split count that minimises it (ties: fewer splits = less reduce traffic)
      const long long tiles = (long long)p.m_blocks * p.n_blocks;
      const int s_max = max(1, min(32, p.kblocks_total / 4));
      double best = 1e30;
      for (int sp = 1; sp <= s_max; ++sp) {
        const double cost = (double)((tiles * sp + sms - 1) / sms) / sp + 0.002 * sp;
        if (cost < best - 1e-9) { best = cost; splits = sp; }
      }
    }
    splits = max(1, min(splits, p.kblocks_total));
  }
  p.kblocks_per_split = (p.kblocks_total + splits - 1) / splits;
  p.k_splits = (p.kblocks_total + p.kblocks_per_split - 1) / p.kblocks_per_split;
  p.group_m = 1;
  if (mode == 0) {
    // wave of `sms` tiles = group_m x (sms / group_m) blocks; footprint group_m BM K + (sms / group_m) BN K is least at
    // group_m = sqrt(sms BN / BM). Only matters when one row of tiles is longer than the wave share.
    int g = 1;
    while ((g + 1) * (g + 1) * BM <= sms * BN) ++g;
    if (p.n_blocks * g > sms) p.group_m = min(g, p.m_blocks);
  }
  p.a_mn = a_mn ? 1 : 0;
  p.b_mn = b_mn ? 1 : 0;
  p.out_f32 = out_f32 ? 1 : 0;
  p.reduce_add = (accumulate || p.k_splits > 1 || mode == 1) ? 1 : 0;
  p.idesc = sm100::make_idesc_f16(dtype == NNB_BF16 ? 1 : 0, p.a_mn, p.b_mn, BM, BN);
  p.out_bf16 = dtype == NNB_BF16 ? 1 : 0;
  p.status = static_cast<int*>(status);
  p.mode = mode;

  CUtensorMap tmA, tmB;
  DMaps tmDs;
  if (!p.a_mn) { if (!nnb_make_tmap_2d(&tmA, in_dt, 2, A, M, K, lda * 2, BM, BK, "gemm A")) return -4; }
  else         { if (!nnb_make_tmap_2d(&tmA, in_dt, 2, A, K, M, lda * 2, BK, 64, "gemm A^T")) return -4; }
  if (!p.b_mn) { if (!nnb_make_tmap_2d(&tmB, in_dt, 2, B, N, K, ldb * 2, BN, BK, "gemm B")) return -4; }
  else         { if (!nnb_make_tmap_2d(&tmB, in_dt, 2, B, K, N, ldb * 2, BK, 64, "gemm B^T")) return -4; }
  const CUtensorMapDataType d_dt = out_f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : in_dt;
  const int d_bytes = out_f32 ? 4 : 2, d_box = out_f32 ? 32 : 64;
  if (mode == 1) {
    NNB_REQUIRE(comm->world >= 1 && comm->world <= 8, "gemm_rs: world %d not supported (1..8)", comm->world);
    NNB_REQUIRE(!a_mn && M % (BM * comm->world) == 0, "gemm_rs: M=%d must be a multiple of %d x world", M, BM);
    const int rows = M / comm->world;
    for (int r = 0; r < comm->world; ++r)
      if (!nnb_make_tmap_2d(&tmDs.m[r], d_dt, d_bytes, comm->data_ptrs[r], rows, N, ldd * d_bytes, BM, d_box, "gemm_rs D")) return -4;
    for (int r = comm->world; r < 8; ++r) tmDs.m[r] = tmDs.m[0];
  } else {
    if (!nnb_make_tmap_2d(&tmDs.m[0], d_dt, d_bytes, D, M, N, ldd * d_bytes, BM, d_box, "gemm D")) return -4;
    for (int r = 1; r < 8; ++r) tmDs.m[r] = tmDs.m[0];
  }
  if (mode != 0) {
    p.world = comm->world; p.rank = comm->rank;
    p.mblocks_per_rank = p.m_blocks / comm->world;
    p.gather_ctas = (mode == 2 || mode == 3) ? comm->gather_ctas : 0;
    p.epoch = (uint32_t)comm->epoch;
    p.local_flags = static_cast<uint32_t*>(comm->local_flags);
    p.comm_status = static_cast<int*>(comm->comm_status);
    p.a_row_bytes = lda * 2;
    if (nnbcomm::fill_peers(p.peers, (mode == 2 || mode == 3) ? comm->data_ptrs : nullptr, comm->flag_ptrs, comm->world) != 0) return -1;
    if (mode == 3) {
      NNB_REQUIRE(!a_mn && !b_mn && ldb == K, "gather_b_gemm: K-major operands with a contiguous weight expected");
      NNB_REQUIRE(comm->gather_ctas >= 1 && comm->gather_ctas < sms, "gather_b_gemm: bad gather CTA count %d", comm->gather_ctas);
      NNB_REQUIRE(comm->per_bytes > 0 && comm->per_bytes % 16 == 0 && comm->src_off % 16 == 0 && nnb_aligned16(comm->dst),
                  "gather_b_gemm: shards must be 16-byte aligned");
      p.g_src_off = comm->src_off; p.g_per_bytes = comm->per_bytes; p.g_b_off = comm->b_off;
      p.g_dst = static_cast<uint8_t*>(comm->dst);
      p.g_chunk_bytes = 32768;  // fits one operand stage of every tile width; 16-byte multiple
      p.g_chunks_per_rank = (int)((comm->per_bytes + p.g_chunk_bytes - 1) / p.g_chunk_bytes);
      NNB_REQUIRE((long long)p.g_chunks_per_rank * comm->world <= 16000, "gather_b_gemm: unit too large for the chunk table");
    }
    if (mode == 2) {
      NNB_REQUIRE(!a_mn && lda == K && M % (BM * comm->world) == 0, "ag_gemm: A must be contiguous [M, K] with M a multiple of %d x world", BM);
      NNB_REQUIRE(comm->gather_ctas >= 1 && comm->gather_ctas < sms, "ag_gemm: bad gather CTA count %d", comm->gather_ctas);
    }
  }

  if (out_f32 && !accumulate && p.k_splits > 1) {
    // partial tiles are reduce-added: start from zero
    if (ldd == N) cudaMemsetAsync(D, 0, (size_t)M * N * 4, st);
    else cudaMemset2DAsync(D, ldd * 4, 0, (size_t)N * 4, M, st);
  }
  const int items = p.m_blocks * p.n_blocks * p.k_splits;
  int grid = min(items, sms);
  if (mode == 2 || mode == 3) grid = min(items + p.gather_ctas, sms);
  const int rc = BN == 256 ? launch<256>(tmA, tmB, tmDs, p, grid, st)
               : BN == 192 ? launch<192>(tmA, tmB, tmDs, p, grid, st) : launch<128>(tmA, tmB, tmDs, p, grid, st);
  if (rc != 0) return rc;
  NNB_LAUNCH_OK("gemm_tcgen05");
  return 0;
}

}  // namespace

// A, B: 16-bit (dtype: 1 = bf16, 2 = fp16). lda/ldb/ldd: row strides in ELEMENTS of the stored matrices:
//   A K-major stored [M, K] (lda >= K); A MN-major stored [K, M] (lda >= M); same for B with N.
// D stored [M, N] row-major with ldd; out_f32 selects fp32 output, accumulate adds into D (fp32 only).
// k_splits <= 0 picks a split automatically (only used with fp32 output). status: device int[4] or null.
extern "C" int nnb_gemm_bf16(const void* A, const void* B, void* D, int M, int N, int K, long long lda, long long ldb,
                             long long ldd, int a_mn, int b_mn, int dtype, int out_f32, int accumulate, int k_splits,
                             int bn_hint, int max_ctas, void* status, cudaStream_t st) {
  return gemm_impl(A, B, D, M, N, K, lda, ldb, ldd, a_mn, b_mn, dtype, out_f32, accumulate, k_splits, bn_hint, max_ctas, status,
                   nullptr, st);
}

// ---- GEMMs with a fused epilogue (CTA-pair kernel only; return code 1 = shape not served, the caller runs the unfused ops)
static int fused_gemm_common(NnbGemm2Args& g, const void* A, const void* B, void* D, int M, int N, int K, long long lda,
                             long long ldb, long long ldd, int dtype, void* status) {
  NNB_REQUIRE(M > 0 && N > 0 && K > 0, "gemm: empty problem %dx%dx%d", M, N, K);
  NNB_REQUIRE(dtype == NNB_BF16 || dtype == NNB_F16, "gemm: inputs must be bf16 or fp16 (dtype code %d)", dtype);
  g.A = A; g.B = B; g.D = D; g.M = M; g.N = N; g.K = K; g.lda = lda; g.ldb = ldb; g.ldd = ldd;
  g.a_mn = 0; g.b_mn = 0; g.dtype = dtype; g.out_f32 = 0; g.accumulate = 0; g.k_splits = 1; g.max_ctas = 0; g.status = status;
  return 0;
}

// gu[M, 2F] = x[M, K] @ w_gu[2F, K]^T (gate rows first, then up rows) and act[M, F] = silu(gate) * up, one kernel.
extern "C" int nnb_gemm_swiglu(const void* X, const void* Wgu, void* GU, void* ACT, int M, int F, int K, long long lda, long long ldw,
                               long long ldgu, long long ldact, int dtype, void* status, cudaStream_t st) {
  NnbGemm2Args g{};
  if (int rc = fused_gemm_common(g, X, Wgu, GU, M, 2 * F, K, lda, ldw, ldgu, dtype, status)) return rc;
  g.epilogue = EPI_SWIGLU; g.E = ACT; g.lde = ldact;
  return nnb_gemm2_launch(g, st);
}

// qkv[M, N] = x[M, K] @ w[N, K]^T with rotate-half RoPE applied to columns [0, rope_cols) (heads of head_dim columns, row m
// at position m % t_len; cos / sin: fp32 [t_len, head_dim / 2]); the remaining columns (V) pass through.
extern "C" int nnb_gemm_rope(const void* X, const void* W, void* QKV, const void* cos_t, const void* sin_t, int M, int N, int K,
                             long long lda, long long ldw, long long ldd, int t_len, int rope_cols, int head_dim, int dtype,
                             void* status, cudaStream_t st) {
  NnbGemm2Args g{};
  if (int rc = fused_gemm_common(g, X, W, QKV, M, N, K, lda, ldw, ldd, dtype, status)) return rc;
  g.epilogue = EPI_ROPE; g.cos_t = cos_t; g.sin_t = sin_t; g.t_len = t_len; g.rope_cols = rope_cols; g.head_dim = head_dim;
  return nnb_gemm2_launch(g, st);
}

// dgu[M, 2F] = SwiGLU backward of (dy[M, K] @ w_down[K, F]) against the saved projection gu[M, 2F]: the gradient of the
// activation is formed in tensor memory and leaves as d(gate) | d(up), never as a tensor of its own. w_down is the
// row-parallel weight as stored ([K = d_model, F], i.e. MN-major for this product).
extern "C" int nnb_gemm_swiglu_bwd(const void* dY, const void* Wdown, const void* GU, void* dGU, int M, int F, int K, long long lda,
                                   long long ldw, long long ldgu, long long lddgu, int dtype, void* status, cudaStream_t st) {
  NnbGemm2Args g{};
  if (int rc = fused_gemm_common(g, dY, Wdown, dGU, M, F, K, lda, ldw, lddgu, dtype, status)) return rc;
  g.b_mn = 1;
  g.epilogue = EPI_SWIGLU_BWD; g.E = const_cast<void*>(GU); g.lde = ldgu;
  return nnb_gemm2_launch(g, st);
}

// logits[M, N] = x[M, K] @ w[N, K]^T (16-bit) plus stats[M, 2 ceil(N / 256), 2] = (max, sum of exp(x - max)) of every row in
// two parts per 256-column tile (its even and its odd 64-column chunks), computed on the stored (rounded) logits; a part
// without columns holds (-inf, 0). N must be a multiple of 64.
extern "C" int nnb_gemm_ce_stats(const void* X, const void* W, void* logits, void* stats, int M, int N, int K, long long lda,
                                 long long ldw, long long ldd, int dtype, void* status, cudaStream_t st) {
  NnbGemm2Args g{};
  if (int rc = fused_gemm_common(g, X, W, logits, M, N, K, lda, ldw, ldd, dtype, status)) return rc;
  g.epilogue = EPI_CE_STATS; g.stats = stats;
  return nnb_gemm2_launch(g, st);
}

// GEMM -> reduce-scatter in one kernel (row-parallel linear under tensor + sequence parallelism):
//   out_shard[rank r] [M / world, N]  +=  (A[M, K] @ B[N, K]^T) rows [r M / world, (r + 1) M / world)   summed over ranks.
// Every output tile is TMA-reduce-added into the owner's buffer over NVLink as soon as it leaves TMEM, so the
// transfer overlaps the math tile by tile. out_ptrs: every rank's shard buffer (symmetric memory), ZEROED by its
// owner earlier on this stream; the kernel itself waits until every rank has done so and, before it ends, until
// every rank has finished adding. local_flags: device uint32[>= 2], zero before the first call.
extern "C" int nnb_gemm_rs_bf16(const void* A, const void* B, void* const* out_ptrs, void* const* flag_ptrs, void* local_flags,
                                void* comm_status, int rank, int world, int epoch, int M, int N, int K, long long lda,
                                long long ldb, long long ldd, int b_mn, int dtype, int out_f32, void* status, cudaStream_t st) {
  CommArgs c{1, world, rank, 0, out_ptrs, flag_ptrs, local_flags, comm_status, epoch};
  return gemm_impl(A, B, nullptr, M, N, K, lda, ldb, ldd, 0, b_mn, dtype, out_f32, 1, 1, 0, 0, status, &c, st);
}

// all-gather -> GEMM in one kernel (column-parallel linear under tensor + sequence parallelism):
//   D[M, N] = A_full[M, K] @ B[N, K]^T where rank r owns rows [r M / world, (r + 1) M / world) of A_full.
// a_ptrs: every rank's full-size A buffer (symmetric memory) holding valid data in ITS OWN row range; the first
// gather_ctas CTAs copy the peers' ranges into this rank's buffer m-block by m-block while the other CTAs
// multiply, starting with the local rows. local_flags: device uint32[2 + M / 128], zero before the first call.
extern "C" int nnb_ag_gemm_bf16(void* const* a_ptrs, const void* B, void* D, void* const* flag_ptrs, void* local_flags,
                                void* comm_status, int rank, int world, int epoch, int gather_ctas, int M, int N, int K,
                                long long ldb, long long ldd, int b_mn, int dtype, void* status, cudaStream_t st) {
  CommArgs c{2, world, rank, gather_ctas, a_ptrs, flag_ptrs, local_flags, comm_status, epoch};
  return gemm_impl(a_ptrs[rank], B, D, M, N, K, K, ldb, ldd, 0, b_mn, dtype, 0, 0, 1, 0, 0, status, &c, st);
}

// parameter all-gather -> GEMM in one kernel (first linear of an FSDP unit):
//   D[M, N] = A[M, K] @ B[N, K]^T where B lives b_off bytes into a unit of parameters whose bytes are sharded evenly over the
//   ranks: rank r holds bytes [r per_bytes, (r + 1) per_bytes) of the unit in ITS wire buffer at src_off. The first
//   gather_ctas CTAs copy all shards of the WHOLE unit into unit_dst (this rank's unsharded copy), B's chunks first; the
//   other CTAs multiply, each waiting only for the chunks under its own B tile. local_flags: device uint32
//   [2 + world * ceil(per_bytes / 32768)], zero before the first call. After the kernel the whole unit is valid in unit_dst.
extern "C" int nnb_gather_b_gemm_bf16(const void* A, void* const* wire_ptrs, void* unit_dst, void* D, void* const* flag_ptrs,
                                      void* local_flags, void* comm_status, int rank, int world, int epoch, int gather_ctas,
                                      long long src_off, long long per_bytes, long long b_off, int M, int N, int K, long long lda,
                                      long long ldd, int dtype, void* status, cudaStream_t st) {
  CommArgs c{3, world, rank, gather_ctas, wire_ptrs, flag_ptrs, local_flags, comm_status, epoch};
  c.src_off = src_off; c.per_bytes = per_bytes; c.b_off = b_off; c.dst = unit_dst;
  NNB_REQUIRE(b_off % 16 == 0 && b_off >= 0 && b_off + (long long)N * K * 2 <= per_bytes * world, "gather_b_gemm: B outside the unit");
  const void* B = static_cast<const uint8_t*>(unit_dst) + b_off;
  return gemm_impl(A, B, D, M, N, K, lda, K, ldd, 0, 0, dtype, 0, 0, 1, 256, 0, status, &c, st);
}

// MXFP8 GEMM on the block-scaled tensor-core path: D[M, N] (+)= (A * sfa) (B * sfb)^T.
//   A: e4m3 bytes [M, K] row-major (lda bytes per row), B: e4m3 bytes [N, K]; both contract along their rows (K-major).
//   sfa / sfb: e8m0 scales, one per 32 K-elements of every row, in the chunked layout written by nnb_mxfp8_quantize_sw:
//   chunk [row / 128][k / 128] of 512 bytes, scale of (row, k-block) at byte (row % 32) * 16 + ((row % 128) / 32) * 4 + (k / 32) % 4.
//   D: bf16 (out_f32 = 0) or fp32 (out_f32 = 1; accumulate adds into D; split-K partial tiles are reduce-added).
// M, N and K must be multiples of 128. The reference has no FP8 GEMM of its own (it defers to Transformer Engine,
// nanonemo/te/__init__.py:20-39).
extern "C" int nnb_gemm_mxfp8(const void* A, const void* sfa, const void* B, const void* sfb, void* D, int M, int N, int K,
                              long long lda, long long ldb, long long ldd, int out_f32, int accumulate, int k_splits, int max_ctas,
                              void* status, cudaStream_t st) {
  constexpr int BN = 128, KB = 2 * BK;
  NNB_REQUIRE(M > 0 && N > 0 && K > 0 && M % 128 == 0 && N % 128 == 0 && K % 128 == 0,
              "gemm_mxfp8: M=%d, N=%d, K=%d must be positive multiples of 128", M, N, K);
  NNB_REQUIRE(!accumulate || out_f32, "gemm_mxfp8: accumulate needs an fp32 output");
  NNB_REQUIRE(lda % 16 == 0 && ldb % 16 == 0 && nnb_aligned16(A) && nnb_aligned16(B) && nnb_aligned16(sfa) && nnb_aligned16(sfb),
              "gemm_mxfp8: operands and scales must be 16-byte aligned with row strides that are multiples of 16");
  const int sms = max_ctas > 0 ? min(max_ctas, nnb_num_sms()) : nnb_num_sms();
  Params p{};
  p.M = M; p.N = N; p.K = K;
  p.m_blocks = M / BM;
  p.n_blocks = N / BN;
  p.kblocks_total = K / KB;
  int splits = 1;
  if (out_f32) {
    if (k_splits > 0) splits = k_splits;
    else {
      const long long tiles = (long long)p.m_blocks * p.n_blocks;
      const int s_max = max(1, min(32, p.kblocks_total / 4));
      double best = 1e30;
      for (int sp = 1; sp <= s_max; ++sp) {
        const double cost = (double)((tiles * sp + sms - 1) / sms) / sp + 0.002 * sp;
        if (cost < best - 1e-9) { best = cost; splits = sp; }
      }
    }
    splits = max(1, min(splits, p.kblocks_total));
  }
  p.kblocks_per_split = (p.kblocks_total + splits - 1) / splits;
  p.k_splits = (p.kblocks_total + p.kblocks_per_split - 1) / p.kblocks_per_split;
  p.group_m = 1;
  {
    int g = 1;
    while ((g + 1) * (g + 1) * BM <= sms * BN) ++g;
    if (p.n_blocks * g > sms) p.group_m = min(g, p.m_blocks);
  }
  p.out_f32 = out_f32 ? 1 : 0;
  p.reduce_add = (accumulate || p.k_splits > 1) ? 1 : 0;
  p.idesc = sm100::make_idesc_mxf8(BM, BN);
  p.out_bf16 = 1;
  p.sfa = static_cast<const uint8_t*>(sfa);
  p.sfb = static_cast<const uint8_t*>(sfb);
  p.status = static_cast<int*>(status);
  CUtensorMap tmA, tmB;
  DMaps tmDs;
  if (!nnb_make_tmap_2d(&tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, A, M, K, lda, BM, KB, "gemm_mxfp8 A")) return -4;
  if (!nnb_make_tmap_2d(&tmB, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, B, N, K, ldb, BN, KB, "gemm_mxfp8 B")) return -4;
  const CUtensorMapDataType d_dt = out_f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const int d_bytes = out_f32 ? 4 : 2, d_box = out_f32 ? 32 : 64;
  if (!nnb_make_tmap_2d(&tmDs.m[0], d_dt, d_bytes, D, M, N, ldd * d_bytes, BM, d_box, "gemm_mxfp8 D")) return -4;
  for (int r = 1; r < 8; ++r) tmDs.m[r] = tmDs.m[0];
  if (out_f32 && !accumulate && p.k_splits > 1) {
    if (ldd == N) cudaMemsetAsync(D, 0, (size_t)M * N * 4, st);
    else cudaMemset2DAsync(D, ldd * 4, 0, (size_t)N * 4, M, st);
  }
  const int items = p.m_blocks * p.n_blocks * p.k_splits;
  const int rc = launch<BN, true>(tmA, tmB, tmDs, p, min(items, sms), st);
  if (rc != 0) return rc;
  NNB_LAUNCH_OK("gemm_mxfp8");
  return 0;
}
