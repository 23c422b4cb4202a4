// bf16/fp16 GEMM with CTA PAIRS on the 5th-generation tensor cores: D[M,N] (+)= A[M,K] * B[N,K]^T, fp32 accumulate.
//
// Two CTAs of a cluster (two SMs) own one 256 x 256 output tile. Each CTA loads its own 128 rows of A and its own
// 128 of the 256 rows of B; ONE thread of the even ("leader") CTA issues tcgen05.mma.cta_group::2 (M = 256), which
// reads A and B from the shared memory of both CTAs and accumulates each CTA's 128 rows into that CTA's own tensor
// memory. Per 128 x 256 of output a CTA therefore stages 32 KB per k-block instead of the 48 KB of the single-CTA
// kernel (gemm.cu): the L2 -> shared-memory fill, which bounds these GEMMs at K = 768..2048, drops by a third.
// No multicast is used: every CTA fetches its own tiles; the pair is coupled only through
//   * TMA loads of both CTAs completing on the leader's "full" barrier (cta_group::2 form of the load),
//   * tcgen05.commit.cta_group::2 arriving on the "empty" / "accumulator full" barriers of BOTH CTAs (one commit per CTA),
//   * the peer's epilogue warps arriving remotely on the leader's "accumulator empty" barrier.
// Roles per CTA as in gemm.cu: warp 0 TMA producer, warp 1 MMA issuer (leader only; both allocate TMEM), warps 2..5
// epilogue (tcgen05.ld -> swizzled staging -> TMA store / reduce-add). All waits are bounded.
// Replaces the cuBLAS calls behind nn.Linear in the reference (nanonemo/model/layers.py:80-83, 128-130).
//
// Fused epilogues (template parameter EPI), each replacing a separate pass over HBM of the reference's elementwise kernels:
//   EPI_SWIGLU    gate||up projection: the leader stages 128 GATE rows of the weight, its peer the matching 128 UP rows, so
//                 one accumulator holds gate (columns 0..127) and up (128..255) of the same 128 features; the epilogue
//                 writes both halves of the projection (kept for backward) AND act = silu(gate) * up
//                 (nanonemo/kernels/triton/swiglu.py:19-38).
//   EPI_ROPE      QKV projection: rotate-half RoPE applied to the query / key heads while the tile leaves tensor memory
//                 (one cos / sin row per token; a 64-column chunk is one head, two chunks at head_dim 128)
//                 (nanonemo/kernels/triton/rope.py:18-47).
//   EPI_CE_STATS  LM head: besides the 16-bit logits, every (row, 256-column tile) gets its (max, sum of exp(x - max)), so
//                 the cross-entropy kernel needs one sweep over the logits instead of two
//                 (nanonemo/kernels/triton/linear_ce.py:21-41).
// All three compute on the values ROUNDED to the 16-bit output type, so they match the unfused kernels bit for bit.
#include "gemm2.cuh"

#include "common.cuh"
#include "sm100.cuh"

namespace {

using namespace sm100;

constexpr int BM = 128;   // rows per CTA (256 per pair)
constexpr int BN = 256;   // columns per pair tile; each CTA stages BN / 2 rows of B
constexpr int BK = 64;
constexpr int kEpilogueThreads = 128;  // one epilogue GROUP: four warps, one per tensor-memory lane quadrant
constexpr int kStageBytesA = BM * BK * 2, kStageBytesB = (BN / 2) * BK * 2, kStageBytes = kStageBytesA + kStageBytesB;
constexpr int kTmemCols = 512;
// The SwiGLU epilogue fills three staging tiles per 64-feature round (gate, up, act); its backward keeps two (gate, up)
// tile pairs in flight: both pay for the staging with one stage of the operand ring.
template <int EPI> struct Cfg {
  static constexpr int kStages = (EPI == EPI_SWIGLU || EPI == EPI_SWIGLU_BWD) ? 5 : 6;
  static constexpr int kStagingTiles = EPI == EPI_SWIGLU ? 3 : (EPI == EPI_SWIGLU_BWD ? 4 : 2);
  static constexpr int kStagingBytes = kStagingTiles * BM * 128;
  // Epilogue groups of four warps. The SwiGLU backward does the most arithmetic per accumulator element (a sigmoid and both
  // products, operands read from shared memory): two groups take alternate 64-column chunks, each with its own staging
  // pair, barrier and elected thread, so one group's stores and loads overlap the other's arithmetic.
  // The softmax statistics (an exponential per logit) get the same split, one staging tile per group.
  // (The SwiGLU forward stays with one group: a second one needs six staging tiles, which leaves four operand stages, and
  // measured slower: 0.201 vs 0.182 ms at M = 32768, N = 4096, K = 768.)
  static constexpr int kEpiGroups = (EPI == EPI_SWIGLU_BWD || EPI == EPI_CE_STATS) ? 2 : 1;
  static constexpr int kThreads = 64 + kEpiGroups * kEpilogueThreads;
  static constexpr int kSmemBytes = kStages * kStageBytes + kStagingBytes + 1024 + 256;
};

struct Params2 {
  int M, N, K;
  int m_pairs, n_blocks, k_splits, kblocks_total, kblocks_per_split;
  int group_m;  // tile order: groups of group_m 256-row blocks are swept n-block by n-block
  int a_mn, b_mn, out_f32, reduce_add, out_bf16;
  uint32_t idesc;
  int* status;
  // fused epilogues
  int epi_cols;        // EPI_SWIGLU: F (the up rows of the weight start at row F); EPI_ROPE: columns that are rotated
  int t_len, half_dim; // EPI_ROPE: sequence length (row m uses table row m % t_len), head_dim / 2
  const float* cos_t;  // EPI_ROPE: [t_len, half_dim] fp32
  const float* sin_t;
  float* stats;        // EPI_CE_STATS: [M, 2 n_blocks, 2] fp32 (max, sum of exp(x - max)): two entries per 256-column tile (64-column
                       // chunks 0, 2 and 1, 3 of the tile: one entry per epilogue warp group; (-inf, 0) when the group had no chunk)
};

__device__ __forceinline__ uint32_t pack16(float lo, float hi, bool bf) {
  if (bf) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float2 unpack16(uint32_t w, bool bf) {
  if (bf) return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&w));
  return __half22float2(*reinterpret_cast<__half2*>(&w));
}
__device__ __forceinline__ float round16(float x, bool bf) {
  return bf ? __bfloat162float(__float2bfloat16_rn(x)) : __half2float(__float2half_rn(x));
}
// 32 consecutive columns (16 packed words) of this thread's row into 16-byte units [u0, u0 + 4) of a swizzled staging row.
__device__ __forceinline__ void stage32(uint8_t* my_row, int sw, int u0, const uint32_t (&w)[16]) {
#pragma unroll
  for (int j = 0; j < 4; ++j)
    *reinterpret_cast<uint4*>(my_row + (((u0 + j) ^ sw) << 4)) = make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
}
// Rotate-half on 32 (lo, hi) column pairs of one token: lo' = lo c - hi s, hi' = lo s + hi c, computed on the rounded values.
__device__ __forceinline__ void rope32(uint32_t (&lo)[32], uint32_t (&hi)[32], const float (&cc)[32], const float (&ss)[32], bool bf) {
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const float a = round16(__uint_as_float(lo[i]), bf), b = round16(__uint_as_float(hi[i]), bf);
    lo[i] = __float_as_uint(a * cc[i] - b * ss[i]);
    hi[i] = __float_as_uint(a * ss[i] + b * cc[i]);
  }
}
// 32 consecutive fp32 table entries of one token (16-byte aligned: the tables have 32 or 64 entries per row).
__device__ __forceinline__ void load_table32(const float* __restrict__ src, float (&dst)[32]) {
#pragma unroll
  for (int i = 0; i < 32; i += 4) {
    const float4 v = __ldg(reinterpret_cast<const float4*>(src + i));
    dst[i] = v.x; dst[i + 1] = v.y; dst[i + 2] = v.z; dst[i + 3] = v.w;
  }
}
__device__ __forceinline__ void pack32(const uint32_t (&r)[32], uint32_t (&w)[16], bool bf) {
#pragma unroll
  for (int e = 0; e < 16; ++e) w[e] = pack16(__uint_as_float(r[2 * e]), __uint_as_float(r[2 * e + 1]), bf);
}

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// TMA tile load issued by either CTA of the pair; the bytes are counted on the LEADER's mbarrier.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* m, uint32_t leader_bar, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
               ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(leader_bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}"
               ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrive on ONE mbarrier (a shared::cluster address, own or the peer's) once the pair MMAs issued so far have completed.
__device__ __forceinline__ void umma_commit_pair(uint32_t cluster_bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_bar) : "memory");
}

// BF16: the 16-bit format of operands and output (false = fp16). A template parameter rather than a launch argument so that the
// epilogues' conversions are straight-line code: with a run-time flag every pack / unpack is a branch, the unrolled per-element
// arithmetic is cut into hundreds of basic blocks and the epilogue warps (two per scheduler at most) lose the overlap between
// independent elements that hides the special-function and conversion latencies.
template <int EPI, bool BF16>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(Cfg<EPI>::kThreads, 1)
gemm2_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                     const __grid_constant__ CUtensorMap tmD, const __grid_constant__ CUtensorMap tmE, const Params2 p) {
  constexpr int kStages = Cfg<EPI>::kStages, kStagingBytes = Cfg<EPI>::kStagingBytes;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stage_base = smem;
  uint8_t* staging = smem + kStages * kStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(staging + kStagingBytes);
  const uint32_t bar_full = smem_u32(bars), bar_empty = bar_full + 8 * kStages;
  const uint32_t bar_tfull = bar_empty + 8 * kStages, bar_tempty = bar_tfull + 16;
  const uint32_t bar_in = bar_tempty + 16;  // EPI_SWIGLU_BWD: the (gate, up) tiles of staging pair 0 / 1 have landed
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 6);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* epi_abort_base = abort_flag + 1;  // one word per epilogue group

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar_full + 8 * s, 1);    // leader: its producer's expect-tx arrival (bytes of both CTAs)
      mbar_init(bar_empty + 8 * s, 1);   // one commit per CTA
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(bar_tfull + 8 * a, 1);
      mbar_init(bar_tempty + 8 * a, 2 * Cfg<EPI>::kEpiGroups * (kEpilogueThreads / 32));  // leader: epilogue warps of both CTAs
      mbar_init(bar_in + 8 * a, 1);
    }
    *abort_flag = 0;
    epi_abort_base[0] = 0;
    epi_abort_base[1] = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  if (warp == 1) {
    tmem_alloc2(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish2();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    tma_prefetch_desc(&tmD);
    if (EPI == EPI_SWIGLU || EPI == EPI_SWIGLU_BWD) tma_prefetch_desc(&tmE);
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before anybody signals the peer
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int items = p.m_pairs * p.n_blocks * p.k_splits;
  const int pair0 = (int)blockIdx.x >> 1, npairs = (int)gridDim.x >> 1;
  int fail_role = 0, fail_item = -1;
  // consecutive tiles (the ones the persistent pairs work on at the same time) cover group_m x (pairs / group_m) blocks
  auto tile_coords = [&](int tile, int& m_pair, int& n_blk) {
    const int per_group = p.group_m * p.n_blocks, g = tile / per_group, r = tile - g * per_group;
    const int gm = min(p.group_m, p.m_pairs - g * p.group_m);
    m_pair = g * p.group_m + r % gm;
    n_blk = r / gm;
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      const uint32_t leader_full0 = map_to_cta(bar_full, 0);  // the same barrier slot in the even CTA of the pair
      for (int item = pair0; item < items && ok; item += npairs) {
        const int ks = item % p.k_splits, tile = item / p.k_splits;
        int m_pair, n_blk;
        tile_coords(tile, m_pair, n_blk);
        const int m_row0 = (m_pair * 2 + (int)rank) * BM;
        // SwiGLU: the leader stages gate rows, the peer the up rows (F further down) of the same 128 features
        const int n_row0 = EPI == EPI_SWIGLU ? n_blk * (BN / 2) + (int)rank * p.epi_cols : n_blk * BN + (int)rank * (BN / 2);
        const int kb0 = ks * p.kblocks_per_split, kb1 = min(kb0 + p.kblocks_per_split, p.kblocks_total);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const uint32_t s = it % kStages, ph = (it / kStages) & 1;
          if (!mbar_wait(bar_empty + 8 * s, ph ^ 1, abort_flag)) { ok = false; fail_role = 1; fail_item = item; break; }
          const uint32_t full = bar_full + 8 * s, leader_full = leader_full0 + 8 * s;
          if (rank == 0) mbar_expect_tx(full, 2 * kStageBytes);
          const uint32_t sa = smem_u32(stage_base + s * kStageBytes), sb = sa + kStageBytesA;
          if (!p.a_mn) {
            tma_load_2d_pair(sa, &tmA, leader_full, kb * BK, m_row0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d_pair(sa + j * (BK * 128), &tmA, leader_full, m_row0 + j * 64, kb * BK);
          }
          if (!p.b_mn) {
            tma_load_2d_pair(sb, &tmB, leader_full, kb * BK, n_row0);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 128; ++j) tma_load_2d_pair(sb + j * (BK * 128), &tmB, leader_full, n_row0 + j * 64, kb * BK);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && rank == 0) {
      uint32_t it = 0, tile_iter = 0;
      bool ok = true;
      const uint32_t a_step = p.a_mn ? (16 * 128) >> 4 : 32 >> 4, b_step = p.b_mn ? (16 * 128) >> 4 : 32 >> 4;
      const uint32_t a_lbo = p.a_mn ? BK * 128 : 16, b_lbo = p.b_mn ? BK * 128 : 16;
      const uint32_t peer_empty = map_to_cta(bar_empty, 1), peer_tfull = map_to_cta(bar_tfull, 1);
      for (int item = pair0; item < items && ok; item += npairs, ++tile_iter) {
        const int ks = item % p.k_splits;
        const int kb0 = ks * p.kblocks_per_split, kb1 = min(kb0 + p.kblocks_per_split, p.kblocks_total);
        const uint32_t acc = tile_iter & 1, acc_ph = (tile_iter >> 1) & 1;
        if (!mbar_wait(bar_tempty + 8 * acc, acc_ph ^ 1, abort_flag)) { ok = false; fail_role = 2; fail_item = item; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const uint32_t s = it % kStages, ph = (it / kStages) & 1;
          if (!mbar_wait(bar_full + 8 * s, ph, abort_flag)) { ok = false; fail_role = 2; fail_item = item; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(stage_base + s * kStageBytes), sb = sa + kStageBytesA;
          const uint64_t da = make_smem_desc(sa, a_lbo, 1024), db = make_smem_desc(sb, b_lbo, 1024);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            umma_f16_pair(d_tmem, da + (uint64_t)(k * a_step), db + (uint64_t)(k * b_step), p.idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          umma_commit_pair(bar_empty + 8 * s);    // this CTA's stage is free once the MMAs have read it
          umma_commit_pair(peer_empty + 8 * s);   // ... and so is the peer's
        }
        if (ok) {
          umma_commit_pair(bar_tfull + 8 * acc);
          umma_commit_pair(peer_tfull + 8 * acc);
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5, both CTAs)
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const int grp = Cfg<EPI>::kEpiGroups == 1 ? 0 : (threadIdx.x - 64) / kEpilogueThreads;  // epilogue group
    const int et = (threadIdx.x - 64) % kEpilogueThreads;           // thread within the group; et == 0 issues its TMA traffic
    const int epi_bar = 1 + grp;                                    // the group's named barrier
    volatile int* epi_abort = epi_abort_base + grp;
    uint32_t tile_iter = 0, gchunk = 0;
    uint32_t in_count = 0;  // EPI_SWIGLU_BWD: loads this group has consumed from its staging pair (parity of the next wait)
    int pending_stores = 0;
    const uint32_t leader_tempty = map_to_cta(bar_tempty, 0);
    for (int item = pair0; item < items; item += npairs, ++tile_iter) {
      const int tile = item / p.k_splits;
      int m_pair, n_blk;
      tile_coords(tile, m_pair, n_blk);
      const int d_row = (m_pair * 2 + (int)rank) * BM;
      const uint32_t acc = tile_iter & 1, acc_ph = (tile_iter >> 1) & 1;
      float rope_c[32], rope_s[32];  // EPI_ROPE, head_dim 64: this token's table row, fetched while the tile is still being multiplied
      if constexpr (EPI == EPI_ROPE) {
        if (p.half_dim == 32 && n_blk * BN < p.epi_cols) {
          const int t = (d_row + row) % p.t_len;
          load_table32(p.cos_t + (size_t)t * 32, rope_c);
          load_table32(p.sin_t + (size_t)t * 32, rope_s);
        }
      }
      // EPI_SWIGLU_BWD: the saved (gate, up) values of this tile arrive by TMA in 64-column chunks; group g takes chunks g,
      // g + 2 into staging pair g. Its first chunk is requested here, while the tile is still being multiplied.
      int bwd_chunks = 0;
      auto load_gu_chunk = [&](int c) {  // the group's thread et == 0 only; its staging pair must not be the source of a store in flight
        const uint32_t bar = bar_in + 8 * grp, dst = smem_u32(staging + grp * 2 * (BM * 128));
        mbar_expect_tx(bar, 2 * BM * 128);
        tma_load_2d(dst, &tmE, bar, n_blk * BN + c * 64, d_row);
        tma_load_2d(dst + BM * 128, &tmE, bar, p.N + n_blk * BN + c * 64, d_row);
      };
      if constexpr (EPI == EPI_SWIGLU_BWD) {
        if (d_row < p.M) bwd_chunks = min(BN / 64, (p.N - n_blk * BN) / 64);
        if (et == 0) {
          if (grp < bwd_chunks) {
            if (pending_stores > 0) tma_wait_group_read<0>();
            load_gu_chunk(grp);
          }
          // The group's loads form a chain (a pair is reloaded only after its stores have drained), so their latency is
          // exposed: pull this tile's later chunk and the NEXT tile's chunks into L2 now, a whole tile ahead of their use.
          auto prefetch_gu = [&](int nb, int r0, int c) {
            tma_prefetch_l2_2d(&tmE, nb * BN + c * 64, r0);
            tma_prefetch_l2_2d(&tmE, p.N + nb * BN + c * 64, r0);
          };
          if (grp + 2 < bwd_chunks) prefetch_gu(n_blk, d_row, grp + 2);
          if (item + npairs < items) {
            int m2, n2;
            tile_coords((item + npairs) / p.k_splits, m2, n2);
            const int r2 = (m2 * 2 + (int)rank) * BM;
            const int ch2 = r2 < p.M ? min(BN / 64, (p.N - n2 * BN) / 64) : 0;
            for (int c = grp; c < ch2; c += 2) prefetch_gu(n2, r2, c);
          }
        }
      }
      const bool ok = mbar_wait(bar_tfull + 8 * acc, acc_ph, abort_flag);
      if (!ok) { fail_role = 3; fail_item = item; }
      if (et == 0) *epi_abort = *abort_flag;
      named_barrier_sync(epi_bar, kEpilogueThreads);
      if (*epi_abort) {
        if constexpr (EPI == EPI_SWIGLU_BWD) {  // the tile loads requested above must have landed before shared memory is given up
          if (grp < bwd_chunks) mbar_wait(bar_in + 8 * grp, (in_count++) & 1, abort_flag);
        }
        break;
      }
      tc_fence_after();
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN;
      const bool rows_live = d_row < p.M;  // an odd number of 128-row blocks leaves the peer's last block outside the matrix
      constexpr bool bf = BF16;
      const int sw = row & 7;
      if constexpr (EPI == EPI_SWIGLU) {
        // accumulator columns [0, 128) = gate, [128, 256) = up of features n_blk * 128 ...; 64 features per round, all three
        // staging tiles (gate | up | act) filled in two half rounds of 32 columns, then three TMA stores
        const int F = p.epi_cols;
        uint8_t* tiles = staging + grp * 3 * (BM * 128);  // this group's gate | up | act staging tiles
        for (int c = grp; c < 2 && rows_live; c += Cfg<EPI>::kEpiGroups) {
          const int fcol = n_blk * (BN / 2) + c * 64;
          if (fcol >= F) break;
          if (et == 0 && pending_stores > 0) tma_wait_group_read<0>();
          named_barrier_sync(epi_bar, kEpilogueThreads);
          uint8_t* row_g = tiles + row * 128;
          uint8_t* row_u = row_g + BM * 128;
          uint8_t* row_a = row_u + BM * 128;
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint32_t g[32], u[32], wg[16], wu[16], wa[16];
            tmem_ld_32x32b_x32(t_row + c * 64 + h * 32, g);
            tmem_ld_32x32b_x32(t_row + BN / 2 + c * 64 + h * 32, u);
            tmem_ld_wait();
            pack32(g, wg, bf);
            pack32(u, wu, bf);
#pragma unroll
            for (int e = 0; e < 16; ++e) {
              const float2 gg = unpack16(wg[e], bf), uu = unpack16(wu[e], bf);
              wa[e] = pack16(gg.x / (1.f + __expf(-gg.x)) * uu.x, gg.y / (1.f + __expf(-gg.y)) * uu.y, bf);
            }
            stage32(row_g, sw, h * 4, wg);
            stage32(row_u, sw, h * 4, wu);
            stage32(row_a, sw, h * 4, wa);
          }
          fence_proxy_async_smem();
          named_barrier_sync(epi_bar, kEpilogueThreads);
          if (et == 0) {
            tma_store_2d(&tmD, smem_u32(tiles), fcol, d_row);
            tma_store_2d(&tmD, smem_u32(tiles + BM * 128), F + fcol, d_row);
            tma_store_2d(&tmE, smem_u32(tiles + 2 * BM * 128), fcol, d_row);
            tma_commit_group();
          }
          pending_stores = 1;
        }
      } else if constexpr (EPI == EPI_SWIGLU_BWD) {
        // accumulator = d(act); the group's staging pair holds gate | up of the chunk's 64 features for this CTA's 128 rows
        // (same swizzled layout the stores use). Each thread turns its own row's slots into d(gate) | d(up) in place:
        //   s = sigmoid(g), d(gate) = d(act) u s (1 + g (1 - s)), d(up) = d(act) g s
        // then the two tiles are stored at columns col and F + col of the projection's gradient.
        for (int c = grp; c < bwd_chunks; c += 2) {
          uint8_t* g_tile = staging + grp * 2 * (BM * 128);
          if (!mbar_wait(bar_in + 8 * grp, (in_count++) & 1, abort_flag)) { fail_role = 3; fail_item = item; }
          uint32_t r0[32], r1[32];
          tmem_ld_32x32b_x32(t_row + c * 64, r0);
          tmem_ld_32x32b_x32(t_row + c * 64 + 32, r1);
          tmem_ld_wait();
          uint8_t* row_g = g_tile + row * 128;
          uint8_t* row_u = row_g + BM * 128;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            uint4* pg = reinterpret_cast<uint4*>(row_g + ((j ^ sw) << 4));
            uint4* pu = reinterpret_cast<uint4*>(row_u + ((j ^ sw) << 4));
            const uint4 gw = *pg, uw = *pu;
            const uint32_t gin[4] = {gw.x, gw.y, gw.z, gw.w}, uin[4] = {uw.x, uw.y, uw.z, uw.w};
            uint32_t og[4], ou[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int i = (j & 3) * 8 + 2 * e;
              const float d0 = __uint_as_float(j < 4 ? r0[i] : r1[i]), d1 = __uint_as_float(j < 4 ? r0[i + 1] : r1[i + 1]);
              const float2 g2 = unpack16(gin[e], bf), u2 = unpack16(uin[e], bf);
              const float s0 = 1.f / (1.f + __expf(-g2.x)), s1 = 1.f / (1.f + __expf(-g2.y));
              og[e] = pack16(d0 * u2.x * s0 * (1.f + g2.x * (1.f - s0)), d1 * u2.y * s1 * (1.f + g2.y * (1.f - s1)), bf);
              ou[e] = pack16(d0 * g2.x * s0, d1 * g2.y * s1, bf);
            }
            *pg = make_uint4(og[0], og[1], og[2], og[3]);
            *pu = make_uint4(ou[0], ou[1], ou[2], ou[3]);
          }
          fence_proxy_async_smem();
          named_barrier_sync(epi_bar, kEpilogueThreads);
          if (et == 0) {
            const int col = n_blk * BN + c * 64;
            tma_store_2d(&tmD, smem_u32(g_tile), col, d_row);
            tma_store_2d(&tmD, smem_u32(g_tile + BM * 128), p.N + col, d_row);
            tma_commit_group();
            if (c + 2 < bwd_chunks) {
              tma_wait_group_read<0>();  // the stores just issued have left this pair: it can take the chunk after next
              load_gu_chunk(c + 2);
            }
          }
          pending_stores = 1;
        }
      } else if constexpr (EPI == EPI_ROPE) {
        if (p.half_dim == 32) {
          // head_dim 64: a 64-column chunk is one head; its two 32-column halves are the rotation partners
          for (int c = 0; c < BN / 64 && rows_live; ++c) {
            const int gcol = n_blk * BN + c * 64;
            if (gcol >= p.N) break;
            uint8_t* buf = staging + (gchunk & 1) * (BM * 128);
            ++gchunk;
            if (et == 0 && pending_stores >= 2) tma_wait_group_read<1>();
            named_barrier_sync(epi_bar, kEpilogueThreads);
            uint32_t r0[32], r1[32], w0[16], w1[16];
            tmem_ld_32x32b_x32(t_row + c * 64, r0);
            tmem_ld_32x32b_x32(t_row + c * 64 + 32, r1);
            tmem_ld_wait();
            if (gcol < p.epi_cols) rope32(r0, r1, rope_c, rope_s, bf);
            pack32(r0, w0, bf);
            pack32(r1, w1, bf);
            stage32(buf + row * 128, sw, 0, w0);
            stage32(buf + row * 128, sw, 4, w1);
            fence_proxy_async_smem();
            named_barrier_sync(epi_bar, kEpilogueThreads);
            if (et == 0) {
              tma_store_2d(&tmD, smem_u32(buf), gcol, d_row);
              tma_commit_group();
            }
            if (pending_stores < 2) ++pending_stores;
          }
        } else {
          // head_dim 128: a head is two chunks; column i of the first rotates with column i of the second, so both
          // staging tiles are filled together (32 column pairs per half round) and stored as two tiles
          const int t = (d_row + row) % p.t_len;
          for (int g = 0; g < BN / 128 && rows_live; ++g) {
            const int gcol = n_blk * BN + g * 128;
            if (gcol >= p.N) break;
            if (et == 0 && pending_stores > 0) tma_wait_group_read<0>();
            named_barrier_sync(epi_bar, kEpilogueThreads);
            uint8_t* row_lo = staging + row * 128;
            uint8_t* row_hi = row_lo + BM * 128;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              uint32_t lo[32], hi[32], w0[16], w1[16];
              tmem_ld_32x32b_x32(t_row + g * 128 + h * 32, lo);
              tmem_ld_32x32b_x32(t_row + g * 128 + 64 + h * 32, hi);
              tmem_ld_wait();
              if (gcol < p.epi_cols) {
                float cc[32], ss[32];
                load_table32(p.cos_t + (size_t)t * 64 + h * 32, cc);
                load_table32(p.sin_t + (size_t)t * 64 + h * 32, ss);
                rope32(lo, hi, cc, ss, bf);
              }
              pack32(lo, w0, bf);
              pack32(hi, w1, bf);
              stage32(row_lo, sw, h * 4, w0);
              stage32(row_hi, sw, h * 4, w1);
            }
            fence_proxy_async_smem();
            named_barrier_sync(epi_bar, kEpilogueThreads);
            if (et == 0) {
              tma_store_2d(&tmD, smem_u32(staging), gcol, d_row);
              tma_store_2d(&tmD, smem_u32(staging + BM * 128), gcol + 64, d_row);
              tma_commit_group();
            }
            pending_stores = 2;
          }
        }
      } else {
        const int cols_per_chunk = p.out_f32 ? 32 : 64;
        const int chunks = BN / cols_per_chunk;
        constexpr int G = Cfg<EPI>::kEpiGroups;  // with two groups: group g takes chunks g, g + 2 through staging tile g
        float st_m = -INFINITY, st_s = 0.f;  // EPI_CE_STATS: this row's running (max, sum of exp) over the group's chunks of the tile
        for (int c = (G == 2 ? grp : 0); c < chunks && rows_live; c += G) {
          const int col0 = c * cols_per_chunk;
          if (n_blk * BN + col0 >= p.N) break;
          uint8_t* buf = staging + (G == 2 ? grp : (int)(gchunk & 1)) * (BM * 128);
          ++gchunk;
          if (G == 2) {
            if (et == 0 && pending_stores >= 1) tma_wait_group_read<0>();
          } else if (et == 0 && pending_stores >= 2) {
            tma_wait_group_read<1>();
          }
          named_barrier_sync(epi_bar, kEpilogueThreads);
          uint8_t* my_row = buf + row * 128;
          if (p.out_f32) {
            uint32_t r[32];
            tmem_ld_32x32b_x32(t_row + col0, r);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 8; ++j)
              *reinterpret_cast<uint4*>(my_row + ((j ^ sw) << 4)) = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
          } else {
            uint32_t r0[32], r1[32], w0[16], w1[16];
            tmem_ld_32x32b_x32(t_row + col0, r0);
            tmem_ld_32x32b_x32(t_row + col0 + 32, r1);
            tmem_ld_wait();
            pack32(r0, w0, bf);
            pack32(r1, w1, bf);
            if constexpr (EPI == EPI_CE_STATS) {
              constexpr float kLog2e = 1.4426950408889634f;
              float x[64];
              float cm = -INFINITY;
#pragma unroll
              for (int e = 0; e < 16; ++e) {
                const float2 a = unpack16(w0[e], bf), b = unpack16(w1[e], bf);
                x[2 * e] = a.x; x[2 * e + 1] = a.y; x[32 + 2 * e] = b.x; x[32 + 2 * e + 1] = b.y;
                cm = fmaxf(cm, fmaxf(fmaxf(a.x, a.y), fmaxf(b.x, b.y)));
              }
              if (cm > st_m) {
                st_s *= exp2f((st_m - cm) * kLog2e);
                st_m = cm;
              }
              const float mb = st_m * kLog2e;
#pragma unroll
              for (int i = 0; i < 64; ++i) st_s += exp2f(x[i] * kLog2e - mb);
            }
            stage32(my_row, sw, 0, w0);
            stage32(my_row, sw, 4, w1);
          }
          fence_proxy_async_smem();
          named_barrier_sync(epi_bar, kEpilogueThreads);
          if (et == 0) {
            if (p.reduce_add) tma_reduce_add_2d(&tmD, smem_u32(buf), n_blk * BN + col0, d_row);
            else tma_store_2d(&tmD, smem_u32(buf), n_blk * BN + col0, d_row);
            tma_commit_group();
          }
          if (pending_stores < 2) ++pending_stores;
        }
        if constexpr (EPI == EPI_CE_STATS) {
          if (rows_live && d_row + row < p.M)
            *reinterpret_cast<float2*>(p.stats + (((size_t)(d_row + row) * p.n_blocks + n_blk) * G + grp) * 2) = make_float2(st_m, st_s);
        }
      }
      // this CTA's half of the accumulator has been read: tell the leader's MMA thread
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (rank == 0) mbar_arrive(bar_tempty + 8 * acc);
        else mbar_arrive_cluster(leader_tempty + 8 * acc);
      }
    }
    if (et == 0) tma_wait_group<0>();
  }

  if (fail_item >= 0 && p.status != nullptr) {
    if (atomicCAS(p.status, 0, 1) == 0) {
      p.status[1] = fail_role;
      p.status[2] = blockIdx.x;
      p.status[3] = fail_item;
    }
  }
  // The peer's shared memory and barriers are in use until the leader's last MMA and commit have completed, and the pair
  // frees its tensor memory together: meet before leaving.
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc2(tmem_base, kTmemCols);
  }
}

}  // namespace

namespace {

template <int EPI, bool BF16>
int max_resident_pairs() {
  static int max_clusters = -1;
  if (max_clusters < 0) {
    auto kern = gemm2_tcgen05_kernel<EPI, BF16>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<EPI>::kSmemBytes) != cudaSuccess) {
      nnb_set_error("gemm2: cannot reserve %d bytes of shared memory", Cfg<EPI>::kSmemBytes);
      cudaGetLastError();
      return -3;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(2 * (nnb_num_sms() / 2));
    cfg.blockDim = dim3(Cfg<EPI>::kThreads);
    cfg.dynamicSmemBytes = Cfg<EPI>::kSmemBytes;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n < 1) { cudaGetLastError(); n = 0; }
    max_clusters = n;
  }
  return max_clusters;
}

template <int EPI, bool BF16>
int launch2(const NnbGemm2Args& a, cudaStream_t st) {
  const int sms = a.max_ctas > 0 ? min(a.max_ctas, nnb_num_sms()) : nnb_num_sms();
  const int resident = max_resident_pairs<EPI, BF16>();
  if (resident < 0) return resident;
  const int pairs = min(sms / 2, resident);  // persistent pairs must all be resident at once
  if (pairs < 1 || a.M < 2 * BM || a.N < BN / 2) return 1;
  Params2 p{};
  p.M = a.M; p.N = a.N; p.K = a.K;
  p.m_pairs = (a.M + 2 * BM - 1) / (2 * BM);
  p.n_blocks = (a.N + BN - 1) / BN;
  p.kblocks_total = (a.K + BK - 1) / BK;
  if (EPI == EPI_SWIGLU) {
    // a.N = 2 F (rows of the gate||up weight); one tile = 128 features = gate and up columns of the same features
    NNB_REQUIRE(!a.out_f32 && !a.a_mn && !a.b_mn && !a.accumulate && a.E != nullptr, "gemm_swiglu: plain K-major 16-bit problem expected");
    NNB_REQUIRE(a.N % 256 == 0, "gemm_swiglu: F = %d must be a multiple of 128", a.N / 2);
    p.epi_cols = a.N / 2;
    p.n_blocks = p.epi_cols / (BN / 2);
  } else if (EPI == EPI_ROPE) {
    NNB_REQUIRE(!a.out_f32 && !a.accumulate, "gemm_rope: 16-bit output expected");
    NNB_REQUIRE((a.head_dim == 64 || a.head_dim == 128) && a.rope_cols % a.head_dim == 0 && a.N % a.head_dim == 0 && a.t_len > 0 &&
                    a.cos_t != nullptr && a.sin_t != nullptr && nnb_aligned16(a.cos_t) && nnb_aligned16(a.sin_t),
                "gemm_rope: head_dim must be 64 or 128, columns whole heads, tables 16-byte aligned");
    p.epi_cols = a.rope_cols; p.t_len = a.t_len; p.half_dim = a.head_dim / 2;
    p.cos_t = static_cast<const float*>(a.cos_t); p.sin_t = static_cast<const float*>(a.sin_t);
  } else if (EPI == EPI_CE_STATS) {
    NNB_REQUIRE(!a.out_f32 && !a.accumulate && a.N % 64 == 0 && a.stats != nullptr, "gemm_ce_stats: 16-bit output with N a multiple of 64 expected");
    p.stats = static_cast<float*>(a.stats);
  } else if (EPI == EPI_SWIGLU_BWD) {
    NNB_REQUIRE(!a.out_f32 && !a.accumulate && a.N % 64 == 0 && a.E != nullptr && nnb_aligned16(a.E) && a.lde % 8 == 0,
                "gemm_swiglu_bwd: 16-bit output, F a multiple of 64 and an aligned saved projection expected");
    p.epi_cols = a.N;
  }
  int splits = 1;
  if (a.out_f32) {
    if (a.k_splits > 0) splits = a.k_splits;
    else {
      const long long tiles = (long long)p.m_pairs * p.n_blocks;
      const int s_max = max(1, min(32, p.kblocks_total / 4));
      double best = 1e30;
      for (int sp = 1; sp <= s_max; ++sp) {
        const double cost = (double)((tiles * sp + pairs - 1) / pairs) / sp + 0.002 * sp;
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
    while ((g + 1) * (g + 1) * 2 * BM <= pairs * BN) ++g;  // least wave footprint: group_m = sqrt(pairs BN / (2 BM))
    if (p.n_blocks * g > pairs) p.group_m = min(g, p.m_pairs);
  }
  p.a_mn = a.a_mn ? 1 : 0;
  p.b_mn = a.b_mn ? 1 : 0;
  p.out_f32 = a.out_f32 ? 1 : 0;
  p.reduce_add = (a.accumulate || p.k_splits > 1) ? 1 : 0;
  p.out_bf16 = a.dtype == NNB_BF16 ? 1 : 0;
  p.idesc = sm100::make_idesc_f16(a.dtype == NNB_BF16 ? 1 : 0, p.a_mn, p.b_mn, 2 * BM, BN);
  p.status = static_cast<int*>(a.status);
  const CUtensorMapDataType in_dt = a.dtype == NNB_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUtensorMap tmA, tmB, tmD, tmE;
  if (!p.a_mn) { if (!nnb_make_tmap_2d(&tmA, in_dt, 2, a.A, a.M, a.K, a.lda * 2, BM, BK, "gemm2 A")) return -4; }
  else         { if (!nnb_make_tmap_2d(&tmA, in_dt, 2, a.A, a.K, a.M, a.lda * 2, BK, 64, "gemm2 A^T")) return -4; }
  if (!p.b_mn) { if (!nnb_make_tmap_2d(&tmB, in_dt, 2, a.B, a.N, a.K, a.ldb * 2, BN / 2, BK, "gemm2 B")) return -4; }
  else         { if (!nnb_make_tmap_2d(&tmB, in_dt, 2, a.B, a.K, a.N, a.ldb * 2, BK, 64, "gemm2 B^T")) return -4; }
  const CUtensorMapDataType d_dt = a.out_f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : in_dt;
  const int d_bytes = a.out_f32 ? 4 : 2, d_box = a.out_f32 ? 32 : 64;
  // (EPI_SWIGLU_BWD writes d(gate) | d(up): its output, like the projection it reads through tmE, is 2 N columns wide)
  const int d_cols = EPI == EPI_SWIGLU_BWD ? 2 * a.N : a.N;
  if (!nnb_make_tmap_2d(&tmD, d_dt, d_bytes, a.D, a.M, d_cols, a.ldd * d_bytes, BM, d_box, "gemm2 D")) return -4;
  tmE = tmD;
  if (EPI == EPI_SWIGLU_BWD && !nnb_make_tmap_2d(&tmE, in_dt, 2, a.E, a.M, 2 * a.N, a.lde * 2, BM, 64, "gemm2 gate|up")) return -4;
  if (EPI == EPI_SWIGLU && !nnb_make_tmap_2d(&tmE, in_dt, 2, a.E, a.M, a.N / 2, a.lde * 2, BM, 64, "gemm2 act")) return -4;
  if (a.out_f32 && !a.accumulate && p.k_splits > 1) {
    if (a.ldd == a.N) cudaMemsetAsync(a.D, 0, (size_t)a.M * a.N * 4, st);
    else cudaMemset2DAsync(a.D, a.ldd * 4, 0, (size_t)a.N * 4, a.M, st);
  }
  const int items = p.m_pairs * p.n_blocks * p.k_splits;
  const int grid = 2 * min(items, pairs);
  gemm2_tcgen05_kernel<EPI, BF16><<<grid, Cfg<EPI>::kThreads, Cfg<EPI>::kSmemBytes, st>>>(tmA, tmB, tmD, tmE, p);
  NNB_LAUNCH_OK("gemm2_tcgen05");
  return 0;
}

}  // namespace

int nnb_gemm2_launch(const NnbGemm2Args& a, cudaStream_t st) {
  switch (a.epilogue) {
#define NNB_LAUNCH2(E) (a.dtype == NNB_BF16 ? launch2<E, true>(a, st) : launch2<E, false>(a, st))
    case EPI_NONE: return NNB_LAUNCH2(EPI_NONE);
    case EPI_SWIGLU: return NNB_LAUNCH2(EPI_SWIGLU);
    case EPI_ROPE: return NNB_LAUNCH2(EPI_ROPE);
    case EPI_CE_STATS: return NNB_LAUNCH2(EPI_CE_STATS);
    case EPI_SWIGLU_BWD: return NNB_LAUNCH2(EPI_SWIGLU_BWD);
#undef NNB_LAUNCH2
    default: nnb_set_error("gemm2: unknown epilogue %d", a.epilogue); return -1;
  }
}
