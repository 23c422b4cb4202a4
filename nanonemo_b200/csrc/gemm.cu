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
#include "sm100.cuh"

namespace {

using namespace sm100;

constexpr int BM = 128;
constexpr int BK = 64;  // 64 x 16-bit = 128 bytes = one swizzle span
constexpr int kThreads = 192;
constexpr int kEpilogueThreads = 128;
constexpr int kStagingBytes = 2 * BM * 128;  // two 128-row x 128-byte staging tiles

template <int BN>
struct Cfg {
  static constexpr int kStageBytesA = BM * BK * 2;
  static constexpr int kStageBytesB = BN * BK * 2;
  static constexpr int kStageBytes = kStageBytesA + kStageBytesB;
  static constexpr int kStages = (BN == 256) ? 4 : (BN == 192 ? 4 : 6);
  static constexpr int kTmemCols = (2 * BN <= 256) ? 256 : 512;  // two accumulators; allocations are powers of two
  static constexpr int kSmemBytes = kStages * kStageBytes + kStagingBytes + 1024 /*align*/ + 256 /*barriers*/;
};

struct Params {
  int M, N, K;
  int m_blocks, n_blocks, k_splits, kblocks_total, kblocks_per_split;
  int a_mn, b_mn;       // operand majors
  int out_f32;          // output dtype: 0 = 16-bit (same as inputs), 1 = fp32
  int reduce_add;       // epilogue uses TMA reduce-add (fp32 only)
  uint32_t idesc;
  int* status;          // device int[4]: {code, role, block, item}; code 0 = ok
};

template <int BN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ CUtensorMap tmD, const Params p) {
  using C = Cfg<BN>;
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
    tma_prefetch_desc(&tmD);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int items = p.m_blocks * p.n_blocks * p.k_splits;
  int fail_role = 0, fail_item = -1;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < items && ok; item += gridDim.x) {
        const int ks = item % p.k_splits, tile = item / p.k_splits;
        const int n_blk = tile % p.n_blocks, m_blk = tile / p.n_blocks;
        const int kb0 = ks * p.kblocks_per_split, kb1 = min(kb0 + p.kblocks_per_split, p.kblocks_total);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const uint32_t s = it % C::kStages, ph = (it / C::kStages) & 1;
          if (!mbar_wait(bar_empty + 8 * s, ph ^ 1, abort_flag)) { ok = false; fail_role = 1; fail_item = item; break; }
          const uint32_t full = bar_full + 8 * s;
          mbar_expect_tx(full, C::kStageBytes);
          const uint32_t sa = smem_u32(stage_base + s * C::kStageBytes), sb = sa + C::kStageBytesA;
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
      for (int item = blockIdx.x; item < items && ok; item += gridDim.x, ++tile_iter) {
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
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            umma_f16(d_tmem, da + (uint64_t)(k * a_step), db + (uint64_t)(k * b_step), p.idesc, (kb > kb0 || k > 0) ? 1u : 0u);
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
    for (int item = blockIdx.x; item < items; item += gridDim.x, ++tile_iter) {
      const int tile = item / p.k_splits;
      const int n_blk = tile % p.n_blocks, m_blk = tile / p.n_blocks;
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
          const bool is_bf16 = ((p.idesc >> 7) & 7) == 1;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int i = (j & 3) * 8 + 2 * e;
              const float lo = __uint_as_float(j < 4 ? r0[i] : r1[i]), hi = __uint_as_float(j < 4 ? r0[i + 1] : r1[i + 1]);
              if (is_bf16) {
                __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
                w[e] = *reinterpret_cast<uint32_t*>(&v);
              } else {
                __half2 v = __floats2half2_rn(lo, hi);
                w[e] = *reinterpret_cast<uint32_t*>(&v);
              }
            }
            *reinterpret_cast<uint4*>(my_row + ((j ^ sw) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
        fence_proxy_async_smem();
        named_barrier_sync(1, kEpilogueThreads);
        if (et == 0) {
          if (p.reduce_add) tma_reduce_add_2d(&tmD, smem_u32(buf), n_blk * BN + col0, m_blk * BM);
          else tma_store_2d(&tmD, smem_u32(buf), n_blk * BN + col0, m_blk * BM);
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
}

template <int BN>
int launch(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmD, const Params& p, int grid, cudaStream_t st) {
  auto kern = gemm_tcgen05_kernel<BN>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<BN>::kSmemBytes) != cudaSuccess) {
      nnb_set_error("gemm: cannot reserve %d bytes of shared memory", Cfg<BN>::kSmemBytes);
      return -3;
    }
    configured = true;
  }
  kern<<<grid, kThreads, Cfg<BN>::kSmemBytes, st>>>(tmA, tmB, tmD, p);
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
  NNB_REQUIRE(M > 0 && N > 0 && K > 0, "gemm: empty problem %dx%dx%d", M, N, K);
  NNB_REQUIRE(dtype == NNB_BF16 || dtype == NNB_F16, "gemm: inputs must be bf16 or fp16 (dtype code %d)", dtype);
  NNB_REQUIRE(!accumulate || out_f32, "gemm: accumulate needs an fp32 output");
  const CUtensorMapDataType in_dt = dtype == NNB_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const int sms = max_ctas > 0 ? min(max_ctas, nnb_num_sms()) : nnb_num_sms();
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
    const int cands[3] = {256, 192, 128};
    const double eff[3] = {1.0, 1.03, 1.10};  // narrower tiles re-read A more often: small penalty
    for (int i = 0; i < 3; ++i) {
      const int bn = cands[i];
      if (bn == 192) continue;  // measured slower than 256-wide tiles even where it fills the waves better; kept behind bn_hint
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
  if (out_f32) {
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
  p.a_mn = a_mn ? 1 : 0;
  p.b_mn = b_mn ? 1 : 0;
  p.out_f32 = out_f32 ? 1 : 0;
  p.reduce_add = (accumulate || p.k_splits > 1) ? 1 : 0;
  p.idesc = sm100::make_idesc_f16(dtype == NNB_BF16 ? 1 : 0, p.a_mn, p.b_mn, BM, BN);
  p.status = static_cast<int*>(status);

  CUtensorMap tmA, tmB, tmD;
  if (!p.a_mn) { if (!nnb_make_tmap_2d(&tmA, in_dt, 2, A, M, K, lda * 2, BM, BK, "gemm A")) return -4; }
  else         { if (!nnb_make_tmap_2d(&tmA, in_dt, 2, A, K, M, lda * 2, BK, 64, "gemm A^T")) return -4; }
  if (!p.b_mn) { if (!nnb_make_tmap_2d(&tmB, in_dt, 2, B, N, K, ldb * 2, BN, BK, "gemm B")) return -4; }
  else         { if (!nnb_make_tmap_2d(&tmB, in_dt, 2, B, K, N, ldb * 2, BK, 64, "gemm B^T")) return -4; }
  if (out_f32) { if (!nnb_make_tmap_2d(&tmD, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, D, M, N, ldd * 4, BM, 32, "gemm D")) return -4; }
  else         { if (!nnb_make_tmap_2d(&tmD, in_dt, 2, D, M, N, ldd * 2, BM, 64, "gemm D")) return -4; }

  if (out_f32 && !accumulate && p.k_splits > 1) {
    // partial tiles are reduce-added: start from zero
    if (ldd == N) cudaMemsetAsync(D, 0, (size_t)M * N * 4, st);
    else cudaMemset2DAsync(D, ldd * 4, 0, (size_t)N * 4, M, st);
  }
  const int items = p.m_blocks * p.n_blocks * p.k_splits;
  const int grid = min(items, sms);
  const int rc = BN == 256 ? launch<256>(tmA, tmB, tmD, p, grid, st)
               : BN == 192 ? launch<192>(tmA, tmB, tmD, p, grid, st) : launch<128>(tmA, tmB, tmD, p, grid, st);
  if (rc != 0) return rc;
  NNB_LAUNCH_OK("gemm_tcgen05");
  return 0;
}
