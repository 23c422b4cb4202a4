// Causal grouped-query FlashAttention backward on tcgen05 / TMEM / TMA for sm_100a (head_dim 64).
//
// One CTA owns 128 keys of one (batch, KV head) and visits every (query head of the group, query tile)
// at or after its keys; dK and dV of the tile accumulate in TMEM over the whole GQA group, so they are
// written once and need no atomics (as in the reference kernel, nanonemo/kernels/cuda/flash_attn.cu:
// 176-340, which keeps them in registers). Per visit, five tensor-core products:
//     S  = Q K^T            dP = dO V^T                       (M = queries, N = keys, K = head_dim)
//     P  = exp(S*scale - L) ; dS = P * (dP - D) * scale       (128 compute threads, one per query row)
//     dV += P^T dO          dK += dS^T Q                      (M = keys, N = head_dim, K = queries)
//     dQ  = dS K                                              (M = queries, N = head_dim, K = keys)
// P and dS are written once to shared memory as bf16 [query][key] tiles with the 128-byte swizzle; the
// same bytes serve as the K-major A operand of dQ and, read through an MN-major descriptor, as the
// transposed A operand of dV / dK. Q and dO tiles arrive by TMA and are read both K-major (S, dP) and
// MN-major (dK, dV) without any transposed copy. dQ partial tiles leave through a swizzled fp32
// staging tile and a TMA reduce-add (cp.reduce.async.bulk.tensor .add.f32) into an fp32 buffer that a
// small kernel converts at the end. D = rowsum(dO * O) is a pre-pass kernel in this file.
// 320 threads: warp 0 TMA producer, warp 1 MMA issuer, warps 2..9 compute: two threads per query row,
// one for keys 0..63 of the tile and one for keys 64..127 (same TMEM lanes, different columns).
//
// Software pipeline. The score tile is double buffered in tensor memory (S0 | S1 | dP | dV | dK = 512 columns; the dQ
// partial product of a visit is accumulated into the first 64 columns of THAT visit's S buffer, which is free once P has
// been computed from it), and the compute work of a visit is split into  A: P = exp(S scale - L)  /  B: dS = P (dP - D) scale,
// with the dQ drain of the PREVIOUS visit between them. The tensor core then always has work that does not depend on the
// phase the compute warps are in:
//     compute :  A(n)          drain dQ(n-1)     B(n)                    A(n+1)   ...
//     tensor  :        dV(n)               S(n+1)      dK(n) dQ(n) dP(n+1)
// S(n+1) is ready long before A(n+1) starts, dP(n+1) before B(n+1), dQ(n) before its drain, so neither side waits for the
// other in steady state; a visit costs about the compute warps' own work instead of the sum of all phases.
// All waits are bounded.
#include <cstdlib>
#include <type_traits>

#include "sm100.cuh"

namespace {

using namespace sm100;

constexpr int BQ = 128, BKV = 128, HD = 64;
constexpr int kThreads = 320;           // TMA warp, MMA warp, 2 x 4 compute warps
constexpr int kComputeThreads = 256;
constexpr int kTile16 = 128 * 64 * 2;     // a [128 x 64] 16-bit tile = 16 KB
constexpr int kStagesQ = 3;             // a stage is released when dK / dQ of its visit are done and refilled two visits ahead
// shared memory map (bytes)
constexpr int kOffK = 0, kOffV = kTile16, kOffQdO = 2 * kTile16;               // ring of (Q | dO)
constexpr int kOffP = kOffQdO + kStagesQ * 2 * kTile16, kOffdS = kOffP + 2 * kTile16;
constexpr int kOffStage = kOffdS + 2 * kTile16;                                // fp32 [128 x 64] = 32 KB
constexpr int kOffBars = kOffStage + 2 * kTile16;
constexpr int kSmem = kOffBars + 256 + 1024;
// tensor memory columns
constexpr int kColS = 0 /* two buffers: + 128 * (visit & 1) */, kColdP = 256, kColdV = 384, kColdK = 448, kTmemCols = 512;
constexpr int kColdQ = kColS;            // dQ(n) lands in columns [0, 64) of S buffer (n & 1), after P(n) has been taken from it

struct BParams {
  int B, H, KVH, T, n_q_tiles, group;
  float scale, scale_log2;
  const float* lse;    // [B, H, T]
  const float* delta;  // [B, H, T]
  uint32_t idesc_s, idesc_dkv, idesc_dq;
  int* status;
  // Optional inverse RoPE on dK (and on dQ in the convert kernel): fp32 tables [T, 32] of the forward rotation. When given,
  // the attention inputs were rotated by the producer of Q / K and the gradients leave here un-rotated, i.e. with respect to
  // the projection before RoPE, so no separate inverse-RoPE pass over the packed gradient is needed.
  const float* rope_cos;
  const float* rope_sin;
};

template <bool F16>
__global__ void __launch_bounds__(kThreads, 1)
flash_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                 const __grid_constant__ CUtensorMap tmdQacc, const __grid_constant__ CUtensorMap tmdK,
                 const __grid_constant__ CUtensorMap tmdV, const BParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t s_base = smem_u32(smem);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kOffBars);
  // barriers: kv_full, q_full[3], q_empty[3], s_full[2], dp_full, p_written, ds_written, dq_full, dq_read
  const uint32_t bar_kv = smem_u32(bars), bar_qf = bar_kv + 8, bar_qe = bar_qf + 8 * kStagesQ;
  const uint32_t bar_s = bar_qe + 8 * kStagesQ, bar_dp = bar_s + 16, bar_p = bar_dp + 8, bar_ds = bar_p + 8;
  const uint32_t bar_dq = bar_ds + 8, bar_dqr = bar_dq + 8;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 1 + 2 * kStagesQ + 7);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Longest-job-first over the whole grid: key tile 0 is visited by every query tile, the last one by a single tile, and the
  // key tile is the slowest-varying block index, so the heavy CTAs all start first and the kernel ends on the short ones.
  const int kt = blockIdx.z;          // key tile
  const int kvh = blockIdx.x, b = blockIdx.y;
  const int first_qt = (kt * BKV) / BQ;                     // first query tile that can see these keys
  const int n_qt = p.n_q_tiles - first_qt;                  // query tiles per head of the group
  const int iters = n_qt * p.group;

  if (threadIdx.x == 0) {
    mbar_init(bar_kv, 1);
    for (int s = 0; s < kStagesQ; ++s) {
      mbar_init(bar_qf + 8 * s, 1);
      mbar_init(bar_qe + 8 * s, 1);
    }
    mbar_init(bar_s, 1);
    mbar_init(bar_s + 8, 1);
    mbar_init(bar_dp, 1);
    mbar_init(bar_p, kComputeThreads);
    mbar_init(bar_ds, kComputeThreads);
    mbar_init(bar_dq, 1);
    mbar_init(bar_dqr, kComputeThreads);
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  int fail_role = 0;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      mbar_expect_tx(bar_kv, 2 * kTile16);
      tma_load_4d(s_base + kOffK, &tmK, bar_kv, 0, kvh, kt * BKV, b);
      tma_load_4d(s_base + kOffV, &tmV, bar_kv, 0, kvh, kt * BKV, b);
      for (int n = 0; n < iters; ++n) {
        const int hq = kvh * p.group + n / n_qt, qt = first_qt + n % n_qt;
        const uint32_t s = n % kStagesQ, ph = (n / kStagesQ) & 1;
        if (!mbar_wait(bar_qe + 8 * s, ph ^ 1, abort_flag)) { fail_role = 1; break; }
        const uint32_t dst = s_base + kOffQdO + s * 2 * kTile16;
        mbar_expect_tx(bar_qf + 8 * s, 2 * kTile16);
        tma_load_4d(dst, &tmQ, bar_qf + 8 * s, 0, hq, qt * BQ, b);
        tma_load_4d(dst + kTile16, &tmdO, bar_qf + 8 * s, 0, hq, qt * BQ, b);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      bool ok = mbar_wait(bar_kv, 0, abort_flag);
      const uint32_t sK = s_base + kOffK, sV = s_base + kOffV, sP = s_base + kOffP, sdS = s_base + kOffdS;
      auto stage_of = [&](int n) { return s_base + kOffQdO + (uint32_t)(n % kStagesQ) * 2 * kTile16; };
      auto wait_q = [&](int n) { return mbar_wait(bar_qf + 8 * (n % kStagesQ), (n / kStagesQ) & 1, abort_flag); };
      // S(n) = Q K^T into score buffer n & 1 (K-major operands, 4 k-steps of 16 over head_dim)
      auto issue_s = [&](int n) {
        const uint32_t sQ = stage_of(n);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k)
          umma_f16(tmem_base + kColS + (n & 1) * BKV, make_smem_desc(sQ + k * 32, 16, 1024), make_smem_desc(sK + k * 32, 16, 1024), p.idesc_s, k > 0);
        umma_commit(bar_s + 8 * (n & 1));
      };
      // dP(n) = dO V^T
      auto issue_dp = [&](int n) {
        const uint32_t sdO = stage_of(n) + kTile16;
#pragma unroll
        for (int k = 0; k < HD / 16; ++k)
          umma_f16(tmem_base + kColdP, make_smem_desc(sdO + k * 32, 16, 1024), make_smem_desc(sV + k * 32, 16, 1024), p.idesc_s, k > 0);
        umma_commit(bar_dp);
      };
      if (ok && iters > 0) {
        ok = wait_q(0);
        if (ok) {
          tc_fence_after();
          issue_s(0);
          issue_dp(0);
        }
      }
      for (int n = 0; n < iters && ok; ++n) {
        const uint32_t sQ = stage_of(n), sdO = sQ + kTile16;
        if (!mbar_wait(bar_p, n & 1, abort_flag)) { ok = false; break; }     // P(n) is in shared memory, S(n) has been read
        tc_fence_after();
        // dV += P^T dO: A = [query][key] tile read MN-major (M = keys: two 64-key groups 16 KB apart), B = [query][hd]
        // tile read MN-major; 8 k-steps of 16 query rows (2048 bytes each).
#pragma unroll
        for (int k = 0; k < BQ / 16; ++k)
          umma_f16(tmem_base + kColdV, make_smem_desc(sP + k * 2048, kTile16, 1024), make_smem_desc(sdO + k * 2048, kTile16, 1024),
                   p.idesc_dkv, (n > 0 || k > 0) ? 1u : 0u);
        if (n + 1 < iters) {
          // S(n + 1) goes into the other score buffer, whose first columns held dQ(n - 1): wait until that was drained.
          // Its commit also covers dV(n) above, so P may be overwritten as soon as S(n + 1) is seen complete.
          if (n >= 1 && !mbar_wait(bar_dqr, (n - 1) & 1, abort_flag)) { ok = false; break; }
          if (!wait_q(n + 1)) { ok = false; break; }
          tc_fence_after();
          issue_s(n + 1);
        }
        if (!mbar_wait(bar_ds, n & 1, abort_flag)) { ok = false; break; }    // dS(n) is in shared memory, dP(n) has been read
        tc_fence_after();
        // dK += dS^T Q (operands as for dV)
#pragma unroll
        for (int k = 0; k < BQ / 16; ++k)
          umma_f16(tmem_base + kColdK, make_smem_desc(sdS + k * 2048, kTile16, 1024), make_smem_desc(sQ + k * 2048, kTile16, 1024),
                   p.idesc_dkv, (n > 0 || k > 0) ? 1u : 0u);
        // dQ(n) = dS K into the score buffer of this visit: A = dS K-major over keys (two 64-key blocks), B = K tile read
        // MN-major (16 key rows per step)
#pragma unroll
        for (int k = 0; k < BKV / 16; ++k)
          umma_f16(tmem_base + kColdQ + (n & 1) * BKV, make_smem_desc(sdS + (k / 4) * kTile16 + (k % 4) * 32, 16, 1024),
                   make_smem_desc(sK + k * 2048, kTile16, 1024), p.idesc_dq, k > 0);
        umma_commit(bar_dq);
        umma_commit(bar_qe + 8 * (n % kStagesQ));
        if (n + 1 < iters) issue_dp(n + 1);   // dP(n) was consumed (bar_ds), Q / dO of visit n + 1 were awaited above
      }
      if (!ok) fail_role = 2;
    }
  } else {
    // ------------------------------------------------------------------ compute warps (two threads per query row)
    const int half = (warp - 2) >> 2;          // 0: keys 0..63 / dQ columns 0..31 / dV; 1: keys 64..127 / dQ columns 32..63 / dK
    const int q = warp & 3, row = q * 32 + lane, sw = row & 7;
    const bool leader = half == 0 && row == 0;
    const uint32_t t_lane = tmem_base + ((uint32_t)(q * 32) << 16);
    uint8_t* my_p = smem + kOffP + half * kTile16 + row * 128;
    uint8_t* my_ds = smem + kOffdS + half * kTile16 + row * 128;
    uint8_t* my_stage = smem + kOffStage + half * kTile16 + row * 128;
    const int key0 = kt * BKV + half * 64;
    bool ok = true;
    NNB_PROF_DECL;
    constexpr float kLog2e = 1.4426950408889634f;
    // dQ partial tile of visit m: TMEM (score buffer m & 1) -> swizzled fp32 staging (one [128 x 32] box per half) -> TMA
    // reduce-add. Every compute thread runs it, good or bad, so the two block barriers inside always see all 256 threads.
    auto drain_dq = [&](int m) {
      const int hq = kvh * p.group + m / n_qt, qt = first_qt + m % n_qt;
      if (ok && !mbar_wait(bar_dq, m & 1, abort_flag)) ok = false;
      tc_fence_after();
      if (leader) tma_wait_group_read<0>();      // the previous reduce has finished reading the staging tile
      if (named_barrier_or(1, kComputeThreads, !ok)) ok = false;
      if (ok) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(t_lane + kColdQ + (m & 1) * BKV + half * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int jj = 0; jj < 8; ++jj)
          *reinterpret_cast<uint4*>(my_stage + ((jj ^ sw) << 4)) = make_uint4(r[4 * jj], r[4 * jj + 1], r[4 * jj + 2], r[4 * jj + 3]);
      }
      tc_fence_before();
      mbar_arrive(bar_dqr);
      fence_proxy_async_smem();
      named_barrier_sync(1, kComputeThreads);
      if (leader && ok) {
        tma_reduce_add_4d(&tmdQacc, s_base + kOffStage, 0, hq, qt * BQ, b);
        tma_reduce_add_4d(&tmdQacc, s_base + kOffStage + kTile16, 32, hq, qt * BQ, b);
        tma_commit_group();
      }
    };
    for (int n = 0; n < iters; ++n) {
      NNB_PROF_T0;
      const int hq = kvh * p.group + n / n_qt, qt = first_qt + n % n_qt;
      const int qi = qt * BQ + row;
      const bool row_ok = qi < p.T;
      const size_t stat = ((size_t)b * p.H + hq) * p.T + (row_ok ? qi : 0);
      const float L = row_ok ? p.lse[stat] * kLog2e : 0.f;
      const float D = row_ok ? p.delta[stat] : 0.f;
      // Only tiles on the diagonal, past the end of the sequence, or with padded query rows need the
      // per-element mask; every other tile takes the branch-free version.
      const bool need_mask = key0 + 63 > qt * BQ || key0 + 63 >= p.T || qt * BQ + BQ > p.T;
      const float Ds = D * p.scale;
      const uint32_t t_s = t_lane + kColS + (n & 1) * BKV + half * 64;
      float prob[64];  // P of this thread's 64 keys, kept in fp32 from phase A to phase B
      // ---- phase A: P = exp2(S scale log2e - L log2e)
      if (ok && !mbar_wait(bar_s + 8 * (n & 1), (n >> 1) & 1, abort_flag)) ok = false;
      tc_fence_after();
      NNB_PROF_ADD(0);
      auto phase_a = [&](auto masked) {
        constexpr bool kMask = decltype(masked)::value;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t rs[32], pk[16];
          tmem_ld_32x32b_x32(t_s + c * 32, rs);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            float pr = exp2f(__uint_as_float(rs[i]) * p.scale_log2 - L);
            if (kMask) {
              const int key = key0 + c * 32 + i;
              pr = (row_ok && key <= qi && key < p.T) ? pr : 0.f;
            }
            prob[c * 32 + i] = pr;
          }
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            pk[i >> 1] = pack2_16<F16>(prob[c * 32 + i], prob[c * 32 + i + 1]);
          }
#pragma unroll
          for (int jj = 0; jj < 4; ++jj)
            *reinterpret_cast<uint4*>(my_p + (((c * 4 + jj) ^ sw) << 4)) = make_uint4(pk[4 * jj], pk[4 * jj + 1], pk[4 * jj + 2], pk[4 * jj + 3]);
        }
      };
      if (ok) {
        if (need_mask) phase_a(std::true_type{});
        else phase_a(std::false_type{});
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(bar_p);
      NNB_PROF_ADD(1);
      // ---- the previous visit's dQ leaves while the tensor core works on dV(n) and S(n + 1)
      if (n > 0) drain_dq(n - 1);
      NNB_PROF_ADD(2);
      // ---- phase B: dS = P (dP scale - D scale)
      if (ok && !mbar_wait(bar_dp, n & 1, abort_flag)) ok = false;
      tc_fence_after();
      NNB_PROF_ADD(3);
      if (ok) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t rp[32], dk[16];
          tmem_ld_32x32b_x32(t_lane + kColdP + half * 64 + c * 32, rp);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float d0 = prob[c * 32 + i] * (__uint_as_float(rp[i]) * p.scale - Ds);
            const float d1 = prob[c * 32 + i + 1] * (__uint_as_float(rp[i + 1]) * p.scale - Ds);
            dk[i >> 1] = pack2_16<F16>(d0, d1);
          }
#pragma unroll
          for (int jj = 0; jj < 4; ++jj)
            *reinterpret_cast<uint4*>(my_ds + (((c * 4 + jj) ^ sw) << 4)) = make_uint4(dk[4 * jj], dk[4 * jj + 1], dk[4 * jj + 2], dk[4 * jj + 3]);
        }
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(bar_ds);
      NNB_PROF_ADD(4);
      if (named_barrier_or(2, kComputeThreads, !ok)) { ok = false; fail_role = 3; break; }  // all leave together
    }
    if (iters > 0) drain_dq(iters - 1);
    if (!ok && fail_role == 0) fail_role = 3;
    NNB_PROF_FLUSH_N(iters);
    // dV (half 0) and dK (half 1) of this key tile: TMEM -> bf16 staging (reuse the P / dS tiles) -> TMA store
    if (ok && iters > 0) {
      // bar_dq of the last visit was awaited above, so every MMA (including dV / dK accumulation) has completed
      if (leader) tma_wait_group_read<0>();
      named_barrier_sync(1, kComputeThreads);
      uint8_t* dst = (half == 0 ? smem + kOffP : smem + kOffdS) + row * 128;
      uint32_t r0[32], r1[32];
      tmem_ld_32x32b_x32(t_lane + (half == 0 ? kColdV : kColdK), r0);
      tmem_ld_32x32b_x32(t_lane + (half == 0 ? kColdV : kColdK) + 32, r1);
      tmem_ld_wait();
      if (half == 1 && p.rope_cos != nullptr && kt * BKV + row < p.T) {
        // dK of key position t leaves through the transpose of the forward rotation: lo' = lo c + hi s, hi' = hi c - lo s
        const float* cr = p.rope_cos + (size_t)(kt * BKV + row) * (HD / 2);
        const float* sr = p.rope_sin + (size_t)(kt * BKV + row) * (HD / 2);
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          const float4 c4 = __ldg(reinterpret_cast<const float4*>(cr + i)), s4 = __ldg(reinterpret_cast<const float4*>(sr + i));
          const float cc[4] = {c4.x, c4.y, c4.z, c4.w}, ss[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float lo = __uint_as_float(r0[i + e]), hi = __uint_as_float(r1[i + e]);
            r0[i + e] = __float_as_uint(lo * cc[e] + hi * ss[e]);
            r1[i + e] = __float_as_uint(hi * cc[e] - lo * ss[e]);
          }
        }
      }
#pragma unroll
      for (int jj = 0; jj < 8; ++jj) {
        uint32_t w[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int i = (jj & 3) * 8 + 2 * e;
          w[e] = pack2_16<F16>(__uint_as_float(jj < 4 ? r0[i] : r1[i]), __uint_as_float(jj < 4 ? r0[i + 1] : r1[i + 1]));
        }
        *reinterpret_cast<uint4*>(dst + ((jj ^ sw) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
      }
      fence_proxy_async_smem();
      named_barrier_sync(1, kComputeThreads);
      if (leader) {
        tma_store_4d(&tmdV, s_base + kOffP, 0, kvh, kt * BKV, b);
        tma_store_4d(&tmdK, s_base + kOffdS, 0, kvh, kt * BKV, b);
        tma_commit_group();
      }
    }
    if (leader) tma_wait_group<0>();
  }

  if (fail_role != 0 && p.status != nullptr) {
    if (atomicCAS(p.status, 0, 3) == 0) {
      p.status[1] = fail_role;
      p.status[2] = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
      p.status[3] = 0;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// delta[b, h, t] = sum_d dO[b, t, h, d] * O[b, t, h, d]; 8 lanes per (b, t, h) row of 64 elements,
// 16 bytes per lane per tensor. The same pass clears the fp32 dQ accumulator (its rows are visited in the same order).
template <typename T16>
__global__ void flash_delta_kernel(const T16* __restrict__ o, const T16* __restrict__ d_o,
                                   float* __restrict__ delta, float* __restrict__ dq_acc, int B, int T, int H, long long o_sb, long long o_st,
                                   long long o_sh, long long do_sb, long long do_st, long long do_sh) {
  const long long gid = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const long long w = gid >> 3;
  const int sub = threadIdx.x & 7;
  const long long rows = (long long)B * T * H;
  float s = 0.f;
  int h = 0, t = 0, b = 0;
  if (w < rows) {
    h = (int)(w % H);
    const long long bt = w / H;
    t = (int)(bt % T);
    b = (int)(bt / T);
    float a[8], g[8];
    Chunk8<T16>::load(o + b * o_sb + t * o_st + h * o_sh + sub * 8, a);
    Chunk8<T16>::load(d_o + b * do_sb + t * do_st + h * do_sh + sub * 8, g);
#pragma unroll
    for (int i = 0; i < 8; ++i) s += a[i] * g[i];
    float4* z = reinterpret_cast<float4*>(dq_acc + w * HD + sub * 8);
    z[0] = make_float4(0.f, 0.f, 0.f, 0.f);
    z[1] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  s += __shfl_xor_sync(0xffffffffu, s, 4);
  s += __shfl_xor_sync(0xffffffffu, s, 2);
  s += __shfl_xor_sync(0xffffffffu, s, 1);
  if (w < rows && sub == 0) delta[((size_t)b * H + h) * T + t] = s;
}

// dq[b, t, h, :] (bf16, strided) = dq_acc[b, t, h, :] (fp32, contiguous); with tables, the inverse RoPE of position t is
// applied on the way (columns j and j + 32 are partners, so one thread converts 8 + 8 elements).
template <typename T16>
__global__ void flash_dq_convert_kernel(const float* __restrict__ acc, T16* __restrict__ dq, long long rows, int H,
                                        int T, long long sb, long long st, long long sh, const float* __restrict__ rope_cos,
                                        const float* __restrict__ rope_sin) {
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;  // one thread per 8 + 8 elements
  const long long total = rows * (HD / 16);
  if (idx >= total) return;
  const long long r = idx / (HD / 16);
  const int j = (int)(idx % (HD / 16)) * 8;
  const int h = (int)(r % H);
  const long long bt = r / H;
  const int t = (int)(bt % T);
  const long long b = bt / T;
  float lo[8], hi[8];
  Chunk8<float>::load(acc + r * HD + j, lo);
  Chunk8<float>::load(acc + r * HD + HD / 2 + j, hi);
  if (rope_cos != nullptr) {
    float c[8], s[8];
    Chunk8<float>::load(rope_cos + (size_t)t * (HD / 2) + j, c);
    Chunk8<float>::load(rope_sin + (size_t)t * (HD / 2) + j, s);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float a = lo[i], bb = hi[i];
      lo[i] = a * c[i] + bb * s[i];
      hi[i] = bb * c[i] - a * s[i];
    }
  }
  T16* dst = dq + b * sb + t * st + h * sh;
  Chunk8<T16>::store(dst + j, lo);
  Chunk8<T16>::store(dst + HD / 2 + j, hi);
}

}  // namespace

int nnb_flash_bwd_t_impl(int hd, const void* q, const void* k, const void* v, const void* o, const void* d_o, const void* lse, void* delta,
                          void* dq_acc, void* dq, void* dk, void* dv, int B, int T, int H, int KVH, const long long* qs,
                          const long long* ks, const long long* vs, const long long* os, const long long* dos, const long long* dqs,
                          const long long* dks, const long long* dvs, float scale, int dtype, void* status, cudaStream_t st);

#ifdef NNB_PROFILE
extern "C" int nnb_flash_bwd_prof_read(unsigned long long* out) { return (int)cudaMemcpyFromSymbol(out, g_flash_prof, sizeof(g_flash_prof)); }
#endif

// All tensors are [B, T, heads, 64] views given by element strides (contiguous last dim), bf16 or fp16 (one dtype for all).
// lse: fp32 [B, H, T] from the forward pass; delta: fp32 [B, H, T] scratch (written here);
// dq_acc: fp32 [B, T, H, hd] contiguous scratch (cleared by the delta pre-pass; partial tiles are reduce-added into it).
// rope_cos / rope_sin: null, or fp32 [T, 32] tables: dQ and dK are then returned through the inverse rotation (head_dim 64).
extern "C" int nnb_flash_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o, const void* lse,
                             void* delta, void* dq_acc, void* dq, void* dk, void* dv, int B, int T, int H, int KVH, int hd,
                             long long q_sb, long long q_st, long long q_sh, long long k_sb, long long k_st, long long k_sh,
                             long long v_sb, long long v_st, long long v_sh, long long o_sb, long long o_st, long long o_sh,
                             long long do_sb, long long do_st, long long do_sh, long long dq_sb, long long dq_st,
                             long long dq_sh, long long dk_sb, long long dk_st, long long dk_sh, long long dv_sb,
                             long long dv_st, long long dv_sh, float scale, int dtype, const void* rope_cos, const void* rope_sin,
                             void* status, cudaStream_t st) {
  NNB_REQUIRE(hd == HD || hd == 128, "flash_bwd: head_dim %d not supported (64, 128)", hd);
  NNB_REQUIRE(dtype == NNB_BF16 || dtype == NNB_F16, "flash_bwd: bf16 or fp16 only (dtype code %d)", dtype);
  const bool f16 = dtype == NNB_F16;
  NNB_REQUIRE(H % KVH == 0 && B > 0 && T > 0, "flash_bwd: bad shape");
  // head_dim 128 runs on the transposed-tile kernel (flash_bwd_t.cu). It also serves head_dim 64
  // (NANONEMO_FLASH_BWD=transposed), but there the 128 x 128 formulation of this file measured faster (0.43 vs 0.57 ms at
  // B32 H12/4 T1024): with 64-wide tiles every MMA has N = 64 and is bound by shared-memory operand reads.
  static const bool square = [] { const char* e = getenv("NANONEMO_FLASH_BWD"); return !(e && e[0] == 't'); }();
  NNB_REQUIRE((rope_cos == nullptr) == (rope_sin == nullptr), "flash_bwd: give both RoPE tables or neither");
  NNB_REQUIRE(rope_cos == nullptr || (hd == HD && square && nnb_aligned16(rope_cos) && nnb_aligned16(rope_sin)),
              "flash_bwd: the fused inverse RoPE exists for head_dim 64 on the 128 x 128 kernel only");
  if (hd == 128 || !square) {
    const long long qs[3] = {q_sb, q_st, q_sh}, ks[3] = {k_sb, k_st, k_sh}, vs[3] = {v_sb, v_st, v_sh}, os[3] = {o_sb, o_st, o_sh};
    const long long dos[3] = {do_sb, do_st, do_sh}, dqs[3] = {dq_sb, dq_st, dq_sh}, dks[3] = {dk_sb, dk_st, dk_sh};
    const long long dvs[3] = {dv_sb, dv_st, dv_sh};
    return nnb_flash_bwd_t_impl(hd, q, k, v, o, d_o, lse, delta, dq_acc, dq, dk, dv, B, T, H, KVH, qs, ks, vs, os, dos, dqs, dks, dvs,
                                scale, dtype, status, st);
  }
  const CUtensorMapDataType dt = f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUtensorMap tq, tk, tv, tdo, tdq, tdk, tdv;
  if (!nnb_make_tmap_4d(&tq, dt, 2, q, hd, H, T, B, q_sh * 2, q_st * 2, q_sb * 2, 64, 1, BQ, "flash_bwd Q")) return -4;
  if (!nnb_make_tmap_4d(&tk, dt, 2, k, hd, KVH, T, B, k_sh * 2, k_st * 2, k_sb * 2, 64, 1, BKV, "flash_bwd K")) return -4;
  if (!nnb_make_tmap_4d(&tv, dt, 2, v, hd, KVH, T, B, v_sh * 2, v_st * 2, v_sb * 2, 64, 1, BKV, "flash_bwd V")) return -4;
  if (!nnb_make_tmap_4d(&tdo, dt, 2, d_o, hd, H, T, B, do_sh * 2, do_st * 2, do_sb * 2, 64, 1, BQ, "flash_bwd dO")) return -4;
  if (!nnb_make_tmap_4d(&tdq, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, dq_acc, hd, H, T, B, (uint64_t)hd * 4, (uint64_t)H * hd * 4,
                        (uint64_t)T * H * hd * 4, 32, 1, BQ, "flash_bwd dQ acc")) return -4;
  if (!nnb_make_tmap_4d(&tdk, dt, 2, dk, hd, KVH, T, B, dk_sh * 2, dk_st * 2, dk_sb * 2, 64, 1, BKV, "flash_bwd dK")) return -4;
  if (!nnb_make_tmap_4d(&tdv, dt, 2, dv, hd, KVH, T, B, dv_sh * 2, dv_st * 2, dv_sb * 2, 64, 1, BKV, "flash_bwd dV")) return -4;

  const long long rows = (long long)B * T * H;
  const unsigned delta_blocks = (unsigned)((rows * 8 + 255) / 256);
  if (f16)
    flash_delta_kernel<__half><<<delta_blocks, 256, 0, st>>>((const __half*)o, (const __half*)d_o, (float*)delta, (float*)dq_acc, B, T, H, o_sb,
                                                            o_st, o_sh, do_sb, do_st, do_sh);
  else
    flash_delta_kernel<__nv_bfloat16><<<delta_blocks, 256, 0, st>>>((const __nv_bfloat16*)o, (const __nv_bfloat16*)d_o, (float*)delta,
                                                                   (float*)dq_acc, B, T, H, o_sb, o_st, o_sh, do_sb, do_st, do_sh);
  NNB_LAUNCH_OK("flash_delta");

  BParams p{};
  p.B = B; p.H = H; p.KVH = KVH; p.T = T;
  p.n_q_tiles = (T + BQ - 1) / BQ;
  p.group = H / KVH;
  p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.lse = static_cast<const float*>(lse);
  p.delta = static_cast<const float*>(delta);
  const int fmt = f16 ? 0 : 1;
  p.idesc_s = sm100::make_idesc_f16(fmt, 0, 0, BQ, BKV);
  p.idesc_dkv = sm100::make_idesc_f16(fmt, 1, 1, BKV, HD);
  p.idesc_dq = sm100::make_idesc_f16(fmt, 0, 1, BQ, HD);
  p.status = static_cast<int*>(status);
  p.rope_cos = static_cast<const float*>(rope_cos);
  p.rope_sin = static_cast<const float*>(rope_sin);
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(flash_bwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem) != cudaSuccess ||
        cudaFuncSetAttribute(flash_bwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem) != cudaSuccess) {
      nnb_set_error("flash_bwd: cannot reserve %d bytes of shared memory", kSmem);
      return -3;
    }
    configured = true;
  }
  dim3 grid(KVH, B, (T + BKV - 1) / BKV);
  if (f16) flash_bwd_kernel<true><<<grid, kThreads, kSmem, st>>>(tq, tk, tv, tdo, tdq, tdk, tdv, p);
  else flash_bwd_kernel<false><<<grid, kThreads, kSmem, st>>>(tq, tk, tv, tdo, tdq, tdk, tdv, p);
  NNB_LAUNCH_OK("flash_bwd");
  const unsigned conv_blocks = (unsigned)((rows * (HD / 16) + 255) / 256);
  if (f16)
    flash_dq_convert_kernel<__half><<<conv_blocks, 256, 0, st>>>((const float*)dq_acc, (__half*)dq, rows, H, T, dq_sb, dq_st, dq_sh, p.rope_cos,
                                                                p.rope_sin);
  else
    flash_dq_convert_kernel<__nv_bfloat16><<<conv_blocks, 256, 0, st>>>((const float*)dq_acc, (__nv_bfloat16*)dq, rows, H, T, dq_sb, dq_st, dq_sh,
                                                                       p.rope_cos, p.rope_sin);
  NNB_LAUNCH_OK("flash_dq_convert");
  return 0;
}
