// Causal grouped-query FlashAttention backward on TRANSPOSED score tiles (tcgen05 / TMEM / TMA, sm_100a), head_dim 64 and 128.
//
// One CTA owns 128 keys of one (batch, KV head) and visits every (query head of the group, 64-query block) at or after its
// keys. Per visit, on score tiles of 128 keys x 64 queries:
//     S^T  = K Q^T          dP^T = V dO^T                  (M = 128 keys,  N = 64 queries, K = head_dim)
//     P^T  = exp(S^T scale - L[q]) ; dS^T = P^T (dP^T - D[q]) scale     (256 threads: key row x half of the queries)
//     dV  += P^T dO         dK  += dS^T Q                  (M = 128 keys,  N = head_dim,   K = 64 queries)
//     dQ^T = K^T dS^T                                      (M = head_dim,  N = 64 queries, K = 128 keys)
// Why transposed: with 64-query tiles the scores take 64 TMEM columns each, so at head_dim 64 S^T and dP^T are DOUBLE
// BUFFERED (2 x 64 + 2 x 64 + dV 64 + dK 64 + dQ^T 64 = 448 columns) and the softmax-gradient math of visit n + 1 runs while
// the tensor core accumulates dV / dK / dQ^T of visit n — in the 128 x 128 formulation (flash_bwd.cu) the two phases
// alternate, because two score buffers alone would fill the 512 columns. At head_dim 128 the accumulators are twice as wide
// (64 + 64 + 128 + 128 + 64 = 448 columns), the scores single buffered; the 128 x 128 formulation does not fit at all.
// P^T / dS^T are written once to shared memory as bf16 [key][query] tiles (128-byte rows, swizzled) and serve as K-major A
// operand (dV, dK) and MN-major B operand (dQ^T); K is read K-major (S^T) and MN-major (dQ^T), Q / dO K-major (scores) and
// MN-major (dK, dV): no transposed copies. dQ^T (lanes = head_dim index; at head_dim 64 an M = 64 accumulator: row m in
// lane m % 16 of lane quarter m / 16) leaves through an fp32 [query][head_dim] staging tile — the transpose happens in the
// shared-memory write — and a TMA reduce-add into an fp32 buffer. dK / dV accumulate over the GQA group and are stored once.
// With double-buffered scores the compute warps are software pipelined: math(n), then the drain of dQ^T(n - 1), so they do
// not wait for the MMAs they have just unblocked. Same contract as the reference backward (nanonemo/kernels/cuda/flash_attn.cu:176-340; head_dim 64 only).
#include <type_traits>

#include "sm100.cuh"

namespace {

using namespace sm100;

constexpr int BQ = 64, BKV = 128;
constexpr int kThreads = 320, kComputeThreads = 256;
constexpr int kHalfK = BKV * 64 * 2;   // [128 keys x 64] 16-bit tile = 16 KB
constexpr int kHalfQ = BQ * 64 * 2;    // [64 queries x 64] 16-bit tile = 8 KB
constexpr int kTmemCols = 512;

template <int HD>
struct Cfg {
  static constexpr int NH = HD / 64;                 // 64-wide head_dim groups (one TMA box / swizzle span each)
  static constexpr int NBUF = HD == 64 ? 2 : 1;      // buffers of S^T / dP^T (TMEM) and P^T / dS^T (shared memory)
  static constexpr int kStagesQ = HD == 64 ? 4 : 2;  // ring of (Q | dO) blocks
  static constexpr int kTileK = NH * kHalfK;         // K or V tile
  static constexpr int kStageQdO = 2 * NH * kHalfQ;  // Q block + dO block
  static constexpr int kOffK = 0, kOffV = kTileK, kOffQdO = 2 * kTileK;
  static constexpr int kOffP = kOffQdO + kStagesQ * kStageQdO, kOffdS = kOffP + NBUF * kHalfK;
  static constexpr int kOffStage = kOffdS + NBUF * kHalfK;     // fp32 [64 queries x HD]
  static constexpr int kOffBars = kOffStage + BQ * HD * 4;
  static constexpr int kOffLD = kOffBars + 256;                // float [2 parities][2 (L, D)][64]
  static constexpr int kSmem = kOffLD + 2 * 2 * 64 * 4 + 1024;
  static constexpr int kColS = 0, kColdP = 64 * NBUF, kColdV = 128 * NBUF, kColdK = kColdV + HD, kColdQ = kColdK + HD;
  static_assert(kColdQ + 64 <= kTmemCols, "TMEM budget");
  static_assert(kStagesQ * kStageQdO >= 2 * kTileK, "the (Q | dO) ring doubles as the dV / dK staging area");
};

struct BParams {
  int B, H, KVH, T, n_q_blocks, group;
  float scale, scale_log2;
  const float* lse;
  const float* delta;
  uint32_t idesc_s, idesc_dkv, idesc_dq;
  int* status;
};

template <int HD, bool F16>
__global__ void __launch_bounds__(kThreads, 1)
flash_bwd_t_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                   const __grid_constant__ CUtensorMap tmdQacc, const __grid_constant__ CUtensorMap tmdK,
                   const __grid_constant__ CUtensorMap tmdV, const BParams p) {
  using C = Cfg<HD>;
  constexpr int NH = C::NH, NBUF = C::NBUF, S = C::kStagesQ;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t s_base = smem_u32(smem);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kOffBars);
  // barriers: kv, q_full[4], q_empty[4], sdp[2], pds[2], pfree[2], dq, dq_read
  const uint32_t bar_kv = smem_u32(bars), bar_qf = bar_kv + 8, bar_qe = bar_qf + 32;
  const uint32_t bar_sdp = bar_qe + 32, bar_pds = bar_sdp + 16, bar_pfree = bar_pds + 16, bar_dq = bar_pfree + 16, bar_dqr = bar_dq + 8;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 17);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* s_ld = reinterpret_cast<float*>(smem + C::kOffLD);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kt = blockIdx.z, kvh = blockIdx.x, b = blockIdx.y;  // key tile slowest: the heavy CTAs (early keys) are scheduled first
  const int first_qb = (kt * BKV) / BQ;
  const int n_qb = p.n_q_blocks - first_qb;
  const int iters = n_qb * p.group;

  if (threadIdx.x == 0) {
    mbar_init(bar_kv, 1);
    for (int s = 0; s < 4; ++s) {
      mbar_init(bar_qf + 8 * s, 1);
      mbar_init(bar_qe + 8 * s, 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar_sdp + 8 * i, 1);
      mbar_init(bar_pds + 8 * i, kComputeThreads);
      mbar_init(bar_pfree + 8 * i, 1);
    }
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
      mbar_expect_tx(bar_kv, 2 * C::kTileK);
#pragma unroll
      for (int g = 0; g < NH; ++g) {
        tma_load_4d(s_base + C::kOffK + g * kHalfK, &tmK, bar_kv, g * 64, kvh, kt * BKV, b);
        tma_load_4d(s_base + C::kOffV + g * kHalfK, &tmV, bar_kv, g * 64, kvh, kt * BKV, b);
      }
      for (int n = 0; n < iters; ++n) {
        const int hq = kvh * p.group + n / n_qb, qb = first_qb + n % n_qb;
        const uint32_t s = n % S, ph = (n / S) & 1;
        if (!mbar_wait(bar_qe + 8 * s, ph ^ 1, abort_flag)) { fail_role = 1; break; }
        const uint32_t dst = s_base + C::kOffQdO + s * C::kStageQdO;
        mbar_expect_tx(bar_qf + 8 * s, C::kStageQdO);
#pragma unroll
        for (int g = 0; g < NH; ++g) {
          tma_load_4d(dst + g * kHalfQ, &tmQ, bar_qf + 8 * s, g * 64, hq, qb * BQ, b);
          tma_load_4d(dst + (NH + g) * kHalfQ, &tmdO, bar_qf + 8 * s, g * 64, hq, qb * BQ, b);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      bool ok = mbar_wait(bar_kv, 0, abort_flag);
      const uint32_t sK = s_base + C::kOffK, sV = s_base + C::kOffV;
      // S^T = K Q^T and dP^T = V dO^T of visit n into score buffer n % NBUF: K-major operands, k-steps of 16 over head_dim
      auto issue_sdp = [&](int n) -> bool {
        const uint32_t s = n % S, ph = (n / S) & 1, buf = n % NBUF;
        const uint32_t sQ = s_base + C::kOffQdO + s * C::kStageQdO, sdO = sQ + NH * kHalfQ;
        if (!mbar_wait(bar_qf + 8 * s, ph, abort_flag)) return false;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < HD / 16; ++k)
          umma_f16(tmem_base + C::kColS + 64 * buf, make_smem_desc(sK + (k / 4) * kHalfK + (k % 4) * 32, 16, 1024),
                   make_smem_desc(sQ + (k / 4) * kHalfQ + (k % 4) * 32, 16, 1024), p.idesc_s, k > 0);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k)
          umma_f16(tmem_base + C::kColdP + 64 * buf, make_smem_desc(sV + (k / 4) * kHalfK + (k % 4) * 32, 16, 1024),
                   make_smem_desc(sdO + (k / 4) * kHalfQ + (k % 4) * 32, 16, 1024), p.idesc_s, k > 0);
        umma_commit(bar_sdp + 8 * buf);
        return true;
      };
      for (int i = 0; i < NBUF && i < iters && ok; ++i) ok = issue_sdp(i);
      for (int n = 0; n < iters && ok; ++n) {
        const uint32_t s = n % S, buf = n % NBUF;
        const uint32_t sQ = s_base + C::kOffQdO + s * C::kStageQdO, sdO = sQ + NH * kHalfQ;
        const uint32_t sP = s_base + C::kOffP + buf * kHalfK, sdS = s_base + C::kOffdS + buf * kHalfK;
        if (!mbar_wait(bar_pds + 8 * buf, (n / NBUF) & 1, abort_flag)) { ok = false; break; }  // P^T, dS^T written; scores consumed
        if (n > 0 && !mbar_wait(bar_dqr, (n - 1) & 1, abort_flag)) { ok = false; break; }       // dQ^T of the previous visit drained
        tc_fence_after();
        // dV += P^T dO, dK += dS^T Q: A = [key][query] tile K-major (4 k-steps of 16 queries = 32 bytes), B = [query][head_dim]
        // block read MN-major (64-wide head_dim groups kHalfQ apart; 16 query rows = 2048 bytes per step)
#pragma unroll
        for (int k = 0; k < BQ / 16; ++k)
          umma_f16(tmem_base + C::kColdV, make_smem_desc(sP + k * 32, 16, 1024), make_smem_desc(sdO + k * 2048, kHalfQ, 1024),
                   p.idesc_dkv, (n > 0 || k > 0) ? 1u : 0u);
#pragma unroll
        for (int k = 0; k < BQ / 16; ++k)
          umma_f16(tmem_base + C::kColdK, make_smem_desc(sdS + k * 32, 16, 1024), make_smem_desc(sQ + k * 2048, kHalfQ, 1024),
                   p.idesc_dkv, (n > 0 || k > 0) ? 1u : 0u);
        // dQ^T = K^T dS^T: A = K tile read MN-major (M = head_dim in 64-wide groups kHalfK apart), B = dS^T tile read MN-major
        // (N = 64 queries: one group); 8 k-steps of 16 key rows = 2048 bytes
#pragma unroll
        for (int k = 0; k < BKV / 16; ++k)
          umma_f16(tmem_base + C::kColdQ, make_smem_desc(sK + k * 2048, kHalfK, 1024), make_smem_desc(sdS + k * 2048, kHalfK, 1024),
                   p.idesc_dq, k > 0);
        umma_commit(bar_dq);
        umma_commit(bar_qe + 8 * s);
        umma_commit(bar_pfree + 8 * buf);
        if (n + NBUF < iters) ok = issue_sdp(n + NBUF);  // its score buffer was released by bar_pds above
      }
      if (!ok) fail_role = 2;
    }
  } else {
    // ------------------------------------------------------------------ compute warps: (key row) x (half of the 64 queries)
    const int half = (warp - 2) >> 2;
    const int q4 = warp & 3, row = q4 * 32 + lane, sw = row & 7;
    const int ct = threadIdx.x - 64;  // 0..255
    const bool leader = ct == 0;
    const uint32_t t_lane = tmem_base + ((uint32_t)(q4 * 32) << 16);
    float* stage = reinterpret_cast<float*>(smem + C::kOffStage);
    const int key = kt * BKV + row;
    bool ok = true;
    constexpr float kLog2e = 1.4426950408889634f;
    NNB_PROF_DECL;
    // dQ^T of visit m: TMEM (lane = head_dim index, columns = queries) -> fp32 staging [query][head_dim] -> TMA reduce-add
    auto drain_dq = [&](int m) -> bool {
      const int hq = kvh * p.group + m / n_qb, q0 = (first_qb + m % n_qb) * BQ;
      if (!mbar_wait(bar_dq, m & 1, abort_flag)) ok = false;
      tc_fence_after();
      if (leader) tma_wait_group_read<0>();      // the previous reduce has finished reading the staging tile
      if (named_barrier_or(1, kComputeThreads, !ok)) return false;
      NNB_PROF_ADD(2);
      uint32_t r[32];
      tmem_ld_32x32b_x32(t_lane + C::kColdQ + half * 32, r);
      tmem_ld_wait();
      if (HD == 128) {
#pragma unroll
        for (int c = 0; c < 32; ++c) stage[(half * 32 + c) * HD + row] = __uint_as_float(r[c]);
      } else if (lane < 16) {                    // M = 64 accumulator: row 16 q4 + lane lives in lane `lane` of this quarter
#pragma unroll
        for (int c = 0; c < 32; ++c) stage[(half * 32 + c) * HD + q4 * 16 + lane] = __uint_as_float(r[c]);
      }
      tc_fence_before();
      mbar_arrive(bar_dqr);
      fence_proxy_async_smem();
      named_barrier_sync(1, kComputeThreads);
      if (leader) {
        tma_reduce_add_4d(&tmdQacc, s_base + C::kOffStage, 0, hq, q0, b);
        tma_commit_group();
      }
      NNB_PROF_ADD(3);
      return true;
    };
    // L (log-sum-exp, log2 units) and D * scale of the 64 queries of a visit: threads 0..63 fetch L, 64..127 fetch D, one
    // visit AHEAD into a register, so the global-memory latency hides behind the previous visit
    auto fetch_ld = [&](int n) -> float {
      if (ct >= 128 || n >= iters) return 0.f;
      const int hq = kvh * p.group + n / n_qb, qi = (first_qb + n % n_qb) * BQ + (ct & 63);
      if (qi >= p.T) return 0.f;
      const size_t stat = ((size_t)b * p.H + hq) * p.T + qi;
      return ct < 64 ? p.lse[stat] * kLog2e : p.delta[stat] * p.scale;
    };
    float ld_next = fetch_ld(0);
    for (int n = 0; n < iters; ++n) {
      NNB_PROF_T0;
      const int q0 = (first_qb + n % n_qb) * BQ;
      const int buf = n % NBUF;
      uint8_t* my_p = smem + C::kOffP + buf * kHalfK + row * 128;
      uint8_t* my_ds = smem + C::kOffdS + buf * kHalfK + row * 128;
      float* sL = s_ld + (n & 1) * 128;
      float* sD = sL + 64;
      if (ct < 128) sL[ct] = ld_next;  // sD = sL + 64: threads 64..127 land in the D half
      ld_next = fetch_ld(n + 1);
      if (!mbar_wait(bar_sdp + 8 * buf, (n / NBUF) & 1, abort_flag)) ok = false;
      // the MMAs of the visit that last read this P^T / dS^T buffer have completed
      if (n >= NBUF && !mbar_wait(bar_pfree + 8 * buf, (n / NBUF - 1) & 1, abort_flag)) ok = false;
      if (named_barrier_or(1, kComputeThreads, !ok)) { ok = false; fail_role = 3; break; }  // L / D visible; all leave together
      tc_fence_after();
      NNB_PROF_ADD(0);
      // per-element mask only on the diagonal blocks, at the end of the sequence or for padded key rows
      const bool need_mask = q0 < kt * BKV + BKV - 1 || q0 + BQ > p.T || kt * BKV + BKV > p.T;
      auto tile = [&](auto masked) {
        constexpr bool kMask = decltype(masked)::value;
        uint32_t rs[32], rp[32];
        tmem_ld_32x32b_x32(t_lane + C::kColS + 64 * buf + half * 32, rs);
        tmem_ld_32x32b_x32(t_lane + C::kColdP + 64 * buf + half * 32, rp);
        tmem_ld_wait();
        uint32_t pk[16], dk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float pv[2], dv[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int c = half * 32 + i + e;
            float prob = exp2f(__uint_as_float(rs[i + e]) * p.scale_log2 - sL[c]);
            if (kMask) {
              const int qi = q0 + c;
              prob = (key <= qi && qi < p.T && key < p.T) ? prob : 0.f;
            }
            pv[e] = prob;
            dv[e] = prob * (__uint_as_float(rp[i + e]) * p.scale - sD[c]);
          }
          pk[i >> 1] = pack2_16<F16>(pv[0], pv[1]);
          dk[i >> 1] = pack2_16<F16>(dv[0], dv[1]);
        }
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
          const int chunk = ((half * 4 + jj) ^ sw) << 4;
          *reinterpret_cast<uint4*>(my_p + chunk) = make_uint4(pk[4 * jj], pk[4 * jj + 1], pk[4 * jj + 2], pk[4 * jj + 3]);
          *reinterpret_cast<uint4*>(my_ds + chunk) = make_uint4(dk[4 * jj], dk[4 * jj + 1], dk[4 * jj + 2], dk[4 * jj + 3]);
        }
      };
      if (need_mask) tile(std::true_type{});
      else tile(std::false_type{});
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(bar_pds + 8 * buf);
      NNB_PROF_ADD(1);
      if (NBUF == 1) {
        // single score buffer: the next visit's math needs this visit's MMAs anyway, so drain dQ^T right away
        if (!drain_dq(n)) { ok = false; fail_role = 3; break; }
      } else if (n > 0 && !drain_dq(n - 1)) {
        // double buffered: the MMAs of this visit are now unblocked; drain the PREVIOUS visit's dQ^T meanwhile
        ok = false; fail_role = 3; break;
      }
    }
    if (NBUF == 2 && ok && iters > 0 && !drain_dq(iters - 1)) { ok = false; fail_role = 3; }
    NNB_PROF_FLUSH_N(iters);
    // dV then dK of this key tile: TMEM -> bf16 staging (the (Q | dO) ring: every load has been consumed) -> TMA store
    if (ok && iters > 0) {
      // bar_dq of the last visit was awaited in drain_dq, so every MMA (including the dV / dK accumulation) has completed
      if (leader) tma_wait_group_read<0>();
      named_barrier_sync(1, kComputeThreads);
#pragma unroll
      for (int u = half; u < 2 * NH; u += 2) {
        const int which = u / NH, g = u % NH;  // 0 = dV, 1 = dK; 64-wide head_dim group
        uint8_t* dst = smem + C::kOffQdO + which * C::kTileK + g * kHalfK + row * 128;
        const uint32_t col = (which == 0 ? C::kColdV : C::kColdK) + g * 64;
        uint32_t r0[32], r1[32];
        tmem_ld_32x32b_x32(t_lane + col, r0);
        tmem_ld_32x32b_x32(t_lane + col + 32, r1);
        tmem_ld_wait();
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
      }
      fence_proxy_async_smem();
      named_barrier_sync(1, kComputeThreads);
      if (leader) {
#pragma unroll
        for (int g = 0; g < NH; ++g) {
          tma_store_4d(&tmdV, s_base + C::kOffQdO + g * kHalfK, g * 64, kvh, kt * BKV, b);
          tma_store_4d(&tmdK, s_base + C::kOffQdO + C::kTileK + g * kHalfK, g * 64, kvh, kt * BKV, b);
        }
        tma_commit_group();
      }
    }
    if (leader) tma_wait_group<0>();
  }

  if (fail_role != 0 && p.status != nullptr) {
    if (atomicCAS(p.status, 0, 3) == 0) {
      p.status[1] = fail_role;
      p.status[2] = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
      p.status[3] = HD;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// delta[b, h, t] = sum_d dO[b, t, h, d] * O[b, t, h, d]; HD / 8 lanes per row, 16 bytes per lane per tensor. The same pass
// clears the fp32 dQ accumulator (its rows are visited in the same order).
template <int HD, typename T16>
__global__ void flash_delta_t_kernel(const T16* __restrict__ o, const T16* __restrict__ d_o,
                                     float* __restrict__ delta, float* __restrict__ dq_acc, int B, int T, int H, long long o_sb, long long o_st,
                                     long long o_sh, long long do_sb, long long do_st, long long do_sh) {
  constexpr int L = HD / 8;
  const long long gid = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const long long w = gid / L;
  const int sub = threadIdx.x % L;
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
#pragma unroll
  for (int o2 = L / 2; o2 > 0; o2 >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o2);
  if (w < rows && sub == 0) delta[((size_t)b * H + h) * T + t] = s;
}

// dq[b, t, h, :] (bf16, strided) = dq_acc[b, t, h, :] (fp32, contiguous)
template <int HD, typename T16>
__global__ void flash_dq_convert_t_kernel(const float* __restrict__ acc, T16* __restrict__ dq, long long rows, int H,
                                          int T, long long sb, long long st, long long sh) {
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;  // one thread per 8 elements
  const long long total = rows * (HD / 8);
  if (idx >= total) return;
  const long long r = idx / (HD / 8);
  const int j = (int)(idx % (HD / 8)) * 8;
  const int h = (int)(r % H);
  const long long bt = r / H;
  const int t = (int)(bt % T);
  const long long b = bt / T;
  float v[8];
  Chunk8<float>::load(acc + r * HD + j, v);
  Chunk8<T16>::store(dq + b * sb + t * st + h * sh + j, v);
}

template <int HD, bool F16>
int launch_bwd_t(const void* q, const void* k, const void* v, const void* o, const void* d_o, const void* lse, void* delta,
                 void* dq_acc, void* dq, void* dk, void* dv, int B, int T, int H, int KVH, const long long* qs, const long long* ks,
                 const long long* vs, const long long* os, const long long* dos, const long long* dqs, const long long* dks,
                 const long long* dvs, float scale, void* status, cudaStream_t st) {
  using C = Cfg<HD>;
  using T16 = typename sm100::Operand16<F16>::type;
  const CUtensorMapDataType dt = F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUtensorMap tq, tk, tv, tdo, tdq, tdk, tdv;
  if (!nnb_make_tmap_4d(&tq, dt, 2, q, HD, H, T, B, qs[2] * 2, qs[1] * 2, qs[0] * 2, 64, 1, BQ, "flash_bwd Q")) return -4;
  if (!nnb_make_tmap_4d(&tk, dt, 2, k, HD, KVH, T, B, ks[2] * 2, ks[1] * 2, ks[0] * 2, 64, 1, BKV, "flash_bwd K")) return -4;
  if (!nnb_make_tmap_4d(&tv, dt, 2, v, HD, KVH, T, B, vs[2] * 2, vs[1] * 2, vs[0] * 2, 64, 1, BKV, "flash_bwd V")) return -4;
  if (!nnb_make_tmap_4d(&tdo, dt, 2, d_o, HD, H, T, B, dos[2] * 2, dos[1] * 2, dos[0] * 2, 64, 1, BQ, "flash_bwd dO")) return -4;
  if (!nnb_make_tmap_4d(&tdq, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, dq_acc, HD, H, T, B, (uint64_t)HD * 4, (uint64_t)H * HD * 4,
                        (uint64_t)T * H * HD * 4, HD, 1, BQ, "flash_bwd dQ acc")) return -4;
  if (!nnb_make_tmap_4d(&tdk, dt, 2, dk, HD, KVH, T, B, dks[2] * 2, dks[1] * 2, dks[0] * 2, 64, 1, BKV, "flash_bwd dK")) return -4;
  if (!nnb_make_tmap_4d(&tdv, dt, 2, dv, HD, KVH, T, B, dvs[2] * 2, dvs[1] * 2, dvs[0] * 2, 64, 1, BKV, "flash_bwd dV")) return -4;

  const long long rows = (long long)B * T * H;
  flash_delta_t_kernel<HD, T16><<<(unsigned)((rows * (HD / 8) + 255) / 256), 256, 0, st>>>(
      (const T16*)o, (const T16*)d_o, (float*)delta, (float*)dq_acc, B, T, H, os[0], os[1], os[2], dos[0], dos[1], dos[2]);
  NNB_LAUNCH_OK("flash_delta");
  BParams p{};
  p.B = B; p.H = H; p.KVH = KVH; p.T = T;
  p.n_q_blocks = (T + BQ - 1) / BQ;
  p.group = H / KVH;
  p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.lse = static_cast<const float*>(lse);
  p.delta = static_cast<const float*>(delta);
  constexpr int fmt = F16 ? 0 : 1;
  p.idesc_s = sm100::make_idesc_f16(fmt, 0, 0, BKV, BQ);
  p.idesc_dkv = sm100::make_idesc_f16(fmt, 0, 1, BKV, HD);
  p.idesc_dq = sm100::make_idesc_f16(fmt, 1, 1, HD, BQ);
  p.status = static_cast<int*>(status);
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(flash_bwd_t_kernel<HD, F16>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmem) != cudaSuccess) {
      nnb_set_error("flash_bwd: cannot reserve %d bytes of shared memory", C::kSmem);
      return -3;
    }
    configured = true;
  }
  dim3 grid(KVH, B, (T + BKV - 1) / BKV);
  flash_bwd_t_kernel<HD, F16><<<grid, kThreads, C::kSmem, st>>>(tq, tk, tv, tdo, tdq, tdk, tdv, p);
  NNB_LAUNCH_OK("flash_bwd_t");
  flash_dq_convert_t_kernel<HD, T16><<<(unsigned)((rows * (HD / 8) + 255) / 256), 256, 0, st>>>((const float*)dq_acc, (T16*)dq, rows, H, T,
                                                                                                dqs[0], dqs[1], dqs[2]);
  NNB_LAUNCH_OK("flash_dq_convert");
  return 0;
}

}  // namespace

#ifdef NNB_PROFILE
extern "C" int nnb_flash_bwd_t_prof_read(unsigned long long* out) { return (int)cudaMemcpyFromSymbol(out, g_flash_prof, sizeof(g_flash_prof)); }
#endif

// Same contract as nnb_flash_bwd (flash_bwd.cu), which forwards here. All tensors are [B, T, heads, hd] views given by
// element strides {batch, t, head}; dq_acc: fp32 [B, T, H, hd] contiguous scratch (cleared by the delta pre-pass).
int nnb_flash_bwd_t_impl(int hd, const void* q, const void* k, const void* v, const void* o, const void* d_o, const void* lse,
                         void* delta, void* dq_acc, void* dq, void* dk, void* dv, int B, int T, int H, int KVH, const long long* qs,
                         const long long* ks, const long long* vs, const long long* os, const long long* dos, const long long* dqs,
                         const long long* dks, const long long* dvs, float scale, int dtype, void* status, cudaStream_t st) {
#define NNB_BWD_T(HD_, F16_) \
  launch_bwd_t<HD_, F16_>(q, k, v, o, d_o, lse, delta, dq_acc, dq, dk, dv, B, T, H, KVH, qs, ks, vs, os, dos, dqs, dks, dvs, scale, status, st)
  const bool f16 = dtype == NNB_F16;
  if (hd == 64) return f16 ? NNB_BWD_T(64, true) : NNB_BWD_T(64, false);
  return f16 ? NNB_BWD_T(128, true) : NNB_BWD_T(128, false);
#undef NNB_BWD_T
}
