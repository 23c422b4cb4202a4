// Causal grouped-query FlashAttention forward on tcgen05 / TMEM / TMA for sm_100a.
//
// One CTA owns a PAIR of 128-row query tiles of one (batch, query head) and walks the key/value
// tiles up to the diagonal. 320 threads, warp-specialised:
//   warp 0        TMA producer: Q tiles once, then K_j / V_j into a ring of stages (4-D tensor maps
//                 over (head_dim, head, t, batch), so any (B,T,H,hd)/(B,H,T,hd)/packed-QKV strides work
//                 and query head h reads KV head h / group directly — nothing is repeated or copied);
//   warp 1        MMA issuer: S_g = Q_g K_j^T and O_g = P_g V_j with tcgen05.mma, accumulators in TMEM;
//   warps 2..5    softmax group 0 (query tile 2p), warps 6..9 softmax group 1 (query tile 2p+1): one
//                 thread per query row (= TMEM lane): tcgen05.ld the scores, online max / sum in fp32
//                 with exp2, write P as bf16 into a 128-byte swizzled shared tile (the A operand of the
//                 second MMA), then fold the partial O from TMEM into register accumulators.
// The two groups ping-pong: while one does softmax the tensor core works for the other.
// Outputs: O (16-bit) through a swizzled staging tile + TMA store, and L = m * scale + ln(l) per row
// (fp32) for the backward pass. Every mbarrier wait is bounded; on expiry the kernel records a status
// word and leaves cleanly.
//
// Replaces the reference's WMMA kernel for sm_75 (nanonemo/kernels/cuda/flash_attn.cu:52-174) and
// the mem-efficient SDPA path it benchmarks against; same math contract (causal, GQA-direct, saves
// the log-sum-exp per row).
#include "sm100.cuh"

namespace {

using namespace sm100;

constexpr int BQ = 128;  // query rows per tile (= TMEM lanes)
constexpr int kThreads = 320;

template <int HD>
struct FCfg {
  static constexpr int BN = (HD == 64) ? 128 : 64;          // keys per KV tile
  static constexpr int kStages = 3;
  static constexpr int kQBytes = BQ * HD * 2;               // one Q tile (HD/64 swizzled K-blocks of 16 KB)
  static constexpr int kKBytes = BN * HD * 2;
  static constexpr int kVBytes = BN * HD * 2;
  static constexpr int kPBytes = BQ * BN * 2;               // BN/64 swizzled K-blocks of 16 KB
  static constexpr int kSmem = 2 * kQBytes + kStages * (kKBytes + kVBytes) + 2 * kPBytes + 1024 + 256;
  static constexpr int kTmemCols = 512;                     // S0 | S1 | O0 | O1
  static constexpr int kColS0 = 0, kColS1 = 128, kColO0 = 256, kColO1 = 256 + HD;
};

struct FParams {
  int B, H, KVH, T;
  int n_q_tiles, n_pairs;
  float scale_log2;   // softmax scale * log2(e)
  float scale;        // softmax scale
  float* lse;         // [B, H, T]
  uint32_t idesc_qk, idesc_pv;
  int* status;
};

template <int HD>
__global__ void __launch_bounds__(kThreads, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO, const FParams p) {
  using C = FCfg<HD>;
  constexpr int BN = C::BN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                                   // [2][kQBytes]
  uint8_t* sKV = sQ + 2 * C::kQBytes;                   // [stages][K | V]
  uint8_t* sP = sKV + C::kStages * (C::kKBytes + C::kVBytes);  // [2][kPBytes]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + 2 * C::kPBytes);
  // barriers: q_full, k_full[S], v_full[S], kv_empty[S], s_full[2], p_full[2], o_full[2]
  const uint32_t bar_q = smem_u32(bars);
  const uint32_t bar_k = bar_q + 8, bar_v = bar_k + 8 * C::kStages, bar_e = bar_v + 8 * C::kStages;
  const uint32_t bar_s = bar_e + 8 * C::kStages, bar_p = bar_s + 16, bar_o = bar_p + 16;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 1 + 3 * C::kStages + 6);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pair = p.n_pairs - 1 - blockIdx.x;  // heaviest (latest) query tiles first
  const int h = blockIdx.y, b = blockIdx.z;
  const int kvh = h / (p.H / p.KVH);
  const int qt0 = 2 * pair, qt1 = 2 * pair + 1;
  const bool has1 = qt1 < p.n_q_tiles;
  // KV tiles needed by each query tile: keys <= last row of the tile, and < T
  const int kv_total = (p.T + BN - 1) / BN;
  const int n_kv0 = min(((qt0 + 1) * BQ + BN - 1) / BN, kv_total);
  const int n_kv1 = has1 ? min(((qt1 + 1) * BQ + BN - 1) / BN, kv_total) : 0;
  const int n_kv = max(n_kv0, n_kv1);

  if (threadIdx.x == 0) {
    mbar_init(bar_q, 1);
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(bar_k + 8 * s, 1);
      mbar_init(bar_v + 8 * s, 1);
      mbar_init(bar_e + 8 * s, 1);
    }
    for (int g = 0; g < 2; ++g) {
      mbar_init(bar_s + 8 * g, 1);
      mbar_init(bar_p + 8 * g, 128);
      mbar_init(bar_o + 8 * g, 1);
    }
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), C::kTmemCols);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmO);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  int fail_role = 0;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      mbar_expect_tx(bar_q, (has1 ? 2 : 1) * C::kQBytes);
#pragma unroll
      for (int c = 0; c < HD / 64; ++c) {
        tma_load_4d(smem_u32(sQ) + c * (BQ * 128), &tmQ, bar_q, c * 64, h, qt0 * BQ, b);
        if (has1) tma_load_4d(smem_u32(sQ) + C::kQBytes + c * (BQ * 128), &tmQ, bar_q, c * 64, h, qt1 * BQ, b);
      }
      bool ok = true;
      for (int j = 0; j < n_kv && ok; ++j) {
        const uint32_t s = j % C::kStages, ph = (j / C::kStages) & 1;
        if (!mbar_wait(bar_e + 8 * s, ph ^ 1, abort_flag)) { ok = false; fail_role = 1; break; }
        const uint32_t sk = smem_u32(sKV) + s * (C::kKBytes + C::kVBytes), sv = sk + C::kKBytes;
        mbar_expect_tx(bar_k + 8 * s, C::kKBytes);
#pragma unroll
        for (int c = 0; c < HD / 64; ++c) tma_load_4d(sk + c * (BN * 128), &tmK, bar_k + 8 * s, c * 64, kvh, j * BN, b);
        mbar_expect_tx(bar_v + 8 * s, C::kVBytes);
#pragma unroll
        for (int c = 0; c < HD / 64; ++c) tma_load_4d(sv + c * (BN * 128), &tmV, bar_v + 8 * s, c * 64, kvh, j * BN, b);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      bool ok = mbar_wait(bar_q, 0, abort_flag);
      if (!ok) fail_role = 2;
      tc_fence_after();
      auto issue_s = [&](int g, int j) {
        const uint32_t s = j % C::kStages;
        const uint32_t sq = smem_u32(sQ) + g * C::kQBytes, sk = smem_u32(sKV) + s * (C::kKBytes + C::kVBytes);
        const uint32_t d = tmem_base + (g ? C::kColS1 : C::kColS0);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t off_q = (k / 4) * (BQ * 128) + (k % 4) * 32, off_k = (k / 4) * (BN * 128) + (k % 4) * 32;
          umma_f16(d, make_smem_desc(sq + off_q, 16, 1024), make_smem_desc(sk + off_k, 16, 1024), p.idesc_qk, k > 0 ? 1u : 0u);
        }
        umma_commit(bar_s + 8 * g);
      };
      auto issue_pv = [&](int g, int j) {
        const uint32_t s = j % C::kStages;
        const uint32_t sp = smem_u32(sP) + g * C::kPBytes;
        const uint32_t sv = smem_u32(sKV) + s * (C::kKBytes + C::kVBytes) + C::kKBytes;
        const uint32_t d = tmem_base + (g ? C::kColO1 : C::kColO0);
#pragma unroll
        for (int k = 0; k < BN / 16; ++k) {
          const uint32_t off_p = (k / 4) * (BQ * 128) + (k % 4) * 32;   // P is K-major over keys
          const uint32_t off_v = k * (16 * 128);                         // V is MN-major: 16 key rows per step
          umma_f16(d, make_smem_desc(sp + off_p, 16, 1024), make_smem_desc(sv + off_v, BN * 128, 1024), p.idesc_pv, k > 0 ? 1u : 0u);
        }
        umma_commit(bar_o + 8 * g);
      };
      if (ok && n_kv > 0) {
        ok = mbar_wait(bar_k, 0, abort_flag);
        if (ok) {
          tc_fence_after();
          issue_s(0, 0);
          if (has1) issue_s(1, 0);
        } else fail_role = 2;
      }
      for (int j = 0; j < n_kv && ok; ++j) {
        const uint32_t s = j % C::kStages, ph = (j / C::kStages) & 1;
        if (!mbar_wait(bar_v + 8 * s, ph, abort_flag)) { ok = false; fail_role = 2; break; }
        for (int g = 0; g < 2 && ok; ++g) {
          const int n_g = g ? n_kv1 : n_kv0;
          if (j >= n_g) continue;
          if (!mbar_wait(bar_p + 8 * g, j & 1, abort_flag)) { ok = false; fail_role = 2; break; }
          tc_fence_after();
          issue_pv(g, j);
          if (j + 1 < n_g) {
            const uint32_t s2 = (j + 1) % C::kStages, ph2 = ((j + 1) / C::kStages) & 1;
            if (!mbar_wait(bar_k + 8 * s2, ph2, abort_flag)) { ok = false; fail_role = 2; break; }
            tc_fence_after();
            issue_s(g, j + 1);
          }
        }
        if (ok) umma_commit(bar_e + 8 * s);  // K_j and V_j are free once everything issued so far has run
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax groups
    const int g = (warp - 2) >> 2;           // 0: query tile qt0, 1: query tile qt1
    const int q = warp & 3;                  // TMEM lane quarter
    const int row = q * 32 + lane;
    const int qt = g ? qt1 : qt0;
    const int n_g = g ? n_kv1 : n_kv0;
    const int qi = qt * BQ + row;            // query index inside the sequence
    const uint32_t t_s = tmem_base + ((uint32_t)(q * 32) << 16) + (g ? C::kColS1 : C::kColS0);
    const uint32_t t_o = tmem_base + ((uint32_t)(q * 32) << 16) + (g ? C::kColO1 : C::kColO0);
    uint8_t* my_p = sP + g * C::kPBytes + row * 128;
    const int sw = row & 7;
    float o[HD];
#pragma unroll
    for (int i = 0; i < HD; ++i) o[i] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int j = 0; j < n_g; ++j) {
      if (!mbar_wait(bar_s + 8 * g, j & 1, abort_flag)) { ok = false; fail_role = 3; break; }
      tc_fence_after();
      const int key0 = j * BN;
      const bool need_mask = key0 + BN - 1 > qt * BQ;  // the tile reaches past the first row of the query tile
      // pass 1: row maximum
      float mx = m_run;
#pragma unroll
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(t_s + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float sv = __uint_as_float(r[i]);
          const bool keep = !need_mask || (key0 + c * 32 + i <= qi);
          mx = fmaxf(mx, keep ? sv : -INFINITY);
        }
      }
      const float m_new = mx;
      const float alpha = exp2f((m_run - m_new) * p.scale_log2);
      const float m_scaled = m_new * p.scale_log2;
      l_run *= alpha;
      // pass 2: probabilities -> bf16 P tile in shared memory (128-byte swizzle, K-major over keys)
#pragma unroll
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(t_s + c * 32, r);
        tmem_ld_wait();
        uint32_t packed[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const bool k0 = !need_mask || (key0 + c * 32 + i <= qi), k1 = !need_mask || (key0 + c * 32 + i + 1 <= qi);
          const float p0 = k0 ? exp2f(__uint_as_float(r[i]) * p.scale_log2 - m_scaled) : 0.f;
          const float p1 = k1 ? exp2f(__uint_as_float(r[i + 1]) * p.scale_log2 - m_scaled) : 0.f;
          l_run += p0 + p1;
          __nv_bfloat162 v = __floats2bfloat162_rn(p0, p1);
          packed[i >> 1] = *reinterpret_cast<uint32_t*>(&v);
        }
        uint8_t* blk = my_p + (c >> 1) * (BQ * 128);  // 64 keys per swizzled K-block
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
          const int chunk = (c & 1) * 4 + jj;
          *reinterpret_cast<uint4*>(blk + ((chunk ^ sw) << 4)) =
              make_uint4(packed[4 * jj], packed[4 * jj + 1], packed[4 * jj + 2], packed[4 * jj + 3]);
        }
      }
      m_run = m_new;
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(bar_p + 8 * g);
      // fold the partial O of this tile into the running accumulators
      if (!mbar_wait(bar_o + 8 * g, j & 1, abort_flag)) { ok = false; fail_role = 3; break; }
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(t_o + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) o[c * 32 + i] = o[c * 32 + i] * alpha + __uint_as_float(r[i]);
      }
      tc_fence_before();
    }
    // epilogue: normalise, stage (reusing this group's Q tile: every MMA that read it has completed), store
    if (ok && n_g > 0) {
      const float inv_l = 1.f / l_run;
      if (qi < p.T) p.lse[((size_t)b * p.H + h) * p.T + qi] = m_run * p.scale + logf(l_run);
      uint8_t* stage_o = sQ + g * C::kQBytes + row * 128;
#pragma unroll
      for (int c = 0; c < HD / 64; ++c) {
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) {
          uint32_t w[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int i = c * 64 + jj * 8 + 2 * e;
            __nv_bfloat162 v = __floats2bfloat162_rn(o[i] * inv_l, o[i + 1] * inv_l);
            w[e] = *reinterpret_cast<uint32_t*>(&v);
          }
          *reinterpret_cast<uint4*>(stage_o + c * (BQ * 128) + ((jj ^ sw) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
      fence_proxy_async_smem();
      named_barrier_sync(1 + g, 128);
      if (row == 0) {
#pragma unroll
        for (int c = 0; c < HD / 64; ++c)
          tma_store_4d(&tmO, smem_u32(sQ) + g * C::kQBytes + c * (BQ * 128), c * 64, h, qt * BQ, b);
        tma_commit_group();
        tma_wait_group<0>();
      }
    }
  }

  if (fail_role != 0 && p.status != nullptr) {
    if (atomicCAS(p.status, 0, 2) == 0) {
      p.status[1] = fail_role;
      p.status[2] = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
      p.status[3] = 0;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

template <int HD>
int launch_fwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& to, const FParams& p,
               cudaStream_t st) {
  auto kern = flash_fwd_kernel<HD>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, FCfg<HD>::kSmem) != cudaSuccess) {
      nnb_set_error("flash_fwd: cannot reserve %d bytes of shared memory", FCfg<HD>::kSmem);
      return -3;
    }
    configured = true;
  }
  dim3 grid(p.n_pairs, p.H, p.B);
  kern<<<grid, kThreads, FCfg<HD>::kSmem, st>>>(tq, tk, tv, to, p);
  return 0;
}

}  // namespace

// q: [B, T, H, hd] addressed by element strides (q_sb, q_st, q_sh) with a contiguous last dim; k, v:
// [B, T, KVH, hd] likewise; o: [B, T, H, hd] likewise; lse: fp32 [B, H, T] contiguous.
extern "C" int nnb_flash_fwd(const void* q, const void* k, const void* v, void* o, void* lse, int B, int T, int H, int KVH,
                             int hd, long long q_sb, long long q_st, long long q_sh, long long k_sb, long long k_st,
                             long long k_sh, long long v_sb, long long v_st, long long v_sh, long long o_sb, long long o_st,
                             long long o_sh, float scale, int dtype, void* status, cudaStream_t st) {
  NNB_REQUIRE(hd == 64 || hd == 128, "flash_fwd: head_dim %d not supported (64 or 128)", hd);
  NNB_REQUIRE(dtype == NNB_BF16, "flash_fwd: bf16 only (dtype code %d)", dtype);
  NNB_REQUIRE(H % KVH == 0 && B > 0 && T > 0, "flash_fwd: bad shape B=%d T=%d H=%d KVH=%d", B, T, H, KVH);
  const CUtensorMapDataType dt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const int BN = hd == 64 ? 128 : 64;
  CUtensorMap tq, tk, tv, to;
  if (!nnb_make_tmap_4d(&tq, dt, 2, q, hd, H, T, B, q_sh * 2, q_st * 2, q_sb * 2, 64, 1, BQ, "flash Q")) return -4;
  if (!nnb_make_tmap_4d(&tk, dt, 2, k, hd, KVH, T, B, k_sh * 2, k_st * 2, k_sb * 2, 64, 1, BN, "flash K")) return -4;
  if (!nnb_make_tmap_4d(&tv, dt, 2, v, hd, KVH, T, B, v_sh * 2, v_st * 2, v_sb * 2, 64, 1, BN, "flash V")) return -4;
  if (!nnb_make_tmap_4d(&to, dt, 2, o, hd, H, T, B, o_sh * 2, o_st * 2, o_sb * 2, 64, 1, BQ, "flash O")) return -4;
  FParams p{};
  p.B = B; p.H = H; p.KVH = KVH; p.T = T;
  p.n_q_tiles = (T + BQ - 1) / BQ;
  p.n_pairs = (p.n_q_tiles + 1) / 2;
  p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.lse = static_cast<float*>(lse);
  p.idesc_qk = sm100::make_idesc_f16(1, 0, 0, BQ, BN);
  p.idesc_pv = sm100::make_idesc_f16(1, 0, 1, BQ, hd);
  p.status = static_cast<int*>(status);
  const int rc = hd == 64 ? launch_fwd<64>(tq, tk, tv, to, p, st) : launch_fwd<128>(tq, tk, tv, to, p, st);
  if (rc != 0) return rc;
  NNB_LAUNCH_OK("flash_fwd");
  return 0;
}
