// Causal grouped-query FlashAttention forward on tcgen05 / TMEM / TMA for sm_100a.
//
// One CTA owns one 128-row query tile of one (batch, query head) and walks the key/value tiles (64 keys
// each) up to the diagonal; two CTAs are resident per SM at head_dim 64. 192 threads per CTA:
//   warp 0        TMA producer: Q once, then K_j / V_j into a ring of stages (4-D tensor maps over
//                 (head_dim, head, t, batch), so any (B,T,H,hd) / (B,H,T,hd) / packed-QKV strides work and
//                 query head h reads KV head h / group directly — nothing is repeated or copied);
//   warp 1        MMA issuer: S_j = Q K_j^T and O_j = P_j V_j with tcgen05.mma, accumulators in TMEM;
//   warps 2..5    softmax, one thread per query row (= TMEM lane): tcgen05.ld the scores, online max and
//                 sum with exp2, bf16 P_j into a 128-byte swizzled shared tile (the A operand of the second
//                 MMA). O accumulates IN TENSOR MEMORY over the key tiles; the row maximum used for the
//                 exponentials is only raised when a tile exceeds it by more than 2^8 (probabilities then
//                 stay below 256, exact in fp32 / safe in bf16), so the accumulator has to be rescaled —
//                 tcgen05.ld, multiply, tcgen05.st by the softmax threads — on a few tiles only.
// The score tile and the P tile are DOUBLE BUFFERED and the MMA warp runs two tiles ahead: S_{j+2} is
// issued as soon as the softmax threads have read S_j, and P_j V_j runs while they work on tile j+1, so
// neither side waits for a hand-off in steady state.
// Outputs: O (bf16) through a swizzled staging tile + TMA store, and L = m * scale + ln(l) per row (fp32)
// for the backward pass. Every mbarrier wait is bounded; on expiry the kernel records a status word
// and leaves cleanly.
//
// Replaces the reference's WMMA kernel for sm_75 (nanonemo/kernels/cuda/flash_attn.cu:52-174) and
// the mem-efficient SDPA path it benchmarks against; same math contract (causal, GQA-direct, saves
// the log-sum-exp per row).
#include <type_traits>

#include "sm100.cuh"

#ifdef NNB_PROFILE
extern "C" int nnb_flash_prof_read(unsigned long long* out) { return (int)cudaMemcpyFromSymbol(out, g_flash_prof, sizeof(g_flash_prof)); }
#endif

namespace {

using namespace sm100;

constexpr int BQ = 128;  // query rows per tile (= TMEM lanes)
constexpr int kThreads = 192;
constexpr int kSoftmaxThreads = 128;

template <int HD>
struct FCfg {
  static constexpr int BN = 64;                             // keys per KV tile
  static constexpr int kStages = 3;  // 3 x 16 KB at head_dim 64: two CTAs (2 x ~100 KB) fit in one SM
  static constexpr int kCtasPerSm = (HD == 64) ? 2 : 1;
  static constexpr int kQBytes = BQ * HD * 2;               // HD/64 swizzled K-blocks of 16 KB
  static constexpr int kKBytes = BN * HD * 2;
  static constexpr int kVBytes = BN * HD * 2;
  static constexpr int kPBytes = BQ * BN * 2;               // one swizzled K-block of 16 KB per buffer
  static constexpr int kSmem = kQBytes + kStages * (kKBytes + kVBytes) + 2 * kPBytes + 1024 + 256;
  static constexpr int kColS = 0;                           // S buffers at columns 0 and 64
  static constexpr int kColO = 128;                         // O accumulator from column 128
  static constexpr int kTmemCols = 256;
};

struct FParams {
  int B, H, KVH, T;
  int n_q_tiles;
  float scale_log2;   // softmax scale * log2(e)
  float scale;        // softmax scale
  float* lse;         // [B, H, T]
  uint32_t idesc_qk, idesc_pv;
  int* status;
};

template <int HD, bool F16>
__global__ void __launch_bounds__(kThreads, FCfg<HD>::kCtasPerSm)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO, const FParams p) {
  using C = FCfg<HD>;
  constexpr int BN = C::BN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sKV = sQ + C::kQBytes;                              // [stages][K | V]
  uint8_t* sP = sKV + C::kStages * (C::kKBytes + C::kVBytes);  // [2][kPBytes]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + 2 * C::kPBytes);
  // barriers: q_full, k_full[S], v_full[S], kv_empty[S], s_full[2], p_full[2], o_tile, o_all (+ 2 unused slots)
  const uint32_t bar_q = smem_u32(bars);
  const uint32_t bar_k = bar_q + 8, bar_v = bar_k + 8 * C::kStages, bar_e = bar_v + 8 * C::kStages;
  const uint32_t bar_s = bar_e + 8 * C::kStages, bar_p = bar_s + 16, bar_o = bar_p + 16;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 1 + 3 * C::kStages + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Longest-job-first over the WHOLE grid: the query tile is the slowest-varying block index, so every CTA of the latest
  // (heaviest) query tile is scheduled before any of the next one and the kernel ends on the one-key-tile CTAs.
  const int qt = p.n_q_tiles - 1 - blockIdx.z;
  const int h = blockIdx.x, b = blockIdx.y;
  const int kvh = h / (p.H / p.KVH);
  const int kv_total = (p.T + BN - 1) / BN;
  const int n_kv = min(((qt + 1) * BQ + BN - 1) / BN, kv_total);  // KV tiles holding keys <= the tile's last row

  if (threadIdx.x == 0) {
    mbar_init(bar_q, 1);
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(bar_k + 8 * s, 1);
      mbar_init(bar_v + 8 * s, 1);
      mbar_init(bar_e + 8 * s, 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar_s + 8 * i, 1);
      mbar_init(bar_p + 8 * i, kSoftmaxThreads);
      mbar_init(bar_o + 8 * i, 1);
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
      mbar_expect_tx(bar_q, C::kQBytes);
#pragma unroll
      for (int c = 0; c < HD / 64; ++c) tma_load_4d(smem_u32(sQ) + c * (BQ * 128), &tmQ, bar_q, c * 64, h, qt * BQ, b);
      for (int j = 0; j < n_kv; ++j) {
        const uint32_t s = j % C::kStages, ph = (j / C::kStages) & 1;
        if (!mbar_wait(bar_e + 8 * s, ph ^ 1, abort_flag)) { fail_role = 1; break; }
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
      auto issue_s = [&](int j) -> bool {  // S_j = Q K_j^T into score buffer j & 1
        const uint32_t s = j % C::kStages, ph = (j / C::kStages) & 1;
        if (!mbar_wait(bar_k + 8 * s, ph, abort_flag)) return false;
        tc_fence_after();
        const uint32_t sk = smem_u32(sKV) + s * (C::kKBytes + C::kVBytes);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t off_q = (k / 4) * (BQ * 128) + (k % 4) * 32, off_k = (k / 4) * (BN * 128) + (k % 4) * 32;
          umma_f16(tmem_base + C::kColS + (j & 1) * BN, make_smem_desc(smem_u32(sQ) + off_q, 16, 1024),
                   make_smem_desc(sk + off_k, 16, 1024), p.idesc_qk, k > 0 ? 1u : 0u);
        }
        umma_commit(bar_s + 8 * (j & 1));
        return true;
      };
      if (ok && n_kv > 0) ok = issue_s(0);
      if (ok && n_kv > 1) ok = issue_s(1);
      for (int j = 0; j < n_kv && ok; ++j) {
        const uint32_t s = j % C::kStages, ph = (j / C::kStages) & 1;
        const int pb = j & 1;
        if (!mbar_wait(bar_v + 8 * s, ph, abort_flag)) { ok = false; break; }
        if (!mbar_wait(bar_p + 8 * pb, (j >> 1) & 1, abort_flag)) { ok = false; break; }   // P_j written, S_j consumed, O rescaled if needed
        tc_fence_after();
        const uint32_t sv = smem_u32(sKV) + s * (C::kKBytes + C::kVBytes) + C::kKBytes;
        const uint32_t sp = smem_u32(sP) + pb * C::kPBytes;
#pragma unroll
        for (int k = 0; k < BN / 16; ++k)  // P is K-major over keys; V is MN-major: 16 key rows (2048 B) per step
          umma_f16(tmem_base + C::kColO, make_smem_desc(sp + k * 32, 16, 1024),
                   make_smem_desc(sv + k * (16 * 128), BN * 128, 1024), p.idesc_pv, (j > 0 || k > 0) ? 1u : 0u);
        umma_commit(bar_o);  // one completion per tile: O holds the sum over tiles 0..j
        if (j == n_kv - 1) umma_commit(bar_o + 8);  // one-shot "all products done" for the epilogue (no phase aliasing)
        umma_commit(bar_e + 8 * s);  // K_j and V_j are free once everything issued so far has run
        if (j + 2 < n_kv) ok = issue_s(j + 2);  // score buffer j & 1 was released by bar_p above
      }
      if (!ok) fail_role = 2;
    }
  } else {
#include "flash_fwd_softmax.inc"
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

template <int HD, bool F16>
int launch_fwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& to, const FParams& p,
               cudaStream_t st) {
  auto kern = flash_fwd_kernel<HD, F16>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, FCfg<HD>::kSmem) != cudaSuccess) {
      nnb_set_error("flash_fwd: cannot reserve %d bytes of shared memory", FCfg<HD>::kSmem);
      return -3;
    }
    configured = true;
  }
  dim3 grid(p.H, p.B, p.n_q_tiles);
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
  NNB_REQUIRE(dtype == NNB_BF16 || dtype == NNB_F16, "flash_fwd: bf16 or fp16 only (dtype code %d)", dtype);
  const bool f16 = dtype == NNB_F16;
  NNB_REQUIRE(H % KVH == 0 && B > 0 && T > 0, "flash_fwd: bad shape B=%d T=%d H=%d KVH=%d", B, T, H, KVH);
  const CUtensorMapDataType dt = f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const int BN = 64;
  CUtensorMap tq, tk, tv, to;
  if (!nnb_make_tmap_4d(&tq, dt, 2, q, hd, H, T, B, q_sh * 2, q_st * 2, q_sb * 2, 64, 1, BQ, "flash Q")) return -4;
  if (!nnb_make_tmap_4d(&tk, dt, 2, k, hd, KVH, T, B, k_sh * 2, k_st * 2, k_sb * 2, 64, 1, BN, "flash K")) return -4;
  if (!nnb_make_tmap_4d(&tv, dt, 2, v, hd, KVH, T, B, v_sh * 2, v_st * 2, v_sb * 2, 64, 1, BN, "flash V")) return -4;
  if (!nnb_make_tmap_4d(&to, dt, 2, o, hd, H, T, B, o_sh * 2, o_st * 2, o_sb * 2, 64, 1, BQ, "flash O")) return -4;
  FParams p{};
  p.B = B; p.H = H; p.KVH = KVH; p.T = T;
  p.n_q_tiles = (T + BQ - 1) / BQ;
  p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.lse = static_cast<float*>(lse);
  p.idesc_qk = sm100::make_idesc_f16(f16 ? 0 : 1, 0, 0, BQ, BN);
  p.idesc_pv = sm100::make_idesc_f16(f16 ? 0 : 1, 0, 1, BQ, hd);
  p.status = static_cast<int*>(status);
  const int rc = hd == 64 ? (f16 ? launch_fwd<64, true>(tq, tk, tv, to, p, st) : launch_fwd<64, false>(tq, tk, tv, to, p, st))
                          : (f16 ? launch_fwd<128, true>(tq, tk, tv, to, p, st) : launch_fwd<128, false>(tq, tk, tv, to, p, st));
  if (rc != 0) return rc;
  NNB_LAUNCH_OK("flash_fwd");
  return 0;
}
