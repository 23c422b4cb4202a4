// Cross-entropy half of the fused linear + cross-entropy over the tied head.
//
// The head is processed in row chunks: logits_c = x_c W^T (tcgen05 GEMM, bf16 [R, V]) -> this kernel
// -> dx_c = g W and dW += g^T x_c (tcgen05 GEMMs). The kernel reads each logit from HBM once and
// writes it once: a block owns a row, reduces max and sum-exp in fp32, writes
// loss_row = logsumexp - logit[target], and overwrites the row in place with
// g = (softmax - onehot) * grad_scale. Only 16-bit logits of one chunk exist, never the fp32 copy of
// the full [B*T, V] matrix that the unfused path makes (6.6 GB at the 114M shape).
// Same contract as the reference's Triton kernel (nanonemo/kernels/triton/linear_ce.py:21-41).
#include "common.cuh"

namespace {

constexpr int kCeThreads = 256;

template <typename T>
__device__ __forceinline__ float2 unpack2(uint32_t w);
template <>
__device__ __forceinline__ float2 unpack2<__nv_bfloat16>(uint32_t w) {
  return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&w));
}
template <>
__device__ __forceinline__ float2 unpack2<__half>(uint32_t w) {
  return __half22float2(*reinterpret_cast<__half2*>(&w));
}
template <typename T>
__device__ __forceinline__ uint32_t pack2(float a, float b);
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Sweep 1 of a row: every thread keeps a running (max, sum-exp) over its 16-byte vectors, then the block combines the
// pairs. Returns the row's (max, sum of exp(x - max)) to every thread.
template <typename T>
__device__ __forceinline__ float2 row_max_sumexp(const T* __restrict__ x, int nvec, float* s_m, float* s_s) {
  constexpr float kLog2e = 1.4426950408889634f;
  float m = -INFINITY, s = 0.f;
  for (int v = threadIdx.x; v < nvec; v += kCeThreads) {
    const uint4 raw = reinterpret_cast<const uint4*>(x)[v];
    const uint32_t* w = reinterpret_cast<const uint32_t*>(&raw);
    float f[8];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 t = unpack2<T>(w[k]);
      f[2 * k] = t.x; f[2 * k + 1] = t.y;
    }
    float lm = f[0];
#pragma unroll
    for (int k = 1; k < 8; ++k) lm = fmaxf(lm, f[k]);
    if (lm > m) {
      s *= exp2f((m - lm) * kLog2e);
      m = lm;
    }
    const float mb = m * kLog2e;
#pragma unroll
    for (int k = 0; k < 8; ++k) s += exp2f(f[k] * kLog2e - mb);
  }
  // combine (m, s) pairs: warp, then block
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
    const float mn = fmaxf(m, m2);
    s = (m == -INFINITY ? 0.f : s * exp2f((m - mn) * kLog2e)) + (m2 == -INFINITY ? 0.f : s2 * exp2f((m2 - mn) * kLog2e));
    m = mn;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) { s_m[warp] = m; s_s[warp] = s; }
  __syncthreads();
  float M = s_m[0];
#pragma unroll
  for (int i = 1; i < kCeThreads / 32; ++i) M = fmaxf(M, s_m[i]);
  float S = 0.f;
#pragma unroll
  for (int i = 0; i < kCeThreads / 32; ++i) S += s_m[i] == -INFINITY ? 0.f : s_s[i] * exp2f((s_m[i] - M) * kLog2e);
  return make_float2(M, S);
}

// Sweep 2 of a row: overwrite it with (softmax - onehot) * gs, softmax = exp(x - lse). tgt outside [0, 8 nvec) = no onehot here.
template <typename T>
__device__ __forceinline__ void row_write_grad(T* __restrict__ x, int nvec, long long tgt, float lse, float gs) {
  constexpr float kLog2e = 1.4426950408889634f;
  const float lb = lse * kLog2e;
  for (int v = threadIdx.x; v < nvec; v += kCeThreads) {
    uint4 raw = reinterpret_cast<const uint4*>(x)[v];
    uint32_t* w = reinterpret_cast<uint32_t*>(&raw);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = unpack2<T>(w[k]);
      const int col = v * 8 + 2 * k;
      float g0 = exp2f(f.x * kLog2e - lb) * gs, g1 = exp2f(f.y * kLog2e - lb) * gs;
      if (col == tgt) g0 -= gs;
      if (col + 1 == tgt) g1 -= gs;
      w[k] = pack2<T>(g0, g1);
    }
    reinterpret_cast<uint4*>(x)[v] = raw;
  }
}

// One block per row, two sweeps. Sweep 1 reads the row from HBM; sweep 2 re-reads it and overwrites it with the gradient.
// A row is ~100 KB and a few hundred rows are in flight, so the re-read is meant to hit L2; measured, about half of it still
// reaches HBM (the GEMM that wrote the logits and the gradient writes compete for the same L2), which is why the fused
// head uses ce_grad_from_stats_kernel (one sweep) whenever the GEMM epilogue could produce the statistics.
template <typename T>
__global__ void __launch_bounds__(kCeThreads) ce_inplace_kernel(T* __restrict__ logits, const long long* __restrict__ targets,
                                                                float* __restrict__ loss_rows, int V, long long ld,
                                                                float grad_scale) {
  extern __shared__ uint8_t s_occupancy_pad[];  // sized by the launcher to cap resident blocks per SM (see nnb_ce_inplace)
  (void)s_occupancy_pad;
  __shared__ float s_m[kCeThreads / 32], s_s[kCeThreads / 32];
  const long long row = blockIdx.x;
  T* x = logits + row * ld;
  const long long tgt = targets[row];
  const bool valid = tgt >= 0 && tgt < V;
  const float x_t = valid ? to_f32(x[tgt]) : 0.f;
  const float2 ms = row_max_sumexp<T>(x, V >> 3, s_m, s_s);
  const float lse = ms.x + logf(ms.y);
  if (threadIdx.x == 0) loss_rows[row] = valid ? lse - x_t : 0.f;
  row_write_grad<T>(x, V >> 3, tgt, lse, valid ? grad_scale : 0.f);  // ignored rows contribute no gradient
}

// One-sweep form: the head GEMM's epilogue already reduced every 256-column tile of the row to (max, sum of exp(x - max))
// (`tile_stats` [R, n_tiles, 2], written by nnb_gemm_ce_stats); the block combines the n_tiles pairs, writes the row loss and
// overwrites the row with the gradient. The logits are read once and written once.
template <typename T>
__global__ void __launch_bounds__(kCeThreads) ce_grad_from_stats_kernel(T* __restrict__ logits, const long long* __restrict__ targets,
                                                                        const float* __restrict__ tile_stats, int n_tiles,
                                                                        float* __restrict__ loss_rows, int V, long long ld,
                                                                        float grad_scale) {
  constexpr float kLog2e = 1.4426950408889634f;
  __shared__ float s_m[kCeThreads / 32], s_s[kCeThreads / 32];
  const long long row = blockIdx.x;
  T* x = logits + row * ld;
  const long long tgt = targets[row];
  const bool valid = tgt >= 0 && tgt < V;
  const float x_t = valid ? to_f32(x[tgt]) : 0.f;
  const float2* st = reinterpret_cast<const float2*>(tile_stats) + row * n_tiles;
  float m = -INFINITY, s = 0.f;
  for (int i = threadIdx.x; i < n_tiles; i += kCeThreads) {
    const float2 v = st[i];
    const float mn = fmaxf(m, v.x);
    s = (m == -INFINITY ? 0.f : s * exp2f((m - mn) * kLog2e)) + (v.x == -INFINITY ? 0.f : v.y * exp2f((v.x - mn) * kLog2e));
    m = mn;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
    const float mn = fmaxf(m, m2);
    s = (m == -INFINITY ? 0.f : s * exp2f((m - mn) * kLog2e)) + (m2 == -INFINITY ? 0.f : s2 * exp2f((m2 - mn) * kLog2e));
    m = mn;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) { s_m[warp] = m; s_s[warp] = s; }
  __syncthreads();
  float M = s_m[0];
#pragma unroll
  for (int i = 1; i < kCeThreads / 32; ++i) M = fmaxf(M, s_m[i]);
  float S = 0.f;
#pragma unroll
  for (int i = 0; i < kCeThreads / 32; ++i) S += s_m[i] == -INFINITY ? 0.f : s_s[i] * exp2f((s_m[i] - M) * kLog2e);
  const float lse = M + logf(S);
  if (threadIdx.x == 0) loss_rows[row] = valid ? lse - x_t : 0.f;
  row_write_grad<T>(x, V >> 3, tgt, lse, valid ? grad_scale : 0.f);
}

// Vocabulary-parallel variant, first half: this rank's slice of the row -> stats[row] = (max, sum-exp, target logit or 0).
// `targets` are GLOBAL ids; this rank owns columns [v0, v0 + V).
template <typename T>
__global__ void __launch_bounds__(kCeThreads) ce_stats_kernel(const T* __restrict__ logits, const long long* __restrict__ targets,
                                                              float* __restrict__ stats, int V, long long ld, long long v0) {
  __shared__ float s_m[kCeThreads / 32], s_s[kCeThreads / 32];
  const long long row = blockIdx.x;
  const T* x = logits + row * ld;
  const long long tgt = targets[row] - v0;
  const float2 ms = row_max_sumexp<T>(x, V >> 3, s_m, s_s);
  if (threadIdx.x == 0) {
    stats[row * 4 + 0] = ms.x;
    stats[row * 4 + 1] = ms.y;
    stats[row * 4 + 2] = (tgt >= 0 && tgt < V) ? to_f32(x[tgt]) : 0.f;
    stats[row * 4 + 3] = 0.f;
  }
}

// Second half: stats_all [world, R, 4] holds every rank's (max, sum-exp, target logit); each block combines them to the
// row's global logsumexp, writes the row loss (identical on all ranks) and overwrites this rank's slice with the gradient.
template <typename T>
__global__ void __launch_bounds__(kCeThreads) ce_grad_vp_kernel(T* __restrict__ logits, const long long* __restrict__ targets,
                                                                const float* __restrict__ stats_all, float* __restrict__ loss_rows,
                                                                int V, long long ld, long long v0, long long v_total, int world,
                                                                long long R, float grad_scale) {
  const long long row = blockIdx.x;
  T* x = logits + row * ld;
  const long long tg = targets[row];
  const bool valid = tg >= 0 && tg < v_total;
  float M = -INFINITY;
  for (int r = 0; r < world; ++r) M = fmaxf(M, stats_all[((long long)r * R + row) * 4]);
  float S = 0.f, x_t = 0.f;
  for (int r = 0; r < world; ++r) {
    const float* st = stats_all + ((long long)r * R + row) * 4;
    S += st[0] == -INFINITY ? 0.f : st[1] * expf(st[0] - M);
    x_t += st[2];
  }
  const float lse = M + logf(S);
  if (threadIdx.x == 0) loss_rows[row] = valid ? lse - x_t : 0.f;
  row_write_grad<T>(x, V >> 3, valid ? tg - v0 : -1, lse, valid ? grad_scale : 0.f);
}

}  // namespace

// logits: 16-bit [R, V] with row stride ld (elements), overwritten with the scaled gradient;
// targets: int64 [R] (out-of-range = ignored row); loss_rows: fp32 [R].
extern "C" int nnb_ce_inplace(void* logits, const void* targets, void* loss_rows, long long R, int V, long long ld,
                              float grad_scale, int dtype, cudaStream_t st) {
  NNB_REQUIRE(V % 8 == 0 && V > 0, "ce: V=%d must be a positive multiple of 8", V);
  NNB_REQUIRE(ld % 8 == 0 && nnb_aligned16(logits), "ce: logits rows must be 16-byte aligned");
  if (R == 0) return 0;
  // The second sweep must hit L2: keep the rows in flight (resident blocks x row bytes) well below the L2 size by
  // padding each block's dynamic shared memory so that only a few blocks fit per SM.
  int l2 = 0, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&l2, cudaDevAttrL2CacheSize, dev);
  const long long row_bytes = (long long)V * 2;
  int per_sm = (int)(((long long)l2 / 2) / (row_bytes * nnb_num_sms()));
  per_sm = per_sm < 1 ? 1 : (per_sm > 8 ? 8 : per_sm);
  size_t pad = 0;  // 47 KB of padding (no opt-in needed) leaves room for 4 blocks per SM
  if (per_sm < 8) pad = (size_t)min(47 * 1024, (220 * 1024) / per_sm);
  NNB_DISPATCH_16(dtype, T, {
    ce_inplace_kernel<T><<<(unsigned)R, kCeThreads, pad, st>>>((T*)logits, (const long long*)targets, (float*)loss_rows, V, ld, grad_scale);
  });
  NNB_LAUNCH_OK("ce_inplace");
  return 0;
}


// One-sweep cross-entropy on logits whose per-tile statistics came out of the head GEMM (nnb_gemm_ce_stats):
// tile_stats fp32 [R, n_tiles, 2]. Same outputs as nnb_ce_inplace.
extern "C" int nnb_ce_grad_from_stats(void* logits, const void* targets, const void* tile_stats, int n_tiles, void* loss_rows,
                                      long long R, int V, long long ld, float grad_scale, int dtype, cudaStream_t st) {
  NNB_REQUIRE(V % 8 == 0 && V > 0 && n_tiles > 0, "ce_from_stats: V=%d must be a positive multiple of 8", V);
  NNB_REQUIRE(ld % 8 == 0 && nnb_aligned16(logits) && nnb_aligned16(tile_stats), "ce_from_stats: rows must be 16-byte aligned");
  if (R == 0) return 0;
  NNB_DISPATCH_16(dtype, T, {
    ce_grad_from_stats_kernel<T><<<(unsigned)R, kCeThreads, 0, st>>>((T*)logits, (const long long*)targets, (const float*)tile_stats,
                                                                     n_tiles, (float*)loss_rows, V, ld, grad_scale);
  });
  NNB_LAUNCH_OK("ce_grad_from_stats");
  return 0;
}


// Vocabulary-parallel cross-entropy in two launches with one small all-gather of `stats` between them (done by the caller).
// logits: this rank's [R, V] slice of the row (columns v0 .. v0+V of v_total); targets: global ids.
extern "C" int nnb_ce_stats(const void* logits, const void* targets, void* stats, long long R, int V, long long ld,
                            long long v0, int dtype, cudaStream_t st) {
  NNB_REQUIRE(V % 8 == 0 && V > 0, "ce_stats: V=%d must be a positive multiple of 8", V);
  NNB_REQUIRE(ld % 8 == 0 && nnb_aligned16(logits), "ce_stats: logits rows must be 16-byte aligned");
  if (R == 0) return 0;
  NNB_DISPATCH_16(dtype, T, {
    ce_stats_kernel<T><<<(unsigned)R, kCeThreads, 0, st>>>((const T*)logits, (const long long*)targets, (float*)stats, V, ld, v0);
  });
  NNB_LAUNCH_OK("ce_stats");
  return 0;
}

extern "C" int nnb_ce_grad_vp(void* logits, const void* targets, const void* stats_all, void* loss_rows, long long R, int V,
                              long long ld, long long v0, long long v_total, int world, float grad_scale, int dtype,
                              cudaStream_t st) {
  NNB_REQUIRE(V % 8 == 0 && V > 0, "ce_grad_vp: V=%d must be a positive multiple of 8", V);
  NNB_REQUIRE(ld % 8 == 0 && nnb_aligned16(logits), "ce_grad_vp: logits rows must be 16-byte aligned");
  NNB_REQUIRE(world >= 1 && world <= 64, "ce_grad_vp: world=%d out of range", world);
  if (R == 0) return 0;
  NNB_DISPATCH_16(dtype, T, {
    ce_grad_vp_kernel<T><<<(unsigned)R, kCeThreads, 0, st>>>((T*)logits, (const long long*)targets, (const float*)stats_all,
                                                             (float*)loss_rows, V, ld, v0, v_total, world, R, grad_scale);
  });
  NNB_LAUNCH_OK("ce_grad_vp");
  return 0;
}
