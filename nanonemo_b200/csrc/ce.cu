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

// One block per row, two sweeps. Sweep 1 reads the row from HBM and keeps a running (max, sum-exp)
// per thread; sweep 2 re-reads it — a row is ~100 KB and a few hundred rows are in flight, far below
// the 126 MB L2, so the second read does not reach HBM — and overwrites it with the gradient.
template <typename T>
__global__ void __launch_bounds__(kCeThreads) ce_inplace_kernel(T* __restrict__ logits, const long long* __restrict__ targets,
                                                                float* __restrict__ loss_rows, int V, long long ld,
                                                                float grad_scale) {
  extern __shared__ uint8_t s_occupancy_pad[];  // sized by the launcher to cap resident blocks per SM (see nnb_ce_inplace)
  (void)s_occupancy_pad;
  __shared__ float s_m[kCeThreads / 32], s_s[kCeThreads / 32];
  constexpr float kLog2e = 1.4426950408889634f;
  const long long row = blockIdx.x;
  T* x = logits + row * ld;
  const int nvec = V >> 3;
  const long long tgt = targets[row];
  const bool valid = tgt >= 0 && tgt < V;
  const float x_t = valid ? to_f32(x[tgt]) : 0.f;

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
  const float lse = M + logf(S);
  if (threadIdx.x == 0) loss_rows[row] = valid ? lse - x_t : 0.f;
  const float gs = valid ? grad_scale : 0.f;  // ignored rows contribute no gradient
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
