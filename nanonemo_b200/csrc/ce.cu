// Cross-entropy half of the fused linear + cross-entropy over the tied head.
//
// The head is processed in row chunks: logits_c = x_c W^T (tcgen05 GEMM, bf16 [R, V]) -> this kernel
// -> dx_c = g W and dW += g^T x_c (tcgen05 GEMMs). The kernel makes ONE pass over the chunk's logits:
// a block owns a row, holds it in registers as packed 16-bit pairs, reduces max and sum-exp in fp32,
// writes loss_row = logsumexp - logit[target], and overwrites the row in place with
// g = (softmax - onehot) * grad_scale. The [B*T, V] logits never exist (at the 114M shape they would
// be 3.3 GB in bf16 plus 6.6 GB for the fp32 copy the unfused path makes).
// Same contract as the reference's Triton kernel (nanonemo/kernels/triton/linear_ce.py:21-41), which
// re-reads each row in 4096-wide blocks; here the row stays on chip between the two phases.
#include "common.cuh"

namespace {

constexpr int kCeThreads = 512;
constexpr int kMaxVec = 16;  // uint4 (8 x 16-bit) per thread: rows up to 512 * 16 * 8 = 65536 columns

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

__device__ __forceinline__ float block_reduce(float v, float* s_buf, bool is_max) {
  v = is_max ? warp_max(v) : warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) s_buf[warp] = v;
  __syncthreads();
  float r = (lane < (int)(blockDim.x >> 5)) ? s_buf[lane] : (is_max ? -INFINITY : 0.f);
  r = is_max ? warp_max(r) : warp_sum(r);
  return r;
}

template <typename T>
__global__ void __launch_bounds__(kCeThreads) ce_inplace_kernel(T* __restrict__ logits, const long long* __restrict__ targets,
                                                                float* __restrict__ loss_rows, int V, long long ld,
                                                                float grad_scale) {
  __shared__ float s_buf[kCeThreads / 32];
  const long long row = blockIdx.x;
  T* x = logits + row * ld;
  const int nvec = V >> 3;
  const long long tgt = targets[row];
  const bool valid = tgt >= 0 && tgt < V;
  const float x_t = valid ? to_f32(x[tgt]) : 0.f;

  uint4 regs[kMaxVec];
  float m = -INFINITY;
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) {
    const int v = threadIdx.x + i * kCeThreads;
    if (v < nvec) {
      regs[i] = reinterpret_cast<const uint4*>(x)[v];
      const uint32_t* w = reinterpret_cast<const uint32_t*>(&regs[i]);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = unpack2<T>(w[k]);
        m = fmaxf(m, fmaxf(f.x, f.y));
      }
    }
  }
  m = block_reduce(m, s_buf, true);
  float s = 0.f;
  constexpr float kLog2e = 1.4426950408889634f;
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) {
    const int v = threadIdx.x + i * kCeThreads;
    if (v < nvec) {
      const uint32_t* w = reinterpret_cast<const uint32_t*>(&regs[i]);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = unpack2<T>(w[k]);
        s += exp2f((f.x - m) * kLog2e) + exp2f((f.y - m) * kLog2e);
      }
    }
  }
  s = block_reduce(s, s_buf, false);
  const float lse = m + logf(s);
  if (threadIdx.x == 0) loss_rows[row] = valid ? lse - x_t : 0.f;
  const float gs = valid ? grad_scale : 0.f;  // ignored rows contribute no gradient
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) {
    const int v = threadIdx.x + i * kCeThreads;
    if (v < nvec) {
      uint32_t* w = reinterpret_cast<uint32_t*>(&regs[i]);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = unpack2<T>(w[k]);
        const int col = v * 8 + 2 * k;
        float g0 = exp2f((f.x - lse) * kLog2e) * gs, g1 = exp2f((f.y - lse) * kLog2e) * gs;
        if (col == tgt) g0 -= gs;
        if (col + 1 == tgt) g1 -= gs;
        w[k] = pack2<T>(g0, g1);
      }
      reinterpret_cast<uint4*>(x)[v] = regs[i];
    }
  }
}

}  // namespace

// logits: 16-bit [R, V] with row stride ld (elements), overwritten with the scaled gradient;
// targets: int64 [R] (out-of-range = ignored row); loss_rows: fp32 [R].
extern "C" int nnb_ce_inplace(void* logits, const void* targets, void* loss_rows, long long R, int V, long long ld,
                              float grad_scale, int dtype, cudaStream_t st) {
  NNB_REQUIRE(V % 8 == 0 && V <= kCeThreads * kMaxVec * 8, "ce: V=%d must be a multiple of 8 and <= %d", V, kCeThreads * kMaxVec * 8);
  NNB_REQUIRE(ld % 8 == 0 && nnb_aligned16(logits), "ce: logits rows must be 16-byte aligned");
  if (R == 0) return 0;
  NNB_DISPATCH_16(dtype, T, {
    ce_inplace_kernel<T><<<(unsigned)R, kCeThreads, 0, st>>>((T*)logits, (const long long*)targets, (float*)loss_rows, V, ld, grad_scale);
  });
  NNB_LAUNCH_OK("ce_inplace");
  return 0;
}
