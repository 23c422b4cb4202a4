// MXFP8 (OCP microscaling: 1 x 32 blocks along the contraction dimension, e4m3 elements, e8m0 scales)
// quantisation kernels.
//   nnb_mxfp8_quantize     x [M, K] (bf16)  ->  q [M, K] (e4m3 bytes) + scales [M, K/32] (e8m0 bytes)
//   nnb_mxfp8_fake_quant   x -> dequant(quant(x)) in bf16: the exact values an MXFP8 GEMM would multiply
// One warp per 32-element block row segment group: a lane owns 8 consecutive elements, four lanes share a
// block; amax by shuffles; scale = 2^(floor(log2(amax)) - 8) so the block maximum lands in [256, 448],
// the top binade of e4m3 (max 448). This is the quantiser the reference delegates to Transformer
// Engine's recipes (nanonemo/te/__init__.py:28-39, per-tensor scaling there; block scaling here).
#include <cuda_fp8.h>

#include "common.cuh"

namespace {

__device__ __forceinline__ float block_scale_e8m0(float amax, uint8_t* biased) {
  // e8m0: value 2^(b - 127); pick b so that amax / 2^(b-127) <= 448 with the exponent of amax mapped to 8
  int e = amax > 0.f ? ((__float_as_int(amax) >> 23) & 0xff) - 127 : -127;  // floor(log2(amax)) for normals
  int b = e - 8 + 127;
  b = b < 0 ? 0 : (b > 254 ? 254 : b);
  *biased = (uint8_t)b;
  return __int_as_float(b << 23);  // 2^(b-127) (b = 0 gives 0 -> treated as the smallest scale below)
}

template <bool kFake>
__global__ void mxfp8_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q, uint8_t* __restrict__ scales,
                             __nv_bfloat16* __restrict__ y, long long M, int K, long long ldx, long long ldo) {
  const int vec_per_row = K >> 3;
  const long long total = M * vec_per_row;
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const bool live = idx < total;
  const long long m = live ? idx / vec_per_row : 0;
  const int j = live ? (int)(idx - m * vec_per_row) * 8 : 0;
  float v[8];
  if (live) Chunk8<__nv_bfloat16>::load(x + m * ldx + j, v);
  else {
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = 0.f;
  }
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));  // 4 lanes x 8 elements = one 32-element block
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  uint8_t sb;
  float scale = block_scale_e8m0(amax, &sb);
  if (scale == 0.f) scale = __int_as_float(1 << 23);
  const float inv = 1.f / scale;
  if (!live) return;
  uint8_t bytes[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) bytes[i] = (uint8_t)__nv_cvt_float_to_fp8(v[i] * inv, __NV_SATFINITE, __NV_E4M3);
  if (kFake) {
    float o[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const __half_raw h = __nv_cvt_fp8_to_halfraw(bytes[i], __NV_E4M3);
      o[i] = __half2float(*reinterpret_cast<const __half*>(&h)) * scale;
    }
    Chunk8<__nv_bfloat16>::store(y + m * ldo + j, o);
  } else {
    *reinterpret_cast<uint2*>(q + m * ldo + j) = *reinterpret_cast<uint2*>(bytes);
    if ((j & 31) == 0) scales[m * (K >> 5) + (j >> 5)] = sb;
  }
}

}  // namespace

extern "C" int nnb_mxfp8_fake_quant(const void* x, void* y, long long M, int K, long long ldx, long long ldy, cudaStream_t st) {
  NNB_REQUIRE(K % 32 == 0 && ldx % 8 == 0 && ldy % 8 == 0, "mxfp8: K=%d must be a multiple of 32 and strides multiples of 8", K);
  if (M == 0) return 0;
  const long long total = M * (K / 8);
  mxfp8_kernel<true><<<(unsigned)((total + 255) / 256), 256, 0, st>>>((const __nv_bfloat16*)x, nullptr, nullptr, (__nv_bfloat16*)y, M, K, ldx, ldy);
  NNB_LAUNCH_OK("mxfp8_fake_quant");
  return 0;
}

extern "C" int nnb_mxfp8_quantize(const void* x, void* q, void* scales, long long M, int K, long long ldx, long long ldq, cudaStream_t st) {
  NNB_REQUIRE(K % 32 == 0 && ldx % 8 == 0 && ldq % 8 == 0, "mxfp8: K=%d must be a multiple of 32 and strides multiples of 8", K);
  if (M == 0) return 0;
  const long long total = M * (K / 8);
  mxfp8_kernel<false><<<(unsigned)((total + 255) / 256), 256, 0, st>>>((const __nv_bfloat16*)x, (uint8_t*)q, (uint8_t*)scales, nullptr, M, K, ldx, ldq);
  NNB_LAUNCH_OK("mxfp8_quantize");
  return 0;
}
