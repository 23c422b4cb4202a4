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

// Tile quantiser for the tensor-core path. A block owns a 128 x 128 tile of x [R, C] (bf16) held in shared memory and writes
//   ROW: q  [R, C] e4m3, blocks of 32 along C, scales chunked for a GEMM that contracts over C;
//   COL: qt [C, R] e4m3 (the transpose), blocks of 32 along R, scales chunked for a GEMM that contracts over R
// from ONE read of x. Scale layout ("chunked"): for a matrix of `rows` x `k`, chunk [row / 128][k / 128] of 512 bytes, the four
// scales of (row, 128-wide k chunk) form one 32-bit word at byte (row % 32) * 16 + ((row % 128) / 32) * 4 — the order in which
// tcgen05.cp (32x128b, warpx4) expects to find them in shared memory.
constexpr int kTile = 128, kTilePad = 8;

__device__ __forceinline__ uint32_t quant4(const float* v, float inv) {
  const uint16_t lo = __nv_cvt_float2_to_fp8x2(make_float2(v[0] * inv, v[1] * inv), __NV_SATFINITE, __NV_E4M3);
  const uint16_t hi = __nv_cvt_float2_to_fp8x2(make_float2(v[2] * inv, v[3] * inv), __NV_SATFINITE, __NV_E4M3);
  return (uint32_t)lo | ((uint32_t)hi << 16);
}

template <bool ROW, bool COL>
__global__ void __launch_bounds__(256) mxfp8_tile_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, uint8_t* __restrict__ q,
                                                         long long ldq, uint8_t* __restrict__ sf, uint8_t* __restrict__ qt,
                                                         long long ldqt, uint8_t* __restrict__ sft, int R, int C) {
  __shared__ __align__(16) __nv_bfloat16 tile[kTile][kTile + kTilePad];
  const int c0 = blockIdx.x * kTile, r0 = blockIdx.y * kTile;
  for (int i = threadIdx.x; i < kTile * (kTile / 8); i += 256) {
    const int r = i >> 4, cc = (i & 15) * 8;
    *reinterpret_cast<uint4*>(&tile[r][cc]) = *reinterpret_cast<const uint4*>(x + (long long)(r0 + r) * ldx + c0 + cc);
  }
  __syncthreads();
  const int t = threadIdx.x & 127;
  const bool do_row = ROW && (!COL || threadIdx.x < 128), do_col = COL && (!ROW || threadIdx.x >= 128);
  if (do_row) {
    // row r0 + t: four blocks of 32 columns
    uint32_t sfw = 0;
    uint8_t* out = q + (long long)(r0 + t) * ldq + c0;
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      float v[32];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint4 raw = *reinterpret_cast<const uint4*>(&tile[t][b * 32 + j * 8]);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __bfloat1622float2(h[e]);
          v[j * 8 + 2 * e] = f.x; v[j * 8 + 2 * e + 1] = f.y;
        }
      }
      float amax = 0.f;
#pragma unroll
      for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(v[i]));
      uint8_t sb;
      float scale = block_scale_e8m0(amax, &sb);
      if (scale == 0.f) scale = __int_as_float(1 << 23);
      const float inv = 1.f / scale;
      sfw |= (uint32_t)sb << (8 * b);
#pragma unroll
      for (int j = 0; j < 2; ++j)
        *reinterpret_cast<uint4*>(out + b * 32 + j * 16) = make_uint4(quant4(v + j * 16, inv), quant4(v + j * 16 + 4, inv),
                                                                       quant4(v + j * 16 + 8, inv), quant4(v + j * 16 + 12, inv));
    }
    const long long chunk = (long long)blockIdx.y * (C / kTile) + blockIdx.x;
    *reinterpret_cast<uint32_t*>(sf + chunk * 512 + (t & 31) * 16 + (t >> 5) * 4) = sfw;
  }
  if (do_col) {
    // column c0 + t = row c0 + t of the transpose: four blocks of 32 rows
    uint32_t sfw = 0;
    uint8_t* out = qt + (long long)(c0 + t) * ldqt + r0;
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      float v[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = __bfloat162float(tile[b * 32 + i][t]);
      float amax = 0.f;
#pragma unroll
      for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(v[i]));
      uint8_t sb;
      float scale = block_scale_e8m0(amax, &sb);
      if (scale == 0.f) scale = __int_as_float(1 << 23);
      const float inv = 1.f / scale;
      sfw |= (uint32_t)sb << (8 * b);
#pragma unroll
      for (int j = 0; j < 2; ++j)
        *reinterpret_cast<uint4*>(out + b * 32 + j * 16) = make_uint4(quant4(v + j * 16, inv), quant4(v + j * 16 + 4, inv),
                                                                       quant4(v + j * 16 + 8, inv), quant4(v + j * 16 + 12, inv));
    }
    const long long chunk = (long long)blockIdx.x * (R / kTile) + blockIdx.y;
    *reinterpret_cast<uint32_t*>(sft + chunk * 512 + (t & 31) * 16 + (t >> 5) * 4) = sfw;
  }
}

}  // namespace

// x [R, C] bf16 (row stride ldx elements) -> any of
//   q [R, C] e4m3 (row stride ldq bytes) + sf (chunked scales, R / 128 x C / 128 chunks of 512 bytes), blocks along C;
//   qt [C, R] e4m3 (row stride ldqt bytes) + sft (C / 128 x R / 128 chunks), blocks along R.
// Pass null for the pair that is not wanted. R and C must be multiples of 128.
extern "C" int nnb_mxfp8_quantize_sw(const void* x, long long ldx, void* q, long long ldq, void* sf, void* qt, long long ldqt,
                                     void* sft, int R, int C, cudaStream_t st) {
  NNB_REQUIRE(R > 0 && C > 0 && R % 128 == 0 && C % 128 == 0, "mxfp8_quantize_sw: R=%d and C=%d must be positive multiples of 128", R, C);
  NNB_REQUIRE(ldx % 8 == 0 && nnb_aligned16(x), "mxfp8_quantize_sw: x must be 16-byte aligned with a row stride that is a multiple of 8");
  const bool row = q != nullptr, col = qt != nullptr;
  NNB_REQUIRE(row || col, "mxfp8_quantize_sw: nothing to do");
  NNB_REQUIRE(!row || (sf != nullptr && ldq % 16 == 0 && nnb_aligned16(q)), "mxfp8_quantize_sw: bad row-wise output");
  NNB_REQUIRE(!col || (sft != nullptr && ldqt % 16 == 0 && nnb_aligned16(qt)), "mxfp8_quantize_sw: bad transposed output");
  const dim3 grid(C / 128, R / 128);
#define NNB_MX_LAUNCH(ROW, COL) mxfp8_tile_kernel<ROW, COL><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, ldx, (uint8_t*)q, ldq, \
    (uint8_t*)sf, (uint8_t*)qt, ldqt, (uint8_t*)sft, R, C)
  if (row && col) NNB_MX_LAUNCH(true, true);
  else if (row) NNB_MX_LAUNCH(true, false);
  else NNB_MX_LAUNCH(false, true);
#undef NNB_MX_LAUNCH
  NNB_LAUNCH_OK("mxfp8_quantize_sw");
  return 0;
}

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
