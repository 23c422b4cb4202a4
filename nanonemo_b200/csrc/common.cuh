// Shared host/device helpers for the sm_100a kernel library: error reporting for the extern "C"
// launchers, dtype codes, 16-byte vector load/store helpers and warp reductions.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

// ---- host-side error channel: launchers return 0 or a negative code and leave a message here
extern "C" const char* nnb_last_error();
void nnb_set_error(const char* fmt, ...);

#define NNB_REQUIRE(cond, ...)           \
  do {                                   \
    if (!(cond)) {                       \
      nnb_set_error(__VA_ARGS__);        \
      return -1;                         \
    }                                    \
  } while (0)

#define NNB_LAUNCH_OK(name)                                                      \
  do {                                                                           \
    cudaError_t e_ = cudaGetLastError();                                         \
    if (e_ != cudaSuccess) {                                                     \
      nnb_set_error("%s: launch failed: %s", name, cudaGetErrorString(e_));      \
      return -100;                                                               \
    }                                                                            \
  } while (0)

enum NnbDtype : int { NNB_F32 = 0, NNB_BF16 = 1, NNB_F16 = 2 };

static inline int nnb_num_sms() {
  static int sms = 0;
  if (!sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
  }
  return sms;
}

static inline bool nnb_aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

#ifdef __CUDACC__
// ---- 8-element (one "chunk") loads/stores converting to/from fp32 registers
template <typename T>
struct Chunk8;

template <>
struct Chunk8<float> {
  static __device__ __forceinline__ void load(const float* p, float (&v)[8]) {
    float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&v)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
  }
};

template <>
struct Chunk8<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
    uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 f = __bfloat1622float2(h[i]);
      v[2 * i] = f.x; v[2 * i + 1] = f.y;
    }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[8]) {
    uint4 raw;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = raw;
  }
};

template <>
struct Chunk8<__half> {
  static __device__ __forceinline__ void load(const __half* p, float (&v)[8]) {
    uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 f = __half22float2(h[i]);
      v[2 * i] = f.x; v[2 * i + 1] = f.y;
    }
  }
  static __device__ __forceinline__ void store(__half* p, const float (&v)[8]) {
    uint4 raw;
    __half2* h = reinterpret_cast<__half2*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = raw;
  }
};

template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <> __device__ __forceinline__ __half from_f32<__half>(float x) { return __float2half_rn(x); }
__device__ __forceinline__ float to_f32(float x) { return x; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 x) { return __bfloat162float(x); }
__device__ __forceinline__ float to_f32(__half x) { return __half2float(x); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Dispatch a dtype code to a type tag: NNB_DISPATCH(code, T, { body using T })
#define NNB_DISPATCH(code, T, ...)                                  \
  switch (code) {                                                   \
    case NNB_F32: { using T = float; __VA_ARGS__; break; }          \
    case NNB_BF16: { using T = __nv_bfloat16; __VA_ARGS__; break; } \
    case NNB_F16: { using T = __half; __VA_ARGS__; break; }         \
    default: nnb_set_error("unknown dtype code %d", code); return -2; \
  }
#define NNB_DISPATCH_16(code, T, ...)                               \
  switch (code) {                                                   \
    case NNB_BF16: { using T = __nv_bfloat16; __VA_ARGS__; break; } \
    case NNB_F16: { using T = __half; __VA_ARGS__; break; }         \
    default: nnb_set_error("expected a 16-bit float dtype, got code %d", code); return -2; \
  }
#endif
