// Flat-buffer optimizer kernels: the squared gradient norm and the fused AdamW update.
//
// nnb_adamw_flat does, in ONE pass over memory: clip coefficient from the device-resident squared
// norm, decoupled weight decay (per 256-element block flag), both moment updates, the fp32 master
// update (the operations of torch.optim.AdamW in the same order; this file is compiled WITHOUT
// --use_fast_math, so the square root and the division are IEEE-rounded and denormal moments are
// kept), the 16-bit compute copy, and zeroing of the gradient for the next step. The reference does this with clip_grad_norm_ + foreach AdamW +
// zero_grad (nanonemo/train/trainer.py:183-193): about a dozen passes and ~10^3 small launches.
#include <cmath>

#include "common.cuh"

// ---------------------------------------------------------------- sum of squares
// Stage 1: every block writes a partial into `scratch`; the last block to finish (ticket counter at
// scratch[blocks]) adds the partials in index order, so the result does not depend on scheduling.
__global__ void __launch_bounds__(512) sumsq_kernel(const float* __restrict__ x, long long n, float* __restrict__ scratch,
                                                    float* __restrict__ out, int accumulate) {
  __shared__ float s_part[16];
  __shared__ bool s_last;
  float acc = 0.f;
  const long long n4 = n >> 2;
  const float4* x4 = reinterpret_cast<const float4*>(x);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    const float4 v = x4[i];
    acc += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  for (long long i = (n4 << 2) + blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    acc += x[i] * x[i];
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < (blockDim.x >> 5) ? s_part[threadIdx.x] : 0.f;
    v = warp_sum(v);
    if (threadIdx.x == 0) {
      scratch[blockIdx.x] = v;
      __threadfence();
      unsigned* counter = reinterpret_cast<unsigned*>(scratch + gridDim.x);
      s_last = atomicAdd(counter, 1u) == gridDim.x - 1;
    }
  }
  __syncthreads();
  if (s_last && threadIdx.x < 32) {
    __threadfence();
    float v = 0.f;
    for (int i = threadIdx.x; i < (int)gridDim.x; i += 32) v += reinterpret_cast<volatile float*>(scratch)[i];
    v = warp_sum(v);
    if (threadIdx.x == 0) {
      *out = accumulate ? *out + v : v;
      *reinterpret_cast<unsigned*>(scratch + gridDim.x) = 0u;  // ready for the next call
    }
  }
}

extern "C" int nnb_sumsq_blocks() { return 2 * nnb_num_sms(); }

// scratch: fp32 [nnb_sumsq_blocks() + 1], the last word (the ticket counter) zero on entry (the
// kernel leaves it zero). out: fp32 scalar.
extern "C" int nnb_sumsq_f32(const void* x, long long n, void* scratch, void* out, int accumulate, cudaStream_t st) {
  NNB_REQUIRE(nnb_aligned16(x), "sumsq: input must be 16-byte aligned");
  NNB_REQUIRE(scratch != nullptr && out != nullptr, "sumsq: null scratch/out");
  const int blocks = nnb_sumsq_blocks();
  sumsq_kernel<<<blocks, 512, 0, st>>>((const float*)x, n, (float*)scratch, (float*)out, accumulate);
  NNB_LAUNCH_OK("sumsq");
  return 0;
}

// ---------------------------------------------------------------- fused AdamW
template <typename TS>
__global__ void __launch_bounds__(256) adamw_flat_kernel(float* __restrict__ p, float* __restrict__ g, float* __restrict__ m,
                                                         float* __restrict__ v, TS* __restrict__ shadow,
                                                         const unsigned char* __restrict__ decay_flags, long long n4,
                                                         float lr, float beta1, float beta2, float eps, float wd,
                                                         float bc1, float bc2_sqrt, const float* __restrict__ norm_sq,
                                                         float max_norm, int zero_grad) {
  float coef = 1.f;
  if (norm_sq != nullptr) {
    const float norm = sqrtf(*norm_sq);
    coef = fminf(1.f, max_norm / (norm + 1e-6f));
  }
  const float step_size = lr / bc1;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    float4 pp = reinterpret_cast<float4*>(p)[i], gg = reinterpret_cast<float4*>(g)[i];
    float4 mm = reinterpret_cast<float4*>(m)[i], vv = reinterpret_cast<float4*>(v)[i];
    const float decay = decay_flags[i >> 6] ? 1.f - lr * wd : 1.f;  // 64 float4 = one 256-element block
    float* P = &pp.x; float* G = &gg.x; float* Mo = &mm.x; float* V = &vv.x;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float gk = G[k] * coef;
      P[k] *= decay;
      Mo[k] = Mo[k] + (gk - Mo[k]) * (1.f - beta1);
      V[k] = V[k] * beta2 + gk * gk * (1.f - beta2);
      const float denom = sqrtf(V[k]) / bc2_sqrt + eps;
      P[k] -= step_size * (Mo[k] / denom);
    }
    reinterpret_cast<float4*>(p)[i] = pp;
    reinterpret_cast<float4*>(m)[i] = mm;
    reinterpret_cast<float4*>(v)[i] = vv;
    if (zero_grad) reinterpret_cast<float4*>(g)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (shadow != nullptr) {
      TS* s = shadow + i * 4;
      s[0] = from_f32<TS>(pp.x); s[1] = from_f32<TS>(pp.y); s[2] = from_f32<TS>(pp.z); s[3] = from_f32<TS>(pp.w);
    }
  }
}

// p, g, m, v: fp32 [n]; shadow: 16-bit [n] or null; decay_flags: uint8 [n / 256]; norm_sq: device
// fp32 scalar or null (no clipping). n must be a multiple of 256.
extern "C" int nnb_adamw_flat(void* p, void* g, void* m, void* v, void* shadow, const void* decay_flags, long long n,
                              float lr, float beta1, float beta2, float eps, float wd, int step, const void* norm_sq,
                              float max_norm, int zero_grad, int shadow_dtype, cudaStream_t st) {
  NNB_REQUIRE(n % 256 == 0, "adamw_flat: n=%lld must be a multiple of 256", n);
  NNB_REQUIRE(step >= 1, "adamw_flat: step must be >= 1");
  if (n == 0) return 0;
  // bias corrections in double on the host, as torch.optim.AdamW computes them (python floats)
  const float bc1 = (float)(1.0 - pow((double)beta1, (double)step));
  const float bc2_sqrt = (float)sqrt(1.0 - pow((double)beta2, (double)step));
  const long long n4 = n / 4;
  const int blocks = (int)min((n4 + 255) / 256, (long long)nnb_num_sms() * 8);
  if (shadow == nullptr || shadow_dtype == NNB_BF16) {
    adamw_flat_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>((float*)p, (float*)g, (float*)m, (float*)v, (__nv_bfloat16*)shadow,
                                                             (const unsigned char*)decay_flags, n4, lr, beta1, beta2, eps, wd,
                                                             bc1, bc2_sqrt, (const float*)norm_sq, max_norm, zero_grad);
  } else if (shadow_dtype == NNB_F16) {
    adamw_flat_kernel<__half><<<blocks, 256, 0, st>>>((float*)p, (float*)g, (float*)m, (float*)v, (__half*)shadow,
                                                      (const unsigned char*)decay_flags, n4, lr, beta1, beta2, eps, wd, bc1,
                                                      bc2_sqrt, (const float*)norm_sq, max_norm, zero_grad);
  } else {
    nnb_set_error("adamw_flat: shadow dtype code %d unsupported", shadow_dtype);
    return -2;
  }
  NNB_LAUNCH_OK("adamw_flat");
  return 0;
}

// ---------------------------------------------------------------- sum of squares without allocation
#include "nnb_noalloc.h"

// Scratch for nnb_sumsq_f32_noalloc: block partials followed by the ticket word. In host code this
// name is only a handle for cudaGetSymbolAddress, never a device address to pass to a kernel.
static __device__ __align__(256) float g_sumsq_noalloc_scratch[NNB_SUMSQ_NOALLOC_MAX_BLOCKS + 1];

extern "C" int nnb_sumsq_f32_noalloc(const void* x, long long n, void* out, cudaStream_t st) {
  constexpr int kMaxDevices = 64;
  static float* scratch_of[kMaxDevices] = {nullptr};
  NNB_REQUIRE(out != nullptr && (x != nullptr || n == 0), "sumsq_noalloc: null pointer");  // an empty input may come without a buffer
  NNB_REQUIRE(nnb_aligned16(x), "sumsq_noalloc: input must be 16-byte aligned");
  NNB_REQUIRE(n >= 0 && n <= NNB_SUMSQ_NOALLOC_MAX_ELEMS, "sumsq_noalloc: n=%lld is outside [0, %lld]", n,
              (long long)NNB_SUMSQ_NOALLOC_MAX_ELEMS);
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  NNB_REQUIRE(e == cudaSuccess && dev >= 0 && dev < kMaxDevices, "sumsq_noalloc: cudaGetDevice failed or device %d >= %d", dev, kMaxDevices);
  if (scratch_of[dev] == nullptr) {  // once per device, with that device current
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_sumsq_noalloc_scratch);
    NNB_REQUIRE(e == cudaSuccess && p != nullptr, "sumsq_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
    scratch_of[dev] = p;
  }
  float* scratch = scratch_of[dev];
  const int blocks = min(nnb_sumsq_blocks(), NNB_SUMSQ_NOALLOC_MAX_BLOCKS);
  // the array keeps whatever the last call left: the ticket word must start at zero
  e = cudaMemsetAsync(scratch + blocks, 0, sizeof(unsigned), st);
  NNB_REQUIRE(e == cudaSuccess, "sumsq_noalloc: clearing the ticket word failed: %s", cudaGetErrorString(e));
  sumsq_kernel<<<blocks, 512, 0, st>>>(static_cast<const float*>(x), n, scratch, static_cast<float*>(out), 0);
  NNB_LAUNCH_OK("sumsq_noalloc");
  return 0;
}
