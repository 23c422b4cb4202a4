// Host entry of the CTA-pair GEMM (gemm2.cu); called by the dispatcher in gemm.cu.
#pragma once
#include <cuda_runtime.h>

struct NnbGemm2Args {
  const void *A, *B;
  void* D;
  int M, N, K;
  long long lda, ldb, ldd;  // row strides in elements of the stored matrices
  int a_mn, b_mn;           // operand majors (0 = K-major, 1 = MN-major)
  int dtype;                // NNB_BF16 / NNB_F16
  int out_f32, accumulate, k_splits, max_ctas;
  void* status;             // device int[4] or null
};

// Returns 0 on success, 1 when the shape is not served by the pair kernel (caller falls back), < 0 on error.
int nnb_gemm2_launch(const NnbGemm2Args& a, cudaStream_t st);
