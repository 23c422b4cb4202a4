// Host entry of the CTA-pair GEMM (gemm2.cu); called by the dispatcher in gemm.cu.
#pragma once
#include <cuda_runtime.h>

// Work fused into the epilogue while a tile leaves tensor memory (see gemm2.cu).
enum NnbGemm2Epilogue : int { EPI_NONE = 0, EPI_SWIGLU = 1, EPI_ROPE = 2, EPI_CE_STATS = 3, EPI_SWIGLU_BWD = 4 };

struct NnbGemm2Args {
  const void *A, *B;
  void* D;
  int M, N, K;
  long long lda, ldb, ldd;  // row strides in elements of the stored matrices
  int a_mn, b_mn;           // operand majors (0 = K-major, 1 = MN-major)
  int dtype;                // NNB_BF16 / NNB_F16
  int out_f32, accumulate, k_splits, max_ctas;
  void* status;             // device int[4] or null
  int epilogue = EPI_NONE;
  // EPI_SWIGLU: B = gate||up weight [2 F, K] (N = 2 F), D = projection [M, 2 F], E = act [M, F] with row stride lde
  void* E = nullptr;
  long long lde = 0;
  // EPI_ROPE: rotate-half on columns [0, rope_cols) in heads of head_dim columns; row m uses table row m % t_len of the
  // fp32 tables [t_len, head_dim / 2]
  const void *cos_t = nullptr, *sin_t = nullptr;
  int t_len = 0, rope_cols = 0, head_dim = 0;
  // EPI_SWIGLU_BWD: the product [M, N = F] is the gradient of act = silu(gate) * up; E = the saved projection gate||up
  // [M, 2 F] (row stride lde), D = its gradient [M, 2 F] (row stride ldd); the product itself is never stored
  // EPI_CE_STATS: fp32 [M, 2 ceil(N / 256), 2] receiving (max, sum of exp(x - max)) of every row's logits in two parts per
  // 256-column tile (the tile's even and odd 64-column chunks); a part without columns holds (-inf, 0)
  void* stats = nullptr;
};

// Returns 0 on success, 1 when the shape is not served by the pair kernel (caller falls back), < 0 on error.
int nnb_gemm2_launch(const NnbGemm2Args& a, cudaStream_t st);
