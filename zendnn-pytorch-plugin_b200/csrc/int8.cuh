// Internal interface between the dispatcher (api.cu) and the int8 kernels.
#pragma once

#include "common.cuh"

namespace zt {

// One int8 GEMM with (optionally) the dynamic-qlinear epilogue.
struct Int8GemmArgs {
  const void *q;           // [M,K] s8 or u8, row-major
  bool q_is_u8;
  const int8_t *w;         // [N,K] s8, row-major
  int64_t M, N, K;
  bool raw_s32;            // true: y is int32 [M,N] = the accumulators, no epilogue
  const float *src_scale;  // [M]
  const int32_t *src_zp;   // [M] or null
  const void *w_scale;     // [N]
  int w_scale_dtype;
  const int32_t *w_rowsum; // [N] or null
  const void *bias;        // [N] or null
  int bias_dtype;
  int y_dtype;
  void *y;
  PostOpsDev post;
  int force_bn;            // 0 = choose
};

bool int8_tcgen05_supported(int64_t M, int64_t N, int64_t K, const void *q, const void *w);
int int8_tcgen05_launch(const Int8GemmArgs &a, cudaStream_t st);
int int8_generic_launch(const Int8GemmArgs &a, cudaStream_t st);

int dynamic_quantize_launch(const void *x, int x_dtype, int64_t M, int64_t K, int act_quant, void *q, float *scales,
                            int32_t *zps, cudaStream_t st);

}  // namespace zt
