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
  int64_t q_rows;          // rows addressable behind q when more than M (scratch padded by the caller), else 0
  // Static-quantisation form (zt_static_qlinear): src_scale / src_zp hold one element for the whole tensor,
  // w_scale is fp32 and may be one element, binary post-op operands have their own dtype, rows of y are ldy
  // elements apart, and with out_scale the result is requantised to y_dtype (ZT_U8 with out_zp, else ZT_S8).
  bool static_mode;
  bool w_scale_per_tensor;
  int post_dtype;
  const float *out_scale;  // one element or null
  const int32_t *out_zp;   // one element or null
  int64_t ldy;
};

// Output side of the static form, shared by the kernels: requantisation parameters read once per thread.
struct OutQuant {
  float inv_scale;   // 1 / s_o, 0 when the output stays floating point
  float zp, lo, hi;
};
__device__ __forceinline__ OutQuant load_out_quant(const float *out_scale, const int32_t *out_zp, int y_dtype) {
  OutQuant o{0.f, 0.f, 0.f, 0.f};
  if (out_scale) {
    o.inv_scale = 1.0f / *out_scale;                   // IEEE division, as the reference computes 1 / output_scales
    o.zp = out_zp ? (float)*out_zp : 0.f;
    o.lo = y_dtype == ZT_U8 ? 0.f : -128.f;
    o.hi = y_dtype == ZT_U8 ? 255.f : 127.f;
  }
  return o;
}
__device__ __forceinline__ int requantize(float v, const OutQuant &o) {
  return (int)fminf(fmaxf(rintf(v * o.inv_scale) + o.zp, o.lo), o.hi);
}
// one element of y in the static form
__device__ __forceinline__ void store_static(void *y, int64_t i, int y_dtype, float v, const OutQuant &o) {
  if (y_dtype == ZT_U8)
    reinterpret_cast<uint8_t *>(y)[i] = (uint8_t)requantize(v, o);
  else if (y_dtype == ZT_S8)
    reinterpret_cast<int8_t *>(y)[i] = (int8_t)requantize(v, o);
  else
    store_from_float(y, i, y_dtype, v);
}

// The quantised activations of a call with fewer rows live in scratch padded to this many rows.
constexpr int64_t kMinQRows = 16;

bool int8_tcgen05_supported(int64_t M, int64_t N, int64_t K, const void *q, const void *w);
int int8_tcgen05_launch(const Int8GemmArgs &a, cudaStream_t st);
int int8_generic_launch(const Int8GemmArgs &a, cudaStream_t st);

int static_quantize_launch(const void *x, int x_dtype, int64_t numel, const float *scale, const int32_t *zero_point,
                           void *q, cudaStream_t st);
int dynamic_quantize_launch(const void *x, int x_dtype, int64_t M, int64_t K, int act_quant, void *q, float *scales,
                            int32_t *zps, cudaStream_t st);

}  // namespace zt
