// int8 GEMM + dynamic-qlinear epilogue for shapes the tensor-core kernel does not take (K not a
// multiple of 16, unaligned pointers), and the weight row-sum used by the unsigned-activation mode.
//
// One warp owns one output column n; lanes split K (dp4a on whole words, scalar tail), partial sums
// are combined with warp shuffles.  Integer accumulation makes the result independent of the order.
#include "int8.cuh"

namespace zt {

namespace {

constexpr int kRowsPerPass = 4;

template <bool U8>
__device__ __forceinline__ int dot4(int q, int w, int acc) {
  int d;
  if (U8)
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(q), "r"(w), "r"(acc));
  else
    asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(q), "r"(w), "r"(acc));
  return d;
}

template <bool U8>
__global__ void __launch_bounds__(256) int8_generic_kernel(const Int8GemmArgs a) {
  const int lane = threadIdx.x & 31;
  const int64_t n = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (n >= a.N) return;
  const int8_t *wrow = a.w + n * a.K;
  const uint8_t *q = reinterpret_cast<const uint8_t *>(a.q);
  const bool words_ok = (a.K % 4 == 0) && ((reinterpret_cast<uintptr_t>(a.w) & 3) == 0) &&
                        ((reinterpret_cast<uintptr_t>(a.q) & 3) == 0);
  const int64_t kw = words_ok ? a.K / 4 : 0;

  for (int64_t m0 = (int64_t)blockIdx.y * kRowsPerPass; m0 < a.M; m0 += (int64_t)gridDim.y * kRowsPerPass) {
    int acc[kRowsPerPass];
#pragma unroll
    for (int r = 0; r < kRowsPerPass; ++r) acc[r] = 0;
    for (int64_t w = lane; w < kw; w += 32) {
      const int wv = reinterpret_cast<const int *>(wrow)[w];
#pragma unroll
      for (int r = 0; r < kRowsPerPass; ++r) {
        if (m0 + r < a.M) {
          const int qv = reinterpret_cast<const int *>(q + (m0 + r) * a.K)[w];
          acc[r] = dot4<U8>(qv, wv, acc[r]);
        }
      }
    }
    for (int64_t k = kw * 4 + lane; k < a.K; k += 32) {
      const int wv = wrow[k];
#pragma unroll
      for (int r = 0; r < kRowsPerPass; ++r) {
        if (m0 + r < a.M) {
          const int qv = U8 ? (int)q[(m0 + r) * a.K + k] : (int)reinterpret_cast<const int8_t *>(q)[(m0 + r) * a.K + k];
          acc[r] += qv * wv;
        }
      }
    }
#pragma unroll
    for (int r = 0; r < kRowsPerPass; ++r) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) acc[r] += __shfl_xor_sync(0xffffffffu, acc[r], o);
    }
    if (lane == 0) {
#pragma unroll
      for (int r = 0; r < kRowsPerPass; ++r) {
        const int64_t m = m0 + r;
        if (m >= a.M) continue;
        const int64_t idx = m * a.N + n;
        if (a.raw_s32) {
          reinterpret_cast<int32_t *>(a.y)[idx] = acc[r];
          continue;
        }
        const int64_t ms = a.static_mode ? 0 : m;     // per-tensor activation parameters in the static form
        float af;
        if (a.src_zp) {
          af = (float)((int64_t)acc[r] - (int64_t)a.src_zp[ms] * (a.w_rowsum ? a.w_rowsum[n] : 0));
        } else {
          af = (float)acc[r];
        }
        const float sw = a.src_scale[ms] * load_as_float(a.w_scale, a.w_scale_per_tensor ? 0 : n, a.w_scale_dtype);
        float v;
        if (a.static_mode) {
          // separately rounded product and sum (no fused multiply-add): a requantised output sits on rounding
          // boundaries of the float result
          v = __fmul_rn(af, sw);
          if (a.bias) v = __fadd_rn(v, load_as_float(a.bias, n, a.bias_dtype));
        } else {
          v = af * sw;
          if (a.bias) v += load_as_float(a.bias, n, a.bias_dtype);
        }
        if (a.static_mode) {
          v = apply_post_ops(v, a.post, idx, a.post_dtype);
          store_static(a.y, m * a.ldy + n, a.y_dtype, v, load_out_quant(a.out_scale, a.out_zp, a.y_dtype));
        } else {
          v = apply_post_ops(v, a.post, idx, a.y_dtype);
          store_from_float(a.y, idx, a.y_dtype, v);
        }
      }
    }
  }
}

__global__ void __launch_bounds__(256) int8_rowsum_kernel(const int8_t *__restrict__ w, int64_t N, int64_t K,
                                                          int32_t *__restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int64_t n = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (n >= N) return;
  int acc = 0;
  for (int64_t k = lane; k < K; k += 32) acc += w[n * K + k];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) out[n] = acc;
}

}  // namespace

int int8_generic_launch(const Int8GemmArgs &a, cudaStream_t st) {
  if (a.M == 0 || a.N == 0) return ZT_SUCCESS;
  const int warps = 8;
  const int64_t mblocks = ceil_div<int64_t>(a.M, kRowsPerPass);
  dim3 grid((unsigned)ceil_div<int64_t>(a.N, warps), (unsigned)(mblocks < 4096 ? mblocks : 4096));
  if (a.q_is_u8)
    int8_generic_kernel<true><<<grid, warps * 32, 0, st>>>(a);
  else
    int8_generic_kernel<false><<<grid, warps * 32, 0, st>>>(a);
  return launch_status("int8_generic_kernel");
}

}  // namespace zt

using namespace zt;

extern "C" int zt_int8_weight_rowsum(const int8_t *w, int64_t N, int64_t K, int32_t *rowsum, void *stream) {
  ZT_REQUIRE(w && rowsum, ZT_INVALID_ARGUMENT, "zt_int8_weight_rowsum: null pointer");
  ZT_REQUIRE(N >= 0 && K >= 0, ZT_INVALID_ARGUMENT, "zt_int8_weight_rowsum: negative size");
  if (N == 0) return ZT_SUCCESS;
  int8_rowsum_kernel<<<(unsigned)ceil_div<int64_t>(N, 8), 256, 0, (cudaStream_t)stream>>>(w, N, K, rowsum);
  return launch_status("int8_rowsum_kernel");
}
