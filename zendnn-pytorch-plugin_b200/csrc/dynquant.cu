// Per-token dynamic quantisation of activations: the first phase of zentorch_dynamic_qlinear.
//
// One CTA per row.  The row is read once into registers (up to 32 values per thread; longer rows
// re-read the tail, which then comes from L2), reduced to its absolute maximum (s8) or min/max (u8)
// with warp shuffles, and written back as 8-bit values with 8-byte stores.  The scale uses IEEE
// division and the quantised value round-half-even, so the bytes equal those of the CPU formula
//   s = max(absmax, 1e-12) / 127,   q = clamp(rint(x / s), -128, 127).
// A NaN anywhere in a row makes that row's scale NaN (as a maximum that propagates NaNs does, which is what
// the CPU formula's amax is), so the whole output row of the linear is NaN; the row's quantised bytes are
// then unspecified.  Other rows are not affected.  -0.0 counts as 0.
#include "int8.cuh"

namespace zt {

namespace {

constexpr int kThreads = 256;
constexpr int kVec = 8;        // elements per thread per chunk
constexpr int kCached = 4;     // chunks kept in registers

__device__ __forceinline__ void load8(const void *x, int dtype, int64_t off, float (&v)[8]) {
  if (dtype == ZT_BF16) {
    const uint4 raw = *reinterpret_cast<const uint4 *>(reinterpret_cast<const __nv_bfloat16 *>(x) + off);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  } else {
    const float4 a = *reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(x) + off);
    const float4 b = *reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(x) + off + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
}

// Row maximum of hi and row minimum of lo over the CTA in one pass: warp shuffles, one shared-memory slot per
// warp and value, one barrier, and every thread folds the eight warp results itself (max and min are exact, so
// the order does not matter).
// fmaxf / fminf return the other operand when one is NaN; these keep it.
__device__ __forceinline__ float nan_max(float a, float b) { return (a != a) ? a : (b != b) ? b : fmaxf(a, b); }
__device__ __forceinline__ float nan_min(float a, float b) { return (a != a) ? a : (b != b) ? b : fminf(a, b); }

__device__ __forceinline__ void block_reduce_max_min(float &hi, float &lo, bool saw_nan, float *scratch) {
  if (saw_nan) hi = lo = __int_as_float(0x7fc00000);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    hi = nan_max(hi, __shfl_xor_sync(0xffffffffu, hi, o));
    lo = nan_min(lo, __shfl_xor_sync(0xffffffffu, lo, o));
  }
  constexpr int kWarps = kThreads / 32;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) {
    scratch[warp] = hi;
    scratch[kWarps + warp] = lo;
  }
  __syncthreads();
#pragma unroll
  for (int w = 0; w < kWarps; ++w) {
    hi = nan_max(hi, scratch[w]);
    lo = nan_min(lo, scratch[kWarps + w]);
  }
}

// Row scale (and zero point) from the reduced extremes; NaN extremes give a NaN scale.
template <bool U8>
__device__ __forceinline__ void row_scale(float hi, float lo, float &s, float &zp) {
  zp = 0.f;
  if (U8) {
    const float range = hi - lo;
    s = (range != range) ? range : __fdiv_rn(fmaxf(range, 1e-12f), 255.0f);
    zp = fminf(fmaxf(rintf(__fdiv_rn(-lo, s)), 0.f), 255.f);
  } else {
    s = (hi != hi) ? hi : __fdiv_rn(fmaxf(hi, 1e-12f), 127.0f);
  }
}

template <bool U8>
__device__ __forceinline__ uint32_t quant_one(float x, float s, float zp) {
  const float r = rintf(__fdiv_rn(x, s));
  if (U8) {
    const float v = fminf(fmaxf(r + zp, 0.f), 255.f);
    return (uint32_t)(int)v;
  }
  const float v = fminf(fmaxf(r, -128.f), 127.f);
  return (uint32_t)((int)v) & 0xffu;
}

// Vector path: K % 8 == 0 and 16-byte aligned rows.
template <bool U8>
__global__ void __launch_bounds__(kThreads) dynquant_vec_kernel(const void *__restrict__ x, int x_dtype, int64_t K,
                                                                uint8_t *__restrict__ q, float *__restrict__ scales,
                                                                int32_t *__restrict__ zps) {
  __shared__ float scratch[16];
  // programmatic dependent launch: let the GEMM that follows start its prologue and weight prefetch now;
  // wait for the kernel before this one (it may still read the buffers written here) before any access
  grid_launch_dependents();
  grid_dependency_wait();
  const int64_t row = blockIdx.x;
  const int64_t base = row * K;
  const int64_t chunks = K / kVec;
  float v[kCached][8];
  float hi = 0.f, lo = 0.f;  // u8: max(x,0), min(x,0); s8: hi = absmax
  bool saw_nan = false;
#pragma unroll
  for (int c = 0; c < kCached; ++c) {
    const int64_t ch = (int64_t)c * kThreads + threadIdx.x;
    if (ch < chunks) {
      load8(x, x_dtype, base + ch * kVec, v[c]);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        saw_nan |= (v[c][i] != v[c][i]);
        if (U8) {
          hi = fmaxf(hi, v[c][i]);
          lo = fminf(lo, v[c][i]);
        } else {
          hi = fmaxf(hi, fabsf(v[c][i]));
        }
      }
    }
  }
  for (int64_t ch = (int64_t)kCached * kThreads + threadIdx.x; ch < chunks; ch += kThreads) {
    float t[8];
    load8(x, x_dtype, base + ch * kVec, t);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      saw_nan |= (t[i] != t[i]);
      if (U8) {
        hi = fmaxf(hi, t[i]);
        lo = fminf(lo, t[i]);
      } else {
        hi = fmaxf(hi, fabsf(t[i]));
      }
    }
  }
  block_reduce_max_min(hi, lo, saw_nan, scratch);
  float s, zp;
  row_scale<U8>(hi, lo, s, zp);
  if (threadIdx.x == 0) {
    scales[row] = s;
    if (U8 && zps) zps[row] = (int32_t)zp;
  }
  auto emit = [&](const float(&t)[8], int64_t ch) {
    uint32_t w0 = 0, w1 = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      w0 |= quant_one<U8>(t[i], s, zp) << (8 * i);
      w1 |= quant_one<U8>(t[4 + i], s, zp) << (8 * i);
    }
    *reinterpret_cast<uint2 *>(q + base + ch * kVec) = make_uint2(w0, w1);
  };
#pragma unroll
  for (int c = 0; c < kCached; ++c) {
    const int64_t ch = (int64_t)c * kThreads + threadIdx.x;
    if (ch < chunks) emit(v[c], ch);
  }
  for (int64_t ch = (int64_t)kCached * kThreads + threadIdx.x; ch < chunks; ch += kThreads) {
    float t[8];
    load8(x, x_dtype, base + ch * kVec, t);
    emit(t, ch);
  }
}

// Any K, any alignment.
template <bool U8>
__global__ void __launch_bounds__(kThreads) dynquant_scalar_kernel(const void *__restrict__ x, int x_dtype, int64_t K,
                                                                   uint8_t *__restrict__ q, float *__restrict__ scales,
                                                                   int32_t *__restrict__ zps) {
  __shared__ float scratch[16];
  grid_launch_dependents();
  grid_dependency_wait();
  const int64_t row = blockIdx.x;
  const int64_t base = row * K;
  float hi = 0.f, lo = 0.f;
  bool saw_nan = false;
  for (int64_t k = threadIdx.x; k < K; k += kThreads) {
    const float t = load_as_float(x, base + k, x_dtype);
    saw_nan |= (t != t);
    if (U8) {
      hi = fmaxf(hi, t);
      lo = fminf(lo, t);
    } else {
      hi = fmaxf(hi, fabsf(t));
    }
  }
  block_reduce_max_min(hi, lo, saw_nan, scratch);
  float s, zp;
  row_scale<U8>(hi, lo, s, zp);
  if (threadIdx.x == 0) {
    scales[row] = s;
    if (U8 && zps) zps[row] = (int32_t)zp;
  }
  for (int64_t k = threadIdx.x; k < K; k += kThreads)
    q[base + k] = (uint8_t)quant_one<U8>(load_as_float(x, base + k, x_dtype), s, zp);
}

// Per-tensor quantisation with the caller's scale and zero point (the static form):
// q = clamp(rint(x * (1 / s)) + zp).  Element-wise over the flattened tensor, eight elements per thread where
// the alignment allows.
template <bool U8>
__device__ __forceinline__ uint32_t static_quant_one(float x, float inv, float zp) {
  const float r = rintf(__fmul_rn(x, inv)) + zp;
  if (U8) return (uint32_t)(int)fminf(fmaxf(r, 0.f), 255.f);
  return (uint32_t)((int)fminf(fmaxf(r, -128.f), 127.f)) & 0xffu;
}

template <bool U8>
__global__ void __launch_bounds__(kThreads) static_quant_kernel(const void *__restrict__ x, int x_dtype, int64_t numel,
                                                                const float *__restrict__ scale,
                                                                const int32_t *__restrict__ zero_point,
                                                                uint8_t *__restrict__ q, bool vec) {
  grid_launch_dependents();
  grid_dependency_wait();
  const float inv = 1.0f / *scale;                       // IEEE division
  const float zp = U8 ? (float)*zero_point : 0.f;
  const int64_t stride = (int64_t)gridDim.x * kThreads;
  if (vec) {
    for (int64_t ch = (int64_t)blockIdx.x * kThreads + threadIdx.x; ch < numel / kVec; ch += stride) {
      float t[8];
      load8(x, x_dtype, ch * kVec, t);
      uint32_t w0 = 0, w1 = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        w0 |= static_quant_one<U8>(t[i], inv, zp) << (8 * i);
        w1 |= static_quant_one<U8>(t[4 + i], inv, zp) << (8 * i);
      }
      *reinterpret_cast<uint2 *>(q + ch * kVec) = make_uint2(w0, w1);
    }
    for (int64_t i = numel / kVec * kVec + (int64_t)blockIdx.x * kThreads + threadIdx.x; i < numel; i += stride)
      q[i] = (uint8_t)static_quant_one<U8>(load_as_float(x, i, x_dtype), inv, zp);
  } else {
    for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < numel; i += stride)
      q[i] = (uint8_t)static_quant_one<U8>(load_as_float(x, i, x_dtype), inv, zp);
  }
}

}  // namespace

int static_quantize_launch(const void *x, int x_dtype, int64_t numel, const float *scale, const int32_t *zero_point,
                           void *q, cudaStream_t st) {
  if (numel == 0) return ZT_SUCCESS;
  const bool vec = ((reinterpret_cast<uintptr_t>(x) & 15) == 0) && ((reinterpret_cast<uintptr_t>(q) & 7) == 0);
  const int64_t work = vec ? (numel + kVec - 1) / kVec : numel;
  int64_t blocks = (work + kThreads - 1) / kThreads;
  const int64_t cap = (int64_t)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  uint8_t *qq = reinterpret_cast<uint8_t *>(q);
  if (zero_point)
    ZT_CUDA_OK(launch_overlapped(static_quant_kernel<true>, dim3((unsigned)blocks), dim3(kThreads), (size_t)0, st, x,
                                 x_dtype, numel, scale, zero_point, qq, vec));
  else
    ZT_CUDA_OK(launch_overlapped(static_quant_kernel<false>, dim3((unsigned)blocks), dim3(kThreads), (size_t)0, st, x,
                                 x_dtype, numel, scale, zero_point, qq, vec));
  return launch_status("static_quant_kernel");
}

int dynamic_quantize_launch(const void *x, int x_dtype, int64_t M, int64_t K, int act_quant, void *q, float *scales,
                            int32_t *zps, cudaStream_t st) {
  if (M == 0 || K == 0) return ZT_SUCCESS;
  ZT_REQUIRE(M <= 0x7fffffffLL, ZT_UNSUPPORTED, "zt_dynamic_quantize: M = %lld exceeds the grid limit", (long long)M);
  const bool u8 = act_quant == ZT_ACT_U8_ASYM;
  const size_t esz = x_dtype == ZT_BF16 ? 2 : 4;
  const bool vec = (K % kVec == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0) && ((K * esz) % 16 == 0) &&
                   ((reinterpret_cast<uintptr_t>(q) & 7) == 0);
  uint8_t *qq = reinterpret_cast<uint8_t *>(q);
  const dim3 grid((unsigned)M);
  if (vec) {
    if (u8)
      ZT_CUDA_OK(launch_overlapped(dynquant_vec_kernel<true>, dim3(grid), dim3(kThreads), (size_t)0, st, x, x_dtype, K, qq, scales, zps));
    else
      ZT_CUDA_OK(launch_overlapped(dynquant_vec_kernel<false>, dim3(grid), dim3(kThreads), (size_t)0, st, x, x_dtype, K, qq, scales, zps));
  } else {
    if (u8)
      ZT_CUDA_OK(launch_overlapped(dynquant_scalar_kernel<true>, dim3(grid), dim3(kThreads), (size_t)0, st, x, x_dtype, K, qq, scales, zps));
    else
      ZT_CUDA_OK(launch_overlapped(dynquant_scalar_kernel<false>, dim3(grid), dim3(kThreads), (size_t)0, st, x, x_dtype, K, qq, scales, zps));
  }
  return launch_status("dynquant_kernel");
}

}  // namespace zt
