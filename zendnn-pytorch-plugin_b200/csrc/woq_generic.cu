// Weight-only int4 linear for shapes the streaming and tensor-core kernels do not take (K not a
// multiple of 128, group sizes below 128, unaligned pointers), plus the two weight repack ops.
//
// One warp owns one output column n.  Lanes split the row's packed words; each nibble is
// dequantised in fp32 exactly as the reference's test oracle does, dq = bf16(q*s) or
// bf16((q-8)*s + z), multiplied with the activation in fp32 and reduced with warp shuffles.
#include "common.cuh"
#include "woq.cuh"

namespace zt {

namespace {

constexpr int kRowsPerPass = 4;

struct GenericParams {
  const __nv_bfloat16 *x;
  const int32_t *wq;
  const void *scales;
  const void *zeros;
  const void *bias;
  __nv_bfloat16 *y;
  int64_t M, N, K;
  int64_t gs;
  int scale_dtype, bias_dtype;
  PostOpsDev post;
};

__global__ void __launch_bounds__(256) woq_generic_kernel(const GenericParams p) {
  const int lane = threadIdx.x & 31;
  const int64_t n = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (n >= p.N) return;
  const int64_t k8 = p.K >> 3;
  const int32_t *row = p.wq + n * k8;
  const bool asym = p.zeros != nullptr;

  for (int64_t m0 = (int64_t)blockIdx.y * kRowsPerPass; m0 < p.M; m0 += (int64_t)gridDim.y * kRowsPerPass) {
    float acc[kRowsPerPass];
#pragma unroll
    for (int r = 0; r < kRowsPerPass; ++r) acc[r] = 0.f;
    for (int64_t w = lane; w < k8; w += 32) {
      const uint32_t word = (uint32_t)row[w];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int64_t k = w * 8 + i;
        const int64_t gi = (k / p.gs) * p.N + n;
        int q = (word >> (4 * i)) & 0xF;
        const float s = load_as_float(p.scales, gi, p.scale_dtype);
        float dq;
        if (asym) {
          dq = __fadd_rn(__fmul_rn((float)q - 8.f, s), load_as_float(p.zeros, gi, p.scale_dtype));
        } else {
          if (q >= 8) q -= 16;
          dq = __fmul_rn((float)q, s);
        }
        dq = __bfloat162float(__float2bfloat16_rn(dq));
#pragma unroll
        for (int r = 0; r < kRowsPerPass; ++r) {
          if (m0 + r < p.M) acc[r] = fmaf(__bfloat162float(p.x[(m0 + r) * p.K + k]), dq, acc[r]);
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
        if (m0 + r < p.M) {
          float v = acc[r];
          if (p.bias) v += load_as_float(p.bias, n, p.bias_dtype);
          const int64_t idx = (m0 + r) * p.N + n;
          v = apply_post_ops(v, p.post, idx, ZT_BF16);
          p.y[idx] = __float2bfloat16_rn(v);
        }
      }
    }
  }
}

__global__ void woq_repack_weight_kernel(const int8_t *__restrict__ w, int64_t total_words, int32_t *__restrict__ out) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total_words) return;
  // eight consecutive bytes -> one word, byte j to bits [4j, 4j+4)
  const uint2 v = *reinterpret_cast<const uint2 *>(w + i * 8);
  uint32_t word = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    word |= ((v.x >> (8 * j)) & 0xFu) << (4 * j);
    word |= ((v.y >> (8 * j)) & 0xFu) << (4 * (j + 4));
  }
  out[i] = (int32_t)word;
}

// One thread produces one output word: row n, k = 8c .. 8c+7.  Row n lives in 64-row block n/64 at
// in-block row d' = n%64: byte index (d' % 16) + 16 * ((d' / 16) & 1) of the column's 32 bytes,
// low nibble when d' < 32, high nibble otherwise.
__global__ void woq_repack_from_int4pack_kernel(const uint8_t *__restrict__ packed, int64_t N, int64_t K,
                                                int32_t *__restrict__ out) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t k8 = K >> 3;
  if (i >= N * k8) return;
  const int64_t n = i / k8, c = i - n * k8;
  const int64_t blk = n >> 6;
  const int dr = (int)(n & 63);
  const int byte = (dr & 15) + 16 * ((dr >> 4) & 1);
  const int shift = (dr >= 32) ? 4 : 0;
  const uint8_t *src = packed + blk * K * 32 + byte;
  uint32_t word = 0;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const uint32_t b = src[(c * 8 + j) * 32];
    word |= ((b >> shift) & 0xFu) << (4 * j);
  }
  out[i] = (int32_t)word;
}

}  // namespace

int woq_generic_launch(const zt_woq_linear_args_t &a, cudaStream_t st) {
  GenericParams p{};
  p.x = reinterpret_cast<const __nv_bfloat16 *>(a.x);
  p.wq = a.wq;
  p.scales = a.scales;
  p.zeros = a.zeros;
  p.bias = a.bias;
  p.y = reinterpret_cast<__nv_bfloat16 *>(a.y);
  p.M = a.M;
  p.N = a.N;
  p.K = a.K;
  p.gs = a.K / a.n_groups;
  p.scale_dtype = a.scale_dtype;
  p.bias_dtype = a.bias_dtype;
  p.post = to_dev(a.post);
  const int warps = 8;
  const int64_t mblocks = ceil_div<int64_t>(a.M, kRowsPerPass);
  dim3 grid((unsigned)ceil_div<int64_t>(a.N, warps), (unsigned)(mblocks < 4096 ? mblocks : 4096));
  woq_generic_kernel<<<grid, warps * 32, 0, st>>>(p);
  return launch_status("woq_generic_kernel");
}

}  // namespace zt

using namespace zt;

extern "C" int zt_woq_repack_weight(const int8_t *unpacked, int64_t N, int64_t K, int32_t *packed, void *stream) {
  ZT_REQUIRE(N >= 0, ZT_INVALID_ARGUMENT, "zt_woq_repack_weight: N must be non-negative, got %lld", (long long)N);
  ZT_REQUIRE(K >= 8, ZT_INVALID_ARGUMENT, "K must be at least 8, got %lld", (long long)K);
  ZT_REQUIRE(K % 8 == 0, ZT_INVALID_ARGUMENT, "K must be divisible by 8, got %lld", (long long)K);
  if (N == 0) return ZT_SUCCESS;
  ZT_REQUIRE(unpacked && packed, ZT_INVALID_ARGUMENT, "zt_woq_repack_weight: null pointer");
  ZT_REQUIRE((reinterpret_cast<uintptr_t>(unpacked) & 7) == 0, ZT_INVALID_ARGUMENT,
             "zt_woq_repack_weight: unpacked weight must be 8-byte aligned");
  const int64_t words = N * (K / 8);
  if (words == 0) return ZT_SUCCESS;
  woq_repack_weight_kernel<<<(unsigned)ceil_div<int64_t>(words, 256), 256, 0, (cudaStream_t)stream>>>(unpacked, words,
                                                                                                     packed);
  return launch_status("woq_repack_weight_kernel");
}

extern "C" int zt_woq_repack_from_int4pack(const uint8_t *int4pack, int64_t N, int64_t K_half, int32_t *packed,
                                           void *stream) {
  ZT_REQUIRE(N % 64 == 0, ZT_INVALID_ARGUMENT, "packed_weight row count (%lld) must be a multiple of 64",
             (long long)N);
  const int64_t K = 2 * K_half;
  ZT_REQUIRE(K >= 8, ZT_INVALID_ARGUMENT, "K must be at least 8, got %lld", (long long)K);
  ZT_REQUIRE(K % 8 == 0, ZT_INVALID_ARGUMENT, "K must be divisible by 8, got %lld", (long long)K);
  const int64_t words = N * (K / 8);
  if (words == 0) return ZT_SUCCESS;
  ZT_REQUIRE(int4pack && packed, ZT_INVALID_ARGUMENT, "zt_woq_repack_from_int4pack: null pointer");
  woq_repack_from_int4pack_kernel<<<(unsigned)ceil_div<int64_t>(words, 256), 256, 0, (cudaStream_t)stream>>>(
      int4pack, N, K, packed);
  return launch_status("woq_repack_from_int4pack_kernel");
}
