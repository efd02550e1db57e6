// Mixture-of-experts FFN with int4 weight-only experts (Mixtral style): routing bookkeeping, token
// gather, two grouped WOQ GEMMs on the tcgen05 kernel, silu(gate) * up, weighted combine.
//
// The reference's fused MoE (src/cpu/cpp/FusedMoE.cpp:289-436 for the token grouping, :470-718 for the
// FFN) accepts bf16 / fp32 / int8 expert weights only (src/cpu/cpp/GroupMatmul.cpp:104-108); the int4
// form here follows its structure: one pass builds per-expert contiguous token groups, the first GEMM
// produces [gate | up] (gate first, src/cpu/python/zentorch/vllm/_int8_moe_patch.py:48-50), the second
// GEMM maps back to the hidden size, and each token sums its top-k expert outputs with the routing
// weights.  Everything stays on the device: the GEMMs read the number of row tiles from device memory.
#include "common.cuh"
#include "woq.cuh"

namespace zt {

namespace {

constexpr int kRowTile = 64;  // token rows per GEMM tile (about the mean group size of the target config)

struct MoeLayout {
  size_t counts, offsets, cursor, tile_count, tiles, sorted_src, inv_pos, xs, h, a, o, total;
};

size_t align256(size_t v) { return (v + 255) / 256 * 256; }

MoeLayout moe_layout(int64_t T, int64_t H, int64_t I, int E, int top_k) {
  const size_t R = (size_t)T * top_k;
  const size_t max_tiles = (R + kRowTile - 1) / kRowTile + E;
  MoeLayout l{};
  size_t off = 0;
  auto take = [&](size_t bytes) {
    const size_t at = off;
    off += align256(bytes);
    return at;
  };
  l.counts = take(sizeof(int) * E);
  l.offsets = take(sizeof(int) * (E + 1));
  l.cursor = take(sizeof(int) * E);
  l.tile_count = take(sizeof(int));
  l.tiles = take(sizeof(int4) * max_tiles);
  l.sorted_src = take(sizeof(int) * R);
  l.inv_pos = take(sizeof(int) * R);
  l.xs = take(R * H * 2);
  l.h = take(R * 2 * I * 2);
  l.a = take(R * I * 2);
  l.o = take(R * H * 2);
  l.total = off;
  return l;
}

// One CTA: histogram of expert ids, exclusive offsets, placement of every (token, slot) into its
// expert's group, and the list of row tiles for the grouped GEMMs.  Ids outside [0, E) are skipped
// (tokens owned by another rank in expert-parallel runs).
__global__ void __launch_bounds__(1024) moe_route_kernel(const int32_t *__restrict__ ids, int R, int E, int *counts,
                                                         int *offsets, int *cursor, int *tile_count, int4 *tiles,
                                                         int *sorted_src, int *inv_pos) {
  extern __shared__ int sh[];  // counts[E], offsets[E+1], cursor[E]
  int *s_counts = sh, *s_off = sh + E, *s_cur = sh + 2 * E + 1;
  for (int e = threadIdx.x; e < E; e += blockDim.x) s_counts[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < R; i += blockDim.x) {
    const int e = ids[i];
    if (e >= 0 && e < E) atomicAdd(&s_counts[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0, nt = 0;
    for (int e = 0; e < E; ++e) {
      s_off[e] = acc;
      s_cur[e] = acc;
      for (int m0 = acc; m0 < acc + s_counts[e]; m0 += kRowTile)
        tiles[nt++] = make_int4(e, m0, min(kRowTile, acc + s_counts[e] - m0), 0);
      acc += s_counts[e];
    }
    s_off[E] = acc;
    *tile_count = nt;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < R; i += blockDim.x) {
    const int e = ids[i];
    if (e >= 0 && e < E) {
      const int pos = atomicAdd(&s_cur[e], 1);
      sorted_src[pos] = i;
      inv_pos[i] = pos;
    } else {
      inv_pos[i] = -1;
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) {
    offsets[e] = s_off[e];
    if (e < E) {
      counts[e] = s_counts[e];
      cursor[e] = s_cur[e];
    }
  }
}

// xs[pos, :] = x[token(pos), :]   (16-byte vectors; H % 8 == 0)
__global__ void moe_gather_kernel(const uint4 *__restrict__ x, const int *__restrict__ sorted_src,
                                  const int *__restrict__ offsets, int E, int top_k, int h_vec, uint4 *__restrict__ xs) {
  const int pos = blockIdx.x;
  if (pos >= offsets[E]) return;
  const int token = sorted_src[pos] / top_k;
  for (int v = threadIdx.x; v < h_vec; v += blockDim.x) xs[(size_t)pos * h_vec + v] = x[(size_t)token * h_vec + v];
}

// a[r, i] = silu(h[r, i]) * h[r, I + i]
__global__ void moe_silu_mul_kernel(const __nv_bfloat16 *__restrict__ h, const int *__restrict__ offsets, int E, int I,
                                    __nv_bfloat16 *__restrict__ a) {
  const int r = blockIdx.x;
  if (r >= offsets[E]) return;
  const __nv_bfloat162 *gate = reinterpret_cast<const __nv_bfloat162 *>(h + (size_t)r * 2 * I);
  const __nv_bfloat162 *up = reinterpret_cast<const __nv_bfloat162 *>(h + (size_t)r * 2 * I + I);
  __nv_bfloat162 *dst = reinterpret_cast<__nv_bfloat162 *>(a + (size_t)r * I);
  for (int i = threadIdx.x; i < I / 2; i += blockDim.x) {
    const float2 g = __bfloat1622float2(gate[i]), u = __bfloat1622float2(up[i]);
    dst[i] = __floats2bfloat162_rn(unary_post(g.x, ZT_POST_SILU) * u.x, unary_post(g.y, ZT_POST_SILU) * u.y);
  }
}

// y[t, :] = sum_j w[t, j] * o[inv_pos[t, j], :]   (fixed order j = 0 .. top_k-1)
__global__ void moe_combine_kernel(const __nv_bfloat16 *__restrict__ o, const int *__restrict__ inv_pos,
                                   const float *__restrict__ w, int top_k, int H, __nv_bfloat16 *__restrict__ y) {
  const int t = blockIdx.x;
  for (int c = threadIdx.x; c < H / 2; c += blockDim.x) {
    float2 acc = make_float2(0.f, 0.f);
    for (int j = 0; j < top_k; ++j) {
      const int pos = inv_pos[t * top_k + j];
      if (pos < 0) continue;
      const float2 v = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162 *>(o + (size_t)pos * H)[c]);
      const float wj = w[t * top_k + j];
      acc.x = fmaf(wj, v.x, acc.x);
      acc.y = fmaf(wj, v.y, acc.y);
    }
    reinterpret_cast<__nv_bfloat162 *>(y + (size_t)t * H)[c] = __floats2bfloat162_rn(acc.x, acc.y);
  }
}

}  // namespace
}  // namespace zt

using namespace zt;

extern "C" size_t zt_moe_woq_workspace_bytes(int64_t T, int64_t H, int64_t I, int32_t num_experts, int32_t top_k) {
  if (T <= 0 || H <= 0 || I <= 0 || num_experts <= 0 || top_k <= 0) return 256;
  return moe_layout(T, H, I, num_experts, top_k).total;
}

extern "C" int zt_moe_woq(const zt_moe_woq_args_t *a, void *stream) {
  ZT_REQUIRE(a != nullptr, ZT_INVALID_ARGUMENT, "zt_moe_woq: null argument block");
  ZT_REQUIRE(a->T >= 0 && a->H > 0 && a->I > 0, ZT_INVALID_ARGUMENT, "zt_moe_woq: invalid sizes");
  ZT_REQUIRE(a->num_experts >= 1 && a->num_experts <= 1024 && a->top_k >= 1 && a->top_k <= a->num_experts,
             ZT_INVALID_ARGUMENT, "zt_moe_woq: need 1 <= top_k <= num_experts <= 1024");
  if (a->T == 0) return ZT_SUCCESS;
  ZT_REQUIRE(a->x && a->topk_ids && a->topk_weights && a->w13 && a->s13 && a->w2 && a->s2 && a->y, ZT_INVALID_ARGUMENT,
             "zt_moe_woq: null tensor pointer");
  ZT_REQUIRE(a->scale_dtype == ZT_F32 || a->scale_dtype == ZT_BF16, ZT_INVALID_ARGUMENT,
             "zt_moe_woq: scales must be float32 or bfloat16");
  ZT_REQUIRE(a->group_size >= 32 && a->group_size % 32 == 0 && a->H % a->group_size == 0 && a->I % a->group_size == 0,
             ZT_UNSUPPORTED, "zt_moe_woq: group size must be a multiple of 32 that divides H and I");
  ZT_REQUIRE(a->H % 64 == 0 && a->I % 64 == 0, ZT_UNSUPPORTED, "zt_moe_woq: H and I must be multiples of 64");
  const int64_t R64 = a->T * a->top_k;
  ZT_REQUIRE(R64 <= (1 << 24), ZT_UNSUPPORTED, "zt_moe_woq: too many routed rows (%lld)", (long long)R64);
  const MoeLayout l = moe_layout(a->T, a->H, a->I, a->num_experts, a->top_k);
  ZT_REQUIRE(a->workspace && a->workspace_bytes >= l.total, ZT_WORKSPACE_TOO_SMALL,
             "zt_moe_woq: workspace of %zu bytes is smaller than the %zu required", a->workspace_bytes, l.total);
  ZT_REQUIRE((reinterpret_cast<uintptr_t>(a->workspace) & 255) == 0 && (reinterpret_cast<uintptr_t>(a->x) & 15) == 0,
             ZT_INVALID_ARGUMENT, "zt_moe_woq: workspace must be 256-byte and x 16-byte aligned");
  cudaStream_t st = (cudaStream_t)stream;
  char *ws = reinterpret_cast<char *>(a->workspace);
  const int R = (int)R64, E = a->num_experts;
  int *counts = reinterpret_cast<int *>(ws + l.counts), *offsets = reinterpret_cast<int *>(ws + l.offsets);
  int *cursor = reinterpret_cast<int *>(ws + l.cursor), *tile_count = reinterpret_cast<int *>(ws + l.tile_count);
  int4 *tiles = reinterpret_cast<int4 *>(ws + l.tiles);
  int *sorted_src = reinterpret_cast<int *>(ws + l.sorted_src), *inv_pos = reinterpret_cast<int *>(ws + l.inv_pos);
  void *xs = ws + l.xs, *h = ws + l.h, *act = ws + l.a, *o = ws + l.o;
  const int max_tiles = (R + kRowTile - 1) / kRowTile + E;

  moe_route_kernel<<<1, 1024, sizeof(int) * (3 * E + 1), st>>>(a->topk_ids, R, E, counts, offsets, cursor, tile_count,
                                                              tiles, sorted_src, inv_pos);
  int rc = launch_status("moe_route_kernel");
  if (rc != ZT_SUCCESS) return rc;
  moe_gather_kernel<<<R, 128, 0, st>>>(reinterpret_cast<const uint4 *>(a->x), sorted_src, offsets, E, a->top_k,
                                       (int)(a->H / 8), reinterpret_cast<uint4 *>(xs));
  rc = launch_status("moe_gather_kernel");
  if (rc != ZT_SUCCESS) return rc;
  rc = woq_tcgen05_grouped_launch(xs, R, 2 * a->I, a->H, a->w13, a->s13, a->scale_dtype, a->H / a->group_size, E, h,
                                  tile_count, tiles, max_tiles, kRowTile, st);
  if (rc != ZT_SUCCESS) return rc;
  moe_silu_mul_kernel<<<R, 256, 0, st>>>(reinterpret_cast<const __nv_bfloat16 *>(h), offsets, E, (int)a->I,
                                         reinterpret_cast<__nv_bfloat16 *>(act));
  rc = launch_status("moe_silu_mul_kernel");
  if (rc != ZT_SUCCESS) return rc;
  rc = woq_tcgen05_grouped_launch(act, R, a->H, a->I, a->w2, a->s2, a->scale_dtype, a->I / a->group_size, E, o,
                                  tile_count, tiles, max_tiles, kRowTile, st);
  if (rc != ZT_SUCCESS) return rc;
  moe_combine_kernel<<<(unsigned)a->T, 256, 0, st>>>(reinterpret_cast<const __nv_bfloat16 *>(o), inv_pos, a->topk_weights,
                                                     a->top_k, (int)a->H, reinterpret_cast<__nv_bfloat16 *>(a->y));
  return launch_status("moe_combine_kernel");
}
