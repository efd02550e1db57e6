// Weight-only int4 linear for mid-size M (17..64 rows per launch) on mma.sync tensor cores.
//
// Work decomposition.  A CTA of four warps owns 32 output columns (= 32 rows of the N-major packed
// weight) and one K-slice.  The warps take the slice's 128-wide k-steps round-robin.  Within a
// k-step every lane streams its rows with 128-bit loads (32 nibbles each; the four lanes of a quad
// cover the 128 consecutive k of one step), turns nibbles into bf16 pairs in registers with one
// lop3 per pair, and feeds them as the A operand of mma.sync.m16n8k16 (rows = output columns n).
// The B operand is the activation slice, staged once per CTA in shared memory in the nibble-pair
// order (k, k+4),(k+1, k+5),.. so that a lane's 16-byte shared load is its B fragment as is.
// The scale of the step's quantisation group is applied to the step's fp32 partial sum, outside the
// MMA.  Warp partials are reduced through shared memory; K-slices are reduced through a global fp32
// scratch by the last CTA to arrive (fixed order, so the result is deterministic), which also
// applies bias and post-ops.
//
// Nibble decoding.  (w >> 4p) & 0x000f000f picks nibbles p and p+4; or-ing 0x4300 into each half
// makes the bf16 number 128 + u.  For signed weights the nibble is xor-ed with 8 in the same lop3,
// so u = q + 8 in both the signed and the unsigned (zero-point) format and the true value is
// (128 + u) - 136.  With FOLD the subtraction is not done per element: the MMA runs on 128 + u and
// 136 * sum_k x[m,k] of the step is subtracted from the step's partial sum instead.
#include "common.cuh"
#include "woq.cuh"

namespace zt {

namespace {

constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;
constexpr int kTileN = 32;    // output columns per CTA
constexpr int kStepK = 128;   // k per step
constexpr int kRowBlocks = 2; // 16-row MMA blocks per warp

struct SkinnyParams {
  const __nv_bfloat16 *x;
  const int32_t *wq;
  const void *scales;
  const void *zeros;
  const void *bias;
  __nv_bfloat16 *y;
  float *partial;    // [nsplit][M][N]
  int *counters;     // one per n-tile, zero on entry and on exit
  int M, N, K;
  int gs;            // quantisation group size along K
  int kslice;        // k per CTA (multiple of 128)
  int nsplit;
  int scale_dtype, bias_dtype;
  PostOpsDev post;
};

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}

template <bool SIGNED>
__device__ __forceinline__ uint32_t nib_pair_to_bf16x2(uint32_t w) {
  uint32_t r;
  if (SIGNED) {  // (w & 0x000f000f) ^ 0x43084308
    asm("lop3.b32 %0, %1, %2, %3, 0x6a;" : "=r"(r) : "r"(w), "n"(0x000f000f), "n"(0x43084308));
  } else {       // (w & 0x000f000f) | 0x43004300
    asm("lop3.b32 %0, %1, %2, %3, 0xea;" : "=r"(r) : "r"(w), "n"(0x000f000f), "n"(0x43004300));
  }
  return r;
}

__device__ __forceinline__ uint32_t sub136(uint32_t v) {
  uint32_t r;
  // bf16x2: v - 136 is exact (both are small integers).
  asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(v), "r"(0x43084308u));
  return r;
}

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Shared-memory slot (16-byte units) of the eight activations k = 8b .. 8b+7 of the slice: the two
// 2-bit fields "which word of the lane's 128-bit load" and "which lane of the quad" are swapped so
// that the eight lanes of a shared-load phase hit eight different 16-byte bank groups.
__device__ __forceinline__ int x_slot(int b) { return (b & ~15) | ((b & 3) << 2) | ((b >> 2) & 3); }

template <int MT, bool ASYM, bool FOLD>
__global__ void __launch_bounds__(kThreads) woq_skinny_kernel(const SkinnyParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr int kCols = MT * 8;                  // activation rows held (padded M)
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int n0 = blockIdx.x * kTileN;
  const int split = blockIdx.y;
  const int k0 = split * p.kslice;
  const int klen = min(p.kslice, p.K - k0);
  const int steps = klen / kStepK;
  const int row_slots = p.kslice / 8 + 4;        // 16-byte slots per activation row (+4: bank skew)

  uint4 *xs = reinterpret_cast<uint4 *>(smem_raw);
  float *sx = reinterpret_cast<float *>(smem_raw + (size_t)kCols * row_slots * 16);  // [kCols][steps]
  const int sx_stride = p.kslice / kStepK;

  // ---- issue the first weight loads before anything else --------------------------------------
  const int k8 = p.K >> 3;
  const int32_t *wrow[kRowBlocks][2];
  int nrow[kRowBlocks][2];
#pragma unroll
  for (int r = 0; r < kRowBlocks; ++r) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      int n = n0 + 16 * r + 8 * h + g;
      nrow[r][h] = n;
      n = min(n, p.N - 1);
      wrow[r][h] = p.wq + (size_t)n * k8 + (k0 >> 3) + 4 * t;
    }
  }
  uint4 wcur[kRowBlocks][2], wnext[kRowBlocks][2];
  int q = warp;
  if (q < steps) {
#pragma unroll
    for (int r = 0; r < kRowBlocks; ++r)
#pragma unroll
      for (int h = 0; h < 2; ++h) wcur[r][h] = ldg_nc_v4(wrow[r][h] + q * 16);
  }

  // ---- stage the activation slice ---------------------------------------------------------------
  {
    const int blocks = klen / 8;
    for (int i = tid; i < kCols * blocks; i += kThreads) {
      const int c = i / blocks, b = i - c * blocks;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (c < p.M) v = *reinterpret_cast<const uint4 *>(p.x + (size_t)c * p.K + k0 + 8 * b);
      uint4 o;
      o.x = prmt(v.x, v.z, 0x5410);  // (x0, x4)
      o.y = prmt(v.x, v.z, 0x7632);  // (x1, x5)
      o.z = prmt(v.y, v.w, 0x5410);  // (x2, x6)
      o.w = prmt(v.y, v.w, 0x7632);  // (x3, x7)
      xs[c * row_slots + x_slot(b)] = o;
    }
  }
  __syncthreads();
  if (ASYM || FOLD) {
    for (int i = tid; i < kCols * steps; i += kThreads) {
      const int c = i / steps, s = i - c * steps;
      float acc = 0.f;
      const uint4 *row = xs + c * row_slots + s * 16;
#pragma unroll 4
      for (int j = 0; j < 16; ++j) {
        const uint4 v = row[j];
        const uint32_t wds[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) acc += bf16_bits_to_float(wds[e] & 0xffff) + bf16_bits_to_float(wds[e] >> 16);
      }
      sx[c * sx_stride + s] = acc;
    }
    __syncthreads();
  }

  // ---- main loop over this warp's k-steps -------------------------------------------------------
  float acc[kRowBlocks][MT][4];
#pragma unroll
  for (int r = 0; r < kRowBlocks; ++r)
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[r][m][e] = 0.f;

  for (; q < steps; q += kWarps) {
    const int qn = q + kWarps;
    if (qn < steps) {
#pragma unroll
      for (int r = 0; r < kRowBlocks; ++r)
#pragma unroll
        for (int h = 0; h < 2; ++h) wnext[r][h] = ldg_nc_v4(wrow[r][h] + qn * 16);
    }
    float part[kRowBlocks][MT][4];
#pragma unroll
    for (int r = 0; r < kRowBlocks; ++r)
#pragma unroll
      for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int e = 0; e < 4; ++e) part[r][m][e] = 0.f;

#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint4 bfrag[MT];
#pragma unroll
      for (int m = 0; m < MT; ++m) bfrag[m] = xs[(m * 8 + g) * row_slots + q * 16 + 4 * i + t];
#pragma unroll
      for (int r = 0; r < kRowBlocks; ++r) {
        const uint32_t wa = (i == 0) ? wcur[r][0].x : (i == 1) ? wcur[r][0].y : (i == 2) ? wcur[r][0].z : wcur[r][0].w;
        const uint32_t wb = (i == 0) ? wcur[r][1].x : (i == 1) ? wcur[r][1].y : (i == 2) ? wcur[r][1].z : wcur[r][1].w;
        uint32_t ra[4], rb[4];
#pragma unroll
        for (int pp = 0; pp < 4; ++pp) {
          ra[pp] = nib_pair_to_bf16x2<!ASYM>(wa >> (4 * pp));
          rb[pp] = nib_pair_to_bf16x2<!ASYM>(wb >> (4 * pp));
          if (!FOLD) {
            ra[pp] = sub136(ra[pp]);
            rb[pp] = sub136(rb[pp]);
          }
        }
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          mma_bf16_16816(part[r][m], ra[0], rb[0], ra[1], rb[1], bfrag[m].x, bfrag[m].y);
          mma_bf16_16816(part[r][m], ra[2], rb[2], ra[3], rb[3], bfrag[m].z, bfrag[m].w);
        }
      }
    }

    // fold the step into the running sums with the group's scale (and zero point)
    const int gidx = (k0 + q * kStepK) / p.gs;
#pragma unroll
    for (int r = 0; r < kRowBlocks; ++r) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int n = min(nrow[r][h], p.N - 1);
        const float s = load_as_float(p.scales, (int64_t)gidx * p.N + n, p.scale_dtype);
        float z = 0.f;
        if (ASYM) z = load_as_float(p.zeros, (int64_t)gidx * p.N + n, p.scale_dtype);
#pragma unroll
        for (int m = 0; m < MT; ++m) {
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            float v = part[r][m][2 * h + e];
            if (ASYM || FOLD) {
              const float sxv = sx[(m * 8 + 2 * t + e) * sx_stride + q];
              if (FOLD) v -= 136.f * sxv;
              acc[r][m][2 * h + e] += s * v + z * sxv;
            } else {
              acc[r][m][2 * h + e] += s * v;
            }
          }
        }
      }
    }
#pragma unroll
    for (int r = 0; r < kRowBlocks; ++r)
#pragma unroll
      for (int h = 0; h < 2; ++h) wcur[r][h] = wnext[r][h];
  }

  // ---- reduce the four warps through shared memory --------------------------------------------
  __syncthreads();  // everyone is done with xs / sx
  float *red = reinterpret_cast<float *>(smem_raw);  // [kWarps][kCols][kTileN + 1]
  constexpr int kRedStride = kTileN + 1;
#pragma unroll
  for (int r = 0; r < kRowBlocks; ++r)
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int nl = 16 * r + 8 * (e >> 1) + g;
        const int ml = m * 8 + 2 * t + (e & 1);
        red[(warp * kCols + ml) * kRedStride + nl] = acc[r][m][e];
      }
  __syncthreads();

  const int nl = tid & 31;
  const int n = n0 + nl;
  __shared__ int s_ticket;
  if (p.nsplit > 1) {
    for (int ml = tid >> 5; ml < p.M; ml += kWarps) {
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) v += red[(w * kCols + ml) * kRedStride + nl];
      if (n < p.N) p.partial[((size_t)split * p.M + ml) * p.N + n] = v;
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) s_ticket = atomicAdd(&p.counters[blockIdx.x], 1);
    __syncthreads();
    if (s_ticket != p.nsplit - 1) return;
    __threadfence();
    if (tid == 0) p.counters[blockIdx.x] = 0;
  }
  for (int ml = tid >> 5; ml < p.M; ml += kWarps) {
    if (n >= p.N) continue;
    float v = 0.f;
    if (p.nsplit > 1) {
      for (int s = 0; s < p.nsplit; ++s) v += __ldcg(&p.partial[((size_t)s * p.M + ml) * p.N + n]);
    } else {
#pragma unroll
      for (int w = 0; w < kWarps; ++w) v += red[(w * kCols + ml) * kRedStride + nl];
    }
    if (p.bias) v += load_as_float(p.bias, n, p.bias_dtype);
    const int64_t idx = (int64_t)ml * p.N + n;
    v = apply_post_ops(v, p.post, idx, ZT_BF16);
    p.y[idx] = __float2bfloat16_rn(v);
  }
}

size_t skinny_smem_bytes(int mt, int kslice) {
  const size_t cols = (size_t)mt * 8;
  const size_t stage = cols * (kslice / 8 + 4) * 16 + cols * (kslice / kStepK) * sizeof(float);
  const size_t red = (size_t)kWarps * cols * (kTileN + 1) * sizeof(float);
  return stage > red ? stage : red;
}

template <int MT, bool ASYM, bool FOLD>
int launch(const SkinnyParams &p, dim3 grid, size_t smem, cudaStream_t st) {
  auto kern = woq_skinny_kernel<MT, ASYM, FOLD>;
  static PerDeviceOnce configured;
  if (int rc_cfg = allow_dynamic_smem(configured, kern, 160 * 1024)) return rc_cfg;
  kern<<<grid, kThreads, smem, st>>>(p);
  return launch_status("woq_skinny_kernel");
}

template <int MT>
int launch_mt(const SkinnyParams &p, bool asym, bool fold, dim3 grid, size_t smem, cudaStream_t st) {
  (void)fold;
  return asym ? launch<MT, true, false>(p, grid, smem, st) : launch<MT, false, false>(p, grid, smem, st);
}

}  // namespace

// Picks the K-slice: as long as possible (fewer partial sums) while the grid still fills the GPU.
WoqSkinnyPlan woq_skinny_plan(int64_t M, int64_t N, int64_t K) {
  WoqSkinnyPlan pl{};
  const int mchunk = (int)(M < 64 ? M : 64);
  pl.mt = mchunk <= 32 ? 4 : 8;
  const int64_t ntiles = ceil_div<int64_t>(N, kTileN);
  const int64_t want = 3LL * sm_count();
  int kslice = pl.mt <= 2 ? 2048 : (pl.mt == 4 ? 1024 : 512);
  if (kslice > K) kslice = (int)K;
  while (kslice > 512 && kslice % 256 == 0 && ntiles * ceil_div<int64_t>(K, kslice) < want) kslice /= 2;
  pl.kslice = kslice;
  pl.nsplit = (int)ceil_div<int64_t>(K, kslice);
  if (ntiles * (int64_t)sizeof(int) > ZT_WOQ_COUNTER_BYTES) {  // no counter per tile: one slice only
    pl.nsplit = 1;
    pl.kslice = (int)K;
  }
  pl.partial_bytes = pl.nsplit > 1 ? (size_t)pl.nsplit * mchunk * N * sizeof(float) : 0;
  return pl;
}

bool woq_skinny_supported(const zt_woq_linear_args_t &a) {
  if (a.K % kStepK != 0 || a.n_groups <= 0 || a.K % a.n_groups != 0) return false;
  const int64_t gs = a.K / a.n_groups;
  if (gs % kStepK != 0) return false;
  if ((reinterpret_cast<uintptr_t>(a.x) | reinterpret_cast<uintptr_t>(a.wq)) & 15) return false;
  const WoqSkinnyPlan pl = woq_skinny_plan(a.M, a.N, a.K);
  if (skinny_smem_bytes(pl.mt, pl.kslice) > 160 * 1024) return false;
  return a.M >= 1 && a.N >= 1 && a.K <= (1 << 30) && a.N <= (1 << 30);
}

int woq_skinny_launch(const zt_woq_linear_args_t &a, bool fold, cudaStream_t st) {
  const WoqSkinnyPlan pl = woq_skinny_plan(a.M, a.N, a.K);
  ZT_REQUIRE(a.workspace_bytes >= ZT_WOQ_COUNTER_BYTES + pl.partial_bytes || pl.nsplit == 1, ZT_WORKSPACE_TOO_SMALL,
             "zt_woq_linear: workspace of %zu bytes is smaller than the %zu required", a.workspace_bytes,
             (size_t)ZT_WOQ_COUNTER_BYTES + pl.partial_bytes);
  ZT_REQUIRE(pl.nsplit == 1 || a.workspace != nullptr, ZT_WORKSPACE_TOO_SMALL, "zt_woq_linear: workspace is NULL");
  const size_t smem = skinny_smem_bytes(pl.mt, pl.kslice);
  const dim3 grid((unsigned)ceil_div<int64_t>(a.N, kTileN), (unsigned)pl.nsplit);
  for (int64_t m0 = 0; m0 < a.M; m0 += 64) {
    SkinnyParams p{};
    p.M = (int)((a.M - m0) < 64 ? (a.M - m0) : 64);
    p.N = (int)a.N;
    p.K = (int)a.K;
    p.x = reinterpret_cast<const __nv_bfloat16 *>(a.x) + m0 * a.K;
    p.y = reinterpret_cast<__nv_bfloat16 *>(a.y) + m0 * a.N;
    p.wq = a.wq;
    p.scales = a.scales;
    p.zeros = a.zeros;
    p.bias = a.bias;
    p.scale_dtype = a.scale_dtype;
    p.bias_dtype = a.bias_dtype;
    p.gs = (int)(a.K / a.n_groups);
    p.kslice = pl.kslice;
    p.nsplit = pl.nsplit;
    p.counters = reinterpret_cast<int *>(a.workspace);
    p.partial = reinterpret_cast<float *>(reinterpret_cast<char *>(a.workspace) + ZT_WOQ_COUNTER_BYTES);
    p.post = to_dev(a.post);
    for (int i = 0; i < ZT_MAX_POST_OPS; ++i)
      if (p.post.bufs[i]) p.post.bufs[i] = reinterpret_cast<const __nv_bfloat16 *>(p.post.bufs[i]) + m0 * a.N;
    const bool asym = a.zeros != nullptr;
    int rc;
    if (pl.mt == 4)
      rc = launch_mt<4>(p, asym, fold, grid, smem, st);
    else
      rc = launch_mt<8>(p, asym, fold, grid, smem, st);
    if (rc != ZT_SUCCESS) return rc;
  }
  return ZT_SUCCESS;
}

}  // namespace zt
