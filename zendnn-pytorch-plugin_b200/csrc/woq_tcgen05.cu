// Weight-only int4 linear for M > 16 (prefill and large decode batches) on tcgen05 tensor cores.
//
//   Y[M,N] = post_ops( X[M,K] . dq(Wq)[K,N] + bias ),   dq = bf16(q*s)  or  bf16((q-8)*s + z)
//
// The weight is the 128-row operand of the MMA (UMMA M = 128 output columns n), the activations are
// the other operand (UMMA N = BT tokens, up to 256), so a CTA dequantises a 128 x 64 block of weights
// per k-block and reuses it for up to 256 tokens.  One persistent CTA per SM walks over
// (128 columns) x (BT tokens) tiles; tiles that share a weight block are adjacent in the order.
//
//   warp 0        TMA producer for the activation tile (2-D tile load, 128-byte swizzle, no multicast)
//   warp 1        TMEM allocation, tcgen05.mma.kind::f16 issue (bf16 x bf16 -> fp32), TMEM release
//   warps 2..9    dequantisation: 128-bit loads of packed nibbles straight from global memory
//                 (prefetched four k-blocks ahead, with the group's scale / zero point), nibble -> bf16
//                 with lop3, exact subtraction of the encoding bias, multiplication by the scale in
//                 bf16x2 arithmetic, byte-permute into k order, 16-byte stores into the canonical
//                 K-major 128-byte-swizzled operand layout, fence.proxy.async, mbarrier arrive
//   warps 10..13  epilogue: tcgen05.ld (lane = output column n, register j = token), transpose
//                 through shared memory so that stores run along n, bias + post-ops, bf16 stores
//
// Accumulators are double buffered in tensor memory: the epilogue of a tile overlaps the next tile's
// main loop.  All waits are bounded (see tc05.cuh).
//
// Rounding.  q (an integer in [-8, 7]) is exact in bf16.  With bf16 scales q*s is one bf16x2
// multiplication, i.e. exactly bf16(q*s).  With fp32 scales s is split into s_hi + s_lo (both bf16) and
// dq = fma(q, s_hi, q*s_lo), which equals bf16(q*s) except for rare double-rounding cases one bf16 ulp
// apart.  The zero-point form is evaluated in fp32, (q - 8) * s + z, and rounded once.
#include <algorithm>
#include <mutex>
#include <unordered_map>

#include "tc05.cuh"
#include "woq.cuh"

namespace zt {

namespace {

constexpr int kBN = 128;  // output columns per tile (UMMA M)
constexpr int kBK = 64;   // k per stage: 128 bytes of bf16
constexpr int kDqWarps = 8;
constexpr int kEpiWarps = 4;
constexpr int kThreads = 64 + 32 * (kDqWarps + kEpiWarps);
constexpr int kEpiRowStride = 36;  // floats; 144 bytes keeps 16-byte alignment and spreads banks

struct TcParams {
  int M, N, K;
  int m_tiles, n_tiles;
  int gs;
  const int32_t *wq;
  const void *scales;
  const void *zeros;
  int scale_dtype;
  const void *bias;
  int bias_dtype;
  __nv_bfloat16 *y;
  PostOpsDev post;
  int *status;
};

template <int BT, int STAGES>
struct SmemLayout {
  static constexpr int kWBytes = kBN * 128;
  static constexpr int kXBytes = BT * 128;
  static constexpr int kStageBytes = kWBytes + kXBytes;
  static constexpr int kTileBytes = STAGES * kStageBytes;
  static constexpr int kEpiBytes = kEpiWarps * 32 * kEpiRowStride * 4;
  static constexpr int kBarBytes = (3 * STAGES + 4) * 8 + 8;
  static constexpr int kTotal = kTileBytes + kEpiBytes + kBarBytes + 1024;
};

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}
template <bool SIGNED>
__device__ __forceinline__ uint32_t nib_pair_to_bf16x2(uint32_t w) {
  uint32_t r;
  if (SIGNED) {
    asm("lop3.b32 %0, %1, %2, %3, 0x6a;" : "=r"(r) : "r"(w), "n"(0x000f000f), "n"(0x43084308));
  } else {
    asm("lop3.b32 %0, %1, %2, %3, 0xea;" : "=r"(r) : "r"(w), "n"(0x000f000f), "n"(0x43004300));
  }
  return r;
}
__device__ __forceinline__ uint32_t bf2_sub(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ uint32_t bf2_mul(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ uint32_t bf2_fma(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t r;
  asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
  return r;
}
// value -> (hi, lo) bf16 parts replicated into both halves of a register each
__device__ __forceinline__ void split_bf16x2(float v, uint32_t &hi2, uint32_t &lo2) {
  const __nv_bfloat16 h = __float2bfloat16_rn(v);
  const __nv_bfloat16 l = __float2bfloat16_rn(v - __bfloat162float(h));
  const uint32_t hb = __bfloat16_as_ushort(h), lb = __bfloat16_as_ushort(l);
  hi2 = hb | (hb << 16);
  lo2 = lb | (lb << 16);
}

struct DqRegs {
  uint4 w;
  float s, z;
};

template <int BT, int STAGES, bool ASYM>
__global__ void __launch_bounds__(kThreads, 1) woq_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_x,
                                                                  const TcParams p) {
  using L = SmemLayout<BT, STAGES>;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char *smem = smem_dyn + ((1024u - (smem_u32(smem_dyn) & 1023u)) & 1023u);
  float *epi_scratch = reinterpret_cast<float *>(smem + L::kTileBytes);
  uint64_t *full_x = reinterpret_cast<uint64_t *>(smem + L::kTileBytes + L::kEpiBytes);
  uint64_t *full_w = full_x + STAGES;
  uint64_t *empty_bar = full_w + STAGES;
  uint64_t *tmem_full = empty_bar + STAGES;  // [2]
  uint64_t *tmem_empty = tmem_full + 2;      // [2]
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(tmem_empty + 2);

  constexpr uint32_t kTmemCols = 2 * BT <= 32 ? 32 : 2 * BT <= 64 ? 64 : 2 * BT <= 128 ? 128 : 2 * BT <= 256 ? 256 : 512;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_kb = p.K / kBK;
  const int total_tiles = p.m_tiles * p.n_tiles;

  if (threadIdx.x == 0) {
    tc::prefetch_tensormap(&tmap_x);
    for (int s = 0; s < STAGES; ++s) {
      tc::mbar_init(&full_x[s], 1);
      tc::mbar_init(&full_w[s], kDqWarps);
      tc::mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      tc::mbar_init(&tmem_full[b], 1);
      tc::mbar_init(&tmem_empty[b], kEpiWarps);
    }
    tc::mbar_fence_init();
  }
  if (warp == 1) tc::tmem_alloc(tmem_slot, kTmemCols);
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer: activation tiles ----------------
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        const int m0 = (tile % p.m_tiles) * BT;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const uint32_t s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!tc::mbar_wait(&empty_bar[s], ph ^ 1)) {
            tc::report_timeout(p.status, kStatusProducerTimeout);
            ok = false;
            break;
          }
          tc::mbar_expect_tx(&full_x[s], L::kXBytes);
          tc::tma_load_2d(smem + s * L::kStageBytes + L::kWBytes, &tmap_x, &full_x[s], kb * kBK, m0);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = tc::instr_desc(1u, 1u, 1u, kBN, BT);  // f32 accumulate, bf16 x bf16
      uint32_t it = 0;
      bool ok = true;
      int local = 0;
      for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++local) {
        const uint32_t buf = local & 1;
        const uint32_t use = (uint32_t)local >> 1;
        if (ok && !tc::mbar_wait(&tmem_empty[buf], (use & 1) ^ 1)) {
          tc::report_timeout(p.status, kStatusMmaTimeout);
          ok = false;
        }
        tc::fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * BT;
        for (int kb = 0; kb < num_kb && ok; ++kb, ++it) {
          const uint32_t s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!tc::mbar_wait(&full_x[s], ph) || !tc::mbar_wait(&full_w[s], ph)) {
            tc::report_timeout(p.status, kStatusMmaTimeout);
            ok = false;
            break;
          }
          tc::fence_after_sync();
          const uint32_t w_addr = smem_u32(smem + s * L::kStageBytes);
          const uint64_t a_desc = tc::smem_desc_k_sw128(w_addr);
          const uint64_t b_desc = tc::smem_desc_k_sw128(w_addr + L::kWBytes);
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) {
            // 16 bf16 = 32 bytes of K per instruction: advance the start addresses by 32 >> 4 = 2
            tc::mma_f16(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          tc::mma_commit(&empty_bar[s]);
        }
        tc::mma_commit(&tmem_full[buf]);
      }
    }
  } else if (warp < 2 + kDqWarps) {
    // ---------------- dequantisation warps ----------------
    const int d = threadIdx.x - 64;   // 0..255
    const int row = d >> 1;           // weight row (output column) within the tile
    const int half = d & 1;           // which 32 k of the 64-wide k-block
    const int k8 = p.K >> 3;
    auto fetch = [&](int tile, int kb, DqRegs &r) {
      const int n = min((tile / p.m_tiles) * kBN + row, p.N - 1);
      const int k = kb * kBK + 32 * half;
      r.w = ldg_nc_v4(p.wq + (size_t)n * k8 + (k >> 3));
      const int64_t gi = (int64_t)(k / p.gs) * p.N + n;
      r.s = load_as_float(p.scales, gi, p.scale_dtype);
      r.z = ASYM ? load_as_float(p.zeros, gi, p.scale_dtype) : 0.f;
    };
    // The packed words and scales are fetched kPrefetch k-blocks ahead into a register ring, so that
    // several global loads per thread are in flight while one k-block is converted.
    constexpr int kPrefetch = 4;
    DqRegs ring[kPrefetch];
    int ftile = blockIdx.x, fkb = 0;  // next (tile, k-block) to fetch
    auto fetch_next = [&](DqRegs &slot) {
      if (ftile < total_tiles) {
        fetch(ftile, fkb, slot);
        if (++fkb == num_kb) {
          fkb = 0;
          ftile += gridDim.x;
        }
      }
    };
#pragma unroll
    for (int i = 0; i < kPrefetch; ++i) fetch_next(ring[i]);
    uint32_t it = 0;
    bool ok = true;
    const bool exact_scale = (p.scale_dtype == ZT_BF16);
    const int my_tiles = blockIdx.x < total_tiles ? (total_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    const uint32_t total_it = (uint32_t)my_tiles * (uint32_t)num_kb;
    while (it < total_it) {
#pragma unroll
      for (int slot_i = 0; slot_i < kPrefetch; ++slot_i) {
        if (it < total_it) {
          const DqRegs cur = ring[slot_i];
          fetch_next(ring[slot_i]);
          const uint32_t s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (ok && !tc::mbar_wait(&empty_bar[s], ph ^ 1)) {
            tc::report_timeout(p.status, kStatusConvertTimeout);
            ok = false;
          }
          if (ok) {
            unsigned char *wrow = smem + s * L::kStageBytes + row * 128;
            const uint32_t words[4] = {cur.w.x, cur.w.y, cur.w.z, cur.w.w};
            uint32_t s_hi = 0, s_lo = 0;
            if (!ASYM) split_bf16x2(cur.s, s_hi, s_lo);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint4 o;
              if (ASYM) {
                // zero-point form in fp32, one rounding: bf16((q - 8) * s + z), pairs come out in k order
                float f[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                  const uint32_t bits = ((words[i] >> (4 * e)) & 0xFu) | 0x4B000000u;  // 2^23 + q
                  f[e] = fmaf(__uint_as_float(bits) - 8388616.0f, cur.s, cur.z);     // (q - 8) * s + z
                }
                __nv_bfloat162 p0 = __floats2bfloat162_rn(f[0], f[1]);
                __nv_bfloat162 p1 = __floats2bfloat162_rn(f[2], f[3]);
                __nv_bfloat162 p2 = __floats2bfloat162_rn(f[4], f[5]);
                __nv_bfloat162 p3 = __floats2bfloat162_rn(f[6], f[7]);
                o.x = *reinterpret_cast<uint32_t *>(&p0);
                o.y = *reinterpret_cast<uint32_t *>(&p1);
                o.z = *reinterpret_cast<uint32_t *>(&p2);
                o.w = *reinterpret_cast<uint32_t *>(&p3);
              } else {
                uint32_t r[4];
#pragma unroll
                for (int pp = 0; pp < 4; ++pp) {
                  uint32_t v = nib_pair_to_bf16x2<true>(words[i] >> (4 * pp));
                  v = bf2_sub(v, 0x43084308u);  // exact: (128 + u) - 136 = q
                  r[pp] = exact_scale ? bf2_mul(v, s_hi) : bf2_fma(v, s_hi, bf2_mul(v, s_lo));  // (k = p, k = p + 4)
                }
                o.x = prmt(r[0], r[1], 0x5410);  // (k0, k1)
                o.y = prmt(r[2], r[3], 0x5410);  // (k2, k3)
                o.z = prmt(r[0], r[1], 0x7632);  // (k4, k5)
                o.w = prmt(r[2], r[3], 0x7632);  // (k6, k7)
              }
              const int chunk = 4 * half + i;  // 16-byte chunk of the 128-byte row
              *reinterpret_cast<uint4 *>(wrow + ((chunk ^ (row & 7)) << 4)) = o;
            }
            tc::fence_proxy_async_smem();  // generic-proxy stores -> visible to the tensor core's reads
          }
          __syncwarp();
          if (lane == 0) tc::mbar_arrive(&full_w[s]);
          ++it;
        }
      }
    }
  } else {
    // ---------------- epilogue warps ----------------
    const int ew = warp - (2 + kDqWarps);  // 0..3
    const int quarter = warp & 3;          // TMEM lanes 32*quarter .. +31
    float *scratch = epi_scratch + ew * 32 * kEpiRowStride;
    int local = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++local) {
      const int m0 = (tile % p.m_tiles) * BT;
      const int n0 = (tile / p.m_tiles) * kBN;
      const uint32_t buf = local & 1;
      const uint32_t use = (uint32_t)local >> 1;
      if (ok && !tc::mbar_wait(&tmem_full[buf], use & 1)) {
        tc::report_timeout(p.status, kStatusEpilogueTimeout);
        ok = false;
      }
      tc::fence_after_sync();
      const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * BT;
      const int nq = n0 + quarter * 32;        // first output column of this warp
      // phase-2 mapping: lane -> (token row within a group of 4, four consecutive columns)
      const int sub_row = lane >> 3;
      const int col4 = (lane & 7) * 4;
      float bias4[4] = {0.f, 0.f, 0.f, 0.f};
      if (p.bias) {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (nq + col4 + e < p.N) bias4[e] = load_as_float(p.bias, nq + col4 + e, p.bias_dtype);
      }
#pragma unroll 1
      for (int c = 0; c < BT; c += 32) {
        uint32_t r[32];
        tc::tmem_ld_32x32b_x32(t_row + c, r);
        tc::tmem_ld_wait();
        // phase 1: scratch[token j][column lane]
#pragma unroll
        for (int j = 0; j < 32; ++j) scratch[j * kEpiRowStride + lane] = __uint_as_float(r[j]);
        __syncwarp();
        // phase 2: rows of 32 columns, 4 token rows per pass
#pragma unroll 1
        for (int pass = 0; pass < 8; ++pass) {
          const int j = pass * 4 + sub_row;
          const int m = m0 + c + j;
          const float4 v4 = *reinterpret_cast<const float4 *>(&scratch[j * kEpiRowStride + col4]);
          if (m < p.M && nq + col4 < p.N) {
            float v[4] = {v4.x + bias4[0], v4.y + bias4[1], v4.z + bias4[2], v4.w + bias4[3]};
            const int64_t base = (int64_t)m * p.N + nq + col4;
            if (p.post.n_ops > 0) {
#pragma unroll
              for (int e = 0; e < 4; ++e)
                if (nq + col4 + e < p.N) v[e] = apply_post_ops(v[e], p.post, base + e, ZT_BF16);
            }
            __nv_bfloat16 *dst = p.y + base;
            if (nq + col4 + 4 <= p.N && (p.N & 3) == 0) {
              __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]);
              __nv_bfloat162 hi = __floats2bfloat162_rn(v[2], v[3]);
              uint2 o;
              o.x = *reinterpret_cast<uint32_t *>(&lo);
              o.y = *reinterpret_cast<uint32_t *>(&hi);
              *reinterpret_cast<uint2 *>(dst) = o;
            } else {
#pragma unroll
              for (int e = 0; e < 4; ++e)
                if (nq + col4 + e < p.N) dst[e] = __float2bfloat16_rn(v[e]);
            }
          }
        }
        __syncwarp();  // scratch is rewritten by the next chunk; tcgen05.ld is warp-collective
      }
      tc::fence_before_sync();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(&tmem_empty[buf]);
    }
  }

  tc::fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc::fence_after_sync();
    tc::tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---- host ----------------------------------------------------------------------------------------
struct MapKey {
  const void *ptr;
  uint64_t inner, rows;
  uint32_t box_rows;
  bool operator==(const MapKey &o) const {
    return ptr == o.ptr && inner == o.inner && rows == o.rows && box_rows == o.box_rows;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey &k) const {
    return std::hash<const void *>()(k.ptr) ^ (k.inner * 1315423911u) ^ (k.rows << 17) ^ k.box_rows;
  }
};

int cached_x_map(CUtensorMap *out, const void *ptr, uint64_t k, uint64_t rows, uint32_t box_rows) {
  static std::mutex mu;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  const MapKey key{ptr, k, rows, box_rows};
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it != cache.end()) {
    *out = it->second;
    return ZT_SUCCESS;
  }
  int rc = make_tensor_map_2d(out, ptr, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, k, rows, k * 2, kBK, box_rows);
  if (rc != ZT_SUCCESS) return rc;
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, *out);
  return ZT_SUCCESS;
}

template <int BT, int STAGES>
int launch_bt(const TcParams &p0, const void *x, bool asym, cudaStream_t st) {
  using L = SmemLayout<BT, STAGES>;
  TcParams p = p0;
  p.m_tiles = ceil_div(p.M, BT);
  p.n_tiles = ceil_div(p.N, kBN);
  CUtensorMap tx;
  int rc = cached_x_map(&tx, x, (uint64_t)p.K, (uint64_t)p.M, BT);
  if (rc != ZT_SUCCESS) return rc;
  const int tiles = p.m_tiles * p.n_tiles;
  const int sms = sm_count();
  dim3 grid((unsigned)(tiles < sms ? tiles : sms));
  if (asym) {
    auto kern = woq_tcgen05_kernel<BT, STAGES, true>;
    static bool configured = false;
    if (!configured) {
      ZT_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal));
      configured = true;
    }
    kern<<<grid, kThreads, L::kTotal, st>>>(tx, p);
  } else {
    auto kern = woq_tcgen05_kernel<BT, STAGES, false>;
    static bool configured = false;
    if (!configured) {
      ZT_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal));
      configured = true;
    }
    kern<<<grid, kThreads, L::kTotal, st>>>(tx, p);
  }
  return launch_status("woq_tcgen05_kernel");
}

}  // namespace

bool woq_tcgen05_supported(const zt_woq_linear_args_t &a) {
  if (a.M < 1 || a.N < 1 || a.K < kBK || a.K % kBK != 0) return false;
  if (a.n_groups <= 0 || a.K % a.n_groups != 0) return false;
  const int64_t gs = a.K / a.n_groups;
  if (gs % 32 != 0) return false;
  if ((reinterpret_cast<uintptr_t>(a.x) | reinterpret_cast<uintptr_t>(a.wq)) & 15) return false;
  return a.M <= (1 << 30) && a.N <= (1 << 30) && a.K <= (1 << 30);
}

int woq_tcgen05_launch(const zt_woq_linear_args_t &a, cudaStream_t st) {
  TcParams p{};
  p.M = (int)a.M;
  p.N = (int)a.N;
  p.K = (int)a.K;
  p.gs = (int)(a.K / a.n_groups);
  p.wq = a.wq;
  p.scales = a.scales;
  p.zeros = a.zeros;
  p.scale_dtype = a.scale_dtype;
  p.bias = a.bias;
  p.bias_dtype = a.bias_dtype;
  p.y = reinterpret_cast<__nv_bfloat16 *>(a.y);
  p.post = to_dev(a.post);
  p.status = device_status_ptr();
  const bool asym = a.zeros != nullptr;
  int bt = (a.algo >> 8) & 0xffff;
  if (bt == 0) bt = a.M <= 32 ? 32 : a.M <= 64 ? 64 : a.M <= 128 ? 128 : 256;
  switch (bt) {
    case 32: return launch_bt<32, 8>(p, a.x, asym, st);
    case 64: return launch_bt<64, 7>(p, a.x, asym, st);
    case 128: return launch_bt<128, 5>(p, a.x, asym, st);
    case 256: return launch_bt<256, 4>(p, a.x, asym, st);
    default: break;
  }
  set_error("zt_woq_linear: unsupported token-tile width %d for the tcgen05 kernel", bt);
  return ZT_UNSUPPORTED;
}

}  // namespace zt
