// int8 x int8 -> int32 GEMM on tcgen05 tensor cores with the dynamic-qlinear epilogue fused.
//
//   acc[M,N] = Q[M,K] . W[N,K]^T          (Q: per-token quantised activations, s8 or u8; W: s8)
//   Y = post_ops( (acc - zp_m * wsum_n) * (s_m * w_n) + bias_n )
//
// Both operands are K-major, so they go from global memory to shared memory with plain 2-D TMA tile
// loads (128 bytes of K per row, 128-byte swizzle) and are consumed in place by
// tcgen05.mma.kind::i8 (K = 32 per instruction, four per 128-byte k-block).  The kernel is
// persistent: one CTA per SM walks over (MH*128) x BN output tiles (MH = 2 reuses each weight
// stage for two 128-row accumulators, which halves the weight bytes pulled per MAC) (tiles that share a weight column
// block are adjacent in the order, so they run at the same time on neighbouring SMs and the weight
// block is fetched from HBM once).  The int32 accumulator lives in tensor memory and is double
// buffered, so the epilogue of tile i overlaps the main loop of tile i+1:
//
//   warp 0      TMA producer (one lane): fills the shared-memory ring, across tile boundaries
//   warp 1      allocates tensor memory, issues the MMAs (one lane), frees tensor memory
//   warps 2..9  epilogue: tcgen05.ld the accumulator (lane == output row; two warps per 32-lane
//               quarter, each taking every other 32-column chunk), scale, bias, post-op, cast,
//               16-byte stores
//
// Ring stages are recycled through full/empty mbarriers (tcgen05.commit frees a stage when the MMAs
// that read it retire); accumulator buffers through tmem_full/tmem_empty mbarriers.  Every wait is
// bounded: on expiry the role records a status code and stops, the other roles run into their own
// bounded waits, tensor memory is freed and the kernel returns.
#pragma once

#include "int8.cuh"
#include "tc05.cuh"

namespace zt {

namespace i8tc {

constexpr int kBM = 128;
constexpr int kBK = 128;  // bytes (= int8 elements) of K per stage
constexpr int kEpiWarps = 8;
constexpr int kThreads = 64 + kEpiWarps * 32;

// kEpiStatic: the static-quantisation form (per-tensor activation parameters, optional per-tensor weight scale,
// requantised or strided output); kept apart so that the dynamic form's epilogue carries none of it
enum EpiMode { kEpiS32 = 0, kEpiLinear = 1, kEpiStatic = 2 };

struct TcParams {
  int M, N, K;
  int m_tiles, n_tiles;
  // epilogue
  const float *src_scale;  // [M]
  const int32_t *src_zp;   // [M] or null
  const void *w_scale;     // [N]
  const int32_t *w_rowsum; // [N] or null
  const void *bias;        // [N] or null
  int w_scale_dtype, bias_dtype, y_dtype;
  void *y;                 // [M,N] (y_dtype) or int32 for kEpiS32
  PostOpsDev post;
  int *status;             // device status word (bounded-wait failures)
  // kEpiStatic only
  bool w_scale_per_tensor;
  int post_dtype;
  const float *out_scale;
  const int32_t *out_zp;
  int64_t ldy;
};

template <int MH, int BN, int STAGES>
struct SmemLayout {
  static constexpr int kABytes = MH * kBM * kBK;
  static constexpr int kBBytes = BN * kBK;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kTileBytes = STAGES * kStageBytes;
  static constexpr int kVecBytes = 2 * 3 * BN * 4;      // per accumulator buffer: w_scale, bias, rowsum
  static constexpr int kBarBytes = (2 * STAGES + 4) * 8 + 8;
  static constexpr int kTotal = kTileBytes + kVecBytes + kBarBytes + 1024;  // + slack to align to 1024
};

// Scale, bias and post-op for 32 consecutive outputs of one row, then the store.
template <int UNARY>
__device__ __forceinline__ void finish_chunk(const TcParams &p, const uint32_t (&r)[32], float s_m, int zp_m,
                                             const float *wscale, const float *bias, const int32_t *rowsum, int m,
                                             int nb) {
  float v[32];
  // per-column vectors of the chunk, read as 16-byte shared loads (same address in every lane: broadcast)
  float wsc[32], bia[32];
#pragma unroll
  for (int j = 0; j < 32; j += 4) {
    const float4 a = *reinterpret_cast<const float4 *>(wscale + j);
    const float4 b = *reinterpret_cast<const float4 *>(bias + j);
    wsc[j] = a.x; wsc[j + 1] = a.y; wsc[j + 2] = a.z; wsc[j + 3] = a.w;
    bia[j] = b.x; bia[j + 1] = b.y; bia[j + 2] = b.z; bia[j + 3] = b.w;
  }
  if (p.src_zp) {
    // u8 activations: remove zp_m * sum_k W[n,k].  |acc|, |zp*rowsum| and their difference are all
    // bounded by 255 * 127 * K, which fits 32 bits for K <= 65536; longer rows take 64 bits.
    if (p.K <= 65536) {
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        const int4 rs = *reinterpret_cast<const int4 *>(rowsum + j);
        v[j] = (float)((int32_t)r[j] - zp_m * rs.x);
        v[j + 1] = (float)((int32_t)r[j + 1] - zp_m * rs.y);
        v[j + 2] = (float)((int32_t)r[j + 2] - zp_m * rs.z);
        v[j + 3] = (float)((int32_t)r[j + 3] - zp_m * rs.w);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = (float)((int64_t)(int32_t)r[j] - (int64_t)zp_m * rowsum[j]);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = (float)(int32_t)r[j];
  }
#pragma unroll
  for (int j = 0; j < 32; ++j) v[j] = v[j] * (s_m * wsc[j]) + bia[j];
  const int64_t base = (int64_t)m * p.N + nb;
  if (UNARY >= 0) {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = unary_post(v[j], UNARY);
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (nb + j < p.N) v[j] = apply_post_ops(v[j], p.post, base + j, p.y_dtype);
  }
  const bool full = nb + 32 <= p.N;
  if (p.y_dtype == ZT_BF16) {
    __nv_bfloat16 *dst = reinterpret_cast<__nv_bfloat16 *>(p.y) + base;
    if (full && (p.N & 7) == 0) {
#pragma unroll
      for (int j = 0; j < 32; j += 8) {
        uint4 o;
        __nv_bfloat162 t0 = __floats2bfloat162_rn(v[j], v[j + 1]);
        __nv_bfloat162 t1 = __floats2bfloat162_rn(v[j + 2], v[j + 3]);
        __nv_bfloat162 t2 = __floats2bfloat162_rn(v[j + 4], v[j + 5]);
        __nv_bfloat162 t3 = __floats2bfloat162_rn(v[j + 6], v[j + 7]);
        o.x = *reinterpret_cast<uint32_t *>(&t0);
        o.y = *reinterpret_cast<uint32_t *>(&t1);
        o.z = *reinterpret_cast<uint32_t *>(&t2);
        o.w = *reinterpret_cast<uint32_t *>(&t3);
        *reinterpret_cast<uint4 *>(dst + j) = o;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (nb + j < p.N) dst[j] = __float2bfloat16_rn(v[j]);
    }
  } else {
    float *dst = reinterpret_cast<float *>(p.y) + base;
    if (full && (p.N & 3) == 0) {
#pragma unroll
      for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4 *>(dst + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (nb + j < p.N) dst[j] = v[j];
    }
  }
}

// The same for the static-quantisation form: separately rounded product and sum (a requantised output sits
// on rounding boundaries of the float result), post-op operands of their own dtype, and a store that
// requantises or honours a row stride.
__device__ __forceinline__ void finish_chunk_static(const TcParams &p, const uint32_t (&r)[32], float s_x, int zp_x,
                                                    const float *wscale, const float *bias, const int32_t *rowsum,
                                                    const OutQuant &oq, int m, int nb) {
  float v[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    const float af = p.src_zp ? (float)((int64_t)(int32_t)r[j] - (int64_t)zp_x * rowsum[j]) : (float)(int32_t)r[j];
    v[j] = __fadd_rn(__fmul_rn(af, s_x * wscale[j]), bias[j]);
  }
  const int64_t base = (int64_t)m * p.N + nb;
#pragma unroll
  for (int j = 0; j < 32; ++j)
    if (nb + j < p.N) v[j] = apply_post_ops(v[j], p.post, base + j, p.post_dtype);
  const int64_t out = (int64_t)m * p.ldy + nb;
  const bool full = nb + 32 <= p.N;
  if (p.y_dtype == ZT_U8 || p.y_dtype == ZT_S8) {
    uint8_t *dst = reinterpret_cast<uint8_t *>(p.y) + out;
    if (full && ((reinterpret_cast<uintptr_t>(dst)) & 15) == 0) {
#pragma unroll
      for (int j = 0; j < 32; j += 16) {
        uint32_t w4[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          w4[q] = 0;
#pragma unroll
          for (int b = 0; b < 4; ++b) w4[q] |= ((uint32_t)requantize(v[j + 4 * q + b], oq) & 0xffu) << (8 * b);
        }
        *reinterpret_cast<uint4 *>(dst + j) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (nb + j < p.N) dst[j] = (uint8_t)requantize(v[j], oq);
    }
  } else if (p.y_dtype == ZT_BF16) {
    __nv_bfloat16 *dst = reinterpret_cast<__nv_bfloat16 *>(p.y) + out;
    if (full && ((reinterpret_cast<uintptr_t>(dst)) & 15) == 0) {
#pragma unroll
      for (int j = 0; j < 32; j += 8) {
        uint4 o;
        __nv_bfloat162 t0 = __floats2bfloat162_rn(v[j], v[j + 1]);
        __nv_bfloat162 t1 = __floats2bfloat162_rn(v[j + 2], v[j + 3]);
        __nv_bfloat162 t2 = __floats2bfloat162_rn(v[j + 4], v[j + 5]);
        __nv_bfloat162 t3 = __floats2bfloat162_rn(v[j + 6], v[j + 7]);
        o.x = *reinterpret_cast<uint32_t *>(&t0);
        o.y = *reinterpret_cast<uint32_t *>(&t1);
        o.z = *reinterpret_cast<uint32_t *>(&t2);
        o.w = *reinterpret_cast<uint32_t *>(&t3);
        *reinterpret_cast<uint4 *>(dst + j) = o;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (nb + j < p.N) dst[j] = __float2bfloat16_rn(v[j]);
    }
  } else {
    float *dst = reinterpret_cast<float *>(p.y) + out;
    if (full && ((reinterpret_cast<uintptr_t>(dst)) & 15) == 0) {
#pragma unroll
      for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4 *>(dst + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (nb + j < p.N) dst[j] = v[j];
    }
  }
}

template <int MH, int BN, int STAGES, int NBUF, int EPI, bool A_SIGNED>
__global__ void __launch_bounds__(kThreads, 1) int8_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a,
                                                                   const __grid_constant__ CUtensorMap tmap_b,
                                                                   const TcParams p) {
  using L = SmemLayout<MH, BN, STAGES>;
  static_assert(NBUF * MH * BN <= 512, "accumulators exceed tensor memory");
  extern __shared__ unsigned char smem_dyn[];
  // align on the shared-window address (what the descriptors and TMA see), not the generic one
  unsigned char *smem = smem_dyn + ((1024u - (smem_u32(smem_dyn) & 1023u)) & 1023u);
  float *s_vec = reinterpret_cast<float *>(smem + L::kTileBytes);  // [2][3][BN]
  uint64_t *full_bar = reinterpret_cast<uint64_t *>(smem + L::kTileBytes + L::kVecBytes);
  uint64_t *empty_bar = full_bar + STAGES;
  uint64_t *tmem_full = empty_bar + STAGES;   // [2]
  uint64_t *tmem_empty = tmem_full + 2;       // [2]
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(tmem_empty + 2);

  constexpr int kAccCols = NBUF * MH * BN;
  constexpr uint32_t kTmemCols = kAccCols <= 32 ? 32 : kAccCols <= 64 ? 64 : kAccCols <= 128 ? 128 : kAccCols <= 256 ? 256 : 512;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_kb = (p.K + kBK - 1) / kBK;
  const int total_tiles = p.m_tiles * p.n_tiles;

  if (threadIdx.x == 0) {
    tc::prefetch_tensormap(&tmap_a);
    tc::prefetch_tensormap(&tmap_b);
    for (int s = 0; s < STAGES; ++s) {
      tc::mbar_init(&full_bar[s], 1);
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
  // Programmatic dependent launch: the next kernel on the stream may start its prologue now; this one waits
  // for its predecessor (the per-token quantisation) only where it touches what that kernel writes.
  grid_launch_dependents();

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      uint32_t it = 0;  // ring position, runs across tiles
      bool ok = true;
      // First pass over the ring: the weight tiles do not depend on the preceding kernel, so they are
      // requested before the dependency wait and the activation tiles of the same stages after it.
      int pre = 0;
      if ((int)blockIdx.x < total_tiles) {
        const int m0 = ((int)blockIdx.x % p.m_tiles) * (MH * kBM);
        const int n0 = ((int)blockIdx.x / p.m_tiles) * BN;
        pre = num_kb < STAGES ? num_kb : STAGES;
        for (int kb = 0; kb < pre; ++kb) {
          tc::mbar_expect_tx(&full_bar[kb], L::kStageBytes);
          tc::tma_load_2d(smem + kb * L::kStageBytes + L::kABytes, &tmap_b, &full_bar[kb], kb * kBK, n0);
        }
        grid_dependency_wait();
        for (int kb = 0; kb < pre; ++kb)
          tc::tma_load_2d(smem + kb * L::kStageBytes, &tmap_a, &full_bar[kb], kb * kBK, m0);
        it = (uint32_t)pre;
      }
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        const int m0 = (tile % p.m_tiles) * (MH * kBM);
        const int n0 = (tile / p.m_tiles) * BN;
        for (int kb = (tile == (int)blockIdx.x ? pre : 0); kb < num_kb; ++kb, ++it) {
          const uint32_t s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!tc::mbar_wait(&empty_bar[s], ph ^ 1)) {
            tc::report_timeout(p.status, kStatusProducerTimeout);
            ok = false;
            break;
          }
          unsigned char *a_dst = smem + s * L::kStageBytes;
          unsigned char *b_dst = a_dst + L::kABytes;
          tc::mbar_expect_tx(&full_bar[s], L::kStageBytes);
          tc::tma_load_2d(a_dst, &tmap_a, &full_bar[s], kb * kBK, m0);
          tc::tma_load_2d(b_dst, &tmap_b, &full_bar[s], kb * kBK, n0);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = tc::instr_desc(2u, A_SIGNED ? 1u : 0u, 1u, kBM, BN);
      uint32_t it = 0;
      bool ok = true;
      int local = 0;
      for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++local) {
        const uint32_t buf = (uint32_t)local % NBUF;
        const uint32_t use = (uint32_t)local / NBUF;  // how many times this buffer was used before
        if (ok && !tc::mbar_wait(&tmem_empty[buf], (use & 1) ^ 1)) {
          tc::report_timeout(p.status, kStatusMmaTimeout);
          ok = false;
        }
        tc::fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * (MH * BN);
        for (int kb = 0; kb < num_kb && ok; ++kb, ++it) {
          const uint32_t s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!tc::mbar_wait(&full_bar[s], ph)) {
            tc::report_timeout(p.status, kStatusMmaTimeout);
            ok = false;
            break;
          }
          tc::fence_after_sync();
          const uint32_t a_addr = smem_u32(smem + s * L::kStageBytes);
          const uint64_t a_desc = tc::smem_desc_k_sw128(a_addr);
          const uint64_t b_desc = tc::smem_desc_k_sw128(a_addr + L::kABytes);
#pragma unroll
          for (int h = 0; h < MH; ++h) {
#pragma unroll
            for (int k = 0; k < kBK / 32; ++k) {
              // 32 bytes of K per instruction: advance both start addresses by 32 >> 4 = 2; the second
              // 128-row half of the A stage starts 128 * 128 bytes further (>> 4 = 1024)
              tc::mma_i8(d_tmem + h * BN, a_desc + h * (kBM * kBK / 16) + 2 * k, b_desc + 2 * k, idesc,
                         (kb > 0 || k > 0) ? 1u : 0u);
            }
          }
          tc::mma_commit(&empty_bar[s]);
        }
        // Arrive on the accumulator barrier in every case so that the epilogue never waits for a
        // commit that will not come; after a timeout the result is garbage but the kernel ends.
        tc::mma_commit(&tmem_full[buf]);
      }
    }
  } else {
    // ---------------- epilogue warps (2..9) ----------------
    grid_dependency_wait();                    // activation scales / zero points come from the preceding kernel
    const int et = threadIdx.x - 64;           // 0..255
    const int quarter = warp & 3;              // TMEM lanes this warp may read: 32*quarter ..
    const int parity = (warp - 2) >> 2;        // which 32-column chunks this warp takes
    const int row = quarter * 32 + lane;
    // a single unary post-op is resolved once, outside the element loops
    int unary = -1;
    if (p.post.n_ops == 0) unary = ZT_POST_NONE;
    else if (p.post.n_ops == 1 && p.post.ids[0] < ZT_POST_MUL) unary = p.post.ids[0];
    OutQuant out_quant{0.f, 0.f, 0.f, 0.f};
    if (EPI == kEpiStatic) out_quant = load_out_quant(p.out_scale, p.out_zp, p.y_dtype);
    int local = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++local) {
      const int m0 = (tile % p.m_tiles) * (MH * kBM);
      const int n0 = (tile / p.m_tiles) * BN;
      const uint32_t buf = (uint32_t)local % NBUF;
      const uint32_t use = (uint32_t)local / NBUF;
      float *v_wscale = s_vec + (local & 1) * 3 * BN;
      float *v_bias = v_wscale + BN;
      int32_t *v_rowsum = reinterpret_cast<int32_t *>(v_bias + BN);
      if (EPI != kEpiS32) {
        for (int j = et; j < BN; j += kEpiWarps * 32) {
          const int n = n0 + j;
          const bool in = n < p.N;
          v_wscale[j] = in ? load_as_float(p.w_scale, (EPI == kEpiStatic && p.w_scale_per_tensor) ? 0 : n, p.w_scale_dtype) : 0.f;
          v_bias[j] = (in && p.bias) ? load_as_float(p.bias, n, p.bias_dtype) : 0.f;
          v_rowsum[j] = (in && p.w_rowsum) ? p.w_rowsum[n] : 0;
        }
      }
      // All epilogue threads: the vectors of this tile are visible, and everybody has finished
      // reading the vectors of the tile two back (same buffer).
      asm volatile("bar.sync 1, %0;" ::"n"(kEpiWarps * 32) : "memory");
      if (ok && !tc::mbar_wait(&tmem_full[buf], use & 1)) {
        tc::report_timeout(p.status, kStatusEpilogueTimeout);
        ok = false;
      }
      tc::fence_after_sync();
#pragma unroll 1
      for (int h = 0; h < MH; ++h) {
        const int m = m0 + h * kBM + row;
        const bool row_ok = m < p.M;
        float s_m = 0.f;
        int zp_m = 0;
        if (EPI == kEpiLinear && row_ok) {
          s_m = p.src_scale[m];
          if (p.src_zp) zp_m = p.src_zp[m];
        }
        if (EPI == kEpiStatic) {                     // one scale and zero point for the whole tensor
          s_m = p.src_scale[0];
          if (p.src_zp) zp_m = p.src_zp[0];
        }
        const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + (buf * MH + h) * BN;
#pragma unroll 1
        for (int c = parity * 32; c < BN; c += 64) {
          uint32_t r[32];
          tc::tmem_ld_32x32b_x32(t_row + c, r);
          tc::tmem_ld_wait();
          const int nb = n0 + c;
          if (row_ok && nb < p.N) {
            if (EPI == kEpiS32) {
              int32_t *dst = reinterpret_cast<int32_t *>(p.y) + (size_t)m * p.N + nb;
              if (nb + 32 <= p.N && (p.N & 3) == 0) {
#pragma unroll
                for (int j = 0; j < 32; j += 4)
                  *reinterpret_cast<uint4 *>(dst + j) = make_uint4(r[j], r[j + 1], r[j + 2], r[j + 3]);
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  if (nb + j < p.N) dst[j] = (int32_t)r[j];
              }
            } else if (EPI == kEpiStatic) {
              finish_chunk_static(p, r, s_m, zp_m, v_wscale + c, v_bias + c, v_rowsum + c, out_quant, m, nb);
            } else {
              const float *ws = v_wscale + c, *bs = v_bias + c;
              const int32_t *rs = v_rowsum + c;
              switch (unary) {
                case ZT_POST_NONE: finish_chunk<ZT_POST_NONE>(p, r, s_m, zp_m, ws, bs, rs, m, nb); break;
                case ZT_POST_RELU: finish_chunk<ZT_POST_RELU>(p, r, s_m, zp_m, ws, bs, rs, m, nb); break;
                case ZT_POST_SILU: finish_chunk<ZT_POST_SILU>(p, r, s_m, zp_m, ws, bs, rs, m, nb); break;
                case ZT_POST_GELU_TANH: finish_chunk<ZT_POST_GELU_TANH>(p, r, s_m, zp_m, ws, bs, rs, m, nb); break;
                case ZT_POST_GELU_ERF: finish_chunk<ZT_POST_GELU_ERF>(p, r, s_m, zp_m, ws, bs, rs, m, nb); break;
                default: finish_chunk<-1>(p, r, s_m, zp_m, ws, bs, rs, m, nb); break;
              }
            }
          }
          __syncwarp();  // the next tcgen05.ld is warp-collective
        }
      }
      // this warp has drained its part of the accumulator buffer
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

// ---- launch of one configuration ---------------------------------------------------------------------
template <int MH, int BN, int STAGES, int NBUF, int EPI, bool A_SIGNED>
int launch_cfg(const CUtensorMap &ta, const CUtensorMap &tb, const TcParams &p, cudaStream_t st) {
  using L = SmemLayout<MH, BN, STAGES>;
  static_assert(L::kTotal <= 227 * 1024, "stage ring exceeds shared memory");
  auto kern = int8_tcgen05_kernel<MH, BN, STAGES, NBUF, EPI, A_SIGNED>;
  static PerDeviceOnce configured;
  if (int rc_cfg = allow_dynamic_smem(configured, kern, L::kTotal)) return rc_cfg;
  TcParams q = p;
  q.m_tiles = ceil_div(p.M, MH * kBM);
  q.n_tiles = ceil_div(p.N, BN);
  const int tiles = q.m_tiles * q.n_tiles;
  const int sms = sm_count();
  dim3 grid((unsigned)(tiles < sms ? tiles : sms));
  ZT_CUDA_OK(launch_overlapped(kern, grid, dim3(kThreads), (size_t)L::kTotal, st, ta, tb, q));
  return launch_status("int8_tcgen05_kernel");
}

template <int MH, int BN, int STAGES, int NBUF>
int launch_bn(const CUtensorMap &ta, const CUtensorMap &tb, const TcParams &p, int epi, bool a_signed, cudaStream_t st) {
  if (epi == kEpiS32)
    return a_signed ? launch_cfg<MH, BN, STAGES, NBUF, kEpiS32, true>(ta, tb, p, st)
                    : launch_cfg<MH, BN, STAGES, NBUF, kEpiS32, false>(ta, tb, p, st);
  if (epi == kEpiStatic)
    return a_signed ? launch_cfg<MH, BN, STAGES, NBUF, kEpiStatic, true>(ta, tb, p, st)
                    : launch_cfg<MH, BN, STAGES, NBUF, kEpiStatic, false>(ta, tb, p, st);
  return a_signed ? launch_cfg<MH, BN, STAGES, NBUF, kEpiLinear, true>(ta, tb, p, st)
                  : launch_cfg<MH, BN, STAGES, NBUF, kEpiLinear, false>(ta, tb, p, st);
}

// CTA pairs (tcgen05.mma.cta_group::2): 512 x bn tiles, each CTA loads half of every weight block.  Linear
// epilogue only.  Own translation unit (int8_tcgen05_pair.cu).
bool int8_pair_supported(int64_t M, int bn);
int launch_pair(int bn, const Int8GemmArgs &a, const TcParams &p, bool a_signed, cudaStream_t st);

// 256-row tiles, instantiated in their own translation unit.
int launch_mh2(int bn, const CUtensorMap &ta, const CUtensorMap &tb, const TcParams &p, int epi, bool a_signed,
               cudaStream_t st);

}  // namespace i8tc
}  // namespace zt
