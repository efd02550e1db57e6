// int8 GEMM on CTA pairs: tcgen05.mma.cta_group::2.
//
// The one-CTA kernel (int8_tcgen05.cuh) is bound by the operand bytes an SM can pull from L2: with a
// 256 x 160 tile it needs 32 KB of activations and 20 KB of weights per 128 bytes of K.  Here two CTAs of a
// cluster share every weight block: the pair computes 512 rows x BN columns, each CTA holds 256 of the rows
// (two 128-row accumulators in its own tensor memory) and loads only half of the weight block (BN/2 rows);
// one MMA instruction of the leader CTA multiplies 128 rows of either CTA by the whole block, reading the
// other half of it from the peer's shared memory.  Per CTA and k-block that is 32 KB + BN/2 * 128 bytes
// instead of 32 KB + BN * 128.
//
// Every CTA issues its own TMA loads into its own shared memory; nothing is multicast on the load side.  What
// crosses the pair:
//   * both CTAs' loads of a stage count their bytes on the leader's "stage full" barrier (the peer's loads name
//     it by its cluster address), so the leader's MMA thread waits on one barrier per stage;
//   * the leader's tcgen05.commit arrives on the stage's empty barrier and on the accumulator barrier of
//     both CTAs (commit with a CTA mask);
//   * the peer's epilogue warps tell the leader that they have drained the accumulator (remote arrive);
//   * a cluster barrier before tensor memory is freed, because the leader's MMAs read the peer's shared
//     memory and write the peer's tensor memory until the very end.
// All waits are bounded as in the one-CTA kernel.
#include <mutex>
#include <unordered_map>

#include "int8_tcgen05.cuh"

namespace zt {
namespace i8tc {

namespace {

constexpr int kPairRows = 2 * kBM;   // rows per CTA (two accumulators)

template <int BN, int STAGES>
struct PairLayout {
  static constexpr int kABytes = kPairRows * kBK;          // 32 KB
  static constexpr int kBBytes = (BN / 2) * kBK;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kTileBytes = STAGES * kStageBytes;
  static constexpr int kVecBytes = 3 * BN * 4;              // w_scale, bias, rowsum of the tile
  static constexpr int kBarBytes = (2 * STAGES + 2) * 8 + 8;
  static constexpr int kTotal = kTileBytes + kVecBytes + kBarBytes + 1024;
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_to_cta(const void *smem_ptr, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(smem_ptr)), "r"(rank));
  return remote;
}
__device__ __forceinline__ void remote_arrive(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t *slot_in_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot_in_smem)), "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void mma_i8_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on the barrier at this shared-memory offset in both CTAs of the pair once every MMA issued so far
// has completed.
__device__ __forceinline__ void mma_commit_pair(uint64_t *bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
                   smem_u32(bar)),
               "h"((uint16_t)3)
               : "memory");
}

// Tile load of this CTA into its own shared memory whose completion is counted on a barrier of the pair's leader
// (a shared::cluster address): the cta_group::2 form of the load exists for exactly this.  Not a multicast: the
// bytes land in one CTA only.
__device__ __forceinline__ void tma_load_2d_to_leader_bar(void *dst, const CUtensorMap *m, uint32_t bar_cluster_addr, int c0,
                                                          int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
      : "memory");
}

template <int BN, int STAGES, bool A_SIGNED>
__global__ void __launch_bounds__(kThreads, 1) int8_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap tmap_a,
                                                                        const __grid_constant__ CUtensorMap tmap_b,
                                                                        const TcParams p) {
  using L = PairLayout<BN, STAGES>;
  static_assert(2 * BN <= 512 && BN % 32 == 0, "two accumulators of BN columns must fit tensor memory");
  extern __shared__ unsigned char smem_dyn[];
  unsigned char *smem = smem_dyn + ((1024u - (smem_u32(smem_dyn) & 1023u)) & 1023u);
  float *s_vec = reinterpret_cast<float *>(smem + L::kTileBytes);  // [3][BN]
  uint64_t *full_bar = reinterpret_cast<uint64_t *>(smem + L::kTileBytes + L::kVecBytes);   // used in the leader only
  uint64_t *empty_bar = full_bar + STAGES;
  uint64_t *tmem_full = empty_bar + STAGES;    // accumulators complete (both CTAs, by the leader's commit)
  uint64_t *tmem_empty = tmem_full + 1;        // leader only: both CTAs' epilogue warps have drained them
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(tmem_empty + 1);

  constexpr uint32_t kTmemCols = 2 * BN <= 128 ? 128 : 2 * BN <= 256 ? 256 : 512;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();          // 0: leader (issues the MMAs), 1: peer
  const int num_kb = (p.K + kBK - 1) / kBK;
  const int total_tiles = p.m_tiles * p.n_tiles;    // pair tiles of 512 x BN
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    tc::prefetch_tensormap(&tmap_a);
    tc::prefetch_tensormap(&tmap_b);
    for (int s = 0; s < STAGES; ++s) {
      tc::mbar_init(&full_bar[s], 1);
      tc::mbar_init(&empty_bar[s], 1);
    }
    tc::mbar_init(tmem_full, 1);
    tc::mbar_init(tmem_empty, 2 * kEpiWarps);
    tc::mbar_fence_init();
  }
  __syncthreads();
  cluster_sync_all();   // both CTAs' barriers exist before anything arrives on them from the other side
  if (warp == 1) tmem_alloc_pair(tmem_slot, kTmemCols);
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  grid_launch_dependents();

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs): own 256 activation rows, own half of the weight block ----------------
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      uint32_t leader_full[STAGES];   // the leader's "stage full" barriers as cluster addresses
#pragma unroll
      for (int s = 0; s < STAGES; ++s) leader_full[s] = map_to_cta(&full_bar[s], 0);
      // First pass over the ring: the weight blocks do not depend on the preceding kernel, so they are requested
      // before the dependency wait and the activation tiles of the same stages after it.
      int pre = 0;
      if (pair < total_tiles) {
        const int m0 = (pair % p.m_tiles) * (2 * kPairRows) + (int)rank * kPairRows;
        const int n0 = (pair / p.m_tiles) * BN + (int)rank * (BN / 2);
        pre = num_kb < STAGES ? num_kb : STAGES;
#pragma unroll
        for (int kb = 0; kb < STAGES; ++kb)
          if (kb < pre) {
            if (rank == 0) tc::mbar_expect_tx(&full_bar[kb], 2 * L::kStageBytes);   // both CTAs' bytes
            tma_load_2d_to_leader_bar(smem + kb * L::kStageBytes + L::kABytes, &tmap_b, leader_full[kb], kb * kBK, n0);
          }
        grid_dependency_wait();
#pragma unroll
        for (int kb = 0; kb < STAGES; ++kb)
          if (kb < pre) tma_load_2d_to_leader_bar(smem + kb * L::kStageBytes, &tmap_a, leader_full[kb], kb * kBK, m0);
        it = (uint32_t)pre;
      }
      uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
      for (int tile = pair; tile < total_tiles && ok; tile += num_pairs) {
        const int m0 = (tile % p.m_tiles) * (2 * kPairRows) + (int)rank * kPairRows;
        const int n0 = (tile / p.m_tiles) * BN + (int)rank * (BN / 2);
        for (int kb = (tile == pair ? pre : 0); kb < num_kb; ++kb) {
          if (!tc::mbar_wait(&empty_bar[s], ph ^ 1)) {
            tc::report_timeout(p.status, kStatusProducerTimeout);
            ok = false;
            break;
          }
          unsigned char *a_dst = smem + s * L::kStageBytes;
          uint32_t bar = leader_full[0];
#pragma unroll
          for (int j = 1; j < STAGES; ++j)
            if ((uint32_t)j == s) bar = leader_full[j];
          if (rank == 0) tc::mbar_expect_tx(&full_bar[s], 2 * L::kStageBytes);
          tma_load_2d_to_leader_bar(a_dst, &tmap_a, bar, kb * kBK, m0);
          tma_load_2d_to_leader_bar(a_dst + L::kABytes, &tmap_b, bar, kb * kBK, n0);
          if (++s == STAGES) {
            s = 0;
            ph ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (rank == 0) {
      // ---------------- MMA issuer (leader) ----------------
      if (lane == 0) {
        constexpr uint32_t idesc = tc::instr_desc(2u, A_SIGNED ? 1u : 0u, 1u, 2 * kBM, BN);   // M = 256 over the pair
        uint32_t it = 0;
        bool ok = true;
        int local = 0;
        for (int tile = pair; tile < total_tiles; tile += num_pairs, ++local) {
          if (local > 0 && ok && !tc::mbar_wait(tmem_empty, (uint32_t)(local - 1) & 1)) {
            tc::report_timeout(p.status, kStatusMmaTimeout);
            ok = false;
          }
          tc::fence_after_sync();
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
            for (int h = 0; h < 2; ++h) {
#pragma unroll
              for (int k = 0; k < kBK / 32; ++k)
                mma_i8_pair(tmem_base + h * BN, a_desc + h * (kBM * kBK / 16) + 2 * k, b_desc + 2 * k, idesc,
                            (kb > 0 || k > 0) ? 1u : 0u);
            }
            mma_commit_pair(&empty_bar[s]);
          }
          mma_commit_pair(tmem_full);
        }
      }
    }
  } else {
    // ---------------- epilogue warps (both CTAs): own 256 rows ----------------
    grid_dependency_wait();
    const int et = threadIdx.x - 64;
    const int quarter = warp & 3;
    const int parity = (warp - 2) >> 2;
    const int row = quarter * 32 + lane;
    int unary = -1;
    if (p.post.n_ops == 0) unary = ZT_POST_NONE;
    else if (p.post.n_ops == 1 && p.post.ids[0] < ZT_POST_MUL) unary = p.post.ids[0];
    float *v_wscale = s_vec, *v_bias = s_vec + BN;
    int32_t *v_rowsum = reinterpret_cast<int32_t *>(s_vec + 2 * BN);
    const uint32_t leader_empty = map_to_cta(tmem_empty, 0);
    int local = 0;
    bool ok = true;
    for (int tile = pair; tile < total_tiles; tile += num_pairs, ++local) {
      const int m0 = (tile % p.m_tiles) * (2 * kPairRows) + (int)rank * kPairRows;
      const int n0 = (tile / p.m_tiles) * BN;
      asm volatile("bar.sync 1, %0;" ::"n"(kEpiWarps * 32) : "memory");   // the previous tile's vectors are no longer read
      for (int j = et; j < BN; j += kEpiWarps * 32) {
        const int n = n0 + j;
        const bool in = n < p.N;
        v_wscale[j] = in ? load_as_float(p.w_scale, n, p.w_scale_dtype) : 0.f;
        v_bias[j] = (in && p.bias) ? load_as_float(p.bias, n, p.bias_dtype) : 0.f;
        v_rowsum[j] = (in && p.w_rowsum) ? p.w_rowsum[n] : 0;
      }
      asm volatile("bar.sync 1, %0;" ::"n"(kEpiWarps * 32) : "memory");
      if (ok && !tc::mbar_wait(tmem_full, (uint32_t)local & 1)) {
        tc::report_timeout(p.status, kStatusEpilogueTimeout);
        ok = false;
      }
      tc::fence_after_sync();
#pragma unroll 1
      for (int h = 0; h < 2; ++h) {
        const int m = m0 + h * kBM + row;
        const bool row_ok = m < p.M;
        float s_m = 0.f;
        int zp_m = 0;
        if (row_ok) {
          s_m = p.src_scale[m];
          if (p.src_zp) zp_m = p.src_zp[m];
        }
        const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + h * BN;
#pragma unroll 1
        for (int c = parity * 32; c < BN; c += 64) {
          uint32_t r[32];
          tc::tmem_ld_32x32b_x32(t_row + c, r);
          tc::tmem_ld_wait();
          const int nb = n0 + c;
          if (row_ok && nb < p.N) {
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
          __syncwarp();
        }
      }
      tc::fence_before_sync();
      __syncwarp();
      if (lane == 0) remote_arrive(leader_empty);   // the leader's barrier counts the warps of both CTAs
    }
  }

  tc::fence_before_sync();
  __syncthreads();
  cluster_sync_all();   // the leader's MMAs touch the peer's shared and tensor memory until here
  if (warp == 1) {
    tc::fence_after_sync();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

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
int cached_map(CUtensorMap *out, const void *ptr, uint64_t inner, uint64_t rows, uint32_t box_rows) {
  static std::mutex mu;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  const MapKey key{ptr, inner, rows, box_rows};
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it != cache.end()) {
    *out = it->second;
    return ZT_SUCCESS;
  }
  int rc = make_tensor_map_2d(out, ptr, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, inner, rows, inner, kBK, box_rows);
  if (rc != ZT_SUCCESS) return rc;
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, *out);
  return ZT_SUCCESS;
}

template <int BN, int STAGES, bool A_SIGNED>
int launch_pair_cfg(const Int8GemmArgs &a, const TcParams &p0, cudaStream_t st) {
  using L = PairLayout<BN, STAGES>;
  static_assert(L::kTotal <= 227 * 1024, "stage ring exceeds shared memory");
  auto kern = int8_tcgen05_pair_kernel<BN, STAGES, A_SIGNED>;
  static PerDeviceOnce configured;
  if (int rc = allow_dynamic_smem(configured, kern, L::kTotal)) return rc;
  CUtensorMap ta, tb;
  int rc = cached_map(&ta, a.q, (uint64_t)a.K, (uint64_t)a.M, (uint32_t)kPairRows);
  if (rc != ZT_SUCCESS) return rc;
  rc = cached_map(&tb, a.w, (uint64_t)a.K, (uint64_t)a.N, (uint32_t)(BN / 2));
  if (rc != ZT_SUCCESS) return rc;
  TcParams p = p0;
  p.m_tiles = ceil_div(p.M, 2 * kPairRows);
  p.n_tiles = ceil_div(p.N, BN);
  const int tiles = p.m_tiles * p.n_tiles;
  const int pairs = sm_count() / 2;
  const dim3 grid((unsigned)(2 * (tiles < pairs ? tiles : pairs)));
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = (size_t)L::kTotal;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = overlap_launches() ? 2 : 1;
  ZT_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, ta, tb, p));
  return launch_status("int8_tcgen05_pair_kernel");
}

}  // namespace

bool int8_pair_supported(int64_t M, int bn) { return M > kPairRows && (bn == 128 || bn == 160 || bn == 192 || bn == 256); }

// The epilogue form only (scale, bias, post-ops); the raw int32 form stays with the one-CTA kernel.
int launch_pair(int bn, const Int8GemmArgs &a, const TcParams &p, bool a_signed, cudaStream_t st) {
  switch (bn) {
    case 128: return a_signed ? launch_pair_cfg<128, 5, true>(a, p, st) : launch_pair_cfg<128, 5, false>(a, p, st);
    case 160: return a_signed ? launch_pair_cfg<160, 5, true>(a, p, st) : launch_pair_cfg<160, 5, false>(a, p, st);
    case 192: return a_signed ? launch_pair_cfg<192, 5, true>(a, p, st) : launch_pair_cfg<192, 5, false>(a, p, st);
    case 256: return a_signed ? launch_pair_cfg<256, 4, true>(a, p, st) : launch_pair_cfg<256, 4, false>(a, p, st);
    default: break;
  }
  set_error("int8_tcgen05_launch: unsupported pair tile width %d", bn);
  return ZT_UNSUPPORTED;
}

}  // namespace i8tc
}  // namespace zt
