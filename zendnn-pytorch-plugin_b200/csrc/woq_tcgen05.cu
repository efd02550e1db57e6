// Weight-only int4 linear for M > 16 (prefill and large decode batches) on tcgen05 tensor cores.
//
//   Y[M,N] = post_ops( X[M,K] . dq(Wq)[K,N] + bias ),   dq = bf16(q*s)  or  bf16((q-8)*s + z)
//
// The weight is the 128-row operand of the MMA (UMMA M = 128 output columns n), the activations are
// the other operand (UMMA N = BT tokens, up to 256), so a CTA dequantises a 128 x 64 block of weights
// per k-block and reuses it for up to 256 tokens.  One persistent CTA per SM walks over
// (128 columns) x (BT tokens) tiles; tiles that share a weight block are adjacent in the order.
//
//   warp 0        TMA producer of the activation tiles (plain per-CTA loads)
//   warp 1        TMEM allocation, tcgen05.mma.kind::f16 issue (bf16 x bf16 -> fp32), TMEM release
//   warps 2..17   dequantisation in four teams (a thread converts one weight row of a k-block): shared-memory
//                 loads of packed nibbles and of the group's scale / zero point from the chunk ring, nibble ->
//                 bf16 with lop3, exact subtraction of the encoding bias, multiplication by the scale in bf16x2
//                 arithmetic, byte-permute into k order, 16-byte stores into the canonical K-major
//                 128-byte-swizzled operand layout, fence.proxy.async, mbarrier arrive
//   warps 18..21  epilogue: tcgen05.ld (lane = output column n, register j = token), transpose
//                 through shared memory so that stores run along n, bias + post-ops, bf16 stores
//   warp 22       TMA producer of the packed weights in chunks of four k-blocks (128 rows x 128 B, 128-byte
//                 swizzle) with their scales / zero points, into a ring of their own, several chunks ahead and
//                 without ever waiting for the preceding kernel
//   warp 23       second MMA issuer (token tiles up to 128): alternate ring positions, own accumulator
//
// Grouped mode (mixture-of-experts): the rows of X are sorted by expert, a device-side table lists the
// row tiles {expert, first row, valid rows}, and each tile uses its expert's slice of the stacked
// weight and scale tensors; the number of tiles is read from device memory, so no host
// synchronisation is needed between routing and the GEMM.
//
// Conversion teams.  One k-block's conversion is a chain of dependent steps (wait for the stage, shared-memory
// load, ALU, shared-memory store, proxy fence, barrier arrive) whose latency, about 1200 cycles, is several
// times its issue time; with all sixteen warps on the same k-block the kernel converted one k-block per such
// latency.  For token tiles up to 128 the sixteen warps therefore form four teams of four warps, team t
// taking the ring positions congruent to t modulo 4 (a thread converts one whole weight row of the k-block:
// 32 packed bytes in, 128 bytes of bf16 out), so four k-blocks are in flight at once.  This is sound because
// the number of stages is a multiple of the number of teams: a stage is always converted by the same team,
// so a team sees every phase of the stage barriers it waits on.  (With a stage count that is not, consecutive
// uses of a stage belong to different teams, a team can reach its wait two uses ahead of the barrier, and
// an mbarrier parity wait that far ahead passes at once.)  A stage count that is not a multiple of four falls back to
// all sixteen warps converting every k-block together.
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
constexpr int kDqWarps = 16;
constexpr int kWPT = 32 / kDqWarps;   // packed words per dequantisation thread and k-block (4 with 8 warps, 2 with 16)
constexpr int kEpiWarps = 4;
constexpr int kAuxWarps = 2;        // packed-weight producer, second MMA issuer (24 warps leave 80 registers a thread)
constexpr int kThreads = 64 + 32 * (kDqWarps + kEpiWarps + kAuxWarps);
constexpr int kPackedProducer = 2 + kDqWarps + kEpiWarps;   // warp index
constexpr int kIssuerB = kPackedProducer + 1;
constexpr int kEpiRowStride = 36;  // floats; 144 bytes keeps 16-byte alignment and spreads banks
constexpr int kChunkKB = 4;        // k-blocks per packed-weight chunk: 4 x 32 B = one 128-byte row
constexpr int kChunkBytes = kBN * 128;
// per packed chunk: up to two groups x 128 columns of fp32 scales (1 KB), then the same for zero points
constexpr int kScaleSlotBytes = 2048;
constexpr int kZeroSlotOffset = 1024;

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
  // grouped mode (g_count != nullptr)
  const int *g_count;     // number of row tiles
  const int4 *g_tiles;    // per row tile: {expert, first row, valid rows, 0}
  long long s_estride;    // elements between two experts' scale tables
  // split K (dense mode, layers with fewer tiles than SMs): every tile is cut into ksplit work items of kps
  // k-blocks each (kps a multiple of the packed chunk, ksplit * kps = K / 64); the items write fp32 partial
  // sums [ksplit][M][N] that a second kernel adds.  ksplit = 1: kps = K / 64, partial unused.
  int ksplit, kps;
  float *partial;
  // Scales (and zero points) staged in shared memory with every packed chunk: groups per chunk (1 or 2; 0 = the
  // conversion threads fetch them from global memory), log2 of the group size, groups per expert.
  int staged_gpc, gs_log2, groups;
  int single_issuer;   // host side: launch the one-issuer form
#ifdef ZT_TCPROF
  TimelineSink prof;   // 4 records of 8 counters per CTA: conversion team 0, MMA issuer, producer, epilogue warp 0
  int dbg;             // ZENTORCH_B200_TCDBG: 1 no MMA issue, 2 no activation loads, 4 no conversion arithmetic (timing only, results are garbage)
#endif
};

struct TileInfo {
  int m0, rows, n0, expert;
  int kb0, ks;   // first k-block and index of the K slice (0, 0 without split K)
};

__device__ __forceinline__ TileInfo decode_tile(const TcParams &p, int tile, int n_mt, int bt) {
  TileInfo t;
  t.ks = p.ksplit > 1 ? tile % p.ksplit : 0;
  t.kb0 = t.ks * p.kps;
  if (p.ksplit > 1) tile /= p.ksplit;
  const int mt = tile % n_mt;
  t.n0 = (tile / n_mt) * kBN;
  if (p.g_count) {
    const int4 g = p.g_tiles[mt];
    t.expert = g.x;
    t.m0 = g.y;
    t.rows = g.z;
  } else {
    t.expert = 0;
    t.m0 = mt * bt;
    t.rows = min(bt, p.M - t.m0);
  }
  return t;
}

// Three rings: STAGES converted weight blocks (bf16, 16 KB each), XSTAGES activation tiles, PSTAGES packed chunks.
// The activation tiles have a ring of their own so that they can be requested many k-blocks ahead: a tile
// load takes about a microsecond, and a slot that could only be refilled once its weight stage was free again
// would limit the kernel to (stages / that latency) k-blocks per second.
template <int BT, int STAGES, int XSTAGES, int PSTAGES>
struct SmemLayout {
  static constexpr int kWBytes = kBN * 128;
  static constexpr int kXBytes = BT * 128;
  static constexpr int kWRingBytes = STAGES * kWBytes;
  static constexpr int kTileBytes = kWRingBytes + XSTAGES * kXBytes;
  static constexpr int kPackedBytes = PSTAGES * kChunkBytes;
  static constexpr int kScaleBytes = PSTAGES * kScaleSlotBytes;   // scales / zero points of every packed chunk
  static constexpr int kEpiBytes = kEpiWarps * 32 * kEpiRowStride * 4;
  static constexpr int kBarBytes = (2 * STAGES + 2 * XSTAGES + 2 * PSTAGES + 4) * 8 + 8;
  static constexpr int kTotal = kTileBytes + kPackedBytes + kScaleBytes + kEpiBytes + kBarBytes + 1024;
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
  float s, z;
};

// Adds the K slices of a split-K run: y = post_ops(sum_s partial[s] + bias), four columns per thread.
__global__ void __launch_bounds__(256) woq_splitk_reduce_kernel(const float *__restrict__ partial, int ksplit, int M, int N,
                                                                const void *__restrict__ bias, int bias_dtype,
                                                                PostOpsDev post, __nv_bfloat16 *__restrict__ y) {
  grid_launch_dependents();
  grid_dependency_wait();
  const int64_t quad = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;   // N % 4 == 0 here
  const int64_t base = quad * 4;
  if (base >= (int64_t)M * N) return;
  const int n = (int)(base % N);
  float v[4] = {0.f, 0.f, 0.f, 0.f};
  for (int s = 0; s < ksplit; ++s) {
    const float4 t = __ldcg(reinterpret_cast<const float4 *>(partial + (int64_t)s * M * N + base));
    v[0] += t.x;
    v[1] += t.y;
    v[2] += t.z;
    v[3] += t.w;
  }
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    if (bias) v[e] += load_as_float(bias, n + e, bias_dtype);
    v[e] = apply_post_ops(v[e], post, base + e, ZT_BF16);
  }
  __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]);
  __nv_bfloat162 hi = __floats2bfloat162_rn(v[2], v[3]);
  uint2 o;
  o.x = *reinterpret_cast<uint32_t *>(&lo);
  o.y = *reinterpret_cast<uint32_t *>(&hi);
  *reinterpret_cast<uint2 *>(y + base) = o;
}

#ifdef ZT_TCPROF
#define TCP_T0() const long long tcp_t0 = clock64()
#define TCP_ADD(acc) acc += (tcp_warm ? clock64() - tcp_t0 : 0)
#define TCP_DBG(bit) ((p.dbg & (bit)) != 0)
#else
#define TCP_T0()
#define TCP_ADD(acc)
#define TCP_DBG(bit) false
#endif
// Waits of the two pacing threads poll; the conversion teams and the epilogue warps, which wait most of the time,
// let the hardware suspend them between polls (fewer barrier reads competing with the pacing threads).
#define TC_WAIT1(bar, par) tc::mbar_wait(bar, par)
#define TC_WAITN(bar, par) tc::mbar_wait_suspend(bar, par)
constexpr int kTeams = 4;                      // conversion teams (token tiles up to 128)
constexpr int kTeamWarps = kDqWarps / kTeams;  // 4 warps = 128 threads = one weight row per thread

// NI = 2: two MMA issuers take alternate ring positions, each issuer summing its
// k-blocks into an accumulator of its own; the epilogue adds the two.  One thread issuing a block's MMAs, its two
// commits and waiting on its two barriers needs about a thousand cycles per block whatever the tile, which is
// what paced the kernel with a single issuer.  The accumulators are double buffered when NI * 2 * BT columns fit
// tensor memory (BT <= 128), single buffered otherwise.
template <int BT, int STAGES, int XSTAGES, int PSTAGES, bool ASYM, int NI>
__global__ void __launch_bounds__(kThreads, 1) woq_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_x,
                                                                  const __grid_constant__ CUtensorMap tmap_w,
                                                                  const __grid_constant__ CUtensorMap tmap_s,
                                                                  const __grid_constant__ CUtensorMap tmap_z,
                                                                  const TcParams p) {
  using L = SmemLayout<BT, STAGES, XSTAGES, PSTAGES>;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char *smem = smem_dyn + ((1024u - (smem_u32(smem_dyn) & 1023u)) & 1023u);
  unsigned char *packed = smem + L::kTileBytes;  // ring of packed-weight chunks (1024-byte aligned)
  unsigned char *sc_ring = smem + L::kTileBytes + L::kPackedBytes;   // scales / zero points of the packed chunks
  float *epi_scratch = reinterpret_cast<float *>(sc_ring + L::kScaleBytes);
  uint64_t *full_x = reinterpret_cast<uint64_t *>(sc_ring + L::kScaleBytes + L::kEpiBytes);
  uint64_t *empty_x = full_x + XSTAGES;      // activation slot read by the MMAs of its k-block
  uint64_t *full_w = empty_x + XSTAGES;      // converted weight block written
  uint64_t *empty_bar = full_w + STAGES;     // converted weight block read by the MMAs of its k-block
  uint64_t *full_p = empty_bar + STAGES;     // packed chunk landed
  uint64_t *empty_p = full_p + PSTAGES;      // packed chunk consumed by all dequantisation warps
  uint64_t *tmem_full = empty_p + PSTAGES;   // [2]
  uint64_t *tmem_empty = tmem_full + 2;      // [2]
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(tmem_empty + 2);

  // With two issuers alternate ring positions belong to different threads.  A ring
  // of even length keeps every slot with one thread, which then waits on the slot's barriers strictly in order;
  // on an odd ring two threads would share a slot, one could reach its wait two phases ahead of the barrier,
  // and an mbarrier parity wait that far ahead passes at once.
  static_assert(NI == 1 || (STAGES % 2 == 0 && XSTAGES % 2 == 0), "two issuers need rings of even length");
  // When the activation ring is as long as the converted-weight ring, a ring position is one stage: its "full"
  // barrier counts the conversion team's warps and the activation producer (whose bulk copy adds the bytes), its
  // "free" barrier is waited on by both.  The MMA issuer then waits once and commits once per k-block instead
  // of twice -- barrier and tensor-core instructions are what a block's time is made of.
  constexpr bool kUnified = (XSTAGES == STAGES);
  constexpr int NBUF = (2 * NI * BT <= 512) ? 2 : 1;
  static_assert(NBUF * NI * BT <= 512, "accumulators exceed tensor memory");
  constexpr uint32_t kAccCols = NBUF * NI * BT;
  constexpr uint32_t kTmemCols = kAccCols <= 32 ? 32 : kAccCols <= 64 ? 64 : kAccCols <= 128 ? 128 : kAccCols <= 256 ? 256 : 512;
  constexpr bool kUseTeams = (STAGES % kTeams == 0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Programmatic dependent launch: packed weights and scales are read before the wait for the preceding
  // kernel, activations, partial sums and output after it.  The grouped form reads its tile list (made by the
  // routing kernels before it) at once, so it waits first.
  if (p.g_count) grid_dependency_wait();
  const int num_kb = p.kps;   // k-blocks per work item (all of K unless the host split it)
  const int num_chunks = (num_kb + kChunkKB - 1) / kChunkKB;
  const int n_mt = p.g_count ? *p.g_count : p.m_tiles;
  const int total_tiles = n_mt * p.n_tiles * p.ksplit;   // work items

  if (threadIdx.x == 0) {
    tc::prefetch_tensormap(&tmap_x);
    tc::prefetch_tensormap(&tmap_w);
    if (p.staged_gpc) {
      tc::prefetch_tensormap(&tmap_s);
      if (ASYM) tc::prefetch_tensormap(&tmap_z);
    }
    for (int s = 0; s < XSTAGES; ++s) {
      tc::mbar_init(&full_x[s], 1);
      tc::mbar_init(&empty_x[s], 1);
    }
    for (int s = 0; s < STAGES; ++s) {
      tc::mbar_init(&full_w[s], (kUseTeams ? kTeamWarps : kDqWarps) + (kUnified ? 1 : 0));
      tc::mbar_init(&empty_bar[s], 1);
    }
    for (int s = 0; s < PSTAGES; ++s) {
      tc::mbar_init(&full_p[s], 1);
      tc::mbar_init(&empty_p[s], kDqWarps);
    }
    for (int b = 0; b < 2; ++b) {
      tc::mbar_init(&tmem_full[b], NI);
      tc::mbar_init(&tmem_empty[b], kEpiWarps);
    }
    tc::mbar_fence_init();
  }
  if (warp == 1) tc::tmem_alloc(tmem_slot, kTmemCols);
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  grid_launch_dependents();

  if (warp == kPackedProducer) {
    // ---------------- TMA producer of the packed-weight chunks (with their scales / zero points) ----------------
    // Weights are constants: this thread never waits for the preceding kernel, it runs as far ahead as its ring
    // allows.  It has a thread of its own because every bulk-copy or barrier instruction costs the issuing thread
    // a few hundred cycles, and the activation producers are on the pipeline's critical path.
    if (lane == 0) {
      const uint32_t full_p0 = smem_u32(full_p), empty_p0 = smem_u32(empty_p);
      const uint32_t packed0 = smem_u32(packed), sc0 = smem_u32(sc_ring);
      const uint32_t chunk_tx = kChunkBytes + (ASYM ? 2u : 1u) * (uint32_t)p.staged_gpc * kBN * (p.scale_dtype == ZT_F32 ? 4u : 2u);
      uint32_t p_s = 0, p_ph = 1;          // ring slot and the parity of its "free" barrier
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        const TileInfo pt = decode_tile(p, tile, n_mt, BT);
        const int row = pt.expert * p.N + pt.n0;     // rows of the stacked weight: expert * N + n0
        for (int pchunk = 0; pchunk < num_chunks; ++pchunk) {
          if (!tc::mbar_wait_addr(empty_p0 + p_s * 8, p_ph)) {
            tc::report_timeout(p.status, kStatusProducerTimeout);
            ok = false;
            break;
          }
          const int chunk = pt.kb0 / kChunkKB + pchunk;            // chunk of 256 k within K
          const uint32_t bar = full_p0 + p_s * 8;
          tc::mbar_expect_tx_addr(bar, chunk_tx);
          tc::tma_load_2d_addr(packed0 + p_s * kChunkBytes, &tmap_w, bar, chunk * (kChunkKB * 8), row);   // 32 words per row
          if (p.staged_gpc) {
            // the chunk's groups x 128 columns of the scale table (rows = expert * groups + group)
            const int g0 = pt.expert * p.groups + ((chunk * (kChunkKB * kBK)) >> p.gs_log2);
            tc::tma_load_2d_addr(sc0 + p_s * kScaleSlotBytes, &tmap_s, bar, pt.n0, g0);
            if (ASYM) tc::tma_load_2d_addr(sc0 + p_s * kScaleSlotBytes + kZeroSlotOffset, &tmap_z, bar, pt.n0, g0);
          }
          if (++p_s == PSTAGES) {
            p_s = 0;
            p_ph ^= 1;
          }
        }
      }
    }
  } else if (warp == 0) {
    // ---------------- TMA producer of the activation tiles ----------------
    // Ring positions and phases as counters, shared-window addresses computed once.
    if (lane == 0) {
      const uint32_t which = 0u;
      // unified stages: the activation tile is announced on, and its slot freed by, the stage's barriers
      const uint32_t full_x0 = kUnified ? smem_u32(full_w) : smem_u32(full_x);
      const uint32_t empty_x0 = kUnified ? smem_u32(empty_bar) : smem_u32(empty_x);
      const uint32_t x0 = smem_u32(smem + L::kWRingBytes);
#ifdef ZT_TCPROF
      long long pc_total = 0, pc_emptyx = 0, pc_must = 0;
      bool tcp_warm = false;
#endif
      grid_dependency_wait();
      uint32_t x_s = 0, x_ph = 1, x_it = 0;   // slot, parity of its "free" barrier, ring position
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        const TileInfo t = decode_tile(p, tile, n_mt, BT);
        int kx = t.kb0 * kBK;
        for (int kb = 0; kb < num_kb; ++kb, kx += kBK, ++x_it) {
#ifdef ZT_TCPROF
          if (x_it == 8) { tcp_warm = true; pc_total = clock64(); }
#endif
          if (kUnified || !TCP_DBG(2)) {      // (the no-activation-loads knob has no unified form)
            {
              TCP_T0();
              const bool got = tc::mbar_wait_addr(empty_x0 + x_s * 8, x_ph);
              TCP_ADD(pc_emptyx);
              if (!got) {
                tc::report_timeout(p.status, kStatusProducerTimeout);
                ok = false;
                break;
              }
            }
            const uint32_t bar = full_x0 + x_s * 8;
            tc::mbar_expect_tx_addr(bar, L::kXBytes);
            tc::tma_load_2d_addr(x0 + x_s * L::kXBytes, &tmap_x, bar, kx, t.m0);
          }
          if (++x_s == XSTAGES) {
            x_s = 0;
            x_ph ^= 1;
          }
        }
      }
#ifdef ZT_TCPROF
      if (p.prof.base && which == 0) {
        unsigned long long *o = p.prof.base + ((size_t)blockIdx.x * 4 + 2) * kTimelineSlots;
        o[0] = clock64() - pc_total; o[1] = pc_emptyx; o[2] = pc_must; o[3] = x_it - 8;
      }
#endif
    }
  } else if (warp == 1 || (NI == 2 && warp == kIssuerB)) {
    // ---------------- MMA issuer(s) ----------------
    // A thread that paces the pipeline: ring positions and phases as counters, descriptors put together from a
    // constant high word and a start-address field that advances by a constant per stage.  With two issuers
    // each takes every other ring position and accumulates into its own columns of tensor memory.
    if (lane == 0) {
      const uint32_t which = warp == 1 ? 0u : 1u;
      constexpr uint32_t idesc = tc::instr_desc(1u, 1u, 1u, kBN, BT);  // f32 accumulate, bf16 x bf16
      bool ok = true;
      int local = 0;
#ifdef ZT_TCPROF
      long long mc_total = 0, mc_fullx = 0, mc_fullw = 0, mc_issue = 0, mc_tmem = 0, mc_commit = 0;
      bool tcp_warm = false;
      uint32_t it = 0;
#endif
      const uint64_t d0 = tc::smem_desc_k_sw128(0);
      const uint32_t desc_hi = (uint32_t)(d0 >> 32), desc_lo = (uint32_t)d0;
      const uint32_t w_field0 = desc_lo | ((smem_u32(smem) & 0x3FFFF) >> 4);
      const uint32_t x_field0 = desc_lo | ((smem_u32(smem + L::kWRingBytes) & 0x3FFFF) >> 4);
      const uint32_t full_x0 = smem_u32(full_x), empty_x0 = smem_u32(empty_x);
      const uint32_t full_w0 = smem_u32(full_w), empty_w0 = smem_u32(empty_bar);
      uint32_t w_s = 0, w_ph = 0, x_s = 0, x_ph = 0, pos = 0;
      for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++local) {
        const uint32_t buf = (uint32_t)local % NBUF;
        const uint32_t use = (uint32_t)local / NBUF;
        {
          TCP_T0();
          if (ok && !TC_WAIT1(&tmem_empty[buf], (use & 1) ^ 1)) {
            tc::report_timeout(p.status, kStatusMmaTimeout);
            ok = false;
          }
          TCP_ADD(mc_tmem);
        }
        tc::fence_after_sync();
        const uint32_t d_tmem = tmem_base + (buf * NI + which) * BT;
        bool first = true;                 // this issuer's first block of the tile overwrites its accumulator
        for (int kb = 0; kb < num_kb && ok; ++kb, ++pos) {
          if (NI == 1 || (pos & 1u) == which) {
#ifdef ZT_TCPROF
            if (it == 8) { tcp_warm = true; mc_total = clock64(); }
#endif
            bool got;
            {
              TCP_T0();
              got = kUnified || TCP_DBG(2) || tc::mbar_wait_addr(full_x0 + x_s * 8, x_ph);
              TCP_ADD(mc_fullx);
            }
            {
              TCP_T0();
              got = got && tc::mbar_wait_addr(full_w0 + w_s * 8, w_ph);
              TCP_ADD(mc_fullw);
            }
            if (!got) {
              tc::report_timeout(p.status, kStatusMmaTimeout);
              ok = false;
              break;
            }
#ifdef ZT_TCPROF
            if (p.prof.base && which == 0 && it == 16) p.prof.base[((size_t)blockIdx.x * 4 + 3) * kTimelineSlots + 1] = clock64();   // MMA issuer saw W(16)
#endif
            TCP_T0();
            tc::fence_after_sync();
            const uint32_t a_lo = w_field0 + w_s * (L::kWBytes >> 4);
            const uint32_t b_lo = x_field0 + x_s * (L::kXBytes >> 4);
            if (!TCP_DBG(1)) {
#pragma unroll
              for (int k = 0; k < kBK / 16; ++k) {
                // 16 bf16 = 32 bytes of K per instruction: the start-address fields advance by 32 >> 4 = 2
                tc::mma_f16(d_tmem, tc::smem_desc_from_words(a_lo + 2 * k, desc_hi), tc::smem_desc_from_words(b_lo + 2 * k, desc_hi),
                            idesc, (!first || k > 0) ? 1u : 0u);
              }
            }
            first = false;
#ifdef ZT_TCPROF
            const long long tcp_c0 = clock64();
            if (p.prof.base && which == 0 && it == 16) p.prof.base[((size_t)blockIdx.x * 4 + 3) * kTimelineSlots + 2] = tcp_c0;      // MMAs of block 16 issued
#endif
            tc::mma_commit_addr(empty_w0 + w_s * 8);   // both rings' slots are free once these MMAs have read them
            if (!kUnified && !TCP_DBG(2)) tc::mma_commit_addr(empty_x0 + x_s * 8);
            TCP_ADD(mc_issue);
#ifdef ZT_TCPROF
            if (tcp_warm) mc_commit += clock64() - tcp_c0;
#endif
          }
#ifdef ZT_TCPROF
          ++it;
#endif
          if (++w_s == STAGES) {
            w_s = 0;
            w_ph ^= 1;
          }
          if (++x_s == XSTAGES) {
            x_s = 0;
            x_ph ^= 1;
          }
        }
        tc::mma_commit(&tmem_full[buf]);     // one arrival per issuer
      }
#ifdef ZT_TCPROF
      if (p.prof.base && which == 0) {
        unsigned long long *o = p.prof.base + ((size_t)blockIdx.x * 4 + 1) * kTimelineSlots;
        o[0] = clock64() - mc_total; o[1] = mc_fullx; o[2] = mc_fullw; o[3] = mc_issue; o[4] = mc_tmem; o[5] = mc_commit; o[6] = (it - 8) / NI;
      }
#endif
    }
  } else if (kUseTeams && warp < 2 + kDqWarps) {
    // ---------------- dequantisation warps, four teams: a thread converts one weight row of a k-block ----------------
    const int dw = warp - 2;
    const uint32_t team = (uint32_t)dw / kTeamWarps;       // takes ring positions it with it % 4 == team
    const int row = (dw % kTeamWarps) * 32 + lane;          // weight row (output column) within the tile
    const uint32_t row_x = row & 7;
    const int gs_shift = (p.gs & (p.gs - 1)) == 0 ? __ffs(p.gs) - 1 : -1;
    const bool exact_scale = (p.scale_dtype == ZT_BF16);
    const int my_tiles = blockIdx.x < total_tiles ? (total_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    // Scales (zero points) of the two 32-k halves of a k-block, fetched from global memory one k-block of this
    // team ahead.  Position = (local tile index, chunk); the team's k-block in a chunk is 4 * chunk + jt with
    // jt = (team - local * num_kb) mod 4, when that k-block exists.
    struct Sc {
      float s0, s1, z0, z1;
    };
    auto fetch = [&](int local, int chunk, Sc &out) {
      if (local >= my_tiles) return;
      const uint32_t jt = (team - (uint32_t)local * (uint32_t)num_kb) & 3u;
      const int kb = chunk * kChunkKB + (int)jt;
      if (kb >= num_kb) return;
      const TileInfo t = decode_tile(p, blockIdx.x + local * gridDim.x, n_mt, BT);
      const int64_t base = (int64_t)t.expert * p.s_estride + min(t.n0 + row, p.N - 1);
      const int k = (t.kb0 + kb) * kBK;
      const int g0 = gs_shift >= 0 ? (k >> gs_shift) : (k / p.gs);
      const int g1 = gs_shift >= 0 ? ((k + 32) >> gs_shift) : ((k + 32) / p.gs);
      out.s0 = load_as_float(p.scales, base + (int64_t)g0 * p.N, p.scale_dtype);
      out.s1 = g1 == g0 ? out.s0 : load_as_float(p.scales, base + (int64_t)g1 * p.N, p.scale_dtype);
      if (ASYM) {
        out.z0 = load_as_float(p.zeros, base + (int64_t)g0 * p.N, p.scale_dtype);
        out.z1 = g1 == g0 ? out.z0 : load_as_float(p.zeros, base + (int64_t)g1 * p.N, p.scale_dtype);
      }
    };
    Sc nxt{0.f, 0.f, 0.f, 0.f};
    const bool staged = p.staged_gpc != 0;
    if (!staged) fetch(0, 0, nxt);
    uint32_t pit = 0;   // packed chunks walked so far (every team walks every chunk)
    bool ok = true;
#ifdef ZT_TCPROF
    long long tc_total = 0, tc_fullp = 0, tc_empty = 0, tc_conv = 0, tc_blocks = 0;
    bool tcp_warm = false;
#endif
    for (int local = 0; local < my_tiles; ++local) {
      const uint32_t it0 = (uint32_t)local * (uint32_t)num_kb;   // ring position of the tile's first k-block
      const uint32_t jt = (team - it0) & 3u;
      for (int chunk = 0; chunk < num_chunks; ++chunk, ++pit) {
#ifdef ZT_TCPROF
        if (pit == 2) { tcp_warm = true; tc_total = clock64(); }
#endif
        Sc cur = nxt;
        if (!staged) {
          if (chunk + 1 < num_chunks) fetch(local, chunk + 1, nxt); else fetch(local + 1, 0, nxt);
        }
        const uint32_t ps = pit % PSTAGES;
        {
          TCP_T0();
          if (ok && !TC_WAITN(&full_p[ps], (pit / PSTAGES) & 1)) {
            tc::report_timeout(p.status, kStatusConvertTimeout);
            ok = false;
          }
          TCP_ADD(tc_fullp);
        }
        if (staged && ok) {
          // groups are at least 128 k wide here, so both halves of a k-block share one; with two groups per chunk
          // the k-blocks 0, 1 take the first and 2, 3 the second
          const int gl = p.staged_gpc == 2 ? (int)(jt >> 1) : 0;
          const unsigned char *slot = sc_ring + ps * kScaleSlotBytes;
          cur.s0 = cur.s1 = load_as_float(slot, gl * kBN + row, p.scale_dtype);
          if (ASYM) cur.z0 = cur.z1 = load_as_float(slot + kZeroSlotOffset, gl * kBN + row, p.scale_dtype);
        }
        const int kb = chunk * kChunkKB + (int)jt;
        if (kb < num_kb) {
          const uint32_t it = it0 + (uint32_t)kb;
          const uint32_t s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          {
            TCP_T0();
            if (ok && !TC_WAITN(&empty_bar[s], ph ^ 1)) {
              tc::report_timeout(p.status, kStatusConvertTimeout);
              ok = false;
            }
            TCP_ADD(tc_empty);
          }
#ifdef ZT_TCPROF
          if (p.prof.base && dw == 0 && lane == 0 && it == 20) p.prof.base[((size_t)blockIdx.x * 4 + 3) * kTimelineSlots + 3] = clock64();   // team saw stage of block 16 free
#endif
          TCP_T0();
          if (ok && !TCP_DBG(4)) {
            // the row's 32 packed bytes of this k-block: 16-byte chunks 2 jt and 2 jt + 1 of the swizzled 128-byte row
            const unsigned char *prow = packed + ps * kChunkBytes + row * 128;
            const uint4 w0 = *reinterpret_cast<const uint4 *>(prow + (((2u * jt) ^ row_x) << 4));
            const uint4 w1 = *reinterpret_cast<const uint4 *>(prow + (((2u * jt + 1u) ^ row_x) << 4));
            const uint32_t words[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
            unsigned char *wrow = smem + s * L::kWBytes + row * 128;
            uint32_t sh[2] = {0, 0}, sl[2] = {0, 0};
            if (!ASYM) {
              split_bf16x2(cur.s0, sh[0], sl[0]);
              split_bf16x2(cur.s1, sh[1], sl[1]);
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int hf = i >> 2;   // which 32 k of the k-block
              uint4 o;
              if (ASYM) {
                const float sc = hf ? cur.s1 : cur.s0, zp = hf ? cur.z1 : cur.z0;
                float f[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                  const uint32_t bits = ((words[i] >> (4 * e)) & 0xFu) | 0x4B000000u;  // 2^23 + q
                  f[e] = fmaf(__uint_as_float(bits) - 8388616.0f, sc, zp);           // (q - 8) * s + z
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
                  r[pp] = exact_scale ? bf2_mul(v, sh[hf]) : bf2_fma(v, sh[hf], bf2_mul(v, sl[hf]));  // (k = p, k = p + 4)
                }
                o.x = prmt(r[0], r[1], 0x5410);  // (k0, k1)
                o.y = prmt(r[2], r[3], 0x5410);  // (k2, k3)
                o.z = prmt(r[0], r[1], 0x7632);  // (k4, k5)
                o.w = prmt(r[2], r[3], 0x7632);  // (k6, k7)
              }
              *reinterpret_cast<uint4 *>(wrow + (((uint32_t)i ^ row_x) << 4)) = o;
            }
            tc::fence_proxy_async_smem();  // generic-proxy stores -> visible to the tensor core's reads
          }
          __syncwarp();
          if (lane == 0) tc::mbar_arrive(&full_w[s]);
#ifdef ZT_TCPROF
          if (p.prof.base && dw == 0 && lane == 0 && it == 16) p.prof.base[((size_t)blockIdx.x * 4 + 3) * kTimelineSlots + 0] = clock64();   // W(16) announced
          if (p.prof.base && dw == 0 && lane == 0 && it == 20) p.prof.base[((size_t)blockIdx.x * 4 + 3) * kTimelineSlots + 4] = clock64();   // W(20) announced
#endif
          TCP_ADD(tc_conv);
#ifdef ZT_TCPROF
          if (tcp_warm) ++tc_blocks;
#endif
        }
        __syncwarp();
        if (lane == 0) tc::mbar_arrive(&empty_p[ps]);   // this warp is done with the chunk (or had nothing in it)
      }
    }
#ifdef ZT_TCPROF
    if (p.prof.base && dw == 0 && lane == 0) {
      unsigned long long *o = p.prof.base + ((size_t)blockIdx.x * 4 + 0) * kTimelineSlots;
      o[0] = clock64() - tc_total; o[1] = tc_fullp; o[2] = tc_empty; o[3] = tc_conv; o[4] = tc_blocks;
    }
#endif
  } else if (warp < 2 + kDqWarps) {
    // ---------------- dequantisation warps ----------------
    const int d = threadIdx.x - 64;                 // 0 .. 32 * kDqWarps - 1
    constexpr int kThreadsPerRow = 8 / kWPT;        // a k-block row is 8 packed words
    const int row = d / kThreadsPerRow;             // weight row (output column) within the tile
    const int sub = d % kThreadsPerRow;
    const int half = sub * kWPT / 4;                // which 32 k of the 64-wide k-block (one scale each)
    const int word0 = sub * kWPT % 4;               // first of this thread's words within that half
    // scales (and zero points) come from global memory, fetched kPrefetch k-blocks ahead.  The fetch
    // cursor keeps its tile's column and expert offset; they change only when it moves to a new tile.
    const int gs_shift = (p.gs & (p.gs - 1)) == 0 ? __ffs(p.gs) - 1 : -1;
    constexpr int kPrefetch = 4;
    DqRegs ring[kPrefetch];
    int ftile = blockIdx.x, fkb = 0;  // next (tile, k-block) to fetch
    int64_t fbase = 0;                // expert offset + column of the fetch cursor's tile
    int fkb0 = 0;                     // first k-block of the fetch cursor's work item
    auto set_fetch_tile = [&]() {
      if (ftile < total_tiles) {
        const TileInfo t = decode_tile(p, ftile, n_mt, BT);
        fbase = (int64_t)t.expert * p.s_estride + min(t.n0 + row, p.N - 1);
        fkb0 = t.kb0;
      }
    };
    set_fetch_tile();
    auto fetch_next = [&](DqRegs &slot) {
      if (ftile < total_tiles) {
        const int k = (fkb0 + fkb) * kBK + 32 * half;
        const int g = gs_shift >= 0 ? (k >> gs_shift) : (k / p.gs);
        const int64_t gi = fbase + (int64_t)g * p.N;
        slot.s = load_as_float(p.scales, gi, p.scale_dtype);
        slot.z = ASYM ? load_as_float(p.zeros, gi, p.scale_dtype) : 0.f;
        if (++fkb == num_kb) {
          fkb = 0;
          ftile += gridDim.x;
          set_fetch_tile();
        }
      }
    };
#pragma unroll
    for (int i = 0; i < kPrefetch; ++i) fetch_next(ring[i]);
    // loop-invariant shared-memory offsets of this thread: where it reads its 16 packed bytes of
    // k-block j of a chunk, and where it writes its four 16-byte bf16 chunks of a stage row
    uint32_t st_off[kWPT];
    const uint32_t row_off = row * 128, row_x = row & 7;
#pragma unroll
    for (int i = 0; i < kWPT; ++i) st_off[i] = row * 128 + (((4 * half + word0 + i) ^ (row & 7)) << 4);
    uint32_t it = 0;    // k-blocks converted so far (bf16 stage ring position)
    uint32_t pit = 0;   // packed chunks consumed so far
    int kb = 0;         // k-block within the current tile
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
          const int j = kb % kChunkKB;  // k-block within the packed chunk
          const uint32_t ps = pit % PSTAGES;
          if (j == 0 && ok && !tc::mbar_wait(&full_p[ps], (pit / PSTAGES) & 1)) {
            tc::report_timeout(p.status, kStatusConvertTimeout);
            ok = false;
          }
          const uint32_t s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (ok && !tc::mbar_wait(&empty_bar[s], ph ^ 1)) {
            tc::report_timeout(p.status, kStatusConvertTimeout);
            ok = false;
          }
          if (ok) {
            // this thread's 32 nibbles of the k-block: 16-byte chunk (2j + half) of the swizzled 128-byte row
            const unsigned char *src = packed + ps * kChunkBytes + row_off + ((((uint32_t)(2 * j + half)) ^ row_x) << 4) +
                                       4 * word0;
            uint32_t words[kWPT];
            if (kWPT == 4) {
              const uint4 wv = *reinterpret_cast<const uint4 *>(src);
              words[0] = wv.x;
              words[1] = wv.y;
              words[kWPT - 2] = wv.z;
              words[kWPT - 1] = wv.w;
            } else {
              const uint2 wv = *reinterpret_cast<const uint2 *>(src);
              words[0] = wv.x;
              words[1] = wv.y;
            }
            unsigned char *wstage = smem + s * L::kWBytes;
            uint32_t s_hi = 0, s_lo = 0;
            if (!ASYM) split_bf16x2(cur.s, s_hi, s_lo);
#pragma unroll
            for (int i = 0; i < kWPT; ++i) {
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
              *reinterpret_cast<uint4 *>(wstage + st_off[i]) = o;
            }
            tc::fence_proxy_async_smem();  // generic-proxy stores -> visible to the tensor core's reads
          }
          __syncwarp();
          if (lane == 0) tc::mbar_arrive(&full_w[s]);
          ++it;
          ++kb;
          const bool tile_done = (kb == num_kb);
          if (j == kChunkKB - 1 || tile_done) {  // the packed chunk is used up
            if (lane == 0) tc::mbar_arrive(&empty_p[ps]);
            ++pit;
          }
          if (tile_done) kb = 0;
        }
      }
    }
  } else if (warp >= 2 + kDqWarps && warp < 2 + kDqWarps + kEpiWarps) {
    // ---------------- epilogue warps ----------------
    grid_dependency_wait();                // output, partial sums and post-op operands are shared with earlier work
    const int ew = warp - (2 + kDqWarps);  // 0..3
    const int quarter = warp & 3;          // TMEM lanes 32*quarter .. +31
    float *scratch = epi_scratch + ew * 32 * kEpiRowStride;
    int local = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++local) {
      const TileInfo ti = decode_tile(p, tile, n_mt, BT);
      const int m0 = ti.m0, n0 = ti.n0;
      const int m_end = ti.m0 + ti.rows;  // rows past the tile's valid rows belong to nobody (or to the next expert)
      const uint32_t buf = (uint32_t)local % NBUF;
      const uint32_t use = (uint32_t)local / NBUF;
      if (ok && !TC_WAITN(&tmem_full[buf], use & 1)) {
        tc::report_timeout(p.status, kStatusEpilogueTimeout);
        ok = false;
      }
      tc::fence_after_sync();
      const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * NI * BT;
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
        if (NI == 2) {
          // the second issuer's accumulator: same lanes, BT columns further
          tc::tmem_ld_32x32b_x32(t_row + BT + c, r);
          tc::tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) scratch[j * kEpiRowStride + lane] += __uint_as_float(r[j]);
        }
        __syncwarp();
        // phase 2: rows of 32 columns, 4 token rows per pass
#pragma unroll 1
        for (int pass = 0; pass < 8; ++pass) {
          const int j = pass * 4 + sub_row;
          const int m = m0 + c + j;
          const float4 v4 = *reinterpret_cast<const float4 *>(&scratch[j * kEpiRowStride + col4]);
          if (p.ksplit > 1) {
            // split K: raw fp32 sums of this K slice; bias and post-ops belong to the kernel that adds the slices
            if (m < m_end) {
              float *dst = p.partial + ((int64_t)ti.ks * p.M + m) * p.N + nq + col4;
              if (nq + col4 + 4 <= p.N && (p.N & 3) == 0) {
                *reinterpret_cast<float4 *>(dst) = v4;
              } else {
                const float v[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
                for (int e = 0; e < 4; ++e)
                  if (nq + col4 + e < p.N) dst[e] = v[e];
              }
            }
          } else if (m < m_end && nq + col4 < p.N) {
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

// Tensor maps: activations [rows, K] bf16 with a (64 x BT) box; packed weights [rows, K/8] u32 with a
// (32 words x 128 rows) box; both 128-byte swizzled.  Memoised per process.
int cached_map(CUtensorMap *out, const void *ptr, CUtensorMapDataType dt, uint64_t inner, uint64_t rows,
               uint64_t pitch_bytes, uint32_t box_inner, uint32_t box_rows, bool swizzle = true) {
  static std::mutex mu;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  const MapKey key{ptr, inner * 4 + (uint64_t)dt % 4, rows, (box_rows * 1024 + box_inner) * 2 + (swizzle ? 1u : 0u)};
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it != cache.end()) {
    *out = it->second;
    return ZT_SUCCESS;
  }
  const uint64_t dims[2] = {inner, rows}, strides[1] = {pitch_bytes};
  const uint32_t box[2] = {box_inner, box_rows};
  int rc = make_tensor_map(out, ptr, dt, 2, dims, strides, box, swizzle);
  if (rc != ZT_SUCCESS) return rc;
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, *out);
  return ZT_SUCCESS;
}

template <int BT, int STAGES, int XSTAGES, int PSTAGES, int NI>
int launch_bt(const TcParams &p0, const void *x, int64_t x_rows, int64_t w_rows, int max_row_tiles, bool asym,
              cudaStream_t st) {
  using L = SmemLayout<BT, STAGES, XSTAGES, PSTAGES>;
  static_assert(L::kTotal <= 227 * 1024, "rings exceed shared memory");
  TcParams p = p0;
  p.m_tiles = ceil_div(p.M, BT);
  p.n_tiles = ceil_div(p.N, kBN);
  CUtensorMap tx, tw;
  int rc = cached_map(&tx, x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (uint64_t)p.K, (uint64_t)x_rows, (uint64_t)p.K * 2, kBK, BT);
  if (rc != ZT_SUCCESS) return rc;
  rc = cached_map(&tw, p.wq, CU_TENSOR_MAP_DATA_TYPE_UINT32, (uint64_t)p.K / 8, (uint64_t)w_rows, (uint64_t)p.K / 2,
                  kChunkKB * 8, kBN);
  if (rc != ZT_SUCCESS) return rc;
  // Scales and zero points travel with the packed chunks (one or two groups x 128 columns per chunk) when a
  // group is a power of two of at least 128 k and the tables can be addressed by TMA; otherwise the conversion
  // threads fetch them from global memory.
  CUtensorMap ts = tw, tz = tw;
  p.staged_gpc = 0;
  {
    const uint64_t esz = p.scale_dtype == ZT_F32 ? 4 : 2;
    const bool pow2 = (p.gs & (p.gs - 1)) == 0;
    const bool aligned = ((uint64_t)p.N * esz) % 16 == 0 && (reinterpret_cast<uintptr_t>(p.scales) & 15) == 0 &&
                         (!asym || (reinterpret_cast<uintptr_t>(p.zeros) & 15) == 0);
    if (pow2 && p.gs >= 128 && aligned) {
      int lg = 0;
      while ((1 << lg) < p.gs) ++lg;
      p.gs_log2 = lg;
      p.groups = p.K / p.gs;
      p.staged_gpc = p.gs == 128 ? 2 : 1;
      const uint64_t table_rows = (uint64_t)(w_rows / p.N) * (uint64_t)p.groups;   // experts x groups
      const CUtensorMapDataType sdt = p.scale_dtype == ZT_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
      rc = cached_map(&ts, p.scales, sdt, (uint64_t)p.N, table_rows, (uint64_t)p.N * esz, kBN, (uint32_t)p.staged_gpc, false);
      if (rc != ZT_SUCCESS) return rc;
      if (asym) {
        rc = cached_map(&tz, p.zeros, sdt, (uint64_t)p.N, table_rows, (uint64_t)p.N * esz, kBN, (uint32_t)p.staged_gpc, false);
        if (rc != ZT_SUCCESS) return rc;
      }
    }
  }
  const long long tiles = (long long)(p.g_count ? max_row_tiles : p.m_tiles) * p.n_tiles * p.ksplit;
  const int sms = sm_count();
  dim3 grid((unsigned)(tiles < sms ? tiles : sms));
#ifdef ZT_TCPROF
  p.prof = timeline_for_launch((int)grid.x * 4);
  {
    const char *e = getenv("ZENTORCH_B200_TCDBG");
    p.dbg = e ? atoi(e) : 0;
  }
#endif
  // every instantiation needs its own once-per-device attribute set-up
  static PerDeviceOnce configured[2];
  auto launch = [&](auto kern, int which) -> int {
    if (int rc_cfg = allow_dynamic_smem(configured[which], kern, L::kTotal)) return rc_cfg;
    ZT_CUDA_OK(launch_overlapped(kern, grid, dim3(kThreads), (size_t)L::kTotal, st, tx, tw, ts, tz, p));
    return ZT_SUCCESS;
  };
  rc = asym ? launch(woq_tcgen05_kernel<BT, STAGES, XSTAGES, PSTAGES, true, NI>, 0)
            : launch(woq_tcgen05_kernel<BT, STAGES, XSTAGES, PSTAGES, false, NI>, 1);
  if (rc != ZT_SUCCESS) return rc;
  return launch_status("woq_tcgen05_kernel");
}

int launch_any(int bt, const TcParams &p, const void *x, int64_t x_rows, int64_t w_rows, int max_row_tiles, bool asym,
               cudaStream_t st) {
  // two issuers need at least two k-blocks per work item; ZENTORCH_B200_WOQ_ISSUERS=1 keeps the single issuer
  static const int forced_ni = [] { const char *e = getenv("ZENTORCH_B200_WOQ_ISSUERS"); return e ? atoi(e) : 0; }();
  // 256-token tiles keep one issuer: two would leave room for two activation slots and one accumulator buffer
  // only, which measured 13 - 40 % slower than three slots and double-buffered accumulators.
  const bool two = forced_ni != 1 && !p.single_issuer && p.kps >= 2 && bt <= 128;
  if (two) {
    switch (bt) {
      // <token tile, converted-weight stages, activation slots, packed chunks, issuers>; rings of even length
      case 32: return launch_bt<32, 4, 4, 5, 2>(p, x, x_rows, w_rows, max_row_tiles, asym, st);
      case 64: return launch_bt<64, 4, 4, 5, 2>(p, x, x_rows, w_rows, max_row_tiles, asym, st);
      case 128: return launch_bt<128, 4, 4, 4, 2>(p, x, x_rows, w_rows, max_row_tiles, asym, st);
      default: break;
    }
  } else {
    switch (bt) {
      case 32: return launch_bt<32, 4, 4, 5, 1>(p, x, x_rows, w_rows, max_row_tiles, asym, st);
      case 64: return launch_bt<64, 4, 4, 5, 1>(p, x, x_rows, w_rows, max_row_tiles, asym, st);
      case 128: return launch_bt<128, 4, 4, 4, 1>(p, x, x_rows, w_rows, max_row_tiles, asym, st);
      case 256: return launch_bt<256, 4, 3, 2, 1>(p, x, x_rows, w_rows, max_row_tiles, asym, st);
      default: break;
    }
  }
  set_error("zt_woq_linear: unsupported token-tile width %d for the tcgen05 kernel", bt);
  return ZT_UNSUPPORTED;
}

}  // namespace

// Split-K plan of the dense mode: the largest number of equal K slices (each a multiple of the packed chunk) that keeps tiles x slices within one round of the SMs.  1 = no split.
int woq_tcgen05_ksplit(int64_t M, int64_t N, int64_t K) {
  if (M > 256 || (N & 3) != 0 || K % kBK != 0) return 1;
  const int bt = M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
  const int64_t tiles = ceil_div<int64_t>(M, bt) * ceil_div<int64_t>(N, kBN);
  const int64_t num_kb = K / kBK;
  const int sms = sm_count();
  int best = 1;
  for (int ks = 2; ks <= 32; ++ks) {
    if (tiles * ks > sms) break;
    if (num_kb % ks != 0) continue;
    const int64_t kps = num_kb / ks;
    if (kps % kChunkKB != 0) continue;
    best = ks;
  }
  return best;
}
size_t woq_tcgen05_workspace_bytes(int64_t M, int64_t N, int64_t K) {
  const int ks = woq_tcgen05_ksplit(M, N, K);
  return ks > 1 ? (size_t)ks * M * N * sizeof(float) : 0;
}

bool woq_tcgen05_supported(const zt_woq_linear_args_t &a) {
  if (a.M < 1 || a.N < 1 || a.K < kBK || a.K % kBK != 0) return false;
  if (a.n_groups <= 0 || a.K % a.n_groups != 0) return false;
  const int64_t gs = a.K / a.n_groups;
  if (gs % 32 != 0) return false;
  if (a.K % 32 != 0) return false;  // packed rows are fetched by TMA: pitch K/2 bytes must be a multiple of 16
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
  p.single_issuer = (a.algo & ZT_ALGO_SINGLE_ISSUER) ? 1 : 0;
  p.ksplit = 1;
  p.kps = (int)(a.K / kBK);
  if (bt == 0) {
    bt = a.M <= 32 ? 32 : a.M <= 64 ? 64 : a.M <= 128 ? 128 : 256;
    // few tiles: split K over the idle SMs when the caller's workspace has room for the partial sums
    const int ks = woq_tcgen05_ksplit(a.M, a.N, a.K);
    const size_t need = ZT_WOQ_COUNTER_BYTES + (size_t)ks * a.M * a.N * sizeof(float);
    if (ks > 1 && a.workspace != nullptr && a.workspace_bytes >= need) {
      p.ksplit = ks;
      p.kps = (int)(a.K / kBK / ks);
      p.partial = reinterpret_cast<float *>(reinterpret_cast<char *>(a.workspace) + ZT_WOQ_COUNTER_BYTES);
    }
  }
  int rc = launch_any(bt, p, a.x, a.M, a.N, 0, asym, st);
  if (rc != ZT_SUCCESS || p.ksplit == 1) return rc;
  const int64_t quads = a.M * a.N / 4;
  ZT_CUDA_OK(launch_overlapped(woq_splitk_reduce_kernel, dim3((unsigned)ceil_div<int64_t>(quads, 256)), dim3(256), (size_t)0, st,
                               (const float *)p.partial, p.ksplit, p.M, p.N, p.bias, p.bias_dtype, p.post, p.y));
  return launch_status("woq_splitk_reduce_kernel");
}

// Grouped form for mixture-of-experts: `x` holds `total_rows` rows sorted by expert; `tiles` / `tile_count`
// (device memory) list the row tiles; weights and scales are stacked per expert.
int woq_tcgen05_grouped_launch(const void *x, int64_t total_rows, int64_t N, int64_t K, const int32_t *wq,
                               const void *scales, int scale_dtype, int64_t n_groups, int num_experts, void *y,
                               const int *tile_count, const int4 *tiles, int max_row_tiles, int bt, cudaStream_t st) {
  TcParams p{};
  p.M = (int)total_rows;
  p.N = (int)N;
  p.K = (int)K;
  p.gs = (int)(K / n_groups);
  p.wq = wq;
  p.scales = scales;
  p.zeros = nullptr;
  p.scale_dtype = scale_dtype;
  p.bias = nullptr;
  p.bias_dtype = ZT_BF16;
  p.y = reinterpret_cast<__nv_bfloat16 *>(y);
  p.status = device_status_ptr();
  p.ksplit = 1;
  p.kps = (int)(K / kBK);
  p.g_count = tile_count;
  p.g_tiles = tiles;
  p.s_estride = n_groups * N;
  return launch_any(bt, p, x, total_rows, (int64_t)num_experts * N, max_row_tiles, false, st);
}

}  // namespace zt
