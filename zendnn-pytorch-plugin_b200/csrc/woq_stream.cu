// Weight-only int4 linear for decode (M <= 16): an HBM-bound streaming kernel.
//
// Work decomposition.  A CTA owns 16*R output columns (= rows of the N-major packed weight) and one
// K-slice; its W warps split the slice's 128-wide k-steps round-robin, so every warp streams its own
// part of the same rows.  A lane reads 128 bits (32 nibbles) per row and step, the four lanes of a
// quad cover the 128 consecutive k of the step (= one quantisation group when the group size is
// 128).  Weight loads run RING steps ahead of the arithmetic in a register ring, together with the
// scales (and zero points) of those steps, so that each thread keeps RING * 2R 16-byte loads in flight
// (R = 4 with RING = 2 for wide layers: the activation-side work of a step is shared by 64 columns).
// Activations are staged asynchronously (cp.async, double buffered, one chunk = two steps per warp)
// so that staging never stalls the weight stream.
//
// Arithmetic.  Nibbles become bf16 pairs in registers with one lop3 each ((w >> 4p) & 0x000f000f
// picks nibbles p and p+4; or-ing 0x4300 into both halves gives the bf16 number 128 + u; signed
// nibbles are xor-ed with 8 in the same lop3, so u = q + 8 in both formats).  Those pairs are the A
// operand of mma.sync.m16n8k16 (rows = output columns); the B operand is read from the staged
// activations and permuted to the matching order (k, k+4), (k+1, k+5), ... with four byte-permutes
// per 16 bytes.  A second MMA per k-block with an all-ones A operand yields sum_k x[m,k] of the step
// in the same fragment layout; with it the bias of 136 is removed on the step's partial sum
// (part - 136 * sum), the group scale multiplies the corrected partial sum in fp32, and the zero point
// contributes z * sum.  Dequantised weights are therefore never rounded to bf16: the result is the
// fp32-accumulated product with exact q*s.
//
// Reduction.  Warp partials are combined through shared memory; K-slices (only used when N alone
// cannot fill the GPU) through a global fp32 scratch by the last CTA to arrive, in a fixed order.
#include <cstdlib>
#include <type_traits>

#include "common.cuh"
#include "woq.cuh"

namespace zt {

namespace {

constexpr int kStepK = 128;  // k per step
constexpr int kSPC = 2;      // steps per warp and activation chunk

struct StreamParams {
  const __nv_bfloat16 *x;
  const int32_t *wq;
  const void *scales;
  const void *zeros;
  const void *bias;
  __nv_bfloat16 *y;
  float *partial;  // [nsplit][M][N]
  int *counters;   // one per n-tile, zero on entry and on exit
  int M, N, K;
  int gs;
  int kslice;
  int nsplit;
  int scale_dtype, bias_dtype;
  int early_trigger;  // the grid is resident at once: let the next kernel in at entry rather than after the main loop
  int cluster;        // the K slices of a column tile are one thread-block cluster: reduce through its shared memory
  int cluster_off;    // byte offset of the cluster reduction buffer [nsplit][M][columns] in dynamic shared memory
  TimelineSink timeline;
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
  } else {  // (w & 0x000f000f) | 0x43004300
    asm("lop3.b32 %0, %1, %2, %3, 0xea;" : "=r"(r) : "r"(w), "n"(0x000f000f), "n"(0x43004300));
  }
  return r;
}

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void cp_async_16(void *smem_dst, const void *gmem_src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem_dst)), "l"(gmem_src), "r"(src_bytes)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// 16-byte slot of activations k = 8b .. 8b+7 within a chunk row: the fields "which word of the lane's
// 128-bit weight load" (b & 3) and "which lane of the quad" ((b >> 2) & 3) are swapped so that the
// eight lanes of a shared-load phase hit eight different bank groups.
__device__ __forceinline__ int x_slot(int b) { return (b & ~15) | ((b & 3) << 2) | ((b >> 2) & 3); }

template <int R>
struct RingSlot {
  uint4 w[R][2];
  float s[R][2];
  float z[R][2];
};

template <int MT, int R, int RING, int W, bool ASYM, bool SF32>
__global__ void __launch_bounds__(W * 32) woq_stream_kernel(const StreamParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr int kThreads = W * 32;
  constexpr int kCols = MT * 8;                        // padded M held in MMA column blocks
  constexpr int kChunkK = W * kSPC * kStepK;           // k staged per chunk
  constexpr int kRowSlots = kChunkK / 8 + 4;           // +4 slots: bank skew between rows
  constexpr int kTileN = 16 * R;
  constexpr int kUnroll = RING / kSPC;  // chunks per trip of the main loop (ring slots are static)
  static_assert(RING % kSPC == 0 && (kUnroll == 1 || kUnroll == 2), "ring must hold one or two chunks");
  using ScaleT = typename std::conditional<SF32, float, __nv_bfloat16>::type;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int n0 = blockIdx.x * kTileN;
  const int split = blockIdx.y;
  const int k0 = split * p.kslice;
  const int k1 = min(p.K, k0 + p.kslice);
  const int nchunks = (k1 - k0 + kChunkK - 1) / kChunkK;
  const int mrows = min(p.M, kCols);
  uint4 *xs = reinterpret_cast<uint4 *>(smem_raw);     // [2][mrows][kRowSlots]
  const int buf_slots = mrows * kRowSlots;

  // per-row base pointers: weights as 16-byte vectors (4*t words into the step), scales at column n
  const uint4 *wrow[R][2];
  const ScaleT *srow[R][2];
  const ScaleT *zrow[R][2];
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int n = min(n0 + 16 * r + 8 * h + g, p.N - 1);
      wrow[r][h] = reinterpret_cast<const uint4 *>(p.wq + (size_t)n * (p.K >> 3)) + t;
      srow[r][h] = reinterpret_cast<const ScaleT *>(p.scales) + n;
      zrow[r][h] = ASYM ? reinterpret_cast<const ScaleT *>(p.zeros) + n : nullptr;
    }

  // step j of chunk c covers k = k0 + c*kChunkK + (j*W + warp)*128 .. +127
  auto step_k = [&](int c, int j) { return k0 + c * kChunkK + (j * W + warp) * kStepK; };
  RingSlot<R> ring[RING];
  auto prefetch = [&](RingSlot<R> &slot, int k) {
    if (k < k1) {
      const uint32_t woff = (uint32_t)k >> 5;                       // 16-byte vectors into the row
      const uint32_t soff = (uint32_t)(k / p.gs) * (uint32_t)p.N;  // group row of the scale table
#pragma unroll
      for (int r = 0; r < R; ++r)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          slot.w[r][h] = ldg_nc_v4(wrow[r][h] + woff);
          slot.s[r][h] = SF32 ? (float)__ldg(reinterpret_cast<const float *>(srow[r][h]) + soff)
                              : __bfloat162float(__ldg(reinterpret_cast<const __nv_bfloat16 *>(srow[r][h]) + soff));
          if (ASYM)
            slot.z[r][h] = SF32 ? (float)__ldg(reinterpret_cast<const float *>(zrow[r][h]) + soff)
                                : __bfloat162float(__ldg(reinterpret_cast<const __nv_bfloat16 *>(zrow[r][h]) + soff));
        }
    }
  };
  auto stage = [&](int c, int buf) {
    const int kc = k0 + c * kChunkK;
    for (int i = tid; i < mrows * (kChunkK / 8); i += kThreads) {
      const int row = i / (kChunkK / 8), b = i - row * (kChunkK / 8);
      const int k = kc + 8 * b;
      const bool in = k < k1;
      cp_async_16(&xs[buf * buf_slots + row * kRowSlots + x_slot(b)], p.x + (size_t)row * p.K + (in ? k : 0),
                  in ? 16 : 0);  // beyond the slice: zero-fill
    }
    cp_async_commit();
  };

  // Weights and scales do not depend on the kernel before this one: fill the register ring, and only then
  // wait for that kernel before touching activations, scratch and output.
  // The next kernel may come in at once when this grid is resident as a whole; otherwise only after the main
  // loop, when every CTA of this grid has started (its CTAs would take the places of this grid's later ones).
  const int cta = blockIdx.y * gridDim.x + blockIdx.x;
  stamp(p.timeline, cta, 0);
  if (p.early_trigger) grid_launch_dependents();
  // cluster form: every CTA of the cluster must be running before a peer's shared memory is written; the
  // matching wait sits right before the first remote store
  if (p.cluster) asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
#pragma unroll
  for (int s = 0; s < RING; ++s) prefetch(ring[s], step_k(s / kSPC, s % kSPC));
  stamp(p.timeline, cta, 1);
  grid_dependency_wait();
  stamp(p.timeline, cta, 2);
  stage(0, 0);

  float acc[R][MT][4];
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[r][m][e] = 0.f;

  for (int c2 = 0; c2 < nchunks; c2 += kUnroll) {
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int c = c2 + u;
      const int h2 = c & 1;  // activation buffer of this chunk
      if (c < nchunks) {
        cp_async_wait_all();
        __syncthreads();  // chunk c has landed for everybody; chunk c-1 (other buffer) is no longer read
        if (c == 0) stamp(p.timeline, cta, 3);
        if (c + 1 < nchunks) stage(c + 1, h2 ^ 1);
        const uint4 *xb = xs + h2 * buf_slots;
#pragma unroll
        for (int j = 0; j < kSPC; ++j) {
          RingSlot<R> &slot = ring[u * kSPC + j];
          const int k = step_k(c, j);
          if (k < k1) {
            const int sidx = j * W + warp;  // step index within the chunk
            float part[R][MT][4];
            float xsum[MT][4];
#pragma unroll
            for (int m = 0; m < MT; ++m)
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                xsum[m][e] = 0.f;
#pragma unroll
                for (int r = 0; r < R; ++r) part[r][m][e] = 0.f;
              }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint32_t bf[MT][4];
#pragma unroll
              for (int m = 0; m < MT; ++m) {
                const int col = m * 8 + g;
                uint4 v = make_uint4(0u, 0u, 0u, 0u);
                if (col < mrows) v = xb[col * kRowSlots + sidx * 16 + 4 * i + t];
                bf[m][0] = prmt(v.x, v.z, 0x5410);  // (x0, x4)
                bf[m][1] = prmt(v.x, v.z, 0x7632);  // (x1, x5)
                bf[m][2] = prmt(v.y, v.w, 0x5410);  // (x2, x6)
                bf[m][3] = prmt(v.y, v.w, 0x7632);  // (x3, x7)
                constexpr uint32_t kOnes = 0x3f803f80u;  // bf16 (1.0, 1.0)
                mma_bf16_16816(xsum[m], kOnes, kOnes, kOnes, kOnes, bf[m][0], bf[m][1]);
                mma_bf16_16816(xsum[m], kOnes, kOnes, kOnes, kOnes, bf[m][2], bf[m][3]);
              }
#pragma unroll
              for (int r = 0; r < R; ++r) {
                const uint4 &qa = slot.w[r][0];
                const uint4 &qb = slot.w[r][1];
                const uint32_t wa = (i == 0) ? qa.x : (i == 1) ? qa.y : (i == 2) ? qa.z : qa.w;
                const uint32_t wb = (i == 0) ? qb.x : (i == 1) ? qb.y : (i == 2) ? qb.z : qb.w;
                uint32_t ra[4], rb[4];
#pragma unroll
                for (int pp = 0; pp < 4; ++pp) {
                  ra[pp] = nib_pair_to_bf16x2<!ASYM>(wa >> (4 * pp));
                  rb[pp] = nib_pair_to_bf16x2<!ASYM>(wb >> (4 * pp));
                }
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                  mma_bf16_16816(part[r][m], ra[0], rb[0], ra[1], rb[1], bf[m][0], bf[m][1]);
                  mma_bf16_16816(part[r][m], ra[2], rb[2], ra[3], rb[3], bf[m][2], bf[m][3]);
                }
              }
            }
            // fold the step: acc += s * (part - 136 * sum_x) + z * sum_x   (sum_x per output column m)
#pragma unroll
            for (int m = 0; m < MT; ++m)
#pragma unroll
              for (int e = 0; e < 2; ++e) {
                const float sxv = xsum[m][e];  // every row of the ones-MMA holds the column sums
#pragma unroll
                for (int r = 0; r < R; ++r)
#pragma unroll
                  for (int h = 0; h < 2; ++h) {
                    float v = slot.s[r][h] * fmaf(-136.f, sxv, part[r][m][2 * h + e]);
                    if (ASYM) v = fmaf(slot.z[r][h], sxv, v);
                    acc[r][m][2 * h + e] += v;
                  }
              }
          }
          prefetch(slot, step_k(c + kUnroll, j));
        }
      }
    }
  }

  // ---- reduce the warps (they split K) through shared memory ------------------------------------------
  stamp(p.timeline, cta, 4);
  if (!p.early_trigger) grid_launch_dependents();
  __syncthreads();
  float *red = reinterpret_cast<float *>(smem_raw);  // [W][kCols][kTileN + 1]
  constexpr int kRedStride = kTileN + 1;
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int nl = 16 * r + 8 * (e >> 1) + g;
        const int ml = m * 8 + 2 * t + (e & 1);
        red[(warp * kCols + ml) * kRedStride + nl] = acc[r][m][e];
      }
  __syncthreads();
  stamp(p.timeline, cta, 5);

  __shared__ int s_ticket;
  constexpr int kRowsPerPass = kThreads / kTileN;
  const int nl = tid % kTileN;
  const int n = n0 + nl;
  float *cl = reinterpret_cast<float *>(smem_raw + p.cluster_off);   // [nsplit][M][kTileN], used in the first CTA
  if (p.nsplit > 1 && p.cluster) {
    // K slices of this column tile form a cluster (rank = slice): every CTA puts its sums into the first
    // CTA's shared memory, which adds them in slice order after the cluster barrier -- no global round trip.
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");   // pairs with the arrive at kernel entry
    for (int ml = tid / kTileN; ml < p.M; ml += kRowsPerPass) {
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < W; ++w) v += red[(w * kCols + ml) * kRedStride + nl];
      const uint32_t local = smem_u32(cl + ((size_t)split * p.M + ml) * kTileN + nl);
      uint32_t remote;
      asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(0));
      asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
    }
    __syncwarp();   // the loop's trip count differs between lanes; the aligned barrier needs the warp converged
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (split != 0) return;
  } else if (p.nsplit > 1) {
    for (int ml = tid / kTileN; ml < p.M; ml += kRowsPerPass) {
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < W; ++w) v += red[(w * kCols + ml) * kRedStride + nl];
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
  stamp(p.timeline, cta, 6);
  for (int ml = tid / kTileN; ml < p.M; ml += kRowsPerPass) {
    if (n >= p.N) continue;
    float v = 0.f;
    if (p.nsplit > 1 && p.cluster) {
      for (int s = 0; s < p.nsplit; ++s) v += cl[((size_t)s * p.M + ml) * kTileN + nl];
    } else if (p.nsplit > 1) {
      for (int s = 0; s < p.nsplit; ++s) v += __ldcg(&p.partial[((size_t)s * p.M + ml) * p.N + n]);
    } else {
#pragma unroll
      for (int w = 0; w < W; ++w) v += red[(w * kCols + ml) * kRedStride + nl];
    }
    if (p.bias) v += load_as_float(p.bias, n, p.bias_dtype);
    const int64_t idx = (int64_t)ml * p.N + n;
    v = apply_post_ops(v, p.post, idx, ZT_BF16);
    p.y[idx] = __float2bfloat16_rn(v);
  }
  stamp(p.timeline, cta, 7);
}

// Kernel shapes.  cfg 0: 16 columns per CTA, cfg 1: 32 columns (both 8 warps for M <= 8, ring of 4);
// cfg 2: 64 columns, 4 warps, ring of 2 (wide layers).  M in 9..16 always uses 4 warps.
template <int MT, int CFG>
struct Shape {
  static constexpr int R = CFG == 0 ? 1 : CFG == 1 ? 2 : 4;
  static constexpr int RING = CFG == 2 ? 2 : 4;
  static constexpr int W = (MT == 1 && CFG != 2) ? 8 : 4;
};

template <int MT, int CFG>
size_t stream_smem_bytes(int M) {
  using S = Shape<MT, CFG>;
  constexpr int kChunkK = S::W * kSPC * kStepK;
  const size_t mrows = (size_t)(M < MT * 8 ? M : MT * 8);
  const size_t stage = 2 * mrows * (kChunkK / 8 + 4) * 16;
  const size_t red = (size_t)S::W * MT * 8 * (16 * S::R + 1) * sizeof(float);
  return stage > red ? stage : red;
}

constexpr int kMaxDynSmem = 160 * 1024;

template <int MT, int CFG, bool ASYM, bool SF32>
int launch(const StreamParams &p_in, dim3 grid, cudaStream_t st) {
  using S = Shape<MT, CFG>;
  auto kern = woq_stream_kernel<MT, S::R, S::RING, S::W, ASYM, SF32>;
  static PerDeviceOnce configured;
  if (int rc_cfg = allow_dynamic_smem(configured, kern, kMaxDynSmem)) return rc_cfg;
  // clusters of up to eight K slices (the portable cluster size) reduce through shared memory
  static const bool use_clusters = [] {
    const char *e = std::getenv("ZENTORCH_B200_WOQ_CLUSTER");
    return !(e && e[0] == '0');
  }();
  const size_t base_smem = (stream_smem_bytes<MT, CFG>(p_in.M) + 15) / 16 * 16;
  const size_t cl_bytes = (size_t)p_in.nsplit * p_in.M * (16 * S::R) * sizeof(float);
  bool cluster = use_clusters && p_in.nsplit >= 2 && p_in.nsplit <= 8 && (int)grid.y == p_in.nsplit &&
                 base_smem + cl_bytes <= (size_t)kMaxDynSmem;
  size_t smem = base_smem + (cluster ? cl_bytes : 0);
  // resident CTAs per SM: depends on the device and on the shared-memory size (M, and the cluster buffer),
  // so it is asked for every launch (a host-side computation from the function's attributes)
  int per_sm = 0;
  ZT_CUDA_OK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, S::W * 32, smem));
  StreamParams p = p_in;
  p.timeline = timeline_for_launch((int)(grid.x * grid.y));
  p.cluster = cluster ? 1 : 0;
  p.cluster_off = (int)base_smem;
  // half the resident capacity at most: the next kernel's CTAs then find room beside this grid's
  p.early_trigger = (long long)grid.x * grid.y * 2 <= (long long)per_sm * sm_count() ? 1 : 0;
  if (cluster) {
    // a cluster shape the device cannot place is refused at launch: fall back to the reduction through the workspace
    if (launch_overlapped_cluster(kern, grid, dim3(S::W * 32), smem, st, (unsigned)p.nsplit, p) == cudaSuccess)
      return launch_status("woq_stream_kernel");
    (void)cudaGetLastError();
    cluster = false;
    p.cluster = 0;
    smem = base_smem;
  }
  ZT_CUDA_OK(launch_overlapped(kern, grid, dim3(S::W * 32), smem, st, p));
  return launch_status("woq_stream_kernel");
}

template <int MT, int CFG>
int launch_q(const StreamParams &p, dim3 grid, cudaStream_t st) {
  const bool asym = p.zeros != nullptr, sf32 = p.scale_dtype == ZT_F32;
  if (asym) return sf32 ? launch<MT, CFG, true, true>(p, grid, st) : launch<MT, CFG, true, false>(p, grid, st);
  return sf32 ? launch<MT, CFG, false, true>(p, grid, st) : launch<MT, CFG, false, false>(p, grid, st);
}

}  // namespace

// Columns per CTA grow with N (64 once that still gives every SM about two CTAs); K is split across
// CTAs only when the column tiles alone cannot occupy the GPU.
WoqStreamPlan woq_stream_plan(int64_t M, int64_t N, int64_t K) {
  WoqStreamPlan pl{};
  pl.mt = M <= 8 ? 1 : 2;
  const int64_t sms = sm_count();
  // Wide CTAs (64 columns) re-read the activations least and measured fastest wherever column tiles x K
  // slices still give every other SM a CTA; narrower ones only for layers too small for that.
  const int64_t max_split0 = K / 512 > 0 ? K / 512 : 1;
  int cfg = 0;
  if (ceil_div<int64_t>(N, 64) * max_split0 >= sms / 2) cfg = 2;
  else if (ceil_div<int64_t>(N, 32) * max_split0 >= sms / 2) cfg = 1;
  const char *force = std::getenv("ZENTORCH_B200_WOQ_STREAM_CFG");
  if (force && *force) cfg = std::atoi(force) < 0 ? 0 : std::atoi(force) > 2 ? 2 : std::atoi(force);
  pl.r = cfg;  // kernel shape index (see Shape<>)
  const int64_t tile_n = cfg == 0 ? 16 : cfg == 1 ? 32 : 64;
  const int64_t ntiles = ceil_div<int64_t>(N, tile_n);
  int nsplit = 1;
  if (ntiles < (3 * sms) / 2) {
    nsplit = (int)ceil_div<int64_t>(2 * sms, ntiles);
    const int64_t max_split = K / 512 > 0 ? K / 512 : 1;  // at least four steps per CTA
    if (nsplit > max_split) nsplit = (int)max_split;
  } else if (ntiles < 3 * sms) {
    // one to two CTAs per SM: four K slices (a cluster each, reduced through shared memory) measured 10-15 %
    // faster than none
    nsplit = (int)(K / 512 >= 4 ? 4 : 1);
  }
  int64_t kslice = ceil_div<int64_t>(ceil_div<int64_t>(K, nsplit), kStepK) * kStepK;
  pl.kslice = (int)kslice;
  pl.nsplit = (int)ceil_div<int64_t>(K, kslice);
  if (ntiles * (int64_t)sizeof(int) > ZT_WOQ_COUNTER_BYTES) {
    pl.nsplit = 1;
    pl.kslice = (int)K;
  }
  pl.partial_bytes = pl.nsplit > 1 ? (size_t)pl.nsplit * M * N * sizeof(float) : 0;
  return pl;
}

bool woq_stream_supported(const zt_woq_linear_args_t &a) {
  if (a.M < 1 || a.M > 16 || a.N < 1) return false;
  if (a.K % kStepK != 0 || a.n_groups <= 0 || a.K % a.n_groups != 0) return false;
  const int64_t gs = a.K / a.n_groups;
  if (gs % kStepK != 0) return false;
  if ((reinterpret_cast<uintptr_t>(a.x) | reinterpret_cast<uintptr_t>(a.wq)) & 15) return false;
  return a.K <= (1 << 30) && a.N <= (1 << 30);
}

int woq_stream_launch(const zt_woq_linear_args_t &a, cudaStream_t st) {
  const WoqStreamPlan pl = woq_stream_plan(a.M, a.N, a.K);
  if (pl.nsplit > 1) {
    ZT_REQUIRE(a.workspace != nullptr && a.workspace_bytes >= ZT_WOQ_COUNTER_BYTES + pl.partial_bytes,
               ZT_WORKSPACE_TOO_SMALL, "zt_woq_linear: workspace of %zu bytes is smaller than the %zu required",
               a.workspace_bytes, (size_t)ZT_WOQ_COUNTER_BYTES + pl.partial_bytes);
  }
  StreamParams p{};
  p.M = (int)a.M;
  p.N = (int)a.N;
  p.K = (int)a.K;
  p.x = reinterpret_cast<const __nv_bfloat16 *>(a.x);
  p.y = reinterpret_cast<__nv_bfloat16 *>(a.y);
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
  const int tile_n = pl.r == 0 ? 16 : pl.r == 1 ? 32 : 64;
  const dim3 grid((unsigned)ceil_div<int64_t>(a.N, tile_n), (unsigned)pl.nsplit);
  if (pl.mt == 1) {
    if (pl.r == 0) return launch_q<1, 0>(p, grid, st);
    if (pl.r == 1) return launch_q<1, 1>(p, grid, st);
    return launch_q<1, 2>(p, grid, st);
  }
  if (pl.r == 0) return launch_q<2, 0>(p, grid, st);
  if (pl.r == 1) return launch_q<2, 1>(p, grid, st);
  return launch_q<2, 2>(p, grid, st);
}

}  // namespace zt
