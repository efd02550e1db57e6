// Weight-only int4 linear for decode (M <= 16): the HBM-bound kernel, bulk-copy staged and
// work-balanced ("stream-K").
//
// Work.  The problem is cut into cells of 64 output columns x 128 k (one k-step, one quantisation
// group when the group size is 128).  Cells are ordered column-tile major; each of the G CTAs (one
// per SM) takes a contiguous range of total/G cells, so every SM streams the same number of weight
// bytes whatever N and K are.  A range may end inside a column tile; such a tile's partial sums go
// through a small global scratch and the last CTA to arrive at the tile adds them in CTA order
// (deterministic) and applies bias and post-ops.
//
// Memory pipeline.  One producer warp stages chunks of up to eight cells of a tile into a ring of
// shared-memory stages with tiled TMA loads (completion counted on an mbarrier).  The packed weight is
// described to TMA as a 3-D tensor (16 words of one cell's row, K/128 cells along K, N rows), so one
// instruction brings 64 rows x 8 cells = 32 KB laid out [row][cell][64 B]; the activations likewise
// ([row][cell][256 B]) and the scales / zero points of the chunk's groups ([group][64 columns]).  A
// chunk always loads the full 8-cell box (cells past the CTA's range are simply not used; rows and
// cells beyond N and K read as zero).  Nothing is
// staged through registers, so the bytes in flight per SM are bounded by shared memory (> 100 KB), not
// by occupancy.  No multicast is used.
//
// Arithmetic (16 compute warps; warp w takes cell w/2 of the chunk and 32 of its 64 columns).  Nibbles
// become bf16 pairs with one lop3 each ((w >> 4p) & 0x000f000f picks nibbles p and p+4; or-ing 0x4300
// into both halves gives 128 + u, signed nibbles are xor-ed with 8 in the same lop3 so that u = q + 8 in
// both formats) and feed mma.sync.m16n8k16 as the A operand; the activations are the B operand,
// permuted to the same (k, k+4) pairing with byte-permutes; an all-ones A operand yields sum_k x per
// cell, with which the bias of 136 is removed on the cell's partial sum and the zero point applied:
// acc += s * (part - 136 * sum) + z * sum, in fp32.  Dequantised weights are never rounded to bf16.
#include <cstdlib>
#include <mutex>
#include <type_traits>
#include <unordered_map>

#include "tc05.cuh"
#include "woq.cuh"

namespace zt {

namespace {

constexpr int kTileN = 64;        // output columns per cell
constexpr int kStepK = 128;       // k per cell
constexpr int kChunkSteps = 8;    // cells per stage
constexpr int kComputeWarps = 16;
constexpr int kThreads = 32 * (kComputeWarps + 1);
constexpr int kWRowBytes = kChunkSteps * 64;      // one weight row of a stage: [8 cells][64 B]
constexpr int kWBytes = kTileN * kWRowBytes;
constexpr int kXRowBytes = kChunkSteps * 256;     // one activation row of a stage: [8 cells][256 B]
constexpr int kMaxStages = 6;

struct SKParams {
  const __nv_bfloat16 *x;
  const int32_t *wq;
  const void *scales;
  const void *zeros;
  const void *bias;
  __nv_bfloat16 *y;
  float *partial;  // [G][2][16][64]
  int *counters;   // one per column tile, zero on entry and on exit
  int *status;
  int M, N, K;
  int gs, spg;  // group size in k and in cells
  int ksteps, ntiles;
  long long total_cells;
  int scale_dtype, bias_dtype;
  int stages, stage_bytes;
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
  if (SIGNED) {
    asm("lop3.b32 %0, %1, %2, %3, 0x6a;" : "=r"(r) : "r"(w), "n"(0x000f000f), "n"(0x43084308));
  } else {
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
__device__ __forceinline__ void compute_barrier() {
  asm volatile("bar.sync 1, %0;" ::"n"(kComputeWarps * 32) : "memory");
}

// The CTA whose cell range contains cell c, for ranges [b*total/G, (b+1)*total/G).
__device__ __forceinline__ int cta_of_cell(long long c, long long total, int G) {
  return (int)(((c + 1) * G + total - 1) / total - 1);
}

// One chunk = up to kChunkSteps consecutive cells of one column tile.
struct Chunk {
  int tile, step0, nsteps;
  bool last_of_segment;
};

// Walks the chunks of this CTA's cell range in order.  The only division is in the constructor; the
// per-chunk step is additions and compares (the loop runs once per chunk in every warp).
struct ChunkIter {
  int tile, step, ksteps;
  long long remaining;
  __device__ ChunkIter(long long c0, long long c1, int ks) : ksteps(ks), remaining(c1 - c0) {
    tile = (int)(c0 / ks);
    step = (int)(c0 - (long long)tile * ks);
  }
  __device__ bool next(Chunk &ch) {
    if (remaining <= 0) return false;
    int n = ksteps - step;                      // cells left in this column tile
    const bool tile_ends = (long long)n <= remaining && n <= kChunkSteps;
    if ((long long)n > remaining) n = (int)remaining;
    const bool range_ends = (long long)n == remaining && n <= kChunkSteps;
    if (n > kChunkSteps) n = kChunkSteps;
    ch.tile = tile;
    ch.step0 = step;
    ch.nsteps = n;
    ch.last_of_segment = tile_ends || range_ends;
    remaining -= n;
    step += n;
    if (step == ksteps) {
      step = 0;
      ++tile;
    }
    return true;
  }
};

template <int MT, bool ASYM, bool SF32>
__global__ void __launch_bounds__(kThreads, 1)
    woq_streamk_kernel(const __grid_constant__ CUtensorMap map_w8, const __grid_constant__ CUtensorMap map_x8,
                       const __grid_constant__ CUtensorMap map_s, const __grid_constant__ CUtensorMap map_z,
                       const SKParams p) {
  extern __shared__ __align__(128) unsigned char smem[];
  constexpr int kCols = MT * 8;
  constexpr int kScaleBytes = SF32 ? 4 : 2;
  constexpr int kSBytes = kChunkSteps * kTileN * kScaleBytes;  // scales of the chunk: [8 groups][64]
  constexpr int kSOff = kWBytes;
  constexpr int kZOff = kSOff + 2048;                          // zero points (same shape)
  constexpr int kXOff = kZOff + (ASYM ? 2048 : 0);             // activations: [mrows][cell][256 B]
  constexpr int kRedStride = 33;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int G = gridDim.x;
  const int mrows = min(p.M, kCols);
  float *red = reinterpret_cast<float *>(smem + (size_t)p.stages * p.stage_bytes);  // [16][kCols][33]
  uint64_t *full_bar = reinterpret_cast<uint64_t *>(red + kComputeWarps * kCols * kRedStride);
  uint64_t *empty_bar = full_bar + kMaxStages;
  __shared__ int s_ticket;

  const long long c_begin = (long long)blockIdx.x * p.total_cells / G;
  const long long c_end = (long long)(blockIdx.x + 1) * p.total_cells / G;

  if (tid == 0) {
    tc::prefetch_tensormap(&map_w8);
    tc::prefetch_tensormap(&map_x8);
    tc::prefetch_tensormap(&map_s);
    for (int s = 0; s < p.stages; ++s) {
      tc::mbar_init(&full_bar[s], 1);
      tc::mbar_init(&empty_bar[s], kComputeWarps);
    }
    tc::mbar_fence_init();
  }
  __syncthreads();

  if (warp == kComputeWarps) {
    // ---------------- producer warp ----------------
    ChunkIter iter(c_begin, c_end, p.ksteps);
    Chunk ch;
    uint32_t s = 0, ph = 0;  // ring position and its phase bit
    bool ok = true;
    while (ok && iter.next(ch)) {
      if (!tc::mbar_wait(&empty_bar[s], ph ^ 1)) {
        tc::report_timeout(p.status, kStatusProducerTimeout);
        ok = false;
        break;
      }
      unsigned char *stage = smem + (size_t)s * p.stage_bytes;
      const int n0 = ch.tile * kTileN;
      const int g0 = p.spg == 1 ? ch.step0 : ch.step0 / p.spg;
      if (lane == 0) {
        tc::mbar_expect_tx(&full_bar[s], (uint32_t)kWBytes + (uint32_t)mrows * kXRowBytes +
                                             (uint32_t)kSBytes * (ASYM ? 2u : 1u));
        tc::tma_load_3d(stage, &map_w8, &full_bar[s], 0, ch.step0, n0);
        tc::tma_load_3d(stage + kXOff, &map_x8, &full_bar[s], 0, ch.step0, 0);
        tc::tma_load_2d(stage + kSOff, &map_s, &full_bar[s], n0, g0);
        if (ASYM) tc::tma_load_2d(stage + kZOff, &map_z, &full_bar[s], n0, g0);
      }
      __syncwarp();
      if (++s == (uint32_t)p.stages) {
        s = 0;
        ph ^= 1;
      }
    }
  } else {
    // ---------------- compute warps ----------------
    const int g = lane >> 2, t = lane & 3;
    const int my_step = warp >> 1;
    const int rb = 32 * (warp & 1);  // first of this warp's 32 columns within the tile
    float acc[2][MT][4];
#pragma unroll
    for (int r = 0; r < 2; ++r)
#pragma unroll
      for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[r][m][e] = 0.f;

    ChunkIter iter(c_begin, c_end, p.ksteps);
    Chunk ch;
    uint32_t s = 0, ph = 0;
    bool ok = true;
    while (iter.next(ch)) {
      if (ok && !tc::mbar_wait(&full_bar[s], ph)) {
        tc::report_timeout(p.status, kStatusConvertTimeout);
        ok = false;
      }
      const unsigned char *stage = smem + (size_t)s * p.stage_bytes;
      if (ok && my_step < ch.nsteps) {
        // group of this warp's cell, relative to the chunk's first group (spg = cells per group)
        const int gl = p.spg == 1 ? my_step : (ch.step0 + my_step) / p.spg - ch.step0 / p.spg;
        uint4 wv[2][2];
        float sc[2][2], zp[2][2];
#pragma unroll
        for (int r = 0; r < 2; ++r)
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int row = rb + 16 * r + 8 * h + g;
            wv[r][h] = *reinterpret_cast<const uint4 *>(stage + row * kWRowBytes + my_step * 64 + 16 * t);
            const unsigned char *sp = stage + kSOff + gl * kTileN * kScaleBytes;
            sc[r][h] = SF32 ? reinterpret_cast<const float *>(sp)[row]
                            : __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(sp)[row]);
            if (ASYM) {
              const unsigned char *zq = stage + kZOff + gl * kTileN * kScaleBytes;
              zp[r][h] = SF32 ? reinterpret_cast<const float *>(zq)[row]
                              : __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(zq)[row]);
            }
          }
        float part[2][MT][4], xsum[MT][4];
#pragma unroll
        for (int m = 0; m < MT; ++m)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            xsum[m][e] = 0.f;
            part[0][m][e] = 0.f;
            part[1][m][e] = 0.f;
          }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint32_t bf[MT][4];
#pragma unroll
          for (int m = 0; m < MT; ++m) {
            const int col = m * 8 + g;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (col < mrows)
              v = *reinterpret_cast<const uint4 *>(stage + kXOff + col * kXRowBytes + my_step * 256 + 64 * t + 16 * i);
            bf[m][0] = prmt(v.x, v.z, 0x5410);  // (x0, x4)
            bf[m][1] = prmt(v.x, v.z, 0x7632);  // (x1, x5)
            bf[m][2] = prmt(v.y, v.w, 0x5410);  // (x2, x6)
            bf[m][3] = prmt(v.y, v.w, 0x7632);  // (x3, x7)
            constexpr uint32_t kOnes = 0x3f803f80u;
            mma_bf16_16816(xsum[m], kOnes, kOnes, kOnes, kOnes, bf[m][0], bf[m][1]);
            mma_bf16_16816(xsum[m], kOnes, kOnes, kOnes, kOnes, bf[m][2], bf[m][3]);
          }
#pragma unroll
          for (int r = 0; r < 2; ++r) {
            const uint32_t wa = (i == 0) ? wv[r][0].x : (i == 1) ? wv[r][0].y : (i == 2) ? wv[r][0].z : wv[r][0].w;
            const uint32_t wb = (i == 0) ? wv[r][1].x : (i == 1) ? wv[r][1].y : (i == 2) ? wv[r][1].z : wv[r][1].w;
            uint32_t ra[4], rbv[4];
#pragma unroll
            for (int pp = 0; pp < 4; ++pp) {
              ra[pp] = nib_pair_to_bf16x2<!ASYM>(wa >> (4 * pp));
              rbv[pp] = nib_pair_to_bf16x2<!ASYM>(wb >> (4 * pp));
            }
#pragma unroll
            for (int m = 0; m < MT; ++m) {
              mma_bf16_16816(part[r][m], ra[0], rbv[0], ra[1], rbv[1], bf[m][0], bf[m][1]);
              mma_bf16_16816(part[r][m], ra[2], rbv[2], ra[3], rbv[3], bf[m][2], bf[m][3]);
            }
          }
        }
#pragma unroll
        for (int m = 0; m < MT; ++m)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const float sxv = xsum[m][e];
#pragma unroll
            for (int r = 0; r < 2; ++r)
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                float v = sc[r][h] * fmaf(-136.f, sxv, part[r][m][2 * h + e]);
                if (ASYM) v = fmaf(zp[r][h], sxv, v);
                acc[r][m][2 * h + e] += v;
              }
          }
      }
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(&empty_bar[s]);
      if (++s == (uint32_t)p.stages) {
        s = 0;
        ph ^= 1;
      }

      if (ch.last_of_segment) {
        // ---- the segment of tile ch.tile is complete: combine the warps, then finish or hand over ----
#pragma unroll
        for (int r = 0; r < 2; ++r)
#pragma unroll
          for (int m = 0; m < MT; ++m)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int nl = 16 * r + 8 * (e >> 1) + g;  // within this warp's 32 columns
              const int ml = m * 8 + 2 * t + (e & 1);
              red[(warp * kCols + ml) * kRedStride + nl] = acc[r][m][e];
              acc[r][m][e] = 0.f;
            }
        compute_barrier();
        const int n0 = ch.tile * kTileN;
        const long long t_first = (long long)ch.tile * p.ksteps;
        const int b_first = cta_of_cell(t_first, p.total_cells, G);
        const int b_last = cta_of_cell(t_first + p.ksteps - 1, p.total_cells, G);
        const bool shared_tile = b_first != b_last;
        const int nl = tid & 63;       // column within the tile
        const int half = nl >> 5;      // which row-half's warps hold it
        const int n = n0 + nl;
        float mine[2] = {0.f, 0.f};    // up to two output rows per thread (M <= 16, 8 rows per pass)
#pragma unroll
        for (int pass = 0; pass < 2; ++pass) {
          const int ml = (tid >> 6) + 8 * pass;
          if (ml < p.M) {
            float v = 0.f;
#pragma unroll
            for (int w8 = 0; w8 < kComputeWarps / 2; ++w8)
              v += red[((2 * w8 + half) * kCols + ml) * kRedStride + (nl & 31)];
            mine[pass] = v;
          }
        }
        bool finish = true;
        if (shared_tile) {
          const int slot = (c_begin / p.ksteps == ch.tile) ? 0 : 1;
          float *dst = p.partial + ((size_t)(blockIdx.x * 2 + slot) * 16) * kTileN;
#pragma unroll
          for (int pass = 0; pass < 2; ++pass) {
            const int ml = (tid >> 6) + 8 * pass;
            if (ml < p.M) dst[ml * kTileN + nl] = mine[pass];
          }
          __threadfence();
          compute_barrier();
          if (tid == 0) s_ticket = atomicAdd(&p.counters[ch.tile], 1);
          compute_barrier();
          finish = (s_ticket == b_last - b_first);
          if (finish) {
            __threadfence();
            if (tid == 0) p.counters[ch.tile] = 0;
#pragma unroll
            for (int pass = 0; pass < 2; ++pass) {
              const int ml = (tid >> 6) + 8 * pass;
              if (ml < p.M) {
                float v = 0.f;
                for (int b = b_first; b <= b_last; ++b) {
                  const long long bs = (long long)b * p.total_cells / G;
                  const int bslot = (bs / p.ksteps == ch.tile) ? 0 : 1;
                  v += __ldcg(p.partial + ((size_t)(b * 2 + bslot) * 16 + ml) * kTileN + nl);
                }
                mine[pass] = v;
              }
            }
          }
        }
        if (finish && n < p.N) {
#pragma unroll
          for (int pass = 0; pass < 2; ++pass) {
            const int ml = (tid >> 6) + 8 * pass;
            if (ml < p.M) {
              float v = mine[pass];
              if (p.bias) v += load_as_float(p.bias, n, p.bias_dtype);
              const int64_t idx = (int64_t)ml * p.N + n;
              v = apply_post_ops(v, p.post, idx, ZT_BF16);
              p.y[idx] = __float2bfloat16_rn(v);
            }
          }
        }
        compute_barrier();  // red[] and s_ticket are reused by the next segment
      }
    }
  }
}

size_t streamk_stage_bytes(int mt, int M, bool asym) {
  const int mrows = M < mt * 8 ? M : mt * 8;
  size_t b = (size_t)kWBytes + 2048 * (asym ? 2 : 1) + (size_t)mrows * kXRowBytes;
  return (b + 127) / 128 * 128;
}
size_t streamk_tail_bytes(int mt) {
  return (size_t)kComputeWarps * mt * 8 * 33 * sizeof(float) + 2 * kMaxStages * sizeof(uint64_t) + 64;
}

struct Maps {
  CUtensorMap w8, x8, s, z;
};

struct MapKey {
  const void *ptr;
  uint64_t d0, d1, d2, s0, s1;
  uint32_t b0, b1, b2;
  int dtype;
  bool operator==(const MapKey &o) const {
    return ptr == o.ptr && d0 == o.d0 && d1 == o.d1 && d2 == o.d2 && s0 == o.s0 && s1 == o.s1 && b0 == o.b0 &&
           b1 == o.b1 && b2 == o.b2 && dtype == o.dtype;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey &k) const {
    return std::hash<const void *>()(k.ptr) ^ (k.d0 * 1315423911u) ^ (k.d1 << 17) ^ (k.d2 << 29) ^ k.b1 ^ (k.b2 << 9) ^
           (k.s0 << 3) ^ (size_t)k.dtype;
  }
};

// Tensor maps depend only on (pointer, element type, shape, strides, box); they are memoised per
// process.  The element type and strides are part of the key: the allocator reuses addresses.
int cached_map(CUtensorMap *out, const void *ptr, CUtensorMapDataType dt, int rank, const uint64_t *dims,
               const uint64_t *strides, const uint32_t *box) {
  static std::mutex mu;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  const MapKey key{ptr,    dims[0], dims[1], rank > 2 ? dims[2] : 0, strides[0], rank > 2 ? strides[1] : 0,
                   box[0], box[1],  rank > 2 ? box[2] : 0, (int)dt};
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it != cache.end()) {
    *out = it->second;
    return ZT_SUCCESS;
  }
  int rc = make_tensor_map(out, ptr, dt, rank, dims, strides, box, false);
  if (rc != ZT_SUCCESS) return rc;
  if (cache.size() > 8192) cache.clear();
  cache.emplace(key, *out);
  return ZT_SUCCESS;
}

int build_maps(const zt_woq_linear_args_t &a, int mrows, Maps &m) {
  const uint64_t ksteps = (uint64_t)a.K / kStepK;
  {  // packed weight: [N rows][K/128 cells][16 words]
    const uint64_t dims[3] = {16, ksteps, (uint64_t)a.N};
    const uint64_t strides[2] = {64, (uint64_t)a.K / 2};
    const uint32_t box[3] = {16, kChunkSteps, kTileN};
    int rc = cached_map(&m.w8, a.wq, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, dims, strides, box);
    if (rc != ZT_SUCCESS) return rc;
  }
  {  // activations: [M rows][K/128 cells][128 bf16]
    const uint64_t dims[3] = {128, ksteps, (uint64_t)a.M};
    const uint64_t strides[2] = {256, (uint64_t)a.K * 2};
    const uint32_t box[3] = {128, kChunkSteps, (uint32_t)mrows};
    int rc = cached_map(&m.x8, a.x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, dims, strides, box);
    if (rc != ZT_SUCCESS) return rc;
  }
  {  // scales / zero points: [groups][N]
    const bool f32 = a.scale_dtype == ZT_F32;
    const CUtensorMapDataType dt = f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    const uint64_t dims[2] = {(uint64_t)a.N, (uint64_t)a.n_groups};
    const uint64_t strides[1] = {(uint64_t)a.N * (f32 ? 4 : 2)};
    const uint32_t box[2] = {kTileN, kChunkSteps};
    int rc = cached_map(&m.s, a.scales, dt, 2, dims, strides, box);
    if (rc != ZT_SUCCESS) return rc;
    if (a.zeros) {
      rc = cached_map(&m.z, a.zeros, dt, 2, dims, strides, box);
      if (rc != ZT_SUCCESS) return rc;
    } else {
      m.z = m.s;
    }
  }
  return ZT_SUCCESS;
}

template <int MT, bool ASYM, bool SF32>
int launch(const Maps &m, const SKParams &p, int grid, size_t smem_bytes, cudaStream_t st) {
  auto kern = woq_streamk_kernel<MT, ASYM, SF32>;
  static bool configured = false;
  if (!configured) {
    ZT_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024));
    configured = true;
  }
  kern<<<grid, kThreads, smem_bytes, st>>>(m.w8, m.x8, m.s, m.z, p);
  return launch_status("woq_streamk_kernel");
}

template <int MT>
int launch_q(const Maps &m, const SKParams &p, int grid, size_t smem_bytes, cudaStream_t st) {
  const bool asym = p.zeros != nullptr, sf32 = p.scale_dtype == ZT_F32;
  if (asym)
    return sf32 ? launch<MT, true, true>(m, p, grid, smem_bytes, st) : launch<MT, true, false>(m, p, grid, smem_bytes, st);
  return sf32 ? launch<MT, false, true>(m, p, grid, smem_bytes, st) : launch<MT, false, false>(m, p, grid, smem_bytes, st);
}

}  // namespace

size_t woq_streamk_workspace_bytes() { return (size_t)sm_count() * 2 * 16 * kTileN * sizeof(float); }

bool woq_streamk_supported(const zt_woq_linear_args_t &a) {
  if (a.M < 1 || a.M > 16 || a.N < 1) return false;
  if (a.K % kStepK != 0 || a.n_groups <= 0 || a.K % a.n_groups != 0) return false;
  const int64_t gs = a.K / a.n_groups;
  if (gs % kStepK != 0) return false;
  const int ssz = a.scale_dtype == ZT_F32 ? 4 : 2;
  if ((a.N * ssz) % 16 != 0) return false;  // TMA row pitch of the scale table must be a multiple of 16 bytes
  const uintptr_t ptrs = reinterpret_cast<uintptr_t>(a.x) | reinterpret_cast<uintptr_t>(a.wq) |
                         reinterpret_cast<uintptr_t>(a.scales) | reinterpret_cast<uintptr_t>(a.zeros);
  if (ptrs & 15) return false;
  if (ceil_div<int64_t>(a.N, kTileN) * (int64_t)sizeof(int) > ZT_WOQ_COUNTER_BYTES) return false;
  return a.K <= (1 << 30) && a.N <= (1 << 30);
}

int woq_streamk_launch(const zt_woq_linear_args_t &a, cudaStream_t st) {
  const size_t need = ZT_WOQ_COUNTER_BYTES + woq_streamk_workspace_bytes();
  ZT_REQUIRE(a.workspace != nullptr && a.workspace_bytes >= need, ZT_WORKSPACE_TOO_SMALL,
             "zt_woq_linear: workspace of %zu bytes is smaller than the %zu required", a.workspace_bytes, need);
  SKParams p{};
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
  p.spg = p.gs / kStepK;
  p.ksteps = (int)(a.K / kStepK);
  p.ntiles = (int)ceil_div<int64_t>(a.N, kTileN);
  p.total_cells = (long long)p.ntiles * p.ksteps;
  p.counters = reinterpret_cast<int *>(a.workspace);
  p.partial = reinterpret_cast<float *>(reinterpret_cast<char *>(a.workspace) + ZT_WOQ_COUNTER_BYTES);
  p.status = device_status_ptr();
  p.post = to_dev(a.post);
  const int mt = a.M <= 8 ? 1 : 2;
  const size_t stage = streamk_stage_bytes(mt, (int)a.M, a.zeros != nullptr);
  const size_t tail = streamk_tail_bytes(mt);
  int stages = (int)((216 * 1024 - tail) / stage);
  if (stages > kMaxStages) stages = kMaxStages;
  ZT_REQUIRE(stages >= 2, ZT_UNSUPPORTED, "zt_woq_linear: stream-K stage of %zu bytes does not fit twice", stage);
  p.stages = stages;
  p.stage_bytes = (int)stage;
  int grid = sm_count();
  if ((long long)grid > p.total_cells) grid = (int)p.total_cells;
  const size_t smem_bytes = (size_t)stages * stage + tail;
  Maps maps;
  const int mrows = (int)(a.M < mt * 8 ? a.M : mt * 8);
  int rc = build_maps(a, mrows, maps);
  if (rc != ZT_SUCCESS) return rc;
  return mt == 1 ? launch_q<1>(maps, p, grid, smem_bytes, st) : launch_q<2>(maps, p, grid, smem_bytes, st);
}

}  // namespace zt
