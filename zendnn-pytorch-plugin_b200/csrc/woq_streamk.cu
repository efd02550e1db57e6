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
// chunk always loads the full box (cells past the CTA's range are simply not used; rows and cells
// beyond N and K read as zero).  Nothing is staged through registers, so the bytes in flight per SM
// are bounded by shared memory (> 100 KB), not by occupancy.  Loads are plain per-CTA loads.
//
// Arithmetic: integer tensor-core MMAs on exact operands.  A packed word holds eight nibbles;
// (w & 0x0f0f0f0f) is four of them as bytes and ((w >> 4) & 0x0f0f0f0f) the other four (signed nibbles
// are xor-ed with 8 in the same lop3, so u = q + 8 in both formats): three ALU operations per eight
// weights, and the bytes are the A operand of mma.sync.m16n8k32 (u8 x s8 -> s32) as they stand.  The
// activations are made integer once per staged cell by converter warps: the 128 bf16 values of one
// token's cell are scaled by the power of two that puts the largest below 2^21 (tokens <= 2) or 2^14
// (more tokens), rounded to an integer X and split into signed base-256 digits X = d2 2^16 + d1 2^8 + d0.
// bf16 values carry 8 significant bits, so every value within 2^-13 (2^-6) of the cell's largest is
// represented exactly and the rest to 2^-22 (2^-15) of the largest.  Each (token, digit) is one column
// of the B operand (n = 8 per MMA), stored in the fragment order the MMA wants, next to the column's
// power of two and its digit sum.  The accumulators start at -8 * (digit sum), which removes the +8 of u
// exactly; a cell's integer result is converted once and scaled in fp32:
// acc[col] += s * 2^e(col) * float(part[col]) (+ z * sum_k x), and a token's columns are added at the
// end.  Dequantised weights are never rounded and products are exact integers.
//
// Launch overlap.  The kernel is launched with programmatic stream serialisation: it lets its successor
// start as soon as every CTA is running, and itself stages the first weight chunks before waiting for
// its predecessor (only the activations, the scratch and the output depend on earlier work; weights,
// scales and zero points must not be written by the kernel launched directly before this one on the
// same stream unless that kernel completes normally, which every kernel except this one does).
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
constexpr int kComputeWarps = 16;
// Warps: 16 compute, weight producer, activation producer, epilogue, converters -- five converters up to two
// tokens (24 warps; a chunk needs one or two of them, so the groups take chunks in turn), eight for three and
// four tokens (27 warps: still two groups).
__host__ __device__ constexpr int sk_threads(int conv_warps) { return 32 * (kComputeWarps + 3 + conv_warps); }
constexpr int kMaxStages = 8;   // weight stages and activation slots, each
constexpr int kRedStride = 33;
constexpr int kMaxTokens = 4;

// NB = 8-column blocks of the B operand: columns = tokens x digits (3 digits up to 2 tokens, else 2).
__host__ __device__ constexpr int digits_for(int m) { return m <= 2 ? 3 : 2; }
__host__ __device__ constexpr int col_blocks(int m) { return (m * digits_for(m) + 7) / 8; }
// Cells per stage and 16-row blocks per compute warp: one cell x 32 columns per warp with 8-cell chunks,
// one cell x 16 columns with 4-cell chunks (more than 8 tokens: twice the activation bytes per cell).
__host__ __device__ constexpr int chunk_steps(int nb) { return nb <= 2 ? 8 : 4; }
__host__ __device__ constexpr int row_blocks(int nb) { return nb <= 2 ? 2 : 1; }

struct SKParams {
  const __nv_bfloat16 *x;
  const int32_t *wq;
  const void *scales;
  const void *zeros;
  const void *bias;
  __nv_bfloat16 *y;
  float *partial;  // [G][2][16][64]
  int *counters;   // two per column tile ([2][ntiles]: arrived, published), zero on entry and on exit
  int *status;
  int M, N, K;
  int gs, spg;  // group size in k and in cells
  uint32_t spg_mul;  // 0 when spg == 1, else floor(2^32 / spg) + 1: n / spg == umulhi(n, spg_mul) for n * spg < 2^32
  int ksteps, ntiles;
  long long total_cells;
  int scale_dtype, bias_dtype;
  int stages, stage_bytes;   // ring of weight stages
  int xslots, xslot_bytes;   // ring of activation slots
  TimelineSink timeline;
  PostOpsDev post;
};

// Four nibbles of w as bytes: u = q + 8 for signed nibbles (and-then-xor), u itself for unsigned ones.
// mask = 0x0f0f0f0f and flip = 0x08080808 are passed in registers: lop3 takes one immediate only, and
// constants known to the compiler get re-materialised next to every use when registers are short.
template <bool SIGNED>
__device__ __forceinline__ uint32_t nib_bytes(uint32_t w, uint32_t mask, uint32_t flip) {
  uint32_t r;
  if (SIGNED) {
    asm("lop3.b32 %0, %1, %2, %3, 0x6a;" : "=r"(r) : "r"(w), "r"(mask), "r"(flip));
  } else {
    r = w & mask;
  }
  return r;
}
__device__ __forceinline__ void mma_u8s8_16832(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}
__device__ __forceinline__ int byte_sum(uint32_t v, int acc) {  // acc + the four signed bytes of v
  int r;
  asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(r) : "r"(v), "r"(0x01010101), "r"(acc));
  return r;
}

// The CTA whose cell range contains cell c, for ranges [b*total/G, (b+1)*total/G).
__device__ __forceinline__ int cta_of_cell(long long c, long long total, int G) {
  return (int)(((c + 1) * G + total - 1) / total - 1);
}

// One chunk = up to CS consecutive cells of one column tile.
struct Chunk {
  int tile, step0, nsteps;
  bool last_of_segment;
};

// Walks the chunks of this CTA's cell range in order.  The only division is in the constructor; the
// per-chunk step is a handful of 32-bit additions and compares (it runs once per chunk in every warp).
template <int CS>
struct ChunkIter {
  int tile, step, ksteps, remaining;
  __device__ ChunkIter(long long c0, long long c1, int ks) : ksteps(ks), remaining((int)(c1 - c0)) {
    tile = (int)(c0 / ks);
    step = (int)(c0 - (long long)tile * ks);
  }
  __device__ bool next(Chunk &ch) {
    if (remaining <= 0) return false;
    int n = min(min(ksteps - step, remaining), CS);
    ch.tile = tile;
    ch.step0 = step;
    ch.nsteps = n;
    remaining -= n;
    step += n;
    const bool tile_ends = step == ksteps;
    ch.last_of_segment = tile_ends || remaining == 0;
    if (tile_ends) {
      step = 0;
      ++tile;
    }
    return true;
  }
};

template <int NB, int CW, bool ASYM, bool SF32>
__global__ void __launch_bounds__(sk_threads(CW), 1)
    woq_streamk_kernel(const __grid_constant__ CUtensorMap map_w8, const __grid_constant__ CUtensorMap map_x8,
                       const __grid_constant__ CUtensorMap map_s, const __grid_constant__ CUtensorMap map_z,
                       const SKParams p) {
  extern __shared__ __align__(128) unsigned char smem[];
  constexpr int NC = 8 * NB;                  // B-operand columns held (tokens x digits, padded)
  constexpr int CS = chunk_steps(NB);         // cells per chunk
  constexpr int R = row_blocks(NB);           // 16-row blocks per compute warp
  constexpr int kWarpsPerCell = kComputeWarps / CS;
  constexpr int kConvWarps = CW;
  constexpr int kThreads = sk_threads(CW);
  constexpr int kWRowBytes = CS * 64;         // one weight row of a stage: [CS cells][64 B]
  constexpr int kWBytes = kTileN * kWRowBytes;
  constexpr int kXRowBytes = CS * 256;        // one activation row of a slot: [CS cells][256 B]
  constexpr int kScaleBytes = SF32 ? 4 : 2;
  constexpr int kSBytes = CS * kTileN * kScaleBytes;  // scales of the chunk: [CS groups][64]
  // weight stage: packed weights, scales, zero points
  constexpr int kSOff = kWBytes;
  constexpr int kZOff = kSOff + CS * 256;
  // activation slot: per (cell, column) tables (2^e, -8 * digit sum, sum of x), staged bf16, digit fragments
  constexpr int kEBytes = CS * NC * 4;
  constexpr int kXOff = (ASYM ? 3 : 2) * kEBytes;              // [M][cell][256 B] bf16
  using Iter = ChunkIter<CS>;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int G = gridDim.x;
  const int nd = digits_for(p.M);
  const int ncols = p.M * nd;
  const int kDOff = kXOff + p.M * kXRowBytes;                  // digit fragments: [cell][word pair][column][t][16 B]
  // A chunk's CS * M (token, cell) conversions take four lanes each; conv_group warps share one chunk and
  // the groups take chunks in turn, so that a small chunk's conversion latency is spread over several chunks.
  // A group must see every phase of the barriers it waits on, so it owns fixed slots: the number of groups
  // divides the number of slots.
  const int conv_group = min(kConvWarps, (CS * p.M + 7) / 8);
  int conv_ngroups = kConvWarps / conv_group;
  while (p.xslots % conv_ngroups != 0) --conv_ngroups;
  unsigned char *xring = smem + (size_t)p.stages * p.stage_bytes;
  // Two reduction buffers [16 warps][rrows][33]: rows are the columns themselves with three digits, tokens else.
  const int rrows = nd == 3 ? ncols : p.M;
  const int red_buf_floats = kComputeWarps * rrows * kRedStride;
  float *red = reinterpret_cast<float *>(xring + (size_t)p.xslots * p.xslot_bytes);
  uint64_t *full_bar = reinterpret_cast<uint64_t *>(red + 2 * red_buf_floats);
  uint64_t *empty_bar = full_bar + kMaxStages;   // weight stage consumed by all compute warps
  uint64_t *xfull_bar = empty_bar + kMaxStages;  // staged activations have landed
  uint64_t *frag_bar = xfull_bar + kMaxStages;   // digit fragments and tables are written
  uint64_t *xempty_bar = frag_bar + kMaxStages;  // activation slot consumed by all compute warps
  uint64_t *red_full = xempty_bar + kMaxStages;  // [2] every compute warp has written its sums
  uint64_t *red_free = red_full + 2;             // [2] the epilogue warp has read them

  const long long c_begin = (long long)blockIdx.x * p.total_cells / G;
  const long long c_end = (long long)(blockIdx.x + 1) * p.total_cells / G;

  // The weight producer sets up its own barriers and fills the ring once before anybody else is ready:
  // weights do not depend on earlier work, and the first bytes take the longest to arrive.
  stamp(p.timeline, blockIdx.x, 0);
  Iter w_iter(c_begin, c_end, p.ksteps);
  constexpr uint32_t kWTxBytes = (uint32_t)kWBytes + (uint32_t)kSBytes * (ASYM ? 2u : 1u);
  int w_pre = 0;
  if (warp == kComputeWarps) {
    if (lane == 0) {
      tc::prefetch_tensormap(&map_w8);
      tc::prefetch_tensormap(&map_s);
      for (int s = 0; s < kMaxStages; ++s) {
        tc::mbar_init(&full_bar[s], 1);
        tc::mbar_init(&empty_bar[s], kComputeWarps);
      }
      tc::mbar_fence_init();
    }
    __syncwarp();
    Chunk ch;
    while (w_pre < p.stages && w_iter.next(ch)) {
      if (lane == 0) {
        unsigned char *stage = smem + (size_t)w_pre * p.stage_bytes;
        const int n0 = ch.tile * kTileN;
        const int g0 = p.spg == 1 ? ch.step0 : ch.step0 / p.spg;
        tc::mbar_expect_tx(&full_bar[w_pre], kWTxBytes);
        tc::tma_load_3d(stage, &map_w8, &full_bar[w_pre], 0, ch.step0, n0);
        tc::tma_load_2d(stage + kSOff, &map_s, &full_bar[w_pre], n0, g0);
        if (ASYM) tc::tma_load_2d(stage + kZOff, &map_z, &full_bar[w_pre], n0, g0);
      }
      ++w_pre;
    }
    if (lane == 0) stamp_here(p.timeline, blockIdx.x, 1);
  }
  if (tid == 0) {
    tc::prefetch_tensormap(&map_x8);
    for (int s = 0; s < kMaxStages; ++s) {
      tc::mbar_init(&xfull_bar[s], 1);
      tc::mbar_init(&frag_bar[s], conv_group);
      tc::mbar_init(&xempty_bar[s], kComputeWarps);
    }
    for (int b = 0; b < 2; ++b) {
      tc::mbar_init(&red_full[b], kComputeWarps);
      tc::mbar_init(&red_free[b], 1);
    }
    tc::mbar_fence_init();
  }
  // table entries of columns that do not exist are read (and meet zero sums): keep them zero
  {
    constexpr int kWords = (ASYM ? 3 : 2) * CS * NC;
    for (int i = tid; i < p.xslots * kWords; i += kThreads) {
      const int s = i / kWords, r = i - s * kWords;
      reinterpret_cast<float *>(xring + (size_t)s * p.xslot_bytes)[r] = 0.f;
    }
  }
  __syncthreads();
  grid_launch_dependents();

  if (warp == kComputeWarps) {
    // ---------------- weight producer: never touches anything an earlier kernel writes ----------------
    Chunk ch;
    uint32_t s = 0, ph = 1;   // the ring has been filled once (or the range is exhausted)
    while (w_iter.next(ch)) {
      if (!tc::mbar_wait_suspend(&empty_bar[s], ph ^ 1, 300)) {
        tc::report_timeout(p.status, kStatusProducerTimeout);
        break;
      }
      if (lane == 0) {
        unsigned char *stage = smem + (size_t)s * p.stage_bytes;
        const int n0 = ch.tile * kTileN;
        const int g0 = p.spg == 1 ? ch.step0 : ch.step0 / p.spg;
        tc::mbar_expect_tx(&full_bar[s], kWTxBytes);
        tc::tma_load_3d(stage, &map_w8, &full_bar[s], 0, ch.step0, n0);
        tc::tma_load_2d(stage + kSOff, &map_s, &full_bar[s], n0, g0);
        if (ASYM) tc::tma_load_2d(stage + kZOff, &map_z, &full_bar[s], n0, g0);
      }
      __syncwarp();
      if (++s == (uint32_t)p.stages) {
        s = 0;
        ph ^= 1;
      }
    }
  } else if (warp == kComputeWarps + 1) {
    // ---------------- activation producer: its own, deeper ring of small slots ----------------
    grid_dependency_wait();
    if (lane == 0) stamp_here(p.timeline, blockIdx.x, 2);
    Iter iter(c_begin, c_end, p.ksteps);
    Chunk ch;
    uint32_t s = 0, ph = 0;
    while (iter.next(ch)) {
      if (!tc::mbar_wait_suspend(&xempty_bar[s], ph ^ 1, 300)) {
        tc::report_timeout(p.status, kStatusProducerTimeout);
        break;
      }
      if (lane == 0) {
        tc::mbar_expect_tx(&xfull_bar[s], (uint32_t)p.M * kXRowBytes);
        tc::tma_load_3d(xring + (size_t)s * p.xslot_bytes + kXOff, &map_x8, &xfull_bar[s], 0, ch.step0, 0);
      }
      __syncwarp();
      if (++s == (uint32_t)p.xslots) {
        s = 0;
        ph ^= 1;
      }
    }
  } else if (warp == kComputeWarps + 2) {
    // ---------------- epilogue warp: finishes the segments while the compute warps go on ----------------
    // A tile shared by several CTAs is finished by the last of them to reach it.  Roles are drawn from an
    // arrival counter as soon as the segment's turn comes (the atomic's latency overlaps the compute warps'
    // last chunk); the others publish their partial sums and bump a second counter, for which the finisher
    // waits (bounded) before it adds the partial sums in CTA order.
    grid_dependency_wait();   // scratch, counters and output are shared with earlier work
    Iter iter(c_begin, c_end, p.ksteps);
    Chunk ch;
    uint32_t buf = 0, bph = 0;
    bool ok = true;
    int *arrived = p.counters, *published = p.counters + p.ntiles;
    const int nrow = nd == 2 ? 1 : 3;
    while (iter.next(ch)) {
      if (!ch.last_of_segment) continue;
      const int n0 = ch.tile * kTileN;
      const long long t_first = (long long)ch.tile * p.ksteps;
      const int b_first = cta_of_cell(t_first, p.total_cells, G);
      const int b_last = cta_of_cell(t_first + p.ksteps - 1, p.total_cells, G);
      const bool shared_tile = b_first != b_last;
      int ticket = 0;
      if (shared_tile && lane == 0) ticket = atomicAdd(&arrived[ch.tile], 1);
      float bias_v[2] = {0.f, 0.f};
      if (p.bias) {
#pragma unroll
        for (int half = 0; half < 2; ++half)
          if (n0 + lane + 32 * half < p.N) bias_v[half] = load_as_float(p.bias, n0 + lane + 32 * half, p.bias_dtype);
      }
      ticket = __shfl_sync(0xffffffffu, ticket, 0);
      const bool finisher = !shared_tile || ticket == b_last - b_first;
      // A CTA has two scratch slots: 0 for the tile its range starts in, 1 for the tile it ends in.  Every
      // CTA of a shared tile but the first starts inside the tile; the first does only if it starts on it.
      const int slot = (c_begin / p.ksteps == ch.tile) ? 0 : 1;
      const int first_slot = ((long long)b_first * p.total_cells / G >= t_first) ? 0 : 1;
      // The usual shared tile has one other CTA, which was there long ago: fetch its partial sums now, while
      // the compute warps are still on this segment.
      const bool early = shared_tile && finisher && b_last - b_first == 1 && p.M <= 8;
      float other[2][8];
#pragma unroll
      for (int half = 0; half < 2; ++half)
#pragma unroll
        for (int j = 0; j < 8; ++j) other[half][j] = 0.f;
      if (ok && shared_tile && finisher) {
        // wait until every other CTA of the tile has published
        bool seen = false;
        for (uint32_t i = 0; i < tc::kSpinLimit && !seen; ++i) {
          int v = 0;
          if (lane == 0) asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(published + ch.tile) : "memory");
          seen = __shfl_sync(0xffffffffu, v, 0) == b_last - b_first;
          if (!seen && i > 16) __nanosleep(200);
        }
        if (!seen) {
          tc::report_timeout(p.status, kStatusEpilogueTimeout);
          ok = false;
        }
        if (ok && early) {
          const int b = b_first == (int)blockIdx.x ? b_last : b_first;
          const float *src = p.partial + ((size_t)(b * 2 + (b == b_first ? first_slot : 0)) * 16) * kTileN;
#pragma unroll
          for (int half = 0; half < 2; ++half)
#pragma unroll
            for (int j = 0; j < 8; ++j)
              if (j < p.M) other[half][j] = __ldcg(src + j * kTileN + lane + 32 * half);
        }
      }
      if (ok && !tc::mbar_wait_suspend(&red_full[buf], bph, 400)) {
        tc::report_timeout(p.status, kStatusEpilogueTimeout);
        ok = false;
      }
      if (ok) {
        const float *rb = red + (size_t)buf * red_buf_floats;
        float *mine = p.partial + ((size_t)(blockIdx.x * 2 + slot) * 16) * kTileN;
        // a lane finishes columns lane and lane + 32 of the tile, one token at a time
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int nl = lane + 32 * half;
          const int sub = nl / (16 * R), nw = nl % (16 * R);   // which of a cell's warps holds the column, and where
          const int n = n0 + nl;
#pragma unroll 2
          for (int ml = 0; ml < p.M; ++ml) {
            // all the loads first (they are independent), then the sum in a fixed order
            float part[3][CS];
#pragma unroll
            for (int rr = 0; rr < 3; ++rr)
#pragma unroll
              for (int cell = 0; cell < CS; ++cell)
                part[rr][cell] = rr < nrow ? rb[((cell * kWarpsPerCell + sub) * rrows + nrow * ml + rr) * kRedStride + nw]
                                           : 0.f;
            float own = 0.f;
#pragma unroll
            for (int rr = 0; rr < 3; ++rr)
#pragma unroll
              for (int cell = 0; cell < CS; ++cell) own += part[rr][cell];
            if (!finisher) {
              mine[ml * kTileN + nl] = own;
            } else if (n < p.N) {
              float v = own;
              if (early) {
                float o = 0.f;   // ml < 8 here; a select chain keeps other[][] in registers
#pragma unroll
                for (int j = 0; j < 8; ++j)
                  if (j == ml) o = other[half][j];
                v = b_first == (int)blockIdx.x ? own + o : o + own;   // CTA order
              } else if (shared_tile) {
                // partial sums in CTA order, own term in its place; four loads in flight at a time
                v = 0.f;
                for (int b0 = b_first; b0 <= b_last; b0 += 4) {
                  float term[4];
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    const int b = b0 + j;
                    term[j] = 0.f;
                    if (b <= b_last && b != (int)blockIdx.x)
                      term[j] = __ldcg(p.partial + ((size_t)(b * 2 + (b == b_first ? first_slot : 0)) * 16 + ml) * kTileN + nl);
                    if (b == (int)blockIdx.x) term[j] = own;
                  }
#pragma unroll
                  for (int j = 0; j < 4; ++j) v += term[j];
                }
              }
              v += bias_v[half];
              const int64_t idx = (int64_t)ml * p.N + n;
              v = apply_post_ops(v, p.post, idx, ZT_BF16);
              p.y[idx] = __float2bfloat16_rn(v);
            }
          }
        }
        if (shared_tile) {
          if (!finisher) {
            __threadfence();
            __syncwarp();
            if (lane == 0) atomicAdd(&published[ch.tile], 1);
          } else if (lane == 0) {   // both counters return to zero for the next launch
            arrived[ch.tile] = 0;
            published[ch.tile] = 0;
          }
        }
      }
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(&red_free[buf]);
      buf ^= 1;
      if (buf == 0) bph ^= 1;
    }
    if (lane == 0) stamp_here(p.timeline, blockIdx.x, 7);
  } else if (warp > kComputeWarps + 2) {
    // ---------------- converter warps: bf16 activations -> integer digit fragments ----------------
    // Four lanes per (token, cell); a lane converts four of the cell's sixteen 8-value pieces.
    const int cw = warp - kComputeWarps - 3;
    const int my_group = cw / conv_group, my_slot = cw - my_group * conv_group;   // warps past the last group idle
    int turn = 0;                                                                   // group whose chunk this is
    const int q = lane >> 2, sub = lane & 3;
    const uint32_t qmask = 0xfu << (lane & 28);
    const int sh = nd == 3 ? 20 : 13;                       // |X| < 2^(sh + 1)
    // 1.5 * 2^23 + 0x8080: after the add, bytes 0 and 1 of the float hold digits 0 and 1 in excess 128 and
    // bits 16..22 hold 0x40 + digit 2
    const float magic = 12582912.f + 32896.f;
    Iter iter(c_begin, c_end, p.ksteps);
    Chunk ch;
    uint32_t s = 0, ph = 0;
    bool ok = true;
    while (iter.next(ch)) {
      const bool mine = turn == my_group;
      if (++turn == conv_ngroups) turn = 0;
      if (mine && ok && !tc::mbar_wait_suspend(&xfull_bar[s], ph, 300)) {
        tc::report_timeout(p.status, kStatusConvertTimeout);
        ok = false;
      }
      unsigned char *stage = xring + (size_t)s * p.xslot_bytes;
      if (mine && ok) {
        for (int base = my_slot * 8; base < CS * p.M; base += 8 * conv_group) {
          const int idx = base + q;
          if (idx < CS * p.M) {   // uniform within a quad
            const int m = idx / CS, cell = idx % CS;
            const unsigned char *src = stage + kXOff + m * kXRowBytes + cell * 256;
            uint4 v[4];
            uint32_t amax = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int kk = (4 * i + sub + 4 * (q & 1)) & 15;   // rotated so that a quarter-warp covers all banks
              v[i] = *reinterpret_cast<const uint4 *>(src + kk * 16);
              const uint32_t w[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
#pragma unroll
              for (int j = 0; j < 4; ++j) amax = max(amax, max(w[j] & 0x7fffu, (w[j] >> 16) & 0x7fffu));
            }
            amax = max(amax, __shfl_xor_sync(qmask, amax, 1));
            amax = max(amax, __shfl_xor_sync(qmask, amax, 2));
            const int e_raw = (int)(amax >> 7);                       // biased exponent of the largest magnitude
            const int e = min(max(e_raw, sh + 1), 253);
            const float scale = __uint_as_float((uint32_t)(254 + sh - e) << 23);   // 2^(127 + sh - e)
            int dsum[3] = {0, 0, 0};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int kk = (4 * i + sub + 4 * (q & 1)) & 15;
              const uint32_t w[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
              uint32_t yb[8];   // float bit patterns whose low bytes are the excess-coded digits
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                yb[2 * j] = __float_as_uint(fmaf(__uint_as_float(w[j] << 16), scale, magic));
                yb[2 * j + 1] = __float_as_uint(fmaf(__uint_as_float(w[j] & 0xffff0000u), scale, magic));
              }
              // even elements feed b0 (k slots of nibbles 0,2,4,6), odd elements b1 (nibbles 1,3,5,7)
              const uint32_t pe = prmt(yb[0], yb[2], 0x5140), qe = prmt(yb[4], yb[6], 0x5140);
              const uint32_t po = prmt(yb[1], yb[3], 0x5140), qo = prmt(yb[5], yb[7], 0x5140);
              uint32_t b0[3], b1[3];
              b0[0] = prmt(pe, qe, 0x5410) ^ 0x80808080u;
              b1[0] = prmt(po, qo, 0x5410) ^ 0x80808080u;
              b0[1] = prmt(pe, qe, 0x7632) ^ 0x80808080u;
              b1[1] = prmt(po, qo, 0x7632) ^ 0x80808080u;
              if (nd == 3) {
                const uint32_t te = prmt(prmt(yb[0], yb[2], 0x0062), prmt(yb[4], yb[6], 0x0062), 0x5410) ^ 0x40404040u;
                const uint32_t to = prmt(prmt(yb[1], yb[3], 0x0062), prmt(yb[5], yb[7], 0x0062), 0x5410) ^ 0x40404040u;
                b0[2] = te | ((te & 0x40404040u) << 1);   // excess 64 -> two's complement
                b1[2] = to | ((to & 0x40404040u) << 1);
              }
              const int t = kk >> 2, c = kk & 3;
              unsigned char *dst = stage + kDOff + (((cell * 2 + (c >> 1)) * ncols + m * nd) * 4 + t) * 16 + (c & 1) * 8;
#pragma unroll
              for (int d = 0; d < 3; ++d)
                if (d < nd) {
                  *reinterpret_cast<uint2 *>(dst + d * 64) = make_uint2(b0[d], b1[d]);
                  dsum[d] = byte_sum(b1[d], byte_sum(b0[d], dsum[d]));
                }
            }
#pragma unroll
            for (int d = 0; d < 3; ++d) {
              dsum[d] += __shfl_xor_sync(qmask, dsum[d], 1);
              dsum[d] += __shfl_xor_sync(qmask, dsum[d], 2);
            }
            if (sub == 0) {
              float *ftab = reinterpret_cast<float *>(stage) + cell * NC + m * nd;
              int *ntab = reinterpret_cast<int *>(stage + kEBytes) + cell * NC + m * nd;
              const float f0 = e_raw == 255 ? __uint_as_float(0x7fc00000u)             // inf / NaN in the cell
                                            : __uint_as_float((uint32_t)(e - sh) << 23);  // 2^(e - 127 - sh)
#pragma unroll
              for (int d = 0; d < 3; ++d)
                if (d < nd) {
                  ftab[d] = f0 * (d == 0 ? 1.f : d == 1 ? 256.f : 65536.f);
                  ntab[d] = -8 * dsum[d];
                }
              if (ASYM) {
                float *xtab = reinterpret_cast<float *>(stage + 2 * kEBytes) + cell * NC + m * nd;
                xtab[0] = f0 * (float)(dsum[0] + 256 * dsum[1] + 65536 * dsum[2]);   // sum_k x of the cell
              }
            }
          }
        }
      }
      __syncwarp();
      if (mine && lane == 0) tc::mbar_arrive(&frag_bar[s]);
      if (++s == (uint32_t)p.xslots) {
        s = 0;
        ph ^= 1;
      }
    }
  } else {
    // ---------------- compute warps ----------------
    const int g = lane >> 2, t = lane & 3;
    uint32_t kmask, kflip;   // opaque to the compiler so that they stay in registers
    asm volatile("mov.b32 %0, 0x0f0f0f0f;" : "=r"(kmask));
    asm volatile("mov.b32 %0, 0x08080808;" : "=r"(kflip));
    const int my_step = warp / kWarpsPerCell;
    const int rb = 16 * R * (warp % kWarpsPerCell);  // first of this warp's 16 R columns within the tile
    float acc[R][NB][4];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int m = 0; m < NB; ++m)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[r][m][e] = 0.f;
    // byte offsets inside a stage that do not change from chunk to chunk
    const int w_off = (rb + g) * kWRowBytes + my_step * 64 + 16 * t;
    const int d_off = kDOff + ((my_step * 2 * ncols + g) * 4 + t) * 16;   // + (pair * ncols + 8 m) * 64
    const int d_pstride = ncols * 64;
    const int e_off = (my_step * NC + 2 * t) * 4;                          // + 8 m * 4

    Iter iter(c_begin, c_end, p.ksteps);
    Chunk ch;
    uint32_t s = 0, ph = 0, xs_i = 0, xph = 0;   // weight stage / activation slot and their phase bits
    uint32_t rbuf = 0, rph = 0;                  // reduction buffer and its phase bit
    bool ok = true;
    bool first_chunk = true;
    while (iter.next(ch)) {
      if (ok && !(tc::mbar_wait_suspend(&full_bar[s], ph, 60) && tc::mbar_wait_suspend(&frag_bar[xs_i], xph, 60))) {
        tc::report_timeout(p.status, kStatusConvertTimeout);
        ok = false;
      }
      if (first_chunk && tid == 0) stamp_here(p.timeline, blockIdx.x, 3);
      first_chunk = false;
      const unsigned char *stage = smem + (size_t)s * p.stage_bytes;
      const unsigned char *xslot = xring + (size_t)xs_i * p.xslot_bytes;
      if (ok && my_step < ch.nsteps) {
        // group of this warp's cell, relative to the chunk's first group (spg = cells per group)
        const int gl = p.spg_mul == 0 ? my_step
                                      : (int)(__umulhi((uint32_t)(ch.step0 + my_step), p.spg_mul) -
                                              __umulhi((uint32_t)ch.step0, p.spg_mul));
        uint4 wv[R][2];
        float sc[R][2], zp[R][2];
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int row = rb + 16 * r + 8 * h + g;
            wv[r][h] = *reinterpret_cast<const uint4 *>(stage + w_off + (16 * r + 8 * h) * kWRowBytes);
            const unsigned char *sp = stage + kSOff + gl * kTileN * kScaleBytes;
            sc[r][h] = SF32 ? reinterpret_cast<const float *>(sp)[row]
                            : __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(sp)[row]);
            if (ASYM) {
              const unsigned char *zq = stage + kZOff + gl * kTileN * kScaleBytes;
              zp[r][h] = SF32 ? reinterpret_cast<const float *>(zq)[row]
                              : __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(zq)[row]);
            }
          }
        // integer accumulators start at -8 * (digit sum of the column): sum_k (q + 8) d - 8 sum_k d
        int part[R][NB][4];
#pragma unroll
        for (int m = 0; m < NB; ++m) {
          const int2 nb = *reinterpret_cast<const int2 *>(xslot + e_off + kEBytes + m * 32);
#pragma unroll
          for (int r = 0; r < R; ++r) {
            part[r][m][0] = nb.x;
            part[r][m][1] = nb.y;
            part[r][m][2] = nb.x;
            part[r][m][3] = nb.y;
          }
        }
#pragma unroll
        for (int pr = 0; pr < 2; ++pr) {   // pairs of packed words (c = 2 pr, 2 pr + 1)
          uint4 xb[NB];
#pragma unroll
          for (int m = 0; m < NB; ++m) {
            xb[m] = make_uint4(0u, 0u, 0u, 0u);
            if (m * 8 + g < ncols)
              xb[m] = *reinterpret_cast<const uint4 *>(xslot + d_off + pr * d_pstride + m * 8 * 64);
          }
#pragma unroll
          for (int ci = 0; ci < 2; ++ci) {
#pragma unroll
            for (int r = 0; r < R; ++r) {
              const uint32_t wa = pr == 0 ? (ci == 0 ? wv[r][0].x : wv[r][0].y) : (ci == 0 ? wv[r][0].z : wv[r][0].w);
              const uint32_t wb = pr == 0 ? (ci == 0 ? wv[r][1].x : wv[r][1].y) : (ci == 0 ? wv[r][1].z : wv[r][1].w);
              const uint32_t a0 = nib_bytes<!ASYM>(wa, kmask, kflip), a1 = nib_bytes<!ASYM>(wb, kmask, kflip);  // nibbles 0,2,4,6
              const uint32_t a2 = nib_bytes<!ASYM>(wa >> 4, kmask, kflip);                                     // nibbles 1,3,5,7
              const uint32_t a3 = nib_bytes<!ASYM>(wb >> 4, kmask, kflip);
#pragma unroll
              for (int m = 0; m < NB; ++m)
                mma_u8s8_16832(part[r][m], a0, a1, a2, a3, ci == 0 ? xb[m].x : xb[m].z, ci == 0 ? xb[m].y : xb[m].w);
            }
          }
        }
#pragma unroll
        for (int m = 0; m < NB; ++m) {
          const float2 f = *reinterpret_cast<const float2 *>(xslot + e_off + m * 32);
          float2 xs = make_float2(0.f, 0.f);
          if (ASYM) xs = *reinterpret_cast<const float2 *>(xslot + e_off + 2 * kEBytes + m * 32);
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const float fv = e ? f.y : f.x, xsv = e ? xs.y : xs.x;
#pragma unroll
            for (int r = 0; r < R; ++r)
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                float v = (sc[r][h] * fv) * __int2float_rn(part[r][m][2 * h + e]);
                if (ASYM) v = fmaf(zp[r][h], xsv, v);
                acc[r][m][2 * h + e] += v;
              }
          }
        }
      }
      __syncwarp();
      if (lane == 0) {
        tc::mbar_arrive(&empty_bar[s]);
        tc::mbar_arrive(&xempty_bar[xs_i]);
      }
      if (++s == (uint32_t)p.stages) {
        s = 0;
        ph ^= 1;
      }
      if (++xs_i == (uint32_t)p.xslots) {
        xs_i = 0;
        xph ^= 1;
      }

      if (ch.last_of_segment) {
        // ---- the segment of tile ch.tile is complete: hand the warp's sums to the epilogue warp and go on ----
        // With two digits a lane's column pair (2t, 2t+1) is one token: add the pair.  With three digits the
        // columns go out as they are and are added when the rows are read back.
        if (ok && !tc::mbar_wait_suspend(&red_free[rbuf], rph ^ 1)) {
          tc::report_timeout(p.status, kStatusEpilogueTimeout);
          ok = false;
        }
        float *rw = red + (size_t)rbuf * red_buf_floats + warp * rrows * kRedStride;
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
          for (int m = 0; m < NB; ++m)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const int nl = 16 * r + 8 * h + g;  // within this warp's 16 R columns
              if (nd == 2) {
                if (4 * m + t < rrows) rw[(4 * m + t) * kRedStride + nl] = acc[r][m][2 * h] + acc[r][m][2 * h + 1];
              } else if (m == 0) {
                if (2 * t < rrows) rw[(2 * t) * kRedStride + nl] = acc[r][m][2 * h];
                if (2 * t + 1 < rrows) rw[(2 * t + 1) * kRedStride + nl] = acc[r][m][2 * h + 1];
              }
              acc[r][m][2 * h] = 0.f;
              acc[r][m][2 * h + 1] = 0.f;
            }
        __syncwarp();
        if (lane == 0) tc::mbar_arrive(&red_full[rbuf]);
        rbuf ^= 1;
        if (rbuf == 0) rph ^= 1;
      }
    }
    if (tid == 0) stamp_here(p.timeline, blockIdx.x, 4);
  }
}

// Weight stage: packed weights, scales (+ zero points).
size_t streamk_stage_bytes(int M, bool asym) {
  const size_t cs = chunk_steps(col_blocks(M));
  return kTileN * cs * 64 + cs * 256 * (asym ? 2 : 1);
}
// Activation slot: per-column tables, staged bf16 activations, digit fragments.
size_t streamk_xslot_bytes(int M, bool asym) {
  const size_t nb = col_blocks(M), cs = chunk_steps((int)nb), ncols = (size_t)M * digits_for(M);
  const size_t b = (asym ? 3 : 2) * cs * nb * 8 * 4 + (size_t)M * cs * 256 + cs * 128 * ncols;
  return (b + 127) / 128 * 128;
}
size_t streamk_tail_bytes(int M) {   // two reduction buffers and the barriers
  const size_t rrows = digits_for(M) == 3 ? (size_t)M * 3 : (size_t)M;
  return 2 * kComputeWarps * rrows * kRedStride * sizeof(float) + (5 * kMaxStages + 4) * sizeof(uint64_t) + 64;
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

int build_maps(const zt_woq_linear_args_t &a, int mrows, uint32_t cs, Maps &m) {
  const uint64_t ksteps = (uint64_t)a.K / kStepK;
  {  // packed weight: [N rows][K/128 cells][16 words]
    const uint64_t dims[3] = {16, ksteps, (uint64_t)a.N};
    const uint64_t strides[2] = {64, (uint64_t)a.K / 2};
    const uint32_t box[3] = {16, cs, kTileN};
    int rc = cached_map(&m.w8, a.wq, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, dims, strides, box);
    if (rc != ZT_SUCCESS) return rc;
  }
  {  // activations: [M rows][K/128 cells][128 bf16]
    const uint64_t dims[3] = {128, ksteps, (uint64_t)a.M};
    const uint64_t strides[2] = {256, (uint64_t)a.K * 2};
    const uint32_t box[3] = {128, cs, (uint32_t)mrows};
    int rc = cached_map(&m.x8, a.x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, dims, strides, box);
    if (rc != ZT_SUCCESS) return rc;
  }
  {  // scales / zero points: [groups][N]
    const bool f32 = a.scale_dtype == ZT_F32;
    const CUtensorMapDataType dt = f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    const uint64_t dims[2] = {(uint64_t)a.N, (uint64_t)a.n_groups};
    const uint64_t strides[1] = {(uint64_t)a.N * (f32 ? 4 : 2)};
    const uint32_t box[2] = {kTileN, cs};
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

template <int NB, int CW, bool ASYM, bool SF32>
int launch(const Maps &m, const SKParams &p, int grid, size_t smem_bytes, cudaStream_t st) {
  auto kern = woq_streamk_kernel<NB, CW, ASYM, SF32>;
  static PerDeviceOnce configured;
  if (int rc_cfg = allow_dynamic_smem(configured, kern, 226 * 1024)) return rc_cfg;
  ZT_CUDA_OK(launch_overlapped(kern, dim3((unsigned)grid), dim3((unsigned)sk_threads(CW)), smem_bytes, st, m.w8, m.x8, m.s,
                               m.z, p));
  return launch_status("woq_streamk_kernel");
}

template <int NB, int CW>
int launch_q(const Maps &m, const SKParams &p, int grid, size_t smem_bytes, cudaStream_t st) {
  const bool asym = p.zeros != nullptr, sf32 = p.scale_dtype == ZT_F32;
  if (asym)
    return sf32 ? launch<NB, CW, true, true>(m, p, grid, smem_bytes, st) : launch<NB, CW, true, false>(m, p, grid, smem_bytes, st);
  return sf32 ? launch<NB, CW, false, true>(m, p, grid, smem_bytes, st) : launch<NB, CW, false, false>(m, p, grid, smem_bytes, st);
}

}  // namespace

size_t woq_streamk_workspace_bytes() { return (size_t)sm_count() * 2 * 16 * kTileN * sizeof(float); }

bool woq_streamk_supported(const zt_woq_linear_args_t &a) {
  // Beyond four tokens the conversion of the activations (redone by every CTA) outweighs the cheaper
  // weight path and the register-ring decode kernel is faster.
  if (a.M < 1 || a.M > kMaxTokens || a.N < 1) return false;
  if (a.K % kStepK != 0 || a.n_groups <= 0 || a.K % a.n_groups != 0) return false;
  const int64_t gs = a.K / a.n_groups;
  if (gs % kStepK != 0) return false;
  const int ssz = a.scale_dtype == ZT_F32 ? 4 : 2;
  if ((a.N * ssz) % 16 != 0) return false;  // TMA row pitch of the scale table must be a multiple of 16 bytes
  const uintptr_t ptrs = reinterpret_cast<uintptr_t>(a.x) | reinterpret_cast<uintptr_t>(a.wq) |
                         reinterpret_cast<uintptr_t>(a.scales) | reinterpret_cast<uintptr_t>(a.zeros);
  if (ptrs & 15) return false;
  if (2 * ceil_div<int64_t>(a.N, kTileN) * (int64_t)sizeof(int) > ZT_WOQ_COUNTER_BYTES) return false;  // two counters per tile
  return a.K <= (1 << 22) && a.N <= (1 << 30);  // group lookups divide by multiplication: (K/128)^2 < 2^32
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
  p.spg_mul = p.spg == 1 ? 0u : (uint32_t)((1ull << 32) / (uint64_t)p.spg + 1);
  p.ksteps = (int)(a.K / kStepK);
  p.ntiles = (int)ceil_div<int64_t>(a.N, kTileN);
  p.total_cells = (long long)p.ntiles * p.ksteps;
  p.counters = reinterpret_cast<int *>(a.workspace);
  p.partial = reinterpret_cast<float *>(reinterpret_cast<char *>(a.workspace) + ZT_WOQ_COUNTER_BYTES);
  p.status = device_status_ptr();
  p.post = to_dev(a.post);
  const int nb = col_blocks((int)a.M);
  const size_t stage = streamk_stage_bytes((int)a.M, a.zeros != nullptr);
  const size_t xslot = streamk_xslot_bytes((int)a.M, a.zeros != nullptr);
  const size_t tail = streamk_tail_bytes((int)a.M);
  const size_t avail = 226 * 1024 - tail;   // dynamic shared memory left for the two rings
  // Activation slots are small and let the conversion run ahead of the weights: six of them for up to two
  // tokens, four up to four, three beyond; fewer when that buys no weight stage less than three.
  int xslots = a.M <= 2 ? 6 : a.M <= 4 ? 4 : 3;
  while (xslots > 2 && (avail - xslots * xslot) / stage < 3) --xslots;
  int stages = (int)((avail - xslots * xslot) / stage);
  if (stages > kMaxStages) stages = kMaxStages;
  ZT_REQUIRE(stages >= 2, ZT_UNSUPPORTED, "zt_woq_linear: stream-K stage of %zu bytes does not fit twice", stage);
  p.stages = stages;
  p.stage_bytes = (int)stage;
  p.xslots = xslots;
  p.xslot_bytes = (int)xslot;
  int grid = sm_count();
  if ((long long)grid > p.total_cells) grid = (int)p.total_cells;
  const size_t smem_bytes = (size_t)stages * stage + (size_t)xslots * xslot + tail;
  p.timeline = timeline_for_launch(grid);
  Maps maps;
  int rc = build_maps(a, (int)a.M, (uint32_t)chunk_steps(nb), maps);
  if (rc != ZT_SUCCESS) return rc;
  ZT_REQUIRE(nb == 1, ZT_UNSUPPORTED, "zt_woq_linear: the stream-K kernel takes at most %d tokens", kMaxTokens);
  return a.M <= 2 ? launch_q<1, 5>(maps, p, grid, smem_bytes, st) : launch_q<1, 8>(maps, p, grid, smem_bytes, st);
}

}  // namespace zt
