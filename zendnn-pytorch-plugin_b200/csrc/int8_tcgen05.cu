// Host side of the int8 tcgen05 GEMM: tensor-map cache, tile-shape choice, dispatch to the compiled
// configurations (the kernel itself is in int8_tcgen05.cuh).
#include <algorithm>
#include <mutex>
#include <unordered_map>

#include "int8_tcgen05.cuh"

namespace zt {

using namespace i8tc;

namespace {

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

// Tensor maps depend only on (pointer, shape, box); encoding one costs a driver call, so they are
// memoised per process.
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

// Tile shape: the candidate (rows per CTA tile, tile width) that minimises rounds x tile time.  A tile's
// main loop costs, per byte of K, the larger of the tensor-pipe time (rows/128 * BN/64 cycles) and the
// operand-delivery time ((rows + BN) bytes at about 64 B/clk per SM); narrow tiles additionally pay
// shared-memory reads of the A block that every instruction repeats.  A tile whose accumulator cannot
// be double buffered, or that is the only one of its CTA, exposes its epilogue.
struct TileChoice {
  int mh, bn;
};
TileChoice pick_tile(int64_t M, int64_t N, int64_t K) {
  struct Cand {
    int mh, bn, nbuf;
  };
  const Cand cands[] = {{1, 256, 2}, {1, 224, 2}, {1, 192, 2}, {1, 160, 2}, {1, 128, 2}, {1, 96, 2}, {1, 64, 2},
                        {2, 256, 1}, {2, 192, 1}, {2, 160, 1}, {2, 128, 2}};
  const int64_t sms = sm_count();
  double best = 1e30;
  TileChoice pick{1, 128};
  for (const Cand &c : cands) {
    if (c.mh == 2 && M <= kBM) continue;
    const int64_t tiles = ceil_div<int64_t>(M, (int64_t)c.mh * kBM) * ceil_div<int64_t>(N, c.bn);
    const int64_t rounds = ceil_div<int64_t>(tiles, sms);
    const double mma = c.mh * std::max(c.bn / 64.0, (32.0 + c.bn / 4.0) / 32.0);
    const double data = (c.mh * 128.0 + c.bn) / 64.0;
    const double epilogue = c.mh * c.bn * 4.0;  // cycles, when not hidden behind the next tile
    const double exposed = (c.nbuf == 1) ? rounds * epilogue : epilogue;
    const double cost = rounds * std::max(mma, data) * (double)K + exposed;
    if (cost < best * (1.0 - 1e-9)) {
      best = cost;
      pick = {c.mh, c.bn};
    }
  }
  return pick;
}

}  // namespace

bool int8_tcgen05_supported(int64_t M, int64_t N, int64_t K, const void *q, const void *w) {
  if (M < 1 || N < 1 || K < 16 || K % 16 != 0) return false;
  if (M > (1 << 30) || N > (1 << 30) || K > (1 << 30)) return false;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(w)) & 15) return false;
  return true;
}

int int8_tcgen05_launch(const Int8GemmArgs &a, cudaStream_t st) {
  TcParams p{};
  p.M = (int)a.M;
  p.N = (int)a.N;
  p.K = (int)a.K;
  p.src_scale = a.src_scale;
  p.src_zp = a.src_zp;
  p.w_scale = a.w_scale;
  p.w_rowsum = a.w_rowsum;
  p.bias = a.bias;
  p.w_scale_dtype = a.w_scale_dtype;
  p.bias_dtype = a.bias_dtype;
  p.y_dtype = a.y_dtype;
  p.y = a.y;
  p.post = a.post;
  p.status = device_status_ptr();
  p.w_scale_per_tensor = a.w_scale_per_tensor;
  p.post_dtype = a.post_dtype;
  p.out_scale = a.out_scale;
  p.out_zp = a.out_zp;
  p.ldy = a.ldy;
  const int epi = a.raw_s32 ? kEpiS32 : a.static_mode ? kEpiStatic : kEpiLinear;
  // force_bn: tile width, + 1000 for 256-row tiles (e.g. 1160 = 256 x 160), + 2000 for CTA pairs (512 x width)
  TileChoice tile = pick_tile(a.M, a.N, a.K);
  if (a.force_bn >= 2000) {
    ZT_REQUIRE(!a.raw_s32 && !a.static_mode && int8_pair_supported(a.M, a.force_bn % 1000), ZT_UNSUPPORTED,
               "int8_tcgen05_launch: CTA-pair tiles need the linear epilogue, M > 256 and a width of 128, 160, 192 or 256");
    return launch_pair(a.force_bn % 1000, a, p, !a.q_is_u8, st);
  }
  if (a.force_bn > 0) tile = {a.force_bn >= 1000 ? 2 : 1, a.force_bn % 1000};
  const int bn = tile.bn;
  CUtensorMap ta, tb;
  // q_rows: rows that may be addressed behind q (the caller's scratch is padded to kMinQRows rows so that the
  // activation map never has fewer; rows beyond M hold stale bytes whose products are never stored)
  const uint64_t q_rows = a.q_rows > a.M ? (uint64_t)a.q_rows : (uint64_t)a.M;
  int rc = cached_map(&ta, a.q, (uint64_t)a.K, q_rows, (uint32_t)(tile.mh * kBM));
  if (rc != ZT_SUCCESS) return rc;
  rc = cached_map(&tb, a.w, (uint64_t)a.K, (uint64_t)a.N, (uint32_t)bn);
  if (rc != ZT_SUCCESS) return rc;
  const bool sgn = !a.q_is_u8;
  if (tile.mh == 2) return launch_mh2(bn, ta, tb, p, epi, sgn, st);
  switch (bn) {
    case 256: return launch_bn<1, 256, 4, 2>(ta, tb, p, epi, sgn, st);
    case 224: return launch_bn<1, 224, 4, 2>(ta, tb, p, epi, sgn, st);
    case 192: return launch_bn<1, 192, 5, 2>(ta, tb, p, epi, sgn, st);
    case 160: return launch_bn<1, 160, 6, 2>(ta, tb, p, epi, sgn, st);
    case 128: return launch_bn<1, 128, 6, 2>(ta, tb, p, epi, sgn, st);
    case 96: return launch_bn<1, 96, 7, 2>(ta, tb, p, epi, sgn, st);
    case 64: return launch_bn<1, 64, 8, 2>(ta, tb, p, epi, sgn, st);
    default: break;
  }
  set_error("int8_tcgen05_launch: unsupported tile width %d", bn);
  return ZT_UNSUPPORTED;
}

}  // namespace zt
