// Entry points of libzentorch_b200: argument validation, kernel selection, and the process-wide
// pieces (error message, device status word, tensor-map encoder).
#include <cuda.h>
#include <cudaTypedefs.h>

#include <cstdlib>
#include <cstring>
#include <mutex>

#include "int8.cuh"
#include "tc05.cuh"
#include "woq.cuh"

namespace zt {

__device__ int g_device_status = 0;

int *device_status_ptr() {
  static int *ptrs[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!ptrs[dev]) {
    void *p = nullptr;
    if (cudaGetSymbolAddress(&p, g_device_status) != cudaSuccess) return nullptr;
    ptrs[dev] = reinterpret_cast<int *>(p);
  }
  return ptrs[dev];
}

namespace {
thread_local char g_error[512] = "";
}

void set_error(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

int cuda_fail(cudaError_t e, const char *what) {
  set_error("CUDA error in %s: %s (%s)", what, cudaGetErrorName(e), cudaGetErrorString(e));
  return ZT_CUDA_ERROR;
}

namespace {
thread_local bool g_call_overlap = true;
}

bool overlap_launches() {
  static const bool on = [] {
    const char *e = std::getenv("ZENTORCH_B200_PDL");
    return !(e && e[0] == '0');
  }();
  return on && g_call_overlap;
}

CallOverlap::CallOverlap(bool allowed) : saved_(g_call_overlap) { g_call_overlap = allowed; }
CallOverlap::~CallOverlap() { g_call_overlap = saved_; }

namespace {
std::mutex g_timeline_mu;
unsigned long long *g_timeline_buf = nullptr;
size_t g_timeline_entries = 0, g_timeline_used = 0;
}  // namespace

TimelineSink timeline_for_launch(int ctas) {
  std::lock_guard<std::mutex> lock(g_timeline_mu);
  const size_t need = (size_t)ctas * kTimelineSlots;
  if (!g_timeline_buf || g_timeline_used + need > g_timeline_entries) return TimelineSink{nullptr};
  TimelineSink t{g_timeline_buf + g_timeline_used};
  g_timeline_used += need;
  return t;
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

int validate_post_ops(const zt_post_ops_t &p) {
  ZT_REQUIRE(p.n_ops >= 0 && p.n_ops <= ZT_MAX_POST_OPS, ZT_INVALID_ARGUMENT, "post-op count %d out of range [0, %d]",
             p.n_ops, ZT_MAX_POST_OPS);
  int b = 0;
  for (int i = 0; i < p.n_ops; ++i) {
    ZT_REQUIRE(p.ids[i] >= ZT_POST_NONE && p.ids[i] <= ZT_POST_ADD, ZT_INVALID_ARGUMENT, "unknown post-op id %d",
               p.ids[i]);
    if (p.ids[i] == ZT_POST_MUL || p.ids[i] == ZT_POST_ADD) {
      ZT_REQUIRE(p.buffers[b] != nullptr, ZT_INVALID_ARGUMENT, "post-op %d needs a binary operand buffer", i);
      ++b;
    }
  }
  return ZT_SUCCESS;
}

namespace {
PFN_cuTensorMapEncodeTiled_v12000 tensor_map_encoder() {
  static PFN_cuTensorMapEncodeTiled_v12000 encode = nullptr;
  if (!encode) {
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
    if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !fn) return nullptr;
    encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
  }
  return encode;
}
}  // namespace

int make_tensor_map(CUtensorMap *out, const void *base, CUtensorMapDataType dtype, int rank, const uint64_t *dims,
                    const uint64_t *strides_bytes, const uint32_t *box, bool swizzle128) {
  PFN_cuTensorMapEncodeTiled_v12000 encode = tensor_map_encoder();
  if (!encode) {
    set_error("cuTensorMapEncodeTiled is not available from the CUDA driver");
    return ZT_CUDA_ERROR;
  }
  cuuint64_t d[5], st[4];
  cuuint32_t b[5], es[5];
  for (int i = 0; i < rank; ++i) {
    d[i] = dims[i];
    b[i] = box[i];
    es[i] = 1;
    if (i + 1 < rank) st[i] = strides_bytes[i];
  }
  CUresult r = encode(out, dtype, (cuuint32_t)rank, const_cast<void *>(base), d, st, b, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                      swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with CUresult %d (rank %d, dims %llu x %llu, box %u x %u)", (int)r, rank,
              (unsigned long long)dims[0], (unsigned long long)dims[1], box[0], box[1]);
    return ZT_CUDA_ERROR;
  }
  return ZT_SUCCESS;
}

int make_tensor_map_2d(CUtensorMap *out, const void *base, CUtensorMapDataType dtype, uint32_t elem_bytes,
                       uint64_t inner, uint64_t rows, uint64_t pitch_bytes, uint32_t box_inner, uint32_t box_rows) {
  (void)elem_bytes;
  const uint64_t dims[2] = {inner, rows};
  const uint64_t strides[1] = {pitch_bytes};
  const uint32_t box[2] = {box_inner, box_rows};
  return make_tensor_map(out, base, dtype, 2, dims, strides, box, true);
}

namespace {

bool valid_dtype(int d) { return d == ZT_BF16 || d == ZT_F32; }

int env_int(const char *name, int dflt) {
  const char *v = std::getenv(name);
  return v && *v ? std::atoi(v) : dflt;
}

// Read-once 0/1 style switches, in the manner of the reference's EnvReader
// (src/cpu/cpp/EnvReader.hpp:41-60).
struct Env {
  int woq_streamk;     // ZENTORCH_B200_WOQ_STREAMK: 0 = use the register-ring decode kernel instead of stream-K
  int woq_skinny_max;  // ZENTORCH_B200_WOQ_SKINNY_MAX_M: largest M given to the streaming kernel
  int int8_bn;         // ZENTORCH_B200_INT8_BN: force the int8 tensor-core tile width
  Env() {
    woq_streamk = env_int("ZENTORCH_B200_WOQ_STREAMK", 1);
    woq_skinny_max = env_int("ZENTORCH_B200_WOQ_SKINNY_MAX_M", 256);
    int8_bn = env_int("ZENTORCH_B200_INT8_BN", 0);
  }
};
const Env &env() {
  static Env e;
  return e;
}

}  // namespace
}  // namespace zt

using namespace zt;

extern "C" const char *zt_last_error(void) { return g_error; }
extern "C" const char *zt_version(void) { return "zentorch_b200 0.1 (sm_100a)"; }

extern "C" int zt_device_supported(void) {
  int dev = 0, major = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return 0;
  return major == 10 ? 1 : 0;
}

extern "C" int zt_poll_device_status(int *status, int reset) {
  ZT_REQUIRE(status != nullptr, ZT_INVALID_ARGUMENT, "zt_poll_device_status: null pointer");
  ZT_CUDA_OK(cudaMemcpyFromSymbol(status, g_device_status, sizeof(int)));
  if (reset && *status != 0) {
    const int zero = 0;
    ZT_CUDA_OK(cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int)));
  }
  return ZT_SUCCESS;
}

extern "C" int zt_debug_set_timeline(void *device_buffer, size_t bytes) {
  std::lock_guard<std::mutex> lock(g_timeline_mu);
  g_timeline_buf = reinterpret_cast<unsigned long long *>(device_buffer);
  g_timeline_entries = device_buffer ? bytes / sizeof(unsigned long long) : 0;
  g_timeline_used = 0;
  return ZT_SUCCESS;
}

// ---- self-test of the bounded-wait path ------------------------------------------------------------
namespace zt {
namespace {
// One thread waits on an mbarrier that nothing ever arrives at, with a short poll limit; the wait gives up,
// the status word is set, and the kernel returns normally.
__global__ void expire_wait_kernel(int *status, uint32_t polls) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    tc::mbar_init(&bar, 1);
    tc::mbar_fence_init();
    if (!tc::mbar_wait(&bar, 0, polls)) tc::report_timeout(status, kStatusSelfTest);
  }
}
}  // namespace
}  // namespace zt

extern "C" int zt_selftest_expire_wait(void *stream) {
  int *status = device_status_ptr();
  ZT_REQUIRE(status != nullptr, ZT_CUDA_ERROR, "zt_selftest_expire_wait: no device status word");
  expire_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(status, 2048u);
  return launch_status("expire_wait_kernel");
}

// ---- weight-only int4 ---------------------------------------------------------------------------
extern "C" size_t zt_woq_linear_workspace_bytes(int64_t M, int64_t N, int64_t K) {
  if (M <= 0 || N <= 0 || K <= 0) return ZT_WOQ_COUNTER_BYTES;
  const size_t a = woq_skinny_plan(M, N, K).partial_bytes;
  const size_t b = woq_stream_plan(M < 16 ? M : 16, N, K).partial_bytes;
  const size_t c = woq_streamk_workspace_bytes();
  const size_t d = woq_tcgen05_workspace_bytes(M, N, K);
  size_t m = a > b ? a : b;
  m = m > c ? m : c;
  return ZT_WOQ_COUNTER_BYTES + (m > d ? m : d);
}

extern "C" int zt_woq_linear(const zt_woq_linear_args_t *a, void *stream) {
  ZT_REQUIRE(a != nullptr, ZT_INVALID_ARGUMENT, "zt_woq_linear: null argument block");
  ZT_REQUIRE(a->M >= 0 && a->N >= 0 && a->K >= 0, ZT_INVALID_ARGUMENT, "zt_woq_linear: negative size");
  ZT_REQUIRE(a->K % 8 == 0, ZT_INVALID_ARGUMENT, "K must be divisible by 8, got %lld", (long long)a->K);
  if (a->M == 0 || a->N == 0) return ZT_SUCCESS;
  ZT_REQUIRE(a->K >= 8, ZT_INVALID_ARGUMENT, "K must be at least 8, got %lld", (long long)a->K);
  ZT_REQUIRE(a->x && a->wq && a->scales && a->y, ZT_INVALID_ARGUMENT, "zt_woq_linear: null tensor pointer");
  ZT_REQUIRE(a->n_groups >= 1 && a->K % a->n_groups == 0, ZT_INVALID_ARGUMENT,
             "zt_woq_linear: K (%lld) must be divisible by the number of scale groups (%lld)", (long long)a->K,
             (long long)a->n_groups);
  ZT_REQUIRE(valid_dtype(a->scale_dtype), ZT_INVALID_ARGUMENT, "zt_woq_linear: weight_scales must be float32 or bfloat16");
  ZT_REQUIRE(!a->bias || valid_dtype(a->bias_dtype), ZT_INVALID_ARGUMENT, "zt_woq_linear: bias must be float32 or bfloat16");
  int rc = validate_post_ops(a->post);
  if (rc != ZT_SUCCESS) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  CallOverlap overlap(!(a->flags & ZT_FLAG_WEIGHTS_VOLATILE));

  int algo = a->algo & 0xff;
  const bool stream_ok = woq_stream_supported(*a);
  if (algo == ZT_ALGO_AUTO) {
    // Very small problems are launch-bound whatever runs them; they take the generic kernel, whose
    // per-element dequantisation rounds exactly like the reference's test oracle.
    const bool tiny = a->N * a->K < (1 << 18);
    if (stream_ok && !tiny)
      algo = ZT_ALGO_SKINNY;
    else if (woq_tcgen05_supported(*a))
      algo = ZT_ALGO_TCGEN05;
    else if (woq_skinny_supported(*a) && !tiny && a->M <= env().woq_skinny_max)
      algo = ZT_ALGO_SKINNY;
    else
      algo = ZT_ALGO_GENERIC;
  }
  switch (algo) {
    case ZT_ALGO_GENERIC: return woq_generic_launch(*a, st);
    case ZT_ALGO_SKINNY:
      // Two decode kernels: the work-balanced TMA-staged one streams faster but has a longer fixed
      // latency (cross-CTA reduction), so it takes the layers with at least 48 MB of packed weights (at 30 MB the two measured equal).
      // Tile hint 1 forces the register-ring kernel, 2 the stream-K kernel (tests, benchmarks).
      if (((a->algo >> 8) & 0xffff) != 1 &&
          ((env().woq_streamk && a->N * a->K / 2 >= (48 << 20)) || ((a->algo >> 8) & 0xffff) == 2) &&
          woq_streamk_supported(*a) &&
          a->workspace_bytes >= ZT_WOQ_COUNTER_BYTES + woq_streamk_workspace_bytes())
        return woq_streamk_launch(*a, st);
      if (stream_ok) return woq_stream_launch(*a, st);
      ZT_REQUIRE(woq_skinny_supported(*a), ZT_UNSUPPORTED,
                 "zt_woq_linear: the streaming kernels need K and the group size to be multiples of 128 and 16-byte "
                 "aligned x / weight");
      return woq_skinny_launch(*a, false, st);
    case ZT_ALGO_TCGEN05:
      ZT_REQUIRE(woq_tcgen05_supported(*a), ZT_UNSUPPORTED, "zt_woq_linear: shape not supported by the tcgen05 kernel");
      return woq_tcgen05_launch(*a, st);
    default: break;
  }
  set_error("zt_woq_linear: unknown algo %d", a->algo);
  return ZT_INVALID_ARGUMENT;
}

// ---- dynamic int8 -------------------------------------------------------------------------------
namespace {
size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
}

extern "C" size_t zt_dynamic_qlinear_workspace_bytes(int64_t M, int64_t K) {
  if (M <= 0 || K <= 0) return 256;
  const int64_t rows = M < kMinQRows ? kMinQRows : M;   // the quantised activations are padded to kMinQRows rows
  return align_up((size_t)rows * K, 256) + 2 * align_up((size_t)M * 4, 256);
}

extern "C" int zt_dynamic_quantize(const void *x, int32_t x_dtype, int64_t M, int64_t K, int32_t act_quant, void *q,
                                   float *scales, int32_t *zero_points, void *stream) {
  ZT_REQUIRE(M >= 0 && K >= 0, ZT_INVALID_ARGUMENT, "zt_dynamic_quantize: negative size");
  if (M == 0 || K == 0) return ZT_SUCCESS;
  ZT_REQUIRE(x && q && scales, ZT_INVALID_ARGUMENT, "zt_dynamic_quantize: null pointer");
  ZT_REQUIRE(valid_dtype(x_dtype), ZT_INVALID_ARGUMENT, "zentorch_dynamic_qlinear: input must be bfloat16 or float32");
  ZT_REQUIRE(act_quant == ZT_ACT_S8_SYM || act_quant == ZT_ACT_U8_ASYM, ZT_INVALID_ARGUMENT,
             "zt_dynamic_quantize: unknown activation quantisation mode %d", act_quant);
  ZT_REQUIRE(act_quant == ZT_ACT_S8_SYM || zero_points, ZT_INVALID_ARGUMENT,
             "zt_dynamic_quantize: the u8 mode needs a zero-point output");
  return dynamic_quantize_launch(x, x_dtype, M, K, act_quant, q, scales, zero_points, (cudaStream_t)stream);
}

namespace {
int run_int8_gemm(Int8GemmArgs &g, int algo_and_tile, cudaStream_t st) {
  int algo = algo_and_tile & 0xff;
  const int tile_hint = (algo_and_tile >> 8) & 0xffff;
  if (algo == ZT_ALGO_AUTO || algo == ZT_ALGO_SKINNY)
    algo = int8_tcgen05_supported(g.M, g.N, g.K, g.q, g.w) ? ZT_ALGO_TCGEN05 : ZT_ALGO_GENERIC;
  if (algo == ZT_ALGO_TCGEN05) {
    ZT_REQUIRE(int8_tcgen05_supported(g.M, g.N, g.K, g.q, g.w), ZT_UNSUPPORTED,
               "int8 tcgen05 kernel needs K %% 16 == 0 and 16-byte aligned operands");
    g.force_bn = tile_hint ? tile_hint : env().int8_bn;
    // a width forced through the environment applies where that tile form exists; a hint is taken literally
    if (!tile_hint && g.force_bn >= 2000 && (g.raw_s32 || g.M <= 256)) g.force_bn = 0;
    return int8_tcgen05_launch(g, st);
  }
  if (algo == ZT_ALGO_GENERIC) return int8_generic_launch(g, st);
  set_error("int8 gemm: unknown algo %d", algo);
  return ZT_INVALID_ARGUMENT;
}
}  // namespace

extern "C" int zt_int8_gemm_s32(const void *q, int32_t q_is_u8, const int8_t *w, int64_t M, int64_t N, int64_t K,
                                int32_t *acc, int32_t algo, void *stream) {
  ZT_REQUIRE(M >= 0 && N >= 0 && K >= 0, ZT_INVALID_ARGUMENT, "zt_int8_gemm_s32: negative size");
  if (M == 0 || N == 0) return ZT_SUCCESS;
  ZT_REQUIRE(q && w && acc, ZT_INVALID_ARGUMENT, "zt_int8_gemm_s32: null pointer");
  Int8GemmArgs g{};
  g.q = q;
  g.q_is_u8 = q_is_u8 != 0;
  g.w = w;
  g.M = M;
  g.N = N;
  g.K = K;
  g.raw_s32 = true;
  g.y = acc;
  return run_int8_gemm(g, algo, (cudaStream_t)stream);
}

static int qlinear_prequantized_impl(const zt_dynamic_qlinear_args_t *a, const void *q, int64_t q_rows,
                                     const float *src_scales, const int32_t *src_zero_points, void *stream);

extern "C" int zt_dynamic_qlinear(const zt_dynamic_qlinear_args_t *a, void *stream) {
  ZT_REQUIRE(a != nullptr, ZT_INVALID_ARGUMENT, "zt_dynamic_qlinear: null argument block");
  ZT_REQUIRE(a->M >= 0 && a->N >= 0 && a->K >= 0, ZT_INVALID_ARGUMENT, "zt_dynamic_qlinear: negative size");
  ZT_REQUIRE(valid_dtype(a->x_dtype), ZT_INVALID_ARGUMENT, "zentorch_dynamic_qlinear: input must be bfloat16 or float32");
  ZT_REQUIRE(valid_dtype(a->w_scale_dtype), ZT_INVALID_ARGUMENT,
             "zentorch_dynamic_qlinear: weight_scales must be float32, bfloat16");
  ZT_REQUIRE(!a->bias || valid_dtype(a->bias_dtype), ZT_INVALID_ARGUMENT,
             "zentorch_dynamic_qlinear: bias must be float32 or bfloat16");
  ZT_REQUIRE(a->act_quant == ZT_ACT_S8_SYM || a->act_quant == ZT_ACT_U8_ASYM, ZT_INVALID_ARGUMENT,
             "zt_dynamic_qlinear: unknown activation quantisation mode %d", a->act_quant);
  if (a->M == 0 || a->N == 0) return ZT_SUCCESS;
  ZT_REQUIRE(a->K >= 1, ZT_INVALID_ARGUMENT, "zt_dynamic_qlinear: K must be positive");
  ZT_REQUIRE(a->x && a->w && a->w_scales && a->y, ZT_INVALID_ARGUMENT, "zt_dynamic_qlinear: null tensor pointer");
  ZT_REQUIRE(a->act_quant == ZT_ACT_S8_SYM || a->w_rowsum, ZT_INVALID_ARGUMENT,
             "zt_dynamic_qlinear: the u8 mode needs w_rowsum (zt_int8_weight_rowsum)");
  int rc = validate_post_ops(a->post);
  if (rc != ZT_SUCCESS) return rc;
  // the size asked for includes the padding of the quantised activations to kMinQRows rows; a workspace
  // that only holds the M rows is accepted and used without the padding
  const size_t padded = zt_dynamic_qlinear_workspace_bytes(a->M, a->K);
  const size_t need = align_up((size_t)a->M * a->K, 256) + 2 * align_up((size_t)a->M * 4, 256);
  ZT_REQUIRE(a->workspace && a->workspace_bytes >= need, ZT_WORKSPACE_TOO_SMALL,
             "zt_dynamic_qlinear: workspace of %zu bytes is smaller than the %zu required", a->workspace_bytes, need);
  ZT_REQUIRE((reinterpret_cast<uintptr_t>(a->workspace) & 255) == 0, ZT_INVALID_ARGUMENT,
             "zt_dynamic_qlinear: workspace must be 256-byte aligned");
  cudaStream_t st = (cudaStream_t)stream;
  CallOverlap overlap(!(a->flags & ZT_FLAG_WEIGHTS_VOLATILE));
  char *ws = reinterpret_cast<char *>(a->workspace);
  void *q = ws;
  const int64_t q_rows = (a->M < kMinQRows && a->workspace_bytes >= padded) ? kMinQRows : a->M;
  float *scales = reinterpret_cast<float *>(ws + align_up((size_t)q_rows * a->K, 256));
  int32_t *zps = reinterpret_cast<int32_t *>(reinterpret_cast<char *>(scales) + align_up((size_t)a->M * 4, 256));
  rc = dynamic_quantize_launch(a->x, a->x_dtype, a->M, a->K, a->act_quant, q, scales, zps, st);
  if (rc != ZT_SUCCESS) return rc;
  return qlinear_prequantized_impl(a, q, q_rows, scales, zps, stream);
}

extern "C" int zt_qlinear_prequantized(const zt_dynamic_qlinear_args_t *a, const void *q, const float *src_scales,
                                       const int32_t *src_zero_points, void *stream) {
  return qlinear_prequantized_impl(a, q, 0, src_scales, src_zero_points, stream);
}

// q_rows: rows addressable behind q (0: exactly M)
static int qlinear_prequantized_impl(const zt_dynamic_qlinear_args_t *a, const void *q, int64_t q_rows,
                                     const float *src_scales, const int32_t *src_zero_points, void *stream) {
  ZT_REQUIRE(a != nullptr, ZT_INVALID_ARGUMENT, "zt_qlinear_prequantized: null argument block");
  ZT_REQUIRE(a->M >= 0 && a->N >= 0 && a->K >= 0, ZT_INVALID_ARGUMENT, "zt_qlinear_prequantized: negative size");
  ZT_REQUIRE(valid_dtype(a->x_dtype) && valid_dtype(a->w_scale_dtype) && (!a->bias || valid_dtype(a->bias_dtype)),
             ZT_INVALID_ARGUMENT, "zt_qlinear_prequantized: dtypes must be float32 or bfloat16");
  if (a->M == 0 || a->N == 0) return ZT_SUCCESS;
  const bool u8 = a->act_quant == ZT_ACT_U8_ASYM;
  ZT_REQUIRE(q && src_scales && a->w && a->w_scales && a->y, ZT_INVALID_ARGUMENT,
             "zt_qlinear_prequantized: null tensor pointer");
  ZT_REQUIRE(!u8 || (src_zero_points && a->w_rowsum), ZT_INVALID_ARGUMENT,
             "zt_qlinear_prequantized: the u8 mode needs zero points and w_rowsum");
  int rc = validate_post_ops(a->post);
  if (rc != ZT_SUCCESS) return rc;
  CallOverlap overlap(overlap_launches() && !(a->flags & ZT_FLAG_WEIGHTS_VOLATILE));
  Int8GemmArgs g{};
  g.q = q;
  g.q_is_u8 = u8;
  g.w = a->w;
  g.M = a->M;
  g.N = a->N;
  g.K = a->K;
  g.raw_s32 = false;
  g.q_rows = q_rows;
  g.src_scale = src_scales;
  g.src_zp = u8 ? src_zero_points : nullptr;
  g.w_scale = a->w_scales;
  g.w_scale_dtype = a->w_scale_dtype;
  g.w_rowsum = u8 ? a->w_rowsum : nullptr;
  g.bias = a->bias;
  g.bias_dtype = a->bias_dtype;
  g.y_dtype = a->x_dtype;
  g.y = a->y;
  g.post = to_dev(a->post);
  return run_int8_gemm(g, a->algo, (cudaStream_t)stream);
}

// ---- static-quantisation qlinear ------------------------------------------------------------------------
extern "C" size_t zt_static_qlinear_workspace_bytes(int64_t M, int64_t K, int32_t x_dtype) {
  if (M <= 0 || K <= 0 || x_dtype == ZT_U8 || x_dtype == ZT_S8) return 256;
  return align_up((size_t)M * K, 256);
}

extern "C" int zt_static_quantize(const void *x, int32_t x_dtype, int64_t numel, const float *scale,
                                  const int32_t *zero_point, void *q, void *stream) {
  ZT_REQUIRE(numel >= 0, ZT_INVALID_ARGUMENT, "zt_static_quantize: negative size");
  if (numel == 0) return ZT_SUCCESS;
  ZT_REQUIRE(x && scale && q, ZT_INVALID_ARGUMENT, "zt_static_quantize: null pointer");
  ZT_REQUIRE(valid_dtype(x_dtype), ZT_INVALID_ARGUMENT, "zt_static_quantize: input must be bfloat16 or float32");
  return static_quantize_launch(x, x_dtype, numel, scale, zero_point, q, (cudaStream_t)stream);
}

extern "C" int zt_static_qlinear(const zt_static_qlinear_args_t *a, void *stream) {
  ZT_REQUIRE(a != nullptr, ZT_INVALID_ARGUMENT, "zt_static_qlinear: null argument block");
  ZT_REQUIRE(a->M >= 0 && a->N >= 0 && a->K >= 0, ZT_INVALID_ARGUMENT, "zt_static_qlinear: negative size");
  const bool x_quantized = a->x_dtype == ZT_U8 || a->x_dtype == ZT_S8;
  ZT_REQUIRE(valid_dtype(a->x_dtype) || x_quantized, ZT_INVALID_ARGUMENT,
             "unsupported dtype for input tensor, only float32/bfloat16/uint8/int8 is supported");
  ZT_REQUIRE(!a->bias || valid_dtype(a->bias_dtype), ZT_INVALID_ARGUMENT,
             "unsupported dtype for bias tensor, only float32 or bfloat16 is supported");
  ZT_REQUIRE(a->y_dtype == ZT_F32 || a->y_dtype == ZT_BF16 || a->y_dtype == ZT_U8 || a->y_dtype == ZT_S8,
             ZT_INVALID_ARGUMENT, "unsupported dtype for result tensor, only float32/bfloat16/uint8/int8 is supported");
  if (a->out_scale) {
    ZT_REQUIRE(a->y_dtype == (a->out_zero_point ? ZT_U8 : ZT_S8), ZT_INVALID_ARGUMENT,
               "unsupported dtype for result tensor when output_scales are defined: uint8 with output_zero_points, "
               "int8 without");
  } else {
    ZT_REQUIRE(!a->out_zero_point && valid_dtype(a->y_dtype), ZT_INVALID_ARGUMENT,
               "unsupported dtype for result tensor, only float32/bfloat16 is supported when output_scales are not "
               "defined");
  }
  ZT_REQUIRE(a->x_dtype != ZT_U8 || a->x_zero_point, ZT_INVALID_ARGUMENT,
             "zt_static_qlinear: an unsigned 8-bit input needs input_zero_points");
  ZT_REQUIRE(a->x_dtype != ZT_S8 || !a->x_zero_point, ZT_INVALID_ARGUMENT,
             "zt_static_qlinear: a signed 8-bit input takes no input_zero_points");
  ZT_REQUIRE(a->w_scales_numel == 1 || a->w_scales_numel == a->N, ZT_INVALID_ARGUMENT,
             "unsupported number of elements for weight_scales with respect to weight tensor");
  ZT_REQUIRE(valid_dtype(a->post_buffer_dtype), ZT_INVALID_ARGUMENT,
             "unsupported dtype for post_ops, only float32/bfloat16 is supported");
  if (a->M == 0 || a->N == 0) return ZT_SUCCESS;
  ZT_REQUIRE(a->K >= 1, ZT_INVALID_ARGUMENT, "zt_static_qlinear: K must be positive");
  ZT_REQUIRE(a->x && a->x_scale && a->w && a->w_scales && a->y, ZT_INVALID_ARGUMENT,
             "zt_static_qlinear: null tensor pointer");
  ZT_REQUIRE(!a->x_zero_point || a->w_rowsum, ZT_INVALID_ARGUMENT,
             "zt_static_qlinear: input_zero_points need w_rowsum (zt_int8_weight_rowsum)");
  ZT_REQUIRE(a->ldy >= a->N, ZT_INVALID_ARGUMENT, "zt_static_qlinear: ldy (%lld) is smaller than N (%lld)",
             (long long)a->ldy, (long long)a->N);
  int rc = validate_post_ops(a->post);
  if (rc != ZT_SUCCESS) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  CallOverlap overlap(!(a->flags & ZT_FLAG_WEIGHTS_VOLATILE));
  const void *q = a->x;
  if (!x_quantized) {
    const size_t need = zt_static_qlinear_workspace_bytes(a->M, a->K, a->x_dtype);
    ZT_REQUIRE(a->workspace && a->workspace_bytes >= need, ZT_WORKSPACE_TOO_SMALL,
               "zt_static_qlinear: workspace of %zu bytes is smaller than the %zu required", a->workspace_bytes, need);
    ZT_REQUIRE((reinterpret_cast<uintptr_t>(a->workspace) & 255) == 0, ZT_INVALID_ARGUMENT,
               "zt_static_qlinear: workspace must be 256-byte aligned");
    rc = static_quantize_launch(a->x, a->x_dtype, a->M * a->K, a->x_scale, a->x_zero_point, a->workspace, st);
    if (rc != ZT_SUCCESS) return rc;
    q = a->workspace;
  }
  Int8GemmArgs g{};
  g.q = q;
  g.q_is_u8 = a->x_zero_point != nullptr;
  g.w = a->w;
  g.M = a->M;
  g.N = a->N;
  g.K = a->K;
  g.raw_s32 = false;
  g.src_scale = a->x_scale;
  g.src_zp = a->x_zero_point;
  g.w_scale = a->w_scales;
  g.w_scale_dtype = ZT_F32;
  g.w_rowsum = a->x_zero_point ? a->w_rowsum : nullptr;
  g.bias = a->bias;
  g.bias_dtype = a->bias_dtype;
  g.y_dtype = a->y_dtype;
  g.y = a->y;
  g.post = to_dev(a->post);
  g.static_mode = true;
  g.w_scale_per_tensor = a->w_scales_numel == 1 && a->N != 1;
  g.post_dtype = a->post_buffer_dtype;
  g.out_scale = a->out_scale;
  g.out_zp = a->out_zero_point;
  g.ldy = a->ldy;
  return run_int8_gemm(g, a->algo, st);
}

// ---- allocation-free variant of zt_dynamic_qlinear ------------------------------------------------------
// The scratch lives in the library's device image.  In host code the array's name is only a handle
// for the runtime, not a device address: the address is looked up once per device with
// cudaGetSymbolAddress (that device being current) and only that pointer is handed to kernels.
namespace {
constexpr size_t kStaticRowBytes = (size_t)ZT_STATIC_SCRATCH_MAX_ROWS * 4;  // scales, then zero points
constexpr size_t kStaticScratchBytes = (size_t)ZT_STATIC_SCRATCH_Q_BYTES + 2 * kStaticRowBytes;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

int static_scratch_ptr(void **out) {
  static void *ptrs[64] = {nullptr};
  int dev = 0;
  ZT_CUDA_OK(cudaGetDevice(&dev));
  ZT_REQUIRE(dev >= 0 && dev < 64, ZT_UNSUPPORTED, "zt_dynamic_qlinear_static: device index %d out of range", dev);
  if (!ptrs[dev]) {
    void *p = nullptr;
    ZT_CUDA_OK(cudaGetSymbolAddress(&p, g_static_scratch));
    ZT_REQUIRE(p != nullptr, ZT_CUDA_ERROR, "zt_dynamic_qlinear_static: no device address for the scratch array");
    ptrs[dev] = p;
  }
  *out = ptrs[dev];
  return ZT_SUCCESS;
}
}  // namespace

extern "C" int zt_dynamic_qlinear_static(const zt_dynamic_qlinear_args_t *a, void *stream) {
  ZT_REQUIRE(a != nullptr, ZT_INVALID_ARGUMENT, "zt_dynamic_qlinear_static: null argument block");
  ZT_REQUIRE(a->M >= 0 && a->N >= 0 && a->K >= 0, ZT_INVALID_ARGUMENT, "zt_dynamic_qlinear_static: negative size");
  ZT_REQUIRE(a->M <= ZT_STATIC_SCRATCH_MAX_ROWS, ZT_UNSUPPORTED,
             "zt_dynamic_qlinear_static: M = %lld exceeds the built-in scratch (at most %d rows); use "
             "zt_dynamic_qlinear with a caller workspace",
             (long long)a->M, ZT_STATIC_SCRATCH_MAX_ROWS);
  ZT_REQUIRE(a->K == 0 || a->M <= (int64_t)ZT_STATIC_SCRATCH_Q_BYTES / a->K, ZT_UNSUPPORTED,
             "zt_dynamic_qlinear_static: M*K = %lld x %lld exceeds the built-in scratch (at most %u bytes of "
             "quantised activations); use zt_dynamic_qlinear with a caller workspace",
             (long long)a->M, (long long)a->K, (unsigned)ZT_STATIC_SCRATCH_Q_BYTES);
  void *scratch = nullptr;
  int rc = static_scratch_ptr(&scratch);
  if (rc != ZT_SUCCESS) return rc;
  // Same layout as the caller-workspace path expects: q | scales | zero points, each 256-byte aligned.
  zt_dynamic_qlinear_args_t b = *a;
  b.workspace = scratch;
  b.workspace_bytes = kStaticScratchBytes;
  return zt_dynamic_qlinear(&b, stream);
}
