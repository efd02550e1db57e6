/* C ABI of libzentorch_b200.so: the quantized-linear hot path of zentorch on NVIDIA B200 (sm_100a).
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream (passed as void*, i.e. a
 * cudaStream_t; NULL is the legacy default stream).  Nothing here allocates device memory, nothing
 * synchronises the host with the device, and every call may be captured in a CUDA graph unless its
 * comment says otherwise.  Calls return ZT_SUCCESS or an error code; zt_last_error() gives the
 * message of the last failure on the calling thread.  There is no CPU fallback: on a machine
 * without an sm_100 GPU the compute entry points fail with ZT_CUDA_ERROR.
 *
 * Each declaration cites the reference interface it stands in for (paths are those of the
 * amd/ZenDNN-pytorch-plugin tree).
 */
#ifndef ZENTORCH_B200_H_
#define ZENTORCH_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ZT_API __attribute__((visibility("default")))

typedef enum {
  ZT_SUCCESS = 0,
  ZT_INVALID_ARGUMENT = 1,
  ZT_UNSUPPORTED = 2,
  ZT_CUDA_ERROR = 3,
  ZT_WORKSPACE_TOO_SMALL = 4,
  ZT_DEVICE_TIMEOUT = 5 /* a bounded device-side wait expired; the context stays usable */
} zt_status_t;

typedef enum { ZT_BF16 = 0, ZT_F32 = 1, ZT_U8 = 2, ZT_S8 = 3 } zt_dtype_t; /* 8-bit types: static qlinear only */

/* Post-op ids; same values as UNARY_POST_OP / BINARY_POST_OP in src/cpu/cpp/Utils.hpp:56-72. */
typedef enum {
  ZT_POST_NONE = 0,
  ZT_POST_RELU = 1,
  ZT_POST_GELU_TANH = 2,
  ZT_POST_GELU_ERF = 3,
  ZT_POST_SILU = 4,
  ZT_POST_SIGMOID = 5,
  ZT_POST_TANH = 6,
  ZT_POST_MUL = 7,
  ZT_POST_ADD = 8
} zt_post_op_t;

#define ZT_MAX_POST_OPS 4

/* Argument-block flags.
 *
 * The linears treat weights, weight scales, zero points and row sums as constants (the reference passes
 * is_weights_const = true to the library for the same tensors, src/cpu/cpp/WOQ_Linear.cpp:107,
 * src/cpu/cpp/DynamicQLinear.cpp:128): kernels start fetching them while the work submitted before on the
 * same stream may still be running, and order themselves after that work only before they touch
 * activations, scratch and output.  ZT_FLAG_WEIGHTS_VOLATILE tells a call that one of those tensors may
 * have been written by work submitted to the stream directly before it (a repack, a copy, a cast): every
 * kernel of the call then starts only after all earlier work on the stream has completed. */
#define ZT_FLAG_WEIGHTS_VOLATILE 1

/* Ordered post-op chain applied to the fp32 result after the bias (matmul_post_ops,
 * src/cpu/cpp/MatmulUtils.hpp:36-77).  MUL/ADD consume `buffers` in order; each buffer is a
 * contiguous [M, N] array of the output dtype. */
typedef struct {
  int32_t n_ops;
  int32_t ids[ZT_MAX_POST_OPS];
  const void *buffers[ZT_MAX_POST_OPS];
} zt_post_ops_t;

/* Kernel selection.  AUTO picks by shape; the others force one kernel and fail with
 * ZT_UNSUPPORTED when the shape does not fit it (used by tests and the benchmark). */
typedef enum {
  ZT_ALGO_AUTO = 0,
  ZT_ALGO_GENERIC = 1, /* any shape, CUDA cores */
  ZT_ALGO_SKINNY = 2,  /* small M, HBM-bound streaming kernel */
  ZT_ALGO_TCGEN05 = 3  /* large M, tcgen05 tensor cores with TMEM accumulators */
} zt_algo_t;
/* An `algo` argument may carry a tile-width hint for the tcgen05 kernels in bits 8..23 (0 = choose);
 * tests and benchmarks use it to exercise every compiled tile shape. */
#define ZT_ALGO_WITH_TILE(algo, tile_n) ((int32_t)(algo) | ((int32_t)(tile_n) << 8))
/* Bit 24: the weight-only tcgen05 kernel with a single MMA issuer instead of two (tests compare the two forms). */
#define ZT_ALGO_SINGLE_ISSUER (1 << 24)

ZT_API const char *zt_last_error(void);
ZT_API const char *zt_version(void);
/* 1 when the current CUDA device is compute capability 10.x, else 0 (replaces the AVX-512 gate
 * is_avx512_supported, src/cpu/cpp/Utils.hpp:28-35). */
ZT_API int zt_device_supported(void);
/* Reads the device-side status word that a kernel sets when one of its bounded waits expires
 * (0 = none; 101..104 name the waiting role of a linear, 105 a peer that did not show up in zt_allreduce_bf16).  Synchronises with the device; `reset` clears it.
 * No counterpart in the reference (its failures are host exceptions, src/cpu/cpp/Utils.hpp:21-23). */
ZT_API int zt_poll_device_status(int *status, int reset);
/* Exercises that path without a fault: launches a one-thread kernel whose wait on a barrier nobody
 * signals gives up after a few thousand polls (microseconds), records status 199 and returns normally.
 * For tests of the host-side handling; no counterpart in the reference. */
ZT_API int zt_selftest_expire_wait(void *stream);
/* Latency analysis of the decode kernels (no counterpart in the reference).  While a device buffer is set,
 * every launch of zt_woq_linear's decode kernels reserves one record per CTA in it, in launch order, and
 * one thread of each CTA stores the GPU's nanosecond timer at up to eight points: 0 entry, 1 weight
 * prefetch issued, 2 ordered after earlier work, 3 first activations ready for the arithmetic, 4 main loop
 * done, 5 CTA reduction done, 6 cross-CTA reduction done, 7 output written (points a kernel does not have
 * stay zero).  Records hold 8 uint64 each; launches that no longer fit are not recorded.  Pass NULL to
 * switch it off (the default). */
ZT_API int zt_debug_set_timeline(void *device_buffer, size_t bytes);

/* ---------------------------------------------------------------------------------------------
 * Weight-only int4 linear.   zentorch_woq_linear_impl, src/cpu/cpp/WOQ_Linear.cpp:14-176, and the
 * eight op variants built on it (:178-292, :482-507).
 *
 *   Y[M,N] = post_ops( X[M,K] . dq(Wq)[K,N] + bias[N] )
 *
 * wq      int32 words, N-major: the nibble of logical element (k, n) is bits [4(k%8), 4(k%8)+4) of
 *         word n*(K/8) + k/8.  This is the storage behind the op's weight argument of shape
 *         [K/8, N] with strides (1, K/8)  (WOQ_Linear.cpp:138-146).
 * scales  [n_groups, N] contiguous, fp32 or bf16; group size = K / n_groups (n_groups = 1 is
 *         per-channel).
 * zeros   NULL: nibbles are signed (-8..7) and dq = q*s.  Otherwise same shape/dtype as scales,
 *         nibbles are unsigned (0..15) and dq = (q-8)*s + z  (WOQ_Linear.cpp:47-49).
 * x, y    bf16, row-major, leading dimensions K and N.
 * workspace  device scratch of at least zt_woq_linear_workspace_bytes(M,N,K) bytes.  Its first
 *         ZT_WOQ_COUNTER_BYTES must be zero before the first call; every call that completes normally
 *         leaves them zero.  A call in which a bounded device-side wait expired (zt_poll_device_status
 *         reports a non-zero code) may leave counters behind: zero those bytes again before the
 *         workspace is reused, or later calls elect no finisher for the affected column tiles.
 *         Calls that share a workspace must be ordered on one stream.
 */
#define ZT_WOQ_COUNTER_BYTES 16384

typedef struct {
  const void *x;
  int64_t M, K, N;
  const int32_t *wq;
  const void *scales;
  const void *zeros;
  int32_t scale_dtype; /* zt_dtype_t, also the dtype of zeros */
  int64_t n_groups;
  const void *bias; /* may be NULL */
  int32_t bias_dtype;
  zt_post_ops_t post;
  void *y;
  void *workspace;
  size_t workspace_bytes;
  int32_t algo;  /* zt_algo_t */
  int32_t flags; /* ZT_FLAG_* bits, 0 for constant weights */
} zt_woq_linear_args_t;

ZT_API size_t zt_woq_linear_workspace_bytes(int64_t M, int64_t N, int64_t K);
ZT_API int zt_woq_linear(const zt_woq_linear_args_t *args, void *stream);

/* zentorch_woq_repack_weight, src/cpu/cpp/WOQ_Linear.cpp:294-357: [N,K] int8 (one 4-bit value per
 * byte) -> [N,K/8] int32.  K must be a positive multiple of 8. */
ZT_API int zt_woq_repack_weight(const int8_t *unpacked, int64_t N, int64_t K, int32_t *packed, void *stream);

/* zentorch_woq_repack_from_int4pack, src/cpu/cpp/WOQ_Linear.cpp:361-433: PyTorch CPU int4pack
 * layout ([N, K/2] uint8 in 64-row blocks, device copy of it) -> [N,K/8] int32.  N % 64 == 0. */
ZT_API int zt_woq_repack_from_int4pack(const uint8_t *int4pack, int64_t N, int64_t K_half, int32_t *packed,
                                       void *stream);

/* ---------------------------------------------------------------------------------------------
 * Dynamic int8 linear.   zentorch_dynamic_qlinear(_impl), src/cpu/cpp/DynamicQLinear.cpp:74-181.
 *
 *   s_m = max(absmax_k |x[m,k]|, 1e-12) / 127 ;  q = clamp(rint(x / s_m), -128, 127)      (s8)
 *   acc[m,n] = sum_k q[m,k] * W[n,k]  (int32) ;  Y = post_ops( acc * (s_m * w_n) + bias[n] )
 *
 * act_quant ZT_ACT_U8_ASYM (not in the reference op) quantises each row to unsigned 8 bit with a
 * zero point and corrects the accumulator with zp_m * sum_k W[n,k]; it needs `w_rowsum`.
 * Post-ops are likewise an extension: the reference op has none.
 *
 * x        [M,K] bf16 or fp32 row-major;  y has the same dtype, [M,N].
 * w        [N,K] int8 row-major (nn.Linear layout).
 * w_scales [N] fp32 or bf16.      bias [N] fp32 or bf16, may be NULL.
 * workspace at least zt_dynamic_qlinear_workspace_bytes(M,K) bytes: holds the quantised
 *          activations, their scales and zero points between the two kernels.
 */
typedef enum { ZT_ACT_S8_SYM = 0, ZT_ACT_U8_ASYM = 1 } zt_act_quant_t;

typedef struct {
  const void *x;
  int32_t x_dtype;
  int64_t M, K, N;
  const int8_t *w;
  const void *w_scales;
  int32_t w_scale_dtype;
  const void *bias;
  int32_t bias_dtype;
  int32_t act_quant;       /* zt_act_quant_t */
  const int32_t *w_rowsum; /* [N], required for ZT_ACT_U8_ASYM (zt_int8_weight_rowsum) */
  zt_post_ops_t post;
  void *y;
  void *workspace;
  size_t workspace_bytes;
  int32_t algo;
  int32_t flags; /* ZT_FLAG_* bits, 0 for constant weights */
} zt_dynamic_qlinear_args_t;

ZT_API size_t zt_dynamic_qlinear_workspace_bytes(int64_t M, int64_t K);
ZT_API int zt_dynamic_qlinear(const zt_dynamic_qlinear_args_t *args, void *stream);

/* zt_dynamic_qlinear for callers that cannot allocate device memory.
 *
 * This entry point has no counterpart in the reference.  Some hosts of this library cannot call
 * cudaMalloc at the point where they run a linear: a runtime that hands out all device memory up
 * front from its own arena and forbids later driver allocations, code running inside a region where
 * allocation is illegal, or a plugin loaded into a process whose allocator it may not touch.  For
 * them the scratch that zt_dynamic_qlinear needs between its two kernels (the quantised activations,
 * their scales and zero points) lives in a fixed array inside the library's device image instead of a
 * caller-provided workspace: `workspace` / `workspace_bytes` of the argument block are ignored, inputs
 * and outputs are still the caller's.
 *
 * Limits: M * K <= ZT_STATIC_SCRATCH_Q_BYTES (8 MiB of quantised activations, e.g. 2048 x 4096) and
 * M <= ZT_STATIC_SCRATCH_MAX_ROWS; larger problems are rejected with ZT_UNSUPPORTED and a message
 * naming the limit.  Every GPU on which the library is loaded holds the array (8 MiB + 128 KiB) until
 * the process exits.  The call performs no cudaMalloc / cudaFree and calls no allocating library
 * routine.
 *
 * The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that
 * device current) and caches it; make that first call before starting any stream capture.  All calls
 * on a device share the one array and every call overwrites what it uses of it, so two calls that can
 * overlap on the GPU (different streams without an ordering between them) race on it: order them.
 * Nothing in the array has to be zero on entry. */
#define ZT_STATIC_SCRATCH_Q_BYTES (8u << 20)
#define ZT_STATIC_SCRATCH_MAX_ROWS 16384
ZT_API int zt_dynamic_qlinear_static(const zt_dynamic_qlinear_args_t *args, void *stream);

/* The first phase of zentorch_dynamic_qlinear on its own: per-row quantisation.  q is [M,K] int8
 * (s8) or uint8 (u8); scales [M] fp32; zero_points [M] int32 (u8 mode only, else may be NULL). */
ZT_API int zt_dynamic_quantize(const void *x, int32_t x_dtype, int64_t M, int64_t K, int32_t act_quant, void *q,
                               float *scales, int32_t *zero_points, void *stream);

/* The second phase on its own: the int8 GEMM with the scale/bias/post-op epilogue, on activations
 * that were quantised before (by zt_dynamic_quantize).  `args->x` is ignored; x_dtype still names the
 * output dtype; `q` is [M,K] s8/u8 per args->act_quant, `src_scales` [M] fp32, `src_zero_points` [M]
 * int32 (u8 mode).  No workspace is needed. */
ZT_API int zt_qlinear_prequantized(const zt_dynamic_qlinear_args_t *args, const void *q, const float *src_scales,
                                   const int32_t *src_zero_points, void *stream);

/* The second phase without its epilogue: acc[M,N] = q[M,K] . W[N,K]^T in exact int32.  Exposed so
 * that the accumulators can be compared bit for bit. */
ZT_API int zt_int8_gemm_s32(const void *q, int32_t q_is_u8, const int8_t *w, int64_t M, int64_t N, int64_t K,
                            int32_t *acc, int32_t algo, void *stream);

/* rowsum[n] = sum_k W[n,k]; a one-off weight-prepack by-product used by ZT_ACT_U8_ASYM. */
ZT_API int zt_int8_weight_rowsum(const int8_t *w, int64_t N, int64_t K, int32_t *rowsum, void *stream);

/* ---------------------------------------------------------------------------------------------
 * zentorch_qlinear and its _relu / _sigmoid / _mul_add / .out variants: the static-quantisation linear
 * (zentorch_quantized_matmul_impl, src/cpu/cpp/QLinear.cpp:66-366; operators :368-591).
 *
 *   q   = x                                             when x is u8 / s8 already, else
 *   q   = clamp(rint(x * (1 / s_x)) + zp_x)             u8 when x_zero_point is given, s8 (zp = 0) otherwise
 *   acc = sum_k (q[m,k] - zp_x) * W[n,k]                exact int32
 *   v   = post_ops( acc * (s_x * s_w[n]) + bias[n] )    fp32
 *   y   = v                                             as fp32 / bf16 when out_scale is NULL, else
 *   y   = clamp(rint(v * (1 / s_o)) + zp_o)             u8 when out_zero_point is given, s8 otherwise
 *
 * Scales and zero points are per tensor and live in device memory (they are tensors at the operator
 * level; nothing is read back to the host): one float / one int32 each.  The weight is symmetric s8 [N, K]
 * with one scale or one per output channel; weight zero points are not supported by the reference either
 * (QLinear.cpp:255-270).
 *
 * x          [M, K] row-major: ZT_F32 / ZT_BF16 (quantised by the call) or ZT_U8 / ZT_S8.  An unsigned
 *            input needs x_zero_point, a signed one must not have it.
 * w_rowsum   [N] int32 (zt_int8_weight_rowsum), required when x_zero_point is given.
 * post       chain of zt_post_op_t; binary operands are [M, N] contiguous arrays of post_buffer_dtype
 *            (ZT_F32 / ZT_BF16), whatever the output dtype (src/cpu/cpp/MatmulUtils.hpp:418-429).
 * y, ldy     output of y_dtype, row m at y + m * ldy elements (ldy >= N; the .out operators write into
 *            views of wider buffers, QLinear.cpp:409-411).
 * workspace  at least zt_static_qlinear_workspace_bytes(M, K, x_dtype) bytes, 256-byte aligned: holds the
 *            quantised activations (nothing when x is quantised already). */
typedef struct {
  const void *x;
  int32_t x_dtype;
  int64_t M, K, N;
  const float *x_scale;
  const int32_t *x_zero_point; /* NULL: signed activations */
  const int8_t *w;
  const float *w_scales;
  int64_t w_scales_numel;      /* 1 or N */
  const int32_t *w_rowsum;
  const void *bias;            /* [N] or NULL */
  int32_t bias_dtype;
  zt_post_ops_t post;
  int32_t post_buffer_dtype;
  const float *out_scale;          /* NULL: float output */
  const int32_t *out_zero_point;   /* NULL with out_scale: s8 output */
  void *y;
  int32_t y_dtype;
  int64_t ldy;
  void *workspace;
  size_t workspace_bytes;
  int32_t algo;
  int32_t flags; /* ZT_FLAG_* bits */
} zt_static_qlinear_args_t;

ZT_API size_t zt_static_qlinear_workspace_bytes(int64_t M, int64_t K, int32_t x_dtype);
ZT_API int zt_static_qlinear(const zt_static_qlinear_args_t *args, void *stream);

/* The quantisation step of zt_static_qlinear on its own (quantize_bf16_to_int8 and the
 * at::quantize_per_tensor call of src/cpu/cpp/QLinear.cpp:14-64,140-157): numel elements of fp32 / bf16 to
 * u8 (zero_point given) or s8. */
ZT_API int zt_static_quantize(const void *x, int32_t x_dtype, int64_t numel, const float *scale,
                              const int32_t *zero_point, void *q, void *stream);

/* ---------------------------------------------------------------------------------------------
 * Mixture-of-experts FFN with int4 weight-only experts (Mixtral style, symmetric group-wise scales).
 * The reference's zentorch_fused_moe (src/cpu/cpp/FusedMoE.cpp:470-744) takes bf16 / fp32 / int8 expert
 * weights only (src/cpu/cpp/GroupMatmul.cpp:104-108); this is the int4 form with the same structure:
 * per-expert token groups (FusedMoE.cpp:289-436), h = x_e . W13_e with [gate | up] columns, gate first
 * (src/cpu/python/zentorch/vllm/_int8_moe_patch.py:48-50), a = silu(gate) * up, o = a . W2_e,
 * y[t] = sum_j topk_weights[t,j] * o_j[t].
 *
 * x            [T, H] bf16                      y  [T, H] bf16
 * topk_ids     [T, top_k] int32; ids outside [0, num_experts) are skipped (expert-parallel ranks)
 * topk_weights [T, top_k] fp32
 * w13          [E, 2I, H/8] int32, every expert in the zentorch_woq_linear weight layout (N-major)
 * s13          [E, H/group_size, 2I]            w2 [E, H, I/8]        s2 [E, I/group_size, H]
 * workspace    zt_moe_woq_workspace_bytes() bytes, 256-byte aligned
 * No host synchronisation: group sizes stay on the device. */
typedef struct {
  const void *x;
  int64_t T, H, I;
  int32_t num_experts, top_k;
  const int32_t *topk_ids;
  const float *topk_weights;
  const int32_t *w13;
  const void *s13;
  const int32_t *w2;
  const void *s2;
  int32_t scale_dtype;
  int64_t group_size;
  void *y;
  void *workspace;
  size_t workspace_bytes;
} zt_moe_woq_args_t;

ZT_API size_t zt_moe_woq_workspace_bytes(int64_t T, int64_t H, int64_t I, int32_t num_experts, int32_t top_k);
ZT_API int zt_moe_woq(const zt_moe_woq_args_t *args, void *stream);

/* ---------------------------------------------------------------------------------------------
 * All-reduce of a small bf16 tensor over peer memory, for the collective that follows a row-parallel decode
 * linear.  The reference has no communication code (it only makes its int4 tensors sliceable for vLLM's
 * tensor-parallel loader, src/cpu/python/zentorch/vllm/_torchao_int4_opaque_patch.py:93-163); this is the
 * B200 side of that sharding: one process per GPU, every GPU owns a symmetric buffer of
 * zt_allreduce_symmetric_bytes(max_bytes) bytes that all peers can address (peer access enabled or an
 * imported allocation), zero before the first call.
 *
 *   peer_base[r]  base address of rank r's symmetric buffer as seen from this GPU (r = rank: its own)
 *   in, out       [numel] bf16 on this GPU, 16-byte aligned, numel a multiple of 8; may alias
 *   epochs        two uint32 in this GPU's own memory, zero before the first call; the kernel numbers the
 *                 calls with them (so a captured launch can be replayed)
 *
 * Every rank must issue the same sequence of calls with the same sizes.  Each rank adds the partial sums in
 * rank order in fp32, so all ranks hold identical results.  A peer that does not show up within the poll
 * limit (about a second) makes the call give up: the device status word is set (105) and `out` is left
 * unwritten.  Tensors larger than max_bytes are refused (ZT_UNSUPPORTED): use the library collective. */
#define ZT_AR_MAX_RANKS 8
#define ZT_AR_MAX_SLICES 64
typedef struct {
  const void *in;
  void *out;
  int64_t numel;
  void *peer_base[ZT_AR_MAX_RANKS];
  int32_t rank, world;
  size_t max_bytes; /* largest tensor, as given to zt_allreduce_symmetric_bytes */
  uint32_t *epochs;
} zt_allreduce_args_t;

ZT_API size_t zt_allreduce_symmetric_bytes(size_t max_bytes);
ZT_API int zt_allreduce_bf16(const zt_allreduce_args_t *args, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* ZENTORCH_B200_H_ */
