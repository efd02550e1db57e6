// Thin PyTorch boundary: the reference's operator schemas with a CUDA dispatch key.
//
// The schema strings are those of src/cpu/cpp/WOQ_Linear.cpp:435-480 and
// src/cpu/cpp/DynamicQLinear.cpp:184-189; they are defined here only when no other library has
// defined them already (a real zentorch registers CPU kernels for the same names, and both can be
// loaded in one process).  Every CUDA implementation marshals tensors into the plain-pointer C ABI
// of libzentorch_b200 (include/zentorch_b200.h) and launches on the current CUDA stream; nothing
// here computes.  The AOTInductor C shims mirror src/cpu/cpp/shim_cpu_zentorch.hpp:150-197 with the
// device name Inductor derives for CUDA tensors.
#include <ATen/ATen.h>
#include <ATen/core/dispatch/Dispatcher.h>
#include <ATen/cuda/CUDAContext.h>
#include <ATen/record_function.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/csrc/inductor/aoti_torch/c/shim.h>
#include <torch/csrc/inductor/aoti_torch/utils.h>
#include <torch/library.h>

#include <functional>
#include <map>
#include <tuple>
#include <mutex>
#include <optional>
#include <string>
#include <vector>

#include "../../include/zentorch_b200.h"

namespace zentorch_b200 {

namespace {

#define ZT_TORCH_CALL(expr)                                         \
  do {                                                              \
    const int rc__ = (expr);                                        \
    TORCH_CHECK(rc__ == ZT_SUCCESS, zt_last_error());               \
  } while (0)

int to_zt_dtype(const at::Tensor &t, const char *what) {
  if (t.scalar_type() == at::kBFloat16) return ZT_BF16;
  if (t.scalar_type() == at::kFloat) return ZT_F32;
  TORCH_CHECK(false, what, " must be float32 or bfloat16, got ", t.scalar_type());
  return -1;
}

// Flattens all but the last dimension (get_contiguous_view + get_2d_size_for_tensor,
// src/cpu/cpp/MatmulUtils.hpp:79-92, 554-563).
at::Tensor as_2d(const at::Tensor &t) {
  const bool zero_stride = std::any_of(t.strides().begin(), t.strides().end(), [](int64_t s) { return s == 0; });
  at::Tensor c = (t.is_contiguous() && !zero_stride) ? t : t.contiguous();
  const int64_t last = c.size(c.dim() - 1);
  return c.view({last == 0 ? 0 : c.numel() / last, last});
}

// Every tensor argument must live on the input's GPU: the kernels take raw pointers, and a host pointer or
// another device's pointer would fault on the GPU instead of raising here.
void check_on_device(const at::Tensor &t, const at::Tensor &input, const char *op, const char *name) {
  TORCH_CHECK(t.is_cuda() && t.device() == input.device(), op, ": ", name, " must be on the input's device (",
              input.device(), "), got ", t.device());
}
void check_on_device(const std::optional<at::Tensor> &t, const at::Tensor &input, const char *op, const char *name) {
  if (t.has_value() && t->defined()) check_on_device(*t, input, op, name);
}

// Weights are constants of a model, and the kernels read them before ordering themselves after earlier work
// on the stream.  That is only sound for a tensor that earlier work cannot still be writing, so the boundary
// keeps a record of the weight tensors it has seen: (storage, offset, version) with a weak reference that
// tells a live storage from a new one at a recycled address.  A tensor seen in an earlier call, with its
// storage still alive and its version unchanged, was produced before that call; anything else (first sight,
// a temporary made inside this call) is passed on as ZT_FLAG_WEIGHTS_VOLATILE.
//
// The same record is the prepacked-weight cache (the reference lets ZenDNN reorder a constant weight once and
// keep it: is_weights_const = true, src/cpu/cpp/WOQ_Linear.cpp:107, src/cpu/cpp/DynamicQLinear.cpp:128): an
// entry can carry a by-product of the weight that is computed on first sight and reused afterwards -- here the
// int32 row sums of an int8 weight, which the u8 activation mode needs in its epilogue.
class SeenWeights {
 public:
  bool seen_before(const at::Tensor &t) {
    at::Tensor unused;
    return lookup(t, nullptr, &unused);
  }
  // `make` is called on first sight (or after the tensor changed) and its result kept with the entry; returns
  // whether the tensor had been seen before, `*payload` receives the kept by-product.
  bool lookup(const at::Tensor &t, const std::function<at::Tensor()> *make, at::Tensor *payload) {
    if (!t.defined() || !t.has_storage()) {
      if (make) *payload = (*make)();
      return false;
    }
    c10::StorageImpl *impl = t.storage().unsafeGetStorageImpl();
    const Key key{impl, t.storage_offset(), t.numel()};
    const int64_t version = t.is_inference() ? 0 : (int64_t)t._version();
    std::lock_guard<std::mutex> lock(mu_);
    auto it = map_.find(key);
    if (it != map_.end() && !it->second.storage.expired() && it->second.version == version) {
      if (make && !it->second.payload.defined()) it->second.payload = (*make)();
      *payload = it->second.payload;
      return true;
    }
    if (map_.size() >= kMaxEntries) purge();
    Entry e{t.storage().getWeakStorageImpl(), version, make ? (*make)() : at::Tensor()};
    *payload = e.payload;
    map_.insert_or_assign(key, std::move(e));
    return false;
  }

 private:
  struct Key {
    const void *storage;
    int64_t offset, numel;
    bool operator<(const Key &o) const { return std::tie(storage, offset, numel) < std::tie(o.storage, o.offset, o.numel); }
  };
  struct Entry {
    c10::weak_intrusive_ptr<c10::StorageImpl> storage;
    int64_t version;
    at::Tensor payload;   // prepack by-product, may be undefined
  };
  static constexpr size_t kMaxEntries = 1 << 16;
  void purge() {
    for (auto it = map_.begin(); it != map_.end();) it = it->second.storage.expired() ? map_.erase(it) : std::next(it);
    if (map_.size() >= kMaxEntries) map_.clear();
  }
  std::mutex mu_;
  std::map<Key, Entry> map_;
};
SeenWeights &seen_weights() {
  static SeenWeights s;
  return s;
}

// Persistent scratch per (device, stream) for the split-K kernel: the counters at its front must
// stay zero between calls, so it cannot come from a fresh allocation every time.
std::mutex &workspace_mutex() {
  static std::mutex mu;
  return mu;
}
std::map<std::pair<int, void *>, at::Tensor> &workspace_pool() {
  static std::map<std::pair<int, void *>, at::Tensor> pool;
  return pool;
}

at::Tensor &woq_workspace(size_t bytes, c10::DeviceIndex dev, cudaStream_t stream) {
  std::lock_guard<std::mutex> lock(workspace_mutex());
  at::Tensor &t = workspace_pool()[{(int)dev, (void *)stream}];
  if (!t.defined() || (size_t)t.numel() < bytes) {
    const size_t grow = std::max<size_t>(bytes, 1 << 20);
    t = at::zeros({(int64_t)grow}, at::TensorOptions().dtype(at::kByte).device(at::kCUDA, dev));
  }
  return t;
}

struct PostSpec {
  std::vector<int> ids;
  std::vector<at::Tensor> operands;  // in consumption order
};

at::Tensor woq_linear_impl(const at::Tensor &input, const at::Tensor &weight, const at::Tensor &weight_scales,
                           const std::optional<at::Tensor> &weight_zero_points, const std::optional<at::Tensor> &bias,
                           const PostSpec &post, const std::string &op_name) {
  RECORD_FUNCTION(op_name, std::vector<c10::IValue>({input, weight}));
  TORCH_CHECK(input.is_cuda(), "zentorch_woq_linear (CUDA): input must be a CUDA tensor");
  check_on_device(weight, input, "zentorch_woq_linear", "weight");
  check_on_device(weight_scales, input, "zentorch_woq_linear", "weight_scales");
  check_on_device(weight_zero_points, input, "zentorch_woq_linear", "weight_zero_points");
  check_on_device(bias, input, "zentorch_woq_linear", "bias");
  for (const at::Tensor &t : post.operands) check_on_device(t, input, "zentorch_woq_linear", "binary post-op operand");
  TORCH_CHECK(weight.dtype() == at::kInt, "weight must have dtype int32, got ", weight.dtype());
  TORCH_CHECK(weight.dim() == 2, "weight must be 2D, got ", weight.dim(), "D");
  TORCH_CHECK(weight_scales.dim() == 2, "weight_scales must be 2D [groups, N], got ", weight_scales.dim(), "D");
  TORCH_CHECK(weight_scales.size(1) == weight.size(1), "weight_scales dim 1 (", weight_scales.size(1),
              ") must match weight dim 1 (", weight.size(1), ")");
  TORCH_CHECK(input.scalar_type() == at::kBFloat16, "zentorch_woq_linear: input must be bfloat16, got ",
              input.scalar_type());
  const int64_t k8 = weight.size(0), N = weight.size(1), K = k8 * 8;
  TORCH_CHECK(input.dim() >= 1 && input.size(-1) == K, "zentorch_woq_linear: input last dim (", input.size(-1),
              ") must match the unpacked weight rows (", K, ")");
  // The op's weight is the transposed view of the row-wise packed [N, K/8] tensor: element (k8, n)
  // at n*(K/8) + k8.  A row-major [K/8, N] tensor has no defined meaning in the reference either
  // (it hard-codes ldb = K, src/cpu/cpp/WOQ_Linear.cpp:100), so it is rejected rather than re-laid out.
  TORCH_CHECK((weight.stride(0) == 1 || k8 == 1) && (weight.stride(1) == k8 || N == 1),
              "zentorch_woq_linear: weight must be the transposed view of a contiguous [N, K/8] packed tensor "
              "(shape [K/8, N], strides (1, K/8)); got strides (",
              weight.stride(0), ", ", weight.stride(1), ")");
  c10::cuda::CUDAGuard device_guard(input.device());
  cudaStream_t stream = at::cuda::getCurrentCUDAStream();

  at::Tensor x2 = as_2d(input);
  std::vector<int64_t> out_sizes = input.sizes().vec();
  out_sizes.back() = N;
  at::Tensor result = at::empty(out_sizes, input.options());
  const int64_t M = x2.size(0);
  if (M == 0 || N == 0) return result;

  at::Tensor scales = weight_scales.contiguous();
  // constants of the call: tensors seen in an earlier call and passed through unchanged (no temporary made here)
  bool weights_const = seen_weights().seen_before(weight);
  weights_const = seen_weights().seen_before(weight_scales) && scales.is_same(weight_scales) && weights_const;
  at::Tensor zeros;
  if (weight_zero_points.has_value() && weight_zero_points->defined()) {
    TORCH_CHECK(weight_zero_points->sizes() == weight_scales.sizes(),
                "weight_zero_points must have the shape of weight_scales");
    zeros = weight_zero_points->to(scales.scalar_type()).contiguous();
    weights_const = seen_weights().seen_before(*weight_zero_points) && zeros.is_same(*weight_zero_points) && weights_const;
  }
  at::Tensor bias_c;
  if (bias.has_value() && bias->defined()) {
    TORCH_CHECK(bias->dim() == 1 && bias->size(0) == N, "bias must be 1D with size N (", N, ")");
    bias_c = bias->contiguous();
  }

  zt_woq_linear_args_t a{};
  a.x = x2.data_ptr();
  a.M = M;
  a.K = K;
  a.N = N;
  a.wq = reinterpret_cast<const int32_t *>(weight.data_ptr());
  a.scales = scales.data_ptr();
  a.zeros = zeros.defined() ? zeros.data_ptr() : nullptr;
  a.scale_dtype = to_zt_dtype(scales, "weight_scales");
  a.n_groups = scales.size(0);
  a.bias = bias_c.defined() ? bias_c.data_ptr() : nullptr;
  a.bias_dtype = bias_c.defined() ? to_zt_dtype(bias_c, "bias") : ZT_BF16;
  a.y = result.data_ptr();
  a.algo = ZT_ALGO_AUTO;
  a.flags = weights_const ? 0 : ZT_FLAG_WEIGHTS_VOLATILE;
  std::vector<at::Tensor> keep;
  a.post.n_ops = (int)post.ids.size();
  size_t b = 0;
  for (size_t i = 0; i < post.ids.size(); ++i) {
    a.post.ids[i] = post.ids[i];
    if (post.ids[i] == ZT_POST_MUL || post.ids[i] == ZT_POST_ADD) {
      const at::Tensor &t = post.operands.at(b);
      TORCH_CHECK(t.numel() == M * N, "binary post-op operand must have the shape of the result");
      TORCH_CHECK(t.scalar_type() == input.scalar_type(), "binary post-op operand must have the dtype of the input");
      keep.push_back(as_2d(t));
      a.post.buffers[b] = keep.back().data_ptr();
      ++b;
    }
  }
  const size_t ws_bytes = zt_woq_linear_workspace_bytes(M, N, K);
  at::Tensor &ws = woq_workspace(ws_bytes, input.device().index(), stream);
  a.workspace = ws.data_ptr();
  a.workspace_bytes = (size_t)ws.numel();
  ZT_TORCH_CALL(zt_woq_linear(&a, stream));
  return result;
}

template <int UNARY>
at::Tensor woq_linear_unary(const at::Tensor &input, const at::Tensor &weight, const at::Tensor &weight_scales,
                            const std::optional<at::Tensor> &zp, const std::optional<at::Tensor> &bias,
                            std::string zentorch_op_name) {
  PostSpec ps;
  if (UNARY != ZT_POST_NONE) ps.ids.push_back(UNARY);
  return woq_linear_impl(input, weight, weight_scales, zp, bias, ps, zentorch_op_name);
}

at::Tensor woq_linear_add(const at::Tensor &input, const at::Tensor &weight, const at::Tensor &weight_scales,
                          const std::optional<at::Tensor> &zp, const at::Tensor &add_input,
                          const std::optional<at::Tensor> &bias, std::string zentorch_op_name) {
  PostSpec ps{{ZT_POST_ADD}, {add_input}};
  return woq_linear_impl(input, weight, weight_scales, zp, bias, ps, zentorch_op_name);
}

template <int B1, int B2>
at::Tensor woq_linear_binary_binary(const at::Tensor &input, const at::Tensor &weight, const at::Tensor &weight_scales,
                                    const std::optional<at::Tensor> &zp, const at::Tensor &binary1,
                                    const at::Tensor &binary2, const std::optional<at::Tensor> &bias,
                                    std::string zentorch_op_name) {
  PostSpec ps{{B1, B2}, {binary1, binary2}};
  return woq_linear_impl(input, weight, weight_scales, zp, bias, ps, zentorch_op_name);
}

at::Tensor woq_repack_weight(const at::Tensor &unpacked_weight) {
  TORCH_CHECK(unpacked_weight.dtype() == at::kChar, "unpacked_weight must have dtype int8, got ",
              unpacked_weight.dtype());
  TORCH_CHECK(unpacked_weight.dim() == 2, "unpacked_weight must be 2D, got ", unpacked_weight.dim(), "D");
  TORCH_CHECK(unpacked_weight.is_cuda(), "zentorch_woq_repack_weight (CUDA): unpacked_weight must be a CUDA tensor");
  const int64_t N = unpacked_weight.size(0), K = unpacked_weight.size(1);
  TORCH_CHECK(K >= 8, "K must be at least 8, got ", K);
  TORCH_CHECK(K % 8 == 0, "K must be divisible by 8, got ", K);
  c10::cuda::CUDAGuard device_guard(unpacked_weight.device());
  at::Tensor w = unpacked_weight.contiguous();
  at::Tensor out = at::empty({N, K / 8}, w.options().dtype(at::kInt));
  ZT_TORCH_CALL(zt_woq_repack_weight(w.data_ptr<int8_t>(), N, K, out.data_ptr<int32_t>(),
                                     at::cuda::getCurrentCUDAStream().stream()));
  return out;
}

at::Tensor woq_repack_from_int4pack(const at::Tensor &packed_weight) {
  TORCH_CHECK(packed_weight.dtype() == at::kByte, "packed_weight must have dtype uint8, got ", packed_weight.dtype());
  TORCH_CHECK(packed_weight.dim() == 2, "packed_weight must be 2D, got ", packed_weight.dim(), "D");
  TORCH_CHECK(packed_weight.is_cuda(), "zentorch_woq_repack_from_int4pack (CUDA): packed_weight must be a CUDA tensor");
  const int64_t N = packed_weight.size(0), K_half = packed_weight.size(1);
  TORCH_CHECK(N % 64 == 0, "packed_weight row count (", N, ") must be a multiple of ", 64,
              ". The int4pack format from PyTorch pads N to BLOCK_N; "
              "receiving an unpadded tensor indicates a packing mismatch.");
  c10::cuda::CUDAGuard device_guard(packed_weight.device());
  at::Tensor w = packed_weight.contiguous();
  at::Tensor out = at::empty({N, K_half / 4}, w.options().dtype(at::kInt));
  ZT_TORCH_CALL(zt_woq_repack_from_int4pack(w.data_ptr<uint8_t>(), N, K_half, out.data_ptr<int32_t>(),
                                            at::cuda::getCurrentCUDAStream().stream()));
  return out;
}

// ---- dynamic qlinear ------------------------------------------------------------------------------
at::Tensor dynamic_qlinear_impl(const at::Tensor &input, const at::Tensor &weight, const at::Tensor &weight_scales,
                                const std::optional<at::Tensor> &bias, int act_quant, int post_op,
                                const std::optional<at::Tensor> &weight_rowsum, const std::string &op_name) {
  RECORD_FUNCTION(op_name, std::vector<c10::IValue>({input, weight}));
  // checks and messages of check_valid_dtypes/sizes_for_dynamic_qlinear, src/cpu/cpp/DynamicQLinear.cpp:15-70
  TORCH_CHECK(input.scalar_type() == at::kBFloat16 || input.scalar_type() == at::kFloat,
              "zentorch_dynamic_qlinear: input must be bfloat16 or float32, got ", input.scalar_type());
  TORCH_CHECK(weight_scales.scalar_type() == at::kFloat || weight_scales.scalar_type() == at::kBFloat16,
              "zentorch_dynamic_qlinear: weight_scales must be float32, bfloat16, got ", weight_scales.scalar_type());
  TORCH_CHECK(weight.scalar_type() == at::kChar, "zentorch_dynamic_qlinear: weight must be int8 (c10::kChar), got ",
              weight.scalar_type());
  const bool has_bias = bias.has_value() && bias->defined();
  if (has_bias) {
    TORCH_CHECK(bias->scalar_type() == at::kFloat || bias->scalar_type() == at::kBFloat16,
                "zentorch_dynamic_qlinear: bias must be float32 or bfloat16, got ", bias->scalar_type());
  }
  TORCH_CHECK(input.dim() >= 2, "zentorch_dynamic_qlinear: input must be at least 2D");
  TORCH_CHECK(weight.dim() == 2, "zentorch_dynamic_qlinear: weight must be 2D [N, K], got ", weight.dim(), "D");
  const int64_t N = weight.size(0), K = weight.size(1);
  TORCH_CHECK(input.size(input.dim() - 1) == K, "zentorch_dynamic_qlinear: input last dim (", input.size(-1),
              ") must match weight dim 1 (", K, ")");
  if (has_bias) {
    TORCH_CHECK(bias->dim() == 1 && bias->size(0) == N, "zentorch_dynamic_qlinear: bias must be 1D with size N (", N,
                ")");
  }
  TORCH_CHECK(weight_scales.numel() == N, "zentorch_dynamic_qlinear: weight_scales must hold N (", N, ") values");
  TORCH_CHECK(input.is_cuda(), "zentorch_dynamic_qlinear (CUDA): input must be a CUDA tensor");
  check_on_device(weight, input, "zentorch_dynamic_qlinear", "weight");
  check_on_device(weight_scales, input, "zentorch_dynamic_qlinear", "weight_scales");
  check_on_device(bias, input, "zentorch_dynamic_qlinear", "bias");
  check_on_device(weight_rowsum, input, "zentorch_dynamic_qlinear", "weight_rowsum");
  c10::cuda::CUDAGuard device_guard(input.device());
  cudaStream_t stream = at::cuda::getCurrentCUDAStream();

  std::vector<int64_t> out_sizes = input.sizes().vec();
  out_sizes.back() = N;
  at::Tensor result = at::empty(out_sizes, input.options());
  at::Tensor x2 = as_2d(input);
  const int64_t M = x2.size(0);
  if (M == 0 || N == 0) return result;
  at::Tensor w = weight.contiguous();
  at::Tensor ws = weight_scales.contiguous();
  at::Tensor b = has_bias ? bias->contiguous() : at::Tensor();
  const bool given_rowsum = weight_rowsum.has_value() && weight_rowsum->defined();
  at::Tensor rowsum;
  bool weights_const;
  if (act_quant == ZT_ACT_U8_ASYM && !given_rowsum) {
    // prepack by-product, computed when the weight is first seen and kept with its record
    bool computed_now = false;
    const std::function<at::Tensor()> make = [&]() {
      at::Tensor r = at::empty({N}, w.options().dtype(at::kInt));
      const int rc = zt_int8_weight_rowsum(w.data_ptr<int8_t>(), N, K, r.data_ptr<int32_t>(), stream);
      TORCH_CHECK(rc == ZT_SUCCESS, zt_last_error());
      computed_now = true;
      return r;
    };
    weights_const = seen_weights().lookup(weight, &make, &rowsum) && !computed_now;
  } else {
    weights_const = seen_weights().seen_before(weight);
  }
  weights_const = seen_weights().seen_before(weight_scales) && w.is_same(weight) && ws.is_same(weight_scales) && weights_const;
  if (act_quant == ZT_ACT_U8_ASYM && given_rowsum) {
    TORCH_CHECK(weight_rowsum->scalar_type() == at::kInt && weight_rowsum->numel() == N,
                "weight_rowsum must be int32 with N values");
    rowsum = weight_rowsum->contiguous();
    weights_const = seen_weights().seen_before(*weight_rowsum) && rowsum.is_same(*weight_rowsum) && weights_const;
  }
  const size_t ws_bytes = zt_dynamic_qlinear_workspace_bytes(M, K);
  at::Tensor scratch = at::empty({(int64_t)ws_bytes}, w.options().dtype(at::kByte));

  zt_dynamic_qlinear_args_t a{};
  a.x = x2.data_ptr();
  a.x_dtype = to_zt_dtype(x2, "input");
  a.M = M;
  a.K = K;
  a.N = N;
  a.w = w.data_ptr<int8_t>();
  a.w_scales = ws.data_ptr();
  a.w_scale_dtype = to_zt_dtype(ws, "weight_scales");
  a.bias = b.defined() ? b.data_ptr() : nullptr;
  a.bias_dtype = b.defined() ? to_zt_dtype(b, "bias") : ZT_F32;
  a.act_quant = act_quant;
  a.w_rowsum = rowsum.defined() ? rowsum.data_ptr<int32_t>() : nullptr;
  if (post_op != ZT_POST_NONE) {
    a.post.n_ops = 1;
    a.post.ids[0] = post_op;
  }
  a.y = result.data_ptr();
  a.workspace = scratch.data_ptr();
  a.workspace_bytes = ws_bytes;
  a.algo = ZT_ALGO_AUTO;
  a.flags = weights_const ? 0 : ZT_FLAG_WEIGHTS_VOLATILE;
  ZT_TORCH_CALL(zt_dynamic_qlinear(&a, stream));
  return result;
}

at::Tensor dynamic_qlinear(const at::Tensor &input, const at::Tensor &weight, const at::Tensor &weight_scales,
                           const std::optional<at::Tensor> &bias, std::string zentorch_op_name) {
  return dynamic_qlinear_impl(input, weight, weight_scales, bias, ZT_ACT_S8_SYM, ZT_POST_NONE, std::nullopt,
                              zentorch_op_name);
}

int post_id_from_name(const std::string &s) {
  static const std::map<std::string, int> names = {{"none", ZT_POST_NONE},         {"relu", ZT_POST_RELU},
                                                   {"gelu_tanh", ZT_POST_GELU_TANH}, {"gelu_erf", ZT_POST_GELU_ERF},
                                                   {"silu", ZT_POST_SILU},         {"sigmoid", ZT_POST_SIGMOID},
                                                   {"tanh", ZT_POST_TANH}};
  auto it = names.find(s);
  TORCH_CHECK(it != names.end(), "unknown post_op '", s, "'");
  return it->second;
}

// Extension (no reference counterpart): per-token u8 asymmetric activations and a fused unary post-op.
at::Tensor dynamic_qlinear_ext(const at::Tensor &input, const at::Tensor &weight, const at::Tensor &weight_scales,
                               const std::optional<at::Tensor> &bias, const std::optional<at::Tensor> &weight_rowsum,
                               std::string act_quant, std::string post_op, std::string zentorch_op_name) {
  TORCH_CHECK(act_quant == "s8_sym" || act_quant == "u8_asym", "act_quant must be 's8_sym' or 'u8_asym'");
  return dynamic_qlinear_impl(input, weight, weight_scales, bias, act_quant == "u8_asym" ? ZT_ACT_U8_ASYM : ZT_ACT_S8_SYM,
                              post_id_from_name(post_op), weight_rowsum, zentorch_op_name);
}

// ---- static-quantisation qlinear (src/cpu/cpp/QLinear.cpp:66-591) ------------------------------------------
int to_zt_dtype8(c10::ScalarType t) {
  switch (t) {
    case at::kBFloat16: return ZT_BF16;
    case at::kFloat: return ZT_F32;
    case at::kByte: return ZT_U8;
    case at::kChar: return ZT_S8;
    default: return -1;
  }
}

// Checks of check_valid_dtypes_for_quantized_matmul / check_valid_sizes_for_quantized_matmul
// (src/cpu/cpp/MatmulUtils.hpp:331-525) with their messages, then one zt_static_qlinear call that writes
// `result` (any float / 8-bit dtype; a 2-D view may have a row stride).
void qlinear_into(at::Tensor &result, const at::Tensor &input, const at::Tensor &weight, const at::Tensor &input_scales,
                  const at::Tensor &input_zero_points, const at::Tensor &weight_scales,
                  const at::Tensor &weight_zero_points, const std::optional<at::Tensor> &bias,
                  const std::optional<at::Tensor> &output_scales, const std::optional<at::Tensor> &output_zero_points,
                  const std::vector<int> &post_ops, const std::vector<at::Tensor> &post_buffers,
                  const std::string &op_name) {
  RECORD_FUNCTION(op_name, std::vector<c10::IValue>({input, weight}));
  const bool has_bias = bias.has_value() && bias->defined();
  const bool has_oscale = output_scales.has_value() && output_scales->defined();
  const bool has_ozp = output_zero_points.has_value() && output_zero_points->defined();
  const bool has_xzp = input_zero_points.defined();
  const int x_dtype = to_zt_dtype8(input.scalar_type());
  const int y_dtype = to_zt_dtype8(result.scalar_type());
  TORCH_CHECK(x_dtype >= 0, "unsupported dtype for input tensor, only float32/bfloat16/uint8/int8 is supported");
  TORCH_CHECK(weight.scalar_type() == at::kChar, "unsupported dtype for weight tensor, only int8 is supported");
  TORCH_CHECK(y_dtype >= 0, "unsupported dtype for result tensor, only float32/bfloat16/uint8/int8 is supported");
  if (has_bias)
    TORCH_CHECK(bias->scalar_type() == at::kFloat || bias->scalar_type() == at::kBFloat16,
                "unsupported dtype for bias tensor, only float32 or bfloat16 is supported");
  TORCH_CHECK(input_scales.scalar_type() == at::kFloat, "unsupported dtype for input_scales, only float32 is supported");
  if (has_xzp)
    TORCH_CHECK(input_zero_points.scalar_type() == at::kInt, "unsupported dtype for input_zero_points, only int32 supported");
  TORCH_CHECK(weight_scales.scalar_type() == at::kFloat, "unsupported dtype for weight_scales, only float32 is supported");
  if (weight_zero_points.defined())
    TORCH_CHECK(weight_zero_points.scalar_type() == at::kInt,
                "unsupported dtype for weight_zero_points, only int32 is supported");
  if (has_oscale) {
    TORCH_CHECK(output_scales->scalar_type() == at::kFloat, "unsupported dtype for output_scales, only float32 is supported");
    if (has_ozp) {
      TORCH_CHECK(output_zero_points->scalar_type() == at::kInt,
                  "unsupported dtype for output_zero_points, only int32 is supported");
      TORCH_CHECK(result.scalar_type() == at::kByte,
                  "unsupported dtype for result tensor when output_zero_points are defined, uint8 are supported dtype");
    } else {
      TORCH_CHECK(result.scalar_type() == at::kChar,
                  "unsupported dtype for result tensor when output_zero_points are not defined while output_scales are "
                  "defined, int8 are supported dtype");
    }
  } else {
    TORCH_CHECK(result.scalar_type() == at::kFloat || result.scalar_type() == at::kBFloat16,
                "unsupported dtype for result tensor, only float32/bfloat16 is supported when output_scales are not "
                "defined");
  }
  for (const at::Tensor &b : post_buffers)
    TORCH_CHECK(b.scalar_type() == at::kFloat || b.scalar_type() == at::kBFloat16,
                "unsupported dtype for post_ops, only float32/bfloat16 is supported");
  if (post_buffers.size() == 2)
    TORCH_CHECK(post_buffers[0].scalar_type() == post_buffers[1].scalar_type(),
                "unsupported dtype for post_ops, only float32/bfloat16 is supported");
  // sizes
  TORCH_CHECK(input.dim() >= 2 && weight.dim() == 2, "unsupported dims for input and weight");
  const int64_t N = weight.size(0), K = weight.size(1);
  TORCH_CHECK(input.size(input.dim() - 1) == K, "unsupported shapes for input and weight");
  if (has_bias) TORCH_CHECK(bias->dim() == 1 && bias->size(0) == N, "unsupported shapes for input, weight and bias");
  TORCH_CHECK(input_scales.dim() <= 1, "unsupported dims for input_scales with respect to input tensor");
  if (has_xzp) {
    TORCH_CHECK(input_zero_points.dim() <= 1, "only scalar and 1-d input_zero_points are supported");
    TORCH_CHECK(input_zero_points.numel() == 1, "only supporting per-tensor quantization for input");
  }
  TORCH_CHECK(input_scales.numel() == 1, "unsupported number of elements for input_scales with respect to input tensor");
  TORCH_CHECK(weight_scales.dim() <= 1, "unsupported dims for weight_scales with respect to weight tensor");
  TORCH_CHECK(weight_scales.numel() == 1 || weight_scales.numel() == N,
              "unsupported number of elements for weight_scales with respect to weight tensor");
  if (weight_zero_points.defined()) {
    TORCH_CHECK(weight_zero_points.dim() <= 1, "only scalar and 1-d weight_zero_points are supported");
    TORCH_CHECK(weight_zero_points.numel() == 1 || weight_zero_points.numel() == N,
                "only supporting per-tensor and per-channel quantization for weight");
  }
  if (has_oscale && has_ozp) {
    TORCH_CHECK(output_scales->dim() <= 1, "unsupported dims for output_scales with respect to output tensor");
    TORCH_CHECK(output_zero_points->dim() <= 1, "unsupported dims for output_zero_points with respect to output tensor");
    TORCH_CHECK(output_scales->numel() == 1, "unsupported number of elements for output_scales with respect to output tensor");
    TORCH_CHECK(output_zero_points->numel() == 1,
                "unsupported number of elements for output_zero_points with respect to output tensor");
  } else if (has_oscale) {
    TORCH_CHECK(output_scales->numel() == 1, "unsupported number of elements for output_scales with respect to output tensor");
  }
  std::vector<int64_t> out_sizes = input.sizes().vec();
  out_sizes.back() = N;
  TORCH_CHECK(result.sizes() == c10::IntArrayRef(out_sizes), "unsupported shapes for input, weight and result");
  for (const at::Tensor &b : post_buffers) {
    TORCH_CHECK(b.dim() == input.dim(), "unsupported dims for post op buffers for input and weight");
    TORCH_CHECK(b.sizes() == c10::IntArrayRef(out_sizes), "unsupported shapes for post op buffers for input and weight");
  }
  // the unsigned / signed form of the activations follows from the zero points, as in the reference
  // (QLinear.cpp:17,379-383): an unsigned input needs them, a signed one has none
  if (input.scalar_type() == at::kByte)
    TORCH_CHECK(has_xzp, "zentorch_qlinear: a uint8 input needs input_zero_points");
  if (input.scalar_type() == at::kChar)
    TORCH_CHECK(!has_xzp, "zentorch_qlinear: an int8 input takes no input_zero_points");
  TORCH_CHECK(input.is_cuda(), "zentorch_qlinear (CUDA): input must be a CUDA tensor");
  check_on_device(weight, input, "zentorch_qlinear", "weight");
  check_on_device(input_scales, input, "zentorch_qlinear", "input_scales");
  if (has_xzp) check_on_device(input_zero_points, input, "zentorch_qlinear", "input_zero_points");
  check_on_device(weight_scales, input, "zentorch_qlinear", "weight_scales");
  check_on_device(bias, input, "zentorch_qlinear", "bias");
  check_on_device(output_scales, input, "zentorch_qlinear", "output_scales");
  check_on_device(output_zero_points, input, "zentorch_qlinear", "output_zero_points");
  check_on_device(result, input, "zentorch_qlinear", "out");
  for (const at::Tensor &b : post_buffers) check_on_device(b, input, "zentorch_qlinear", "post-op operand");
  c10::cuda::CUDAGuard device_guard(input.device());
  cudaStream_t stream = at::cuda::getCurrentCUDAStream();

  at::Tensor x2 = as_2d(input);
  const int64_t M = x2.size(0);
  if (M == 0 || N == 0) return;
  // the result as rows of N elements `ldy` apart: contiguous tensors of any rank, or a 2-D view of a wider buffer
  int64_t ldy = N;
  if (result.dim() == 2 && result.stride(1) == 1 && result.stride(0) >= N) {
    ldy = M > 1 ? result.stride(0) : N;
  } else {
    TORCH_CHECK(result.is_contiguous(), "zentorch_qlinear: out must be contiguous or a 2-D view with unit inner stride");
  }
  at::Tensor w = weight.contiguous();
  at::Tensor ws = weight_scales.contiguous();
  at::Tensor b = has_bias ? bias->contiguous() : at::Tensor();
  std::vector<at::Tensor> bufs;
  for (const at::Tensor &t : post_buffers) bufs.push_back(t.contiguous());
  at::Tensor rowsum;
  bool weights_const;
  if (has_xzp) {
    bool computed_now = false;
    const std::function<at::Tensor()> make = [&]() {
      at::Tensor r = at::empty({N}, w.options().dtype(at::kInt));
      const int rc = zt_int8_weight_rowsum(w.data_ptr<int8_t>(), N, K, r.data_ptr<int32_t>(), stream);
      TORCH_CHECK(rc == ZT_SUCCESS, zt_last_error());
      computed_now = true;
      return r;
    };
    weights_const = seen_weights().lookup(weight, &make, &rowsum) && !computed_now;
  } else {
    weights_const = seen_weights().seen_before(weight);
  }
  weights_const = seen_weights().seen_before(weight_scales) && w.is_same(weight) && ws.is_same(weight_scales) && weights_const;
  const size_t ws_bytes = zt_static_qlinear_workspace_bytes(M, K, x_dtype);
  at::Tensor scratch = at::empty({(int64_t)ws_bytes}, w.options().dtype(at::kByte));

  zt_static_qlinear_args_t a{};
  a.x = x2.data_ptr();
  a.x_dtype = x_dtype;
  a.M = M;
  a.K = K;
  a.N = N;
  a.x_scale = input_scales.data_ptr<float>();
  a.x_zero_point = has_xzp ? input_zero_points.data_ptr<int32_t>() : nullptr;
  a.w = w.data_ptr<int8_t>();
  a.w_scales = ws.data_ptr<float>();
  a.w_scales_numel = ws.numel();
  a.w_rowsum = rowsum.defined() ? rowsum.data_ptr<int32_t>() : nullptr;
  a.bias = b.defined() ? b.data_ptr() : nullptr;
  a.bias_dtype = b.defined() ? to_zt_dtype(b, "bias") : ZT_F32;
  int nb = 0;
  for (int id : post_ops) {
    if (id == ZT_POST_NONE) continue;
    a.post.ids[a.post.n_ops++] = id;
    if (id == ZT_POST_MUL || id == ZT_POST_ADD) {
      a.post.buffers[nb] = bufs[nb].data_ptr();
      ++nb;
    }
  }
  a.post_buffer_dtype = bufs.empty() ? ZT_F32 : to_zt_dtype(bufs[0], "post-op operand");
  a.out_scale = has_oscale ? output_scales->data_ptr<float>() : nullptr;
  a.out_zero_point = has_ozp ? output_zero_points->data_ptr<int32_t>() : nullptr;
  a.y = result.data_ptr();
  a.y_dtype = y_dtype;
  a.ldy = ldy;
  a.workspace = scratch.data_ptr();
  a.workspace_bytes = ws_bytes;
  a.algo = ZT_ALGO_AUTO;
  a.flags = weights_const ? 0 : ZT_FLAG_WEIGHTS_VOLATILE;
  ZT_TORCH_CALL(zt_static_qlinear(&a, stream));
}

c10::ScalarType qlinear_output_dtype(std::optional<c10::ScalarType> output_dtype) {
  const c10::ScalarType t = output_dtype.value_or(at::kFloat);
  TORCH_CHECK(t == at::kFloat || t == at::kBFloat16 || t == at::kByte || t == at::kChar,
              "output_dtype received is not yet supported, only float32/bfloat16/uint8/int8 is supported");
  return t;
}

at::Tensor qlinear_result(const at::Tensor &input, const at::Tensor &weight, c10::ScalarType dtype) {
  TORCH_CHECK(input.dim() >= 1 && weight.dim() == 2, "unsupported dims for input and weight");
  std::vector<int64_t> out_sizes = input.sizes().vec();
  out_sizes.back() = weight.size(0);
  return at::empty(out_sizes, input.options().dtype(dtype));
}

// zentorch_qlinear / _relu / _sigmoid (zentorch_qlinear_unary, QLinear.cpp:420-454)
template <int POST>
at::Tensor qlinear_unary(const at::Tensor &input, const at::Tensor &weight, const at::Tensor &input_scales,
                         const at::Tensor &input_zero_points, const at::Tensor &weight_scales,
                         const at::Tensor &weight_zero_points, std::optional<at::Tensor> bias,
                         std::optional<at::Tensor> output_scales, std::optional<at::Tensor> output_zero_points,
                         std::optional<c10::ScalarType> output_dtype, std::string zentorch_op_name) {
  at::Tensor result = qlinear_result(input, weight, qlinear_output_dtype(output_dtype));
  qlinear_into(result, input, weight, input_scales, input_zero_points, weight_scales, weight_zero_points, bias,
               output_scales, output_zero_points, {POST}, {}, zentorch_op_name);
  return result;
}

// zentorch_qlinear.out / zentorch_qlinear_relu.out (zentorch_qlinear_out_unary, QLinear.cpp:368-418)
template <int POST>
void qlinear_out_unary(at::Tensor &out, const at::Tensor &input, const at::Tensor &weight,
                       const at::Tensor &input_scales, const at::Tensor &input_zero_points,
                       const at::Tensor &weight_scales, const at::Tensor &weight_zero_points,
                       std::optional<at::Tensor> bias, std::optional<at::Tensor> output_scales,
                       std::optional<at::Tensor> output_zero_points, std::optional<c10::ScalarType> output_dtype,
                       std::string zentorch_op_name) {
  TORCH_CHECK(output_dtype.has_value() && *output_dtype == out.scalar_type(),
              "output_dtype received does not match the dtype of the output tensor");
  qlinear_output_dtype(output_dtype);
  qlinear_into(out, input, weight, input_scales, input_zero_points, weight_scales, weight_zero_points, bias,
               output_scales, output_zero_points, {POST}, {}, zentorch_op_name);
}

// zentorch_qlinear_mul_add (zentorch_qlinear_binary_binary<MUL, ADD>, QLinear.cpp:456-531)
at::Tensor qlinear_mul_add(const at::Tensor &input, const at::Tensor &weight, const at::Tensor &input_scales,
                           const at::Tensor &input_zero_points, const at::Tensor &weight_scales,
                           const at::Tensor &weight_zero_points, const at::Tensor &mul_input,
                           const at::Tensor &add_input, std::optional<at::Tensor> bias,
                           std::optional<at::Tensor> output_scales, std::optional<at::Tensor> output_zero_points,
                           std::optional<c10::ScalarType> output_dtype, std::string zentorch_op_name) {
  at::Tensor result = qlinear_result(input, weight, qlinear_output_dtype(output_dtype));
  qlinear_into(result, input, weight, input_scales, input_zero_points, weight_scales, weight_zero_points, bias,
               output_scales, output_zero_points, {ZT_POST_MUL, ZT_POST_ADD}, {mul_input, add_input}, zentorch_op_name);
  return result;
}

// ---- meta kernels (src/cpu/python/zentorch/_meta_registrations.py:552-714, 755-797) --------------------
at::Tensor meta_woq(const at::Tensor &input, const at::Tensor &weight) {
  std::vector<c10::SymInt> sizes = input.sym_sizes().vec();
  sizes.back() = weight.sym_size(1);
  return at::empty_symint(sizes, input.options());
}
at::Tensor meta_woq_unary(const at::Tensor &input, const at::Tensor &weight, const at::Tensor &,
                          const std::optional<at::Tensor> &, const std::optional<at::Tensor> &, std::string) {
  return meta_woq(input, weight);
}
at::Tensor meta_woq_add(const at::Tensor &input, const at::Tensor &weight, const at::Tensor &,
                        const std::optional<at::Tensor> &, const at::Tensor &, const std::optional<at::Tensor> &,
                        std::string) {
  return meta_woq(input, weight);
}
at::Tensor meta_woq_binary_binary(const at::Tensor &input, const at::Tensor &weight, const at::Tensor &,
                                  const std::optional<at::Tensor> &, const at::Tensor &, const at::Tensor &,
                                  const std::optional<at::Tensor> &, std::string) {
  return meta_woq(input, weight);
}
at::Tensor meta_repack_weight(const at::Tensor &w) {
  return at::empty_symint({w.sym_size(0), w.sym_size(1) / 8}, w.options().dtype(at::kInt));
}
at::Tensor meta_repack_from_int4pack(const at::Tensor &w) {
  return at::empty_symint({w.sym_size(0), w.sym_size(1) * 2 / 8}, w.options().dtype(at::kInt));
}
at::Tensor meta_dynamic_qlinear(const at::Tensor &input, const at::Tensor &weight, const at::Tensor &,
                                const std::optional<at::Tensor> &, std::string) {
  std::vector<c10::SymInt> sizes = input.sym_sizes().vec();
  sizes.back() = weight.sym_size(0);
  return at::empty_symint(sizes, input.options());
}
at::Tensor meta_dynamic_qlinear_ext(const at::Tensor &input, const at::Tensor &weight, const at::Tensor &,
                                    const std::optional<at::Tensor> &, const std::optional<at::Tensor> &, std::string,
                                    std::string, std::string) {
  std::vector<c10::SymInt> sizes = input.sym_sizes().vec();
  sizes.back() = weight.sym_size(0);
  return at::empty_symint(sizes, input.options());
}

// static qlinear (src/cpu/python/zentorch/_meta_registrations.py:424-550)
at::Tensor meta_qlinear_shape(const at::Tensor &input, const at::Tensor &weight, std::optional<c10::ScalarType> dtype) {
  std::vector<c10::SymInt> sizes = input.sym_sizes().vec();
  sizes.back() = weight.sym_size(0);
  return at::empty_symint(sizes, input.options().dtype(dtype.value_or(at::kFloat)));
}
at::Tensor meta_qlinear(const at::Tensor &input, const at::Tensor &weight, const at::Tensor &, const at::Tensor &,
                        const at::Tensor &, const at::Tensor &, std::optional<at::Tensor>, std::optional<at::Tensor>,
                        std::optional<at::Tensor>, std::optional<c10::ScalarType> output_dtype, std::string) {
  return meta_qlinear_shape(input, weight, output_dtype);
}
at::Tensor meta_qlinear_mul_add(const at::Tensor &input, const at::Tensor &weight, const at::Tensor &, const at::Tensor &,
                                const at::Tensor &, const at::Tensor &, const at::Tensor &, const at::Tensor &,
                                std::optional<at::Tensor>, std::optional<at::Tensor>, std::optional<at::Tensor>,
                                std::optional<c10::ScalarType> output_dtype, std::string) {
  return meta_qlinear_shape(input, weight, output_dtype);
}
void meta_qlinear_out(at::Tensor &, const at::Tensor &, const at::Tensor &, const at::Tensor &, const at::Tensor &,
                      const at::Tensor &, const at::Tensor &, std::optional<at::Tensor>, std::optional<at::Tensor>,
                      std::optional<at::Tensor>, std::optional<c10::ScalarType>, std::string) {}

bool has_schema(const char *name, const char *overload = "") {
  return c10::Dispatcher::singleton().findSchema({std::string("zentorch::") + name, overload}).has_value();
}

struct Registrar {
  std::vector<std::unique_ptr<torch::Library>> libs;
  Registrar() {
    auto frag = std::make_unique<torch::Library>(torch::Library::FRAGMENT, "zentorch", std::nullopt, __FILE__, __LINE__);
    auto def = [&](const char *name, const char *schema, std::vector<at::Tag> tags = {}) {
      if (!has_schema(name)) frag->def(schema, static_cast<const std::vector<at::Tag> &>(tags));
    };
    def("zentorch_woq_linear",
        "zentorch_woq_linear(Tensor input, Tensor weight, Tensor weight_scales, Tensor? weight_zero_points, "
        "Tensor? bias=None, *, str zentorch_op_name='zentorch::zentorch_woq_linear') -> Tensor");
    def("zentorch_woq_linear_relu",
        "zentorch_woq_linear_relu(Tensor input, Tensor weight, Tensor weight_scales, Tensor? weight_zero_points, "
        "Tensor? bias=None, *, str zentorch_op_name='zentorch::zentorch_woq_linear_relu') -> Tensor");
    def("zentorch_woq_linear_sigmoid",
        "zentorch_woq_linear_sigmoid(Tensor input, Tensor weight, Tensor weight_scales, Tensor? weight_zero_points, "
        "Tensor? bias=None, *, str zentorch_op_name='zentorch::zentorch_woq_linear_sigmoid') -> Tensor");
    def("zentorch_woq_linear_gelu_tanh",
        "zentorch_woq_linear_gelu_tanh(Tensor input, Tensor weight, Tensor weight_scales, Tensor? weight_zero_points, "
        "Tensor? bias=None, *, str zentorch_op_name='zentorch::zentorch_woq_linear_gelu_tanh') -> Tensor");
    def("zentorch_woq_linear_gelu_erf",
        "zentorch_woq_linear_gelu_erf(Tensor input, Tensor weight, Tensor weight_scales, Tensor? weight_zero_points, "
        "Tensor? bias=None, *, str zentorch_op_name='zentorch::zentorch_woq_linear_gelu_erf') -> Tensor");
    def("zentorch_woq_linear_add",
        "zentorch_woq_linear_add(Tensor input, Tensor weight, Tensor weight_scales, Tensor? weight_zero_points, "
        "Tensor add_input, Tensor? bias=None, *, str zentorch_op_name='zentorch::zentorch_woq_linear_add') -> Tensor",
        {at::Tag::needs_contiguous_strides});
    def("zentorch_woq_linear_mul_add",
        "zentorch_woq_linear_mul_add(Tensor input, Tensor weight, Tensor weight_scales, Tensor? weight_zero_points, "
        "Tensor mul_input, Tensor add_input, Tensor? bias=None, *, str zentorch_op_name="
        "'zentorch::zentorch_woq_linear_mul_add') -> Tensor",
        {at::Tag::needs_fixed_stride_order});
    def("zentorch_woq_linear_add_add",
        "zentorch_woq_linear_add_add(Tensor input, Tensor weight, Tensor weight_scales, Tensor? weight_zero_points, "
        "Tensor add_input, Tensor add_input_2, Tensor? bias=None, *, str zentorch_op_name="
        "'zentorch::zentorch_woq_linear_add_add') -> Tensor",
        {at::Tag::needs_fixed_stride_order});
    def("zentorch_woq_repack_weight", "zentorch_woq_repack_weight(Tensor unpacked_weight) -> Tensor");
    def("zentorch_woq_repack_from_int4pack", "zentorch_woq_repack_from_int4pack(Tensor packed_weight) -> Tensor");
    def("zentorch_dynamic_qlinear",
        "zentorch_dynamic_qlinear(Tensor input, Tensor weight, Tensor weight_scales, Tensor? bias=None, *, "
        "str zentorch_op_name='zentorch::zentorch_dynamic_qlinear') -> Tensor");
    def("zentorch_dynamic_qlinear_ext",
        "zentorch_dynamic_qlinear_ext(Tensor input, Tensor weight, Tensor weight_scales, Tensor? bias=None, "
        "Tensor? weight_rowsum=None, *, str act_quant='s8_sym', str post_op='none', "
        "str zentorch_op_name='zentorch::zentorch_dynamic_qlinear_ext') -> Tensor");
    // static-quantisation family, schema strings of src/cpu/cpp/QLinear.cpp:535-575
#define ZT_QLINEAR_ARGS                                                                                           \
  "Tensor input, Tensor weight, Tensor input_scales, Tensor input_zero_points, Tensor weight_scales, "            \
  "Tensor weight_zero_points, "
#define ZT_QLINEAR_TAIL "Tensor? bias, Tensor? output_scales, Tensor? output_zero_points, ScalarType? output_dtype=None, "
    def("zentorch_qlinear", "zentorch_qlinear(" ZT_QLINEAR_ARGS ZT_QLINEAR_TAIL
        "str zentorch_op_name='zentorch::zentorch_qlinear') -> Tensor");
    def("zentorch_qlinear_relu", "zentorch_qlinear_relu(" ZT_QLINEAR_ARGS ZT_QLINEAR_TAIL
        "str zentorch_op_name='zentorch::zentorch_qlinear_relu') -> Tensor");
    def("zentorch_qlinear_sigmoid", "zentorch_qlinear_sigmoid(" ZT_QLINEAR_ARGS ZT_QLINEAR_TAIL
        "str zentorch_op_name='zentorch::zentorch_qlinear_sigmoid') -> Tensor");
    def("zentorch_qlinear_mul_add", "zentorch_qlinear_mul_add(" ZT_QLINEAR_ARGS "Tensor mul_input, Tensor add_input, "
        ZT_QLINEAR_TAIL "str zentorch_op_name='zentorch::zentorch_qlinear_mul_add') -> Tensor");
    if (!has_schema("zentorch_qlinear", "out"))
      frag->def("zentorch_qlinear.out(Tensor(a!) out, " ZT_QLINEAR_ARGS ZT_QLINEAR_TAIL
                "str zentorch_op_name='zentorch::zentorch_qlinear.out') -> ()");
    if (!has_schema("zentorch_qlinear_relu", "out"))
      frag->def("zentorch_qlinear_relu.out(Tensor(a!) out, " ZT_QLINEAR_ARGS ZT_QLINEAR_TAIL
                "str zentorch_op_name='zentorch::zentorch_qlinear_relu.out') -> ()");
#undef ZT_QLINEAR_ARGS
#undef ZT_QLINEAR_TAIL
    libs.push_back(std::move(frag));

    auto cuda = std::make_unique<torch::Library>(torch::Library::IMPL, "zentorch", c10::DispatchKey::CUDA, __FILE__, __LINE__);
    cuda->impl("zentorch_woq_linear", woq_linear_unary<ZT_POST_NONE>);
    cuda->impl("zentorch_woq_linear_relu", woq_linear_unary<ZT_POST_RELU>);
    cuda->impl("zentorch_woq_linear_sigmoid", woq_linear_unary<ZT_POST_SIGMOID>);
    cuda->impl("zentorch_woq_linear_gelu_tanh", woq_linear_unary<ZT_POST_GELU_TANH>);
    cuda->impl("zentorch_woq_linear_gelu_erf", woq_linear_unary<ZT_POST_GELU_ERF>);
    cuda->impl("zentorch_woq_linear_add", woq_linear_add);
    cuda->impl("zentorch_woq_linear_mul_add", woq_linear_binary_binary<ZT_POST_MUL, ZT_POST_ADD>);
    cuda->impl("zentorch_woq_linear_add_add", woq_linear_binary_binary<ZT_POST_ADD, ZT_POST_ADD>);
    cuda->impl("zentorch_woq_repack_weight", woq_repack_weight);
    cuda->impl("zentorch_woq_repack_from_int4pack", woq_repack_from_int4pack);
    cuda->impl("zentorch_dynamic_qlinear", dynamic_qlinear);
    cuda->impl("zentorch_dynamic_qlinear_ext", dynamic_qlinear_ext);
    cuda->impl("zentorch_qlinear", qlinear_unary<ZT_POST_NONE>);
    cuda->impl("zentorch_qlinear_relu", qlinear_unary<ZT_POST_RELU>);
    cuda->impl("zentorch_qlinear_sigmoid", qlinear_unary<ZT_POST_SIGMOID>);
    cuda->impl("zentorch_qlinear_mul_add", qlinear_mul_add);
    cuda->impl("zentorch_qlinear.out", qlinear_out_unary<ZT_POST_NONE>);
    cuda->impl("zentorch_qlinear_relu.out", qlinear_out_unary<ZT_POST_RELU>);
    libs.push_back(std::move(cuda));

    // A real zentorch registers its own Meta kernels from Python; only fill the gap when absent.
    auto meta = std::make_unique<torch::Library>(torch::Library::IMPL, "zentorch", c10::DispatchKey::Meta, __FILE__, __LINE__);
    auto has_meta = [](const char *name, const char *overload = "") {
      auto op = c10::Dispatcher::singleton().findOp({std::string("zentorch::") + name, overload});
      return op.has_value() && op->hasKernelForDispatchKey(c10::DispatchKey::Meta);
    };
#define ZT_META(name, fn) \
  if (!has_meta(name)) meta->impl(name, fn)
    ZT_META("zentorch_woq_linear", meta_woq_unary);
    ZT_META("zentorch_woq_linear_relu", meta_woq_unary);
    ZT_META("zentorch_woq_linear_sigmoid", meta_woq_unary);
    ZT_META("zentorch_woq_linear_gelu_tanh", meta_woq_unary);
    ZT_META("zentorch_woq_linear_gelu_erf", meta_woq_unary);
    ZT_META("zentorch_woq_linear_add", meta_woq_add);
    ZT_META("zentorch_woq_linear_mul_add", meta_woq_binary_binary);
    ZT_META("zentorch_woq_linear_add_add", meta_woq_binary_binary);
    ZT_META("zentorch_woq_repack_weight", meta_repack_weight);
    ZT_META("zentorch_woq_repack_from_int4pack", meta_repack_from_int4pack);
    ZT_META("zentorch_dynamic_qlinear", meta_dynamic_qlinear);
    ZT_META("zentorch_dynamic_qlinear_ext", meta_dynamic_qlinear_ext);
    ZT_META("zentorch_qlinear", meta_qlinear);
    ZT_META("zentorch_qlinear_relu", meta_qlinear);
    ZT_META("zentorch_qlinear_sigmoid", meta_qlinear);
    ZT_META("zentorch_qlinear_mul_add", meta_qlinear_mul_add);
    if (!has_meta("zentorch_qlinear", "out")) meta->impl("zentorch_qlinear.out", meta_qlinear_out);
    if (!has_meta("zentorch_qlinear_relu", "out")) meta->impl("zentorch_qlinear_relu.out", meta_qlinear_out);
#undef ZT_META
    libs.push_back(std::move(meta));
  }
};

static Registrar g_registrar;

}  // namespace

}  // namespace zentorch_b200

// Zeroes the split-K counters of every pooled WOQ workspace; to be called after zt_poll_device_status
// reported an expired device-side wait (the kernel that gave up may have left counters non-zero).
extern "C" ZT_API void zentorch_b200_reset_workspaces() {
  std::lock_guard<std::mutex> lock(zentorch_b200::workspace_mutex());
  for (auto &kv : zentorch_b200::workspace_pool())
    if (kv.second.defined()) kv.second.zero_();
}

// ---- AOTInductor C shims -------------------------------------------------------------------------------
// Same parameter lists as aoti_torch_cpu_zentorch_* (src/cpu/cpp/shim_cpu_zentorch.hpp:150-197);
// inputs are borrowed handles, *ret0 receives a new owning handle (shim_cpu_zentorch.cpp:367-381).
using torch::aot_inductor::new_tensor_handle;
using torch::aot_inductor::pointer_to_optional;
using torch::aot_inductor::tensor_handle_to_tensor_pointer;
using namespace zentorch_b200;

#define ZT_SHIM_UNARY(suffix, POST)                                                                          \
  extern "C" ZT_API AOTITorchError aoti_torch_cuda_zentorch_woq_linear##suffix(                              \
      AtenTensorHandle X, AtenTensorHandle W, AtenTensorHandle weight_scales, AtenTensorHandle *weight_zero_points, \
      AtenTensorHandle *B, const char *zentorch_op_name, AtenTensorHandle *ret0) {                           \
    AOTI_TORCH_CONVERT_EXCEPTION_TO_ERROR_CODE({                                                             \
      auto tmp = woq_linear_unary<POST>(*tensor_handle_to_tensor_pointer(X), *tensor_handle_to_tensor_pointer(W), \
                                        *tensor_handle_to_tensor_pointer(weight_scales),                     \
                                        pointer_to_optional<at::Tensor>(weight_zero_points),                 \
                                        pointer_to_optional<at::Tensor>(B), zentorch_op_name);               \
      *ret0 = new_tensor_handle(std::move(tmp));                                                             \
    });                                                                                                      \
  }

ZT_SHIM_UNARY(, ZT_POST_NONE)
ZT_SHIM_UNARY(_relu, ZT_POST_RELU)
ZT_SHIM_UNARY(_sigmoid, ZT_POST_SIGMOID)
ZT_SHIM_UNARY(_gelu_tanh, ZT_POST_GELU_TANH)
ZT_SHIM_UNARY(_gelu_erf, ZT_POST_GELU_ERF)

extern "C" ZT_API AOTITorchError aoti_torch_cuda_zentorch_woq_linear_add(
    AtenTensorHandle X, AtenTensorHandle W, AtenTensorHandle weight_scales, AtenTensorHandle *weight_zero_points,
    AtenTensorHandle add_input, AtenTensorHandle *B, const char *zentorch_op_name, AtenTensorHandle *ret0) {
  AOTI_TORCH_CONVERT_EXCEPTION_TO_ERROR_CODE({
    auto tmp = woq_linear_add(*tensor_handle_to_tensor_pointer(X), *tensor_handle_to_tensor_pointer(W),
                              *tensor_handle_to_tensor_pointer(weight_scales),
                              pointer_to_optional<at::Tensor>(weight_zero_points),
                              *tensor_handle_to_tensor_pointer(add_input), pointer_to_optional<at::Tensor>(B),
                              zentorch_op_name);
    *ret0 = new_tensor_handle(std::move(tmp));
  });
}

extern "C" ZT_API AOTITorchError aoti_torch_cuda_zentorch_woq_linear_mul_add(
    AtenTensorHandle X, AtenTensorHandle W, AtenTensorHandle weight_scales, AtenTensorHandle *weight_zero_points,
    AtenTensorHandle mul_input, AtenTensorHandle add_input, AtenTensorHandle *B, const char *zentorch_op_name,
    AtenTensorHandle *ret0) {
  AOTI_TORCH_CONVERT_EXCEPTION_TO_ERROR_CODE({
    auto tmp = woq_linear_binary_binary<ZT_POST_MUL, ZT_POST_ADD>(
        *tensor_handle_to_tensor_pointer(X), *tensor_handle_to_tensor_pointer(W),
        *tensor_handle_to_tensor_pointer(weight_scales), pointer_to_optional<at::Tensor>(weight_zero_points),
        *tensor_handle_to_tensor_pointer(mul_input), *tensor_handle_to_tensor_pointer(add_input),
        pointer_to_optional<at::Tensor>(B), zentorch_op_name);
    *ret0 = new_tensor_handle(std::move(tmp));
  });
}

extern "C" ZT_API AOTITorchError aoti_torch_cuda_zentorch_woq_linear_add_add(
    AtenTensorHandle X, AtenTensorHandle W, AtenTensorHandle weight_scales, AtenTensorHandle *weight_zero_points,
    AtenTensorHandle add_input, AtenTensorHandle add_input_2, AtenTensorHandle *B, const char *zentorch_op_name,
    AtenTensorHandle *ret0) {
  AOTI_TORCH_CONVERT_EXCEPTION_TO_ERROR_CODE({
    auto tmp = woq_linear_binary_binary<ZT_POST_ADD, ZT_POST_ADD>(
        *tensor_handle_to_tensor_pointer(X), *tensor_handle_to_tensor_pointer(W),
        *tensor_handle_to_tensor_pointer(weight_scales), pointer_to_optional<at::Tensor>(weight_zero_points),
        *tensor_handle_to_tensor_pointer(add_input), *tensor_handle_to_tensor_pointer(add_input_2),
        pointer_to_optional<at::Tensor>(B), zentorch_op_name);
    *ret0 = new_tensor_handle(std::move(tmp));
  });
}

extern "C" ZT_API AOTITorchError aoti_torch_cuda_zentorch_dynamic_qlinear(AtenTensorHandle X, AtenTensorHandle W,
                                                                         AtenTensorHandle weight_scales,
                                                                         AtenTensorHandle *B,
                                                                         const char *zentorch_op_name,
                                                                         AtenTensorHandle *ret0) {
  AOTI_TORCH_CONVERT_EXCEPTION_TO_ERROR_CODE({
    auto tmp = dynamic_qlinear(*tensor_handle_to_tensor_pointer(X), *tensor_handle_to_tensor_pointer(W),
                               *tensor_handle_to_tensor_pointer(weight_scales), pointer_to_optional<at::Tensor>(B),
                               zentorch_op_name);
    *ret0 = new_tensor_handle(std::move(tmp));
  });
}

// Static-quantisation family (src/cpu/cpp/shim_cpu_zentorch.hpp:28-75, shim_cpu_zentorch.cpp:72-230).
#define ZT_QL_ARGS                                                                                       \
  AtenTensorHandle X, AtenTensorHandle W, AtenTensorHandle X_scales, AtenTensorHandle X_zero_points,     \
      AtenTensorHandle W_scales, AtenTensorHandle W_zero_points
#define ZT_QL_TAIL                                                                                       \
  AtenTensorHandle *B, AtenTensorHandle *output_scales, AtenTensorHandle *output_zero_points,            \
      const int32_t *output_dtype, const char *zentorch_op_name
#define ZT_QL_PASS                                                                                       \
  *tensor_handle_to_tensor_pointer(X), *tensor_handle_to_tensor_pointer(W),                              \
      *tensor_handle_to_tensor_pointer(X_scales), *tensor_handle_to_tensor_pointer(X_zero_points),       \
      *tensor_handle_to_tensor_pointer(W_scales), *tensor_handle_to_tensor_pointer(W_zero_points)
#define ZT_QL_PASS_TAIL                                                                                  \
  pointer_to_optional<at::Tensor>(B), pointer_to_optional<at::Tensor>(output_scales),                    \
      pointer_to_optional<at::Tensor>(output_zero_points), pointer_to_optional<c10::ScalarType>(output_dtype), \
      zentorch_op_name

#define ZT_SHIM_QLINEAR(suffix, POST)                                                                    \
  extern "C" ZT_API AOTITorchError aoti_torch_cuda_zentorch_qlinear##suffix(ZT_QL_ARGS, ZT_QL_TAIL,      \
                                                                            AtenTensorHandle *ret0) {    \
    AOTI_TORCH_CONVERT_EXCEPTION_TO_ERROR_CODE({                                                         \
      auto tmp = qlinear_unary<POST>(ZT_QL_PASS, ZT_QL_PASS_TAIL);                                       \
      *ret0 = new_tensor_handle(std::move(tmp));                                                         \
    });                                                                                                  \
  }
ZT_SHIM_QLINEAR(, ZT_POST_NONE)
ZT_SHIM_QLINEAR(_relu, ZT_POST_RELU)
ZT_SHIM_QLINEAR(_sigmoid, ZT_POST_SIGMOID)

extern "C" ZT_API AOTITorchError aoti_torch_cuda_zentorch_qlinear_mul_add(ZT_QL_ARGS, AtenTensorHandle mul_input,
                                                                         AtenTensorHandle add_input, ZT_QL_TAIL,
                                                                         AtenTensorHandle *ret0) {
  AOTI_TORCH_CONVERT_EXCEPTION_TO_ERROR_CODE({
    auto tmp = qlinear_mul_add(ZT_QL_PASS, *tensor_handle_to_tensor_pointer(mul_input),
                               *tensor_handle_to_tensor_pointer(add_input), ZT_QL_PASS_TAIL);
    *ret0 = new_tensor_handle(std::move(tmp));
  });
}

extern "C" ZT_API AOTITorchError aoti_torch_cuda_zentorch_qlinear_out(AtenTensorHandle out, ZT_QL_ARGS, ZT_QL_TAIL) {
  AOTI_TORCH_CONVERT_EXCEPTION_TO_ERROR_CODE(
      { qlinear_out_unary<ZT_POST_NONE>(*tensor_handle_to_tensor_pointer(out), ZT_QL_PASS, ZT_QL_PASS_TAIL); });
}

extern "C" ZT_API AOTITorchError aoti_torch_cuda_zentorch_qlinear_relu_out(AtenTensorHandle out, ZT_QL_ARGS, ZT_QL_TAIL) {
  AOTI_TORCH_CONVERT_EXCEPTION_TO_ERROR_CODE(
      { qlinear_out_unary<ZT_POST_RELU>(*tensor_handle_to_tensor_pointer(out), ZT_QL_PASS, ZT_QL_PASS_TAIL); });
}
