/* AOTInductor C shims of the zentorch quantized-linear operators for CUDA tensors.
 *
 * Inductor's cpp_wrapper names the shim of an extern kernel after the device of its first input
 * (aoti_torch_<device>_<op>); the reference ships the CPU set in
 * src/cpu/cpp/shim_cpu_zentorch.hpp:150-197.  These are the same parameter lists for "cuda",
 * exported by libzentorch_b200_torch.so.  Inputs are borrowed handles; *ret0 receives a new owning
 * handle that the caller frees (src/cpu/cpp/shim_cpu_zentorch.cpp:367-381).  Optional tensors are
 * passed as pointer-to-handle, NULL when absent.
 */
#pragma once

#include <torch/csrc/inductor/aoti_torch/c/shim.h>

#ifdef __cplusplus
extern "C" {
#endif

AOTI_TORCH_EXPORT AOTITorchError aoti_torch_cuda_zentorch_woq_linear(
    AtenTensorHandle X, AtenTensorHandle W, AtenTensorHandle weight_scales, AtenTensorHandle *weight_zero_points,
    AtenTensorHandle *B, const char *zentorch_op_name, AtenTensorHandle *ret0);
AOTI_TORCH_EXPORT AOTITorchError aoti_torch_cuda_zentorch_woq_linear_relu(
    AtenTensorHandle X, AtenTensorHandle W, AtenTensorHandle weight_scales, AtenTensorHandle *weight_zero_points,
    AtenTensorHandle *B, const char *zentorch_op_name, AtenTensorHandle *ret0);
AOTI_TORCH_EXPORT AOTITorchError aoti_torch_cuda_zentorch_woq_linear_sigmoid(
    AtenTensorHandle X, AtenTensorHandle W, AtenTensorHandle weight_scales, AtenTensorHandle *weight_zero_points,
    AtenTensorHandle *B, const char *zentorch_op_name, AtenTensorHandle *ret0);
AOTI_TORCH_EXPORT AOTITorchError aoti_torch_cuda_zentorch_woq_linear_gelu_tanh(
    AtenTensorHandle X, AtenTensorHandle W, AtenTensorHandle weight_scales, AtenTensorHandle *weight_zero_points,
    AtenTensorHandle *B, const char *zentorch_op_name, AtenTensorHandle *ret0);
AOTI_TORCH_EXPORT AOTITorchError aoti_torch_cuda_zentorch_woq_linear_gelu_erf(
    AtenTensorHandle X, AtenTensorHandle W, AtenTensorHandle weight_scales, AtenTensorHandle *weight_zero_points,
    AtenTensorHandle *B, const char *zentorch_op_name, AtenTensorHandle *ret0);
AOTI_TORCH_EXPORT AOTITorchError aoti_torch_cuda_zentorch_woq_linear_add(
    AtenTensorHandle X, AtenTensorHandle W, AtenTensorHandle weight_scales, AtenTensorHandle *weight_zero_points,
    AtenTensorHandle add_input, AtenTensorHandle *B, const char *zentorch_op_name, AtenTensorHandle *ret0);
AOTI_TORCH_EXPORT AOTITorchError aoti_torch_cuda_zentorch_woq_linear_mul_add(
    AtenTensorHandle X, AtenTensorHandle W, AtenTensorHandle weight_scales, AtenTensorHandle *weight_zero_points,
    AtenTensorHandle mul_input, AtenTensorHandle add_input, AtenTensorHandle *B, const char *zentorch_op_name,
    AtenTensorHandle *ret0);
AOTI_TORCH_EXPORT AOTITorchError aoti_torch_cuda_zentorch_woq_linear_add_add(
    AtenTensorHandle X, AtenTensorHandle W, AtenTensorHandle weight_scales, AtenTensorHandle *weight_zero_points,
    AtenTensorHandle add_input, AtenTensorHandle add_input_2, AtenTensorHandle *B, const char *zentorch_op_name,
    AtenTensorHandle *ret0);
AOTI_TORCH_EXPORT AOTITorchError aoti_torch_cuda_zentorch_dynamic_qlinear(
    AtenTensorHandle X, AtenTensorHandle W, AtenTensorHandle weight_scales, AtenTensorHandle *B,
    const char *zentorch_op_name, AtenTensorHandle *ret0);

/* Static-quantisation qlinear family (src/cpu/cpp/shim_cpu_zentorch.hpp:28-75).  X_zero_points and
 * W_zero_points are handles of possibly undefined tensors, output_dtype points at a c10::ScalarType value or
 * is NULL; the .out forms write into `out` and return nothing. */
#define ZT_QLINEAR_SHIM_ARGS                                                                                        \
  AtenTensorHandle X, AtenTensorHandle W, AtenTensorHandle X_scales, AtenTensorHandle X_zero_points,                \
      AtenTensorHandle W_scales, AtenTensorHandle W_zero_points
#define ZT_QLINEAR_SHIM_TAIL                                                                                        \
  AtenTensorHandle *B, AtenTensorHandle *output_scales, AtenTensorHandle *output_zero_points,                       \
      const int32_t *output_dtype, const char *zentorch_op_name
AOTI_TORCH_EXPORT AOTITorchError aoti_torch_cuda_zentorch_qlinear(ZT_QLINEAR_SHIM_ARGS, ZT_QLINEAR_SHIM_TAIL,
                                                                  AtenTensorHandle *ret0);
AOTI_TORCH_EXPORT AOTITorchError aoti_torch_cuda_zentorch_qlinear_relu(ZT_QLINEAR_SHIM_ARGS, ZT_QLINEAR_SHIM_TAIL,
                                                                       AtenTensorHandle *ret0);
AOTI_TORCH_EXPORT AOTITorchError aoti_torch_cuda_zentorch_qlinear_sigmoid(ZT_QLINEAR_SHIM_ARGS, ZT_QLINEAR_SHIM_TAIL,
                                                                          AtenTensorHandle *ret0);
AOTI_TORCH_EXPORT AOTITorchError aoti_torch_cuda_zentorch_qlinear_mul_add(ZT_QLINEAR_SHIM_ARGS,
                                                                          AtenTensorHandle mul_input,
                                                                          AtenTensorHandle add_input,
                                                                          ZT_QLINEAR_SHIM_TAIL, AtenTensorHandle *ret0);
AOTI_TORCH_EXPORT AOTITorchError aoti_torch_cuda_zentorch_qlinear_out(AtenTensorHandle out, ZT_QLINEAR_SHIM_ARGS,
                                                                      ZT_QLINEAR_SHIM_TAIL);
AOTI_TORCH_EXPORT AOTITorchError aoti_torch_cuda_zentorch_qlinear_relu_out(AtenTensorHandle out, ZT_QLINEAR_SHIM_ARGS,
                                                                           ZT_QLINEAR_SHIM_TAIL);
#undef ZT_QLINEAR_SHIM_ARGS
#undef ZT_QLINEAR_SHIM_TAIL

#ifdef __cplusplus
}
#endif
