"""Host-side checks that need no GPU: the C-ABI library loads, exports every symbol the header
declares, validates arguments before touching the device, and the torch boundary registers the
reference's schemas with meta kernels."""
import ctypes as C
import re
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent


def _declared_symbols():
    text = (ROOT / "include" / "zentorch_b200.h").read_text()
    return sorted(set(re.findall(r"ZT_API[^;(]*?\b(zt_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol(zt):
    from zentorch_b200 import _capi
    lib = _capi.lib()
    declared = _declared_symbols()
    assert len(declared) >= 12
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in include/zentorch_b200.h but not exported"
    assert sorted(_capi.EXPORTED_SYMBOLS) == declared


def test_aoti_shims_exported(zt):
    lib = C.CDLL(str(ROOT / "zendnn-pytorch-plugin_b200" / "lib" / "libzentorch_b200_torch.so"))
    for suffix in ("", "_relu", "_sigmoid", "_gelu_tanh", "_gelu_erf", "_add", "_mul_add", "_add_add"):
        assert hasattr(lib, f"aoti_torch_cuda_zentorch_woq_linear{suffix}")
    assert hasattr(lib, "aoti_torch_cuda_zentorch_dynamic_qlinear")
    text = (ROOT / "include" / "shim_cuda_zentorch.h").read_text()
    for name in re.findall(r"\b(aoti_torch_cuda_zentorch_\w+)\s*\(", text):
        assert hasattr(lib, name), name


def test_aoti_shim_returns_an_error_code_for_host_tensors(zt):
    """The shims never let an exception cross the C boundary: CPU tensors (no CUDA kernel would accept
    them) come back as a non-zero AOTITorchError and *ret0 stays untouched."""
    lib = C.CDLL(str(ROOT / "zendnn-pytorch-plugin_b200" / "lib" / "libzentorch_b200_torch.so"))
    from _util import aoti_handle, aoti_release
    x = torch.zeros(2, 64, dtype=torch.bfloat16)
    w = torch.zeros(32, 8, dtype=torch.int32).t()
    sc = torch.ones(1, 32)
    handles = [aoti_handle(t) for t in (x, w, sc)]
    ret = C.c_void_p(None)
    fn = lib.aoti_torch_cuda_zentorch_woq_linear
    fn.restype = C.c_int32
    rc = fn(*(C.c_void_p(addr) for _, addr in handles), None, None, b"zentorch::zentorch_woq_linear", C.byref(ret))
    assert rc != 0 and ret.value is None
    for cap, _ in handles:
        aoti_release(cap)


def test_argument_validation_precedes_device_work(zt):
    from zentorch_b200 import _capi
    lib = _capi.lib()
    assert lib.zt_version().startswith(b"zentorch_b200")
    one = C.c_void_p(16)  # never dereferenced: validation fails first
    assert lib.zt_woq_repack_weight(one, 4, 12, one, None) == 1
    assert b"K must be divisible by 8" in lib.zt_last_error()
    assert lib.zt_woq_repack_weight(one, 4, 4, one, None) == 1
    assert b"K must be at least 8" in lib.zt_last_error()
    assert lib.zt_woq_repack_from_int4pack(one, 32, 16, one, None) == 1
    assert b"multiple of 64" in lib.zt_last_error()
    a = _capi.WoqLinearArgs()
    a.M, a.K, a.N = 2, 20, 8
    assert lib.zt_woq_linear(C.byref(a), None) == 1 and b"divisible by 8" in lib.zt_last_error()
    a.K = 64
    assert lib.zt_woq_linear(C.byref(a), None) == 1 and b"null tensor pointer" in lib.zt_last_error()
    d = _capi.DynamicQLinearArgs()
    d.M, d.K, d.N, d.x_dtype = 2, 8, 4, 7
    assert lib.zt_dynamic_qlinear(C.byref(d), None) == 1
    assert b"input must be bfloat16 or float32" in lib.zt_last_error()
    assert lib.zt_woq_linear_workspace_bytes(1, 4096, 4096) >= _capi.ZT_WOQ_COUNTER_BYTES
    assert lib.zt_dynamic_qlinear_workspace_bytes(512, 4096) >= 512 * 4096 + 2 * 512 * 4
    # decode batches on a layer with few 128-column tiles are split over K: room for the fp32 partial sums
    # (32 tiles on a 148-SM part -> 4 slices), none when the tiles already cover the SMs or M is large
    base = lib.zt_woq_linear_workspace_bytes(1, 4096, 4096)
    assert lib.zt_woq_linear_workspace_bytes(64, 4096, 4096) >= _capi.ZT_WOQ_COUNTER_BYTES + 2 * 64 * 4096 * 4
    assert lib.zt_woq_linear_workspace_bytes(2048, 4096, 4096) <= max(base, lib.zt_woq_linear_workspace_bytes(64, 4096, 4096))


def test_schemas_match_the_reference(zt):
    ops = torch.ops.zentorch
    s = str(ops.zentorch_woq_linear.default._schema)
    assert "Tensor input, Tensor weight, Tensor weight_scales, Tensor? weight_zero_points, Tensor? bias=None" in s
    assert 'zentorch_op_name="zentorch::zentorch_woq_linear"' in s
    for name in ("relu", "sigmoid", "gelu_tanh", "gelu_erf"):
        assert getattr(ops, f"zentorch_woq_linear_{name}") is not None
    assert "Tensor add_input, Tensor? bias=None" in str(ops.zentorch_woq_linear_add.default._schema)
    assert "Tensor mul_input, Tensor add_input, Tensor? bias=None" in str(ops.zentorch_woq_linear_mul_add.default._schema)
    assert "Tensor add_input, Tensor add_input_2, Tensor? bias=None" in str(ops.zentorch_woq_linear_add_add.default._schema)
    assert torch.Tag.needs_contiguous_strides in ops.zentorch_woq_linear_add.default.tags
    assert torch.Tag.needs_fixed_stride_order in ops.zentorch_woq_linear_mul_add.default.tags
    assert torch.Tag.needs_fixed_stride_order in ops.zentorch_woq_linear_add_add.default.tags
    d = str(ops.zentorch_dynamic_qlinear.default._schema)
    assert "Tensor input, Tensor weight, Tensor weight_scales, Tensor? bias=None" in d


def test_meta_kernels(zt):
    ops = torch.ops.zentorch
    x = torch.empty(2, 3, 64, dtype=torch.bfloat16, device="meta")
    w = torch.empty(8, 48, dtype=torch.int32, device="meta")
    s = torch.empty(1, 48, device="meta")
    other = torch.empty(2, 3, 48, dtype=torch.bfloat16, device="meta")
    assert ops.zentorch_woq_linear(x, w, s, None, None).shape == (2, 3, 48)
    assert ops.zentorch_woq_linear_gelu_erf(x, w, s, None, None).dtype == torch.bfloat16
    assert ops.zentorch_woq_linear_add(x, w, s, None, other).shape == (2, 3, 48)
    assert ops.zentorch_woq_linear_mul_add(x, w, s, None, other, other).shape == (2, 3, 48)
    assert ops.zentorch_woq_linear_add_add(x, w, s, None, other, other).shape == (2, 3, 48)
    assert ops.zentorch_woq_repack_weight(torch.empty(48, 64, dtype=torch.int8, device="meta")).shape == (48, 8)
    assert ops.zentorch_woq_repack_from_int4pack(torch.empty(64, 32, dtype=torch.uint8, device="meta")).shape == (64, 8)
    xi = torch.empty(5, 16, device="meta")
    wi = torch.empty(10, 16, dtype=torch.int8, device="meta")
    out = ops.zentorch_dynamic_qlinear(xi, wi, torch.empty(10, device="meta"), None)
    assert out.shape == (5, 10) and out.dtype == torch.float32


def test_no_cpu_fallback(zt):
    x = torch.zeros(4, 64, dtype=torch.bfloat16)
    w = torch.zeros(32, 8, dtype=torch.int32).t()
    with pytest.raises((RuntimeError, NotImplementedError)):
        torch.ops.zentorch.zentorch_woq_linear(x, w, torch.ones(1, 32), None, None)
    with pytest.raises((RuntimeError, NotImplementedError)):
        torch.ops.zentorch.zentorch_dynamic_qlinear(torch.zeros(2, 8), torch.zeros(4, 8, dtype=torch.int8), torch.ones(4), None)


def test_static_qlinear_validation_schemas_and_meta(zt):
    """The static-quantisation family on a box without a GPU: argument checks of the C entry point fail before any
    device work with the reference's messages (src/cpu/cpp/QLinear.cpp:66-366), the schemas are the reference's
    (QLinear.cpp:525-573), and the Meta kernels give the output shape and dtype rule."""
    from zentorch_b200 import _capi
    lib = _capi.lib()
    one = C.c_void_p(16)  # never dereferenced: validation fails first
    a = _capi.StaticQLinearArgs()
    a.M, a.K, a.N, a.w_scales_numel, a.ldy = 2, 8, 4, 4, 4
    a.x_dtype, a.y_dtype, a.post_buffer_dtype = 9, _capi.ZT_F32, _capi.ZT_F32
    assert lib.zt_static_qlinear(C.byref(a), None) == 1
    assert b"unsupported dtype for input tensor" in lib.zt_last_error()
    a.x_dtype, a.y_dtype = _capi.ZT_F32, _capi.ZT_U8
    assert lib.zt_static_qlinear(C.byref(a), None) == 1
    assert b"only float32/bfloat16 is supported when output_scales are not defined" in lib.zt_last_error()
    a.y_dtype, a.w_scales_numel = _capi.ZT_F32, 3
    assert lib.zt_static_qlinear(C.byref(a), None) == 1
    assert b"unsupported number of elements for weight_scales" in lib.zt_last_error()
    a.w_scales_numel, a.x_dtype = 4, _capi.ZT_U8
    assert lib.zt_static_qlinear(C.byref(a), None) == 1 and b"needs input_zero_points" in lib.zt_last_error()
    a.x_dtype = _capi.ZT_F32
    assert lib.zt_static_qlinear(C.byref(a), None) == 1 and b"null tensor pointer" in lib.zt_last_error()
    a.x = a.x_scale = a.w = a.w_scales = a.y = one
    a.x_zero_point = one
    assert lib.zt_static_qlinear(C.byref(a), None) == 1 and b"need w_rowsum" in lib.zt_last_error()
    a.x_zero_point, a.ldy = None, 3
    assert lib.zt_static_qlinear(C.byref(a), None) == 1 and b"smaller than N" in lib.zt_last_error()
    a.M = 0          # an empty batch succeeds without touching anything
    assert lib.zt_static_qlinear(C.byref(a), None) == 0
    assert lib.zt_static_quantize(None, _capi.ZT_F32, 0, None, None, None, None) == 0
    assert lib.zt_static_quantize(None, _capi.ZT_F32, 4, None, None, None, None) == 1
    assert lib.zt_static_qlinear_workspace_bytes(512, 4096, _capi.ZT_BF16) >= 512 * 4096
    assert lib.zt_static_qlinear_workspace_bytes(512, 4096, _capi.ZT_U8) <= 256    # nothing to quantise

    ops = torch.ops.zentorch
    head = ("Tensor input, Tensor weight, Tensor input_scales, Tensor input_zero_points, Tensor weight_scales, "
            "Tensor weight_zero_points, ")
    tail = "Tensor? bias, Tensor? output_scales, Tensor? output_zero_points, ScalarType? output_dtype=None"
    for name in ("zentorch_qlinear", "zentorch_qlinear_relu", "zentorch_qlinear_sigmoid"):
        s = str(getattr(ops, name).default._schema)
        assert head + tail in s and f'zentorch_op_name="zentorch::{name}"' in s
    assert head + "Tensor mul_input, Tensor add_input, " + tail in str(ops.zentorch_qlinear_mul_add.default._schema)
    for name in ("zentorch_qlinear", "zentorch_qlinear_relu"):
        s = str(getattr(ops, name).out._schema)
        assert "Tensor(a!) out, " + head + tail in s and s.endswith("-> ()")

    x = torch.empty(3, 5, 64, device="meta")
    w = torch.empty(48, 64, dtype=torch.int8, device="meta")
    sc = torch.empty(1, device="meta")
    zp = torch.empty(1, dtype=torch.int32, device="meta")
    ws = torch.empty(48, device="meta")
    wz = torch.empty(48, dtype=torch.int32, device="meta")
    y = ops.zentorch_qlinear(x, w, sc, zp, ws, wz, None, None, None)
    assert y.shape == (3, 5, 48) and y.dtype == torch.float32
    y = ops.zentorch_qlinear(x, w, sc, zp, ws, wz, None, sc, zp, output_dtype=torch.uint8)
    assert y.shape == (3, 5, 48) and y.dtype == torch.uint8
    y = ops.zentorch_qlinear_relu(x.bfloat16(), w, sc, zp, ws, wz, None, None, None, output_dtype=torch.bfloat16)
    assert y.dtype == torch.bfloat16
    other = torch.empty(3, 5, 48, device="meta")
    assert ops.zentorch_qlinear_mul_add(x, w, sc, zp, ws, wz, other, other, None, None, None).shape == (3, 5, 48)

    # and no CPU kernel behind it
    with pytest.raises((RuntimeError, NotImplementedError)):
        ops.zentorch_qlinear(torch.zeros(2, 8), torch.zeros(4, 8, dtype=torch.int8), torch.ones(1),
                             torch.zeros(1, dtype=torch.int32), torch.ones(4), torch.zeros(4, dtype=torch.int32),
                             None, None, None)
