"""ctypes binding of the C ABI declared in ``include/zentorch_b200.h``.

This is the binding a maintainer of the reference would write to call the library from Python
without going through ``torch.ops``; the parity tests use it so that what they exercise is the
shipped C entry points themselves.  Tensors are passed as raw device pointers.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent.parent / "lib" / "libzentorch_b200.so"

ZT_SUCCESS = 0
ZT_BF16, ZT_F32, ZT_U8, ZT_S8 = 0, 1, 2, 3
ZT_MAX_POST_OPS = 4
ZT_WOQ_COUNTER_BYTES = 16384
ZT_ALGO_AUTO, ZT_ALGO_GENERIC, ZT_ALGO_SKINNY, ZT_ALGO_TCGEN05 = 0, 1, 2, 3
ZT_ALGO_SINGLE_ISSUER = 1 << 24
ZT_ACT_S8_SYM, ZT_ACT_U8_ASYM = 0, 1
ZT_FLAG_WEIGHTS_VOLATILE = 1
ZT_STATIC_SCRATCH_Q_BYTES, ZT_STATIC_SCRATCH_MAX_ROWS = 8 << 20, 16384
(ZT_POST_NONE, ZT_POST_RELU, ZT_POST_GELU_TANH, ZT_POST_GELU_ERF, ZT_POST_SILU, ZT_POST_SIGMOID,
 ZT_POST_TANH, ZT_POST_MUL, ZT_POST_ADD) = range(9)

# Every symbol include/zentorch_b200.h declares; the CPU test-suite checks the library exports all.
EXPORTED_SYMBOLS = (
    "zt_last_error", "zt_version", "zt_device_supported", "zt_poll_device_status", "zt_selftest_expire_wait", "zt_debug_set_timeline",
    "zt_woq_linear_workspace_bytes", "zt_woq_linear", "zt_woq_repack_weight", "zt_woq_repack_from_int4pack",
    "zt_dynamic_qlinear_workspace_bytes", "zt_dynamic_qlinear", "zt_dynamic_quantize", "zt_int8_gemm_s32",
    "zt_int8_weight_rowsum", "zt_qlinear_prequantized", "zt_dynamic_qlinear_static",
    "zt_static_qlinear_workspace_bytes", "zt_static_qlinear", "zt_static_quantize",
    "zt_moe_woq_workspace_bytes", "zt_moe_woq", "zt_allreduce_symmetric_bytes", "zt_allreduce_bf16",
)


class PostOps(C.Structure):
    _fields_ = [("n_ops", C.c_int32), ("ids", C.c_int32 * ZT_MAX_POST_OPS), ("buffers", C.c_void_p * ZT_MAX_POST_OPS)]


class WoqLinearArgs(C.Structure):
    _fields_ = [
        ("x", C.c_void_p), ("M", C.c_int64), ("K", C.c_int64), ("N", C.c_int64),
        ("wq", C.c_void_p), ("scales", C.c_void_p), ("zeros", C.c_void_p), ("scale_dtype", C.c_int32),
        ("n_groups", C.c_int64), ("bias", C.c_void_p), ("bias_dtype", C.c_int32), ("post", PostOps),
        ("y", C.c_void_p), ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("algo", C.c_int32),
        ("flags", C.c_int32),
    ]


class DynamicQLinearArgs(C.Structure):
    _fields_ = [
        ("x", C.c_void_p), ("x_dtype", C.c_int32), ("M", C.c_int64), ("K", C.c_int64), ("N", C.c_int64),
        ("w", C.c_void_p), ("w_scales", C.c_void_p), ("w_scale_dtype", C.c_int32), ("bias", C.c_void_p),
        ("bias_dtype", C.c_int32), ("act_quant", C.c_int32), ("w_rowsum", C.c_void_p), ("post", PostOps),
        ("y", C.c_void_p), ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("algo", C.c_int32),
        ("flags", C.c_int32),
    ]


class StaticQLinearArgs(C.Structure):
    _fields_ = [
        ("x", C.c_void_p), ("x_dtype", C.c_int32), ("M", C.c_int64), ("K", C.c_int64), ("N", C.c_int64),
        ("x_scale", C.c_void_p), ("x_zero_point", C.c_void_p), ("w", C.c_void_p), ("w_scales", C.c_void_p),
        ("w_scales_numel", C.c_int64), ("w_rowsum", C.c_void_p), ("bias", C.c_void_p), ("bias_dtype", C.c_int32),
        ("post", PostOps), ("post_buffer_dtype", C.c_int32), ("out_scale", C.c_void_p),
        ("out_zero_point", C.c_void_p), ("y", C.c_void_p), ("y_dtype", C.c_int32), ("ldy", C.c_int64),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("algo", C.c_int32), ("flags", C.c_int32),
    ]


class MoeWoqArgs(C.Structure):
    _fields_ = [
        ("x", C.c_void_p), ("T", C.c_int64), ("H", C.c_int64), ("I", C.c_int64), ("num_experts", C.c_int32),
        ("top_k", C.c_int32), ("topk_ids", C.c_void_p), ("topk_weights", C.c_void_p), ("w13", C.c_void_p),
        ("s13", C.c_void_p), ("w2", C.c_void_p), ("s2", C.c_void_p), ("scale_dtype", C.c_int32),
        ("group_size", C.c_int64), ("y", C.c_void_p), ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
    ]


ZT_AR_MAX_RANKS, ZT_AR_MAX_SLICES = 8, 64


class AllReduceArgs(C.Structure):
    _fields_ = [
        ("in_", C.c_void_p), ("out", C.c_void_p), ("numel", C.c_int64), ("peer_base", C.c_void_p * ZT_AR_MAX_RANKS),
        ("rank", C.c_int32), ("world", C.c_int32), ("max_bytes", C.c_size_t), ("epochs", C.c_void_p),
    ]


class ZtError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(message or f"zentorch_b200 error {code}")
        self.code = code


_lib = None


def lib() -> C.CDLL:
    """Loads libzentorch_b200.so (RTLD_GLOBAL, as the reference loads libzentorch.so:
    src/cpu/python/zentorch/__init__.py:69-78).  Raises when it has not been built: there is no
    fallback implementation."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m zentorch_b200._build` "
            "(there is no CPU or PyTorch fallback for these operators)")
    L = C.CDLL(str(LIB_PATH), mode=C.RTLD_GLOBAL)
    L.zt_last_error.restype = C.c_char_p
    L.zt_version.restype = C.c_char_p
    L.zt_device_supported.restype = C.c_int
    L.zt_poll_device_status.argtypes = [C.POINTER(C.c_int), C.c_int]
    L.zt_selftest_expire_wait.argtypes = [C.c_void_p]
    L.zt_debug_set_timeline.argtypes = [C.c_void_p, C.c_size_t]
    L.zt_woq_linear_workspace_bytes.restype = C.c_size_t
    L.zt_woq_linear_workspace_bytes.argtypes = [C.c_int64, C.c_int64, C.c_int64]
    L.zt_woq_linear.argtypes = [C.POINTER(WoqLinearArgs), C.c_void_p]
    L.zt_woq_repack_weight.argtypes = [C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p]
    L.zt_woq_repack_from_int4pack.argtypes = [C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p]
    L.zt_dynamic_qlinear_workspace_bytes.restype = C.c_size_t
    L.zt_dynamic_qlinear_workspace_bytes.argtypes = [C.c_int64, C.c_int64]
    L.zt_dynamic_qlinear.argtypes = [C.POINTER(DynamicQLinearArgs), C.c_void_p]
    L.zt_dynamic_qlinear_static.argtypes = [C.POINTER(DynamicQLinearArgs), C.c_void_p]
    L.zt_dynamic_quantize.argtypes = [C.c_void_p, C.c_int32, C.c_int64, C.c_int64, C.c_int32, C.c_void_p,
                                      C.c_void_p, C.c_void_p, C.c_void_p]
    L.zt_int8_gemm_s32.argtypes = [C.c_void_p, C.c_int32, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_void_p,
                                   C.c_int32, C.c_void_p]
    L.zt_qlinear_prequantized.argtypes = [C.POINTER(DynamicQLinearArgs), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    L.zt_static_qlinear_workspace_bytes.restype = C.c_size_t
    L.zt_static_qlinear_workspace_bytes.argtypes = [C.c_int64, C.c_int64, C.c_int32]
    L.zt_static_qlinear.argtypes = [C.POINTER(StaticQLinearArgs), C.c_void_p]
    L.zt_static_quantize.argtypes = [C.c_void_p, C.c_int32, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    L.zt_moe_woq_workspace_bytes.restype = C.c_size_t
    L.zt_moe_woq_workspace_bytes.argtypes = [C.c_int64, C.c_int64, C.c_int64, C.c_int32, C.c_int32]
    L.zt_moe_woq.argtypes = [C.POINTER(MoeWoqArgs), C.c_void_p]
    L.zt_int8_weight_rowsum.argtypes = [C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p]
    L.zt_allreduce_symmetric_bytes.restype = C.c_size_t
    L.zt_allreduce_symmetric_bytes.argtypes = [C.c_size_t]
    L.zt_allreduce_bf16.argtypes = [C.POINTER(AllReduceArgs), C.c_void_p]
    _lib = L
    return L


def check(rc: int) -> None:
    if rc != ZT_SUCCESS:
        raise ZtError(rc, lib().zt_last_error().decode())


def poll_device_status(reset: bool = True) -> int:
    """The device status word (0 = no bounded wait expired).  With ``reset`` a non-zero status is cleared
    and the split-K counters at the front of every cached WOQ workspace are zeroed again, as the header
    asks after a timeout (a kernel that gave up may have left them non-zero)."""
    st = C.c_int(0)
    check(lib().zt_poll_device_status(C.byref(st), 1 if reset else 0))
    if reset and st.value != 0:
        for t in _woq_ws.values():
            t[:ZT_WOQ_COUNTER_BYTES].zero_()
        torch_lib = _torch_boundary()
        if torch_lib is not None:
            torch_lib.zentorch_b200_reset_workspaces()
    return st.value


def _torch_boundary():
    """The operator library, when the package has loaded it (it keeps its own workspace pool)."""
    path = LIB_PATH.with_name("libzentorch_b200_torch.so")
    try:
        return C.CDLL(str(path), mode=os.RTLD_NOLOAD | os.RTLD_NOW)
    except OSError:
        return None


# ---- torch-tensor conveniences (raw pointers underneath) ------------------------------------------
def _dtype_code(t) -> int:
    import torch
    if t.dtype == torch.bfloat16:
        return ZT_BF16
    if t.dtype == torch.float32:
        return ZT_F32
    raise TypeError(f"unsupported dtype {t.dtype}")


def _dtype_code8(dtype) -> int:
    """Codes of the four tensor dtypes of the static qlinear."""
    import torch
    return {torch.bfloat16: ZT_BF16, torch.float32: ZT_F32, torch.uint8: ZT_U8, torch.int8: ZT_S8}[dtype]


def _stream_ptr():
    import torch
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _post(post_ops, buffers) -> PostOps:
    p = PostOps()
    p.n_ops = len(post_ops)
    for i, op in enumerate(post_ops):
        p.ids[i] = int(op)
    for i, b in enumerate(buffers):
        p.buffers[i] = b.data_ptr()
    return p


_woq_ws = {}


def woq_workspace(nbytes: int, device):
    """Zero-initialised scratch kept per device (the counters at its front must stay zero)."""
    import torch
    key = (device.index, torch.cuda.current_stream().cuda_stream)
    t = _woq_ws.get(key)
    if t is None or t.numel() < nbytes:
        t = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _woq_ws[key] = t
    return t


def woq_linear(x, wq_rows, scales, zeros=None, bias=None, post_ops=(), buffers=(), algo=ZT_ALGO_AUTO, flags=0):
    """x: [M, K] bf16 CUDA; wq_rows: the contiguous [N, K/8] int32 packed tensor (i.e. the op's
    weight argument transposed back); scales/zeros: [G, N]."""
    import torch
    assert x.is_cuda and x.is_contiguous() and wq_rows.is_contiguous() and scales.is_contiguous()
    m, k = x.shape
    n = wq_rows.shape[0]
    y = torch.empty(m, n, dtype=x.dtype, device=x.device)
    a = WoqLinearArgs()
    a.x, a.M, a.K, a.N = x.data_ptr(), m, k, n
    a.wq, a.scales = wq_rows.data_ptr(), scales.data_ptr()
    a.zeros = zeros.data_ptr() if zeros is not None else None
    a.scale_dtype, a.n_groups = _dtype_code(scales), scales.shape[0]
    a.bias = bias.data_ptr() if bias is not None else None
    a.bias_dtype = _dtype_code(bias) if bias is not None else ZT_BF16
    a.post = _post(post_ops, buffers)
    a.y = y.data_ptr()
    ws = woq_workspace(lib().zt_woq_linear_workspace_bytes(m, n, k), x.device)
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    a.algo = algo
    a.flags = flags
    check(lib().zt_woq_linear(C.byref(a), _stream_ptr()))
    return y


def woq_repack_weight(unpacked):
    import torch
    n, k = unpacked.shape
    out = torch.empty(n, max(k // 8, 0), dtype=torch.int32, device=unpacked.device)
    check(lib().zt_woq_repack_weight(unpacked.data_ptr(), n, k, out.data_ptr(), _stream_ptr()))
    return out


def woq_repack_from_int4pack(packed):
    import torch
    n, k_half = packed.shape
    out = torch.empty(n, k_half // 4, dtype=torch.int32, device=packed.device)
    check(lib().zt_woq_repack_from_int4pack(packed.data_ptr(), n, k_half, out.data_ptr(), _stream_ptr()))
    return out


def dynamic_quantize(x, act_quant=ZT_ACT_S8_SYM):
    import torch
    m, k = x.shape
    q = torch.empty(m, k, dtype=torch.uint8 if act_quant == ZT_ACT_U8_ASYM else torch.int8, device=x.device)
    s = torch.empty(m, dtype=torch.float32, device=x.device)
    zp = torch.zeros(m, dtype=torch.int32, device=x.device)
    check(lib().zt_dynamic_quantize(x.data_ptr(), _dtype_code(x), m, k, act_quant, q.data_ptr(), s.data_ptr(),
                                    zp.data_ptr(), _stream_ptr()))
    return q, s, zp


def int8_gemm_s32(q, w, algo=ZT_ALGO_AUTO):
    import torch
    m, k = q.shape
    n = w.shape[0]
    acc = torch.empty(m, n, dtype=torch.int32, device=q.device)
    check(lib().zt_int8_gemm_s32(q.data_ptr(), 1 if q.dtype == torch.uint8 else 0, w.data_ptr(), m, n, k,
                                 acc.data_ptr(), algo, _stream_ptr()))
    return acc


def int8_weight_rowsum(w):
    import torch
    n, k = w.shape
    out = torch.empty(n, dtype=torch.int32, device=w.device)
    check(lib().zt_int8_weight_rowsum(w.data_ptr(), n, k, out.data_ptr(), _stream_ptr()))
    return out


def dynamic_qlinear_args(x, w, w_scales, bias, act_quant, post_ops, buffers, w_rowsum, y, ws, algo):
    """Fills the argument block of zt_dynamic_qlinear / zt_qlinear_prequantized from torch tensors."""
    m, k = x.shape
    n = w.shape[0]
    a = DynamicQLinearArgs()
    a.x, a.x_dtype, a.M, a.K, a.N = x.data_ptr(), _dtype_code(x), m, k, n
    a.w, a.w_scales, a.w_scale_dtype = w.data_ptr(), w_scales.data_ptr(), _dtype_code(w_scales)
    a.bias = bias.data_ptr() if bias is not None else None
    a.bias_dtype = _dtype_code(bias) if bias is not None else ZT_F32
    a.act_quant = act_quant
    a.w_rowsum = w_rowsum.data_ptr() if w_rowsum is not None else None
    a.post = _post(post_ops, buffers)
    a.y = y.data_ptr()
    a.workspace, a.workspace_bytes = (ws.data_ptr(), ws.numel()) if ws is not None else (None, 0)
    a.algo = algo
    return a


def dynamic_qlinear(x, w, w_scales, bias=None, act_quant=ZT_ACT_S8_SYM, post_ops=(), buffers=(), w_rowsum=None,
                    algo=ZT_ALGO_AUTO, flags=0):
    import torch
    m, k = x.shape
    n = w.shape[0]
    y = torch.empty(m, n, dtype=x.dtype, device=x.device)
    nbytes = lib().zt_dynamic_qlinear_workspace_bytes(m, k)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=x.device)
    if act_quant == ZT_ACT_U8_ASYM and w_rowsum is None:
        w_rowsum = int8_weight_rowsum(w)
    a = DynamicQLinearArgs()
    a.x, a.x_dtype, a.M, a.K, a.N = x.data_ptr(), _dtype_code(x), m, k, n
    a.w, a.w_scales, a.w_scale_dtype = w.data_ptr(), w_scales.data_ptr(), _dtype_code(w_scales)
    a.bias = bias.data_ptr() if bias is not None else None
    a.bias_dtype = _dtype_code(bias) if bias is not None else ZT_F32
    a.act_quant = act_quant
    a.w_rowsum = w_rowsum.data_ptr() if w_rowsum is not None else None
    a.post = _post(post_ops, buffers)
    a.y, a.workspace, a.workspace_bytes, a.algo = y.data_ptr(), ws.data_ptr(), nbytes, algo
    a.flags = flags
    check(lib().zt_dynamic_qlinear(C.byref(a), _stream_ptr()))
    return y


def dynamic_qlinear_static(x, w, w_scales, bias=None, act_quant=ZT_ACT_S8_SYM, post_ops=(), buffers=(), w_rowsum=None,
                           algo=ZT_ALGO_AUTO):
    """zt_dynamic_qlinear_static: same result as dynamic_qlinear, but the library's built-in scratch is
    used, so nothing is allocated for the call besides the output the caller asks for here.  The u8 mode
    needs `w_rowsum` from the caller (it is an input, not scratch)."""
    import torch
    m, _ = x.shape
    n = w.shape[0]
    y = torch.empty(m, n, dtype=x.dtype, device=x.device)
    a = dynamic_qlinear_args(x, w, w_scales, bias, act_quant, post_ops, buffers, w_rowsum, y, None, algo)
    check(lib().zt_dynamic_qlinear_static(C.byref(a), _stream_ptr()))
    return y


def static_quantize(x, scale, zero_point=None):
    """zt_static_quantize: per-tensor quantisation of x (fp32 / bf16) to u8 (zero point given) or s8."""
    import torch
    q = torch.empty(x.shape, dtype=torch.uint8 if zero_point is not None else torch.int8, device=x.device)
    check(lib().zt_static_quantize(x.data_ptr(), _dtype_code(x), x.numel(), scale.data_ptr(),
                                   zero_point.data_ptr() if zero_point is not None else None, q.data_ptr(),
                                   _stream_ptr()))
    return q


def static_qlinear(x, w, x_scale, x_zero_point, w_scales, bias=None, out_scale=None, out_zero_point=None,
                   out_dtype=None, post_ops=(), buffers=(), w_rowsum=None, algo=ZT_ALGO_AUTO, out=None, flags=0):
    """zt_static_qlinear on 2-D operands: x [M, K] fp32 / bf16 / u8 / s8, w [N, K] int8, one-element x_scale
    (fp32) and x_zero_point (int32 or None), w_scales fp32 with 1 or N elements, optional requantisation.
    `out` may be a view with a row stride (its last dimension contiguous)."""
    import torch
    m, k = x.shape
    n = w.shape[0]
    if out_dtype is None:
        out_dtype = torch.float32
    y = out if out is not None else torch.empty(m, n, dtype=out_dtype, device=x.device)
    nbytes = lib().zt_static_qlinear_workspace_bytes(m, k, _dtype_code8(x.dtype))
    ws = torch.empty(nbytes, dtype=torch.uint8, device=x.device)
    if x_zero_point is not None and w_rowsum is None:
        w_rowsum = int8_weight_rowsum(w)
    a = StaticQLinearArgs()
    a.x, a.x_dtype, a.M, a.K, a.N = x.data_ptr(), _dtype_code8(x.dtype), m, k, n
    a.x_scale = x_scale.data_ptr()
    a.x_zero_point = x_zero_point.data_ptr() if x_zero_point is not None else None
    a.w, a.w_scales, a.w_scales_numel = w.data_ptr(), w_scales.data_ptr(), w_scales.numel()
    a.w_rowsum = w_rowsum.data_ptr() if w_rowsum is not None else None
    a.bias = bias.data_ptr() if bias is not None else None
    a.bias_dtype = _dtype_code(bias) if bias is not None else ZT_F32
    a.post = _post(post_ops, buffers)
    a.post_buffer_dtype = _dtype_code(buffers[0]) if buffers else ZT_F32
    a.out_scale = out_scale.data_ptr() if out_scale is not None else None
    a.out_zero_point = out_zero_point.data_ptr() if out_zero_point is not None else None
    a.y, a.y_dtype, a.ldy = y.data_ptr(), _dtype_code8(y.dtype), y.stride(0) if m > 1 or out is not None else n
    a.workspace, a.workspace_bytes, a.algo, a.flags = ws.data_ptr(), nbytes, algo, flags
    check(lib().zt_static_qlinear(C.byref(a), _stream_ptr()))
    return y


def moe_woq(x, topk_weights, topk_ids, w13, s13, w2, s2):
    """x [T,H] bf16; w13 [E, 2I, H/8] int32; s13 [E, H/gs, 2I]; w2 [E, H, I/8]; s2 [E, I/gs, H]."""
    import torch
    t, h = x.shape
    e, two_i, _ = w13.shape
    i = two_i // 2
    k = topk_ids.shape[1]
    y = torch.empty(t, h, dtype=x.dtype, device=x.device)
    nbytes = lib().zt_moe_woq_workspace_bytes(t, h, i, e, k)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=x.device)
    a = MoeWoqArgs()
    a.x, a.T, a.H, a.I, a.num_experts, a.top_k = x.data_ptr(), t, h, i, e, k
    a.topk_ids, a.topk_weights = topk_ids.data_ptr(), topk_weights.data_ptr()
    a.w13, a.s13, a.w2, a.s2 = w13.data_ptr(), s13.data_ptr(), w2.data_ptr(), s2.data_ptr()
    a.scale_dtype, a.group_size = _dtype_code(s13), h // s13.shape[1]
    a.y, a.workspace, a.workspace_bytes = y.data_ptr(), ws.data_ptr(), nbytes
    check(lib().zt_moe_woq(C.byref(a), _stream_ptr()))
    return y
