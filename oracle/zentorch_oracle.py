"""CPU oracle for the zentorch quantized-linear hot path.  TEST INFRASTRUCTURE ONLY.

This module restates, on the CPU with plain torch/numpy arithmetic, what the reference
operators ``zentorch_woq_linear`` (+ fused variants), ``zentorch_woq_repack_weight``,
``zentorch_woq_repack_from_int4pack``, ``zentorch_dynamic_qlinear`` and the ``zentorch_qlinear`` family compute.  Nothing in the
shipped package imports it: only the tests, the smoke entry and the CPU-baseline leg of the
benchmark do, and only as the checker.

The arithmetic of the reference lives in AMD ZenDNN (tag ``zendnn-2026-WW29``), which is not part
of the reference tree; the restatement therefore follows the reference's wrapper code and the
formulas its own tests use as ground truth.  Pin status per function:

* repack / unpack ops ............ pinned (bit-exact against the reference's independent Python
  packer ``test/unittests/op_tests/_pack.py`` and against ``aten._convert_weight_to_int4pack_for_cpu``).
* WOQ symmetric per-channel ...... pinned (formula of ``test/unittests/op_tests/test_woq_linear.py:107-136``).
* WOQ asymmetric per-group ....... pinned against ``aten._weight_int4pack_mm_for_cpu``
  (``test/unittests/op_tests/test_woq_linear_asymmetric.py:100-142``).
* WOQ symmetric per-GROUP ........ parity unpinned (the reference's only tests for it are skipped:
  ``test/unittests/model_tests/test_woq_linear.py:215-251``); formula ``dq = q * s[k // gs, n]``.
* dynamic qlinear (symmetric s8) . pinned (formula of ``test/unittests/op_tests/test_dynamic_qlinear.py:32-36``
  and the integer restatement ``test/unittests/op_tests/test_group_matmul.py:394-409``).
* static-quant qlinear family ..... pinned (the reference's own ``qdq_linear``,
  ``test/unittests/quant_utils.py:13-83``, over input dtype x zero point x weight granularity x output dtype).
* dynamic qlinear u8-asymmetric + fused post-op, int4 MoE, tensor-parallel shards: parity unpinned
  (no reference implementation); composed from the pinned pieces.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence

import torch

# Post-op ids: values of UNARY_POST_OP / BINARY_POST_OP in src/cpu/cpp/Utils.hpp:56-72.
POST_NONE, POST_RELU, POST_GELU_TANH, POST_GELU_ERF, POST_SILU, POST_SIGMOID, POST_TANH = range(7)
POST_MUL, POST_ADD = 7, 8
POST_NAMES = {
    "none": POST_NONE, "relu": POST_RELU, "gelu_tanh": POST_GELU_TANH, "gelu_erf": POST_GELU_ERF,
    "silu": POST_SILU, "sigmoid": POST_SIGMOID, "tanh": POST_TANH, "mul": POST_MUL, "add": POST_ADD,
}


# --------------------------------------------------------------------------------------------
# Weight repack / unpack  (src/cpu/cpp/WOQ_Linear.cpp:294-433)
# --------------------------------------------------------------------------------------------
def woq_repack_weight(unpacked: torch.Tensor) -> torch.Tensor:
    """[N, K] int8 (one 4-bit value per byte) -> [N, K/8] int32, value i of each run of eight
    at bits [4i, 4i+4).  Follows src/cpu/cpp/WOQ_Linear.cpp:294-357 (order map is the identity)."""
    if unpacked.dtype != torch.int8:
        raise RuntimeError(f"unpacked_weight must have dtype int8, got {unpacked.dtype}")
    if unpacked.dim() != 2:
        raise RuntimeError(f"unpacked_weight must be 2D, got {unpacked.dim()}D")
    n, k = unpacked.shape
    if k < 8:
        raise RuntimeError(f"K must be at least 8, got {k}")
    if k % 8 != 0:
        raise RuntimeError(f"K must be divisible by 8, got {k}")
    nib = (unpacked.to(torch.int64) & 0xF).view(n, k // 8, 8)
    shifts = torch.arange(8, dtype=torch.int64) * 4
    word = (nib << shifts).sum(dim=-1)                       # 0 .. 2^32-1
    word = torch.where(word >= 2 ** 31, word - 2 ** 32, word)  # two's complement int32
    return word.to(torch.int32).contiguous()


def unpack_int4pack_to_int8(packed: torch.Tensor) -> torch.Tensor:
    """PyTorch CPU int4pack layout ([N, K/2] uint8, 64-row blocks) -> [N, K] int8 in 0..15.
    Follows src/cpu/cpp/WOQ_Linear.cpp:361-428."""
    if packed.dtype != torch.uint8:
        raise RuntimeError(f"packed_weight must have dtype uint8, got {packed.dtype}")
    if packed.dim() != 2:
        raise RuntimeError(f"packed_weight must be 2D, got {packed.dim()}D")
    n, k_half = packed.shape
    k = 2 * k_half
    if n % 64 != 0:
        raise RuntimeError(f"packed_weight row count ({n}) must be a multiple of 64")
    nb = n // 64
    src = packed.contiguous().view(nb, k, 32).to(torch.int16)   # block, column, 32 bytes
    p02, p13 = src[:, :, :16], src[:, :, 16:]
    out = torch.empty(nb, 64, k, dtype=torch.int8)
    out[:, 0:16, :] = (p02 & 0xF).transpose(1, 2).to(torch.int8)
    out[:, 32:48, :] = ((p02 >> 4) & 0xF).transpose(1, 2).to(torch.int8)
    out[:, 16:32, :] = (p13 & 0xF).transpose(1, 2).to(torch.int8)
    out[:, 48:64, :] = ((p13 >> 4) & 0xF).transpose(1, 2).to(torch.int8)
    return out.view(n, k)


def woq_repack_from_int4pack(packed: torch.Tensor) -> torch.Tensor:
    """src/cpu/cpp/WOQ_Linear.cpp:430-433."""
    return woq_repack_weight(unpack_int4pack_to_int8(packed))


def woq_unpack(weight: torch.Tensor, signed: bool) -> torch.Tensor:
    """Packed int32 weight as the op receives it (shape [K/8, N], stride (1, K/8)) -> [N, K] int8.
    Nibble of logical element (k, n) is bits [4(k%8), +4) of word n*(K/8) + k//8
    (src/cpu/cpp/WOQ_Linear.cpp:138-146)."""
    k8, n = weight.shape
    rows = weight.t().contiguous().to(torch.int64) & 0xFFFFFFFF          # [N, K/8]
    shifts = torch.arange(8, dtype=torch.int64) * 4
    nib = ((rows.unsqueeze(-1) >> shifts) & 0xF).view(n, k8 * 8)
    if signed:
        nib = torch.where(nib >= 8, nib - 16, nib)
    return nib.to(torch.int8)


# --------------------------------------------------------------------------------------------
# Post-ops  (src/cpu/cpp/MatmulUtils.hpp:19-77)
# --------------------------------------------------------------------------------------------
def apply_post_ops(y: torch.Tensor, post_ops: Sequence[int], buffers: Sequence[torch.Tensor]) -> torch.Tensor:
    """y is fp32 [M, N]; post-ops are applied in order, binary operands consumed in order."""
    b = 0
    for op in post_ops:
        if op == POST_NONE:
            continue
        if op == POST_RELU:
            y = torch.relu(y)
        elif op == POST_GELU_TANH:
            y = torch.nn.functional.gelu(y, approximate="tanh")
        elif op == POST_GELU_ERF:
            y = torch.nn.functional.gelu(y, approximate="none")
        elif op == POST_SILU:
            y = y * torch.sigmoid(y)
        elif op == POST_SIGMOID:
            y = torch.sigmoid(y)
        elif op == POST_TANH:
            y = torch.tanh(y)
        elif op == POST_MUL:
            y = y * buffers[b].reshape(y.shape).float()
            b += 1
        elif op == POST_ADD:
            y = y + buffers[b].reshape(y.shape).float()
            b += 1
        else:
            raise RuntimeError(f"unknown post-op id {op}")
    return y


# --------------------------------------------------------------------------------------------
# WOQ linear  (src/cpu/cpp/WOQ_Linear.cpp:14-292)
# --------------------------------------------------------------------------------------------
def woq_dequant(q: torch.Tensor, scales: torch.Tensor, zeros: Optional[torch.Tensor],
                dq_round: Optional[torch.dtype] = torch.bfloat16) -> torch.Tensor:
    """q: [N, K] int8; scales/zeros: [G, N].  Returns W_dq as fp32 [N, K].

    Symmetric (zeros is None): dq = q * s, q in [-8, 7].  Asymmetric: q in [0, 15] and the zero
    point is a float-domain offset in the tinygemm convention, dq = (q - 8) * s + z
    (test/unittests/op_tests/test_woq_linear_asymmetric.py:30-41).  The reference's test oracle
    rounds dq to the activation dtype before the GEMM (test_woq_linear.py:123,130); dq_round=None
    keeps full fp32 precision instead.
    """
    n, k = q.shape
    g = scales.shape[0]
    if scales.shape[1] != n:
        raise RuntimeError(f"weight_scales dim 1 ({scales.shape[1]}) must match weight dim 1 ({n})")
    if k % g != 0:
        raise RuntimeError("K must be divisible by the number of groups")
    gs = k // g
    s = scales.float().t().repeat_interleave(gs, dim=1)       # [N, K]
    if zeros is None:
        dq = q.float() * s
    else:
        z = zeros.float().t().repeat_interleave(gs, dim=1)
        dq = (q.float() - 8.0) * s + z
    if dq_round is not None:
        dq = dq.to(dq_round).float()
    return dq


def woq_linear(x: torch.Tensor, weight: torch.Tensor, scales: torch.Tensor,
               zeros: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None,
               post_ops: Sequence[int] = (), buffers: Sequence[torch.Tensor] = (),
               dq_round: Optional[torch.dtype] = torch.bfloat16,
               return_fp32: bool = False) -> torch.Tensor:
    """Y = X . dq(Wq) + b, post-ops in fp32, one cast to the input dtype at the end."""
    if weight.dtype != torch.int32:
        raise RuntimeError(f"weight must have dtype int32, got {weight.dtype}")
    if weight.dim() != 2:
        raise RuntimeError(f"weight must be 2D, got {weight.dim()}D")
    n = weight.shape[1]
    k = weight.shape[0] * 8
    q = woq_unpack(weight, signed=zeros is None)
    dq = woq_dequant(q, scales, zeros, dq_round)                          # [N, K] fp32
    x2 = x.reshape(-1, k).float()
    y = (x2.double() @ dq.double().t()).float() if x2.shape[0] * n * k <= (1 << 28) else x2 @ dq.t()
    if bias is not None:
        y = y + bias.float()
    y = apply_post_ops(y, post_ops, [b.reshape(-1, n) for b in buffers])
    y = y.reshape(*x.shape[:-1], n)
    return y if return_fp32 else y.to(x.dtype)


# --------------------------------------------------------------------------------------------
# Dynamic int8 qlinear  (src/cpu/cpp/DynamicQLinear.cpp:74-181)
# --------------------------------------------------------------------------------------------
def dynamic_quantize_s8(x2: torch.Tensor):
    """Per-row symmetric s8: s = max(absmax, 1e-12) / 127 ; q = clamp(rint(x / s), -128, 127),
    all in fp32 with IEEE division and round-half-even
    (test/unittests/op_tests/test_dynamic_qlinear.py:32-36)."""
    xf = x2.float()
    absmax = xf.abs().amax(dim=1, keepdim=True).clamp(min=1e-12)
    s = absmax / 127.0
    q = torch.clamp(torch.round(xf / s), -128, 127).to(torch.int8)
    return q, s.squeeze(1)


def dynamic_quantize_u8(x2: torch.Tensor):
    """Per-row affine u8 (not in the reference op; standard scheme of
    test/unittests/quant_utils.py:13-83 applied per token): lo = min(x, 0), hi = max(x, 0),
    s = max(hi - lo, 1e-12) / 255, zp = clamp(rint(-lo / s), 0, 255),
    q = clamp(rint(x / s) + zp, 0, 255)."""
    xf = x2.float()
    lo = xf.amin(dim=1, keepdim=True).clamp(max=0.0)
    hi = xf.amax(dim=1, keepdim=True).clamp(min=0.0)
    s = (hi - lo).clamp(min=1e-12) / 255.0
    zp = torch.clamp(torch.round(-lo / s), 0, 255)
    q = torch.clamp(torch.round(xf / s) + zp, 0, 255).to(torch.uint8)
    return q, s.squeeze(1), zp.squeeze(1).to(torch.int32)


def int_gemm(q: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """Exact int32 accumulation of q [M, K] (int8/uint8) against w [N, K] int8.  Large signed cases
    use torch's CPU int8 GEMM; unsigned activations are shifted by 128 into the signed range and the
    shift is put back with the weight row sums (both steps exact in integers)."""
    m, k = q.shape
    if q.dtype == torch.uint8:
        if m > 16 and k % 8 == 0 and w.shape[0] % 8 == 0:
            shifted = (q.to(torch.int16) - 128).to(torch.int8)
            return int_gemm(shifted, w) + 128 * w.sum(dim=1, dtype=torch.int32).unsqueeze(0)
        return (q.long() @ w.long().t()).to(torch.int32)
    if m > 16 and k % 8 == 0 and w.shape[0] % 8 == 0:
        return torch._int_mm(q.contiguous(), w.t().contiguous())
    return (q.long() @ w.long().t()).to(torch.int32)


def dynamic_qlinear(x: torch.Tensor, weight: torch.Tensor, weight_scales: torch.Tensor,
                    bias: Optional[torch.Tensor] = None, act_quant: str = "s8_sym",
                    post_ops: Sequence[int] = (), buffers: Sequence[torch.Tensor] = (),
                    return_parts: bool = False):
    """y = acc * (s_m * w_n) + b_n with acc = sum_k q[m,k] W[n,k] (int32).  ``act_quant='u8_asym'``
    and post-ops are extensions that the reference op does not have
    (docs/zentorch_dynamic_qlinear.md:96,99)."""
    if x.dtype not in (torch.bfloat16, torch.float32):
        raise RuntimeError(f"zentorch_dynamic_qlinear: input must be bfloat16 or float32, got {x.dtype}")
    if weight.dtype != torch.int8:
        raise RuntimeError(f"zentorch_dynamic_qlinear: weight must be int8 (c10::kChar), got {weight.dtype}")
    n, k = weight.shape
    if x.shape[-1] != k:
        raise RuntimeError(f"zentorch_dynamic_qlinear: input last dim ({x.shape[-1]}) must match weight dim 1 ({k})")
    if bias is not None and (bias.dim() != 1 or bias.shape[0] != n):
        raise RuntimeError(f"zentorch_dynamic_qlinear: bias must be 1D with size N ({n})")
    x2 = x.reshape(-1, k)
    ws = weight_scales.reshape(-1).float()
    if act_quant == "s8_sym":
        q, s = dynamic_quantize_s8(x2)
        zp = None
        acc = int_gemm(q, weight)
        accf = acc.float()
    elif act_quant == "u8_asym":
        q, s, zp = dynamic_quantize_u8(x2)
        acc = int_gemm(q, weight)
        wsum = weight.sum(dim=1, dtype=torch.int64)                     # [N]
        accf = (acc.long() - zp.long().unsqueeze(1) * wsum.unsqueeze(0)).float()
    else:
        raise RuntimeError(f"unknown act_quant {act_quant}")
    y = accf * (s.unsqueeze(1) * ws.unsqueeze(0))
    if bias is not None:
        y = y + bias.float()
    y = apply_post_ops(y, post_ops, [b.reshape(-1, n) for b in buffers])
    y = y.reshape(*x.shape[:-1], n).to(x.dtype)
    if return_parts:
        return q, s, zp, acc, y
    return y


# --------------------------------------------------------------------------------------------
# Static-quant qlinear  (src/cpu/cpp/QLinear.cpp:66-591)
# --------------------------------------------------------------------------------------------
_QRANGE = {torch.uint8: (0, 255), torch.int8: (-128, 127)}


def quantize_per_tensor(x: torch.Tensor, scale: torch.Tensor, zero_point: Optional[torch.Tensor]) -> torch.Tensor:
    """q = clamp(rint(x * (1 / s)) + zp, lo, hi) in fp32: unsigned 8 bit when a zero point is given, signed 8
    bit with zp = 0 otherwise (src/cpu/cpp/QLinear.cpp:14-17,120-157; the multiplication by the reciprocal is
    what torch.fake_quantize_per_tensor_affine and quantized_decomposed.quantize_per_tensor do, which the
    reference's tests use as the truth: test/unittests/quant_utils.py:33-36,72-79)."""
    inv = 1.0 / scale.reshape(()).float()
    dt = torch.uint8 if zero_point is not None else torch.int8
    lo, hi = _QRANGE[dt]
    zp = 0 if zero_point is None else int(zero_point.reshape(()).item())
    return torch.clamp(torch.round(x.float() * inv) + zp, lo, hi).to(dt)


def static_qlinear(x: torch.Tensor, weight: torch.Tensor, input_scales: torch.Tensor,
                   input_zero_points: Optional[torch.Tensor], weight_scales: torch.Tensor,
                   weight_zero_points: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None,
                   output_scales: Optional[torch.Tensor] = None, output_zero_points: Optional[torch.Tensor] = None,
                   output_dtype: Optional[torch.dtype] = None, post_ops: Sequence[int] = (),
                   buffers: Sequence[torch.Tensor] = (), return_parts: bool = False):
    """zentorch_qlinear and its _relu / _sigmoid / _mul_add variants.

    The activations are quantised per tensor with the caller's scale and zero point (or arrive as u8 / s8
    already), the weight is symmetric s8 [N, K] with one scale or one per output channel; with integer
    accumulation acc = sum_k (q - zp_x) W,  y = post_ops(acc * (s_x * s_w[n]) + bias[n]) in fp32.  Without
    output scales y is cast to float32 / bfloat16; with them it is requantised per tensor,
    clamp(rint(y * (1 / s_o)) + zp_o), to u8 when a zero point is given and to s8 otherwise
    (test/unittests/quant_utils.py:13-83 is the float restatement the reference's tests compare with;
    checks and their messages: src/cpu/cpp/MatmulUtils.hpp:331-525)."""
    if x.dtype not in (torch.float32, torch.bfloat16, torch.uint8, torch.int8):
        raise RuntimeError("unsupported dtype for input tensor, only float32/bfloat16/uint8/int8 is supported")
    if weight.dtype != torch.int8:
        raise RuntimeError("unsupported dtype for weight tensor, only int8 is supported")
    if bias is not None and bias.dtype not in (torch.float32, torch.bfloat16):
        raise RuntimeError("unsupported dtype for bias tensor, only float32 or bfloat16 is supported")
    if input_scales.dtype != torch.float32:
        raise RuntimeError("unsupported dtype for input_scales, only float32 is supported")
    if input_zero_points is not None and input_zero_points.dtype != torch.int32:
        raise RuntimeError("unsupported dtype for input_zero_points, only int32 supported")
    if weight_scales.dtype != torch.float32:
        raise RuntimeError("unsupported dtype for weight_scales, only float32 is supported")
    if weight_zero_points is not None and weight_zero_points.dtype != torch.int32:
        raise RuntimeError("unsupported dtype for weight_zero_points, only int32 is supported")
    if output_dtype is None:
        output_dtype = torch.float32
    if output_dtype not in (torch.float32, torch.bfloat16, torch.uint8, torch.int8):
        raise RuntimeError("output_dtype received is not yet supported, only float32/bfloat16/uint8/int8 is supported")
    n, k = weight.shape
    if x.shape[-1] != k:
        raise RuntimeError("unsupported shapes for input and weight")
    if input_scales.dim() > 1:
        raise RuntimeError("unsupported dims for input_scales with respect to input tensor")
    if input_zero_points is not None and input_zero_points.numel() != 1:
        raise RuntimeError("only supporting per-tensor quantization for input")
    if input_scales.numel() != 1:
        raise RuntimeError("unsupported number of elements for input_scales with respect to input tensor")
    if weight_scales.dim() > 1:
        raise RuntimeError("unsupported dims for weight_scales with respect to weight tensor")
    if weight_scales.numel() not in (1, n):
        raise RuntimeError("unsupported number of elements for weight_scales with respect to weight tensor")
    if output_scales is not None:
        want = torch.uint8 if output_zero_points is not None else torch.int8
        if output_dtype != want:
            raise RuntimeError("unsupported dtype for result tensor when output_scales are defined")
    elif output_dtype not in (torch.float32, torch.bfloat16):
        raise RuntimeError("unsupported dtype for result tensor, only float32/bfloat16 is supported when "
                           "output_scales are not defined")
    x2 = x.reshape(-1, k)
    if x.dtype in (torch.uint8, torch.int8):
        q = x2
    else:
        q = quantize_per_tensor(x2, input_scales, input_zero_points)
    zp = 0 if input_zero_points is None else int(input_zero_points.reshape(()).item())
    acc = int_gemm(q, weight)
    wsum = weight.sum(dim=1, dtype=torch.int64)
    accf = (acc.long() - zp * wsum.unsqueeze(0)).float()
    ws = weight_scales.reshape(-1).float()
    y = accf * (input_scales.reshape(()).float() * ws.unsqueeze(0))
    if bias is not None:
        y = y + bias.float()
    y = apply_post_ops(y, post_ops, [b.reshape(-1, n) for b in buffers])
    if output_scales is not None:
        lo, hi = _QRANGE[output_dtype]
        zo = 0 if output_zero_points is None else int(output_zero_points.reshape(()).item())
        inv = 1.0 / output_scales.reshape(()).float()
        y = torch.clamp(torch.round(y * inv) + zo, lo, hi)
    y = y.reshape(*x.shape[:-1], n).to(output_dtype)
    if return_parts:
        return q, acc, y
    return y


# --------------------------------------------------------------------------------------------
# Compositions without a reference counterpart (parity unpinned)
# --------------------------------------------------------------------------------------------
def route_top2(logits: torch.Tensor, top_k: int = 2):
    """softmax -> top-k -> renormalise; returns (weights [T, k] fp32, ids [T, k] int32)."""
    p = torch.softmax(logits.float(), dim=-1)
    w, ids = torch.topk(p, top_k, dim=-1)
    w = w / w.sum(dim=-1, keepdim=True)
    return w, ids.to(torch.int32)


def moe_woq(x: torch.Tensor, topk_w: torch.Tensor, topk_ids: torch.Tensor,
            w13: Sequence[torch.Tensor], s13: Sequence[torch.Tensor],
            w2: Sequence[torch.Tensor], s2: Sequence[torch.Tensor]) -> torch.Tensor:
    """Mixtral-style expert FFN with int4 WOQ experts.  Structure follows
    src/cpu/cpp/FusedMoE.cpp:289-436 (token grouping) and the gate-first silu-and-mul of
    src/cpu/python/zentorch/vllm/_int8_moe_patch.py:48-50.  Per expert: h = woq_linear(x_e, w13),
    a = silu(h[:, :I]) * h[:, I:], o = woq_linear(a, w2); out[t] = sum_j topk_w[t, j] * o_j[t]."""
    t, _ = x.shape
    out = torch.zeros(t, w2[0].shape[1], dtype=torch.float32)
    for e in range(len(w13)):
        tok, slot = torch.nonzero(topk_ids == e, as_tuple=True)
        if tok.numel() == 0:
            continue
        h = woq_linear(x[tok], w13[e], s13[e], return_fp32=True)
        inter = h.shape[1] // 2
        a = (torch.nn.functional.silu(h[:, :inter]) * h[:, inter:]).to(x.dtype)
        o = woq_linear(a, w2[e], s2[e], return_fp32=True)
        out.index_add_(0, tok, o * topk_w[tok, slot].unsqueeze(1))
    return out.to(x.dtype)


def quantize_woq_sym(w: torch.Tensor, group_size: int):
    """Synthetic-weight quantiser of the benchmark configs: per group of ``group_size`` along K,
    s = max|w| / 7 (clamped at 1e-8), q = clamp(round(w / s), -8, 7).  Returns (q int8 [N, K],
    scales fp32 [K/gs, N]).  Same scheme as test/unittests/op_tests/test_woq_linear.py:71-96
    applied per group."""
    n, k = w.shape
    g = k // group_size
    wg = w.float().view(n, g, group_size)
    s = (wg.abs().amax(dim=2) / 7.0).clamp(min=1e-8)
    q = torch.clamp(torch.round(wg / s.unsqueeze(2)), -8, 7).to(torch.int8).view(n, k)
    return q, s.t().contiguous()


def quantize_int8_per_channel(w: torch.Tensor):
    """s = max|w_row| / 127, q = clamp(round(w / s), -127, 127); returns (q int8 [N, K], s fp32 [N])."""
    s = (w.float().abs().amax(dim=1) / 127.0).clamp(min=1e-12)
    q = torch.clamp(torch.round(w.float() / s.unsqueeze(1)), -127, 127).to(torch.int8)
    return q, s


def tp_shard_woq(weight: torch.Tensor, scales: torch.Tensor, zeros, bias, mode: str, rank: int, world: int):
    """Slice a packed WOQ linear for one tensor-parallel rank.  'column' shards N, 'row' shards K
    on group boundaries (slicing rules of
    src/cpu/python/zentorch/vllm/_torchao_int4_opaque_patch.py:93-163).  The weight slice keeps the
    op's layout contract (shape [K/8, N] with stride (1, K/8))."""
    k8, n = weight.shape
    g = scales.shape[0]
    if mode == "column":
        n0, n1 = rank * n // world, (rank + 1) * n // world
        w = weight.t()[n0:n1].contiguous().t()
        return (w, scales[:, n0:n1].contiguous(), None if zeros is None else zeros[:, n0:n1].contiguous(),
                None if bias is None else bias[n0:n1].contiguous())
    if mode == "row":
        if g % world != 0:
            raise RuntimeError("row-parallel shards must fall on quantization-group boundaries")
        gs = k8 * 8 // g
        g0, g1 = rank * g // world, (rank + 1) * g // world
        w = weight.t()[:, g0 * gs // 8: g1 * gs // 8].contiguous().t()
        return (w, scales[g0:g1].contiguous(), None if zeros is None else zeros[g0:g1].contiguous(),
                bias if rank == 0 else None)
    raise RuntimeError(f"unknown shard mode {mode}")
