"""Helpers shared by the tests: seeded synthetic inputs of the benchmark configs, bf16 bit views,
and the ctypes handle of the C oracle."""
import ctypes as C
import subprocess
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent.parent


def bf16_from_bits(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a)).view(torch.bfloat16)


QLINEAR_POST = {"none": (), "relu": (1,), "sigmoid": (5,), "mul_add": (7, 8)}   # post-op ids of the oracle / C ABI


def qlinear_golden_cases():
    """The static-qlinear cases of tests/golden/zentorch_qlinear_golden.npz (made by the reference's qdq_linear)
    as dictionaries of torch tensors: x, xs, xzp (None for signed activations), w, ws, bias, os / ozp (None
    unless the output is requantised), out_dtype, post (post-op ids), buffers, y (the reference result)."""
    g = np.load(ROOT / "tests" / "golden" / "zentorch_qlinear_golden.npz")
    w, bias = torch.from_numpy(g["w"]), torch.from_numpy(g["bias"])
    cases = []
    for name in g["cases"]:
        tag, x_kind, asym, per_channel, out_kind, eltwise = str(name).split(":")
        x = bf16_from_bits(g[tag + "_x"]) if x_kind == "bfloat16" else torch.from_numpy(g[tag + "_x"])
        y = bf16_from_bits(g[tag + "_y"]) if out_kind == "bfloat16" else torch.from_numpy(g[tag + "_y"])
        c = dict(name=str(name), x=x, xs=torch.from_numpy(g[tag + "_xs"]), w=w, ws=torch.from_numpy(g[tag + "_ws"]),
                 xzp=torch.from_numpy(g[tag + "_xzp"]) if asym == "1" else None, bias=bias, os=None, ozp=None,
                 out_dtype=getattr(torch, out_kind), post=QLINEAR_POST[eltwise], buffers=(), y=y, eltwise=eltwise)
        if out_kind in ("uint8", "int8"):
            c["os"] = torch.from_numpy(g[tag + "_os"])
            c["ozp"] = torch.from_numpy(g[tag + "_ozp"]) if out_kind == "uint8" else None
        if eltwise == "mul_add":
            c["buffers"] = (torch.from_numpy(g[tag + "_mul"]), torch.from_numpy(g[tag + "_add"]))
        cases.append(c)
    return cases


def assert_qlinear_close(got, ref, what):
    """Float outputs: the reference's own tolerance for zentorch_qlinear (atol = rtol = 1e-2,
    test/unittests/op_tests/test_qlinear.py:607-609) and a hundred times tighter in the mean.  Requantised
    outputs: the float restatement and the integer evaluation may land on different sides of a rounding
    boundary, so at most one step apart anywhere and equal in at least 99 % of the elements."""
    assert got.dtype == ref.dtype and got.shape == ref.shape, what
    if ref.dtype in (torch.uint8, torch.int8):
        d = (got.to(torch.int32) - ref.to(torch.int32)).abs()
        assert int(d.max()) <= 1, f"{what}: requantised outputs differ by {int(d.max())} steps"
        assert float((d == 0).float().mean()) >= 0.99, f"{what}: {float((d != 0).float().mean()):.3%} of the outputs differ"
    else:
        g, r = got.float(), ref.float()
        assert torch.allclose(g, r, atol=1e-2, rtol=1e-2), f"{what}: max diff {float((g - r).abs().max()):.3e}"
        lim = 1e-4 if ref.dtype == torch.float32 else 4e-3
        assert float((g - r).abs().mean()) <= lim * max(1.0, float(r.abs().mean())), what


def load_c_oracle() -> C.CDLL:
    so = ROOT / "oracle" / "_build" / "libzentorch_oracle.so"
    src = ROOT / "oracle" / "zentorch_oracle.c"
    if not so.exists() or so.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(ROOT / "oracle")], check=True, capture_output=True)
    lib = C.CDLL(str(so))
    p, i64, i32 = C.c_void_p, C.c_int64, C.c_int
    lib.zt_oracle_woq_repack_weight.argtypes = [p, i64, i64, p]
    lib.zt_oracle_unpack_int4pack.argtypes = [p, i64, i64, p]
    lib.zt_oracle_woq_linear.argtypes = [p, i64, i64, p, i64, p, p, i64, p, i32, p, p, i32, p, p]
    lib.zt_oracle_dynamic_quantize_s8.argtypes = [p, i64, i64, p, p]
    lib.zt_oracle_dynamic_quantize_u8.argtypes = [p, i64, i64, p, p, p]
    lib.zt_oracle_int8_gemm.argtypes = [p, i32, p, i64, i64, i64, p]
    lib.zt_oracle_qlinear_epilogue.argtypes = [p, i64, i64, p, p, p, p, p, i32, p]
    return lib


def make_woq_case(m, k, n, gs, seed=0, asym=False, scale_dtype=torch.float32, bias=True, x_shape=None):
    """Synthetic WOQ linear of the benchmark configs: x ~ N(0,1) bf16, W ~ N(0,0.02) quantised per
    group of gs along K (symmetric: s = max|w|/7; asymmetric: tinygemm min/max scheme), bias ~
    N(0,0.01) bf16.  Returns CPU tensors: x, q [N,K] int8, scales [G,N], zeros or None, bias."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(*(x_shape or (m, k)), generator=g).to(torch.bfloat16)
    w = torch.randn(n, k, generator=g) * 0.02
    ng = k // gs
    wg = w.view(n, ng, gs)
    if not asym:
        s = (wg.abs().amax(dim=2) / 7.0).clamp(min=1e-8)
        q = torch.clamp(torch.round(wg / s.unsqueeze(2)), -8, 7).to(torch.int8).view(n, k)
        scales, zeros = s.t().contiguous().to(scale_dtype), None
    else:
        mn, mx = wg.amin(dim=2), wg.amax(dim=2)
        s = ((mx - mn) / 15.0).clamp(min=1e-6)
        z = mn + s * 8.0
        q = torch.clamp(torch.round((wg - mn.unsqueeze(2)) / s.unsqueeze(2)), 0, 15).to(torch.int8).view(n, k)
        scales, zeros = s.t().contiguous().to(scale_dtype), z.t().contiguous().to(scale_dtype)
    b = (torch.randn(n, generator=g) * 0.01).to(torch.bfloat16) if bias else None
    return x, q, scales, zeros, b


def make_int8_case(m, k, n, seed=0, x_dtype=torch.bfloat16, bias_dtype=torch.float32, bias=True):
    """Synthetic dynamic-int8 linear: x ~ N(0,1), W ~ N(0,0.02) quantised per output channel
    (s = max|w|/127), bias ~ N(0,0.01)."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(m, k, generator=g).to(x_dtype)
    w = torch.randn(n, k, generator=g) * 0.02
    s = (w.abs().amax(dim=1) / 127.0).clamp(min=1e-12)
    q = torch.clamp(torch.round(w / s.unsqueeze(1)), -127, 127).to(torch.int8)
    b = (torch.randn(n, generator=g) * 0.01).to(bias_dtype) if bias else None
    return x, q, s, b


def assert_close_bf16(actual, expected, rtol=1e-2, atol=1e-2, what="", frob=5e-3):
    """The stated tolerance for bf16 results, 1e-2 relative: |a - e| <= rtol * |e| + atol * max(1, rms(e)).
    The absolute floor scales with the output's RMS because the oracle rounds every dequantised weight
    to bf16 (as the reference's test formula does), which by itself scatters results by about
    1e-3 * rms around the exactly computed product.

    The element-wise floor is loose for outputs whose RMS is far below 1, so an aggregate bound goes with
    it: the relative Frobenius error ||a - e|| / ||e|| must stay below `frob`.  Unbiased rounding noise
    (bf16 rounding of the dequantised weights in the oracle, of both outputs) adds up to about 2e-3 there;
    a kernel with a systematic error of one percent cannot hide under it.  Pass frob=None to skip it."""
    a, e = actual.float().cpu(), expected.float().cpu()
    diff = (a - e).abs()
    rms = float(e.pow(2).mean().sqrt()) if e.numel() else 0.0
    bound = atol * max(1.0, rms) + rtol * e.abs()
    bad = diff > bound
    assert not bad.any(), (f"{what}: {int(bad.sum())} of {a.numel()} elements off; max abs diff "
                           f"{diff.max().item():.5f} at value {e.flatten()[diff.argmax()].item():.5f} (rms {rms:.3f})")
    if frob is not None and e.numel() >= 64:
        mask = torch.isfinite(e)
        norm = float(e[mask].double().pow(2).sum().sqrt())
        if norm > 0:
            rel = float((a[mask] - e[mask]).double().pow(2).sum().sqrt()) / norm
            assert rel <= frob, f"{what}: relative Frobenius error {rel:.2e} exceeds {frob:.1e}"


def make_woq_fast(k, n, gs=128, seed=0, asym=False, scale_dtype=torch.float32):
    """Large synthetic WOQ weights without a float master copy: uniform nibbles (signed -8..7, or 0..15
    with zero points) and group scales around max|w|/7 of N(0, 0.02) weights.  Returns CPU tensors
    q [N,K] int8, scales [K/gs, N], zeros or None, bias [N] bf16."""
    g = torch.Generator().manual_seed(seed)
    lo, hi = (0, 16) if asym else (-8, 8)
    q = torch.randint(lo, hi, (n, k), generator=g, dtype=torch.int8)
    scales = (torch.rand(k // gs, n, generator=g) * 0.006 + 0.007).to(scale_dtype)
    zeros = ((torch.rand(k // gs, n, generator=g) - 0.5) * 0.02).to(scale_dtype) if asym else None
    bias = (torch.randn(n, generator=g) * 0.01).to(torch.bfloat16)
    return q, scales, zeros, bias


def woq_oracle_columns(x, q, scales, zeros, bias, cols, gs, dq_round=torch.bfloat16):
    """The WOQ oracle restricted to the output columns `cols` (a LongTensor): dequantise only those weight
    rows (bf16-rounded like the reference's test formula unless dq_round is None), fp32 product, bias.
    Returns fp32 [M, len(cols)].  Lets a test check a 100-MB-class layer without a full CPU product."""
    qs = q[cols].float()                                            # [C, K]
    k = qs.shape[1]
    s = scales.float()[:, cols].t().repeat_interleave(gs, dim=1)    # [C, K]
    if zeros is None:
        dq = qs * s
    else:
        dq = (qs - 8.0) * s + zeros.float()[:, cols].t().repeat_interleave(gs, dim=1)
    if dq_round is not None:
        dq = dq.to(dq_round).float()
    y = x.float() @ dq.t()
    if bias is not None:
        y = y + bias.float()[cols]
    return y


# ---- AtenTensorHandle plumbing for calling the AOTInductor C shims from a test ---------------------------
def aoti_handle(t):
    """A new AtenTensorHandle (heap at::Tensor) for `t`: returns (capsule, address).  Give the capsule back
    with aoti_release() after the call; the shims only borrow their inputs."""
    cap = torch._C._aoti.unsafe_alloc_void_ptr_from_tensor(t)
    get = C.pythonapi.PyCapsule_GetPointer
    get.restype, get.argtypes = C.c_void_p, [C.py_object, C.c_char_p]
    return cap, get(cap, None)


def aoti_release(cap):
    torch._C._aoti.alloc_tensor_by_stealing_from_void_ptr(cap)


def aoti_take(address):
    """The tensor behind an owning handle that a shim returned in *ret0 (the handle is consumed)."""
    new = C.pythonapi.PyCapsule_New
    new.restype, new.argtypes = C.py_object, [C.c_void_p, C.c_char_p, C.c_void_p]
    return torch._C._aoti.alloc_tensor_by_stealing_from_void_ptr(new(address, None, None))
