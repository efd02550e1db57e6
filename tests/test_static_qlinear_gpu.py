"""Parity of the static-quantisation linear (zentorch_qlinear family) on a B200: through the C ABI against the
CPU oracle and against the golden vectors made by the reference's own test formula, and through
torch.ops.zentorch.zentorch_qlinear* / the AOTInductor shims.

Quantised activations are compared bit for bit.  Float outputs: 1e-4 (fp32) / 1e-2 (bf16) of the oracle.
Requantised outputs sit on rounding boundaries of a float result that the GPU and the CPU evaluate with the
same operations in the same order, so they are compared bit for bit with the oracle too; against the
reference's float restatement (which sums in another order) one quantisation step in at most 1 % of the
elements is allowed, as in the oracle's own pin."""
import ctypes as C

import pytest
import torch

import zentorch_oracle as O
from _util import aoti_handle, aoti_release, aoti_take, assert_qlinear_close, qlinear_golden_cases

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def capi(zt):
    from zentorch_b200 import _capi
    assert torch.cuda.is_available() and _capi.lib().zt_device_supported() == 1
    return _capi


def _cuda(t):
    return None if t is None else t.cuda()


def _case(m, k, n, x_kind, per_channel, out_kind, seed, bias_dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    asym = x_kind in ("float32", "uint8") or (x_kind == "bfloat16" and seed % 2 == 0)
    if x_kind == "uint8":
        x = torch.randint(0, 256, (m, k), generator=g, dtype=torch.uint8)
    elif x_kind == "int8":
        x = torch.randint(-128, 128, (m, k), generator=g, dtype=torch.int8)
        asym = False
    else:
        x = (torch.randn(m, k, generator=g) * 1.5).to(getattr(torch, x_kind))
    w = torch.randint(-128, 128, (n, k), generator=g, dtype=torch.int8)
    c = dict(x=x, w=w, xs=torch.rand(1, generator=g) * 0.03 + 0.01,
             xzp=torch.randint(100, 156, (1,), generator=g, dtype=torch.int32) if asym else None,
             ws=torch.rand(n if per_channel else 1, generator=g) * 0.004 + 0.001,
             bias=torch.randn(n, generator=g).to(bias_dtype), os=None, ozp=None, out_dtype=getattr(torch, out_kind))
    if out_kind in ("uint8", "int8"):
        # the output scale follows the magnitude of the result so that the quantised range is used
        c["os"] = torch.rand(1, generator=g) * 0.02 * (k / 96) ** 0.5 + 0.03 * (k / 96) ** 0.5
        c["ozp"] = torch.randint(90, 166, (1,), generator=g, dtype=torch.int32) if out_kind == "uint8" else None
    return c


def _run(capi, c, post=(), buffers=(), algo=None, out=None):
    return capi.static_qlinear(c["x"].cuda(), c["w"].cuda(), c["xs"].cuda(), _cuda(c["xzp"]), c["ws"].cuda(),
                               _cuda(c["bias"]), _cuda(c["os"]), _cuda(c["ozp"]), c["out_dtype"], post,
                               tuple(b.cuda() for b in buffers), algo=capi.ZT_ALGO_AUTO if algo is None else algo,
                               out=out)


def _oracle(c, post=(), buffers=()):
    return O.static_qlinear(c["x"], c["w"], c["xs"], c["xzp"], c["ws"], None, c["bias"], c["os"], c["ozp"],
                            c["out_dtype"], post, buffers)


def _compare(y, ref, what, exact=True):
    """exact=False (a transcendental post-op before the requantisation: the device's and the host's sigmoid
    differ in the last bits): one step in at most 1 % of the elements."""
    y = y.cpu()
    assert y.dtype == ref.dtype and y.shape == ref.shape
    if ref.dtype in (torch.uint8, torch.int8):
        if exact:
            assert torch.equal(y, ref), f"{what}: {int((y != ref).sum())} of {ref.numel()} requantised outputs differ"
        else:
            assert_qlinear_close(y, ref, what)
    elif ref.dtype == torch.float32:
        assert torch.allclose(y, ref, rtol=1e-4, atol=1e-4 * max(1.0, float(ref.abs().mean()))), \
            f"{what}: max diff {float((y - ref).abs().max()):.3e}"
    else:
        assert torch.allclose(y.float(), ref.float(), rtol=1e-2, atol=1e-2), what


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("numel", [1, 7, 8, 4096, 100003])
def test_static_quantize_bit_exact(capi, dtype, numel):
    g = torch.Generator().manual_seed(numel)
    x = (torch.randn(numel, generator=g) * 2).to(dtype)
    x[0] = 0.5
    s = torch.tensor([0.0173])
    zp = torch.tensor([131], dtype=torch.int32)
    assert torch.equal(capi.static_quantize(x.cuda(), s.cuda(), zp.cuda()).cpu(), O.quantize_per_tensor(x, s, zp))
    assert torch.equal(capi.static_quantize(x.cuda(), s.cuda(), None).cpu(), O.quantize_per_tensor(x, s, None))


def test_golden_cases_through_the_c_abi(capi):
    """Every case of the golden file (input dtype x zero-point kind x weight granularity x output dtype,
    relu / sigmoid / mul_add), small shapes: the kernel for unaligned shapes."""
    for c in qlinear_golden_cases():
        y = _run(capi, c, c["post"], c["buffers"])
        _compare(y, _oracle(c, c["post"], c["buffers"]), c["name"] + " vs oracle")
        assert_qlinear_close(y.cpu(), c["y"], c["name"] + " vs reference formula")


@pytest.mark.parametrize("out_kind", ["float32", "bfloat16", "uint8", "int8"])
@pytest.mark.parametrize("x_kind", ["float32", "bfloat16", "uint8", "int8"])
@pytest.mark.parametrize("m,k,n,per_channel", [(5, 256, 96, True), (130, 512, 384, True), (300, 1024, 200, False),
                                               (513, 4096, 1024, True)])
def test_tensor_core_path_matches_oracle(capi, m, k, n, per_channel, x_kind, out_kind):
    c = _case(m, k, n, x_kind, per_channel, out_kind, seed=m + k + n)
    y = _run(capi, c, algo=capi.ZT_ALGO_TCGEN05)
    ref = _oracle(c)
    _compare(y, ref, f"M={m} K={k} N={n} {x_kind}->{out_kind}")
    if ref.dtype in (torch.uint8, torch.int8):      # the case exercises the quantised range, not one clamped value
        assert int(ref.to(torch.int32).max()) - int(ref.to(torch.int32).min()) > 60
    # the dispatcher's own choice gives the same bytes
    assert torch.equal(_run(capi, c), y)


@pytest.mark.parametrize("post,name", [((O.POST_RELU,), "relu"), ((O.POST_SIGMOID,), "sigmoid"),
                                       ((O.POST_MUL, O.POST_ADD), "mul_add")])
@pytest.mark.parametrize("out_kind", ["bfloat16", "uint8"])
@pytest.mark.parametrize("buf_dtype", [torch.float32, torch.bfloat16])
def test_post_ops(capi, post, name, out_kind, buf_dtype):
    m, k, n = 200, 768, 320
    c = _case(m, k, n, "bfloat16", True, out_kind, seed=len(name), bias_dtype=torch.bfloat16)
    g = torch.Generator().manual_seed(3)
    buffers = (torch.randn(m, n, generator=g).to(buf_dtype), torch.randn(m, n, generator=g).to(buf_dtype)) \
        if name == "mul_add" else ()
    if name == "sigmoid" and out_kind == "uint8":
        c["os"], c["ozp"] = torch.tensor([1.0 / 255]), torch.tensor([0], dtype=torch.int32)
    for algo in (capi.ZT_ALGO_TCGEN05, capi.ZT_ALGO_GENERIC):
        _compare(_run(capi, c, post, buffers, algo), _oracle(c, post, buffers), f"{name} -> {out_kind} algo {algo}",
                 exact=(name != "sigmoid"))


def test_u8_dynamic_rows_agree_with_the_static_form(capi):
    """Ties the per-token u8 mode of the dynamic linear (an extension without a reference fixture) to the static
    form, which is pinned by the reference's formula: a row's quantised bytes, scale and zero point from
    zt_dynamic_quantize, fed to zt_static_qlinear, give the dynamic linear's row (the two epilogues differ only in
    whether product and sum are fused: 1e-6 relative)."""
    from _util import make_int8_case
    x, w, ws, b = make_int8_case(6, 512, 96, seed=8)
    xd, wd, wsd, bd = x.float().cuda(), w.cuda(), ws.reshape(-1).float().cuda(), b.float().cuda()
    y = capi.dynamic_qlinear(xd, wd, wsd, bd, act_quant=capi.ZT_ACT_U8_ASYM)
    q, s, zp = capi.dynamic_quantize(xd, capi.ZT_ACT_U8_ASYM)
    for m in range(x.shape[0]):
        row = capi.static_qlinear(q[m:m + 1].contiguous(), wd, s[m:m + 1].contiguous(), zp[m:m + 1].contiguous(), wsd, bd,
                                  out_dtype=torch.float32)
        assert torch.allclose(row, y[m:m + 1], rtol=1e-6, atol=1e-6 * float(y.abs().max()))
        ref = O.static_qlinear(q[m:m + 1].cpu(), w, s[m:m + 1].cpu(), zp[m:m + 1].cpu(), ws.reshape(-1).float(), None,
                               b.float(), output_dtype=torch.float32)
        assert torch.equal(row.cpu(), ref)


def test_strided_output(capi):
    """The .out operators write into views of wider buffers: rows ldy elements apart, the rest untouched."""
    m, k, n = 70, 256, 48
    for out_kind, width in (("float32", 64), ("uint8", 80), ("bfloat16", 51)):
        c = _case(m, k, n, "float32", True, out_kind, seed=width)
        wide = torch.full((m, width), 7, dtype=c["out_dtype"], device="cuda")
        first = 3 if width == 51 else 16            # 3: rows that are not 16-byte aligned
        view = wide[:, first:first + n]
        _run(capi, c, out=view)
        _compare(view.contiguous(), _oracle(c), f"strided {out_kind}")
        outside = torch.ones(width, dtype=torch.bool)
        outside[first:first + n] = False
        assert bool((wide[:, outside.cuda()] == 7).all())


def test_argument_checks(capi):
    c = _case(4, 64, 16, "float32", True, "float32", seed=1)
    with pytest.raises(RuntimeError, match="output_scales are not defined"):
        capi.static_qlinear(c["x"].cuda(), c["w"].cuda(), c["xs"].cuda(), c["xzp"].cuda(), c["ws"].cuda(),
                            out_dtype=torch.uint8)
    with pytest.raises(RuntimeError, match="unsupported number of elements for weight_scales"):
        capi.static_qlinear(c["x"].cuda(), c["w"].cuda(), c["xs"].cuda(), c["xzp"].cuda(), c["ws"][:5].cuda())
    with pytest.raises(RuntimeError, match="needs input_zero_points"):
        capi.static_qlinear(torch.zeros(4, 64, dtype=torch.uint8, device="cuda"), c["w"].cuda(), c["xs"].cuda(), None,
                            c["ws"].cuda())


# ---- torch.ops.zentorch.zentorch_qlinear* -----------------------------------------------------------------
def test_torch_ops_match_oracle(capi):
    ops = torch.ops.zentorch
    m, k, n = 3 * 50, 512, 256
    c = _case(m, k, n, "bfloat16", True, "float32", seed=9)
    x3 = c["x"].reshape(3, 50, k)
    c["xzp"] = torch.tensor([117], dtype=torch.int32)
    args = (c["w"].cuda(), c["xs"].cuda(), c["xzp"].cuda(), c["ws"].cuda(), None)
    ref = _oracle(c)
    y = ops.zentorch_qlinear(x3.cuda(), *args, c["bias"].cuda(), None, None, torch.float32)
    assert y.shape == (3, 50, n)
    _compare(y.reshape(m, n), ref, "zentorch_qlinear")
    # default output dtype is float32 (src/cpu/cpp/QLinear.cpp:433-435)
    assert ops.zentorch_qlinear(x3.cuda(), *args, c["bias"].cuda(), None, None).dtype == torch.float32
    _compare(ops.zentorch_qlinear_relu(x3.cuda(), *args, c["bias"].cuda(), None, None, torch.float32).reshape(m, n),
             _oracle(c, (O.POST_RELU,)), "zentorch_qlinear_relu")
    _compare(ops.zentorch_qlinear_sigmoid(x3.cuda(), *args, c["bias"].cuda(), None, None, torch.bfloat16).reshape(m, n),
             O.static_qlinear(c["x"], c["w"], c["xs"], c["xzp"], c["ws"], None, c["bias"], None, None, torch.bfloat16,
                              (O.POST_SIGMOID,)), "zentorch_qlinear_sigmoid")
    g = torch.Generator().manual_seed(5)
    mul, add = torch.randn(3, 50, n, generator=g), torch.randn(3, 50, n, generator=g)
    _compare(ops.zentorch_qlinear_mul_add(x3.cuda(), *args, mul.cuda(), add.cuda(), c["bias"].cuda(), None, None,
                                          torch.float32).reshape(m, n),
             _oracle(c, (O.POST_MUL, O.POST_ADD), (mul.reshape(m, n), add.reshape(m, n))), "zentorch_qlinear_mul_add")
    # requantised: u8 with output zero points, s8 without
    os_, ozp = torch.tensor([0.11]), torch.tensor([120], dtype=torch.int32)
    y8 = ops.zentorch_qlinear(x3.cuda(), *args, c["bias"].cuda(), os_.cuda(), ozp.cuda(), torch.uint8)
    _compare(y8.reshape(m, n), O.static_qlinear(c["x"], c["w"], c["xs"], c["xzp"], c["ws"], None, c["bias"], os_, ozp,
                                                torch.uint8), "u8 output")
    ys = ops.zentorch_qlinear(x3.cuda(), *args, c["bias"].cuda(), os_.cuda(), None, torch.int8)
    _compare(ys.reshape(m, n), O.static_qlinear(c["x"], c["w"], c["xs"], c["xzp"], c["ws"], None, c["bias"], os_, None,
                                                torch.int8), "s8 output")
    # a quantised output feeds the next qlinear as it is
    c2 = _case(m, n, 64, "float32", True, "float32", seed=4)
    y2 = ops.zentorch_qlinear(y8.reshape(m, n), c2["w"].cuda(), os_.cuda(), ozp.cuda(), c2["ws"].cuda(), None, None,
                              None, None, torch.float32)
    ref2 = O.static_qlinear(y8.reshape(m, n).cpu(), c2["w"], os_, ozp, c2["ws"])
    _compare(y2, ref2, "chained qlinear")
    # signed activations: no zero points (None for the non-optional Tensor argument, as the reference's tests pass it)
    cs = _case(m, k, n, "float32", False, "float32", seed=12)
    cs["xzp"] = None
    ysig = ops.zentorch_qlinear(cs["x"].cuda(), cs["w"].cuda(), cs["xs"].cuda(), None, cs["ws"].cuda(), None,
                                cs["bias"].cuda(), None, None, torch.float32)
    _compare(ysig, _oracle(cs), "signed activations, per-tensor weight scale")


def test_torch_out_variants(capi):
    ops = torch.ops.zentorch
    m, k, n = 64, 256, 80
    c = _case(m, k, n, "float32", True, "float32", seed=21)
    args = (c["x"].cuda(), c["w"].cuda(), c["xs"].cuda(), c["xzp"].cuda(), c["ws"].cuda(), None, c["bias"].cuda(),
            None, None)
    wide = torch.zeros(m, 2 * n + 8, device="cuda")
    ops.zentorch_qlinear.out(wide[:, 8:8 + n], *args, torch.float32)
    ops.zentorch_qlinear_relu.out(wide[:, 8 + n:], *args, torch.float32)
    _compare(wide[:, 8:8 + n].contiguous(), _oracle(c), "qlinear.out")
    _compare(wide[:, 8 + n:].contiguous(), _oracle(c, (O.POST_RELU,)), "qlinear_relu.out")
    assert bool((wide[:, :8] == 0).all())
    with pytest.raises(RuntimeError, match="output_dtype received does not match the dtype of the output tensor"):
        ops.zentorch_qlinear.out(wide[:, 8:8 + n], *args, torch.bfloat16)


def test_torch_error_messages(capi):
    """Messages of src/cpu/cpp/MatmulUtils.hpp:357-415,453-501 that the reference's tests match on
    (test/unittests/op_tests/test_qlinear.py:78-505)."""
    ops = torch.ops.zentorch
    c = _case(4, 64, 16, "float32", True, "float32", seed=2)
    x, w, xs, xzp, ws, b = (t.cuda() for t in (c["x"], c["w"], c["xs"], c["xzp"], c["ws"], c["bias"]))

    def call(**kw):
        a = dict(x=x, w=w, xs=xs, xzp=xzp, ws=ws, wzp=None, b=b, os=None, ozp=None, dt=torch.float32)
        a.update(kw)
        return ops.zentorch_qlinear(a["x"], a["w"], a["xs"], a["xzp"], a["ws"], a["wzp"], a["b"], a["os"], a["ozp"], a["dt"])

    cases = [
        (dict(x=x.half()), "unsupported dtype for input tensor, only float32/bfloat16/uint8/int8 is supported"),
        (dict(w=w.float()), "unsupported dtype for weight tensor, only int8 is supported"),
        (dict(b=b.half()), "unsupported dtype for bias tensor, only float32 or bfloat16 is supported"),
        (dict(xs=xs.half()), "unsupported dtype for input_scales"),
        (dict(xzp=xzp.float()), "unsupported dtype for input_zero_points"),
        (dict(ws=ws.half()), "unsupported dtype for weight_scales"),
        (dict(wzp=torch.zeros(16, device="cuda")), "unsupported dtype for weight_zero_points"),
        (dict(os=xs.half(), dt=torch.int8), "unsupported dtype for output_scales"),
        (dict(os=xs, ozp=xzp.float(), dt=torch.uint8), "unsupported dtype for output_zero_points"),
        (dict(dt=torch.float16), "output_dtype received is not yet supported"),
        (dict(dt=torch.uint8), "only float32/bfloat16 is supported when output_scales are not defined"),
        (dict(xs=torch.ones(2, device="cuda")), "unsupported number of elements for input_scales"),
        (dict(xs=torch.ones(1, 1, device="cuda")), "unsupported dims for input_scales"),
        (dict(xzp=torch.zeros(2, dtype=torch.int32, device="cuda")), "only supporting per-tensor quantization for input"),
        (dict(ws=torch.ones(5, device="cuda")), "unsupported number of elements for weight_scales"),
        (dict(ws=torch.ones(1, 16, device="cuda")), "unsupported dims for weight_scales"),
        (dict(x=x[:, :32]), "unsupported shapes for input and weight"),
        (dict(b=b[:8]), "unsupported shapes for input, weight and bias"),
        (dict(ws=ws.cpu()), "must be on the input's device"),
    ]
    for kw, msg in cases:
        with pytest.raises(RuntimeError, match=msg):
            call(**kw)


def test_meta_kernels(capi):
    ops = torch.ops.zentorch
    x = torch.empty(2, 5, 64, device="meta")
    w = torch.empty(24, 64, dtype=torch.int8, device="meta")
    s = torch.empty(1, device="meta")
    z = torch.empty(1, dtype=torch.int32, device="meta")
    y = ops.zentorch_qlinear(x, w, s, z, torch.empty(24, device="meta"), None, None, None, None, torch.uint8)
    assert y.shape == (2, 5, 24) and y.dtype == torch.uint8
    y = ops.zentorch_qlinear_mul_add(x, w, s, z, torch.empty(24, device="meta"), None, torch.empty(2, 5, 24, device="meta"),
                                     torch.empty(2, 5, 24, device="meta"), None, None, None)
    assert y.shape == (2, 5, 24) and y.dtype == torch.float32


def test_aoti_shim(capi):
    """aoti_torch_cuda_zentorch_qlinear_relu with the parameter list of src/cpu/cpp/shim_cpu_zentorch.hpp:36-42."""
    from zentorch_b200 import _capi
    lib = _capi._torch_boundary()
    m, k, n = 40, 256, 64
    c = _case(m, k, n, "bfloat16", True, "bfloat16", seed=6)
    w_zero_points = torch.zeros(1, dtype=torch.int32, device="cuda")   # symmetric weights, as the reference expects
    tensors = [c["x"].cuda(), c["w"].cuda(), c["xs"].cuda(), c["xzp"].cuda(), c["ws"].cuda(), w_zero_points,
               c["bias"].cuda()]
    handles = [aoti_handle(t) for t in tensors]                  # (capsule, address) pairs
    vp = C.c_void_p
    bias_slot, ret = vp(handles[6][1]), vp(None)
    dtype_code = C.c_int32(15)                                     # c10::ScalarType::BFloat16
    fn = lib.aoti_torch_cuda_zentorch_qlinear_relu
    fn.restype = C.c_int32
    rc = fn(*(vp(a) for _, a in handles[:6]), C.byref(bias_slot), None, None, C.byref(dtype_code),
            b"zentorch::zentorch_qlinear_relu", C.byref(ret))
    assert rc == 0
    y = aoti_take(ret.value)
    for cap, _ in handles:
        aoti_release(cap)
    ref = O.static_qlinear(c["x"], c["w"], c["xs"], c["xzp"], c["ws"], None, c["bias"], None, None, torch.bfloat16,
                           (O.POST_RELU,))
    _compare(y, ref, "shim")
