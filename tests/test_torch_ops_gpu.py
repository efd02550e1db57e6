"""The torch.ops.zentorch operators on CUDA tensors: what a user of the reference calls."""
import pytest
import torch

import zentorch_oracle as O
from _util import assert_close_bf16, bf16_from_bits, make_int8_case, make_woq_case

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops(zt):
    assert torch.cuda.is_available()
    return torch.ops.zentorch


@pytest.mark.parametrize("shape", [(7, 256), (2, 3, 256), (2, 2, 3, 256)])
def test_woq_linear_op_ranks(ops, shape):
    x, q, s, z, b = make_woq_case(0, 256, 80, 128, seed=1, x_shape=shape)
    packed = ops.zentorch_woq_repack_weight(q.cuda())
    y = ops.zentorch_woq_linear(x.cuda(), packed.t(), s.cuda(), None, b.cuda())
    assert y.shape == (*shape[:-1], 80) and y.dtype == torch.bfloat16 and y.is_contiguous()
    assert_close_bf16(y, O.woq_linear(x, packed.cpu().t(), s, None, b))
    # non-contiguous input is made contiguous by the op
    xt = x.cuda().transpose(0, -2) if len(shape) > 2 else x.cuda()[::2]
    xt_cpu = x.transpose(0, -2) if len(shape) > 2 else x[::2]
    y2 = ops.zentorch_woq_linear(xt, packed.t(), s.cuda(), None, None)
    assert_close_bf16(y2, O.woq_linear(xt_cpu.contiguous(), packed.cpu().t(), s, None, None))


def test_woq_fused_variants(ops):
    m, k, n = 12, 384, 64
    x, q, s, z, b = make_woq_case(m, k, n, 128, seed=2)
    packed = ops.zentorch_woq_repack_weight(q.cuda())
    wt, sd, bd, xd = packed.t(), s.cuda(), b.cuda(), x.cuda()
    pc = packed.cpu().t()
    g = torch.Generator().manual_seed(3)
    a1 = torch.randn(m, n, generator=g).to(torch.bfloat16)
    a2 = torch.randn(m, n, generator=g).to(torch.bfloat16)
    for name, post in (("relu", O.POST_RELU), ("sigmoid", O.POST_SIGMOID), ("gelu_tanh", O.POST_GELU_TANH),
                       ("gelu_erf", O.POST_GELU_ERF)):
        y = getattr(ops, f"zentorch_woq_linear_{name}")(xd, wt, sd, None, bd)
        assert_close_bf16(y, O.woq_linear(x, pc, s, None, b, [post]), what=name)
    y = ops.zentorch_woq_linear_add(xd, wt, sd, None, a1.cuda(), bd)
    assert_close_bf16(y, O.woq_linear(x, pc, s, None, b, [O.POST_ADD], [a1]), what="add")
    y = ops.zentorch_woq_linear_mul_add(xd, wt, sd, None, a1.cuda(), a2.cuda(), bd)
    assert_close_bf16(y, O.woq_linear(x, pc, s, None, b, [O.POST_MUL, O.POST_ADD], [a1, a2]), what="mul_add")
    y = ops.zentorch_woq_linear_add_add(xd, wt, sd, None, a1.cuda(), a2.cuda(), bd)
    assert_close_bf16(y, O.woq_linear(x, pc, s, None, b, [O.POST_ADD, O.POST_ADD], [a1, a2]), what="add_add")


def test_woq_asymmetric_from_int4pack(ops, golden):
    x = bf16_from_bits(golden["asym_x"])
    repacked = ops.zentorch_woq_repack_from_int4pack(torch.from_numpy(golden["asym_int4pack"]).cuda())
    s, z = bf16_from_bits(golden["asym_scale"]), bf16_from_bits(golden["asym_zero"])
    y = ops.zentorch_woq_linear(x.cuda(), repacked.t(), s.cuda(), z.cuda(), None, zentorch_op_name="zentorch_woq_linear")
    ref = bf16_from_bits(golden["asym_y"])
    assert torch.allclose(y.cpu().float(), ref.float(), rtol=0.1, atol=2.0)


def test_woq_error_messages(ops):
    x = torch.zeros(2, 64, dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(32, 8, dtype=torch.int32, device="cuda")
    s = torch.ones(1, 32, device="cuda")
    with pytest.raises(RuntimeError, match="weight must have dtype int32"):
        ops.zentorch_woq_linear(x, w.t().to(torch.int8), s, None, None)
    with pytest.raises(RuntimeError, match=r"weight_scales dim 1 \(16\) must match weight dim 1 \(32\)"):
        ops.zentorch_woq_linear(x, w.t(), torch.ones(1, 16, device="cuda"), None, None)
    with pytest.raises(RuntimeError, match="transposed view"):
        ops.zentorch_woq_linear(x, w.t().contiguous(), s, None, None)
    with pytest.raises(RuntimeError, match="K must be divisible by 8"):
        ops.zentorch_woq_repack_weight(torch.zeros(4, 12, dtype=torch.int8, device="cuda"))
    with pytest.raises(RuntimeError, match="must have dtype int8"):
        ops.zentorch_woq_repack_weight(torch.zeros(4, 16, dtype=torch.int32, device="cuda"))
    with pytest.raises(RuntimeError, match="multiple of 64"):
        ops.zentorch_woq_repack_from_int4pack(torch.zeros(32, 16, dtype=torch.uint8, device="cuda"))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_dynamic_qlinear_op(ops, dtype, golden):
    x, w, ws, b = make_int8_case(40, 256, 96, seed=5, x_dtype=dtype)
    x3 = x.view(5, 8, 256)
    y = ops.zentorch_dynamic_qlinear(x3.cuda(), w.cuda(), ws.cuda().unsqueeze(0), b.cuda())
    ref = O.dynamic_qlinear(x3, w, ws, b)
    assert y.shape == (5, 8, 96) and y.dtype == dtype
    if dtype == torch.float32:
        assert torch.allclose(y.cpu(), ref, rtol=1e-4, atol=1e-4)
    else:
        assert_close_bf16(y, ref)
    # deliberately non-contiguous weight / scales / bias (model_tests/test_dynamic_qlinear.py:171-205)
    w_nc = w.t().contiguous().cuda().t()
    ws_nc = torch.stack([ws, ws], dim=1).cuda()[:, 0]
    b_nc = torch.stack([b, b], dim=1).cuda()[:, 0]
    y2 = ops.zentorch_dynamic_qlinear(x3.cuda(), w_nc, ws_nc, b_nc)
    assert torch.equal(y2, y)
    if dtype == torch.float32:
        gx = torch.from_numpy(golden["dyn_x"])
        gy = ops.zentorch_dynamic_qlinear(gx.cuda(), torch.from_numpy(golden["dyn_w"]).cuda(),
                                          torch.from_numpy(golden["dyn_ws"]).cuda().unsqueeze(0),
                                          torch.from_numpy(golden["dyn_b"]).cuda())
        assert torch.allclose(gy.cpu(), torch.from_numpy(golden["dyn_y"]), rtol=1e-2, atol=1e-2)


def test_dynamic_qlinear_ext_and_errors(ops):
    x, w, ws, b = make_int8_case(20, 128, 48, seed=6)
    y = ops.zentorch_dynamic_qlinear_ext(x.cuda(), w.cuda(), ws.cuda(), b.cuda(), act_quant="u8_asym", post_op="silu")
    assert_close_bf16(y, O.dynamic_qlinear(x, w, ws, b, act_quant="u8_asym", post_ops=[O.POST_SILU]))
    with pytest.raises(RuntimeError, match="input must be bfloat16 or float32"):
        ops.zentorch_dynamic_qlinear(x.cuda().half(), w.cuda(), ws.cuda(), None)
    with pytest.raises(RuntimeError, match="weight must be int8"):
        ops.zentorch_dynamic_qlinear(x.cuda(), w.cuda().int(), ws.cuda(), None)
    with pytest.raises(RuntimeError, match="bias must be 1D with size N"):
        ops.zentorch_dynamic_qlinear(x.cuda(), w.cuda(), ws.cuda(), b.cuda()[:3])
    with pytest.raises(RuntimeError, match=r"input last dim \(64\) must match weight dim 1 \(128\)"):
        ops.zentorch_dynamic_qlinear(x.cuda()[:, :64], w.cuda(), ws.cuda(), None)


def test_cuda_graph_capture(ops):
    """Both ops launch on the current stream without host synchronisation and can be captured."""
    x, q, s, z, b = make_woq_case(4, 512, 256, 128, seed=8)
    packed = ops.zentorch_woq_repack_weight(q.cuda())
    xd, sd, bd = x.cuda(), s.cuda(), b.cuda()
    xi, wi, wsi, bi = [t.cuda() for t in make_int8_case(64, 256, 128, seed=9)]
    y_eager = ops.zentorch_woq_linear(xd, packed.t(), sd, None, bd)
    yi_eager = ops.zentorch_dynamic_qlinear(xi, wi, wsi, bi)
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        ops.zentorch_woq_linear(xd, packed.t(), sd, None, bd)      # warm-up on the capture stream
        ops.zentorch_dynamic_qlinear(xi, wi, wsi, bi)
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            y = ops.zentorch_woq_linear(xd, packed.t(), sd, None, bd)
            yi = ops.zentorch_dynamic_qlinear(xi, wi, wsi, bi)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(y, y_eager) and torch.equal(yi, yi_eager)


def test_arguments_on_other_devices_are_refused(ops):
    """Every tensor argument must live on the input's GPU; a host tensor raises before anything is launched."""
    x, q, s, z, b = make_woq_case(2, 256, 64, 128, seed=12)
    packed = ops.zentorch_woq_repack_weight(q.cuda())
    with pytest.raises(RuntimeError, match="weight_scales must be on the input's device"):
        ops.zentorch_woq_linear(x.cuda(), packed.t(), s, None, b.cuda())
    with pytest.raises(RuntimeError, match="bias must be on the input's device"):
        ops.zentorch_woq_linear(x.cuda(), packed.t(), s.cuda(), None, b)
    with pytest.raises(RuntimeError, match="binary post-op operand must be on the input's device"):
        ops.zentorch_woq_linear_add(x.cuda(), packed.t(), s.cuda(), None, torch.zeros(2, 64, dtype=torch.bfloat16), b.cuda())
    xi, wi, wsi, bi = make_int8_case(4, 64, 16, seed=13)
    with pytest.raises(RuntimeError, match="weight must be on the input's device"):
        ops.zentorch_dynamic_qlinear(xi.cuda(), wi, wsi.cuda(), None)
    with pytest.raises(RuntimeError, match="weight_scales must be on the input's device"):
        ops.zentorch_dynamic_qlinear(xi.cuda(), wi.cuda(), wsi, None)
    torch.cuda.synchronize()


def test_weights_fresh_every_call_through_the_ops(ops):
    """Weights that are made right before each call (no constant folding): the boundary has not seen them
    before, or sees a new storage at an old address, and tells the kernels not to prefetch them."""
    m, k, n = 3, 2048, 512
    x, q, s, z, b = make_woq_case(m, k, n, 128, seed=14)
    ref = O.woq_linear(x, O.woq_repack_weight(q).t(), s, None, b)
    xd, qd, s_t, bd = x.cuda(), q.cuda(), s.t().contiguous().cuda(), b.cuda()
    junk = torch.empty(64 << 20, dtype=torch.uint8, device="cuda")
    for rep in range(10):
        junk.random_(0, 255)
        y = ops.zentorch_woq_linear(xd, ops.zentorch_woq_repack_weight(qd).t(), s_t.t().contiguous(), None, bd)
        assert_close_bf16(y, ref, what=f"fresh weights rep {rep}")
    xi, wi, wsi, bi = make_int8_case(64, 512, 256, seed=15)
    refi = O.dynamic_qlinear(xi, wi, wsi, bi)
    wt = wi.t().contiguous().cuda()
    for rep in range(10):
        junk.random_(0, 255)
        yi = ops.zentorch_dynamic_qlinear(xi.cuda(), wt.t(), wsi.cuda(), bi.cuda())   # non-contiguous: copied in the op
        assert_close_bf16(yi, refi, what=f"int8 fresh weights rep {rep}")


def test_aoti_shims_compute(zt):
    """The C shims Inductor's cpp_wrapper calls (same parameter lists as aoti_torch_cpu_zentorch_*,
    src/cpu/cpp/shim_cpu_zentorch.hpp:150-197), called for real: borrowed input handles, nullable optional
    handles, a new owning handle in *ret0, zero return code."""
    import ctypes as C
    from pathlib import Path
    from _util import aoti_handle, aoti_release, aoti_take
    lib = C.CDLL(str(Path(zt.__file__).resolve().parent.parent / "lib" / "libzentorch_b200_torch.so"))
    m, k, n = 9, 512, 128
    x, q, s, z, b = make_woq_case(m, k, n, 128, seed=16)
    packed = torch.ops.zentorch.zentorch_woq_repack_weight(q.cuda())
    g = torch.Generator().manual_seed(17)
    a1 = torch.randn(m, n, generator=g).to(torch.bfloat16)
    a2 = torch.randn(m, n, generator=g).to(torch.bfloat16)
    pc = packed.cpu().t()
    vp = C.c_void_p

    def call(name, extra, post, bufs):
        """X, W, scales, no zero points, the binary operands, an optional bias passed by address."""
        hs = [aoti_handle(t) for t in (x.cuda(), packed.t(), s.cuda())]
        hextra = [aoti_handle(t.cuda()) for t in extra]
        hb = aoti_handle(b.cuda())
        bias_slot, ret = vp(hb[1]), vp(None)
        fn = getattr(lib, name)
        fn.restype = C.c_int32
        rc = fn(*(vp(a) for _, a in hs), None, *(vp(a) for _, a in hextra), C.byref(bias_slot), b"from_test", C.byref(ret))
        assert rc == 0, f"{name} returned {rc}"
        y = aoti_take(ret.value)
        for cap, _ in hs + hextra + [hb]:
            aoti_release(cap)
        assert_close_bf16(y, O.woq_linear(x, pc, s, None, b, post, bufs), what=name)

    call("aoti_torch_cuda_zentorch_woq_linear", [], [], [])
    call("aoti_torch_cuda_zentorch_woq_linear_gelu_tanh", [], [O.POST_GELU_TANH], [])
    call("aoti_torch_cuda_zentorch_woq_linear_add", [a1], [O.POST_ADD], [a1])
    call("aoti_torch_cuda_zentorch_woq_linear_mul_add", [a1, a2], [O.POST_MUL, O.POST_ADD], [a1, a2])
    call("aoti_torch_cuda_zentorch_woq_linear_add_add", [a1, a2], [O.POST_ADD, O.POST_ADD], [a1, a2])

    xi, wi, wsi, bi = make_int8_case(33, 256, 80, seed=18)
    hs = [aoti_handle(t.cuda()) for t in (xi, wi, wsi, bi)]
    bias_slot, ret = vp(hs[3][1]), vp(None)
    fn = lib.aoti_torch_cuda_zentorch_dynamic_qlinear
    fn.restype = C.c_int32
    assert fn(vp(hs[0][1]), vp(hs[1][1]), vp(hs[2][1]), C.byref(bias_slot), b"from_test", C.byref(ret)) == 0
    yi = aoti_take(ret.value)
    for cap, _ in hs:
        aoti_release(cap)
    assert_close_bf16(yi, O.dynamic_qlinear(xi, wi, wsi, bi), what="aoti dynamic_qlinear")
    # an invalid call comes back as a non-zero error code, not as an exception across the C boundary
    hs = [aoti_handle(t) for t in (xi.cuda(), wi.cuda().int(), wsi.cuda())]
    ret = vp(None)
    assert fn(vp(hs[0][1]), vp(hs[1][1]), vp(hs[2][1]), None, b"from_test", C.byref(ret)) != 0
    for cap, _ in hs:
        aoti_release(cap)


def test_rowsum_cache_follows_the_weight(ops):
    """The u8 mode keeps the weight's row sums with the boundary's record of the weight.  Repeated calls give the
    same result, and a weight that is modified in place (its version changes) or replaced by a new tensor at
    the same address gets fresh row sums."""
    x, w, ws, b = make_int8_case(48, 256, 64, seed=22)
    xd, wd, wsd, bd = x.cuda(), w.cuda(), ws.cuda(), b.cuda()
    ref = O.dynamic_qlinear(x, w, ws, b, act_quant="u8_asym")
    for _ in range(3):
        y = ops.zentorch_dynamic_qlinear_ext(xd, wd, wsd, bd, act_quant="u8_asym")
        assert_close_bf16(y, ref, what="u8 with cached row sums")
    w2 = w.clone()
    w2[::2] = -w2[::2]                                   # row sums change sign on every other row
    wd.copy_(w2.cuda())                                  # in place: same storage, new version
    ref2 = O.dynamic_qlinear(x, w2, ws, b, act_quant="u8_asym")
    assert_close_bf16(ops.zentorch_dynamic_qlinear_ext(xd, wd, wsd, bd, act_quant="u8_asym"), ref2, what="after in-place update")
    del wd
    w3 = torch.roll(w, 1, 0).cuda()                      # very likely the same address, a new storage
    ref3 = O.dynamic_qlinear(x, w3.cpu(), ws, b, act_quant="u8_asym")
    assert_close_bf16(ops.zentorch_dynamic_qlinear_ext(xd, w3, wsd, bd, act_quant="u8_asym"), ref3, what="new tensor")


def test_expired_device_wait_is_reported_and_cleared(zt):
    """A kernel whose bounded wait gives up (a barrier nobody signals, a few thousand polls) sets the device
    status word and returns; the host reads the code, clearing it also re-zeroes the split-K counters of the
    cached workspaces, and the context stays usable."""
    from zentorch_b200 import _capi
    dev = torch.device("cuda", torch.cuda.current_device())
    ws = _capi.woq_workspace(1 << 20, dev)
    ws[:8].fill_(1)                                     # pretend a kernel that gave up left a counter behind
    _capi.check(_capi.lib().zt_selftest_expire_wait(None))
    torch.cuda.synchronize()
    assert _capi.poll_device_status(reset=True) == 199
    assert _capi.poll_device_status(reset=True) == 0
    assert int(ws[:_capi.ZT_WOQ_COUNTER_BYTES].sum()) == 0
    x, q, s, z, b = make_woq_case(1, 4096, 1024, 128, seed=19)     # a split-K shape works right after
    y = _capi.woq_linear(x.cuda(), _capi.woq_repack_weight(q.cuda()), s.cuda(), None, b.cuda())
    assert_close_bf16(y, O.woq_linear(x, O.woq_repack_weight(q).t(), s, None, b))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs in one process")
def test_one_process_two_devices(ops):
    """Per-device kernel attributes: the same process runs both linears on cuda:0 and then on cuda:1."""
    x, q, s, z, b = make_woq_case(40, 1024, 256, 128, seed=20)
    ref = O.woq_linear(x, O.woq_repack_weight(q).t(), s, None, b)
    xi, wi, wsi, bi = make_int8_case(130, 512, 192, seed=21)
    refi = O.dynamic_qlinear(xi, wi, wsi, bi)
    for d in (0, 1):
        dev = torch.device("cuda", d)
        with torch.cuda.device(dev):
            packed = ops.zentorch_woq_repack_weight(q.to(dev))
            for m in (40, 2):
                y = ops.zentorch_woq_linear(x[:m].to(dev), packed.t(), s.to(dev), None, b.to(dev))
                assert_close_bf16(y, ref[:m], what=f"woq on cuda:{d} M={m}")
            yi = ops.zentorch_dynamic_qlinear(xi.to(dev), wi.to(dev), wsi.to(dev), bi.to(dev))
            assert_close_bf16(yi, refi, what=f"int8 on cuda:{d}")
            torch.cuda.synchronize(dev)
