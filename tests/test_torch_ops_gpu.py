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
