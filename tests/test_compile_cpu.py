"""The FX passes on CPU-traced ATen graphs (no kernel runs): dequantise+matmul subgraphs become
zentorch_woq_linear, element-wise consumers fold into the fused variants, counters are bumped."""
import pytest
import torch
from torch.fx.experimental.proxy_tensor import make_fx


def _trace(fn, *args):
    from torch._inductor.decomposition import select_decomp_table
    gm = make_fx(fn, decomposition_table=select_decomp_table(), tracing_mode="fake")(*args)
    gm.graph.eliminate_dead_code()   # Inductor hands its passes a graph without dead nodes
    return gm


def _targets(gm):
    return [n.target for n in gm.graph.nodes if n.op == "call_function"]


@pytest.fixture()
def comp(zt):
    from zentorch_b200 import _compile
    _compile.counters.clear()
    return _compile


def _inputs(n=32, k=64, m=4, groups=None):
    x = torch.randn(m, k, dtype=torch.bfloat16)
    if groups is None:
        w = torch.randint(-8, 8, (n, k), dtype=torch.int8)
        zp = torch.zeros(n, 1, dtype=torch.int8)
        s = torch.rand(n, 1, dtype=torch.bfloat16)
    else:
        w = torch.randint(-8, 8, (n, groups, k // groups), dtype=torch.int8)
        zp = torch.zeros(n, groups, 1, dtype=torch.int8)
        s = torch.rand(n, groups, 1, dtype=torch.bfloat16)
    return x, w, zp, s, torch.randn(n, dtype=torch.bfloat16)


def test_per_channel_patterns(comp):
    x, w, zp, s, b = _inputs()

    def no_bias(x, w, zp, s):
        dq = (w.to(torch.bfloat16) - zp.to(torch.bfloat16)) * s
        return torch.mm(x, dq.permute(1, 0))

    def with_bias(x, w, zp, s, b):
        dq = (w.to(torch.bfloat16) - zp.to(torch.bfloat16)) * s
        return torch.addmm(b, x, dq.permute(1, 0))

    for fn, args in ((no_bias, (x, w, zp, s)), (with_bias, (x, w, zp, s, b))):
        gm = _trace(fn, *args)
        comp.optimize(gm.graph, require_device=False)
        t = _targets(gm)
        assert torch.ops.zentorch.zentorch_woq_linear.default in t
        assert torch.ops.zentorch.zentorch_woq_repack_weight.default in t
        assert torch.ops.aten.mm.default not in t and torch.ops.aten.addmm.default not in t
    assert comp.counters["zentorch"]["zentorch_woq_linear"] == 2


def test_per_group_pattern_and_output_meta(comp):
    x, w, zp, s, b = _inputs(groups=2)

    def fn(x, w, zp, s, b):
        dq = ((w.to(torch.bfloat16) - zp.to(torch.bfloat16)) * s).view(32, 64)
        return torch.addmm(b, x, dq.permute(1, 0))

    gm = _trace(fn, x, w, zp, s, b)
    comp.optimize(gm.graph, require_device=False)
    lin = [n for n in gm.graph.nodes if n.target == torch.ops.zentorch.zentorch_woq_linear.default]
    assert len(lin) == 1
    # weight argument is the transposed view [K/8, N]; scales are [groups, N]
    assert tuple(lin[0].args[1].meta["val"].shape) == (8, 32)
    assert tuple(lin[0].args[1].meta["val"].stride()) == (1, 8)
    assert tuple(lin[0].args[2].meta["val"].shape) == (2, 32)
    assert tuple(lin[0].meta["val"].shape) == (4, 32)


def test_fusions(comp):
    x, w, zp, s, b = _inputs()
    a1, a2 = torch.randn(4, 32, dtype=torch.bfloat16), torch.randn(4, 32, dtype=torch.bfloat16)

    def lin(x, w, zp, s, b):
        dq = (w.to(torch.bfloat16) - zp.to(torch.bfloat16)) * s
        return torch.addmm(b, x, dq.permute(1, 0))

    cases = {
        "zentorch_woq_linear_relu": lambda x, w, zp, s, b, a1, a2: torch.relu(lin(x, w, zp, s, b)),
        "zentorch_woq_linear_add_add": lambda x, w, zp, s, b, a1, a2: lin(x, w, zp, s, b) + a1 + a2,
        "zentorch_woq_linear_mul_add": lambda x, w, zp, s, b, a1, a2: lin(x, w, zp, s, b) * a1 + a2,
        "zentorch_woq_linear_gelu_erf": lambda x, w, zp, s, b, a1, a2: torch.nn.functional.gelu(lin(x, w, zp, s, b)),
        "zentorch_woq_linear_gelu_tanh": lambda x, w, zp, s, b, a1, a2: torch.nn.functional.gelu(
            lin(x, w, zp, s, b), approximate="tanh"),
    }
    for name, fn in cases.items():
        gm = _trace(fn, x, w, zp, s, b, a1, a2)
        comp.optimize(gm.graph, require_device=False)
        t = _targets(gm)
        assert getattr(torch.ops.zentorch, name).default in t, (name, t)
        assert torch.ops.zentorch.zentorch_woq_linear.default not in t, name
        assert comp.counters["zentorch"][name] == 1


def test_gate_without_device(comp):
    x, w, zp, s, b = _inputs()

    def fn(x, w, zp, s):
        return torch.mm(x, ((w.to(torch.bfloat16) - zp.to(torch.bfloat16)) * s).permute(1, 0))

    gm = _trace(fn, x, w, zp, s)
    comp.optimize(gm.graph)   # no sm_100 device here: the graph is left alone
    if not torch.cuda.is_available():
        assert torch.ops.aten.mm.default in _targets(gm)
