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


# ---- horizontal fusion of sibling weight-only linears (opt-in pass) ------------------------------------------
class _OracleInterpreter(torch.fx.Interpreter):
    """Runs an FX graph on CPU tensors with the zentorch operators evaluated by the CPU oracle."""

    def call_function(self, target, args, kwargs):
        import zentorch_oracle as O
        if target == torch.ops.zentorch.zentorch_woq_repack_weight.default:
            return O.woq_repack_weight(args[0])
        if target == torch.ops.zentorch.zentorch_woq_linear.default:
            x, w, s, z, b = (list(args) + [None] * 5)[:5]
            return O.woq_linear(x, w, s, z, b)
        return super().call_function(target, args, kwargs)


def _qkv_graph(bias: bool, groups: int = 2):
    g = torch.Generator().manual_seed(3)
    k, ns = 128, (64, 32, 32)
    x = torch.randn(5, k, generator=g).to(torch.bfloat16)
    params = []
    for n in ns:
        q = torch.randint(-8, 8, (n, k), generator=g, dtype=torch.int8)
        s = (torch.rand(groups, n, generator=g) * 0.05 + 0.01)
        b = torch.randn(n, generator=g).to(torch.bfloat16) if bias else None
        params += [q, s] + ([b] if bias else [])

    def fn(x, *p):
        step = 3 if bias else 2
        outs = []
        for i in range(3):
            q, s = p[step * i], p[step * i + 1]
            b = p[step * i + 2] if bias else None
            w = torch.ops.zentorch.zentorch_woq_repack_weight(q).t()
            outs.append(torch.ops.zentorch.zentorch_woq_linear(x, w, s, None, b))
        return outs[0].float().sum(-1, keepdim=True) + outs[1].float().mean(-1, keepdim=True), outs[2] * 2

    return fn, (x, *params)


@pytest.mark.parametrize("bias", [False, True])
def test_parallel_woq_linears_fuse_into_one(comp, bias):
    fn, args = _qkv_graph(bias)
    gm = _trace(fn, *args)
    before = _OracleInterpreter(gm).run(*args)
    assert _targets(gm).count(torch.ops.zentorch.zentorch_woq_linear.default) == 3
    assert comp.fuse_parallel_woq_linears(gm.graph) == 1
    gm.recompile()
    t = _targets(gm)
    assert t.count(torch.ops.zentorch.zentorch_woq_linear.default) == 1
    assert comp.counters["zentorch"]["fused_parallel_woq_linear"] == 1
    lin = next(n for n in gm.graph.nodes if n.target == torch.ops.zentorch.zentorch_woq_linear.default)
    # the fused weight keeps the layout contract: [K/8, sum N] with strides (1, K/8); scales [groups, sum N]
    assert tuple(lin.args[1].meta["val"].shape) == (16, 128) and tuple(lin.args[1].meta["val"].stride()) == (1, 16)
    assert tuple(lin.args[2].meta["val"].shape) == (2, 128)
    assert (lin.args[4] is None) == (not bias)
    assert tuple(lin.meta["val"].shape) == (5, 128)
    after = _OracleInterpreter(gm).run(*args)
    for a, b in zip(before, after):
        assert torch.equal(a, b)           # the same columns computed by the same arithmetic


def test_parallel_woq_linears_left_alone_when_they_differ(comp):
    g = torch.Generator().manual_seed(4)
    x = torch.randn(3, 64, generator=g).to(torch.bfloat16)
    q1 = torch.randint(-8, 8, (32, 64), generator=g, dtype=torch.int8)
    q2 = torch.randint(0, 16, (32, 64), generator=g, dtype=torch.int8)
    s1, s2 = torch.rand(1, 32, generator=g), torch.rand(2, 32, generator=g)
    z2 = torch.rand(2, 32, generator=g)

    def fn(x, q1, s1, q2, s2, z2):
        a = torch.ops.zentorch.zentorch_woq_linear(x, torch.ops.zentorch.zentorch_woq_repack_weight(q1).t(), s1, None)
        b = torch.ops.zentorch.zentorch_woq_linear(x, torch.ops.zentorch.zentorch_woq_repack_weight(q2).t(), s2, z2)
        return a, b

    gm = _trace(fn, x, q1, s1, q2, s2, z2)
    assert comp.fuse_parallel_woq_linears(gm.graph) == 0      # different group counts and zero-point presence
    assert _targets(gm).count(torch.ops.zentorch.zentorch_woq_linear.default) == 2

    def chained(x, q1, s1):
        w = torch.ops.zentorch.zentorch_woq_repack_weight(q1).t()
        a = torch.ops.zentorch.zentorch_woq_linear(x, w, s1, None)
        b = torch.ops.zentorch.zentorch_woq_linear(x, w, s1, None, a[0, :32].contiguous())   # bias from the sibling
        return a, b

    q3 = torch.randint(-8, 8, (64, 64), generator=g, dtype=torch.int8)
    gm = _trace(chained, x, q3, torch.rand(1, 64, generator=g))
    assert comp.fuse_parallel_woq_linears(gm.graph) == 0      # one depends on the other
