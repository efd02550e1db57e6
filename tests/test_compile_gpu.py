"""torch.compile(backend="zentorch_b200") on a CUDA module: the dequantise+matmul subgraphs of a
weight-only-quantised MLP are rewritten to the fused operators and the compiled result matches the
oracle.  Mirrors the reference's model-level WOQ tests (test/unittests/model_tests/test_woq_*.py)."""
import pytest
import torch

import zentorch_oracle as O
from _util import assert_close_bf16

pytestmark = pytest.mark.gpu


class DequantLinear(torch.nn.Module):
    """What a torchao int4 weight-only linear looks like to Inductor: int8-held nibbles, group scales."""

    def __init__(self, n, k, group, seed, bias=True):
        super().__init__()
        g = torch.Generator().manual_seed(seed)
        self.n, self.k = n, k
        self.w = torch.nn.Buffer(torch.randint(-8, 8, (n, k // group, group), generator=g, dtype=torch.int8))
        self.zp = torch.nn.Buffer(torch.zeros(n, k // group, 1, dtype=torch.int8))
        self.s = torch.nn.Buffer((torch.rand(n, k // group, 1, generator=g) * 0.02 + 0.005).to(torch.bfloat16))
        self.b = torch.nn.Buffer(torch.randn(n, generator=g).to(torch.bfloat16)) if bias else None

    def forward(self, x):
        dq = ((self.w.to(torch.bfloat16) - self.zp.to(torch.bfloat16)) * self.s).view(self.n, self.k)
        if self.b is not None:
            return torch.addmm(self.b, x, dq.permute(1, 0))
        return torch.mm(x, dq.permute(1, 0))

    def oracle(self, x, post=()):
        q = self.w.cpu().view(self.n, self.k)
        packed = O.woq_repack_weight(q)
        s = self.s.cpu().view(self.n, -1).t().contiguous()
        return O.woq_linear(x, packed.t(), s, None, None if self.b is None else self.b.cpu(), list(post))


class MLP(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.up = DequantLinear(512, 256, 128, 1)
        self.down = DequantLinear(256, 512, 128, 2, bias=False)

    def forward(self, x):
        return self.down(torch.nn.functional.gelu(self.up(x), approximate="tanh"))


def test_compiled_mlp_uses_fused_ops(zt):
    from zentorch_b200 import _compile
    zt.register_backend()
    _compile.counters.clear()
    torch._dynamo.reset()
    model = MLP().cuda()
    x = torch.randn(24, 256, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16)
    with torch.no_grad():
        y = torch.compile(model, backend="zentorch_b200")(x.cuda())
    assert _compile.counters["zentorch"]["zentorch_woq_linear"] == 2
    assert _compile.counters["zentorch"]["zentorch_woq_linear_gelu_tanh"] == 1
    h = model.up.oracle(x, [O.POST_GELU_TANH])
    assert_close_bf16(y, model.down.oracle(h))


class DynLinear(torch.nn.Module):
    """A dynamic-int8 linear calling the reference's operator directly (what the torchao / compressed-tensors
    handlers emit)."""

    def __init__(self, n, k, seed):
        super().__init__()
        from _util import make_int8_case
        _, w, ws, b = make_int8_case(1, k, n, seed=seed)
        self.w, self.ws, self.b = torch.nn.Buffer(w), torch.nn.Buffer(ws), torch.nn.Buffer(b)

    def forward(self, x):
        return torch.ops.zentorch.zentorch_dynamic_qlinear(x, self.w, self.ws, self.b)


@pytest.mark.parametrize("cpp_wrapper", [False, True])
def test_lowerings_python_and_cpp_wrapper(zt, cpp_wrapper, monkeypatch):
    """The operators lowered to extern kernels: the Python wrapper calls the overload, the C++ wrapper calls the
    aoti_torch_cuda_zentorch_* shims (the generated code is checked for the shim names, so this is the test
    that runs them from Inductor's own caller).  Also compiles through backend="zentorch"."""
    from zentorch_b200 import _compile
    from torch._inductor.utils import run_and_get_code
    zt.register_backend()
    _compile.counters.clear()
    torch._dynamo.reset()
    model = MLP().cuda()
    dyn = DynLinear(96, 256, seed=4).cuda()

    def fn(x):
        return dyn(torch.relu(model(x)))

    x = torch.randn(24, 256, generator=torch.Generator().manual_seed(5)).to(torch.bfloat16)
    options = {"cpp_wrapper": True} if cpp_wrapper else {}
    if cpp_wrapper:
        # Inductor builds its C++ wrapper with -fopenmp; where the compiler driver runs under another prefix it
        # does not find its own libgomp.spec unless the directory is on the library search path
        import glob
        import os
        specs = glob.glob("/usr/lib/gcc/x86_64-linux-gnu/*/libgomp.spec")
        if specs:
            extra = os.path.dirname(specs[0])
            monkeypatch.setenv("LIBRARY_PATH", extra + os.pathsep + os.environ.get("LIBRARY_PATH", ""))
    with torch.no_grad():
        y, codes = run_and_get_code(torch.compile(fn, backend="zentorch", options=options), x.cuda())
    code = "\n".join(codes)
    if cpp_wrapper:
        # the relu after the second linear is folded into it by the unary-fusion pass
        for shim in ("aoti_torch_cuda_zentorch_woq_linear_gelu_tanh", "aoti_torch_cuda_zentorch_woq_linear_relu",
                     "aoti_torch_cuda_zentorch_dynamic_qlinear"):
            assert shim in code, f"{shim} not called by the generated C++ wrapper"
    else:
        assert "zentorch_woq_linear" in code and "zentorch_dynamic_qlinear" in code
    h = model.up.oracle(x, [O.POST_GELU_TANH])
    h2 = torch.relu(model.down.oracle(h).float()).to(torch.bfloat16)
    ref = O.dynamic_qlinear(h2, dyn.w.cpu(), dyn.ws.cpu(), dyn.b.cpu())
    assert_close_bf16(y, ref, rtol=2e-2, atol=2e-2, frob=1e-2, what=f"compiled chain cpp_wrapper={cpp_wrapper}")
