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
