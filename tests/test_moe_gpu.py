"""Int4 mixture-of-experts FFN on a B200 against the CPU oracle (composition of the pinned WOQ linear;
the reference has no int4 MoE, so parity of the composition is unpinned)."""
import pytest
import torch

import zentorch_oracle as O
from _util import assert_close_bf16

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def capi(zt):
    from zentorch_b200 import _capi
    assert torch.cuda.is_available() and _capi.lib().zt_device_supported() == 1
    return _capi


def make_moe(t, h, inter, e, gs, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(t, h, generator=g).to(torch.bfloat16)
    logits = torch.randn(t, e, generator=g)
    w13q, s13, w2q, s2 = [], [], [], []
    for _ in range(e):
        q, s = O.quantize_woq_sym(torch.randn(2 * inter, h, generator=g) * 0.02, gs)
        w13q.append(q)
        s13.append(s)
        q, s = O.quantize_woq_sym(torch.randn(h, inter, generator=g) * 0.02, gs)
        w2q.append(q)
        s2.append(s)
    return x, logits, w13q, s13, w2q, s2


def run_gpu(capi, x, tw, ids, w13q, s13, w2q, s2):
    dev = "cuda"
    w13 = torch.stack([capi.woq_repack_weight(q.to(dev)) for q in w13q])
    w2 = torch.stack([capi.woq_repack_weight(q.to(dev)) for q in w2q])
    return capi.moe_woq(x.to(dev), tw.to(dev).contiguous(), ids.to(dev).contiguous(), w13,
                        torch.stack(s13).to(dev), w2, torch.stack(s2).to(dev)).cpu()


@pytest.mark.parametrize("t,h,inter,e,k", [(64, 256, 512, 8, 2), (5, 128, 192, 4, 1), (300, 512, 256, 8, 2),
                                           (17, 256, 128, 16, 4)])
def test_moe_vs_oracle(capi, t, h, inter, e, k):
    x, logits, w13q, s13, w2q, s2 = make_moe(t, h, inter, e, 64, seed=t)
    tw, ids = O.route_top2(logits, k)
    y = run_gpu(capi, x, tw, ids, w13q, s13, w2q, s2)
    ref = O.moe_woq(x, tw, ids, [O.woq_repack_weight(q).t() for q in w13q], s13,
                    [O.woq_repack_weight(q).t() for q in w2q], s2)
    assert_close_bf16(y, ref, rtol=2e-2, atol=2e-2, what=f"moe T={t}")


def test_moe_skipped_and_empty_experts(capi):
    """Ids outside [0, E) are skipped (tokens of another expert-parallel rank); experts may be empty."""
    t, h, inter, e = 40, 256, 256, 8
    x, logits, w13q, s13, w2q, s2 = make_moe(t, h, inter, e, 128, seed=9)
    tw, ids = O.route_top2(logits, 2)
    ids[ids == 3] = 5            # expert 3 gets no tokens
    ids[::7, 1] = -1             # some slots belong to a remote rank
    y = run_gpu(capi, x, tw, ids, w13q, s13, w2q, s2)
    ref = O.moe_woq(x, tw, ids, [O.woq_repack_weight(q).t() for q in w13q], s13,
                    [O.woq_repack_weight(q).t() for q in w2q], s2)
    assert_close_bf16(y, ref, rtol=2e-2, atol=2e-2, what="moe with skipped slots")


def test_moe_config4_properties(capi):
    """BASELINE config 4 at full size (8 experts, top-2, 256 tokens, H=4096, I=14336) through size-independent
    properties: permuting the tokens permutes the outputs, and the tokens routed only to experts {0, 1}
    match the oracle evaluated for those two experts."""
    t, h, inter, e = 256, 4096, 14336, 8
    g = torch.Generator().manual_seed(0)
    x = torch.randn(t, h, generator=g).to(torch.bfloat16)
    logits = torch.randn(t, e, generator=g)
    logits[:6, :2] += 8.0                                  # make sure a few tokens use experts 0 and 1 only
    tw, ids = O.route_top2(logits, 2)
    dev = "cuda"
    w13, s13, w2, s2, keep = [], [], [], [], {}
    for ei in range(e):
        q13, sc13 = O.quantize_woq_sym(torch.randn(2 * inter, h, generator=g) * 0.02, 128)
        q2, sc2 = O.quantize_woq_sym(torch.randn(h, inter, generator=g) * 0.02, 128)
        w13.append(capi.woq_repack_weight(q13.to(dev)))
        w2.append(capi.woq_repack_weight(q2.to(dev)))
        s13.append(sc13.to(dev))
        s2.append(sc2.to(dev))
        if ei < 2:
            keep[ei] = (q13, sc13, q2, sc2)
    w13, w2, s13, s2 = torch.stack(w13), torch.stack(w2), torch.stack(s13), torch.stack(s2)
    y = capi.moe_woq(x.to(dev), tw.to(dev), ids.to(dev), w13, s13, w2, s2).cpu()
    perm = torch.randperm(t, generator=g)
    y_perm = capi.moe_woq(x[perm].to(dev), tw[perm].to(dev).contiguous(), ids[perm].to(dev).contiguous(), w13, s13, w2,
                          s2).cpu()
    assert torch.equal(y_perm, y[perm])
    sel = torch.nonzero((ids < 2).all(dim=1)).flatten()
    assert sel.numel() >= 6
    sel = sel[:8]
    out = torch.zeros(sel.numel(), h)
    for ei, (q13, sc13, q2, sc2) in keep.items():
        hh = x[sel].float() @ O.woq_dequant(q13, sc13, None).t()
        a = (torch.nn.functional.silu(hh[:, :inter]) * hh[:, inter:]).to(torch.bfloat16)
        o = a.float() @ O.woq_dequant(q2, sc2, None).t()
        wsel = (tw[sel] * (ids[sel] == ei)).sum(dim=1, keepdim=True)
        out += o * wsel
    assert_close_bf16(y[sel], out.to(torch.bfloat16), rtol=2e-2, atol=2e-2, what="config 4 sample tokens")
