"""Parity of the dynamic int8 path on a B200 against the CPU oracle, through the C ABI.
Quantised activations, scales, zero points and int32 accumulators are compared bit for bit; final
outputs within 1e-2 relative (bf16) or 1e-4 (fp32)."""
import pytest
import torch

import zentorch_oracle as O
from _util import assert_close_bf16, make_int8_case

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def capi(zt):
    from zentorch_b200 import _capi
    assert torch.cuda.is_available() and _capi.lib().zt_device_supported() == 1
    return _capi


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("m,k", [(1, 4), (3, 12), (7, 16), (5, 100), (33, 4096), (4, 8192), (2, 28672), (3, 10248)])
def test_dynamic_quantize_bit_exact(capi, dtype, m, k):
    g = torch.Generator().manual_seed(m + k)
    x = (torch.randn(m, k, generator=g) * 3).to(dtype)
    x[0, 0] = 0.5  # an exact tie candidate after scaling is likely somewhere; also test zero row below
    if m > 1:
        x[1].zero_()
    q, s, _ = capi.dynamic_quantize(x.cuda(), capi.ZT_ACT_S8_SYM)
    q_ref, s_ref = O.dynamic_quantize_s8(x)
    assert torch.equal(s.cpu(), s_ref) and torch.equal(q.cpu(), q_ref)
    qu, su, zpu = capi.dynamic_quantize(x.cuda(), capi.ZT_ACT_U8_ASYM)
    qu_ref, su_ref, zp_ref = O.dynamic_quantize_u8(x)
    assert torch.equal(su.cpu(), su_ref) and torch.equal(zpu.cpu(), zp_ref) and torch.equal(qu.cpu(), qu_ref)


def test_dynamic_quantize_nan_and_signed_zero(capi):
    """A NaN makes its own row's scale NaN (the CPU formula's amax propagates it) and with it the whole output
    row of the linear; the other rows keep their exact bytes.  A row of -0.0 quantises like a row of zeros."""
    g = torch.Generator().manual_seed(11)
    m, k, n = 6, 512, 48
    x = (torch.randn(m, k, generator=g) * 2).to(torch.bfloat16)
    x[2, 77] = float("nan")
    x[4] = -0.0
    w = torch.randint(-127, 128, (n, k), generator=g, dtype=torch.int8)
    ws = torch.rand(n, generator=g) * 1e-3 + 1e-4
    for act in (capi.ZT_ACT_S8_SYM, capi.ZT_ACT_U8_ASYM):
        q, s, zp = capi.dynamic_quantize(x.cuda(), act)
        if act == capi.ZT_ACT_S8_SYM:
            q_ref, s_ref = O.dynamic_quantize_s8(x)
            zp_ref = torch.zeros(m, dtype=torch.int32)
        else:
            q_ref, s_ref, zp_ref = O.dynamic_quantize_u8(x)
        assert torch.isnan(s_ref[2]) and torch.isnan(s.cpu()[2])
        keep = [0, 1, 3, 4, 5]
        assert torch.equal(s.cpu()[keep], s_ref[keep]) and torch.equal(q.cpu()[keep], q_ref[keep])
        if act == capi.ZT_ACT_U8_ASYM:
            assert torch.equal(zp.cpu()[keep], zp_ref[keep])
        assert float(s.cpu()[4]) == float(s_ref[4]) and not torch.signbit(s.cpu()[4])
        y = capi.dynamic_qlinear(x.cuda(), w.cuda(), ws.cuda(), None, act_quant=act).float().cpu()
        assert torch.isnan(y[2]).all() and torch.isfinite(y[keep]).all()
        assert (y[4] == 0).all()


TILES = [0, 64, 96, 128, 160, 192, 224, 256, 1128, 1160, 1192, 1256]  # +1000: 256-row CTA tiles


@pytest.mark.parametrize("tile", TILES)
def test_int8_accumulators_bit_exact_tcgen05(capi, tile):
    g = torch.Generator().manual_seed(tile)
    for (m, n, k) in ((128, 256, 128), (130, 200, 144), (1, 40, 16), (257, 523, 400), (64, 1024, 4096)):
        q = torch.randint(-128, 128, (m, k), generator=g, dtype=torch.int8)
        w = torch.randint(-128, 128, (n, k), generator=g, dtype=torch.int8)
        algo = capi.ZT_ALGO_TCGEN05 | (tile << 8)
        acc = capi.int8_gemm_s32(q.cuda(), w.cuda(), algo=algo).cpu()
        assert torch.equal(acc, O.int_gemm(q, w)), f"tile {tile} shape {(m, n, k)}"
    qu = torch.randint(0, 256, (70, 272), generator=g, dtype=torch.uint8)
    w = torch.randint(-128, 128, (90, 272), generator=g, dtype=torch.int8)
    accu = capi.int8_gemm_s32(qu.cuda(), w.cuda(), algo=capi.ZT_ALGO_TCGEN05 | (tile << 8)).cpu()
    assert torch.equal(accu, (qu.long() @ w.long().t()).to(torch.int32))


def test_int8_accumulators_bit_exact_generic(capi):
    g = torch.Generator().manual_seed(1)
    for (m, n, k) in ((5, 7, 4), (6, 10, 12), (3, 9, 13), (40, 33, 260)):
        q = torch.randint(-128, 128, (m, k), generator=g, dtype=torch.int8)
        w = torch.randint(-128, 128, (n, k), generator=g, dtype=torch.int8)
        acc = capi.int8_gemm_s32(q.cuda(), w.cuda(), algo=capi.ZT_ALGO_GENERIC).cpu()
        assert torch.equal(acc, (q.long() @ w.long().t()).to(torch.int32))
        acc = capi.int8_gemm_s32(q.cuda(), w.cuda(), algo=capi.ZT_ALGO_AUTO).cpu()
        assert torch.equal(acc, (q.long() @ w.long().t()).to(torch.int32))


def test_reference_op_test_grid(capi):
    """Shapes and formula of test/unittests/op_tests/test_dynamic_qlinear.py: fp32 input, K in
    {4,8,12,16}, N in 2..10, scales 1+|randn|, optional fp32 bias; tolerance 1e-2 there, 1e-4 here."""
    g = torch.Generator().manual_seed(0)
    for k in (4, 8, 12, 16):
        for n in (2, 5, 10):
            for with_bias in (False, True):
                x = torch.randn(6, k, generator=g)
                w = torch.randint(-128, 127, (n, k), generator=g, dtype=torch.int8)
                ws = 1 + torch.randn(n, generator=g).abs()
                b = torch.randn(n, generator=g) if with_bias else None
                y = capi.dynamic_qlinear(x.cuda(), w.cuda(), ws.cuda(), None if b is None else b.cuda()).cpu()
                ref = O.dynamic_qlinear(x, w, ws, b)
                assert torch.allclose(y, ref, rtol=1e-4, atol=1e-4), (k, n, with_bias)


@pytest.mark.parametrize("x_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("act", ["s8_sym", "u8_asym"])
@pytest.mark.parametrize("post", ["none", "relu", "silu", "gelu_tanh", "gelu_erf"])
def test_dynamic_qlinear_outputs(capi, x_dtype, act, post):
    m, k, n = 150, 512, 328
    x, w, ws, b = make_int8_case(m, k, n, seed=4, x_dtype=x_dtype)
    ops = [] if post == "none" else [O.POST_NAMES[post]]
    mode = capi.ZT_ACT_U8_ASYM if act == "u8_asym" else capi.ZT_ACT_S8_SYM
    y = capi.dynamic_qlinear(x.cuda(), w.cuda(), ws.cuda(), b.cuda(), act_quant=mode, post_ops=ops).cpu()
    ref = O.dynamic_qlinear(x, w, ws, b, act_quant=act, post_ops=ops)
    if x_dtype == torch.float32:
        assert torch.allclose(y, ref, rtol=1e-4, atol=1e-4)
    else:
        assert_close_bf16(y, ref, what=f"{act}/{post}")


def test_config2_full_size(capi):
    """M=512, K=4096, N=11008, fp32 bias, fused SiLU, both activation modes: quantised bytes and
    accumulators bit-exact against the oracle, outputs within tolerance."""
    m, k, n = 512, 4096, 11008
    x, w, ws, b = make_int8_case(m, k, n, seed=0)
    xd, wd = x.cuda(), w.cuda()
    q, s, _ = capi.dynamic_quantize(xd, capi.ZT_ACT_S8_SYM)
    q_ref, s_ref, _, acc_ref, y_ref = O.dynamic_qlinear(x, w, ws, b, return_parts=True)
    assert torch.equal(q.cpu(), q_ref) and torch.equal(s.cpu(), s_ref)
    acc = capi.int8_gemm_s32(q, wd).cpu()
    assert torch.equal(acc, acc_ref)
    y = capi.dynamic_qlinear(xd, wd, ws.cuda(), b.cuda()).cpu()
    assert_close_bf16(y, y_ref, what="config 2, s8, no post-op")
    y_silu = capi.dynamic_qlinear(xd, wd, ws.cuda(), b.cuda(), act_quant=capi.ZT_ACT_U8_ASYM,
                                  post_ops=[O.POST_SILU]).cpu()
    ref_silu = O.dynamic_qlinear(x, w, ws, b, act_quant="u8_asym", post_ops=[O.POST_SILU])
    assert_close_bf16(y_silu, ref_silu, what="config 2, u8 + silu")


def test_full_size_checksum_70b(capi):
    """Llama-3-70B gate/up projection as int8 (K=8192, N=28672) at M=4096: the sum over n of the
    accumulators of a row equals q[m,:] . (sum_n W[n,:]) exactly, which needs no CPU GEMM."""
    m, k, n = 4096, 8192, 28672
    g = torch.Generator().manual_seed(3)
    q = torch.randint(-128, 128, (m, k), generator=g, dtype=torch.int8)
    w = torch.randint(-127, 128, (n, k), generator=g, dtype=torch.int8)
    acc = capi.int8_gemm_s32(q.cuda(), w.cuda())
    rows = acc.sum(dim=1, dtype=torch.int64).cpu()
    cols = acc.sum(dim=0, dtype=torch.int64).cpu()
    del acc
    w_colsum = w.sum(dim=0, dtype=torch.int64)
    q_colsum = q.sum(dim=0, dtype=torch.int64)
    assert torch.equal(rows, (q.double() @ w_colsum.double()).round().long())
    expect_cols = torch.cat([(w[i:i + 4096].double() @ q_colsum.double()).round().long() for i in range(0, n, 4096)])
    assert torch.equal(cols, expect_cols)


@pytest.mark.parametrize("bn", [128, 160, 192, 256])
def test_cta_pair_tiles_match_the_one_cta_kernel(capi, bn):
    """The tcgen05.mma.cta_group::2 form (two CTAs share every weight block): same int32 sums and the same fp32
    epilogue as the one-CTA kernel, so the outputs are identical bit for bit.  Ragged M (a last pair tile with
    one CTA partly or wholly past M), ragged N, K shorter than the ring, several tiles per CTA pair, both
    activation forms, a post-op chain with a binary operand."""
    cases = [(512, 4096, 1000, capi.ZT_ACT_U8_ASYM, (capi.ZT_POST_SILU,)), (600, 256, 3 * bn + 40, capi.ZT_ACT_S8_SYM, ()),
             (257, 144, 72, capi.ZT_ACT_U8_ASYM, ()), (1300, 1024, 75 * bn, capi.ZT_ACT_S8_SYM, (capi.ZT_POST_GELU_TANH,))]
    for (m, k, n, act, post) in cases:
        x, w, ws, b = [t.cuda() for t in make_int8_case(m, k, n, seed=m + n)]
        rowsum = capi.int8_weight_rowsum(w)
        expect = capi.dynamic_qlinear(x, w, ws, b, act_quant=act, post_ops=post, w_rowsum=rowsum)
        got = capi.dynamic_qlinear(x, w, ws, b, act_quant=act, post_ops=post, w_rowsum=rowsum,
                                   algo=capi.ZT_ALGO_TCGEN05 | ((2000 + bn) << 8))
        assert torch.equal(got, expect), f"pair tile {bn}: {(m, k, n)}"
    m, k, n = 700, 512, 2 * bn + 8
    x, w, ws, b = [t.cuda() for t in make_int8_case(m, k, n, seed=9)]
    add = torch.randn(m, n, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16).cuda()
    expect = capi.dynamic_qlinear(x, w, ws, b, post_ops=(capi.ZT_POST_ADD,), buffers=(add,))
    got = capi.dynamic_qlinear(x, w, ws, b, post_ops=(capi.ZT_POST_ADD,), buffers=(add,),
                               algo=capi.ZT_ALGO_TCGEN05 | ((2000 + bn) << 8))
    assert torch.equal(got, expect)
    ref = O.dynamic_qlinear(x.cpu(), w.cpu(), ws.cpu(), b.cpu(), post_ops=[O.POST_ADD], buffers=[add.cpu()])
    assert_close_bf16(got, ref, what=f"pair tile {bn} vs oracle")
