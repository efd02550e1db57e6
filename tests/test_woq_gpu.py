"""Parity of the weight-only int4 path on a B200 against the CPU oracle, through the C ABI."""
import pytest
import torch

import zentorch_oracle as O
from _util import assert_close_bf16, bf16_from_bits, make_woq_case

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def capi(zt):
    from zentorch_b200 import _capi
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    assert _capi.lib().zt_device_supported() == 1, "GPU tests need an sm_100 device"
    return _capi


def _run(capi, x, q, scales, zeros, bias, algo, post_ops=(), buffers=()):
    dev = "cuda"
    packed = capi.woq_repack_weight(q.to(dev))                     # [N, K/8] on device
    y = capi.woq_linear(x.to(dev), packed, scales.to(dev), None if zeros is None else zeros.to(dev),
                        None if bias is None else bias.to(dev), post_ops, [b.to(dev) for b in buffers], algo=algo)
    torch.cuda.synchronize()
    return y.cpu(), packed.cpu()


POST_CASES = {  # used by the streaming-kernel and the tensor-core-kernel tests
    "relu": ([O.POST_RELU], 0), "sigmoid": ([O.POST_SIGMOID], 0), "gelu_tanh": ([O.POST_GELU_TANH], 0),
    "gelu_erf": ([O.POST_GELU_ERF], 0), "silu": ([O.POST_SILU], 0), "tanh": ([O.POST_TANH], 0),
    "add": ([O.POST_ADD], 1), "mul_add": ([O.POST_MUL, O.POST_ADD], 2), "add_add": ([O.POST_ADD, O.POST_ADD], 2),
}


# ---- repack ops: bit-exact -------------------------------------------------------------------------
def test_repack_weight_bit_exact(capi, golden):
    for key in ("pack", "packu"):
        w = torch.from_numpy(golden[f"{key}_in"])
        got = capi.woq_repack_weight(w.cuda()).cpu()
        assert torch.equal(got, torch.from_numpy(golden[f"{key}_out"]))
    g = torch.Generator().manual_seed(5)
    for n, k in ((1, 8), (3, 24), (48, 128), (1024, 4096)):
        w = torch.randint(-8, 8, (n, k), generator=g, dtype=torch.int8)
        assert torch.equal(capi.woq_repack_weight(w.cuda()).cpu(), O.woq_repack_weight(w))
    with pytest.raises(capi.ZtError, match="K must be divisible by 8"):
        capi.woq_repack_weight(torch.zeros(4, 12, dtype=torch.int8, device="cuda"))
    with pytest.raises(capi.ZtError, match="K must be at least 8"):
        capi.woq_repack_weight(torch.zeros(4, 4, dtype=torch.int8, device="cuda"))


def test_repack_from_int4pack_bit_exact(capi, golden):
    packed = torch.from_numpy(golden["int4pack_packed"])
    expect = O.woq_repack_weight(torch.from_numpy(golden["int4pack_int_data"]))
    assert torch.equal(capi.woq_repack_from_int4pack(packed.cuda()).cpu(), expect)
    int_data = torch.randint(0, 16, (192, 1024), dtype=torch.int32)
    p = torch.ops.aten._convert_weight_to_int4pack_for_cpu(int_data, 1)
    assert torch.equal(capi.woq_repack_from_int4pack(p.cuda()).cpu(), O.woq_repack_weight(int_data.to(torch.int8)))
    with pytest.raises(capi.ZtError, match="multiple of 64"):
        capi.woq_repack_from_int4pack(torch.zeros(32, 16, dtype=torch.uint8, device="cuda"))


# ---- the reference's own test grid: per-channel symmetric, tiny shapes (generic kernel) --------------------
@pytest.mark.parametrize("n", [32, 48, 64])
@pytest.mark.parametrize("k", [32, 64, 128])
@pytest.mark.parametrize("m", [1, 4, 24])
def test_reference_grid_per_channel(capi, m, k, n):
    g = torch.Generator().manual_seed(m * 1000 + k + n)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16)
    w = torch.randn(n, k, generator=g).to(torch.bfloat16)
    s = torch.clamp(w.abs().max(dim=1, keepdim=True)[0] / 8, min=1e-8).float()
    q = torch.clamp(torch.round(w / s), -8, 7).to(torch.int8)
    bias = torch.randn(n, generator=g).to(torch.bfloat16)
    scales = s.t().contiguous()
    y, packed = _run(capi, x, q, scales, None, bias, capi.ZT_ALGO_AUTO)
    ref = O.woq_linear(x, packed.t(), scales, None, bias)
    # reference tolerance rtol = atol = 1e-3, or the same value up to one bf16 rounding step
    close = torch.isclose(y.float(), ref.float(), rtol=1e-3, atol=1e-3)
    one_ulp = (y.view(torch.int16).int() - ref.view(torch.int16).int()).abs() <= 1
    assert (close | one_ulp).all()


def test_golden_fixture_through_capi(capi, golden):
    x = bf16_from_bits(golden["sym_x"]).reshape(-1, 128)
    q = torch.from_numpy(golden["sym_q"])
    scale = torch.from_numpy(golden["sym_scale"])
    bias = bf16_from_bits(golden["sym_bias"])
    y, _ = _run(capi, x, q, scale, None, bias, capi.ZT_ALGO_AUTO)
    ref = bf16_from_bits(golden["sym_y"]).reshape(-1, 48)
    one_ulp = (y.view(torch.int16).int() - ref.view(torch.int16).int()).abs() <= 1
    assert (torch.isclose(y.float(), ref.float(), rtol=1e-3, atol=1e-3) | one_ulp).all()
    # asymmetric fixture (truth: aten._weight_int4pack_mm_for_cpu); reference tolerance 0.1 / 2.0
    xa = bf16_from_bits(golden["asym_x"])
    packed = capi.woq_repack_from_int4pack(torch.from_numpy(golden["asym_int4pack"]).cuda())
    sa, za = bf16_from_bits(golden["asym_scale"]), bf16_from_bits(golden["asym_zero"])
    for algo in (capi.ZT_ALGO_GENERIC, capi.ZT_ALGO_SKINNY):
        ya = capi.woq_linear(xa.cuda(), packed, sa.cuda(), za.cuda(), None, algo=algo).cpu()
        refa = bf16_from_bits(golden["asym_y"])
        assert torch.allclose(ya.float(), refa.float(), rtol=0.1, atol=2.0)
        assert (ya.float() - refa.float()).abs().max() < 0.05


# ---- streaming kernel: every M 1..17, group sizes, asymmetric, scale dtypes, ragged N ------------------------
@pytest.mark.parametrize("m", list(range(1, 18)) + [31, 32, 33, 64])
def test_skinny_every_m(capi, m):
    x, q, s, z, b = make_woq_case(m, 512, 96, 128, seed=m)
    y, packed = _run(capi, x, q, s, None, b, capi.ZT_ALGO_SKINNY)
    assert_close_bf16(y, O.woq_linear(x, packed.t(), s, None, b), what=f"skinny M={m}")
    # against the exact (un-rounded dq) product the kernel is much tighter than the tolerance
    exact = O.woq_linear(x, packed.t(), s, None, b, dq_round=None)
    assert_close_bf16(y, exact, rtol=8e-3, atol=4e-3, what=f"skinny M={m} vs exact")


@pytest.mark.parametrize("asym", [False, True])
@pytest.mark.parametrize("scale_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("k,gs,n", [(256, 128, 40), (1024, 256, 100), (2048, 2048, 33), (4096, 128, 1024)])
def test_skinny_quant_modes(capi, asym, scale_dtype, k, gs, n):
    x, q, s, z, b = make_woq_case(5, k, n, gs, seed=k + n, asym=asym, scale_dtype=scale_dtype)
    for algo in (capi.ZT_ALGO_SKINNY, capi.ZT_ALGO_GENERIC):
        y, packed = _run(capi, x, q, s, z, b, algo)
        assert_close_bf16(y, O.woq_linear(x, packed.t(), s, z, b), what=f"algo {algo}")


@pytest.mark.parametrize("cfg", [0, 1, 2])
@pytest.mark.parametrize("m", [1, 7, 13, 16])
def test_stream_kernel_shapes(capi, cfg, m, monkeypatch):
    """Every compiled shape of the decode kernel (16 / 32 / 64 columns per CTA), with and without a
    K split across CTAs, ragged N, a K that is not a multiple of the activation chunk."""
    monkeypatch.setenv("ZENTORCH_B200_WOQ_STREAM_CFG", str(cfg))
    for (k, n, gs, asym, sdt) in ((4096, 200, 128, False, torch.float32), (1152, 1000, 128, True, torch.bfloat16),
                                  (8192, 72, 256, False, torch.bfloat16), (2048, 4100, 128, True, torch.float32),
                                  (4096, 1024, 128, False, torch.float32)):   # eight K slices in one cluster
        x, q, s, z, b = make_woq_case(m, k, n, gs, seed=cfg * 100 + m, asym=asym, scale_dtype=sdt)
        y, packed = _run(capi, x, q, s, z, b, capi.ZT_ALGO_SKINNY | (1 << 8))   # hint 1: register-ring kernel
        assert_close_bf16(y, O.woq_linear(x, packed.t(), s, z, b), what=f"cfg {cfg} M={m} K={k} N={n}")
        exact = O.woq_linear(x, packed.t(), s, z, b, dq_round=None)
        assert_close_bf16(y, exact, rtol=8e-3, atol=4e-3, what=f"cfg {cfg} M={m} K={k} N={n} vs exact")


@pytest.mark.parametrize("m", [1, 2, 3, 4])
def test_streamk_kernel(capi, m):
    """The work-balanced decode kernel: column tiles shared between CTAs (small N, long K), ragged N,
    both quantisation forms and scale dtypes; run twice to check that the arrival counters reset."""
    cases = ((4096, 64, 128, False, torch.float32), (28672, 192, 128, False, torch.float32),
             (8192, 1000, 256, True, torch.float32), (1024, 4104, 128, True, torch.bfloat16),
             (4096, 4096, 4096, False, torch.bfloat16), (14336, 136, 128, False, torch.float32),
             (7168, 4096, 256, True, torch.float32))   # many chunks per CTA: the stage ring wraps several times
    for (k, n, gs, asym, sdt) in cases:
        x, q, s, z, b = make_woq_case(m, k, n, gs, seed=m * 7 + n, asym=asym, scale_dtype=sdt)
        ref = O.woq_linear(x, O.woq_repack_weight(q).t(), s, z, b)
        exact = O.woq_linear(x, O.woq_repack_weight(q).t(), s, z, b, dq_round=None)
        for rep in range(2):
            y, _ = _run(capi, x, q, s, z, b, capi.ZT_ALGO_SKINNY | (2 << 8))   # hint 2: stream-K kernel
            assert_close_bf16(y, ref, what=f"stream-K M={m} K={k} N={n} rep {rep}")
            assert_close_bf16(y, exact, rtol=8e-3, atol=4e-3, what=f"stream-K M={m} K={k} N={n} vs exact")


def test_generic_odd_shapes(capi):
    for (m, k, n, gs) in ((3, 24, 7, 8), (2, 64, 5, 32), (9, 136, 17, 136), (1, 8, 1, 8)):
        x, q, s, z, b = make_woq_case(m, k, n, gs, seed=k)
        y, packed = _run(capi, x, q, s, None, b, capi.ZT_ALGO_AUTO)
        assert_close_bf16(y, O.woq_linear(x, packed.t(), s, None, b), what=f"{m}x{k}x{n}")




@pytest.mark.parametrize("name", sorted(POST_CASES))
@pytest.mark.parametrize("algo_name", ["SKINNY", "GENERIC"])
def test_post_ops(capi, name, algo_name):
    ops, nbuf = POST_CASES[name]
    m, k, n = 6, 256, 72
    x, q, s, z, b = make_woq_case(m, k, n, 128, seed=3)
    g = torch.Generator().manual_seed(9)
    bufs = [torch.randn(m, n, generator=g).to(torch.bfloat16) for _ in range(nbuf)]
    y, packed = _run(capi, x, q, s, None, b, getattr(capi, f"ZT_ALGO_{algo_name}"), ops, bufs)
    assert_close_bf16(y, O.woq_linear(x, packed.t(), s, None, b, ops, bufs), what=name)


# ---- tensor-core kernel (M > 16): every token-tile width, ragged M / N, both quantisation forms ------------
@pytest.mark.parametrize("tile", [0, 32, 64, 128, 256])
@pytest.mark.parametrize("asym,scale_dtype", [(False, torch.float32), (False, torch.bfloat16), (True, torch.float32),
                                              (True, torch.bfloat16)])
def test_tcgen05_kernel(capi, tile, asym, scale_dtype):
    # K = 128, 320, 448: packed-weight chunks of four k-blocks that end in a partial chunk
    for (m, k, n, gs) in ((17, 256, 128, 128), (100, 512, 200, 64), (300, 1024, 136, 128), (64, 128, 8, 32),
                          (257, 2048, 384, 2048), (40, 320, 72, 32), (129, 448, 260, 64),
                          (64, 1024, 256, 128), (200, 2048, 136, 64)):   # few tiles, long K: split over K when tile == 0
        x, q, s, z, b = make_woq_case(m, k, n, gs, seed=m + n, asym=asym, scale_dtype=scale_dtype)
        algo = capi.ZT_ALGO_TCGEN05 | (tile << 8)
        y, packed = _run(capi, x, q, s, z, b, algo)
        ref = O.woq_linear(x, packed.t(), s, z, b)
        assert_close_bf16(y, ref, what=f"tcgen05 tile={tile} {m}x{k}x{n} gs={gs}")
        # this kernel rounds dq to bf16 like the oracle: agreement is much tighter than the tolerance
        tight = 1.5e-2 if asym else 8e-3
        assert (y.float() - ref.float()).abs().max() <= tight * max(1.0, float(ref.float().abs().max())), (m, k, n)


@pytest.mark.parametrize("m,k,n", [(40, 128, 136), (33, 192, 128), (64, 4096, 256), (128, 1024, 384), (300, 2048, 200)])
def test_tcgen05_one_and_two_issuers_agree(capi, m, k, n):
    """The kernel's default form has two MMA issuers, each summing every other k-block into an accumulator of
    its own (the epilogue adds them); the one-issuer form sums all k-blocks in order.  Both against the oracle,
    and against each other to fp32 summation-order noise (K = 192: three k-blocks, the issuers swap parity from
    tile to tile)."""
    x, q, s, z, b = make_woq_case(m, k, n, 64, seed=k + n)
    y2, packed = _run(capi, x, q, s, None, b, capi.ZT_ALGO_TCGEN05)
    y1, _ = _run(capi, x, q, s, None, b, capi.ZT_ALGO_TCGEN05 | capi.ZT_ALGO_SINGLE_ISSUER)
    ref = O.woq_linear(x, packed.t(), s, None, b)
    assert_close_bf16(y2, ref, what=f"two issuers {m}x{k}x{n}")
    assert_close_bf16(y1, ref, what=f"one issuer {m}x{k}x{n}")
    # the two forms round one fp32 sum differently: at most one bf16 ulp apart, and mostly equal
    d = (y1.float() - y2.float()).abs()
    assert float(d.max()) <= 2 ** -7 * max(1.0, float(ref.float().abs().max()))
    assert float((d == 0).float().mean()) > 0.9


@pytest.mark.parametrize("name", sorted(["relu", "gelu_erf", "silu", "add", "mul_add", "add_add"]))
def test_tcgen05_post_ops(capi, name):
    ops, nbuf = POST_CASES[name]
    m, k, n = 150, 512, 264
    x, q, s, z, b = make_woq_case(m, k, n, 128, seed=4)
    g = torch.Generator().manual_seed(10)
    bufs = [torch.randn(m, n, generator=g).to(torch.bfloat16) for _ in range(nbuf)]
    y, packed = _run(capi, x, q, s, None, b, capi.ZT_ALGO_TCGEN05, ops, bufs)
    assert_close_bf16(y, O.woq_linear(x, packed.t(), s, None, b, ops, bufs), what=name)


def test_prefill_shape_vs_oracle(capi):
    """Llama-3-8B q projection at prefill M=2048 (config 3) against the full CPU oracle."""
    m, k, n = 2048, 4096, 4096
    x, q, s, z, b = make_woq_case(m, k, n, 128, seed=5)
    packed = capi.woq_repack_weight(q.cuda())
    y = capi.woq_linear(x.cuda(), packed, s.cuda(), None, b.cuda()).cpu()
    ref = (x.float() @ O.woq_dequant(q, s, None).t() + b.float()).to(torch.bfloat16)
    assert_close_bf16(y, ref, what="prefill 2048x4096x4096")


# ---- benchmark shapes ---------------------------------------------------------------------------------
@pytest.mark.parametrize("k,n", [(4096, 4096), (4096, 1024), (4096, 14336), (14336, 4096)])
def test_config_shapes_vs_oracle(capi, k, n):
    """Projection shapes of the benchmark configs at M in {1, 8, 32, 64, 128}; the weight is
    dequantised once on the CPU and shared by all M."""
    _, q, s, z, b = make_woq_case(1, k, n, 128, seed=0)
    packed = capi.woq_repack_weight(q.cuda())
    assert torch.equal(packed.cpu(), O.woq_repack_weight(q))
    dq = O.woq_dequant(q, s, None)                                   # [N, K] fp32, bf16-rounded
    sd, bd = s.cuda(), b.cuda()
    for m in (1, 8, 32, 64, 128):
        x = torch.randn(m, k, generator=torch.Generator().manual_seed(m)).to(torch.bfloat16)
        y = capi.woq_linear(x.cuda(), packed, sd, None, bd).cpu()
        ref = (x.float() @ dq.t() + b.float()).to(torch.bfloat16)
        assert_close_bf16(y, ref, what=f"M={m} K={k} N={n}")


def test_full_size_linearity_and_checksum(capi):
    """Llama-3-70B down projection (K=28672, N=8192) at M=32: size-independent properties instead of
    a full CPU product.  (1) without bias the op is linear in x; (2) the sum of each output row equals
    x[m,:] . (sum_n dq[:,n]), which needs only one pass over the weight on the CPU."""
    m, k, n = 32, 28672, 8192
    x, q, s, z, b = make_woq_case(m, k, n, 128, seed=1, bias=False)
    dev = "cuda"
    packed = capi.woq_repack_weight(q.to(dev))
    sd = s.to(dev)
    y1 = capi.woq_linear(x.to(dev), packed, sd).float()
    x2 = torch.randn(m, k, generator=torch.Generator().manual_seed(2)).to(torch.bfloat16)
    y2 = capi.woq_linear(x2.to(dev), packed, sd).float()
    xs = (x.float() + x2.float()).to(torch.bfloat16)
    ys = capi.woq_linear(xs.to(dev), packed, sd).float()
    # x + x2 is rounded to bf16 before the call: compare against the same rounded input's parts
    resid = (xs.float() - x.float() - x2.float()).to(dev)
    tol = 3e-2 * (y1.abs() + y2.abs()).mean() + 1e-2
    assert ((ys - y1 - y2).abs().mean() < tol) and resid.abs().max() < 0.1
    colsum = torch.zeros(k, dtype=torch.float64)
    sg = s.double()
    for n0 in range(0, n, 1024):
        qq = q[n0:n0 + 1024].double().view(-1, k // 128, 128) * sg[:, n0:n0 + 1024].t().unsqueeze(2)
        colsum += qq.view(-1, k).sum(dim=0)
    expect = x.double() @ colsum
    got = y1.double().sum(dim=1).cpu()
    scale = y1.abs().sum(dim=1).double().cpu()
    assert ((got - expect).abs() <= 4e-3 * scale + 0.5).all()


# ---- weights written directly before the call -----------------------------------------------------------
@pytest.mark.parametrize("m,k,n,algo_hint", [(1, 4096, 1024, 1), (2, 8192, 256, 2), (40, 1024, 512, 0), (24, 1096, 64, 0)])
def test_weights_written_just_before_the_call(capi, m, k, n, algo_hint):
    """ZT_FLAG_WEIGHTS_VOLATILE: the packed weight and the scale table are produced on the same stream right
    before every call (a repack and a copy into fresh buffers), as a non-frozen graph does.  The kernels
    normally fetch weights before they order themselves after earlier work; with the flag they must not.
    Covered: the register-ring kernel (hint 1), the work-balanced decode kernel (hint 2), the tensor-core
    kernel (M = 40) and the mma.sync kernel for shapes the tensor-core kernel does not take (K % 64 != 0)."""
    gs = 128 if k % 128 == 0 else 8
    x, q, s, z, b = make_woq_case(m, k, n, gs, seed=k + m)
    dev = "cuda"
    xd, qd, s_t, bd = x.to(dev), q.to(dev), s.t().contiguous().to(dev), b.to(dev)
    algo = capi.ZT_ALGO_SKINNY | (algo_hint << 8) if algo_hint else capi.ZT_ALGO_AUTO
    ref = O.woq_linear(x, O.woq_repack_weight(q).t(), s, None, b)
    junk = torch.empty(64 << 20, dtype=torch.uint8, device=dev)
    for rep in range(12):
        junk.random_(0, 255)                                  # a long-running kernel ahead on the stream
        packed = capi.woq_repack_weight(qd)                   # fresh buffers, written just before the linear
        scales = s_t.t().contiguous()
        y = capi.woq_linear(xd, packed, scales, None, bd, algo=algo, flags=capi.ZT_FLAG_WEIGHTS_VOLATILE)
        del packed, scales
        assert_close_bf16(y, ref, what=f"volatile weights rep {rep} M={m} K={k} N={n}")
