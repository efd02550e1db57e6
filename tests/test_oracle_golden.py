"""The CPU oracle against the golden vectors made from the reference's own test utilities
(tests/golden/make_golden.py), and the C restatement against the Python one."""
import ctypes as C

import numpy as np
import torch

import zentorch_oracle as O
from _util import assert_qlinear_close, bf16_from_bits, make_woq_case, make_int8_case, qlinear_golden_cases


def _ptr(t):
    return C.c_void_p(t.data_ptr())


def test_repack_matches_reference_packer(golden):
    for key in ("pack", "packu"):
        w = torch.from_numpy(golden[f"{key}_in"])
        expect = torch.from_numpy(golden[f"{key}_out"])
        got = O.woq_repack_weight(w)
        assert got.dtype == torch.int32 and torch.equal(got, expect)
        # and unpacking the op-layout view gives the values back
        back = O.woq_unpack(got.t(), signed=(key == "pack"))
        assert torch.equal(back, w)


def test_int4pack_unpack_matches_aten(golden):
    packed = torch.from_numpy(golden["int4pack_packed"])
    int_data = torch.from_numpy(golden["int4pack_int_data"])
    assert torch.equal(O.unpack_int4pack_to_int8(packed), int_data)
    assert torch.equal(O.woq_repack_from_int4pack(packed), O.woq_repack_weight(int_data))


def test_asymmetric_linear_matches_native_int4_mm(golden):
    x = bf16_from_bits(golden["asym_x"])
    scale, zero = bf16_from_bits(golden["asym_scale"]), bf16_from_bits(golden["asym_zero"])
    packed = O.woq_repack_from_int4pack(torch.from_numpy(golden["asym_int4pack"]))
    y = O.woq_linear(x, packed.t(), scale, zero, None)
    ref = bf16_from_bits(golden["asym_y"])
    # the reference accepts rtol=0.1, atol=2.0 here; the oracle is far inside that
    assert torch.allclose(y.float(), ref.float(), rtol=0.1, atol=2.0)
    assert (y.float() - ref.float()).abs().max() < 0.05


def test_symmetric_per_channel_matches_reference_formula(golden):
    x = bf16_from_bits(golden["sym_x"])
    q = torch.from_numpy(golden["sym_q"])
    scale = torch.from_numpy(golden["sym_scale"])
    bias = bf16_from_bits(golden["sym_bias"])
    packed = O.woq_repack_weight(q)
    y = O.woq_linear(x, packed.t(), scale, None, bias)
    ref = bf16_from_bits(golden["sym_y"])
    assert y.shape == ref.shape and y.dtype == torch.bfloat16
    # reference tolerance: rtol = atol = 1e-3 (test_woq_linear.py:133-136) up to one bf16 rounding
    close = torch.isclose(y.float(), ref.float(), rtol=1e-3, atol=1e-3)
    one_ulp = (y.view(torch.int16).int() - ref.view(torch.int16).int()).abs() <= 1
    assert (close | one_ulp).all()
    assert close.float().mean() > 0.98
    a1, a2 = bf16_from_bits(golden["sym_add1"]), bf16_from_bits(golden["sym_add2"])
    cases = {
        "gelu_tanh": ([O.POST_GELU_TANH], []), "gelu_erf": ([O.POST_GELU_ERF], []),
        "add_add": ([O.POST_ADD, O.POST_ADD], [a1, a2]), "mul_add": ([O.POST_MUL, O.POST_ADD], [a1, a2]),
    }
    for name, (ops, bufs) in cases.items():
        yf = O.woq_linear(x, packed.t(), scale, None, bias, ops, bufs)
        reff = bf16_from_bits(golden[f"sym_y_{name}"])
        # fused variants: rtol = atol = 1e-2 (test_woq_linear.py:163-165); the golden applies the
        # post-op to an already rounded bf16 linear output, the oracle rounds once at the end
        assert torch.allclose(yf.float(), reff.float(), rtol=1e-2, atol=6e-2), name


def test_dynamic_qlinear_matches_reference_formula(golden):
    x = torch.from_numpy(golden["dyn_x"])
    w = torch.from_numpy(golden["dyn_w"])
    ws, b = torch.from_numpy(golden["dyn_ws"]), torch.from_numpy(golden["dyn_b"])
    y = O.dynamic_qlinear(x, w, ws.unsqueeze(0), b)
    ref = torch.from_numpy(golden["dyn_y"])
    assert y.shape == ref.shape
    assert torch.allclose(y, ref, atol=1e-2, rtol=1e-2)      # test_dynamic_qlinear.py:102-103
    assert torch.allclose(y, ref, atol=1e-3, rtol=1e-5)


def test_static_qlinear_matches_reference_formula():
    """zentorch_qlinear and its relu / sigmoid / mul_add variants against the reference's qdq_linear
    (test/unittests/quant_utils.py:13-83) over input dtype x zero-point kind x weight granularity x output dtype."""
    cases = qlinear_golden_cases()
    assert len(cases) >= 48
    seen = set()
    for c in cases:
        y = O.static_qlinear(c["x"], c["w"], c["xs"], c["xzp"], c["ws"], None, c["bias"], c["os"], c["ozp"],
                             c["out_dtype"], c["post"], c["buffers"])
        assert_qlinear_close(y, c["y"], c["name"])
        seen.add((c["x"].dtype, c["out_dtype"], c["eltwise"]))
    assert {d for d, _, _ in seen} == {torch.float32, torch.bfloat16, torch.uint8, torch.int8}
    assert {e for _, _, e in seen} == {"none", "relu", "sigmoid", "mul_add"}


def test_u8_dynamic_rows_are_static_qlinear_rows():
    """The per-token u8 mode (no reference counterpart) shares everything after the choice of a row's scale and
    zero point with the static qlinear, whose arithmetic is pinned by the reference's formula above: feeding a
    row's quantised bytes, scale and zero point to the static form gives the same fp32 row bit for bit."""
    x, w, ws, b = make_int8_case(5, 192, 40, seed=3)
    xf = x.float()
    q, s, zp, acc, y = O.dynamic_qlinear(xf, w, ws, b, act_quant="u8_asym", return_parts=True)
    for m in range(x.shape[0]):
        row = O.static_qlinear(q[m:m + 1], w, s[m:m + 1].clone(), zp[m:m + 1].clone(), ws.reshape(-1).float(), None, b,
                               output_dtype=torch.float32)
        assert torch.equal(row, y[m:m + 1])


def test_static_qlinear_error_messages():
    import pytest
    x, w = torch.zeros(2, 8), torch.zeros(4, 8, dtype=torch.int8)
    s1, z1, sw = torch.ones(1), torch.zeros(1, dtype=torch.int32), torch.ones(4)
    # messages of src/cpu/cpp/MatmulUtils.hpp:357-415,453-475 and src/cpu/cpp/QLinear.cpp:379-383
    with pytest.raises(RuntimeError, match="unsupported dtype for input tensor"):
        O.static_qlinear(x.half(), w, s1, z1, sw)
    with pytest.raises(RuntimeError, match="unsupported dtype for weight tensor, only int8 is supported"):
        O.static_qlinear(x, w.float(), s1, z1, sw)
    with pytest.raises(RuntimeError, match="unsupported dtype for bias tensor"):
        O.static_qlinear(x, w, s1, z1, sw, None, torch.zeros(4, dtype=torch.float16))
    with pytest.raises(RuntimeError, match="unsupported dtype for input_scales"):
        O.static_qlinear(x, w, s1.half(), z1, sw)
    with pytest.raises(RuntimeError, match="unsupported dtype for input_zero_points"):
        O.static_qlinear(x, w, s1, z1.float(), sw)
    with pytest.raises(RuntimeError, match="unsupported number of elements for input_scales"):
        O.static_qlinear(x, w, torch.ones(2), z1, sw)
    with pytest.raises(RuntimeError, match="unsupported number of elements for weight_scales"):
        O.static_qlinear(x, w, s1, z1, torch.ones(3))
    with pytest.raises(RuntimeError, match="output_dtype received is not yet supported"):
        O.static_qlinear(x, w, s1, z1, sw, output_dtype=torch.float16)
    with pytest.raises(RuntimeError, match="when output_scales are not defined"):
        O.static_qlinear(x, w, s1, z1, sw, output_dtype=torch.uint8)


def test_error_messages_follow_the_reference():
    import pytest
    with pytest.raises(RuntimeError, match="K must be divisible by 8"):
        O.woq_repack_weight(torch.zeros(4, 12, dtype=torch.int8))
    with pytest.raises(RuntimeError, match="K must be at least 8"):
        O.woq_repack_weight(torch.zeros(4, 4, dtype=torch.int8))
    with pytest.raises(RuntimeError, match="must have dtype int8"):
        O.woq_repack_weight(torch.zeros(4, 8, dtype=torch.int32))
    with pytest.raises(RuntimeError, match="multiple of 64"):
        O.unpack_int4pack_to_int8(torch.zeros(32, 16, dtype=torch.uint8))
    with pytest.raises(RuntimeError, match="weight must have dtype int32"):
        O.woq_linear(torch.zeros(1, 8, dtype=torch.bfloat16), torch.zeros(1, 4, dtype=torch.int8), torch.ones(1, 4))
    with pytest.raises(RuntimeError, match="input must be bfloat16 or float32"):
        O.dynamic_qlinear(torch.zeros(2, 8, dtype=torch.float16), torch.zeros(4, 8, dtype=torch.int8), torch.ones(4))
    with pytest.raises(RuntimeError, match="bias must be 1D with size N"):
        O.dynamic_qlinear(torch.zeros(2, 8), torch.zeros(4, 8, dtype=torch.int8), torch.ones(4), torch.zeros(3))


# ---- C restatement == Python restatement --------------------------------------------------------------
def test_c_oracle_repack_and_unpack(c_oracle, golden):
    w = torch.from_numpy(golden["pack_in"]).contiguous()
    out = torch.empty(w.shape[0], w.shape[1] // 8, dtype=torch.int32)
    assert c_oracle.zt_oracle_woq_repack_weight(_ptr(w), w.shape[0], w.shape[1], _ptr(out)) == 0
    assert torch.equal(out, torch.from_numpy(golden["pack_out"]))
    assert c_oracle.zt_oracle_woq_repack_weight(_ptr(w), w.shape[0], 12, _ptr(out)) == 1
    packed = torch.from_numpy(golden["int4pack_packed"]).contiguous()
    un = torch.empty(packed.shape[0], packed.shape[1] * 2, dtype=torch.int8)
    assert c_oracle.zt_oracle_unpack_int4pack(_ptr(packed), packed.shape[0], packed.shape[1], _ptr(un)) == 0
    assert torch.equal(un, torch.from_numpy(golden["int4pack_int_data"]))


def test_c_oracle_woq_linear_equals_python(c_oracle):
    for asym, gs, (m, k, n) in ((False, 128, (3, 256, 40)), (True, 64, (2, 128, 24)), (False, 256, (1, 256, 16))):
        x, q, s, z, b = make_woq_case(m, k, n, gs, seed=7, asym=asym)
        packed = O.woq_repack_weight(q)
        add = torch.randn(m, n).to(torch.bfloat16)
        ops = [O.POST_SILU, O.POST_ADD]
        y_py = O.woq_linear(x, packed.t(), s, z, b, ops, [add])
        y_c = torch.empty(m, n, dtype=torch.bfloat16)
        bias_f = b.float().contiguous()
        ids = (C.c_int * 2)(*ops)
        bufs = (C.c_void_p * 1)(add.data_ptr())
        rc = c_oracle.zt_oracle_woq_linear(_ptr(x), m, k, _ptr(packed), n, _ptr(s), _ptr(z) if z is not None else None,
                                           s.shape[0], _ptr(bias_f), 2, ids, bufs, 1, None, _ptr(y_c))
        assert rc == 0
        ulp = (y_c.view(torch.int16).int() - y_py.view(torch.int16).int()).abs()
        assert ulp.max() <= 1 and (ulp == 0).float().mean() > 0.99


def test_c_oracle_dynamic_qlinear_equals_python(c_oracle):
    x, w, ws, b = make_int8_case(9, 64, 20, seed=3, x_dtype=torch.float32)
    q_py, s_py, _, acc_py, y_py = O.dynamic_qlinear(x, w, ws, b, return_parts=True)
    q_c = torch.empty_like(q_py)
    s_c = torch.empty_like(s_py)
    c_oracle.zt_oracle_dynamic_quantize_s8(_ptr(x), 9, 64, _ptr(q_c), _ptr(s_c))
    assert torch.equal(q_c, q_py) and torch.equal(s_c, s_py)
    acc_c = torch.empty(9, 20, dtype=torch.int32)
    c_oracle.zt_oracle_int8_gemm(_ptr(q_c), 0, _ptr(w), 9, 20, 64, _ptr(acc_c))
    assert torch.equal(acc_c, acc_py)
    y_c = torch.empty(9, 20)
    c_oracle.zt_oracle_qlinear_epilogue(_ptr(acc_c), 9, 20, _ptr(s_c), _ptr(ws), _ptr(b), None, None, 0, _ptr(y_c))
    assert torch.allclose(y_c, y_py, rtol=1e-6, atol=1e-6)
    # unsigned mode
    qu_py, su_py, zp_py, accu_py, yu_py = O.dynamic_qlinear(x, w, ws, b, act_quant="u8_asym",
                                                           post_ops=[O.POST_SILU], return_parts=True)
    qu_c, su_c, zp_c = torch.empty_like(qu_py), torch.empty_like(su_py), torch.empty_like(zp_py)
    c_oracle.zt_oracle_dynamic_quantize_u8(_ptr(x), 9, 64, _ptr(qu_c), _ptr(su_c), _ptr(zp_c))
    assert torch.equal(qu_c, qu_py) and torch.equal(su_c, su_py) and torch.equal(zp_c, zp_py)
    accu_c = torch.empty(9, 20, dtype=torch.int32)
    c_oracle.zt_oracle_int8_gemm(_ptr(qu_c), 1, _ptr(w), 9, 20, 64, _ptr(accu_c))
    assert torch.equal(accu_c, accu_py)
    wsum = w.int().sum(dim=1).to(torch.int32).contiguous()
    c_oracle.zt_oracle_qlinear_epilogue(_ptr(accu_c), 9, 20, _ptr(su_c), _ptr(ws), _ptr(b), _ptr(zp_c), _ptr(wsum), 4,
                                        _ptr(y_c))
    assert torch.allclose(y_c, yu_py, rtol=1e-5, atol=1e-5)


def test_u8_quantisation_reconstructs_input():
    x = torch.randn(16, 256) * 3 + 1
    q, s, zp = O.dynamic_quantize_u8(x)
    rec = (q.float() - zp.unsqueeze(1).float()) * s.unsqueeze(1)
    assert (rec - x).abs().max() <= s.max() * 0.5 + 1e-6
    q8, s8 = O.dynamic_quantize_s8(x)
    assert ((q8.float() * s8.unsqueeze(1)) - x).abs().max() <= s8.max() * 0.5 + 1e-6


def test_tp_shards_recompose():
    x, q, s, z, b = make_woq_case(4, 512, 64, 128, seed=11)
    packed = O.woq_repack_weight(q).t()
    full = O.woq_linear(x, packed, s, None, b, return_fp32=True)
    for world in (2, 4):
        cols = [O.woq_linear(x, *O.tp_shard_woq(packed, s, None, b, "column", r, world), return_fp32=True)
                for r in range(world)]
        assert torch.allclose(torch.cat(cols, dim=1), full, rtol=1e-5, atol=1e-5)
        rows = []
        for r in range(world):
            w_r, s_r, _, b_r = O.tp_shard_woq(packed, s, None, b, "row", r, world)
            k0, k1 = r * 512 // world, (r + 1) * 512 // world
            rows.append(O.woq_linear(x[:, k0:k1].contiguous(), w_r, s_r, None, b_r, return_fp32=True))
        assert torch.allclose(sum(rows), full, rtol=1e-4, atol=1e-4)


def test_c_oracle_static_qlinear_equals_python_and_golden(c_oracle):
    """The C restatement of the static qlinear against the Python one on every golden case (float inputs are
    quantised in C too), bit for bit; the Python one is pinned by the reference's qdq_linear above."""
    lib = c_oracle
    lib.zt_oracle_static_quantize.argtypes = [C.c_void_p, C.c_int64, C.c_float, C.c_int32, C.c_int, C.c_void_p]
    lib.zt_oracle_static_qlinear_epilogue.argtypes = [C.c_void_p, C.c_int64, C.c_int64, C.c_float, C.c_int32,
                                                      C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int,
                                                      C.c_void_p, C.c_void_p, C.c_float, C.c_int32, C.c_int, C.c_void_p]
    lib.zt_oracle_int8_gemm.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_void_p]
    n_checked = 0
    for c in qlinear_golden_cases():
        x, w = c["x"], c["w"]
        m, k, n = x.shape[0], x.shape[1], w.shape[0]
        is_u8 = c["xzp"] is not None
        xs, xzp = float(c["xs"]), (int(c["xzp"]) if is_u8 else 0)
        if x.dtype in (torch.uint8, torch.int8):
            q = x.contiguous()
        else:
            xf = x.float().contiguous()
            q = torch.empty(m, k, dtype=torch.uint8 if is_u8 else torch.int8)
            lib.zt_oracle_static_quantize(_ptr(xf), m * k, xs, xzp, int(is_u8), _ptr(q))
        acc = torch.empty(m, n, dtype=torch.int32)
        lib.zt_oracle_int8_gemm(_ptr(q), int(is_u8), _ptr(w), m, n, k, _ptr(acc))
        wsum = w.sum(dim=1, dtype=torch.int32).contiguous()
        ws = c["ws"].float().contiguous()
        bias = c["bias"].float().contiguous()
        unary = {"none": 0, "relu": O.POST_RELU, "sigmoid": O.POST_SIGMOID, "mul_add": 0}[c["eltwise"]]
        mul, add = (c["buffers"][0].float().contiguous(), c["buffers"][1].float().contiguous()) if c["buffers"] else (None, None)
        requant = c["os"] is not None
        y = torch.empty(m, n)
        lib.zt_oracle_static_qlinear_epilogue(
            _ptr(acc), m, n, xs, xzp, _ptr(wsum) if is_u8 else None, _ptr(ws), int(ws.numel() == 1), _ptr(bias), unary,
            _ptr(mul) if mul is not None else None, _ptr(add) if add is not None else None,
            float(c["os"]) if requant else 0.0, int(c["ozp"]) if c["ozp"] is not None else 0,
            int(c["out_dtype"] == torch.uint8), _ptr(y))
        ref = O.static_qlinear(x, w, c["xs"], c["xzp"], c["ws"], None, c["bias"], c["os"], c["ozp"], c["out_dtype"],
                               c["post"], c["buffers"])
        got = y.to(c["out_dtype"])
        if c["eltwise"] == "sigmoid":       # libm's and torch's exp differ in the last bits
            assert_qlinear_close(got, ref, c["name"])
        else:
            assert torch.equal(got, ref), c["name"]
        n_checked += 1
    assert n_checked >= 48


def test_moe_oracle_equals_token_loop():
    """The grouped-by-expert MoE oracle against a second, token-by-token statement of the same FFN built from the
    raw int4 values and scales (no packing, no grouping): out[t] = sum_j w[t,j] * W2_e(silu(W1_e x) * W3_e x).
    The reference has no int4 MoE to pin this on; the check is that grouping, slot weights and the gate-first
    split of the fused w13 are consistent with the per-token definition, and that token order does not matter."""
    g = torch.Generator().manual_seed(5)
    t, h, inter, e, gs = 9, 128, 64, 4, 64
    x = torch.randn(t, h, generator=g).to(torch.bfloat16)
    tw, ids = O.route_top2(torch.randn(t, e, generator=g))
    assert torch.allclose(tw.sum(dim=1), torch.ones(t)) and (ids[:, 0] != ids[:, 1]).all()
    w13q, s13, w2q, s2 = [], [], [], []
    for _ in range(e):
        q, s = O.quantize_woq_sym(torch.randn(2 * inter, h, generator=g) * 0.05, gs)
        w13q.append(q), s13.append(s)
        q, s = O.quantize_woq_sym(torch.randn(h, inter, generator=g) * 0.05, gs)
        w2q.append(q), s2.append(s)
    got = O.moe_woq(x, tw, ids, [O.woq_repack_weight(q).t() for q in w13q], s13,
                    [O.woq_repack_weight(q).t() for q in w2q], s2)

    def dense(q, s):                      # [N, K] int8, [K/gs, N] -> fp32 [N, K], rounded to bf16 like the op
        w = q.float().view(q.shape[0], -1, gs) * s.t().unsqueeze(2)
        return w.view(q.shape).to(torch.bfloat16).float()

    want = torch.zeros(t, h)
    for i in range(t):
        for j in range(ids.shape[1]):
            ex = int(ids[i, j])
            hh = dense(w13q[ex], s13[ex]) @ x[i].float()
            a = (torch.nn.functional.silu(hh[:inter]) * hh[inter:]).to(torch.bfloat16).float()
            want[i] += tw[i, j] * (dense(w2q[ex], s2[ex]) @ a)
    assert torch.allclose(got.float(), want, rtol=2e-2, atol=1e-3)

    perm = torch.randperm(t, generator=g)
    got_p = O.moe_woq(x[perm], tw[perm], ids[perm], [O.woq_repack_weight(q).t() for q in w13q], s13,
                      [O.woq_repack_weight(q).t() for q in w2q], s2)
    assert torch.equal(got_p, got[perm])


def test_c_oracle_quantisation_edge_rows(c_oracle):
    """Rows the two restatements could round differently: all zero, constant of either sign, one huge outlier,
    denormals, one-sided ranges.  Bytes, scales and zero points must agree bit for bit, and the u8 zero point of a
    one-sided row sits at the matching end of the range."""
    k = 64
    x = torch.zeros(8, k)
    x[1], x[2], x[4] = 3.0, -2.5, 1e-41
    x[3, 5] = 1e30
    x[5], x[6], x[7] = torch.linspace(-1, 1, k), torch.linspace(0, 5, k), torch.linspace(-5, -1, k)
    q, s = O.dynamic_quantize_s8(x)
    qc, sc = torch.empty_like(q), torch.empty_like(s)
    c_oracle.zt_oracle_dynamic_quantize_s8(_ptr(x), 8, k, _ptr(qc), _ptr(sc))
    assert torch.equal(q, qc) and torch.equal(s, sc)
    assert (q[0] == 0).all() and (q[1] == 127).all() and (q[2] == -127).all() and int(q[3, 5]) == 127
    qu, su, zp = O.dynamic_quantize_u8(x)
    quc, suc, zpc = torch.empty_like(qu), torch.empty_like(su), torch.empty_like(zp)
    c_oracle.zt_oracle_dynamic_quantize_u8(_ptr(x), 8, k, _ptr(quc), _ptr(suc), _ptr(zpc))
    assert torch.equal(qu, quc) and torch.equal(su, suc) and torch.equal(zp, zpc)
    assert zp.tolist() == [0, 0, 255, 0, 0, 127, 0, 255]
    assert torch.isfinite(s).all() and torch.isfinite(su).all() and (s > 0).all() and (su > 0).all()
