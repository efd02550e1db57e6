"""Generates tests/golden/zentorch_golden.npz from the reference's own Python test utilities.

Run once where a checkout of the reference (amd/ZenDNN-pytorch-plugin) is available, with
ZENTORCH_REFERENCE_ROOT pointing at it; the resulting file is committed and is what the test-suite
reads -- the reference tree is not needed at test time.

Sources of truth used here (none of them is our code):
  * test/unittests/op_tests/_pack.py           -- the reference's independent int4 packer
    (``Pack_4_bits.pack(reorder=False)`` has the bit order of zentorch_woq_repack_weight).
  * aten._convert_weight_to_int4pack_for_cpu / aten._weight_int4pack_mm_for_cpu -- what
    test/unittests/op_tests/test_woq_linear_asymmetric.py:100-142 compares the op against.
  * the formulas written out in test_woq_linear.py:71-96,107-136 and test_dynamic_qlinear.py:32-36,83-92,
    evaluated with stock torch ops exactly as those tests evaluate them.
  * test/unittests/quant_utils.py:13-83 (``qdq_linear``), imported and called as it is: the float restatement
    that test/unittests/op_tests/test_qlinear*.py compare zentorch_qlinear with.  Its cases go into
    tests/golden/zentorch_qlinear_golden.npz (``python make_golden.py qlinear`` writes only that file).
"""
import importlib.util
import os
import sys
from pathlib import Path

import numpy as np
import torch

if "ZENTORCH_REFERENCE_ROOT" not in os.environ:
    raise SystemExit("set ZENTORCH_REFERENCE_ROOT to a checkout of amd/ZenDNN-pytorch-plugin")
REF = Path(os.environ["ZENTORCH_REFERENCE_ROOT"])
OUT = Path(__file__).resolve().parent / "zentorch_golden.npz"
OUT_QLINEAR = Path(__file__).resolve().parent / "zentorch_qlinear_golden.npz"


def _load_pack_module():
    spec = importlib.util.spec_from_file_location("ref_pack", REF / "test/unittests/op_tests/_pack.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def bits(t: torch.Tensor) -> np.ndarray:
    """bf16 tensors are stored as their 16-bit patterns."""
    if t.dtype == torch.bfloat16:
        return t.contiguous().view(torch.int16).numpy()
    return t.contiguous().numpy()


def main():
    torch.manual_seed(1234)
    torch.set_num_threads(1)
    pack = _load_pack_module()
    out = {}

    # 1. repack bit order (signed nibbles), against the reference's own packer
    w = torch.randint(-8, 8, (24, 64), dtype=torch.int8)
    packer = pack.Pack_4_bits(None, "int4")
    packed = packer.pack(w.to(torch.int32), reorder=False, transpose=False)
    out["pack_in"], out["pack_out"] = bits(w), bits(packed)
    # unsigned nibbles too (asymmetric weights are 0..15)
    wu = torch.randint(0, 16, (8, 32), dtype=torch.int8)
    out["packu_in"], out["packu_out"] = bits(wu), bits(packer.pack(wu.to(torch.int32), reorder=False, transpose=False))

    # 2. PyTorch CPU int4pack layout
    n, k, gs = 128, 512, 128
    int_data = torch.randint(0, 16, (n, k), dtype=torch.int32)
    int4pack = torch.ops.aten._convert_weight_to_int4pack_for_cpu(int_data, 1)
    out["int4pack_int_data"], out["int4pack_packed"] = bits(int_data.to(torch.int8)), bits(int4pack)

    # 3. asymmetric per-group linear: test_woq_linear_asymmetric.py:47-89 quantiser, native int4 mm as truth
    wf = (torch.randn(n, k, dtype=torch.bfloat16) * 0.02)
    wv = wf.view(n, k // gs, gs)
    mn, mx = wv.amin(dim=2), wv.amax(dim=2)
    scale = ((mx - mn) / 15.0).clamp(min=torch.finfo(wf.dtype).eps)
    zero = mn + scale * 8.0
    scale, zero = scale.to(wf.dtype), zero.to(wf.dtype)
    mn_rec = zero.unsqueeze(2) - scale.unsqueeze(2) * 8.0
    q_asym = torch.clamp(torch.round((wv - mn_rec) / scale.unsqueeze(2)), 0, 15).to(torch.int32).view(n, k)
    scale_and_zero = torch.cat([scale.unsqueeze(-1), zero.unsqueeze(-1)], dim=-1).transpose(0, 1).contiguous()
    x = torch.randn(5, k, dtype=torch.bfloat16)
    p = torch.ops.aten._convert_weight_to_int4pack_for_cpu(q_asym, 1)
    y = torch.ops.aten._weight_int4pack_mm_for_cpu(x, p, gs, scale_and_zero)
    out["asym_x"], out["asym_q"], out["asym_int4pack"] = bits(x), bits(q_asym.to(torch.int8)), bits(p)
    out["asym_scale"] = bits(scale_and_zero.select(2, 0).contiguous())
    out["asym_zero"] = bits(scale_and_zero.select(2, 1).contiguous())
    out["asym_y"] = bits(y)

    # 4. symmetric per-channel linear: test_woq_linear.py:71-96 quantiser, F.linear on bf16 dq weight as truth
    n2, k2 = 48, 128
    w2 = torch.randn(n2, k2, dtype=torch.bfloat16)
    s2 = torch.clamp(w2.abs().max(dim=1, keepdim=True)[0] / 8, min=1e-8).to(torch.float32)
    q2 = torch.clamp(torch.round(w2 / s2), -8, 7).to(torch.int8)
    x2 = torch.randn(3, 4, k2, dtype=torch.bfloat16)
    b2 = torch.randn(n2, dtype=torch.bfloat16)
    dq2 = (q2.to(torch.bfloat16) * s2).to(torch.bfloat16)
    y2 = torch.nn.functional.linear(x2, dq2, b2)
    out["sym_x"], out["sym_q"], out["sym_scale"], out["sym_bias"], out["sym_y"] = (
        bits(x2), bits(q2), bits(s2.transpose(0, 1).contiguous()), bits(b2), bits(y2))
    # fused variants of the same case: gelu (both forms), add_add, mul_add (test_woq_linear.py:176-290)
    a1 = torch.randn(3, 4, n2, dtype=torch.bfloat16)
    a2 = torch.randn(3, 4, n2, dtype=torch.bfloat16)
    out["sym_add1"], out["sym_add2"] = bits(a1), bits(a2)
    out["sym_y_gelu_tanh"] = bits(torch.nn.functional.gelu(y2, approximate="tanh"))
    out["sym_y_gelu_erf"] = bits(torch.nn.functional.gelu(y2, approximate="none"))
    out["sym_y_add_add"] = bits(y2 + a1 + a2)
    out["sym_y_mul_add"] = bits(y2 * a1 + a2)

    # 5. dynamic qlinear: test_dynamic_qlinear.py:32-36, 83-92
    m3, k3, n3 = 6, 16, 10
    x3 = torch.randn(2, 3, k3)
    w3 = torch.randint(-128, 127, (n3, k3), dtype=torch.int8)
    ws3 = 1 + torch.randn(n3).abs()
    b3 = torch.randn(n3)
    flat = x3.reshape(-1, k3)
    amax = flat.abs().amax(dim=1, keepdim=True).clamp(min=1e-12)
    sc = amax / 127.0
    qdq = torch.clamp(torch.round(flat / sc), -128, 127) * sc
    y3 = (torch.matmul(qdq, (w3.float() * ws3.unsqueeze(1)).t()) + b3).reshape(2, 3, n3)
    out["dyn_x"], out["dyn_w"], out["dyn_ws"], out["dyn_b"], out["dyn_y"] = bits(x3), bits(w3), bits(ws3), bits(b3), bits(y3)

    np.savez_compressed(OUT, **out)
    print("wrote", OUT, OUT.stat().st_size, "bytes")


def _load_quant_utils():
    import torch.ao.quantization.fx._decomposed  # noqa: F401  (registers torch.ops.quantized_decomposed)
    spec = importlib.util.spec_from_file_location("ref_quant_utils", REF / "test/unittests/quant_utils.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main_qlinear():
    """Static-quant qlinear cases: every combination of input dtype (fp32, bf16, already-quantised u8 / s8),
    input zero-point kind, weight-scale granularity and output dtype that
    test/unittests/op_tests/test_qlinear.py:540-610 runs, plus relu / sigmoid (test_qlinear_eltwise.py) and
    mul_add (test_qlinear_mul_add.py), all evaluated by the reference's qdq_linear."""
    torch.manual_seed(4321)
    torch.set_num_threads(1)
    qu = _load_quant_utils()
    out, names = {}, []
    m, k, n = 9, 96, 40
    w = torch.randint(-128, 128, (n, k), dtype=torch.int8)
    bias = torch.randn(n)
    idx = 0
    for x_kind in ("float32", "bfloat16", "uint8", "int8"):
        for per_channel in (False, True):
            for out_kind in ("float32", "bfloat16", "uint8", "int8"):
                for eltwise in ("none", "relu", "sigmoid"):
                    if eltwise != "none" and (x_kind in ("uint8", "int8") or per_channel is False):
                        continue                      # the element-wise variants on the main float cases only
                    xs = torch.rand(1) * 0.03 + 0.01
                    asym = x_kind in ("float32", "uint8") or (x_kind == "bfloat16" and idx % 2 == 0)
                    if x_kind == "int8":
                        asym = False
                    xzp = torch.randint(100, 156, (1,), dtype=torch.uint8) if asym else torch.zeros(1, dtype=torch.int8)
                    if x_kind == "uint8":
                        x = torch.randint(0, 256, (m, k), dtype=torch.uint8)
                    elif x_kind == "int8":
                        x = torch.randint(-128, 128, (m, k), dtype=torch.int8)
                    else:
                        x = (torch.randn(m, k) * 1.5).to(getattr(torch, x_kind))
                    ws = torch.rand(n if per_channel else 1) * 0.004 + 0.001
                    wzp = torch.zeros(n if per_channel else 1, dtype=torch.int8)
                    os_, ozp = None, None
                    if out_kind in ("uint8", "int8"):
                        os_ = torch.rand(1) * 0.02 + 0.03
                        ozp = (torch.randint(90, 166, (1,), dtype=torch.uint8) if out_kind == "uint8"
                               else torch.zeros(1, dtype=torch.int8))
                    fn = {"none": None, "relu": torch.relu, "sigmoid": torch.sigmoid}[eltwise]
                    y = qu.qdq_linear(x, w, bias, xs, xzp, ws, wzp, fn, getattr(torch, out_kind), os_, ozp)
                    tag = f"c{idx}"
                    names.append(f"{tag}:{x_kind}:{int(asym)}:{int(per_channel)}:{out_kind}:{eltwise}")
                    out[tag + "_x"], out[tag + "_xs"], out[tag + "_xzp"] = bits(x), bits(xs), bits(xzp.to(torch.int32))
                    out[tag + "_ws"] = bits(ws)
                    if os_ is not None:
                        out[tag + "_os"], out[tag + "_ozp"] = bits(os_), bits(ozp.to(torch.int32))
                    out[tag + "_y"] = bits(y)
                    idx += 1
    # mul_add: (linear * mul) + add, float outputs (test_qlinear_mul_add.py)
    for x_kind in ("float32", "bfloat16"):
        x = (torch.randn(m, k) * 1.5).to(getattr(torch, x_kind))
        xs, xzp = torch.rand(1) * 0.03 + 0.01, torch.randint(100, 156, (1,), dtype=torch.uint8)
        ws, wzp = torch.rand(n) * 0.004 + 0.001, torch.zeros(n, dtype=torch.int8)
        mul, add = torch.randn(m, n), torch.randn(m, n)
        y = qu.qdq_linear(x, w, bias, xs, xzp, ws, wzp, lambda t: t * mul + add, torch.float32)
        tag = f"c{idx}"
        names.append(f"{tag}:{x_kind}:1:1:float32:mul_add")
        out[tag + "_x"], out[tag + "_xs"], out[tag + "_xzp"], out[tag + "_ws"] = (
            bits(x), bits(xs), bits(xzp.to(torch.int32)), bits(ws))
        out[tag + "_mul"], out[tag + "_add"], out[tag + "_y"] = bits(mul), bits(add), bits(y)
        idx += 1
    out["w"], out["bias"] = bits(w), bits(bias)
    out["cases"] = np.array(names)
    np.savez_compressed(OUT_QLINEAR, **out)
    print("wrote", OUT_QLINEAR, OUT_QLINEAR.stat().st_size, "bytes,", idx, "cases")


if __name__ == "__main__":
    if sys.argv[1:] != ["qlinear"]:
        main()
    main_qlinear()
