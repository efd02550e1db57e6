"""zt_dynamic_qlinear_static: the variant of the dynamic int8 linear for callers that cannot allocate
device memory (runtimes that own all device memory through their own arena, code in regions where
cudaMalloc is not allowed, plugins that must not touch the host's allocator).  Its scratch is a
fixed array inside the library, so the test checks three things through the C ABI:

* two calls in a row, on different inputs, each give exactly what zt_dynamic_qlinear gives with a
  caller workspace (the second call must not be disturbed by what the first left in the array);
* no device memory is allocated by the calls themselves;
* problems larger than the built-in scratch are refused with a message that names the limit.

The file sorts last so that a run stopping at the first failure has already run everything else.
"""
import ctypes as C

import pytest
import torch

from _util import make_int8_case

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def capi(zt):
    from zentorch_b200 import _capi
    assert torch.cuda.is_available() and _capi.lib().zt_device_supported() == 1
    return _capi


def test_static_scratch_matches_workspace_variant_twice(capi):
    dev = "cuda"
    cases = [(300, 1024, 520, capi.ZT_ACT_S8_SYM, ()), (64, 4096, 264, capi.ZT_ACT_U8_ASYM, (capi.ZT_POST_SILU,))]
    prepared = []
    for i, (m, k, n, act, post) in enumerate(cases):
        x, w, ws, b = [t.to(dev) for t in make_int8_case(m, k, n, seed=20 + i)]
        rowsum = capi.int8_weight_rowsum(w)
        expect = capi.dynamic_qlinear(x, w, ws, b, act_quant=act, post_ops=post, w_rowsum=rowsum)
        prepared.append((x, w, ws, b, rowsum, act, post, expect))
    torch.cuda.synchronize()
    # first call on the device resolves the array's address; do it before measuring allocations
    x, w, ws, b, rowsum, act, post, _ = prepared[0]
    capi.dynamic_qlinear_static(x, w, ws, b, act_quant=act, post_ops=post, w_rowsum=rowsum)
    torch.cuda.synchronize()
    outs = [torch.empty_like(p[-1]) for p in prepared]
    free_before, _ = torch.cuda.mem_get_info()
    for (x, w, ws, b, rowsum, act, post, _), y in zip(prepared, outs):      # two calls in a row
        a = capi.dynamic_qlinear_args(x, w, ws, b, act, post, (), rowsum, y, None, capi.ZT_ALGO_AUTO)
        capi.check(capi.lib().zt_dynamic_qlinear_static(C.byref(a), C.c_void_p(torch.cuda.current_stream().cuda_stream)))
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, "the allocation-free entry point changed the device's free memory"
    for (_, _, _, _, _, _, _, expect), y in zip(prepared, outs):
        assert torch.equal(y, expect)
    # and once more in the opposite order: the array still holds the other problem's data
    for idx in (1, 0):
        x, w, ws, b, rowsum, act, post, expect = prepared[idx]
        y = capi.dynamic_qlinear_static(x, w, ws, b, act_quant=act, post_ops=post, w_rowsum=rowsum)
        assert torch.equal(y, expect)


def test_static_scratch_limits(capi):
    dev = "cuda"
    k = 4096
    m_too_big = capi.ZT_STATIC_SCRATCH_Q_BYTES // k + 1
    x = torch.zeros(m_too_big, k, dtype=torch.bfloat16, device=dev)
    w = torch.zeros(16, k, dtype=torch.int8, device=dev)
    ws = torch.ones(16, device=dev)
    with pytest.raises(capi.ZtError, match="exceeds the built-in scratch") as err:
        capi.dynamic_qlinear_static(x, w, ws)
    assert err.value.code == 2  # ZT_UNSUPPORTED
    x2 = torch.zeros(capi.ZT_STATIC_SCRATCH_MAX_ROWS + 1, 16, dtype=torch.bfloat16, device=dev)
    w2 = torch.zeros(16, 16, dtype=torch.int8, device=dev)
    with pytest.raises(capi.ZtError, match="at most 16384 rows"):
        capi.dynamic_qlinear_static(x2, w2, ws)
    # the largest problem that fits is accepted
    m_fit = capi.ZT_STATIC_SCRATCH_Q_BYTES // k
    xf = torch.randn(m_fit, k, device=dev).to(torch.bfloat16)
    wf = torch.randint(-127, 128, (64, k), dtype=torch.int8, device=dev)
    wsf = torch.rand(64, device=dev) * 0.01
    assert torch.equal(capi.dynamic_qlinear_static(xf, wf, wsf), capi.dynamic_qlinear(xf, wf, wsf))
