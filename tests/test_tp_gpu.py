"""Tensor-parallel shards of the 70B-class projections on one GPU.

Every rank's shard (sliced by zentorch_b200.tp exactly as a tensor-parallel run slices it, following
src/cpu/python/zentorch/vllm/_torchao_int4_opaque_patch.py:93-163) is run on cuda:0 through
torch.ops.zentorch.*, the pieces are put together the way the collectives would (concatenation for
column-parallel, an fp32 sum for row-parallel), and the result is compared with the CPU oracle of the
unsharded layer.  The layers are too large for a full CPU product, so the oracle is evaluated on a sample
of output columns that touches every shard; the unsharded GPU result is checked the same way (which also
covers the kernels the dispatcher picks by itself at these sizes) and the sharded result is compared with
it in full.
"""
import pytest
import torch

import zentorch_oracle as O
from _util import assert_close_bf16, make_woq_fast, woq_oracle_columns

pytestmark = pytest.mark.gpu

GS = 128
# (K, N, mode): q/k/v-like narrow projection, up projection, down projection of a 70B-class layer
LAYERS = {"kv": (8192, 1024, "column"), "up": (8192, 28672, "column"), "down": (28672, 8192, "row")}


@pytest.fixture(scope="module")
def env(zt):
    from zentorch_b200 import _capi, tp
    assert torch.cuda.is_available() and _capi.lib().zt_device_supported() == 1
    return torch.ops.zentorch, tp, _capi


@pytest.fixture(scope="module")
def woq_layers(env):
    """Packed weights of the three layers on the device (made once per module) plus their CPU copies."""
    ops, _, _ = env
    out = {}
    for name, (k, n, mode) in LAYERS.items():
        q, s, _, b = make_woq_fast(k, n, GS, seed=len(name))
        packed = ops.zentorch_woq_repack_weight(q.cuda())          # [N, K/8]
        g = torch.Generator().manual_seed(k + n)
        cols = torch.randperm(n, generator=g)[:192].sort().values  # sample spread over all shards
        out[name] = dict(q=q, s=s, b=b, packed=packed, sd=s.cuda(), bd=b.cuda(), cols=cols, mode=mode)
    return out


def _x(m, k, seed):
    return torch.randn(m, k, generator=torch.Generator().manual_seed(seed)).to(torch.bfloat16)


@pytest.mark.parametrize("m", [1, 4, 32])
@pytest.mark.parametrize("name", sorted(LAYERS))
def test_unsharded_layer_auto_dispatch(env, woq_layers, name, m):
    """The whole layer through the op with the dispatcher's own choice: at M <= 4 the 117 MB layers take the
    work-balanced decode kernel (>= 48 MB of packed weights), the 4 MB one the register-ring kernel, M = 32
    the tensor-core kernel.  Checked on sampled columns against the oracle."""
    ops, _, _ = env
    L = woq_layers[name]
    k = L["q"].shape[1]
    x = _x(m, k, seed=m)
    y = ops.zentorch_woq_linear(x.cuda(), L["packed"].t(), L["sd"], None, L["bd"]).cpu()
    ref = woq_oracle_columns(x, L["q"], L["s"], None, L["b"], L["cols"], GS)
    assert_close_bf16(y[:, L["cols"]], ref.to(torch.bfloat16), what=f"{name} M={m} unsharded")


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("m", [1, 32])
@pytest.mark.parametrize("name", sorted(LAYERS))
def test_woq_shards_reassemble(env, woq_layers, name, m, world):
    ops, tp, _ = env
    L = woq_layers[name]
    k, n = L["q"].shape[1], L["q"].shape[0]
    x = _x(m, k, seed=10 * m + world)
    xd = x.cuda()
    weight = L["packed"].t()                                        # the op's argument: [K/8, N], strides (1, K/8)
    parts = []
    for rank in range(world):
        w, s, z, b = tp.shard_woq(weight, L["sd"], None, L["bd"], L["mode"], rank, world)
        assert w.stride(0) == 1 or w.shape[0] == 1                  # shards keep the layout contract
        if L["mode"] == "column":
            assert w.shape == (k // 8, n // world)
            parts.append(ops.zentorch_woq_linear(xd, w, s, z, b))
        else:
            k0, k1 = rank * k // world, (rank + 1) * k // world
            assert w.shape == (k // 8 // world, n) and s.shape[0] == k // GS // world
            parts.append(ops.zentorch_woq_linear(xd[:, k0:k1].contiguous(), w, s, z, b).float())
    if L["mode"] == "column":
        y = torch.cat(parts, dim=-1).cpu()
    else:
        y = torch.stack(parts).sum(dim=0).to(torch.bfloat16).cpu()   # what the all-reduce adds (fp32 here)
    ref = woq_oracle_columns(x, L["q"], L["s"], None, L["b"], L["cols"], GS)
    assert_close_bf16(y[:, L["cols"]], ref.to(torch.bfloat16), what=f"{name} M={m} tp={world} vs oracle")
    full = ops.zentorch_woq_linear(xd, weight, L["sd"], None, L["bd"]).cpu()
    assert_close_bf16(y, full, what=f"{name} M={m} tp={world} vs unsharded GPU")


@pytest.mark.parametrize("world", [2, 8])
@pytest.mark.parametrize("m", [1, 32])
def test_woq_asymmetric_row_shards(env, m, world):
    """Zero points travel with the scales: a row-parallel slice of an asymmetric layer."""
    ops, tp, _ = env
    k, n = 7168, 1024
    q, s, z, b = make_woq_fast(k, n, GS, seed=5, asym=True, scale_dtype=torch.bfloat16)
    packed = ops.zentorch_woq_repack_weight(q.cuda())
    x = _x(m, k, seed=m + world)
    parts = []
    for rank in range(world):
        w, ss, zz, bb = tp.shard_woq(packed.t(), s.cuda(), z.cuda(), b.cuda(), "row", rank, world)
        k0, k1 = rank * k // world, (rank + 1) * k // world
        parts.append(ops.zentorch_woq_linear(x.cuda()[:, k0:k1].contiguous(), w, ss, zz, bb).float())
    y = torch.stack(parts).sum(dim=0).to(torch.bfloat16).cpu()
    ref = O.woq_linear(x, O.woq_repack_weight(q).t(), s, z, b)
    assert_close_bf16(y, ref, what=f"asymmetric row-parallel M={m} tp={world}")


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("m", [1, 32])
@pytest.mark.parametrize("mode,k,n", [("column", 8192, 1024), ("column", 8192, 3584), ("row", 28672, 1024)])
def test_int8_shards_reassemble(env, mode, k, n, m, world):
    """Dynamic-int8 shards.  Column-parallel ranks quantise the same activations, so the concatenation is
    the unsharded result bit for bit.  A row-parallel rank quantises its own K slice with its own per-token
    scale: the oracle is evaluated the same way (per-slice scales, fp32 sum) at the 1e-2 tolerance, and the
    sum also stays close to the unsharded oracle (2e-2 in the Frobenius norm)."""
    ops, tp, _ = env
    g = torch.Generator().manual_seed(k + n + m)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16)
    w = torch.randint(-127, 128, (n, k), generator=g, dtype=torch.int8)
    ws = torch.rand(n, generator=g) * 4e-4 + 2e-4
    b = torch.randn(n, generator=g) * 0.01
    xd, wd, wsd, bd = x.cuda(), w.cuda(), ws.cuda(), b.cuda()
    full_ref = O.dynamic_qlinear(x, w, ws, b)
    parts, ref_parts = [], []
    for rank in range(world):
        wr, sr, br = tp.shard_int8(wd, wsd, bd, mode, rank, world)
        if mode == "column":
            parts.append(ops.zentorch_dynamic_qlinear(xd, wr, sr, br))
        else:
            k0, k1 = rank * k // world, (rank + 1) * k // world
            parts.append(ops.zentorch_dynamic_qlinear(xd[:, k0:k1].contiguous(), wr, sr, br).float())
            ref_parts.append(O.dynamic_qlinear(x[:, k0:k1].contiguous(), w[:, k0:k1].contiguous(), ws,
                                               b if rank == 0 else None).float())
    if mode == "column":
        y = torch.cat(parts, dim=-1)
        assert torch.equal(y, ops.zentorch_dynamic_qlinear(xd, wd, wsd, bd))
        assert_close_bf16(y, full_ref, what=f"int8 column M={m} tp={world}")
    else:
        y = torch.stack(parts).sum(dim=0).to(torch.bfloat16).cpu()
        ref = torch.stack(ref_parts).sum(dim=0).to(torch.bfloat16)
        assert_close_bf16(y, ref, what=f"int8 row M={m} tp={world} vs per-slice oracle")
        # against the unsharded oracle only the quantisation noise differs (other scales per slice): it is a
        # few percent of an element's magnitude with long tails, so the comparison is an aggregate one
        rel = float((y.float() - full_ref.float()).norm() / full_ref.float().norm())
        assert rel < 2e-2, f"int8 row M={m} tp={world} vs unsharded: relative Frobenius error {rel:.3e}"
