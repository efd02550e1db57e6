"""Tensor-parallel sharding and collectives on CPU: two gloo ranks, the oracle as each rank's linear.
Checks that column-parallel + all-gather, row-parallel + all-reduce, and the gate/up -> down MLP
reproduce the unsharded oracle."""
import os
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _worker(rank, world, port, results):
    for p in (ROOT / "zendnn-pytorch-plugin_b200", ROOT / "oracle", ROOT / "tests"):
        sys.path.insert(0, str(p))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import zentorch_oracle as O
        from zentorch_b200 import tp
        from _util import make_woq_case, make_int8_case

        def woq_fn(x, w, s, z, b):
            return O.woq_linear(x, w, s, z, b, return_fp32=True)

        def int8_fn(x, w, s, b):
            return O.dynamic_qlinear(x.float(), w, s, b)

        m, k, n = 6, 1024, 256
        x, q, s, _, b = make_woq_case(m, k, n, 128, seed=3)
        packed = O.woq_repack_weight(q).t()
        full = O.woq_linear(x, packed, s, None, b, return_fp32=True)

        col = tp.make_parallel_woq(packed, s, None, b, "column", linear_fn=woq_fn)
        y_col = col(x, gather_output=True)
        assert y_col.shape == full.shape and torch.allclose(y_col, full, rtol=1e-5, atol=1e-5)
        assert col(x).shape == (m, n // world)

        row = tp.make_parallel_woq(packed, s, None, b, "row", linear_fn=woq_fn)
        y_row = row(tp.slice_activation_for_row_parallel(x))
        assert torch.allclose(y_row, full, rtol=1e-4, atol=1e-4)

        # MLP: gate/up column-parallel, down row-parallel, exactly one all-reduce
        inter = 512
        _, qg, sg, _, _ = make_woq_case(1, k, inter, 128, seed=4, bias=False)
        _, qu, su, _, _ = make_woq_case(1, k, inter, 128, seed=5, bias=False)
        _, qd, sd, _, bd = make_woq_case(1, inter, k, 128, seed=6)
        pg, pu, pd = (O.woq_repack_weight(t).t() for t in (qg, qu, qd))
        mlp = tp.ParallelMLP(tp.make_parallel_woq(pg, sg, None, None, "column", linear_fn=woq_fn),
                             tp.make_parallel_woq(pu, su, None, None, "column", linear_fn=woq_fn),
                             tp.make_parallel_woq(pd, sd, None, bd, "row", linear_fn=woq_fn))
        calls = []
        orig = dist.all_reduce
        dist.all_reduce = lambda *a, **kw: (calls.append(1), orig(*a, **kw))[1]
        y_mlp = mlp(x)
        dist.all_reduce = orig
        assert len(calls) == 1
        h = torch.nn.functional.silu(O.woq_linear(x, pg, sg, return_fp32=True)) * O.woq_linear(x, pu, su, return_fp32=True)
        ref = O.woq_linear(h.to(torch.bfloat16), pd, sd, None, bd, return_fp32=True)
        assert torch.allclose(y_mlp.float(), ref, rtol=2e-2, atol=2e-2)

        # int8: column-parallel is exact; row-parallel quantises each K-slice with its own scale
        xi, wi, wsi, bi = make_int8_case(8, 256, 64, seed=7, x_dtype=torch.float32)
        full_i = O.dynamic_qlinear(xi, wi, wsi, bi)
        ci = tp.make_parallel_int8(wi, wsi, bi, "column", linear_fn=int8_fn)
        assert torch.allclose(ci(xi, gather_output=True), full_i, rtol=1e-6, atol=1e-6)
        ri = tp.make_parallel_int8(wi, wsi, bi, "row", linear_fn=int8_fn)
        y_ri = ri(tp.slice_activation_for_row_parallel(xi))
        assert torch.allclose(y_ri, full_i, rtol=5e-2, atol=5e-2)

        # error paths
        with pytest.raises(ValueError, match="group boundaries"):
            tp.shard_woq(packed, s[:3], None, None, "row", 0, 2)
        results[rank] = "ok"
    except Exception as e:  # surface the failure in the parent
        results[rank] = f"{type(e).__name__}: {e}"
    finally:
        dist.destroy_process_group()


def _layer_worker(rank, world, port, results):
    """The whole sharded decoder layer (fused q/k/v and gate/up, two all-reduces) against the same class at
    world 1, the oracle standing in for the CUDA ops."""
    for p in (ROOT / "zendnn-pytorch-plugin_b200", ROOT / "oracle", ROOT / "tests"):
        sys.path.insert(0, str(p))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import zentorch_oracle as O
        from zentorch_b200 import tp
        from _util import make_woq_case, make_int8_case

        hidden, kv, inter, m = 256, 128, 512, 5
        shapes = {"q": (hidden, hidden), "k": (hidden, kv), "v": (hidden, kv), "o": (hidden, hidden),
                  "gate": (hidden, inter), "up": (hidden, inter), "down": (inter, hidden)}

        def woq_fn(x, w, s, z, b):
            return O.woq_linear(x, w, s, z, b, return_fp32=True)

        def int8_fn(x, w, s, b):
            return O.dynamic_qlinear(x.float(), w, s, b)

        for asym in (False, True):
            full = {}
            for i, (name, (k, n)) in enumerate(shapes.items()):
                _, q, s, z, b = make_woq_case(1, k, n, 128, seed=20 + i, asym=asym, bias=name in ("q", "down"))
                if name in ("k", "v"):           # fused with q, whose bias decides for all three
                    b = torch.zeros(n, dtype=torch.bfloat16)
                full[name] = (O.woq_repack_weight(q).t(), s, z, b)
            g = torch.Generator().manual_seed(99)
            x = torch.randn(m, hidden, generator=g).to(torch.bfloat16)
            attn = torch.randn(m, hidden, generator=g).to(torch.bfloat16)
            one = tp.DecoderLayerLinears("woq", full, 0, 1, linear_fn=woq_fn)
            qkv1, down1 = one(x, attn)
            many = tp.DecoderLayerLinears("woq", full, rank, world, linear_fn=woq_fn)
            qkv, down = many(x, tp.slice_activation_for_row_parallel(attn))
            want = torch.cat([t.chunk(world, dim=-1)[rank] for t in
                              qkv1.split([hidden, kv, kv], dim=-1)], dim=-1)
            assert qkv.shape == want.shape and torch.allclose(qkv, want, rtol=1e-5, atol=1e-5), "woq qkv"
            assert torch.allclose(down, down1, rtol=1e-3, atol=1e-3), "woq down"
            assert many.weight_bytes() * world == one.weight_bytes(), "weight bytes"

        full = {}
        for i, (name, (k, n)) in enumerate(shapes.items()):
            _, w, ws, b = make_int8_case(1, k, n, seed=40 + i, x_dtype=torch.float32)
            full[name] = (w, ws, b)
        xf, af = x.float(), attn.float()
        one = tp.DecoderLayerLinears("int8", full, 0, 1, linear_fn=int8_fn)
        qkv1, down1 = one(xf, af)
        many = tp.DecoderLayerLinears("int8", full, rank, world, linear_fn=int8_fn)
        qkv, down = many(xf, tp.slice_activation_for_row_parallel(af))
        want = torch.cat([t.chunk(world, dim=-1)[rank] for t in qkv1.split([hidden, kv, kv], dim=-1)], dim=-1)
        assert torch.allclose(qkv, want, rtol=1e-6, atol=1e-6), "int8 qkv"      # column-parallel is exact
        # row-parallel quantises each K slice with its own scale: close, not equal
        err = (down - down1).abs().max() / down1.abs().max()
        assert err < 5e-2, f"int8 down {err}"
        results[rank] = "ok"
    except Exception as e:
        results[rank] = f"{type(e).__name__}: {e}"
    finally:
        dist.destroy_process_group()


def test_decoder_layer_two_gloo_ranks():
    world = 2
    port = 31500 + (os.getpid() % 2000)
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_layer_worker, args=(world, port, results), nprocs=world, join=True)
    assert dict(results) == {0: "ok", 1: "ok"}, dict(results)


def test_tp_two_gloo_ranks():
    world = 2
    port = 29500 + (os.getpid() % 2000)
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
    assert dict(results) == {0: "ok", 1: "ok"}, dict(results)
