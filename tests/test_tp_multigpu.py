"""Tensor-parallel pieces that need more than one GPU: the all-reduce over peer memory and a sharded decoder
layer that uses it.  One child process per GPU (NCCL for the rendezvous and as the comparison), two ranks;
skipped on a box with a single GPU.  NVLS is switched off: the kernels under test use plain peer loads and
stores, and a rank that dies while bound to a multicast object must not disturb its peers."""
import os
import time
import sys
from pathlib import Path

import pytest
import torch
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
pytestmark = pytest.mark.gpu


def _worker(rank, world, port, results):
    for p in (ROOT / "zendnn-pytorch-plugin_b200", ROOT / "oracle", ROOT / "tests"):
        sys.path.insert(0, str(p))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import zentorch_b200  # noqa: F401
        from zentorch_b200 import _capi, tp
        ar = tp.PeerAllReduce(max_bytes=1 << 20)

        def part(r, n, seed):
            g = torch.Generator().manual_seed(1000 * seed + r)
            return torch.randn(n, generator=g).to(torch.bfloat16)

        # every size class: one slice, several slices, the largest that fits; epochs advance call by call
        for call, n in enumerate([8192, 8, 32 * 8192, 1 << 19, 8192, 24 * 8192]):
            parts = [part(r, n, call) for r in range(world)]
            expect = torch.zeros(n)
            for t in parts:                      # rank order, fp32: what the kernel computes
                expect += t.float()
            y = parts[rank].to(dev)
            assert ar.fits(y)
            ar(y)
            torch.cuda.synchronize()
            assert torch.equal(y.cpu(), expect.to(torch.bfloat16)), f"call {call} n={n}"
        assert not ar.fits(torch.empty((1 << 19) + 8, dtype=torch.bfloat16, device=dev))
        # replayed from a CUDA graph: the kernel numbers the calls itself
        n = 16 * 8192
        src = part(rank, n, 99).to(dev)
        buf = torch.empty_like(src)
        stream = torch.cuda.Stream()
        with torch.cuda.stream(stream):
            buf.copy_(src)
            ar(buf)
            stream.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                buf.copy_(src)
                ar(buf)
            expect = sum(part(r, n, 99).float() for r in range(world)).to(torch.bfloat16)
            for _ in range(4):
                g.replay()
                stream.synchronize()
                assert torch.equal(buf.cpu(), expect)
        # a sharded decoder layer: the peer all-reduce and NCCL give the same layer output up to bf16 rounding
        # of the sum (NCCL adds in its own order)
        from bench import LLAMA8B, make_layer_params, seeded_x
        full = make_layer_params(torch, _capi, dev, "woq", LLAMA8B, seed0=7)
        with_peer = tp.DecoderLayerLinears("woq", full, rank, world, peer_allreduce=ar)
        with_nccl = tp.DecoderLayerLinears("woq", full, rank, world)
        for m in (1, 32):
            x = seeded_x(torch, dev, m, 4096, seed=m)
            attn = seeded_x(torch, dev, m, 4096, seed=m + 1)[:, rank * 4096 // world:(rank + 1) * 4096 // world].contiguous()
            _, y1 = with_peer(x, attn)
            _, y2 = with_nccl(x, attn)
            torch.cuda.synchronize()
            err = float((y1.float() - y2.float()).norm() / y2.float().norm())
            assert err < 1e-2, f"layer M={m}: peer all-reduce vs NCCL {err:.3e}"
        assert _capi.poll_device_status() == 0
        results[rank] = "ok"
    except Exception as e:  # surface the failure in the parent
        import traceback
        results[rank] = f"{type(e).__name__}: {e}\n{traceback.format_exc()[-1500:]}"
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_peer_allreduce_and_sharded_layer_two_ranks():
    world = 2
    port = 29600 + (os.getpid() % 2000)
    mgr = mp.Manager()
    results = mgr.dict()
    # bounded: ranks that wait for each other forever are killed (by their own process handles) and the test fails
    ctx = mp.spawn(_worker, args=(world, port, results), nprocs=world, join=False)
    deadline = time.time() + 300
    while not ctx.join(timeout=5):
        if time.time() > deadline:
            for proc in ctx.processes:
                if proc.is_alive():
                    proc.kill()
            pytest.fail(f"the ranks did not finish within 300 s: {dict(results)}")
    assert dict(results) == {0: "ok", 1: "ok"}, dict(results)
