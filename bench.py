#!/usr/bin/env python
"""Benchmark of the zentorch quantized-linear hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (BASELINE config 2): dynamic int8 linear, x bf16 [512, 4096] ~ N(0,1) quantised per token
at run time, W int8 [11008, 4096] (per-channel scales), fp32 bias, fused SiLU.  Metric: achieved
int8 TOP/s = 2*M*N*K / time.  One "step" is one pass over a batch of CALLS_PER_STEP such linears
(each call = the per-token quantisation kernel + the tcgen05 GEMM with fused epilogue), rotating
over operand sets whose total size exceeds L2 so that no call finds its weights cached.

The JSON line carries, besides the driver contract's keys:
  roofline       the tcgen05 GEMM kernel alone against the tensor roofline
  woq_decode     the weight-only int4 GEMV (config 1, M=1) against the HBM roofline
  cpu_baseline   the CPU oracle (torch CPU kernels) timed on this box's host cores
  e2e            the same metric through torch.ops.zentorch with host buffers (pinned H2D of x,
                 D2H of y inside the timed region)
With N > 1 (torchrun) every rank runs the same workload on its own batch (data-parallel replicas,
no collective on the data path) and the value is the sum over ranks: weak scaling.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
for p in (ROOT / "zendnn-pytorch-plugin_b200", ROOT / "oracle", ROOT / "tests"):
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))

M, K, N = 512, 4096, 11008
CALLS_PER_STEP = 256
OPS_PER_CALL = 2.0 * M * N * K
L2_BYTES = 126 * 1024 * 1024
METRIC = "dynamic int8 qlinear (u8 per-token act x s8 per-channel weight, fused SiLU) achieved TOP/s"


def peaks():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        d = json.loads(f.read_text())
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed regions run."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.samples, self.proc, self.thread = [], None, None
        self.gpu_index = gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 7:
                self.samples.append(parts)

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm, reasons, smax = [], set(), None
        for s in self.samples:
            try:
                sm.append(float(s[0]))
                smax = float(s[1])
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), s[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": smax, "reasons": [], "samples": 0}
        busy = [v for v in sm if v >= 0.5 * max(sm)]
        return {"sm_mhz": statistics.median(busy), "sm_max_mhz": smax, "reasons": sorted(reasons), "samples": len(sm)}


def make_operands(torch, device, seed):
    """One operand set of config 2, generated on the CPU from a seed and copied to the device."""
    from _util import make_int8_case
    x, w, ws, b = make_int8_case(M, K, N, seed=seed)
    return x, w, ws, b


def time_region(torch, fn, reps):
    """CUDA-event time in ms of `reps` back-to-back invocations of fn on the current stream."""
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for _ in range(reps):
        fn()
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end)


def run_ours(args):
    import torch
    import torch.distributed as dist
    import zentorch_b200
    from zentorch_b200 import _capi
    import ctypes as C

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    assert zentorch_b200.is_supported_device(), "bench.py needs an sm_100 GPU; there is no fallback path"
    pk = peaks()
    lib = _capi.lib()

    # ---- operands: enough distinct sets that the rotation exceeds L2 ---------------------------------
    set_bytes = N * K + M * K * 2 + M * N * 2
    n_sets = max(4, -(-int(1.5 * L2_BYTES) // set_bytes))
    x0, w0, ws0, b0 = make_operands(torch, dev, seed=rank)
    sets = []
    for i in range(n_sets):
        xs = x0.roll(i, 0).contiguous().to(dev)
        wsd = w0.roll(i, 0).contiguous().to(dev)
        sets.append({
            "x": xs, "w": wsd, "ws": ws0.roll(i, 0).contiguous().to(dev), "b": b0.roll(i, 0).contiguous().to(dev),
            "rowsum": _capi.int8_weight_rowsum(wsd), "y": torch.empty(M, N, dtype=torch.bfloat16, device=dev),
            "ws_buf": torch.empty(lib.zt_dynamic_qlinear_workspace_bytes(M, K), dtype=torch.uint8, device=dev),
        })
    stream = torch.cuda.Stream()
    sptr = C.c_void_p(stream.cuda_stream)
    SILU = 4

    def args_for(s, act, post):
        return _capi.dynamic_qlinear_args(s["x"], s["w"], s["ws"], s["b"], act, post, (), s["rowsum"], s["y"], s["ws_buf"],
                                          _capi.ZT_ALGO_AUTO)

    arg_u8 = [args_for(s, _capi.ZT_ACT_U8_ASYM, (SILU,)) for s in sets]
    arg_s8 = [args_for(s, _capi.ZT_ACT_S8_SYM, ()) for s in sets]

    def one_pass(arglist):
        for i in range(CALLS_PER_STEP):
            _capi.check(lib.zt_dynamic_qlinear(C.byref(arglist[i % n_sets]), sptr))

    def capture(body):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.stream(stream):
            body()
            stream.synchronize()
            with torch.cuda.graph(g, stream=stream):
                body()
        return g

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    with torch.cuda.stream(stream):
        graph_u8 = capture(lambda: one_pass(arg_u8))
        graph_s8 = capture(lambda: one_pass(arg_s8))
        for _ in range(max(args.warmup, 3)):
            graph_u8.replay()
        stream.synchronize()
        if world > 1:
            dist.barrier()
        ms = time_region(torch, graph_u8.replay, args.steps)
        if world > 1:
            dist.barrier()
        t = torch.tensor([ms], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_max = float(t.item())
        for _ in range(3):
            graph_s8.replay()
        ms_s8 = time_region(torch, graph_s8.replay, args.steps)

        # ---- roofline of the dominant kernel: the tcgen05 GEMM alone ---------------------------------
        pre = []
        for s in sets:
            q, sc, zp = _capi.dynamic_quantize(s["x"], _capi.ZT_ACT_U8_ASYM)
            pre.append((q, sc, zp))

        def gemm_pass():
            for i in range(CALLS_PER_STEP):
                q, sc, zp = pre[i % n_sets]
                _capi.check(lib.zt_qlinear_prequantized(C.byref(arg_u8[i % n_sets]), q.data_ptr(), sc.data_ptr(),
                                                        zp.data_ptr(), sptr))

        def quant_pass():
            for i in range(CALLS_PER_STEP):
                s = sets[i % n_sets]
                q, sc, zp = pre[i % n_sets]
                _capi.check(lib.zt_dynamic_quantize(s["x"].data_ptr(), _capi.ZT_BF16, M, K, _capi.ZT_ACT_U8_ASYM,
                                                    q.data_ptr(), sc.data_ptr(), zp.data_ptr(), sptr))

        graph_gemm, graph_quant = capture(gemm_pass), capture(quant_pass)
        for _ in range(3):
            graph_gemm.replay()
            graph_quant.replay()
        ms_gemm = time_region(torch, graph_gemm.replay, args.steps) / (args.steps * CALLS_PER_STEP)
        ms_quant = time_region(torch, graph_quant.replay, args.steps) / (args.steps * CALLS_PER_STEP)

        # ---- weight-only int4 decode GEMV (config 1, M = 1), HBM-bound ---------------------------------
        woq = bench_woq(torch, _capi, lib, dev, stream, sptr, args.steps, pk) if rank == 0 else {}
        layer_cfg = bench_layer_configs(torch, _capi, lib, dev, stream, sptr, pk) if rank == 0 else None
    moe_cfg = bench_moe_config(torch, _capi, dev, pk) if rank == 0 else None

    # ---- end to end through torch.ops with host buffers ---------------------------------------------------
    e2e = bench_e2e(torch, dev, sets, args.steps, world)
    tp_mlp = bench_tp_mlp(torch, dist, dev, args.steps, world)
    clocks = sampler.stop() if rank == 0 else None
    torch.cuda.synchronize()
    status = _capi.poll_device_status()
    assert status == 0, f"a kernel reported a bounded-wait timeout (code {status})"

    total_calls = args.steps * CALLS_PER_STEP
    value = world * total_calls * OPS_PER_CALL / (ms_max * 1e-3) / 1e12
    if world > 1:
        te = torch.tensor([e2e["ms"]], device=dev)
        dist.all_reduce(te, op=dist.ReduceOp.MAX)
        e2e["ms"] = float(te.item())
    e2e_value = world * args.steps * OPS_PER_CALL / (e2e["ms"] * 1e-3) / 1e12

    if rank == 0:
        int8_peak = 2.0 * pk["bf16_tflops"]
        cpu = cpu_baseline_sample()
        line = {
            "metric": METRIC, "value": round(value, 2), "unit": "TOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": round(ms_max / args.steps, 5), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "s8/u8 x s8 -> s32, fp32 epilogue", "data": "synthetic",
            "config": {
                "workload": f"BASELINE config 2: dynamic int8 linear M={M} K={K} N={N}, per-token u8 asymmetric "
                            "activations, per-channel s8 weights, fp32 bias, fused SiLU",
                "calls_per_step": CALLS_PER_STEP,
                "l2": f"rotating over {n_sets} operand sets ({n_sets * set_bytes / 2**20:.0f} MiB > L2)",
                "parallelism": f"dp{world} (independent batches per GPU, no collective on the data path)",
                "launch": "CUDA graph of one step",
            },
            "variants": {
                "s8_symmetric_no_postop (the reference op zentorch_dynamic_qlinear)": {
                    "value": round(total_calls * OPS_PER_CALL / (ms_s8 * 1e-3) / 1e12, 2), "unit": "TOP/s"},
                "quant_kernel_us": round(ms_quant * 1e3, 3), "gemm_kernel_us": round(ms_gemm * 1e3, 3),
            },
            "roofline": {
                "kernel": "int8_tcgen05_kernel", "bound": "tensor",
                "achieved": round(OPS_PER_CALL / (ms_gemm * 1e-3) / 1e12, 2), "peak": round(int8_peak, 1),
                "unit": "TOP/s", "frac": round(OPS_PER_CALL / (ms_gemm * 1e-3) / 1e12 / int8_peak, 4),
                "peak_note": f"2 x cuBLAS bf16 burst ({pk['bf16_tflops']} TF/s, {pk['source']}): kind::i8 issues at "
                             "twice the kind::f16 rate",
                "frac_of_sustained_peak": round(OPS_PER_CALL / (ms_gemm * 1e-3) / 1e12 / (2.0 * pk["bf16_tflops_sustained"]), 4),
                "traffic": None,
            },
            "woq_decode": woq.get("woq_decode"), "woq_decode_large_layer": woq.get("woq_decode_large_layer"),
            "woq_prefill": woq.get("woq_prefill"), "tp_mlp": tp_mlp,
            "llama8b_layer": layer_cfg, "moe_int4": moe_cfg,
            "cpu_baseline": cpu,
            "e2e": {"value": round(e2e_value, 3), "unit": "TOP/s", "h2d_bytes_per_step": e2e["h2d"],
                    "d2h_bytes_per_step": e2e["d2h"], "calls_per_step": 1,
                    "api": "torch.ops.zentorch.zentorch_dynamic_qlinear_ext(act_quant='u8_asym', post_op='silu')"},
            "gpu_launches": total_calls * 2,
            "clocks": clocks,
        }
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def device_woq_weights(torch, _capi, dev, k, n, seed, gs=128):
    """Synthetic int4 weights made on the device: uniform nibbles in [-8, 7], fp32 group scales around
    0.01 (the magnitude max|w|/7 of N(0, 0.02) weights gives), packed by the repack kernel."""
    g = torch.Generator(device=dev).manual_seed(seed)
    q = torch.randint(-8, 8, (n, k), generator=g, device=dev, dtype=torch.int8)
    scales = (torch.rand(k // gs, n, generator=g, device=dev) * 0.006 + 0.007).contiguous()
    packed = _capi.woq_repack_weight(q)
    del q
    return packed, scales


def bench_woq_case(torch, _capi, lib, dev, stream, sptr, steps, pk, m, k, n, label):
    """One weight-only int4 linear y = x[m,k] . dq(W)[k,n] + bias (fp32 scales per group of 128, bf16
    bias), rotating over enough weight copies to exceed L2.  Small m is HBM-bound (reported as algorithmic
    GB/s of the HBM roofline), large m tensor-bound (TFLOP/s of the bf16 roofline)."""
    import ctypes as C
    gs = 128
    w_bytes = n * k // 2 + (k // gs) * n * 4
    alg_bytes = w_bytes + m * k * 2 + m * n * 2 + n * 2
    copies = max(2, -(-int(2.0 * L2_BYTES) // w_bytes))
    packed0, scales0 = device_woq_weights(torch, _capi, dev, k, n, seed=0)
    xs = torch.randn(m, k, device=dev).to(torch.bfloat16)
    bs = (torch.randn(n, device=dev) * 0.01).to(torch.bfloat16)
    ws = _capi.woq_workspace(lib.zt_woq_linear_workspace_bytes(m, n, k), dev)
    arglist, keep = [], []
    for i in range(copies):
        wq = packed0.clone()
        sc = scales0.clone()
        y = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
        a = _capi.WoqLinearArgs()
        a.x, a.M, a.K, a.N = xs.data_ptr(), m, k, n
        a.wq, a.scales, a.zeros = wq.data_ptr(), sc.data_ptr(), None
        a.scale_dtype, a.n_groups = _capi.ZT_F32, k // gs
        a.bias, a.bias_dtype = bs.data_ptr(), _capi.ZT_BF16
        a.y, a.workspace, a.workspace_bytes, a.algo = y.data_ptr(), ws.data_ptr(), ws.numel(), _capi.ZT_ALGO_AUTO
        arglist.append(a)
        keep.append((wq, sc, y))

    def one_pass():
        for a in arglist:
            _capi.check(lib.zt_woq_linear(C.byref(a), sptr))

    g = torch.cuda.CUDAGraph()
    one_pass()
    stream.synchronize()
    with torch.cuda.graph(g, stream=stream):
        one_pass()
    for _ in range(3):
        g.replay()
    reps = max(steps, 10)
    ms = time_region(torch, g.replay, reps) / (reps * copies)
    out = {"workload": f"{label}: WOQ int4 (group 128, fp32 scales) M={m} K={k} N={n}, bf16 bias",
           "us_per_call": round(ms * 1e3, 3), "l2": f"rotating over {copies} weight copies",
           "launch": "CUDA graph, back-to-back"}
    if m <= 16:
        gbs = alg_bytes / (ms * 1e-3) / 1e9
        # the dispatcher's rule: TMA-staged stream-K kernel from 48 MB of packed weights, register ring below
        kernel = "woq_streamk_kernel" if n * k // 2 >= (48 << 20) else "woq_stream_kernel"
        out.update({"kernel": kernel, "bound": "hbm", "algorithmic_bytes": alg_bytes, "achieved": round(gbs, 1),
                    "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": round(gbs / pk["hbm_gbs"], 4),
                    "peak_note": f"STREAM-style copy, {pk['source']}"})
    else:
        tf = 2.0 * m * n * k / (ms * 1e-3) / 1e12
        out.update({"kernel": "woq_tcgen05_kernel", "bound": "tensor", "achieved": round(tf, 1),
                    "peak": pk["bf16_tflops"], "unit": "TFLOP/s", "frac": round(tf / pk["bf16_tflops"], 4),
                    "peak_note": f"cuBLAS bf16 burst, {pk['source']}"})
    del keep
    return out


def bench_woq(torch, _capi, lib, dev, stream, sptr, steps, pk):
    cases = {"woq_decode": (1, 4096, 4096, "BASELINE config 1 at M=1"),
             "woq_decode_large_layer": (1, 8192, 28672, "BASELINE config 3 layer (70B-class up-projection) at M=1"),
             "woq_prefill": (2048, 4096, 4096, "BASELINE config 1 at M=2048")}
    return {name: bench_woq_case(torch, _capi, lib, dev, stream, sptr, steps, pk, m, k, n, label)
            for name, (m, k, n, label) in cases.items()}


def bench_layer_configs(torch, _capi, lib, dev, stream, sptr, pk):
    """BASELINE config 2: the seven WOQ int4 projections of a Llama-3-8B decoder layer at decode batch
    M in {1, 8, 32, 64} and prefill M = 2048.  Per M: the layer's summed time, its algorithmic bytes per
    second (decode) or flops per second (prefill).  Weights rotate over copies larger than L2 in total."""
    import ctypes as C
    shapes = [("q", 4096, 4096), ("k", 4096, 1024), ("v", 4096, 1024), ("o", 4096, 4096), ("gate", 4096, 14336),
              ("up", 4096, 14336), ("down", 14336, 4096)]
    gs = 128
    weights = {}
    for _, k, n in shapes:
        if (k, n) not in weights:
            w_bytes = n * k // 2 + (k // gs) * n * 4
            copies = max(2, -(-int(1.5 * L2_BYTES) // w_bytes))
            packed0, scales0 = device_woq_weights(torch, _capi, dev, k, n, seed=k + n)
            weights[(k, n)] = [(packed0.clone(), scales0.clone()) for _ in range(copies)]
    out = {}
    for m in (1, 8, 32, 64, 2048):
        total_us, total_bytes, total_flops = 0.0, 0, 0.0
        for _, k, n in shapes:
            xs = torch.randn(m, k, device=dev).to(torch.bfloat16)
            bs = torch.zeros(n, dtype=torch.bfloat16, device=dev)
            ws = _capi.woq_workspace(lib.zt_woq_linear_workspace_bytes(m, n, k), dev)
            ys = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
            arglist = []
            for wq, sc in weights[(k, n)]:
                a = _capi.WoqLinearArgs()
                a.x, a.M, a.K, a.N = xs.data_ptr(), m, k, n
                a.wq, a.scales, a.zeros = wq.data_ptr(), sc.data_ptr(), None
                a.scale_dtype, a.n_groups = _capi.ZT_F32, k // gs
                a.bias, a.bias_dtype = bs.data_ptr(), _capi.ZT_BF16
                a.y, a.workspace, a.workspace_bytes, a.algo = ys.data_ptr(), ws.data_ptr(), ws.numel(), _capi.ZT_ALGO_AUTO
                arglist.append(a)

            def one_pass():
                for a in arglist:
                    _capi.check(lib.zt_woq_linear(C.byref(a), sptr))

            g = torch.cuda.CUDAGraph()
            one_pass()
            stream.synchronize()
            with torch.cuda.graph(g, stream=stream):
                one_pass()
            g.replay()
            reps = 5
            us = time_region(torch, g.replay, reps) * 1e3 / (reps * len(arglist))
            total_us += us
            total_bytes += n * k // 2 + (k // gs) * n * 4 + m * k * 2 + m * n * 2 + n * 2
            total_flops += 2.0 * m * n * k
        entry = {"layer_us": round(total_us, 2)}
        if m <= 64:
            gbs = total_bytes / (total_us * 1e-6) / 1e9
            entry.update({"algorithmic_GBps": round(gbs, 1), "frac_of_hbm_peak": round(gbs / pk["hbm_gbs"], 4)})
        else:
            tf = total_flops / (total_us * 1e-6) / 1e12
            entry.update({"TFLOPps": round(tf, 1), "frac_of_bf16_peak": round(tf / pk["bf16_tflops"], 4)})
        out[f"M={m}"] = entry
    return {"workload": "BASELINE config 2: Llama-3-8B decoder layer, seven WOQ int4 (group 128) projections, "
                        "one launch each, weights not in L2", "per_batch": out}


def bench_moe_config(torch, _capi, dev, pk):
    """BASELINE config 3: Mixtral-style int4 expert FFN, 8 experts, top-2 over 256 tokens, hidden 4096, ffn 14336."""
    t, h, inter, e, topk, gs = 256, 4096, 14336, 8, 2, 128
    g = torch.Generator(device=dev).manual_seed(3)
    x = torch.randn(t, h, generator=g, device=dev).to(torch.bfloat16)
    logits = torch.randn(t, e, generator=g, device=dev)
    wts, ids = torch.topk(torch.softmax(logits, dim=-1), topk, dim=-1)
    wts = (wts / wts.sum(dim=-1, keepdim=True)).float().contiguous()
    ids = ids.to(torch.int32).contiguous()
    w13 = torch.randint(-2**31, 2**31 - 1, (e, 2 * inter, h // 8), generator=g, device=dev, dtype=torch.int32)
    s13 = (torch.rand(e, h // gs, 2 * inter, generator=g, device=dev) * 0.006 + 0.007).contiguous()
    w2 = torch.randint(-2**31, 2**31 - 1, (e, h, inter // 8), generator=g, device=dev, dtype=torch.int32)
    s2 = (torch.rand(e, inter // gs, h, generator=g, device=dev) * 0.006 + 0.007).contiguous()
    for _ in range(2):
        _capi.moe_woq(x, wts, ids, w13, s13, w2, s2)
    torch.cuda.synchronize()
    reps = 5
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(reps):
        _capi.moe_woq(x, wts, ids, w13, s13, w2, s2)
    end.record()
    torch.cuda.synchronize()
    us = start.elapsed_time(end) * 1e3 / reps
    w_bytes = w13.numel() * 4 + w2.numel() * 4 + s13.numel() * 4 + s2.numel() * 4
    flops = 2.0 * t * topk * (h * 2 * inter + inter * h)
    return {"workload": "BASELINE config 3: int4 MoE FFN, 8 experts, top-2, 256 tokens, hidden 4096, ffn 14336 "
                        "(routing, grouping, two grouped tcgen05 GEMMs, SiLU-mul, combine)",
            "us_per_call": round(us, 1), "weight_bytes": w_bytes, "weight_GBps": round(w_bytes / (us * 1e-6) / 1e9, 1),
            "frac_of_hbm_peak": round(w_bytes / (us * 1e-6) / 1e9 / pk["hbm_gbs"], 4),
            "TFLOPps": round(flops / (us * 1e-6) / 1e12, 1),
            "l2": "705 MB of expert weights per call exceed L2", "launch": "plain launches on the current stream"}


def bench_tp_mlp(torch, dist, dev, steps, world):
    """Tensor-parallel WOQ MLP at decode size (M=16): up-projection column-parallel [8192 -> 28672/world],
    SiLU-gated product, down-projection row-parallel [28672/world -> 8192] followed by the NCCL all-reduce.
    Device-timed per call, max over ranks.  Shards are generated directly (weights are synthetic)."""
    from zentorch_b200 import _capi, tp
    m, hidden, inter = 16, 8192, 28672
    shard = inter // world
    ops = torch.ops.zentorch

    def shard_params(k, n, seed):
        packed, scales = device_woq_weights(torch, _capi, dev, k, n, seed)
        return packed.t(), scales, None, None

    rank = dist.get_rank() if world > 1 else 0
    gate = tp.ParallelLinear("woq", "column", shard_params(hidden, shard, 10 + rank))
    up = tp.ParallelLinear("woq", "column", shard_params(hidden, shard, 20 + rank))
    down = tp.ParallelLinear("woq", "row", shard_params(shard, hidden, 30 + rank))
    mlp = tp.ParallelMLP(gate, up, down)
    x = torch.randn(m, hidden, device=dev).to(torch.bfloat16)
    for _ in range(3):
        mlp(x)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    reps = max(steps, 10)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(reps):
        mlp(x)
    end.record()
    torch.cuda.synchronize()
    t = torch.tensor([start.elapsed_time(end) / reps], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    w_bytes = 3 * (hidden * shard // 2 + (hidden // 128) * shard * 4)
    us = float(t.item()) * 1e3
    return {"workload": f"WOQ int4 SiLU-gated MLP {hidden}->{inter}->{hidden}, M={m}, tensor-parallel over {world} GPU(s)",
            "us_per_call": round(us, 2), "weight_bytes_per_gpu": w_bytes,
            "weight_stream_gbs_per_gpu": round(w_bytes / (us * 1e-6) / 1e9, 1),
            "collective": "one NCCL all-reduce of [16, 8192] bf16 per call" if world > 1 else "none"}


def bench_e2e(torch, dev, sets, steps, world):
    """The user-facing call with host buffers: pinned x -> device, op, y -> pinned host, every step."""
    ops = torch.ops.zentorch
    s = sets[0]
    x_host = s["x"].cpu().pin_memory()
    y_host = torch.empty(M, N, dtype=torch.bfloat16).pin_memory()
    x_dev = torch.empty_like(s["x"])

    def step(i):
        st = sets[i % len(sets)]
        x_dev.copy_(x_host, non_blocking=True)
        y = ops.zentorch_dynamic_qlinear_ext(x_dev, st["w"], st["ws"], st["b"], st["rowsum"], act_quant="u8_asym",
                                             post_op="silu")
        y_host.copy_(y, non_blocking=True)

    for i in range(3):
        step(i)
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(steps):
        step(i)
    end.record()
    torch.cuda.synchronize()
    return {"ms": start.elapsed_time(end), "h2d": M * K * 2, "d2h": M * N * 2}


def run_profile_case(name):
    """A few plain launches (no CUDA graph) of one kernel on a case that is small enough to profile
    with `ncu --set full` and still larger than L2:  python bench.py --profile int8_gemm|woq_decode|dynquant"""
    import ctypes as C
    import torch
    import zentorch_b200  # noqa: F401
    from zentorch_b200 import _capi
    from _util import make_woq_case
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    lib = _capi.lib()
    if name in ("int8_gemm", "dynquant"):
        x0, w0, ws0, b0 = make_operands(torch, dev, seed=0)
        sets = []
        for i in range(4):
            w = w0.roll(i, 0).contiguous().to(dev)
            sets.append((x0.roll(i, 0).contiguous().to(dev), w, ws0.to(dev), b0.to(dev), _capi.int8_weight_rowsum(w)))
        y = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
        for i in range(8):
            x, w, ws, b, rs = sets[i % 4]
            q, sc, zp = _capi.dynamic_quantize(x, _capi.ZT_ACT_U8_ASYM)
            if name == "int8_gemm":
                a = _capi.dynamic_qlinear_args(x, w, ws, b, _capi.ZT_ACT_U8_ASYM, (4,), (), rs, y, None, _capi.ZT_ALGO_AUTO)
                _capi.check(lib.zt_qlinear_prequantized(C.byref(a), q.data_ptr(), sc.data_ptr(), zp.data_ptr(), None))
    elif name == "woq_decode":
        m, k, n, gs = 1, 8192, 28672, 128
        x = torch.randn(m, k, device=dev).to(torch.bfloat16)
        bias = torch.zeros(n, dtype=torch.bfloat16, device=dev)
        copies = [(torch.randint(-2**31, 2**31 - 1, (n, k // 8), dtype=torch.int32, device=dev),
                   torch.rand(k // gs, n, device=dev) * 0.01) for _ in range(2)]
        for i in range(6):
            wq, sc = copies[i % 2]
            _capi.woq_linear(x, wq, sc, None, bias)
    elif name == "woq_prefill":
        m, k, n, gs = 2048, 4096, 14336, 128
        x = torch.randn(m, k, device=dev).to(torch.bfloat16)
        bias = torch.zeros(n, dtype=torch.bfloat16, device=dev)
        copies = [(torch.randint(-2**31, 2**31 - 1, (n, k // 8), dtype=torch.int32, device=dev),
                   torch.rand(k // gs, n, device=dev) * 0.01) for _ in range(2)]
        for i in range(4):
            wq, sc = copies[i % 2]
            _capi.woq_linear(x, wq, sc, None, bias)
    else:
        raise SystemExit(f"unknown profile case {name}")
    torch.cuda.synchronize()
    assert _capi.poll_device_status() == 0
    print(json.dumps({"profile_case": name, "status": "ok"}))


def cpu_oracle_call():
    """The reference's CPU path is not installable here (its kernels live in ZenDNN, fetched from the
    network at build time), so the timed CPU arm is the oracle port on stock torch CPU kernels."""
    import torch
    import zentorch_oracle as O
    from _util import make_int8_case
    x, w, ws, b = make_int8_case(M, K, N, seed=0)
    torch.set_num_threads(os.cpu_count() or 1)

    def call():
        return O.dynamic_qlinear(x, w, ws, b, act_quant="u8_asym", post_ops=[O.POST_SILU])
    return call


def cpu_baseline_sample():
    import torch
    call = cpu_oracle_call()
    call()
    n = 5
    t0 = time.perf_counter()
    for _ in range(n):
        call()
    dt = (time.perf_counter() - t0) / n
    return {"value": round(OPS_PER_CALL / dt / 1e12, 4), "unit": "TOP/s", "cores": torch.get_num_threads(),
            "kind": "port", "sample": f"{n} full calls of the config-2 linear (1 warm-up), {dt * 1e3:.1f} ms each",
            "note": "oracle port on torch CPU kernels (row-wise quantise + torch._int_mm + fp32 epilogue); "
                    "zentorch's own CPU path is unavailable on this box"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    import torch
    call = cpu_oracle_call()
    for _ in range(max(args.warmup, 1)):
        call()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        call()
    dt = time.perf_counter() - t0
    value = args.steps * OPS_PER_CALL / dt / 1e12
    sample = f"{args.steps} steps of one full config-2 call each"
    line = {
        "impl": "reference", "metric": METRIC, "value": round(value, 4), "unit": "TOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 1), "ms_per_step": round(dt / args.steps * 1e3, 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "s8/u8 x s8 -> s32, fp32 epilogue",
        "data": "synthetic",
        "config": {"workload": f"BASELINE config 2: dynamic int8 linear M={M} K={K} N={N}, per-token u8 asymmetric "
                               "activations, per-channel s8 weights, fp32 bias, fused SiLU", "calls_per_step": 1,
                   "parallelism": "host cores of rank 0"},
        "cpu_baseline": {"value": round(value, 4), "unit": "TOP/s", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": sample,
                         "note": "oracle port on torch CPU kernels; zentorch's own CPU path (ZenDNN) cannot be "
                                 "built or installed here"},
        "e2e": {"value": round(value, 4), "unit": "TOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--profile", default=None, help="run a few plain launches of one kernel (for ncu): "
                                                    "int8_gemm | woq_decode | woq_prefill | dynquant")
    args = ap.parse_args()
    if args.profile:
        run_profile_case(args.profile)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
