"""Tensor-parallel sharding of the quantized linears across the GPUs of one box.

The reference has no communication code; it only makes its int4 tensors sliceable so that vLLM's
tensor-parallel loader can ``narrow()`` them (slicing rules:
src/cpu/python/zentorch/vllm/_torchao_int4_opaque_patch.py:93-163).  This module is the B200-side
equivalent for 70B-class layers: Megatron-style column-parallel (shard N) and row-parallel (shard K on
quantisation-group boundaries) linears, one process per GPU, with NCCL collectives only at the shard
boundaries -- an all-reduce after a row-parallel linear, an all-gather when a column-parallel output
is needed whole.

The compute is ``torch.ops.zentorch.*`` (the CUDA kernels); ``linear_fn`` can be replaced, which is
how the CPU test-suite checks the sharding and collective logic with gloo ranks.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.distributed as dist


# ---- slicing ------------------------------------------------------------------------------------------
def shard_woq(weight: torch.Tensor, scales: torch.Tensor, zeros: Optional[torch.Tensor],
              bias: Optional[torch.Tensor], mode: str, rank: int, world: int):
    """Slice a packed WOQ linear for one rank.  ``weight`` is the op's argument: shape [K/8, N], strides
    (1, K/8).  'column' keeps columns [rank*N/world, (rank+1)*N/world); 'row' keeps the K range of the
    same fraction, which must fall on quantisation-group boundaries.  Slices keep the layout contract."""
    k8, n = weight.shape
    groups = scales.shape[0]
    if mode == "column":
        if n % world != 0:
            raise ValueError(f"N ({n}) must be divisible by the tensor-parallel size ({world})")
        n0, n1 = rank * n // world, (rank + 1) * n // world
        w = weight.t()[n0:n1].contiguous().t()
        return (w, scales[:, n0:n1].contiguous(), None if zeros is None else zeros[:, n0:n1].contiguous(),
                None if bias is None else bias[n0:n1].contiguous())
    if mode == "row":
        if groups % world != 0:
            raise ValueError("row-parallel shards must fall on quantization-group boundaries: "
                             f"{groups} groups over {world} ranks")
        gs = k8 * 8 // groups
        g0, g1 = rank * groups // world, (rank + 1) * groups // world
        w = weight.t()[:, g0 * gs // 8: g1 * gs // 8].contiguous().t()
        return (w, scales[g0:g1].contiguous(), None if zeros is None else zeros[g0:g1].contiguous(),
                bias if rank == 0 else None)
    raise ValueError(f"unknown shard mode {mode!r}")


def shard_int8(weight: torch.Tensor, w_scales: torch.Tensor, bias: Optional[torch.Tensor], mode: str, rank: int,
               world: int):
    """Slice a dynamic-int8 linear ([N, K] int8, per-channel scales [N]).  Row-parallel ranks quantise
    their own K-slice of the activations with their own per-token scale."""
    n, k = weight.shape
    if mode == "column":
        n0, n1 = rank * n // world, (rank + 1) * n // world
        return weight[n0:n1].contiguous(), w_scales.reshape(-1)[n0:n1].contiguous(), \
            None if bias is None else bias[n0:n1].contiguous()
    if mode == "row":
        if k % (16 * world) != 0:
            raise ValueError(f"K ({k}) must split into multiples of 16 over {world} ranks")
        k0, k1 = rank * k // world, (rank + 1) * k // world
        return weight[:, k0:k1].contiguous(), w_scales.reshape(-1).contiguous(), bias if rank == 0 else None
    raise ValueError(f"unknown shard mode {mode!r}")


# ---- layers -------------------------------------------------------------------------------------------
def _woq_op(x, w, s, z, b):
    return torch.ops.zentorch.zentorch_woq_linear(x, w, s, z, b)


def _int8_op(x, w, s, b):
    return torch.ops.zentorch.zentorch_dynamic_qlinear(x, w, s, b)


@dataclass
class ParallelLinear:
    """One shard of a column- or row-parallel quantized linear.

    kind 'woq':  params = (weight [K/8, N_shard] view, scales, zeros, bias)
    kind 'int8': params = (weight [N_shard, K_shard], w_scales, bias)
    """
    kind: str
    mode: str
    params: tuple
    group: Optional[dist.ProcessGroup] = None
    linear_fn: Optional[Callable] = None
    reduce_dtype: Optional[torch.dtype] = None   # e.g. torch.float32 for a tighter row-parallel sum

    def local(self, x: torch.Tensor) -> torch.Tensor:
        fn = self.linear_fn or (_woq_op if self.kind == "woq" else _int8_op)
        return fn(x, *self.params)

    def __call__(self, x: torch.Tensor, gather_output: bool = False) -> torch.Tensor:
        """column: x is replicated, the result is this rank's columns (all-gathered when asked).
        row: x is this rank's K-slice, the result is the all-reduced full output."""
        y = self.local(x)
        world = dist.get_world_size(self.group) if dist.is_initialized() else 1
        if world == 1:
            return y
        if self.mode == "row":
            if self.reduce_dtype is not None and y.dtype != self.reduce_dtype:
                yr = y.to(self.reduce_dtype)
                dist.all_reduce(yr, group=self.group)
                return yr.to(y.dtype)
            dist.all_reduce(y, group=self.group)
            return y
        if gather_output:
            parts = [torch.empty_like(y) for _ in range(world)]
            dist.all_gather(parts, y.contiguous(), group=self.group)
            return torch.cat(parts, dim=-1)
        return y


def make_parallel_woq(weight, scales, zeros, bias, mode, group=None, linear_fn=None, reduce_dtype=None):
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    return ParallelLinear("woq", mode, shard_woq(weight, scales, zeros, bias, mode, rank, world), group, linear_fn,
                          reduce_dtype)


def make_parallel_int8(weight, w_scales, bias, mode, group=None, linear_fn=None, reduce_dtype=None):
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    return ParallelLinear("int8", mode, shard_int8(weight, w_scales, bias, mode, rank, world), group, linear_fn,
                          reduce_dtype)


class ParallelMLP:
    """gate/up column-parallel -> silu(gate) * up -> down row-parallel: one collective per call (the
    all-reduce of the down projection), activations between the two stay sharded."""

    def __init__(self, gate: ParallelLinear, up: ParallelLinear, down: ParallelLinear):
        self.gate, self.up, self.down = gate, up, down

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        h = torch.nn.functional.silu(self.gate(x).float()) * self.up(x).float()
        return self.down(h.to(x.dtype))


def slice_activation_for_row_parallel(x: torch.Tensor, group=None) -> torch.Tensor:
    """The K-slice of a replicated activation that a row-parallel shard consumes."""
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    k = x.shape[-1]
    return x[..., rank * k // world:(rank + 1) * k // world].contiguous()


# ---- all-reduce over peer memory for decode sizes -----------------------------------------------------
class PeerAllReduce:
    """In-place sum of a small bf16 tensor over the ranks of `group` with zt_allreduce_bf16: one kernel that
    writes this rank's partial sums into its symmetric buffer, flags the peers and adds everybody's partial sums
    read over NVLink.  The symmetric buffers come from torch's symmetric-memory allocator (one rendezvous at
    construction); nothing is allocated per call and the call can be captured in a CUDA graph.  Tensors larger
    than `max_bytes` are not accepted (`fits()`): the caller keeps the NCCL collective for those."""

    def __init__(self, group=None, max_bytes=1 << 20, device=None):
        import ctypes as C

        import torch.distributed._symmetric_memory as symm_mem

        from . import _capi
        self._capi, self._C = _capi, C
        group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if self.world > _capi.ZT_AR_MAX_RANKS:
            raise ValueError(f"at most {_capi.ZT_AR_MAX_RANKS} ranks")
        self.max_bytes = int(max_bytes)
        device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        total = _capi.lib().zt_allreduce_symmetric_bytes(self.max_bytes)
        self._buf = symm_mem.empty(total, dtype=torch.uint8, device=device)
        self._buf.zero_()
        self._hdl = symm_mem.rendezvous(self._buf, group)
        self._epochs = torch.zeros(_capi.ZT_AR_MAX_SLICES, dtype=torch.int32, device=device)
        torch.cuda.synchronize(device)
        self._hdl.barrier()          # every rank's flags are zero before anybody's first call
        self._args = _capi.AllReduceArgs()
        for r in range(self.world):
            self._args.peer_base[r] = int(self._hdl.buffer_ptrs[r])
        self._args.rank, self._args.world = self.rank, self.world
        self._args.max_bytes = self.max_bytes
        self._args.epochs = self._epochs.data_ptr()

    def fits(self, t: torch.Tensor) -> bool:
        """Every rank sends its whole tensor to every peer (twice the bytes: each word carries the call number), so
        the one-shot form pays off while (world - 1) x bytes stays small; beyond 4 MB of that product the library's
        bandwidth-optimal collective is the better choice."""
        nbytes = t.numel() * 2
        return (t.dtype == torch.bfloat16 and t.is_contiguous() and t.numel() % 8 == 0 and nbytes <= self.max_bytes
                and (self.world - 1) * nbytes <= (4 << 20) and t.data_ptr() % 16 == 0)

    def __call__(self, t: torch.Tensor) -> torch.Tensor:
        a = self._args
        a.in_, a.out, a.numel = t.data_ptr(), t.data_ptr(), t.numel()
        stream = self._C.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)
        self._capi.check(self._capi.lib().zt_allreduce_bf16(self._C.byref(a), stream))
        return t


# ---- fused projections and a whole decoder layer's linears --------------------------------------------
def fuse_woq_columns(parts):
    """Horizontal fusion of WOQ linears that share their input (q/k/v, gate/up): one linear whose output is
    the concatenation of theirs.  The packed layout is N-major, so fusing is a row concatenation of the
    packed tensors and a column concatenation of the scale tables; it is done once at load time (the
    reference's qkv fusion concatenates weights the same way at compile time,
    src/cpu/python/zentorch/_custom_op_replacement.py:675-810).  `parts` is a list of (weight, scales, zeros,
    bias) with weight in the op's [K/8, N_i] form."""
    ws, ss, zs, bs = zip(*parts)
    w = torch.cat([x.t() for x in ws], dim=0).contiguous().t()
    s = torch.cat(ss, dim=1).contiguous()
    z = None if zs[0] is None else torch.cat(zs, dim=1).contiguous()
    b = None if bs[0] is None else torch.cat(bs, dim=0).contiguous()
    return w, s, z, b


def fuse_int8_rows(parts):
    """The same for dynamic-int8 linears: (weight [N_i, K], w_scales [N_i], bias) concatenated along N."""
    ws, ss, bs = zip(*parts)
    return (torch.cat(ws, dim=0).contiguous(), torch.cat([x.reshape(-1) for x in ss]).contiguous(),
            None if bs[0] is None else torch.cat(bs).contiguous())


class DecoderLayerLinears:
    """The seven projections of a Llama-style decoder layer as four launches and two collectives per rank:

        qkv  = x . [Wq | Wk | Wv]   column-parallel (each of q, k, v sharded, then fused per rank)
        o    = attn . Wo            row-parallel, all-reduce
        gu   = o . [Wgate | Wup]    column-parallel, fused; h = silu(gate) * up stays sharded
        down = h . Wdown            row-parallel, all-reduce

    Attention itself is outside this path; `attn` is whatever buffer the caller passes (its shard of the
    attention output).  `kind` is 'woq' or 'int8'; `full` maps a projection name to its unsharded
    parameters (woq: weight [K/8, N] view, scales, zeros, bias; int8: weight [N, K], w_scales, bias).
    Every step is plain launches on the current stream plus NCCL calls, so a whole step can be captured
    in a CUDA graph and replayed without host code between the kernels."""

    def __init__(self, kind, full, rank=0, world=1, group=None, peer_allreduce=None, overlap_rows=None,
                 linear_fn=None):
        self.kind, self.rank, self.world, self.group = kind, rank, world, group
        self.linear_fn = linear_fn               # replaces the CUDA op (CPU tests pass a checker here); None = the op
        self.peer_allreduce = peer_allreduce     # a PeerAllReduce for the decode-size collectives, or None
        # Opt-in: batches of at least `overlap_rows` rows are cut into two halves that run on two streams, so that
        # the library all-reduce of one half can overlap the GEMMs of the other.  Off by default (0 / None): at two
        # ranks it measured 6 % slower, and it is never used while a stream capture is in progress (collectives of
        # one communicator captured on two streams have no order between them in the graph).
        self.overlap_rows = int(overlap_rows) if overlap_rows else 0
        self._side = None
        shard = (lambda p, mode: shard_woq(*p, mode, rank, world)) if kind == "woq" else \
            (lambda p, mode: shard_int8(*p, mode, rank, world))
        fuse = fuse_woq_columns if kind == "woq" else fuse_int8_rows
        self.qkv = fuse([shard(full[n], "column") for n in ("q", "k", "v")])
        self.o = shard(full["o"], "row")
        self.gate_up = fuse([shard(full[n], "column") for n in ("gate", "up")])
        self.down = shard(full["down"], "row")

    def _lin(self, x, params):
        if self.linear_fn is not None:
            return self.linear_fn(x, *params)
        if self.kind == "woq":
            return torch.ops.zentorch.zentorch_woq_linear(x, *params)
        return torch.ops.zentorch.zentorch_dynamic_qlinear(x, *params)

    def _reduce(self, y):
        if self.world > 1:
            if self.peer_allreduce is not None and self.peer_allreduce.fits(y):
                return self.peer_allreduce(y)
            dist.all_reduce(y, group=self.group)
        return y

    def _forward(self, x, attn):
        qkv = self._lin(x, self.qkv)
        o = self._reduce(self._lin(attn, self.o))
        gu = self._lin(o, self.gate_up)
        half = gu.shape[-1] // 2
        h = torch.nn.functional.silu(gu[..., :half]) * gu[..., half:]
        return qkv, self._reduce(self._lin(h, self.down))

    def __call__(self, x, attn):
        m = x.shape[0]
        if (self.world == 1 or not self.overlap_rows or m < self.overlap_rows or x.dim() != 2 or not x.is_cuda
                or torch.cuda.is_current_stream_capturing()):
            return self._forward(x, attn)
        # two half batches on two streams; the collectives are issued in the same order on every rank (second
        # half's, then first half's), and outside a capture torch's process group runs them on its own stream in
        # that order.
        if self._side is None:
            self._side = torch.cuda.Stream(device=x.device)
        main = torch.cuda.current_stream(x.device)
        cut = (m // 2 + 127) // 128 * 128
        self._side.wait_stream(main)
        with torch.cuda.stream(self._side):
            qkv_b, down_b = self._forward(x[cut:], attn[cut:])
        qkv_a, down_a = self._forward(x[:cut], attn[:cut])
        main.wait_stream(self._side)
        for t in (qkv_b, down_b):
            t.record_stream(main)
        return torch.cat([qkv_a, qkv_b]), torch.cat([down_a, down_b])

    def weight_bytes(self):
        """Bytes of weights, scales and zero points this rank streams per step."""
        total = 0
        for p in (self.qkv, self.o, self.gate_up, self.down):
            for t in p[:-1]:
                if t is not None:
                    total += t.numel() * t.element_size()
        return total
