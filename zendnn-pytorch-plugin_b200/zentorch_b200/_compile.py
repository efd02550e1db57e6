"""torch.compile glue for CUDA graphs: the FX passes that turn dequantise-then-matmul subgraphs into
``torch.ops.zentorch.zentorch_woq_linear`` and fold element-wise consumers into its fused variants.

Contract mirrored from the reference (same ATen-level patterns, same replacement graph, same counter
keys, so that the reference's model tests read the same):

* op replacement: src/cpu/python/zentorch/_op_replacements_new.py:297-677 -- ``mm`` / ``addmm`` of
  ``permute([view(]mul(sub(to_bf16(W_int8), to_bf16(zp)), scale)[)])`` becomes
  ``zentorch_woq_repack_weight(W).transpose(0, 1)`` + ``scale.transpose(0, 1).contiguous()`` ->
  ``zentorch_woq_linear(x, Wp, S, None, bias)``.  Under freezing the repack constant-folds.
* fusions: _woq_linear_unary_fusion.py (GELU erf / tanh) and _woq_linear_binary_binary_fusion.py
  (add+add, mul+add), plus relu / sigmoid / single add which the kernels also fuse.
* pass order and gate: _optimize.py:80-160; the AVX-512 gate (:87-91) becomes "a compute-capability
  10.x CUDA device is present".
* backend: _compile_backend.py:70-95 (Inductor ``compile_fx`` with the pass as ``joint_custom_post_pass``).

The ``aten._weight_int4pack_mm_for_cpu`` patterns of the reference (:684-799) cannot occur in a CUDA graph
(that ATen op is CPU-only); ``zentorch_woq_repack_from_int4pack`` stays available for converting such
checkpoints.
"""
from __future__ import annotations

import collections
import functools
from typing import Any

import torch
from torch._inductor.pattern_matcher import (
    Arg,
    CallFunction,
    Match,
    PatternMatcherPass,
    register_graph_pattern,
    stable_topological_sort,
)

aten = torch.ops.aten
prims = torch.ops.prims
zt = torch.ops.zentorch

# counters["zentorch"][op_name] += 1 per replacement, as in src/cpu/python/zentorch/_utils.py:23
counters: dict = collections.defaultdict(collections.Counter)

replace_pass = PatternMatcherPass(pass_name="zentorch_b200_woq_replace")
binary_pass = PatternMatcherPass(pass_name="zentorch_b200_woq_binary_fusion")
unary_pass = PatternMatcherPass(pass_name="zentorch_b200_woq_unary_fusion")


def _val(node):
    return node.meta.get("val") if hasattr(node, "meta") else None


def _is_int8_weight(idx: int):
    def check(match: Match) -> bool:
        v = _val(match.args[idx])
        return v is not None and v.dtype == torch.int8 and v.dim() in (2, 3)
    return check


def _bias_and_weight_ok(bias_idx: int, weight_idx: int):
    def check(match: Match) -> bool:
        b = _val(match.args[bias_idx])
        return b is not None and b.dim() == 1 and _is_int8_weight(weight_idx)(match)
    return check


def _dequant(view: bool):
    """to_bf16(W) - to_bf16(zp), times scale, optionally viewed back to 2-D (per-group), permuted."""
    core = CallFunction(
        aten.mul,
        CallFunction(
            aten.sub,
            CallFunction(prims.convert_element_type.default, Arg(), torch.bfloat16),   # int8 weight
            CallFunction(prims.convert_element_type.default, Arg(), torch.bfloat16),   # int8 zero points
        ),
        Arg(),                                                                         # scales
    )
    if view:
        core = CallFunction(aten.view, core, Arg())
    return CallFunction(aten.permute, core, Arg())


def _replacement(view: bool, with_bias: bool):
    def repl(*args):
        if with_bias:
            bias, x, w, _zp, scales = args[:5]
            rest = args[5:]
        else:
            x, w, _zp, scales = args[:4]
            bias, rest = None, args[4:]
        if view:
            view_shape = rest[0]
            w = w.view(view_shape)
            scales = scales.view(scales.shape[0], -1)
        packed = zt.zentorch_woq_repack_weight(w).transpose(0, 1)            # [N, K/8] -> [K/8, N] view
        scales = scales.transpose(0, 1).contiguous()                           # [N, G] -> [G, N]
        return zt.zentorch_woq_linear(x, packed, scales, None, bias, zentorch_op_name="zentorch_woq_linear")
    return repl


def _register_replacements():
    for view in (False, True):
        @register_graph_pattern(CallFunction(aten.mm, Arg(), _dequant(view)), pass_dict=replace_pass,
                                extra_check=_is_int8_weight(1))
        def _no_bias(match: Match, *args, _view=view):
            counters["zentorch"]["zentorch_woq_linear"] += 1
            match.replace_by_example(_replacement(_view, False), list(args))

        @register_graph_pattern(CallFunction(aten.addmm, Arg(), Arg(), _dequant(view)), pass_dict=replace_pass,
                                extra_check=_bias_and_weight_ok(0, 2))
        def _with_bias(match: Match, *args, _view=view):
            counters["zentorch"]["zentorch_woq_linear"] += 1
            match.replace_by_example(_replacement(_view, True), list(args))


# ---- fusions ---------------------------------------------------------------------------------------------
def _woq(users: int = 1, with_bias: bool = True):
    args = [Arg(), Arg(), Arg(), Arg()] + ([Arg()] if with_bias else [])
    return CallFunction(zt.zentorch_woq_linear.default, *args, _users=users)


def _same_shape_as_output(match: Match) -> bool:
    out = _val(match.output_node())
    if out is None:
        return False
    for a in match.args[-2:]:
        v = _val(a) if isinstance(a, torch.fx.Node) else None
        if v is None or tuple(v.shape) != tuple(out.shape) or v.dtype != out.dtype:
            return False
    return True


def _register_binary_fusions():
    combos = {("add", "add"): (aten.add.Tensor, aten.add.Tensor, "zentorch_woq_linear_add_add"),
              ("mul", "add"): (aten.mul.Tensor, aten.add.Tensor, "zentorch_woq_linear_mul_add")}
    for (inner, outer), (op_in, op_out, name) in combos.items():
        target = getattr(zt, name)
        for with_bias in (True, False):
            lin = _woq(1, with_bias)
            shapes = [CallFunction(op_out, CallFunction(op_in, lin, Arg()), Arg()),
                      CallFunction(op_out, Arg(), CallFunction(op_in, lin, Arg())),
                      CallFunction(op_out, CallFunction(op_in, Arg(), lin), Arg()),
                      CallFunction(op_out, Arg(), CallFunction(op_in, Arg(), lin))]
            for variant, pat in enumerate(shapes):
                @register_graph_pattern(pat, pass_dict=binary_pass, extra_check=_same_shape_as_output)
                def _fuse(match: Match, *args, _variant=variant, _with_bias=with_bias, _target=target, _name=name):
                    nlin = 5 if _with_bias else 4
                    # locate the linear's arguments and the two element-wise operands in pattern order
                    flat = list(args)
                    if _variant == 0:      # out(in(lin, a), b)
                        lin_args, first, second = flat[:nlin], flat[nlin], flat[nlin + 1]
                    elif _variant == 1:    # out(b, in(lin, a))
                        second, lin_args, first = flat[0], flat[1:1 + nlin], flat[1 + nlin]
                    elif _variant == 2:    # out(in(a, lin), b)
                        first, lin_args, second = flat[0], flat[1:1 + nlin], flat[1 + nlin]
                    else:                  # out(b, in(a, lin))
                        second, first, lin_args = flat[0], flat[1], flat[2:2 + nlin]
                    bias = lin_args[4] if _with_bias else None

                    def repl(x, w, s, zp, first, second, *maybe_bias):
                        b = maybe_bias[0] if maybe_bias else None
                        return _target(x, w, s, zp, first, second, b, zentorch_op_name=_name)

                    counters["zentorch"][_name] += 1
                    ex = list(lin_args[:4]) + [first, second] + ([bias] if _with_bias else [])
                    match.replace_by_example(repl, ex)


def _register_unary_fusions():
    simple = {aten.relu.default: "zentorch_woq_linear_relu", aten.sigmoid.default: "zentorch_woq_linear_sigmoid"}
    for op, name in simple.items():
        for with_bias in (True, False):
            @register_graph_pattern(CallFunction(op, _woq(1, with_bias)), pass_dict=unary_pass)
            def _fuse(match: Match, *args, _name=name, _with_bias=with_bias):
                target = getattr(zt, _name)

                def repl(x, w, s, zp, *maybe_bias):
                    return target(x, w, s, zp, maybe_bias[0] if maybe_bias else None, zentorch_op_name=_name)

                counters["zentorch"][_name] += 1
                match.replace_by_example(repl, list(args))
    # GELU arrives decomposed; reuse Inductor's own description of the two decompositions, as the
    # reference does (_woq_linear_unary_fusion.py:11-14, 211-245).
    try:
        from torch._inductor.fx_passes.mkldnn_fusion import _gelu_fusion_1, _gelu_fusion_2
    except Exception:  # pragma: no cover - private Inductor helpers moved
        return
    def wrapped(make, users, with_bias, lowp):
        # bf16 linears reach GELU through an fp32 up-cast that carries the fan-out; the result is cast back
        if not lowp:
            return make(_woq(users, with_bias))
        up = CallFunction(prims.convert_element_type.default, _woq(1, with_bias), torch.float32, _users=users)
        return CallFunction(prims.convert_element_type.default, make(up), torch.bfloat16)

    for make, users, name in ((_gelu_fusion_1, 2, "zentorch_woq_linear_gelu_erf"),
                              (_gelu_fusion_2, 4, "zentorch_woq_linear_gelu_tanh")):
        for with_bias in (True, False):
            for lowp in (True, False):
                @register_graph_pattern(wrapped(make, users, with_bias, lowp), pass_dict=unary_pass)
                def _fuse(match: Match, *args, _name=name):
                    target = getattr(zt, _name)

                    def repl(x, w, s, zp, *maybe_bias):
                        return target(x, w, s, zp, maybe_bias[0] if maybe_bias else None, zentorch_op_name=_name)

                    counters["zentorch"][_name] += 1
                    match.replace_by_example(repl, list(args))


_registered = False


def _register_all():
    global _registered
    if not _registered:
        _register_replacements()
        _register_binary_fusions()
        _register_unary_fusions()
        _registered = True


# ---- horizontal fusion of weight-only linears that share their input (q / k / v, gate / up) ------------------
def _ancestors_include(node, targets, limit=64):
    """True when one of `targets` is reachable upwards from `node` (bounded walk over parameter chains)."""
    stack, seen = [node], set()
    while stack and len(seen) < limit:
        n = stack.pop()
        if not isinstance(n, torch.fx.Node) or n in seen:
            continue
        if n in targets:
            return True
        seen.add(n)
        stack.extend(a for a in n.all_input_nodes)
    return False


def _fake(target, args):
    """meta["val"] of a new node, computed from its arguments' fake values."""
    vals = torch.fx.node.map_arg(args, lambda n: n.meta["val"])
    return target(*vals)


def fuse_parallel_woq_linears(fx_graph: torch.fx.Graph) -> int:
    """zentorch_woq_linear nodes with the same input (and no post-op, the same zero-point / bias presence, the
    same group count and scale dtype) become one zentorch_woq_linear on concatenated parameters followed by
    slices of its output: one launch instead of two or three, which is what a decode step is made of.  The
    packed layout is N-major, so the fused weight is a row concatenation of the packed tensors
    ([N_i, K/8] each) viewed back as [K/8, sum N_i]; scale and zero-point tables are concatenated along their
    columns, biases along their only axis.

    The concatenations are graph nodes: with frozen parameters (Inductor's freezing) they fold into
    constants, otherwise they would run on every call and cost more than the launches they save, which is why
    this pass is not part of `optimize()` and has to be asked for.  The reference fuses q / k / v of its bf16
    linear the same way (src/cpu/python/zentorch/_custom_op_replacement.py:675-810: same input, exactly three
    users, consistent bias and post-ops, `cat` of the weights, split of the output); this is that idea for
    the weight-only operator, for any number of siblings.  Returns the number of fused groups."""
    target = zt.zentorch_woq_linear.default
    order = {n: i for i, n in enumerate(fx_graph.nodes)}
    fused_groups = 0
    for x in list(fx_graph.nodes):
        group = [u for u in x.users if u.op == "call_function" and u.target == target and u.args[0] is x]
        if len(group) < 2:
            continue
        group.sort(key=order.get)

        def arg(n, i):
            return n.args[i] if len(n.args) > i else None
        vals = [(_val(arg(n, 1)), _val(arg(n, 2))) for n in group]
        if any(w is None or sc is None for w, sc in vals):
            continue
        w0, s0 = vals[0]
        same = all(w.shape[0] == w0.shape[0] and sc.shape[0] == s0.shape[0] and sc.dtype == s0.dtype for w, sc in vals)
        same = same and len({arg(n, 3) is None for n in group}) == 1 and len({arg(n, 4) is None for n in group}) == 1
        # parameters must not depend on a member of the group, and every consumer must come after the last member
        members = set(group)
        same = same and not any(_ancestors_include(a, members) for n in group for a in n.args[1:] if a is not None)
        last = group[-1]
        same = same and all(order[u] > order[last] for n in group for u in n.users)
        if not same:
            continue
        with fx_graph.inserting_before(last):
            def make(tgt, args):
                node = fx_graph.call_function(tgt, args)
                node.meta["val"] = _fake(tgt, args)
                return node
            rows = [make(aten.t.default, (arg(n, 1),)) for n in group]                  # [N_i, K/8] each
            wf = make(aten.t.default, (make(aten.cat.default, (rows, 0)),))             # [K/8, sum N_i], strides (1, K/8)
            sf = make(aten.cat.default, ([arg(n, 2) for n in group], 1))
            zf = None if arg(group[0], 3) is None else make(aten.cat.default, ([arg(n, 3) for n in group], 1))
            bf = None if arg(group[0], 4) is None else make(aten.cat.default, ([arg(n, 4) for n in group], 0))
            fused = make(target, (x, wf, sf, zf, bf))
            start = 0
            for n in group:
                width = _val(arg(n, 1)).shape[1]
                piece = make(aten.slice.Tensor, (fused, -1, start, start + width))
                n.replace_all_uses_with(piece)
                start += width
        for n in reversed(group):
            fx_graph.erase_node(n)
        counters["zentorch"]["fused_parallel_woq_linear"] += 1
        fused_groups += 1
    if fused_groups:
        stable_topological_sort(fx_graph)
        fx_graph.lint()
    return fused_groups


def device_gate() -> bool:
    """The replacement of the reference's AVX-512 gate (_optimize.py:87-91)."""
    from . import is_supported_device
    return is_supported_device()


def optimize(fx_graph: torch.fx.Graph, require_device: bool = True) -> torch.fx.Graph:
    """Apply the passes to an ATen-level FX graph (Inductor's joint graph), in the reference's order:
    op replacement, binary-binary fusions, unary fusions."""
    if require_device and not device_gate():
        return fx_graph
    _register_all()
    for p in (replace_pass, binary_pass, unary_pass):
        p.apply(fx_graph)
    stable_topological_sort(fx_graph)
    fx_graph.lint()
    return fx_graph


class OptimizePass:
    """Callable with the interface Inductor expects of ``joint_custom_post_pass``."""

    def __call__(self, graph: torch.fx.Graph) -> None:
        optimize(graph)

    def uuid(self) -> Any:
        return "zentorch_b200_optimize_pass_v1"


def zentorch_b200_backend(gm: torch.fx.GraphModule, example_inputs, **kwargs):
    """``torch.compile(model, backend="zentorch_b200")`` (and ``backend="zentorch"`` when no other package
    has taken that name).  ``options={"cpp_wrapper": True}`` and the other Inductor options pass through."""
    from torch._inductor import config as inductor_config
    from torch._inductor.compile_fx import compile_fx

    options = kwargs.pop("options", None) or {}
    with inductor_config.patch({"joint_custom_post_pass": OptimizePass(), **options}):
        return compile_fx(gm, example_inputs, **kwargs)


@functools.lru_cache(None)
def register_backend() -> None:
    """Registers the Inductor lowerings of the operators and the compile backend.  The reference registers its
    backend as "zentorch" (src/cpu/python/zentorch/_compile_backend.py:93-95); that name is taken here as well
    unless a real zentorch has registered it already, so ``torch.compile(model, backend="zentorch")`` keeps
    working for a model that moved to CUDA."""
    from torch._dynamo import list_backends, register_backend as _reg

    from . import _lowerings
    _lowerings.register()
    _reg(name="zentorch_b200", compiler_fn=zentorch_b200_backend)
    if "zentorch" not in list_backends(exclude_tags=()):
        _reg(name="zentorch", compiler_fn=zentorch_b200_backend)
