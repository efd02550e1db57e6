"""Inductor lowerings of the zentorch quantized-linear operators for CUDA graphs.

Without a lowering Inductor treats ``torch.ops.zentorch.*`` as opaque fallback kernels; under ``cpp_wrapper``
that means a round trip through the Python dispatcher for every call.  The reference lowers each operator to
an ``ExternKernelAlloc`` node whose C++ name is the operator's AOTInductor shim
(src/cpu/python/zentorch/_lowerings.py:1399-1701 for the weight-only int4 family, :1870-1951 for
``zentorch_dynamic_qlinear``), so that generated C++ calls ``aoti_torch_cpu_zentorch_*`` directly.  This module
does the same for CUDA tensors: the shim name is built from the device type of the first input
(``aoti_torch_cuda_zentorch_*``, exported by ``libzentorch_b200_torch.so`` and declared in
``include/shim_cuda_zentorch.h``), the Python wrapper path keeps calling the operator overload.

As in the reference, only the activation is forced contiguous at the IR level; the packed weight and the
scale tables are merely realized (the packed weight is a strided view whose layout is the contract,
src/cpu/python/zentorch/_lowerings.py:1445-1453).

One table drives everything: for each operator the tensor arguments in schema order, each required or
optional.  Present tensors become the node's inputs; ``codegen_args`` puts ``None`` back where an optional
tensor is absent, so that positional order matches the schema in both wrapper flavours.
"""
from __future__ import annotations

from pathlib import Path

import torch
from torch._inductor.ir import ExternKernelAlloc, FixedLayout, TensorBox
from torch._inductor.lowering import register_lowering
from torch._inductor.virtualized import V

SHIM_HEADER = str(Path(__file__).resolve().parent.parent.parent / "include" / "shim_cuda_zentorch.h")

_REQ, _OPT = True, False
_WOQ_HEAD = (("input", _REQ), ("weight", _REQ), ("weight_scales", _REQ), ("weight_zero_points", _OPT))
# operator -> (tensor arguments in schema order, index of the argument whose last dimension gives out_features,
#              which dimension of it)
_OPS = {
    "zentorch_woq_linear": (_WOQ_HEAD + (("bias", _OPT),), 1, 1),
    "zentorch_woq_linear_relu": (_WOQ_HEAD + (("bias", _OPT),), 1, 1),
    "zentorch_woq_linear_sigmoid": (_WOQ_HEAD + (("bias", _OPT),), 1, 1),
    "zentorch_woq_linear_gelu_tanh": (_WOQ_HEAD + (("bias", _OPT),), 1, 1),
    "zentorch_woq_linear_gelu_erf": (_WOQ_HEAD + (("bias", _OPT),), 1, 1),
    "zentorch_woq_linear_add": (_WOQ_HEAD + (("add_input", _REQ), ("bias", _OPT)), 1, 1),
    "zentorch_woq_linear_mul_add": (_WOQ_HEAD + (("mul_input", _REQ), ("add_input", _REQ), ("bias", _OPT)), 1, 1),
    "zentorch_woq_linear_add_add": (_WOQ_HEAD + (("add_input", _REQ), ("add_input_2", _REQ), ("bias", _OPT)), 1, 1),
    "zentorch_dynamic_qlinear": ((("input", _REQ), ("weight", _REQ), ("weight_scales", _REQ), ("bias", _OPT)), 1, 0),
}


class ZentorchExternLinear(ExternKernelAlloc):
    """One zentorch linear as an extern kernel: inputs are the tensors that are present, `present` says which
    schema slots they fill."""

    def __init__(self, layout, inputs, present, op_overload, shim_name, kwargs):
        super().__init__(layout, inputs, (), kwargs, op_overload=op_overload, cpp_kernel_name=shim_name)
        self.present = tuple(present)

    def codegen(self, wrapper):
        if V.graph.cpp_wrapper:
            wrapper.include_extra_header(SHIM_HEADER)
        super().codegen(wrapper)

    def codegen_args(self):
        tensors = iter(self.inputs)
        ordered = [next(tensors) if here else None for here in self.present]
        to_str = V.graph.wrapper_code.val_to_arg_str
        if V.graph.cpp_wrapper:
            # positional arguments the schema has beyond the tensors (none today) come from kwargs / defaults
            ordered = list(self.fill_non_provided_args(ordered, self.kwargs))
            return [to_str(v, self.arg_properties[i].get("type")) for i, v in enumerate(ordered)]
        return [to_str(v) for v in ordered]

    def apply_constraint(self):
        pass


def _make_lowering(op_name, slots, out_arg, out_dim):
    overload = getattr(torch.ops.zentorch, op_name).default

    def lowering(*args, zentorch_op_name=f"zentorch::{op_name}"):
        assert len(args) <= len(slots), f"{op_name}: too many positional arguments"
        args = list(args) + [None] * (len(slots) - len(args))
        # the activation is made contiguous here so that the operator's own contiguity fix-up never copies;
        # everything else (the packed weight above all) keeps its strides
        x = ExternKernelAlloc.require_contiguous(ExternKernelAlloc.realize_input(args[0]))
        inputs, present = [x], [True]
        for (name, required), value in zip(slots[1:], args[1:]):
            if value is None:
                assert not required, f"{op_name}: {name} is required"
                present.append(False)
                continue
            value.realize()
            inputs.append(value)
            present.append(True)
        *lead, _k = x.get_size()
        out_features = args[out_arg].get_size()[out_dim]
        device = x.get_device()
        assert device is not None
        node = ZentorchExternLinear(
            FixedLayout(device=device, dtype=x.get_dtype(), size=[*lead, out_features]), inputs, present, overload,
            f"aoti_torch_{device.type}_{op_name}", {"zentorch_op_name": zentorch_op_name})
        return TensorBox.create(node)

    lowering.__name__ = f"{op_name}_lowering"
    return lowering


_registered = False


def register() -> None:
    """Registers the lowerings (idempotent).  Called when the compile backend is set up."""
    global _registered
    if _registered:
        return
    for op_name, (slots, out_arg, out_dim) in _OPS.items():
        overload = getattr(torch.ops.zentorch, op_name).default
        register_lowering(overload, type_promotion_kind=None)(_make_lowering(op_name, slots, out_arg, out_dim))
    _registered = True
