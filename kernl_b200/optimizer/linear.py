"""Linear-layer graph rewrites (reference: src/kernl/optimizer/linear.py)."""
from typing import Callable

import torch

from kernl_b200.implementations.linear_layer import linear_layer
from kernl_b200.utils.extended_matcher import replace_pattern


def linear_wrapper(v: torch.Tensor, linear: torch.nn.Linear, activation=""):
    return linear_wrapper_functional(v, linear.weight, linear.bias, activation=activation)


torch.fx.wrap("linear_wrapper")


def linear_wrapper_functional(v: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, activation=""):
    """fp32 parameters are converted to fp16 IN PLACE the first time they are seen, so the cast is
    paid once and not per call (reference: optimizer/linear.py:31-38)."""
    if weight.dtype == torch.float32:
        weight.data = weight.data.half()
    if bias is not None and bias.dtype == torch.float32:
        bias.data = bias.data.half()
    return linear_layer(v, weight, bias, activation=activation)


torch.fx.wrap("linear_wrapper_functional")


class _EagerLinear(torch.nn.Module):
    """What the models contain: an nn.Linear, optionally followed by an activation (a module such
    as nn.Tanh() or a function such as F.gelu)."""

    def __init__(self, activation_fn=None):
        super().__init__()
        self.linear = torch.nn.Linear(1, 1)
        self.activation = activation_fn

    def forward(self, v):
        out = self.linear(v)
        return out if self.activation is None else self.activation(out)


class _KernelLinear(torch.nn.Module):
    """What replaces it: one call of the fused kernel, the activation named by its string."""

    def __init__(self, activation_name=""):
        super().__init__()
        self.linear = torch.nn.Linear(1, 1)
        self.activation_name = activation_name

    def forward(self, v):
        return linear_wrapper(v, self.linear, activation=self.activation_name)


def replace_linear_activation(gm: torch.fx.GraphModule, activation_module: Callable, activation: str):
    """nn.Linear followed by an activation → one fused call (reference: optimizer/linear.py:44-66)."""
    replace_pattern(gm, _EagerLinear(activation_module), _KernelLinear(activation))


def replace_linear(gm: torch.fx.GraphModule):
    """Bare nn.Linear modules (reference: optimizer/linear.py:69-86)."""
    replace_pattern(gm, _EagerLinear(), _KernelLinear())


def replace_linear_fn(gm: torch.fx.GraphModule):
    """F.linear(v, weight, bias) calls (reference: optimizer/linear.py:89-98), and the same call with
    a literal None for the bias, which has to be part of the pattern to match (:101-110)."""
    replace_pattern(gm, lambda v, weight, bias: torch.nn.functional.linear(v, weight, bias),
                    lambda v, weight, bias: linear_wrapper_functional(v, weight, bias))


def replace_linear_fn_constant_match(gm: torch.fx.GraphModule):
    replace_pattern(gm, lambda v, weight: torch.nn.functional.linear(v, weight, None),
                    lambda v, weight: linear_wrapper_functional(v, weight, None))


class FusedLinear(torch.nn.Linear):
    """Several nn.Linear modules that read the same input, stacked along the output dimension."""

    def __init__(self, linears):
        first = linears[0]
        out_features = sum(l.out_features for l in linears)
        super().__init__(first.in_features, out_features, bias=first.bias is not None,
                         device=first.weight.device, dtype=first.weight.dtype)
        with torch.no_grad():
            self.weight.copy_(torch.cat([l.weight for l in linears], dim=0))
            if self.bias is not None:
                self.bias.copy_(torch.cat([l.bias for l in linears], dim=0))
        self.requires_grad_(False)


def fuse_parallel_linears(gm: torch.fx.GraphModule):
    """Bare linears that read the same tensor (the q, k and v projections of an attention block, the
    k and v projections of a cross-attention) become ONE linear over the stacked weights; each
    original output is a column slice of its result (a strided view, which the attention kernel's
    tensor maps take as they are). Not in the reference: there a projection at batch 1 is a 7 µs
    kernel of which most is fixed cost, and three of them per block are a fifth of BERT's latency.
    Runs after `replace_all_linear`; linears with a fused activation are left alone."""
    import operator

    groups = {}
    for n in gm.graph.nodes:
        if n.op != "call_function" or n.target is not linear_wrapper or len(n.args) != 2:
            continue
        if n.kwargs.get("activation", ""):
            continue
        mod_node = n.args[1]
        if not isinstance(mod_node, torch.fx.Node) or mod_node.op != "get_attr":
            continue
        try:
            lin = gm.get_submodule(mod_node.target)
        except AttributeError:
            continue
        if type(lin) is not torch.nn.Linear:
            continue
        key = (n.args[0], lin.in_features, lin.bias is not None, lin.weight.dtype, str(lin.weight.device))
        groups.setdefault(key, []).append((n, lin))
    fused_count = 0
    for (v, *_), members in groups.items():
        if len(members) < 2:
            continue
        name = f"kernl_fused_linear_{fused_count}"
        fused_count += 1
        gm.add_submodule(name, FusedLinear([lin for _, lin in members]))
        order = {node: i for i, node in enumerate(gm.graph.nodes)}
        first = min((n for n, _ in members), key=lambda node: order[node])
        with gm.graph.inserting_before(first):
            mod = gm.graph.get_attr(name)
            fused = gm.graph.call_function(linear_wrapper, (v, mod))
            start = 0
            for n, lin in members:
                piece = gm.graph.call_function(operator.getitem, (fused, (Ellipsis, slice(start, start + lin.out_features))))
                start += lin.out_features
                n.replace_all_uses_with(piece)
        for n, _ in members:
            mod_node = n.args[1]
            gm.graph.erase_node(n)
            if len(mod_node.users) == 0:
                gm.graph.erase_node(mod_node)
    if fused_count:
        gm.graph.lint()
        gm.recompile()
    return gm


def replace_all_linear(gm: torch.fx.GraphModule):
    """Fused variants first, then what is left (reference: optimizer/linear.py:113-119). The
    nn.GELU / nn.SiLU module forms are additions for current model code."""
    replace_linear_activation(gm, torch.nn.Tanh(), "tanh")
    replace_linear_activation(gm, torch.nn.ReLU(), "relu")
    replace_linear_activation(gm, torch.nn.functional.gelu, "gelu")
    replace_linear_activation(gm, torch.nn.GELU(), "gelu")
    replace_linear(gm)
    replace_linear_fn(gm)
    replace_linear_fn_constant_match(gm)
