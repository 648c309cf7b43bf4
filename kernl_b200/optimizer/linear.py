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


def replace_linear_activation(gm: torch.fx.GraphModule, activation_module: Callable, activation: str):
    """nn.Linear followed by an activation → one fused call (reference: optimizer/linear.py:44-66)."""

    class Pattern(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.linear = torch.nn.Linear(1, 1)
            self.activation = activation_module

        def forward(self, v):
            return self.activation(self.linear(v))

    class Replacement(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.linear = torch.nn.Linear(1, 1)
            self.activation = activation_module

        def forward(self, v):
            return linear_wrapper(v, self.linear, activation=activation)

    replace_pattern(gm, Pattern(), Replacement())


def replace_linear(gm: torch.fx.GraphModule):
    """Bare nn.Linear modules (reference: optimizer/linear.py:69-86)."""

    class Pattern(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.linear = torch.nn.Linear(1, 1)

        def forward(self, v):
            return self.linear(v)

    class Replacement(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.linear = torch.nn.Linear(1, 1)

        def forward(self, v):
            return linear_wrapper(v, self.linear)

    replace_pattern(gm, Pattern(), Replacement())


def replace_linear_fn(gm: torch.fx.GraphModule):
    """F.linear(v, weight, bias) calls (reference: optimizer/linear.py:89-98)."""

    def pattern(v, weight, bias):
        return torch.nn.functional.linear(v, weight, bias)

    def replace(v, weight, bias):
        return linear_wrapper_functional(v, weight, bias)

    replace_pattern(gm, pattern, replace)


def replace_linear_fn_constant_match(gm: torch.fx.GraphModule):
    """F.linear(v, weight, None): the literal None has to be part of the pattern
    (reference: optimizer/linear.py:101-110)."""

    def pattern(v, weight):
        return torch.nn.functional.linear(v, weight, None)

    def replace(v, weight):
        return linear_wrapper_functional(v, weight, None)

    replace_pattern(gm, pattern, replace)


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
