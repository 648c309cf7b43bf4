"""LayerNorm / RMSNorm graph rewrites (reference: src/kernl/optimizer/layer_norm.py)."""
import torch

from kernl_b200.implementations.layer_norm import layer_norm
from kernl_b200.utils.extended_matcher import replace_pattern


def layer_norm_wrapper(v: torch.Tensor, layernorm: torch.nn.LayerNorm):
    """fp32 affine parameters are converted to fp16 in place once (reference: optimizer/layer_norm.py:22-29)."""
    if layernorm.weight.dtype == torch.float32:
        layernorm.weight.data = layernorm.weight.data.half()
    if layernorm.bias is not None and layernorm.bias.dtype == torch.float32:
        layernorm.bias.data = layernorm.bias.data.half()
    return layer_norm(v, layernorm.weight, layernorm.bias, layernorm.eps)


def layer_norm_rms_wrapper(v: torch.Tensor, weight: torch.Tensor, eps: float):
    if weight.dtype == torch.float32 and v.dtype == torch.float16:
        weight.data = weight.data.half()
    return layer_norm(v, weight, None, eps, use_rms_norm=True)


torch.fx.wrap("layer_norm_wrapper")
torch.fx.wrap("layer_norm_rms_wrapper")


def replace_layer_norm(gm: torch.fx.GraphModule):
    """nn.LayerNorm modules (reference: optimizer/layer_norm.py:40-57)."""

    class Pattern(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.layernorm = torch.nn.LayerNorm((1, 1))

        def forward(self, v):
            return self.layernorm(v)

    class Replacement(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.layernorm = torch.nn.LayerNorm((1, 1))

        def forward(self, v):
            return layer_norm_wrapper(v, self.layernorm)

    replace_pattern(gm, Pattern(), Replacement())


def replace_layer_norm_rms(gm: torch.fx.GraphModule):
    """The T5 LayerNorm expression with its literal eps 1e-06 (reference: optimizer/layer_norm.py:60-74)."""

    def pattern(v, weight):
        variance = v.to(torch.float32).pow(2).mean(-1, keepdim=True)
        variance = variance + 1e-06
        scaled = v * torch.rsqrt(variance)
        return weight * scaled

    def replace(v, weight):
        return layer_norm_rms_wrapper(v, weight, 1e-06)

    replace_pattern(gm, pattern, replace)
