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


def layer_norm_residual_wrapper(a: torch.Tensor, b: torch.Tensor, layernorm: torch.nn.LayerNorm):
    """LayerNorm(a + b): the add runs inside the norm kernel."""
    if layernorm.weight.dtype == torch.float32:
        layernorm.weight.data = layernorm.weight.data.half()
    if layernorm.bias is not None and layernorm.bias.dtype == torch.float32:
        layernorm.bias.data = layernorm.bias.data.half()
    if a.shape != b.shape or a.dtype != b.dtype or a.shape[-1] % 8 != 0 or a.shape[-1] > 6144:
        return layer_norm(a + b, layernorm.weight, layernorm.bias, layernorm.eps)
    y, _ = layer_norm(a, layernorm.weight, layernorm.bias, layernorm.eps, residual=b)
    return y


torch.fx.wrap("layer_norm_residual_wrapper")


def fuse_add_layer_norm(gm: torch.fx.GraphModule):
    """`layer_norm_wrapper(a + b, ln)` where the sum has no other reader (the post-LayerNorm residual of
    BERT-style blocks) becomes one call whose kernel adds and normalises. Not in the reference; an
    elementwise add at batch 1 is a 2-3 µs launch, and there are two per block. Runs after
    `replace_layer_norm`."""
    import operator

    changed = False
    for n in list(gm.graph.nodes):
        if n.op != "call_function" or n.target is not layer_norm_wrapper or len(n.args) != 2:
            continue
        src = n.args[0]
        if not isinstance(src, torch.fx.Node) or len(src.users) != 1:
            continue
        is_add = (src.op == "call_function" and src.target in (operator.add, torch.add)) or (
            src.op == "call_method" and src.target == "add")
        if not is_add or len(src.args) != 2 or src.kwargs:
            continue
        a, b = src.args
        if not (isinstance(a, torch.fx.Node) and isinstance(b, torch.fx.Node)):
            continue
        with gm.graph.inserting_before(n):
            fused = gm.graph.call_function(layer_norm_residual_wrapper, (a, b, n.args[1]))
        n.replace_all_uses_with(fused)
        gm.graph.erase_node(n)
        gm.graph.erase_node(src)
        changed = True
    if changed:
        gm.graph.lint()
        gm.recompile()
    return gm
