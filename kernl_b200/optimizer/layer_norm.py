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


def layer_norm_residual_sum_wrapper(a: torch.Tensor, b: torch.Tensor, layernorm: torch.nn.LayerNorm):
    """(LayerNorm(a + b), a + b) from one kernel, for blocks that keep the sum as their residual."""
    if layernorm.weight.dtype == torch.float32:
        layernorm.weight.data = layernorm.weight.data.half()
    if layernorm.bias is not None and layernorm.bias.dtype == torch.float32:
        layernorm.bias.data = layernorm.bias.data.half()
    fits = (a.shape == b.shape and a.dtype == b.dtype and a.dtype in (torch.float16, torch.bfloat16)
            and a.shape[-1] % 8 == 0 and a.shape[-1] <= 6144)
    if not fits:
        total = a + b
        return layer_norm(total, layernorm.weight, layernorm.bias, layernorm.eps), total
    return layer_norm(a, layernorm.weight, layernorm.bias, layernorm.eps, residual=b)


torch.fx.wrap("layer_norm_residual_wrapper")
torch.fx.wrap("layer_norm_residual_sum_wrapper")


def fuse_add_layer_norm(gm: torch.fx.GraphModule):
    """`layer_norm_wrapper(a + b, ln)` becomes one call whose kernel adds and normalises: where the sum
    has no other reader (the post-LayerNorm residual of BERT-style blocks) it returns the normalised
    tensor; where it has (pre-LayerNorm blocks: Whisper, GPT-2, ViT) it returns the sum as well. Not in the reference; an
    elementwise add at batch 1 is a 2-3 µs launch, and there are two per block. Runs after
    `replace_layer_norm`."""
    import operator

    changed = False
    for n in list(gm.graph.nodes):
        if n.op != "call_function" or n.target is not layer_norm_wrapper or len(n.args) != 2:
            continue
        src = n.args[0]
        if not isinstance(src, torch.fx.Node):
            continue
        is_add = (src.op == "call_function" and src.target in (operator.add, torch.add)) or (
            src.op == "call_method" and src.target == "add")
        if not is_add or len(src.args) != 2 or src.kwargs:
            continue
        a, b = src.args
        if not (isinstance(a, torch.fx.Node) and isinstance(b, torch.fx.Node)):
            continue
        if len(src.users) == 1:
            with gm.graph.inserting_before(n):
                fused = gm.graph.call_function(layer_norm_residual_wrapper, (a, b, n.args[1]))
            n.replace_all_uses_with(fused)
            gm.graph.erase_node(n)
            gm.graph.erase_node(src)
        else:
            # pre-LayerNorm blocks: the sum is also the next residual; the kernel stores it
            module_node = n.args[1]
            if not (isinstance(module_node, torch.fx.Node) and module_node.op == "get_attr"):
                continue
            src.prepend(module_node)
            with gm.graph.inserting_after(src):
                fused = gm.graph.call_function(layer_norm_residual_sum_wrapper, (a, b, module_node))
            with gm.graph.inserting_after(fused):
                normed = gm.graph.call_function(operator.getitem, (fused, 0))
                total = gm.graph.call_function(operator.getitem, (fused, 1))
            n.replace_all_uses_with(normed)
            gm.graph.erase_node(n)
            src.replace_all_uses_with(total)
            gm.graph.erase_node(src)
        changed = True
    if changed:
        gm.graph.lint()
        gm.recompile()
    return gm


# ------------------------------------------------------------------------------------------------
# RMSNorm as current decoder models spell it, and its residual add
# ------------------------------------------------------------------------------------------------
def _is_call(n, kind: str, *targets) -> bool:
    return isinstance(n, torch.fx.Node) and n.op == kind and n.target in targets


def _match_rms_norm(out: torch.fx.Node):
    """`weight * (h * rsqrt(h32.pow(2).mean(-1, keepdim=True) + eps)).to(dtype)` with
    h32 = x.to(float32) and h either h32 (Llama-style modules) or x itself (T5 style), eps any float.
    Returns (x, weight, eps, [interior nodes from the output inwards]) or None."""
    import operator

    mul = (operator.mul, torch.mul)
    if not _is_call(out, "call_function", *mul) or len(out.args) != 2 or out.kwargs:
        return None
    for weight, scaled in ((out.args[0], out.args[1]), (out.args[1], out.args[0])):
        if not (isinstance(weight, torch.fx.Node) and weight.op == "get_attr"):
            continue
        interior = []
        cast = scaled
        if _is_call(cast, "call_method", "to") and len(cast.args) == 2 and isinstance(cast.args[1], torch.dtype) and not cast.kwargs:
            interior.append(cast)
            scaled = cast.args[0]
        if not _is_call(scaled, "call_function", *mul) or len(scaled.args) != 2 or scaled.kwargs:
            continue
        for h, r in ((scaled.args[0], scaled.args[1]), (scaled.args[1], scaled.args[0])):
            if not _is_call(r, "call_function", torch.rsqrt) or len(r.args) != 1:
                continue
            add = r.args[0]
            if not _is_call(add, "call_function", operator.add, torch.add) or len(add.args) != 2 or add.kwargs:
                continue
            var, eps = add.args
            if not isinstance(eps, float):
                continue
            if not (_is_call(var, "call_method", "mean") and len(var.args) == 2 and var.args[1] == -1
                    and var.kwargs == {"keepdim": True}):
                continue
            pw = var.args[0]
            if not (_is_call(pw, "call_method", "pow") and len(pw.args) == 2 and pw.args[1] == 2 and not pw.kwargs):
                continue
            h32 = pw.args[0]
            if not (_is_call(h32, "call_method", "to") and len(h32.args) == 2 and h32.args[1] is torch.float32 and not h32.kwargs):
                continue
            x = h32.args[0]
            if h is not h32 and h is not x:
                continue
            chain = interior + [scaled, r, add, var, pw]
            if any(len(n.users) != 1 for n in chain):
                continue
            if set(h32.users) - {pw, scaled}:
                continue
            return x, weight, eps, chain + [h32]
    return None


def replace_rms_norm_any_eps(gm: torch.fx.GraphModule):
    """RMSNorm written out in eager ops with whatever epsilon the model carries (Llama-family
    decoders: `hidden.to(float32)`, mean of squares, rsqrt, cast back, times weight) → the RMSNorm
    kernel. The reference only knows T5's form with the literal 1e-06 (optimizer/layer_norm.py:60-74),
    which `replace_layer_norm_rms` has already taken when this pass runs."""
    changed = False
    for n in list(gm.graph.nodes):
        m = _match_rms_norm(n)
        if m is None:
            continue
        x, weight, eps, interior = m
        with gm.graph.inserting_before(n):
            fused = gm.graph.call_function(layer_norm_rms_wrapper, (x, weight, eps))
        n.replace_all_uses_with(fused)
        gm.graph.erase_node(n)
        for node in interior:
            if len(node.users) == 0:
                gm.graph.erase_node(node)
        changed = True
    if changed:
        gm.graph.lint()
        gm.recompile()
    return gm


def layer_norm_rms_residual_wrapper(a: torch.Tensor, b: torch.Tensor, weight: torch.Tensor, eps: float):
    """(RMSNorm(a + b), a + b): the residual add of a pre-norm block runs inside the norm kernel, which
    also stores the sum for the next residual connection."""
    if weight.dtype == torch.float32 and a.dtype == torch.float16:
        weight.data = weight.data.half()
    fits = (a.shape == b.shape and a.dtype == b.dtype and a.dtype in (torch.float16, torch.bfloat16)
            and a.shape[-1] % 8 == 0 and a.shape[-1] <= 6144)
    if not fits:
        total = a + b
        return layer_norm(total, weight, None, eps, use_rms_norm=True), total
    return layer_norm(a, weight, None, eps, use_rms_norm=True, residual=b)


torch.fx.wrap("layer_norm_rms_residual_wrapper")


def fuse_add_rms_norm(gm: torch.fx.GraphModule):
    """`layer_norm_rms_wrapper(a + b, w, eps)` becomes one call that returns the normalised tensor AND
    the sum; other readers of `a + b` (the next residual connection of a pre-norm block) take the
    stored sum. Not in the reference. Runs after the RMSNorm rewrites."""
    import operator

    changed = False
    for n in list(gm.graph.nodes):
        if not _is_call(n, "call_function", layer_norm_rms_wrapper) or len(n.args) != 3 or n.kwargs:
            continue
        src, weight, eps = n.args
        if not _is_call(src, "call_function", operator.add, torch.add) or len(src.args) != 2 or src.kwargs:
            continue
        a, b = src.args
        if not (isinstance(a, torch.fx.Node) and isinstance(b, torch.fx.Node) and isinstance(weight, torch.fx.Node)):
            continue
        if weight.op != "get_attr":
            continue
        src.prepend(weight)  # the parameter has no inputs: it may sit anywhere before its first reader
        with gm.graph.inserting_after(src):
            fused = gm.graph.call_function(layer_norm_rms_residual_wrapper, (a, b, weight, eps))
        with gm.graph.inserting_after(fused):
            normed = gm.graph.call_function(operator.getitem, (fused, 0))
            total = gm.graph.call_function(operator.getitem, (fused, 1))
        n.replace_all_uses_with(normed)
        gm.graph.erase_node(n)
        src.replace_all_uses_with(total)
        gm.graph.erase_node(src)
        changed = True
    if changed:
        gm.graph.lint()
        gm.recompile()
    return gm

