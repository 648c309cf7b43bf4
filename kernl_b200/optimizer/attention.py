"""Attention graph rewrites (reference: src/kernl/optimizer/attention.py).

`attention_wrapper` is the call site of the fused kernels: the rewrites replace eager attention
sub-graphs by a call to it. Patterns 1-3 are the reference's (BERT-style `/ 8.0`, T5-style fp32
softmax, bmm-style 3-D tensors); a further rewrite covers what current `transformers` emits:
a direct `scaled_dot_product_attention` call (with its `scale=` literal or the default
head_dim ** -0.5, and grouped-query K/V when `enable_gqa` is set).
"""
from typing import Optional

import torch

from kernl_b200.implementations.attention import attention_forward
from kernl_b200.implementations.attention_skinny import skinny_attention_forward
from kernl_b200.utils.extended_matcher import replace_pattern


def attention_wrapper(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    output: torch.Tensor,
    sm_scale: float,
    is_causal: bool,
    attention_mask: Optional[torch.Tensor],
) -> torch.Tensor:
    """Dispatch between the fused and the decode-shape kernel (reference: optimizer/attention.py:24-55).

    3-D (bmm-style) inputs get a unit head dimension. One query row against more than 50 keys goes
    to the split-KV kernel; the reference sends the masked / causal variant of that shape to eager
    PyTorch (:48-49), here the same kernel handles masks, so nothing leaves the CUDA library.
    """
    extend_head = q.dim() == 3
    if extend_head:
        q, k, v, output = q.unsqueeze(1), k.unsqueeze(1), v.unsqueeze(1), output.unsqueeze(1)
    if attention_mask is not None and attention_mask.dtype == torch.bool:
        # boolean keep-masks (scaled_dot_product_attention convention) become additive 0 / -inf
        attention_mask = torch.zeros_like(attention_mask, dtype=q.dtype).masked_fill_(~attention_mask, float("-inf"))
    # The front-ends return the tensor the kernel wrote: under torch.autocast that is an fp16 copy
    # of a non-fp16 `output`, not `output` itself, so the return value is what goes on.
    if q.size(-2) == 1 and k.size(-2) > 50:
        output = skinny_attention_forward(q, k, v, output, sm_scale, is_causal=is_causal, attention_mask=attention_mask)
    else:
        output = attention_forward(q, k, v, output, sm_scale, is_causal=is_causal, attention_mask=attention_mask)
    if extend_head:
        output = output.squeeze(1)
    return output


torch.fx.wrap("attention_wrapper")


def additive_mask(attention_mask: Optional[torch.Tensor], like: torch.Tensor) -> Optional[torch.Tensor]:
    """A boolean keep-mask (scaled_dot_product_attention convention) as an additive 0 / -inf mask of
    `like`'s dtype; any other mask unchanged. A graph node of its own, so that the layers of a model —
    which all receive the same mask — share ONE conversion instead of three small kernels each."""
    if attention_mask is not None and attention_mask.dtype == torch.bool:
        # Broadcast dimensions (stride 0: the usual [B, 1, M, N] expansion of a [B, N] padding mask)
        # stay broadcast: only one copy of them is converted, and the kernel then sees a per-sequence
        # row mask (staged once per tile, padded key blocks skipped) instead of a dense [M, N] mask.
        shape = attention_mask.shape
        core = attention_mask
        for dim in range(core.dim()):
            if core.stride(dim) == 0 and core.size(dim) > 1:
                core = core.narrow(dim, 0, 1)
        additive = torch.zeros(core.shape, dtype=like.dtype, device=core.device).masked_fill_(~core, float("-inf"))
        return additive.expand(shape)
    return attention_mask


torch.fx.wrap("additive_mask")


def fuse_attention_pattern_1(gm: torch.fx.GraphModule, is_causal: bool):
    """softmax(q·kᵀ / 8.0 + mask)·v (reference: optimizer/attention.py:61-76)."""

    def pattern(q, k, attention_mask, v):
        scores = torch.matmul(q, k.transpose(-1, -2))
        scores = scores / 8.0
        scores = scores + attention_mask
        probs = torch.nn.functional.softmax(scores, dim=-1)
        return torch.matmul(probs, v)

    def replace(q, k, attention_mask, v):
        output = torch.empty_like(q)
        output = attention_wrapper(q, k, v, output, 1 / 8.0, is_causal, attention_mask)
        return output

    replace_pattern(gm, pattern, replace)


def fuse_attention_pattern_2(gm: torch.fx.GraphModule, is_causal: bool):
    """T5 form: unscaled scores + position bias, softmax in fp32, cast back (reference: :79-95)."""

    def pattern(q, k, encoder_decoder_position_bias, v):
        scores = torch.matmul(q, k.transpose(3, 2))
        scores = torch.add(scores, encoder_decoder_position_bias)
        probs = torch.nn.functional.softmax(scores.float(), dim=-1)
        probs = probs.type_as(scores)
        return torch.matmul(probs, v)

    def replace(q, k, encoder_decoder_position_bias, v):
        output = torch.empty_like(q)
        output = attention_wrapper(q, k, v, output, 1.0, is_causal, encoder_decoder_position_bias)
        return output

    replace_pattern(gm, pattern, replace)


def fuse_attention_pattern_3(gm: torch.fx.GraphModule, is_causal: bool):
    """bmm form on [batch*heads, seq, dim] tensors, no mask, no scale (reference: :98-112)."""

    def pattern(q, k, v):
        scores = torch.bmm(q, k.transpose(1, 2))
        probs = torch.nn.functional.softmax(scores, dim=-1)
        return torch.bmm(probs, v)

    def replace(q, k, v):
        output = torch.empty_like(q)
        output = attention_wrapper(q, k, v, output, 1.0, is_causal, None)
        return output

    replace_pattern(gm, pattern, replace)


def fuse_attention_sdpa(gm: torch.fx.GraphModule, is_causal: bool):
    """`F.scaled_dot_product_attention(q, k, v, attn_mask=…, scale=…, is_causal=…)` calls, which is
    what current `transformers` models emit by default. Has no counterpart in the reference (its
    target stack predates the op); literals (scale, is_causal) are read from the node."""
    targets = (torch.nn.functional.scaled_dot_product_attention, torch._C._nn.scaled_dot_product_attention)
    changed = False
    converted = {}  # mask node -> its additive form, built before the first attention that uses it
    for node in list(gm.graph.nodes):
        if node.op != "call_function" or node.target not in targets:
            continue
        args = list(node.args)
        kwargs = dict(node.kwargs)
        q, k, v = args[0], args[1], args[2]
        mask = args[3] if len(args) > 3 else kwargs.get("attn_mask")
        dropout_p = args[4] if len(args) > 4 else kwargs.get("dropout_p", 0.0)
        causal = args[5] if len(args) > 5 else kwargs.get("is_causal", False)
        scale = kwargs.get("scale")
        # enable_gqa needs nothing special: the kernels take k/v with fewer heads than q as they are
        if dropout_p not in (0, 0.0) or isinstance(causal, torch.fx.Node):
            continue
        if isinstance(scale, torch.fx.Node):
            continue
        with gm.graph.inserting_before(node):
            if isinstance(mask, torch.fx.Node):
                if mask not in converted:
                    converted[mask] = gm.graph.call_function(additive_mask, (mask, q))
                mask = converted[mask]
            out = gm.graph.call_function(torch.empty_like, (q,))
            if scale is None:
                head_dim = gm.graph.call_method("size", (q, -1))
                scale = gm.graph.call_function(pow, (head_dim, -0.5))
            fused = gm.graph.call_function(attention_wrapper, (q, k, v, out, scale, bool(causal) or is_causal, mask))
        node.replace_all_uses_with(fused)
        gm.graph.erase_node(node)
        changed = True
    if changed:
        gm.graph.lint()
        gm.recompile()


def _repeated_kv_source(node):
    """If `node` is `x[:, :, None, :, :].expand(B, Hkv, rep, S, D).reshape(B, Hkv * rep, S, D)` — how
    grouped-query models repeat their K/V heads before an ordinary attention — return x."""
    if not (isinstance(node, torch.fx.Node) and node.op == "call_method" and node.target == "reshape"):
        return None
    expand = node.args[0]
    if not (isinstance(expand, torch.fx.Node) and expand.op == "call_method" and expand.target == "expand"):
        return None
    index = expand.args[0]
    import operator

    if not (isinstance(index, torch.fx.Node) and index.op == "call_function" and index.target is operator.getitem):
        return None
    source, key = index.args
    full = slice(None, None, None)
    if not (isinstance(key, tuple) and len(key) == 5 and key[2] is None and all(k == full for i, k in enumerate(key) if i != 2)):
        return None
    exp_shape = expand.args[1:] if len(expand.args) > 2 else tuple(expand.args[1])
    new_shape = node.args[1:] if len(node.args) > 2 else tuple(node.args[1])
    if len(exp_shape) != 5 or len(new_shape) != 4:
        return None
    return source


def fuse_repeat_kv(gm: torch.fx.GraphModule):
    """Grouped-query models (Mistral, Llama 2 70B / 3 families) expand K and V to the number of
    query heads with a copy before attention (`repeat_kv`). The kernels index the shared K/V head
    themselves, so the fused call takes the un-repeated tensors and the copies disappear. Has no
    counterpart in the reference."""
    changed = False
    for node in gm.graph.nodes:
        if node.op != "call_function" or node.target is not attention_wrapper:
            continue
        k_src, v_src = _repeated_kv_source(node.args[1]), _repeated_kv_source(node.args[2])
        if k_src is None or v_src is None:
            continue
        args = list(node.args)
        args[1], args[2] = k_src, v_src
        node.args = tuple(args)
        changed = True
    if changed:
        gm.graph.eliminate_dead_code()
        gm.graph.lint()
        gm.recompile()
