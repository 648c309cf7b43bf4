"""Dropout is the identity at inference time: drop the nodes (reference: src/kernl/optimizer/dropout.py)."""
import torch


def remove_dropout(gm: torch.fx.GraphModule):
    modules = dict(gm.named_modules())
    for node in list(gm.graph.nodes):
        is_module = node.op == "call_module" and isinstance(modules.get(node.target), torch.nn.Dropout)
        is_function = node.op == "call_function" and node.target is torch.nn.functional.dropout
        if is_module or is_function:
            node.replace_all_uses_with(node.args[0])
            gm.graph.erase_node(node)
    gm.recompile()
