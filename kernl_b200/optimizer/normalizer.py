"""In-place operators → functional equivalents, so that patterns written with `+`, `torch.add`,
... match graphs traced from code that uses `+=` (reference: src/kernl/optimizer/normalizer.py)."""
import functools
import operator

import torch

NORMALIZED_OPERATORS = {
    operator.iadd: torch.add,
    operator.iand: torch.bitwise_and,
    operator.ifloordiv: functools.partial(torch.div, rounding_mode="floor"),
    operator.imod: torch.remainder,
    operator.imul: torch.mul,
    operator.imatmul: torch.matmul,
    operator.ior: torch.bitwise_or,
    operator.ipow: torch.pow,
    operator.isub: torch.sub,
    operator.itruediv: torch.div,
    operator.ixor: torch.bitwise_xor,
}


def normalize_operators(gm: torch.fx.GraphModule):
    for node in list(gm.graph.nodes):
        if node.op == "call_function" and node.target in NORMALIZED_OPERATORS:
            with gm.graph.inserting_after(node):
                functional = gm.graph.call_function(NORMALIZED_OPERATORS[node.target], node.args, node.kwargs)
            node.replace_all_uses_with(functional)
            gm.graph.erase_node(node)
    gm.recompile()
