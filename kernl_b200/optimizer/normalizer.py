"""In-place operators → functional equivalents, so that patterns written with `+`, `torch.add`,
... match graphs traced from code that uses `+=` (reference: src/kernl/optimizer/normalizer.py)."""
import functools
import operator

import torch

# in-place operator `operator.i<name>` -> the out-of-place torch function with the same meaning
_OUT_OF_PLACE = {
    "add": torch.add, "sub": torch.sub, "mul": torch.mul, "matmul": torch.matmul, "pow": torch.pow,
    "truediv": torch.div, "floordiv": functools.partial(torch.div, rounding_mode="floor"), "mod": torch.remainder,
    "and": torch.bitwise_and, "or": torch.bitwise_or, "xor": torch.bitwise_xor,
}
NORMALIZED_OPERATORS = {getattr(operator, "i" + name): fn for name, fn in _OUT_OF_PLACE.items()}


def normalize_operators(gm: torch.fx.GraphModule):
    for node in list(gm.graph.nodes):
        if node.op == "call_function" and node.target in NORMALIZED_OPERATORS:
            with gm.graph.inserting_after(node):
                functional = gm.graph.call_function(NORMALIZED_OPERATORS[node.target], node.args, node.kwargs)
            node.replace_all_uses_with(functional)
            gm.graph.erase_node(node)
    gm.recompile()


def replace_scalar_tensor_constants(gm: torch.fx.GraphModule):
    """`torch.tensor(<python number>, device=cuda)` builds the value on the host and copies it to the
    device, which is not allowed while a CUDA graph is being captured. `torch.full((), value)` fills
    on the device and gives the same 0-d tensor. Current `transformers` emits such constants when
    it builds additive masks; the reference's target stack did not, so this pass has no
    counterpart there."""
    for node in list(gm.graph.nodes):
        if node.op != "call_function" or node.target is not torch.tensor or len(node.args) != 1:
            continue
        value = node.args[0]
        if isinstance(value, bool) or not isinstance(value, (int, float)):
            continue
        kwargs = {k: v for k, v in node.kwargs.items() if k in ("dtype", "device")}
        if "dtype" not in kwargs:
            kwargs["dtype"] = torch.float32 if isinstance(value, float) else torch.int64
        with gm.graph.inserting_after(node):
            filled = gm.graph.call_function(torch.full, ((), value), kwargs)
        node.replace_all_uses_with(filled)
        gm.graph.erase_node(node)
    gm.recompile()
