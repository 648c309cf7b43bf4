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


class GatedLinear(torch.nn.Linear):
    """The gate and up projections of a gated feed-forward as ONE weight whose rows alternate in
    blocks of eight (eight gate rows, the matching eight up rows, ...): the layout the kernel's
    "swiglu" epilogue reads. `out_features` counts both halves; the call returns half as many columns."""

    def __init__(self, gate: torch.nn.Linear, up: torch.nn.Linear):
        from kernl_b200.implementations.linear_layer import interleave_gate_up

        super().__init__(gate.in_features, 2 * gate.out_features, bias=gate.bias is not None,
                         device=gate.weight.device, dtype=gate.weight.dtype)
        with torch.no_grad():
            self.weight.copy_(interleave_gate_up(gate.weight, up.weight))
            if self.bias is not None:
                self.bias.copy_(interleave_gate_up(gate.bias, up.bias))
        self.requires_grad_(False)


def _bare_linear(gm: torch.fx.GraphModule, n, exact: bool = True):
    """The nn.Linear behind a `linear_wrapper(v, module)` node without a fused activation, else None.
    `exact=False` also accepts the subclasses this package builds (stacked, transposed weights)."""
    if not isinstance(n, torch.fx.Node) or n.op != "call_function" or n.target is not linear_wrapper:
        return None
    if len(n.args) != 2 or n.kwargs.get("activation", ""):
        return None
    mod_node = n.args[1]
    if not isinstance(mod_node, torch.fx.Node) or mod_node.op != "get_attr":
        return None
    try:
        lin = gm.get_submodule(mod_node.target)
    except AttributeError:
        return None
    if exact:
        return lin if type(lin) is torch.nn.Linear else None
    return lin if isinstance(lin, torch.nn.Linear) else None


def _is_silu(gm: torch.fx.GraphModule, n) -> bool:
    if not isinstance(n, torch.fx.Node) or len(n.args) != 1 or set(n.kwargs) - {"inplace"}:
        return False
    if n.op == "call_function":
        return n.target is torch.nn.functional.silu
    if n.op == "call_module":
        return type(gm.get_submodule(n.target)) is torch.nn.SiLU
    return False


def fuse_gated_feed_forward(gm: torch.fx.GraphModule):
    """silu(gate(x)) * up(x) — the feed-forward of Llama-style decoders — becomes one linear over the
    interleaved gate/up weight whose epilogue does the gating, so the two [tokens, F] projections
    are never written out. Not in the reference's dispatched path (its experimental
    llama-v2/kernel/fused_kernel_ff.py:10-114 fuses the same three ops). Runs after
    `replace_all_linear` and before `fuse_parallel_linears` (which would otherwise stack gate and
    up as plain columns). Skipped unless both projections read the same tensor, have the same shape
    with a multiple of eight outputs, agree on having a bias, and feed nothing else."""
    import operator

    fused_count = 0
    for n in list(gm.graph.nodes):
        if n.op != "call_function" or n.target not in (operator.mul, torch.mul) or len(n.args) != 2 or n.kwargs:
            continue
        for act, up in ((n.args[0], n.args[1]), (n.args[1], n.args[0])):
            if not _is_silu(gm, act):
                continue
            gate = act.args[0]
            gate_lin, up_lin = _bare_linear(gm, gate), _bare_linear(gm, up)
            if gate_lin is None or up_lin is None or gate is up:
                continue
            if gate.args[0] is not up.args[0] or len(act.users) != 1 or len(gate.users) != 1 or len(up.users) != 1:
                continue
            if (gate_lin.weight.shape != up_lin.weight.shape or gate_lin.out_features % 8 != 0
                    or (gate_lin.bias is None) != (up_lin.bias is None)
                    or gate_lin.weight.dtype != up_lin.weight.dtype or gate_lin.weight.device != up_lin.weight.device):
                continue
            name = f"kernl_gated_linear_{fused_count}"
            while hasattr(gm, name):
                fused_count += 1
                name = f"kernl_gated_linear_{fused_count}"
            fused_count += 1
            gm.add_submodule(name, GatedLinear(gate_lin, up_lin))
            with gm.graph.inserting_before(n):
                mod = gm.graph.get_attr(name)
                fused = gm.graph.call_function(linear_wrapper, (gate.args[0], mod), {"activation": "swiglu"})
            n.replace_all_uses_with(fused)
            gm.graph.erase_node(n)
            gm.graph.erase_node(act)
            for lin_node in (gate, up):
                mod_node = lin_node.args[1]
                gm.graph.erase_node(lin_node)
                if len(mod_node.users) == 0:
                    gm.graph.erase_node(mod_node)
            break
    if fused_count:
        gm.graph.lint()
        gm.recompile()
    return gm


class TransposedLinear(torch.nn.Linear):
    """An nn.Linear built from a [in, out] weight (the layout of `transformers`' Conv1D, which
    computes addmm(bias, x, weight)): the kernel streams W as [out, in] rows."""

    def __init__(self, weight_in_out: torch.Tensor, bias):
        super().__init__(weight_in_out.shape[0], weight_in_out.shape[1], bias=bias is not None,
                         device=weight_in_out.device, dtype=weight_in_out.dtype)
        with torch.no_grad():
            self.weight.copy_(weight_in_out.t())
            if bias is not None:
                self.bias.copy_(bias)
        self.requires_grad_(False)


def _fetch(gm: torch.fx.GraphModule, node):
    """The tensor behind a get_attr node, else None."""
    if not isinstance(node, torch.fx.Node) or node.op != "get_attr":
        return None
    obj = gm
    for part in node.target.split("."):
        if not hasattr(obj, part):
            return None
        obj = getattr(obj, part)
    return obj if isinstance(obj, torch.Tensor) else None


def replace_addmm(gm: torch.fx.GraphModule):
    """`torch.addmm(bias, x2d, weight)` on parameters — GPT-2's Conv1D — → the fused linear on the
    transposed weight (transposed once, here). Not in the reference."""
    count = 0
    for n in list(gm.graph.nodes):
        if n.op != "call_function" or n.target is not torch.addmm or len(n.args) != 3 or n.kwargs:
            continue
        bias_node, x, weight_node = n.args
        bias, weight = _fetch(gm, bias_node), _fetch(gm, weight_node)
        if bias is None or weight is None or weight.dim() != 2 or bias.shape != (weight.shape[1],):
            continue
        name = f"kernl_transposed_linear_{count}"
        while hasattr(gm, name):
            count += 1
            name = f"kernl_transposed_linear_{count}"
        count += 1
        gm.add_submodule(name, TransposedLinear(weight, bias))
        with gm.graph.inserting_before(n):
            mod = gm.graph.get_attr(name)
            fused = gm.graph.call_function(linear_wrapper, (x, mod), {"activation": ""})
        n.replace_all_uses_with(fused)
        gm.graph.erase_node(n)
        for old in (bias_node, weight_node):
            if len(old.users) == 0:
                gm.graph.erase_node(old)
    if count:
        gm.graph.lint()
        gm.recompile()
    return gm


def _const_and_node(n, targets):
    """For a commutative binary call_function node: (python number, other operand), else None."""
    if not (isinstance(n, torch.fx.Node) and n.op == "call_function" and n.target in targets and len(n.args) == 2 and not n.kwargs):
        return None
    a, b = n.args
    if isinstance(a, (int, float)) and isinstance(b, torch.fx.Node):
        return float(a), b
    if isinstance(b, (int, float)) and isinstance(a, torch.fx.Node):
        return float(b), a
    return None


def _match_tanh_gelu(root):
    """0.5 * x * (1 + tanh(sqrt(2/pi) * (x + 0.044715 * x**3))) as `transformers` writes gelu_new.
    Returns (x, interior nodes) or None."""
    import operator

    mul, add = (operator.mul, torch.mul), (operator.add, torch.add)

    def close(value, target):
        return abs(value - target) < 1e-6

    if not (isinstance(root, torch.fx.Node) and root.op == "call_function" and root.target in mul and len(root.args) == 2):
        return None
    for half, one_plus in ((root.args[0], root.args[1]), (root.args[1], root.args[0])):
        h = _const_and_node(half, mul)
        o = _const_and_node(one_plus, add)
        if h is None or o is None or not close(h[0], 0.5) or not close(o[0], 1.0):
            continue
        x, tanh = h[1], o[1]
        if not (tanh.op == "call_function" and tanh.target is torch.tanh and len(tanh.args) == 1):
            continue
        scaled = _const_and_node(tanh.args[0], mul)
        if scaled is None or not close(scaled[0], 0.7978845608028654):
            continue
        inner = scaled[1]
        if not (inner.op == "call_function" and inner.target in add and len(inner.args) == 2 and not inner.kwargs):
            continue
        for x2, cubic in ((inner.args[0], inner.args[1]), (inner.args[1], inner.args[0])):
            c = _const_and_node(cubic, mul)
            if x2 is not x or c is None or not close(c[0], 0.044715):
                continue
            pw = c[1]
            is_pow = (pw.op == "call_function" and pw.target is torch.pow) or (pw.op == "call_method" and pw.target == "pow")
            if not (is_pow and len(pw.args) == 2 and pw.args[0] is x and pw.args[1] in (3, 3.0)):
                continue
            interior = [one_plus, tanh, tanh.args[0], inner, cubic, pw, half]
            if any(len(node.users) != 1 for node in interior):
                continue
            return x, interior
    return None


def fuse_tanh_gelu_into_linear(gm: torch.fx.GraphModule):
    """A bare fused linear (possibly seen through a view) whose only reader is the tanh form of GELU
    gets activation="fast_gelu" (reference kernel: activation_func.py:40-43) and the eager expression
    goes away. Where the expression does not sit behind such a linear it is left as it is."""
    changed = False
    for root in list(gm.graph.nodes):
        m = _match_tanh_gelu(root)
        if m is None:
            continue
        x, interior = m
        lin = x
        if lin.op == "call_method" and lin.target in ("view", "reshape") and isinstance(lin.args[0], torch.fx.Node):
            if len(lin.args[0].users) != 1:
                continue
            lin = lin.args[0]
        if _bare_linear(gm, lin, exact=False) is None or len(x.users) != 3:  # x feeds 0.5*x, x + ..., pow(x, 3)
            continue
        kwargs = dict(lin.kwargs)
        kwargs["activation"] = "fast_gelu"
        lin.kwargs = kwargs
        root.replace_all_uses_with(x)
        gm.graph.erase_node(root)
        for node in interior:
            gm.graph.erase_node(node)
        changed = True
    if changed:
        gm.graph.lint()
        gm.recompile()
    return gm


def replace_all_linear(gm: torch.fx.GraphModule):
    """Fused variants first, then what is left (reference: optimizer/linear.py:113-119).
    The nn.GELU module form is an addition for current model code; a SiLU is left alone here because
    it belongs to a gated feed-forward, which `fuse_gated_feed_forward` takes as a whole. The last two
    passes cover GPT-2: Conv1D's addmm and the tanh form of GELU written out in eager ops."""
    replace_linear_activation(gm, torch.nn.Tanh(), "tanh")
    replace_linear_activation(gm, torch.nn.ReLU(), "relu")
    replace_linear_activation(gm, torch.nn.functional.gelu, "gelu")
    replace_linear_activation(gm, torch.nn.GELU(), "gelu")
    replace_linear_activation(gm, torch.nn.GELU(approximate="tanh"), "fast_gelu")
    replace_linear(gm)
    replace_linear_fn(gm)
    replace_linear_fn_constant_match(gm)
    replace_addmm(gm)
    fuse_tanh_gelu_into_linear(gm)
