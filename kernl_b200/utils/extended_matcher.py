"""Subgraph matching and replacement on torch.fx graphs.

`replace_pattern(gm, pattern, replacement)` keeps the signature and behaviour of the reference's
`kernl.utils.extended_matcher.replace_pattern` (src/kernl/utils/extended_matcher.py:343-523), which
differs from `torch.fx.replace_pattern` in two ways that the graph rewrites rely on:
  * literal (non-Node) arguments must be equal for two nodes to match (extended_matcher.py:112-115,
    src/kernl/utils/fx.py:21-39) — `x / 8.0` does not match `x / 4.0`;
  * `call_module` nodes match when the MODULE TYPES are equal (extended_matcher.py:116-124), and the
    modules named in the replacement are re-pointed to the modules that were matched (:458-467), so
    a replacement written against a dummy `torch.nn.Linear(1, 1)` ends up calling the real layer.
This is an independent implementation: a recursive structural match anchored on the pattern's
output, a check that no interior value escapes the match, then a node-by-node copy of the traced
replacement.
"""
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Union

import torch
from torch.fx import Graph, GraphModule, Node, symbolic_trace

from kernl_b200.utils.fx import literals_are_equal


@dataclass
class Match:
    anchor: Node  # node of the target graph that produced the matched pattern's output
    nodes_map: Dict[Node, Node] = field(default_factory=dict)  # pattern node -> graph node
    modules_map: Dict[str, str] = field(default_factory=dict)  # pattern module name -> graph module name


def _trace(obj: Union[Callable, GraphModule, Graph]) -> GraphModule:
    if isinstance(obj, GraphModule):
        return obj
    return symbolic_trace(obj)


class _Matcher:
    def __init__(self, pattern_gm: GraphModule, target_gm: GraphModule):
        self.pattern_gm = pattern_gm
        self.target_gm = target_gm
        self.pattern_modules = dict(pattern_gm.named_modules())
        self.target_modules = dict(target_gm.named_modules())

    def _targets_equal(self, pn: Node, gn: Node, m: Match) -> bool:
        if pn.op != gn.op:
            return False
        if pn.op == "call_module":
            pm, tm = self.pattern_modules.get(pn.target), self.target_modules.get(gn.target)
            if pm is None or tm is None or type(pm) is not type(tm):
                return False
            # same type, different function: nn.GELU() is the erf form, nn.GELU(approximate="tanh") is not
            if isinstance(pm, torch.nn.GELU) and pm.approximate != tm.approximate:
                return False
            known = m.modules_map.get(pn.target)
            if known is not None and known != gn.target:
                return False
            m.modules_map[pn.target] = gn.target
            return True
        if pn.op == "get_attr":
            return True
        return pn.target == gn.target

    def _match_arg(self, pa, ga, m: Match) -> bool:
        if isinstance(pa, Node):
            return isinstance(ga, Node) and self._match_node(pa, ga, m)
        if isinstance(ga, Node):
            return False
        if isinstance(pa, (tuple, list)):
            if type(pa) != type(ga) or len(pa) != len(ga):  # noqa: E721
                return False
            return all(self._match_arg(x, y, m) for x, y in zip(pa, ga))
        if isinstance(pa, dict):
            if not isinstance(ga, dict) or pa.keys() != ga.keys():
                return False
            return all(self._match_arg(pa[k], ga[k], m) for k in pa)
        return literals_are_equal(pa, ga)

    @staticmethod
    def _kwargs(node: Node) -> dict:
        """Keyword arguments that carry information: tracing through torch functions records
        private bookkeeping keys (`_stacklevel`) and defaulted `None`s that another tracer omits."""
        return {k: v for k, v in node.kwargs.items() if not k.startswith("_") and v is not None}

    def _match_node(self, pn: Node, gn: Node, m: Match) -> bool:
        if pn in m.nodes_map:
            return m.nodes_map[pn] is gn
        if pn.op == "placeholder":
            m.nodes_map[pn] = gn
            return True
        if not self._targets_equal(pn, gn, m):
            return False
        pk, gk = self._kwargs(pn), self._kwargs(gn)
        if len(pn.args) != len(gn.args) or pk.keys() != gk.keys():
            return False
        m.nodes_map[pn] = gn
        ok = all(self._match_arg(pa, ga, m) for pa, ga in zip(pn.args, gn.args)) and all(
            self._match_arg(pk[k], gk[k], m) for k in pk
        )
        return ok

    def try_match(self, pattern_anchor: Node, gn: Node):
        m = Match(anchor=gn)
        if not self._match_node(pattern_anchor, gn, m):
            return None
        interior = {g for p, g in m.nodes_map.items() if p.op != "placeholder"}
        for p, g in m.nodes_map.items():
            if p.op == "placeholder" or g is gn:
                continue
            if any(user not in interior for user in g.users):
                return None  # an intermediate value is used outside the pattern
        # one pattern placeholder may not swallow an interior node of the same match
        for p, g in m.nodes_map.items():
            if p.op == "placeholder" and g in interior:
                return None
        return m


def replace_pattern(
    gm: GraphModule,
    pattern: Union[Callable, GraphModule],
    replacement: Union[Callable, GraphModule],
) -> List[Match]:
    """Replace every non-overlapping occurrence of `pattern` in `gm` by `replacement`.

    pattern / replacement: callables or nn.Modules with the same positional parameters (they are
    symbolically traced), returning one value. Returns the matches that were replaced.
    """
    pattern_gm, replacement_gm = _trace(pattern), _trace(replacement)
    p_out = [n for n in pattern_gm.graph.nodes if n.op == "output"][0]
    r_out = [n for n in replacement_gm.graph.nodes if n.op == "output"][0]
    pattern_anchor = p_out.args[0]
    assert isinstance(pattern_anchor, Node), "the pattern must return exactly one value"
    p_placeholders = [n for n in pattern_gm.graph.nodes if n.op == "placeholder"]
    r_placeholders = [n for n in replacement_gm.graph.nodes if n.op == "placeholder"]
    assert len(p_placeholders) == len(r_placeholders), "pattern and replacement need the same parameters"

    matcher = _Matcher(pattern_gm, gm)
    matches: List[Match] = []
    consumed = set()
    for gn in reversed(list(gm.graph.nodes)):
        if gn in consumed or gn.op in ("placeholder", "output"):
            continue
        m = matcher.try_match(pattern_anchor, gn)
        if m is None:
            continue
        interior = [g for p, g in m.nodes_map.items() if p.op != "placeholder"]
        if any(g in consumed for g in interior):
            continue
        if any(p not in m.nodes_map for p in p_placeholders):
            continue
        matches.append(m)
        consumed.update(interior)

    replacement_modules = dict(replacement_gm.named_modules())
    for m in matches:
        val_map: Dict[Node, Node] = {rp: m.nodes_map[pp] for pp, rp in zip(p_placeholders, r_placeholders)}
        with gm.graph.inserting_before(m.anchor):
            for rn in replacement_gm.graph.nodes:
                if rn.op in ("placeholder", "output"):
                    continue
                new = gm.graph.node_copy(rn, lambda n: val_map[n])
                if rn.op in ("call_module", "get_attr"):
                    if rn.target in m.modules_map:
                        # a module of the replacement that stands for a matched module
                        new.target = m.modules_map[rn.target]
                    elif rn.op == "call_module" or rn.target in replacement_modules:
                        raise RuntimeError(f"replacement module '{rn.target}' has no counterpart in the pattern")
                    else:
                        # plain attribute (tensor constant) of the replacement: carry it over
                        name = f"_kb_repl_{len(matches)}_{rn.target.replace('.', '_')}"
                        setattr(gm, name, getattr(replacement_gm, rn.target))
                        new.target = name
                val_map[rn] = new
        result = r_out.args[0]
        m.anchor.replace_all_uses_with(val_map[result] if isinstance(result, Node) else result)
        interior = [g for p, g in m.nodes_map.items() if p.op != "placeholder"]
        order = {n: i for i, n in enumerate(gm.graph.nodes)}
        for g in sorted(interior, key=lambda n: order[n], reverse=True):
            if len(g.users) == 0:
                gm.graph.erase_node(g)
    if matches:
        gm.graph.lint()
        gm.recompile()
    return matches
