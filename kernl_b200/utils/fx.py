"""Small helpers over torch.fx nodes (reference: src/kernl/utils/fx.py)."""
from typing import Iterable

from torch.fx import Node


def compare_static_args(arg1, arg2) -> bool:
    """True when two node arguments agree as far as static information goes: Nodes match any Node,
    containers are compared element-wise, literals by type and value (reference: fx.py:21-31)."""
    if type(arg1) != type(arg2):  # noqa: E721
        return False
    if isinstance(arg1, Node):
        return True
    if isinstance(arg1, (str, bytes)):
        return arg1 == arg2
    if isinstance(arg1, Iterable):
        a, b = list(arg1), list(arg2)
        return len(a) == len(b) and all(compare_static_args(x, y) for x, y in zip(a, b))
    return arg1 == arg2


def static_args_are_equal(pn: Node, gn: Node) -> bool:
    """Positional arguments of two nodes agree statically (reference: fx.py:33-39)."""
    return len(pn.args) == len(gn.args) and all(compare_static_args(a, b) for a, b in zip(pn.args, gn.args))


def literals_are_equal(a, b) -> bool:
    """Two non-Node arguments are the same literal: same type (1 and 1.0, or True and 1, differ),
    containers element-wise, slices by their three fields. This is the comparison the pattern
    matcher applies to every literal argument of a candidate node."""
    if isinstance(a, Node) or isinstance(b, Node):
        return False
    if type(a) != type(b):  # noqa: E721
        return False
    if isinstance(a, (tuple, list)):
        return len(a) == len(b) and all(literals_are_equal(x, y) for x, y in zip(a, b))
    if isinstance(a, slice):
        return (a.start, a.stop, a.step) == (b.start, b.stop, b.step)
    return a == b
