"""Drop-in alias: the reference's import paths, served by kernl_b200.

`from kernl.model_optimization import optimize_model` — and every other module path of the
reference's package that this library mirrors (`kernl.implementations.attention`,
`kernl.optimizer.cuda_graph`, `kernl.utils.extended_matcher`, ...) — resolves to the module of the
same name under `kernl_b200`, as the very same module object, so code written against the
reference (src/kernl/model_optimization.py:32 and the modules it imports) runs unchanged.
Modules of the reference that have no counterpart here (its Triton debugger, the benchmark plugin,
`attention_vec_mat`, `batched_matmul`) raise ModuleNotFoundError.
"""
import importlib
import importlib.abc
import importlib.util
import sys

import kernl_b200

_PREFIX = "kernl."
_REAL = "kernl_b200."


class _AliasFinder(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    def find_spec(self, fullname, path=None, target=None):
        if not fullname.startswith(_PREFIX):
            return None
        try:
            importlib.import_module(_REAL + fullname[len(_PREFIX):])
        except ModuleNotFoundError:
            return None
        return importlib.util.spec_from_loader(fullname, self)

    def create_module(self, spec):
        real = sys.modules[_REAL + spec.name[len(_PREFIX):]]
        self._real_spec = real.__spec__
        return real

    def exec_module(self, module):
        module.__spec__ = self._real_spec  # the import machinery put the alias spec on the shared module


if not any(isinstance(f, _AliasFinder) for f in sys.meta_path):
    sys.meta_path.insert(0, _AliasFinder())

__version__ = getattr(kernl_b200, "__version__", "0")
