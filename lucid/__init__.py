"""Import alias: makes ``import lucid`` / ``import lucid.quantization as Q`` /
``from lucid.nn.quantized import dynamic`` resolve to ``lucid_b200`` so code written against
the reference's module paths runs unchanged on the CUDA backend.  Every ``lucid.x.y`` is the
very module object ``lucid_b200.x.y`` (never a second copy, whose classes would fail
``isinstance`` checks against the first)."""
import importlib
import importlib.abc
import importlib.util
import sys

import lucid_b200 as _impl


class _AliasFinder(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    @staticmethod
    def _real(fullname: str) -> str:
        return "lucid_b200" + fullname[len("lucid"):]

    def find_spec(self, fullname, path=None, target=None):
        if not fullname.startswith("lucid."):
            return None
        try:
            importlib.import_module(self._real(fullname))
        except ModuleNotFoundError as e:
            if e.name and self._real(fullname).startswith(e.name):
                return None  # no such submodule: let the import fail as usual
            raise
        return importlib.util.spec_from_loader(fullname, self)

    def create_module(self, spec):
        return sys.modules[self._real(spec.name)]

    def exec_module(self, module) -> None:
        """Nothing to run: the module was executed under its real name."""


sys.meta_path.insert(0, _AliasFinder())
for _name, _mod in list(sys.modules.items()):
    if _name.startswith("lucid_b200."):
        sys.modules["lucid" + _name[len("lucid_b200"):]] = _mod
sys.modules["lucid"] = _impl
