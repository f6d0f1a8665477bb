"""`makani` name for this framework: `python -m makani.train`, `import makani.utils.comm`, `from makani import Trainer`
resolve to the modules of `makani_b200`, so that launch scripts, recipes and plug-ins written against the upstream
package name keep working (upstream layout: makani/__init__.py:16-19, makani/train.py, makani/inference.py).

`makani.X.Y` is the SAME module object as `makani_b200.X.Y` (a meta-path finder aliases it; nothing is imported twice),
with one addition: `makani.mpu.*` maps to `makani_b200.parallel.*`, the name the upstream package uses for its
model-parallel layer.
"""

from __future__ import annotations

import importlib
import importlib.abc
import importlib.util
import sys

import makani_b200 as _impl

__version__ = _impl.__version__

_RENAMES = {"makani.mpu": "makani_b200.parallel"}
_OWN = {"makani.train", "makani.inference", "makani.train_profile", "makani.convert_legacy_to_flexible"}


def _target(name: str) -> str:
    for src, dst in _RENAMES.items():
        if name == src or name.startswith(src + "."):
            return dst + name[len(src):]
    return "makani_b200" + name[len("makani"):]


class _AliasLoader(importlib.abc.Loader):
    def __init__(self, target):
        self.target = target

    def create_module(self, spec):
        return importlib.import_module(self.target)

    def exec_module(self, module):
        pass


class _AliasFinder(importlib.abc.MetaPathFinder):
    def find_spec(self, fullname, path=None, target=None):
        if not fullname.startswith("makani.") or fullname in _OWN:
            return None
        tgt = _target(fullname)
        try:
            real = importlib.util.find_spec(tgt)
        except (ImportError, ValueError):
            return None
        if real is None:
            return None
        spec = importlib.util.spec_from_loader(fullname, _AliasLoader(tgt), is_package=real.submodule_search_locations is not None)
        return spec


if not any(isinstance(f, _AliasFinder) for f in sys.meta_path):
    sys.meta_path.insert(0, _AliasFinder())


def __getattr__(name):
    return getattr(_impl, name)
