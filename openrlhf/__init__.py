"""Alias package: ``openrlhf.*`` resolves to ``openrlhf_b200.*`` so that launch scripts and user agent / reward files
written against the reference (``python -m openrlhf.cli.train_ppo_ray``, ``from openrlhf.utils.agent import ...``) keep
working unchanged."""
import importlib
import importlib.abc
import importlib.util
import sys

_TARGET = "openrlhf_b200"


class _AliasFinder(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    def find_spec(self, fullname, path=None, target=None):
        if fullname == "openrlhf" or not fullname.startswith("openrlhf."):
            return None
        real = _TARGET + fullname[len("openrlhf"):]
        try:
            real_spec = importlib.util.find_spec(real)
        except (ImportError, ValueError):
            return None
        if real_spec is None:
            return None
        return importlib.util.spec_from_loader(fullname, self,
                                               is_package=real_spec.submodule_search_locations is not None)

    def create_module(self, spec):
        real = _TARGET + spec.name[len("openrlhf"):]
        return importlib.import_module(real)

    def exec_module(self, module):
        return None


if not any(isinstance(f, _AliasFinder) for f in sys.meta_path):
    sys.meta_path.append(_AliasFinder())  # after the regular finders: physical modules under openrlhf/ win
__version__ = "0.11.0+b200"
