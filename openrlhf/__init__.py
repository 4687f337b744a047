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
        if fullname == "openrlhf.cli" or fullname.startswith("openrlhf.cli."):
            return None                  # physical launcher stubs of this package
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
        mod = importlib.import_module(real)
        self._real_specs[id(mod)] = mod.__spec__
        return mod

    def exec_module(self, module):
        # the import machinery has just stamped the alias spec on the (shared) module object: put the real one back so
        # that relative imports inside the module keep resolving against its real package
        real = self._real_specs.get(id(module))
        if real is not None:
            module.__spec__ = real
        return None

    _real_specs: dict = {}


if not any(isinstance(f, _AliasFinder) for f in sys.meta_path):
    # ahead of the path finder: a submodule of an aliased package (openrlhf.utils.agent) must be the *same* module
    # object as its target, not a second copy loaded from the target's directory under the alias name, or user classes
    # deriving from openrlhf.utils.agent.AgentExecutorBase would fail the workers' issubclass checks
    sys.meta_path.insert(0, _AliasFinder())
__version__ = "0.11.0+b200"
