"""Alias package: ``openrlhf.*`` resolves to ``openrlhf_b200.*`` so that launch scripts and user agent / reward files
written against the reference (``python -m openrlhf.cli.train_ppo_ray``, ``from openrlhf.utils.agent import ...``) keep
working unchanged."""
import importlib
import importlib.abc
import importlib.util
import sys

_TARGET = "openrlhf_b200"

# module paths of the reference that live elsewhere in this package, and names it uses for the same things
_RENAMED = {
    "openrlhf.trainer.ppo_utils": "openrlhf_b200.rl",
    "openrlhf.trainer.ppo_utils.experience": "openrlhf_b200.rl.experience",
    "openrlhf.trainer.ppo_utils.experience_maker": "openrlhf_b200.rl.experience_maker",
    "openrlhf.trainer.ppo_utils.kl_controller": "openrlhf_b200.rl.kl_controller",
    "openrlhf.trainer.ppo_utils.length_penalty": "openrlhf_b200.rl.length_penalty",
    "openrlhf.trainer.ppo_utils.replay_buffer": "openrlhf_b200.rl.replay_buffer",
    "openrlhf.trainer.ppo_utils.samples_generator": "openrlhf_b200.rl.samples_generator",
    "openrlhf.utils.deepspeed": "openrlhf_b200.utils.strategy",
    "openrlhf.utils.deepspeed.deepspeed": "openrlhf_b200.utils.strategy",
    "openrlhf.models.ring_attn_utils": "openrlhf_b200.parallel.cp",
    "openrlhf.trainer.ray": "openrlhf_b200.runtime",
    "openrlhf.trainer.ray.launcher": "openrlhf_b200.runtime.core",
    "openrlhf.trainer.ray.vllm_engine": "openrlhf_b200.runtime.core",
}
_EXTRA_NAMES = {
    "openrlhf_b200.runtime.core": {"RayActorGroup": "ActorGroup", "batch_vllm_engine_call": "batch_engine_call"},
    "openrlhf_b200.runtime": {"batch_vllm_engine_call": "core.batch_engine_call"},
}


def _real_name(fullname: str) -> str:
    return _RENAMED.get(fullname, _TARGET + fullname[len("openrlhf"):])


class _AliasFinder(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    def find_spec(self, fullname, path=None, target=None):
        if fullname == "openrlhf" or not fullname.startswith("openrlhf."):
            return None
        if fullname == "openrlhf.cli" or fullname.startswith("openrlhf.cli."):
            return None                  # physical launcher stubs of this package
        real = _real_name(fullname)
        try:
            real_spec = importlib.util.find_spec(real)
        except (ImportError, ValueError):
            return None
        if real_spec is None:
            return None
        # a module of this package that stands in for a package of the reference (openrlhf.utils.deepspeed) must
        # still accept submodule imports under the old name
        is_pkg = real_spec.submodule_search_locations is not None or any(k.startswith(fullname + ".") for k in _RENAMED)
        return importlib.util.spec_from_loader(fullname, self, is_package=is_pkg)

    def create_module(self, spec):
        real = _real_name(spec.name)
        mod = importlib.import_module(real)
        self._real_specs[id(mod)] = mod.__spec__
        for alias, target in _EXTRA_NAMES.get(real, {}).items():
            if not hasattr(mod, alias):
                owner, _, attr = target.rpartition(".")
                src = importlib.import_module(real + "." + owner) if owner else mod
                setattr(mod, alias, getattr(src, attr))
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
