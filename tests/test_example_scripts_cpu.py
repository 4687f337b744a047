"""Every flag used by the example launch scripts is accepted by the CLI it targets."""
import glob
import importlib
import os
import re
import shlex

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
NO_CLI = {"docker_run.sh"}     # helper scripts that start no trainer


def _commands(path):
    text = open(path).read().replace("\\\n", " ")
    for line in text.splitlines():
        m = re.search(r"-m (openrlhf\.cli\.\w+)(.*)", line)
        if m:
            yield m.group(1), m.group(2)


@pytest.mark.parametrize("script", sorted(glob.glob(os.path.join(ROOT, "examples", "scripts", "*.sh"))))
def test_script_flags_parse(script):
    found = False
    for module, argstr in _commands(script):
        found = True
        argstr = re.sub(r"\$\{\w+:-([^}]*)\}", lambda m: m.group(1).strip('"'), argstr)
        mod = importlib.import_module(module.replace("openrlhf.", "openrlhf_b200."))
        if not hasattr(mod, "build_parser"):
            continue
        flags = [t for t in shlex.split(argstr) if t.startswith("--")]
        known = set()
        for a in mod.build_parser()._actions:
            known.update(a.option_strings)
        missing = [f for f in flags if f not in known]
        assert not missing, f"{os.path.basename(script)}: {module} does not accept {missing}"
    assert found or os.path.basename(script) in NO_CLI, "no CLI invocation found"
