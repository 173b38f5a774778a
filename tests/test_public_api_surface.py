"""Every public name of the reference package layout (``vrl.<module>``: the ``__all__`` list of a
package, the public classes and functions of a plain module) resolves here, through the ``vrl``
alias.  ``public_api_names.json`` is that list of names; recipes, tests and user code written
against the reference import exactly these."""

import importlib
import json
import os

import pytest

with open(os.path.join(os.path.dirname(__file__), "public_api_names.json")) as fh:
    NAMES = json.load(fh)


def test_the_list_covers_the_whole_layout():
    assert len(NAMES) > 100 and sum(len(v) for v in NAMES.values()) > 400
    for package in ("vrl.algorithms", "vrl.trainers", "vrl.engine", "vrl.rollouts.collector", "vrl.rewards",
                    "vrl.models", "vrl.distributed.ray", "vrl.config"):
        assert package in NAMES


@pytest.mark.parametrize("module", sorted(NAMES))
def test_module_imports_and_has_its_public_names(module):
    mod = importlib.import_module(module)
    missing = [name for name in NAMES[module] if not hasattr(mod, name)]
    assert not missing, f"{module} lacks {missing}"
