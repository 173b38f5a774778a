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


with open(os.path.join(os.path.dirname(__file__), "public_api_signatures.json")) as fh:
    SIGNATURES = json.load(fh)

# Where the native models deliberately differ: the reference hands its policies objects of external
# libraries (a diffusers pipeline, the vendor's multimodal model and processor, a vendor repository
# directory); the native policies are built from ``model.arch`` and have no such arguments.  The
# per-family sampling-state records are private to each policy.
NATIVE_MODEL_DIFFERENCES = {
    "vrl.models.families.sd3_5.policy": {"SD3_5Policy.__init__", "SD3_5Policy.pipeline"},
    "vrl.models.families.cosmos.policy": {"CosmosPredict2Policy.__init__", "CosmosPredict2Policy.pipeline"},
    "vrl.models.families.wan_2_1.diffusers_policy": {"WanT2VDiffusersPolicy.__init__", "WanT2VDiffusersPolicy.pipeline"},
    "vrl.models.families.wan_2_1.official_policy": {"WanT2VOfficialPolicy.__init__"},
    "vrl.models.families.janus_pro.policy": {"JanusProPolicy.__init__", "JanusProPolicy.processor",
                                             "image_token_logits_from_hidden"},
}


def _checks():
    for module, entries in sorted(SIGNATURES.items()):
        for name in sorted(entries):
            if name in NATIVE_MODEL_DIFFERENCES.get(module, ()):
                continue
            yield module, name


@pytest.mark.parametrize("module,name", list(_checks()))
def test_callable_keeps_the_parameter_names_and_positional_order(module, name):
    import inspect

    mod = importlib.import_module(module)
    target = mod
    for part in name.split("."):
        if not hasattr(target, part):
            if part == "__init__":
                return
            pytest.fail(f"{module}.{name} does not exist")
        target = inspect.getattr_static(target, part) if inspect.isclass(target) else getattr(target, part)
    if isinstance(target, property):
        return                                   # a method of the reference served as a property here
    if isinstance(target, (staticmethod, classmethod)):
        target = target.__func__
    if name.endswith(".__init__") and target is object.__init__:
        return
    try:
        sig = inspect.signature(target)
    except (TypeError, ValueError):
        return
    have = [k for k in sig.parameters if k not in ("self", "cls")]
    takes_kwargs = any(p.kind == p.VAR_KEYWORD for p in sig.parameters.values())
    want = SIGNATURES[module][name]
    if not takes_kwargs:
        missing = [w for w in want["positional"] + want["keyword_only"] if w not in have]
        assert not missing, f"{module}.{name} lacks parameters {missing}"
    positional = [k for k, p in sig.parameters.items()
                  if p.kind in (p.POSITIONAL_ONLY, p.POSITIONAL_OR_KEYWORD) and k not in ("self", "cls")]
    if all(w in have for w in want["positional"]):
        assert positional[:len(want["positional"])] == want["positional"], \
            f"{module}.{name}: positional order {positional} differs from {want['positional']}"
